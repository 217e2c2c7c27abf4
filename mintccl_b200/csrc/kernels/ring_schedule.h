// Ring / chain schedules written once against the step interface of a protocol: which role a rank
// plays at which step, which shard or chunk it touches, how a message is cut into FIFO steps.  The same
// code drives the CUDA kernels (SimplePrims / LL128Prims, one CTA per channel) and the host-side
// protocol simulator (one thread per rank and channel), so the simulator checks the very schedule the
// GPU runs.
//
// Every collective is expressed as the standard n-1 step ring schedule, so no rank plays a lagged
// "root" (the reference's reduce and reduce-scatter drain the root several rounds late from a one-round
// buffer, 5_reduce.py:79-89 and 7_reducescatter.py:57-67, which loses data on more than two ranks).
//
// Capability map to the reference kernels:
//   OP_SENDRECV      2_sendrecv_indirect.py:44-93 / 3_sendrecv_buffer.py:23-74 (route of any length)
//   OP_BROADCAST     4_broadcast.py:27-76
//   OP_REDUCE        5_reduce.py:36-95
//   OP_ALLGATHER     6_allgather.py:24-77 (temporal) and 6_allgather.py:79-138 (spatial)
//   OP_REDUCESCATTER 7_reducescatter.py:13-79
//   OP_ALLREDUCE     on the reference's roadmap only (README.md:23)
#pragma once
#include <stdlib.h>
#include "../device/sched.h"

#if defined(__CUDACC__)
#define MT_SCHED_FN __device__ __forceinline__
#else
#define MT_SCHED_FN static inline
#endif

namespace mt {

enum RingOp : int {
  OP_SENDRECV = 0,
  OP_BROADCAST = 1,
  OP_REDUCE = 2,
  OP_ALLGATHER = 3,
  OP_REDUCESCATTER = 4,
  OP_ALLREDUCE = 5,
};

struct RingArgs {
  const void* in[MT_MAX_RANKS];   // per local rank (index 0 outside emulation)
  void* out[MT_MAX_RANKS];
  uint64_t nbytes;                // chain ops and all-reduce: message bytes; AG / RS: bytes per shard
  int32_t op;
  int32_t root;                   // broadcast / reduce
  int32_t spatial;                // AG / RS: CTA groups per shard instead of all CTAs per shard
  int32_t chain_len;              // OP_SENDRECV: number of ranks on the route
  int32_t chain[MT_MAX_RANKS + 1];
  int32_t elem_size;
  uint32_t step_bytes;            // chain ops over the Simple protocol: bytes per FIFO step when smaller than a slot
                                  // (0: whole slots); a multiple of 128
};

// Step size of chain operations (send/recv over a route, broadcast, reduce) over the Simple protocol.  The last of L
// ranks sees its first byte after L - 2 extra steps, so smaller steps shorten the fill of the chain; but every step
// costs a flag round (block barrier, release store, the peer's poll).  Which side wins depends on how the calls
// follow one another.  Blocks of back-to-back calls overlap one another, so the fill hardly counts: there, on 8 B200,
// cutting a channel's share into eight steps took the 64 MiB broadcast from 511 to 373 GB/s.  A call that other work
// surrounds pays the fill in full: fenced calls on 4 B200 took 292 us with whole 1 MiB slots and 190 us with 256 KiB
// steps at 64 MiB (624 -> 551 us at 256 MiB, 99 -> 87 us at 16 MiB with 128 KiB steps), and a step of five mixed
// collectives on 8 B200 went from 1.42 to 0.95 ms.  The default serves the single call: on a chain of more than two
// ranks half a channel's share per step, at least 64 KiB and at most 256 KiB.  MINTCCL_CHAIN_STEP_BYTES overrides it (rounded down to a multiple of
// 128, at least 4 KiB; 0: whole slots, the best for streams of identical calls).
static inline uint32_t mt_chain_step_bytes(uint64_t bytes_per_channel, uint64_t slot_bytes, int chain_len) {
  const char* e = getenv("MINTCCL_CHAIN_STEP_BYTES");
  if (e) {
    long long v = atoll(e);
    if (v <= 0) return 0;
    if (v < 4096) v = 4096;
    if (v > (1ll << 30)) v = 1ll << 30;
    return (uint32_t)(v & ~127ll);
  }
  if (chain_len <= 2) return 0;   // one link: nothing to fill, whole slots cost the fewest flag rounds
  uint64_t step = bytes_per_channel / 2;
  if (step < (64u << 10)) step = 64u << 10;
  if (step > (256u << 10)) step = 256u << 10;
  if (step >= slot_bytes) return 0;
  return (uint32_t)(step & ~127ull);
}

enum Role : int {
  R_NONE = 0,
  R_COPY,                   // local copy (single rank)
  R_SEND,                   // src -> next
  R_COPY_SEND,              // src -> dst, next
  R_RECV,                   // prev -> dst
  R_RECV_SEND,              // prev -> next                  (jump host)
  R_RECV_COPY_SEND,         // prev -> dst, next
  R_RECV_REDUCE_SEND,       // prev + src -> next
  R_RECV_REDUCE_COPY,       // prev + src -> dst
  R_RECV_REDUCE_COPY_SEND,  // prev + src -> dst, next
};

template <class P>
MT_SCHED_FN bool run_role(P& p, int role, const uint8_t* src, uint8_t* dst, uint64_t n) {
  switch (role) {
    case R_COPY: return p.template step<false, false, true, true>(src, dst, n);
    case R_SEND: return p.template step<false, true, true, false>(src, nullptr, n);
    case R_COPY_SEND: return p.template step<false, true, true, true>(src, dst, n);
    case R_RECV: return p.template step<true, false, false, true>(nullptr, dst, n);
    case R_RECV_SEND: return p.template step<true, true, false, false>(nullptr, nullptr, n);
    case R_RECV_COPY_SEND: return p.template step<true, true, false, true>(nullptr, dst, n);
    case R_RECV_REDUCE_SEND: return p.template step<true, true, true, false>(src, nullptr, n);
    case R_RECV_REDUCE_COPY: return p.template step<true, false, true, true>(src, dst, n);
    case R_RECV_REDUCE_COPY_SEND: return p.template step<true, true, true, true>(src, dst, n);
    default: return true;
  }
}

// Alignment of channel boundaries: a multiple of every element size and of the 16-byte vector.
static constexpr uint64_t kSplitAlign = 128;

template <template <class, int> class Proto, class T, int NTHREADS>
MT_SCHED_FN void ring_body(const MtDevComm& c, const RingArgs& a, int lr, int ch, int nch, int* s_fail) {
  const int n = c.nranks, q = c.ring_pos;
  const uint8_t* in = (const uint8_t*)a.in[lr];
  uint8_t* out = (uint8_t*)a.out[lr];
  const int prev = c.ring[mt_mod(q - 1, n)], next = c.ring[mt_mod(q + 1, n)];

  if (a.op == OP_SENDRECV || a.op == OP_BROADCAST || a.op == OP_REDUCE) {
    // ---- open chain --------------------------------------------------------------------------
    int len, idx = -1, up = -1, down = -1;
    if (a.op == OP_SENDRECV) {
      len = a.chain_len;
      for (int i = 0; i < len; ++i)
        if (a.chain[i] == c.rank) idx = i;
      if (idx < 0) return;
      if (idx > 0) up = a.chain[idx - 1];
      if (idx < len - 1) down = a.chain[idx + 1];
    } else {
      len = n;
      int root_pos = 0;
      for (int i = 0; i < n; ++i)
        if (c.ring[i] == a.root) root_pos = i;
      // broadcast: root, root+1, ...; reduce: root+1, ..., root
      idx = a.op == OP_BROADCAST ? mt_mod(q - root_pos, n) : mt_mod(q - root_pos - 1, n);
      if (idx > 0) up = prev;
      if (idx < len - 1) down = next;
    }
    int role;
    if (len == 1) {
      role = (in != out) ? R_COPY : R_NONE;
    } else if (a.op == OP_SENDRECV) {
      role = idx == 0 ? R_SEND : (idx == len - 1 ? R_RECV : R_RECV_SEND);
    } else if (a.op == OP_BROADCAST) {
      role = idx == 0 ? (in != out ? R_COPY_SEND : R_SEND) : (idx == len - 1 ? R_RECV : R_RECV_COPY_SEND);
    } else {
      role = idx == 0 ? R_SEND : (idx == len - 1 ? R_RECV_REDUCE_COPY : R_RECV_REDUCE_SEND);
    }
    if (role == R_NONE) return;
    Proto<T, NTHREADS> p(c, ch, up, down, s_fail);
    const MtRange r = mt_split(a.nbytes, nch, ch, kSplitAlign);
    uint64_t P = p.step_payload();
    if (a.step_bytes && a.step_bytes < P) P = a.step_bytes;  // sub-slot steps: a shorter fill of the chain
    bool ok = true;
    for (uint64_t off = r.lo; ok && off < r.hi; off += P) {
      const uint64_t nb = mt_min64(P, r.hi - off);
      ok = run_role(p, role, in ? in + off : nullptr, out ? out + off : nullptr, nb);
    }
    p.finish();
    return;
  }

  if (a.op == OP_ALLGATHER || a.op == OP_REDUCESCATTER) {
    const uint64_t B = a.nbytes;  // bytes per shard
    const bool ag = a.op == OP_ALLGATHER;
    if (n == 1) {
      if (in != out) {
        Proto<T, NTHREADS> p(c, ch, -1, -1, s_fail);
        const MtRange r = mt_split(B, nch, ch, kSplitAlign);
        const uint64_t P = p.step_payload();
        for (uint64_t off = r.lo; off < r.hi; off += P) run_role(p, R_COPY, in + off, out + off, mt_min64(P, r.hi - off));
        p.finish();
      }
      return;
    }
    Proto<T, NTHREADS> p(c, ch, prev, next, s_fail);
    const uint64_t P = p.step_payload();
    // temporal: every channel walks all n steps over its slice of the shard.
    // spatial : channel group (ch % n) serves exactly one shard, i.e. one value of the step index.
    const bool spatial = a.spatial && nch >= n && nch % n == 0;
    const int sub = spatial ? ch / n : ch, nsub = spatial ? nch / n : nch;
    const MtRange r = mt_split(B, nsub, sub, kSplitAlign);
    bool ok = true;
    for (uint64_t off = r.lo; ok && off < r.hi; off += P) {
      const uint64_t nb = mt_min64(P, r.hi - off);
      for (int j = 0; ok && j < n; ++j) {
        int shard_pos;
        if (spatial) {
          const int s = ch % n;  // shard (by ring position of its owner) this channel serves
          const int jj = ag ? mt_mod(q - s, n) : mt_mod(q - s - 1, n);
          if (jj != j) continue;
          shard_pos = s;
        } else {
          shard_pos = ag ? mt_ag_shard_pos(q, j, n) : mt_rs_shard_pos(q, j, n);
        }
        const uint64_t so = (uint64_t)c.ring[shard_pos] * B + off;
        if (ag) {
          // in: my shard (B bytes); out: [n][B]
          if (j == 0) {
            const bool inplace = (in == out + (uint64_t)c.rank * B);
            ok = run_role(p, inplace ? R_SEND : R_COPY_SEND, in + off, out + so, nb);
          } else if (j < n - 1) {
            ok = run_role(p, R_RECV_COPY_SEND, nullptr, out + so, nb);
          } else {
            ok = run_role(p, R_RECV, nullptr, out + so, nb);
          }
        } else {
          // in: [n][B]; out: my shard (B bytes)
          if (j == 0) ok = run_role(p, R_SEND, in + so, nullptr, nb);
          else if (j < n - 1) ok = run_role(p, R_RECV_REDUCE_SEND, in + so, nullptr, nb);
          else ok = run_role(p, R_RECV_REDUCE_COPY, in + so, out + off, nb);
        }
      }
    }
    p.finish();
    return;
  }

  if (a.op == OP_ALLREDUCE) {
    const uint64_t N = a.nbytes;
    if (n == 1) {
      if (in != out) {
        Proto<T, NTHREADS> p(c, ch, -1, -1, s_fail);
        const MtRange r = mt_split(N, nch, ch, kSplitAlign);
        const uint64_t P = p.step_payload();
        for (uint64_t off = r.lo; off < r.hi; off += P) run_role(p, R_COPY, in + off, out + off, mt_min64(P, r.hi - off));
        p.finish();
      }
      return;
    }
    Proto<T, NTHREADS> p(c, ch, prev, next, s_fail);
    const uint64_t P = p.step_payload();
    const MtRange r = mt_split(N, nch, ch, kSplitAlign);
    bool ok = true;
    // Regions of up to n*P bytes; inside a region chunk k belongs to ring position k.
    for (uint64_t off = r.lo; ok && off < r.hi; off += (uint64_t)n * P) {
      const uint64_t len = mt_min64((uint64_t)n * P, r.hi - off);
      const uint64_t cb = mt_min64(P, mt_round_up(mt_div_up(len, n), 16));  // chunk bytes in this region
      auto chunk_off = [&](int pos) { return mt_min64((uint64_t)pos * cb, len); };
      auto chunk_len = [&](int pos) { return mt_min64((uint64_t)(pos + 1) * cb, len) - mt_min64((uint64_t)pos * cb, len); };
      // reduce-scatter phase
      for (int j = 0; ok && j < n; ++j) {
        const int k = mt_rs_shard_pos(q, j, n);
        const uint64_t o = off + chunk_off(k), nb = chunk_len(k);
        if (nb == 0) continue;
        if (j == 0) ok = run_role(p, R_SEND, in + o, nullptr, nb);
        else if (j < n - 1) ok = run_role(p, R_RECV_REDUCE_SEND, in + o, nullptr, nb);
        else ok = run_role(p, R_RECV_REDUCE_COPY_SEND, in + o, out + o, nb);
      }
      // all-gather phase: step j receives the finished chunk of position q - j
      for (int j = 1; ok && j < n; ++j) {
        const int k = mt_mod(q - j, n);
        const uint64_t o = off + chunk_off(k), nb = chunk_len(k);
        if (nb == 0) continue;
        ok = run_role(p, j < n - 1 ? R_RECV_COPY_SEND : R_RECV, nullptr, out + o, nb);
      }
    }
    p.finish();
    return;
  }
}

}  // namespace mt
