// LL128 protocol: every 128-byte line carries 120 bytes of payload and an 8-byte flag written by
// the same warp-wide store, so the receiver needs no fence: when it reads the expected flag the rest
// of the line is valid (NVLink delivers a 128-byte store of one warp instruction as a unit).
//
// Same capability as the reference's load/save/recv/send/comp/wait/post _ll128 family
// (protocol.py:57-189) with these differences:
//   * a warp moves 16 lines per iteration (4 coalesced 512-byte accesses; the reference moves 2 lines
//     per 8-thread group, protocol.py:44) and lines are paired so that each pair carries 240
//     contiguous, 16-byte aligned payload bytes;
//   * the flag is step+1 of a 64-bit step counter that keeps growing across kernels, so a slot never
//     has to be cleared and a line left over from an earlier call can never match
//     (the reference restarts flags at 1 in every call, 2_sendrecv_indirect.py:61);
//   * credits are a `head` counter written into the sender's memory by the receiver; the sender polls
//     local memory (the reference polls the remote slot for a zero flag, protocol.py:161-179, and the
//     receiver's zero store can overwrite a line that already arrived);
//   * payload tails and lines that a short message does not need are handled per line;
//   * every spin is bounded and reports instead of hanging.
#pragma once
#include "prims.cuh"
#include "reduce_ops.cuh"
#include "sched.h"

namespace mt {

// Load `width` (8 or 16) bytes of payload at p; only the first `valid` bytes exist, the rest read 0.
template <int WIDTH>
__device__ __forceinline__ void ll128_load_piece(const uint8_t* p, int valid, bool aligned, uint64_t& a, uint64_t& b) {
  a = 0;
  b = 0;
  if (valid <= 0) return;
  if (aligned && valid >= WIDTH) {
    if (WIDTH == 16) {
      u128 t = load128_stream(p);
      a = t.x;
      b = t.y;
    } else {
      a = *reinterpret_cast<const uint64_t*>(p);
    }
    return;
  }
  const int n = valid < WIDTH ? valid : WIDTH;
  for (int i = 0; i < n; ++i) {
    uint64_t byte = p[i];
    if (i < 8) a |= byte << (8 * i);
    else b |= byte << (8 * (i - 8));
  }
}
template <int WIDTH>
__device__ __forceinline__ void ll128_store_piece(uint8_t* p, int valid, bool aligned, uint64_t a, uint64_t b) {
  if (valid <= 0) return;
  if (aligned && valid >= WIDTH) {
    if (WIDTH == 16) {
      u128 t;
      t.x = a;
      t.y = b;
      *reinterpret_cast<u128*>(p) = t;
    } else {
      *reinterpret_cast<uint64_t*>(p) = a;
    }
    return;
  }
  const int n = valid < WIDTH ? valid : WIDTH;
  for (int i = 0; i < n; ++i) p[i] = (uint8_t)((i < 8 ? a >> (8 * i) : b >> (8 * (i - 8))) & 0xff);
}

// Which of the four lines a lane touches per warp chunk, and where their payload lives.
struct LL128Lane {
  int g, l;
  bool flag_lane;
  bool need[4];   // line k*4+g carries payload for a chunk of `nbytes`
  int poff[4];    // payload offset (inside the chunk) of this lane's piece of line k
  __device__ __forceinline__ LL128Lane(int nbytes) {
    const int lane = threadIdx.x & 31;
    g = lane >> 3;
    l = lane & 7;
    flag_lane = (l == 7);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int pair = (k >> 1) * 4 + g, half = k & 1;
      const int line_off = MT_LL128_PAIR_PAYLOAD * pair + 128 * half;
      // the second line of a pair also carries payload bytes [120,128) of the pair (in its flag lane)
      need[k] = (MT_LL128_PAIR_PAYLOAD * pair + MT_LL128_LINE_PAYLOAD * half) < nbytes;
      poff[k] = flag_lane ? MT_LL128_PAIR_PAYLOAD * pair + 112 + 8 * half : line_off + 16 * l;
    }
  }
  __device__ __forceinline__ int wire_off(int k) const { return (k * 4 + g) * MT_LL128_LINE + l * 16; }
};

// Payload -> registers in line layout (flag lanes leave v[2k+1] for the flag).
__device__ __forceinline__ void ll128_load_raw(const LL128Lane& L, const uint8_t* src, int nbytes, bool aligned,
                                               uint64_t* v) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    v[2 * k] = 0;
    v[2 * k + 1] = 0;
    if (L.need[k]) {
      if (L.flag_lane) ll128_load_piece<8>(src + L.poff[k], nbytes - L.poff[k], aligned, v[2 * k], v[2 * k + 1]);
      else ll128_load_piece<16>(src + L.poff[k], nbytes - L.poff[k], aligned, v[2 * k], v[2 * k + 1]);
    }
  }
}
__device__ __forceinline__ void ll128_store_raw(const LL128Lane& L, uint8_t* dst, int nbytes, bool aligned,
                                                const uint64_t* v) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (L.need[k]) {
      if (L.flag_lane) ll128_store_piece<8>(dst + L.poff[k], nbytes - L.poff[k], aligned, v[2 * k], 0);
      else ll128_store_piece<16>(dst + L.poff[k], nbytes - L.poff[k], aligned, v[2 * k], v[2 * k + 1]);
    }
  }
}
__device__ __forceinline__ void ll128_store_wire(const LL128Lane& L, uint8_t* wire, const uint64_t* v, uint64_t flag) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (L.need[k]) {
      u128 t;
      t.x = v[2 * k];
      t.y = L.flag_lane ? flag : v[2 * k + 1];
      store128(wire + L.wire_off(k), t);
    }
  }
}
// Poll the needed lines until every flag equals `flag`.  Warp-uniform result; on give-up lane 0 has
// recorded the error and raised *s_fail.
__device__ __forceinline__ bool ll128_poll_wire(const MtDevComm& c, const LL128Lane& L, const uint8_t* wire,
                                                uint64_t flag, uint64_t* v, int* s_fail, int ch, uint32_t where,
                                                uint64_t step) {
  const int lane = threadIdx.x & 31;
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (true) {
    bool bad = false;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (L.need[k]) {
        u128 t = load128(wire + L.wire_off(k));
        v[2 * k] = t.x;
        v[2 * k + 1] = t.y;
        if (L.flag_lane && t.y != flag) bad = true;
      }
    }
    if (!__any_sync(0xffffffffu, bad)) return true;
    ++spins;
    if ((spins & 0xffu) == 0u) {
      int giveup = 0;
      if (lane == 0) {
        if (abort_raised(c) || *(volatile int*)s_fail) {
          giveup = MT_ERR_REMOTE_ABORT;
        } else {
          uint64_t now = globaltimer();
          if (t0 == 0) t0 = now;
          else if (now - t0 > c.timeout_ns) giveup = MT_ERR_TIMEOUT_FLAG;
        }
      }
      giveup = __shfl_sync(0xffffffffu, giveup, 0);
      if (giveup) {
        if (lane == 0) {
          report_error(c, giveup, ch, where, flag, 0, step);
          atomicExch(s_fail, 1);
        }
        return false;
      }
    }
    if (spins > 32u) __nanosleep(20);
  }
}

template <class T, int NTHREADS>
struct LL128Prims {
  static constexpr int kProto = MT_PROTO_LL128;
  static constexpr int kWarps = NTHREADS / 32;
  const MtDevComm& c;
  const int ch;
  int* s_fail;
  int recv_peer, send_peer;
  uint8_t* recv_fifo;
  uint8_t* send_fifo;
  MtConnCtrl* recv_conn;
  MtConnCtrl* send_conn;
  uint64_t* recv_head_rem;
  uint64_t recv_step, send_step;
  uint32_t slots;
  uint64_t slot_bytes;

  __device__ LL128Prims(const MtDevComm& comm, int channel, int recvPeer, int sendPeer, int* sfail)
      : c(comm), ch(channel), s_fail(sfail), recv_peer(recvPeer), send_peer(sendPeer) {
    slots = c.L.fifo_slots[kProto];
    slot_bytes = c.L.fifo_slot_bytes[kProto];
    recv_step = send_step = 0;
    recv_fifo = send_fifo = nullptr;
    recv_conn = send_conn = nullptr;
    recv_head_rem = nullptr;
    if (recv_peer >= 0) {
      recv_fifo = c.heap[c.rank] + mt_fifo_off(c.L, kProto, c.nranks, ch, recv_peer);
      recv_conn = (MtConnCtrl*)(c.heap[c.rank] + mt_conn_off(c.L, kProto, c.nranks, ch, recv_peer));
      recv_head_rem = &((MtConnCtrl*)(c.heap[recv_peer] + mt_conn_off(c.L, kProto, c.nranks, ch, c.rank)))->head;
      recv_step = load64(&recv_conn->recv_step);
    }
    if (send_peer >= 0) {
      send_fifo = c.heap[send_peer] + mt_fifo_off(c.L, kProto, c.nranks, ch, c.rank);
      send_conn = (MtConnCtrl*)(c.heap[c.rank] + mt_conn_off(c.L, kProto, c.nranks, ch, send_peer));
      send_step = load64(&send_conn->send_step);
    }
    if (threadIdx.x == 0) *s_fail = 0;
    __syncthreads();
  }

  __device__ void finish() {
    __syncthreads();
    if (threadIdx.x == 0 && *s_fail == 0) {
      if (recv_peer >= 0) store64(&recv_conn->recv_step, recv_step);
      if (send_peer >= 0) store64(&send_conn->send_step, send_step);
    }
  }

  __device__ __forceinline__ uint64_t step_payload() const { return mt_slot_payload(kProto, slot_bytes); }

  // One warp chunk: up to 16 lines / 1920 payload bytes.  Returns false (warp-uniform) on give-up.
  template <bool RECV, bool SEND, bool SRC, bool DST>
  __device__ __forceinline__ bool chunk(const uint8_t* rwire, uint8_t* swire, const uint8_t* src, uint8_t* dst,
                                        int nbytes, uint64_t rflag, uint64_t sflag, bool src_al, bool dst_al) {
    const LL128Lane L(nbytes);
    uint64_t v[8];
    if (RECV) {
      if (!ll128_poll_wire(c, L, rwire, rflag, v, s_fail, ch, MT_WHERE_LL128_RECV, recv_step)) return false;
      if (SRC) {
        uint64_t r[8];
        ll128_load_raw(L, src, nbytes, src_al, r);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          v[2 * k] = sum64<T>(v[2 * k], r[2 * k]);
          if (!L.flag_lane) v[2 * k + 1] = sum64<T>(v[2 * k + 1], r[2 * k + 1]);
        }
      }
    } else {
      ll128_load_raw(L, src, nbytes, src_al, v);
    }
    if (SEND) ll128_store_wire(L, swire, v, sflag);
    if (DST) ll128_store_raw(L, dst, nbytes, dst_al, v);
    return true;
  }

  // One FIFO step of up to step_payload() bytes; same contract as SimplePrims::step.
  template <bool RECV, bool SEND, bool SRC, bool DST>
  __device__ __noinline__ bool step(const uint8_t* src, uint8_t* dst, uint64_t nbytes) {
    const int tid = threadIdx.x;
    if (SEND) {
      if (tid == 32) {
        const uint64_t want = send_step + 1;
        const uint64_t* w = &send_conn->head;
        const uint64_t nslots = slots;
        if (!bounded_wait(
                c, [&] { return load64_acquire_sys(w) + nslots >= want; }, MT_ERR_TIMEOUT_HEAD, ch,
                MT_WHERE_LL128_SEND, want, send_step, (const volatile uint64_t*)w))
          atomicExch(s_fail, 1);
      }
      __syncthreads();
      if (*s_fail) return false;
    }
    const uint8_t* rslot = RECV ? recv_fifo + (recv_step % slots) * slot_bytes : nullptr;
    uint8_t* sslot = SEND ? send_fifo + (send_step % slots) * slot_bytes : nullptr;
    const uint64_t rflag = recv_step + 1, sflag = send_step + 1;
    const bool src_al = ((uintptr_t)src & 15) == 0, dst_al = ((uintptr_t)dst & 15) == 0;
    const uint32_t nchunks = (uint32_t)mt_div_up(nbytes, MT_LL128_WARP_PAYLOAD);
    for (uint32_t wc = tid >> 5; wc < nchunks; wc += kWarps) {
      const uint64_t po = (uint64_t)wc * MT_LL128_WARP_PAYLOAD, wo = (uint64_t)wc * MT_LL128_WARP_WIRE;
      const uint64_t left = nbytes - po;
      const int nb = left < MT_LL128_WARP_PAYLOAD ? (int)left : MT_LL128_WARP_PAYLOAD;
      if (!chunk<RECV, SEND, SRC, DST>(RECV ? rslot + wo : nullptr, SEND ? sslot + wo : nullptr,
                                       src ? src + po : nullptr, dst ? dst + po : nullptr, nb, rflag, sflag, src_al,
                                       dst_al))
        break;
    }
    __syncthreads();
    if (*s_fail) return false;
    if (SEND) ++send_step;
    if (RECV) {
      ++recv_step;
      if (tid == 32) store64_release_sys(recv_head_rem, recv_step);
    }
    return true;
  }
};

}  // namespace mt
