// Host-side simulator of the ring / chain protocols: one thread per (rank, channel) runs the SAME
// schedule code as the GPU kernels (kernels/ring_schedule.h) over FIFOs, step counters, credits and
// LL128 lines laid out exactly as in a real heap (device/sched.h), with std atomics in place of
// ld/st.acquire/release.  It proves properties that must not be probed on a shared GPU:
//   * no deadlock at 2/4/8 ranks over many back-to-back operations with random scheduling jitter;
//   * flags and counters that grow across operations never match stale data;
//   * a rank that never shows up makes every waiting rank give up after its time limit with an error
//     record (fault injection on the host), instead of spinning forever as the reference's waits do
//     (protocol.py:115,127,177).
#include <string.h>

#include <atomic>
#include <chrono>
#include <cmath>
#include <random>
#include <thread>
#include <vector>

#include "../device/sched.h"
#include "../kernels/ring_schedule.h"
#include "../mintccl.h"

namespace mt {

struct SimF32 {
  using elem = float;
};

static inline uint64_t ld_acq(const uint64_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
static inline void st_rel(uint64_t* p, uint64_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
static inline uint32_t ld_acq32(const uint32_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }

struct SimEnv {
  int jitter_us = 0;
  uint64_t timeout_ns = 2000000000ull;
};
static thread_local SimEnv* t_env = nullptr;
static thread_local std::mt19937* t_rng = nullptr;

static void jitter() {
  if (t_env && t_env->jitter_us > 0 && ((*t_rng)() & 7) == 0)
    std::this_thread::sleep_for(std::chrono::microseconds((*t_rng)() % (t_env->jitter_us + 1)));
}

static void sim_report(const MtDevComm& c, uint32_t code, uint32_t ch, uint32_t where, uint64_t expected, uint64_t seen,
                       uint64_t step) {
  MtStatus* st = (MtStatus*)(c.heap[c.rank] + c.L.status_off);
  uint32_t zero = 0;
  if (__atomic_compare_exchange_n(&st->code, &zero, code, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE)) {
    st->rank = c.rank;
    st->channel = ch;
    st->where = where;
    st->expected = expected;
    st->seen = seen;
    st->step = step;
  }
  for (int p = 0; p < c.nranks; ++p)
    __atomic_store_n(&((MtStatus*)(c.heap[p] + c.L.status_off))->abort, 1u, __ATOMIC_RELEASE);
}

template <class Pred>
static bool sim_wait(const MtDevComm& c, Pred pred, uint32_t code, uint32_t ch, uint32_t where, uint64_t expected,
                     uint64_t step, const uint64_t* seen) {
  auto t0 = std::chrono::steady_clock::now();
  uint32_t spins = 0;
  while (!pred()) {
    if ((++spins & 0x3f) == 0) {
      if (ld_acq32(&((MtStatus*)(c.heap[c.rank] + c.L.status_off))->abort)) {
        sim_report(c, MT_ERR_REMOTE_ABORT, ch, where, expected, seen ? ld_acq(seen) : 0, step);
        return false;
      }
      auto dt = std::chrono::steady_clock::now() - t0;
      if ((uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(dt).count() > c.timeout_ns) {
        sim_report(c, code, ch, where, expected, seen ? ld_acq(seen) : 0, step);
        return false;
      }
      std::this_thread::yield();
    }
  }
  return true;
}

// Shared connection bookkeeping of both host protocols (same fields and addresses as the device classes).
template <int PROTO>
struct HostConn {
  const MtDevComm& c;
  const int ch;
  int* s_fail;
  int recv_peer, send_peer;
  uint8_t *recv_fifo = nullptr, *send_fifo = nullptr;
  MtConnCtrl *recv_conn = nullptr, *send_conn = nullptr;
  uint64_t *recv_head_rem = nullptr, *send_tail_rem = nullptr;
  uint64_t recv_step = 0, send_step = 0;
  uint32_t slots;
  uint64_t slot_bytes;
  HostConn(const MtDevComm& comm, int channel, int rp, int sp, int* sf)
      : c(comm), ch(channel), s_fail(sf), recv_peer(rp), send_peer(sp) {
    slots = c.L.fifo_slots[PROTO];
    slot_bytes = c.L.fifo_slot_bytes[PROTO];
    if (recv_peer >= 0) {
      recv_fifo = c.heap[c.rank] + mt_fifo_off(c.L, PROTO, c.nranks, ch, recv_peer);
      recv_conn = (MtConnCtrl*)(c.heap[c.rank] + mt_conn_off(c.L, PROTO, c.nranks, ch, recv_peer));
      recv_head_rem = &((MtConnCtrl*)(c.heap[recv_peer] + mt_conn_off(c.L, PROTO, c.nranks, ch, c.rank)))->head;
      recv_step = recv_conn->recv_step;
    }
    if (send_peer >= 0) {
      send_fifo = c.heap[send_peer] + mt_fifo_off(c.L, PROTO, c.nranks, ch, c.rank);
      send_conn = (MtConnCtrl*)(c.heap[c.rank] + mt_conn_off(c.L, PROTO, c.nranks, ch, send_peer));
      send_tail_rem = &((MtConnCtrl*)(c.heap[send_peer] + mt_conn_off(c.L, PROTO, c.nranks, ch, c.rank)))->tail;
      send_step = send_conn->send_step;
    }
    *s_fail = 0;
  }
  void finish() {
    if (*s_fail == 0) {
      if (recv_peer >= 0) recv_conn->recv_step = recv_step;
      if (send_peer >= 0) send_conn->send_step = send_step;
    }
  }
  bool wait_credit(uint32_t where) {
    const uint64_t want = send_step + 1, nslots = slots;
    const uint64_t* w = &send_conn->head;
    if (!sim_wait(c, [&] { return ld_acq(w) + nslots >= want; }, MT_ERR_TIMEOUT_HEAD, ch, where, want, send_step, w)) {
      *s_fail = 1;
      return false;
    }
    return true;
  }
};

template <class T, int NTHREADS>
struct HostSimple : HostConn<MT_PROTO_SIMPLE> {
  using HostConn<MT_PROTO_SIMPLE>::HostConn;
  uint64_t step_payload() const { return slot_bytes; }
  template <bool RECV, bool SEND, bool SRC, bool DST>
  bool step(const uint8_t* src, uint8_t* dst, uint64_t nbytes) {
    jitter();
    if (RECV) {
      const uint64_t want = recv_step + 1;
      const uint64_t* w = &recv_conn->tail;
      if (!sim_wait(c, [&] { return ld_acq(w) >= want; }, MT_ERR_TIMEOUT_TAIL, ch, MT_WHERE_SIMPLE_RECV, want, recv_step, w)) {
        *s_fail = 1;
        return false;
      }
    }
    if (SEND && !wait_credit(MT_WHERE_SIMPLE_SEND)) return false;
    const uint8_t* rslot = RECV ? recv_fifo + (recv_step % slots) * slot_bytes : nullptr;
    uint8_t* sslot = SEND ? send_fifo + (send_step % slots) * slot_bytes : nullptr;
    const uint64_t nel = nbytes / sizeof(float);
    for (uint64_t i = 0; i < nel; ++i) {
      float v;
      if (RECV) {
        memcpy(&v, rslot + 4 * i, 4);
        if (SRC) {
          float s;
          memcpy(&s, src + 4 * i, 4);
          v += s;
        }
      } else {
        memcpy(&v, src + 4 * i, 4);
      }
      if (SEND) memcpy(sslot + 4 * i, &v, 4);
      if (DST) memcpy(dst + 4 * i, &v, 4);
    }
    jitter();
    if (SEND) st_rel(send_tail_rem, ++send_step);
    if (RECV) st_rel(recv_head_rem, ++recv_step);
    return true;
  }
};

template <class T, int NTHREADS>
struct HostLL128 : HostConn<MT_PROTO_LL128> {
  using HostConn<MT_PROTO_LL128>::HostConn;
  uint64_t step_payload() const { return mt_slot_payload(MT_PROTO_LL128, slot_bytes); }

  // Payload byte range carried by line (pair, half) of a chunk with `nb` payload bytes: two pieces.
  static void pieces(int pair, int half, int& a_off, int& a_len, int& b_off) {
    a_off = MT_LL128_PAIR_PAYLOAD * pair + 128 * half;  // 112 bytes for lanes 0..6
    a_len = 112;
    b_off = MT_LL128_PAIR_PAYLOAD * pair + 112 + 8 * half;  // 8 bytes in the flag lane
  }

  template <bool RECV, bool SEND, bool SRC, bool DST>
  bool step(const uint8_t* src, uint8_t* dst, uint64_t nbytes) {
    jitter();
    if (SEND && !wait_credit(MT_WHERE_LL128_SEND)) return false;
    const uint8_t* rslot = RECV ? recv_fifo + (recv_step % slots) * slot_bytes : nullptr;
    uint8_t* sslot = SEND ? send_fifo + (send_step % slots) * slot_bytes : nullptr;
    const uint64_t rflag = recv_step + 1, sflag = send_step + 1;
    const uint64_t nchunks = mt_div_up(nbytes, MT_LL128_WARP_PAYLOAD);
    for (uint64_t wc = 0; wc < nchunks; ++wc) {
      const uint64_t po = wc * MT_LL128_WARP_PAYLOAD, wo = wc * MT_LL128_WARP_WIRE;
      const int nb = (int)mt_min64(MT_LL128_WARP_PAYLOAD, nbytes - po);
      const int nlines = (int)mt_ll128_wire_lines(nb);
      for (int li = 0; li < nlines; ++li) {
        const int pair = li / 2, half = li % 2;
        const uint32_t line = mt_ll128_line_of(pair, half);
        uint8_t payload[120];
        memset(payload, 0, sizeof(payload));
        int a_off, a_len, b_off;
        pieces(pair, half, a_off, a_len, b_off);
        auto clip = [&](int off, int len) { return off >= nb ? 0 : (off + len > nb ? nb - off : len); };
        const int la = clip(a_off, a_len), lb = clip(b_off, 8);
        if (RECV) {
          const uint8_t* w = rslot + wo + (uint64_t)line * MT_LL128_LINE;
          const uint64_t* fw = (const uint64_t*)(w + 120);
          if (!sim_wait(c, [&] { return ld_acq(fw) == rflag; }, MT_ERR_TIMEOUT_FLAG, ch, MT_WHERE_LL128_RECV, rflag, recv_step, fw)) {
            *s_fail = 1;
            return false;
          }
          memcpy(payload, w, 120);  // wire bytes [0,112) = piece a, [112,120) = piece b
          if (SRC) {
            for (int i = 0; i + 4 <= la; i += 4) {
              float x, y;
              memcpy(&x, payload + i, 4);
              memcpy(&y, src + po + a_off + i, 4);
              x += y;
              memcpy(payload + i, &x, 4);
            }
            for (int i = 0; i + 4 <= lb; i += 4) {
              float x, y;
              memcpy(&x, payload + 112 + i, 4);
              memcpy(&y, src + po + b_off + i, 4);
              x += y;
              memcpy(payload + 112 + i, &x, 4);
            }
          }
        } else {
          if (la) memcpy(payload, src + po + a_off, la);
          if (lb) memcpy(payload + 112, src + po + b_off, lb);
        }
        if (SEND) {
          uint8_t* w = sslot + wo + (uint64_t)line * MT_LL128_LINE;
          memcpy(w, payload, 120);
          st_rel((uint64_t*)(w + 120), sflag);  // flag last: the line is valid once the flag is seen
        }
        if (DST) {
          if (la) memcpy(dst + po + a_off, payload, la);
          if (lb) memcpy(dst + po + b_off, payload + 112, lb);
        }
      }
      jitter();
    }
    if (SEND) ++send_step;
    if (RECV) st_rel(recv_head_rem, ++recv_step);
    return true;
  }
};

}  // namespace mt

extern "C" {

// Geometry helpers exported for the Python tests of the shared index arithmetic.
void mt_sched_split(uint64_t total, uint32_t parts, uint32_t idx, uint64_t align, uint64_t* lo, uint64_t* hi) {
  MtRange r = mt_split(total, parts, idx, align);
  *lo = r.lo;
  *hi = r.hi;
}
uint64_t mt_sched_ll128_lines(uint64_t payload) { return mt_ll128_wire_lines(payload); }
uint32_t mt_sched_ll128_line_of(uint32_t pair, uint32_t half) { return mt_ll128_line_of(pair, half); }
int mt_sched_ag_shard(int q, int j, int n) { return mt_ag_shard_pos(q, j, n); }
int mt_sched_rs_shard(int q, int j, int n) { return mt_rs_shard_pos(q, j, n); }
uint64_t mt_sched_layout_user_off(int nranks, uint32_t nch, uint64_t ssb, uint32_t ss, uint64_t lsb, uint32_t ls,
                                  uint64_t llb, uint64_t scratch) {
  return mt_make_layout(nranks, nch, ssb, ss, lsb, ls, llb, scratch, 0).user_off;
}

// Runs `iters` back-to-back operations of one collective on a simulated world and checks every result.
// op: ring op codes (0 sendrecv .. 5 allreduce); proto: 0 Simple, 1 LL128; count: fp32 elements (per shard
// for all-gather / reduce-scatter).  dead_rank >= 0: that rank never starts (fault injection).
// Returns 0 ok, 1 wrong data, 2 a wait gave up (statuses copied to status_out[nranks]), -1 bad argument.
int mt_sim_run(int nranks, int nchannels, int proto, int op, uint64_t count, int root, int spatial, const int* chain,
               int chain_len, const int* ring, int iters, int jitter_us, int dead_rank, int timeout_ms, uint32_t seed,
               uint64_t slot_bytes, uint32_t slots, MtStatus* status_out) {
  using namespace mt;
  if (nranks < 1 || nranks > MT_MAX_RANKS || nchannels < 1 || nchannels > MT_MAX_CHANNELS) return -1;
  const uint64_t ll_slot = mt_round_up(slot_bytes, MT_LL128_WARP_WIRE);
  MtHeapLayout L = mt_make_layout(nranks, nchannels, mt_round_up(slot_bytes, 128), slots, ll_slot, slots, 2048, 0, 0);
  const uint64_t heap_bytes = L.user_off;
  std::vector<std::vector<uint64_t>> heaps(nranks, std::vector<uint64_t>(heap_bytes / 8 + 1, 0));
  std::vector<MtDevComm> comms(nranks);
  for (int r = 0; r < nranks; ++r) {
    MtDevComm& d = comms[r];
    memset(&d, 0, sizeof(d));
    d.rank = r;
    d.nranks = nranks;
    d.timeout_ns = (uint64_t)timeout_ms * 1000000ull;
    d.L = L;
    for (int p = 0; p < nranks; ++p) d.heap[p] = (uint8_t*)heaps[p].data();
    for (int i = 0; i < nranks; ++i) {
      d.ring[i] = ring ? ring[i] : i;
      if (d.ring[i] == r) d.ring_pos = i;
    }
  }
  const bool shard_op = op == OP_ALLGATHER || op == OP_REDUCESCATTER;
  const uint64_t in_elems = op == OP_REDUCESCATTER ? count * nranks : count;
  const uint64_t out_elems = op == OP_ALLGATHER ? count * nranks : count;
  std::vector<std::vector<float>> in(nranks, std::vector<float>(in_elems + 4)), out(nranks, std::vector<float>(out_elems + 4));
  SimEnv env;
  env.jitter_us = jitter_us;
  int rc = 0;
  for (int it = 0; it < iters && rc == 0; ++it) {
    for (int r = 0; r < nranks; ++r) {
      std::mt19937 g(seed + 1000003u * it + r);
      for (auto& v : in[r]) v = (float)((int)(g() % 2001) - 1000) / 64.0f;  // exact in fp32 sums
      for (auto& v : out[r]) v = -12345.f;
    }
    RingArgs a;
    memset(&a, 0, sizeof(a));
    a.nbytes = count * 4;
    a.op = op;
    a.root = root;
    if (proto == MT_PROTO_SIMPLE && (op == OP_SENDRECV || op == OP_BROADCAST || op == OP_REDUCE))
      a.step_bytes = mt_chain_step_bytes(a.nbytes / (uint64_t)nchannels, slot_bytes, op == OP_SENDRECV ? chain_len : nranks);  // the same rule as mt_ring
    a.spatial = spatial;
    a.chain_len = chain_len;
    for (int i = 0; i < chain_len; ++i) a.chain[i] = chain[i];
    a.elem_size = 4;
    std::vector<std::thread> threads;
    for (int r = 0; r < nranks; ++r) {
      if (r == dead_rank) continue;
      for (int ch = 0; ch < nchannels; ++ch) {
        threads.emplace_back([&, r, ch] {
          std::mt19937 rng(seed * 7919u + r * 131u + ch + it * 17u);
          t_rng = &rng;
          t_env = &env;
          RingArgs mine = a;
          // in-place conventions of the public API: AG input is row `rank` of out unless given separately
          mine.in[0] = in[r].data();
          mine.out[0] = out[r].data();
          int s_fail = 0;
          if (proto == MT_PROTO_LL128) ring_body<HostLL128, SimF32, 1>(comms[r], mine, 0, ch, nchannels, &s_fail);
          else ring_body<HostSimple, SimF32, 1>(comms[r], mine, 0, ch, nchannels, &s_fail);
          t_rng = nullptr;  // they point into this frame
          t_env = nullptr;
        });
      }
    }
    for (auto& t : threads) t.join();
    for (int r = 0; r < nranks; ++r) {
      MtStatus* st = (MtStatus*)(comms[r].heap[r] + L.status_off);
      if (status_out) status_out[r] = *st;
      if (st->code != 0 || st->abort != 0) rc = 2;
    }
    if (rc) break;
    // verify
    auto sum_at = [&](uint64_t i) {
      float s = 0.f;
      for (int r = 0; r < nranks; ++r) s += in[r][i];
      return s;
    };
    for (int r = 0; r < nranks && rc == 0; ++r) {
      for (uint64_t i = 0; i < out_elems && rc == 0; ++i) {
        float want = -12345.f;
        switch (op) {
          case OP_SENDRECV: want = (r == chain[chain_len - 1]) ? in[chain[0]][i] : -12345.f; break;
          case OP_BROADCAST: want = in[root][i]; break;
          case OP_REDUCE: want = (r == root) ? sum_at(i) : -12345.f; break;
          case OP_ALLGATHER: want = in[i / count][i % count]; break;
          case OP_REDUCESCATTER: want = sum_at((uint64_t)r * count + i); break;
          case OP_ALLREDUCE: want = sum_at(i); break;
        }
        if (std::fabs(out[r][i] - want) > 1e-3f) rc = 1;
      }
    }
    (void)shard_op;
  }
  return rc;
}

}  // extern "C"

#ifdef MT_SIM_MAIN
// Stand-alone driver (used for the ThreadSanitizer build):
//   sim ranks channels proto op count root spatial iters jitter_us slot_bytes slots [chain ranks ...]
#include <stdlib.h>
int main(int argc, char** argv) {
  if (argc < 12) return 64;
  long v[11];
  for (int i = 0; i < 11; ++i) v[i] = atol(argv[i + 1]);
  int chain[MT_MAX_RANKS + 1];
  int chain_len = 0;
  for (int i = 12; i < argc && chain_len <= MT_MAX_RANKS; ++i) chain[chain_len++] = atoi(argv[i]);
  return mt_sim_run((int)v[0], (int)v[1], (int)v[2], (int)v[3], (uint64_t)v[4], (int)v[5], (int)v[6], chain_len ? chain : nullptr,
                    chain_len, nullptr, (int)v[7], (int)v[8], -1, 8000, 1u, (uint64_t)v[9], (uint32_t)v[10], nullptr);
}
#endif
