// Host-side model of the cross-rank protocols of the fused GEMM + collective kernels (kernels/gemm_tc.cu,
// kernels/gemm_tc2.cu, kernels/gemm_fused_parts.cuh): threads stand for CTAs, std atomics for the
// system-scope loads, stores and reductions, stamps for the data.  The tile orders, the arrival counters
// (which only ever grow: call e waits for e x arrivals), the entry barrier of the comm CTAs, the ticketed
// reducers with their two alternating ticket words and the two alternating halves of the staging area are
// the ones of the kernels (the tile order is the kernels' own code, kernels/fused_schedule.h).  Every datum
// carries the number of the call that produced it, so a read that sees another call's data (a buffer reused
// too early) is reported, not just a deadlock.
//
// What it is for: schedules that cannot be forced on a GPU (one rank far ahead of another, reducers that
// stall) and failures that must not be provoked there (a rank that never starts).  The reference has no such
// kernels and no simulator (its self-tests need the GPUs, e.g. 6_allgather.py:186-200).
#include <stdint.h>
#include <string.h>

#include <atomic>
#include <chrono>
#include <random>
#include <thread>
#include <vector>

#include "../kernels/fused_schedule.h"

namespace {

using Clock = std::chrono::steady_clock;

struct Params {
  int op;      // 0 all-gather -> GEMM, 1 GEMM -> reduce-scatter
  int n;       // ranks
  int per;     // 128-row blocks per rank
  int nbs;     // column blocks
  int ngemm;   // GEMM CTAs (single-CTA kernels) or clusters (pair kernels) per rank
  int nextra;  // comm CTAs (op 0) or dedicated reducer CTAs (op 1) per rank
  int pair;    // 1: tiles of two row blocks (CTA pairs), each CTA handles its own block's flag / counter
  int iters;
  int dead_rank;      // >= 0: this rank never starts
  int slow_rank;      // >= 0: this rank's reducers (op 1) / GEMM CTAs (op 0) stall before they read
  int double_buffer;  // op 1: alternate between two halves of the staging area by the parity of the call
  uint64_t timeout_ms;
};

// The payload (gathered rows, partial tiles).  Normally atomics, so that the model itself has no undefined
// behaviour even when it demonstrates a protocol that reuses a buffer too early.  With MT_SIM_PLAIN_DATA the
// payload is plain memory: built with -fsanitize=thread, ThreadSanitizer then checks that the counters and
// barriers (the only atomics left) order every payload write before the reads that depend on it.
#ifdef MT_SIM_PLAIN_DATA
struct Datum {
  uint64_t v = 0;
  void store(uint64_t x, std::memory_order = std::memory_order_relaxed) { v = x; }
  uint64_t load(std::memory_order = std::memory_order_relaxed) const { return v; }
};
#else
using Datum = std::atomic<uint64_t>;
#endif

inline uint64_t stamp(uint64_t call, int rank, int block, int nb) {
  return (call << 32) | ((uint64_t)rank << 24) | ((uint64_t)block << 12) | (uint64_t)nb;
}

struct Rank {
  // all-gather -> GEMM
  std::vector<Datum> gathered;                  // [n][per]: rows of every source rank
  std::vector<std::atomic<uint64_t>> ag_cnt;    // [n][per]
  std::vector<std::atomic<uint64_t>> bar;       // [nextra][n]: entry barrier of comm CTA cc, slot of rank p
  // GEMM -> reduce-scatter
  std::vector<Datum> stage;                     // [2][n][per][nbs]
  std::vector<std::atomic<uint64_t>> rs_cnt;    // [n][per][nbs]
  std::atomic<uint64_t> tickets[2];
  std::vector<std::atomic<uint64_t>> out;       // [per][nbs]: call number of the last reduction
  std::atomic<uint64_t> reduced{0};
  // local "kernel boundary": all CTAs of call e are done before any of call e + 1 starts
  std::atomic<int> done_in_call{0};
  std::atomic<uint64_t> call_open{1};
};

struct World {
  Params p;
  std::vector<Rank> ranks;
  std::atomic<int> error{0};  // 1 wrong data, 2 a wait gave up
  std::atomic<int> abort_flag{0};
  explicit World(const Params& pp) : p(pp), ranks(pp.n) {}
};

struct Ctx {
  World* w;
  std::mt19937 rng;
  void jitter(int max_us = 30) {
    const uint32_t r = rng() % 8;
    if (r == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % max_us));
    else if (r < 3) std::this_thread::yield();
  }
  template <class Pred>
  bool wait(Pred pred) {
    const auto t0 = Clock::now();
    uint32_t spins = 0;
    while (!pred()) {
      if (w->abort_flag.load(std::memory_order_relaxed)) return false;
      if ((++spins & 0xff) == 0) {
        if (std::chrono::duration_cast<std::chrono::milliseconds>(Clock::now() - t0).count() > (long)w->p.timeout_ms) {
          int z = 0;
          w->error.compare_exchange_strong(z, 2);
          w->abort_flag.store(1);
          return false;
        }
        std::this_thread::yield();
      }
    }
    return true;
  }
  void bad_data() {
    int z = 0;
    w->error.compare_exchange_strong(z, 1);
    w->abort_flag.store(1);
  }
};

// ---- all-gather -> GEMM -----------------------------------------------------------------------------------
void ag_comm_cta(Ctx& c, int me, int cc, uint64_t e) {
  const Params& p = c.w->p;
  // entry barrier: every rank has entered call e, so nobody still reads the rows gathered by call e - 1
  for (int q = 0; q < p.n; ++q) c.w->ranks[q].bar[(size_t)cc * p.n + me].store(e, std::memory_order_release);
  for (int q = 0; q < p.n; ++q)
    if (!c.wait([&] { return c.w->ranks[me].bar[(size_t)cc * p.n + q].load(std::memory_order_acquire) >= e; })) return;
  for (int wk = cc; wk < p.per * (p.n - 1); wk += p.nextra) {
    const int peer = (me + 1 + wk / p.per) % p.n, ci = wk % p.per;
    c.jitter();
    Rank& r = c.w->ranks[peer];
    r.gathered[(size_t)me * p.per + ci].store(stamp(e, me, ci, 0), std::memory_order_relaxed);
    r.ag_cnt[(size_t)me * p.per + ci].fetch_add(1, std::memory_order_release);
  }
}

void ag_gemm_cta(Ctx& c, int me, int g, uint64_t e) {
  const Params& p = c.w->p;
  const int bpt = p.pair ? 2 : 1, per_t = p.per / bpt;
  const int tiles = p.n * per_t * p.nbs;
  for (int t = g; t < tiles; t += p.ngemm) {
    // the kernels' own tile order (128-row tiles, or 256-row tiles of a CTA pair)
    const MtTile tl = mt_fused_tile(MT_TILE_AG_GEMM, t, p.n * p.per * 128, p.nbs * 256, p.n, me, 0, 128 * bpt, 256);
    const int owner = tl.owner, j = tl.jb;
    if (owner != me) {
      for (int h = 0; h < bpt; ++h) {  // with pairs, each CTA of the pair waits for its own block
        const int blk = j * bpt + h;
        Rank& r = c.w->ranks[me];
        if (!c.wait([&] { return r.ag_cnt[(size_t)owner * p.per + blk].load(std::memory_order_acquire) >= e; })) return;
        if (me == p.slow_rank) std::this_thread::sleep_for(std::chrono::microseconds(200));
        if (r.gathered[(size_t)owner * p.per + blk].load(std::memory_order_relaxed) != stamp(e, owner, blk, 0)) return c.bad_data();
      }
    }
    c.jitter();
  }
}

// ---- GEMM -> reduce-scatter -------------------------------------------------------------------------------
void rs_reduce_loop(Ctx& c, int me, bool first_cta, uint64_t e) {
  const Params& p = c.w->p;
  Rank& r = c.w->ranks[me];
  const int buf = p.double_buffer ? (int)(e & 1) : 0;
  if (first_cta) r.tickets[(e + 1) & 1].store(0, std::memory_order_relaxed);  // next call's counter
  while (true) {
    const uint64_t ot = r.tickets[e & 1].fetch_add(1, std::memory_order_relaxed);
    if (ot >= (uint64_t)p.per * p.nbs) return;
    const int mbl = (int)(ot / p.nbs), nb = (int)(ot % p.nbs);
    for (int s = 0; s < p.n; ++s)
      if (!c.wait([&] { return r.rs_cnt[((size_t)s * p.per + mbl) * p.nbs + nb].load(std::memory_order_acquire) >= 4 * e; })) return;
    if (me == p.slow_rank) std::this_thread::sleep_for(std::chrono::microseconds(300));
    for (int s = 0; s < p.n; ++s) {
      const uint64_t v = r.stage[(((size_t)buf * p.n + s) * p.per + mbl) * p.nbs + nb].load(std::memory_order_relaxed);
      if (v != stamp(e, s, mbl, nb)) return c.bad_data();  // a partial tile of another call
    }
    if (r.out[(size_t)mbl * p.nbs + nb].exchange(e, std::memory_order_relaxed) != e - 1) return c.bad_data();  // once per call
    r.reduced.fetch_add(1, std::memory_order_relaxed);
  }
}

void rs_gemm_cta(Ctx& c, int me, int g, uint64_t e) {
  const Params& p = c.w->p;
  const int bpt = p.pair ? 2 : 1, per_t = p.per / bpt;
  const int tiles = p.n * per_t * p.nbs;
  const int buf = p.double_buffer ? (int)(e & 1) : 0;
  for (int t = g; t < tiles; t += p.ngemm) {
    const MtTile tl = mt_fused_tile(MT_TILE_GEMM_RS, t, p.n * p.per * 128, p.nbs * 256, p.n, me, 0, 128 * bpt, 256);
    const int nb = tl.nb, j = tl.jb, owner = tl.owner;
    c.jitter();
    Rank& r = c.w->ranks[owner];
    for (int h = 0; h < bpt; ++h) {
      const int blk = j * bpt + h;
      r.stage[(((size_t)buf * p.n + me) * p.per + blk) * p.nbs + nb].store(stamp(e, me, blk, nb), std::memory_order_relaxed);
      for (int q = 0; q < 4; ++q)  // the four epilogue warps
        r.rs_cnt[((size_t)me * p.per + blk) * p.nbs + nb].fetch_add(1, std::memory_order_release);
    }
  }
  rs_reduce_loop(c, me, g == 0, e);
}

void cta_thread(World* w, int me, int idx, uint32_t seed) {
  Ctx c{w, std::mt19937(seed)};
  const Params& p = w->p;
  Rank& r = w->ranks[me];
  const int nthreads = p.ngemm + p.nextra;
  for (uint64_t e = 1; e <= (uint64_t)p.iters && !w->abort_flag.load(); ++e) {
    // kernel boundary: wait until this rank has opened call e
    if (!c.wait([&] { return r.call_open.load(std::memory_order_acquire) >= e; })) return;
    if (p.op == 0) {
      if (idx < p.ngemm) ag_gemm_cta(c, me, idx, e);
      else ag_comm_cta(c, me, idx - p.ngemm, e);
    } else {
      if (idx < p.ngemm) rs_gemm_cta(c, me, idx, e);
      else rs_reduce_loop(c, me, false, e);
    }
    if (r.done_in_call.fetch_add(1, std::memory_order_acq_rel) + 1 == nthreads) {
      // last CTA of the call: checks, then the next launch may start
      if (p.op == 1 && !w->abort_flag.load() && r.reduced.load() != e * (uint64_t)p.per * p.nbs) c.bad_data();
      r.done_in_call.store(0, std::memory_order_relaxed);
      r.call_open.store(e + 1, std::memory_order_release);
    }
  }
}

}  // namespace

extern "C" {

// The kernels' tile order, for tests of its coverage: out = {row block, column block, owner, row block in owner}.
void mt_sched_fused_tile(int mode, int t, int M, int N, int nranks, int rank, int raster, int tile_rows, int tile_cols,
                         int* out) {
  const MtTile c = mt_fused_tile(mode, t, M, N, nranks, rank, raster, tile_rows, tile_cols);
  out[0] = c.mb;
  out[1] = c.nb;
  out[2] = c.owner;
  out[3] = c.jb;
}

// Runs `iters` back-to-back calls of one fused op on a simulated world.  op: 0 all-gather -> GEMM, 1 GEMM ->
// reduce-scatter.  Returns 0 ok, 1 a CTA read data of another call (or a tile was reduced twice / not at all),
// 2 a wait gave up (e.g. `dead_rank` never started), -1 bad argument.
int mt_sim_fused(int op, int nranks, int per, int nbs, int ngemm, int nextra, int pair, int iters, uint32_t seed,
                 int dead_rank, int slow_rank, int double_buffer, uint64_t timeout_ms) {
  if (op < 0 || op > 1 || nranks < 1 || nranks > 16 || per < 1 || nbs < 1 || ngemm < 1 || nextra < 0 || iters < 1) return -1;
  if (pair && per % 2) return -1;
  if (op == 0 && nranks > 1 && nextra < 1) return -1;
  Params p{op, nranks, per, nbs, ngemm, nextra, pair, iters, dead_rank, slow_rank, double_buffer, timeout_ms ? timeout_ms : 2000};
  World w(p);
  for (auto& r : w.ranks) {
    r.gathered = std::vector<Datum>((size_t)nranks * per);
    r.ag_cnt = std::vector<std::atomic<uint64_t>>((size_t)nranks * per);
    r.bar = std::vector<std::atomic<uint64_t>>((size_t)(nextra > 0 ? nextra : 1) * nranks);
    r.stage = std::vector<Datum>((size_t)2 * nranks * per * nbs);
    r.rs_cnt = std::vector<std::atomic<uint64_t>>((size_t)nranks * per * nbs);
    r.out = std::vector<std::atomic<uint64_t>>((size_t)per * nbs);
    for (auto* v : {&r.ag_cnt, &r.bar, &r.rs_cnt, &r.out})
      for (auto& x : *v) x.store(0);
    for (auto* v : {&r.gathered, &r.stage})
      for (auto& x : *v) x.store(0);
    r.tickets[0].store(0);
    r.tickets[1].store(0);
  }
  std::vector<std::thread> ts;
  std::mt19937 seeder(seed);
  for (int me = 0; me < nranks; ++me) {
    if (me == dead_rank) continue;
    for (int idx = 0; idx < ngemm + nextra; ++idx) ts.emplace_back(cta_thread, &w, me, idx, (uint32_t)seeder());
  }
  for (auto& t : ts) t.join();
  return w.error.load();
}

}  // extern "C"

#ifdef MT_SIM_MAIN
// Stand-alone driver (used for the ThreadSanitizer build): the arguments of mt_sim_fused in order.
#include <stdlib.h>
int main(int argc, char** argv) {
  if (argc != 14) return 64;
  long v[13];
  for (int i = 0; i < 13; ++i) v[i] = atol(argv[i + 1]);
  return mt_sim_fused((int)v[0], (int)v[1], (int)v[2], (int)v[3], (int)v[4], (int)v[5], (int)v[6], (int)v[7], (uint32_t)v[8],
                      (int)v[9], (int)v[10], (int)v[11], (uint64_t)v[12]);
}
#endif
