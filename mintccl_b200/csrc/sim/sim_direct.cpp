// Host-side model of the one-hop ("direct") collectives (kernels/direct_engine.cuh) and of the one-shot
// low-latency all-reduce (kernels/p2p_engine.cuh): threads stand for CTAs, std atomics for the system-scope
// flag loads and stores, and the payload is plain memory when built with MT_SIM_PLAIN_DATA, so that
// ThreadSanitizer checks the happens-before edges the protocols rely on.
//
//   direct ops   every CTA i of every rank meets CTA i of the other ranks in a barrier (one slot per CTA index:
//                rank r stores its call number into arrive[r] of every peer's slot and waits for all arrive[]
//                of its own) BEFORE touching peer memory and again AFTER its last access; between the two it
//                reads and writes slices of the peers' symmetric buffers.  Calls follow each other back to
//                back on the same buffers, in place, and the "user" rewrites its input between calls.
//   rooted sum   reduce with a summing root (rooted_reduce_kernel): between the two barriers every rank but the root sums
//                its own slice over the ranks that are not the root, stores the partial sum into the root's output,
//                chunk by chunk, and raises a counter in the root's barrier slot; the root waits for each counter and
//                adds its own input to that chunk.  The counters are tagged with the slot's barrier epoch, so they
//                are never cleared and an older call's value cannot satisfy a wait.  The root changes from call to call.
//   one-shot     no barrier: every rank stores its lines, tagged with the call number, into the peers' staging
//                area of that call's parity and polls its own area until the tag matches.
//
// The checks: every value read must carry the stamp of the call and rank it is expected from; a wait gives up
// after its time limit (a rank that never starts).  `exit_barrier = 0` drops the second barrier and shows why
// it is there: a rank that returns early lets its user overwrite data a slower peer still reads.
//
// The reference has neither these algorithms nor a model (its collectives are rings, README.md:53-55).
#include <stdint.h>
#include <string.h>

#include <atomic>
#include <chrono>
#include <random>
#include <thread>
#include <vector>

namespace {

using Clock = std::chrono::steady_clock;

#ifdef MT_SIM_PLAIN_DATA
struct Datum {
  uint64_t v = 0;
  void store(uint64_t x) { v = x; }
  uint64_t load() const { return v; }
};
#else
struct Datum {
  std::atomic<uint64_t> v{0};
  void store(uint64_t x) { v.store(x, std::memory_order_relaxed); }
  uint64_t load() const { return v.load(std::memory_order_relaxed); }
};
#endif

enum Op { AR_TWO_SHOT = 0, ALLGATHER = 1, REDUCESCATTER = 2, ALLTOALL = 3, LL_ONESHOT = 4, REDUCE_SUMMING_ROOT = 5, NUM_OPS = 6 };
constexpr int kChunks = 3;   // chunks per sub-slice in the rooted sum

struct Params {
  int n, nctas, iters, slow_rank, dead_rank, exit_barrier;
  uint64_t timeout_ms;
};

inline uint64_t stamp(uint64_t call, int rank, int slice, int part) {
  return (call << 32) | ((uint64_t)rank << 24) | ((uint64_t)slice << 12) | (uint64_t)part;
}

struct Rank {
  std::vector<Datum> buf;                       // symmetric buffer [n slices][nctas parts]
  std::vector<Datum> out;                       // second symmetric buffer (all-gather / all-to-all output)
  std::vector<std::atomic<uint64_t>> arrive;    // barrier slots [nctas][n]
  std::vector<uint64_t> bar_epoch;              // [nctas], private to the CTA that owns the slot
  std::vector<std::atomic<uint64_t>> xflag;     // chunk counters of the rooted sum [nctas][n]: [.][q] is written by rank q
  std::vector<Datum> rout;                      // the root's output of the rooted sum [n slices][nctas parts][kChunks]
  std::vector<std::atomic<uint64_t>> ll;        // one-shot area [2 parities][n sources][nctas]: the stamp is the flag
  std::vector<uint64_t> ll_epoch;               // [nctas]
  std::atomic<int> done_in_call{0};
  std::atomic<uint64_t> call_open{1};
};

struct World {
  Params p;
  std::vector<Rank> ranks;
  std::vector<int> ops;  // operation of every call (the same on all ranks)
  std::atomic<int> error{0}, abort_flag{0};
  explicit World(const Params& pp) : p(pp), ranks(pp.n) {}
};

struct Ctx {
  World* w;
  std::mt19937 rng;
  void jitter() {
    const uint32_t r = rng() % 8;
    if (r == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 30));
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
  bool bad() {
    int z = 0;
    w->error.compare_exchange_strong(z, 1);
    w->abort_flag.store(1);
    return false;
  }
};

// The cross-rank barrier of CTA `cta`: same words and orderings as rank_barrier in device/prims.cuh.
bool rank_barrier(Ctx& c, int me, int cta) {
  const Params& p = c.w->p;
  Rank& mine = c.w->ranks[me];
  const uint64_t e = mine.bar_epoch[cta] + 1;
  for (int q = 0; q < p.n; ++q) c.w->ranks[q].arrive[(size_t)cta * p.n + me].store(e, std::memory_order_release);
  for (int q = 0; q < p.n; ++q)
    if (!c.wait([&] { return mine.arrive[(size_t)cta * p.n + q].load(std::memory_order_acquire) >= e; })) return false;
  mine.bar_epoch[cta] = e;
  return true;
}

// One CTA of one direct collective, call number e.  Slice s of a buffer belongs to rank s; part `cta` of every
// slice is handled by CTA `cta` (the kernels split every range over the CTAs the same way on all ranks).
bool direct_cta(Ctx& c, int me, int cta, int op, uint64_t e) {
  const Params& p = c.w->p;
  const int n = p.n, nc = p.nctas;
  auto at = [&](int slice) { return (size_t)slice * nc + cta; };
  if (!rank_barrier(c, me, cta)) return false;  // every rank has entered the call: inputs are final, old readers gone
  if (me == p.slow_rank) std::this_thread::sleep_for(std::chrono::microseconds(150));
  c.jitter();
  switch (op) {
    case AR_TWO_SHOT:
      // sum my slice over all ranks (pull), store the result into everybody's buffer, in place
      for (int q = 0; q < n; ++q)
        if (c.w->ranks[q].buf[at(me)].load() != stamp(e, q, me, cta)) return c.bad();
      c.jitter();
      for (int q = 0; q < n; ++q) c.w->ranks[q].buf[at(me)].store(stamp(e, n + me, me, cta));  // "sum", written by owner
      break;
    case ALLGATHER:
      // push my contribution (slice `me` of my buffer) into slice `me` of everybody's output
      for (int q = 0; q < n; ++q) c.w->ranks[q].out[at(me)].store(c.w->ranks[me].buf[at(me)].load());
      break;
    case REDUCESCATTER:
      // pull slice `me` of everybody's buffer, keep the sum locally
      for (int q = 0; q < n; ++q)
        if (c.w->ranks[q].buf[at(me)].load() != stamp(e, q, me, cta)) return c.bad();
      break;
    case ALLTOALL:
      // slice q of my buffer goes to slice `me` of rank q's output
      for (int q = 0; q < n; ++q) c.w->ranks[q].out[at(me)].store(c.w->ranks[me].buf[at(q)].load());
      break;
    case REDUCE_SUMMING_ROOT: {
      const int root = (int)(e % (uint64_t)n);
      const uint64_t tag = c.w->ranks[me].bar_epoch[cta] << 24;   // the same on every rank after the entry barrier
      auto ro = [&](int slice, int k) { return ((size_t)slice * nc + cta) * kChunks + k; };
      if (n == 1) break;
      if (me != root) {
        for (int k = 0; k < kChunks; ++k) {
          // sum my slice over the ranks that are not the root (the root's memory is never read)
          for (int q = 0; q < n; ++q)
            if (q != root && c.w->ranks[q].buf[at(me)].load() != stamp(e, q, me, cta)) return c.bad();
          c.w->ranks[root].rout[ro(me, k)].store(stamp(e, n + me, me, cta) + (uint64_t)k * 7);   // the partial sum
          c.jitter();
          c.w->ranks[root].xflag[(size_t)cta * n + me].store(tag + k + 1, std::memory_order_release);
        }
      } else {
        for (int k = 0; k < kChunks; ++k)
          for (int q = 0; q < n; ++q) {
            if (q == root) continue;
            const std::atomic<uint64_t>& f = c.w->ranks[root].xflag[(size_t)cta * n + q];
            if (!c.wait([&] { return f.load(std::memory_order_acquire) >= tag + k + 1; })) return false;
            if (c.w->ranks[root].rout[ro(q, k)].load() != stamp(e, n + q, q, cta) + (uint64_t)k * 7) return c.bad();
            if (c.w->ranks[root].buf[at(q)].load() != stamp(e, root, q, cta)) return c.bad();   // my own input
            c.w->ranks[root].rout[ro(q, k)].store(stamp(e, 2 * n + q, q, cta) + (uint64_t)k * 7);   // the sum
          }
      }
      break;
    }
    default: break;
  }
  c.jitter();
  // nobody returns (and lets its user touch the buffers) before every rank has finished reading and writing
  if (p.exit_barrier && !rank_barrier(c, me, cta)) return false;
  // the results this rank may look at after the call
  switch (op) {
    case AR_TWO_SHOT:
      if (!p.exit_barrier) break;  // without the barrier other slices may not be there yet
      for (int s = 0; s < n; ++s)
        if (c.w->ranks[me].buf[at(s)].load() != stamp(e, n + s, s, cta)) return c.bad();
      break;
    case ALLGATHER:
      if (!p.exit_barrier) break;
      for (int s = 0; s < n; ++s)
        if (c.w->ranks[me].out[at(s)].load() != stamp(e, s, s, cta)) return c.bad();
      break;
    case ALLTOALL:
      if (!p.exit_barrier) break;
      for (int s = 0; s < n; ++s)
        if (c.w->ranks[me].out[at(s)].load() != stamp(e, s, me, cta)) return c.bad();
      break;
    case REDUCE_SUMMING_ROOT: {
      const int root = (int)(e % (uint64_t)n);
      if (me != root) break;
      for (int q = 0; q < n; ++q)
        for (int k = 0; q != root && k < kChunks; ++k)
          if (c.w->ranks[me].rout[(((size_t)q * nc + cta) * kChunks) + k].load() != stamp(e, 2 * n + q, q, cta) + (uint64_t)k * 7)
            return c.bad();
      break;
    }
    default: break;
  }
  return true;
}

// One CTA of the one-shot all-reduce: its private call counter is the tag; two parities of the staging area.
bool ll_cta(Ctx& c, int me, int cta, uint64_t) {
  const Params& p = c.w->p;
  Rank& mine = c.w->ranks[me];
  const uint64_t e = mine.ll_epoch[cta] + 1, par = e & 1;
  const int n = p.n, nc = p.nctas;
  for (int d = 1; d < n; ++d) {
    const int q = (me + d) % n;
    c.w->ranks[q].ll[((size_t)par * n + me) * nc + cta].store(stamp(e, me, 0, cta), std::memory_order_release);
  }
  if (me == p.slow_rank) std::this_thread::sleep_for(std::chrono::microseconds(150));
  for (int q = 0; q < n; ++q) {
    if (q == me) continue;
    const std::atomic<uint64_t>& line = mine.ll[((size_t)par * n + q) * nc + cta];
    if (!c.wait([&] { return (line.load(std::memory_order_acquire) >> 32) >= e; })) return false;
    if (line.load(std::memory_order_relaxed) != stamp(e, q, 0, cta)) return c.bad();  // a later call's line: overwritten unread
  }
  mine.ll_epoch[cta] = e;
  return true;
}

void cta_thread(World* w, int me, int cta, uint32_t seed) {
  Ctx c{w, std::mt19937(seed)};
  const Params& p = w->p;
  Rank& r = w->ranks[me];
  for (uint64_t e = 1; e <= (uint64_t)p.iters && !w->abort_flag.load(); ++e) {
    if (!c.wait([&] { return r.call_open.load(std::memory_order_acquire) >= e; })) return;
    const int op = w->ops[e - 1];
    const bool ok = op == LL_ONESHOT ? ll_cta(c, me, cta, e) : direct_cta(c, me, cta, op, e);
    if (!ok) return;
    if (r.done_in_call.fetch_add(1, std::memory_order_acq_rel) + 1 == p.nctas) {
      // kernel boundary reached by the last CTA: the "user" prepares the next call's input in place (its own
      // buffer only), then the next launch may start
      if (e < (uint64_t)p.iters)
        for (int s = 0; s < p.n; ++s)
          for (int k = 0; k < p.nctas; ++k) r.buf[(size_t)s * p.nctas + k].store(stamp(e + 1, me, s, k));
      r.done_in_call.store(0, std::memory_order_relaxed);
      r.call_open.store(e + 1, std::memory_order_release);
    }
  }
}

}  // namespace

extern "C" {

// Runs `iters` back-to-back calls (a seeded random mix of two-shot all-reduce, all-gather, reduce-scatter,
// all-to-all, one-shot all-reduce and the reduce with a summing root; `only_op` >= 0 fixes the operation) on a
// simulated world.
// Returns 0 ok, 1 a value of another call / rank was read, 2 a wait gave up, -1 bad argument.
int mt_sim_direct(int nranks, int nctas, int iters, uint32_t seed, int only_op, int slow_rank, int dead_rank,
                  int exit_barrier, uint64_t timeout_ms) {
  if (nranks < 1 || nranks > 16 || nctas < 1 || nctas > 64 || iters < 1 || only_op >= NUM_OPS) return -1;
  Params p{nranks, nctas, iters, slow_rank, dead_rank, exit_barrier, timeout_ms ? timeout_ms : 2000};
  World w(p);
  std::mt19937 g(seed);
  for (int i = 0; i < iters; ++i) w.ops.push_back(only_op >= 0 ? only_op : (int)(g() % NUM_OPS));
  for (int me = 0; me < nranks; ++me) {
    Rank& r = w.ranks[me];
    r.buf = std::vector<Datum>((size_t)nranks * nctas);
    r.out = std::vector<Datum>((size_t)nranks * nctas);
    r.arrive = std::vector<std::atomic<uint64_t>>((size_t)nctas * nranks);
    r.ll = std::vector<std::atomic<uint64_t>>((size_t)2 * nranks * nctas);
    r.xflag = std::vector<std::atomic<uint64_t>>((size_t)nctas * nranks);
    for (auto& x : r.xflag) x.store(0);
    r.rout = std::vector<Datum>((size_t)nranks * nctas * kChunks);
    for (auto& x : r.arrive) x.store(0);
    for (auto& x : r.ll) x.store(0);
    r.bar_epoch.assign(nctas, 0);
    r.ll_epoch.assign(nctas, 0);
    for (int s = 0; s < nranks; ++s)
      for (int k = 0; k < nctas; ++k) r.buf[(size_t)s * nctas + k].store(stamp(1, me, s, k));
  }
  std::vector<std::thread> ts;
  for (int me = 0; me < nranks; ++me) {
    if (me == dead_rank) continue;
    for (int k = 0; k < nctas; ++k) ts.emplace_back(cta_thread, &w, me, k, (uint32_t)g());
  }
  for (auto& t : ts) t.join();
  return w.error.load();
}

}  // extern "C"

#ifdef MT_SIM_MAIN
#include <stdlib.h>
int main(int argc, char** argv) {
  if (argc != 10) return 64;
  long v[9];
  for (int i = 0; i < 9; ++i) v[i] = atol(argv[i + 1]);
  return mt_sim_direct((int)v[0], (int)v[1], (int)v[2], (uint32_t)v[3], (int)v[4], (int)v[5], (int)v[6], (int)v[7], (uint64_t)v[8]);
}
#endif
