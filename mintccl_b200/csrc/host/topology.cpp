// Topology search on a bandwidth matrix: widest route between two ranks and the best ring.
//
// Same questions as the reference's find_route / find_ring (topology.py:23-93) answered with exact
// searches: the route is the maximum-bottleneck path with the fewest hops among equals (a direct link
// wins when it is at least as wide); the ring is the Hamiltonian cycle through rank 0 that maximises
// the narrowest link (depth-first with pruning, fine for the <= 8 ranks of a node).
#include <algorithm>
#include <limits>
#include <vector>

#include "../mintccl.h"

namespace {
struct RingSearch {
  const double* bw = nullptr;
  int n = 0;
  std::vector<int> path, best;
  std::vector<char> used;
  double best_bw = 0;
  void dfs(int u, double min_bw) {
    if ((int)path.size() == n) {
      const double back = bw[u * n + path[0]];
      const double w = std::min(min_bw, back);
      if (back > 0 && w > best_bw) {
        best_bw = w;
        best = path;
      }
      return;
    }
    for (int v = 0; v < n; ++v) {
      if (used[v]) continue;
      const double e = bw[u * n + v];
      if (e <= 0) continue;
      const double w = std::min(min_bw, e);
      if (w <= best_bw) continue;  // cannot beat the best ring found so far
      used[v] = 1;
      path.push_back(v);
      dfs(v, w);
      path.pop_back();
      used[v] = 0;
    }
  }
};
}  // namespace

extern "C" int mt_find_ring(const double* bw, int n, int* out) {
  if (n < 1 || n > 64) return 0;
  if (n == 1) {
    out[0] = 0;
    out[1] = 0;
    return 2;
  }
  RingSearch s;
  s.bw = bw;
  s.n = n;
  s.used.assign(n, 0);
  s.used[0] = 1;
  s.path.push_back(0);
  s.dfs(0, std::numeric_limits<double>::infinity());
  if (s.best.empty()) return 0;
  for (int i = 0; i < n; ++i) out[i] = s.best[i];
  out[n] = s.best[0];
  return n + 1;
}

extern "C" int mt_find_route(const double* bw, int n, int src, int dst, int* out) {
  if (n < 1 || src < 0 || dst < 0 || src >= n || dst >= n) return 0;
  if (src == dst) {
    out[0] = src;
    return 1;
  }
  // widest path; ties broken by hop count (O(n^2) Dijkstra on (width desc, hops asc))
  std::vector<double> width(n, 0.0);
  std::vector<int> hops(n, 1 << 30), prev(n, -1);
  std::vector<char> done(n, 0);
  width[src] = std::numeric_limits<double>::infinity();
  hops[src] = 0;
  for (int it = 0; it < n; ++it) {
    int u = -1;
    for (int v = 0; v < n; ++v) {
      if (done[v] || width[v] <= 0) continue;
      if (u < 0 || width[v] > width[u] || (width[v] == width[u] && hops[v] < hops[u])) u = v;
    }
    if (u < 0) break;
    done[u] = 1;
    for (int v = 0; v < n; ++v) {
      const double e = bw[u * n + v];
      if (e <= 0 || done[v]) continue;
      const double w = std::min(width[u], e);
      if (w > width[v] || (w == width[v] && hops[u] + 1 < hops[v])) {
        width[v] = w;
        hops[v] = hops[u] + 1;
        prev[v] = u;
      }
    }
  }
  if (width[dst] <= 0) return 0;
  std::vector<int> rev;
  for (int v = dst; v != -1; v = prev[v]) rev.push_back(v);
  if (rev.back() != src) return 0;
  int len = 0;
  for (auto it = rev.rbegin(); it != rev.rend(); ++it) out[len++] = *it;
  return len;
}
