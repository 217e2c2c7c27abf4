// Link discovery: which device pairs can access each other, and (optionally) how fast.
//
// Counterpart of get_p2p_speed / get_topology (topology.py:96-150 of the reference).  The probe warms
// the path up once and times the second copy; the reference times a single cold copy.  On an NVSwitch
// node every pair reports the same bandwidth, so measuring is optional: without it a link counts 1.0.
#include <cuda_runtime.h>

#include "../mintccl.h"

// Times one peer copy s -> d of probe_bytes after a warm-up copy.  Returns GB/s, or 0 when a step failed.
static double probe_pair(int s, int d, uint64_t probe_bytes) {
  void *ps = nullptr, *pd = nullptr;
  cudaStream_t st;
  cudaEvent_t e0, e1;
  double gbs = 0.0;
  cudaSetDevice(s);
  if (cudaMalloc(&ps, probe_bytes) != cudaSuccess) return 0.0;
  cudaStreamCreate(&st);
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaSetDevice(d);
  if (cudaMalloc(&pd, probe_bytes) == cudaSuccess) {
    cudaSetDevice(s);
    cudaMemcpyPeerAsync(pd, d, ps, s, probe_bytes, st);  // warm-up: maps the path, wakes the links
    cudaEventRecord(e0, st);
    cudaMemcpyPeerAsync(pd, d, ps, s, probe_bytes, st);
    cudaEventRecord(e1, st);
    cudaStreamSynchronize(st);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    if (ms > 0.f) gbs = (double)probe_bytes / (ms * 1e-3) / 1e9;
    cudaSetDevice(d);
    cudaFree(pd);
  }
  cudaSetDevice(s);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaStreamDestroy(st);
  cudaFree(ps);
  return gbs;
}

// One pair only: 0 = no peer access (or the probe failed), else GB/s of the timed copy src -> dst.
extern "C" int mt_topo_probe_pair(int src, int dst, uint64_t probe_bytes, double* gbs) {
  int count = 0;
  *gbs = 0.0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) return -1;
  if (src < 0 || dst < 0 || src >= count || dst >= count || src == dst) return -1;
  int prev_dev = 0;
  cudaGetDevice(&prev_dev);
  int a = 0, b = 0;
  cudaDeviceCanAccessPeer(&a, src, dst);
  cudaDeviceCanAccessPeer(&b, dst, src);
  if (a && b) *gbs = probe_pair(src, dst, probe_bytes);
  cudaSetDevice(prev_dev);
  return 0;
}

extern "C" int mt_topo_probe(int ndev, double* bw, int measure, uint64_t probe_bytes) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) return -1;
  if (ndev > count) ndev = count;
  int prev_dev = 0;
  cudaGetDevice(&prev_dev);
  for (int i = 0; i < ndev * ndev; ++i) bw[i] = 0.0;
  for (int s = 0; s < ndev; ++s) {
    for (int d = s + 1; d < ndev; ++d) {
      int a = 0, b = 0;
      cudaDeviceCanAccessPeer(&a, s, d);
      cudaDeviceCanAccessPeer(&b, d, s);
      if (!a || !b) continue;
      double gbs = 1.0;
      if (measure) {
        gbs = probe_pair(s, d, probe_bytes);
        if (gbs <= 0.0) continue;
      }
      bw[s * ndev + d] = gbs;
      bw[d * ndev + s] = gbs;
    }
  }
  cudaSetDevice(prev_dev);
  return ndev;
}
