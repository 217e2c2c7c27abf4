// Link discovery: which device pairs can access each other, and (optionally) how fast.
//
// Counterpart of get_p2p_speed / get_topology (topology.py:96-150 of the reference).  The probe warms
// the path up once and times the second copy; the reference times a single cold copy.  On an NVSwitch
// node every pair reports the same bandwidth, so measuring is optional: without it a link counts 1.0.
#include <cuda_runtime.h>

#include "../mintccl.h"

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
        void *ps = nullptr, *pd = nullptr;
        cudaStream_t st;
        cudaEvent_t e0, e1;
        cudaSetDevice(s);
        if (cudaMalloc(&ps, probe_bytes) != cudaSuccess) continue;
        cudaStreamCreate(&st);
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaSetDevice(d);
        if (cudaMalloc(&pd, probe_bytes) != cudaSuccess) {
          cudaSetDevice(s);
          cudaFree(ps);
          continue;
        }
        cudaSetDevice(s);
        cudaMemcpyPeerAsync(pd, d, ps, s, probe_bytes, st);  // warm-up: maps the path, wakes the links
        cudaEventRecord(e0, st);
        cudaMemcpyPeerAsync(pd, d, ps, s, probe_bytes, st);
        cudaEventRecord(e1, st);
        cudaStreamSynchronize(st);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (ms > 0.f) gbs = (double)probe_bytes / (ms * 1e-3) / 1e9;
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        cudaStreamDestroy(st);
        cudaFree(ps);
        cudaSetDevice(d);
        cudaFree(pd);
      }
      bw[s * ndev + d] = gbs;
      bw[d * ndev + s] = gbs;
    }
  }
  cudaSetDevice(prev_dev);
  return ndev;
}
