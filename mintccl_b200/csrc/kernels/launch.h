// Internal interface between the host runtime and the translation units that hold the kernels.
#pragma once
#include <cuda_runtime.h>
#include "../device/layout.h"

namespace mt {
struct RingArgs;
struct DirectArgs;
struct P2pArgs;
struct LLArgs;

constexpr int kRingThreads = 512;
constexpr int kDirectThreads = 512;
constexpr int kP2pThreads = 512;
constexpr int kLLThreads = 256;

// Launch helper: plain launch for one local rank, cooperative launch (all CTAs guaranteed resident)
// for an emulated world whose ranks wait on each other inside one grid.
cudaError_t launch_any(const void* fn, dim3 grid, dim3 block, void** args, cudaStream_t s, bool cooperative,
                       size_t dyn_smem = 0);
void count_launch();

cudaError_t launch_ring_simple(int dtype, const MtDevComm* comms, const RingArgs& a, int nch, int nlocal, cudaStream_t s);
cudaError_t launch_ring_ll128(int dtype, const MtDevComm* comms, const RingArgs& a, int nch, int nlocal, cudaStream_t s);
cudaError_t launch_direct(int dtype, int out_dtype, const MtDevComm* comms, const DirectArgs& a, int nctas, int nlocal, cudaStream_t s);
cudaError_t launch_p2p(const MtDevComm* comms, const P2pArgs& a, int nctas, int nlocal, cudaStream_t s);
cudaError_t launch_ll_allreduce(int dtype, const MtDevComm* comms, const LLArgs& a, int nctas, int nlocal, cudaStream_t s);
// one-rank communicators: every collective is this copy (invalid value: pointers not co-aligned, use the ring kernel)
cudaError_t launch_local_copy(void* dst, const void* src, uint64_t nbytes, int sms, cudaStream_t s);
cudaError_t launch_wait_timeout_test(const MtDevComm* comms, int nlocal, cudaStream_t s);
}  // namespace mt
