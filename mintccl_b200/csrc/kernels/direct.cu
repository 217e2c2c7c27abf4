// One-hop / NVLS collectives, point-to-point copy, one-shot all-reduce: instantiations and launchers.
#include <type_traits>
#include "launch.h"
#include "direct_engine.cuh"
#include "p2p_engine.cuh"

namespace mt {
template <class TI, class TO>
static cudaError_t go_direct(const MtDevComm* comms, const DirectArgs& a, int nctas, int nlocal, cudaStream_t s) {
  DirectArgs args = a;
  void* p[] = {(void*)&comms, (void*)&args};
  if (a.op == DOP_REDUCE && a.variant == 5) {   // counters per chunk: a kernel of its own
    if constexpr (std::is_same<TI, TO>::value)
      return launch_any((const void*)rooted_reduce_kernel<TI, kDirectThreads>, dim3(nctas, nlocal), dim3(kDirectThreads), p, s,
                        nlocal > 1, 0);
    return cudaErrorInvalidValue;
  }
  const void* fn = (const void*)direct_kernel<TI, TO, kDirectThreads>;
  size_t smem = 0;
  if (a.variant >= 4) {  // the copy-engine variants stage their pieces in dynamic shared memory
    static bool raised = false;   // per instantiation; the attribute belongs to the function, not to a device
    if (!raised) {
      cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBulkSmemBytes);
      if (e != cudaSuccess) return e;
      raised = true;
    }
    smem = kBulkSmemBytes;
  }
  return launch_any(fn, dim3(nctas, nlocal), dim3(kDirectThreads), p, s, nlocal > 1, smem);
}
// dtype: elements of the input; out_dtype: elements of the output (the same, or fp32 for a 16-bit input, or a
// 16-bit type for an fp32 input: the sum is rounded once, into the output type).
cudaError_t launch_direct(int dtype, int out_dtype, const MtDevComm* comms, const DirectArgs& a, int nctas, int nlocal,
                          cudaStream_t s) {
  if (dtype != out_dtype) {
    if (dtype == DT_F16 && out_dtype == DT_F32) return go_direct<F16, F32>(comms, a, nctas, nlocal, s);
    if (dtype == DT_BF16 && out_dtype == DT_F32) return go_direct<BF16, F32>(comms, a, nctas, nlocal, s);
    if (dtype == DT_F32 && out_dtype == DT_F16) return go_direct<F32, F16>(comms, a, nctas, nlocal, s);
    if (dtype == DT_F32 && out_dtype == DT_BF16) return go_direct<F32, BF16>(comms, a, nctas, nlocal, s);
    return cudaErrorInvalidValue;
  }
  switch (dtype) {
    case DT_F32: return go_direct<F32, F32>(comms, a, nctas, nlocal, s);
    case DT_F16: return go_direct<F16, F16>(comms, a, nctas, nlocal, s);
    case DT_BF16: return go_direct<BF16, BF16>(comms, a, nctas, nlocal, s);
    default: return go_direct<U8, U8>(comms, a, nctas, nlocal, s);
  }
}
cudaError_t launch_p2p(const MtDevComm* comms, const P2pArgs& a, int nctas, int nlocal, cudaStream_t s) {
  P2pArgs args = a;
  void* p[] = {(void*)&comms, (void*)&args};
  const void* fn = (const void*)p2p_kernel<kP2pThreads>;
  size_t smem = 0;
  if (a.mode == 2) {
    static bool raised = false;
    if (!raised) {
      cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBulkSmemBytes);
      if (e != cudaSuccess) return e;
      raised = true;
    }
    smem = kBulkSmemBytes;
  }
  return launch_any(fn, dim3(nctas, nlocal), dim3(kP2pThreads), p, s, nlocal > 1, smem);
}
template <class T>
static cudaError_t go_ll(const MtDevComm* comms, const LLArgs& a, int nctas, int nlocal, cudaStream_t s) {
  LLArgs args = a;
  void* p[] = {(void*)&comms, (void*)&args};
  return launch_any((const void*)ll_allreduce_kernel<T, kLLThreads>, dim3(nctas, nlocal), dim3(kLLThreads), p, s,
                    nlocal > 1);
}
cudaError_t launch_ll_allreduce(int dtype, const MtDevComm* comms, const LLArgs& a, int nctas, int nlocal, cudaStream_t s) {
  switch (dtype) {
    case DT_F32: return go_ll<F32>(comms, a, nctas, nlocal, s);
    case DT_F16: return go_ll<F16>(comms, a, nctas, nlocal, s);
    case DT_BF16: return go_ll<BF16>(comms, a, nctas, nlocal, s);
    default: return cudaErrorInvalidValue;
  }
}

// A wait on a word that nothing ever writes: must give up after the communicator's time limit, record
// MT_ERR_TIMEOUT_SIGNAL and return, leaving the context usable.
__global__ void wait_timeout_test_kernel(const MtDevComm* comms) {
  const MtDevComm& c = comms[blockIdx.y];
  if (threadIdx.x == 0) {
    const uint64_t* w = (const uint64_t*)(c.heap[c.rank] + c.L.ll_epoch_off + 4088);  // never written
    bounded_wait(
        c, [&] { return load64_acquire_sys(w) == 0x5eedull; }, MT_ERR_TIMEOUT_SIGNAL, 0, MT_WHERE_TEST, 0x5eedull, 0,
        (const volatile uint64_t*)w);
  }
}
cudaError_t launch_wait_timeout_test(const MtDevComm* comms, int nlocal, cudaStream_t s) {
  void* p[] = {(void*)&comms};
  return launch_any((const void*)wait_timeout_test_kernel, dim3(1, nlocal), dim3(32), p, s, false);
}
}  // namespace mt
