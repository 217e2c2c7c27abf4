// Ring / chain collectives, LL128 protocol instantiations.
#include "launch.h"
#include "ring_engine.cuh"

namespace mt {
template <class T>
static cudaError_t go(const MtDevComm* comms, const RingArgs& a, int nch, int nlocal, cudaStream_t s) {
  RingArgs args = a;
  void* p[] = {(void*)&comms, (void*)&args};
  return launch_any((const void*)ring_kernel<LL128Prims, T, kRingThreads>, dim3(nch, nlocal), dim3(kRingThreads), p, s,
                    nlocal > 1);
}
cudaError_t launch_ring_ll128(int dtype, const MtDevComm* comms, const RingArgs& a, int nch, int nlocal, cudaStream_t s) {
  switch (dtype) {
    case DT_F32: return go<F32>(comms, a, nch, nlocal, s);
    case DT_F16: return go<F16>(comms, a, nch, nlocal, s);
    case DT_BF16: return go<BF16>(comms, a, nch, nlocal, s);
    default: return go<U8>(comms, a, nch, nlocal, s);
  }
}
}  // namespace mt
