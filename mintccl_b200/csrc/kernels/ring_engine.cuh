// CUDA kernels of the ring / chain collectives: the schedules of ring_schedule.h instantiated with the
// Simple and LL128 protocols.  One CTA is one channel; channels never wait on each other.
#pragma once
#include "../device/proto_ll128.cuh"
#include "../device/proto_simple.cuh"
#include "ring_schedule.h"

namespace mt {

// grid = (channels, local ranks); local ranks > 1 only in single-GPU emulation (cooperative launch).
template <template <class, int> class Proto, class T, int NTHREADS>
__global__ void __launch_bounds__(NTHREADS, 1) ring_kernel(const MtDevComm* comms, RingArgs a) {
  __shared__ int s_fail;
  const int lr = blockIdx.y;
  ring_body<Proto, T, NTHREADS>(comms[lr], a, lr, blockIdx.x, gridDim.x, &s_fail);
}

}  // namespace mt
