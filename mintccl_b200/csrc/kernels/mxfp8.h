// Arguments of the block-scaled fp8 reduction kernel.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../device/layout.h"

namespace mt {
enum Mxfp8Op : int { MX_ALLREDUCE = 0, MX_REDUCESCATTER = 1 };
struct Mxfp8Args {
  void* data_out[MT_MAX_RANKS];   // reduce-scatter: local shard payload, per local rank
  void* scale_out[MT_MAX_RANKS];  // reduce-scatter: local shard scales
  uint64_t data_in_off, scale_in_off;    // heap offsets of the quantised input (every rank)
  uint64_t data_out_off, scale_out_off;  // all-reduce: heap offsets of the output (every rank)
  uint64_t nblocks;                      // 32-element blocks in the whole tensor
  int32_t op;
};
cudaError_t launch_mxfp8(const MtDevComm* comms, const Mxfp8Args& a, int nctas, int nlocal, cudaStream_t s);
}  // namespace mt
