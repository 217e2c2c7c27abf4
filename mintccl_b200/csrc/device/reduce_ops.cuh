// Element-wise sum on packed words, accumulated in fp32.
//
// The reference reduces fp16 only, with fp16 accumulation (`SumFP16`, primitive.py:230-247: two
// add.f16x2 on a 64-bit word).  Here every 16-bit type is widened to fp32, added, and rounded once per
// combine; kernels that see all contributions at once (direct and NVLS algorithms) keep the running
// sum in fp32 registers across all ranks and round a single time.  The MXFP8 helpers implement the
// block-scaled fp8 sum: e4m3 payload with one ue8m0 scale per 32 elements, fp32 accumulate, one
// requantisation at the end.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include "prims.cuh"

namespace mt {

enum DType : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2, DT_U8 = 3, DT_MXFP8 = 4 };

__host__ __device__ __forceinline__ int dtype_size(int dt) { return dt == DT_F32 ? 4 : (dt == DT_U8 || dt == DT_MXFP8) ? 1 : 2; }

struct F32 {
  using elem = float;
  static constexpr int kPer64 = 2;
  static __device__ __forceinline__ void unpack(uint64_t w, float* f) {
    f[0] = __uint_as_float((uint32_t)w);
    f[1] = __uint_as_float((uint32_t)(w >> 32));
  }
  static __device__ __forceinline__ uint64_t pack(const float* f) {
    return (uint64_t)__float_as_uint(f[0]) | ((uint64_t)__float_as_uint(f[1]) << 32);
  }
};
struct F16 {
  using elem = __half;
  static constexpr int kPer64 = 4;
  static __device__ __forceinline__ void unpack(uint64_t w, float* f) {
    __half2 lo = *reinterpret_cast<__half2*>(&w);
    uint32_t h = (uint32_t)(w >> 32);
    __half2 hi = *reinterpret_cast<__half2*>(&h);
    float2 a = __half22float2(lo), b = __half22float2(hi);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
  static __device__ __forceinline__ uint64_t pack(const float* f) {
    __half2 lo = __floats2half2_rn(f[0], f[1]), hi = __floats2half2_rn(f[2], f[3]);
    return (uint64_t)(*reinterpret_cast<uint32_t*>(&lo)) | ((uint64_t)(*reinterpret_cast<uint32_t*>(&hi)) << 32);
  }
};
struct BF16 {
  using elem = __nv_bfloat16;
  static constexpr int kPer64 = 4;
  static __device__ __forceinline__ void unpack(uint64_t w, float* f) {
    // bf16 -> fp32 is a 16-bit shift
    f[0] = __uint_as_float((uint32_t)(w << 16) & 0xffff0000u);
    f[1] = __uint_as_float((uint32_t)w & 0xffff0000u);
    f[2] = __uint_as_float((uint32_t)(w >> 16) & 0xffff0000u);
    f[3] = __uint_as_float((uint32_t)(w >> 32) & 0xffff0000u);
  }
  static __device__ __forceinline__ uint64_t pack(const float* f) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(f[0], f[1]), hi = __floats2bfloat162_rn(f[2], f[3]);
    return (uint64_t)(*reinterpret_cast<uint32_t*>(&lo)) | ((uint64_t)(*reinterpret_cast<uint32_t*>(&hi)) << 32);
  }
};
// Opaque bytes: "sum" is not defined; used by copy-only collectives so that one template serves all.
struct U8 {
  using elem = uint8_t;
  static constexpr int kPer64 = 8;
  static __device__ __forceinline__ void unpack(uint64_t, float*) {}
  static __device__ __forceinline__ uint64_t pack(const float*) { return 0; }
};

// a + b on one 64-bit word of packed T, fp32 arithmetic, one rounding.
template <class T>
__device__ __forceinline__ uint64_t sum64(uint64_t a, uint64_t b) {
  float fa[T::kPer64], fb[T::kPer64];
  T::unpack(a, fa);
  T::unpack(b, fb);
#pragma unroll
  for (int i = 0; i < T::kPer64; ++i) fa[i] += fb[i];
  return T::pack(fa);
}
template <>
__device__ __forceinline__ uint64_t sum64<U8>(uint64_t a, uint64_t) { return a; }

template <class T>
__device__ __forceinline__ u128 sum128(u128 a, u128 b) {
  u128 r;
  r.x = sum64<T>(a.x, b.x);
  r.y = sum64<T>(a.y, b.y);
  return r;
}

// fp32 accumulator for one 16-byte vector of packed T (direct algorithms: add all ranks, round once).
template <class T>
struct Acc128 {
  float f[2 * T::kPer64];
  __device__ __forceinline__ void set(u128 v) {
    T::unpack(v.x, f);
    T::unpack(v.y, f + T::kPer64);
  }
  __device__ __forceinline__ void add(u128 v) {
    float g[2 * T::kPer64];
    T::unpack(v.x, g);
    T::unpack(v.y, g + T::kPer64);
#pragma unroll
    for (int i = 0; i < 2 * T::kPer64; ++i) f[i] += g[i];
  }
  __device__ __forceinline__ u128 get() const {
    u128 r;
    r.x = T::pack(f);
    r.y = T::pack(f + T::kPer64);
    return r;
  }
};

// Scalar sum for unaligned tails.
template <class T>
__device__ __forceinline__ typename T::elem sum_elem(typename T::elem a, typename T::elem b);
template <>
__device__ __forceinline__ float sum_elem<F32>(float a, float b) { return a + b; }
template <>
__device__ __forceinline__ __half sum_elem<F16>(__half a, __half b) { return __float2half_rn(__half2float(a) + __half2float(b)); }
template <>
__device__ __forceinline__ __nv_bfloat16 sum_elem<BF16>(__nv_bfloat16 a, __nv_bfloat16 b) {
  return __float2bfloat16_rn(__bfloat162float(a) + __bfloat162float(b));
}
template <>
__device__ __forceinline__ uint8_t sum_elem<U8>(uint8_t a, uint8_t) { return a; }

template <class T>
__device__ __forceinline__ float elem_to_float(typename T::elem v);
template <>
__device__ __forceinline__ float elem_to_float<F32>(float v) { return v; }
template <>
__device__ __forceinline__ float elem_to_float<F16>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float elem_to_float<BF16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float elem_to_float<U8>(uint8_t v) { return (float)v; }
template <class T>
__device__ __forceinline__ typename T::elem float_to_elem(float v);
template <>
__device__ __forceinline__ float float_to_elem<F32>(float v) { return v; }
template <>
__device__ __forceinline__ __half float_to_elem<F16>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 float_to_elem<BF16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ uint8_t float_to_elem<U8>(float v) { return (uint8_t)v; }

// ---- MXFP8 (e4m3 payload, ue8m0 scale per 32 elements) ----------------------------------------------
__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ uint8_t float_to_e4m3(float f) {
  return (uint8_t)__nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3);
}
// ue8m0: value = 2^(e - 127); e == 255 is NaN and is never produced here.
__device__ __forceinline__ float ue8m0_to_float(uint8_t e) { return __uint_as_float((uint32_t)(e == 0 ? 0x00400000u : ((uint32_t)e << 23))); }
// Smallest power-of-two scale such that amax / scale <= 448 (the largest e4m3 value).
__device__ __forceinline__ uint8_t ue8m0_for_amax(float amax) {
  if (!(amax > 0.f)) return 127 - 8;  // all-zero block: any scale works, use a small finite one
  // amax = m * 2^e with m in [1,2); need 2^s >= amax / 448, 448 = 1.75 * 2^8.
  int e;
  float m = frexpf(amax, &e);       // amax = m * 2^e, m in [0.5,1)
  int s = e - 9 + (m * 2.f > 1.75f ? 1 : 0);  // (m*2) * 2^(e-1) / (1.75 * 2^8) <= 2^s
  s += 127;
  s = s < 1 ? 1 : (s > 254 ? 254 : s);
  return (uint8_t)s;
}

}  // namespace mt
