// Small device helpers shared by the kernels: element types at the boundary, sign bits, the 128-point
// Walsh-Hadamard butterfly across one warp, and the status codes of the C interface.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/htr_b200.h"

namespace htr {

constexpr float kInvSqrt128 = 0.08838834764831845f;  // 1/sqrt(128)
constexpr unsigned kFullWarp = 0xFFFFFFFFu;

// four consecutive elements of a row, widened to float (element index idx is a multiple of 4)
__device__ __forceinline__ float4 load_quad(const void* base, size_t idx, int dtype) {
  if (dtype == HTR_DTYPE_F32) return *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
  const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(base) + idx);
  if (dtype == HTR_DTYPE_BF16)
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u), __uint_as_float(raw.y << 16),
                       __uint_as_float(raw.y & 0xFFFF0000u));
  const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
  const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// narrow four floats (round to nearest even) and store them at element index idx (multiple of 4)
__device__ __forceinline__ void store_quad(void* base, size_t idx, int dtype, float4 v) {
  if (dtype == HTR_DTYPE_F32) {
    *reinterpret_cast<float4*>(static_cast<float*>(base) + idx) = v;
    return;
  }
  uint2 raw;
  if (dtype == HTR_DTYPE_BF16) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    raw.x = *reinterpret_cast<const uint32_t*>(&a);
    raw.y = *reinterpret_cast<const uint32_t*>(&b);
  } else {
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    raw.x = *reinterpret_cast<const uint32_t*>(&a);
    raw.y = *reinterpret_cast<const uint32_t*>(&b);
  }
  *reinterpret_cast<uint2*>(static_cast<uint16_t*>(base) + idx) = raw;
}

// packed sign vector: bit (j & 7) of byte j >> 3 set means -1 (docs/FORMAT.md:28-29)
__device__ __forceinline__ float sign_of(const uint8_t* packed, int j) { return ((packed[j >> 3] >> (j & 7)) & 1) ? -1.0f : 1.0f; }

// the four sign bits of elements 4*g .. 4*g+3 (a nibble of the packed vector)
__device__ __forceinline__ unsigned sign_nibble(const uint8_t* packed, int g) { return (packed[g >> 1] >> ((g & 1) * 4)) & 15u; }

__device__ __forceinline__ float flip(float v, unsigned bit) { return __uint_as_float(__float_as_uint(v) ^ (bit << 31)); }

// Unnormalised 128-point Walsh-Hadamard transform (Sylvester order, htr/wire.py:80-87) of a vector spread
// over one warp, four elements per lane.  The element held in v[k] may be 4*lane+k or lane+32*k: the
// butterfly network is the same for both because the transform treats all seven index bits alike.
__device__ __forceinline__ void wht128(float (&v)[4], int lane) {
  const float p = v[0] + v[1], m = v[0] - v[1], q = v[2] + v[3], n = v[2] - v[3];
  v[0] = p + q;
  v[1] = m + n;
  v[2] = p - q;
  v[3] = m - n;
#pragma unroll
  for (int bit = 1; bit < 32; bit <<= 1) {
    const float sgn = (lane & bit) ? -1.0f : 1.0f;  // the upper partner of a butterfly keeps (other - own)
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = fmaf(sgn, v[k], __shfl_xor_sync(kFullWarp, v[k], bit));
  }
}

}  // namespace htr
