// Hooks around the wire format: raw integer decode, the stand-alone activation transform and the
// original-basis weight materialisation.  None of them is on the decode hot path (the packed GEMV fuses
// what it needs); they exist so that each stage can be compared with the CPU decoder on its own.
#include "htr_codec.cuh"
#include "htr_common.cuh"

namespace htr {

// ------------------------------------------------------------------------------------------------
// int16 v(s_t) for every step of every tile, [ntiles, 256] in stream order.  One thread = one row pair.
template <int K>
__global__ void __launch_bounds__(256) decode_raw_kernel(const uint32_t* __restrict__ qw, int16_t* __restrict__ out, long long ntiles) {
  const long long unit = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (unit >= ntiles * 8) return;
  const long long tile = unit >> 3;
  const int q = (int)(unit & 7);
  const uint32_t* words = qw + tile * (8 * K);
  uint32_t V[K + 1];
  V[0] = words[history_word<K>(q)];
#pragma unroll
  for (int k = 0; k < K; ++k) V[k + 1] = words[q * K + k];
  uint32_t s[32];
  unit_states<K>(V, s);
  uint4* dst = reinterpret_cast<uint4*>(out + tile * 256 + q * 32);
#pragma unroll
  for (int v4 = 0; v4 < 4; ++v4) {
    uint32_t packed[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t lo = (uint32_t)code_value(s[v4 * 8 + 2 * e]) & 0xFFFFu, hi = (uint32_t)code_value(s[v4 * 8 + 2 * e + 1]) & 0xFFFFu;
      packed[e] = lo | (hi << 16);
    }
    dst[v4] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

// ------------------------------------------------------------------------------------------------
// xt[r, 128b + :] = H128/sqrt(128) (su * x[r, 128b + :]).  One warp per (row, 128-column block).
__global__ void __launch_bounds__(256) rht_kernel(const void* __restrict__ x, int dtype, int M, int n, const uint8_t* __restrict__ su,
                                                  float* __restrict__ xt) {
  const int lane = threadIdx.x & 31;
  const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int blocks = n >> 7;
  if (item >= (long long)M * blocks) return;
  const int r = (int)(item / blocks), hb = (int)(item % blocks);
  const size_t at = (size_t)r * n + hb * 128 + 4 * lane;
  const float4 xv = load_quad(x, at, dtype);
  const unsigned sg = sign_nibble(su, hb * 32 + lane);
  float v[4] = {flip(xv.x, sg & 1u), flip(xv.y, (sg >> 1) & 1u), flip(xv.z, (sg >> 2) & 1u), flip(xv.w, sg >> 3)};
  wht128(v, lane);
  *reinterpret_cast<float4*>(xt + at) = make_float4(v[0] * kInvSqrt128, v[1] * kInvSqrt128, v[2] * kInvSqrt128, v[3] * kInvSqrt128);
}

// ------------------------------------------------------------------------------------------------
// W block (128 x 128) = sv * Ho Q Hi * su.  One CTA per block: decode into shared memory, transform down
// the columns, then along the rows, apply the signs and write.
constexpr int kDqLd = 129;  // padded leading dimension: conflict-free for both transform directions

template <int K>
__global__ void __launch_bounds__(256) dequant_w_kernel(const uint32_t* __restrict__ qw, const __half* __restrict__ scales,
                                                        const uint8_t* __restrict__ su, const uint8_t* __restrict__ sv, float cb,
                                                        void* __restrict__ W, int out_dtype, int nt) {
  extern __shared__ float blk[];  // [128][kDqLd]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cbk = blockIdx.x, rb = blockIdx.y, n = nt * 16;

  // decode: 64 tiles x 8 row pairs = 512 lane units, two per thread
  for (int unit = tid; unit < 512; unit += 256) {
    const int q = unit & 7, tl = unit >> 3, tr = tl >> 3, tc = tl & 7;  // tile (tr, tc) of the block
    const uint32_t* words = qw + ((size_t)(rb * 8 + tr) * nt + (cbk * 8 + tc)) * (8 * K);
    uint32_t V[K + 1];
    V[0] = words[history_word<K>(q)];
#pragma unroll
    for (int k = 0; k < K; ++k) V[k + 1] = words[q * K + k];
    uint32_t s[32];
    unit_states<K>(V, s);
#pragma unroll
    for (int u = 0; u < 32; ++u) {
      const int row = tr * 16 + 2 * q + (u >> 4), col = tc * 16 + (u & 15);
      blk[row * kDqLd + col] = (float)code_value(s[u]) * (__half2float(scales[rb * 128 + row]) * cb);
    }
  }
  __syncthreads();
  // Hadamard over the 128 rows, column by column (htr/wire.py:111): lane holds rows lane + 32k
  for (int col = warp; col < 128; col += 8) {
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = blk[(lane + 32 * k) * kDqLd + col];
    wht128(v, lane);
#pragma unroll
    for (int k = 0; k < 4; ++k) blk[(lane + 32 * k) * kDqLd + col] = v[k];
  }
  __syncthreads();
  // Hadamard over the 128 columns of each row (htr/wire.py:112), signs (htr/wire.py:113), store
  for (int row = warp; row < 128; row += 8) {
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = blk[row * kDqLd + lane + 32 * k];
    wht128(v, lane);
    const int gi = rb * 128 + row;
    const float rs = sign_of(sv, gi) * (1.0f / 128.0f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int gj = cbk * 128 + lane + 32 * k;
      const float w = v[k] * rs * sign_of(su, gj);
      const size_t at = (size_t)gi * n + gj;
      if (out_dtype == HTR_DTYPE_F32) static_cast<float*>(W)[at] = w;
      else if (out_dtype == HTR_DTYPE_BF16) static_cast<__nv_bfloat16*>(W)[at] = __float2bfloat16_rn(w);
      else static_cast<__half*>(W)[at] = __float2half_rn(w);
    }
  }
}

template <int K>
static int launch_decode_raw(const uint32_t* qw, int16_t* out, long long ntiles, cudaStream_t st) {
  const long long blocks = (ntiles * 8 + 255) / 256;
  decode_raw_kernel<K><<<(unsigned)blocks, 256, 0, st>>>(qw, out, ntiles);
  return (int)cudaGetLastError();
}

template <int K>
static int launch_dequant_w(const uint32_t* qw, const __half* scales, const uint8_t* su, const uint8_t* sv, float cb, void* W,
                            int out_dtype, int mt, int nt, cudaStream_t st) {
  const size_t smem = sizeof(float) * 128 * kDqLd;
  cudaError_t e = cudaFuncSetAttribute(dequant_w_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dequant_w_kernel<K><<<dim3(nt / 8, mt / 8), 256, smem, st>>>(qw, scales, su, sv, cb, W, out_dtype, nt);
  return (int)cudaGetLastError();
}

int run_decode_raw(int K, const uint32_t* qw, int16_t* out, long long ntiles, cudaStream_t st) {
  switch (K) {
    case 2: return launch_decode_raw<2>(qw, out, ntiles, st);
    case 3: return launch_decode_raw<3>(qw, out, ntiles, st);
    case 4: return launch_decode_raw<4>(qw, out, ntiles, st);
    case 5: return launch_decode_raw<5>(qw, out, ntiles, st);
    case 6: return launch_decode_raw<6>(qw, out, ntiles, st);
    case 8: return launch_decode_raw<8>(qw, out, ntiles, st);
  }
  return (int)cudaErrorInvalidValue;
}

int run_rht(const void* x, int dtype, int M, int n, const uint8_t* su, float* xt, cudaStream_t st) {
  const long long warps = (long long)M * (n >> 7);
  const long long blocks = (warps + 7) / 8;
  rht_kernel<<<(unsigned)blocks, 256, 0, st>>>(x, dtype, M, n, su, xt);
  return (int)cudaGetLastError();
}

int run_dequant_w(int K, const uint32_t* qw, const __half* scales, const uint8_t* su, const uint8_t* sv, float cb, void* W,
                  int out_dtype, int mt, int nt, cudaStream_t st) {
  switch (K) {
    case 2: return launch_dequant_w<2>(qw, scales, su, sv, cb, W, out_dtype, mt, nt, st);
    case 3: return launch_dequant_w<3>(qw, scales, su, sv, cb, W, out_dtype, mt, nt, st);
    case 4: return launch_dequant_w<4>(qw, scales, su, sv, cb, W, out_dtype, mt, nt, st);
    case 5: return launch_dequant_w<5>(qw, scales, su, sv, cb, W, out_dtype, mt, nt, st);
    case 6: return launch_dequant_w<6>(qw, scales, su, sv, cb, W, out_dtype, mt, nt, st);
    case 8: return launch_dequant_w<8>(qw, scales, su, sv, cb, W, out_dtype, mt, nt, st);
  }
  return (int)cudaErrorInvalidValue;
}

}  // namespace htr
