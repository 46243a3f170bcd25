// C entry points of the tensor-core packed GEMM (batches of 9..128 activation rows per call).
#include <cmath>

#include "packed_gemm_tc.cuh"

namespace htr {

// ------------------------------------------------------------------------------------------------
// Activation transform for the GEMM: xt = H128(su * x) / sqrt(128) / tok as two fp16 planes, their row sum, tok.
// One CTA per activation row (rows beyond `rows` are written as zeros so that the padded batch is harmless).
__global__ void __launch_bounds__(256) rht_f16_kernel(const void* __restrict__ x, int dtype, int rows, int n, int planes,
                                                      const uint8_t* __restrict__ su,
                                                      __half* __restrict__ xh, __half* __restrict__ xl, float* __restrict__ xsum,
                                                      float* __restrict__ tok) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int blocks = n >> 7;
  if (r >= rows) {
    for (int e = tid; e < n / 8; e += 256) {
      reinterpret_cast<uint4*>(xh + (size_t)r * n)[e] = make_uint4(0u, 0u, 0u, 0u);
      reinterpret_cast<uint4*>(xl + (size_t)r * n)[e] = make_uint4(0u, 0u, 0u, 0u);
    }
    if (tid == 0) { xsum[r] = 0.f; tok[r] = 1.f; }
    return;
  }
  float amax = 0.f;
  for (int hb = warp; hb < blocks; hb += 8) {
    const float4 v = load_quad(x, (size_t)r * n + hb * 128 + 4 * lane, dtype);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(kFullWarp, amax, o));
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  if (tid == 0) {
    float mx = 0.f;
    for (int k = 0; k < 8; ++k) mx = fmaxf(mx, red[k]);
    const float bound = mx * 11.32f;                       // |H128 x| / sqrt(128) <= sqrt(128) * amax
    s_scale = bound > 16384.f ? exp2f(ceilf(log2f(bound / 16384.f))) : 1.f;
    tok[r] = s_scale;
  }
  __syncthreads();
  const float inv = kInvSqrt128 / s_scale;
  float sum = 0.f;
  for (int hb = warp; hb < blocks; hb += 8) {
    const size_t at = (size_t)r * n + hb * 128 + 4 * lane;
    const float4 xv = load_quad(x, at, dtype);
    const unsigned sg = sign_nibble(su, hb * 32 + lane);
    float v[4] = {flip(xv.x, sg & 1u), flip(xv.y, (sg >> 1) & 1u), flip(xv.z, (sg >> 2) & 1u), flip(xv.w, sg >> 3)};
    wht128(v, lane);
    __half hi[4], lo[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float t = v[k] * inv;
      hi[k] = __float2half_rn(t);
      lo[k] = __float2half_rn(t - __half2float(hi[k]));
      sum += planes == 2 ? __half2float(hi[k]) + __half2float(lo[k]) : __half2float(hi[k]);   // exactly what the MMA will see
    }
    *reinterpret_cast<uint2*>(xh + at) = *reinterpret_cast<const uint2*>(hi);
    *reinterpret_cast<uint2*>(xl + at) = *reinterpret_cast<const uint2*>(lo);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(kFullWarp, sum, o);
  __syncthreads();
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (tid == 0) {
    float s = 0.f;
    for (int k = 0; k < 8; ++k) s += red[k];
    xsum[r] = s;
  }
}

int run_rht_f16(const void* x, int dtype, int rows, int np, int n, int planes, const uint8_t* su, __half* xh, __half* xl, float* xsum,
                float* tok, cudaStream_t st) {
  rht_f16_kernel<<<np, 256, 0, st>>>(x, dtype, rows, n, planes, su, xh, xl, xsum, tok);
  return (int)cudaGetLastError();
}

namespace {

thread_local int t_gemm_cuda = 0;
constexpr size_t kCounterRegion = 1 << 16;   // same fixed counter region as the GEMV workspace
constexpr size_t kErrorRegion = 256;

struct GemmPlan {
  int np, rbs, hb, split, grid;
  size_t off_xh, off_xl, off_xsum, off_tok, off_part, total;
};

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

bool width_ok(int K) { return K == 2 || K == 3 || K == 4 || K == 5 || K == 6 || K == 8; }

double codebook_scale() {
  static const double value = [] {
    double acc = 0.0;
    for (uint32_t s = 0; s < 65536u; ++s) {
      const double v = (double)code_value(s);
      acc += v * v;
    }
    return 1.0 / std::sqrt(acc / 65536.0);
  }();
  return value;
}

int make_gemm_plan(int M, int m, int n, int K, int planes, GemmPlan* out) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HTR_ERR_CUDA;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return HTR_ERR_CUDA;
  GemmPlan g;
  g.np = (M + 15) / 16 * 16;
  g.rbs = m / 128;
  g.hb = n / 128;
  int per_sm = (227 * 1024) / (gemm_smem_bytes(g.np, planes, K) + 1024);   // bounded by shared memory ...
  if (per_sm > 3) per_sm = 3;
  if (per_sm * 2 * g.np > 512) per_sm = 512 / (2 * g.np);                   // ... and by the 512 TMEM columns of an SM
  if (per_sm < 1) per_sm = 1;
  long long s = (long long)sms * per_sm / g.rbs;
  if (s < 1) s = 1;
  if (s > g.hb) s = g.hb;
  g.split = (int)s;
  g.grid = g.rbs * g.split;
  size_t off = kCounterRegion + kErrorRegion;
  g.off_xh = off; off += align256((size_t)g.np * n * 2);
  g.off_xl = off; off += align256((size_t)g.np * n * 2);
  g.off_xsum = off; off += align256((size_t)g.np * 4);
  g.off_tok = off; off += align256((size_t)g.np * 4);
  g.off_part = off; off += align256((size_t)g.rbs * g.split * g.np * 128 * 4);
  g.total = off;
  *out = g;
  return HTR_OK;
}

}  // namespace
}  // namespace htr

using namespace htr;

extern "C" {

size_t htr_linear_gemm_workspace_bytes(int M, int m, int n, int K) {
  if (!width_ok(K) || M < 1 || M > HTR_GEMM_MAX_ROWS || m <= 0 || n <= 0 || m % 128 || n % 128) return 0;
  GemmPlan g1, g2;      // the scratch of either activation form (one or two fp16 planes) must fit
  if (make_gemm_plan(M, m, n, K, 1, &g1) != HTR_OK || make_gemm_plan(M > HTR_GEMM_MAX_ROWS_F32 ? HTR_GEMM_MAX_ROWS_F32 : M, m, n, K, 2, &g2) != HTR_OK) return 0;
  return g1.total > g2.total ? g1.total : g2.total;
}

int htr_linear_gemm(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su,
                    const uint8_t* sv, const void* bias, void* y, void* workspace, size_t workspace_bytes, htr_stream_t stream) {
  if (!width_ok(K)) return HTR_ERR_BAD_K;
  if (dtype < HTR_DTYPE_BF16 || dtype > HTR_DTYPE_F32) return HTR_ERR_BAD_DTYPE;
  if (M < 0 || M > HTR_GEMM_MAX_ROWS || mt <= 0 || nt <= 0 || mt % 8 || nt % 8) return HTR_ERR_BAD_SHAPE;
  if (mt / 8 > (int)(kCounterRegion / 4)) return HTR_ERR_TOO_LARGE;
  if (M == 0) return HTR_OK;
  if (!x || !qweight || !scales || !su || !sv || !y) return HTR_ERR_NULL;
  const auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!a16(x) || !a16(qweight) || !a16(y) || (bias && !a16(bias)) || !a16(workspace) || !a16(scales)) return HTR_ERR_ALIGNMENT;
  const int m = mt * 16, n = nt * 16;
  GemmPlan g;
  const int planes = dtype == HTR_DTYPE_F32 ? 2 : 1;      // 16-bit activations need no lo plane
  if (planes == 2 && M > HTR_GEMM_MAX_ROWS_F32) return HTR_ERR_BAD_SHAPE;
  const int rc = make_gemm_plan(M, m, n, K, planes, &g);
  if (rc != HTR_OK) return rc;
  if (!workspace || workspace_bytes < g.total) return HTR_ERR_WORKSPACE;
  char* ws = static_cast<char*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  GemmParams p;
  p.qw = static_cast<const uint32_t*>(qweight);
  p.scales = static_cast<const __half*>(scales);
  p.sv = sv;
  p.bias = bias;
  p.y = y;
  p.xh = reinterpret_cast<const __half*>(ws + g.off_xh);
  p.xl = reinterpret_cast<const __half*>(ws + g.off_xl);
  p.xsum = reinterpret_cast<const float*>(ws + g.off_xsum);
  p.tok = reinterpret_cast<const float*>(ws + g.off_tok);
  p.part = reinterpret_cast<float*>(ws + g.off_part);
  p.counters = reinterpret_cast<int*>(ws);
  p.error = reinterpret_cast<int*>(ws + kCounterRegion);
  p.rows = M;
  p.np = g.np;
  p.planes = planes;
  p.mt = mt;
  p.nt = nt;
  p.dtype = dtype;
  p.hb = g.hb;
  p.split = g.split;
  p.cb = (float)codebook_scale();
  int e = run_rht_f16(x, dtype, M, g.np, n, planes, su, reinterpret_cast<__half*>(ws + g.off_xh), reinterpret_cast<__half*>(ws + g.off_xl),
                      reinterpret_cast<float*>(ws + g.off_xsum), reinterpret_cast<float*>(ws + g.off_tok), st);
  if (e) { t_gemm_cuda = e; return HTR_ERR_CUDA; }
  switch (K) {
    case 2: e = launch_packed_gemm_tc<2>(p, g.grid, st); break;
    case 3: e = launch_packed_gemm_tc<3>(p, g.grid, st); break;
    case 4: e = launch_packed_gemm_tc<4>(p, g.grid, st); break;
    case 5: e = launch_packed_gemm_tc<5>(p, g.grid, st); break;
    case 6: e = launch_packed_gemm_tc<6>(p, g.grid, st); break;
    case 8: e = launch_packed_gemm_tc<8>(p, g.grid, st); break;
  }
  if (e) t_gemm_cuda = e;
  return e ? HTR_ERR_CUDA : HTR_OK;
}

int htr_linear_gemm_last_cuda_error(void) { return t_gemm_cuda; }

size_t htr_linear_gemm_error_offset(void) { return kCounterRegion; }

}  // extern "C"
