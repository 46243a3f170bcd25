// C entry points of the tensor-core packed GEMM (batches of 9..128 activation rows per call).
#include <cmath>

#include "packed_gemm_tc.cuh"

namespace htr {

// ------------------------------------------------------------------------------------------------
// Activation transform for the GEMM: xt = H128(su * x) / sqrt(128) / tok as one or two fp16 planes, their sums, tok.
// Output layout = the B operand tiles of the GEMM, ready for one bulk copy per 64-column chunk:
//   xb[chunk][column group g][k-group kc][column r][8 k]   column = g*8 + r: activation row (hi plane), np + row (lo plane)
// grid (np, slices): a CTA transforms one 1024-column slice of one activation row (one 128-column block per warp), after
// finding the range of the whole row itself (every CTA of a row reads the row once; that is cheaper than a second launch
// or a grid-wide exchange).  xsum[row][slice] holds the slice's sum, added up in slice order by the GEMM's epilogue.
// Rows beyond `rows` are written as zeros so that the padded batch is harmless.
template <int DT>
__global__ void __launch_bounds__(256) rht_f16_kernel(const void* __restrict__ x, int rows, int np, int n, int planes, int per,
                                                      const uint8_t* __restrict__ su, __half* __restrict__ xb, float* __restrict__ xsum,
                                                      float* __restrict__ tok) {
  __shared__ float red[8];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the GEMM may start fetching packed words now
  const int r = blockIdx.x, slice = blockIdx.y, slices = gridDim.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int blocks = n >> 7;
  const int hb0 = slice * 8 * per + warp;                    // this warp's 128-column blocks: hb0, hb0 + 8, ... (`per` of them)
  const int ncols = np * planes;
  const size_t chunk_halves = (size_t)ncols * 64;
  // element offset of (column c, k) = chunk*chunk_halves + ((c/8)*8 + (k%64)/8)*64 + (c%8)*8 + k%8
  const size_t col_hi = (size_t)(r >> 3) * 512 + (r & 7) * 8, col_lo = (size_t)((np + r) >> 3) * 512 + ((np + r) & 7) * 8;
  auto tile_offset = [&](int hb) {
    const int k0 = hb * 128 + 4 * lane;                      // four consecutive k, inside one 8-wide k group
    return (size_t)(k0 >> 6) * chunk_halves + (size_t)((k0 & 63) >> 3) * 64 + (k0 & 7);
  };
  if (r >= rows) {
    for (int i = 0; i < per; ++i) {
      const int hb = hb0 + 8 * i;
      if (hb < blocks) {
        *reinterpret_cast<uint2*>(xb + tile_offset(hb) + col_hi) = make_uint2(0u, 0u);
        if (planes == 2) *reinterpret_cast<uint2*>(xb + tile_offset(hb) + col_lo) = make_uint2(0u, 0u);
      }
    }
    if (tid == 0) {
      xsum[(size_t)r * slices + slice] = 0.f;
      if (slice == 0) tok[r] = 1.f;
    }
    return;
  }
  float amax = 0.f;
#pragma unroll 4
  for (int e = tid; e < n / 4; e += 256) {                   // range of the whole row
    const float4 v = load_quad(x, (size_t)r * n + 4 * e, DT);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(kFullWarp, amax, o));
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  float mx = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) mx = fmaxf(mx, red[k]);
  const float bound = mx * 11.32f;                           // |H128 x| / sqrt(128) <= sqrt(128) * amax
  const float scale = bound > 16384.f ? exp2f(ceilf(log2f(bound / 16384.f))) : 1.f;
  if (tid == 0 && slice == 0) tok[r] = scale;
  const float inv = kInvSqrt128 / scale;
  float sum = 0.f;
#pragma unroll 2
  for (int i = 0; i < per; ++i) {
    const int hb = hb0 + 8 * i;
    if (hb >= blocks) break;                                 // warp-uniform: the shuffles inside stay converged
    const float4 mine = load_quad(x, (size_t)r * n + hb * 128 + 4 * lane, DT);   // second touch: L1
    const unsigned sg = sign_nibble(su, hb * 32 + lane);
    float v[4] = {flip(mine.x, sg & 1u), flip(mine.y, (sg >> 1) & 1u), flip(mine.z, (sg >> 2) & 1u), flip(mine.w, sg >> 3)};
    wht128(v, lane);
    __half hi[4], lo[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float t = v[k] * inv;
      hi[k] = __float2half_rn(t);
      lo[k] = __float2half_rn(t - __half2float(hi[k]));
      sum += planes == 2 ? __half2float(hi[k]) + __half2float(lo[k]) : __half2float(hi[k]);   // exactly what the MMA will see
    }
    const size_t at = tile_offset(hb);
    *reinterpret_cast<uint2*>(xb + at + col_hi) = *reinterpret_cast<const uint2*>(hi);
    if (planes == 2) *reinterpret_cast<uint2*>(xb + at + col_lo) = *reinterpret_cast<const uint2*>(lo);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(kFullWarp, sum, o);
  __syncthreads();
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (tid == 0) {
    float s = 0.f;
    for (int k = 0; k < 8; ++k) s += red[k];
    xsum[(size_t)r * slices + slice] = s;
  }
}

// 128-column blocks per warp of the transform: one for small batches (most CTAs), more when the rows alone fill the GPU
int gemm_rht_per(int np, int n) {
  const int max_per = (n / 128 + 7) / 8;
  int per = np / 48;
  if (per < 1) per = 1;
  return per > max_per ? max_per : per;
}
int gemm_rht_slices(int np, int n) {
  const int per = gemm_rht_per(np, n);
  return (n / 128 + 8 * per - 1) / (8 * per);
}

int run_rht_f16(const void* x, int dtype, int rows, int np, int n, int planes, const uint8_t* su, __half* xb, float* xsum, float* tok,
                cudaStream_t st) {
  const dim3 grid(np, gemm_rht_slices(np, n));
  const int per = gemm_rht_per(np, n);
  switch (dtype) {
    case HTR_DTYPE_BF16: rht_f16_kernel<HTR_DTYPE_BF16><<<grid, 256, 0, st>>>(x, rows, np, n, planes, per, su, xb, xsum, tok); break;
    case HTR_DTYPE_F16: rht_f16_kernel<HTR_DTYPE_F16><<<grid, 256, 0, st>>>(x, rows, np, n, planes, per, su, xb, xsum, tok); break;
    default: rht_f16_kernel<HTR_DTYPE_F32><<<grid, 256, 0, st>>>(x, rows, np, n, planes, per, su, xb, xsum, tok); break;
  }
  return (int)cudaGetLastError();
}

namespace {

thread_local int t_gemm_cuda = 0;
constexpr size_t kCounterRegion = 1 << 16;   // same fixed counter region as the GEMV workspace
constexpr size_t kErrorRegion = 256;

struct GemmPlan {
  int np, rbs, hb, split, grid, stages;
  size_t off_xb, off_xsum, off_tok, off_part, total;
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
  const int ncols = g.np * planes;
  int tmem_cols = 32;
  while (tmem_cols < ncols) tmem_cols <<= 1;
  // two CTAs per SM when shared memory and the 512 TMEM columns allow, else one; the deepest ring of chunk pairs that fits
#ifndef HTR_GEMM_MAX_CTAS
#define HTR_GEMM_MAX_CTAS 2
#endif
  const int budget = 227 * 1024;
  int per_sm = 1;
  g.stages = 2;
  bool found = false;
  for (int ctas = HTR_GEMM_MAX_CTAS; ctas >= 1 && !found; --ctas) {
    if (ctas * tmem_cols > 512) continue;
    for (int st = kMaxStages; st >= 2; --st) {
      if (ctas * (gemm_smem_bytes(g.np, planes, K, st) + 1024) <= budget) {
        per_sm = ctas;
        g.stages = st;
        found = true;
        break;
      }
    }
  }
  if (!found) return HTR_ERR_TOO_LARGE;
  long long s = (long long)sms * per_sm / g.rbs;
  if (s < 1) s = 1;
  if (s > g.hb) s = g.hb;
  g.split = (int)s;
  g.grid = g.rbs * g.split;
  size_t off = kCounterRegion + kErrorRegion;
  g.off_xb = off; off += align256((size_t)ncols * n * 2);
  g.off_xsum = off; off += align256((size_t)g.np * gemm_rht_slices(g.np, n) * 4);
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

// rows of the first launch when a batch is too wide for the shared memory of one CTA (two fp16 planes of many rows, wide streams)
static int first_half_rows(int M) { return ((M + 1) / 2 + 15) / 16 * 16; }

static size_t plan_bytes(int M, int m, int n, int K, int planes) {
  GemmPlan g;
  const int rc = make_gemm_plan(M, m, n, K, planes, &g);
  if (rc == HTR_OK) return g.total;
  if (rc == HTR_ERR_TOO_LARGE && M > 16) return plan_bytes(first_half_rows(M), m, n, K, planes);   // the halves run one after the other
  return 0;
}

size_t htr_linear_gemm_workspace_bytes(int M, int m, int n, int K) {
  if (!width_ok(K) || M < 1 || M > HTR_GEMM_MAX_ROWS || m <= 0 || n <= 0 || m % 128 || n % 128) return 0;
  // the scratch of either activation form (one or two fp16 planes) must fit
  const size_t b1 = plan_bytes(M, m, n, K, 1), b2 = plan_bytes(M > HTR_GEMM_MAX_ROWS_F32 ? HTR_GEMM_MAX_ROWS_F32 : M, m, n, K, 2);
  if (!b1 || !b2) return 0;
  return b1 > b2 ? b1 : b2;
}

static int gemm_launch(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su,
                       const uint8_t* sv, const void* bias, void* y, void* const* peer_y, int npeer, int64_t peer_offset, void* workspace,
                       size_t workspace_bytes, htr_stream_t stream);

int htr_linear_gemm(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su,
                    const uint8_t* sv, const void* bias, void* y, void* workspace, size_t workspace_bytes, htr_stream_t stream) {
  return gemm_launch(x, dtype, M, qweight, mt, nt, K, scales, su, sv, bias, y, nullptr, 0, 0, workspace, workspace_bytes, stream);
}

int htr_linear_gemm_peers(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su,
                          const uint8_t* sv, const void* bias, void* const* peer_y, int npeer, int64_t peer_offset, void* workspace,
                          size_t workspace_bytes, htr_stream_t stream) {
  if (npeer < 1 || npeer > 8 || !peer_y || peer_offset < 0 || (peer_offset & 7)) return HTR_ERR_BAD_SHAPE;
  for (int i = 0; i < npeer; ++i)
    if (!peer_y[i] || (reinterpret_cast<uintptr_t>(peer_y[i]) & 15u)) return peer_y[i] ? HTR_ERR_ALIGNMENT : HTR_ERR_NULL;
  // a batch too wide for one launch would need the halves at different offsets: the row-shard form serves one launch
  GemmPlan g;
  if (M > 0 && width_ok(K) && mt > 0 && nt > 0 && make_gemm_plan(M, mt * 16, nt * 16, K, dtype == HTR_DTYPE_F32 ? 2 : 1, &g) != HTR_OK)
    return HTR_ERR_TOO_LARGE;
  return gemm_launch(x, dtype, M, qweight, mt, nt, K, scales, su, sv, bias, nullptr, peer_y, npeer, peer_offset, workspace, workspace_bytes, stream);
}

static int gemm_launch(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su,
                       const uint8_t* sv, const void* bias, void* y, void* const* peer_y, int npeer, int64_t peer_offset, void* workspace,
                       size_t workspace_bytes, htr_stream_t stream) {
  if (!width_ok(K)) return HTR_ERR_BAD_K;
  if (dtype < HTR_DTYPE_BF16 || dtype > HTR_DTYPE_F32) return HTR_ERR_BAD_DTYPE;
  if (M < 0 || M > HTR_GEMM_MAX_ROWS || mt <= 0 || nt <= 0 || mt % 8 || nt % 8) return HTR_ERR_BAD_SHAPE;
  if (mt / 8 > (int)(kCounterRegion / 4)) return HTR_ERR_TOO_LARGE;
  if (M == 0) return HTR_OK;
  if (!x || !qweight || !scales || !su || !sv || (!y && npeer == 0)) return HTR_ERR_NULL;
  const auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!a16(x) || !a16(qweight) || !a16(y) || (bias && !a16(bias)) || !a16(workspace) || !a16(scales)) return HTR_ERR_ALIGNMENT;
  const int m = mt * 16, n = nt * 16;
  GemmPlan g;
  const int planes = dtype == HTR_DTYPE_F32 ? 2 : 1;      // 16-bit activations need no lo plane
  if (planes == 2 && M > HTR_GEMM_MAX_ROWS_F32) return HTR_ERR_BAD_SHAPE;
  const int rc = make_gemm_plan(M, m, n, K, planes, &g);
  if (rc == HTR_ERR_TOO_LARGE && M > 16 && npeer == 0) {  // too wide for one CTA's shared memory: two launches over row halves
    const int M1 = first_half_rows(M);
    const size_t esz = dtype == HTR_DTYPE_F32 ? 4 : 2;
    const int r1 = htr_linear_gemm(x, dtype, M1, qweight, mt, nt, K, scales, su, sv, bias, y, workspace, workspace_bytes, stream);
    if (r1 != HTR_OK) return r1;
    return htr_linear_gemm(static_cast<const char*>(x) + (size_t)M1 * n * esz, dtype, M - M1, qweight, mt, nt, K, scales, su, sv, bias,
                           static_cast<char*>(y) + (size_t)M1 * m * esz, workspace, workspace_bytes, stream);
  }
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
  p.xb = reinterpret_cast<const __half*>(ws + g.off_xb);
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
  p.stages = g.stages;
  p.xsum_slices = gemm_rht_slices(g.np, n);
  p.cb = (float)codebook_scale();
  p.npeer = npeer;
  p.peer_offset = peer_offset;
  for (int i = 0; i < 8; ++i) p.peer_y[i] = i < npeer ? peer_y[i] : nullptr;
  int e = run_rht_f16(x, dtype, M, g.np, n, planes, su, reinterpret_cast<__half*>(ws + g.off_xb), reinterpret_cast<float*>(ws + g.off_xsum),
                      reinterpret_cast<float*>(ws + g.off_tok), st);
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
