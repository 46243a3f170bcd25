// Tail-biting Viterbi search over the 16-bit bit-shift trellis: the encoder-side inverse of the decode path.
//
// For every tile (batch row) it finds the states s_0 .. s_{T-1}, s_t = ((s_{t-1} << K) & 0xFFFF) | new bits, that minimise
// sum_t w[t] * (x[t] - cb[s_t])^2 with cb[s] = float32(v(s) / rms), and -- with tail-biting -- close the stream into a circle
// (the high 16-K bits of s_0 equal the low 16-K bits of s_{T-1}), so that the rate is exactly K bits per weight.
// Same result as the reference's portable search (htr/reference.py:7-50) and its CUDA version (htr/vit_v2.py:28-73, built there
// for sm_86 / sm_120 only): same float32 operation order per candidate, first minimum wins on ties.
//
// Formulation.  The reference keeps all 65536 path costs; here only their minima over the top K bits survive a step:
//   m_{t+1}[j] = min_top ( m_t[(top << (16-2K)) | (j >> K)] + w_t * (x_t - cb[(top << (16-K)) | j])^2 ),   bp_t[j] = argmin,
// with m_0 = 0 (or, in the second pass, +inf except at the required start).  That is 2 * 2^(16-K) floats of state, which fits
// shared memory for every K (128 KB at K = 2), so one CTA owns a tile from the first step to the traceback and touches global
// memory only for the back-pointers (one byte per (step, j), second pass only; each resident CTA has its own region).
// The codebook value is recomputed per candidate from the hash: v(s) lands in a float through the 1.5 * 2^23 mantissa trick
// and float32(v / rms) = fma(v, inv_hi, v * inv_lo) with 1/rms split in two floats -- exact for all 1021 possible v (checked
// by the tests against the oracle's table, bit for bit), so no table lookups with their bank conflicts.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

#include "../../include/htr_b200.h"
#include "htr_codec.cuh"

namespace htr {
namespace {

constexpr int kVitMaxT = 256;

struct VitParams {
  const float* x;
  const float* w;
  int32_t* states;
  float* total;
  uint8_t* bps;      // [grid][T][2^(16-K)]
  int B, T, tailbite;
  float inv_hi, inv_lo;
};

template <int K>
struct VitCfg {
  static constexpr int kSj = 1 << (16 - K);
  // a thread owns groups of kJb consecutive j (they share the predecessor minima: kJb divides 2^K) and works on them in pairs
  static constexpr int kJb = K == 2 ? 4 : K <= 4 ? 8 : K == 5 ? 4 : 2;
  static constexpr int kThreads = K == 2 ? 1024 : (kSj / kJb < 512 ? kSj / kJb : 512);
  static constexpr int kGroups = kSj / (kThreads * kJb);
  static constexpr int kSmem = 2 * kSj * 4 + 2 * kVitMaxT * 4 + kSj;   // two cost arrays, targets, weights, last back-pointers
};

__device__ __forceinline__ float codebook_value(uint32_t hash, float inv_hi, float inv_lo) {
  const float v = __uint_as_float(__dp4a(hash, 0x01010101u, kMagicBits - 510u)) - 12582912.0f;   // the integer v(s), exactly
  return __fmaf_rn(v, inv_hi, __fmul_rn(v, inv_lo));
}

// packed float32 pairs: one instruction, two candidates
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

struct Best {
  float v;
  uint32_t key;      // (top << 16) | j : state order, so "smaller key" = "earlier state"
};
__device__ __forceinline__ bool better(const Best& a, const Best& b) { return a.v < b.v || (a.v == b.v && a.key < b.key); }

template <int K>
__global__ void __launch_bounds__(VitCfg<K>::kThreads) viterbi_kernel(const VitParams p) {
  constexpr int NB = 1 << K, SJ = VitCfg<K>::kSj, SH = 16 - 2 * K, THREADS = VitCfg<K>::kThreads, JB = VitCfg<K>::kJb, GROUPS = VitCfg<K>::kGroups;
  static_assert(JB >= 2 && JB % 2 == 0 && NB % JB == 0 && GROUPS * THREADS * JB == SJ, "thread-to-state mapping");
  constexpr uint32_t kTopStep = kGenMul << (16 - K);                      // hash difference between consecutive top values
  extern __shared__ __align__(16) unsigned char vsm[];
  float* m_a = reinterpret_cast<float*>(vsm);
  float* m_b = m_a + SJ;
  float* xs = m_b + SJ;
  float* ws = xs + kVitMaxT;
  uint8_t* lastarg = reinterpret_cast<uint8_t*>(ws + kVitMaxT);
  __shared__ Best s_red[32];
  __shared__ Best s_win;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int T = p.T;
  uint8_t* bp = p.bps + (size_t)blockIdx.x * T * SJ;
  const float2 unmagic = make_float2(-12582912.0f, -12582912.0f);
  const float2 ninv_hi = make_float2(-p.inv_hi, -p.inv_hi), ninv_lo = make_float2(-p.inv_lo, -p.inv_lo);

  for (int tile = blockIdx.x; tile < p.B; tile += gridDim.x) {
    __syncthreads();                                                     // the previous tile's traceback is over
    for (int t = tid; t < T; t += THREADS) {
      xs[t] = p.x[(size_t)tile * T + t];
      ws[t] = p.w[(size_t)tile * T + t];
    }
    int j0 = -1;
    const int passes = p.tailbite ? 2 : 1;
    for (int pass = 0; pass < passes; ++pass) {
      const bool keep = pass == passes - 1;                              // back-pointers are needed for the last pass only
      float* mc = m_a;
      float* mn = m_b;
      for (int j = tid; j < SJ; j += THREADS) mc[j] = (j0 < 0 || j == j0) ? 0.f : INFINITY;
      __syncthreads();
      for (int t = 0; t < T; ++t) {
        const float2 xt2 = make_float2(xs[t], xs[t]), wt2 = make_float2(ws[t], ws[t]);
        const bool last = t == T - 1;
#pragma unroll 1
        for (int g = 0; g < GROUPS; ++g) {
          const int jbase = (g * THREADS + tid) * JB;
          const float* prev_col = mc + (jbase >> K);                     // predecessor minima of this group: stride 2^(16-2K) per top
          uint32_t hash[JB];
          float best[JB];
          int arg[JB];
#pragma unroll
          for (int b = 0; b < JB; ++b) {
            hash[b] = (uint32_t)(jbase + b) * kGenMul + kGenAdd;
            best[b] = INFINITY;
            arg[b] = 0;
          }
#pragma unroll 4
          for (int top = 0; top < NB; ++top) {
            const float prev = prev_col[top << SH];
#pragma unroll
            for (int b = 0; b < JB; b += 2) {
              // two candidates per packed float instruction; per lane the reference's operation order:
              // c = float32(v / rms); d = x - c; cost = prev + w * (d * d)
              const float2 vm = make_float2(__uint_as_float(bytesum_add_alu(hash[b], kMagicBits - 510u)),
                                            __uint_as_float(bytesum_add(hash[b + 1], kMagicBits - 510u)));
              const float2 v = add2(vm, unmagic);
              const float2 negc = fma2(v, ninv_hi, mul2(v, ninv_lo));              // -c: negation commutes with rounding
              const float2 d = add2(xt2, negc);
              const float2 wd = mul2(wt2, mul2(d, d));
              // the last addition stays scalar: a packed multiply followed by a packed add was observed to come out fused (one
              // rounding instead of two, costs 1 ulp off the reference's), which separate scalar adds rule out
              const float2 val = make_float2(__fadd_rn(prev, wd.x), __fadd_rn(prev, wd.y));
              if (val.x < best[b]) { best[b] = val.x; arg[b] = top; }              // strict: the first minimum wins, as torch.min does
              if (val.y < best[b + 1]) { best[b + 1] = val.y; arg[b + 1] = top; }
              hash[b] += kTopStep;
              hash[b + 1] += kTopStep;
            }
          }
          uint32_t packed_arg[(JB + 3) / 4];
#pragma unroll
          for (int q = 0; q < (JB + 3) / 4; ++q) packed_arg[q] = 0u;
#pragma unroll
          for (int b = 0; b < JB; ++b) {
            mn[jbase + b] = best[b];
            packed_arg[b >> 2] |= (uint32_t)arg[b] << (8 * (b & 3));
          }
          if constexpr (JB >= 4) {
            if (keep) {
#pragma unroll
              for (int q = 0; q < JB / 4; ++q) *reinterpret_cast<uint32_t*>(bp + (size_t)t * SJ + jbase + 4 * q) = packed_arg[q];
            }
            if (last) {
#pragma unroll
              for (int q = 0; q < JB / 4; ++q) *reinterpret_cast<uint32_t*>(lastarg + jbase + 4 * q) = packed_arg[q];
            }
          } else {
            if (keep) *reinterpret_cast<uint16_t*>(bp + (size_t)t * SJ + jbase) = (uint16_t)packed_arg[0];
            if (last) *reinterpret_cast<uint16_t*>(lastarg + jbase) = (uint16_t)packed_arg[0];
          }
        }
        __syncthreads();
        float* sw = mc; mc = mn; mn = sw;
      }
      // mc[j] = min over top of the final costs, lastarg[j] = its first top.  First pass of a tail-biting search, or an open
      // search: the first state (in state order) of minimal cost.
      if (!(p.tailbite && keep)) {
        Best mine = {INFINITY, 0xFFFFFFFFu};
        for (int j = tid; j < SJ; j += THREADS) {
          const Best cand = {mc[j], ((uint32_t)lastarg[j] << 16) | (uint32_t)j};
          if (better(cand, mine)) mine = cand;
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
          Best other = {__shfl_xor_sync(0xFFFFFFFFu, mine.v, o), __shfl_xor_sync(0xFFFFFFFFu, mine.key, o)};
          if (better(other, mine)) mine = other;
        }
        if (lane == 0) s_red[warp] = mine;
        __syncthreads();
        if (tid == 0) {
          Best win = s_red[0];
          for (int i = 1; i < THREADS / 32; ++i)
            if (better(s_red[i], win)) win = s_red[i];
          s_win = win;
        }
        __syncthreads();
        j0 = (int)(s_win.key & 0xFFFFu);                                 // low 16-K bits of the winner (j < 2^(16-K))
      }
      if (keep && tid == 0) {
        // last state: with tail-biting the cheapest state whose low bits equal j0, else the overall winner
        uint32_t s = p.tailbite ? ((uint32_t)lastarg[j0] * SJ + (uint32_t)j0) : ((s_win.key >> 16) * SJ + (s_win.key & 0xFFFFu));
        if (p.total) p.total[tile] = p.tailbite ? mc[j0] : s_win.v;
        int32_t* out = p.states + (size_t)tile * T;
        out[T - 1] = (int32_t)s;
        for (int t = T - 1; t >= 1; --t) {                                // htr/reference.py:45-49
          const uint32_t low = s >> K;
          s = (uint32_t)bp[(size_t)(t - 1) * SJ + low] * SJ + low;
          out[t - 1] = (int32_t)s;
        }
      }
      __syncthreads();
    }
  }
}

// every codebook value through the device function above (test hook)
__global__ void codebook_kernel(float* out, float inv_hi, float inv_lo) {
  const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s < 65536u) out[s] = codebook_value(s * kGenMul + kGenAdd, inv_hi, inv_lo);
}

double inverse_rms() {
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

bool width_ok(int K) { return K == 2 || K == 3 || K == 4 || K == 5 || K == 6 || K == 8; }

thread_local int t_vit_cuda = 0;

template <int K>
int resident_ctas(int* out) {
  static int cached[64] = {0};
  int dev = 0, sms = 0, per = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return (int)cudaErrorInvalidDevice;
  if (dev >= 0 && dev < 64 && cached[dev]) { *out = cached[dev]; return 0; }
  cudaError_t e = cudaFuncSetAttribute(viterbi_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, VitCfg<K>::kSmem);
  if (e != cudaSuccess) return (int)e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
  if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, viterbi_kernel<K>, VitCfg<K>::kThreads, VitCfg<K>::kSmem)) != cudaSuccess) return (int)e;
  if (per < 1) return (int)cudaErrorLaunchOutOfResources;
  *out = sms * per;
  if (dev >= 0 && dev < 64) cached[dev] = *out;
  return 0;
}

int resident_for(int K, int* out) {
  switch (K) {
    case 2: return resident_ctas<2>(out);
    case 3: return resident_ctas<3>(out);
    case 4: return resident_ctas<4>(out);
    case 5: return resident_ctas<5>(out);
    case 6: return resident_ctas<6>(out);
    case 8: return resident_ctas<8>(out);
  }
  return (int)cudaErrorInvalidValue;
}

template <int K>
int launch(const VitParams& p, int grid, cudaStream_t st) {
  viterbi_kernel<K><<<grid, VitCfg<K>::kThreads, VitCfg<K>::kSmem, st>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace
}  // namespace htr

using namespace htr;

extern "C" {

size_t htr_viterbi_workspace_bytes(int B, int T, int K) {
  if (!width_ok(K) || B < 1 || T < 1 || T > kVitMaxT) return 0;
  int resident = 0;
  if (resident_for(K, &resident) != 0) return 0;
  const int grid = B < resident ? B : resident;
  return (size_t)grid * T * ((size_t)65536 >> K);
}

int htr_viterbi(const float* x, const float* w, int B, int T, int K, int tailbite, int32_t* states, float* total, void* workspace,
                size_t workspace_bytes, htr_stream_t stream) {
  if (!width_ok(K)) return HTR_ERR_BAD_K;
  if (B < 0 || T < 1 || T > kVitMaxT) return HTR_ERR_BAD_SHAPE;
  if (B == 0) return HTR_OK;
  if (!x || !w || !states) return HTR_ERR_NULL;
  int resident = 0;
  int e = resident_for(K, &resident);
  if (e) { t_vit_cuda = e; return HTR_ERR_CUDA; }
  const int grid = B < resident ? B : resident;
  if (!workspace || workspace_bytes < (size_t)grid * T * ((size_t)65536 >> K)) return HTR_ERR_WORKSPACE;
  const double inv = inverse_rms();
  VitParams p;
  p.x = x;
  p.w = w;
  p.states = states;
  p.total = total;
  p.bps = static_cast<uint8_t*>(workspace);
  p.B = B;
  p.T = T;
  p.tailbite = tailbite ? 1 : 0;
  p.inv_hi = (float)inv;
  p.inv_lo = (float)(inv - (double)p.inv_hi);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (K) {
    case 2: e = launch<2>(p, grid, st); break;
    case 3: e = launch<3>(p, grid, st); break;
    case 4: e = launch<4>(p, grid, st); break;
    case 5: e = launch<5>(p, grid, st); break;
    case 6: e = launch<6>(p, grid, st); break;
    case 8: e = launch<8>(p, grid, st); break;
  }
  if (e) { t_vit_cuda = e; return HTR_ERR_CUDA; }
  return HTR_OK;
}

int htr_viterbi_last_cuda_error(void) { return t_vit_cuda; }

int htr_codebook_f32(float* out, htr_stream_t stream) {
  if (!out) return HTR_ERR_NULL;
  const double inv = inverse_rms();
  const float hi = (float)inv, lo = (float)(inv - (double)hi);
  codebook_kernel<<<256, 256, 0, static_cast<cudaStream_t>(stream)>>>(out, hi, lo);
  const int e = (int)cudaGetLastError();
  if (e) { t_vit_cuda = e; return HTR_ERR_CUDA; }
  return HTR_OK;
}

}  // extern "C"
