// Streaming packed GEMV for HTR-W1 weights on sm_100a: one launch per linear.
//
//   y = sv * Ho( diag(scale * CB) * V * Hi(su * x) ),  V[i,j] = v(s_ij) integer codebook values
//
// (docs/FORMAT.md:7-13 of the reference; replaces its prologue + gemv_epi pair, htr/ops.py:95-98.)
//
// Decomposition.  The weight is cut into units of (128-row block) x (4 tile columns = 64 input columns);
// unit u = rb * CG + cg.  The grid has G persistent CTAs and CTA b owns the contiguous unit range
// [b*U/G, (b+1)*U/G), so every CTA streams the same number of packed bytes (+-1 unit) whatever the
// shape.  A range may end inside a row block and continue in the next one.  For every row block it
// touches, a CTA publishes one partial result [M,128]; the CTA that arrives last at the block's counter
// adds the partials in CTA order (deterministic), applies row scales, the output Hadamard, output signs
// and bias, and resets the counter.  No CTA ever waits for another one.
//
// Inside a CTA (256 threads): warp = (half h of the row block: strips 4h..4h+3) x (tile column c of the
// unit); lane = (strip g, row pair q).  Per unit a lane loads its K words (+1 history word from the
// neighbouring lane), rebuilds 32 codebook integers in registers and multiplies them with the transformed
// activations, which all lanes of the warp read from shared memory at the same address (broadcast).
// The integer->float step uses the 1.5*2^23 bit trick; products are accumulated in float32 with the
// packed two-wide FMA of sm_100.
#pragma once
#include "htr_codec.cuh"
#include "htr_common.cuh"

namespace htr {

constexpr int kGemvThreads = 256;
constexpr int kStageBlocks = 8;                  // 128-column blocks staged in shared memory at a time
constexpr int kStageCols = kStageBlocks * 128;   // 1024 activations per row

struct GemvParams {
  const void* x;
  const uint32_t* qw;
  const __half* scales;
  const uint8_t* su;
  const uint8_t* sv;
  const void* bias;
  void* y;
  float* part;      // [row blocks][slots][MT][128]
  int* counters;    // [row blocks], zero between launches
  int rows;         // activation rows actually present (<= MT)
  int mt, nt;       // tiles along m and n
  int dtype;        // element type of x, y, bias
  int cg;           // column groups per row block (nt / 4)
  long long units;  // row blocks * cg
  int slots;        // partial slots per row block
  float cb;         // 1 / rms of the codebook integers
};

// owner CTA of unit x when CTA b starts at floor(b*U/G)
__device__ __host__ inline int unit_owner(long long x, long long G, long long U) { return (int)(((x + 1) * G - 1) / U); }

template <int K>
__device__ __forceinline__ void load_unit_words(const uint32_t* __restrict__ p, uint32_t (&w)[K]) {
  if constexpr (K % 4 == 0) {
#pragma unroll
    for (int i = 0; i < K / 4; ++i) {
      const uint4 t = __ldg(reinterpret_cast<const uint4*>(p) + i);
      w[4 * i] = t.x; w[4 * i + 1] = t.y; w[4 * i + 2] = t.z; w[4 * i + 3] = t.w;
    }
  } else if constexpr (K % 2 == 0) {
#pragma unroll
    for (int i = 0; i < K / 2; ++i) {
      const uint2 t = __ldg(reinterpret_cast<const uint2*>(p) + i);
      w[2 * i] = t.x; w[2 * i + 1] = t.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < K; ++i) w[i] = __ldg(p + i);
  }
}

// column of the tile stored at staged position pos (inverse of staged_col)
template <int K>
__device__ __forceinline__ constexpr int staged_col_inv(int pos) {
  constexpr int P = PairStride<K>::value;
  if (P == 1) return pos;
  const int pair = pos >> 1, hi = pos & 1;
  return (pair / P) * 2 * P + (pair % P) + hi * P;
}

// 32 weights x MT activation rows of one lane unit.  xs points at the 16 staged activations of this tile
// for row 0; consecutive activation rows are kStageCols floats apart.
template <int K, int MT>
__device__ __forceinline__ void unit_fma(const uint32_t (&V)[K + 1], const float* __restrict__ xs, float2 (&acc)[MT][2]) {
  uint32_t s[32];
  unit_states<K>(V, s);
  const float2 unbias = make_float2(-kMagic, -kMagic);
#pragma unroll
  for (int quad = 0; quad < 4; ++quad) {
    float4 xv[MT];
#pragma unroll
    for (int r = 0; r < MT; ++r) xv[r] = *reinterpret_cast<const float4*>(xs + r * kStageCols + quad * 4);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int c0 = staged_col_inv<K>(quad * 4 + half * 2), c1 = staged_col_inv<K>(quad * 4 + half * 2 + 1);
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const float2 w = __fadd2_rn(
            make_float2(__uint_as_float(code_magic_bits(s[rr * 16 + c0])), __uint_as_float(code_magic_bits(s[rr * 16 + c1]))), unbias);
#pragma unroll
        for (int r = 0; r < MT; ++r) {
          const float2 xp = half ? make_float2(xv[r].z, xv[r].w) : make_float2(xv[r].x, xv[r].y);
          acc[r][rr] = __ffma2_rn(w, xp, acc[r][rr]);
        }
      }
    }
  }
}

template <int K, int MT>
__global__ void __launch_bounds__(kGemvThreads) packed_gemv_kernel(const GemvParams p) {
  // staged activations during the sweep; reused for the cross-warp reduction at the end of a row block
  __shared__ __align__(16) float smem[MT * kStageCols];
  __shared__ int s_arrival;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = warp & 1, c = warp >> 1, g = lane >> 3, q = lane & 7;
  const long long U = p.units, G = gridDim.x;
  const long long u_begin = (long long)blockIdx.x * U / G, u_end = ((long long)blockIdx.x + 1) * U / G;
  const int CG = p.cg, nt = p.nt, n = nt * 16, m = p.mt * 16;
  const int hist_lane = (lane & ~7) | ((q + 7) & 7);

  auto unit_ptr = [&](long long u) -> const uint32_t* {
    const int rb = (int)(u / CG), cgi = (int)(u - (long long)rb * CG);
    const size_t tile = (size_t)(rb * 8 + 4 * h + g) * nt + (size_t)(4 * cgi + c);
    return p.qw + tile * (8 * K) + q * K;
  };

  uint32_t next[K];
  if (u_begin < u_end) load_unit_words<K>(unit_ptr(u_begin), next);

  float2 acc[MT][2];
#pragma unroll
  for (int r = 0; r < MT; ++r) acc[r][0] = acc[r][1] = make_float2(0.f, 0.f);

  int staged_rb = -1, stage_lo = 0, stage_hi = 0;  // staged tile columns [stage_lo, stage_hi) of row block staged_rb

  for (long long u = u_begin; u < u_end; ++u) {
    uint32_t V[K + 1];
#pragma unroll
    for (int k = 0; k < K; ++k) V[k + 1] = next[k];
    if (u + 1 < u_end) load_unit_words<K>(unit_ptr(u + 1), next);
    V[0] = __shfl_sync(kFullWarp, V[K], hist_lane);

    const int rb = (int)(u / CG), cgi = (int)(u - (long long)rb * CG);
    const int tj = 4 * cgi + c;

    if (rb != staged_rb || 4 * cgi >= stage_hi) {
      // ---- stage the transformed activations of the next kStageBlocks column blocks (CTA-uniform branch)
      const int hb0 = cgi >> 1;                                   // first 128-column block needed
      const int cg_stop = (int)min((long long)CG, cgi + (u_end - u));   // this CTA's last column group in rb, exclusive
      const int hb1 = min(hb0 + kStageBlocks, (cg_stop + 1) >> 1);
      __syncthreads();
      for (int item = warp; item < MT * (hb1 - hb0); item += kGemvThreads / 32) {
        const int r = item / (hb1 - hb0), hb = hb0 + item % (hb1 - hb0);
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < p.rows) {
          const float4 xv = load_quad(p.x, (size_t)r * n + hb * 128 + 4 * lane, p.dtype);
          const unsigned sg = sign_nibble(p.su, hb * 32 + lane);
          v[0] = flip(xv.x, sg & 1u); v[1] = flip(xv.y, (sg >> 1) & 1u); v[2] = flip(xv.z, (sg >> 2) & 1u); v[3] = flip(xv.w, sg >> 3);
          wht128(v, lane);
        }
        float* dst = smem + r * kStageCols + (hb - hb0) * 128 + (lane >> 2) * 16;
#pragma unroll
        for (int k = 0; k < 4; ++k) dst[staged_col<K>(4 * (lane & 3) + k)] = v[k] * kInvSqrt128;
      }
      __syncthreads();
      staged_rb = rb; stage_lo = hb0 * 8; stage_hi = hb1 * 8;
    }

    unit_fma<K, MT>(V, smem + (tj - stage_lo) * 16, acc);

    const bool block_done = (cgi == CG - 1) || (u + 1 == u_end);
    if (!block_done) continue;

    // ---- this CTA's contribution to row block rb is complete: reduce the four column warps
    __syncthreads();                                   // everyone is done reading the staged activations
    float* red = smem;                                  // [4][MT][128]
#pragma unroll
    for (int r = 0; r < MT; ++r)
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        red[(c * MT + r) * 128 + h * 64 + g * 16 + 2 * q + rr] = acc[r][rr].x + acc[r][rr].y;
        acc[r][rr] = make_float2(0.f, 0.f);
      }
    staged_rb = -1;                                     // the staging buffer is clobbered
    __syncthreads();

    const int first = unit_owner((long long)rb * CG, G, U), last = unit_owner((long long)(rb + 1) * CG - 1, G, U);
    const int contributors = last - first + 1;
    float* ytil = smem + 4 * MT * 128;                  // [MT][128], disjoint from red (needs MT*kStageCols >= 5*MT*128)
    bool finish = true;
    if (contributors > 1) {
      float* mine = p.part + ((size_t)rb * p.slots + (blockIdx.x - first)) * (MT * 128);
      for (int e = tid; e < MT * 128; e += kGemvThreads)
        __stcg(mine + e, red[e] + red[MT * 128 + e] + red[2 * MT * 128 + e] + red[3 * MT * 128 + e]);
      __threadfence();
      __syncthreads();
      if (tid == 0) s_arrival = atomicAdd(p.counters + rb, 1);
      __syncthreads();
      finish = (s_arrival == contributors - 1);
      if (finish) {
        __threadfence();
        const float* slot0 = p.part + (size_t)rb * p.slots * (MT * 128);
        for (int e = tid; e < MT * 128; e += kGemvThreads) {
          float sum = 0.f;
          for (int sl = 0; sl < contributors; ++sl) sum += __ldcg(slot0 + (size_t)sl * (MT * 128) + e);
          ytil[e] = sum;
        }
        if (tid == 0) p.counters[rb] = 0;
      }
    } else {
      for (int e = tid; e < MT * 128; e += kGemvThreads)
        ytil[e] = red[e] + red[MT * 128 + e] + red[2 * MT * 128 + e] + red[3 * MT * 128 + e];
    }
    __syncthreads();
    if (finish && warp < p.rows) {
      // ---- epilogue of row block rb, one warp per activation row
      const int r = warp, row0 = rb * 128 + 4 * lane;
      float v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = ytil[r * 128 + 4 * lane + k] * (__half2float(p.scales[row0 + k]) * p.cb);
      wht128(v, lane);
      const unsigned sg = sign_nibble(p.sv, rb * 32 + lane);
      float4 o = make_float4(flip(v[0] * kInvSqrt128, sg & 1u), flip(v[1] * kInvSqrt128, (sg >> 1) & 1u),
                             flip(v[2] * kInvSqrt128, (sg >> 2) & 1u), flip(v[3] * kInvSqrt128, sg >> 3));
      if (p.bias) {
        const float4 b = load_quad(p.bias, row0, p.dtype);
        o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
      }
      store_quad(p.y, (size_t)r * m + row0, p.dtype, o);
    }
    // the next row block restages before it touches smem again (staged_rb == -1 forces the barrier)
  }
}

// host-side launcher of one instantiation, defined once per K in packed_gemv_k*.cu
template <int K>
int launch_packed_gemv(const GemvParams& p, int mt_rows, int grid, cudaStream_t stream);
template <int K>
int packed_gemv_ctas_per_sm(int mt_rows);

}  // namespace htr
