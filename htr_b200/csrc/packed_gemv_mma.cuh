// Packed GEMV for HTR-W1 weights with the byte sums and the dot product on the tensor cores (warp-level int8 MMA).
//
//   y = sv * Ho( diag(scale * CB) * V * Hi(su * x) ),  V[i,j] = bytesum(h_ij) - 510,  h_ij = (s_ij * 0xDF6ADF + 0x34983) mod 2^32
//
// (docs/FORMAT.md:7-13 of the reference; the same linear as packed_gemv.cuh, for up to four activation rows.)
//
// The 32-bit hash of a weight is fed to mma.sync.m16n8k32 (u8 x s8 -> s32) as four consecutive u8 k-elements of the A
// fragment, straight from the register the multiply-add left it in; the B fragment holds the activation of that column four
// times (one s8 value splatted over a word).  The MMA then performs byte sum, multiply and accumulation of 128 weights per
// instruction: per weight the thread is left with the window extraction and the hash multiply-add (about half the
// instructions of the CUDA-core kernel, which is bounded by instruction issue).
//
// Activations: per window of columns a power-of-two scale per row and four signed 7-bit planes,
// xt * sc = q0 + q1/128 + q2/128^2 + q3/128^3 (|q| <= 64; 27 bits, more than float32 holds).  The eight B columns of an MMA
// are (row parity, plane): one MMA set serves two activation rows, two sets serve four.  Accumulators are exact integers; the
// constant 510 leaves through the exact plane sums; planes are recombined in 64-bit integers, one rounding per window.
//
// Fragment use.  A warp owns one 16-row strip of the 128-row block and the four tiles of a unit (64 columns).  Lane
// (g = lane >> 2, c = lane & 3) decodes the lane unit "rows 2g, 2g+1 of tile c" exactly as in packed_gemv.cuh (same words,
// same compile-time windows).  For MMA j (0..7) it supplies a0 = hash(row 2g, col 2j), a1 = hash(row 2g+1, col 2j),
// a2 = hash(row 2g, col 2j+1), a3 = hash(row 2g+1, col 2j+1): MMA row g is tile row 2g, MMA row g+8 is tile row 2g+1, k-group c
// is (tile c, column 2j), k-group c+4 is (tile c, column 2j+1).  Its B registers are the splatted planes of B column g for the
// same two columns, read from shared memory where the staging pass laid them out per reader lane (conflict-free 16-byte loads).
// The accumulator fragment leaves lane (g, c) with B columns 2c, 2c+1 of both rows: two of the four planes of one activation
// row; a shuffle inside the quad joins the halves.
//
// Decomposition, ring, split reduction, epilogue, launch overlap: packed_gemv.cuh (same GemvParams, plan and workspace).
#pragma once
#include "packed_gemv.cuh"

#ifndef HTR_MMA_CTAS
#define HTR_MMA_CTAS 3
#endif

namespace htr {

constexpr int kMmaRows = 4;                              // activation rows per launch (two per MMA set)

// units (64 columns) of activations staged at a time: 2 KB of B operand per unit and MMA set
template <int NS>
struct MmaWinUnits {
  static constexpr int value = NS == 1 ? 16 : 8;
};
// Words between the tiles of a warp's ring slot.  The four lanes of a quad read the same row pair of four different tiles, so
// with the tiles back to back (8K words) their loads would hit the same banks; a few words of padding spread them out
// (wavefronts per lane unit: K2 6 -> 4, K4 20 -> 8, K6 14 -> 8, K8 40 -> 20; K3 and K5 are conflict-free as they are).
template <int K>
struct MmaTileStride {
  static constexpr int value = 8 * K + (K == 8 ? 4 : K % 2 == 0 ? 8 : 0);
};
template <int K, int NS>
constexpr int gemv_mma_smem_bytes() { return MmaWinUnits<NS>::value * NS * 2048 + kRing * kGemvWarps * 4 * (4 * MmaTileStride<K>::value); }

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int K, int NS>
__global__ void __launch_bounds__(kGemvThreads, (NS == 1 ? HTR_MMA_CTAS : 2)) packed_gemv_mma_kernel(const GemvParams p) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  constexpr int kWinUnits = MmaWinUnits<NS>::value, kWinBlocks = kWinUnits / 2;
  unsigned char* bwin = dyn_smem;                                                   // [unit][set][4 word groups][32 reader lanes][16 B]
  uint32_t* ring = reinterpret_cast<uint32_t*>(dyn_smem + kWinUnits * NS * 2048);  // [kRing][warps][4 tiles][tile stride]
  __shared__ int s_arrival;
  __shared__ unsigned s_amax[kMmaRows];
  __shared__ int s_psum[kMmaRows * 4];
  __shared__ float s_row_inv[kMmaRows];
  __shared__ float s_ss[kGemvWarps];
  __shared__ __align__(16) float ytil[kMmaRows * 128];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;               // consumer roles: row pair of the strip, tile column of the unit
  // planes per activation: four (27 bits), or two (13 bits below the largest value of the window: enough for bf16, whose
  // results are rounded to 8 bits) when an MMA set has to serve four rows instead of two
  const int P = p.rows > 2 * NS ? 2 : 4, RPS = 8 / P;
  const int U = p.units, G = gridDim.x, CG = p.cg, nt = p.nt, n = nt * 16, m = p.mt * 16;
  int u_begin, u_end;
  if (p.split > 0) {
    const int brb = blockIdx.x / p.split, part = blockIdx.x - brb * p.split;
    u_begin = brb * CG + part * CG / p.split;
    u_end = brb * CG + (part + 1) * CG / p.split;
  } else {
    u_begin = (int)((long long)blockIdx.x * U / G);
    u_end = (int)(((long long)blockIdx.x + 1) * U / G);
  }
  constexpr int kTileStride = MmaTileStride<K>::value, kTileBytes = 32 * K, kTileChunks = 2 * K;
  constexpr int kStageBytes = kGemvWarps * 4 * kTileStride * 4;

  // ring slot of this warp: the four tiles of its strip; copy roles: tile lane >> 3, 16-byte chunk lane & 7
  const uint32_t* my_ring = ring + (warp * 4) * kTileStride;
  const uint32_t ring_dst = (uint32_t)__cvta_generic_to_shared(my_ring + (lane >> 3) * kTileStride) + (lane & 7) * 16;

  int rb = u_begin / CG, cgi = u_begin - rb * CG;
  const char* lane_base = reinterpret_cast<const char*>(p.qw) + ((size_t)(rb * 8 + warp) * nt + (size_t)(4 * cgi + (lane >> 3))) * kTileBytes + (lane & 7) * 16;
  constexpr int kStep16 = 4 * kTileBytes / 16;
  const int wrap_extra16 = (7 * nt + 4) * (kTileBytes / 16) - kStep16;
  int pf_off16 = 0, pf_left = u_end - u_begin, pf_in_rb = CG - cgi;
  auto issue = [&](int stage_bytes) {
    const int on = pf_left > 0;
    const char* src = lane_base + (size_t)(unsigned)pf_off16 * 16;
#pragma unroll
    for (int j = 0; j < (kTileChunks + 7) / 8; ++j) {
      if (8 * j + 8 <= kTileChunks) async_copy16_if(ring_dst + stage_bytes + j * 128, src + j * 128, on);
      else async_copy16_if(ring_dst + stage_bytes + j * 128, src + j * 128, on && ((lane & 7) + 8 * j < kTileChunks));
    }
    --pf_left;
    pf_off16 += kStep16;
    if (--pf_in_rb == 0) {
      pf_off16 += wrap_extra16;
      pf_in_rb = CG;
    }
    async_commit();
  };
  issue(0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  bool predecessor_done = false;
  if (!p.independent) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    predecessor_done = true;
  }
#pragma unroll
  for (int sgi = 1; sgi < kDepth; ++sgi) issue(sgi * kStageBytes);
  if (tid < kMmaRows) s_amax[tid] = 0u;
  if (tid < kMmaRows * 4) s_psum[tid] = 0;
  if (p.prologue == 1) {
    for (int r = 0; r < p.rows; ++r) {
      float ss = 0.f;
      for (int e = tid; e < (n >> 2); e += kGemvThreads) {
        const float4 v = load_quad(p.x, (size_t)r * p.x_stride + 4 * e, p.dtype);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(kFullWarp, ss, o);
      __syncthreads();
      if (lane == 0) s_ss[warp] = ss;
      __syncthreads();
      if (tid == 0) {
        float tot = 0.f;
        for (int k = 0; k < kGemvWarps; ++k) tot += s_ss[k];
        s_row_inv[r] = rsqrtf(tot / (float)n + p.eps);
      }
    }
  }
  __syncthreads();

  float accf[NS][2];                                   // rows 2g, 2g+1 of the strip for activation row 2t + (c >> 1), summed over windows
#pragma unroll
  for (int t = 0; t < NS; ++t) accf[t][0] = accf[t][1] = 0.f;

  int stage_bytes = 0, refill_bytes = (kRing - 1) * kStageBytes;
  int u = u_begin;
  while (u < u_end) {
    // ---- window: units [u, seg_end) lie in row block rb and inside kWinBlocks staged 128-column blocks
    const int hb0 = cgi >> 1;
    const int cg_stop = min(CG, cgi + (u_end - u));
    const int hb1 = min(hb0 + kWinBlocks, (cg_stop + 1) >> 1);
    const int seg_cg_end = min(cg_stop, hb1 * 2);
    const int seg_units = seg_cg_end - cgi;
    const int nblk = hb1 - hb0, items = p.rows * nblk;  // <= 4 x 8 = 32 items over 8 warps (two planes), else <= 16
    constexpr int kRounds = NS == 1 ? 4 : 2;

    // -- stage 1: transform the activations of the window, find the range of every row
    float xv[kRounds][4];
#pragma unroll
    for (int it = 0; it < kRounds; ++it) {
      const int item = warp + it * kGemvWarps;
      xv[it][0] = xv[it][1] = xv[it][2] = xv[it][3] = 0.f;
      if (item < items) {
        const int r = item / nblk, hb = hb0 + item % nblk;
        const float4 x4 = fused_x(p, p.x, r, hb * 128 + 4 * lane, p.prologue == 1 ? s_row_inv[r] : 1.f);
        const unsigned sg = sign_nibble(p.su, hb * 32 + lane);
        float v[4] = {flip(x4.x, sg & 1u), flip(x4.y, (sg >> 1) & 1u), flip(x4.z, (sg >> 2) & 1u), flip(x4.w, sg >> 3)};
        wht128(v, lane);
        unsigned mb = __float_as_uint(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
        if (v[0] != v[0] || v[1] != v[1] || v[2] != v[2] || v[3] != v[3]) mb = 0x7FC00000u;
#pragma unroll
        for (int o = 16; o; o >>= 1) mb = max(mb, __shfl_xor_sync(kFullWarp, mb, o));
        if (lane == 0) atomicMax(&s_amax[r], mb);
#pragma unroll
        for (int k = 0; k < 4; ++k) xv[it][k] = v[k];
      }
    }
    __syncthreads();

    // -- stage 2: 7-bit planes of every activation, splatted over a word, laid out per reader lane
#pragma unroll
    for (int it = 0; it < kRounds; ++it) {
      const int item = warp + it * kGemvWarps;
      if (item < items) {
        const int r = item / nblk, hbi = item % nblk;
        const unsigned mb = s_amax[r];
        int ex = (int)(mb >> 23) - 127;
        ex = ex < -100 ? -100 : ex;
        const float sc = __uint_as_float((unsigned)(5 - ex + 127) << 23);     // max * sc in [32, 64)
        int q[4][4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float yv = mb < 0x7F800000u ? xv[it][k] * sc : 0.f;
#pragma unroll
          for (int pl = 0; pl < 4; ++pl) {
            const float rq = rintf(yv);
            q[pl][k] = (int)rq;
            yv = (yv - rq) * 128.f;
          }
        }
        // this lane holds columns 4 lane .. 4 lane + 3 of the block: unit lane >> 4, tile (lane >> 2) & 3, word group lane & 3;
        // reader lane (B column n, tile) = 4 n + tile, with n = P (r % RPS) + plane, in MMA set r / RPS
        const int ul = 2 * hbi + (lane >> 4);
        unsigned char* dst = bwin + ((((ul * NS + r / RPS) * 4 + (lane & 3)) * 32 + ((lane >> 2) & 3)) * 16);
#pragma unroll
        for (int pl = 0; pl < 4; ++pl)
          if (pl < P)
            *reinterpret_cast<uint4*>(dst + (4 * (P * (r % RPS) + pl)) * 16) =
                make_uint4((unsigned)(q[pl][0] & 255) * 0x01010101u, (unsigned)(q[pl][1] & 255) * 0x01010101u,
                           (unsigned)(q[pl][2] & 255) * 0x01010101u, (unsigned)(q[pl][3] & 255) * 0x01010101u);
        const int cgu = 2 * (hb0 + hbi) + (lane >> 4);
        const bool mine = cgu >= cgi && cgu < seg_cg_end;
#pragma unroll
        for (int pl = 0; pl < 4; ++pl) {
          const int sum = __reduce_add_sync(kFullWarp, mine ? q[pl][0] + q[pl][1] + q[pl][2] + q[pl][3] : 0);
          if (lane == 0) atomicAdd(&s_psum[r * 4 + pl], sum);
        }
      }
    }
    __syncthreads();

    // -- main loop of the window
    int d[NS][4];
#pragma unroll
    for (int t = 0; t < NS; ++t) d[t][0] = d[t][1] = d[t][2] = d[t][3] = 0;
    const unsigned char* bunit = bwin + (size_t)(cgi - 2 * hb0) * (NS * 2048) + lane * 16;
#pragma unroll 1
    for (int i = 0; i < seg_units; ++i) {
      uint32_t V[K + 1];
      async_wait<kDepth - 1>();
      __syncwarp();
      read_unit_words<K>(reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(my_ring) + stage_bytes) + c * kTileStride, g, V);
      issue(refill_bytes);
      refill_bytes = stage_bytes;
      stage_bytes = (stage_bytes + kStageBytes == kRing * kStageBytes) ? 0 : stage_bytes + kStageBytes;
      uint32_t s[32];
      unit_states<K>(V, s);
#pragma unroll
      for (int j4 = 0; j4 < 4; ++j4) {
        uint4 b[NS];
#pragma unroll
        for (int t = 0; t < NS; ++t) b[t] = *reinterpret_cast<const uint4*>(bunit + (t * 4 + j4) * 512);
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int col = 4 * j4 + 2 * jj;
          const uint32_t a0 = s[col] * kGenMul + kGenAdd, a1 = s[16 + col] * kGenMul + kGenAdd;
          const uint32_t a2 = s[col + 1] * kGenMul + kGenAdd, a3 = s[17 + col] * kGenMul + kGenAdd;
#pragma unroll
          for (int t = 0; t < NS; ++t) mma_u8s8(d[t], a0, a1, a2, a3, jj ? b[t].z : b[t].x, jj ? b[t].w : b[t].y);
        }
      }
      bunit += NS * 2048;
    }

    // -- the window's integers leave for float.  Four planes: lane (g, c) holds planes 2 (c & 1), 2 (c & 1) + 1 of activation row
    // 2t + (c >> 1), the other two sit in the neighbouring lane.  Two planes: both planes of activation row 4t + c.
#pragma unroll
    for (int t = 0; t < NS; ++t) {
      const int r = P == 4 ? 2 * t + (c >> 1) : 4 * t + c, p0 = P == 4 ? 2 * (c & 1) : 0;
      const int rr_ok = r < p.rows;
      const int ra = rr_ok ? r : 0;
      const long long hi = (P == 4 && (c & 1) == 0) ? 16384ll : 1ll;    // 128^2 for planes 0, 1 of four
      long long v0 = ((long long)(d[t][0] - 510 * s_psum[ra * 4 + p0]) * 128 + (long long)(d[t][1] - 510 * s_psum[ra * 4 + p0 + 1])) * hi;
      long long v1 = ((long long)(d[t][2] - 510 * s_psum[ra * 4 + p0]) * 128 + (long long)(d[t][3] - 510 * s_psum[ra * 4 + p0 + 1])) * hi;
      if (P == 4) {
        v0 += __shfl_xor_sync(kFullWarp, v0, 1);
        v1 += __shfl_xor_sync(kFullWarp, v1, 1);
      }
      const unsigned mb = s_amax[ra];
      int ex = (int)(mb >> 23) - 127;
      ex = ex < -100 ? -100 : ex;
      // 1 / (sc * 128^(P-1)), sc = 2^(5 - ex)
      const double w = __longlong_as_double((long long)(1023 - 7 * (P - 1) - 5 + ex) << 52);
      if (rr_ok) {
        accf[t][0] += mb < 0x7F800000u ? (float)((double)v0 * w) : __uint_as_float(0x7FC00000u);
        accf[t][1] += mb < 0x7F800000u ? (float)((double)v1 * w) : __uint_as_float(0x7FC00000u);
      }
    }
    __syncthreads();                                   // statistics and B window read by everyone: the next window may overwrite them
    if (tid < kMmaRows) s_amax[tid] = 0u;
    if (tid < kMmaRows * 4) s_psum[tid] = 0;

    u += seg_units;
    cgi += seg_units;
    if (cgi < CG && u < u_end) { __syncthreads(); continue; }   // same row block, next window (zeroed statistics visible)

    // ---- this CTA's contribution to row block rb is complete
    if (P == 2 || (c & 1) == 0) {
#pragma unroll
      for (int t = 0; t < NS; ++t) {
        const int r = P == 4 ? 2 * t + (c >> 1) : 4 * t + c;
        if (r < kMmaRows) {
          ytil[r * 128 + warp * 16 + 2 * g] = accf[t][0] * kInvSqrt128;
          ytil[r * 128 + warp * 16 + 2 * g + 1] = accf[t][1] * kInvSqrt128;
        }
      }
    }
#pragma unroll
    for (int t = 0; t < NS; ++t) accf[t][0] = accf[t][1] = 0.f;
    int first, contributors;
    if (p.split > 0) {
      first = rb * p.split;
      contributors = p.split;
    } else {
      first = unit_owner((long long)rb * CG, G, U);
      contributors = unit_owner((long long)(rb + 1) * CG - 1, G, U) - first + 1;
    }
    const int row0 = rb * 128 + 4 * lane;
    uint2 sc_raw = make_uint2(0u, 0u);
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
    unsigned sv_bits = 0;
    if (warp < p.rows) {
      sc_raw = __ldg(reinterpret_cast<const uint2*>(p.scales + row0));
      sv_bits = sign_nibble(p.sv, rb * 32 + lane);
      if (p.bias && row0 < p.m_out) bias4 = load_quad(p.bias, row0, p.dtype);
    }
    if (!predecessor_done) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      predecessor_done = true;
    }
    __syncthreads();
    bool finish = true;
    const int width = (p.rows <= 1 ? 1 : p.rows <= 2 ? 2 : 4) * 128;
    if (contributors > 1) {
      float* mine = p.part + ((size_t)rb * p.slots + (blockIdx.x - first)) * width;
      for (int e = tid; e < width; e += kGemvThreads) __stcg(mine + e, ytil[e]);
      __syncthreads();
      if (tid == 0) {
        __threadfence();
        s_arrival = atomicAdd(p.counters + rb, 1);
        __threadfence();
      }
      __syncthreads();
      finish = (s_arrival == contributors - 1);
      if (finish) {
        const float* slot0 = p.part + (size_t)rb * p.slots * width;
        for (int e = tid; e < width; e += kGemvThreads) {
          float sum = 0.f;
          for (int base = 0; base < contributors; base += 16) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = base + j < contributors ? __ldcg(slot0 + (size_t)(base + j) * width + e) : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) sum += v[j];
          }
          ytil[e] = sum;
        }
        if (tid == 0) p.counters[rb] = 0;
      }
      __syncthreads();
    }
    if (finish && warp < p.rows) {
      const int r = warp;
      const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sc_raw.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&sc_raw.y));
      float v[4] = {ytil[r * 128 + 4 * lane] * (s01.x * p.cb), ytil[r * 128 + 4 * lane + 1] * (s01.y * p.cb),
                    ytil[r * 128 + 4 * lane + 2] * (s23.x * p.cb), ytil[r * 128 + 4 * lane + 3] * (s23.y * p.cb)};
      wht128(v, lane);
      float4 o = make_float4(flip(v[0] * kInvSqrt128, sv_bits & 1u), flip(v[1] * kInvSqrt128, (sv_bits >> 1) & 1u),
                             flip(v[2] * kInvSqrt128, (sv_bits >> 2) & 1u), flip(v[3] * kInvSqrt128, sv_bits >> 3));
      o.x += bias4.x; o.y += bias4.y; o.z += bias4.z; o.w += bias4.w;
      if (p.npeer == 0) {
        if (p.residual) {
          const float4 old = load_quad(p.y, (size_t)r * p.m_out + row0, p.dtype);
          o = make_float4(old.x + bf16_round(o.x), old.y + bf16_round(o.y), old.z + bf16_round(o.z), old.w + bf16_round(o.w));
        }
        if (row0 < p.m_out) store_quad(p.y, (size_t)r * p.m_out + row0, p.dtype, o);
      } else {
#pragma unroll 1
        for (int pe = 0; pe < p.npeer; ++pe) store_quad(p.peer_y[pe], (size_t)p.peer_offset + (size_t)r * m + row0, p.dtype, o);
      }
    }
    __syncthreads();                                   // ytil is free again
    if (cgi == CG) { cgi = 0; ++rb; }
  }
  async_wait<0>();
}

template <int K>
int launch_packed_gemv_mma(const GemvParams& p, int grid, cudaStream_t stream);
template <int K>
int packed_gemv_mma_ctas_per_sm(int rows, int dtype);
// one MMA set (and, beyond two rows, two planes per activation) when the results are rounded to bf16 anyway
inline bool mma_one_set(int rows, int dtype) { return rows <= 2 || dtype == HTR_DTYPE_BF16; }

}  // namespace htr
