// Packed GEMM for prefill-sized batches on sm_100a: decoded tiles feed tcgen05.mma, accumulators live in TMEM.
//
//   Y[j, i] = sum_k Xt[j, k] * V[i, k]   for one 128-row block i of the weight, batch rows j (up to 128 per launch)
//
// Replaces the reference's prefill route (dequant_w to bf16 in DRAM + library GEMM, htr/ops.py:89-93, kernels
// htr_kernels.cu:658-903): the packed words are decoded once per launch straight into the shared-memory A operand
// and never reach DRAM as 16-bit weights.  This is the only kernel of the library that uses tensor cores.
//
// Operands.  A (128 x 64 per k-chunk) holds the codebook integers as exact fp16 values 1024 + bytesum (the fp16 bit
// pattern 0x6400 + bytesum needs no conversion instruction); the constant 1534 = 1024 + 510 is removed in the
// epilogue with the row sums of the activations, as the reference does (htr_kernels.cu:312-313).  B holds the
// transformed activations as two fp16 planes, hi and lo = fp16(xt - hi), concatenated along N, so that the
// products carry ~22 bits of the activations; the two accumulator halves are added after the MMA.  A per-row
// power-of-two scale keeps |xt| inside the fp16 range (htr_kernels.cu:205-206).
//
// Both operands use the K-major, no-swizzle canonical layout of the UMMA shared-memory descriptor: 8 rows x 16 bytes
// form a contiguous 128-byte core matrix; core matrices adjacent in K are LBO = 128 bytes apart, 8-row groups are
// SBO bytes apart.  SBO is padded by 16 bytes so that the decode threads' 16-byte stores spread over all banks.
//
// Every wait on an mbarrier is bounded: when it expires the CTA records an error code, stops issuing work, frees its
// TMEM columns and returns; the host sees the code in the workspace header.
#pragma once
#include "htr_codec.cuh"
#include "htr_common.cuh"

namespace htr {

constexpr int kGemmThreads = 256;
constexpr int kGemmWarps = 8;
constexpr int kChunkK = 64;                                 // k extent of one shared-memory stage
constexpr int kLbo = 128;                                   // bytes between core matrices adjacent in K
constexpr int kSbo = (kChunkK / 8) * 128 + 16;              // bytes between 8-row groups (padded: 1040)
constexpr int kATileBytes = (128 / 8) * kSbo;               // 16640
constexpr int kGemmStages = 2;                              // A tiles: one being read by the tensor core, one being decoded
constexpr int kAhead = 3;                                   // chunks of packed words and activations in flight (cp.async)
constexpr int kRawSlots = kAhead + 1;                       // packed-word ring per warp
constexpr int kBStages = kAhead + 2;                        // activation tiles: + one read by the MMA, + one being decoded against
constexpr unsigned kSpinLimit = 4000000u;                   // iterations of a try_wait loop before giving up

struct GemmParams {
  const uint32_t* qw;
  const __half* scales;
  const uint8_t* sv;
  const void* bias;
  void* y;
  const __half* xh;       // [np][n] hi plane of the transformed activations (rows >= rows are zero)
  const __half* xl;       // [np][n] lo plane
  const float* xsum;      // [np] sum over k of the planes in use (hi, or hi + lo)
  const float* tok;       // [np] power-of-two range scale per activation row
  float* part;            // [row blocks][slots][np][128]
  int* counters;          // [row blocks]
  int* error;             // one word: first failure code seen by any CTA (0 = none)
  int rows, np;           // activation rows present / padded to a multiple of 16 (16..128)
  int planes;             // 1: hi plane only (16-bit activations), 2: hi + lo (float32 activations)
  int mt, nt;
  int dtype;
  int hb;                 // 128-column blocks per row (n / 128) = units per row block
  int split;              // CTAs per row block
  float cb;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, int sbo_bytes) {
  // start address, LBO, SBO in 16-byte units; descriptor version 1 (sm_100); layout type 0 = no swizzle
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((kLbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) |
         (1ull << 46);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// bounded wait for the phase with the given parity; false when the limit ran out
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned it = 0; it < kSpinLimit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 16 consecutive accumulator columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_load16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// dynamic shared memory: A tiles, activation tiles, packed-word ring -- later reused for the [np][128] float result
__host__ __device__ inline int gemm_b_tile_bytes(int ncols) { return (ncols / 8) * kSbo; }
__host__ __device__ inline int gemm_raw_bytes(int K) { return kRawSlots * kGemmWarps * 4 * 32 * K; }
__host__ __device__ inline int gemm_smem_bytes(int np, int planes, int K) {
  const int stages = kGemmStages * kATileBytes + kBStages * gemm_b_tile_bytes(np * planes) + gemm_raw_bytes(K);
  const int result = np * 128 * 4;
  return (stages > result ? stages : result) + 128;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

template <int K>
__device__ __forceinline__ void load_lane_words(const uint32_t* __restrict__ p, uint32_t (&w)[K]) {
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

template <int K>
__global__ void __launch_bounds__(kGemmThreads) packed_gemm_tc_kernel(const GemmParams p) {
  extern __shared__ __align__(128) unsigned char gsm[];
  __shared__ __align__(8) unsigned long long s_bar[kGemmStages];
  __shared__ uint32_t s_tmem;
  __shared__ int s_arrival, s_fail;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int np = p.np, ncols = p.planes * np;               // accumulator columns: hi plane, then lo plane if present
  const int nt = p.nt, n = nt * 16, m = p.mt * 16, HB = p.hb;
  const int rb = blockIdx.x / p.split, part_id = blockIdx.x - rb * p.split;
  const int hb_begin = part_id * HB / p.split, hb_end = (part_id + 1) * HB / p.split;
  const int b_tile_bytes = gemm_b_tile_bytes(ncols);
  unsigned char* stage0 = gsm + (128 - (smem_u32(gsm) & 127)) % 128;   // 128-byte aligned start: A tiles
  unsigned char* b_stage0 = stage0 + kGemmStages * kATileBytes;        // activation tiles
  unsigned char* raw0 = b_stage0 + kBStages * b_tile_bytes;            // packed-word ring [slot][warp][4 tiles][8K words]
  const uint32_t stage0_addr = smem_u32(stage0), b_stage0_addr = smem_u32(b_stage0), raw0_addr = smem_u32(raw0);

  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < ncols) tmem_cols <<= 1;
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kGemmStages; ++s) mbar_init(smem_u32(&s_bar[s]), 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = s_tmem;

  // instruction descriptor: D = f32, A = B = f16, both K-major, M = 128, N = ncols
  const uint32_t idesc = (1u << 4) | ((uint32_t)(ncols >> 3) << 17) | ((128u >> 4) << 24);

  // decode role of this thread inside a k-chunk: strip = warp, tile column tc = lane >> 3, row pair q = lane & 7
  const int tc = lane >> 3, q = lane & 7;
  const size_t strip_tile0 = (size_t)(rb * 8 + warp) * nt;
  const int chunks = (hb_end - hb_begin) * 2;                // two 64-column chunks per 128-column block
  constexpr int kWarpRawBytes = 4 * 32 * K, kSlotBytes = kGemmWarps * kWarpRawBytes;

  // asynchronous fetch of chunk c: this warp's four packed tiles (contiguous) and the CTA's activation tile
  auto prefetch = [&](int c) {
    if (c < chunks) {
      const int tile_col0 = hb_begin * 8 + c * 4;
      const char* wsrc = reinterpret_cast<const char*>(p.qw + (strip_tile0 + tile_col0) * (8 * K));
      const uint32_t wdst = raw0_addr + (c % kRawSlots) * kSlotBytes + warp * kWarpRawBytes;
#pragma unroll
      for (int j = 0; j < (8 * K + 31) / 32; ++j)
        if (32 * j + 32 <= 8 * K || lane + 32 * j < 8 * K) cp_async16(wdst + (lane + 32 * j) * 16, wsrc + (lane + 32 * j) * 16);
      const uint32_t bdst = b_stage0_addr + (c % kBStages) * b_tile_bytes;
      const int k0 = tile_col0 * 16;
      for (int v = tid; v < ncols * 8; v += kGemmThreads) {
        const int row = v % ncols, kc = v / ncols;           // row fastest: conflict-free 16-byte stores
        const __half* src = (row < np ? p.xh + (size_t)row * n : p.xl + (size_t)(row - np) * n) + k0 + kc * 8;
        cp_async16(bdst + (row >> 3) * kSbo + (row & 7) * 16 + kc * kLbo, src);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int c = 0; c < kAhead; ++c) prefetch(c);

  uint32_t phase_bits = 0u;                                 // bit s = parity of the next completion of stage s's barrier
  bool failed = false;
  for (int ch = 0; ch < chunks; ++ch) {
    const int s = ch & 1;
    asm volatile("cp.async.wait_group %0;" ::"n"(kAhead - 1) : "memory");   // this chunk's words and activations have landed
    // the MMAs that read A stage s (and the activation tile of chunk ch-2) must have finished (bounded wait, all threads)
    if (ch >= kGemmStages && !failed) {
      if (!mbar_wait(smem_u32(&s_bar[s]), (phase_bits >> s) & 1u)) failed = true;
      phase_bits ^= 1u << s;
    }
    __syncwarp();
    prefetch(ch + kAhead);                                   // overwrites the activation tile of chunk ch-2 and the word slot of ch-1

    uint32_t V[K + 1];
    {
      const uint32_t* tile = reinterpret_cast<const uint32_t*>(raw0 + (ch % kRawSlots) * kSlotBytes + warp * kWarpRawBytes) + tc * (8 * K);
      const uint32_t* own = tile + q * K;
      if constexpr (K % 4 == 0) {
#pragma unroll
        for (int i = 0; i < K / 4; ++i) {
          const uint4 t = *reinterpret_cast<const uint4*>(own + 4 * i);
          V[4 * i + 1] = t.x; V[4 * i + 2] = t.y; V[4 * i + 3] = t.z; V[4 * i + 4] = t.w;
        }
      } else if constexpr (K % 2 == 0) {
#pragma unroll
        for (int i = 0; i < K / 2; ++i) {
          const uint2 t = *reinterpret_cast<const uint2*>(own + 2 * i);
          V[2 * i + 1] = t.x; V[2 * i + 2] = t.y;
        }
      } else {
#pragma unroll
        for (int k = 0; k < K; ++k) V[k + 1] = own[k];
      }
      V[0] = tile[history_word<K>(q)];
    }
    unsigned char* a_tile = stage0 + s * kATileBytes;

    // ---- A: 32 codebook integers of this lane unit as fp16 (1024 + bytesum), rows 2q and 2q+1 of strip `warp`
    {
      uint32_t st[32];
      unit_states<K>(V, st);
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int row = warp * 16 + 2 * q + rr;
        unsigned char* dst = a_tile + (row >> 3) * kSbo + (row & 7) * 16 + (2 * tc) * kLbo;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t lo = bytesum_add_alu(st[rr * 16 + half * 8 + 2 * e] * kGenMul + kGenAdd, 0x6400u);
            const uint32_t hi = bytesum_add(st[rr * 16 + half * 8 + 2 * e + 1] * kGenMul + kGenAdd, 0x6400u);
            w[e] = __byte_perm(lo, hi, 0x5410);
          }
          *reinterpret_cast<uint4*>(dst + half * kLbo) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && !failed && !s_fail) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_addr = stage0_addr + s * kATileBytes, b_addr = b_stage0_addr + (ch % kBStages) * b_tile_bytes;
#pragma unroll
      for (int kk = 0; kk < kChunkK / 16; ++kk)
        umma_f16(tmem_base, umma_desc(a_addr + kk * 2 * kLbo, kSbo), umma_desc(b_addr + kk * 2 * kLbo, kSbo), idesc, (ch | kk) ? 1u : 0u);
      umma_commit(smem_u32(&s_bar[s]));
    }
    if (failed) s_fail = 1;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // ---- all MMAs of this CTA done?  (the last commit covers every earlier MMA)
  if (chunks > 0 && !failed) {
    const int s = (chunks - 1) & 1;
    if (!mbar_wait(smem_u32(&s_bar[s]), (phase_bits >> s) & 1u)) failed = true;
  }
  if (failed) s_fail = 1;
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  __syncthreads();
  const bool bad = s_fail != 0;
  if (bad && tid == 0) atomicCAS(p.error, 0, 1);

  // ---- accumulator -> registers -> shared [np][128]: thread = row of the block, hi + lo added here
  float* result = reinterpret_cast<float*>(stage0);          // the stages are idle now
  if (!bad && chunks > 0) {
    const int row = 32 * (warp & 3) + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16);
    for (int j0 = (warp >> 2) * 16; j0 < np; j0 += 32) {     // warps 0-3 and 4-7 take alternate groups of 16 batch rows
      float hi[16], lo[16];
      tmem_load16(lane_addr + j0, hi);
      if (p.planes == 2) {
        tmem_load16(lane_addr + np + j0, lo);
#pragma unroll
        for (int j = 0; j < 16; ++j) hi[j] += lo[j];
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) result[(j0 + j) * 128 + row] = hi[j];
    }
  } else {
    for (int e = tid; e < np * 128; e += kGemmThreads) result[e] = 0.f;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");

  // ---- split reduction across the CTAs of this row block (same scheme as the GEMV), then the epilogue
  bool finish = true;
  const int contributors = p.split;
  if (contributors > 1) {
    float* mine = p.part + ((size_t)rb * contributors + part_id) * ((size_t)np * 128);
    for (int e = tid; e < np * 128; e += kGemmThreads) __stcg(mine + e, result[e]);
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      s_arrival = atomicAdd(p.counters + rb, 1);
      __threadfence();
    }
    __syncthreads();
    finish = (s_arrival == contributors - 1);
    if (finish) {
      const float* slot0 = p.part + (size_t)rb * contributors * ((size_t)np * 128);
      for (int e = tid; e < np * 128; e += kGemmThreads) {
        float sum = 0.f;
        for (int sl = 0; sl < contributors; ++sl) sum += __ldcg(slot0 + (size_t)sl * np * 128 + e);
        result[e] = sum;
      }
      if (tid == 0) p.counters[rb] = 0;
    }
    __syncthreads();
  }
  if (!finish) return;
  // epilogue: one warp per activation row j; lane holds rows 4*lane .. 4*lane+3 of the block
  const int row0 = rb * 128 + 4 * lane;
  const uint2 sc_raw = __ldg(reinterpret_cast<const uint2*>(p.scales + row0));
  const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sc_raw.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&sc_raw.y));
  const unsigned sv_bits = sign_nibble(p.sv, rb * 32 + lane);
  float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (p.bias) bias4 = load_quad(p.bias, row0, p.dtype);
  for (int j = warp; j < p.rows; j += kGemmWarps) {
    const float off = 1534.0f * p.xsum[j], rs = p.cb * p.tok[j];
    float v[4] = {(result[j * 128 + 4 * lane] - off) * (s01.x * rs), (result[j * 128 + 4 * lane + 1] - off) * (s01.y * rs),
                  (result[j * 128 + 4 * lane + 2] - off) * (s23.x * rs), (result[j * 128 + 4 * lane + 3] - off) * (s23.y * rs)};
    wht128(v, lane);
    float4 o = make_float4(flip(v[0] * kInvSqrt128, sv_bits & 1u), flip(v[1] * kInvSqrt128, (sv_bits >> 1) & 1u),
                           flip(v[2] * kInvSqrt128, (sv_bits >> 2) & 1u), flip(v[3] * kInvSqrt128, sv_bits >> 3));
    o.x += bias4.x; o.y += bias4.y; o.z += bias4.z; o.w += bias4.w;
    store_quad(p.y, (size_t)j * m + row0, p.dtype, o);
  }
}

int run_rht_f16(const void* x, int dtype, int rows, int np, int n, int planes, const uint8_t* su, __half* xh, __half* xl, float* xsum,
                float* tok, cudaStream_t st);
template <int K>
int launch_packed_gemm_tc(const GemmParams& p, int grid, cudaStream_t st);

}  // namespace htr
