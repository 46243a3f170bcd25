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
// SBO bytes apart.  For A, SBO is padded by 16 bytes so that the decode threads' 16-byte stores spread over all
// banks.  The activation transform writes B to global memory already in this layout, one contiguous block per
// 64-column chunk, so a B tile arrives with a single bulk copy.
//
// Roles (576 threads).  Warps 0-15 decode: two groups of eight warps take alternate 64-column chunks; inside a group
// warp w owns the 16-row strip w of the 128-row block, fetches that strip's packed words itself (cp.async ring, the
// same scheme as the GEMV) and writes its rows of the A tile.  One lane of warp 16 brings the B tiles (one bulk copy
// per pair of chunks, completion counted on an mbarrier); one lane of warp 17 issues the MMAs.  The ring holds pairs of
// consecutive chunks (one chunk per decode group): {A tile, A tile, B tile, B tile} with a_full[s] (all sixteen decode
// warps stored and fenced), b_full[s] (bytes landed) and freed[s] (tcgen05.commit: the MMAs that read the pair have
// retired), so the MMA lane pays one round of barrier traffic per 128 columns.  No CTA-wide barrier inside the main loop.
//
// Every wait on an mbarrier is bounded: when it expires the CTA records an error code, stops issuing work, waits
// (bounded) for its copies in flight, frees its TMEM columns and returns; the host sees the code in the workspace
// header.
#pragma once
#include "htr_codec.cuh"
#include "htr_common.cuh"

namespace htr {

constexpr int kStripWarps = 8;                              // warps of one decode group = 16-row strips of a row block
constexpr int kDecodeGroups = 2;                            // groups take alternate chunks
constexpr int kGemmDecodeWarps = kStripWarps * kDecodeGroups;
constexpr int kGemmWarps = kGemmDecodeWarps + 2;            // + B-tile warp + MMA warp
constexpr int kGemmThreads = kGemmWarps * 32;
constexpr int kChunkK = 64;                                 // k extent of one stage
constexpr int kLbo = 128;                                   // bytes between core matrices adjacent in K
#ifndef HTR_GEMM_SBOA_PAD
#define HTR_GEMM_SBOA_PAD 16
#endif
#ifndef HTR_GEMM_MMAS
#define HTR_GEMM_MMAS (kChunkK / 16)
#endif
constexpr int kSboA = (kChunkK / 8) * 128 + HTR_GEMM_SBOA_PAD;   // bytes between 8-row groups of A (padded: 1040)
constexpr int kSboB = (kChunkK / 8) * 128;                  // ... of B (as written by the activation transform)
constexpr int kATileBytes = (128 / 8) * kSboA;              // 16640
constexpr int kMaxStages = 3;                               // stage pairs in flight (2..3, chosen by the host); a pair = two consecutive
                                                            // chunks, one per decode group: {A tile, A tile, B tile, B tile}
constexpr unsigned kSpinLimit = 4000000u;                   // iterations of a try_wait loop before giving up
constexpr int kGemmMaxCols = 256;                           // accumulator columns (activation rows x planes) per launch
#ifndef HTR_GEMM_WAIT_HINT
#define HTR_GEMM_WAIT_HINT 200
#endif
#ifndef HTR_GEMM_PACK_MODE
#define HTR_GEMM_PACK_MODE 1
#endif
// packed-word ring of a decode warp: chunks in flight + the one being read
#ifndef HTR_GEMM_RAW_SLOTS
#define HTR_GEMM_RAW_SLOTS(K) ((K) <= 2 ? 6 : (K) <= 3 ? 5 : 4)
#endif
__host__ __device__ constexpr int gemm_raw_slots(int K) { return HTR_GEMM_RAW_SLOTS(K); }

struct GemmParams {
  const uint32_t* qw;
  const __half* scales;
  const uint8_t* sv;
  const void* bias;
  void* y;
  const __half* xb;       // transformed activations, [chunk][column group of 8][8 k-groups][8 columns][8 k] fp16:
                          // columns 0..np-1 = hi plane of the activation rows, np..2np-1 = lo plane (planes == 2)
  const float* xsum;      // [np][xsum_slices] sums over k (per 1024-column slice) of the planes in use (hi, or hi + lo)
  const float* tok;       // [np] power-of-two range scale per activation row
  float* part;            // [row blocks][slots][np][128]
  int* counters;          // [row blocks]
  int* error;             // one word: first failure code seen by any CTA (0 = none)
  int rows, np;           // activation rows present / padded to a multiple of 16
  int planes;             // 1: hi plane only (16-bit activations), 2: hi + lo (float32 activations)
  int mt, nt;
  int dtype;
  int hb;                 // 128-column blocks per row (n / 128) = units per row block
  int split;              // CTAs per row block
  int cluster;            // 1: the CTAs of a row block were launched as one thread-block cluster (split <= 8): the split reduction
                          // goes through distributed shared memory instead of global partial sums
  int stages;             // stage pairs in the ring (2..kMaxStages)
  int xsum_slices;
  float cb;
  // row-shard form: the output rows go, with plain peer stores, to element offset peer_offset + j * m + row of every buffer in
  // peer_y (the gather buffers of all ranks of an NVLink box as mapped into this process) instead of y
  void* peer_y[8];
  int npeer;
  long long peer_offset;
};

__device__ __forceinline__ void gemm_store_rows(const GemmParams& p, int j, int m, int row0, float4 o) {
  if (p.npeer == 0) {
    store_quad(p.y, (size_t)j * m + row0, p.dtype, o);
  } else {
#pragma unroll 1
    for (int pe = 0; pe < p.npeer; ++pe) store_quad(p.peer_y[pe], (size_t)p.peer_offset + (size_t)j * m + row0, p.dtype, o);
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, int sbo_bytes) {
  // start address, LBO, SBO in 16-byte units; descriptor version 1 (sm_100); layout type 0 = no swizzle
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((kLbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) |
         (1ull << 46);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// bounded wait for the phase with the given parity; false when the limit ran out or another role has already failed
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const volatile int* fail) {
  for (unsigned it = 0; it < kSpinLimit; ++it) {
    uint32_t done;
#if HTR_GEMM_WAIT_HINT > 0
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"((unsigned)HTR_GEMM_WAIT_HINT)
        : "memory");
#else
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
#endif
    if (done) return true;
    if ((it & 255u) == 255u && *fail) return false;
  }
  return false;
}

// the same without the early exit: used on the failure path to let copies and MMAs in flight drain
__device__ __forceinline__ bool mbar_wait_plain(uint32_t bar, uint32_t parity) {
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

// global -> shared bulk copy (16-byte aligned, size a multiple of 16), completion counted in bytes on an mbarrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
               "r"(bar)
               : "memory");
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

// dynamic shared memory: stages {A tile, B tile}, then the packed-word rings of the decode warps -- later reused for
// the [np][128] float result
__host__ __device__ inline int gemm_stage_bytes(int ncols) { return kDecodeGroups * (kATileBytes + ncols * 128); }   // one pair
__host__ __device__ inline int gemm_smem_bytes(int np, int planes, int K, int stages) {
  const int pipe = stages * gemm_stage_bytes(np * planes) + kGemmDecodeWarps * gemm_raw_slots(K) * (4 * 32 * K);
  const int result = np * 128 * 4;
  return (pipe > result ? pipe : result) + 128;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

template <int K>
__global__ void __launch_bounds__(kGemmThreads) packed_gemm_tc_kernel(const GemmParams p) {
  extern __shared__ __align__(128) unsigned char gsm[];
  __shared__ __align__(8) unsigned long long s_afull[kMaxStages], s_bfull[kMaxStages], s_freed[kMaxStages], s_done;
  __shared__ uint32_t s_tmem;
  __shared__ int s_arrival;
  __shared__ volatile int s_fail;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int np = p.np, ncols = p.planes * np;               // accumulator columns: hi plane, then lo plane if present
  const int nt = p.nt, m = p.mt * 16, HB = p.hb, NS = p.stages;
  const int rb = blockIdx.x / p.split, part_id = blockIdx.x - rb * p.split;
  const int hb_begin = part_id * HB / p.split, hb_end = (part_id + 1) * HB / p.split;
  const int chunks = (hb_end - hb_begin) * 2;                // two 64-column chunks per 128-column block
  constexpr int kStripBytes = 4 * 32 * K, R = gemm_raw_slots(K);
  const int b_tile_bytes = ncols * 128, stage_bytes = kDecodeGroups * (kATileBytes + b_tile_bytes);   // pair: A0 | A1 | B0 | B1
  unsigned char* stage0 = gsm + (128 - (smem_u32(gsm) & 127)) % 128;   // 128-byte aligned start: stage s = {A tile, B tile}
  unsigned char* raw0 = stage0 + NS * stage_bytes;                     // packed-word rings [decode warp][slot][4 tiles][8K words]
  const uint32_t stage0_addr = smem_u32(stage0), raw0_addr = smem_u32(raw0);

  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < ncols) tmem_cols <<= 1;
  if (tid == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&s_afull[s]), kGemmDecodeWarps);              // one arrival per decode warp (both groups)
      mbar_init(smem_u32(&s_bfull[s]), 1);                             // the B lane's arrive.expect_tx
      mbar_init(smem_u32(&s_freed[s]), 1);                             // tcgen05.commit
    }
    mbar_init(smem_u32(&s_done), 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  if (warp < kGemmDecodeWarps) {
    // ================= decode warps: group = warp / 8 takes chunks group, group + 2, ...; strip = warp % 8;
    // inside the strip: tile column tc = lane >> 3, row pair q = lane & 7
    const int group = warp / kStripWarps, strip = warp % kStripWarps;
    const int tc = lane >> 3, q = lane & 7;
    const uint32_t ring_addr = raw0_addr + warp * (R * kStripBytes);
    const unsigned char* ring = raw0 + warp * (R * kStripBytes);
    const char* wsrc = reinterpret_cast<const char*>(p.qw) + ((size_t)(rb * 8 + strip) * nt + (size_t)hb_begin * 8) * (32 * K);
    // asynchronous fetch of chunk c (contiguous: four tiles of this strip) into ring slot `slot`; always commits a group
    auto prefetch = [&](int c, int slot) {
      if (c < chunks) {
        const char* src = wsrc + (size_t)c * kStripBytes;
        const uint32_t dst = ring_addr + slot * kStripBytes;
#pragma unroll
        for (int j = 0; j < (kStripBytes / 16 + 31) / 32; ++j)
          if (32 * j + 32 <= kStripBytes / 16 || lane + 32 * j < kStripBytes / 16) cp_async16(dst + (lane + 32 * j) * 16, src + (lane + 32 * j) * 16);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int i = 0; i < R - 1; ++i) prefetch(group + kDecodeGroups * i, i);   // the weights do not depend on the preceding kernel
    // the barriers and the TMEM address become visible here (first CTA-wide barrier)
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    const int hist = history_word<K>(q);
    const int row_a = strip * 16 + 2 * q;
    const uint32_t a_off = (uint32_t)((row_a >> 3) * kSboA + (row_a & 7) * 16 + (2 * tc) * kLbo);
    int slot = 0;
    int st_idx = 0;                                         // ring slot of the pair (c / 2) % NS
    uint32_t use = 0u;                                      // how many times that slot was used before this pair
    bool ok = true;
    for (int c = group; c < chunks; c += kDecodeGroups) {
      asm volatile("cp.async.wait_group %0;" ::"n"(R - 2) : "memory");   // this chunk's words have landed (own copies) ...
      __syncwarp();                                                       // ... and those of the other lanes; slot of the previous chunk is free
      prefetch(c + kDecodeGroups * (R - 1), slot == 0 ? R - 1 : slot - 1);
      uint32_t V[K + 1];
      {
        const uint32_t* tile = reinterpret_cast<const uint32_t*>(ring + slot * kStripBytes) + tc * (8 * K);
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
        V[0] = tile[hist];
      }
      // the MMAs that read this ring slot (NS pairs ago) must have retired
      if (use > 0 && !__all_sync(kFullWarp, mbar_wait(smem_u32(&s_freed[st_idx]), (use - 1u) & 1u, &s_fail))) { ok = false; break; }
      unsigned char* dst0 = stage0 + st_idx * stage_bytes + group * kATileBytes + a_off;
      // 32 codebook integers of this lane unit as fp16 (1024 + bytesum): rows 2q and 2q+1 of the strip, 16 k each
      uint32_t st[32];
      unit_states<K>(V, st);
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
#if HTR_GEMM_PACK_MODE == 0
            const uint32_t lo = bytesum_add_alu(st[rr * 16 + half * 8 + 2 * e] * kGenMul + kGenAdd, 0x6400u);
            const uint32_t hi = bytesum_add(st[rr * 16 + half * 8 + 2 * e + 1] * kGenMul + kGenAdd, 0x6400u);
            w[e] = __byte_perm(lo, hi, 0x5410);
#elif HTR_GEMM_PACK_MODE == 1
            const uint32_t lo = bytesum_add(st[rr * 16 + half * 8 + 2 * e] * kGenMul + kGenAdd, 0x6400u);
            const uint32_t hi = bytesum_add(st[rr * 16 + half * 8 + 2 * e + 1] * kGenMul + kGenAdd, 0x6400u);
            w[e] = hi * 65536u + lo;                         // multiply-add: keeps the pack off the shift/logic pipe
#else
            const uint32_t lo = bytesum_add_alu(st[rr * 16 + half * 8 + 2 * e] * kGenMul + kGenAdd, 0x6400u);
            const uint32_t hi = bytesum_add(st[rr * 16 + half * 8 + 2 * e + 1] * kGenMul + kGenAdd, 0x6400u);
            w[e] = hi * 65536u + lo;
#endif
          }
          *reinterpret_cast<uint4*>(dst0 + rr * 16 + half * kLbo) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_afull[st_idx]));
      if (++slot == R) slot = 0;
      if (++st_idx == NS) { st_idx = 0; ++use; }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (!ok) s_fail = 1;
  } else {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == kGemmDecodeWarps) {
      // ================= B lane: one bulk copy per chunk (the activation transform wrote the tiles contiguously)
      if (lane == 0) {
        asm volatile("griddepcontrol.wait;" ::: "memory");   // the transformed activations come from the preceding kernel
        const char* bsrc = reinterpret_cast<const char*>(p.xb) + (size_t)(hb_begin * 2) * b_tile_bytes;
        int s = 0, issued = 0;
        uint32_t use = 0u;
        const uint32_t pair_b_bytes = (uint32_t)(kDecodeGroups * b_tile_bytes);
        for (int pr = 0; pr < chunks / kDecodeGroups; ++pr) {      // the B tiles of a pair are contiguous in global memory: one copy
          if (use > 0 && !mbar_wait(smem_u32(&s_freed[s]), (use - 1u) & 1u, &s_fail)) { s_fail = 1; break; }
          const uint32_t bar = smem_u32(&s_bfull[s]);
          mbar_expect_tx(bar, pair_b_bytes);
          bulk_load(stage0_addr + s * stage_bytes + kDecodeGroups * kATileBytes, bsrc + (size_t)pr * pair_b_bytes, pair_b_bytes, bar);
          ++issued;
          if (++s == NS) { s = 0; ++use; }
        }
        if (s_fail) {
          // copies still in flight write into this CTA's shared memory: wait (bounded) for every slot last filled
          for (int pr = issued > NS ? issued - NS : 0; pr < issued; ++pr) mbar_wait_plain(smem_u32(&s_bfull[pr % NS]), (uint32_t)(pr / NS) & 1u);
        }
      }
    } else if (lane == 0) {
      // ================= MMA lane
      const uint32_t tmem_acc = s_tmem;
      // instruction descriptor: D = f32, A = B = f16, both K-major, M = 128, N = ncols
      const uint32_t idesc = (1u << 4) | ((uint32_t)(ncols >> 3) << 17) | ((128u >> 4) << 24);
      int s = 0;
      uint32_t ph = 0u;
      bool ok = true;
      for (int pr = 0; pr < chunks / kDecodeGroups; ++pr) {
        if (!mbar_wait(smem_u32(&s_afull[s]), ph, &s_fail)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&s_bfull[s]), ph, &s_fail)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = stage0_addr + s * stage_bytes, b_addr = a_addr + kDecodeGroups * kATileBytes;
#pragma unroll
        for (int g = 0; g < kDecodeGroups; ++g)
#pragma unroll
          for (int kk = 0; kk < HTR_GEMM_MMAS; ++kk)
            umma_f16(tmem_acc, umma_desc(a_addr + g * kATileBytes + kk * 2 * kLbo, kSboA), umma_desc(b_addr + g * b_tile_bytes + kk * 2 * kLbo, kSboB),
                     idesc, (pr | g | kk) ? 1u : 0u);
        umma_commit(smem_u32(&s_freed[s]));
        if (++s == NS) { s = 0; ph ^= 1u; }
      }
      umma_commit(smem_u32(&s_done));                        // covers every MMA issued above
      if (!ok) {
        s_fail = 1;                                          // the other threads stop waiting at once ...
        mbar_wait_plain(smem_u32(&s_done), 0u);              // ... this one lets the MMAs in flight retire first
      }
    }
    __syncwarp();
  }
  const uint32_t tmem_base = s_tmem;

  // ---- all MMAs of this CTA done?
  if (!mbar_wait(smem_u32(&s_done), 0u, &s_fail)) s_fail = 1;
  asm volatile("griddepcontrol.wait;" ::: "memory");         // row sums / scales of the activations, scratch of earlier launches
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  __syncthreads();
  const bool bad = s_fail != 0;
  if (bad && tid == 0) atomicCAS(p.error, 0, 1);

  // ---- accumulator -> registers -> shared [np][128]: thread = row of the block, hi + lo added here
  float* result = reinterpret_cast<float*>(stage0);          // the stages are idle now
  if (!bad) {
    if (warp < 16) {
      const int row = 32 * (warp & 3) + lane;                // a warp reads the TMEM lanes of its quadrant (warp % 4)
      const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16);
      for (int j0 = (warp >> 2) * 16; j0 < np; j0 += 64) {   // the four warps of a quadrant take alternate groups of 16 batch rows
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
    }
  } else {
    // a bounded wait gave up: the rows of this block come out as NaN (visible to any consumer), beside the error word
    for (int e = tid; e < np * 128; e += kGemmThreads) result[e] = __uint_as_float(0x7FC00000u);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");

  if (p.cluster) {
    // ---- split reduction inside the cluster: every CTA keeps its partial [np][128] where it is; CTA r of the cluster sums rows
    // r, r + split, ... over all CTAs (in rank order: the same additions as the global path) and finishes those rows itself
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    const int row0 = rb * 128 + 4 * lane;
    const uint2 sc_raw = __ldg(reinterpret_cast<const uint2*>(p.scales + row0));
    const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sc_raw.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&sc_raw.y));
    const unsigned sv_bits = sign_nibble(p.sv, rb * 32 + lane);
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p.bias) bias4 = load_quad(p.bias, row0, p.dtype);
    const uint32_t result_addr = smem_u32(result);
    for (int j = part_id + p.split * warp; j < p.rows; j += p.split * kGemmWarps) {
      float4 r4 = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < p.split; ++r) {
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(result_addr + (uint32_t)(j * 128 + 4 * lane) * 4u), "r"(r));
        float4 v;
        asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
        r4.x += v.x; r4.y += v.y; r4.z += v.z; r4.w += v.w;
      }
      float xs = 0.f;
      for (int y = 0; y < p.xsum_slices; ++y) xs += p.xsum[j * p.xsum_slices + y];
      const float off = 1534.0f * xs, rs = p.cb * p.tok[j];
      float v[4] = {(r4.x - off) * (s01.x * rs), (r4.y - off) * (s01.y * rs), (r4.z - off) * (s23.x * rs), (r4.w - off) * (s23.y * rs)};
      wht128(v, lane);
      float4 o = make_float4(flip(v[0] * kInvSqrt128, sv_bits & 1u), flip(v[1] * kInvSqrt128, (sv_bits >> 1) & 1u),
                             flip(v[2] * kInvSqrt128, (sv_bits >> 2) & 1u), flip(v[3] * kInvSqrt128, sv_bits >> 3));
      o.x += bias4.x; o.y += bias4.y; o.z += bias4.z; o.w += bias4.w;
      gemm_store_rows(p, j, m, row0, o);
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // nobody leaves while its shared memory may still be read
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    return;
  }

  // ---- split reduction across the CTAs of this row block (same scheme as the GEMV), then the epilogue
  bool finish = true;
  const int contributors = p.split;
  if (contributors > 1) {
    float4* mine = reinterpret_cast<float4*>(p.part + ((size_t)rb * contributors + part_id) * ((size_t)np * 128));
    for (int e = tid; e < np * 32; e += kGemmThreads) __stcg(mine + e, reinterpret_cast<const float4*>(result)[e]);
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      s_arrival = atomicAdd(p.counters + rb, 1);
      __threadfence();
    }
    __syncthreads();
    finish = (s_arrival == contributors - 1);
    if (finish) {
      const float4* slot0 = reinterpret_cast<const float4*>(p.part + (size_t)rb * contributors * ((size_t)np * 128));
      for (int e = tid; e < np * 32; e += kGemmThreads) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sl = 0; sl < contributors; ++sl) {
          const float4 v = __ldcg(slot0 + (size_t)sl * np * 32 + e);
          sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        reinterpret_cast<float4*>(result)[e] = sum;
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
    float xs = 0.f;
    for (int y = 0; y < p.xsum_slices; ++y) xs += p.xsum[j * p.xsum_slices + y];   // fixed order: results do not depend on scheduling
    const float off = 1534.0f * xs, rs = p.cb * p.tok[j];
    const float4 r4 = *reinterpret_cast<const float4*>(result + j * 128 + 4 * lane);
    float v[4] = {(r4.x - off) * (s01.x * rs), (r4.y - off) * (s01.y * rs), (r4.z - off) * (s23.x * rs), (r4.w - off) * (s23.y * rs)};
    wht128(v, lane);
    float4 o = make_float4(flip(v[0] * kInvSqrt128, sv_bits & 1u), flip(v[1] * kInvSqrt128, (sv_bits >> 1) & 1u),
                           flip(v[2] * kInvSqrt128, (sv_bits >> 2) & 1u), flip(v[3] * kInvSqrt128, sv_bits >> 3));
    o.x += bias4.x; o.y += bias4.y; o.z += bias4.z; o.w += bias4.w;
    gemm_store_rows(p, j, m, row0, o);
  }
}

int gemm_rht_slices(int np, int n);
int run_rht_f16(const void* x, int dtype, int rows, int np, int n, int planes, const uint8_t* su, __half* xb, float* xsum, float* tok,
                cudaStream_t st);
template <int K>
int launch_packed_gemm_tc(const GemmParams& p, int grid, cudaStream_t st);

}  // namespace htr
