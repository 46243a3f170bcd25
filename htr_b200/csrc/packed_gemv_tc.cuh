// Packed GEMV for HTR-W1 weights on the sm_100a tensor cores: the hash words themselves are the A operand.
//
//   y = sv * Ho( diag(scale * CB) * V * Hi(su * x) ),  V[i,j] = bytesum(h_ij) - 510,  h_ij = (s_ij * 0xDF6ADF + 0x34983) mod 2^32
//
// (docs/FORMAT.md:7-13 of the reference; the same linear as packed_gemv.cuh, which it replaces for up to four activation rows.)
//
// Idea.  A codebook integer is the sum of the four bytes of a 32-bit hash.  An 8-bit integer MMA whose A operand holds the
// hash word as four consecutive u8 k-elements and whose B operand holds the activation four times (one s8 value splatted over
// the four k-elements) computes sum_j bytesum(h_ij) * q_j: byte sum, multiply and accumulate of a weight cost no instruction
// of the decoding threads at all.  What is left per weight is the window extraction, one multiply-add for the hash, and 1/16 of
// a tcgen05.st that puts sixteen hash words of one row into tensor memory, where tcgen05.mma (kind::i8, A from TMEM, B from shared
// memory, s32 accumulators in TMEM) picks them up.
//
// Activations.  The transformed activations of a window of columns are split into four signed 7-bit planes around a
// power-of-two scale, xt * sc = q0 + q1/128 + q2/128^2 + q3/128^3 (|q| <= 64, 27 bits: more than a float32 holds), one B
// column per (activation row, plane): N = 16 = 4 rows x 4 planes.  The accumulators are exact integers; the constant 510 is
// removed with the exact plane sums, the planes are recombined in 64-bit integers and leave the integer domain with a single
// rounding per window.  Results therefore do not depend on the order of anything.
//
// Decomposition, split reduction, epilogue, launch overlap: as in packed_gemv.cuh (same GemvParams, same plan, same
// workspace).  Inside a CTA (384 threads at <= 80 registers, two CTAs per SM, 256 TMEM columns each):
//   * warps 0-7 decode.  Warp = (quarter qd = warp & 3, unit slot cs = warp >> 2); the two slots take alternate units
//     (unit = 128 rows x 64 columns).  Thread t of quarter qd owns row 32 qd + t of the row block = TMEM lane 32 qd + t,
//     i.e. one tile row of four consecutive tiles per unit: 64 weights = four tcgen05.st of 16 words.  The packed words travel
//     global -> shared memory through a per-warp cp.async ring as in the other kernels.
//   * lane 0 of warps 8-11 issues the MMAs ("MMA lanes", two per slot): per unit 8 instructions of K = 32 bytes (8 columns
//     of A), four per lane, into the lane's own 16 accumulator columns (32 columns apart); tcgen05.commit frees the A stage
//     (two stages of 64 TMEM columns, used in turn).  One thread gets an MMA of this size out only every 45 cycles at best (measured; ~150 in
//     this kernel), whatever N up to 64: hence several lanes.
// A window of activations (1536 columns for one or two rows, 768 for three or four) ends with a drain: all MMAs retired,
// accumulators read out (tcgen05.ld) and converted, next window staged.
//
// Every wait on an mbarrier is bounded; when one expires the CTA stops issuing work, lets copies and MMAs in flight finish
// (bounded), frees its TMEM columns, counts the failure in a device counter the host can read (htr_gemv_tc_failures), and
// writes NaN results.
//
// Status: correct (bit-stable, exact integer accumulation) but slower than the CUDA-core GEMV at every size measured so far;
// the library therefore uses it only on request (htr_set_gemv_tc / HTR_GEMV_TC=1).
#pragma once
#include <cstdio>

#include "packed_gemm_tc.cuh"
#include "packed_gemv.cuh"

namespace htr {

constexpr int kTcDecodeWarps = 8;
constexpr int kTcSlots = 2;                                // decode warp groups taking alternate units
constexpr int kTcLanes = 2 * kTcSlots;                     // MMA lanes: two per slot, each issues half of a unit's MMAs
constexpr int kTcWarps = kTcDecodeWarps + kTcLanes;
constexpr int kTcThreads = kTcWarps * 32;                 // 384: 3 warps per scheduler, two CTAs per SM at <= 80 registers
// TMEM columns between the accumulators of two MMA lanes.  Each accumulator is 16 columns wide, but they must not share a
// 32-column granule: with a spacing of 16, MMAs issued concurrently by two threads into neighbouring accumulators gave a wrong
// sum about once in 5000 launches and, rarely, an MMA that never completed (24000 launches each way: 5 + 1 against 0 + 0).
constexpr int kTcDStride = 32;
constexpr int kTcStages = 2;                               // A stages in TMEM, used in turn by the units of a CTA
constexpr int kTcStageCols = 64;                           // one unit: 64 weights per row
constexpr int kTcAcol0 = 4 * kTcDStride;                   // first A column (the accumulators of the four MMA lanes come first)
constexpr int kTcTmemCols = 256;
constexpr int kTcWinBytes = 48 * 1024;                     // B operand of one window of activations
constexpr int kTcRows = 4;                                 // activation rows per launch (x 4 planes = 16 accumulator columns)
// B operand of one unit: 16 k-groups x n-groups x (8 x 16 bytes).  With one or two activation rows only the first n-group
// (8 accumulator columns) carries data: it is stored alone and the descriptor repeats it for the second one (stride 0), whose
// accumulator columns nobody reads.  So a window holds 24 units (1536 columns) for up to two rows and 12 units for three or four.
__host__ __device__ constexpr int tc_unit_b_bytes(int rows) { return rows <= 2 ? 16 * 128 : 16 * 2 * 128; }

__host__ __device__ constexpr int tc_ring_slots(int K) { return K <= 3 ? 6 : K == 4 ? 5 : K <= 6 ? 4 : 3; }
__host__ __device__ constexpr int tc_slot_bytes(int K) { return 2 * 4 * 32 * K; }   // two strips x four tiles
__host__ __device__ constexpr int gemv_tc_smem_bytes(int K) {
  return kTcWinBytes + kTcDecodeWarps * tc_ring_slots(K) * tc_slot_bytes(K) + 128 + 64;
}

// D[128 x 16] (+)= A[128 x 32 u8, TMEM] * B[32 x 16 s8, shared memory]
__device__ __forceinline__ void umma_i8_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

__device__ __forceinline__ void tmem_store16(uint32_t taddr, const uint32_t (&h)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
               "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]), "r"(h[4]), "r"(h[5]), "r"(h[6]), "r"(h[7]), "r"(h[8]), "r"(h[9]), "r"(h[10]), "r"(h[11]),
               "r"(h[12]), "r"(h[13]), "r"(h[14]), "r"(h[15])
               : "memory");
}

__device__ __forceinline__ void tmem_load16_s32(uint32_t taddr, int (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
        "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// bounded wait with an explicit suspend-time hint (nanoseconds the hardware may park the thread before it looks again)
__device__ __forceinline__ bool mbar_wait_hint(uint32_t bar, uint32_t parity, const volatile int* fail, uint32_t hint_ns) {
  for (unsigned it = 0; it < kSpinLimit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    if (done) return true;
    if ((it & 255u) == 255u && *fail) return false;
  }
  return false;
}

namespace detail {
template <int K, int... CHAIN>
HTR_HD void row_pairs(const uint32_t (&V)[K + 1], uint32_t (&s)[32], std::integer_sequence<int, CHAIN...>) {
  constexpr int P = PairStride<K>::value;
  (pair_chain<K, CHAIN>(V, s, std::make_integer_sequence<int, 8 / P>{}), ...);
}
template <int K, int... U>
HTR_HD void row_singles(const uint32_t (&V)[K + 1], uint32_t (&s)[32], std::integer_sequence<int, U...>) {
  ((s[U] = window16<K, 16 + (U + 1) * K>(V)), ...);
}
}  // namespace detail

// The 16 states of one tile row.  V[0] holds the 16 history bits in its low half, V[1..] the row's own bits from bit 0 on
// (the layout of a lane unit in htr_codec.cuh, cut after 16 steps); s[0..15] are written.
template <int K>
HTR_HD void row_states(const uint32_t (&V)[K + 1], uint32_t (&s)[32]) {
  if constexpr (PairStride<K>::value > 1) detail::row_pairs<K>(V, s, std::make_integer_sequence<int, PairStride<K>::value>{});
  else detail::row_singles<K>(V, s, std::make_integer_sequence<int, 16>{});
}

// words of V a tile row needs: the history word and ceil(16 K / 32) own words
template <int K>
struct RowWords {
  static constexpr int value = 1 + (16 * K + 31) / 32;
};

// Loads V for tile row r (0..15) of a tile that sits in shared memory (8K words, circular).
template <int K>
__device__ __forceinline__ void read_row_words(const uint32_t* __restrict__ tile, int r, uint32_t (&V)[K + 1]) {
  constexpr int NW = RowWords<K>::value;
#pragma unroll
  for (int i = NW; i < K + 1; ++i) V[i] = 0u;
  if constexpr (K % 2 == 0) {
    // 16 K bits = K/2 whole words per row: the row starts at word r K/2, the history is the low half of the word before it
    const int w0 = r * (K / 2);
    V[0] = tile[w0 == 0 ? 8 * K - 1 : w0 - 1];
    if constexpr (K == 4) {
      const uint2 t = *reinterpret_cast<const uint2*>(tile + w0);
      V[1] = t.x; V[2] = t.y;
    } else if constexpr (K == 8) {
      const uint4 t = *reinterpret_cast<const uint4*>(tile + w0);
      V[1] = t.x; V[2] = t.y; V[3] = t.z; V[4] = t.w;
    } else {
#pragma unroll
      for (int i = 0; i < K / 2; ++i) V[1 + i] = tile[w0 + i];
    }
  } else {
    // odd K: odd rows start in the middle of a word.  X[0] is the word that holds the history bits; for rows that start at
    // bit 16 of it the whole run is moved down by 16 bits so that both cases share the window positions.
    const int e = r * K, wb = (e - 1) >> 1, sh = (e & 1) * 16;
    uint32_t X[NW];
    X[0] = tile[wb < 0 ? 8 * K - 1 : wb];
#pragma unroll
    for (int i = 1; i < NW; ++i) X[i] = tile[wb + i];          // the last one may lie past the tile (then unused): the ring is padded
    V[0] = __funnelshift_r(X[0], 0u, sh);
#pragma unroll
    for (int i = 1; i < NW; ++i) V[i] = __funnelshift_r(X[i], X[i - 1], sh);
  }
}

// failures (expired waits) since the library was loaded, over all launches of this kernel on this device
static __device__ int htr_gemv_tc_failures_dev = 0;
// where the last one happened: wait kind (1 freed, 2 operand ready, 3 window done) << 28 | window << 24 | unit of the CTA << 12 | block
static __device__ unsigned htr_gemv_tc_last_failure_dev = 0u;
__device__ __forceinline__ void tc_note_failure(unsigned kind, unsigned window, unsigned unit) {
  htr_gemv_tc_last_failure_dev = (kind << 28) | ((window & 15u) << 24) | ((unit & 4095u) << 12) | (blockIdx.x & 4095u);
}

#ifdef HTR_GEMV_TC_TRACE
// timeline probe for experiments: per-CTA %globaltimer stamps, compiled only on request
static __device__ unsigned long long htr_tc_trace_buf[512 * 160];
__device__ __forceinline__ void tc_stamp(int slot) {
  if (blockIdx.x < 512 && slot < 160) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    htr_tc_trace_buf[blockIdx.x * 160 + slot] = t;
  }
}
#define HTR_TTRACE(cond, slot) do { if (cond) tc_stamp(slot); } while (0)
#define HTR_TFAIL(...) printf(__VA_ARGS__)
#else
#define HTR_TTRACE(cond, slot)
#define HTR_TFAIL(...)
#endif

template <int K>
__global__ void __launch_bounds__(kTcThreads, 2) packed_gemv_tc_kernel(const GemvParams p) {
  extern __shared__ __align__(128) unsigned char tsm[];
  __shared__ __align__(8) unsigned long long s_afull[kTcStages], s_freed[kTcStages], s_done[kTcLanes];
  __shared__ uint32_t s_tmem;
  __shared__ int s_arrival;
  __shared__ volatile int s_fail;
  __shared__ unsigned s_amax[2][kTcRows];            // per window parity: max |xt| bits per activation row
  __shared__ int s_psum[2][kTcRows * 4];             // per window parity: plane sums over the columns this CTA consumes
  __shared__ float s_row_inv[kTcRows];
  __shared__ float s_ss[kTcWarps];
  __shared__ __align__(16) float ytil[kTcRows * 128];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qd = warp & 3, cs = warp >> 2;           // decode warps only
  HTR_TTRACE(tid == 0, 0);
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
  const int total = u_end - u_begin;
  constexpr int kTileBytes = 32 * K, kSlotBytes = tc_slot_bytes(K), R = tc_ring_slots(K), kSlotChunks = kSlotBytes / 16;

  unsigned char* bwin = tsm + (128 - (smem_u32(tsm) & 127)) % 128;              // B operand of the window, [unit][k-group][n-group][8][16]
  unsigned char* ring0 = bwin + kTcWinBytes;                    // [decode warp][slot][strip of the pair][tile][8K words]
  const uint32_t bwin_addr = smem_u32(bwin);

  if (tid == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(smem_u32(&s_afull[s]), kTcDecodeWarps / kTcSlots);            // the four quarter warps of one slot
      mbar_init(smem_u32(&s_freed[s]), kTcLanes / kTcSlots);                   // tcgen05.commit of the slot's two MMA lanes
    }
    for (int g = 0; g < kTcLanes; ++g) mbar_init(smem_u32(&s_done[g]), 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < 2 * kTcRows) (&s_amax[0][0])[tid] = 0u;
  if (tid < 2 * kTcRows * 4) (&s_psum[0][0])[tid] = 0;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "n"(kTcTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    HTR_TTRACE(tid == 0, 3);
  }

  int rb = u_begin / CG, cgi = u_begin - rb * CG;
  const int unit_b = tc_unit_b_bytes(p.rows), ng_stride = p.rows <= 2 ? 0 : 128, kg_stride = p.rows <= 2 ? 128 : 256;
  const int win_blocks = kTcWinBytes / unit_b / 2;    // 128-column blocks of activations per window

  // ---- packed-word ring of this decode warp: units cs, cs + 2, ... of the CTA's range, R - 1 of them in flight
  const uint32_t ring_addr = smem_u32(ring0) + warp * (R * kSlotBytes);
  const unsigned char* ring = ring0 + warp * (R * kSlotBytes);
  const size_t strip_stride = (size_t)nt * kTileBytes;
  int pf_i = cs, pf_rb = rb, pf_cgi = cgi + cs;
  if (pf_cgi >= CG) { pf_cgi -= CG; ++pf_rb; }
  auto prefetch = [&](int slot) {
    if (pf_i < total) {
      const char* src = reinterpret_cast<const char*>(p.qw) + ((size_t)(pf_rb * 8 + 2 * qd) * nt + (size_t)4 * pf_cgi) * kTileBytes;
      const uint32_t dst = ring_addr + slot * kSlotBytes;
#pragma unroll
      for (int j = 0; j < (kSlotChunks + 31) / 32; ++j) {
        const int ch = lane + 32 * j;
        if (32 * j + 32 <= kSlotChunks || ch < kSlotChunks) {
          const int sp = ch >= kSlotChunks / 2 ? 1 : 0;
          cp_async16(dst + ch * 16, src + (sp ? strip_stride : 0) + (size_t)(ch - sp * (kSlotChunks / 2)) * 16);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    pf_i += kTcSlots;
    pf_cgi += kTcSlots;
    if (pf_cgi >= CG) { pf_cgi -= CG; ++pf_rb; }
  };
  if (warp < kTcDecodeWarps) {
#pragma unroll
    for (int i = 0; i < R - 1; ++i) prefetch(i);       // the weights never depend on the preceding kernel
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  bool predecessor_done = false;
  if (!p.independent) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    predecessor_done = true;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();                                     // barriers, TMEM address, zeroed window statistics
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem;
  HTR_TTRACE(tid == 0, 1);

  if (p.prologue == 1) {
    // RMSNorm fused into the activation staging: every CTA finds the row scales itself (the rows are a few KB in L2)
    for (int r = 0; r < p.rows; ++r) {
      float ss = 0.f;
      for (int e = tid; e < (n >> 2); e += kTcThreads) {
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
        for (int k = 0; k < kTcWarps; ++k) tot += s_ss[k];
        s_row_inv[r] = rsqrtf(tot / (float)n + p.eps);
      }
    }
    __syncthreads();
  }

  // instruction descriptor: D = s32, A = u8, B = s8, both K-major, M = 128, N = 16
  constexpr uint32_t kIdesc = (2u << 4) | (0u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

  float accf[kTcRows] = {0.f, 0.f, 0.f, 0.f};        // rows of the block owned by this thread (slot-0 decode warps), summed over windows
  int done_i = 0;                                      // units of the range consumed so far (all roles count alike)
  int ring_slot = 0;
  uint32_t window = 0u;                                // windows finished so far (parity of s_done, index of the statistics)
  bool bad = false;

  int u = u_begin;
  while (u < u_end) {
    // ---- window: units [u, u + seg_units) lie in row block rb and inside kTcBlocks staged 128-column blocks
    const int hb0 = cgi >> 1;
    const int cg_stop = min(CG, cgi + (u_end - u));
    const int hb1 = min(hb0 + win_blocks, (cg_stop + 1) >> 1);
    const int seg_cg_end = min(cg_stop, hb1 * 2);
    const int seg_units = seg_cg_end - cgi;
    const int wp = window & 1u;
    // three rows are staged as four (a row of zeros): every B column of the window is then written by this launch
    const int nblk = hb1 - hb0, items = (p.rows == 3 ? 4 : p.rows) * nblk;

    // -- stage 1: transform the activations of the window, find the range of every row
    constexpr int kStageRounds = 2;                    // rows x blocks <= 2 x 12 or 4 x 6 = 24 items over 12 warps
    float xv[kStageRounds][4];
    {
#pragma unroll
      for (int it = 0; it < kStageRounds; ++it) {
        const int item = warp + it * kTcWarps;
        xv[it][0] = xv[it][1] = xv[it][2] = xv[it][3] = 0.f;
        if (item < items) {
          const int r = item / nblk, hb = hb0 + item % nblk;
          const float4 x4 = r < p.rows ? fused_x(p, p.x, r, hb * 128 + 4 * lane, p.prologue == 1 ? s_row_inv[r] : 1.f) : make_float4(0.f, 0.f, 0.f, 0.f);
          const unsigned sg = sign_nibble(p.su, hb * 32 + lane);
          float v[4] = {flip(x4.x, sg & 1u), flip(x4.y, (sg >> 1) & 1u), flip(x4.z, (sg >> 2) & 1u), flip(x4.w, sg >> 3)};
          wht128(v, lane);
          float mx = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
          unsigned mb = __float_as_uint(mx);           // NaN keeps its (large) bit pattern through the integer maximum below
          if (v[0] != v[0] || v[1] != v[1] || v[2] != v[2] || v[3] != v[3]) mb = 0x7FC00000u;
#pragma unroll
          for (int o = 16; o; o >>= 1) mb = max(mb, __shfl_xor_sync(kFullWarp, mb, o));
          if (lane == 0) atomicMax(&s_amax[wp][r], mb);
#pragma unroll
          for (int k = 0; k < 4; ++k) xv[it][k] = v[k];
        }
      }
    }
    __syncthreads();
    HTR_TTRACE(tid == 0 && window < 4, 4 + 8 * window);

    // -- stage 2: four 7-bit planes per activation, splatted over the four bytes of a weight's hash, in the B operand layout
    {
#pragma unroll
      for (int it = 0; it < kStageRounds; ++it) {
        const int item = warp + it * kTcWarps;
        if (item < items) {
          const int r = item / nblk, hbi = item % nblk;
          const unsigned mb = s_amax[wp][r];
          int ex = (int)(mb >> 23) - 127;              // floor(log2(max)); zero and denormal maxima use the smallest scale that is safe
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
          // columns 4 lane .. 4 lane + 3 of block hb: unit 2 hbi + (lane >> 4) of the window, k-group lane & 15, 16 contiguous bytes
          const int ul = 2 * (hb0 + hbi) + (lane >> 4) - 2 * hb0;
          unsigned char* dst = bwin + ul * unit_b + (lane & 15) * kg_stride + (r >> 1) * 128 + ((r & 1) * 4) * 16;
#pragma unroll
          for (int pl = 0; pl < 4; ++pl)
            *reinterpret_cast<uint4*>(dst + pl * 16) = make_uint4((unsigned)(q[pl][0] & 255) * 0x01010101u, (unsigned)(q[pl][1] & 255) * 0x01010101u,
                                                                  (unsigned)(q[pl][2] & 255) * 0x01010101u, (unsigned)(q[pl][3] & 255) * 0x01010101u);
          // plane sums over the columns this CTA consumes in this window
          const int cgu = 2 * (hb0 + hbi) + (lane >> 4);
          const bool mine = cgu >= cgi && cgu < seg_cg_end;
#pragma unroll
          for (int pl = 0; pl < 4; ++pl) {
            const int sum = __reduce_add_sync(kFullWarp, mine ? q[pl][0] + q[pl][1] + q[pl][2] + q[pl][3] : 0);
            if (lane == 0) atomicAdd(&s_psum[wp][r * 4 + pl], sum);
          }
        }
      }
      HTR_TTRACE(tid == 0 && window < 4, 8 + 8 * window);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
      HTR_TTRACE(tid == 0 && window < 4, 9 + 8 * window);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    HTR_TTRACE(tid == 0 && window < 4, 5 + 8 * window);
    // -- main loop of the window
    if (warp < kTcDecodeWarps) {
      const int sp = lane >> 4, r = lane & 15;
      bool ok = !bad;
      for (int i = done_i + ((cs - done_i) & 1); i < done_i + seg_units; i += kTcSlots) {
        if (!ok) break;
        asm volatile("cp.async.wait_group %0;" ::"n"(R - 2) : "memory");   // this unit's words have landed (own copies) ...
        __syncwarp();                                                       // ... and the other lanes'; the previous slot is free
        prefetch(ring_slot == 0 ? R - 1 : ring_slot - 1);
        HTR_TTRACE(qd == 0 && lane == 0 && i < 16, 36 + 3 * i);
        const int st = i % kTcStages, use = i / kTcStages;
        // the MMAs that read this stage three units ago must have retired
        if (use > 0 && !__all_sync(kFullWarp, mbar_wait_hint(smem_u32(&s_freed[st]), (uint32_t)(use - 1) & 1u, &s_fail, 400u))) { ok = false; if (lane == 0 && !s_fail) tc_note_failure(1u, window, (unsigned)i); if (lane == 0) HTR_TFAIL("tc fail: freed wait, block %d warp %d unit %d stage %d use %d window %u prior fail %d\n", blockIdx.x, warp, i, st, use, window, s_fail); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        HTR_TTRACE(qd == 0 && lane == 0 && i < 16, 37 + 3 * i);
        const uint32_t* tiles = reinterpret_cast<const uint32_t*>(ring + ring_slot * kSlotBytes) + sp * (4 * 8 * K);
        const uint32_t taddr = tmem + ((uint32_t)(32 * qd) << 16) + kTcAcol0 + st * kTcStageCols;
#pragma unroll
        for (int tc = 0; tc < 4; ++tc) {
          uint32_t V[K + 1], st32[32], h[16];
          read_row_words<K>(tiles + tc * (8 * K), r, V);
          row_states<K>(V, st32);
#pragma unroll
          for (int c = 0; c < 16; ++c) h[c] = st32[c] * kGenMul + kGenAdd;
          tmem_store16(taddr + 16 * tc, h);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&s_afull[st]));
        HTR_TTRACE(qd == 0 && lane == 0 && i < 16, 38 + 3 * i);
        if (++ring_slot == R) ring_slot = 0;
      }
      if (!ok) { s_fail = 1; bad = true; }
    } else if (lane == 0) {
      // MMA lane ml = 2 g + hf of slot g: the units of the window with the parity of the slot, MMAs 4 hf .. 4 hf + 3 of each,
      // accumulated in the lane's own 16 TMEM columns.  (A single thread gets an MMA out every 50-150 cycles, whatever its size;
      // several lanes keep the tensor core fed.)
      const int ml = warp - kTcDecodeWarps, g = ml >> 1, hf = ml & 1;
      const uint32_t d_addr = tmem + kTcDStride * ml;
      const uint32_t desc_hi = (uint32_t)((ng_stride >> 4) & 0x3FFF) | (1u << 14);              // SBO, descriptor version 1
      const uint32_t desc_lo_const = (uint32_t)((kg_stride >> 4) & 0x3FFF) << 16;              // LBO
      const uint32_t kk_step = (uint32_t)(2 * kg_stride) >> 4;                                  // one MMA further along k, in 16-byte units
      bool ok = !bad;
      uint32_t accumulate = 0u;
      for (int i = done_i + ((g - done_i) & 1); i < done_i + seg_units && ok; i += kTcSlots) {
        const int st = i % kTcStages, use = i / kTcStages;
        if (!mbar_wait_hint(smem_u32(&s_afull[st]), (uint32_t)use & 1u, &s_fail, 400u)) { ok = false; if (!s_fail) tc_note_failure(2u, window, (unsigned)i); HTR_TFAIL("tc fail: a_full wait, block %d lane warp %d unit %d stage %d use %d window %u prior fail %d\n", blockIdx.x, warp, i, st, use, window, s_fail); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        HTR_TTRACE(hf == 0 && i < 16, 84 + 2 * i);
        const uint32_t lo = ((bwin_addr + (uint32_t)(cgi + (i - done_i) - 2 * hb0) * unit_b) >> 4) + desc_lo_const + (uint32_t)(4 * hf) * kk_step;
        const uint32_t a_addr = tmem + kTcAcol0 + st * kTcStageCols + 32 * hf;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
          umma_i8_tmem_a(d_addr, a_addr + 8 * k4, ((uint64_t)desc_hi << 32) | (lo + (uint32_t)k4 * kk_step), kIdesc, k4 ? 1u : accumulate);
        accumulate = 1u;
        umma_commit(smem_u32(&s_freed[st]));
        HTR_TTRACE(hf == 0 && i < 16, 85 + 2 * i);
      }
      umma_commit(smem_u32(&s_done[ml]));              // covers every MMA this lane has issued so far
      if (!ok) {
        s_fail = 1;
        bad = true;
      }
    }
    __syncwarp();
    // -- drain: the MMAs of the window have retired
#pragma unroll
    for (int g = 0; g < kTcLanes; ++g)
      if (!mbar_wait(smem_u32(&s_done[g]), window & 1u, &s_fail)) {
        if (tid == 0 && !s_fail) tc_note_failure(3u, window, (unsigned)g);
        if (lane == 0) HTR_TFAIL("tc fail: done wait %d, block %d warp %d window %u prior fail %d\n", g, blockIdx.x, warp, window, s_fail);
        s_fail = 1;
        mbar_wait_plain(smem_u32(&s_done[g]), window & 1u);                 // let the MMAs in flight retire all the same
      }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    HTR_TTRACE(tid == 0 && window < 4, 6 + 8 * window);
    if (warp < kTcDecodeWarps && cs == 0) {
      // the MMA lanes hold partial sums: add them (the lanes of a slot without a unit in this window hold old values)
      int d[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) d[j] = 0;
      const int first_par = done_i & 1;                 // parity of the window's first unit
#pragma unroll
      for (int ml = 0; ml < kTcLanes; ++ml) {
        if (seg_units > 1 || first_par == (ml >> 1)) {  // uniform over the CTA
          int dl[16];
          tmem_load16_s32(tmem + ((uint32_t)(32 * qd) << 16) + kTcDStride * ml, dl);
#pragma unroll
          for (int j = 0; j < 16; ++j) d[j] += dl[j];
        }
      }
#pragma unroll
      for (int r = 0; r < kTcRows; ++r) {
        if (r < p.rows) {
          const unsigned mb = s_amax[wp][r];
          int ex = (int)(mb >> 23) - 127;
          ex = ex < -100 ? -100 : ex;
          long long t = 0;
#pragma unroll
          for (int pl = 0; pl < 4; ++pl) t = t * 128 + (long long)(d[4 * r + pl] - 510 * s_psum[wp][4 * r + pl]);
          // t = sum (bytesum - 510) * xt * sc * 128^3, sc = 2^(5 - ex): one rounding on the way to float
          const float val = (float)((double)t * __longlong_as_double((long long)(1023 - 21 - 5 + ex) << 52));
          accf[r] += mb < 0x7F800000u ? val : __uint_as_float(0x7FC00000u);
        }
      }
    }
    done_i += seg_units;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();                                   // statistics read, accumulators read: the next window may overwrite both
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    HTR_TTRACE(tid == 0 && window < 4, 7 + 8 * window);
    if (tid < kTcRows) s_amax[wp][tid] = 0u;            // this parity is used again two windows from now
    if (tid < kTcRows * 4) s_psum[wp][tid] = 0;
    ++window;
    if (s_fail) bad = true;

    u += seg_units;
    cgi += seg_units;
    if (cgi < CG && u < u_end) continue;              // same row block, next window

    // ---- this CTA's contribution to row block rb is complete
    if (warp < kTcDecodeWarps && cs == 0) {
#pragma unroll
      for (int r = 0; r < kTcRows; ++r) {
        ytil[r * 128 + 32 * qd + lane] = bad ? __uint_as_float(0x7FC00000u) : accf[r] * kInvSqrt128;
        accf[r] = 0.f;
      }
    }
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
    if (!predecessor_done) {                           // deferred wait of the independent-input form
      asm volatile("griddepcontrol.wait;" ::: "memory");
      predecessor_done = true;
    }
    __syncthreads();
    bool finish = true;
    if (contributors > 1) {
      float* mine = p.part + ((size_t)rb * p.slots + (blockIdx.x - first)) * (p.rows <= 1 ? 1 : p.rows <= 2 ? 2 : 4) * 128;
      const int width = (p.rows <= 1 ? 1 : p.rows <= 2 ? 2 : 4) * 128;
      for (int e = tid; e < width; e += kTcThreads) __stcg(mine + e, ytil[e]);
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
        for (int e = tid; e < width; e += kTcThreads) {
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
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  HTR_TTRACE(tid == 0, 2);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kTcTmemCols) : "memory");
  if (tid == 0 && s_fail) atomicAdd(&htr_gemv_tc_failures_dev, 1);
}

template <int K>
int launch_packed_gemv_tc(const GemvParams& p, int grid, cudaStream_t stream);
template <int K>
int packed_gemv_tc_ctas_per_sm();
template <int K>
int packed_gemv_tc_failures(int* count, unsigned* last);

}  // namespace htr
