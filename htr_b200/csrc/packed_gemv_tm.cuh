// Packed GEMV for HTR-W1 weights with the weight hashes in tensor memory: byte sums, products and accumulation on tcgen05.
//
//   y = sv * Ho( diag(scale * CB) * V * Hi(su * x) ),  V[i,j] = bytesum(h_ij) - 510,  h_ij = (s_ij * 0xDF6ADF + 0x34983) mod 2^32
//
// (docs/FORMAT.md:7-13 of the reference; the same linear as packed_gemv.cuh, for up to four activation rows, plain activations.)
//
// The 32-bit hash of a weight is four u8 k-elements of the A operand of tcgen05.mma.kind::i8, and the A operand lives in
// tensor memory: thread = one row of the 128-row block (its TMEM lane), and the 16 hashes of one tile row leave the thread's
// registers with ONE tcgen05.st (16 columns).  Per weight the thread is left with the window extraction and the hash
// multiply-add.  The B operand (shared memory, K-major, no swizzle) holds each activation four times in a row (one s8 digit
// splatted over a word), so that the MMA multiplies every byte of the hash with it: sum_b byte_b * y = bytesum * y.
//
// Activations are integers on one grid per activation row for the whole launch: Y = rint(v * sc), v the unnormalised transform,
// sc the power of two that maps the guaranteed bound 128 * max|x| below 2^30.  The B rows are the four signed base-256 digits of
// Y (with Z = Y + 0x80808080, digit i is byte i of Z ^ 0x80808080 read as s8; Y = sum_i 256^i digit_i), N = 16 = four rows x
// four digits.  Accumulators are exact 32-bit integers in tensor memory (a thread block never accumulates more than 16384
// columns: 16384 * 4 * 255 * 128 < 2^31); they leave as sum_i 256^i D_i - 510 * sum_j Y_j in 64-bit integers, are summed
// across thread blocks as integers and rounded once: the result does not depend on the decomposition of the launch.
//
// Thread block: 288 threads, two per SM (256 TMEM columns each).  Warps 0-7 decode, as two groups of four that take alternate
// 64-column units; warp w of a group owns TMEM lane quadrant w & 3, i.e. rows 32 (w & 3) .. + 31 of the row block = two
// 16-row strips, fetches those strips' tiles itself (private cp.async ring) and writes them to A stage (trip % 3).  One lane of
// warp 8 issues the MMAs (eight per unit: K = 32 bytes = 8 weights each) and commits them onto the mbarrier that frees the
// A stage.  Every wait on an mbarrier is bounded; on expiry the thread block records a fault word in the workspace, stops
// issuing, lets its copies and MMAs drain, writes NaN into the rows it still owed, frees its tensor memory and returns.
//
// Decomposition (flat unit ranges), split reduction (64-bit partial sums, last arriver finishes), epilogue and launch overlap
// as in packed_gemv_mma.cuh.
#pragma once
#include <type_traits>

#include "packed_gemv.cuh"

namespace htr {

constexpr int kTmRows = 4;                               // activation rows per launch at most
constexpr int kTmPlanes = 4;                             // signed base-256 digits per activation
constexpr int kTmGroupWarps = 4, kTmDecodeWarps = 8;
constexpr int kTmThreads = (kTmDecodeWarps + 1) * 32;    // + the MMA warp
constexpr int kTmAStages = 3;
constexpr int kTmCols = 256;                             // TMEM columns of a thread block: D at 0..15, A stage s at 64 + 64 s
constexpr int kTmACol = 64;
constexpr int kTmLbo = 144;                              // bytes between core matrices adjacent in K (padded: conflict-free staging stores)
constexpr int kTmSbo = 16 * kTmLbo;                      // bytes between the two 8-row groups of B inside a unit
constexpr int kTmUnitB = 2 * kTmSbo;                     // B operand of one 64-column unit: 16 rows x 256 bytes (+ padding)
constexpr int kTmItems = 64;                             // (activation row, 128-column block) pairs of one staged window at most
constexpr int kTmMaxCols = 16384;                        // columns a thread block may accumulate in 32-bit integers
constexpr unsigned kTmSpin = 4000000u;
constexpr int kTmFaultWord = kCounterBytes / 4 - 2;      // counters[kTmFaultWord] != 0: a bounded wait of this kernel ran out

template <int K>
struct TmRing {
  static constexpr int tile_bytes = 32 * K;
  static constexpr int strip_bytes = 4 * tile_bytes + 16;   // the four tiles of one strip of a unit (+ one spare chunk: a row may read a word past its tile)
  static constexpr int stage_bytes = 2 * strip_bytes;       // one warp, one trip: both strips of its quadrant
  static constexpr int stages = K <= 2 ? 6 : K <= 4 ? 5 : K <= 6 ? 4 : 3;
  static constexpr int bytes = kTmDecodeWarps * stages * stage_bytes;
  static constexpr int chunks = 16 * K;                      // 16-byte chunks of one trip of one warp
  static constexpr int copies = (chunks + 31) / 32;
};
constexpr int tm_window_bytes(int wblocks) { return wblocks * 2 * kTmUnitB; }

__device__ __forceinline__ uint32_t tm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tm_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tm_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bounded wait for the phase with the given parity; false when the limit ran out or another role has already failed
__device__ __forceinline__ bool tm_mbar_wait_slow(uint32_t bar, uint32_t parity, const volatile int* fail) {
  for (unsigned it = 0; it < kTmSpin; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(200u)
        : "memory");
    if (done) return true;
    if ((it & 255u) == 255u && *fail) return false;
  }
  return false;
}
__device__ __forceinline__ bool tm_mbar_wait(uint32_t bar, uint32_t parity, const volatile int* fail) {
  uint32_t done;                                       // the common case: the phase is already complete
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
               : "=r"(done)
               : "r"(bar), "r"(parity)
               : "memory");
  if (done) return true;
  return tm_mbar_wait_slow(bar, parity, fail);
}
__device__ __forceinline__ uint64_t tm_desc_b(uint32_t smem_addr) {
  // start address, LBO, SBO in 16-byte units; descriptor version 1 (sm_100); layout type 0 = no swizzle
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((kTmLbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((kTmSbo >> 4) & 0x3FFF) << 32) |
         (1ull << 46);
}
// D[128 x 16] (+)= A[128 x 32 u8, tensor memory] * B[16 x 32 s8, shared memory]
__device__ __forceinline__ void tm_mma_i8(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tm_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tm_store16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
               "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
               : "memory");
}
__device__ __forceinline__ void tm_load16(uint32_t taddr, int (&d)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]), "=r"(d[9]),
                 "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- one tile row (16 steps) of one thread.
// Row i of a tile needs the stream bits [16 K i + K - 16, 16 K i + 16 K): the 16 windows start K bits apart.  The thread loads
// the words from ((K i) >> 1) - 1 on (circularly for row 0); for even K window 0 then starts at bit 16 + K of the first word.
// For odd K the odd rows start half a word later in the stream: they take the 16-bit funnel of neighbouring words (one PRMT
// per word with a per-lane selector), after which every row has window 0 at bit 16 + K as well.
template <int K>
struct TmRow {
  static constexpr int AE = 16 + K;                                   // bit offset of window 0
  static constexpr int NA = (AE + 15 * K + 16 + 31) / 32;             // aligned words that hold the 16 windows
  static constexpr int NL = NA + (K & 1);                             // words loaded
};

template <int K, int BIT>
__device__ __forceinline__ uint32_t tm_window16(const uint32_t (&A)[TmRow<K>::NA]) {
  constexpr int w = BIT >> 5, off = BIT & 31;
  if constexpr (off == 0) return A[w] >> 16;
  else if constexpr (off == 16) return A[w] & 0xFFFFu;
  else if constexpr (off == 8) return middle_bytes(A[w]);
  else if constexpr (off < 16) return (A[w] >> (16 - off)) & 0xFFFFu;
  else return funnel_left(A[w], A[w + 1], off) >> 16;
}
template <int K, int BIT>
__device__ __forceinline__ uint32_t tm_window32(const uint32_t (&A)[TmRow<K>::NA]) {
  constexpr int w = BIT >> 5, off = BIT & 31;
  if constexpr (off == 0) return A[w];
  else return funnel_left(A[w], A[w + 1], off);
}
namespace detail {
template <int K, int... T>
__device__ __forceinline__ void tm_single(const uint32_t (&A)[TmRow<K>::NA], uint32_t (&h)[16], std::integer_sequence<int, T...>) {
  ((h[T] = tm_window16<K, TmRow<K>::AE + T * K>(A) * kGenMul + kGenAdd), ...);
}
template <int K, int CHAIN, int J>
__device__ __forceinline__ void tm_pair(const uint32_t (&A)[TmRow<K>::NA], uint32_t (&h)[16]) {
  constexpr int P = 16 / K;                                           // steps between the two halves of one 32-bit window
  constexpr int t = CHAIN + 2 * J * P;
  const uint32_t win = tm_window32<K, TmRow<K>::AE + t * K>(A);
  h[t] = (win >> 16) * kGenMul + kGenAdd;
  h[t + P] = (win & 0xFFFFu) * kGenMul + kGenAdd;
}
template <int K, int CHAIN, int... J>
__device__ __forceinline__ void tm_chain(const uint32_t (&A)[TmRow<K>::NA], uint32_t (&h)[16], std::integer_sequence<int, J...>) {
  (tm_pair<K, CHAIN, J>(A, h), ...);
}
template <int K, int... CHAIN>
__device__ __forceinline__ void tm_pairs(const uint32_t (&A)[TmRow<K>::NA], uint32_t (&h)[16], std::integer_sequence<int, CHAIN...>) {
  constexpr int P = 16 / K;
  (tm_chain<K, CHAIN>(A, h, std::make_integer_sequence<int, 8 / P>{}), ...);
}
}  // namespace detail

// hashes of the 16 weights of a tile row; `tile` = the tile's words in shared memory, off0 / off1 = byte offsets of the first
// and the second word this lane loads, sel = PRMT selector of the 16-bit funnel (odd K)
template <int K>
__device__ __forceinline__ void tm_row_hashes(const unsigned char* tile, int off0, int off1, uint32_t sel, uint32_t (&h)[16]) {
  constexpr int NA = TmRow<K>::NA, NL = TmRow<K>::NL;
  uint32_t L[NL];
  L[0] = *reinterpret_cast<const uint32_t*>(tile + off0);
#pragma unroll
  for (int j = 1; j < NL; ++j) L[j] = *reinterpret_cast<const uint32_t*>(tile + off1 + 4 * (j - 1));
  uint32_t A[NA];
  if constexpr (K & 1) {
#pragma unroll
    for (int j = 0; j < NA; ++j) A[j] = __byte_perm(L[j + 1], L[j], sel);
  } else {
#pragma unroll
    for (int j = 0; j < NA; ++j) A[j] = L[j];
  }
  if constexpr (16 % K == 0 && K < 16) detail::tm_pairs<K>(A, h, std::make_integer_sequence<int, 16 / K>{});
  else detail::tm_single<K>(A, h, std::make_integer_sequence<int, 16>{});
}

template <int K>
__global__ void __launch_bounds__(kTmThreads, 2) packed_gemv_tm_kernel(const GemvParams p) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  using Ring = TmRing<K>;
  constexpr int kTileBytes = Ring::tile_bytes, kStageBytes = Ring::stage_bytes, kStages = Ring::stages, kDepth = kStages - 1;
  constexpr int P = kTmPlanes;
  unsigned char* ring = dyn_smem;                                        // [decode warp][stage][strip of the quadrant][4 tiles]
  unsigned char* bwin = dyn_smem + Ring::bytes;                          // [unit of the window][kTmUnitB]
  __shared__ __align__(8) unsigned long long s_full[kTmAStages], s_freed[kTmAStages], s_done;
  __shared__ uint32_t s_tmem;
  __shared__ volatile int s_fail;
  __shared__ int s_arrival;
  __shared__ int s_ilo[kTmItems], s_ihi[kTmItems];          // per staged (row, block): sum of its integers Y over this CTA's units, as hi * 65536 + lo
  __shared__ long long s_ysum[kTmRows];                     // the same summed over the windows of the current row block
  __shared__ unsigned s_rowmax[kTmRows];                    // float bits of the bound of every transformed activation row
  __shared__ float s_red[kTmDecodeWarps + 1];
  __shared__ __align__(16) float ytil[kTmRows * 128];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int U = p.units, G = gridDim.x, CG = p.cg, nt = p.nt, n = nt * 16, m = p.mt * 16, WB = p.wblocks;
  const int u_begin = (int)((long long)blockIdx.x * U / G), u_end = (int)(((long long)blockIdx.x + 1) * U / G);
  const int T = u_end - u_begin;                            // trips (64-column units) of this CTA
  int rb = u_begin / CG;
  int cgi = u_begin - rb * CG;

  if (tid == 0) {
    for (int s = 0; s < kTmAStages; ++s) {
      tm_mbar_init(tm_smem(&s_full[s]), kTmGroupWarps);     // one arrival per warp of the group that decoded the unit
      tm_mbar_init(tm_smem(&s_freed[s]), 1);                // tcgen05.commit
    }
    tm_mbar_init(tm_smem(&s_done), 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < kTmRows) s_ysum[tid] = 0ll;
  if (warp == kTmDecodeWarps) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tm_smem(&s_tmem)), "r"((uint32_t)kTmCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // ---- decode warps: roles and the private copy ring
  const int group = warp >> 2, quad = warp & 3;             // (decode warps only)
  const int row_i = lane & 15, strip_half = lane >> 4;
  const int ws = ((K * row_i) >> 1) - 1;
  const int off0 = (ws < 0 ? 8 * K - 1 : ws) * 4, off1 = (ws + 1) * 4;
  const uint32_t sel = (row_i & 1) ? 0x5432u : 0x7654u;
  unsigned char* my_ring = ring + (warp < kTmDecodeWarps ? warp : 0) * (kStages * kStageBytes);
  const uint32_t my_ring_addr = tm_smem(my_ring);
  // chunk lane + 32 j of the trip: strip (chunk / 8K) of the quadrant, 16-byte piece (chunk % 8K) of its four tiles
  uint32_t cp_dst[Ring::copies];
  int cp_src[Ring::copies];
#pragma unroll
  for (int j = 0; j < Ring::copies; ++j) {
    const int ch = lane + 32 * j, sh = ch >= 8 * K ? 1 : 0, within = ch - sh * 8 * K;
    cp_dst[j] = my_ring_addr + sh * Ring::strip_bytes + within * 16;
    cp_src[j] = sh * nt * kTileBytes + within * 16;
  }
  const int own_trips = warp < kTmDecodeWarps ? (T - group + 1) / 2 : 0;   // trips group, group + 2, ... of the range
  int pf_left = own_trips;
  const char* pf_src = nullptr;
  int pf_in_rb = 0;
  if (own_trips > 0) {
    const int u0 = u_begin + group, rb0 = u0 / CG, cg0 = u0 - rb0 * CG;
    pf_src = reinterpret_cast<const char*>(p.qw) + ((size_t)(rb0 * 8 + 2 * quad) * nt + (size_t)cg0 * 4) * kTileBytes;
    pf_in_rb = (CG - cg0 + 1) >> 1;                         // own trips that remain in the row block, this one included
  }
  auto issue = [&](int stage) {
    // no branches: past the end of the range the copies are predicated off and the cursor runs on harmlessly
#pragma unroll
    for (int j = 0; j < Ring::copies; ++j) {
      const int on = (32 * j + 32 <= Ring::chunks || lane + 32 * j < Ring::chunks) ? pf_left : 0;
      asm volatile("{\n\t.reg .pred p;\n\tsetp.gt.s32 p, %2, 0;\n\t@p cp.async.cg.shared.global [%0], [%1], 16;\n\t}" ::"r"(
                       cp_dst[j] + (uint32_t)(stage * kStageBytes)),
                   "l"(pf_src + cp_src[j]), "r"(on)
                   : "memory");
    }
    --pf_left;
    const bool wrap = pf_in_rb == 1;                        // (an even number of units per row block: the parity of a group's units never changes)
    pf_src += wrap ? (long long)(8 + 7 * nt) * kTileBytes : (long long)8 * kTileBytes;
    pf_in_rb = wrap ? CG >> 1 : pf_in_rb - 1;
    async_commit();
  };
  if (warp < kTmDecodeWarps) {
#pragma unroll
    for (int sgi = 0; sgi < kDepth; ++sgi) issue(sgi);      // the weights do not depend on the preceding kernel
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  bool predecessor_done = false;
  if (!p.independent) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    predecessor_done = true;
  }

  // ---- one power-of-two scale per activation row for the whole launch, from a bound that needs no transform:
  // |v_j| <= 128 max_i |x_i| for the unnormalised transform v.  Every CTA scans the rows (a few KB from L2).
  for (int r = 0; r < p.rows; ++r) {
    unsigned mx = 0u;
    for (int e0 = tid; e0 < (n >> 2); e0 += 4 * kTmThreads) {       // four loads in flight per thread
      float4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = e0 + j * kTmThreads;
        v[j] = e < (n >> 2) ? load_x(p.x, r, 4 * e, p.n_in, p.dtype) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        mx = max(max(mx, __float_as_uint(v[j].x) & 0x7FFFFFFFu), max(__float_as_uint(v[j].y) & 0x7FFFFFFFu,
                 max(__float_as_uint(v[j].z) & 0x7FFFFFFFu, __float_as_uint(v[j].w) & 0x7FFFFFFFu)));   // NaN and Inf patterns compare largest
    }
    mx = __reduce_max_sync(kFullWarp, mx);
    if (lane == 0) s_red[warp] = __uint_as_float(mx);
    __syncthreads();
    if (tid == 0) {
      unsigned all = 0u;
      for (int k = 0; k <= kTmDecodeWarps; ++k) all = max(all, __float_as_uint(s_red[k]));
      s_rowmax[r] = all >= 0x7F800000u ? 0x7FC00000u : min(all + (7u << 23), 0x7F000000u);      // seven binades up: the factor 128
    }
    __syncthreads();
  }
  // the barriers and the TMEM address are visible from here on
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem;
  const uint32_t lane_addr = tmem + ((uint32_t)(32 * quad) << 16);
  // D = s32, A = u8 (tensor memory), B = s8, both K-major, M = 128, N = 16
  const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
  auto scale_exponent = [&](unsigned mb) {
    int ex = (int)(mb >> 23) - 127;
    return ex < -90 ? -90 : ex;
  };

  int ci = 0;                                               // trips consumed by the CTA so far
  int own_stage = 0;                                        // ring stage of this warp's next own trip
  uint32_t done_parity = 0u;
  bool seg_first = true;                                    // the next trip opens a row block's accumulation
  bool ok = true;
  int u = u_begin;
  while (u < u_end) {
    // ---- window: units [cgi, seg_end) of row block rb lie inside at most WB staged 128-column blocks
    const int hb0 = cgi >> 1;
    const int cg_stop = min(CG, cgi + (u_end - u));
    const int hb1 = min(hb0 + WB, (cg_stop + 1) >> 1);
    const int seg_end = min(cg_stop, hb1 * 2);
    const int nblk = hb1 - hb0, items = p.rows * nblk;

    // -- staging: digits of every activation of the window, splatted over a word, in the B operand layout
    if (warp < kTmDecodeWarps) {
      for (int item = warp; item < items; item += kTmDecodeWarps) {
        const int r = item / nblk, hbi = item - r * nblk, hb = hb0 + hbi;
        const float4 x4 = load_x(p.x, r, hb * 128 + 4 * lane, p.n_in, p.dtype);
        const unsigned sg = sign_nibble(p.su, hb * 32 + lane);
        float v[4] = {flip(x4.x, sg & 1u), flip(x4.y, (sg >> 1) & 1u), flip(x4.z, (sg >> 2) & 1u), flip(x4.w, sg >> 3)};
        wht128(v, lane);
        const unsigned mb = s_rowmax[r];
        const float sc = __uint_as_float((unsigned)(8 * P - 3 - scale_exponent(mb) + 127) << 23);   // bound * sc in [2^29, 2^30)
        unsigned z[4];
        int lo = 0, hi = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int y = mb < 0x7F800000u ? __float2int_rn(v[k] * sc) : 0;
          z[k] = ((unsigned)y + 0x80808080u) ^ 0x80808080u;
          lo += y & 0xFFFF;
          hi += y >> 16;
        }
        // this lane holds columns 4 lane .. 4 lane + 3 of the block: unit lane >> 4, core matrix lane & 15 of the unit's K run
        unsigned char* dst = bwin + (hbi * 2 + (lane >> 4)) * kTmUnitB + (lane & 15) * kTmLbo;
#pragma unroll
        for (int pl = 0; pl < P; ++pl) {
          const int nrow = P * r + pl;                       // B row (activation row, digit)
          *reinterpret_cast<uint4*>(dst + (nrow >> 3) * kTmSbo + (nrow & 7) * 16) =
              make_uint4(__byte_perm(z[0], 0u, 0x1111 * pl), __byte_perm(z[1], 0u, 0x1111 * pl), __byte_perm(z[2], 0u, 0x1111 * pl),
                         __byte_perm(z[3], 0u, 0x1111 * pl));
        }
        const int cgu = 2 * hb + (lane >> 4);
        const bool mine = cgu >= cgi && cgu < seg_end;
        lo = __reduce_add_sync(kFullWarp, mine ? lo : 0);
        hi = __reduce_add_sync(kFullWarp, mine ? hi : 0);
        if (lane == 0) {
          s_ilo[item] = lo;
          s_ihi[item] = hi;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
    }
    __syncthreads();
    if (tid < p.rows) {
      long long s = 0ll;
      for (int i = 0; i < nblk; ++i) s += (long long)s_ihi[tid * nblk + i] * 65536ll + (long long)s_ilo[tid * nblk + i];
      s_ysum[tid] += s;
    }

    const int trips = seg_end - cgi;
    if (warp < kTmDecodeWarps) {
      // ================= decode: the trips ci + t with (ci + t) % 2 == group
      for (int t = (group - ci) & 1; t < trips && ok; t += 2) {
        const int c = ci + t, st = c % kTmAStages, use = c / kTmAStages;
        async_wait<kDepth - 1>();                          // the oldest copy group (this trip) has landed
        __syncwarp();                                      // ... for every lane; and every lane is done with the previous slot
        const unsigned char* tiles = my_ring + own_stage * kStageBytes + strip_half * Ring::strip_bytes;
        issue(own_stage == 0 ? kStages - 1 : own_stage - 1);   // refill the slot that was consumed one trip ago (or never used yet)
        own_stage = own_stage + 1 == kStages ? 0 : own_stage + 1;
        // the MMAs that read this A stage three trips ago must have retired
        if (use > 0 && !__all_sync(kFullWarp, tm_mbar_wait(tm_smem(&s_freed[st]), (uint32_t)(use - 1) & 1u, &s_fail))) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = lane_addr + (uint32_t)(kTmACol + 64 * st);
#pragma unroll
        for (int tc = 0; tc < 4; ++tc) {
          uint32_t h[16];
          tm_row_hashes<K>(tiles + tc * kTileBytes, off0, off1, sel, h);
          tm_store16(a_addr + 16 * tc, h);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) tm_mbar_arrive(tm_smem(&s_full[st]));
      }
      if (!ok) s_fail = 1;
    } else if (lane == 0) {
      // ================= MMA lane: every trip in order
      for (int t = 0; t < trips; ++t) {
        const int c = ci + t, st = c % kTmAStages, use = c / kTmAStages;
        if (!tm_mbar_wait(tm_smem(&s_full[st]), (uint32_t)use & 1u, &s_fail)) { s_fail = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = tmem + (uint32_t)(kTmACol + 64 * st);
        const uint32_t b_addr = tm_smem(bwin) + (uint32_t)((cgi + t - 2 * hb0) * kTmUnitB);
#pragma unroll
        for (int j = 0; j < 8; ++j) tm_mma_i8(tmem, a_addr + 8 * j, tm_desc_b(b_addr + j * 2 * kTmLbo), idesc, (seg_first && j == 0) ? 0u : 1u);
        seg_first = false;
        tm_commit(tm_smem(&s_freed[st]));
      }
      tm_commit(tm_smem(&s_done));                          // covers every MMA issued so far
    }
    __syncwarp();
    ci += trips;
    // ---- the MMAs of the window have retired: its B operand may be rewritten, the accumulator read
    if (!tm_mbar_wait(tm_smem(&s_done), done_parity, &s_fail)) s_fail = 1;
    done_parity ^= 1u;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    u += trips;
    cgi = seg_end;
    __syncthreads();
    if (s_fail) break;
    if (cgi < CG && u < u_end) continue;                    // same row block, next window

    // ---- this CTA's contribution to row block rb is complete: accumulator -> 64-bit integers on the rows' grids
    long long* ytil_i = reinterpret_cast<long long*>(bwin);     // [rows][128] (the window is consumed)
    if (warp < 4) {
      int d[16];
      tm_load16(lane_addr, d);                              // warp w reads the lanes of quadrant w
#pragma unroll
      for (int r = 0; r < kTmRows; ++r)
        if (r < p.rows) {
          const long long w = (long long)d[4 * r] + 256ll * (long long)d[4 * r + 1] + 65536ll * (long long)d[4 * r + 2] +
                              16777216ll * (long long)d[4 * r + 3];
          ytil_i[r * 128 + 32 * quad + lane] = w - 510ll * s_ysum[r];
        }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    seg_first = true;
    const int first = unit_owner((long long)rb * CG, G, U);
    const int contributors = unit_owner((long long)(rb + 1) * CG - 1, G, U) - first + 1;
    const int slot_index = blockIdx.x - first;
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
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (tid < kTmRows) s_ysum[tid] = 0ll;                   // (read above, before the barrier)
    bool finish = true;
    const int width = (p.rows <= 1 ? 1 : p.rows <= 2 ? 2 : 4) * 128;
    if (contributors > 1) {
      long long* part_i = reinterpret_cast<long long*>(p.part);
      long long* mine = part_i + ((size_t)rb * p.slots + slot_index) * width;
      for (int e = tid; e < width; e += kTmThreads) __stcg(mine + e, ytil_i[e]);
      __syncthreads();
      if (tid == 0) {
        __threadfence();                                    // the partials of the whole CTA (ordered by the barrier) before the arrival
        s_arrival = atomicAdd(p.counters + rb, 1);         // (the finisher reads the partials with loads served by L2, after this atomic)
      }
      __syncthreads();
      finish = (s_arrival == contributors - 1);
      if (finish) {
        const long long* slot0 = part_i + (size_t)rb * p.slots * width;
        for (int e = tid; e < width; e += kTmThreads) {
          long long sum = 0ll;
          for (int base = 0; base < contributors; base += 8) {
            long long v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = base + j < contributors ? __ldcg(slot0 + (size_t)(base + j) * width + e) : 0ll;
#pragma unroll
            for (int j = 0; j < 8; ++j) sum += v[j];
          }
          ytil_i[e] = sum;
        }
        if (tid == 0) p.counters[rb] = 0;
      }
      __syncthreads();
    }
    if (finish) {
      // the sums leave the integer grid here, once, whatever the launch looked like: one rounding, then the exact power of two
      for (int e = tid; e < p.rows * 128; e += kTmThreads) {
        const unsigned mb = s_rowmax[e >> 7];
        const float inv_sc = __uint_as_float((unsigned)(127 - (8 * P - 3) + scale_exponent(mb)) << 23);
        ytil[e] = mb < 0x7F800000u ? __ll2float_rn(ytil_i[e]) * inv_sc * kInvSqrt128 : __uint_as_float(0x7FC00000u);
      }
    }
    __syncthreads();
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
    if (finish && p.npeer > 0 && p.peer_flag[0] != nullptr) signal_peers_when_last(p, p.counters, p.mt >> 3);
    if (cgi == CG) { cgi = 0; ++rb; }
    __syncthreads();                                         // ytil and the window are free for the next row block
  }
  async_wait<0>();
  if (s_fail && tid == kTmDecodeWarps * 32) {
    // a bounded wait ran out: note it for the host and let the MMAs in flight retire (bounded) before the tensor memory goes
    atomicExch(p.counters + kTmFaultWord, 1);
    for (unsigned it = 0; it < kTmSpin; ++it) {
      uint32_t done;
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                   : "=r"(done)
                   : "r"(tm_smem(&s_done)), "r"(done_parity ^ 1u)
                   : "memory");
      if (done) break;
    }
  }
  if (!predecessor_done) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (s_fail) {
    // the row blocks this thread block still owed never complete (nobody arrives for them): their rows come out as NaN, visible to
    // any consumer, beside the fault word
    const int rb_last = (u_end - 1) / CG;
    const float4 nan4 = make_float4(__uint_as_float(0x7FC00000u), __uint_as_float(0x7FC00000u), __uint_as_float(0x7FC00000u),
                                    __uint_as_float(0x7FC00000u));
    for (int b = rb; b <= rb_last; ++b)
      for (int e = tid; e < p.rows * 32; e += kTmThreads) {
        const int r = e >> 5, row0 = b * 128 + 4 * (e & 31);
        if (p.npeer == 0) {
          if (row0 < p.m_out) store_quad(p.y, (size_t)r * p.m_out + row0, p.dtype, nan4);
        } else {
#pragma unroll 1
          for (int pe = 0; pe < p.npeer; ++pe) store_quad(p.peer_y[pe], (size_t)p.peer_offset + (size_t)r * m + row0, p.dtype, nan4);
        }
      }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kTmDecodeWarps) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kTmCols) : "memory");
}

// host side, defined once per K in packed_gemv_tm_k*.cu
template <int K>
int launch_packed_gemv_tm(const GemvParams& p, int grid, cudaStream_t stream);
// CTAs per SM the kernel is planned for and the largest window (128-column blocks) that fits beside the ring then
template <int K>
int packed_gemv_tm_config(int rows, int* ctas_per_sm, int* window_cap);

}  // namespace htr
