// Packed GEMV for HTR-W1 weights with the byte sums and the dot product on the tensor cores (warp-level int8 MMA).
//
//   y = sv * Ho( diag(scale * CB) * V * Hi(su * x) ),  V[i,j] = bytesum(h_ij) - 510,  h_ij = (s_ij * 0xDF6ADF + 0x34983) mod 2^32
//
// (docs/FORMAT.md:7-13 of the reference; the same linear as packed_gemv.cuh, for up to four activation rows.)
//
// The 32-bit hash of a weight is fed to mma.sync.m16n8k32 (u8 x s8 -> s32) as four consecutive u8 k-elements of the A
// fragment, straight from the register the multiply-add left it in; the B fragment holds the activation of that column four
// times (one s8 value splatted over a word).  The MMA then performs byte sum, multiply and accumulation of 128 weights per
// instruction: per weight the thread is left with the window extraction and the hash multiply-add.
//
// Activations.  Per window of columns and per activation row one power-of-two scale sc is chosen so that the integer
// Y = rint(xt * sc) stays below 2^(8P-2) (P = 4 byte planes, or 2 when an MMA has to carry four bf16 rows).  The planes are the
// signed base-256 digits of Y: with Z = Y + 0x80..80, digit i is byte i of Z minus 128, i.e. byte i of Z ^ 0x80..80 read as s8,
// and Y = sum_i 256^i digit_i exactly.  One add and one xor give all planes of a value; the eight B columns of an MMA are
// (activation row, plane).  Accumulators are exact integers: sum_j bytesum_j * Y_j = sum_i 256^i D_i, and the constant 510 leaves
// as 510 * sum_j Y_j, one 64-bit integer per row and window.  One rounding per window; results do not depend on the order of
// the additions.
//
// Fragment use.  A warp owns one 16-row strip of the 128-row block; a loop trip covers one 128-column block of it (two units
// of four tiles).  Lane (g = lane >> 2, c = lane & 3) decodes rows 2g, 2g+1 of tile c of either unit exactly as in
// packed_gemv.cuh (same words, same compile-time windows).  For MMA j (0..7) of a unit it supplies a0 = hash(row 2g, col 2j),
// a1 = hash(row 2g+1, col 2j), a2 = hash(row 2g, col 2j+1), a3 = hash(row 2g+1, col 2j+1): MMA row g is tile row 2g, MMA row
// g+8 is tile row 2g+1, k-group c is (tile c, column 2j), k-group c+4 is (tile c, column 2j+1).  Its B registers are the
// splatted planes of B column g for the same two columns, read from shared memory where the staging pass laid them out per
// reader lane (conflict-free 16-byte loads); with one activation row only B columns 0..3 carry data and lanes 16..31 skip
// the load.  The accumulator fragment leaves lane (g, c) with B columns 2c, 2c+1 of both rows.
//
// Decomposition, split reduction, epilogue, launch overlap: packed_gemv.cuh (same GemvParams, plan and workspace).
#pragma once
#include <type_traits>

#include "packed_gemv.cuh"

namespace htr {

constexpr int kMmaRows = 4;                              // activation rows per launch at most
constexpr int kMmaItems = 64;                            // (activation row, 128-column block) pairs of one staged window at most

// Words between the tiles of a warp's ring slot.  The four lanes of a quad read the same row pair of four different tiles, so
// with the tiles back to back (8K words) their loads would hit the same banks; a few words of padding spread them out.
template <int K>
struct MmaTileStride {
  static constexpr int value = 8 * K + (K == 8 ? 4 : K % 2 == 0 ? 8 : 0);
};
// ring stages (one trip = two units of every warp each); one less is in flight
template <int K>
struct MmaStages {
  static constexpr int value = K <= 3 ? 4 : 3;
};
template <int K>
struct MmaRing {
  static constexpr int stage_bytes = kGemvWarps * 8 * MmaTileStride<K>::value * 4;
  static constexpr int bytes = MmaStages<K>::value * stage_bytes;
};
template <int K>
constexpr int mma_ring_bytes() { return MmaRing<K>::bytes; }
// B operand of a window of `wblocks` 128-column blocks: two units x four word groups x (NB x 4 reader lanes) x 16 bytes each
constexpr int mma_window_bytes(int nb, int wblocks) { return wblocks * nb * 512; }
// B columns that carry data: four planes of one row, or eight (two rows x four planes, four rows x two planes)
inline int mma_b_columns(int rows) { return rows <= 1 ? 4 : 8; }
// the kernel serves one or two rows of any type and three or four bf16 rows (two planes: enough below an 8-bit rounding)
inline bool mma_serves(int rows, int dtype) { return rows <= 2 || (rows <= kMmaRows && dtype == HTR_DTYPE_BF16); }

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// 16-byte asynchronous copy global -> shared from src + OFF (the offset travels inside the instruction), when `on` is non-zero
template <int OFF>
__device__ __forceinline__ void async_copy16_off_if(uint32_t smem_addr, const void* src, int on) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.gt.s32 p, %2, 0;\n\t@p cp.async.cg.shared.global [%0], [%1+%3], 16;\n\t}" ::"r"(smem_addr),
      "l"(src), "r"(on), "n"(OFF)
      : "memory");
}
template <int J, int N, int CHUNKS>
struct MmaCopies {
  // `left` > 0: trips that remain to be fetched (past the end of the range nothing is copied)
  static __device__ __forceinline__ void run(const uint32_t (&dst)[N], uint32_t stage_bytes, const void* src, int lane, int left) {
    if constexpr (32 * J + 32 <= CHUNKS) async_copy16_off_if<J * 512>(dst[J] + stage_bytes, src, left);
    else async_copy16_off_if<J * 512>(dst[J] + stage_bytes, src, lane + 32 * J < CHUNKS ? left : 0);
    if constexpr (J + 1 < N) MmaCopies<J + 1, N, CHUNKS>::run(dst, stage_bytes, src, lane, left);
  }
};

// one unit of one lane: 32 weights = 8 MMAs, alternating between two accumulator sets
template <int K, int NB>
__device__ __forceinline__ void mma_lane_unit(const uint32_t* __restrict__ tile, int g, uint32_t baddr, int (&d)[2][4]) {
  uint32_t V[K + 1];
  read_unit_words<K>(tile, g, V);
  uint32_t s[32];
  unit_states<K>(V, s);
#pragma unroll
  for (int j4 = 0; j4 < 4; ++j4) {
    const uint4 b = lds128(baddr + j4 * (NB * 64));
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
      const int col = 4 * j4 + 2 * jj;
      const uint32_t a0 = s[col] * kGenMul + kGenAdd, a1 = s[16 + col] * kGenMul + kGenAdd;
      const uint32_t a2 = s[col + 1] * kGenMul + kGenAdd, a3 = s[17 + col] * kGenMul + kGenAdd;
      mma_u8s8(d[jj], a0, a1, a2, a3, jj ? b.z : b.x, jj ? b.w : b.y);
    }
  }
}

template <int K, int NB>
__global__ void __launch_bounds__(kGemvThreads, 3) packed_gemv_mma_kernel(const GemvParams p) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  constexpr int kStride = MmaTileStride<K>::value, kTileBytes = 32 * K;
  constexpr int kStageBytes = MmaRing<K>::stage_bytes, kStages = MmaStages<K>::value, kDepth = kStages - 1;
  constexpr int kChunks = 16 * K;                        // 16-byte chunks of one trip of one warp (eight tiles)
  constexpr int kCopies = (kChunks + 31) / 32;           // copy instructions per lane and trip
  constexpr int kUnitB = NB * 256;                       // B operand of one unit
  uint32_t* ring = reinterpret_cast<uint32_t*>(dyn_smem);                 // [stage][warp][8 tiles][kStride]
  unsigned char* bwin = dyn_smem + kStages * kStageBytes;                 // [block][unit][4 word groups][NB x 4 reader lanes][16 B]
  __shared__ int s_arrival;
  __shared__ unsigned s_imax[kMmaItems];                 // per staged (row, block): largest magnitude (float bits)
  __shared__ int s_ilo[kMmaItems], s_ihi[kMmaItems];     // ... and the sum of its integers Y over this CTA's units, as hi * 65536 + lo
  __shared__ float s_row_inv[kMmaRows];
  __shared__ float s_ss[kGemvWarps];
  __shared__ __align__(16) float ytil[kMmaRows * 128];
  __shared__ unsigned s_rowmax[kMmaRows];                // exact form: float bits of the bound of every transformed activation row

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;               // consumer roles: row pair of the strip, tile column of the unit
  const int P = (NB == 8 && p.rows > 2) ? 2 : 4;       // byte planes per activation
  const int U = p.units, G = gridDim.x, CG = p.cg, CB = CG >> 1, nt = p.nt, n = nt * 16, m = p.mt * 16, WB = p.wblocks;
  // split form: grid (split, row blocks), the parts of a row block differ by at most one unit; flat form: even unit ranges
  int u_begin, u_end, slot_index;
  if (p.split > 0) {
    const int part = blockIdx.x, base = blockIdx.y * CG;
    u_begin = base + part * p.cg_quot + min(part, p.cg_rem);
    u_end = u_begin + p.cg_quot + (part < p.cg_rem ? 1 : 0);
    slot_index = part;
  } else {
    u_begin = (int)((long long)blockIdx.x * U / G);
    u_end = (int)(((long long)blockIdx.x + 1) * U / G);
    slot_index = 0;                                     // found per row block below
  }
  int rb = p.split > 0 ? (int)blockIdx.y : u_begin / CG;
  int cgi = u_begin - rb * CG;

  // one staged item: the 128 transformed activations of (row r, block hb), four per lane (columns 4 lane .. 4 lane + 3)
  auto load_item = [&](int r, int hb) -> float4 { return fused_x(p, p.x, r, hb * 128 + 4 * lane, p.prologue == 1 ? s_row_inv[r] : 1.f); };
  auto transform_item = [&](float4 x4, int hb, float (&v)[4]) {
    const unsigned sg = sign_nibble(p.su, hb * 32 + lane);
    v[0] = flip(x4.x, sg & 1u); v[1] = flip(x4.y, (sg >> 1) & 1u); v[2] = flip(x4.z, (sg >> 2) & 1u); v[3] = flip(x4.w, sg >> 3);
    wht128(v, lane);
  };
  // geometry of the window that starts at unit cgi of a row block when `left` units of the range remain
  struct Window { int hb0, hb1, seg_end, nblk; };
  auto window_at = [&](int cgi_, int left) {
    Window w;
    w.hb0 = cgi_ >> 1;
    const int cg_stop = min(CG, cgi_ + left);
    w.hb1 = min(w.hb0 + WB, (cg_stop + 1) >> 1);
    w.seg_end = min(cg_stop, w.hb1 * 2);
    w.nblk = w.hb1 - w.hb0;
    return w;
  };

  // copy roles: chunk lane + 32 j of the trip's eight tiles; the tiles sit kStride words apart in the ring
  uint32_t cp_dst[kCopies];
#pragma unroll
  for (int j = 0; j < kCopies; ++j) {
    const int ch = lane + 32 * j, t = ch / (2 * K), w = ch - t * (2 * K);
    cp_dst[j] = (uint32_t)__cvta_generic_to_shared(ring + (warp * 8 + (t & 7)) * kStride) + w * 16;
  }
  const int T = ((u_end + 1) >> 1) - (u_begin >> 1);   // trips (128-column blocks) of this CTA
  // Only the first and the last block of the range can be half foreign (row blocks hold an even number of units).  The copies
  // always bring whole blocks; the consumer skips the foreign unit.
  const int first_partial = (u_begin & 1) ? 0 : -1, last_partial = (u_end & 1) ? T - 1 : -1;
  // prefetch cursor: kDepth trips ahead of the consumer along the same sequence of blocks
  const char* pf_src = reinterpret_cast<const char*>(p.qw) + ((size_t)(rb * 8 + warp) * nt + (size_t)(8 * (cgi >> 1))) * kTileBytes + lane * 16;
  constexpr int kStepBytes = 8 * kTileBytes;                           // next 128-column block of the strip
  const long long wrap_bytes = (long long)7 * nt * kTileBytes;         // ... or the first block of the next row block
  int pf_left = T, pf_in_rb = CB - (cgi >> 1);
  auto issue = [&](int stage_bytes) {
    // no branches: past the end of the range the copies are predicated off and the cursor runs on harmlessly
    MmaCopies<0, kCopies, kChunks>::run(cp_dst, (uint32_t)stage_bytes, pf_src, lane, pf_left);
    --pf_left;
    const bool wrap = pf_in_rb == 1;
    pf_src += wrap ? kStepBytes + wrap_bytes : (long long)kStepBytes;
    pf_in_rb = wrap ? CB : pf_in_rb - 1;
    async_commit();
  };

  // the first window's first item: its load goes out before the copies queue up in front of it
  Window win = window_at(cgi, u_end - u_begin);
  float4 x_first = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool first_item = warp < p.rows * win.nblk;
  const int first_r = warp / win.nblk, first_hb = win.hb0 + warp - first_r * win.nblk;
  if (p.independent && p.prologue != 1 && first_item) x_first = load_item(first_r, first_hb);
  issue(0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  bool predecessor_done = false;
  if (!p.independent) {
    // the activations come from the preceding kernel: while it drains, the whole ring is primed
#pragma unroll
    for (int sgi = 1; sgi < kDepth; ++sgi) issue(sgi * kStageBytes);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    predecessor_done = true;
    if (p.prologue != 1 && first_item) x_first = load_item(first_r, first_hb);
  } else {
#pragma unroll
    for (int sgi = 1; sgi < kDepth; ++sgi) issue(sgi * kStageBytes);
  }
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
    __syncthreads();
    if (first_item) x_first = load_item(first_r, first_hb);
  }

  // Exact form (p.exact): one power-of-two scale per activation row for the whole launch, so that every window's integers lie
  // on one grid and all sums -- across windows, across thread blocks -- stay in 64-bit integers.  The scale comes from a bound
  // that needs no transform: |v_j| <= 128 max_i |x_i| for the unnormalised transform v that is quantised below (met when su * x
  // is a row of the Hadamard matrix).  Every CTA scans the row (a few KB from L2).
  const bool exact = p.exact != 0;
  if (exact) {
    for (int r = 0; r < p.rows; ++r) {
      unsigned mx = 0u;
      for (int e = tid; e < (n >> 2); e += kGemvThreads) {
        const float4 v = load_x(p.x, r, 4 * e, p.n_in, p.dtype);
        mx = max(max(mx, __float_as_uint(v.x) & 0x7FFFFFFFu), max(__float_as_uint(v.y) & 0x7FFFFFFFu,
                 max(__float_as_uint(v.z) & 0x7FFFFFFFu, __float_as_uint(v.w) & 0x7FFFFFFFu)));   // NaN and Inf patterns compare largest
      }
      mx = __reduce_max_sync(kFullWarp, mx);
      if (lane == 0) s_ss[warp] = __uint_as_float(mx);
      __syncthreads();
      if (tid == 0) {
        unsigned all = 0u;
        for (int k = 0; k < kGemvWarps; ++k) all = max(all, __float_as_uint(s_ss[k]));
        // seven binades up: the factor 128
        s_rowmax[r] = all >= 0x7F800000u ? 0x7FC00000u : min(all + (7u << 23), 0x7F000000u);
      }
      __syncthreads();
    }
  }
  float accf[2] = {0.f, 0.f};                          // rows 2g, 2g+1 of the strip for this lane's activation row, summed over windows
  long long acci[2] = {0ll, 0ll};                       // the same sums as integers on the row's grid (exact form)
  const uint32_t* my_tiles = ring + (warp * 8 + c) * kStride;
  // with four B columns the lanes 16..31 read what lanes 0..15 read: their B columns (4..7) feed accumulator columns nobody uses
  const uint32_t bwin_addr = (uint32_t)__cvta_generic_to_shared(bwin) + (lane & (NB * 4 - 1)) * 16;
  // statistics of row r of the staged window, for every lane of the calling warp (all lanes call together)
  auto row_amax = [&](int r, int nblk) {
    unsigned mx = 0u;
    for (int i = lane; i < nblk; i += 32) mx = max(mx, s_imax[r * nblk + i]);
    return __reduce_max_sync(kFullWarp, mx);
  };
  auto row_ysum = [&](int r, int nblk) {
    int lo = 0, hi = 0;
    for (int i = lane; i < nblk; i += 32) {
      lo += s_ilo[r * nblk + i];
      hi += s_ihi[r * nblk + i];
    }
    lo = __reduce_add_sync(kFullWarp, lo);
    hi = __reduce_add_sync(kFullWarp, hi);
    return (long long)hi * 65536ll + (long long)lo;
  };

  int stage_bytes = 0, refill_bytes = (kStages - 1) * kStageBytes;
  int u = u_begin, ci = 0;                             // ci: trips consumed
  bool first_window = true;
  while (u < u_end) {
    // ---- window: units [cgi, win.seg_end) of row block rb lie inside at most WB staged 128-column blocks
    if (!first_window) {
      win = window_at(cgi, u_end - u);
      __syncthreads();                                 // the previous window is consumed and its statistics are read
    }
    const int hb0 = win.hb0, nblk = win.nblk, items = p.rows * nblk, seg_cg_end = win.seg_end;

    // -- pass 1: transform the activations of the window, note the range of every item.  The first kKeep items of a warp stay in
    // registers for pass 2; a window with more items per warp transforms the rest a second time there.
    constexpr int kKeep = 4;
    float keep[kKeep][4];
#pragma unroll
    for (int it = 0; it < kKeep; ++it) keep[it][0] = keep[it][1] = keep[it][2] = keep[it][3] = 0.f;
    auto note_range = [&](int item, const float (&v)[4]) {
      unsigned mb = __float_as_uint(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
      if (v[0] != v[0] || v[1] != v[1] || v[2] != v[2] || v[3] != v[3]) mb = 0x7FC00000u;
      mb = __reduce_max_sync(kFullWarp, mb);
      if (lane == 0) s_imax[item] = mb;
    };
#pragma unroll
    for (int it = 0; it < kKeep; ++it) {
      const int item = warp + it * kGemvWarps;
      if (item < items) {
        const int r = item / nblk, hb = hb0 + item - r * nblk;
        transform_item((first_window && it == 0) ? x_first : load_item(r, hb), hb, keep[it]);
        note_range(item, keep[it]);
      }
    }
#pragma unroll 1
    for (int item = warp + kKeep * kGemvWarps; item < items; item += kGemvWarps) {
      const int r = item / nblk, hb = hb0 + item - r * nblk;
      float v[4];
      transform_item(load_item(r, hb), hb, v);
      note_range(item, v);
    }
    __syncthreads();

    // -- pass 2: byte planes of every activation, splatted over a word, laid out per reader lane
    auto emit_item = [&](int item, const float (&v)[4]) {
      const int r = item / nblk, hbi = item - r * nblk;
      const unsigned mb = exact ? s_rowmax[r] : row_amax(r, nblk);
      int ex = (int)(mb >> 23) - 127;
      ex = ex < -90 ? -90 : ex;
      const float sc = __uint_as_float((unsigned)(8 * P - 3 - ex + 127) << 23);   // max * sc in [2^(8P-3), 2^(8P-2))
      const unsigned bias = P == 4 ? 0x80808080u : 0x00008080u;
      unsigned z[4];
      int lo = 0, hi = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int y = mb < 0x7F800000u ? __float2int_rn(v[k] * sc) : 0;
        z[k] = ((unsigned)y + bias) ^ bias;
        lo += y & 0xFFFF;
        hi += y >> 16;
      }
      // this lane holds columns 4 lane .. 4 lane + 3 of the block: unit lane >> 4, tile (lane >> 2) & 3, word group lane & 3;
      // reader lane of (B column nb, tile) = 4 nb + tile, with nb = P r + plane
      unsigned char* dst = bwin + ((hbi * 2 + (lane >> 4)) * kUnitB + (lane & 3) * (NB * 64) + (P * r * 4 + ((lane >> 2) & 3)) * 16);
#pragma unroll
      for (int pl = 0; pl < 4; ++pl)
        if (pl < P)
          *reinterpret_cast<uint4*>(dst + pl * 64) = make_uint4(__byte_perm(z[0], 0u, 0x1111 * pl), __byte_perm(z[1], 0u, 0x1111 * pl),
                                                                 __byte_perm(z[2], 0u, 0x1111 * pl), __byte_perm(z[3], 0u, 0x1111 * pl));
      const int cgu = 2 * (hb0 + hbi) + (lane >> 4);
      const bool mine = cgu >= cgi && cgu < seg_cg_end;
      lo = __reduce_add_sync(kFullWarp, mine ? lo : 0);
      hi = __reduce_add_sync(kFullWarp, mine ? hi : 0);
      if (lane == 0) {
        s_ilo[item] = lo;
        s_ihi[item] = hi;
      }
    };
#pragma unroll
    for (int it = 0; it < kKeep; ++it) {
      const int item = warp + it * kGemvWarps;
      if (item < items) emit_item(item, keep[it]);
    }
#pragma unroll 1
    for (int item = warp + kKeep * kGemvWarps; item < items; item += kGemvWarps) {
      const int r = item / nblk, hb = hb0 + item - r * nblk;
      float v[4];
      transform_item(load_item(r, hb), hb, v);
      emit_item(item, v);
    }
    __syncthreads();

    // -- main loop of the window: one 128-column block per trip
    int d[2][4];
#pragma unroll
    for (int t = 0; t < 2; ++t) d[t][0] = d[t][1] = d[t][2] = d[t][3] = 0;
    uint32_t baddr = bwin_addr;
    const int trips = ((seg_cg_end + 1) >> 1) - hb0;
    // a trip: wait for its slot, refill the slot consumed one trip ago, decode FIRST and / or SECOND unit of the block
    auto trip = [&](auto first, auto second) {
      async_wait<kDepth - 1>();                        // the oldest copy group (this trip) has landed
      __syncwarp();                                    // ... for every lane; and every lane is done with the previous slot
      const uint32_t* tiles = reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(my_tiles) + stage_bytes);
      issue(refill_bytes);                             // refill the slot that was consumed one trip ago (or never used yet)
      refill_bytes = stage_bytes;
      stage_bytes = (stage_bytes + kStageBytes == kStages * kStageBytes) ? 0 : stage_bytes + kStageBytes;
      if constexpr (decltype(first)::value) mma_lane_unit<K, NB>(tiles, g, baddr, d);
      if constexpr (decltype(second)::value) mma_lane_unit<K, NB>(tiles + 4 * kStride, g, baddr + kUnitB, d);
      baddr += 2 * kUnitB;
    };
    // only the first and the last trip of the whole range can be half foreign (never the same trip: such a range would be
    // empty): they are peeled off the steady loop
    const bool head = ci == first_partial, tail = ci + trips - 1 == last_partial;
    const int full = trips - (head ? 1 : 0) - (tail ? 1 : 0);
    if (head) trip(std::false_type{}, std::true_type{});
#pragma unroll 1
    for (int t = 0; t < full; ++t) trip(std::true_type{}, std::true_type{});
    if (tail) trip(std::true_type{}, std::false_type{});
    ci += trips;

    // -- the window's integers leave for float.  Four planes: lane (g, c) holds planes 2 (c & 1), 2 (c & 1) + 1 of activation row
    // c >> 1, the other two sit in the neighbouring lane.  Two planes: both planes of activation row c.
    {
      const int r = P == 4 ? (c >> 1) : c;
      unsigned mb = 0u;
      long long ysum = 0ll;
#pragma unroll
      for (int rr = 0; rr < kMmaRows; ++rr)
        if (rr < p.rows) {                             // (uniform) every lane takes part in the warp-wide reductions
          const unsigned mrow = exact ? s_rowmax[rr] : row_amax(rr, nblk);
          const long long yrow = row_ysum(rr, nblk);
          if (rr == r) {
            mb = mrow;
            ysum = yrow;
          }
        }
      const long long hi = (P == 4 && (c & 1)) ? 65536ll : 1ll;       // 256^2 for planes 2, 3 of four
      long long w0 = ((long long)(d[0][0] + d[1][0]) + 256ll * (long long)(d[0][1] + d[1][1])) * hi;
      long long w1 = ((long long)(d[0][2] + d[1][2]) + 256ll * (long long)(d[0][3] + d[1][3])) * hi;
      if (P == 4) {
        w0 += __shfl_xor_sync(kFullWarp, w0, 1);
        w1 += __shfl_xor_sync(kFullWarp, w1, 1);
      }
      int ex = (int)(mb >> 23) - 127;
      ex = ex < -90 ? -90 : ex;
      const float inv_sc = __uint_as_float((unsigned)(127 - (8 * P - 3) + ex) << 23);   // 1 / sc, a power of two
      if (r < p.rows) {
        if (exact) {                                   // integers on the row's grid: summed as they are
          acci[0] += w0 - 510ll * ysum;
          acci[1] += w1 - 510ll * ysum;
        } else {
          // one rounding (64-bit integer to float); the scaling by a power of two is exact
          accf[0] += mb < 0x7F800000u ? __ll2float_rn(w0 - 510ll * ysum) * inv_sc : __uint_as_float(0x7FC00000u);
          accf[1] += mb < 0x7F800000u ? __ll2float_rn(w1 - 510ll * ysum) * inv_sc : __uint_as_float(0x7FC00000u);
        }
      }
    }
    first_window = false;
    u += seg_cg_end - cgi;
    cgi = seg_cg_end;
    if (cgi < CG && u < u_end) continue;               // same row block, next window

    // ---- this CTA's contribution to row block rb is complete
    long long* ytil_i = reinterpret_cast<long long*>(bwin);     // exact form: [rows][128] 64-bit sums (the window is consumed)
    if (exact) __syncthreads();                                 // every warp is done reading the B window
    if (P == 2 || (c & 1) == 0) {
      const int r = P == 4 ? (c >> 1) : c;
      if (exact) {
        if (r < p.rows) {
          ytil_i[r * 128 + warp * 16 + 2 * g] = acci[0];
          ytil_i[r * 128 + warp * 16 + 2 * g + 1] = acci[1];
        }
      } else {
        ytil[r * 128 + warp * 16 + 2 * g] = accf[0] * kInvSqrt128;
        ytil[r * 128 + warp * 16 + 2 * g + 1] = accf[1] * kInvSqrt128;
      }
    }
    accf[0] = accf[1] = 0.f;
    acci[0] = acci[1] = 0ll;
    int contributors;
    if (p.split > 0) {
      contributors = p.split;
    } else {
      const int first = unit_owner((long long)rb * CG, G, U);
      contributors = unit_owner((long long)(rb + 1) * CG - 1, G, U) - first + 1;
      slot_index = blockIdx.x - first;
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
      if (exact) {
        long long* part_i = reinterpret_cast<long long*>(p.part);
        long long* mine = part_i + ((size_t)rb * p.slots + slot_index) * width;
        for (int e = tid; e < width; e += kGemvThreads) __stcg(mine + e, ytil_i[e]);
      } else {
        float* mine = p.part + ((size_t)rb * p.slots + slot_index) * width;
        for (int e = tid; e < width; e += kGemvThreads) __stcg(mine + e, ytil[e]);
      }
      __syncthreads();
      if (tid == 0) {
        __threadfence();                               // the partials of the whole CTA (ordered by the barrier) before the arrival
        s_arrival = atomicAdd(p.counters + rb, 1);   // (the finisher reads the partials with loads served by L2, after this atomic)
      }
      __syncthreads();
      finish = (s_arrival == contributors - 1);
      if (finish) {
        if (exact) {
          const long long* slot0 = reinterpret_cast<const long long*>(p.part) + (size_t)rb * p.slots * width;
          for (int e = tid; e < width; e += kGemvThreads) {
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
        } else {
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
        }
        if (tid == 0) p.counters[rb] = 0;
      }
      __syncthreads();
    }
    if (exact && finish) {
      // the sums leave the integer grid here, once, whatever the launch looked like: one rounding, then the exact power of two
      for (int e = tid; e < width; e += kGemvThreads) {
        const unsigned mb = s_rowmax[e >> 7];
        int ex = (int)(mb >> 23) - 127;
        ex = ex < -90 ? -90 : ex;
        const float inv_sc = __uint_as_float((unsigned)(127 - (8 * P - 3) + ex) << 23);
        ytil[e] = mb < 0x7F800000u ? __ll2float_rn(ytil_i[e]) * inv_sc * kInvSqrt128 : __uint_as_float(0x7FC00000u);
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
    if (finish && p.npeer > 0 && p.peer_flag[0] != nullptr) signal_peers_when_last(p, p.counters, p.mt >> 3);
    if (cgi == CG) { cgi = 0; ++rb; }                   // (ytil is rewritten only after the barrier that opens the next window)
  }
  async_wait<0>();
}

// host side, defined once per K in packed_gemv_mma_k*.cu
template <int K>
int launch_packed_gemv_mma(const GemvParams& p, int grid, cudaStream_t stream);
// CTAs per SM the kernel is planned for and the largest window (128-column blocks) that fits beside the ring then
template <int K>
int packed_gemv_mma_config(int rows, int* ctas_per_sm, int* window_cap);

}  // namespace htr
