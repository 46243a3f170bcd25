// Streaming packed GEMV for HTR-W1 weights on sm_100a: one launch per linear.
//
//   y = sv * Ho( diag(scale * CB) * V * Hi(su * x) ),  V[i,j] = v(s_ij) integer codebook values
//
// (docs/FORMAT.md:7-13 of the reference; replaces its prologue + gemv_epi pair, htr/ops.py:95-98.)
//
// Decomposition.  The weight is cut into units of (128-row block) x (4 tile columns = 64 input columns);
// unit u = rb * CG + cg.  All CTAs of the grid are resident at once and each owns a contiguous unit range.
// Short matrices use the "split" form: every row block is shared by exactly S CTAs, so no CTA crosses a
// row block.  Tall matrices (more row blocks than resident CTAs, or long ranges) use the "flat" form:
// CTA b owns [b*U/G, (b+1)*U/G), which may end inside a row block and continue in the next one.  For every
// row block it touches, a CTA publishes one partial result [M,128]; the CTA that arrives last at the
// block's counter adds the partials in CTA order (deterministic), applies row scales, the output
// Hadamard, output signs and bias, and resets the counter.  No CTA ever waits for another one.
//
// Launch overlap.  The kernel is launched with programmatic stream serialisation: it starts while its
// predecessor in the stream drains, prefetches its first packed words (weights never depend on earlier
// kernels), and only then waits for the predecessor (griddepcontrol.wait) before it reads activations or
// touches the workspace or the output.
//
// Inside a CTA (256 threads): warp = (half h of the row block: strips 4h..4h+3) x (tile column c of the
// unit); lane = (strip g, row pair q).  A loop trip covers one 128-column block (two units).  The packed words
// travel global -> shared memory through a ring of trip-sized slots per warp, all but one of them in flight
// (16-byte cp.async, no registers held while they fly); a lane then reads its K words and the history word, rebuilds 32
// codebook integers in registers and multiplies them with the transformed activations, which all lanes of
// the warp read from shared memory at the same address (broadcast).
//
// Instruction budget.  On sm_100 the multiply-add of the hash, the byte dot product and the packed
// two-wide float ops all issue to the same half-rate pipe, which is what bounds this kernel; the integer
// to float step uses the exact 1.5*2^23 bit trick with packed adds and FMAs (half the issue slots of
// scalar ones), and part of the byte sums are moved to the shift/logic pipe (see unit_fma).
#pragma once
#include <type_traits>

#include "htr_codec.cuh"

#include "htr_common.cuh"

namespace htr {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kStageBlocks = 8;                  // 128-column blocks of activations staged at a time
constexpr int kStageCols = kStageBlocks * 128;   // 1024 activations per row
constexpr int kCounterBytes = 1 << 16;           // arrival counters at the start of the workspace (16384 row blocks)
constexpr int kDoneCounter = kCounterBytes / 4 - 1;   // the last one counts the finished row blocks of a signalling launch


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
  int units;        // row blocks * cg
  int split;        // > 0: every row block is shared by exactly `split` CTAs (grid = (split, row blocks)); 0: flat unit ranges
  int cg_quot, cg_rem;   // split form: cg / split and cg % split (the first cg_rem parts of a row block hold one unit more)
  int slots;        // partial slots per row block
  int wblocks;      // warp-MMA kernel only: 128-column blocks of activations staged at a time
  int exact;        // warp-MMA kernel only: 1 = one scale per activation row and 64-bit integer sums throughout (the partial sums in
                    // `part` are then 64-bit: twice the bytes); results are independent of the launch decomposition
  int independent;  // 1: x, bias and y are untouched by the preceding kernel of the stream (wait only before publishing)
  int n_in;         // columns present in x (row stride of x); columns n_in .. n-1 of the stored weight see zeros
  int m_out;        // rows written to y (row stride of y, length of bias); rows m_out .. m-1 of the stored weight are dropped
  // Decoder fusions (bf16 only; the roundings of the unfused bf16 operators are reproduced):
  int prologue;     // 0: x as given; 1: x <- rmsnorm(x) * norm_w (row-wise, eps); 2: x holds [gate | up] rows of 2n, x <- silu(gate) * up
  int residual;     // 1: y <- y + result (y is the residual stream, read and written in place)
  int x_stride;     // elements between activation rows (n_in; 2n for prologue 2)
  const void* norm_w;
  float eps;
  float cb;         // 1 / rms of the codebook integers
  // Peer form (row-sharded linears over NVLink): when npeer > 0 the epilogue writes its rows into every listed buffer
  // (peers' and its own, plain stores through peer-mapped addresses) at element offset peer_offset, instead of into y.
  void* peer_y[8];
  int npeer;
  long long peer_offset;
  // Delivery signal of the peer form: when peer_flag[0] is set, the thread block that finishes the launch's last row block adds 1
  // to the word peer_flag[pe] of every peer (system scope, after a system-wide fence): "this rank's rows of this call are in your
  // buffer".  The launch-wide count of finished row blocks lives in the last counter of the workspace (zero between launches).
  unsigned* peer_flag[8];
  // Grouped form (experts of a mixture-of-experts layer): group > 0 problems of identical shape, one activation row each;
  // the per-problem tensors come from device arrays of device pointers, row blocks are numbered problem-major.  A problem whose
  // weight pointer is null is skipped (its output is left untouched).
  int group;
  int rb_per_problem;
  const void* const* g_x;
  const uint32_t* const* g_qw;
  const __half* const* g_scales;
  const uint8_t* const* g_su;
  const uint8_t* const* g_sv;
  void* const* g_y;
  // Routed form: g_route[prob] = index into the four tables above (e.g. the expert of a (token, slot) pair); activations are
  // row prob / g_xdiv of the matrix at x (g_xrow_bytes apart), outputs row prob of the matrix at y (g_yrow_bytes apart).
  const long long* g_route;
  int g_table_rows;  // rows of the four tables: a route entry outside [0, g_table_rows) skips its problem like a null weight pointer
  int g_xdiv;
  long long g_xrow_bytes, g_yrow_bytes;
};

// Called by every thread of the block that has just stored the output rows of a row block into the peers' buffers.
__device__ __forceinline__ void signal_peers_when_last(const GemvParams& p, int* counters, int row_blocks) {
  __syncthreads();                                   // the stores of every warp are issued
  if (threadIdx.x == 0) {
    // Release at GPU scope, then the count; the block that counts last acquires the others' stores with its own fence, which is
    // system-wide and so also releases all of them to the peers ahead of the flags (fences are cumulative).  Only that one block
    // pays for a system-wide fence.
    __threadfence();
    if (atomicAdd(counters + kDoneCounter, 1) == row_blocks - 1) {
      __threadfence_system();
      counters[kDoneCounter] = 0;
#pragma unroll 1
      for (int pe = 0; pe < p.npeer; ++pe) atomicAdd_system(p.peer_flag[pe], 1u);
    }
  }
}

// four consecutive activations of row r at column col (a multiple of 4); columns at or beyond n_in (a multiple of 4) read as zero
__device__ __forceinline__ float4 load_x(const void* x, int r, int col, int n_in, int dtype) {
  return col < n_in ? load_quad(x, (size_t)r * n_in + col, dtype) : make_float4(0.f, 0.f, 0.f, 0.f);
}

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// the activation a decoder layer would have materialised in bf16 before this linear, recomputed from its inputs
__device__ __forceinline__ float4 fused_x(const GemvParams& p, const void* x, int r, int col, float inv) {
  if (p.prologue == 1) {                                  // RMSNorm: normalise, round, scale, round (the order of the unfused operators)
    const float4 v = load_quad(x, (size_t)r * p.x_stride + col, p.dtype);
    const float4 g = load_quad(p.norm_w, col, p.dtype);
    return make_float4(bf16_round(bf16_round(v.x * inv) * g.x), bf16_round(bf16_round(v.y * inv) * g.y),
                       bf16_round(bf16_round(v.z * inv) * g.z), bf16_round(bf16_round(v.w * inv) * g.w));
  }
  if (p.prologue == 2) {                                  // SwiGLU: silu(gate) rounded, times up, rounded
    const float4 g = load_quad(x, (size_t)r * p.x_stride + col, p.dtype);
    const float4 u = load_quad(x, (size_t)r * p.x_stride + (p.x_stride >> 1) + col, p.dtype);
    return make_float4(bf16_round(bf16_round(g.x / (1.f + __expf(-g.x))) * u.x), bf16_round(bf16_round(g.y / (1.f + __expf(-g.y))) * u.y),
                       bf16_round(bf16_round(g.z / (1.f + __expf(-g.z))) * u.z), bf16_round(bf16_round(g.w / (1.f + __expf(-g.w))) * u.w));
  }
  return load_x(x, r, col, p.n_in, p.dtype);
}

// owner CTA of unit x when CTA b starts at floor(b*U/G)
__device__ __host__ inline int unit_owner(long long x, long long G, long long U) { return (int)(((x + 1) * G - 1) / U); }


__device__ __forceinline__ void async_copy16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
// the same copy, performed only when `on` is non-zero (a predicated instruction: no branch, no reconvergence point)
__device__ __forceinline__ void async_copy16_if(uint32_t smem_addr, const void* gptr, int on) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p cp.async.cg.shared.global [%0], [%1], 16;\n\t}" ::"r"(smem_addr),
      "l"(gptr), "r"(on)
      : "memory");
}
__device__ __forceinline__ void async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

// the K own words of row pair q and the history word, from a tile that sits in shared memory
template <int K>
__device__ __forceinline__ void read_unit_words(const uint32_t* __restrict__ tile, int q, uint32_t (&V)[K + 1]) {
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
    for (int i = 0; i < K; ++i) V[i + 1] = own[i];
  }
  V[0] = tile[history_word<K>(q)];
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
//
// Pipe balance (measured on B200 with issue-rate probes): the hash multiply-add, the byte dot product and
// the packed float ops share one half-rate pipe, the shifts/masks and the byte-wise |a-b| sum share another.
// Three of every four byte sums therefore go through the |a-b| form so that both pipes fill up together.
template <int K, int MT, int ALU4 = 3>
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
        const uint32_t b0 = (2 * half + 2 * rr) % 4 < ALU4 ? code_magic_bits_alu(s[rr * 16 + c0]) : code_magic_bits(s[rr * 16 + c0]);
        const uint32_t b1 = (2 * half + 2 * rr + 1) % 4 < ALU4 ? code_magic_bits_alu(s[rr * 16 + c1]) : code_magic_bits(s[rr * 16 + c1]);
        const float2 w = __fadd2_rn(make_float2(__uint_as_float(b0), __uint_as_float(b1)), unbias);
#pragma unroll
        for (int r = 0; r < MT; ++r) {
          const float2 xp = half ? make_float2(xv[r].z, xv[r].w) : make_float2(xv[r].x, xv[r].y);
          acc[r][rr] = __ffma2_rn(w, xp, acc[r][rr]);
        }
      }
    }
  }
}

// 16-byte asynchronous copy global -> shared when `on` is positive; both addresses carry a compile-time offset inside the instruction
template <int OFF>
__device__ __forceinline__ void async_copy16_at_if(uint32_t smem_addr, const void* gptr, int on) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.gt.s32 p, %2, 0;\n\t@p cp.async.cg.shared.global [%0+%3], [%1+%3], 16;\n\t}" ::"r"(smem_addr),
      "l"(gptr), "r"(on), "n"(OFF)
      : "memory");
}
// the copies of one lane for one trip: both units of a 128-column block, chunk q + 8 j of its strip's tile in either unit
template <int K, int U, int J>
struct GemvTripCopies {
  static __device__ __forceinline__ void run(uint32_t dst, const void* src, int on, int on_tail) {
    constexpr int kChunks = 2 * K, kOff = U * 4 * (32 * K) + J * 128;
    async_copy16_at_if<kOff>(dst, src, 8 * J + 8 <= kChunks ? on : on_tail);
    if constexpr (8 * J + 8 < kChunks) GemvTripCopies<K, U, J + 1>::run(dst, src, on, on_tail);
    else if constexpr (U == 0) GemvTripCopies<K, 1, 0>::run(dst, src, on, on_tail);
  }
};

// ring stages (one trip = one 128-column block = two units of every warp each); one less is in flight
template <int K>
struct GemvStages {
  static constexpr int value = K <= 3 ? 4 : 3;
};
template <int K, int MT>
constexpr int gemv_smem_bytes() { return MT * kStageCols * 4 + GemvStages<K>::value * kGemvWarps * 8 * (32 * K); }

template <int K, int MT>
__global__ void __launch_bounds__(kGemvThreads, (MT == 1 ? 3 : MT == 2 ? 2 : 1)) packed_gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  float* smem = reinterpret_cast<float*>(dyn_smem);                               // [MT][kStageCols], later reductions
  uint32_t* ring = reinterpret_cast<uint32_t*>(dyn_smem + MT * kStageCols * 4);   // [stage][warp][unit of the trip][4 strips][8K]
  __shared__ int s_arrival;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = warp & 1, c = warp >> 1, g = lane >> 3, q = lane & 7;
  const int U = p.units, G = gridDim.x, CG = p.cg, nt = p.nt, n = nt * 16, m = p.mt * 16;
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
  constexpr int kTileWords = 8 * K, kTileBytes = 32 * K, kTileChunks = 2 * K;    // 16-byte chunks per tile
  constexpr int kStages = GemvStages<K>::value, kDepth = kStages - 1;
  constexpr int kStageBytes = kGemvWarps * 8 * kTileBytes;

  // ring slot of (this warp, strip g): a lane group of 8 copies and reads its own tile of either unit
  const uint32_t* my_ring = ring + (warp * 8 + g) * kTileWords;
  const uint32_t ring_dst = (uint32_t)__cvta_generic_to_shared(my_ring) + q * 16;

  int rb = p.split > 0 ? (int)blockIdx.y : u_begin / CG;
  int cgi = u_begin - rb * CG;

  // tensors of this CTA's problem (grouped form: one row block per CTA, so they never change inside a launch)
  const void* x_ptr = p.x;
  const uint32_t* qw_ptr = p.qw;
  const __half* scales_ptr = p.scales;
  const uint8_t* su_ptr = p.su;
  const uint8_t* sv_ptr = p.sv;
  void* y_ptr = p.y;
  int rb_base = 0;
  if (p.group > 0) {
    asm volatile("griddepcontrol.wait;" ::: "memory");            // the pointer lists may come from the preceding kernel
    const int prob = rb / p.rb_per_problem;
    rb_base = prob * p.rb_per_problem;
    const long long entry = p.g_route ? p.g_route[prob] : prob;      // which row of the pointer tables
    if (entry < 0 || entry >= p.g_table_rows) return;               // a route that points outside the tables: skipped, like a null weight
    qw_ptr = p.g_qw[entry];
    if (qw_ptr == nullptr) return;                                  // a problem this rank does not own (expert parallelism): nothing to do
    scales_ptr = p.g_scales[entry];
    su_ptr = p.g_su[entry];
    sv_ptr = p.g_sv[entry];
    if (p.g_route) {
      x_ptr = static_cast<const char*>(p.x) + (size_t)(prob / p.g_xdiv) * p.g_xrow_bytes;
      y_ptr = static_cast<char*>(p.y) + (size_t)prob * p.g_yrow_bytes;
    } else {
      x_ptr = p.g_x[prob];
      y_ptr = p.g_y[prob];
    }
  }

  // Prefetch cursor of the current row block.  A trip brings the whole 128-column block (eight tiles of every strip) even where
  // one of its two units belongs to the neighbouring CTA: only the first and the last block of a range can be such a block.
  // The cursor never crosses a row block: at the end of one the ring runs empty and is primed again.
  const int on_tail = (q + 8 * ((kTileChunks - 1) / 8) < kTileChunks) ? -1 : 0;   // all ones where this lane owns a chunk of the last copy
  const char* pf_src = nullptr;
  int pf_left = 0;                                      // trips of the row block that remain to be fetched
  auto issue = [&](int stage_bytes) {
    // no branches: past the end of the row block's range the copies are predicated off and the cursor runs on harmlessly
    GemvTripCopies<K, 0, 0>::run(ring_dst + stage_bytes, pf_src, pf_left, pf_left & on_tail);
    --pf_left;
    pf_src += 8 * kTileBytes;
    async_commit();
  };
  auto open_row_block = [&](int rb_, int cgi_, int units_left) {
    const int stop = min(CG, cgi_ + units_left);
    pf_left = ((stop + 1) >> 1) - (cgi_ >> 1);
    pf_src = reinterpret_cast<const char*>(qw_ptr) + ((size_t)((rb_ - rb_base) * 8 + 4 * h + g) * nt + (size_t)(8 * (cgi_ >> 1) + c)) * kTileBytes + q * 16;
  };
  open_row_block(rb, cgi, u_end - u_begin);
  issue(0);
  // everything above touched only the weights; what follows reads activations and writes shared state
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  bool predecessor_done = false;
  bool ring_primed = false;                        // independent inputs: stages 1.. are issued behind the first activation loads
  if (!p.independent) {
    // the activations come from the preceding kernel: while it drains, the whole ring is primed
#pragma unroll
    for (int sgi = 1; sgi < kDepth; ++sgi) issue(sgi * kStageBytes);
    ring_primed = true;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    predecessor_done = true;
  }
  __shared__ float s_row_inv[MT];                  // RMSNorm scale per activation row (prologue 1)
  if (p.prologue == 1) {
    // RMSNorm fused into the activation staging: every CTA finds the row scale itself (the row is a few KB in L2), with the
    // copy ring fully primed first so that the weights keep streaming meanwhile
    if (!ring_primed) {
#pragma unroll
      for (int sgi = 1; sgi < kDepth; ++sgi) issue(sgi * kStageBytes);
      ring_primed = true;
    }
    __shared__ float s_ss[kGemvWarps];
#pragma unroll
    for (int r = 0; r < MT; ++r) {
      if (r < p.rows) {
        float ss = 0.f;
        for (int e = tid; e < (n >> 2); e += kGemvThreads) {
          const float4 v = load_quad(x_ptr, (size_t)r * p.x_stride + 4 * e, p.dtype);
          ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(kFullWarp, ss, o);
        __syncthreads();
        if (lane == 0) s_ss[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int k = 0; k < kGemvWarps; ++k) tot += s_ss[k];
        if (tid == 0) s_row_inv[r] = rsqrtf(tot / (float)n + p.eps);   // read after the barrier that opens the first staging
      }
    }
  }

  float2 acc[MT][2];
#pragma unroll
  for (int r = 0; r < MT; ++r) acc[r][0] = acc[r][1] = make_float2(0.f, 0.f);

  int stage_bytes = 0, refill_bytes = (kStages - 1) * kStageBytes;
  int u = u_begin;
  while (u < u_end) {
    // ---- segment: units [cgi, seg_cg_end) lie in row block rb and inside one staged window of activations
    const int hb0 = cgi >> 1;                                       // first 128-column block needed
    const int cg_stop = min(CG, cgi + (u_end - u));                 // this CTA's last column group in rb, exclusive
    const int hb1 = min(hb0 + kStageBlocks, (cg_stop + 1) >> 1);
    const int seg_cg_end = min(cg_stop, hb1 * 2);
    __syncthreads();                                                // the previous users of the staging buffer are done
    const int nblk = hb1 - hb0, items = MT * nblk;
    float4 xv_first = make_float4(0.f, 0.f, 0.f, 0.f);
    const int first_r = MT == 1 ? 0 : warp / nblk;                  // (one activation row: no divisions in the staging)
    if (warp < items && first_r < p.rows)                           // the first item's loads go out before the copy burst
      xv_first = fused_x(p, x_ptr, first_r, (hb0 + warp - first_r * nblk) * 128 + 4 * lane, p.prologue == 1 ? s_row_inv[first_r] : 1.f);
    if (!ring_primed) {
#pragma unroll
      for (int sgi = 1; sgi < kDepth; ++sgi) issue(sgi * kStageBytes);
      ring_primed = true;
    }
    for (int item = warp; item < items; item += kGemvWarps) {
      const int r = MT == 1 ? 0 : item / nblk, hb = hb0 + item - r * nblk;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (r < p.rows) {
        const float4 xv = item == warp ? xv_first : fused_x(p, x_ptr, r, hb * 128 + 4 * lane, p.prologue == 1 ? s_row_inv[r] : 1.f);
        const unsigned sg = sign_nibble(su_ptr, hb * 32 + lane);
        v[0] = flip(xv.x, sg & 1u); v[1] = flip(xv.y, (sg >> 1) & 1u); v[2] = flip(xv.z, (sg >> 2) & 1u); v[3] = flip(xv.w, sg >> 3);
        wht128(v, lane);
      }
      float* dst = smem + r * kStageCols + (hb - hb0) * 128 + (lane >> 2) * 16;
#pragma unroll
      for (int k = 0; k < 4; ++k) dst[staged_col<K>(4 * (lane & 3) + k)] = v[k] * kInvSqrt128;
    }
    __syncthreads();

    // ---- the trips of the window.  A trip: wait for its slot, refill the slot consumed one trip ago, decode FIRST and / or SECOND
    // unit of the block.  Only the first and the last trip of the CTA's range can hold a foreign unit (never both in one trip:
    // such a range would be empty); they are peeled off the steady loop, which has no conditional code.
    const float* xs = smem + c * 16;
    auto trip = [&](auto first, auto second) {
      async_wait<kDepth - 1>();                      // the oldest copy group (this trip) has landed
      __syncwarp();                                  // ... for every lane; and every lane is done with the previous slot
      const uint32_t* tiles = reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(my_ring) + stage_bytes);
      issue(refill_bytes);                           // refill the slot that was consumed one trip ago (or never used yet)
      refill_bytes = stage_bytes;
      stage_bytes = (stage_bytes + kStageBytes == kStages * kStageBytes) ? 0 : stage_bytes + kStageBytes;
      if constexpr (decltype(first)::value) {
        uint32_t V[K + 1];
        read_unit_words<K>(tiles, q, V);
        unit_fma<K, MT>(V, xs, acc);
      }
      if constexpr (decltype(second)::value) {
        uint32_t V[K + 1];
        read_unit_words<K>(tiles + 4 * kTileWords, q, V);
        unit_fma<K, MT>(V, xs + 64, acc);
      }
      xs += 128;
    };
    const int trips = ((seg_cg_end + 1) >> 1) - hb0;
    const bool head = (cgi & 1) != 0, tail = (seg_cg_end & 1) != 0;   // (windows end on block boundaries except at the end of the range)
    const int full = trips - (head ? 1 : 0) - (tail ? 1 : 0);
    if (head) trip(std::false_type{}, std::true_type{});
#pragma unroll 1
    for (int t = 0; t < full; ++t) trip(std::true_type{}, std::true_type{});
    if (tail) trip(std::true_type{}, std::false_type{});
    u += seg_cg_end - cgi;
    cgi = seg_cg_end;
    if (cgi < CG && u < u_end) continue;              // same row block, next staged window

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
    __syncthreads();

    int contributors;
    if (p.split > 0) {
      contributors = p.split;
    } else {
      const int first = unit_owner((long long)rb * CG, G, U);
      contributors = unit_owner((long long)(rb + 1) * CG - 1, G, U) - first + 1;
      slot_index = blockIdx.x - first;
    }
    float* ytil = smem + 4 * MT * 128;                  // [MT][128], disjoint from red (MT*kStageCols >= 5*MT*128)
    // operands of the epilogue are fetched now so that their latency hides behind the arrival handshake
    const int row0 = (rb - rb_base) * 128 + 4 * lane;               // row inside this problem's weight
    uint2 sc_raw = make_uint2(0u, 0u);
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
    unsigned sv_bits = 0;
    if (warp < p.rows) {
      sc_raw = __ldg(reinterpret_cast<const uint2*>(scales_ptr + row0));
      sv_bits = sign_nibble(sv_ptr, (rb - rb_base) * 32 + lane);
      if (p.bias && row0 < p.m_out) bias4 = load_quad(p.bias, row0, p.dtype);
    }
    if (!predecessor_done) {                           // deferred wait of the independent-input form
      asm volatile("griddepcontrol.wait;" ::: "memory");
      predecessor_done = true;
    }
    bool finish = true;
    if (contributors > 1) {
      float* mine = p.part + ((size_t)rb * p.slots + slot_index) * (MT * 128);
      for (int e = tid; e < MT * 128; e += kGemvThreads)
        __stcg(mine + e, red[e] + red[MT * 128 + e] + red[2 * MT * 128 + e] + red[3 * MT * 128 + e]);
      __syncthreads();
      if (tid == 0) {
        __threadfence();                               // the partials of the whole CTA (ordered by the barrier) before the arrival
        s_arrival = atomicAdd(p.counters + rb, 1);   // (the finisher reads the partials with loads served by L2, after this atomic)
      }
      __syncthreads();
      finish = (s_arrival == contributors - 1);
      if (finish) {
        const float* slot0 = p.part + (size_t)rb * p.slots * (MT * 128);
        for (int e = tid; e < MT * 128; e += kGemvThreads) {
          float sum = 0.f;
          for (int base = 0; base < contributors; base += 16) {    // 16 loads in flight, added in slot order
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = base + j < contributors ? __ldcg(slot0 + (size_t)(base + j) * (MT * 128) + e) : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) sum += v[j];
          }
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
      // ---- epilogue of the row block, one warp per activation row
      const int r = warp;
      const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sc_raw.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&sc_raw.y));
      float v[4] = {ytil[r * 128 + 4 * lane] * (s01.x * p.cb), ytil[r * 128 + 4 * lane + 1] * (s01.y * p.cb),
                    ytil[r * 128 + 4 * lane + 2] * (s23.x * p.cb), ytil[r * 128 + 4 * lane + 3] * (s23.y * p.cb)};
      wht128(v, lane);
      float4 o = make_float4(flip(v[0] * kInvSqrt128, sv_bits & 1u), flip(v[1] * kInvSqrt128, (sv_bits >> 1) & 1u),
                             flip(v[2] * kInvSqrt128, (sv_bits >> 2) & 1u), flip(v[3] * kInvSqrt128, sv_bits >> 3));
      o.x += bias4.x; o.y += bias4.y; o.z += bias4.z; o.w += bias4.w;
      if (p.npeer == 0) {
        if (p.residual) {                              // y is the residual stream: add the (bf16-rounded) result in place
          const float4 old = load_quad(y_ptr, (size_t)r * p.m_out + row0, p.dtype);
          o = make_float4(old.x + bf16_round(o.x), old.y + bf16_round(o.y), old.z + bf16_round(o.z), old.w + bf16_round(o.w));
        }
        if (row0 < p.m_out) store_quad(y_ptr, (size_t)r * p.m_out + row0, p.dtype, o);
      } else {
        // (routed form: the problem's output row sits at the same byte offset in every peer's matrix as in y)
        const size_t row_bytes = p.g_route ? (size_t)(static_cast<char*>(y_ptr) - static_cast<char*>(p.y)) : 0;
#pragma unroll 1
        for (int pe = 0; pe < p.npeer; ++pe)
          store_quad(static_cast<char*>(p.peer_y[pe]) + row_bytes, (size_t)p.peer_offset + (size_t)r * m + row0, p.dtype, o);
      }
    }
    if (finish && p.npeer > 0 && p.peer_flag[0] != nullptr) signal_peers_when_last(p, p.counters, p.mt >> 3);
    if (cgi == CG) { cgi = 0; ++rb; }
    if (u < u_end) {
      // the next row block of the range: the ring has run empty (every copy group issued for the old block has been consumed);
      // its weights are fetched while the block's reduction above is still in flight on other warps
      open_row_block(rb, cgi, u_end - u);
      stage_bytes = 0;
      refill_bytes = (kStages - 1) * kStageBytes;
#pragma unroll
      for (int sgi = 0; sgi < kDepth; ++sgi) issue(sgi * kStageBytes);
    }
  }
  async_wait<0>();
}

// HTR_GEMV_OVERLAP=0 in the environment launches without programmatic stream serialisation (for A/B timing)
bool gemv_overlap_enabled();

// host-side launcher of one instantiation, defined once per K in packed_gemv_k*.cu
template <int K>
int launch_packed_gemv(const GemvParams& p, int mt_rows, int grid, cudaStream_t stream);
template <int K>
int packed_gemv_ctas_per_sm(int mt_rows);

}  // namespace htr
