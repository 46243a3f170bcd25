// C interface of the library: argument checks, launch planning and dispatch to the kernels.
#include <cmath>
#include <cstdlib>
#include <mutex>

#include "packed_gemv_mma.cuh"
#include "packed_gemv_tm.cuh"

namespace htr {
int run_decode_raw(int K, const uint32_t* qw, int16_t* out, long long ntiles, cudaStream_t st);
int run_rht(const void* x, int dtype, int M, int n, const uint8_t* su, float* xt, cudaStream_t st);
int run_dequant_w(int K, const uint32_t* qw, const __half* scales, const uint8_t* su, const uint8_t* sv, float cb, void* W,
                  int out_dtype, int mt, int nt, cudaStream_t st);

static thread_local int t_last_cuda = 0;

static int cuda_fail(int e) {
  t_last_cuda = e;
  return HTR_ERR_CUDA;
}

static bool width_ok(int K) { return K == 2 || K == 3 || K == 4 || K == 5 || K == 6 || K == 8; }
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// 1/sqrt(mean v(s)^2) over all 65536 states in double (htr/wire.py:27-30), evaluated once
static double codebook_scale() {
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

static int template_rows(int M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8; }

static int gemv_ctas_per_sm(int K, int mt_rows) {
  switch (K) {
    case 2: return packed_gemv_ctas_per_sm<2>(mt_rows);
    case 3: return packed_gemv_ctas_per_sm<3>(mt_rows);
    case 4: return packed_gemv_ctas_per_sm<4>(mt_rows);
    case 5: return packed_gemv_ctas_per_sm<5>(mt_rows);
    case 6: return packed_gemv_ctas_per_sm<6>(mt_rows);
    case 8: return packed_gemv_ctas_per_sm<8>(mt_rows);
  }
  return -1;
}

static int gemv_mma_config(int K, int rows, int* ctas, int* cap) {
  switch (K) {
    case 2: return packed_gemv_mma_config<2>(rows, ctas, cap);
    case 3: return packed_gemv_mma_config<3>(rows, ctas, cap);
    case 4: return packed_gemv_mma_config<4>(rows, ctas, cap);
    case 5: return packed_gemv_mma_config<5>(rows, ctas, cap);
    case 6: return packed_gemv_mma_config<6>(rows, ctas, cap);
    case 8: return packed_gemv_mma_config<8>(rows, ctas, cap);
  }
  return (int)cudaErrorInvalidValue;
}

static int gemv_tm_config(int K, int rows, int* ctas, int* cap) {
  switch (K) {
    case 2: return packed_gemv_tm_config<2>(rows, ctas, cap);
    case 3: return packed_gemv_tm_config<3>(rows, ctas, cap);
    case 4: return packed_gemv_tm_config<4>(rows, ctas, cap);
    case 5: return packed_gemv_tm_config<5>(rows, ctas, cap);
    case 6: return packed_gemv_tm_config<6>(rows, ctas, cap);
    case 8: return packed_gemv_tm_config<8>(rows, ctas, cap);
  }
  return (int)cudaErrorInvalidValue;
}

// Which kernel serves single problems of up to four activation rows: 0 = CUDA-core GEMV, 1 = warp-MMA GEMV, 2 = tensor-memory
// GEMV, -1 = by measurement (gemv_kind below).  HTR_GEMV_KERNEL in the environment sets the default of the process.
static int gemv_kind_default() {
  static const int kind = [] {
    const char* v = std::getenv("HTR_GEMV_KERNEL");
    const int k = v ? std::atoi(v) : -1;
    return k < -1 || k > 2 ? -1 : k;
  }();
  return kind;
}

bool gemv_overlap_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("HTR_GEMV_OVERLAP");
    return !(v && v[0] == '0');
  }();
  return on;
}

struct Plan {
  int grid, slots, rows_t, split;
  int units;
  int cg, rbs;
  int wblocks;       // warp-MMA kernel: 128-column blocks of activations staged at a time
};

// device facts are cached per device; the occupancy of each instantiation is cached per (device, K, rows)
static int device_sms(int dev) {
  static int cache[64] = {0};
  if (dev >= 0 && dev < 64 && cache[dev]) return cache[dev];
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  if (dev >= 0 && dev < 64) cache[dev] = v;
  return v;
}

static int cached_occupancy(int dev, int K, int rows_t) {
  static int cache[64][9][9] = {{{0}}};
  static std::mutex mu;
  if (dev < 0 || dev >= 64) return gemv_ctas_per_sm(K, rows_t);
  std::lock_guard<std::mutex> lock(mu);
  int& slot = cache[dev][K][rows_t];
  if (slot == 0) slot = gemv_ctas_per_sm(K, rows_t);
  return slot;
}

// warp-MMA kernel: CTAs per SM and the window cap, per (device, K, rows)
static int cached_mma_config(int dev, int K, int rows, int* ctas, int* cap) {
  struct Entry { int ctas, cap; };
  static Entry cache[64][9][kMmaRows + 1] = {};
  static std::mutex mu;
  if (dev < 0 || dev >= 64) return gemv_mma_config(K, rows, ctas, cap);
  std::lock_guard<std::mutex> lock(mu);
  Entry& slot = cache[dev][K][rows];
  if (slot.ctas == 0) {
    int c = 0, w = 0;
    if (const int e = gemv_mma_config(K, rows, &c, &w)) return e;
    slot.ctas = c;
    slot.cap = w;
  }
  *ctas = slot.ctas;
  *cap = slot.cap;
  return 0;
}

// tensor-memory kernel: CTAs per SM and the window cap, per (device, K, rows)
static int cached_tm_config(int dev, int K, int rows, int* ctas, int* cap) {
  struct Entry { int ctas, cap; };
  static Entry cache[64][9][kTmRows + 1] = {};
  static std::mutex mu;
  if (dev < 0 || dev >= 64) return gemv_tm_config(K, rows, ctas, cap);
  std::lock_guard<std::mutex> lock(mu);
  Entry& slot = cache[dev][K][rows];
  if (slot.ctas == 0) {
    int c = 0, w = 0;
    if (const int e = gemv_tm_config(K, rows, &c, &w)) return e;
    slot.ctas = c;
    slot.cap = w;
  }
  *ctas = slot.ctas;
  *cap = slot.cap;
  return 0;
}

// the tensor-memory kernel serves up to four rows of plain activations, rows of at most 16384 columns (32-bit accumulators)
static bool tm_serves(int M, int n, int prologue) { return M >= 1 && M <= kTmRows && n <= kTmMaxCols && prologue == 0; }

static int g_kind_override = -1;                       // -1: environment default, else the kind
// Measured policy (4096x12288 K4, bf16): one row is cheapest on the CUDA-core kernel -- an int8 mma.sync costs about as many issue
// slots as the byte sums and multiply-adds it replaces, and its activation staging is heavier; from two rows on the MMA serves the
// extra rows for free.  Three or four float32 / fp16 rows (which would need more planes than an MMA holds) and five to eight rows
// stay on the CUDA-core kernel.
static int gemv_kind(int M, int dtype = HTR_DTYPE_BF16, int n = 0, int prologue = 0) {
  const int kind = g_kind_override >= 0 ? g_kind_override : gemv_kind_default();
  if (kind == 2 && n > 0 && tm_serves(M, n, prologue)) return 2;
  if (!mma_serves(M, dtype)) return 0;
  return kind == 0 || kind == 1 ? kind : (M >= 2 ? 1 : 0);
}

static int make_plan(int M, int m, int n, int K, Plan* out, int kind = 0) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail((int)e);
  const int sms = device_sms(dev);
  if (sms <= 0) return cuda_fail((int)cudaErrorInvalidDevice);
  Plan pl;
  pl.rows_t = template_rows(M);
  int per_sm = 0, window_cap = 0;
  if (kind == 2) {
    // flat ranges of 64-column units over two thread blocks per SM; a run of L units touches at most L/2 + 1 blocks
    if (const int ce = cached_tm_config(dev, K, M, &per_sm, &window_cap)) return cuda_fail(ce);
    pl.rbs = m / 128;
    if (pl.rbs >= kTmFaultWord) return HTR_ERR_TOO_LARGE;
    pl.cg = n / 64;
    pl.units = pl.rbs * pl.cg;
    const long long slots_all = (long long)sms * per_sm;
    pl.split = 0;
    pl.grid = (int)(slots_all < pl.units ? slots_all : pl.units);
    const int per_cta = pl.units / pl.grid;
    pl.slots = (pl.cg + per_cta - 1) / per_cta + 1;
    const int longest = per_cta + 1 < pl.cg ? per_cta + 1 : pl.cg;
    int need = longest / 2 + 1;
    if (need > pl.cg / 2) need = pl.cg / 2;
    const int windows = (need + window_cap - 1) / window_cap;
    pl.wblocks = (need + windows - 1) / windows;
    *out = pl;
    return HTR_OK;
  }
  if (kind == 1) {
    if (const int ce = cached_mma_config(dev, K, M, &per_sm, &window_cap)) return cuda_fail(ce);
  } else {
    per_sm = cached_occupancy(dev, K, pl.rows_t);
  }
  if (per_sm <= 0) return cuda_fail((int)cudaErrorLaunchOutOfResources);
  pl.rbs = m / 128;
  pl.cg = n / 64;
  pl.units = pl.rbs * pl.cg;
  const long long cap = (long long)sms * per_sm;          // CTAs that are resident together
  // Short ranges: give every row block the same number of CTAs so that none crosses a row block (a crossing costs
  // one extra publish + restage, which is only cheap when a CTA owns many units).  Otherwise: flat even ranges.
  const long long flat_grid = cap < pl.units ? cap : pl.units;
  int longest;                                            // units of one row block that a CTA may own
  long long s = pl.rbs <= cap ? cap / pl.rbs : 0;
  if (s > pl.cg) s = pl.cg;
  // (the split form must also fill the GPU: 149 row blocks on 444 slots would leave a third of them empty with two CTAs per block)
  if (s >= 1 && pl.units / flat_grid < 24 && (5 * pl.rbs * s >= 4 * cap || pl.units / flat_grid < 8)) {
    pl.split = (int)s;
    pl.grid = pl.rbs * pl.split;
    pl.slots = pl.split;
    longest = (pl.cg + pl.split - 1) / pl.split;
  } else {
    pl.split = 0;
    pl.grid = (int)flat_grid;
    // a row block holds cg units and a CTA at least floor(U/G) of them
    const int per_cta = pl.units / pl.grid;
    pl.slots = (pl.cg + per_cta - 1) / per_cta + 1;
    longest = per_cta + 1 < pl.cg ? per_cta + 1 : pl.cg;
  }
  pl.wblocks = 0;
  if (kind == 1) {
    // a run of L units touches at most L/2 + 1 blocks; the windows of a run are made equally long
    int need = longest / 2 + 1;
    if (need > pl.cg / 2) need = pl.cg / 2;
    const int windows = (need + window_cap - 1) / window_cap;
    pl.wblocks = (need + windows - 1) / windows;
  }
  *out = pl;
  return HTR_OK;
}

// the counter region has one fixed size, so that calls of any shape share a workspace without moving it
static size_t counter_bytes(int) { return (size_t)kCounterBytes; }

}  // namespace htr

using namespace htr;

extern "C" {

static int launch_linear(const void* x, int dtype, int M, int n_in, const void* qweight, int mt, int nt, int K, const void* scales,
                         const uint8_t* su, const uint8_t* sv, const void* bias, void* y, int m_out, void* const* peer_y, int npeer,
                         int64_t peer_offset, void* workspace, size_t workspace_bytes, htr_stream_t stream, unsigned flags,
                         int prologue = 0, const void* norm_w = nullptr, float eps = 0.f, int residual = 0, unsigned* const* peer_flags = nullptr);
static int launch_grouped(const void* const* x_list, void* const* y_list, const void* x, void* y, int x_div, int64_t x_row_stride,
                          const int64_t* route, int table_rows, int prologue, int dtype, const void* const* qweight_list, int mt, int nt, int K,
                          const void* const* scales_list, const uint8_t* const* su_list, const uint8_t* const* sv_list, int count,
                          void* workspace, size_t workspace_bytes, htr_stream_t stream, void* const* peer_y = nullptr, int npeer = 0,
                          int share = 1);


const char* htr_status_string(int status) {
  switch (status) {
    case HTR_OK: return "ok";
    case HTR_ERR_BAD_K: return "unsupported bits per weight (K must be 2, 3, 4, 5, 6 or 8)";
    case HTR_ERR_BAD_SHAPE: return "bad shape (m and n must be positive multiples of 128; row count out of range)";
    case HTR_ERR_BAD_DTYPE: return "unsupported element type";
    case HTR_ERR_WORKSPACE: return "workspace missing or too small";
    case HTR_ERR_NULL: return "required pointer is NULL";
    case HTR_ERR_ALIGNMENT: return "pointer is not 16-byte aligned";
    case HTR_ERR_CUDA: return "CUDA runtime error";
    case HTR_ERR_TOO_LARGE: return "size exceeds the limit of this entry point";
  }
  return "unknown status";
}

int htr_last_cuda_error(void) { return t_last_cuda; }
int htr_version(void) { return 100; }

void htr_set_gemv_kernel(int kind) { g_kind_override = kind < 0 || kind > 2 ? -1 : kind; }   // -1: back to the default

size_t htr_linear_fault_offset(void) { return (size_t)kTmFaultWord * 4; }

int htr_decode_raw(const void* qweight, int64_t ntiles, int K, int16_t* out, htr_stream_t stream) {
  if (!width_ok(K)) return HTR_ERR_BAD_K;
  if (ntiles < 0 || ntiles > (1ll << 34)) return HTR_ERR_BAD_SHAPE;
  if (ntiles == 0) return HTR_OK;
  if (!qweight || !out) return HTR_ERR_NULL;
  if (!aligned16(qweight) || !aligned16(out)) return HTR_ERR_ALIGNMENT;
  const int e = run_decode_raw(K, static_cast<const uint32_t*>(qweight), out, ntiles, static_cast<cudaStream_t>(stream));
  return e ? cuda_fail(e) : HTR_OK;
}

int htr_rht(const void* x, int dtype, int M, int n, const uint8_t* su, float* xt, htr_stream_t stream) {
  if (dtype < HTR_DTYPE_BF16 || dtype > HTR_DTYPE_F32) return HTR_ERR_BAD_DTYPE;
  if (M < 0 || n <= 0 || n % 128) return HTR_ERR_BAD_SHAPE;
  if (M == 0) return HTR_OK;
  if (!x || !su || !xt) return HTR_ERR_NULL;
  if (!aligned16(x) || !aligned16(xt)) return HTR_ERR_ALIGNMENT;
  const int e = run_rht(x, dtype, M, n, su, xt, static_cast<cudaStream_t>(stream));
  return e ? cuda_fail(e) : HTR_OK;
}

size_t htr_linear_counter_bytes(int m) { return counter_bytes(m); }

size_t htr_linear_workspace_bytes(int M, int m, int n, int K) {
  if (!width_ok(K) || M < 1 || M > HTR_GEMV_MAX_ROWS || m <= 0 || n <= 0 || m % 128 || n % 128) return 0;
  Plan pl;
  if (make_plan(M, m, n, K, &pl) != HTR_OK) return 0;
  size_t slots = (size_t)pl.slots;
  if (M <= kMmaRows) {                                   // any of the kernels may serve the call: size for all
    Plan mma;
    if (make_plan(M, m, n, K, &mma, 1) != HTR_OK) return 0;
    if ((size_t)mma.slots > slots) slots = (size_t)mma.slots;
    if (tm_serves(M, n, 0)) {
      Plan tm;
      if (make_plan(M, m, n, K, &tm, 2) != HTR_OK) return 0;
      if ((size_t)tm.slots > slots) slots = (size_t)tm.slots;
    }
  }
  // up to four rows may run in an integer-exact form, whose partial sums are 64-bit
  return counter_bytes(m) + (size_t)pl.rbs * slots * pl.rows_t * 128 * (M <= kMmaRows ? sizeof(long long) : sizeof(float));
}

int htr_linear_plan(int M, int m, int n, int K, int* grid, int* slots_per_block) {
  if (!width_ok(K)) return HTR_ERR_BAD_K;
  if (M < 1 || M > HTR_GEMV_MAX_ROWS || m <= 0 || n <= 0 || m % 128 || n % 128) return HTR_ERR_BAD_SHAPE;
  Plan pl;
  const int rc = make_plan(M, m, n, K, &pl, gemv_kind(M, HTR_DTYPE_BF16, n, 0));
  if (rc != HTR_OK) return rc;
  if (grid) *grid = pl.grid;
  if (slots_per_block) *slots_per_block = pl.slots;
  return HTR_OK;
}

int htr_linear(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su,
               const uint8_t* sv, const void* bias, void* y, void* workspace, size_t workspace_bytes, htr_stream_t stream) {
  return htr_linear_ex(x, dtype, M, qweight, mt, nt, K, scales, su, sv, bias, y, workspace, workspace_bytes, stream, 0u);
}

int htr_linear_ex(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su,
                  const uint8_t* sv, const void* bias, void* y, void* workspace, size_t workspace_bytes, htr_stream_t stream,
                  unsigned flags) {
  return htr_linear_peers(x, dtype, M, qweight, mt, nt, K, scales, su, sv, bias, y, nullptr, 0, 0, workspace, workspace_bytes, stream, flags);
}

int htr_linear_peers(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su,
                     const uint8_t* sv, const void* bias, void* y, void* const* peer_y, int npeer, int64_t peer_offset, void* workspace,
                     size_t workspace_bytes, htr_stream_t stream, unsigned flags) {
  return launch_linear(x, dtype, M, nt * 16, qweight, mt, nt, K, scales, su, sv, bias, y, mt * 16, peer_y, npeer, peer_offset, workspace,
                       workspace_bytes, stream, flags);
}

int htr_linear_peers_signal(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su,
                            const uint8_t* sv, const void* bias, void* const* peer_y, unsigned* const* peer_flags, int npeer, int64_t peer_offset,
                            void* workspace, size_t workspace_bytes, htr_stream_t stream, unsigned flags) {
  if (!peer_flags) return HTR_ERR_NULL;
  return launch_linear(x, dtype, M, nt * 16, qweight, mt, nt, K, scales, su, sv, bias, nullptr, mt * 16, peer_y, npeer, peer_offset, workspace,
                       workspace_bytes, stream, flags, 0, nullptr, 0.f, 0, peer_flags);
}

int htr_linear_padded(const void* x, int dtype, int M, int n_in, const void* qweight, int mt, int nt, int K, const void* scales,
                      const uint8_t* su, const uint8_t* sv, const void* bias, void* y, int m_out, void* workspace, size_t workspace_bytes,
                      htr_stream_t stream) {
  if (mt <= 0 || nt <= 0) return HTR_ERR_BAD_SHAPE;
  if (n_in < 8 || n_in > nt * 16 || n_in % 8 || m_out < 8 || m_out > mt * 16 || m_out % 8) return HTR_ERR_BAD_SHAPE;
  return launch_linear(x, dtype, M, n_in, qweight, mt, nt, K, scales, su, sv, bias, y, m_out, nullptr, 0, 0, workspace, workspace_bytes,
                       stream, 0u);
}

int htr_linear_fused(const void* x, int M, const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su,
                     const uint8_t* sv, void* y, void* workspace, size_t workspace_bytes, htr_stream_t stream, int prologue,
                     const void* norm_weight, float eps, int residual) {
  if (prologue < HTR_PROLOGUE_NONE || prologue > HTR_PROLOGUE_SWIGLU || (residual != 0 && residual != 1)) return HTR_ERR_BAD_SHAPE;
  if (prologue == HTR_PROLOGUE_RMSNORM && (!norm_weight || !aligned16(norm_weight))) return norm_weight ? HTR_ERR_ALIGNMENT : HTR_ERR_NULL;
  if (mt <= 0 || nt <= 0) return HTR_ERR_BAD_SHAPE;
  return launch_linear(x, HTR_DTYPE_BF16, M, nt * 16, qweight, mt, nt, K, scales, su, sv, nullptr, y, mt * 16, nullptr, 0, 0, workspace,
                       workspace_bytes, stream, 0u, prologue, norm_weight, eps, residual);
}

// shared body of the single-problem entry points: x has n_in <= n columns (the rest read as zeros), y gets the first m_out <= m rows
static int launch_linear(const void* x, int dtype, int M, int n_in, const void* qweight, int mt, int nt, int K, const void* scales,
                         const uint8_t* su, const uint8_t* sv, const void* bias, void* y, int m_out, void* const* peer_y, int npeer,
                         int64_t peer_offset, void* workspace, size_t workspace_bytes, htr_stream_t stream, unsigned flags, int prologue,
                         const void* norm_w, float eps, int residual, unsigned* const* peer_flags) {
  if (!width_ok(K)) return HTR_ERR_BAD_K;
  if (dtype < HTR_DTYPE_BF16 || dtype > HTR_DTYPE_F32) return HTR_ERR_BAD_DTYPE;
  if (M < 0 || M > HTR_GEMV_MAX_ROWS || mt <= 0 || nt <= 0 || mt % 8 || nt % 8) return HTR_ERR_BAD_SHAPE;
  if (mt / 8 > kDoneCounter || (long long)(mt / 8) * (nt / 4) > 0x3FFFFFFFll) return HTR_ERR_TOO_LARGE;
  if (peer_flags) {
    if (npeer < 1) return HTR_ERR_BAD_SHAPE;
    for (int i = 0; i < npeer; ++i)
      if (!peer_flags[i]) return HTR_ERR_NULL;
  }
  if (M == 0) return HTR_OK;
  if (npeer < 0 || npeer > 8 || (npeer > 0 && !peer_y) || peer_offset < 0 || (peer_offset & 7)) return HTR_ERR_BAD_SHAPE;
  if (!x || !qweight || !scales || !su || !sv || (!y && npeer == 0)) return HTR_ERR_NULL;
  for (int i = 0; i < npeer; ++i)
    if (!peer_y[i] || !aligned16(peer_y[i])) return HTR_ERR_ALIGNMENT;
  if (!aligned16(x) || !aligned16(qweight) || !aligned16(y) || (bias && !aligned16(bias)) || !aligned16(workspace) ||
      !aligned16(scales))
    return HTR_ERR_ALIGNMENT;
  const int m = mt * 16, n = nt * 16;
  Plan pl;
  // the integer-exact form: up to two rows (four byte planes per activation), plain activations
  // (the tensor-memory kernel always sums in integers; its grid of integers differs from the warp-MMA kernel's, so a process
  // should keep to one of them where results of differently sharded launches are compared bit for bit)
  int kind = gemv_kind(M, dtype, n, prologue);
  const bool exact = (flags & HTR_LINEAR_EXACT_SUMS) && prologue == 0 && (M <= 2 || kind == 2);
  if (exact && kind != 2) kind = 1;
  const int rc = make_plan(M, m, n, K, &pl, kind);
  if (rc != HTR_OK) return rc;
  const size_t need = counter_bytes(m) + (size_t)pl.rbs * pl.slots * pl.rows_t * 128 * ((exact || kind == 2) ? sizeof(long long) : sizeof(float));
  if (!workspace || workspace_bytes < need) return HTR_ERR_WORKSPACE;

  GemvParams p;
  p.x = x;
  p.qw = static_cast<const uint32_t*>(qweight);
  p.scales = static_cast<const __half*>(scales);
  p.su = su;
  p.sv = sv;
  p.bias = bias;
  p.y = y;
  p.counters = static_cast<int*>(workspace);
  p.part = reinterpret_cast<float*>(static_cast<char*>(workspace) + counter_bytes(m));
  p.rows = M;
  p.mt = mt;
  p.nt = nt;
  p.dtype = dtype;
  p.cg = pl.cg;
  p.units = pl.units;
  p.split = pl.split;
  p.cg_quot = pl.split > 0 ? pl.cg / pl.split : 0;
  p.cg_rem = pl.split > 0 ? pl.cg % pl.split : 0;
  p.independent = (flags & HTR_LINEAR_INPUT_INDEPENDENT) ? 1 : 0;
  p.n_in = n_in;
  p.m_out = m_out;
  p.g_route = nullptr;
  p.g_table_rows = 0;
  p.g_xdiv = 1;
  p.g_xrow_bytes = 0;
  p.g_yrow_bytes = 0;
  p.prologue = prologue;
  p.residual = residual;
  p.x_stride = prologue == 2 ? 2 * n_in : n_in;
  p.norm_w = norm_w;
  p.eps = eps;
  p.group = 0;
  p.rb_per_problem = 0;
  p.g_x = nullptr; p.g_qw = nullptr; p.g_scales = nullptr; p.g_su = nullptr; p.g_sv = nullptr; p.g_y = nullptr;
  p.npeer = npeer;
  p.peer_offset = peer_offset;
  for (int i = 0; i < 8; ++i) p.peer_y[i] = i < npeer ? peer_y[i] : nullptr;
  for (int i = 0; i < 8; ++i) p.peer_flag[i] = (peer_flags && i < npeer) ? peer_flags[i] : nullptr;
  p.slots = pl.slots;
  p.wblocks = pl.wblocks;
  p.exact = exact ? 1 : 0;
  p.cb = (float)codebook_scale();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int e = 0;
  if (kind == 2) {
    switch (K) {
      case 2: e = launch_packed_gemv_tm<2>(p, pl.grid, st); break;
      case 3: e = launch_packed_gemv_tm<3>(p, pl.grid, st); break;
      case 4: e = launch_packed_gemv_tm<4>(p, pl.grid, st); break;
      case 5: e = launch_packed_gemv_tm<5>(p, pl.grid, st); break;
      case 6: e = launch_packed_gemv_tm<6>(p, pl.grid, st); break;
      case 8: e = launch_packed_gemv_tm<8>(p, pl.grid, st); break;
    }
    return e ? cuda_fail(e) : HTR_OK;
  }
  if (kind == 1) {
    switch (K) {
      case 2: e = launch_packed_gemv_mma<2>(p, pl.grid, st); break;
      case 3: e = launch_packed_gemv_mma<3>(p, pl.grid, st); break;
      case 4: e = launch_packed_gemv_mma<4>(p, pl.grid, st); break;
      case 5: e = launch_packed_gemv_mma<5>(p, pl.grid, st); break;
      case 6: e = launch_packed_gemv_mma<6>(p, pl.grid, st); break;
      case 8: e = launch_packed_gemv_mma<8>(p, pl.grid, st); break;
    }
    return e ? cuda_fail(e) : HTR_OK;
  }
  switch (K) {
    case 2: e = launch_packed_gemv<2>(p, pl.rows_t, pl.grid, st); break;
    case 3: e = launch_packed_gemv<3>(p, pl.rows_t, pl.grid, st); break;
    case 4: e = launch_packed_gemv<4>(p, pl.rows_t, pl.grid, st); break;
    case 5: e = launch_packed_gemv<5>(p, pl.rows_t, pl.grid, st); break;
    case 6: e = launch_packed_gemv<6>(p, pl.rows_t, pl.grid, st); break;
    case 8: e = launch_packed_gemv<8>(p, pl.rows_t, pl.grid, st); break;
  }
  return e ? cuda_fail(e) : HTR_OK;
}

size_t htr_linear_grouped_workspace_bytes(int count, int m, int n, int K) {
  if (!width_ok(K) || count < 1 || m <= 0 || n <= 0 || m % 128 || n % 128) return 0;
  Plan pl;
  if (make_plan(1, m, n, K, &pl) != HTR_OK) return 0;
  // at most n/64 CTAs share a row block
  return counter_bytes(m) + (size_t)count * (m / 128) * (size_t)(n / 64) * 128 * sizeof(float);
}

int htr_linear_grouped(const void* const* x_list, int dtype, const void* const* qweight_list, int mt, int nt, int K,
                       const void* const* scales_list, const uint8_t* const* su_list, const uint8_t* const* sv_list, void* const* y_list,
                       int count, void* workspace, size_t workspace_bytes, htr_stream_t stream) {
  if (count > 0 && (!x_list || !y_list)) return HTR_ERR_NULL;
  return launch_grouped(x_list, y_list, nullptr, nullptr, 1, 0, nullptr, count, 0, dtype, qweight_list, mt, nt, K, scales_list, su_list, sv_list, count,
                        workspace, workspace_bytes, stream);
}

int htr_linear_routed(const void* x, int dtype, int x_div, int64_t x_row_stride, const int64_t* route, int count, int table_rows,
                      const void* const* qweight_table, const void* const* scales_table, const uint8_t* const* su_table,
                      const uint8_t* const* sv_table, int mt, int nt, int K, void* y, int prologue, void* workspace, size_t workspace_bytes,
                      htr_stream_t stream) {
  if (count > 0 && (!x || !y || !route)) return HTR_ERR_NULL;
  if (x_div < 1 || x_row_stride < 0 || table_rows < 1 || (prologue != HTR_PROLOGUE_NONE && prologue != HTR_PROLOGUE_SWIGLU))
    return HTR_ERR_BAD_SHAPE;
  if (prologue == HTR_PROLOGUE_SWIGLU && dtype != HTR_DTYPE_BF16) return HTR_ERR_BAD_DTYPE;
  if (count > 0 && (!aligned16(x) || !aligned16(y))) return HTR_ERR_ALIGNMENT;
  return launch_grouped(nullptr, nullptr, x, y, x_div, x_row_stride, route, table_rows, prologue, dtype, qweight_table, mt, nt, K, scales_table, su_table,
                        sv_table, count, workspace, workspace_bytes, stream);
}

int htr_linear_routed_peers(const void* x, int dtype, int x_div, int64_t x_row_stride, const int64_t* route, int count, int table_rows,
                            const void* const* qweight_table, const void* const* scales_table, const uint8_t* const* su_table,
                            const uint8_t* const* sv_table, int mt, int nt, int K, void* y, void* const* peer_y, int npeer, int share,
                            int prologue, void* workspace, size_t workspace_bytes, htr_stream_t stream) {
  if (count > 0 && (!x || !y || !route)) return HTR_ERR_NULL;
  if (npeer < 0 || npeer > 8 || (npeer > 0 && !peer_y) || share < 1 || share > 64) return HTR_ERR_BAD_SHAPE;
  if (x_div < 1 || x_row_stride < 0 || table_rows < 1 || (prologue != HTR_PROLOGUE_NONE && prologue != HTR_PROLOGUE_SWIGLU))
    return HTR_ERR_BAD_SHAPE;
  if (prologue == HTR_PROLOGUE_SWIGLU && dtype != HTR_DTYPE_BF16) return HTR_ERR_BAD_DTYPE;
  if (count > 0 && (!aligned16(x) || !aligned16(y))) return HTR_ERR_ALIGNMENT;
  return launch_grouped(nullptr, nullptr, x, y, x_div, x_row_stride, route, table_rows, prologue, dtype, qweight_table, mt, nt, K, scales_table, su_table,
                        sv_table, count, workspace, workspace_bytes, stream, peer_y, npeer, share);
}

// shared body of the grouped entry points: per-problem pointer lists (x_list / y_list), or a route into per-expert tables with the
// activations and outputs as rows of two matrices
static int launch_grouped(const void* const* x_list, void* const* y_list, const void* x, void* y, int x_div, int64_t x_row_stride,
                          const int64_t* route, int table_rows, int prologue, int dtype, const void* const* qweight_list, int mt, int nt, int K,
                          const void* const* scales_list, const uint8_t* const* su_list, const uint8_t* const* sv_list, int count,
                          void* workspace, size_t workspace_bytes, htr_stream_t stream, void* const* peer_y, int npeer, int share) {
  if (!width_ok(K)) return HTR_ERR_BAD_K;
  if (dtype < HTR_DTYPE_BF16 || dtype > HTR_DTYPE_F32) return HTR_ERR_BAD_DTYPE;
  if (count < 0 || mt <= 0 || nt <= 0 || mt % 8 || nt % 8) return HTR_ERR_BAD_SHAPE;
  if (count == 0) return HTR_OK;
  if (!qweight_list || !scales_list || !su_list || !sv_list) return HTR_ERR_NULL;
  const int m = mt * 16, n = nt * 16, rbp = m / 128;
  if ((long long)count * rbp > kDoneCounter) return HTR_ERR_TOO_LARGE;
  if (!aligned16(workspace)) return HTR_ERR_ALIGNMENT;
  Plan pl;
  const int rc = make_plan(1, m, n, K, &pl);
  if (rc != HTR_OK) return rc;
  int dev = 0;
  cudaGetDevice(&dev);
  const int sms = device_sms(dev);
  const int per_sm = cached_occupancy(dev, K, 1);
  const long long cap = (long long)sms * per_sm;
  const long long rbs = (long long)count * rbp;
  // `share`: only one problem in `share` has its weights here (expert parallelism: the thread blocks of the others leave at once),
  // so the grid is made that many times larger than the GPU
  long long split = cap * (share < 1 ? 1 : share) / rbs;
  if (split < 1) split = 1;
  if (split > pl.cg) split = pl.cg;
  const size_t need = counter_bytes(m) + (size_t)rbs * (size_t)split * 128 * sizeof(float);
  if (!workspace || workspace_bytes < need) return HTR_ERR_WORKSPACE;

  GemvParams p;
  p.x = x; p.qw = nullptr; p.scales = nullptr; p.su = nullptr; p.sv = nullptr; p.bias = nullptr; p.y = y;
  p.counters = static_cast<int*>(workspace);
  p.part = reinterpret_cast<float*>(static_cast<char*>(workspace) + counter_bytes(m));
  p.rows = 1;
  p.mt = mt;
  p.nt = nt;
  p.dtype = dtype;
  p.cg = pl.cg;
  p.units = (int)(rbs * pl.cg);
  p.split = (int)split;
  p.cg_quot = pl.cg / (int)split;
  p.cg_rem = pl.cg % (int)split;
  p.slots = (int)split;
  p.independent = 0;
  p.cb = (float)codebook_scale();
  if (npeer < 0 || npeer > 8 || (npeer > 0 && (!peer_y || !route))) return HTR_ERR_BAD_SHAPE;
  for (int i = 0; i < npeer; ++i)
    if (!peer_y[i] || !aligned16(peer_y[i])) return HTR_ERR_ALIGNMENT;
  p.npeer = npeer;
  p.n_in = nt * 16;
  p.m_out = mt * 16;
  p.prologue = prologue;
  p.residual = 0;
  p.x_stride = prologue == HTR_PROLOGUE_SWIGLU ? 2 * nt * 16 : nt * 16;
  p.norm_w = nullptr;
  p.eps = 0.f;
  p.g_route = reinterpret_cast<const long long*>(route);
  p.g_table_rows = table_rows;
  p.g_xdiv = x_div;
  const long long esz = dtype == HTR_DTYPE_F32 ? 4 : 2;
  p.g_xrow_bytes = (long long)x_row_stride * esz;
  p.g_yrow_bytes = (long long)m * esz;
  p.peer_offset = 0;
  for (int i = 0; i < 8; ++i) p.peer_y[i] = i < npeer ? peer_y[i] : nullptr;
  for (int i = 0; i < 8; ++i) p.peer_flag[i] = nullptr;
  p.wblocks = 0;
  p.exact = 0;
  p.group = count;
  p.rb_per_problem = rbp;
  p.g_x = x_list;
  p.g_qw = reinterpret_cast<const uint32_t* const*>(qweight_list);
  p.g_scales = reinterpret_cast<const __half* const*>(scales_list);
  p.g_su = su_list;
  p.g_sv = sv_list;
  p.g_y = y_list;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = (int)(rbs * split);
  int e = 0;
  switch (K) {
    case 2: e = launch_packed_gemv<2>(p, 1, grid, st); break;
    case 3: e = launch_packed_gemv<3>(p, 1, grid, st); break;
    case 4: e = launch_packed_gemv<4>(p, 1, grid, st); break;
    case 5: e = launch_packed_gemv<5>(p, 1, grid, st); break;
    case 6: e = launch_packed_gemv<6>(p, 1, grid, st); break;
    case 8: e = launch_packed_gemv<8>(p, 1, grid, st); break;
  }
  return e ? cuda_fail(e) : HTR_OK;
}

int htr_dequant_w(const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su, const uint8_t* sv, void* W,
                  int out_dtype, htr_stream_t stream) {
  if (!width_ok(K)) return HTR_ERR_BAD_K;
  if (out_dtype < HTR_DTYPE_BF16 || out_dtype > HTR_DTYPE_F32) return HTR_ERR_BAD_DTYPE;
  if (mt <= 0 || nt <= 0 || mt % 8 || nt % 8 || mt / 8 > 65535) return HTR_ERR_BAD_SHAPE;
  if (!qweight || !scales || !su || !sv || !W) return HTR_ERR_NULL;
  if (!aligned16(qweight) || !aligned16(W)) return HTR_ERR_ALIGNMENT;
  const int e = run_dequant_w(K, static_cast<const uint32_t*>(qweight), static_cast<const __half*>(scales), su, sv,
                              (float)codebook_scale(), W, out_dtype, mt, nt, static_cast<cudaStream_t>(stream));
  return e ? cuda_fail(e) : HTR_OK;
}

}  // extern "C"
