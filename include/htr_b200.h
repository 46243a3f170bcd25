/*
 * htr_b200 -- C interface of the B200 (sm_100a) packed-linear library for HTR-W1 weights.
 *
 * Every entry point takes plain device pointers and sizes, launches on the given CUDA stream
 * without synchronising the host, and returns HTR_OK or a negative status; nothing aborts.
 * Each declaration names the interface of the reference (HawgAuto/HTR) that it stands in for.
 *
 * Tensor contract (docs/FORMAT.md:25-32 of the reference):
 *   qweight  int32/uint32 [m/16, n/16, 8*K] contiguous, 16-byte aligned; K in {2,3,4,5,6,8}
 *   scales   float16 [m]            su  uint8 [n/8]           sv  uint8 [m/8]
 *   m % 128 == 0 and n % 128 == 0.  Activations / outputs are row-major [M, n] / [M, m].
 */
#ifndef HTR_B200_H_
#define HTR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes (0 = success; the reference raises RuntimeError from TORCH_CHECK, htr_kernels.cu:910-915) */
enum {
  HTR_OK = 0,
  HTR_ERR_BAD_K = -1,        /* K outside {2,3,4,5,6,8} */
  HTR_ERR_BAD_SHAPE = -2,    /* m or n not a multiple of 128, negative sizes, M out of range */
  HTR_ERR_BAD_DTYPE = -3,    /* dtype not one of HTR_DTYPE_* */
  HTR_ERR_WORKSPACE = -4,    /* workspace missing or smaller than htr_linear_workspace_bytes() */
  HTR_ERR_NULL = -5,         /* a required pointer is NULL */
  HTR_ERR_ALIGNMENT = -6,    /* a pointer is not 16-byte aligned */
  HTR_ERR_CUDA = -7,         /* a CUDA runtime call failed; see htr_last_cuda_error() */
  HTR_ERR_TOO_LARGE = -8     /* size beyond what the entry point supports */
};

/* activation / output element types; numbering follows the reference's out_dtype (htr/ops.py:79) */
enum { HTR_DTYPE_BF16 = 0, HTR_DTYPE_F16 = 1, HTR_DTYPE_F32 = 2 };

/* largest activation row count a single htr_linear call accepts through the streaming GEMV kernel */
#define HTR_GEMV_MAX_ROWS 8

typedef void* htr_stream_t; /* a cudaStream_t (NULL = the legacy default stream) */

const char* htr_status_string(int status);
int htr_last_cuda_error(void);  /* cudaError_t of the most recent HTR_ERR_CUDA on the calling thread */
int htr_version(void);

/* Integer codebook values of every tile, int16 [ntiles, 256] in stream order.
 * Stands in for decode_raw (htr/csrc/htr_kernels.cpp:4, kernel k_decode_raw htr_kernels.cu:153-172);
 * must equal wire.gen_values(wire.unpack_states(words, K)) bit for bit (htr/wire.py:10-13,54-63). */
int htr_decode_raw(const void* qweight, int64_t ntiles, int K, int16_t* out, htr_stream_t stream);

/* Activation transform xt = blockdiag(H128/sqrt(128)) (su * x), float32 [M, n].
 * Stands in for prologue (htr_kernels.cpp:5, k_prologue htr_kernels.cu:189-234); unlike the reference it
 * keeps float32 and needs no per-token range scale.  Reference math: docs/FORMAT.md:8. */
int htr_rht(const void* x, int dtype, int M, int n, const uint8_t* su, float* xt, htr_stream_t stream);

/* Bytes of scratch one htr_linear call with these sizes may touch (partial sums of the column splits and
 * one arrival counter per 128-row block).  The first htr_linear_counter_bytes(m) bytes hold the counters:
 * they must be zero before the first call and every call leaves them zero again.  One workspace may be
 * shared by calls that are ordered on one stream; concurrent streams need one each.
 * Stands in for the per-call `part` allocation and the persistent `counters` tensor (htr/ops.py:24-28). */
size_t htr_linear_workspace_bytes(int M, int m, int n, int K);
size_t htr_linear_counter_bytes(int m);

/* y[M, m] = x[M, n] @ W^T (+ bias) for one HTR-W1 weight, y/bias in the dtype of x.  One launch: input
 * sign flip + Hadamard, streaming decode of the trellis words with the dot products, split reduction,
 * row scales, output Hadamard, output signs, bias, cast.  1 <= M <= HTR_GEMV_MAX_ROWS (M == 0 returns at once).
 * Stands in for the decode branch of _linear_impl (htr/ops.py:69-101): prologue + gemv_epi / gemv_fused
 * (htr_kernels.cu:337-652).  Must match x.float() @ wire.dequant(...).T (htr/wire.py:105-113). */
int htr_linear(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales,
               const uint8_t* su, const uint8_t* sv, const void* bias /* may be NULL */, void* y, void* workspace,
               size_t workspace_bytes, htr_stream_t stream);

/* htr_linear with flags.  HTR_LINEAR_INPUT_INDEPENDENT promises that x, bias and y are neither written nor read by
 * the kernel that precedes this call in the stream; the launch then overlaps that kernel completely and waits for
 * it only before it touches the shared workspace.  Without the flag the launch still starts early and prefetches
 * packed words, but waits for its predecessor before reading x.  (No counterpart in the reference, whose
 * launches serialise on the stream, htr_kernels.cu:920.) */
#define HTR_LINEAR_INPUT_INDEPENDENT 1u
/* HTR_LINEAR_EXACT_SUMS asks for the kernel that accumulates in exact integers (the warp-MMA GEMV: up to two rows of any type,
 * three or four bf16 rows; other calls ignore the flag).  Its results do not depend on how the launch is cut into thread blocks,
 * so a row shard of a linear reproduces the rows of the unsharded result bit for bit whatever the number of shards.  At one row it
 * costs a few per cent against the default kernel, whose float32 sums follow the launch decomposition. */
#define HTR_LINEAR_EXACT_SUMS 2u
int htr_linear_ex(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales,
                  const uint8_t* su, const uint8_t* sv, const void* bias /* may be NULL */, void* y, void* workspace,
                  size_t workspace_bytes, htr_stream_t stream, unsigned flags);

/* htr_linear_ex for a row shard of a taller linear on one NVLink box: with npeer > 0 the epilogue stores the result rows
 * into every buffer of peer_y[0..npeer) (device addresses of this and the peer GPUs' gather buffers as mapped into this
 * process, e.g. by CUDA IPC or torch symmetric memory) at element offset peer_offset, with plain stores, and y is not
 * written.  The stores are complete when the kernel is; consumers on other GPUs still need their own ordering (a
 * barrier across the ranks) before they read.  peer_offset must be a multiple of 8 elements.  (No counterpart in the
 * reference, which is single-GPU: htr/vllm_plugin.py:91.) */
int htr_linear_peers(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales,
                     const uint8_t* su, const uint8_t* sv, const void* bias /* may be NULL */, void* y /* may be NULL when npeer > 0 */,
                     void* const* peer_y, int npeer, int64_t peer_offset, void* workspace, size_t workspace_bytes,
                     htr_stream_t stream, unsigned flags);

/* htr_linear_peers that also tells the peers when this rank's rows have arrived, so that no barrier across the ranks is needed:
 * peer_flags[i] is the address, as mapped into this process, of the 32-bit word "this rank has delivered" in the memory of the
 * GPU that owns peer_y[i].  The thread block that finishes the launch's last row block adds 1 to each of them (system scope,
 * after a system-wide fence behind the stores).  The consumer orders itself with htr_peer_wait on its own stream.  Uses the last
 * arrival counter of the workspace as the launch-wide count (m / 128 must stay below 16383).  A rank must have consumed the
 * result of call i - 1 (on its stream) before it launches call i + 1 into the same buffer: callers alternate two buffers.
 * (No counterpart in the reference.) */
int htr_linear_peers_signal(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales,
                            const uint8_t* su, const uint8_t* sv, const void* bias /* may be NULL */, void* const* peer_y,
                            unsigned* const* peer_flags, int npeer, int64_t peer_offset, void* workspace, size_t workspace_bytes,
                            htr_stream_t stream, unsigned flags);
/* Consumer side of the delivery flags: one small kernel on `stream` that waits until each of flags[0..nranks) (this GPU's words,
 * one per producing rank) has reached *epoch + count (count deliveries per rank since the last wait), then stores that number to *epoch (both in device memory: the sequence
 * survives CUDA-graph replay).  The wait is bounded (about two seconds); a producer that has not delivered by then gets its bit
 * set in *status (device int, may be NULL) and the kernel returns: the buffer then holds stale rows. */
int htr_peer_wait(const unsigned* flags, unsigned* epoch, int nranks, int count, int* status, htr_stream_t stream);
/* Barrier across the ranks of one NVLink box as one small kernel per rank (no collective library): peer_word[r] = the address, as
 * mapped into this process, of THIS rank's word in rank r's flag array (a DEVICE array of nranks pointers, this rank's own
 * included); flags = this GPU's flag array (word r is raised by rank r); *epoch = barriers passed so far (device memory: survives
 * CUDA-graph replay).  The kernel first waits for everything launched before it on `stream` (peer stores of the preceding kernel are
 * complete and flushed then), raises its word everywhere and waits until every rank has raised its word here.  The wait is bounded
 * (about two seconds): a rank that has not arrived by then gets its bit set in *status (device int, may be NULL) and the kernel
 * returns.  The flag words must be used by nothing else (they count barriers since they were zeroed). */
int htr_peer_barrier(unsigned* const* peer_word, const unsigned* flags, unsigned* epoch, int nranks, int* status, htr_stream_t stream);
/* Combine step of an expert-parallel mixture-of-experts layer without a collective: part[t, :] = sum_j gates[t, j] *
 * dn[t * top_k + j, :] (float32) is stored into every peer's buffer at float offset slot_offset (+ t * hidden), with the same
 * delivery signal as above when peer_flag is given (done_counter: a zeroed device int of this rank); htr_rank_sum then adds the
 * ranks' parts in rank order (every rank obtains the same bits) and casts to the output type. */
int htr_moe_combine_peers(const void* dn, int dtype, const float* gates, int tokens, int top_k, int hidden, float* const* peer_out,
                          int npeer, int64_t slot_offset, unsigned* const* peer_flag /* may be NULL */, int* done_counter,
                          htr_stream_t stream);
/* Closing step of a mixture-of-experts layer: out[t, :] = sum_j gates[t, j] * dn[t * top_k + j, :], float32 sums in slot order, rounded
 * once to `dtype` (dn and out share it).  The same call closes the layer on one GPU and, after htr_linear_routed_peers and a barrier, on several: equal bits.  (The reference leaves the combine to the serving framework.) */
int htr_moe_weighted_sum(const void* dn, int dtype, const float* gates, int tokens, int top_k, int hidden, void* out, htr_stream_t stream);
int htr_rank_sum(const float* buf, int world, int64_t rank_stride, int tokens, int hidden, void* out, int dtype, htr_stream_t stream);

/* Grouped form of htr_linear: `count` packed linears of one shape [m, n] and width K, one activation row each, in ONE launch
 * (the experts hit by the tokens of a mixture-of-experts step).  Every list is a DEVICE array of `count` device pointers
 * (x_list[i] -> n activations, y_list[i] -> m outputs, and the four wire tensors of problem i), so that a routing kernel can
 * fill them without a host round trip; the same expert may appear several times.  count * m/128 must not exceed 16384.
 * A problem whose qweight_list entry is NULL is skipped and its output left untouched (expert parallelism: the pairs routed to
 * another rank's experts).
 * (No counterpart in the reference, which ships no MoE runtime kernel: docs/ADAPTERS.md:19.) */
size_t htr_linear_grouped_workspace_bytes(int count, int m, int n, int K);
int htr_linear_grouped(const void* const* x_list, int dtype, const void* const* qweight_list, int mt, int nt, int K,
                       const void* const* scales_list, const uint8_t* const* su_list, const uint8_t* const* sv_list,
                       void* const* y_list, int count, void* workspace, size_t workspace_bytes, htr_stream_t stream);

/* htr_linear without a workspace argument, for callers that cannot allocate device memory when they need the
 * linear (stream capture in progress, allocation-free real-time loops, hosts whose allocator is not theirs to call).
 * The scratch is a fixed array of HTR_STATIC_WORKSPACE_BYTES inside the library image, held by every GPU that
 * loads the library until the process exits; sizes whose scratch exceeds it return HTR_ERR_TOO_LARGE.  The first
 * call on each device resolves the array's device address and clears its counters on `stream`: make that first
 * call before any stream capture begins.  All calls on a device share the array, so calls that overlap on the GPU
 * (different streams) race; order them on one stream.  The entry point itself calls no allocating routine.
 * This entry point has no counterpart in the reference. */
#define HTR_STATIC_WORKSPACE_BYTES (4u << 20)
int htr_linear_static(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales,
                      const uint8_t* su, const uint8_t* sv, const void* bias /* may be NULL */, void* y, htr_stream_t stream);

#define HTR_PROLOGUE_NONE 0
#define HTR_PROLOGUE_RMSNORM 1
#define HTR_PROLOGUE_SWIGLU 2

/* Routed form of the grouped launch: problem i uses row route[i] of four DEVICE tables of device pointers (table_rows rows, one
 * per expert; a NULL qweight entry, or a route entry outside [0, table_rows), skips the problem and leaves its output row
 * untouched), reads activation row i / x_div of the matrix at x (rows x_row_stride elements apart)
 * and writes row i of y[count][m].  With x_div = top-k and route = the router's expert ids this is the gate_up launch of a
 * mixture-of-experts step with no pointer arithmetic on the host or in framework kernels; the down launch uses x_div = 1 and
 * prologue = HTR_PROLOGUE_SWIGLU, in which x holds [gate | up] rows of 2n bf16 values and the linear sees
 * silu(gate) * up.  Workspace as for htr_linear_grouped. */
int htr_linear_routed(const void* x, int dtype, int x_div, int64_t x_row_stride, const int64_t* route, int count, int table_rows,
                      const void* const* qweight_table, const void* const* scales_table, const uint8_t* const* su_table,
                      const uint8_t* const* sv_table, int mt, int nt, int K, void* y, int prologue, void* workspace,
                      size_t workspace_bytes, htr_stream_t stream);

/* htr_linear_routed for expert parallelism on one NVLink box.
 * share: this rank holds the weights of about one problem in `share` (the number of ranks the experts are dealt to); the launch is
 * planned with that many times more thread blocks than the GPU holds, because those of the other ranks' problems leave at once.
 * npeer > 0: the output row of every problem this rank owns (non-NULL weight entry) is stored, with plain peer stores, into the
 * matrix of each peer at the byte offset it has in y (peer_y[i]: the peers' [count][m] matrices as mapped into this process, this
 * rank's own among them; y itself is then only the base the offsets are taken from and is not written).  After the ranks have
 * ordered themselves (a barrier across them) every rank holds the rows of all problems, each computed by the rank that owns its
 * expert, and combines them exactly as a single GPU would.  npeer == 0: rows go to y as in htr_linear_routed.
 * (No counterpart in the reference.) */
int htr_linear_routed_peers(const void* x, int dtype, int x_div, int64_t x_row_stride, const int64_t* route, int count, int table_rows,
                            const void* const* qweight_table, const void* const* scales_table, const uint8_t* const* su_table,
                            const uint8_t* const* sv_table, int mt, int nt, int K, void* y, void* const* peer_y, int npeer, int share,
                            int prologue, void* workspace, size_t workspace_bytes, htr_stream_t stream);

/* Padded form (the reference's HTRHCLinearMethod.apply, htr/vllm_plugin.py:313-326: F.pad of the input to n_pad, slice of
 * the output to m_out, both as separate copies there): the stored tensors cover a padded [m = 16*mt, n = 16*nt] matrix, x has
 * only n_in <= n columns per row (row stride n_in; the missing columns count as zeros) and y receives only the first
 * m_out <= m rows (row stride m_out; bias, if given, has m_out elements).  n_in and m_out are multiples of 8.  Same kernel,
 * workspace and limits as htr_linear (M <= HTR_GEMV_MAX_ROWS). */
int htr_linear_padded(const void* x, int dtype, int M, int n_in, const void* qweight, int mt, int nt, int K, const void* scales,
                      const uint8_t* su, const uint8_t* sv, const void* bias, void* y, int m_out, void* workspace,
                      size_t workspace_bytes, htr_stream_t stream);

/* Decoder fusions of the GEMV (bf16 activations, M <= HTR_GEMV_MAX_ROWS, no bias; no counterpart in the reference, whose serving
 * stack runs these element-wise steps as separate kernels around HTRLinearMethod.apply, htr/vllm_plugin.py:130-138):
 *   prologue HTR_PROLOGUE_RMSNORM : the linear's input is rmsnorm(x) * norm_weight (row-wise over the n columns, eps), x[M][n]
 *   prologue HTR_PROLOGUE_SWIGLU  : x holds [gate | up] rows of 2n values; the linear's input is silu(gate) * up
 *   residual 1                    : y[M][m] is the residual stream, y <- y + result (in place) instead of y <- result
 * Intermediate values are rounded to bf16 exactly where the unfused bf16 operators round them. */
int htr_linear_fused(const void* x, int M, const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su,
                     const uint8_t* sv, void* y, void* workspace, size_t workspace_bytes, htr_stream_t stream, int prologue,
                     const void* norm_weight, float eps, int residual);

/* Tensor-core form of the packed linear for prefill-sized batches, 1 <= M <= HTR_GEMM_MAX_ROWS rows per call:
 * decoded tiles go straight into the shared-memory operand of tcgen05.mma, accumulators live in TMEM; two launches
 * (activation transform to fp16 hi/lo planes, then the GEMM with the same split reduction and epilogue as the GEMV).
 * The workspace starts with the same zero-initialised counter region as htr_linear's, followed by one status word at
 * htr_linear_gemm_error_offset(): non-zero after a call means a bounded device-side wait expired; the rows of the
 * affected 128-row blocks are then written as NaN.  Stands in for the prefill branch of _linear_impl, dequant_w + F.linear (htr/ops.py:89-93). */
#define HTR_GEMM_MAX_ROWS 256
#define HTR_GEMM_MAX_ROWS_F32 128 /* float32 activations travel as two fp16 planes: half as many rows per call */
size_t htr_linear_gemm_workspace_bytes(int M, int m, int n, int K);
size_t htr_linear_gemm_error_offset(void);
int htr_linear_gemm_last_cuda_error(void);
int htr_linear_gemm(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales,
                    const uint8_t* su, const uint8_t* sv, const void* bias /* may be NULL */, void* y, void* workspace,
                    size_t workspace_bytes, htr_stream_t stream);

/* Row-shard form of htr_linear_gemm (one launch: batches that htr_linear_gemm would split into two are refused with
 * HTR_ERR_TOO_LARGE): the epilogue stores row j, rows [0, m) of this shard, at element offset peer_offset + j * m of every buffer in
 * peer_y (the gather buffers of all ranks of an NVLink box as mapped into this process, plain peer stores) instead of y; the caller
 * then orders the ranks (htr_peer_barrier).  (No counterpart in the reference, which asserts one GPU: htr/vllm_plugin.py:91.) */
int htr_linear_gemm_peers(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales,
                          const uint8_t* su, const uint8_t* sv, const void* bias /* may be NULL */, void* const* peer_y, int npeer,
                          int64_t peer_offset, void* workspace, size_t workspace_bytes, htr_stream_t stream);

/* Original-basis weight W = Sv Ho Q Hi Su as bf16 / f16 / f32 [m, n] (debug and prefill hook).
 * Stands in for dequant_w (htr_kernels.cpp:13, k_dequant_w* htr_kernels.cu:658-903); compared with
 * wire.dequant (htr/wire.py:105-113). */
int htr_dequant_w(const void* qweight, int mt, int nt, int K, const void* scales, const uint8_t* su, const uint8_t* sv,
                  void* W, int out_dtype, htr_stream_t stream);

/* Glue kernels of the decoder harness (bf16 tensors, float32 arithmetic), all asynchronous on `stream`.  They stand in for
 * the framework ops a serving stack runs between the packed linears of a decode step (the model code around
 * HTRLinearMethod.apply, htr/vllm_plugin.py:130-138); the reference ships none of its own.
 *   add_rmsnorm : resid[rows,h] += delta (delta may be NULL); out = rmsnorm(resid, eps) * weight
 *   rope_cache  : rotary embedding (interleaved pairs) of the q and k parts of qkv[rows, (q_heads+2*kv_heads)*head_dim];
 *                 q -> q_out[rows,q_heads,head_dim]; k, v -> cache rows pos[row] of k_cache/v_cache[capacity,kv_heads,head_dim]
 *   attention   : out[row,head,:] = softmax(q . K[0..pos[row]] / sqrt(head_dim)) V, grouped-query, head_dim == 128,
 *                 pos[row] < min(capacity, HTR_DEC_MAX_LEN)
 *   swiglu      : out[rows,I] = silu(gate_up[:, :I]) * gate_up[:, I:]
 * `capacity` is the number of rows of the two caches.  The positions live in device memory, so the kernels check them: a row
 * whose position is negative or not below the limit touches no cache row, gets zeros as its attention output, and ORs a bit into
 * *status (device int, may be NULL; 1 = rope_cache, 2 = attention, 4 = rope_attention).  Nothing traps. */
#define HTR_DEC_MAX_LEN 1024
int htr_dec_add_rmsnorm(void* resid, const void* delta, const void* weight, void* out, int rows, int h, float eps, htr_stream_t stream);
int htr_dec_rope_cache(const void* qkv, const int64_t* pos, const float* cosv, const float* sinv, void* q_out, void* k_cache,
                       void* v_cache, int rows, int q_heads, int kv_heads, int head_dim, int capacity, int* status, htr_stream_t stream);
int htr_dec_attention(const void* q, const void* k_cache, const void* v_cache, const int64_t* pos, void* out, int rows, int q_heads,
                      int kv_heads, int head_dim, int capacity, int* status, htr_stream_t stream);
int htr_dec_swiglu(const void* gate_up, void* out, int rows, int intermediate, htr_stream_t stream);
/* rope_cache + attention of a single-token step (one row) in one launch: the same values, the new key/value rows written once */
int htr_dec_rope_attention(const void* qkv, const int64_t* pos, const float* cosv, const float* sinv, void* k_cache, void* v_cache,
                           void* out, int q_heads, int kv_heads, int head_dim, int capacity, int* status, htr_stream_t stream);

/* Encoder-side search: tail-biting Viterbi over the bit-shift trellis, one tile per row of x[B][T] with weights w[B][T]
 * (float32, T <= 256; the encoder uses T = 256).  Replaces htr/reference.py:7-50 (viterbi) and the CUDA module of
 * htr/vit_v2.py:28-73 (built there for sm_86 / sm_120 only), the callable behind the reference's encode.VITERBI hook
 * (htr/encode.py:7,48): minimises sum_t w[t] * (x[t] - cb[s_t])^2, cb[s] = float32(v(s) / rms), over state sequences
 * s_t = ((s_{t-1} << K) & 0xFFFF) | bits; with tailbite != 0 the sequence closes into a circle.  states[B][T] receives the
 * 16-bit states (as int32), total[B] (may be NULL) the cost of the winning final state.  The workspace holds back-pointers:
 * htr_viterbi_workspace_bytes(B, T, K) bytes (0 = unsupported arguments).
 * htr_codebook_f32 writes cb[0..65535] as the search computes it (test hook). */
size_t htr_viterbi_workspace_bytes(int B, int T, int K);
int htr_viterbi(const float* x, const float* w, int B, int T, int K, int tailbite, int32_t* states, float* total, void* workspace,
                size_t workspace_bytes, htr_stream_t stream);
int htr_viterbi_last_cuda_error(void);
int htr_codebook_f32(float* out, htr_stream_t stream);

/* Which kernel serves htr_linear and its variants for up to four activation rows: 0 = the CUDA-core GEMV, 1 = the warp-MMA GEMV
 * (hash words as int8 mma.sync fragments; one or two rows of any type, three or four bf16 rows), 2 = the tensor-memory GEMV
 * (hash words as the A operand of tcgen05.mma.kind::i8 in tensor memory; up to four rows of any type, plain activations, rows of
 * at most 16384 columns; integer-exact sums always), -1 = the default: environment variable HTR_GEMV_KERNEL if set, else the
 * measured policy.  A kind that does not serve a call falls back to the default policy for that call.  Grouped launches and five
 * to eight rows always run on the CUDA-core GEMV.  (Measurement and test knob; no counterpart in the reference.) */
void htr_set_gemv_kernel(int kind);
/* Byte offset, inside the workspace of htr_linear and its variants, of a 32-bit word that the tensor-memory GEMV sets to 1 when
 * one of its bounded waits ran out (the rows of y that the thread block still owed are then written as NaN).  Zero in a healthy run;
 * the caller clears it. */
size_t htr_linear_fault_offset(void);
/* Grid size and scratch slots the next htr_linear call with these sizes would use (for tests and benches). */
int htr_linear_plan(int M, int m, int n, int K, int* grid, int* slots_per_block);

#ifdef __cplusplus
}
#endif
#endif /* HTR_B200_H_ */
