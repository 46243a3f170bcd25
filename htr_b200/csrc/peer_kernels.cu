// Cross-GPU hand-over for the sharded forms on one NVLink box: delivery flags instead of a barrier across the ranks.
//
// A producer kernel (the GEMV's peer form, or moe_combine_peers_kernel below) stores its share of a result into every rank's
// buffer with plain peer stores and then, once, adds 1 to the word "rank s has delivered" in every rank's flag array (system
// scope, after a system-wide fence).  The consumer runs peer_wait_kernel on its own stream before it reads its buffer: it waits
// until every flag has reached the call's sequence number, which it keeps in device memory (so a captured CUDA graph replays
// correctly).  Every wait is bounded; a wait that runs out sets bits in a status word that the host can read, and returns.
// Only plain loads, stores and atomics cross NVLink: no multicast, no multimem.
// (The reference is single-GPU, htr/vllm_plugin.py:91: no counterpart.)
#include "htr_common.cuh"

namespace {

__device__ __forceinline__ unsigned load_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// flags[r] counts the deliveries of rank r into this GPU's buffer; *epoch counts the calls this GPU has consumed
__global__ void peer_wait_kernel(const unsigned* __restrict__ flags, unsigned* __restrict__ epoch, int nranks, unsigned count,
                                 int* __restrict__ status, unsigned limit) {
  const int lane = threadIdx.x;
  const unsigned want = *epoch + count;
  bool ok = true;
  if (lane < nranks) {
    ok = false;
    for (unsigned it = 0; it < limit; ++it) {
      if ((int)(load_acquire_sys(flags + lane) - want) >= 0) {
        ok = true;
        break;
      }
      __nanosleep(it < 64 ? 32 : 256);
    }
    if (!ok && status) atomicOr(status, 1 << lane);     // rank `lane` did not deliver in time: the buffer holds stale rows
  }
  __syncwarp();
  if (lane == 0) *epoch = want;
}

// Barrier across the ranks of one NVLink box, as one small kernel per rank: lane r adds 1 to this rank's word in rank r's flag array
// (system scope, after a system-wide fence) and then waits, bounded, until rank r has done the same here.  The kernel is launched
// so that it may become resident while its predecessor still runs (programmatic stream serialisation) and begins with
// griddepcontrol.wait: what this rank stored before the barrier -- peer stores of the preceding kernel included -- is complete and
// flushed when the first signal leaves, and the launch latency is hidden behind the predecessor.
__global__ void peer_barrier_kernel(unsigned* const* __restrict__ peer_word, const unsigned* __restrict__ flags, unsigned* __restrict__ epoch,
                                    int nranks, int* __restrict__ status, unsigned limit) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int lane = threadIdx.x;
  const unsigned want = *epoch + 1u;
  if (lane < nranks) {
    __threadfence_system();
    atomicAdd_system(peer_word[lane], 1u);
    bool ok = false;
    for (unsigned it = 0; it < limit; ++it) {
      if ((int)(load_acquire_sys(flags + lane) - want) >= 0) {
        ok = true;
        break;
      }
      __nanosleep(it < 256 ? 20 : 256);
    }
    if (!ok && status) atomicOr(status, 1 << lane);     // rank `lane` did not arrive in time
  }
  __syncwarp();
  if (lane == 0) *epoch = want;
}

// part[t, :] = sum_j w[t, j] * dn[t * k + j, :] (float32), stored into every peer's buffer at [my_rank][t][:]; then the signal.
// grid (h / 1024, T), 256 threads, four columns per thread.
__global__ void __launch_bounds__(256) moe_combine_peers_kernel(const void* __restrict__ dn, int dtype, const float* __restrict__ w, int k, int h,
                                                                float* const* __restrict__ peer_out, int npeer, long long slot_offset,
                                                                unsigned* const* __restrict__ peer_flag, int* __restrict__ done) {
  const int t = blockIdx.y, col = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (col < h) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < k; ++j) {
      const float g = w[t * k + j];
      const float4 v = htr::load_quad(dn, (size_t)(t * k + j) * h + col, dtype);
      acc.x += g * v.x; acc.y += g * v.y; acc.z += g * v.z; acc.w += g * v.w;
    }
#pragma unroll 1
    for (int pe = 0; pe < npeer; ++pe) *reinterpret_cast<float4*>(peer_out[pe] + slot_offset + (size_t)t * h + col) = acc;
  }
  if (peer_flag == nullptr) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();                                   // release at GPU scope; the last block's system-wide fence carries all of it to the peers
    if (atomicAdd(done, 1) == (int)(gridDim.x * gridDim.y) - 1) {
      __threadfence_system();
      *done = 0;
#pragma unroll 1
      for (int pe = 0; pe < npeer; ++pe) atomicAdd_system(peer_flag[pe], 1u);
    }
  }
}

// out[t, :] = sum_j w[t, j] * dn[t * k + j, :], float32 sums in slot order, rounded once to the output type.  The same kernel closes the
// layer on one GPU and on several (where dn holds the rows every rank delivered), so the two give the same bits.
__global__ void __launch_bounds__(256) moe_weighted_sum_kernel(const void* __restrict__ dn, int dtype, const float* __restrict__ w, int k, int h,
                                                               void* __restrict__ out) {
  const int t = blockIdx.y, col = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (col >= h) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j = 0; j < k; ++j) {
    const float g = w[t * k + j];
    const float4 v = htr::load_quad(dn, (size_t)(t * k + j) * h + col, dtype);
    acc.x += g * v.x; acc.y += g * v.y; acc.z += g * v.z; acc.w += g * v.w;
  }
  htr::store_quad(out, (size_t)t * h + col, dtype, acc);
}

// out[t, :] = sum_r buf[r][t][:] in rank order (every rank adds identically), cast to the output type
__global__ void __launch_bounds__(256) rank_sum_kernel(const float* __restrict__ buf, int world, long long rank_stride, int h, void* __restrict__ out,
                                                       int dtype) {
  const int t = blockIdx.y, col = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (col >= h) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r = 0; r < world; ++r) {
    const float4 v = *reinterpret_cast<const float4*>(buf + r * rank_stride + (size_t)t * h + col);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  htr::store_quad(out, (size_t)t * h + col, dtype, acc);
}

}  // namespace

extern "C" {

int htr_peer_wait(const unsigned* flags, unsigned* epoch, int nranks, int count, int* status, htr_stream_t stream) {
  if (!flags || !epoch) return HTR_ERR_NULL;
  if (nranks < 1 || nranks > 32 || count < 1) return HTR_ERR_BAD_SHAPE;
  // about two seconds at the longest: 2^23 polls a quarter of a microsecond apart
  peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, epoch, nranks, (unsigned)count, status, 1u << 23);
  return cudaGetLastError() == cudaSuccess ? HTR_OK : HTR_ERR_CUDA;
}

int htr_peer_barrier(unsigned* const* peer_word, const unsigned* flags, unsigned* epoch, int nranks, int* status, htr_stream_t stream) {
  if (!peer_word || !flags || !epoch) return HTR_ERR_NULL;
  if (nranks < 1 || nranks > 32) return HTR_ERR_BAD_SHAPE;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // about two seconds at the longest
  return cudaLaunchKernelEx(&cfg, peer_barrier_kernel, peer_word, flags, epoch, nranks, status, 1u << 23) == cudaSuccess ? HTR_OK : HTR_ERR_CUDA;
}

int htr_moe_combine_peers(const void* dn, int dtype, const float* gates, int tokens, int top_k, int hidden, float* const* peer_out, int npeer,
                          int64_t slot_offset, unsigned* const* peer_flag, int* done_counter, htr_stream_t stream) {
  if (tokens <= 0) return HTR_OK;
  if (!dn || !gates || !peer_out) return HTR_ERR_NULL;
  if (dtype < HTR_DTYPE_BF16 || dtype > HTR_DTYPE_F32) return HTR_ERR_BAD_DTYPE;
  if (top_k < 1 || hidden < 4 || hidden % 4 || npeer < 1 || npeer > 8 || slot_offset < 0 || (slot_offset & 3) || tokens > 65535) return HTR_ERR_BAD_SHAPE;
  if (peer_flag && !done_counter) return HTR_ERR_NULL;
  moe_combine_peers_kernel<<<dim3((hidden + 1023) / 1024, tokens), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      dn, dtype, gates, top_k, hidden, peer_out, npeer, (long long)slot_offset, peer_flag, done_counter);
  return cudaGetLastError() == cudaSuccess ? HTR_OK : HTR_ERR_CUDA;
}

int htr_moe_weighted_sum(const void* dn, int dtype, const float* gates, int tokens, int top_k, int hidden, void* out, htr_stream_t stream) {
  if (tokens <= 0) return HTR_OK;
  if (!dn || !gates || !out) return HTR_ERR_NULL;
  if (dtype < HTR_DTYPE_BF16 || dtype > HTR_DTYPE_F32) return HTR_ERR_BAD_DTYPE;
  if (top_k < 1 || hidden < 4 || hidden % 4 || tokens > 65535) return HTR_ERR_BAD_SHAPE;
  moe_weighted_sum_kernel<<<dim3((hidden + 1023) / 1024, tokens), 256, 0, static_cast<cudaStream_t>(stream)>>>(dn, dtype, gates, top_k, hidden, out);
  return cudaGetLastError() == cudaSuccess ? HTR_OK : HTR_ERR_CUDA;
}

int htr_rank_sum(const float* buf, int world, int64_t rank_stride, int tokens, int hidden, void* out, int dtype, htr_stream_t stream) {
  if (tokens <= 0) return HTR_OK;
  if (!buf || !out) return HTR_ERR_NULL;
  if (dtype < HTR_DTYPE_BF16 || dtype > HTR_DTYPE_F32) return HTR_ERR_BAD_DTYPE;
  if (world < 1 || hidden < 4 || hidden % 4 || rank_stride < 0 || (rank_stride & 3) || tokens > 65535) return HTR_ERR_BAD_SHAPE;
  rank_sum_kernel<<<dim3((hidden + 1023) / 1024, tokens), 256, 0, static_cast<cudaStream_t>(stream)>>>(buf, world, (long long)rank_stride, hidden, out, dtype);
  return cudaGetLastError() == cudaSuccess ? HTR_OK : HTR_ERR_CUDA;
}

}  // extern "C"
