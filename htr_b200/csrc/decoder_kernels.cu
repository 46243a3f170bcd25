// Small fused kernels of the decoder harness (the non-linear glue between packed linears in a decode step):
// residual add + RMSNorm, rotary embedding + KV-cache write, single-query grouped-query attention, SwiGLU.
// They exist so that a decode step is a short chain of launches around the packed GEMVs instead of dozens of
// framework kernels; every one is launched with programmatic stream serialisation, signals its dependents at once and
// waits for its predecessor before touching data, so the next packed GEMV prefetches its weights while these run.
// bf16 activations, float32 arithmetic.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/htr_b200.h"

namespace {

__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float bf(const __nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = -3.0e38f;
  for (int i = 0; i < nw; ++i) t = fmaxf(t, red[i]);
  return t;
}

// resid += delta (if any); out = rmsnorm(resid) * w.  One CTA per row; the row stays in registers between the two passes
// (h <= 8192: up to 16 bf16 pairs per thread).
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__nv_bfloat16* __restrict__ resid, const __nv_bfloat16* __restrict__ delta,
                                                          const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, int h, float eps) {
  __shared__ float red[8];
  pdl_enter();
  const size_t row = (size_t)blockIdx.x * h;
  constexpr int kMaxPairs = 16;
  float2 v[kMaxPairs];
  float2 g[kMaxPairs];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxPairs; ++j) {
    const int i = (threadIdx.x + j * 256) * 2;
    v[j] = make_float2(0.f, 0.f);
    g[j] = make_float2(0.f, 0.f);
    if (i < h) {
      v[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(resid + row + i));
      g[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + i));
      if (delta) {
        const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(delta + row + i));
        const __nv_bfloat162 r = __floats2bfloat162_rn(v[j].x + d.x, v[j].y + d.y);
        *reinterpret_cast<__nv_bfloat162*>(resid + row + i) = r;
        v[j] = __bfloat1622float2(r);                   // the norm sees the stored (rounded) residual, as a framework would
      }
      ss += v[j].x * v[j].x + v[j].y * v[j].y;
    }
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)h + eps);
#pragma unroll
  for (int j = 0; j < kMaxPairs; ++j) {
    const int i = (threadIdx.x + j * 256) * 2;
    if (i < h) {
      // normalise, round to bf16, then scale: the order of the unfused reference ops
      const float2 nf = __bfloat1622float2(__floats2bfloat162_rn(v[j].x * inv, v[j].y * inv));
      *reinterpret_cast<__nv_bfloat162*>(out + row + i) = __floats2bfloat162_rn(nf.x * g[j].x, nf.y * g[j].y);
    }
  }
}

// rotary embedding of q and k (interleaved pairs), k and v written into the cache rows pos[t].  grid (heads_q + 2*heads_kv, T), D/2 threads.
__global__ void rope_cache_kernel(const __nv_bfloat16* __restrict__ qkv, const long long* __restrict__ pos, const float* __restrict__ cosv,
                                  const float* __restrict__ sinv, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                                  __nv_bfloat16* __restrict__ v_cache, int hq, int hkv, int D, int capacity, int* __restrict__ status) {
  pdl_enter();
  const int head = blockIdx.x, t = blockIdx.y, i = threadIdx.x;           // pair index i: elements 2i, 2i+1
  const long long p = pos[t];
  if (p < 0 || p >= capacity) {                                           // a position outside the cache: nothing is read or written
    if (status && i == 0 && head == 0) atomicOr(status, 1);
    return;
  }
  const size_t row = (size_t)t * (hq + 2 * hkv) * D;
  const __nv_bfloat162 in = *reinterpret_cast<const __nv_bfloat162*>(qkv + row + (size_t)head * D + 2 * i);
  if (head >= hq + hkv) {                                                 // v: plain copy into the cache
    *reinterpret_cast<__nv_bfloat162*>(v_cache + ((size_t)p * hkv + (head - hq - hkv)) * D + 2 * i) = in;
    return;
  }
  const float2 v = __bfloat1622float2(in);
  const float c = cosv[(size_t)p * (D / 2) + i], s = sinv[(size_t)p * (D / 2) + i];
  const __nv_bfloat162 r = __floats2bfloat162_rn(v.x * c - v.y * s, v.x * s + v.y * c);
  if (head < hq) *reinterpret_cast<__nv_bfloat162*>(q_out + ((size_t)t * hq + head) * D + 2 * i) = r;
  else *reinterpret_cast<__nv_bfloat162*>(k_cache + ((size_t)p * hkv + (head - hq)) * D + 2 * i) = r;
}

// out[t, head, :] = softmax(q . K[0..pos[t]] / sqrt(D)) V.  grid (heads_q, T), 128 threads, D == 128, positions < min(capacity,
// HTR_DEC_MAX_LEN); a row whose position lies outside gets zeros and sets the status word.
// Scores: one thread per position (128 positions per pass, the 256-byte key row read as sixteen 16-byte loads);
// values: one thread per dimension, eight positions in flight.
__global__ void __launch_bounds__(128) attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                                                        const __nv_bfloat16* __restrict__ v_cache, const long long* __restrict__ pos,
                                                        __nv_bfloat16* __restrict__ out, int hq, int hkv, int capacity, int* __restrict__ status) {
  constexpr int D = 128;
  __shared__ __align__(16) float sq[D];
  __shared__ float sc[HTR_DEC_MAX_LEN];
  __shared__ float red[4];
  pdl_enter();
  const int head = blockIdx.x, t = blockIdx.y, tid = threadIdx.x;
  const int kvh = head / (hq / hkv);
  const long long pt = pos[t];
  if (pt < 0 || pt >= capacity || pt >= HTR_DEC_MAX_LEN) {                // the whole CTA takes this branch: no barrier is skipped by a part of it
    if (status && tid == 0 && head == 0) atomicOr(status, 2);
    out[((size_t)t * hq + head) * D + tid] = __float2bfloat16_rn(0.f);
    return;
  }
  const int len = (int)pt + 1;
  sq[tid] = bf(q[((size_t)t * hq + head) * D + tid]) * 0.08838834764831845f;   // 1/sqrt(128)
  __syncthreads();
  float mx = -3.0e38f;
  for (int p = tid; p < len; p += 128) {
    const uint4* kr = reinterpret_cast<const uint4*>(k_cache + ((size_t)p * hkv + kvh) * D);
    float d = 0.f;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      const uint4 raw = __ldg(kr + c);
      const float4 q0 = *reinterpret_cast<const float4*>(sq + 8 * c), q1 = *reinterpret_cast<const float4*>(sq + 8 * c + 4);
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      const float2 e = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.z)), f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.w));
      d += a.x * q0.x + a.y * q0.y + b.x * q0.z + b.y * q0.w + e.x * q1.x + e.y * q1.y + f.x * q1.z + f.y * q1.w;
    }
    sc[p] = d;
    mx = fmaxf(mx, d);
  }
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int p = tid; p < len; p += 128) {
    const float e = __expf(sc[p] - mx);
    sc[p] = e;
    sum += e;
  }
  sum = block_sum(sum, red);
  const __nv_bfloat16* vcol = v_cache + (size_t)kvh * D + tid;
  float acc = 0.f;
  int p = 0;
  for (; p + 8 <= len; p += 8) {
    float vv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) vv[j] = bf(vcol[(size_t)(p + j) * hkv * D]);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += sc[p + j] * vv[j];
  }
  for (; p < len; ++p) acc += sc[p] * bf(vcol[(size_t)p * hkv * D]);
  out[((size_t)t * hq + head) * D + tid] = __float2bfloat16_rn(acc / sum);
}

// Single-token step: rotary embedding, cache write and attention of one query head in one kernel.  grid (heads_q), 128 threads,
// D == 128.  The CTA rotates its query and its group's new key itself (the four query heads of a group repeat that small piece
// of work), takes the scores and values of the new position from shared memory and those of older positions from the cache;
// the first head of each group writes the new key and value rows.  Same roundings as rope_cache_kernel + attention_kernel; the
// weighted sum of the value rows runs over four interleaved position streams (one per warp), so it differs from theirs in the last
// float32 bits.
__global__ void __launch_bounds__(128) rope_attention_kernel(const __nv_bfloat16* __restrict__ qkv, const long long* __restrict__ pos,
                                                             const float* __restrict__ cosv, const float* __restrict__ sinv,
                                                             __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                                             __nv_bfloat16* __restrict__ out, int hq, int hkv, int capacity,
                                                             int* __restrict__ status) {
  constexpr int D = 128;
  __shared__ __align__(16) float sq[D];
  __shared__ float sk[D], sv[D];
  __shared__ float sc[HTR_DEC_MAX_LEN];
  __shared__ float red[4];
  pdl_enter();
  const int head = blockIdx.x, tid = threadIdx.x;
  const int rep = hq / hkv, kvh = head / rep;
  const long long p0 = pos[0];
  if (p0 < 0 || p0 >= capacity || p0 >= HTR_DEC_MAX_LEN) {                // outside the cache: no cache row is touched, zeros come out
    if (status && tid == 0 && head == 0) atomicOr(status, 4);
    out[(size_t)head * D + tid] = __float2bfloat16_rn(0.f);
    return;
  }
  const int p = (int)p0, len = p + 1;
  {
    const int i = tid >> 1;                                               // pair (2i, 2i+1); even threads own the first element
    const float c = cosv[(size_t)p * (D / 2) + i], s = sinv[(size_t)p * (D / 2) + i];
    const float2 qv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(qkv + (size_t)head * D + 2 * i));
    const float2 kv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(qkv + (size_t)(hq + kvh) * D + 2 * i));
    const __nv_bfloat16 qr = __float2bfloat16_rn((tid & 1) ? qv.x * s + qv.y * c : qv.x * c - qv.y * s);
    const __nv_bfloat16 kr = __float2bfloat16_rn((tid & 1) ? kv.x * s + kv.y * c : kv.x * c - kv.y * s);
    const __nv_bfloat16 vn = qkv[(size_t)(hq + hkv + kvh) * D + tid];
    sq[tid] = bf(qr) * 0.08838834764831845f;                              // 1/sqrt(128)
    sk[tid] = bf(kr);
    sv[tid] = bf(vn);
    if (head == kvh * rep) {
      k_cache[((size_t)p * hkv + kvh) * D + tid] = kr;
      v_cache[((size_t)p * hkv + kvh) * D + tid] = vn;
    }
  }
  __syncthreads();
  const int lane = tid & 31, warp = tid >> 5;
  float mx = -3.0e38f;
  // scores of the cached positions: one thread per position (the 256-byte key row as sixteen 16-byte loads in flight)
  for (int t = tid; t < p; t += 128) {
    const uint4* kr = reinterpret_cast<const uint4*>(k_cache + ((size_t)t * hkv + kvh) * D);
    float d = 0.f;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      const uint4 raw = __ldg(kr + c);
      const float4 q0 = *reinterpret_cast<const float4*>(sq + 8 * c), q1 = *reinterpret_cast<const float4*>(sq + 8 * c + 4);
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      const float2 e = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.z)), f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.w));
      d += a.x * q0.x + a.y * q0.y + b.x * q0.z + b.y * q0.w + e.x * q1.x + e.y * q1.y + f.x * q1.z + f.y * q1.w;
    }
    sc[t] = d;
    mx = fmaxf(mx, d);
  }
  // score of the new position from shared memory: warp 0, four dimensions per lane
  if (warp == 0) {
    float d = sk[4 * lane] * sq[4 * lane] + sk[4 * lane + 1] * sq[4 * lane + 1] + sk[4 * lane + 2] * sq[4 * lane + 2] + sk[4 * lane + 3] * sq[4 * lane + 3];
#pragma unroll
    for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, o);
    if (lane == 0) sc[p] = d;
    mx = fmaxf(mx, d);
  }
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int t = tid; t < len; t += 128) {
    const float e = __expf(sc[t] - mx);
    sc[t] = e;
    sum += e;
  }
  sum = block_sum(sum, red);
  // values: warp w takes the cached positions w, w + 4, ..., a lane four dimensions of a row (one 8-byte load; a row is one
  // coalesced 256-byte read of the warp), eight rows in flight per warp; the four partial sums meet in shared memory
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  {
    const __nv_bfloat16* vrow = v_cache + (size_t)kvh * D + 4 * lane;
    const size_t stride = (size_t)hkv * D;
    int t = warp;
    for (; t + 28 < p; t += 32) {
      uint2 raw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) raw[j] = __ldg(reinterpret_cast<const uint2*>(vrow + (size_t)(t + 4 * j) * stride));
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float w = sc[t + 4 * j];
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[j].x)), hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[j].y));
        a0 += w * lo.x; a1 += w * lo.y; a2 += w * hi.x; a3 += w * hi.y;
      }
    }
    for (; t < p; t += 4) {
      const uint2 raw = __ldg(reinterpret_cast<const uint2*>(vrow + (size_t)t * stride));
      const float w = sc[t];
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x)), hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      a0 += w * lo.x; a1 += w * lo.y; a2 += w * hi.x; a3 += w * hi.y;
    }
  }
  __shared__ __align__(16) float part[4][D];
  *reinterpret_cast<float4*>(&part[warp][4 * lane]) = make_float4(a0, a1, a2, a3);
  __syncthreads();
  const float acc = part[0][tid] + part[1][tid] + part[2][tid] + part[3][tid] + sc[p] * sv[tid];
  out[(size_t)head * D + tid] = __float2bfloat16_rn(acc / sum);
}

// out = silu(gate) * up, gu = [T, 2I] with the gate half first
__global__ void __launch_bounds__(256) swiglu_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I, int total) {
  pdl_enter();
  const int idx = (blockIdx.x * 256 + threadIdx.x) * 2;
  if (idx >= total) return;
  const int t = idx / I, j = idx - t * I;
  const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + (size_t)t * 2 * I + j));
  const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + (size_t)t * 2 * I + I + j));
  // silu rounded to bf16 before the product, as the unfused ops do
  const __nv_bfloat162 s = __floats2bfloat162_rn(g.x / (1.f + __expf(-g.x)), g.y / (1.f + __expf(-g.y)));
  const float2 sf = __bfloat1622float2(s);
  *reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * I + j) = __floats2bfloat162_rn(sf.x * u.x, sf.y * u.y);
}

template <typename Kern, typename... Args>
int launch_pdl(Kern kern, dim3 grid, dim3 block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, args...);
}

}  // namespace

extern "C" {

int htr_dec_add_rmsnorm(void* resid, const void* delta, const void* weight, void* out, int rows, int h, float eps, htr_stream_t stream) {
  if (rows <= 0) return HTR_OK;
  if (!resid || !weight || !out) return HTR_ERR_NULL;
  if (h <= 0 || h % 2 || h > 8192) return HTR_ERR_BAD_SHAPE;
  const int e = launch_pdl(add_rmsnorm_kernel, dim3(rows), dim3(256), static_cast<cudaStream_t>(stream), static_cast<__nv_bfloat16*>(resid),
                           static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(out), h, eps);
  return e ? HTR_ERR_CUDA : HTR_OK;
}

int htr_dec_rope_cache(const void* qkv, const int64_t* pos, const float* cosv, const float* sinv, void* q_out, void* k_cache, void* v_cache,
                       int rows, int q_heads, int kv_heads, int head_dim, int capacity, int* status, htr_stream_t stream) {
  if (rows <= 0) return HTR_OK;
  if (!qkv || !pos || !cosv || !sinv || !q_out || !k_cache || !v_cache) return HTR_ERR_NULL;
  if (head_dim <= 0 || head_dim % 2 || head_dim > 2048 || q_heads <= 0 || kv_heads <= 0 || capacity <= 0) return HTR_ERR_BAD_SHAPE;
  const int e = launch_pdl(rope_cache_kernel, dim3(q_heads + 2 * kv_heads, rows), dim3(head_dim / 2), static_cast<cudaStream_t>(stream),
                           static_cast<const __nv_bfloat16*>(qkv), reinterpret_cast<const long long*>(pos), cosv, sinv,
                           static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), q_heads,
                           kv_heads, head_dim, capacity, status);
  return e ? HTR_ERR_CUDA : HTR_OK;
}

int htr_dec_attention(const void* q, const void* k_cache, const void* v_cache, const int64_t* pos, void* out, int rows, int q_heads,
                      int kv_heads, int head_dim, int capacity, int* status, htr_stream_t stream) {
  if (rows <= 0) return HTR_OK;
  if (!q || !k_cache || !v_cache || !pos || !out) return HTR_ERR_NULL;
  if (head_dim != 128 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || capacity <= 0) return HTR_ERR_BAD_SHAPE;
  const int e = launch_pdl(attention_kernel, dim3(q_heads, rows), dim3(128), static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(q),
                           static_cast<const __nv_bfloat16*>(k_cache), static_cast<const __nv_bfloat16*>(v_cache),
                           reinterpret_cast<const long long*>(pos), static_cast<__nv_bfloat16*>(out), q_heads, kv_heads, capacity, status);
  return e ? HTR_ERR_CUDA : HTR_OK;
}

int htr_dec_rope_attention(const void* qkv, const int64_t* pos, const float* cosv, const float* sinv, void* k_cache, void* v_cache, void* out,
                           int q_heads, int kv_heads, int head_dim, int capacity, int* status, htr_stream_t stream) {
  if (!qkv || !pos || !cosv || !sinv || !k_cache || !v_cache || !out) return HTR_ERR_NULL;
  if (head_dim != 128 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || capacity <= 0) return HTR_ERR_BAD_SHAPE;
  const int e = launch_pdl(rope_attention_kernel, dim3(q_heads), dim3(128), static_cast<cudaStream_t>(stream),
                           static_cast<const __nv_bfloat16*>(qkv), reinterpret_cast<const long long*>(pos), cosv, sinv,
                           static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), static_cast<__nv_bfloat16*>(out), q_heads,
                           kv_heads, capacity, status);
  return e ? HTR_ERR_CUDA : HTR_OK;
}

int htr_dec_swiglu(const void* gate_up, void* out, int rows, int intermediate, htr_stream_t stream) {
  if (rows <= 0) return HTR_OK;
  if (!gate_up || !out) return HTR_ERR_NULL;
  if (intermediate <= 0 || intermediate % 2) return HTR_ERR_BAD_SHAPE;
  const int total = rows * intermediate;
  const int e = launch_pdl(swiglu_kernel, dim3((total / 2 + 255) / 256), dim3(256), static_cast<cudaStream_t>(stream),
                           static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), intermediate, total);
  return e ? HTR_ERR_CUDA : HTR_OK;
}

}  // extern "C"
