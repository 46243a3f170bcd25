// Instantiates the warp-MMA packed GEMV for one stream width; included by packed_gemv_mma_k<K>.cu with HTR_INST_K set.
#include "packed_gemv_mma.cuh"

namespace htr {

template <int K, int NB>
static int allow_mma_smem() {
  static bool done[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < 64 && done[dev]) return 0;
  int optin = 0;
  e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (e != cudaSuccess) return (int)e;
  e = cudaFuncSetAttribute(packed_gemv_mma_kernel<K, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, optin - 4096);
  if (e != cudaSuccess) return (int)e;
  e = cudaFuncSetAttribute(packed_gemv_mma_kernel<K, NB>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < 64) done[dev] = true;
  return 0;
}

template <int K, int NB>
static int launch_mma_one(const GemvParams& p, int grid, cudaStream_t stream) {
  if (const int e = allow_mma_smem<K, NB>()) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = p.split > 0 ? dim3(p.split, grid / p.split) : dim3(grid);   // split form: (parts of a row block, row blocks)
  cfg.blockDim = dim3(kGemvThreads);
  cfg.dynamicSmemBytes = mma_ring_bytes<K>() + mma_window_bytes(NB, p.wblocks);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gemv_overlap_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, packed_gemv_mma_kernel<K, NB>, p);
}

constexpr int kMmaTargetCtas = 3;                       // CTAs per SM the launches are planned for (registers allow three)

template <int K, int NB>
static int config_mma_one(int rows, int* ctas_per_sm, int* window_cap) {
  if (const int e = allow_mma_smem<K, NB>()) return e;
  int dev = 0, per_sm_bytes = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  e = cudaDeviceGetAttribute(&per_sm_bytes, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
  if (e != cudaSuccess) return (int)e;
  cudaFuncAttributes fa;
  e = cudaFuncGetAttributes(&fa, packed_gemv_mma_kernel<K, NB>);
  if (e != cudaSuccess) return (int)e;
  const int row_cap = kMmaItems / (rows < 1 ? 1 : rows);
  for (int target = kMmaTargetCtas; target >= 1; --target) {
    // every resident CTA costs its static and dynamic shared memory plus 1 KB that the system reserves
    const int budget = per_sm_bytes / target - 1024 - (int)fa.sharedSizeBytes - mma_ring_bytes<K>();
    int cap = budget / (NB * 512);
    if (cap > row_cap) cap = row_cap;
    if (cap < 2 && target > 1) continue;
    if (cap < 1) return (int)cudaErrorLaunchOutOfResources;
    int ctas = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas, packed_gemv_mma_kernel<K, NB>, kGemvThreads,
                                                      mma_ring_bytes<K>() + mma_window_bytes(NB, cap));
    if (e != cudaSuccess) return (int)e;
    if (ctas < 1) continue;
    *ctas_per_sm = ctas < target ? ctas : target;
    *window_cap = cap;
    return 0;
  }
  return (int)cudaErrorLaunchOutOfResources;
}

template <>
int launch_packed_gemv_mma<HTR_INST_K>(const GemvParams& p, int grid, cudaStream_t stream) {
  return mma_b_columns(p.rows) == 4 ? launch_mma_one<HTR_INST_K, 4>(p, grid, stream) : launch_mma_one<HTR_INST_K, 8>(p, grid, stream);
}

template <>
int packed_gemv_mma_config<HTR_INST_K>(int rows, int* ctas_per_sm, int* window_cap) {
  return mma_b_columns(rows) == 4 ? config_mma_one<HTR_INST_K, 4>(rows, ctas_per_sm, window_cap)
                                  : config_mma_one<HTR_INST_K, 8>(rows, ctas_per_sm, window_cap);
}

}  // namespace htr

