// Instantiates the warp-MMA packed GEMV for one stream width; included by packed_gemv_mma_k<K>.cu with HTR_INST_K set.
#include "packed_gemv_mma.cuh"

namespace htr {

template <int K, int NS>
static int allow_mma_smem() {
  static bool done[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < 64 && done[dev]) return 0;
  e = cudaFuncSetAttribute(packed_gemv_mma_kernel<K, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, gemv_mma_smem_bytes<K, NS>());
  if (e != cudaSuccess) return (int)e;
  e = cudaFuncSetAttribute(packed_gemv_mma_kernel<K, NS>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < 64) done[dev] = true;
  return 0;
}

template <int K, int NS>
static int launch_mma_one(const GemvParams& p, int grid, cudaStream_t stream) {
  if (const int e = allow_mma_smem<K, NS>()) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kGemvThreads);
  cfg.dynamicSmemBytes = gemv_mma_smem_bytes<K, NS>();
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gemv_overlap_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, packed_gemv_mma_kernel<K, NS>, p);
}

template <int K, int NS>
static int occupancy_mma_one() {
  int ctas = 0;
  if (allow_mma_smem<K, NS>()) return -1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas, packed_gemv_mma_kernel<K, NS>, kGemvThreads, gemv_mma_smem_bytes<K, NS>()) != cudaSuccess)
    return -1;
  return ctas;
}

// one MMA set serves two rows with four planes each, or four rows of 16-bit activations with two planes each
template <>
int launch_packed_gemv_mma<HTR_INST_K>(const GemvParams& p, int grid, cudaStream_t stream) {
  return mma_one_set(p.rows, p.dtype) ? launch_mma_one<HTR_INST_K, 1>(p, grid, stream) : launch_mma_one<HTR_INST_K, 2>(p, grid, stream);
}

template <>
int packed_gemv_mma_ctas_per_sm<HTR_INST_K>(int rows, int dtype) {
  return mma_one_set(rows, dtype) ? occupancy_mma_one<HTR_INST_K, 1>() : occupancy_mma_one<HTR_INST_K, 2>();
}

}  // namespace htr
