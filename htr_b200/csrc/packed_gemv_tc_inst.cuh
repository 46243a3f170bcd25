// Instantiates the tensor-core packed GEMV for one stream width; included by packed_gemv_tc_k<K>.cu with HTR_INST_K set.
#include "packed_gemv_tc.cuh"

namespace htr {

template <int K>
static int allow_tc_smem() {
  static bool done[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < 64 && done[dev]) return 0;
  e = cudaFuncSetAttribute(packed_gemv_tc_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, gemv_tc_smem_bytes(K));
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < 64) done[dev] = true;
  return 0;
}

template <>
int launch_packed_gemv_tc<HTR_INST_K>(const GemvParams& p, int grid, cudaStream_t stream) {
  if (const int e = allow_tc_smem<HTR_INST_K>()) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = gemv_tc_smem_bytes(HTR_INST_K);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gemv_overlap_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, packed_gemv_tc_kernel<HTR_INST_K>, p);
}

// CTAs of this kernel that one SM holds: bounded by the tensor memory (two allocations of 256 columns), whatever else would fit
template <>
int packed_gemv_tc_ctas_per_sm<HTR_INST_K>() {
  int ctas = 0;
  if (allow_tc_smem<HTR_INST_K>()) return -1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas, packed_gemv_tc_kernel<HTR_INST_K>, kTcThreads, gemv_tc_smem_bytes(HTR_INST_K)) != cudaSuccess)
    return -1;
  return ctas > 512 / kTcTmemCols ? 512 / kTcTmemCols : ctas;
}

template <>
int packed_gemv_tc_failures<HTR_INST_K>(int* count) {
  return (int)cudaMemcpyFromSymbol(count, htr_gemv_tc_failures_dev, sizeof(int));
}

}  // namespace htr
