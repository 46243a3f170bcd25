// Instantiates the tensor-core packed GEMM for one stream width; included by packed_gemm_tc_k<K>.cu with HTR_INST_K set.
#include "packed_gemm_tc.cuh"

namespace htr {

template <>
int launch_packed_gemm_tc<HTR_INST_K>(const GemmParams& p, int grid, cudaStream_t st) {
  const int smem = gemm_smem_bytes(p.np, p.planes, HTR_INST_K);
  cudaError_t e = cudaFuncSetAttribute(packed_gemm_tc_kernel<HTR_INST_K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       gemm_smem_bytes(128, 1, HTR_INST_K));   // = the largest supported form (128 rows x 1 plane, 64 rows x 2 planes)
  if (e != cudaSuccess) return (int)e;
  packed_gemm_tc_kernel<HTR_INST_K><<<grid, kGemmThreads, smem, st>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace htr
