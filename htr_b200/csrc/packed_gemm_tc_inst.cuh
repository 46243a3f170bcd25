// Instantiates the tensor-core packed GEMM for one stream width; included by packed_gemm_tc_k<K>.cu with HTR_INST_K set.
#include "packed_gemm_tc.cuh"

namespace htr {

template <>
int launch_packed_gemm_tc<HTR_INST_K>(const GemmParams& p, int grid, cudaStream_t st) {
  const int smem = gemm_smem_bytes(p.np, p.planes, HTR_INST_K, p.stages);
  cudaError_t e = cudaFuncSetAttribute(packed_gemm_tc_kernel<HTR_INST_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);   // the 227 KB limit includes the static part
  if (e != cudaSuccess) return (int)e;
  // programmatic stream serialisation: the kernel may start while the activation transform before it still runs; it
  // fetches packed words at once and waits (griddepcontrol.wait) before it touches anything that kernel writes
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, packed_gemm_tc_kernel<HTR_INST_K>, p);
}

}  // namespace htr

#ifdef HTR_GEMM_TRACE
#if HTR_INST_K == 4
extern "C" int htr_gemm_trace_read(unsigned long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, htr::htr_gemm_trace_buf, sizeof(unsigned long long) * n);
}
extern "C" int htr_gemm_trace_clear() {
  static unsigned long long zeros[512 * 128];
  return (int)cudaMemcpyToSymbol(htr::htr_gemm_trace_buf, zeros, sizeof(zeros));
}
#endif
#endif
