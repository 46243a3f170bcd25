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
  // two CTAs per SM need the largest shared-memory carve-out; the default preference would size it for one
  e = cudaFuncSetAttribute(packed_gemv_tc_kernel<K>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
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

// CTAs of this kernel that one SM holds: two allocations of 256 tensor-memory columns, if the shared memory fits twice (the
// registers do: 384 threads at <= 80 registers).  Computed by hand: the occupancy query of the runtime answers 1 for every
// kernel that allocates tensor memory, whatever it allocates.
template <>
int packed_gemv_tc_ctas_per_sm<HTR_INST_K>() {
  if (allow_tc_smem<HTR_INST_K>()) return -1;
  int dev = 0, smem_sm = 0, reserved = 0;
  cudaFuncAttributes fa;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaFuncGetAttributes(&fa, packed_gemv_tc_kernel<HTR_INST_K>) != cudaSuccess ||
      cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev) != cudaSuccess)
    return -1;
  const int per_cta = gemv_tc_smem_bytes(HTR_INST_K) + (int)fa.sharedSizeBytes + reserved;
  int ctas = smem_sm / per_cta;
  if (fa.numRegs > 80) ctas = 1;
  if (ctas < 1) return -1;
  return ctas > 512 / kTcTmemCols ? 512 / kTcTmemCols : ctas;
}

template <>
int packed_gemv_tc_failures<HTR_INST_K>(int* count, unsigned* last) {
  if (const cudaError_t e = cudaMemcpyFromSymbol(count, htr_gemv_tc_failures_dev, sizeof(int))) return (int)e;
  return (int)cudaMemcpyFromSymbol(last, htr_gemv_tc_last_failure_dev, sizeof(unsigned));
}

}  // namespace htr

#ifdef HTR_GEMV_TC_TRACE
#if HTR_INST_K == 4
extern "C" int htr_tc_trace_read(unsigned long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, htr::htr_tc_trace_buf, sizeof(unsigned long long) * n);
}
extern "C" int htr_tc_trace_clear() {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, htr::htr_tc_trace_buf) != cudaSuccess) return 1;
  return (int)cudaMemset(p, 0, sizeof(htr::htr_tc_trace_buf));
}
#endif
#endif
