// Instantiates the tensor-memory packed GEMV for one stream width; included by packed_gemv_tm_k<K>.cu with HTR_INST_K set.
#include "packed_gemv_tm.cuh"

namespace htr {

template <int K>
static int allow_tm_smem() {
  static bool done[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < 64 && done[dev]) return 0;
  int optin = 0;
  e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (e != cudaSuccess) return (int)e;
  e = cudaFuncSetAttribute(packed_gemv_tm_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, optin - 8192);
  if (e != cudaSuccess) return (int)e;
  e = cudaFuncSetAttribute(packed_gemv_tm_kernel<K>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < 64) done[dev] = true;
  return 0;
}

template <>
int launch_packed_gemv_tm<HTR_INST_K>(const GemvParams& p, int grid, cudaStream_t stream) {
  if (const int e = allow_tm_smem<HTR_INST_K>()) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kTmThreads);
  cfg.dynamicSmemBytes = TmRing<HTR_INST_K>::bytes + tm_window_bytes(p.wblocks);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gemv_overlap_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, packed_gemv_tm_kernel<HTR_INST_K>, p);
}

// two thread blocks per SM (256 tensor-memory columns each): the window is what fits beside the ring then
template <>
int packed_gemv_tm_config<HTR_INST_K>(int rows, int* ctas_per_sm, int* window_cap) {
  if (const int e = allow_tm_smem<HTR_INST_K>()) return e;
  int dev = 0, per_sm_bytes = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  e = cudaDeviceGetAttribute(&per_sm_bytes, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
  if (e != cudaSuccess) return (int)e;
  cudaFuncAttributes fa;
  e = cudaFuncGetAttributes(&fa, packed_gemv_tm_kernel<HTR_INST_K>);
  if (e != cudaSuccess) return (int)e;
  const int row_cap = kTmItems / (rows < 1 ? 1 : rows);
  // every resident CTA costs its static and dynamic shared memory plus 1 KB that the system reserves
  const int budget = per_sm_bytes / 2 - 1024 - (int)fa.sharedSizeBytes - TmRing<HTR_INST_K>::bytes;
  int cap = budget / tm_window_bytes(1);
  if (cap > row_cap) cap = row_cap;
  if (cap < 1) return (int)cudaErrorLaunchOutOfResources;
  // (two thread blocks fit by the arithmetic above; tensor memory, 256 columns each, allows no more)
  const int ctas = 2;
  *ctas_per_sm = ctas < 2 ? ctas : 2;
  *window_cap = cap;
  return 0;
}

}  // namespace htr
