// Instantiates the packed GEMV for one stream width; included by packed_gemv_k<K>.cu with HTR_INST_K set.
#include "packed_gemv.cuh"

namespace htr {

// dynamic shared memory beyond 48 KB needs an opt-in, done once per device and instantiation
template <int K, int MT>
static int allow_smem() {
  static bool done[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < 64 && done[dev]) return 0;
  e = cudaFuncSetAttribute(packed_gemv_kernel<K, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, gemv_smem_bytes<K, MT>());
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < 64) done[dev] = true;
  return 0;
}

template <int K, int MT>
static int launch_one(const GemvParams& p, int grid, cudaStream_t stream) {
  if (const int e = allow_smem<K, MT>()) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = p.split > 0 ? dim3(p.split, grid / p.split) : dim3(grid);   // split form: (parts of a row block, row blocks)
  cfg.blockDim = dim3(kGemvThreads);
  cfg.dynamicSmemBytes = gemv_smem_bytes<K, MT>();
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gemv_overlap_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, packed_gemv_kernel<K, MT>, p);
}

template <int K, int MT>
static int occupancy_one() {
  int ctas = 0;
  if (allow_smem<K, MT>()) return -1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas, packed_gemv_kernel<K, MT>, kGemvThreads, gemv_smem_bytes<K, MT>()) != cudaSuccess)
    return -1;
  return ctas;
}

template <>
int launch_packed_gemv<HTR_INST_K>(const GemvParams& p, int mt_rows, int grid, cudaStream_t stream) {
  switch (mt_rows) {
    case 1: return launch_one<HTR_INST_K, 1>(p, grid, stream);
    case 2: return launch_one<HTR_INST_K, 2>(p, grid, stream);
    case 4: return launch_one<HTR_INST_K, 4>(p, grid, stream);
    case 8: return launch_one<HTR_INST_K, 8>(p, grid, stream);
  }
  return (int)cudaErrorInvalidValue;
}

template <>
int packed_gemv_ctas_per_sm<HTR_INST_K>(int mt_rows) {
  switch (mt_rows) {
    case 1: return occupancy_one<HTR_INST_K, 1>();
    case 2: return occupancy_one<HTR_INST_K, 2>();
    case 4: return occupancy_one<HTR_INST_K, 4>();
    case 8: return occupancy_one<HTR_INST_K, 8>();
  }
  return -1;
}

}  // namespace htr

