// Instantiates the packed GEMV for one stream width; included by packed_gemv_k<K>.cu with HTR_INST_K set.
#include "packed_gemv.cuh"

namespace htr {

template <int K, int MT>
static int launch_one(const GemvParams& p, int grid, cudaStream_t stream) {
  packed_gemv_kernel<K, MT><<<grid, kGemvThreads, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

template <int K, int MT>
static int occupancy_one() {
  int ctas = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas, packed_gemv_kernel<K, MT>, kGemvThreads, 0) != cudaSuccess) return -1;
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
