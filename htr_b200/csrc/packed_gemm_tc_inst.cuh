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
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  GemmParams q = p;
  q.cluster = 0;
#ifndef HTR_GEMM_NO_CLUSTER
  if (p.split >= 2 && p.split <= 8) {
    // the CTAs of a row block as one cluster, when every cluster of the grid can be resident at once
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)p.split;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
    // the occupancy query costs tens of microseconds on the host: remember the answer per (device, cluster size, shared memory)
    struct Seen { int dev, split, smem, clusters; };
    static thread_local Seen seen[8] = {};
    static thread_local int next_slot = 0;
    int dev = 0, clusters = -1;
    cudaGetDevice(&dev);
    for (const Seen& c : seen)
      if (c.split == p.split && c.smem == smem && c.dev == dev) clusters = c.clusters;
    if (clusters < 0) {
      if (cudaOccupancyMaxActiveClusters(&clusters, packed_gemm_tc_kernel<HTR_INST_K>, &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        clusters = 0;
      }
      seen[next_slot] = Seen{dev, p.split, smem, clusters};
      next_slot = (next_slot + 1) % 8;
    }
    if (clusters * p.split >= grid) q.cluster = 1;
    else cfg.numAttrs = 1;
  }
#endif
  return (int)cudaLaunchKernelEx(&cfg, packed_gemm_tc_kernel<HTR_INST_K>, q);
}

}  // namespace htr

