// warp-MMA packed GEMV kernels for K = 2 bits per weight
#define HTR_INST_K 2
#include "packed_gemv_mma_inst.cuh"
