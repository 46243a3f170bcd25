// warp-MMA packed GEMV kernels for K = 6 bits per weight
#define HTR_INST_K 6
#include "packed_gemv_mma_inst.cuh"
