// warp-MMA packed GEMV kernels for K = 4 bits per weight
#define HTR_INST_K 4
#include "packed_gemv_mma_inst.cuh"
