// warp-MMA packed GEMV kernels for K = 8 bits per weight
#define HTR_INST_K 8
#include "packed_gemv_mma_inst.cuh"
