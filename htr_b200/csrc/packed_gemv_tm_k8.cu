// tensor-memory packed GEMV kernels for K = 8 bits per weight
#define HTR_INST_K 8
#include "packed_gemv_tm_inst.cuh"
