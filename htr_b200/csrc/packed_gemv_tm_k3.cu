// tensor-memory packed GEMV kernels for K = 3 bits per weight
#define HTR_INST_K 3
#include "packed_gemv_tm_inst.cuh"
