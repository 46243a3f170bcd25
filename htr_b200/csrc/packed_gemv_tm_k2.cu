// tensor-memory packed GEMV kernels for K = 2 bits per weight
#define HTR_INST_K 2
#include "packed_gemv_tm_inst.cuh"
