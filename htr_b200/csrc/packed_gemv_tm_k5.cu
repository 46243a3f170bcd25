// tensor-memory packed GEMV kernels for K = 5 bits per weight
#define HTR_INST_K 5
#include "packed_gemv_tm_inst.cuh"
