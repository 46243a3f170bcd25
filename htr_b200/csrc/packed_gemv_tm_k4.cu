// tensor-memory packed GEMV kernels for K = 4 bits per weight
#define HTR_INST_K 4
#include "packed_gemv_tm_inst.cuh"
