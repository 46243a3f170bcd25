// tensor-memory packed GEMV kernels for K = 6 bits per weight
#define HTR_INST_K 6
#include "packed_gemv_tm_inst.cuh"
