// tensor-core packed GEMM kernels for K = 3 bits per weight
#define HTR_INST_K 3
#include "packed_gemm_tc_inst.cuh"
