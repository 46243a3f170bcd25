// tensor-core packed GEMM kernels for K = 5 bits per weight
#define HTR_INST_K 5
#include "packed_gemm_tc_inst.cuh"
