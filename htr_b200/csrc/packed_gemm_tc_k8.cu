// tensor-core packed GEMM kernels for K = 8 bits per weight
#define HTR_INST_K 8
#include "packed_gemm_tc_inst.cuh"
