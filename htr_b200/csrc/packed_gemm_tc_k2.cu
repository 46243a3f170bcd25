// tensor-core packed GEMM kernels for K = 2 bits per weight
#define HTR_INST_K 2
#include "packed_gemm_tc_inst.cuh"
