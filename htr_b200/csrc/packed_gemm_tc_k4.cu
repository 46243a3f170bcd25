// tensor-core packed GEMM kernels for K = 4 bits per weight
#define HTR_INST_K 4
#include "packed_gemm_tc_inst.cuh"
