// tensor-core packed GEMM kernels for K = 6 bits per weight
#define HTR_INST_K 6
#include "packed_gemm_tc_inst.cuh"
