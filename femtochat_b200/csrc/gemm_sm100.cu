#include "common.cuh"
bool gemm_tc_supported(const GemmArgs&) { return false; }
int gemm_tc_bf16(const GemmArgs&, cudaStream_t) { return femto_fail(FEMTO_ERR_UNSUPPORTED, "tcgen05 GEMM not built"); }
