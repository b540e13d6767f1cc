#include "nq_common.cuh"
bool nq_tc_supported(int64_t, int64_t, int64_t) { return false; }
size_t nq_tc_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }
int nq_launch_tc_gemm(const void*, const void*, int64_t, int64_t, int64_t, void*, int, void*, cudaStream_t) { return NQ_ERR_ARG; }
