// Prefill GEMM on tcgen05 tensor cores (placeholder until the kernel lands).
#include "awq_common.cuh"

namespace awq {
bool gemm_tc_supported(int, int, int, int) { return false; }
int launch_gemm_tc(const uint16_t *, const int32_t *, const int32_t *, const uint16_t *, uint16_t *, int, int, int,
                   int, cudaStream_t) {
    return set_error(AWQ_ERR_UNSUPPORTED, "tensor-core gemm not built");
}
}  // namespace awq
