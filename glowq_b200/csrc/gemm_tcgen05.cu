// Tensor-core (tcgen05 / TMEM) corrected W4A16 GEMM for prefill token counts.
#include "../../include/glowq_w4a16.h"
#include "params.h"

namespace glowq {
bool gemm_supported(const glowq_w4a16_group_t&) { return false; }
size_t gemm_workspace_bytes(int, int, int, int, int) { return 0; }
int gemm_group_forward(const glowq_w4a16_group_t&, cudaStream_t, cudaError_t*) { return GLOWQ_ERR_UNSUPPORTED_SHAPE; }
}  // namespace glowq
