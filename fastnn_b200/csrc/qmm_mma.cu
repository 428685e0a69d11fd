// Skinny-M tensor-core kernel (placeholder until the fragment-major path lands).
#include "common.cuh"
namespace fnn {
bool qmm_mma_supported(const fnn_cuda_qweight *, size_t) { return false; }
int launch_qmm_mma(fnn_cuda_ctx *, const QmmArgs &) {
    return set_error(FNN_ERR_UNSUPPORTED, "qmatmul: skinny tensor-core path not built");
}
}  // namespace fnn
