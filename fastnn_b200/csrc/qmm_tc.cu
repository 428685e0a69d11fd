// tcgen05 GEMM (placeholder until the TMA/TMEM path lands).
#include "common.cuh"
namespace fnn {
bool qmm_tc_supported(const fnn_cuda_qweight *, size_t) { return false; }
int prepare_qmm_tc(fnn_cuda_ctx *, fnn_cuda_qweight *) { return FNN_OK; }
int launch_qmm_tc(fnn_cuda_ctx *, const QmmArgs &) {
    return set_error(FNN_ERR_UNSUPPORTED, "qmatmul: tcgen05 path not built");
}
}  // namespace fnn
