// Tensor-core (tcgen05 / TMEM / TMA) path of the perturbed linear layer.
#include "linear.cuh"

namespace hses {

bool tensor_path_supports(const hses_linear_args&) { return false; }
size_t tensor_path_workspace_bytes(const hses_linear_args&) { return 0; }
int run_tensor_path(hses_ctx*, cudaStream_t, const hses_linear_args&) {
    set_error("tensor path not available");
    return HSES_ERR_UNSUPPORTED;
}

}  // namespace hses
