// Interface between the perturbed-linear dispatcher and its tensor-core path.
#pragma once

#include "common.cuh"

namespace hses {

// True when the tcgen05 kernel covers the shapes/pitches of this call.
bool tensor_path_supports(const hses_linear_args& g);
size_t tensor_path_workspace_bytes(const hses_linear_args& g);
int run_tensor_path(hses_ctx* ctx, cudaStream_t stream, const hses_linear_args& g);

}  // namespace hses
