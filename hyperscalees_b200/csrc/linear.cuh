// Interface between the perturbed-linear dispatcher and its tensor-core path.
#pragma once

#include "common.cuh"

namespace hses {

// True when the tcgen05 kernel covers the shapes/pitches of this call.
bool tensor_path_supports(const hses_linear_args& g);
size_t tensor_path_workspace_bytes(const hses_linear_args& g);
int run_tensor_path(hses_ctx* ctx, cudaStream_t stream, const hses_linear_args& g);

// The path for few rows per antithetic pair and wide factors (linear_pair.cu): clean product
// through the other paths, then one CTA per pair that streams the pair's factors once.
bool pair_path_supports(const hses_linear_args& g);
bool pair_path_fuses_scan(const hses_linear_args& g);   // lif == 2 is finished inside the per-pair kernel
size_t pair_path_workspace_bytes(const hses_linear_args& g);
int run_pair_path(hses_ctx* ctx, cudaStream_t stream, const hses_linear_args& g);

// Narrow layers (k, a <= 64, rank <= 16; linear_small.cu): persistent CTAs keep W in shared memory and
// walk over pairs.  Taken by HSES_ALGO_AUTO only.
bool small_path_supports(const hses_linear_args& g);
size_t small_path_workspace_bytes(const hses_linear_args& g);
int run_small_path(hses_ctx* ctx, cudaStream_t stream, const hses_linear_args& g);

// Checks args.cache against the call and returns the cached raw factors of the call's
// first pair: A rows (pair, a, rank) and B rows (pair, k, rank).
int resolve_factor_cache(const hses_linear_args& g, const float** A, const float** B);

}  // namespace hses
