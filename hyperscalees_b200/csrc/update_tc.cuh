// Interface between the update dispatcher (update.cu) and its tensor-core path (update_tc.cu).
#pragma once

#include "common.cuh"

namespace hses {

struct UpdateTcPlan {
    int64_t pairs, chunk_pairs;
    int bn, n_tiles, m_tiles, splits;
    size_t partial_bytes, raw_bytes, bytes;
};

// rank a multiple of 64: the shapes the tcgen05 contraction covers (ragged a and b are zero-filled)
bool update_tc_supports(int a, int b, int rank);
// need_raw: room for one chunk of regenerated fp32 factors (no factor cache)
UpdateTcPlan plan_update_tc(int a, int b, int rank, int64_t n, bool need_raw);
// grad (+)= scale * sum_p (f_2p - f_2p+1) A_p B_pᵀ; arguments already validated by the caller
// reuse_range: the power-of-two range of the pair weights that an earlier call with the same
// fitness vector and workspace left at the start of the workspace is still there (the layers of one
// model share both), so it is not computed again
int run_update_tc(hses_ctx* ctx, cudaStream_t stream, const hses_update_args& u, float scale,
                  bool reuse_range = false);
// hses_es_update_ex with that option; *took_tc tells whether the tensor-core contraction ran
int es_update_ex_impl(hses_ctx* ctx, hses_stream stream, const hses_update_args* args, bool reuse_range,
                      bool* took_tc);

}  // namespace hses
