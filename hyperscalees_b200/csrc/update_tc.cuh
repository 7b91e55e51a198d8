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
int run_update_tc(hses_ctx* ctx, cudaStream_t stream, const hses_update_args& u, float scale);

}  // namespace hses
