// Interface between hses_einsum_pair (update.cu) and its tensor-core path (einsum_tc.cu).
#pragma once

#include "common.cuh"

namespace hses {

struct EinsumTcPlan {
    int bn, n_tiles, m_tiles, splits;
    int rb, ppb, kq;   // rows of a pair per 64-row k-block, pairs per k-block, k-blocks per pair
    int64_t blocks;
    size_t bytes;      // workspace: the three operand ranges and the split-K partial sums
};

// 16-byte aligned bases and strides, r from 32 up or a divisor of 64, and a contraction long
// enough to pay for the set-up; everything else stays on the fp32 kernel
bool einsum_tc_supports(const float* a_t, int64_t a_s0, int64_t a_s1, const float* b_t, int64_t b_s0, int64_t b_s1,
                        int64_t half, int r, int a, int b);
EinsumTcPlan plan_einsum_tc(int64_t half, int r, int a, int b);
// arguments already validated by the caller; workspace 256-byte aligned and of plan.bytes at least
int run_einsum_tc(hses_ctx* ctx, cudaStream_t stream, const float* a_t, int64_t a_s0, int64_t a_s1, const float* b_t,
                  int64_t b_s0, int64_t b_s1, const float* scores, int64_t half, int r, int a, int b, float* g_raw,
                  float* g_ones, void* workspace, size_t workspace_bytes);

}  // namespace hses
