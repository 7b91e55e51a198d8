// Pieces of the token-level spiking transformer (BASELINE's language-model form of the spiking
// self-attention model) that the other translation units do not cover:
//   embedding   do_emb of the noiser surface (src/hyperscalees/noiser/eggroll.py:93 and
//               hyperscalees-noiser/src/eggroll.rs:943-954 leave it unimplemented; the clean
//               gather param[x] is what their comment states): row gather from the (vocab, d)
//               table plus the member's rank-r term on the gathered row, A B^T with A (vocab, r)
//               and B (d, r) drawn like every other LoRA factor pair (eggroll.rs:86-103), plus
//               a learned position row
//   lif_rate    firing rate of a LIF neuron driven by a constant current for T steps: lif_step
//               (hyperscalees-models/src/snn.rs:53-65) T times from v = 0, rate = spikes / T —
//               the Q/K/V encoding of src/hyperscalees/models/snn_self_attention.py:114-131
//               when the projected current does not change over the T steps
//   swish       x * sigmoid(x), the feed-forward activation of snn_transformer.rs:404
//   next-token log-likelihood reduced per member
#include "common.cuh"

namespace hses {

// One thread per (row, 4 columns).  A is already scaled by sign * sigma / sqrt(rank).
__global__ void embedding_kernel(const int32_t* __restrict__ ids, int64_t rows, const float* __restrict__ table,
                                 int64_t table_stride, int vocab, int d, const float* __restrict__ pos, int L,
                                 const float* __restrict__ A, const float* __restrict__ B, int rank,
                                 int64_t rows_per_member, float* __restrict__ out, int64_t out_stride, int* status) {
    const int d4 = d >> 2;
    int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= rows * d4) return;
    const int64_t row = e / d4;
    const int c = (int)(e - row * d4) * 4;
    int id = ids[row];
    if (id < 0 || id >= vocab) {   // an id outside the table: reported, row of zeros
        atomicOr(status, 1 << 15);
        *reinterpret_cast<float4*>(out + (size_t)row * out_stride + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    float4 v = *reinterpret_cast<const float4*>(table + (size_t)id * table_stride + c);
    if (A != nullptr) {
        const int64_t m = row / rows_per_member;
        const float* a = A + ((size_t)m * vocab + id) * rank;
        const float* b = B + ((size_t)m * d + c) * rank;
        float u[4] = {0.f, 0.f, 0.f, 0.f};
        if ((rank & 3) == 0 && (((uintptr_t)A | (uintptr_t)B) & 15u) == 0) {
            // the same sums, q ascending, from 16-byte loads (the scalar form waits for 5 * rank dependent
            // 4-byte loads per thread)
            for (int q = 0; q < rank; q += 4) {
                const float4 a4 = __ldg(reinterpret_cast<const float4*>(a + q));
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 b4 = __ldg(reinterpret_cast<const float4*>(b + j * rank + q));
                    u[j] = __fadd_rn(u[j], __fmul_rn(a4.x, b4.x));
                    u[j] = __fadd_rn(u[j], __fmul_rn(a4.y, b4.y));
                    u[j] = __fadd_rn(u[j], __fmul_rn(a4.z, b4.z));
                    u[j] = __fadd_rn(u[j], __fmul_rn(a4.w, b4.w));
                }
            }
        } else {
            for (int q = 0; q < rank; ++q) {
                const float aq = a[q];
#pragma unroll
                for (int j = 0; j < 4; ++j) u[j] = __fadd_rn(u[j], __fmul_rn(aq, b[j * rank + q]));
            }
        }
        v.x = __fadd_rn(v.x, u[0]); v.y = __fadd_rn(v.y, u[1]);
        v.z = __fadd_rn(v.z, u[2]); v.w = __fadd_rn(v.w, u[3]);
    }
    if (pos != nullptr) {
        const float4 p = *reinterpret_cast<const float4*>(pos + (size_t)(row % L) * d + c);
        v.x = __fadd_rn(v.x, p.x); v.y = __fadd_rn(v.y, p.y);
        v.z = __fadd_rn(v.z, p.z); v.w = __fadd_rn(v.w, p.w);
    }
    *reinterpret_cast<float4*>(out + (size_t)row * out_stride + c) = v;
}

// TC: the number of steps when it is known at compile time (the loop unrolls, the reset mode is a constant
// and the division by a power of two a multiplication with the same result), 0: any T
template <int TC, int RESET>
__global__ void lif_rate_kernel(const float* __restrict__ cur, int64_t n, int T_run, float leak, float v_th, int reset_run,
                                float* __restrict__ out) {
    const int T = TC ? TC : T_run;
    const int reset = TC ? RESET : reset_run;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t n4 = n >> 2;
    if (i < n4) {
        const float4 c4 = __ldcs(reinterpret_cast<const float4*>(cur) + i);
        const float c[4] = {c4.x, c4.y, c4.z, c4.w};
        float r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v = 0.0f, s = 0.0f;
#pragma unroll
            for (int t = 0; t < (TC ? TC : 1); ++t) {
                if (TC) s = __fadd_rn(s, lif_update(v, c[j], leak, v_th, reset));
            }
            if (!TC)
                for (int t = 0; t < T; ++t) s = __fadd_rn(s, lif_update(v, c[j], leak, v_th, reset));
            r[j] = __fdiv_rn(s, (float)T);
        }
        reinterpret_cast<float4*>(out)[i] = make_float4(r[0], r[1], r[2], r[3]);
        return;
    }
    i = n4 * 4 + (i - n4);
    if (i < n) {
        float v = 0.0f, s = 0.0f;
        const float c = cur[i];
        for (int t = 0; t < T; ++t) s = __fadd_rn(s, lif_update(v, c, leak, v_th, reset));
        out[i] = __fdiv_rn(s, (float)T);
    }
}

__global__ void swish_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t n4 = n >> 2;
    auto f = [](float v) { return __fmul_rn(v, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v)))); };
    if (i < n4) {
        const float4 v = reinterpret_cast<const float4*>(x)[i];
        reinterpret_cast<float4*>(out)[i] = make_float4(f(v.x), f(v.y), f(v.z), f(v.w));
        return;
    }
    i = n4 * 4 + (i - n4);
    if (i < n) out[i] = f(x[i]);
}

// acc += y (the residual connections), 16 bytes per thread
__global__ void add_inplace_kernel(float* __restrict__ acc, const float* __restrict__ y, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t n4 = n >> 2;
    if (i < n4) {
        float4 a = reinterpret_cast<float4*>(acc)[i];
        const float4 b = reinterpret_cast<const float4*>(y)[i];
        a.x = __fadd_rn(a.x, b.x); a.y = __fadd_rn(a.y, b.y); a.z = __fadd_rn(a.z, b.z); a.w = __fadd_rn(a.w, b.w);
        reinterpret_cast<float4*>(acc)[i] = a;
        return;
    }
    i = n4 * 4 + (i - n4);
    if (i < n) acc[i] = __fadd_rn(acc[i], y[i]);
}

// Next-token log-likelihood of a member: mean over its sequences and over positions 0..L-2 of
// log_softmax(logits[s, t])[ids[s, t+1]] (max-shifted, like fitness_from_logits_reward,
// hyperscalees-envs/src/snn_mnist.rs:186-193).  One warp per (sequence, position); the per-member
// sum is taken in a second kernel in a fixed order.
__global__ void token_loglik_kernel(const float* __restrict__ logits, int64_t logits_stride, const int32_t* __restrict__ ids,
                                    int64_t n_seq, int L, int vocab, float gain, float* __restrict__ lp) {
    const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= n_seq * L) return;
    const int t = (int)(w % L);
    if (t == L - 1) {   // the last position has no next token
        if (lane == 0) lp[w] = 0.0f;
        return;
    }
    const float* row = logits + (size_t)w * logits_stride;
    // One pass with a running maximum (a row of a 50 277-word vocabulary is 200 KB and thousands of rows are
    // in flight: a second pass would come from HBM again, and the kernel is bound by those bytes).  A lane
    // keeps the maximum mx of what it has seen and s = sum exp(x - mx); a new maximum rescales s, which is
    // rare after the first few values.  Rows that start on a 16-byte boundary are read 16 bytes per lane.
    const int v4 = (((uintptr_t)row & 15u) == 0) ? vocab >> 2 : 0;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    float mx = -INFINITY, s = 0.0f;
    auto take = [&](float raw) {
        const float xv = __fmul_rn(raw, gain);
        if (xv > mx) {
            s = fmaf(s, expf(mx - xv), 1.0f);
            mx = xv;
        } else {
            s += expf(xv - mx);
        }
    };
#pragma unroll 4
    for (int c = lane; c < v4; c += 32) {
        const float4 q = __ldcs(row4 + c);
        take(q.x); take(q.y); take(q.z); take(q.w);
    }
    for (int c = 4 * v4 + lane; c < vocab; c += 32) take(row[c]);
    for (int off = 16; off > 0; off >>= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, mx, off), so = __shfl_xor_sync(0xffffffffu, s, off);
        const float mn = fmaxf(mx, mo);
        // a lane that saw nothing has mx = -inf and s = 0: its term is 0 * exp(-inf) = 0
        s = (mx == mn ? s : s * expf(mx - mn)) + (mo == mn ? so : so * expf(mo - mn));
        mx = mn;
    }
    if (lane == 0) {
        const int target = ids[w + 1];
        lp[w] = (target >= 0 && target < vocab) ? (__fmul_rn(row[target], gain) - mx) - logf(s) : 0.0f;
    }
}
__global__ void member_token_mean_kernel(const float* __restrict__ lp, int64_t n_members, int seqs, int L,
                                         float* __restrict__ out) {
    const int64_t m = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (m >= n_members) return;
    const int64_t cnt = (int64_t)seqs * L;
    float s = 0.0f;
    for (int64_t i = lane; i < cnt; i += 32) s += lp[m * cnt + i];
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) out[m] = s / (float)((int64_t)seqs * (L - 1));
}

}  // namespace hses

using namespace hses;

extern "C" {

int hses_embedding(hses_ctx* ctx, hses_stream stream, const int32_t* ids, int64_t rows, const float* table,
                   int64_t table_stride, int32_t vocab, int32_t d, const float* pos, int32_t L, const float* A,
                   const float* B, int32_t rank, int64_t rows_per_member, float* out, int64_t out_stride) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(rows >= 0 && vocab >= 1 && d >= 4 && d % 4 == 0, "d must be a positive multiple of 4");
    if (rows == 0) return HSES_OK;
    HSES_REQUIRE(ids != nullptr && table != nullptr && out != nullptr, "NULL pointer");
    HSES_REQUIRE(table_stride >= d && table_stride % 4 == 0 && out_stride >= d && out_stride % 4 == 0,
                 "row strides must be multiples of 4 and at least d");
    HSES_REQUIRE((((uintptr_t)table | (uintptr_t)out | (uintptr_t)pos) & 15u) == 0, "table, pos and out must be 16-byte aligned");
    HSES_REQUIRE(pos == nullptr || L >= 1, "L must be positive when a position table is given");
    HSES_REQUIRE((A == nullptr) == (B == nullptr), "A and B come together");
    HSES_REQUIRE(A == nullptr || (rank >= 1 && rows_per_member >= 1 && rows % rows_per_member == 0),
                 "rows must be whole members");
    int64_t work = rows * (d / 4);
    HSES_KERNEL(ctx, as_stream(stream), "embedding");
    embedding_kernel<<<(unsigned)((work + 255) / 256), 256, 0, as_stream(stream)>>>(
        ids, rows, table, table_stride, vocab, d, pos, L > 0 ? L : 1, A, B, rank, rows_per_member > 0 ? rows_per_member : 1,
        out, out_stride, ctx->t.status_word);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_lif_rate(hses_ctx* ctx, hses_stream stream, const float* cur, int64_t n, int32_t T, float tau_m, float v_th,
                  int32_t reset_mode, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n >= 0 && T >= 1 && tau_m != 0.0f, "bad arguments");
    HSES_REQUIRE(reset_mode == HSES_RESET_HARD || reset_mode == HSES_RESET_SUBTRACT, "unknown reset mode");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(cur != nullptr && out != nullptr, "NULL pointer");
    HSES_REQUIRE((((uintptr_t)cur | (uintptr_t)out) & 15u) == 0, "cur and out must be 16-byte aligned");
    int64_t work = n / 4 + n % 4;
    HSES_KERNEL(ctx, as_stream(stream), "lif_rate");
    const unsigned grid = (unsigned)((work + 255) / 256);
    const float leak = 1.0f / tau_m;
    if (T == 4 && reset_mode == HSES_RESET_HARD)
        lif_rate_kernel<4, HSES_RESET_HARD><<<grid, 256, 0, as_stream(stream)>>>(cur, n, T, leak, v_th, reset_mode, out);
    else if (T == 4)
        lif_rate_kernel<4, HSES_RESET_SUBTRACT><<<grid, 256, 0, as_stream(stream)>>>(cur, n, T, leak, v_th, reset_mode, out);
    else if (T == 8 && reset_mode == HSES_RESET_HARD)
        lif_rate_kernel<8, HSES_RESET_HARD><<<grid, 256, 0, as_stream(stream)>>>(cur, n, T, leak, v_th, reset_mode, out);
    else
        lif_rate_kernel<0, 0><<<grid, 256, 0, as_stream(stream)>>>(cur, n, T, leak, v_th, reset_mode, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_swish(hses_ctx* ctx, hses_stream stream, const float* x, int64_t n, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n >= 0, "n must be >= 0");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(x != nullptr && out != nullptr, "NULL pointer");
    HSES_REQUIRE((((uintptr_t)x | (uintptr_t)out) & 15u) == 0, "x and out must be 16-byte aligned");
    int64_t work = n / 4 + n % 4;
    HSES_KERNEL(ctx, as_stream(stream), "swish");
    swish_kernel<<<(unsigned)((work + 255) / 256), 256, 0, as_stream(stream)>>>(x, n, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_add_inplace(hses_ctx* ctx, hses_stream stream, float* acc, const float* y, int64_t n) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n >= 0, "n must be >= 0");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(acc != nullptr && y != nullptr, "NULL pointer");
    HSES_REQUIRE((((uintptr_t)acc | (uintptr_t)y) & 15u) == 0, "acc and y must be 16-byte aligned");
    int64_t work = n / 4 + n % 4;
    HSES_KERNEL(ctx, as_stream(stream), "add_inplace");
    add_inplace_kernel<<<(unsigned)((work + 255) / 256), 256, 0, as_stream(stream)>>>(acc, y, n);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_token_fitness(hses_ctx* ctx, hses_stream stream, const float* logits, int64_t logits_stride,
                       const int32_t* ids, int64_t n_members, int32_t seqs, int32_t L, int32_t vocab, float gain,
                       float* per_token, float* fitness) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n_members >= 0 && seqs >= 1 && L >= 2 && vocab >= 1, "bad shape");
    if (n_members == 0) return HSES_OK;
    HSES_REQUIRE(logits != nullptr && ids != nullptr && per_token != nullptr && fitness != nullptr, "NULL pointer");
    HSES_REQUIRE(logits_stride >= vocab, "logits stride smaller than the vocabulary");
    const int64_t n_seq = n_members * seqs;
    const int64_t warps = n_seq * L;
    {
        HSES_KERNEL(ctx, as_stream(stream), "token_loglik");
        token_loglik_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, as_stream(stream)>>>(logits, logits_stride, ids, n_seq,
                                                                                      L, vocab, gain, per_token);
        HSES_LAUNCH_CHECK();
    }
    HSES_KERNEL(ctx, as_stream(stream), "member_token_mean");
    member_token_mean_kernel<<<(unsigned)((n_members + 7) / 8), 256, 0, as_stream(stream)>>>(per_token, n_members, seqs,
                                                                                          L, fitness);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // extern "C"
