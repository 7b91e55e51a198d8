// Sequence-model kernels on the population path: the RWKV-7 state recurrence and the spiking
// self-attention core.  One CTA per (sequence, head); the recurrent state stays in registers.
#include "common.cuh"

namespace hses {

// ---------------------------------------------------------------------------
// RWKV-7 inner loop (hyperscalees-models/src/llm.rs:235-296; models/llm/rwkv7.py:200-220):
//   dec = exp(-exp(w));  sa = S a;  S = S * dec + v k^T + sa b^T;  out = S r
// Thread i owns row i of the (S, S) state.  Operation order and rounding follow the
// reference's op-by-op evaluation: (S*dec) + v*k, then + sa*b, dot products in index order.
// ---------------------------------------------------------------------------
template <int S>
__global__ void __launch_bounds__(S)
wkv7_kernel(const float* __restrict__ r, const float* __restrict__ w, const float* __restrict__ k,
            const float* __restrict__ v, const float* __restrict__ a, const float* __restrict__ b,
            const uint8_t* __restrict__ new_starts, int T, int H, float* __restrict__ state,
            float* __restrict__ out) {
    __shared__ float sh[6][S];  // r, dec, k, v, a, b of the current step
    const int seq = blockIdx.x / H, h = blockIdx.x % H, i = threadIdx.x;
    float st[S];
    float* sp = state + (((size_t)seq * H + h) * S + i) * S;
#pragma unroll
    for (int j = 0; j < S; j += 4) {
        float4 q = *reinterpret_cast<const float4*>(sp + j);
        st[j] = q.x; st[j + 1] = q.y; st[j + 2] = q.z; st[j + 3] = q.w;
    }
    for (int t = 0; t < T; ++t) {
        size_t o = (((size_t)seq * T + t) * H + h) * S + i;
        __syncthreads();
        sh[0][i] = r[o];
        sh[1][i] = expf(-expf(w[o]));
        sh[2][i] = k[o];
        sh[3][i] = v[o];
        sh[4][i] = a[o];
        sh[5][i] = b[o];
        __syncthreads();
        if (new_starts && new_starts[(size_t)seq * T + t]) {
#pragma unroll
            for (int j = 0; j < S; ++j) st[j] = 0.0f;
        }
        float sa = 0.0f;
#pragma unroll
        for (int j = 0; j < S; ++j) sa = __fadd_rn(sa, __fmul_rn(st[j], sh[4][j]));
        const float vi = sh[3][i];
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < S; ++j) {
            float s1 = __fadd_rn(__fmul_rn(st[j], sh[1][j]), __fmul_rn(vi, sh[2][j]));
            st[j] = __fadd_rn(s1, __fmul_rn(sa, sh[5][j]));
            acc = __fadd_rn(acc, __fmul_rn(st[j], sh[0][j]));
        }
        out[o] = acc;
    }
#pragma unroll
    for (int j = 0; j < S; j += 4) *reinterpret_cast<float4*>(sp + j) = make_float4(st[j], st[j + 1], st[j + 2], st[j + 3]);
}

// ---------------------------------------------------------------------------
// Spiking self-attention core on firing rates Q, K, V of shape (tokens, d) per (sequence, head).
//   mode 0  spike product without softmax:  O = (beta * Q K^T) V
//   mode 1  LIF-count row softmax (src/hyperscalees/models/snn_self_attention.py:45-98): each row
//           of beta*QK^T is scaled by 1/(max|.| + 1e-6), then n_iter LIF steps with hard reset and
//           global inhibition g_inh * sum(counts so far); weights = count / (sum(count) + 1e-6)
// Thread i owns query row i; K and V of the head sit in shared memory.
// ---------------------------------------------------------------------------
constexpr int kMaxTokens = 128, kMaxHeadDim = 64;
__global__ void spiking_attention_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                         const float* __restrict__ V, int tokens, int heads, int d,
                                         int64_t row_stride, int mode, float beta, float tau_m, float v_th,
                                         float g_inh, int n_iter, float* __restrict__ O,
                                         float* __restrict__ A_out) {
    extern __shared__ float sm[];  // K (tokens, d) | V (tokens, d)
    float* ks = sm;
    float* vs = sm + tokens * d;
    const int seq = blockIdx.x / heads, h = blockIdx.x % heads;
    const size_t base = (size_t)seq * tokens * row_stride + (size_t)h * d;
    for (int e = threadIdx.x; e < tokens * d; e += blockDim.x) {
        int tk = e / d, c = e - tk * d;
        ks[e] = K[base + (size_t)tk * row_stride + c];
        vs[e] = V[base + (size_t)tk * row_stride + c];
    }
    __syncthreads();
    const int i = threadIdx.x;
    if (i >= tokens) return;
    float q[kMaxHeadDim];
    for (int c = 0; c < d; ++c) q[c] = Q[base + (size_t)i * row_stride + c];
    float hrow[kMaxTokens];
    float amax = 0.0f;
    for (int j = 0; j < tokens; ++j) {
        float acc = 0.0f;
        for (int c = 0; c < d; ++c) acc = __fadd_rn(acc, __fmul_rn(q[c], ks[j * d + c]));
        hrow[j] = __fmul_rn(beta, acc);
        amax = fmaxf(amax, fabsf(hrow[j]));
    }
    if (mode == 1) {
        const float inv = __fadd_rn(amax, 1e-6f);
        const float leak = 1.0f / tau_m;
        float u[kMaxTokens], cnt[kMaxTokens];
        for (int j = 0; j < tokens; ++j) { hrow[j] = __fdiv_rn(hrow[j], inv); u[j] = 0.0f; cnt[j] = 0.0f; }
        for (int it = 0; it < n_iter; ++it) {
            float G = 0.0f;
            for (int j = 0; j < tokens; ++j) G = __fadd_rn(G, cnt[j]);
            const float inh = __fmul_rn(g_inh, G);
            for (int j = 0; j < tokens; ++j) {
                float cur = __fsub_rn(hrow[j], inh);
                float c = __fadd_rn(u[j], __fmul_rn(__fadd_rn(-u[j], cur), leak));
                float s = c >= v_th ? 1.0f : 0.0f;
                u[j] = __fmul_rn(c, __fadd_rn(-s, 1.0f));
                cnt[j] = __fadd_rn(cnt[j], s);
            }
        }
        float tot = 0.0f;
        for (int j = 0; j < tokens; ++j) tot = __fadd_rn(tot, cnt[j]);
        tot = __fadd_rn(tot, 1e-6f);
        for (int j = 0; j < tokens; ++j) hrow[j] = __fdiv_rn(cnt[j], tot);
    }
    if (mode == 2) {
        // continuous Hopfield relaxation then a stable softmax along the keys
        // (hyperscalees-models/src/snn_transformer.rs:80-102)
        const float one_over_tau = 1.0f / tau_m;
        float u[kMaxTokens];
        for (int j = 0; j < tokens; ++j) u[j] = hrow[j];
        for (int it = 0; it < n_iter; ++it) {
            float m = 0.0f;
            for (int j = 0; j < tokens; ++j) m = __fadd_rn(m, u[j]);
            m = __fdiv_rn(m, (float)tokens);
            const float inh = __fmul_rn(m, g_inh);
            for (int j = 0; j < tokens; ++j)
                u[j] = __fadd_rn(u[j], __fmul_rn(__fsub_rn(__fadd_rn(-u[j], hrow[j]), inh), one_over_tau));
        }
        float mx = u[0];
        for (int j = 1; j < tokens; ++j) mx = fmaxf(mx, u[j]);
        float tot = 0.0f;
        for (int j = 0; j < tokens; ++j) {
            u[j] = expf(__fsub_rn(u[j], mx));
            tot = __fadd_rn(tot, u[j]);
        }
        tot = __fadd_rn(tot, 1e-6f);
        for (int j = 0; j < tokens; ++j) hrow[j] = __fdiv_rn(u[j], tot);
    }
    if (A_out)
        for (int j = 0; j < tokens; ++j)
            A_out[(((size_t)seq * heads + h) * tokens + i) * tokens + j] = hrow[j];
    for (int c = 0; c < d; ++c) {
        float acc = 0.0f;
        for (int j = 0; j < tokens; ++j) acc = __fadd_rn(acc, __fmul_rn(hrow[j], vs[j * d + c]));
        O[base + (size_t)i * row_stride + c] = acc;
    }
}

// ---------------------------------------------------------------------------
// RWKV-7 block pieces around the recurrence (hyperscalees-models/src/llm.rs:64-213)
// ---------------------------------------------------------------------------

// Statistics of `cnt` contiguous values per (row, group): one warp per group.
// layer_norm is the case of one group per row; var = E[x^2] - E[x]^2 as in the reference.
__global__ void group_stats_norm_kernel(const float* __restrict__ x, int64_t n_groups_total, int groups, int inner,
                                        int l, const float* __restrict__ weight, const float* __restrict__ bias,
                                        float eps, float* __restrict__ out) {
    int64_t gidx = (int64_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    int lane = threadIdx.x & 31;
    if (gidx >= n_groups_total) return;
    const int64_t cnt = (int64_t)inner * l;
    const float* xg = x + (size_t)gidx * cnt;
    float sum = 0.0f, sumsq = 0.0f;
    for (int64_t j = lane; j < cnt; j += 32) {
        float v = xg[j];
        sum += v;
        sumsq = fmaf(v, v, sumsq);
    }
    for (int off = 16; off > 0; off >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, off);
        sumsq += __shfl_xor_sync(0xffffffffu, sumsq, off);
    }
    const float mean = __fdiv_rn(sum, (float)cnt);
    const float var = __fsub_rn(__fdiv_rn(sumsq, (float)cnt), __fmul_rn(mean, mean));
    const float sd = __fsqrt_rn(__fadd_rn(var, eps));
    const int g = (int)(gidx % groups);
    float* og = out + (size_t)gidx * cnt;
    for (int64_t j = lane; j < cnt; j += 32) {
        int ch = g * inner + (int)(j / l);
        float nv = __fdiv_rn(__fsub_rn(xg[j], mean), sd);
        og[j] = __fadd_rn(__fmul_rn(nv, weight[ch]), bias[ch]);
    }
}

// out = x + (prev - x) * coef with prev = the previous row (row 0: state), 0 at new starts
__global__ void token_shift_mix_kernel(const float* __restrict__ x, int T, int c, const float* __restrict__ state,
                                       const uint8_t* __restrict__ new_starts, const float* __restrict__ coef,
                                       float* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)T * c) return;
    int t = (int)(i / c), j = (int)(i - (int64_t)t * c);
    float prev = t == 0 ? state[j] : x[i - c];
    if (new_starts && new_starts[t]) prev = 0.0f;
    float xv = x[i];
    out[i] = __fadd_rn(xv, __fmul_rn(__fsub_rn(prev, xv), coef[j]));
}

__global__ void relu_square_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = x[i] > 0.0f ? x[i] : 0.0f;
    out[i] = __fmul_rn(v, v);
}

// rate_encode, snn_transformer.rs:109-116: sigmoid(gain * p / (1 + |p|))
__global__ void rate_encode_kernel(const float* __restrict__ p, int64_t n, float gain, float* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float ss = __fdiv_rn(p[i], __fadd_rn(fabsf(p[i]), 1.0f));
    out[i] = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-__fmul_rn(ss, gain))));
}

}  // namespace hses

using namespace hses;

extern "C" {

int hses_wkv7(hses_ctx* ctx, hses_stream stream, const float* r, const float* w, const float* k,
              const float* v, const float* a, const float* b, const uint8_t* new_starts, int64_t n_seq,
              int32_t T, int32_t H, int32_t S, float* state, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n_seq >= 0 && T >= 1 && H >= 1, "bad shape");
    HSES_REQUIRE(S == 32 || S == 64, "head size must be 32 or 64");
    HSES_REQUIRE(n_seq * H < (1ll << 31), "too many (sequence, head) pairs");
    if (n_seq == 0) return HSES_OK;
    HSES_REQUIRE(r && w && k && v && a && b && state && out, "NULL pointer");
    HSES_REQUIRE(((uintptr_t)state & 15u) == 0, "state must be 16-byte aligned");
    HSES_KERNEL(ctx, as_stream(stream), "wkv7");
    unsigned grid = (unsigned)(n_seq * H);
    if (S == 64)
        wkv7_kernel<64><<<grid, 64, 0, as_stream(stream)>>>(r, w, k, v, a, b, new_starts, T, H, state, out);
    else
        wkv7_kernel<32><<<grid, 32, 0, as_stream(stream)>>>(r, w, k, v, a, b, new_starts, T, H, state, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_spiking_attention(hses_ctx* ctx, hses_stream stream, const float* Q, const float* K, const float* V,
                           int64_t n_seq, int32_t tokens, int32_t heads, int32_t head_dim, int64_t row_stride,
                           int32_t mode, float beta, float tau_m, float v_th, float g_inh, int32_t n_iter,
                           float* O, float* A_out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n_seq >= 0 && tokens >= 1 && tokens <= kMaxTokens, "tokens must be in 1..128");
    HSES_REQUIRE(heads >= 1 && head_dim >= 1 && head_dim <= kMaxHeadDim, "head_dim must be in 1..64");
    HSES_REQUIRE(row_stride >= (int64_t)heads * head_dim, "row stride smaller than heads*head_dim");
    HSES_REQUIRE(mode >= 0 && mode <= 2, "unknown mode");
    HSES_REQUIRE(mode == 0 || (tau_m != 0.0f && n_iter >= 1), "bad LIF parameters");
    HSES_REQUIRE(n_seq * heads < (1ll << 31), "too many (sequence, head) pairs");
    if (n_seq == 0) return HSES_OK;
    HSES_REQUIRE(Q && K && V && O, "NULL pointer");
    int threads = (tokens + 31) / 32 * 32;
    size_t smem = (size_t)2 * tokens * head_dim * sizeof(float);
    HSES_KERNEL(ctx, as_stream(stream), "spiking_attention");
    spiking_attention_kernel<<<(unsigned)(n_seq * heads), threads, smem, as_stream(stream)>>>(
        Q, K, V, tokens, heads, head_dim, row_stride, mode, beta, tau_m, v_th, g_inh, n_iter, O, A_out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_layer_norm(hses_ctx* ctx, hses_stream stream, const float* x, int64_t rows, int32_t c,
                    const float* weight, const float* bias, float eps, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(rows >= 0 && c >= 1, "bad shape");
    if (rows == 0) return HSES_OK;
    HSES_REQUIRE(x != nullptr && weight != nullptr && bias != nullptr && out != nullptr, "NULL pointer");
    HSES_KERNEL(ctx, as_stream(stream), "layer_norm");
    group_stats_norm_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, as_stream(stream)>>>(x, rows, 1, c, 1, weight, bias,
                                                                                      eps, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_group_norm(hses_ctx* ctx, hses_stream stream, const float* x, int64_t n, int32_t c, int32_t l,
                    int32_t groups, const float* weight, const float* bias, float eps, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n >= 0 && c >= 1 && l >= 1 && groups >= 1 && c % groups == 0, "bad shape");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(x != nullptr && weight != nullptr && bias != nullptr && out != nullptr, "NULL pointer");
    int64_t total = n * groups;
    HSES_KERNEL(ctx, as_stream(stream), "group_norm");
    group_stats_norm_kernel<<<(unsigned)((total + 7) / 8), 256, 0, as_stream(stream)>>>(x, total, groups, c / groups, l,
                                                                                       weight, bias, eps, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_token_shift_mix(hses_ctx* ctx, hses_stream stream, const float* x, int32_t T, int32_t c,
                         const float* state, const uint8_t* new_starts, const float* coef, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(T >= 0 && c >= 1, "bad shape");
    if (T == 0) return HSES_OK;
    HSES_REQUIRE(x != nullptr && state != nullptr && coef != nullptr && out != nullptr, "NULL pointer");
    HSES_REQUIRE(x != out, "token_shift_mix cannot run in place");
    int64_t n = (int64_t)T * c;
    HSES_KERNEL(ctx, as_stream(stream), "token_shift_mix");
    token_shift_mix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(x, T, c, state, new_starts, coef,
                                                                                      out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_relu_square(hses_ctx* ctx, hses_stream stream, const float* x, int64_t n, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n >= 0, "n must be >= 0");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(x != nullptr && out != nullptr, "NULL pointer");
    HSES_KERNEL(ctx, as_stream(stream), "relu_square");
    relu_square_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(x, n, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}


int hses_rate_encode(hses_ctx* ctx, hses_stream stream, const float* p, int64_t n, float gain, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n >= 0, "n must be >= 0");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(p != nullptr && out != nullptr, "NULL pointer");
    HSES_KERNEL(ctx, as_stream(stream), "rate_encode");
    rate_encode_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(p, n, gain, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // extern "C"
