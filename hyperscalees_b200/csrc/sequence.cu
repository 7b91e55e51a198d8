// Sequence-model kernels on the population path: the RWKV-7 state recurrence and the spiking
// self-attention core.  One CTA per (sequence, head); the recurrent state stays in registers.
#include "common.cuh"

namespace hses {

// Packed fp32 pairs (sm_100 f32x2 arithmetic): one instruction works on two independent IEEE
// fp32 lanes.  Lane 0 is the low word: a pair loaded from memory holds (p[0], p[1]).
// Measured on B200: a packed instruction issues at half the rate of a scalar one, so the lane
// throughput is the same and only issue slots are saved; and the assembler contracts a packed
// multiply followed by a packed add into a packed fma even when both carry .rn, so code that
// needs two roundings per multiply-add cannot use the packed forms.  The kernels below that use
// them (mode 0 of the attention, the WKV-7 recurrence) therefore round each multiply-add once.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void upk2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// ---------------------------------------------------------------------------
// RWKV-7 inner loop (hyperscalees-models/src/llm.rs:235-296; models/llm/rwkv7.py:200-220):
//   dec = exp(-exp(w));  sa = S a;  S = S * dec + v k^T + sa b^T;  out = S r
// Thread i owns rows 2i and 2i+1 of the (S, S) state as packed pairs.  Every multiply-add is one fused
// operation (S*dec, then fma(v, k, .), then fma(sa, b, .)); the two dot products run as four
// interleaved partial sums that are added at the end.  The reference rounds
// each tensor operation separately: results agree to a few ulp per step (tested to 1e-5).
// ---------------------------------------------------------------------------
template <int S>
__global__ void __launch_bounds__(S / 2)
wkv7_kernel(const float* __restrict__ r, const float* __restrict__ w, const float* __restrict__ k,
            const float* __restrict__ v, const float* __restrict__ a, const float* __restrict__ b,
            const uint8_t* __restrict__ new_starts, int T, int H, float* __restrict__ state,
            float* __restrict__ out) {
    __shared__ __align__(16) float shbuf[2][6][S];  // r, dec, k, v, a, b of a step
    const int seq = blockIdx.x / H, h = blockIdx.x % H, i = threadIdx.x;
    // rows 2i and 2i+1 of the state as S/2 packed pairs (st[2p], st[2p+1]) each: every 16-byte
    // piece of a step vector read from shared memory feeds both rows
    f32x2 sta[S / 2], stb[S / 2];
    float* sp = state + (((size_t)seq * H + h) * S + 2 * i) * S;
#pragma unroll
    for (int p = 0; p < S / 2; p += 2) {
        ulonglong2 q = *reinterpret_cast<const ulonglong2*>(sp + 2 * p);
        sta[p] = q.x;
        sta[p + 1] = q.y;
        q = *reinterpret_cast<const ulonglong2*>(sp + S + 2 * p);
        stb[p] = q.x;
        stb[p + 1] = q.y;
    }
    // The six vectors of a step go through a double-buffered shared-memory block (one barrier per
    // step); those of the next step are fetched into registers while this step computes.
    const size_t o0 = ((size_t)seq * T * H + h) * S + 2 * i, ostep = (size_t)H * S;
    auto ld2 = [](const float* p) { return *reinterpret_cast<const float2*>(p); };
    float2 nr = ld2(r + o0), nw = ld2(w + o0), nk = ld2(k + o0), nv = ld2(v + o0), na = ld2(a + o0), nb = ld2(b + o0);
    for (int t = 0; t < T; ++t) {
        const size_t o = o0 + (size_t)t * ostep;
        float(*sh)[S] = shbuf[t & 1];
        *reinterpret_cast<float2*>(&sh[0][2 * i]) = nr;
        *reinterpret_cast<float2*>(&sh[1][2 * i]) = make_float2(expf(-expf(nw.x)), expf(-expf(nw.y)));
        *reinterpret_cast<float2*>(&sh[2][2 * i]) = nk;
        *reinterpret_cast<float2*>(&sh[4][2 * i]) = na;
        *reinterpret_cast<float2*>(&sh[5][2 * i]) = nb;
        const float via = nv.x, vib = nv.y;   // v of the thread's own rows
        __syncthreads();
        if (t + 1 < T) {
            const size_t on = o + ostep;
            nr = ld2(r + on); nw = ld2(w + on); nk = ld2(k + on); nv = ld2(v + on); na = ld2(a + on); nb = ld2(b + on);
        }
        if (new_starts && new_starts[(size_t)seq * T + t]) {
#pragma unroll
            for (int p = 0; p < S / 2; ++p) sta[p] = stb[p] = 0ull;
        }
        f32x2 saa_p = 0ull, saa_q = 0ull, sab_p = 0ull, sab_q = 0ull;   // (even, odd) partial sums, two chains per row
#pragma unroll
        for (int p = 0; p < S / 2; p += 2) {
            const ulonglong2 av = *reinterpret_cast<const ulonglong2*>(&sh[4][2 * p]);
            saa_p = fma2(sta[p], av.x, saa_p);
            saa_q = fma2(sta[p + 1], av.y, saa_q);
            sab_p = fma2(stb[p], av.x, sab_p);
            sab_q = fma2(stb[p + 1], av.y, sab_q);
        }
        float e0, e1;
        upk2(add2(saa_p, saa_q), e0, e1);
        const float saa = __fadd_rn(e0, e1);
        upk2(add2(sab_p, sab_q), e0, e1);
        const float sab = __fadd_rn(e0, e1);
        const f32x2 via2 = pk2(via, via), vib2 = pk2(vib, vib), saa2 = pk2(saa, saa), sab2 = pk2(sab, sab);
        f32x2 acca_p = 0ull, acca_q = 0ull, accb_p = 0ull, accb_q = 0ull;
#pragma unroll
        for (int p = 0; p < S / 2; p += 2) {
            const ulonglong2 dv = *reinterpret_cast<const ulonglong2*>(&sh[1][2 * p]);
            const ulonglong2 kv = *reinterpret_cast<const ulonglong2*>(&sh[2][2 * p]);
            const ulonglong2 bv = *reinterpret_cast<const ulonglong2*>(&sh[5][2 * p]);
            const ulonglong2 rv = *reinterpret_cast<const ulonglong2*>(&sh[0][2 * p]);
            sta[p] = fma2(saa2, bv.x, fma2(via2, kv.x, mul2(sta[p], dv.x)));
            sta[p + 1] = fma2(saa2, bv.y, fma2(via2, kv.y, mul2(sta[p + 1], dv.y)));
            stb[p] = fma2(sab2, bv.x, fma2(vib2, kv.x, mul2(stb[p], dv.x)));
            stb[p + 1] = fma2(sab2, bv.y, fma2(vib2, kv.y, mul2(stb[p + 1], dv.y)));
            acca_p = fma2(sta[p], rv.x, acca_p);
            acca_q = fma2(sta[p + 1], rv.y, acca_q);
            accb_p = fma2(stb[p], rv.x, accb_p);
            accb_q = fma2(stb[p + 1], rv.y, accb_q);
        }
        float2 res;
        upk2(add2(acca_p, acca_q), e0, e1);
        res.x = __fadd_rn(e0, e1);
        upk2(add2(accb_p, accb_q), e0, e1);
        res.y = __fadd_rn(e0, e1);
        *reinterpret_cast<float2*>(out + o) = res;
    }
#pragma unroll
    for (int p = 0; p < S / 2; p += 2) {
        ulonglong2 q;
        q.x = sta[p];
        q.y = sta[p + 1];
        *reinterpret_cast<ulonglong2*>(sp + 2 * p) = q;
        q.x = stb[p];
        q.y = stb[p + 1];
        *reinterpret_cast<ulonglong2*>(sp + S + 2 * p) = q;
    }
}

// ---------------------------------------------------------------------------
// Spiking self-attention core on firing rates Q, K, V of shape (tokens, d) per (sequence, head).
//   mode 0  spike product without softmax:  O = (beta * Q K^T) V
//   mode 3  the same with a causal mask: the score of key j is zero for j > i (next-token models)
//   mode 1  LIF-count row softmax (src/hyperscalees/models/snn_self_attention.py:45-98): each row
//           of beta*QK^T is scaled by 1/(max|.| + 1e-6), then n_iter LIF steps with hard reset and
//           global inhibition g_inh * sum(counts so far); weights = count / (sum(count) + 1e-6)
// Thread i owns query row i; K and V of the head sit in shared memory.
// ---------------------------------------------------------------------------
constexpr int kMaxTokens = 128, kMaxHeadDim = 64;
__global__ void spiking_attention_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                         const float* __restrict__ V, int tokens, int heads, int d,
                                         int64_t row_stride, int mode, float beta, const float* __restrict__ beta_seq,
                                         float tau_m, float v_th, float g_inh, int n_iter, float* __restrict__ O,
                                         float* __restrict__ A_out) {
    extern __shared__ float sm[];  // K (tokens, d) | V (tokens, d)
    float* ks = sm;
    float* vs = sm + tokens * d;
    const int seq = blockIdx.x / heads, h = blockIdx.x % heads;
    if (beta_seq) beta = beta_seq[seq];   // one scale per sequence (a member's own beta)
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
        if (mode == 3 && j > i) hrow[j] = 0.0f;   // causal spike product: a query sees keys 0..i only
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

// Mode 0 for head sizes 16/32/64 with 16-byte aligned rows: the same sums in the same order as
// the kernel above with one rounding per multiply-add (fma) instead of two; q and the output row
// live in registers (compile-time head size), K and V
// are staged with 16-byte loads and read back as broadcasts, and the score of key j is used as
// soon as it is known, so no row of scores is kept.  Four keys are in flight at a time to give
// the sequential dot products independent chains.
template <int D>
__global__ void __launch_bounds__(128)
attention_product_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                         int tokens, int heads, int64_t row_stride, float beta, const float* __restrict__ beta_seq,
                         int causal, float* __restrict__ O, float* __restrict__ A_out) {
    extern __shared__ __align__(16) float sm[];  // K (tokens, D) | V (tokens, D)
    float4* ks4 = reinterpret_cast<float4*>(sm);
    float4* vs4 = ks4 + tokens * (D / 4);
    const int seq = blockIdx.x / heads, h = blockIdx.x % heads;
    if (beta_seq) beta = beta_seq[seq];   // one scale per sequence (a member's own beta)
    const size_t base = (size_t)seq * tokens * row_stride + (size_t)h * D;
    constexpr int D4 = D / 4;
    for (int e = threadIdx.x; e < tokens * D4; e += blockDim.x) {
        int tk = e / D4, c4 = e - tk * D4;
        ks4[e] = *reinterpret_cast<const float4*>(K + base + (size_t)tk * row_stride + c4 * 4);
        vs4[e] = *reinterpret_cast<const float4*>(V + base + (size_t)tk * row_stride + c4 * 4);
    }
    __syncthreads();
    const int i = threadIdx.x;
    if (i >= tokens) return;
    float q[D], acc[D];
#pragma unroll
    for (int c4 = 0; c4 < D4; ++c4) {
        float4 v = *reinterpret_cast<const float4*>(Q + base + (size_t)i * row_stride + c4 * 4);
        q[4 * c4] = v.x; q[4 * c4 + 1] = v.y; q[4 * c4 + 2] = v.z; q[4 * c4 + 3] = v.w;
    }
#pragma unroll
    for (int c = 0; c < D; ++c) acc[c] = 0.0f;
    float* arow = A_out ? A_out + (((size_t)seq * heads + h) * tokens + i) * tokens : nullptr;
    constexpr int JB = 4;
    for (int j0 = 0; j0 < tokens; j0 += JB) {
        float sc[JB];
#pragma unroll
        for (int u = 0; u < JB; ++u) sc[u] = 0.0f;
#pragma unroll
        for (int c4 = 0; c4 < D4; ++c4) {
#pragma unroll
            for (int u = 0; u < JB; ++u) {
                const int j = j0 + u < tokens ? j0 + u : tokens - 1;
                const float4 kv = ks4[j * D4 + c4];
                sc[u] = fmaf(q[4 * c4], kv.x, sc[u]);
                sc[u] = fmaf(q[4 * c4 + 1], kv.y, sc[u]);
                sc[u] = fmaf(q[4 * c4 + 2], kv.z, sc[u]);
                sc[u] = fmaf(q[4 * c4 + 3], kv.w, sc[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < JB; ++u) {
            if (j0 + u < tokens) {
                const float hj = (causal && j0 + u > i) ? 0.0f : __fmul_rn(beta, sc[u]);
                if (arow) arow[j0 + u] = hj;
#pragma unroll
                for (int c4 = 0; c4 < D4; ++c4) {
                    const float4 vv = vs4[(j0 + u) * D4 + c4];
                    acc[4 * c4] = fmaf(hj, vv.x, acc[4 * c4]);
                    acc[4 * c4 + 1] = fmaf(hj, vv.y, acc[4 * c4 + 1]);
                    acc[4 * c4 + 2] = fmaf(hj, vv.z, acc[4 * c4 + 2]);
                    acc[4 * c4 + 3] = fmaf(hj, vv.w, acc[4 * c4 + 3]);
                }
            }
        }
    }
#pragma unroll
    for (int c4 = 0; c4 < D4; ++c4)
        *reinterpret_cast<float4*>(O + base + (size_t)i * row_stride + c4 * 4) =
            make_float4(acc[4 * c4], acc[4 * c4 + 1], acc[4 * c4 + 2], acc[4 * c4 + 3]);
}

// Modes 1 and 2 for head sizes 16/32/64 with 16-byte aligned rows.  Same operations in the same
// order as the general kernel (two roundings per multiply-add: these modes end in threshold
// decisions or a softmax), but q and the output row live in registers, K and V are read back as
// 16-byte broadcasts, and the per-row arrays (scores, potentials, counts) sit in shared memory
// with an odd pitch instead of local memory.
template <int D>
__global__ void __launch_bounds__(128)
attention_rows_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                      int tokens, int heads, int64_t row_stride, int mode, float beta, const float* __restrict__ beta_seq,
                      float tau_m, float v_th, float g_inh, int n_iter, float* __restrict__ O, float* __restrict__ A_out) {
    extern __shared__ __align__(16) float sm[];
    constexpr int D4 = D / 4;
    const int pitch = tokens + 1;
    float4* ks4 = reinterpret_cast<float4*>(sm);
    float4* vs4 = ks4 + tokens * D4;
    float* hs = sm + 2 * tokens * D;
    float* us = hs + tokens * pitch;
    float* cs = us + tokens * pitch;   // mode 1 only
    const int seq = blockIdx.x / heads, h = blockIdx.x % heads;
    if (beta_seq) beta = beta_seq[seq];   // one scale per sequence (a member's own beta)
    const size_t base = (size_t)seq * tokens * row_stride + (size_t)h * D;
    for (int e = threadIdx.x; e < tokens * D4; e += blockDim.x) {
        int tk = e / D4, c4 = e - tk * D4;
        ks4[e] = *reinterpret_cast<const float4*>(K + base + (size_t)tk * row_stride + c4 * 4);
        vs4[e] = *reinterpret_cast<const float4*>(V + base + (size_t)tk * row_stride + c4 * 4);
    }
    __syncthreads();
    const int i = threadIdx.x;
    if (i >= tokens) return;
    float q[D];
#pragma unroll
    for (int c4 = 0; c4 < D4; ++c4) {
        float4 v = *reinterpret_cast<const float4*>(Q + base + (size_t)i * row_stride + c4 * 4);
        q[4 * c4] = v.x; q[4 * c4 + 1] = v.y; q[4 * c4 + 2] = v.z; q[4 * c4 + 3] = v.w;
    }
    float* hrow = hs + i * pitch;
    float* u = us + i * pitch;
    float* cnt = cs + i * pitch;
    float amax = 0.0f;
    for (int j0 = 0; j0 < tokens; j0 += 4) {
        float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int c4 = 0; c4 < D4; ++c4) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int j = j0 + k < tokens ? j0 + k : tokens - 1;
                const float4 kv = ks4[j * D4 + c4];
                sc[k] = __fadd_rn(sc[k], __fmul_rn(q[4 * c4], kv.x));
                sc[k] = __fadd_rn(sc[k], __fmul_rn(q[4 * c4 + 1], kv.y));
                sc[k] = __fadd_rn(sc[k], __fmul_rn(q[4 * c4 + 2], kv.z));
                sc[k] = __fadd_rn(sc[k], __fmul_rn(q[4 * c4 + 3], kv.w));
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (j0 + k < tokens) {
                const float hv = __fmul_rn(beta, sc[k]);
                hrow[j0 + k] = hv;
                amax = fmaxf(amax, fabsf(hv));
            }
    }
    if (mode == 1) {
        const float inv = __fadd_rn(amax, 1e-6f);
        const float leak = 1.0f / tau_m;
        for (int j = 0; j < tokens; ++j) {
            hrow[j] = __fdiv_rn(hrow[j], inv);
            u[j] = 0.0f;
            cnt[j] = 0.0f;
        }
        // the counts are small integers: their sum is exact in any order, so the inhibition of
        // an iteration is the running number of spikes before it
        float G = 0.0f;
        for (int it = 0; it < n_iter; ++it) {
            const float inh = __fmul_rn(g_inh, G);
            for (int j = 0; j < tokens; ++j) {
                const float uj = u[j];
                float cur = __fsub_rn(hrow[j], inh);
                float c = __fadd_rn(uj, __fmul_rn(__fadd_rn(-uj, cur), leak));
                float sp = c >= v_th ? 1.0f : 0.0f;
                u[j] = __fmul_rn(c, __fadd_rn(-sp, 1.0f));
                cnt[j] = __fadd_rn(cnt[j], sp);
                G = __fadd_rn(G, sp);
            }
        }
        const float tot = __fadd_rn(G, 1e-6f);
        for (int j = 0; j < tokens; ++j) hrow[j] = __fdiv_rn(cnt[j], tot);
    } else {
        // continuous Hopfield relaxation then a stable softmax along the keys
        // (hyperscalees-models/src/snn_transformer.rs:80-102)
        const float one_over_tau = 1.0f / tau_m;
        for (int j = 0; j < tokens; ++j) u[j] = hrow[j];
        for (int it = 0; it < n_iter; ++it) {
            float m = 0.0f;
            for (int j = 0; j < tokens; ++j) m = __fadd_rn(m, u[j]);
            m = __fdiv_rn(m, (float)tokens);
            const float inh = __fmul_rn(m, g_inh);
            for (int j = 0; j < tokens; ++j) {
                const float uj = u[j];
                u[j] = __fadd_rn(uj, __fmul_rn(__fsub_rn(__fadd_rn(-uj, hrow[j]), inh), one_over_tau));
            }
        }
        float mx = u[0];
        for (int j = 1; j < tokens; ++j) mx = fmaxf(mx, u[j]);
        float tot = 0.0f;
        for (int j = 0; j < tokens; ++j) {
            const float e = expf(__fsub_rn(u[j], mx));
            u[j] = e;
            tot = __fadd_rn(tot, e);
        }
        tot = __fadd_rn(tot, 1e-6f);
        for (int j = 0; j < tokens; ++j) hrow[j] = __fdiv_rn(u[j], tot);
    }
    float* arow = A_out ? A_out + (((size_t)seq * heads + h) * tokens + i) * tokens : nullptr;
    float acc[D];
#pragma unroll
    for (int c = 0; c < D; ++c) acc[c] = 0.0f;
    for (int j = 0; j < tokens; ++j) {
        const float hj = hrow[j];
        if (arow) arow[j] = hj;
#pragma unroll
        for (int c4 = 0; c4 < D4; ++c4) {
            const float4 vv = vs4[j * D4 + c4];
            acc[4 * c4] = __fadd_rn(acc[4 * c4], __fmul_rn(hj, vv.x));
            acc[4 * c4 + 1] = __fadd_rn(acc[4 * c4 + 1], __fmul_rn(hj, vv.y));
            acc[4 * c4 + 2] = __fadd_rn(acc[4 * c4 + 2], __fmul_rn(hj, vv.z));
            acc[4 * c4 + 3] = __fadd_rn(acc[4 * c4 + 3], __fmul_rn(hj, vv.w));
        }
    }
#pragma unroll
    for (int c4 = 0; c4 < D4; ++c4)
        *reinterpret_cast<float4*>(O + base + (size_t)i * row_stride + c4 * 4) =
            make_float4(acc[4 * c4], acc[4 * c4 + 1], acc[4 * c4 + 2], acc[4 * c4 + 3]);
}

template <int D>
static cudaError_t launch_attention_rows(cudaStream_t st, unsigned grid, int threads, size_t smem, const float* Q,
                                         const float* K, const float* V, int tokens, int heads, int64_t row_stride,
                                         int mode, float beta, const float* beta_seq, float tau_m, float v_th,
                                         float g_inh, int n_iter, float* O, float* A_out) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_rows_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
    }
    attention_rows_kernel<D><<<grid, threads, smem, st>>>(Q, K, V, tokens, heads, row_stride, mode, beta, beta_seq, tau_m, v_th,
                                                          g_inh, n_iter, O, A_out);
    return cudaSuccess;
}

// The same for head sizes 16 and 32 on packed pairs.  The kernel above is bound by the rate at
// which shared memory feeds registers (every thread reads all of K and V: 128 bytes per cycle and
// SM), so here a thread owns TWO query rows and every 16-byte piece of K or V it loads feeds four
// packed fmas.  K is staged transposed (Kt[c][j]) so that one piece holds column c of four
// consecutive keys, i.e. two (key j, key j+1) pairs whose dot products with q advance together;
// the V row of a key is consumed as (c, c+1) pairs.  Sums run in index order with one rounding
// per multiply-add.
template <int D>
__global__ void __launch_bounds__(64)
attention_product_packed_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                                int tokens, int heads, int64_t row_stride, float beta,
                                const float* __restrict__ beta_seq, int causal, float* __restrict__ O,
                                float* __restrict__ A_out) {
    extern __shared__ __align__(16) float sm[];
    const int tp = (tokens + 3) / 4 * 4 + 4;   // pitch of Kt: keys rounded up to four, plus four
    float* kt = sm;                            // [D][tp]
    float4* vs4 = reinterpret_cast<float4*>(sm + D * tp);  // [tokens][D]
    const int seq = blockIdx.x / heads, h = blockIdx.x % heads;
    if (beta_seq) beta = beta_seq[seq];   // one scale per sequence (a member's own beta)
    const size_t base = (size_t)seq * tokens * row_stride + (size_t)h * D;
    constexpr int D4 = D / 4;
    const int padc = tp - tokens;
    for (int e = threadIdx.x; e < D * padc; e += blockDim.x) kt[(e / padc) * tp + tokens + e % padc] = 0.0f;
    for (int e = threadIdx.x; e < tokens * D4; e += blockDim.x) {
        int tk = e / D4, c4 = e - tk * D4;
        const float4 kv = *reinterpret_cast<const float4*>(K + base + (size_t)tk * row_stride + c4 * 4);
        kt[(4 * c4) * tp + tk] = kv.x;
        kt[(4 * c4 + 1) * tp + tk] = kv.y;
        kt[(4 * c4 + 2) * tp + tk] = kv.z;
        kt[(4 * c4 + 3) * tp + tk] = kv.w;
        vs4[e] = *reinterpret_cast<const float4*>(V + base + (size_t)tk * row_stride + c4 * 4);
    }
    __syncthreads();
    const int i0 = 2 * threadIdx.x;
    if (i0 >= tokens) return;
    const bool two = i0 + 1 < tokens;
    const int i1 = two ? i0 + 1 : i0;
    f32x2 qa[D], qb[D], acca[D / 2], accb[D / 2];
#pragma unroll
    for (int c4 = 0; c4 < D4; ++c4) {
        const float4 va = *reinterpret_cast<const float4*>(Q + base + (size_t)i0 * row_stride + c4 * 4);
        const float4 vb = *reinterpret_cast<const float4*>(Q + base + (size_t)i1 * row_stride + c4 * 4);
        qa[4 * c4] = pk2(va.x, va.x); qa[4 * c4 + 1] = pk2(va.y, va.y);
        qa[4 * c4 + 2] = pk2(va.z, va.z); qa[4 * c4 + 3] = pk2(va.w, va.w);
        qb[4 * c4] = pk2(vb.x, vb.x); qb[4 * c4 + 1] = pk2(vb.y, vb.y);
        qb[4 * c4 + 2] = pk2(vb.z, vb.z); qb[4 * c4 + 3] = pk2(vb.w, vb.w);
    }
#pragma unroll
    for (int c = 0; c < D / 2; ++c) acca[c] = accb[c] = 0ull;
    const f32x2 beta2 = pk2(beta, beta);
    float* arow_a = A_out ? A_out + (((size_t)seq * heads + h) * tokens + i0) * tokens : nullptr;
    float* arow_b = A_out ? A_out + (((size_t)seq * heads + h) * tokens + i1) * tokens : nullptr;
    // with the causal mask the keys after this thread's second row contribute nothing: they are
    // skipped, except that the weight rows, when asked for, are written in full
    const int j_end = (causal && !A_out) ? min(tokens, i1 + 1) : tokens;
    for (int j0 = 0; j0 < j_end; j0 += 4) {
        f32x2 sa01 = 0ull, sa23 = 0ull, sb01 = 0ull, sb23 = 0ull;
#pragma unroll
        for (int c = 0; c < D; ++c) {
            const ulonglong2 kv = *reinterpret_cast<const ulonglong2*>(kt + c * tp + j0);
            sa01 = fma2(qa[c], kv.x, sa01);
            sa23 = fma2(qa[c], kv.y, sa23);
            sb01 = fma2(qb[c], kv.x, sb01);
            sb23 = fma2(qb[c], kv.y, sb23);
        }
        float ha[4], hb[4];
        upk2(mul2(beta2, sa01), ha[0], ha[1]);
        upk2(mul2(beta2, sa23), ha[2], ha[3]);
        upk2(mul2(beta2, sb01), hb[0], hb[1]);
        upk2(mul2(beta2, sb23), hb[2], hb[3]);
        if (causal) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (j0 + u > i0) ha[u] = 0.0f;
                if (j0 + u > i1) hb[u] = 0.0f;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (j0 + u < tokens) {
                if (arow_a) {
                    arow_a[j0 + u] = ha[u];
                    if (two) arow_b[j0 + u] = hb[u];
                }
                const f32x2 ha2 = pk2(ha[u], ha[u]), hb2 = pk2(hb[u], hb[u]);
                const ulonglong2* vrow = reinterpret_cast<const ulonglong2*>(vs4 + (j0 + u) * D4);
#pragma unroll
                for (int c4 = 0; c4 < D4; ++c4) {
                    const ulonglong2 vv = vrow[c4];
                    acca[2 * c4] = fma2(ha2, vv.x, acca[2 * c4]);
                    acca[2 * c4 + 1] = fma2(ha2, vv.y, acca[2 * c4 + 1]);
                    accb[2 * c4] = fma2(hb2, vv.x, accb[2 * c4]);
                    accb[2 * c4 + 1] = fma2(hb2, vv.y, accb[2 * c4 + 1]);
                }
            }
        }
    }
#pragma unroll
    for (int c4 = 0; c4 < D4; ++c4) {
        ulonglong2 o;
        o.x = acca[2 * c4];
        o.y = acca[2 * c4 + 1];
        *reinterpret_cast<ulonglong2*>(O + base + (size_t)i0 * row_stride + c4 * 4) = o;
        if (two) {
            o.x = accb[2 * c4];
            o.y = accb[2 * c4 + 1];
            *reinterpret_cast<ulonglong2*>(O + base + (size_t)i1 * row_stride + c4 * 4) = o;
        }
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

// The same statistics for groups of `cnt` contiguous values with l == 1, cnt a multiple of 4 and
// 16-byte aligned groups: LPG lanes (a power of two <= 32) share a group, every lane keeps its
// 16-byte pieces in registers between the statistics and the normalisation, so x is read once.
// A lane group walks over GPT consecutive groups with all their loads issued first: a short group
// (64 values are one 16-byte piece per lane) would otherwise leave one load in flight per thread.
template <int LPG, int NV, int GPT>
__global__ void __launch_bounds__(256)
group_norm_regs_kernel(const float* __restrict__ x, int64_t n_groups_total, int groups, int cnt,
                       const float* __restrict__ weight, const float* __restrict__ bias, float eps,
                       float* __restrict__ out) {
    constexpr int GPB = 256 / LPG;
    const int sub = threadIdx.x / LPG, lane = threadIdx.x % LPG;
    const int64_t g0 = ((int64_t)blockIdx.x * GPB + sub) * GPT;
    const int n4 = cnt / 4;
    float4 v[GPT][NV];
    float sum[GPT], sumsq[GPT];
#pragma unroll
    for (int t = 0; t < GPT; ++t) {
        int64_t gidx = g0 + t;
        if (gidx >= n_groups_total) gidx = n_groups_total - 1;   // keep the lanes of a warp together for the shuffles
        const float4* xg = reinterpret_cast<const float4*>(x + (size_t)gidx * cnt);
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            const int j = lane + u * LPG;
            v[t][u] = j < n4 ? xg[j] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
#pragma unroll
    for (int t = 0; t < GPT; ++t) {
        sum[t] = 0.0f;
        sumsq[t] = 0.0f;
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            sum[t] += (v[t][u].x + v[t][u].y) + (v[t][u].z + v[t][u].w);
            sumsq[t] = fmaf(v[t][u].x, v[t][u].x, fmaf(v[t][u].y, v[t][u].y,
                            fmaf(v[t][u].z, v[t][u].z, fmaf(v[t][u].w, v[t][u].w, sumsq[t]))));
        }
#pragma unroll
        for (int off = LPG / 2; off > 0; off >>= 1) {
            sum[t] += __shfl_xor_sync(0xffffffffu, sum[t], off);
            sumsq[t] += __shfl_xor_sync(0xffffffffu, sumsq[t], off);
        }
    }
    // the group's position in its row, once per thread (a 64-bit remainder per group would cost as much
    // as the normalisation of a short group)
    int g = n_groups_total <= 0xffffffffll ? (int)((uint32_t)g0 % (uint32_t)groups) : (int)(g0 % groups);
#pragma unroll
    for (int t = 0; t < GPT; ++t, g = g + 1 == groups ? 0 : g + 1) {
        const int64_t gidx = g0 + t;
        if (gidx >= n_groups_total) break;
        const float mean = __fdiv_rn(sum[t], (float)cnt);
        const float var = __fsub_rn(__fdiv_rn(sumsq[t], (float)cnt), __fmul_rn(mean, mean));
        const float sd = __fsqrt_rn(__fadd_rn(var, eps));
        const float4* w4 = reinterpret_cast<const float4*>(weight + (size_t)g * cnt);
        const float4* b4 = reinterpret_cast<const float4*>(bias + (size_t)g * cnt);
        float4* og = reinterpret_cast<float4*>(out + (size_t)gidx * cnt);
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            const int j = lane + u * LPG;
            if (j < n4) {
                const float4 w = w4[j], b = b4[j];
                float4 o;
                o.x = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(v[t][u].x, mean), sd), w.x), b.x);
                o.y = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(v[t][u].y, mean), sd), w.y), b.y);
                o.z = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(v[t][u].z, mean), sd), w.z), b.z);
                o.w = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(v[t][u].w, mean), sd), w.w), b.w);
                og[j] = o;
            }
        }
    }
}

// Launches the register-cached variant when the shape allows it; false = use the general kernel.
static bool launch_group_norm_regs(cudaStream_t st, const float* x, int64_t total, int groups, int cnt,
                                   const float* weight, const float* bias, float eps, float* out) {
    if (cnt % 4 != 0 || cnt > 1024) return false;
    if ((((uintptr_t)x | (uintptr_t)out | (uintptr_t)weight | (uintptr_t)bias) & 15u) != 0) return false;
    const int n4 = cnt / 4;
#define HSES_GN(LPG, NV, GPT)                                                                                    \
    group_norm_regs_kernel<LPG, NV, GPT><<<(unsigned)((total + (256 / LPG) * GPT - 1) / ((256 / LPG) * GPT)), 256, 0, \
                                           st>>>(x, total, groups, cnt, weight, bias, eps, out)
    if (n4 <= 4) HSES_GN(4, 1, 4);
    else if (n4 <= 8) HSES_GN(8, 1, 4);
    else if (n4 <= 16) HSES_GN(16, 1, 4);
    else if (n4 <= 32) HSES_GN(32, 1, 4);
    else if (n4 <= 64) HSES_GN(32, 2, 2);
    else if (n4 <= 128) HSES_GN(32, 4, 1);
    else HSES_GN(32, 8, 1);
#undef HSES_GN
    return true;
}

// out = x + (prev - x) * coef with prev = the previous row (row 0: state), 0 at new starts.
// VEC: 4 (rows and pointers 16-byte aligned, c a multiple of 4) or 1.
template <int VEC>
__global__ void token_shift_mix_kernel(const float* __restrict__ x, int T, int c, const float* __restrict__ state,
                                       const uint8_t* __restrict__ new_starts, const float* __restrict__ coef,
                                       float* __restrict__ out) {
    int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (i >= (int64_t)T * c) return;
    int t = (int)(i / c), j = (int)(i - (int64_t)t * c);
    const bool zero = new_starts && new_starts[t];
    if (VEC == 4) {
        float4 prev = t == 0 ? *reinterpret_cast<const float4*>(state + j) : *reinterpret_cast<const float4*>(x + i - c);
        if (zero) prev = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 xv = *reinterpret_cast<const float4*>(x + i), cf = *reinterpret_cast<const float4*>(coef + j);
        float4 o;
        o.x = __fadd_rn(xv.x, __fmul_rn(__fsub_rn(prev.x, xv.x), cf.x));
        o.y = __fadd_rn(xv.y, __fmul_rn(__fsub_rn(prev.y, xv.y), cf.y));
        o.z = __fadd_rn(xv.z, __fmul_rn(__fsub_rn(prev.z, xv.z), cf.z));
        o.w = __fadd_rn(xv.w, __fmul_rn(__fsub_rn(prev.w, xv.w), cf.w));
        *reinterpret_cast<float4*>(out + i) = o;
    } else {
        float prev = t == 0 ? state[j] : x[i - c];
        if (zero) prev = 0.0f;
        float xv = x[i];
        out[i] = __fadd_rn(xv, __fmul_rn(__fsub_rn(prev, xv), coef[j]));
    }
}

// The same for several coefficient vectors at once (TimeMixing mixes one x six ways, llm.rs:381-392):
// x and its previous row are read once, out[m] = x + (prev - x) * coef[m].  16-byte accesses.
constexpr int kMaxMixes = 8;
struct MixPtrs {
    const float* coef[kMaxMixes];
    float* out[kMaxMixes];
};
__global__ void token_shift_mix_multi_kernel(const float* __restrict__ x, int T, int c, const float* __restrict__ state,
                                             const uint8_t* __restrict__ new_starts, int n_mix, MixPtrs p) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= (int64_t)T * c) return;
    const int t = (int)(i / c), j = (int)(i - (int64_t)t * c);
    float4 prev = t == 0 ? *reinterpret_cast<const float4*>(state + j) : *reinterpret_cast<const float4*>(x + i - c);
    if (new_starts && new_starts[t]) prev = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 xv = *reinterpret_cast<const float4*>(x + i);
    const float4 d = make_float4(__fsub_rn(prev.x, xv.x), __fsub_rn(prev.y, xv.y), __fsub_rn(prev.z, xv.z),
                                 __fsub_rn(prev.w, xv.w));
#pragma unroll
    for (int m = 0; m < kMaxMixes; ++m) {
        if (m >= n_mix) break;
        const float4 cf = __ldg(reinterpret_cast<const float4*>(p.coef[m] + j));
        __stcs(reinterpret_cast<float4*>(p.out[m] + i),
               make_float4(__fadd_rn(xv.x, __fmul_rn(d.x, cf.x)), __fadd_rn(xv.y, __fmul_rn(d.y, cf.y)),
                           __fadd_rn(xv.z, __fmul_rn(d.z, cf.z)), __fadd_rn(xv.w, __fmul_rn(d.w, cf.w))));
    }
}

// ---- element-wise work of TimeMixing::forward around the recurrence (llm.rs:396-440 before it,
// 462-472 after it), one warp per (row, head): the head's S values sit S / 32 per lane, the two sums
// over a head (the norm of kk, the bonus) are warp reductions.
//   before: w    = -softplus(-(w0 + w_lin)) - 0.5                                   (llm.rs:400)
//           v    = v_raw                         in layer 0 (v_lin == NULL), else
//                  v_raw + (v_first - v_raw) * sigmoid(v0 + v_lin)                  (llm.rs:405-415)
//           a    = sigmoid(a0 + a_lin)
//           kk   = (k_raw * k_k) / max(|k_raw * k_k|_2 over the head, 1e-12)        (llm.rs:426-433)
//           k    = k_raw * (k_a * (a - 1) + 1)                                      (llm.rs:437)
//           outputs w, v, k, -kk and kk * a: the recurrence's decay, value, key, a and b inputs
//   after:  y = (y_norm + (sum over the head of r * k * r_k) * v) * gate            (llm.rs:462-472)
__device__ __forceinline__ float sigmoid_f(float z) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-z))); }

// PER consecutive floats of a lane as one 4-, 8- or 16-byte access
template <int PER>
__device__ __forceinline__ void ld_per(const float* __restrict__ p, float (&v)[PER]) {
    if (PER == 4) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(p));
        v[0] = q.x; v[1] = q.y; v[2 % PER] = q.z; v[3 % PER] = q.w;
    } else if (PER == 2) {
        const float2 q = __ldg(reinterpret_cast<const float2*>(p));
        v[0] = q.x; v[1 % PER] = q.y;
    } else {
        v[0] = __ldg(p);
    }
}
template <int PER>
__device__ __forceinline__ void st_per(float* __restrict__ p, const float (&v)[PER]) {
    if (PER == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2 % PER], v[3 % PER]);
    else if (PER == 2) *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1 % PER]);
    else p[0] = v[0];
}

template <int PER>
__global__ void __launch_bounds__(256)
rwkv_mix_prepare_kernel(int64_t heads_total, int H, const float* __restrict__ w_lin, const float* __restrict__ v_raw,
                        const float* __restrict__ v_lin, const float* __restrict__ v_first,
                        const float* __restrict__ a_lin, const float* __restrict__ k_raw,
                        const float* __restrict__ w0, const float* __restrict__ v0, const float* __restrict__ a0,
                        const float* __restrict__ k_k, const float* __restrict__ k_a, float* __restrict__ w_out,
                        float* __restrict__ v_out, float* __restrict__ k_out, float* __restrict__ nkk_out,
                        float* __restrict__ kka_out) {
    constexpr int S = 32 * PER;
    const int64_t wi = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wi >= heads_total) return;   // warp-uniform
    const int lane = threadIdx.x & 31;
    const int h = (int)(wi % H);
    const int64_t e0 = wi * S + lane * PER;   // (row * H + h) * S + the lane's PER consecutive values
    const int c0 = h * S + lane * PER;
    float wl[PER], vr[PER], al[PER], kr[PER], p_w0[PER], p_a0[PER], p_kk[PER], p_ka[PER];
    ld_per<PER>(w_lin + e0, wl); ld_per<PER>(v_raw + e0, vr); ld_per<PER>(a_lin + e0, al); ld_per<PER>(k_raw + e0, kr);
    ld_per<PER>(w0 + c0, p_w0); ld_per<PER>(a0 + c0, p_a0); ld_per<PER>(k_k + c0, p_kk); ld_per<PER>(k_a + c0, p_ka);
    float vl[PER], vf[PER], p_v0[PER];
    if (v_lin != nullptr) {
        ld_per<PER>(v_lin + e0, vl); ld_per<PER>(v_first + e0, vf); ld_per<PER>(v0 + c0, p_v0);
    }
    float kk[PER], a[PER], wo[PER], vo[PER], ko[PER];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const float iw = __fadd_rn(p_w0[i], wl[i]);
        // softplus(-iw) = max(-iw, 0) + log1p(exp(-|iw|))
        const float sp = __fadd_rn(fmaxf(-iw, 0.0f), log1pf(expf(-fabsf(iw))));
        wo[i] = __fsub_rn(-sp, 0.5f);
        float v = vr[i];
        if (v_lin != nullptr) {
            const float sg = sigmoid_f(__fadd_rn(p_v0[i], vl[i]));
            v = __fadd_rn(vr[i], __fmul_rn(__fsub_rn(vf[i], vr[i]), sg));
        }
        vo[i] = v;
        a[i] = sigmoid_f(__fadd_rn(p_a0[i], al[i]));
        kk[i] = __fmul_rn(kr[i], p_kk[i]);
        ss = fmaf(kk[i], kk[i], ss);
        ko[i] = __fmul_rn(kr[i], __fadd_rn(__fmul_rn(p_ka[i], __fsub_rn(a[i], 1.0f)), 1.0f));
    }
    st_per<PER>(w_out + e0, wo); st_per<PER>(v_out + e0, vo); st_per<PER>(k_out + e0, ko);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float nrm = fmaxf(sqrtf(ss), 1e-12f);
    float nk[PER], ka[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const float q = __fdiv_rn(kk[i], nrm);
        nk[i] = -q;
        ka[i] = __fmul_rn(q, a[i]);
    }
    st_per<PER>(nkk_out + e0, nk); st_per<PER>(kka_out + e0, ka);
}

template <int PER>
__global__ void __launch_bounds__(256)
rwkv_mix_finish_kernel(int64_t heads_total, int H, const float* __restrict__ y_norm, const float* __restrict__ r,
                       const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ gate,
                       const float* __restrict__ r_k, float* __restrict__ out) {
    constexpr int S = 32 * PER;
    const int64_t wi = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wi >= heads_total) return;
    const int lane = threadIdx.x & 31;
    const int h = (int)(wi % H);
    const int64_t e0 = wi * S + lane * PER;
    float rv[PER], kv[PER], rk[PER], yn[PER], vv[PER], gv[PER], o[PER];
    ld_per<PER>(r + e0, rv); ld_per<PER>(k + e0, kv); ld_per<PER>(r_k + h * S + lane * PER, rk);
    ld_per<PER>(y_norm + e0, yn); ld_per<PER>(v + e0, vv); ld_per<PER>(gate + e0, gv);
    float bonus = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) bonus = __fadd_rn(bonus, __fmul_rn(__fmul_rn(rv[i], kv[i]), rk[i]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) bonus += __shfl_xor_sync(0xffffffffu, bonus, off);
#pragma unroll
    for (int i = 0; i < PER; ++i) o[i] = __fmul_rn(__fadd_rn(yn[i], __fmul_rn(bonus, vv[i])), gv[i]);
    st_per<PER>(out + e0, o);
}

struct ReluSquareOp {
    __device__ __forceinline__ float operator()(float x) const {
        float v = x > 0.0f ? x : 0.0f;
        return __fmul_rn(v, v);
    }
};
// rate_encode, snn_transformer.rs:109-116: sigmoid(gain * p / (1 + |p|))
struct RateEncodeOp {
    float gain;
    __device__ __forceinline__ float operator()(float p) const {
        float ss = __fdiv_rn(p, __fadd_rn(fabsf(p), 1.0f));
        return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-__fmul_rn(ss, gain))));
    }
};
// out[i] = op(x[i]): one 16-byte piece per thread when VEC4 (aligned pointers), the n % 4 tail
// one value per thread
template <bool VEC4, class Op>
__global__ void map_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ out, Op op) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (VEC4) {
        const int64_t n4 = n / 4;
        if (i < n4) {
            const float4 v = reinterpret_cast<const float4*>(x)[i];
            reinterpret_cast<float4*>(out)[i] = make_float4(op(v.x), op(v.y), op(v.z), op(v.w));
            return;
        }
        i = n4 * 4 + (i - n4);
    }
    if (i < n) out[i] = op(x[i]);
}
template <class Op>
static void launch_map(cudaStream_t st, const float* x, int64_t n, float* out, Op op) {
    if (((((uintptr_t)x | (uintptr_t)out) & 15u) == 0) && n >= 4) {
        int64_t work = n / 4 + n % 4;
        map_kernel<true, Op><<<(unsigned)((work + 255) / 256), 256, 0, st>>>(x, n, out, op);
    } else {
        map_kernel<false, Op><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, n, out, op);
    }
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
    HSES_REQUIRE((((uintptr_t)r | (uintptr_t)w | (uintptr_t)k | (uintptr_t)v | (uintptr_t)a | (uintptr_t)b |
                   (uintptr_t)out) & 7u) == 0, "r, w, k, v, a, b and out must be 8-byte aligned");
    HSES_KERNEL(ctx, as_stream(stream), "wkv7");
    unsigned grid = (unsigned)(n_seq * H);
    if (S == 64)
        wkv7_kernel<64><<<grid, 32, 0, as_stream(stream)>>>(r, w, k, v, a, b, new_starts, T, H, state, out);
    else
        wkv7_kernel<32><<<grid, 16, 0, as_stream(stream)>>>(r, w, k, v, a, b, new_starts, T, H, state, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_spiking_attention(hses_ctx* ctx, hses_stream stream, const float* Q, const float* K, const float* V,
                           int64_t n_seq, int32_t tokens, int32_t heads, int32_t head_dim, int64_t row_stride,
                           int32_t mode, float beta, const float* beta_per_seq, float tau_m, float v_th, float g_inh,
                           int32_t n_iter, float* O, float* A_out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n_seq >= 0 && tokens >= 1 && tokens <= kMaxTokens, "tokens must be in 1..128");
    HSES_REQUIRE(heads >= 1 && head_dim >= 1 && head_dim <= kMaxHeadDim, "head_dim must be in 1..64");
    HSES_REQUIRE(row_stride >= (int64_t)heads * head_dim, "row stride smaller than heads*head_dim");
    HSES_REQUIRE(mode >= 0 && mode <= 3, "unknown mode");
    HSES_REQUIRE(mode == 0 || mode == 3 || (tau_m != 0.0f && n_iter >= 1), "bad LIF parameters");
    const int causal = mode == 3 ? 1 : 0;
    const bool product = mode == 0 || mode == 3;
    HSES_REQUIRE(n_seq * heads < (1ll << 31), "too many (sequence, head) pairs");
    if (n_seq == 0) return HSES_OK;
    HSES_REQUIRE(Q && K && V && O, "NULL pointer");
    int threads = (tokens + 31) / 32 * 32;
    size_t smem = (size_t)2 * tokens * head_dim * sizeof(float);
    HSES_KERNEL(ctx, as_stream(stream), "spiking_attention");
    const bool aligned = ((((uintptr_t)Q | (uintptr_t)K | (uintptr_t)V | (uintptr_t)O) & 15u) == 0) && row_stride % 4 == 0;
    if (product && aligned && (head_dim == 16 || head_dim == 32 || head_dim == 64)) {
        unsigned grid = (unsigned)(n_seq * heads);
        cudaStream_t st = as_stream(stream);
        const int threads2 = ((tokens + 1) / 2 + 31) / 32 * 32;   // two query rows per thread
        const size_t smem_packed = ((size_t)head_dim * ((tokens + 3) / 4 * 4 + 4) + (size_t)tokens * head_dim) * sizeof(float);
        if (head_dim == 16)
            attention_product_packed_kernel<16><<<grid, threads2, smem_packed, st>>>(Q, K, V, tokens, heads, row_stride,
                                                                                     beta, beta_per_seq, causal, O, A_out);
        else if (head_dim == 32)
            attention_product_packed_kernel<32><<<grid, threads2, smem_packed, st>>>(Q, K, V, tokens, heads, row_stride,
                                                                                     beta, beta_per_seq, causal, O, A_out);
        else {
            // up to 64 KB for 128 tokens x 64 values: above the 48 KB a kernel gets without opting in
            if (smem > 48 * 1024)
                HSES_CUDA(cudaFuncSetAttribute(attention_product_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)smem));
            attention_product_kernel<64><<<grid, threads, smem, st>>>(Q, K, V, tokens, heads, row_stride, beta, beta_per_seq,
                                                                      causal, O, A_out);
        }
        HSES_LAUNCH_CHECK();
        return HSES_OK;
    }
    const size_t smem_rows = ((size_t)2 * tokens * head_dim + (size_t)(mode == 1 ? 3 : 2) * tokens * (tokens + 1)) *
                             sizeof(float);
    if (!product && aligned && (head_dim == 16 || head_dim == 32 || head_dim == 64) && smem_rows <= 200 * 1024) {
        unsigned grid = (unsigned)(n_seq * heads);
        cudaStream_t st = as_stream(stream);
        cudaError_t e;
        if (head_dim == 16)
            e = launch_attention_rows<16>(st, grid, threads, smem_rows, Q, K, V, tokens, heads, row_stride, mode, beta, beta_per_seq,
                                          tau_m, v_th, g_inh, n_iter, O, A_out);
        else if (head_dim == 32)
            e = launch_attention_rows<32>(st, grid, threads, smem_rows, Q, K, V, tokens, heads, row_stride, mode, beta, beta_per_seq,
                                          tau_m, v_th, g_inh, n_iter, O, A_out);
        else
            e = launch_attention_rows<64>(st, grid, threads, smem_rows, Q, K, V, tokens, heads, row_stride, mode, beta, beta_per_seq,
                                          tau_m, v_th, g_inh, n_iter, O, A_out);
        HSES_REQUIRE(e == cudaSuccess, "cudaFuncSetAttribute failed");
        HSES_LAUNCH_CHECK();
        return HSES_OK;
    }
    if (smem > 48 * 1024)
        HSES_CUDA(cudaFuncSetAttribute(spiking_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    spiking_attention_kernel<<<(unsigned)(n_seq * heads), threads, smem, as_stream(stream)>>>(
        Q, K, V, tokens, heads, head_dim, row_stride, mode, beta, beta_per_seq, tau_m, v_th, g_inh, n_iter, O, A_out);
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
    if (launch_group_norm_regs(as_stream(stream), x, rows, 1, c, weight, bias, eps, out)) {
        HSES_LAUNCH_CHECK();
        return HSES_OK;
    }
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
    if (l == 1 && launch_group_norm_regs(as_stream(stream), x, total, groups, c / groups, weight, bias, eps, out)) {
        HSES_LAUNCH_CHECK();
        return HSES_OK;
    }
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
    const bool vec4 = c % 4 == 0 &&
                      ((((uintptr_t)x | (uintptr_t)out | (uintptr_t)state | (uintptr_t)coef) & 15u) == 0);
    if (vec4)
        token_shift_mix_kernel<4><<<(unsigned)((n / 4 + 255) / 256), 256, 0, as_stream(stream)>>>(x, T, c, state,
                                                                                                 new_starts, coef, out);
    else
        token_shift_mix_kernel<1><<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(x, T, c, state,
                                                                                             new_starts, coef, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_token_shift_mix_multi(hses_ctx* ctx, hses_stream stream, const float* x, int32_t T, int32_t c,
                               const float* state, const uint8_t* new_starts, int32_t n_mix, const float* const* coefs,
                               float* const* outs) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(T >= 0 && c >= 1 && n_mix >= 1 && n_mix <= kMaxMixes, "bad shape (at most 8 mixes)");
    if (T == 0) return HSES_OK;
    HSES_REQUIRE(x != nullptr && state != nullptr && coefs != nullptr && outs != nullptr, "NULL pointer");
    MixPtrs p{};
    uintptr_t bits = (uintptr_t)x | (uintptr_t)state;
    for (int m = 0; m < n_mix; ++m) {
        HSES_REQUIRE(coefs[m] != nullptr && outs[m] != nullptr && outs[m] != x, "NULL or aliasing pointer");
        p.coef[m] = coefs[m];
        p.out[m] = outs[m];
        bits |= (uintptr_t)coefs[m] | (uintptr_t)outs[m];
    }
    if (c % 4 != 0 || (bits & 15u) != 0) {   // no 16-byte accesses: one mix at a time
        for (int m = 0; m < n_mix; ++m) {
            int rc = hses_token_shift_mix(ctx, stream, x, T, c, state, new_starts, coefs[m], outs[m]);
            if (rc != HSES_OK) return rc;
        }
        return HSES_OK;
    }
    const int64_t n = (int64_t)T * c;
    HSES_KERNEL(ctx, as_stream(stream), "token_shift_mix");
    token_shift_mix_multi_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, as_stream(stream)>>>(x, T, c, state, new_starts,
                                                                                                 n_mix, p);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_rwkv_mix_prepare(hses_ctx* ctx, hses_stream stream, int64_t rows, int32_t H, int32_t S, const float* w_lin,
                          const float* v_raw, const float* v_lin, const float* v_first, const float* a_lin,
                          const float* k_raw, const float* w0, const float* v0, const float* a0, const float* k_k,
                          const float* k_a, float* w_out, float* v_out, float* k_out, float* nkk_out, float* kka_out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(rows >= 0 && H >= 1 && (S == 32 || S == 64 || S == 128), "head size must be 32, 64 or 128");
    if (rows == 0) return HSES_OK;
    HSES_REQUIRE(w_lin && v_raw && a_lin && k_raw && w0 && a0 && k_k && k_a && w_out && v_out && k_out && nkk_out && kka_out,
                 "NULL pointer");
    HSES_REQUIRE(v_lin == nullptr || (v0 != nullptr && v_first != nullptr), "v_lin needs v0 and v_first");
    {   // a lane reads and writes S / 32 consecutive floats at once
        uintptr_t bits = 0;
        for (const void* q : {(const void*)w_lin, (const void*)v_raw, (const void*)v_lin, (const void*)v_first,
                              (const void*)a_lin, (const void*)k_raw, (const void*)w0, (const void*)v0, (const void*)a0,
                              (const void*)k_k, (const void*)k_a, (const void*)w_out, (const void*)v_out,
                              (const void*)k_out, (const void*)nkk_out, (const void*)kka_out})
            bits |= (uintptr_t)q;
        HSES_REQUIRE((bits & 15u) == 0, "pointers must be 16-byte aligned");
    }
    const int64_t heads_total = rows * H;
    const unsigned grid = (unsigned)((heads_total + 7) / 8);
    HSES_KERNEL(ctx, as_stream(stream), "rwkv_mix_prepare");
#define HSES_MIXP(PER)                                                                                           \
    rwkv_mix_prepare_kernel<PER><<<grid, 256, 0, as_stream(stream)>>>(heads_total, H, w_lin, v_raw, v_lin, v_first, \
                                                                      a_lin, k_raw, w0, v0, a0, k_k, k_a, w_out,  \
                                                                      v_out, k_out, nkk_out, kka_out)
    if (S == 32) HSES_MIXP(1);
    else if (S == 64) HSES_MIXP(2);
    else HSES_MIXP(4);
#undef HSES_MIXP
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_rwkv_mix_finish(hses_ctx* ctx, hses_stream stream, int64_t rows, int32_t H, int32_t S, const float* y_norm,
                         const float* r, const float* k, const float* v, const float* gate, const float* r_k,
                         float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(rows >= 0 && H >= 1 && (S == 32 || S == 64 || S == 128), "head size must be 32, 64 or 128");
    if (rows == 0) return HSES_OK;
    HSES_REQUIRE(y_norm && r && k && v && gate && r_k && out, "NULL pointer");
    HSES_REQUIRE((((uintptr_t)y_norm | (uintptr_t)r | (uintptr_t)k | (uintptr_t)v | (uintptr_t)gate | (uintptr_t)r_k |
                   (uintptr_t)out) & 15u) == 0,
                 "pointers must be 16-byte aligned");
    const int64_t heads_total = rows * H;
    const unsigned grid = (unsigned)((heads_total + 7) / 8);
    HSES_KERNEL(ctx, as_stream(stream), "rwkv_mix_finish");
    if (S == 32) rwkv_mix_finish_kernel<1><<<grid, 256, 0, as_stream(stream)>>>(heads_total, H, y_norm, r, k, v, gate, r_k, out);
    else if (S == 64) rwkv_mix_finish_kernel<2><<<grid, 256, 0, as_stream(stream)>>>(heads_total, H, y_norm, r, k, v, gate, r_k, out);
    else rwkv_mix_finish_kernel<4><<<grid, 256, 0, as_stream(stream)>>>(heads_total, H, y_norm, r, k, v, gate, r_k, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_relu_square(hses_ctx* ctx, hses_stream stream, const float* x, int64_t n, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n >= 0, "n must be >= 0");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(x != nullptr && out != nullptr, "NULL pointer");
    HSES_KERNEL(ctx, as_stream(stream), "relu_square");
    launch_map(as_stream(stream), x, n, out, ReluSquareOp{});
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}


int hses_rate_encode(hses_ctx* ctx, hses_stream stream, const float* p, int64_t n, float gain, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n >= 0, "n must be >= 0");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(p != nullptr && out != nullptr, "NULL pointer");
    HSES_KERNEL(ctx, as_stream(stream), "rate_encode");
    launch_map(as_stream(stream), p, n, out, RateEncodeOp{gain});
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // extern "C"
