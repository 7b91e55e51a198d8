// HBM-bound elementwise kernels: Poisson encode, LIF scan, fitness, z-score,
// solver step.  All of them stream their operands once; rows are pitched.
#include <cuda_fp16.h>

#include "common.cuh"

namespace hses {

// ---------------------------------------------------------------------------
// Poisson encode (poisson_encode_fused_oxide.rs:36-105)
// ---------------------------------------------------------------------------
// The reference compares u = fl((k+1)/8388609) with p at every step, k being
// the top 23 bits of the xorshift32 output.  fl(n/8388609) is monotone in n,
// so "u < p" is "n < n*(p)" with n* the smallest n whose quotient reaches p.
// n* is found once per element with exact divisions; the T steps are then
// integer-only.
__device__ __forceinline__ uint32_t poisson_threshold(float p) {
    const float D = 8388609.0f;
    float guess = __fmul_rn(p, D);
    uint32_t c = guess >= 1.0f ? (guess < 8388609.0f ? (uint32_t)guess : 8388609u) : 1u;
    while (c > 1u && __fdiv_rn((float)(c - 1u), D) >= p) --c;
    while (c <= 8388608u && __fdiv_rn((float)c, D) < p) ++c;
    return c;
}

__device__ __forceinline__ uint32_t poisson_seed(uint32_t idx, uint32_t mix) {
    return 1000000007u * idx + mix + 0x9E3779B9u;
}

__device__ __forceinline__ uint32_t xs32(uint32_t x) {
    x ^= x << 13;
    x ^= x >> 17;
    x ^= x << 5;
    return x;
}

// out_half (optional, dense rows of in_dim values): the same spikes as fp16 0/1, the operand
// format of the tensor-core layer that follows, so that it need not convert them itself.
template <int VEC>
__global__ void poisson_kernel(const float* __restrict__ probs, int64_t batch, int in_dim,
                               int64_t stride, int T, uint32_t mix, float* __restrict__ out,
                               __half* __restrict__ out_half) {
    int64_t vec_per_row = in_dim / VEC;
    int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= batch * vec_per_row) return;
    int64_t row = v / vec_per_row;
    int col = (int)(v - row * vec_per_row) * VEC;
    size_t base = (size_t)row * stride + col;
    size_t out_step = (size_t)batch * stride;
    float p[VEC];
    if constexpr (VEC == 4) {
        float4 q = *reinterpret_cast<const float4*>(probs + base);
        p[0] = q.x; p[1] = q.y; p[2] = q.z; p[3] = q.w;
    } else {
        p[0] = probs[base];
    }
    uint32_t x[VEC], thr[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        x[i] = poisson_seed((uint32_t)(row * in_dim + col + i), mix);
        thr[i] = poisson_threshold(p[i]);
    }
    for (int t = 0; t < T; ++t) {
        float s[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            x[i] = xs32(x[i]);
            s[i] = ((x[i] >> 9) + 1u) < thr[i] ? 1.0f : 0.0f;
        }
        float* dst = out + (size_t)t * out_step + base;
        if constexpr (VEC == 4)
            __stcs(reinterpret_cast<float4*>(dst), make_float4(s[0], s[1], s[2], s[3]));
        else
            dst[0] = s[0];
        if (out_half) {
            __half* dh = out_half + ((size_t)t * batch + row) * in_dim + col;
            if constexpr (VEC == 4) {
                // 1.0 in fp16 is 0x3C00
                const uint32_t lo = (s[0] != 0.0f ? 0x3C00u : 0u) | (s[1] != 0.0f ? 0x3C000000u : 0u);
                const uint32_t hi = (s[2] != 0.0f ? 0x3C00u : 0u) | (s[3] != 0.0f ? 0x3C000000u : 0u);
                *reinterpret_cast<uint2*>(dh) = make_uint2(lo, hi);
            } else {
                dh[0] = __float2half_rn(s[0]);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// LIF scan (snn.rs:53-97, lif_fused_oxide.rs:37-70)
// ---------------------------------------------------------------------------
// cur and spikes may be the same buffer (the scan then runs in place: every element is read
// before the same thread overwrites it), so neither pointer is declared restrict.
template <int VEC>
__global__ void lif_scan_kernel(const float* cur, int T, int64_t n, int h,
                                int64_t stride, float* __restrict__ v_io, float leak, float v_th,
                                int reset, float* spikes) {
    int64_t vec_per_row = h / VEC;
    int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n * vec_per_row) return;
    int64_t row = e / vec_per_row;
    int col = (int)(e - row * vec_per_row) * VEC;
    size_t base = (size_t)row * stride + col;
    size_t step = (size_t)n * stride;
    float v[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = 0.0f;
    if (v_io) {
        if constexpr (VEC == 4) {
            float4 q = *reinterpret_cast<const float4*>(v_io + base);
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
            v[0] = v_io[base];
        }
    }
    for (int t = 0; t < T; ++t) {
        float c[VEC], s[VEC];
        const float* src = cur + (size_t)t * step + base;
        if constexpr (VEC == 4) {
            float4 q = __ldcs(reinterpret_cast<const float4*>(src));
            c[0] = q.x; c[1] = q.y; c[2] = q.z; c[3] = q.w;
        } else {
            c[0] = src[0];
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) s[i] = lif_update(v[i], c[i], leak, v_th, reset);
        float* dst = spikes + (size_t)t * step + base;
        if constexpr (VEC == 4)
            __stcs(reinterpret_cast<float4*>(dst), make_float4(s[0], s[1], s[2], s[3]));
        else
            dst[0] = s[0];
    }
    if (v_io) {
        if constexpr (VEC == 4)
            *reinterpret_cast<float4*>(v_io + base) = make_float4(v[0], v[1], v[2], v[3]);
        else
            v_io[base] = v[0];
    }
}

// ---------------------------------------------------------------------------
// mean over time (snn.rs:278): sum in step order, then one division
// ---------------------------------------------------------------------------
__global__ void time_mean_kernel(const float* __restrict__ x, int T, int64_t n, int h,
                                 int64_t stride, float* __restrict__ out, int64_t out_stride) {
    int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n * h) return;
    int64_t row = e / h;
    int col = (int)(e - row * h);
    size_t step = (size_t)n * stride;
    float s = 0.0f;
    for (int t = 0; t < T; ++t) s = __fadd_rn(s, x[(size_t)t * step + (size_t)row * stride + col]);
    out[(size_t)row * out_stride + col] = __fdiv_rn(s, (float)T);
}

// ---------------------------------------------------------------------------
// fitness (snn_mnist.rs:180-201) and per-member mean
// ---------------------------------------------------------------------------
__global__ void fitness_kernel(const float* __restrict__ logits, int64_t n, int classes,
                               const int32_t* __restrict__ labels, int reward,
                               float* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float* row = logits + (size_t)i * classes;
    float mx = row[0];
    int arg = 0;
    for (int c = 1; c < classes; ++c)
        if (row[c] > mx) { mx = row[c]; arg = c; }
    int label = labels[i];
    if (reward == HSES_REWARD_BINARY) {
        out[i] = arg == label ? 1.0f : 0.0f;
    } else {
        float sum = 0.0f;
        for (int c = 0; c < classes; ++c) sum = __fadd_rn(sum, expf(__fsub_rn(row[c], mx)));
        float picked = (label >= 0 && label < classes) ? row[label] : __int_as_float(0x7fc00000);
        out[i] = __fsub_rn(__fsub_rn(picked, mx), logf(sum));
    }
}

__global__ void member_mean_kernel(const float* __restrict__ x, int64_t n_pop, int bm,
                                   float* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pop) return;
    float s = 0.0f;
    for (int j = 0; j < bm; ++j) s = __fadd_rn(s, x[(size_t)i * bm + j]);
    out[i] = __fdiv_rn(s, (float)bm);
}

// ---------------------------------------------------------------------------
// z-score (noiser.rs:517-537): one block, fixed reduction order
// ---------------------------------------------------------------------------
constexpr int kZThreads = 1024;
__global__ void zscore_kernel(const float* __restrict__ raw, int64_t n, int group_size,
                              float* __restrict__ out, float* __restrict__ stats) {
    __shared__ float s_sum[kZThreads];
    __shared__ float s_sq[kZThreads];
    float a = 0.0f, b = 0.0f;
    for (int64_t i = threadIdx.x; i < n; i += kZThreads) {
        float x = raw[i];
        a = __fadd_rn(a, x);
        b = __fadd_rn(b, __fmul_rn(x, x));
    }
    s_sum[threadIdx.x] = a;
    s_sq[threadIdx.x] = b;
    __syncthreads();
    for (int stride = kZThreads / 2; stride > 0; stride >>= 1) {
        if (threadIdx.x < stride) {
            s_sum[threadIdx.x] = __fadd_rn(s_sum[threadIdx.x], s_sum[threadIdx.x + stride]);
            s_sq[threadIdx.x] = __fadd_rn(s_sq[threadIdx.x], s_sq[threadIdx.x + stride]);
        }
        __syncthreads();
    }
    float nf = (float)n;
    float mean = __fdiv_rn(s_sum[0], nf);
    float var = __fsub_rn(__fdiv_rn(s_sq[0], nf), __fmul_rn(mean, mean));
    float sd = __fsqrt_rn(__fadd_rn(var, 1e-5f));
    float inv = __fdiv_rn(1.0f, sd);
    if (threadIdx.x == 0 && stats) { stats[0] = mean; stats[1] = sd; }
    if (group_size == 0) {
        for (int64_t i = threadIdx.x; i < n; i += kZThreads)
            out[i] = __fmul_rn(__fadd_rn(raw[i], -mean), inv);
    } else {
        int64_t groups = n / group_size;
        for (int64_t g = threadIdx.x; g < groups; g += kZThreads) {
            float gs = 0.0f;
            for (int j = 0; j < group_size; ++j) gs = __fadd_rn(gs, raw[g * group_size + j]);
            float gmean = __fdiv_rn(gs, (float)group_size);
            for (int j = 0; j < group_size; ++j)
                out[g * group_size + j] = __fmul_rn(__fsub_rn(raw[g * group_size + j], gmean), inv);
        }
    }
}

// ---------------------------------------------------------------------------
// solver (noiser.rs:155-224)
// ---------------------------------------------------------------------------
constexpr int kSolverMulti = 12;
struct SolverConsts {
    int kind;
    float lr, beta1, beta2, eps, wd;
    float omb1, omb2, ibc1, ibc2, grad_scale;
};
__device__ __forceinline__ void solver_one(const SolverConsts& c, float& p, float g, float& m, float& v) {
    float gi = c.grad_scale == 1.0f ? g : __fmul_rn(g, c.grad_scale);
    if (c.kind == HSES_SGD) {
        p = __fsub_rn(p, __fmul_rn(gi, c.lr));
        return;
    }
    float mn = __fadd_rn(__fmul_rn(m, c.beta1), __fmul_rn(gi, c.omb1));
    float vn = __fadd_rn(__fmul_rn(v, c.beta2), __fmul_rn(__fmul_rn(gi, gi), c.omb2));
    m = mn;
    v = vn;
    float mh = __fmul_rn(mn, c.ibc1), vh = __fmul_rn(vn, c.ibc2);
    float denom = __fadd_rn(__fsqrt_rn(vh), c.eps);
    float term = __fmul_rn(__fdiv_rn(mh, denom), -c.lr);
    p = c.wd == 0.0f ? __fadd_rn(p, term) : __fadd_rn(__fadd_rn(p, term), __fmul_rn(p, c.wd));
}

// One 16-byte piece per thread (VEC4, all pointers 16-byte aligned); the last threads take the
// len % 4 tail one value each.
template <bool VEC4>
__global__ void solver_kernel(SolverConsts c, float* __restrict__ p, const float* __restrict__ g,
                              float* __restrict__ m, float* __restrict__ v, int64_t len) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool adam = c.kind != HSES_SGD;
    if (VEC4) {
        const int64_t n4 = len / 4;
        if (i < n4) {
            float4 pv = reinterpret_cast<float4*>(p)[i];
            const float4 gv = reinterpret_cast<const float4*>(g)[i];
            float4 mv = make_float4(0.f, 0.f, 0.f, 0.f), vv = mv;
            if (adam) {
                mv = reinterpret_cast<float4*>(m)[i];
                vv = reinterpret_cast<float4*>(v)[i];
            }
            solver_one(c, pv.x, gv.x, mv.x, vv.x);
            solver_one(c, pv.y, gv.y, mv.y, vv.y);
            solver_one(c, pv.z, gv.z, mv.z, vv.z);
            solver_one(c, pv.w, gv.w, mv.w, vv.w);
            reinterpret_cast<float4*>(p)[i] = pv;
            if (adam) {
                reinterpret_cast<float4*>(m)[i] = mv;
                reinterpret_cast<float4*>(v)[i] = vv;
            }
            return;
        }
        i = n4 * 4 + (i - n4);
    }
    if (i >= len) return;
    float mi = adam ? m[i] : 0.0f, vi = adam ? v[i] : 0.0f, pi = p[i];
    solver_one(c, pi, g[i], mi, vi);
    p[i] = pi;
    if (adam) {
        m[i] = mi;
        v[i] = vi;
    }
}

// The same step for up to kSolverMulti parameter tensors in one launch (the leaves of a small
// model): block b works on the tensor whose block range contains it; grads are one flat buffer
// in tensor order.
struct SolverMulti {
    int n;
    float* p[kSolverMulti];
    float* m[kSolverMulti];
    float* v[kSolverMulti];
    int64_t len[kSolverMulti];
    int64_t goff[kSolverMulti];
    int first_block[kSolverMulti + 1];
};
__global__ void solver_multi_kernel(SolverConsts c, SolverMulti d, const float* __restrict__ grads) {
    int t = 0;
    while (t + 1 < d.n && (int)blockIdx.x >= d.first_block[t + 1]) ++t;
    const int64_t i = (int64_t)(blockIdx.x - d.first_block[t]) * blockDim.x + threadIdx.x;
    if (i >= d.len[t] || d.p[t] == nullptr) return;
    const bool adam = c.kind != HSES_SGD;
    float mi = adam ? d.m[t][i] : 0.0f, vi = adam ? d.v[t][i] : 0.0f, pi = d.p[t][i];
    solver_one(c, pi, grads[d.goff[t] + i], mi, vi);
    d.p[t][i] = pi;
    if (adam) {
        d.m[t][i] = mi;
        d.v[t][i] = vi;
    }
}

// ---------------------------------------------------------------------------
// prng_normal_half (hyperscalees-kernels/src/lib.rs:26-143, wrapper oxide.rs:233-275): reference
// thread t owns out[128t, 128t+128); its four state words start at 1000000007*t + seed_j, every
// uniform advances three Tausworthe generators and one LCG, a Box-Muller pair keeps cos and sin.
// The integer stream and the uniforms are exact; ln/sqrt/cos/sin are the device functions.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t taus_step(uint32_t z, int s1, int s2, int s3, uint32_t m) {
    uint32_t b = ((z << s1) ^ z) >> s2;
    return ((z & m) << s3) ^ b;
}
__device__ __forceinline__ float taus_unit(uint32_t (&st)[4]) {
    st[0] = taus_step(st[0], 13, 19, 12, 4294967294u);
    st[1] = taus_step(st[1], 2, 25, 4, 4294967288u);
    st[2] = taus_step(st[2], 3, 11, 17, 4294967280u);
    st[3] = st[3] * 1664525u + 1013904223u;
    uint32_t r = st[0] ^ st[1] ^ st[2] ^ st[3];
    return __fdiv_rn(__fadd_rn((float)(r >> 9), 1.0f), 8388609.0f);
}
__global__ void prng_normal_half_kernel(float* __restrict__ out, int64_t total_threads, float mean, float sd,
                                        uint32_t s0, uint32_t s1, uint32_t s2, uint32_t s3) {
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= total_threads) return;
    const uint32_t s = 1000000007u * (uint32_t)t;
    uint32_t st[4] = {s + s0, s + s1, s + s2, s + s3};
    float4* dst = reinterpret_cast<float4*>(out + (size_t)t * 128);
#pragma unroll 2
    for (int i = 0; i < 32; ++i) {
        float z[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float u0 = taus_unit(st), u1 = taus_unit(st);
            const float coeff = __fmul_rn(__fsqrt_rn(__fmul_rn(logf(u0), -2.0f)), sd);
            const float arg = __fmul_rn(__fmul_rn(2.0f, 3.14159274f), u1);
            float sn, cs;
            sincosf(arg, &sn, &cs);
            z[2 * h] = __fadd_rn(__fmul_rn(cs, coeff), mean);
            z[2 * h + 1] = __fadd_rn(__fmul_rn(sn, coeff), mean);
        }
        dst[i] = make_float4(z[0], z[1], z[2], z[3]);
    }
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

// EggRollBS::convert_fitnesses (hyperscalees-noiser/src/eggroll_bs.rs:226-250), first pass: one
// warp per row of the (Q, G) score matrix writes std + 1e-8 with var = E[x^2] - E[x]^2.
__global__ void bs_row_std_kernel(const float* __restrict__ raw, int64_t q, int g, float* __restrict__ row_den) {
    int64_t r = (int64_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    int lane = threadIdx.x & 31;
    if (r >= q) return;
    const float* s = raw + (size_t)r * g;
    float sum = 0.0f, sumsq = 0.0f;
    for (int j = lane; j < g; j += 32) {
        float v = s[j];
        sum += v;
        sumsq = fmaf(v, v, sumsq);
    }
    for (int off = 16; off > 0; off >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, off);
        sumsq += __shfl_xor_sync(0xffffffffu, sumsq, off);
    }
    if (lane == 0) {
        float mean = __fdiv_rn(sum, (float)g);
        float var = __fsub_rn(__fdiv_rn(sumsq, (float)g), __fmul_rn(mean, mean));
        row_den[r] = __fadd_rn(__fsqrt_rn(var), 1e-8f);
    }
}

// Second pass: block j averages (S[q][j] - S[q][0]) / den[q] over the rows; columns 0 and 1 are zero.
__global__ void bs_column_mean_kernel(const float* __restrict__ raw, int64_t q, int g,
                                      const float* __restrict__ row_den, float* __restrict__ out) {
    __shared__ float red[32];
    int j = blockIdx.x;
    float acc = 0.0f;
    if (j >= 2) {
        for (int64_t r = threadIdx.x; r < q; r += blockDim.x) {
            const float* s = raw + (size_t)r * g;
            acc += __fdiv_rn(__fsub_rn(s[j], s[0]), row_den[r]);
        }
    }
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
        out[j] = __fdiv_rn(t, (float)q);
    }
}

__global__ void vector_mul_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                  float* __restrict__ out, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fmul_rn(a[i], b[i]);
}

}  // namespace hses

using namespace hses;

extern "C" {

int hses_prng_normal_half(hses_ctx* ctx, hses_stream stream, float* out, int64_t total_threads, float mean,
                          float std, const uint32_t seeds[4]) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(total_threads >= 0 && total_threads <= 0xffffffffll, "total_threads must fit 32 bits");
    HSES_REQUIRE(seeds != nullptr, "seeds is NULL");
    if (total_threads == 0) return HSES_OK;
    HSES_REQUIRE(out != nullptr && aligned16(out), "out must be a 16-byte aligned device pointer");
    HSES_KERNEL(ctx, as_stream(stream), "prng_normal_half");
    prng_normal_half_kernel<<<(unsigned)((total_threads + 127) / 128), 128, 0, as_stream(stream)>>>(
        out, total_threads, mean, std, seeds[0], seeds[1], seeds[2], seeds[3]);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_poisson_encode(hses_ctx* ctx, hses_stream stream, const float* probs, int64_t batch,
                        int32_t in_dim, int64_t row_stride, int32_t T, const uint32_t seeds[4],
                        float* out) {
    return hses_poisson_encode_dual(ctx, stream, probs, batch, in_dim, row_stride, T, seeds, out, nullptr);
}

int hses_poisson_encode_dual(hses_ctx* ctx, hses_stream stream, const float* probs, int64_t batch,
                             int32_t in_dim, int64_t row_stride, int32_t T, const uint32_t seeds[4],
                             float* out, void* out_half) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(out_half == nullptr || (in_dim % 4 == 0 && ((uintptr_t)out_half & 7u) == 0),
                 "the fp16 copy needs in_dim % 4 == 0 and an 8-byte aligned buffer");
    HSES_REQUIRE(batch >= 0 && in_dim >= 1 && row_stride >= in_dim, "bad shape");
    HSES_REQUIRE(T >= 1, "T must be >= 1");
    HSES_REQUIRE(seeds != nullptr, "seeds is NULL");
    HSES_REQUIRE((double)batch * in_dim < 4294967296.0,
                 "batch*in_dim must fit the 32-bit element index of the reference stream");
    if (batch == 0) return HSES_OK;
    HSES_REQUIRE(probs != nullptr && out != nullptr, "NULL pointer");
    uint32_t mix = seeds[0] ^ seeds[1] ^ seeds[2] ^ seeds[3];
    bool vec = (in_dim % 4 == 0) && (row_stride % 4 == 0) && aligned16(probs) && aligned16(out);
    if (vec) {
        int64_t total = batch * (in_dim / 4);
        HSES_KERNEL(ctx, as_stream(stream), "poisson_encode");
        poisson_kernel<4><<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(
            probs, batch, in_dim, row_stride, T, mix, out, reinterpret_cast<__half*>(out_half));
    } else {
        int64_t total = batch * in_dim;
        HSES_KERNEL(ctx, as_stream(stream), "poisson_encode");
        poisson_kernel<1><<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(
            probs, batch, in_dim, row_stride, T, mix, out, reinterpret_cast<__half*>(out_half));
    }
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_lif_scan(hses_ctx* ctx, hses_stream stream, const float* cur, int32_t T, int64_t n,
                  int32_t h, int64_t row_stride, float* v, float tau_m, float v_th,
                  int32_t reset_mode, float* spikes) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(T >= 1 && n >= 0 && h >= 1 && row_stride >= h, "bad shape");
    HSES_REQUIRE(reset_mode == HSES_RESET_HARD || reset_mode == HSES_RESET_SUBTRACT, "bad reset mode");
    HSES_REQUIRE(tau_m != 0.0f, "tau_m must be non-zero");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(cur != nullptr && spikes != nullptr, "NULL pointer");
    float leak = 1.0f / tau_m;
    bool vec = (h % 4 == 0) && (row_stride % 4 == 0) && aligned16(cur) && aligned16(spikes) &&
               (v == nullptr || aligned16(v));
    if (vec) {
        int64_t total = n * (h / 4);
        HSES_KERNEL(ctx, as_stream(stream), "lif_scan");
        lif_scan_kernel<4><<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(
            cur, T, n, h, row_stride, v, leak, v_th, reset_mode, spikes);
    } else {
        int64_t total = n * h;
        HSES_KERNEL(ctx, as_stream(stream), "lif_scan");
        lif_scan_kernel<1><<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(
            cur, T, n, h, row_stride, v, leak, v_th, reset_mode, spikes);
    }
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_time_mean(hses_ctx* ctx, hses_stream stream, const float* x, int32_t T, int64_t n,
                   int32_t h, int64_t row_stride, float* out, int64_t out_row_stride) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(T >= 1 && n >= 0 && h >= 1 && row_stride >= h && out_row_stride >= h, "bad shape");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(x != nullptr && out != nullptr, "NULL pointer");
    int64_t total = n * h;
    HSES_KERNEL(ctx, as_stream(stream), "time_mean");
    time_mean_kernel<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(
        x, T, n, h, row_stride, out, out_row_stride);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_fitness(hses_ctx* ctx, hses_stream stream, const float* logits, int64_t n, int32_t classes,
                 const int32_t* labels, int32_t reward, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n >= 0 && classes >= 1, "bad shape");
    HSES_REQUIRE(reward == HSES_REWARD_LOGLIK || reward == HSES_REWARD_BINARY, "bad reward");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(logits != nullptr && labels != nullptr && out != nullptr, "NULL pointer");
    HSES_KERNEL(ctx, as_stream(stream), "fitness");
    fitness_kernel<<<(unsigned)((n + 127) / 128), 128, 0, as_stream(stream)>>>(logits, n, classes,
                                                                             labels, reward, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_member_mean(hses_ctx* ctx, hses_stream stream, const float* per_sample, int64_t n_pop,
                     int32_t bm, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n_pop >= 0 && bm >= 1, "bad shape");
    if (n_pop == 0) return HSES_OK;
    HSES_REQUIRE(per_sample != nullptr && out != nullptr, "NULL pointer");
    HSES_KERNEL(ctx, as_stream(stream), "member_mean");
    member_mean_kernel<<<(unsigned)((n_pop + 127) / 128), 128, 0, as_stream(stream)>>>(per_sample,
                                                                                     n_pop, bm, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_convert_fitnesses(hses_ctx* ctx, hses_stream stream, const float* raw, int64_t n,
                           int32_t group_size, float* out, float* stats) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n >= 1, "n must be >= 1");
    HSES_REQUIRE(group_size >= 0, "group_size must be >= 0");
    HSES_REQUIRE(group_size == 0 || n % group_size == 0, "n must be a multiple of group_size");
    HSES_REQUIRE(raw != nullptr && out != nullptr, "NULL pointer");
    HSES_KERNEL(ctx, as_stream(stream), "zscore");
    zscore_kernel<<<1, kZThreads, 0, as_stream(stream)>>>(raw, n, group_size, out, stats);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_convert_fitnesses_bs(hses_ctx* ctx, hses_stream stream, const float* raw, int64_t n,
                              int32_t group_size, float* out, float* row_den) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(group_size >= 1 && n >= group_size && n % group_size == 0,
                 "n must be a positive multiple of group_size");
    HSES_REQUIRE(raw != nullptr && out != nullptr && row_den != nullptr, "NULL pointer");
    int64_t q = n / group_size;
    {
        HSES_KERNEL(ctx, as_stream(stream), "bs_row_std");
        bs_row_std_kernel<<<(unsigned)((q + 7) / 8), 256, 0, as_stream(stream)>>>(raw, q, group_size, row_den);
        HSES_LAUNCH_CHECK();
    }
    {
        HSES_KERNEL(ctx, as_stream(stream), "bs_column_mean");
        bs_column_mean_kernel<<<(unsigned)group_size, 256, 0, as_stream(stream)>>>(raw, q, group_size, row_den, out);
        HSES_LAUNCH_CHECK();
    }
    return HSES_OK;
}

int hses_vector_mul(hses_ctx* ctx, hses_stream stream, const float* a, const float* b, float* out, int64_t n) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n >= 0, "n must be >= 0");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(a != nullptr && b != nullptr && out != nullptr, "NULL pointer");
    HSES_KERNEL(ctx, as_stream(stream), "vector_mul");
    vector_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(a, b, out, n);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // extern "C"

namespace hses {
// One solver step over several parameter tensors whose gradients sit back to back in `grads`
// (tensors with a NULL parameter pointer are skipped but still take their place in `grads`).
int solver_step_multi(hses_ctx* ctx, cudaStream_t st, const hses_solver* solver, int32_t step, int n_tensors,
                      float* const* params, float* const* m_bufs, float* const* v_bufs, const int64_t* lens,
                      const float* grads) {
    HSES_REQUIRE(solver->kind == HSES_SGD || solver->kind == HSES_ADAM || solver->kind == HSES_ADAMW,
                 "unknown solver kind");
    const bool moments = solver->kind != HSES_SGD;
    HSES_REQUIRE(!moments || step >= 1, "step is the counter after the increment (>= 1)");
    SolverConsts c{};
    c.kind = solver->kind;
    c.lr = solver->lr;
    c.grad_scale = 1.0f;
    if (moments) {
        float t = (float)step;
        c.beta1 = solver->beta1;
        c.beta2 = solver->beta2;
        c.eps = solver->eps;
        c.wd = solver->kind == HSES_ADAMW ? solver->weight_decay : 0.0f;
        c.omb1 = 1.0f - solver->beta1;
        c.omb2 = 1.0f - solver->beta2;
        c.ibc1 = 1.0f / (1.0f - powf(solver->beta1, t));
        c.ibc2 = 1.0f / (1.0f - powf(solver->beta2, t));
    }
    int64_t goff = 0;
    for (int t0 = 0; t0 < n_tensors; t0 += kSolverMulti) {
        SolverMulti d{};
        d.n = n_tensors - t0 < kSolverMulti ? n_tensors - t0 : kSolverMulti;
        int blocks = 0;
        for (int t = 0; t < d.n; ++t) {
            d.p[t] = params[t0 + t];
            d.m[t] = moments ? m_bufs[t0 + t] : nullptr;
            d.v[t] = moments ? v_bufs[t0 + t] : nullptr;
            HSES_REQUIRE(d.p[t] == nullptr || !moments || (d.m[t] != nullptr && d.v[t] != nullptr), "Adam needs moment buffers");
            d.len[t] = lens[t0 + t];
            d.goff[t] = goff;
            goff += lens[t0 + t];
            d.first_block[t] = blocks;
            blocks += (int)((lens[t0 + t] + 255) / 256);
        }
        d.first_block[d.n] = blocks;
        if (blocks == 0) continue;
        HSES_KERNEL(ctx, st, "solver");
        solver_multi_kernel<<<(unsigned)blocks, 256, 0, st>>>(c, d, grads);
        HSES_LAUNCH_CHECK();
    }
    return HSES_OK;
}
}  // namespace hses

extern "C" {

int hses_solver_step(hses_ctx* ctx, hses_stream stream, const hses_solver* solver, int32_t step,
                     float grad_scale, float* param, const float* grad, float* m, float* v,
                     int64_t len) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(solver != nullptr, "solver is NULL");
    HSES_REQUIRE(solver->kind == HSES_SGD || solver->kind == HSES_ADAM || solver->kind == HSES_ADAMW,
                 "unknown solver kind");
    HSES_REQUIRE(len >= 0, "len must be >= 0");
    if (len == 0) return HSES_OK;
    HSES_REQUIRE(param != nullptr && grad != nullptr, "NULL pointer");
    SolverConsts c{};
    c.kind = solver->kind;
    c.lr = solver->lr;
    c.grad_scale = grad_scale;
    if (solver->kind != HSES_SGD) {
        HSES_REQUIRE(m != nullptr && v != nullptr, "Adam needs moment buffers");
        HSES_REQUIRE(step >= 1, "step is the counter after the increment (>= 1)");
        float t = (float)step;
        float bc1 = 1.0f - powf(solver->beta1, t);
        float bc2 = 1.0f - powf(solver->beta2, t);
        c.beta1 = solver->beta1;
        c.beta2 = solver->beta2;
        c.eps = solver->eps;
        c.wd = solver->kind == HSES_ADAMW ? solver->weight_decay : 0.0f;
        c.omb1 = 1.0f - solver->beta1;
        c.omb2 = 1.0f - solver->beta2;
        c.ibc1 = 1.0f / bc1;
        c.ibc2 = 1.0f / bc2;
    }
    HSES_KERNEL(ctx, as_stream(stream), "solver");
    const bool vec4 = ((((uintptr_t)param | (uintptr_t)grad | (uintptr_t)m | (uintptr_t)v) & 15u) == 0) && len >= 4;
    if (vec4) {
        int64_t work = len / 4 + len % 4;
        solver_kernel<true><<<(unsigned)((work + 255) / 256), 256, 0, as_stream(stream)>>>(c, param, grad, m, v, len);
    } else {
        solver_kernel<false><<<(unsigned)((len + 255) / 256), 256, 0, as_stream(stream)>>>(c, param, grad, m, v, len);
    }
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // extern "C"
