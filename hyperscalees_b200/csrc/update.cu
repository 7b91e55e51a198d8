// Fitness-weighted update of a LoRA-noised matrix
// (simple_lora_update + do_update_with, hyperscalees-noiser/src/eggroll.rs:353-404):
//   grad = -sqrt(N) * (1/N) * sum_i f_i A_i B_iᵀ.
// Antithetic members 2p and 2p+1 share one draw with A negated, so the sum
// folds to sum_p (f_2p - f_2p+1) * base_sigma * Araw_p Braw_pᵀ — a dense
// contraction (a, K)·(K, b) over K = pairs * rank, the same 2-D GEMM form as
// lora_einsum_raw (eggroll.rs:726-738).
//
// General path: the raw factors of a chunk of pairs are regenerated into
// scratch (A pre-multiplied by the pair weight), a split-K fp32 GEMM writes
// per-split partial sums, and a final pass adds the partials in a fixed order
// so that every rank ends up with bit-identical gradients.
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

#include "common.cuh"
#include "einsum_tc.cuh"
#include "update_tc.cuh"

namespace hses {

constexpr int UM = 128, UN = 128, UK = 16, UT = 256;
constexpr size_t kFactorChunkBytes = 256ull << 20;

struct UpdatePlan {
    int64_t pairs, chunk_pairs;
    int splits;
    size_t a_elems, b_elems, partial_elems, bytes;
};

static UpdatePlan plan_update(int a, int b, int rank, int64_t n) {
    UpdatePlan p;
    p.pairs = n / 2;
    size_t per_pair = (size_t)(a + b) * rank * sizeof(float);
    int64_t fit = (int64_t)(kFactorChunkBytes / per_pair);
    if (fit < 1) fit = 1;
    p.chunk_pairs = p.pairs < fit ? p.pairs : fit;
    int tiles = ((a + UM - 1) / UM) * ((b + UN - 1) / UN);
    int want = (2 * plan_sm_count() + tiles - 1) / tiles;
    if (want > 64) want = 64;
    if (want > p.chunk_pairs) want = (int)p.chunk_pairs;
    if (want < 1) want = 1;
    p.splits = want;
    auto up = [](size_t v) { return (v + 63) / 64 * 64; };
    p.a_elems = up((size_t)p.chunk_pairs * a * rank);
    p.b_elems = up((size_t)p.chunk_pairs * b * rank);
    p.partial_elems = up((size_t)p.splits * a * b);
    p.bytes = (p.a_elems + p.b_elems + p.partial_elems) * sizeof(float);
    return p;
}

// partial[split][m][n] (+)= sum over the split's pairs and q of A[p][m][q]*B[p][n][q]
__global__ void __launch_bounds__(UT)
update_gemm_kernel(const float* __restrict__ A, const float* __restrict__ B, int64_t pairs, int rank,
                   int a, int b, int accumulate, const float* __restrict__ pair_weight, int sign_factors,
                   float* __restrict__ partial) {
    __shared__ __align__(16) float sa[UK][UM + 4];
    __shared__ __align__(16) float sb[UK][UN + 4];
    int m0 = blockIdx.y * UM, n0 = blockIdx.x * UN;
    int split = blockIdx.z, splits = gridDim.z;
    int64_t p_lo = pairs * split / splits, p_hi = pairs * (split + 1) / splits;
    int64_t k_lo = p_lo * rank, k_hi = p_hi * rank;
    int tid = threadIdx.x;
    int tr = (tid / 16) * 4, tc = (tid % 16) * 4;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    for (int64_t k0 = k_lo; k0 < k_hi; k0 += UK) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            int idx = tid + e * UT;
            int r = idx / UK, kk = idx % UK;
            int64_t kg = k0 + kk;
            int64_t p = kg / rank;
            int q = (int)(kg - p * rank);
            bool kin = kg < k_hi;
            float av = (kin && m0 + r < a) ? A[((size_t)p * a + m0 + r) * rank + q] : 0.0f;
            float bv = (kin && n0 + r < b) ? B[((size_t)p * b + n0 + r) * rank + q] : 0.0f;
            if (sign_factors) {  // AltEggRoll contracts the sign patterns of the raw factors
                av = av > 0.0f ? 1.0f : av < 0.0f ? -1.0f : 0.0f;
                bv = bv > 0.0f ? 1.0f : bv < 0.0f ? -1.0f : 0.0f;
            }
            // factors read from a cache are unweighted: apply (f_even - f_odd) of the pair here
            if (pair_weight && kin) av = __fmul_rn(av, __fsub_rn(pair_weight[2 * p], pair_weight[2 * p + 1]));
            sa[kk][r] = av;
            sb[kk][r] = bv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < UK; ++kk) {
            float xa[8], wb[8];
            *reinterpret_cast<float4*>(&xa[0]) = *reinterpret_cast<const float4*>(&sa[kk][tr]);
            *reinterpret_cast<float4*>(&xa[4]) = *reinterpret_cast<const float4*>(&sa[kk][64 + tr]);
            *reinterpret_cast<float4*>(&wb[0]) = *reinterpret_cast<const float4*>(&sb[kk][tc]);
            *reinterpret_cast<float4*>(&wb[4]) = *reinterpret_cast<const float4*>(&sb[kk][64 + tc]);
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(xa[i], wb[j], acc[i][j]);
        }
        __syncthreads();
    }
    float* dst = partial + (size_t)split * a * b;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int m = m0 + (i < 4 ? tr + i : 64 + tr + i - 4);
        if (m >= a) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int n = n0 + (j < 4 ? tc + j : 64 + tc + j - 4);
            if (n >= b) continue;
            size_t o = (size_t)m * b + n;
            dst[o] = accumulate ? dst[o] + acc[i][j] : acc[i][j];
        }
    }
}

__global__ void update_reduce_kernel(const float* __restrict__ partial, int splits, size_t len,
                                     float scale, int accumulate, float* __restrict__ grad) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= len) return;
    float s = 0.0f;
    for (int k = 0; k < splits; ++k) s = __fadd_rn(s, partial[(size_t)k * len + i]);
    s = __fmul_rn(s, scale);
    grad[i] = accumulate ? __fadd_rn(grad[i], s) : s;
}

// ---------------------------------------------------------------------------
// Allocation-free variant: the scratch of the update lives in a fixed array in
// device memory that is part of the library image.  In host code the array's
// name only stands in for the symbol; its device address is looked up once per
// device with cudaGetSymbolAddress and that pointer is what the kernels get.
// ---------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 16ull << 20;
static __device__ __align__(256) unsigned char g_static_update_scratch[kStaticScratchBytes];

static std::mutex g_static_mutex;
static std::map<int, float*> g_static_ptr;  // device ordinal -> address of the array on that device

static int static_scratch_for_device(int device, float** out) {
    // checked on every call: a launch made while another GPU is current would hand that GPU
    // this device's address
    int current = -1;
    HSES_CUDA(cudaGetDevice(&current));
    HSES_REQUIRE(current == device, "the context's device must be the current CUDA device");
    std::lock_guard<std::mutex> lock(g_static_mutex);
    auto it = g_static_ptr.find(device);
    if (it != g_static_ptr.end()) {
        *out = it->second;
        return HSES_OK;
    }
    void* ptr = nullptr;
    HSES_CUDA(cudaGetSymbolAddress(&ptr, g_static_update_scratch));
    HSES_REQUIRE(ptr != nullptr, "cudaGetSymbolAddress returned NULL");
    g_static_ptr[device] = reinterpret_cast<float*>(ptr);
    *out = reinterpret_cast<float*>(ptr);
    return HSES_OK;
}

// Splits the fixed array into per-split partial sums and one chunk of factors.
static bool plan_update_static(int a, int b, int rank, int64_t n, UpdatePlan* out) {
    UpdatePlan p;
    p.pairs = n / 2;
    auto up = [](size_t v) { return (v + 63) / 64 * 64; };
    size_t budget = kStaticScratchBytes / sizeof(float);
    size_t per_pair = (size_t)(a + b) * rank;
    size_t ab = (size_t)a * b;
    int tiles = ((a + UM - 1) / UM) * ((b + UN - 1) / UN);
    int splits = (2 * plan_sm_count() + tiles - 1) / tiles;
    if (splits > 16) splits = 16;
    // partial sums may take at most half of the array; the rest holds factors
    while (splits > 1 && up((size_t)splits * ab) > budget / 2) --splits;
    if (up((size_t)splits * ab) + 2 * 64 + per_pair > budget) return false;
    size_t left = budget - up((size_t)splits * ab) - 2 * 64;
    int64_t fit = (int64_t)(left / per_pair);
    if (fit < 1) return false;
    p.chunk_pairs = p.pairs < fit ? p.pairs : fit;
    if (splits > p.chunk_pairs) splits = (int)p.chunk_pairs;
    p.splits = splits;
    p.a_elems = up((size_t)p.chunk_pairs * a * rank);
    p.b_elems = up((size_t)p.chunk_pairs * b * rank);
    p.partial_elems = up((size_t)p.splits * ab);
    p.bytes = (p.a_elems + p.b_elems + p.partial_elems) * sizeof(float);
    if (p.bytes > kStaticScratchBytes) return false;
    *out = p;
    return true;
}

// ---------------------------------------------------------------------------
// einsum_pair_fused (hyperscalees/src/oxide.rs:318-462, kernel
// hyperscalees-kernels/src/einsum_pair_fused_oxide.rs:94-227) for callers that bring their own
// half-population factors: a_t (half*r, a) and b_t (half*r, b), row k = i*r + j belonging to
// member pair (i, i + half);  g_raw = sum_k (s_i + s_{i+half}) a_t[k] (x) b_t[k],
// g_ones = 2 * sum_k a_t[k] (x) b_t[k].  Split-K partial sums are added in a fixed order
// (the reference merges with float atomics).
// ---------------------------------------------------------------------------
constexpr int EP_TM = 64, EP_TN = 64, EP_TK = 16, EP_THREADS = 256;
__global__ void __launch_bounds__(EP_THREADS)
einsum_pair_kernel(const float* __restrict__ a_t, int64_t a_s0, int64_t a_s1, const float* __restrict__ b_t, int64_t b_s0,
                   int64_t b_s1,
                   const float* __restrict__ scores, int64_t half, int r, int a, int b,
                   float* __restrict__ partial) {
    __shared__ __align__(16) float sa[EP_TK][EP_TM];
    __shared__ __align__(16) float sw[EP_TK][EP_TM];
    __shared__ __align__(16) float sb[EP_TK][EP_TN];
    const int m0 = blockIdx.y * EP_TM, n0 = blockIdx.x * EP_TN;
    const int split = blockIdx.z, splits = gridDim.z;
    const int64_t K = half * r;
    const int64_t k_lo = K * split / splits, k_hi = K * (split + 1) / splits;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    float raw[4][4], ones[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) raw[i][j] = ones[i][j] = 0.0f;
    for (int64_t k0 = k_lo; k0 < k_hi; k0 += EP_TK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int idx = tid + e * EP_THREADS;
            int kk = idx >> 6, c = idx & 63;
            int64_t kg = k0 + kk;
            bool kin = kg < k_hi;
            float f = 0.0f;
            int64_t i = 0, j = 0;
            if (kin) {
                i = kg / r;
                j = kg - i * r;
                f = __fadd_rn(scores[i], scores[i + half]);
            }
            float av = (kin && m0 + c < a) ? a_t[(size_t)(i * a_s0 + j * a_s1) + m0 + c] : 0.0f;
            sa[kk][c] = av;
            sw[kk][c] = __fmul_rn(av, f);
            sb[kk][c] = (kin && n0 + c < b) ? b_t[(size_t)(i * b_s0 + j * b_s1) + n0 + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < EP_TK; ++kk) {
            float4 a4 = *reinterpret_cast<const float4*>(&sa[kk][ty * 4]);
            float4 w4 = *reinterpret_cast<const float4*>(&sw[kk][ty * 4]);
            float4 b4 = *reinterpret_cast<const float4*>(&sb[kk][tx * 4]);
            const float av[4] = {a4.x, a4.y, a4.z, a4.w}, wv[4] = {w4.x, w4.y, w4.z, w4.w};
            const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    raw[i][j] = fmaf(wv[i], bv[j], raw[i][j]);
                    ones[i][j] = fmaf(av[i], bv[j], ones[i][j]);
                }
        }
        __syncthreads();
    }
    float* praw = partial + (size_t)split * 2 * a * b;
    float* pones = praw + (size_t)a * b;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        if (m >= a) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n >= b) continue;
            praw[(size_t)m * b + n] = raw[i][j];
            pones[(size_t)m * b + n] = ones[i][j];
        }
    }
}

__global__ void einsum_pair_reduce_kernel(const float* __restrict__ partial, int splits, size_t len,
                                          float* __restrict__ g_raw, float* __restrict__ g_ones) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= len) return;
    float sr = 0.0f, so = 0.0f;
    for (int k = 0; k < splits; ++k) {
        sr = __fadd_rn(sr, partial[(size_t)k * 2 * len + i]);
        so = __fadd_rn(so, partial[(size_t)k * 2 * len + len + i]);
    }
    g_raw[i] = sr;
    g_ones[i] = __fmul_rn(so, 2.0f);
}

static int einsum_pair_splits(int64_t half, int r, int a, int b) {
    int tiles = ((a + EP_TM - 1) / EP_TM) * ((b + EP_TN - 1) / EP_TN);
    int64_t kblocks = (half * r + 255) / 256;   // at least 256 rows of K per split
    int want = (2 * plan_sm_count() + tiles - 1) / tiles;
    if (want > kblocks) want = (int)kblocks;
    if (want > 256) want = 256;
    return want < 1 ? 1 : want;
}

}  // namespace hses

using namespace hses;

extern "C" {

size_t hses_es_update_workspace_bytes(int32_t a, int32_t b, int32_t rank, int64_t n) {
    if (a < 1 || b < 1 || rank < 1 || n < 2) return 0;
    size_t bytes = plan_update(a, b, rank, n).bytes;
    if (update_tc_supports(a, b, rank)) {
        size_t tc = plan_update_tc(a, b, rank, n, true).bytes;
        if (tc > bytes) bytes = tc;
    }
    return bytes;
}

int hses_es_update_ex(hses_ctx* ctx, hses_stream stream, const hses_update_args* args) {
    return es_update_ex_impl(ctx, stream, args, false, nullptr);
}

}  // extern "C"

int hses::es_update_ex_impl(hses_ctx* ctx, hses_stream stream, const hses_update_args* args, bool reuse_range,
                            bool* took_tc) {
    if (took_tc) *took_tc = false;
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(args != nullptr, "args is NULL");
    const hses_update_args& u = *args;
    const int a = u.a, b = u.b, rank = u.rank;
    HSES_REQUIRE(u.n > 0 && u.n % 2 == 0 && u.first_thread >= 0 && u.first_thread % 2 == 0,
                 "members must form whole antithetic pairs");
    HSES_REQUIRE(u.n_total >= 1, "n_total must be >= 1");
    HSES_REQUIRE(rank >= 1 && rank <= 1024 && a >= 1 && b >= 1, "bad shape");
    HSES_REQUIRE(u.noise_reuse >= 0, "noise_reuse must be >= 0");
    HSES_REQUIRE(u.fitness != nullptr && u.grad != nullptr, "NULL pointer");
    HSES_REQUIRE(u.mode == HSES_UPDATE_GRAD || u.mode == HSES_UPDATE_RAW_ACC, "unknown update mode");
    cudaStream_t st = as_stream(stream);
    const float base_sigma_tc = u.sigma / sqrtf((float)rank);
    HSES_REQUIRE(u.algo == HSES_ALGO_AUTO || u.algo == HSES_ALGO_SIMT || u.algo == HSES_ALGO_TENSOR, "unknown algo");
    const bool tc_ok = update_tc_supports(a, b, rank);
    if (u.algo == HSES_ALGO_TENSOR && !tc_ok) {
        set_error("hses_es_update_ex: the tensor-core contraction does not cover this shape");
        return HSES_ERR_UNSUPPORTED;
    }
    if (tc_ok && u.algo != HSES_ALGO_SIMT) {
        // wide factors on tile-aligned shapes: the contraction runs on the tensor cores
        float nf = (float)u.n_total;
        float sc = u.mode == HSES_UPDATE_GRAD ? -(base_sigma_tc * (1.0f / nf)) * sqrtf(nf) : base_sigma_tc;
        if (took_tc) *took_tc = true;
        return run_update_tc(ctx, st, u, sc, reuse_range);
    }
    UpdatePlan p = plan_update(a, b, rank, u.n);
    HSES_REQUIRE(u.workspace != nullptr && u.workspace_bytes >= p.bytes,
                 "workspace too small; see hses_es_update_workspace_bytes");
    HSES_REQUIRE((a + UM - 1) / UM <= 65535, "a too large");
    float* wsA = reinterpret_cast<float*>(u.workspace);
    float* wsB = wsA + p.a_elems;
    float* partial = wsB + p.b_elems;
    const int32_t te = true_epoch_of(u.epoch, u.noise_reuse);
    const int32_t first_pair = u.first_thread / 2;
    dim3 grid((unsigned)((b + UN - 1) / UN), (unsigned)((a + UM - 1) / UM), (unsigned)p.splits);
    if (u.cache) {
        const hses_factor_cache& c = *u.cache;
        HSES_REQUIRE(c.data != nullptr && c.key == u.key && c.true_epoch == te && c.rank == rank &&
                         c.a == a && c.b == b,
                     "factor cache was built for another parameter, epoch bucket or shape");
        HSES_REQUIRE(first_pair >= c.first_pair && first_pair + p.pairs <= c.first_pair + c.n_pairs,
                     "factor cache does not cover these members");
        const float* cA = c.data + (size_t)(first_pair - c.first_pair) * a * rank;
        const float* cB = c.data + (size_t)c.n_pairs * a * rank + (size_t)(first_pair - c.first_pair) * b * rank;
        HSES_KERNEL(ctx, st, "update_gemm");
        update_gemm_kernel<<<grid, UT, 0, st>>>(cA, cB, p.pairs, rank, a, b, 0, u.fitness, u.sign_factors, partial);
        HSES_LAUNCH_CHECK();
    } else {
        int chunk_idx = 0;
        for (int64_t done = 0; done < p.pairs; done += p.chunk_pairs, ++chunk_idx) {
            int64_t cnt = p.pairs - done < p.chunk_pairs ? p.pairs - done : p.chunk_pairs;
            // the sign variant must see the unweighted factors: the pair weight is applied by the loader
            const float* w = u.fitness + 2 * done;
            int rc = launch_pair_factors(ctx, st, u.key, te, first_pair + (int32_t)done, cnt, rank, a, b,
                                         u.sign_factors ? nullptr : w, wsA, wsB);
            if (rc != HSES_OK) return rc;
            HSES_KERNEL(ctx, st, "update_gemm");
            update_gemm_kernel<<<grid, UT, 0, st>>>(wsA, wsB, cnt, rank, a, b, chunk_idx > 0,
                                                    u.sign_factors ? w : nullptr, u.sign_factors, partial);
            HSES_LAUNCH_CHECK();
        }
    }
    const float base_sigma = u.sigma / sqrtf((float)rank);
    float scale;
    if (u.mode == HSES_UPDATE_GRAD) {
        // grad = -( (sum * base_sigma / N) * sqrt(N) ), eggroll.rs:365-372, 402-403
        float nf = (float)u.n_total;
        scale = -(base_sigma * (1.0f / nf)) * sqrtf(nf);
    } else {
        scale = base_sigma;
    }
    size_t len = (size_t)a * b;
    HSES_KERNEL(ctx, st, "update_reduce");
    update_reduce_kernel<<<(unsigned)((len + 255) / 256), 256, 0, st>>>(
        partial, p.splits, len, scale, u.mode == HSES_UPDATE_RAW_ACC, u.grad);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

extern "C" {

int hses_es_update(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                   int32_t noise_reuse, int32_t first_thread, int64_t n, int64_t n_total,
                   int32_t rank, int32_t a, int32_t b, float sigma, const float* fitness,
                   float* grad, void* workspace, size_t workspace_bytes) {
    hses_update_args u;
    memset(&u, 0, sizeof(u));
    u.key = key;
    u.epoch = epoch;
    u.noise_reuse = noise_reuse;
    u.first_thread = first_thread;
    u.n = n;
    u.n_total = n_total;
    u.rank = rank;
    u.a = a;
    u.b = b;
    u.sigma = sigma;
    u.fitness = fitness;
    u.grad = grad;
    u.workspace = workspace;
    u.workspace_bytes = workspace_bytes;
    u.cache = nullptr;
    u.mode = HSES_UPDATE_GRAD;
    return hses_es_update_ex(ctx, stream, &u);
}

size_t hses_es_update_static_scratch_bytes(void) { return kStaticScratchBytes; }

int hses_es_update_static(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                          int32_t noise_reuse, int32_t first_thread, int64_t n, int64_t n_total,
                          int32_t rank, int32_t a, int32_t b, float sigma, const float* fitness,
                          float* grad) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n > 0 && n % 2 == 0 && first_thread >= 0 && first_thread % 2 == 0,
                 "members must form whole antithetic pairs");
    HSES_REQUIRE(n_total >= 1, "n_total must be >= 1");
    HSES_REQUIRE(rank >= 1 && rank <= 1024 && a >= 1 && b >= 1, "bad shape");
    HSES_REQUIRE(noise_reuse >= 0, "noise_reuse must be >= 0");
    HSES_REQUIRE(fitness != nullptr && grad != nullptr, "NULL pointer");
    HSES_REQUIRE((a + UM - 1) / UM <= 65535, "a too large");
    UpdatePlan p;
    if (!plan_update_static(a, b, rank, n, &p)) {
        set_error("hses_es_update_static: a=" + std::to_string(a) + ", b=" + std::to_string(b) +
                  ", rank=" + std::to_string(rank) + " does not fit the built-in scratch of " +
                  std::to_string(kStaticScratchBytes) + " bytes (partial sums plus the factors of "
                  "one antithetic pair must fit); use hses_es_update with a caller workspace");
        return HSES_ERR_INVALID;
    }
    float* base = nullptr;
    int rc = static_scratch_for_device(ctx->device, &base);
    if (rc != HSES_OK) return rc;
    cudaStream_t st = as_stream(stream);
    float* wsA = base;
    float* wsB = wsA + p.a_elems;
    float* partial = wsB + p.b_elems;
    int32_t te = true_epoch_of(epoch, noise_reuse);
    dim3 grid((unsigned)((b + UN - 1) / UN), (unsigned)((a + UM - 1) / UM), (unsigned)p.splits);
    int chunk_idx = 0;
    for (int64_t done = 0; done < p.pairs; done += p.chunk_pairs, ++chunk_idx) {
        int64_t cnt = p.pairs - done < p.chunk_pairs ? p.pairs - done : p.chunk_pairs;
        rc = launch_pair_factors(ctx, st, key, te, first_thread / 2 + (int32_t)done, cnt, rank, a, b,
                                 fitness + 2 * done, wsA, wsB, /*no_alloc=*/true);
        if (rc != HSES_OK) return rc;
        HSES_KERNEL(ctx, st, "update_gemm");
        // the first chunk overwrites the partial sums, so nothing left behind by an
        // earlier call is read
        update_gemm_kernel<<<grid, UT, 0, st>>>(wsA, wsB, cnt, rank, a, b, chunk_idx > 0, nullptr, 0, partial);
        HSES_LAUNCH_CHECK();
    }
    float nf = (float)n_total;
    float scale = -((sigma / sqrtf((float)rank)) * (1.0f / nf)) * sqrtf(nf);
    size_t len = (size_t)a * b;
    HSES_KERNEL(ctx, st, "update_reduce");
    update_reduce_kernel<<<(unsigned)((len + 255) / 256), 256, 0, st>>>(partial, p.splits, len, scale,
                                                                       0, grad);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

size_t hses_einsum_pair_workspace_bytes(int64_t half, int32_t r, int32_t a, int32_t b) {
    if (half < 1 || r < 1 || a < 1 || b < 1) return 0;
    size_t simt = (size_t)einsum_pair_splits(half, r, a, b) * 2 * (size_t)a * b * sizeof(float);
    size_t tc = plan_einsum_tc(half, r, a, b).bytes;   // whichever kernel the pointers and strides allow
    return simt > tc ? simt : tc;
}

int hses_einsum_pair(hses_ctx* ctx, hses_stream stream, const float* a_t, int64_t a_stride0, int64_t a_stride1,
                     const float* b_t, int64_t b_stride0, int64_t b_stride1, const float* scores, int64_t half,
                     int32_t r, int32_t a, int32_t b, float* g_raw, float* g_ones, void* workspace,
                     size_t workspace_bytes) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(half >= 1 && r >= 1 && a >= 1 && b >= 1, "bad shape");
    HSES_REQUIRE(a_stride1 >= a && b_stride1 >= b && a_stride0 >= 0 && b_stride0 >= 0, "row stride smaller than the row");
    HSES_REQUIRE(a_t != nullptr && b_t != nullptr && scores != nullptr && g_raw != nullptr && g_ones != nullptr,
                 "NULL pointer");
    HSES_REQUIRE(half * r < (1ll << 40), "K too large");
    size_t need = hses_einsum_pair_workspace_bytes(half, r, a, b);
    HSES_REQUIRE(workspace != nullptr && workspace_bytes >= need, "workspace too small; see hses_einsum_pair_workspace_bytes");
    cudaStream_t st = as_stream(stream);
    // long contractions over 16-byte aligned operands run on the tensor cores
    if (einsum_tc_supports(a_t, a_stride0, a_stride1, b_t, b_stride0, b_stride1, half, r, a, b) &&
        ((uintptr_t)workspace & 255u) == 0)
        return run_einsum_tc(ctx, st, a_t, a_stride0, a_stride1, b_t, b_stride0, b_stride1, scores, half, r, a, b, g_raw,
                             g_ones, workspace, workspace_bytes);
    int splits = einsum_pair_splits(half, r, a, b);
    HSES_REQUIRE((a + EP_TM - 1) / EP_TM <= 65535, "a too large");
    float* partial = reinterpret_cast<float*>(workspace);
    dim3 grid((unsigned)((b + EP_TN - 1) / EP_TN), (unsigned)((a + EP_TM - 1) / EP_TM), (unsigned)splits);
    {
        HSES_KERNEL(ctx, st, "einsum_pair");
        einsum_pair_kernel<<<grid, EP_THREADS, 0, st>>>(a_t, a_stride0, a_stride1, b_t, b_stride0, b_stride1, scores, half, r, a,
                                                        b, partial);
        HSES_LAUNCH_CHECK();
    }
    size_t len = (size_t)a * b;
    HSES_KERNEL(ctx, st, "einsum_pair_reduce");
    einsum_pair_reduce_kernel<<<(unsigned)((len + 255) / 256), 256, 0, st>>>(partial, splits, len, g_raw, g_ones);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // extern "C"
