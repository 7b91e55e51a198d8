// Materialising kernels for the noise stream: normal_fill, lora_factors,
// dense_noise and the dense-leaf update.  The fused forward/update kernels
// regenerate the same values in registers; these entry points exist for
// callers that want the tensors (parity checks, the trainer's cached-noise
// path) and for the small PARAM-class leaves.
#include "common.cuh"

namespace hses {

// Normals are produced in chunks of kChunk per thread; a thread reaches its
// chunk with a jump of 2*kChunk*chunk_index generator steps.
constexpr int kChunk = 16;

__global__ void normal_fill_kernel(LibmCal cal, const uint64_t* __restrict__ pow2, uint64_t seed,
                                   float* __restrict__ out, size_t n) {
    size_t chunk = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t begin = chunk * kChunk;
    if (begin >= n) return;
    uint64_t s = jump_by(pow2, seed | 1ull, 2ull * begin);
    size_t end = begin + kChunk < n ? begin + kChunk : n;
    for (size_t i = begin; i < end; ++i) out[i] = next_normal(s, cal);
}

// One thread per (member, row of the (a+b, r) block).  Rows [0,b) are B, rows
// [b,a+b) are A (eggroll.rs:98-101).
__global__ void lora_factors_kernel(LibmCal cal, const uint64_t* __restrict__ pow2, uint64_t key,
                                    int32_t true_epoch, const int32_t* __restrict__ thread_ids,
                                    int32_t first_thread, int64_t n_members, int rank, int a, int b,
                                    float base_sigma, int layout, float* __restrict__ A,
                                    float* __restrict__ B) {
    int64_t member = blockIdx.x;
    int row = blockIdx.y * blockDim.x + threadIdx.x;
    if (member >= n_members || row >= a + b) return;
    bool is_a = row >= b;
    if (is_a ? (A == nullptr) : (B == nullptr)) return;
    int32_t tid = thread_ids ? thread_ids[member] : first_thread + (int32_t)member;
    float scale = (tid % 2 == 0) ? base_sigma : -base_sigma;  // sign * base_sigma
    uint64_t s = noise_seed(key, true_epoch, tid / 2) | 1ull;
    s = jump_by(pow2, s, 2ull * (uint64_t)rank * (uint64_t)row);
    int m = is_a ? row - b : row;
    int dim = is_a ? a : b;
    float* dst = is_a ? A : B;
    for (int q = 0; q < rank; ++q) {
        float z = next_normal(s, cal);
        if (is_a) z = fmul(z, scale);
        size_t off = layout == HSES_LAYOUT_NAR
                         ? ((size_t)member * dim + m) * rank + q
                         : ((size_t)member * rank + q) * dim + m;
        dst[off] = z;
    }
}

__global__ void dense_noise_kernel(LibmCal cal, const uint64_t* __restrict__ pow2, uint64_t key,
                                   int32_t true_epoch, const int32_t* __restrict__ thread_ids,
                                   int32_t first_thread, int64_t n_members, int len,
                                   float base_sigma, float* __restrict__ out) {
    int64_t member = blockIdx.x;
    int begin = (blockIdx.y * blockDim.x + threadIdx.x) * kChunk;
    if (member >= n_members || begin >= len) return;
    int32_t tid = thread_ids ? thread_ids[member] : first_thread + (int32_t)member;
    float scale = (tid % 2 == 0) ? base_sigma : -base_sigma;
    uint64_t s = noise_seed(key, true_epoch, tid / 2) | 1ull;
    s = jump_by(pow2, s, 2ull * (uint64_t)begin);
    int end = begin + kChunk < len ? begin + kChunk : len;
    for (int i = begin; i < end; ++i) out[(size_t)member * len + i] = fmul(next_normal(s, cal), scale);
}

// Dense-leaf update: block c owns elements [c*kChunk, (c+1)*kChunk); its
// threads stride over the antithetic pairs, then reduce in a fixed order so
// that every rank obtains the same bits.
constexpr int kDenseThreads = 1024;  // few blocks (one per chunk of a leaf): all the parallelism is in the block
__global__ void es_update_dense_kernel(LibmCal cal, const uint64_t* __restrict__ pow2, uint64_t key,
                                       int32_t true_epoch, int32_t first_pair, int64_t n_pairs,
                                       int len, float sigma, float out_scale,
                                       const float* __restrict__ fitness, float* __restrict__ grad) {
    __shared__ float red[kDenseThreads];
    int begin = blockIdx.x * kChunk;
    int cnt = len - begin < kChunk ? len - begin : kChunk;
    float acc[kChunk];
#pragma unroll
    for (int i = 0; i < kChunk; ++i) acc[i] = 0.0f;
    for (int64_t p = threadIdx.x; p < n_pairs; p += kDenseThreads) {
        // member 2p has sign +1, member 2p+1 sign -1 (eggroll.rs:60-65)
        float w = fmul(fitness[2 * p] - fitness[2 * p + 1], sigma);
        uint64_t s = noise_seed(key, true_epoch, first_pair + (int32_t)p) | 1ull;
        s = jump_by(pow2, s, 2ull * (uint64_t)begin);
#pragma unroll
        for (int i = 0; i < kChunk; ++i)
            if (i < cnt) acc[i] = fmaf(w, next_normal(s, cal), acc[i]);
    }
    for (int i = 0; i < cnt; ++i) {
        red[threadIdx.x] = acc[i];
        __syncthreads();
        for (int stride = kDenseThreads / 2; stride > 0; stride >>= 1) {
            if (threadIdx.x < stride) red[threadIdx.x] += red[threadIdx.x + stride];
            __syncthreads();
        }
        if (threadIdx.x == 0) grad[begin + i] = red[0] * out_scale;
        __syncthreads();
    }
}

// Pair-folded raw factors for the scratch-based paths (see common.cuh).  CTA (pair, chunk)
// writes kPfBlocks blocks of 128 rows of the pair's (b + a, rank) normal block: a thread jumps
// to its first row once and from then on hops 127 rows ahead after each row it has written.
constexpr int kPfBlocks = 8;
__global__ void __launch_bounds__(128)
pair_factors_kernel(LibmCal cal, const uint64_t* __restrict__ pow2, const uint64_t* __restrict__ hop127,
                    uint64_t key, int32_t true_epoch, int32_t first_pair, int64_t pairs, int rank, int a,
                    int b, const float* __restrict__ pair_weight, float* __restrict__ A,
                    float* __restrict__ B) {
    // tables that every normal reads stay in shared memory
    __shared__ double2 log_tab_s[64];
    __shared__ uint32_t delta_s[512];
    __shared__ uint64_t hop_s[kJumpWords];
    for (int i = threadIdx.x; i < 64; i += blockDim.x) log_tab_s[i] = cal.log_tab[i];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        delta_s[i] = cal.log_delta[i];
        delta_s[256 + i] = cal.cos_delta[i];
    }
    // without a prebuilt hop table a thread advances with the per-context power-of-two tables instead
    if (hop127)
        for (int i = threadIdx.x; i < kJumpWords; i += blockDim.x) hop_s[i] = hop127[i];
    __syncthreads();
    cal.log_tab = log_tab_s;
    cal.log_delta = delta_s;
    cal.cos_delta = delta_s + 256;
    const int64_t p = blockIdx.x;
    int row = blockIdx.y * (128 * kPfBlocks) + threadIdx.x;
    if (p >= pairs || row >= a + b) return;
    uint64_t s = noise_seed(key, true_epoch, first_pair + (int32_t)p) | 1ull;
    s = jump_by(pow2, s, 2ull * (uint64_t)rank * (uint64_t)row);
    float w = 1.0f;
    if (pair_weight) w = __fsub_rn(pair_weight[2 * p], pair_weight[2 * p + 1]);
    for (int blk = 0; blk < kPfBlocks && row < a + b; ++blk, row += 128) {
        const bool is_a = row >= b;
        float* dst = is_a ? A + ((size_t)p * a + (row - b)) * rank : B + ((size_t)p * b + row) * rank;
        const bool weigh = is_a && pair_weight;
        if ((rank & 3) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            for (int q = 0; q < rank; q += 4) {
                float z[4];
                next_normals4(s, cal, z);
                if (weigh) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) z[j] = __fmul_rn(z[j], w);
                }
                *reinterpret_cast<float4*>(dst + q) = make_float4(z[0], z[1], z[2], z[3]);
            }
        } else {
            for (int q = 0; q < rank; ++q) {
                float z = next_normal(s, cal);
                dst[q] = weigh ? __fmul_rn(z, w) : z;
            }
        }
        s = hop127 ? jump_apply(hop_s, s) : jump_by(pow2, s, 2ull * (uint64_t)rank * 127ull);
    }
}

int launch_pair_factors(hses_ctx* ctx, cudaStream_t stream, uint64_t key, int32_t true_epoch,
                        int32_t first_pair, int64_t pairs, int rank, int a, int b,
                        const float* pair_weight, float* A, float* B, bool no_alloc) {
    int rows = a + b;
    int chunks = (rows + 128 * kPfBlocks - 1) / (128 * kPfBlocks);
    HSES_REQUIRE(chunks <= 65535, "a + b too large");
    HSES_REQUIRE(pairs >= 1 && pairs < (1ll << 31), "pair count out of range");
    // the hop table of a rank is built (and allocated) on its first use; callers that must not
    // allocate leave it out and the kernel advances with the context's power-of-two tables
    const uint64_t* hop127 = nullptr;
    if (!no_alloc) {
        int rc = get_hop_table(ctx, 2ull * (uint64_t)rank * 127, &hop127);
        if (rc != HSES_OK) return rc;
    }
    dim3 grid((unsigned)pairs, (unsigned)chunks);
    HSES_KERNEL(ctx, stream, "pair_factors");
    pair_factors_kernel<<<grid, 128, 0, stream>>>(ctx->cal(), ctx->t.jump_pow2, hop127, key, true_epoch,
                                                  first_pair, pairs, rank, a, b, pair_weight, A, B);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // namespace hses

using namespace hses;

extern "C" {

size_t hses_factor_cache_bytes(int64_t n_pairs, int32_t rank, int32_t a, int32_t b) {
    if (n_pairs < 1 || rank < 1 || a < 1 || b < 1) return 0;
    return (size_t)n_pairs * (size_t)(a + b) * (size_t)rank * sizeof(float);
}

int hses_factor_cache_build(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                            int32_t noise_reuse, int32_t first_pair, int64_t n_pairs,
                            int32_t rank, int32_t a, int32_t b, float* data,
                            hses_factor_cache* cache) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(cache != nullptr && data != nullptr, "NULL pointer");
    HSES_REQUIRE(n_pairs >= 1 && first_pair >= 0, "pair range out of bounds");
    HSES_REQUIRE(rank >= 1 && a >= 1 && b >= 1, "rank, a and b must be positive");
    HSES_REQUIRE(noise_reuse >= 0, "noise_reuse must be >= 0");
    HSES_REQUIRE((reinterpret_cast<uintptr_t>(data) & 15) == 0, "cache data must be 16-byte aligned");
    int32_t te = true_epoch_of(epoch, noise_reuse);
    float* A = data;
    float* B = data + (size_t)n_pairs * a * rank;
    int rc = launch_pair_factors(ctx, as_stream(stream), key, te, first_pair, n_pairs, rank, a, b,
                                 nullptr, A, B);
    if (rc != HSES_OK) return rc;
    cache->data = data;
    cache->key = key;
    cache->true_epoch = te;
    cache->first_pair = first_pair;
    cache->n_pairs = n_pairs;
    cache->rank = rank;
    cache->a = a;
    cache->b = b;
    return HSES_OK;
}

int hses_normal_fill(hses_ctx* ctx, hses_stream stream, uint64_t seed, float* out, size_t n) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    if (n == 0) return HSES_OK;
    HSES_REQUIRE(out != nullptr, "out is NULL");
    HSES_REQUIRE(n < (1ull << 40), "n too large");
    size_t chunks = (n + kChunk - 1) / kChunk;
    unsigned blocks = (unsigned)((chunks + 127) / 128);
    HSES_KERNEL(ctx, as_stream(stream), "normal_fill");
    normal_fill_kernel<<<blocks, 128, 0, as_stream(stream)>>>(ctx->cal(), ctx->t.jump_pow2, seed, out, n);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_lora_factors(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                      int32_t noise_reuse, const int32_t* thread_ids, int32_t first_thread,
                      int64_t n_members, int32_t rank, int32_t a, int32_t b, float base_sigma,
                      int32_t layout, float* A, float* B) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n_members >= 0 && n_members < (1ll << 31), "n_members out of range");
    HSES_REQUIRE(rank >= 1 && a >= 1 && b >= 1, "rank, a and b must be positive");
    HSES_REQUIRE(layout == HSES_LAYOUT_NAR || layout == HSES_LAYOUT_NRA, "unknown layout");
    HSES_REQUIRE(noise_reuse >= 0, "noise_reuse must be >= 0");
    HSES_REQUIRE(thread_ids != nullptr || first_thread >= 0, "thread ids must be non-negative");
    if (n_members == 0 || (A == nullptr && B == nullptr)) return HSES_OK;
    int rows = a + b;
    HSES_REQUIRE((rows + 127) / 128 <= 65535, "a + b too large");
    dim3 grid((unsigned)n_members, (unsigned)((rows + 127) / 128));
    HSES_KERNEL(ctx, as_stream(stream), "lora_factors");
    lora_factors_kernel<<<grid, 128, 0, as_stream(stream)>>>(
        ctx->cal(), ctx->t.jump_pow2, key, true_epoch_of(epoch, noise_reuse), thread_ids,
        first_thread, n_members, rank, a, b, base_sigma, layout, A, B);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_dense_noise(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                     int32_t noise_reuse, const int32_t* thread_ids, int32_t first_thread,
                     int64_t n_members, int32_t rows, int32_t cols, float base_sigma, float* out) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n_members >= 0 && n_members < (1ll << 31), "n_members out of range");
    HSES_REQUIRE(rows >= 1 && cols >= 1 && (int64_t)rows * cols < (1ll << 24), "bad leaf shape");
    HSES_REQUIRE(noise_reuse >= 0, "noise_reuse must be >= 0");
    if (n_members == 0) return HSES_OK;
    HSES_REQUIRE(out != nullptr, "out is NULL");
    int len = rows * cols;
    int chunks = (len + kChunk - 1) / kChunk;
    dim3 grid((unsigned)n_members, (unsigned)((chunks + 63) / 64));
    HSES_KERNEL(ctx, as_stream(stream), "dense_noise");
    dense_noise_kernel<<<grid, 64, 0, as_stream(stream)>>>(
        ctx->cal(), ctx->t.jump_pow2, key, true_epoch_of(epoch, noise_reuse), thread_ids,
        first_thread, n_members, len, base_sigma, out);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_es_update_dense(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                         int32_t noise_reuse, int32_t first_thread, int64_t n, int64_t n_total,
                         int32_t len, float sigma, const float* fitness, float* grad) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(n > 0 && n % 2 == 0 && first_thread >= 0 && first_thread % 2 == 0,
                 "members must form whole antithetic pairs");
    HSES_REQUIRE(n_total >= 1, "n_total must be >= 1");
    HSES_REQUIRE(len >= 1 && len <= (1 << 20), "len out of range");
    HSES_REQUIRE(fitness != nullptr && grad != nullptr, "NULL pointer");
    // grad = -( (sum/N) * sqrt(N) ), eggroll.rs:349,402-403
    float nf = (float)n_total;
    float out_scale = -(1.0f / nf) * sqrtf(nf);
    int blocks = (len + kChunk - 1) / kChunk;
    HSES_KERNEL(ctx, as_stream(stream), "es_update_dense");
    es_update_dense_kernel<<<blocks, kDenseThreads, 0, as_stream(stream)>>>(
        ctx->cal(), ctx->t.jump_pow2, key, true_epoch_of(epoch, noise_reuse), first_thread / 2,
        n / 2, len, sigma, out_scale, fitness, grad);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // extern "C"
