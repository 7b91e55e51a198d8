// Tensor-core form of the fitness-weighted update
//   sum_p (f_2p - f_2p+1) * A_p B_pᵀ          (simple_lora_update, eggroll.rs:353-373, pair-folded)
// as one dense contraction (a, K)·(K, b) over K = pairs * rank — the 2-D GEMM form of
// lora_einsum_raw (eggroll.rs:726-738) — for the wide-rank, large-population case in which it
// dominates the step (rank from 48 up; ranks that are not multiples of 64 run with a zero-filled
// last k-block).
//
//   launch 1  pair_weight_range   largest |f_2p - f_2p+1| -> one power-of-two scale for all weights
//   launch 2  update_tc           one CTA per (128 x bn output tile, K split), eighteen warps:
//       warp 1      TMA producer: the raw fp32 [128 x 64] / [bn x 64] tiles of one pair at a time
//                   (factor cache, or scratch pair_factors just filled) through 3-D tensor maps
//                   over (q, row, pair) into a shared-memory stage
//       warps 2-17  converters: read the landed fp32 values, apply the pair weight and fixed
//                   powers of two, split into fp16 hi + lo and write the 128B-swizzled K-major
//                   operand tiles over the same stage (an fp32 row and its hi + lo rows have the
//                   same size)
//       warp 0      MMA issuer: tcgen05.mma kind::f16, hi*hi + hi*lo + lo*hi, fp32 accumulators
//                   in TMEM over all pairs of the split
//       warps 2-17  afterwards drain TMEM into the split's partial sums (four per TMEM quadrant)
//   launch 3  update_tc_reduce    adds the splits in a fixed order, undoes the scales
// The factors are read exactly once, as fp32, and never written back: the kernel is bound by
// those bytes.  Three fp16 passes keep the products fp32-equivalent; normals from 24-bit
// uniforms are bounded by 5.8, so fixed scales cannot overflow.  No multicast, no cluster
// launch, bounded waits.
#include <cuda.h>
#include <cuda_fp16.h>

#include "tc_common.cuh"
#include "update_tc.cuh"

namespace hses {

namespace {

using namespace tc;

constexpr int UT_BM = 128;
constexpr int UT_BK = 64;
constexpr int UT_THREADS = 576;  // warp 0 MMA, warp 1 TMA, warps 2-17 converters and epilogue
constexpr int UT_CONV = 512;     // converter threads
constexpr int kExpA = 12, kExpB = 11;  // A' = (w * 2^-e_w) * A * 2^12 <= 23.7e3, B' = B * 2^11 <= 11.9e3
constexpr size_t kRawChunkBytes = 384ull << 20;  // regenerated fp32 factors of one chunk of pairs

// largest |f_even - f_odd| over the call's pairs -> exponent e with 2^e >= max (0 when all zero)
__global__ void pair_weight_range_kernel(const float* __restrict__ fitness, int64_t pairs, int* __restrict__ e_out) {
    __shared__ float red[32];
    float m = 0.0f;
    for (int64_t p = threadIdx.x; p < pairs; p += blockDim.x)
        m = fmaxf(m, fabsf(__fsub_rn(fitness[2 * p], fitness[2 * p + 1])));
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < (int)(blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
        int e = 0;
        if (m > 0.0f && m < INFINITY) {
            frexpf(m, &e);  // m = f * 2^e, f in [0.5, 1)
            if (e > 100) e = 100;
            if (e < -100) e = -100;
        }
        *e_out = e;
    }
}

struct UtArgs {
    const float* A;     // raw (pairs, a, rank) of this chunk
    const float* B;     // raw (pairs, b, rank)
    const float* fitness;  // of the chunk's first member on
    const int* e_w;
    int sign_factors;
    int a, b, rank, bn;
    int n_tiles;        // output column tiles of bn
    int64_t pairs;      // pairs of this chunk
    int splits;
    int accumulate;     // add to the partial sums of earlier chunks
    int tmem_cols;      // power of two >= bn
    int stages;
    float* partial;     // [splits][a][b]
    int* status;
};

// four fp32 values -> fp16 hi and lo halves of a 16-byte piece of a 128B-swizzled K-major tile
__device__ __forceinline__ void convert_store(float4 v, float mul, int sign_factors, uint8_t* tile_hi,
                                              uint8_t* tile_lo, int row, int f4) {
    if (sign_factors) {  // uniform over the launch
        v.x = v.x > 0.0f ? 1.0f : v.x < 0.0f ? -1.0f : 0.0f;
        v.y = v.y > 0.0f ? 1.0f : v.y < 0.0f ? -1.0f : 0.0f;
        v.z = v.z > 0.0f ? 1.0f : v.z < 0.0f ? -1.0f : 0.0f;
        v.w = v.w > 0.0f ? 1.0f : v.w < 0.0f ? -1.0f : 0.0f;
    }
    // mul = weight * power of two: one rounding, the same value as (v * weight) * power of two
    const float x0 = __fmul_rn(v.x, mul), x1 = __fmul_rn(v.y, mul);
    const float x2 = __fmul_rn(v.z, mul), x3 = __fmul_rn(v.w, mul);
    const __half2 h01 = __floats2half2_rn(x0, x1), h23 = __floats2half2_rn(x2, x3);
    const float2 b01 = __half22float2(h01), b23 = __half22float2(h23);
    const __half2 l01 = __floats2half2_rn(x0 - b01.x, x1 - b01.y), l23 = __floats2half2_rn(x2 - b23.x, x3 - b23.y);
    // row r of the tile is 128 bytes; its 16-byte piece c sits at piece c ^ (r % 8) of the row
    const int off = (row >> 3) * 1024 + (row & 7) * 128 + (((f4 >> 1) ^ (row & 7)) << 4) + ((f4 & 1) << 3);
    *reinterpret_cast<uint2*>(tile_hi + off) =
        make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
    *reinterpret_cast<uint2*>(tile_lo + off) =
        make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
}

__global__ void __launch_bounds__(UT_THREADS, 1)
update_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const UtArgs g) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int a_bytes = UT_BM * UT_BK * 2, b_bytes = g.bn * UT_BK * 2;
    const int stage_bytes = 2 * a_bytes + 2 * b_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)g.stages * stage_bytes);
    uint64_t* full = bars;          // [stages] tiles converted
    uint64_t* empty = bars + 4;     // [stages] MMAs finished reading the stage
    uint64_t* landed = bars + 8;    // [stages] fp32 tiles arrived
    uint64_t* readdone = bars + 12; // [stages] every converter has read its fp32 values
    uint64_t* tfull = bars + 16;    // accumulator complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
    __shared__ int abort_flag_s;
    volatile int* abort_flag = &abort_flag_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int mt = tile / g.n_tiles, nt = tile - mt * g.n_tiles;
    const int64_t p_lo = g.pairs * split / g.splits, p_hi = g.pairs * (split + 1) / g.splits;
    const int kq = (g.rank + UT_BK - 1) / UT_BK;        // k-blocks per pair; columns past the rank of a ragged
                                                        // last block arrive as zeros (TMA fill) and add nothing
    const int64_t k_blocks = (p_hi - p_lo) * kq;

    if (threadIdx.x == 0) {
        abort_flag_s = 0;
        for (int s = 0; s < g.stages; ++s) {
            mbar_init(&full[s], UT_CONV);
            mbar_init(&empty[s], 1);
            mbar_init(&landed[s], 1);
            mbar_init(&readdone[s], UT_CONV);
        }
        mbar_init(tfull, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(g.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc(g.bn);
            bool ok = true;
            for (int64_t it = 0; it < k_blocks; ++it) {
                int s = (int)(it % g.stages);
                uint32_t ph = (uint32_t)(it / g.stages) & 1;
                if (!mbar_wait(&full[s], ph, abort_flag, g.status, 12)) { ok = false; break; }
                tc_fence_after();
                uint8_t* st = smem + (size_t)s * stage_bytes;
                uint64_t dah = make_smem_desc(st), dal = make_smem_desc(st + a_bytes);
                uint64_t dbh = make_smem_desc(st + 2 * a_bytes), dbl = make_smem_desc(st + 2 * a_bytes + b_bytes);
#pragma unroll
                for (int ks = 0; ks < UT_BK / 16; ++ks) {
                    uint64_t off = (uint64_t)(ks * 32 >> 4);  // 16 fp16 = 32 B along K
                    umma_f16(tmem_base, dal + off, dbh + off, idesc, (it | ks) != 0);
                    umma_f16(tmem_base, dah + off, dbl + off, idesc, 1);
                    umma_f16(tmem_base, dah + off, dbh + off, idesc, 1);
                }
                umma_commit(&empty[s]);
            }
            if (ok && k_blocks > 0) umma_commit(tfull);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            int64_t it = 0;
            for (int64_t p = p_lo; p < p_hi && ok; ++p) {
                for (int qb = 0; qb < kq; ++qb, ++it) {
                    const int s = (int)(it % g.stages);
                    const uint32_t ph = (uint32_t)(it / g.stages) & 1;
                    if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, g.status, 11)) { ok = false; break; }
                    uint8_t* st = smem + (size_t)s * stage_bytes;
                    mbar_expect_tx(&landed[s], (uint32_t)stage_bytes);  // boxes count in full, zero fill included
                    tma_load_3d(st, &tm_a, qb * UT_BK, mt * UT_BM, (int)p, &landed[s]);
                    tma_load_3d(st + 2 * a_bytes, &tm_b, qb * UT_BK, nt * g.bn, (int)p, &landed[s]);
                }
            }
            if (!ok) {
                // copies already issued still land in this CTA's shared memory: give them a bounded moment
                for (int s = 0; s < g.stages; ++s)
                    for (uint32_t i = 0; i < 4096; ++i) {
                        if (mbar_try(&landed[s], 0) || mbar_try(&landed[s], 1)) break;
                        __nanosleep(256);
                    }
            }
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------------ converters
        const int ct = threadIdx.x - 64;        // 0..511
        const int crow = ct >> 4, f4 = ct & 15;  // 32 rows per pass, 16 float4 per 64-value row
        const float sc_a = ldexpf(1.0f, kExpA - *g.e_w), sc_b = ldexpf(1.0f, kExpB);
        constexpr int A_PASSES = UT_BM / 32, B_PASSES = 256 / 32;
        bool ok = true;
        int64_t it = 0;
        // the pair weight is fetched one pair ahead: its load latency would otherwise sit between the
        // arrival of a stage and the first converted value
        float2 f_next = p_lo < p_hi ? make_float2(__ldg(g.fitness + 2 * p_lo), __ldg(g.fitness + 2 * p_lo + 1))
                                    : make_float2(0.f, 0.f);
        for (int64_t p = p_lo; p < p_hi && ok; ++p) {
            const float w_sc = __fmul_rn(__fsub_rn(f_next.x, f_next.y), sc_a);   // exact: sc_a is a power of two
            if (p + 1 < p_hi) f_next = make_float2(__ldg(g.fitness + 2 * p + 2), __ldg(g.fitness + 2 * p + 3));
            for (int qb = 0; qb < kq; ++qb, ++it) {
                const int s = (int)(it % g.stages);
                const uint32_t ph = (uint32_t)(it / g.stages) & 1;
                if (!mbar_wait(&landed[s], ph, abort_flag, g.status, 14)) { ok = false; break; }
                uint8_t* st = smem + (size_t)s * stage_bytes;
                // fp32 rows are 256 bytes; thread (crow, f4) owns the float4 f4 of rows crow + 32u
                float4 va[A_PASSES], vb[B_PASSES];
#pragma unroll
                for (int u = 0; u < A_PASSES; ++u)
                    va[u] = *reinterpret_cast<const float4*>(st + (size_t)(u * 32 + crow) * 256 + f4 * 16);
#pragma unroll
                for (int u = 0; u < B_PASSES; ++u) {
                    const int row = u * 32 + crow;
                    vb[u] = row < g.bn ? *reinterpret_cast<const float4*>(st + 2 * a_bytes + (size_t)row * 256 + f4 * 16)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                // the fp16 tiles overwrite the fp32 values: every converter must have read first
                // (an mbarrier with a bounded wait rather than bar.sync: a role that gave up must
                // not leave the others parked for good)
                mbar_arrive(&readdone[s]);
                if (!mbar_wait(&readdone[s], ph, abort_flag, g.status, 15)) { ok = false; break; }
#pragma unroll
                for (int u = 0; u < A_PASSES; ++u)
                    convert_store(va[u], w_sc, g.sign_factors, st, st + a_bytes, u * 32 + crow, f4);
#pragma unroll
                for (int u = 0; u < B_PASSES; ++u) {
                    const int row = u * 32 + crow;
                    if (row < g.bn)
                        convert_store(vb[u], sc_b, g.sign_factors, st + 2 * a_bytes,
                                      st + 2 * a_bytes + b_bytes, row, f4);
                }
                fence_proxy_async();   // the tensor core reads these generic-proxy stores
                mbar_arrive(&full[s]);
            }
        }
        // ------------------------------------------------------------------ epilogue
        // warp w may read TMEM lanes [32*(w%4), 32*(w%4)+32); lane = output row; the four warps of
        // a quadrant take one quarter of the columns each
        const int q4 = warp & 3, eh = (warp - 2) >> 2;
        const int m = mt * UT_BM + q4 * 32 + lane;
        float* dst = g.partial + ((size_t)split * g.a + (m < g.a ? m : 0)) * g.b;
        bool have = k_blocks > 0 && ok;
        if (have) have = mbar_wait(tfull, 0, abort_flag, g.status, 13);
        have = __all_sync(0xffffffffu, have);  // the TMEM loads below are warp-wide
        tc_fence_after();
        const int n0 = nt * g.bn;
        const int quarter = (g.bn / 4 + 7) / 8 * 8;
        const int j_lo = min(eh * quarter, g.bn), j_hi = eh == 3 ? g.bn : min((eh + 1) * quarter, g.bn);
        for (int j0 = j_lo; j0 < j_hi; j0 += 8) {
            uint32_t acc[8];
            if (have) {
                tmem_ld8(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)j0, acc);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                int n = n0 + j0 + j;
                if (n < g.b && m < g.a) {
                    float v = __uint_as_float(acc[j]);
                    dst[n] = g.accumulate ? dst[n] + v : v;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(g.tmem_cols)
                     : "memory");
    }
}

// grad (+)= scale * 2^(e_w - kExpA - kExpB) * sum over splits.  A block of eight warps takes 32 elements:
// warp w adds the splits w, w + 8, .. in index order, then the eight sums are added in warp order (a fixed
// order, the same on every rank).  One thread per element walking all splits had so few threads on the
// 128 x 128 layers (64 blocks) that the launch took 12 us, most of it the latency of 148 loads in a row.
__global__ void __launch_bounds__(256)
update_tc_reduce_kernel(const float* __restrict__ partial, int splits, size_t len, float scale,
                        const int* __restrict__ e_w, int accumulate, float* __restrict__ grad) {
    __shared__ float part[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t i = (size_t)blockIdx.x * 32 + lane;
    float s = 0.0f;
    if (i < len)
        for (int k = warp; k < splits; k += 8) s = __fadd_rn(s, partial[(size_t)k * len + i]);
    part[warp][lane] = s;
    __syncthreads();
    if (warp != 0 || i >= len) return;
#pragma unroll
    for (int w = 1; w < 8; ++w) s = __fadd_rn(s, part[w][lane]);
    s = __fmul_rn(ldexpf(s, *e_w - kExpA - kExpB), scale);
    grad[i] = accumulate ? __fadd_rn(grad[i], s) : s;
}

// 3-D fp32 map over (q, row, pair): `rows` rows of `rank` values per pair; box (64, box_rows, 1), no swizzle
int make_map_3d(CUtensorMap* map, const float* base, int rank, int rows, int64_t pairs, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return HSES_ERR_CUDA;
    }
    cuuint64_t dims[3] = {(cuuint64_t)rank, (cuuint64_t)rows, (cuuint64_t)pairs};
    cuuint64_t strides[2] = {(cuuint64_t)rank * 4, (cuuint64_t)rank * 4 * (cuuint64_t)rows};
    cuuint32_t box[3] = {(cuuint32_t)UT_BK, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (3-D) failed with code " + std::to_string((int)r));
        return HSES_ERR_CUDA;
    }
    return HSES_OK;
}

size_t up256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace

bool update_tc_supports(int a, int b, int rank) {
    // rows of A beyond a and rows of B beyond b are written as zeros, so only the rank is constrained
    // (rows of 16-byte multiples for the tensor map; a last k-block filled to less than three quarters
    // would mostly convert zeros)
    return a >= 1 && rank >= 48 && rank % 4 == 0 && (rank % UT_BK == 0 || rank % UT_BK >= 32) && b >= 1 &&
           b <= (1 << 20) && a <= (1 << 20);
}

UpdateTcPlan plan_update_tc(int a, int b, int rank, int64_t n, bool need_raw) {
    UpdateTcPlan p{};
    p.pairs = n / 2;
    int tiles_n = (b + 255) / 256;
    p.bn = ((b + tiles_n - 1) / tiles_n + 15) / 16 * 16;
    p.n_tiles = (b + p.bn - 1) / p.bn;
    p.m_tiles = (a + UT_BM - 1) / UT_BM;
    // without a factor cache the factors are regenerated chunk by chunk into fp32 scratch
    size_t per_pair = (size_t)(a + b) * rank * sizeof(float);
    int64_t fit = (int64_t)(kRawChunkBytes / per_pair);
    if (fit < 1) fit = 1;
    p.chunk_pairs = (need_raw && p.pairs > fit) ? fit : p.pairs;
    int tiles = p.n_tiles * p.m_tiles;
    // one CTA per SM fits (the operand stages take most of the shared memory): one full wave
    int want = plan_sm_count() / tiles;
    if (want > p.chunk_pairs) want = (int)p.chunk_pairs;
    if (want < 1) want = 1;
    p.splits = want;
    p.partial_bytes = up256((size_t)p.splits * a * b * sizeof(float));
    p.raw_bytes = need_raw ? up256((size_t)p.chunk_pairs * (a + b) * rank * sizeof(float)) : 0;
    p.bytes = 256 + p.partial_bytes + p.raw_bytes;
    return p;
}

int run_update_tc(hses_ctx* ctx, cudaStream_t st, const hses_update_args& u, float scale, bool reuse_range) {
    const int a = u.a, b = u.b, rank = u.rank;
    UpdateTcPlan p = plan_update_tc(a, b, rank, u.n, u.cache == nullptr);
    HSES_REQUIRE(u.workspace != nullptr && u.workspace_bytes >= p.bytes && ((uintptr_t)u.workspace & 255u) == 0,
                 "workspace too small or not 256-byte aligned; see hses_es_update_workspace_bytes");
    uint8_t* base = reinterpret_cast<uint8_t*>(u.workspace);
    int* e_w = reinterpret_cast<int*>(base);
    float* partial = reinterpret_cast<float*>(base + 256);
    float* raw = reinterpret_cast<float*>(base + 256 + p.partial_bytes);
    const int32_t te = true_epoch_of(u.epoch, u.noise_reuse);
    const int32_t first_pair = u.first_thread / 2;

    const float *cA = nullptr, *cB = nullptr;
    if (u.cache) {
        const hses_factor_cache& c = *u.cache;
        HSES_REQUIRE(c.data != nullptr && c.key == u.key && c.true_epoch == te && c.rank == rank && c.a == a &&
                         c.b == b,
                     "factor cache was built for another parameter, epoch bucket or shape");
        HSES_REQUIRE(first_pair >= c.first_pair && first_pair + p.pairs <= c.first_pair + c.n_pairs,
                     "factor cache does not cover these members");
        cA = c.data + (size_t)(first_pair - c.first_pair) * a * rank;
        cB = c.data + (size_t)c.n_pairs * a * rank + (size_t)(first_pair - c.first_pair) * b * rank;
    }
    if (!reuse_range) {
        HSES_KERNEL(ctx, st, "pair_weight_range");
        pair_weight_range_kernel<<<1, 1024, 0, st>>>(u.fitness, p.pairs, e_w);
        HSES_LAUNCH_CHECK();
    }
    UtArgs g{};
    g.e_w = e_w;
    g.sign_factors = u.sign_factors;
    g.a = a;
    g.b = b;
    g.rank = rank;
    g.bn = p.bn;
    g.n_tiles = p.n_tiles;
    g.splits = p.splits;
    g.tmem_cols = p.bn > 128 ? 256 : p.bn > 64 ? 128 : p.bn > 32 ? 64 : 32;
    g.partial = partial;
    g.status = ctx->t.status_word;
    const int stage_bytes = 2 * UT_BM * UT_BK * 2 + 2 * p.bn * UT_BK * 2;
    g.stages = (232448 - 2048) / stage_bytes;
    if (g.stages > 4) g.stages = 4;
    HSES_REQUIRE(g.stages >= 2, "update_tc: tile does not fit in shared memory");
    const int smem_bytes = g.stages * stage_bytes + 1024;
    HSES_CUDA(cudaFuncSetAttribute(update_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));

    int chunk_idx = 0;
    for (int64_t done = 0; done < p.pairs; done += p.chunk_pairs, ++chunk_idx) {
        const int64_t cnt = p.pairs - done < p.chunk_pairs ? p.pairs - done : p.chunk_pairs;
        if (u.cache) {
            g.A = cA + (size_t)done * a * rank;
            g.B = cB + (size_t)done * b * rank;
        } else {
            float* ra = raw;
            float* rb = raw + (size_t)cnt * a * rank;
            int rc = launch_pair_factors(ctx, st, u.key, te, first_pair + (int32_t)done, cnt, rank, a, b, nullptr, ra,
                                         rb);
            if (rc != HSES_OK) return rc;
            g.A = ra;
            g.B = rb;
        }
        g.fitness = u.fitness + 2 * done;
        g.pairs = cnt;
        g.accumulate = chunk_idx > 0;
        CUtensorMap tm_a, tm_b;
        int mrc = make_map_3d(&tm_a, g.A, rank, a, cnt, UT_BM);
        if (mrc == HSES_OK) mrc = make_map_3d(&tm_b, g.B, rank, b, cnt, p.bn);
        if (mrc != HSES_OK) return mrc;
        dim3 grid((unsigned)(p.n_tiles * p.m_tiles), (unsigned)p.splits);
        HSES_KERNEL(ctx, st, "update_tc");
        update_tc_kernel<<<grid, UT_THREADS, smem_bytes, st>>>(tm_a, tm_b, g);
        HSES_LAUNCH_CHECK();
    }
    size_t len = (size_t)a * b;
    HSES_KERNEL(ctx, st, "update_reduce");
    update_tc_reduce_kernel<<<(unsigned)((len + 31) / 32), 256, 0, st>>>(partial, p.splits, len, scale, e_w,
                                                                          u.mode == HSES_UPDATE_RAW_ACC, u.grad);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // namespace hses
