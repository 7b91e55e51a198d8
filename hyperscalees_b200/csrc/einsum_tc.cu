// Tensor-core form of the explicit-input paired einsum (einsum_pair_fused,
// hyperscalees-kernels/src/einsum_pair_fused_oxide.rs:94-227, host side hyperscalees/src/oxide.rs:318-462):
//   g_raw  = sum_k w_k a_t[k] (x) b_t[k],   w_k = s_i + s_{i+half} for the pair i that row k belongs to
//   g_ones = 2 * sum_k a_t[k] (x) b_t[k]
// over K = half * r rows that the CALLER holds as a_t (half, r, a) and b_t (half, r, b) with the
// output dimension innermost.  Both sums are one contraction
//   a_tᵀ (a, K) · [ diag(w) b_t | b_t ] (K, 2b)
// so one fp32 accumulator of 2*bn columns per 128-row output tile serves both.  The tensor core adds
// into its accumulator with truncation, an error that grows with the length of the chain: the MMAs
// therefore alternate between TWO accumulators in TMEM every ET_CHUNK k-blocks, and the converter
// warps add the finished one into the split's fp32 partial sums while the other one fills.
//
//   launches 1-3  abs_max        largest |a_t|, |b_t| and |w|: one power-of-two scale per operand
//   launch 4      einsum_tc      one CTA per (128 x bn output tile, K split), eighteen warps:
//       warp 1      TMA producer: the fp32 [64 x 128] / [64 x bn] row blocks (K outermost, as they
//                   lie in the caller's memory) through 3-D tensor maps over (column, j, i)
//       warps 2-17  converters: read the landed values TRANSPOSED (a thread owns one output
//                   column and eight consecutive K rows), scale, split into fp16 hi + lo and write
//                   128B-swizzled K-major operand tiles over the same stage; the b_t block is
//                   written twice, once multiplied by the row's weight
//       warp 0      MMA issuer: tcgen05.mma kind::f16, hi*hi + hi*lo + lo*hi, N = 2*bn
//       warps 2-17  between chunks and at the end: drain the finished accumulator into the split's
//                   partial sums (stored with the output row innermost, so a warp's 32 rows are one
//                   128-byte line)
//   launch 5      einsum_tc_reduce   adds the splits in a fixed order, undoes the scales
// The factors are read once as fp32 (output tiles that share a K range run at the same time and
// meet in L2).  No multicast, no cluster launch, bounded waits.
#include <cuda.h>
#include <cuda_fp16.h>

#include "einsum_tc.cuh"
#include "tc_common.cuh"

namespace hses {

namespace {

using namespace tc;

constexpr int ET_BM = 128;
constexpr int ET_BK = 64;
constexpr int ET_MAX_BN = 128;
constexpr int ET_THREADS = 576;  // warp 0 MMA, warp 1 TMA, warps 2-17 converters and epilogue
constexpr int ET_CONV = 512;
constexpr int ET_STAGES = 2;
constexpr int ET_CHUNK = 16;     // k-blocks (of 64 rows) accumulated in TMEM before they are added in fp32
constexpr int kExpOp = 13;       // operands are scaled into (-2^13, 2^13)

struct EtArgs {
    const float* scores;
    const unsigned* maxbits;  // [0] |a_t|, [1] |b_t|, [2] |w| as fp32 bit patterns
    int64_t half;
    int r, a, b, bn, n_tiles;
    int rb, ppb, kq;          // rows of a pair per k-block, pairs per k-block, k-blocks per pair
    int64_t blocks;           // k-blocks in all
    int splits;
    int acc_cols;             // TMEM columns of one accumulator: power of two >= 2*bn; two are allocated
    float* partial;           // [splits][2][b][a]: output row innermost
    int* status;
};

// exponent e with 2^e > v >= 2^(e-1) (0 for v = 0 or a non-finite v)
__device__ __forceinline__ int range_exp(unsigned bits) {
    float v = __uint_as_float(bits);
    int e = 0;
    if (v > 0.0f && v < INFINITY) {
        frexpf(v, &e);
        if (e > 100) e = 100;
        if (e < -100) e = -100;
    }
    return e;
}

// largest magnitude of a (n0, n1, cols) tensor with element strides (s0, s1, 1); rows 16-byte aligned;
// one warp per row at a time
__global__ void abs_max_kernel(const float* __restrict__ base, int64_t s0, int64_t s1, int64_t n0, int n1, int cols,
                               unsigned* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t rows = n0 * n1, warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    float m = 0.0f;
    for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
        const int64_t i = row / n1;
        const float* p = base + i * s0 + (row - i * n1) * s1;
        for (int c = lane * 4; c < cols; c += 128) {
            if (c + 3 < cols) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(p + c));
                m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            } else {
                for (int k = c; k < cols; ++k) m = fmaxf(m, fabsf(__ldg(p + k)));
            }
        }
    }
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if (lane == 0 && m > 0.0f) atomicMax(out, __float_as_uint(m));  // non-negative floats order like their bits
}

__global__ void weight_max_kernel(const float* __restrict__ scores, int64_t half, unsigned* __restrict__ out) {
    float m = 0.0f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < half; i += (int64_t)gridDim.x * blockDim.x)
        m = fmaxf(m, fabsf(__fadd_rn(scores[i], scores[i + half])));
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if ((threadIdx.x & 31) == 0 && m > 0.0f) atomicMax(out, __float_as_uint(m));
}

// eight scaled values -> the 16-byte hi and lo pieces (eight fp16 along K) of a K-major tile row
__device__ __forceinline__ void split8(const float (&x)[8], uint4& hi, uint4& lo) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __half2 hh = __floats2half2_rn(x[2 * j], x[2 * j + 1]);
        const float2 back = __half22float2(hh);
        const __half2 ll = __floats2half2_rn(x[2 * j] - back.x, x[2 * j + 1] - back.y);
        h[j] = *reinterpret_cast<const uint32_t*>(&hh);
        l[j] = *reinterpret_cast<const uint32_t*>(&ll);
    }
    hi = make_uint4(h[0], h[1], h[2], h[3]);
    lo = make_uint4(l[0], l[1], l[2], l[3]);
}
// row `row` of a 128B-swizzled K-major tile is 128 bytes; its 16-byte piece c sits at piece c ^ (row % 8)
__device__ __forceinline__ int piece_off(int row, int piece) {
    return (row >> 3) * 1024 + (row & 7) * 128 + ((piece ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__(ET_THREADS, 1)
einsum_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const EtArgs g) {
    extern __shared__ __align__(1024) uint8_t smem[];
    // stage: [A fp32 64x128 -> A hi | A lo] [B fp32 64xbn -> (wB | B) hi] [(wB | B) lo]
    const int a_tile = ET_BM * ET_BK * 2, bx_tile = 2 * g.bn * ET_BK * 2;
    const int stage_bytes = 2 * a_tile + 2 * bx_tile;
    uint8_t* tail = smem + (size_t)ET_STAGES * stage_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
    uint64_t* full = bars;          // [stages] tiles converted
    uint64_t* empty = bars + 2;     // [stages] MMAs finished reading the stage
    uint64_t* landed = bars + 4;    // [stages] fp32 blocks arrived
    uint64_t* readdone = bars + 6;  // [stages] every converter has read its fp32 values
    uint64_t* tfull = bars + 8;     // [2] the chunk in this accumulator is complete
    uint64_t* tempty = bars + 10;   // [2] the accumulator has been drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    float* wrow = reinterpret_cast<float*>(tail + 128);  // [stages][64] row weights, scaled into (-1, 1)
    __shared__ int abort_flag_s;
    volatile int* abort_flag = &abort_flag_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int mt = tile / g.n_tiles, nt = tile - mt * g.n_tiles;
    const int64_t b_lo = g.blocks * split / g.splits, b_hi = g.blocks * (split + 1) / g.splits;
    const int64_t k_blocks = b_hi - b_lo;

    if (threadIdx.x == 0) {
        abort_flag_s = 0;
        for (int s = 0; s < ET_STAGES; ++s) {
            mbar_init(&full[s], ET_CONV);
            mbar_init(&empty[s], 1);
            mbar_init(&landed[s], 1);
            mbar_init(&readdone[s], ET_CONV);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&tfull[t], 1);
            mbar_init(&tempty[t], ET_CONV);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(2 * g.acc_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc(2 * g.bn);
            bool ok = true;
            for (int64_t it = 0; it < k_blocks; ++it) {
                const int s = (int)(it % ET_STAGES);
                const uint32_t ph = (uint32_t)(it / ET_STAGES) & 1;
                const int64_t chunk = it / ET_CHUNK;
                const int in_chunk = (int)(it - chunk * ET_CHUNK);
                const uint32_t acc = tmem_base + (uint32_t)(chunk & 1) * (uint32_t)g.acc_cols;
                if (in_chunk == 0 && chunk >= 2 &&
                    !mbar_wait(&tempty[chunk & 1], (uint32_t)((chunk >> 1) & 1) ^ 1, abort_flag, g.status, 10)) {
                    ok = false;
                    break;
                }
                if (!mbar_wait(&full[s], ph, abort_flag, g.status, 12)) { ok = false; break; }
                tc_fence_after();
                uint8_t* st = smem + (size_t)s * stage_bytes;
                const uint64_t dah = make_smem_desc(st), dal = make_smem_desc(st + a_tile);
                const uint64_t dbh = make_smem_desc(st + 2 * a_tile), dbl = make_smem_desc(st + 2 * a_tile + bx_tile);
#pragma unroll
                for (int ks = 0; ks < ET_BK / 16; ++ks) {
                    const uint64_t off = (uint64_t)(ks * 32 >> 4);  // 16 fp16 = 32 B along K
                    umma_f16(acc, dal + off, dbh + off, idesc, (in_chunk | ks) != 0);
                    umma_f16(acc, dah + off, dbl + off, idesc, 1);
                    umma_f16(acc, dah + off, dbh + off, idesc, 1);
                }
                umma_commit(&empty[s]);
                if (in_chunk == ET_CHUNK - 1 || it == k_blocks - 1) umma_commit(&tfull[chunk & 1]);
            }
            (void)ok;
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            for (int64_t it = 0; it < k_blocks; ++it) {
                const int s = (int)(it % ET_STAGES);
                const uint32_t ph = (uint32_t)(it / ET_STAGES) & 1;
                if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, g.status, 11)) { ok = false; break; }
                const int64_t blk = b_lo + it;
                int c1, c2;   // row inside the pair, pair
                if (g.ppb > 1) {
                    c1 = 0;
                    c2 = (int)(blk * g.ppb);
                } else {
                    c2 = (int)(blk / g.kq);
                    c1 = (int)(blk - (int64_t)c2 * g.kq) * ET_BK;
                }
                uint8_t* st = smem + (size_t)s * stage_bytes;
                // boxes count in full, zero fill of rows and columns outside the tensor included
                mbar_expect_tx(&landed[s], (uint32_t)(ET_BM * ET_BK * 4 + g.bn * ET_BK * 4));
                tma_load_3d(st, &tm_a, mt * ET_BM, c1, c2, &landed[s]);
                tma_load_3d(st + 2 * a_tile, &tm_b, nt * g.bn, c1, c2, &landed[s]);
            }
            if (!ok) {
                // copies already issued still land in this CTA's shared memory: give them a bounded moment
                for (int s = 0; s < ET_STAGES; ++s)
                    for (uint32_t i = 0; i < 4096; ++i) {
                        if (mbar_try(&landed[s], 0) || mbar_try(&landed[s], 1)) break;
                        __nanosleep(256);
                    }
            }
        }
    } else {
        // ------------------------------------------------------------------ converters
        const int ct = threadIdx.x - 64;  // 0..511
        const int e_a = range_exp(g.maxbits[0]), e_b = range_exp(g.maxbits[1]), e_w = range_exp(g.maxbits[2]);
        const float sc_a = ldexpf(1.0f, kExpOp - e_a), sc_b = ldexpf(1.0f, kExpOp - e_b), sc_w = ldexpf(1.0f, -e_w);
        const int am = ct & 127, akg = ct >> 7;   // A: output row am, K groups akg and akg + 4
        const int b_units = g.bn * 8;             // B: unit = (K group, column)
        int bn_[2], bkg[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int id = ct + ET_CONV * u;
            bkg[u] = id / g.bn;
            bn_[u] = id - bkg[u] * g.bn;
            if (id >= b_units) bkg[u] = -1;
        }
        // Adds the accumulator of chunk c into the split's partial sums (the first chunk stores).  Warp w
        // may read TMEM lanes [32*(w%4), 32*(w%4)+32); lane = output row; the four warps of a quadrant
        // take one quarter of the 2*bn columns each (columns bn.. are the unweighted sum).  A chunk that
        // cannot be had (a wait ran out somewhere) counts as zeros, so the sums stay finite.
        const int q4 = warp & 3, eh = (warp - 2) >> 2;
        const int m = mt * ET_BM + q4 * 32 + lane;
        const size_t len = (size_t)g.a * g.b;
        float* const praw = g.partial + (size_t)split * 2 * len + (m < g.a ? m : 0);
        const int n0 = nt * g.bn, quarter = g.bn / 2;   // bn is a multiple of 16: quarters of whole 8-column groups
        auto drain = [&](int64_t c, bool good) {
            const int t = (int)(c & 1);
            bool have = good;
            if (have) have = mbar_wait(&tfull[t], (uint32_t)(c >> 1) & 1, abort_flag, g.status, 13);
            have = __all_sync(0xffffffffu, have);  // the TMEM loads below are warp-wide
            tc_fence_after();
            const uint32_t acc = tmem_base + (uint32_t)t * (uint32_t)g.acc_cols + ((uint32_t)(q4 * 32) << 16);
            for (int j0 = eh * quarter; j0 < (eh + 1) * quarter; j0 += 8) {
                uint32_t v[8];
                if (have) {
                    tmem_ld8(acc + (uint32_t)j0, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = 0u;
                }
                const bool ones = j0 >= g.bn;
                float* dst = (ones ? praw + len : praw) + (size_t)(n0 + j0 - (ones ? g.bn : 0)) * g.a;
                // One thread owns an address for the whole kernel: the first chunk stores, later ones add
                // with a reduction that returns nothing (no load round trip); operations of one thread
                // on one address keep their order, so the sum is the same on every run.
                if (m < g.a) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (n0 + j0 + j - (ones ? g.bn : 0) >= g.b) continue;
                        if (c == 0)
                            dst[(size_t)j * g.a] = __uint_as_float(v[j]);
                        else
                            asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + (size_t)j * g.a), "f"(__uint_as_float(v[j]))
                                         : "memory");
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&tempty[t]);
        };
        bool ok = true;
        for (int64_t it = 0; it < k_blocks; ++it) {
            const int s = (int)(it % ET_STAGES);
            const uint32_t ph = (uint32_t)(it / ET_STAGES) & 1;
            if (it > 0 && it % ET_CHUNK == 0) drain(it / ET_CHUNK - 1, true);
            if (!mbar_wait(&landed[s], ph, abort_flag, g.status, 14)) { ok = false; break; }
            uint8_t* st = smem + (size_t)s * stage_bytes;
            const float* a32 = reinterpret_cast<const float*>(st);
            const float* b32 = reinterpret_cast<const float*>(st + 2 * a_tile);
            float* wr = wrow + s * ET_BK;
            if (ct < ET_BK) {   // the weight of K row ct of this block
                const int64_t blk = b_lo + it;
                const int64_t i = g.ppb > 1 ? blk * g.ppb + ct / g.rb : blk / g.kq;
                wr[ct] = i < g.half ? __fmul_rn(__fadd_rn(g.scores[i], g.scores[i + g.half]), sc_w) : 0.0f;
            }
            float va[2][8], vb[2][8];
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int j = 0; j < 8; ++j) va[u][j] = a32[((akg + 4 * u) * 8 + j) * ET_BM + am];
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int j = 0; j < 8; ++j) vb[u][j] = bkg[u] >= 0 ? b32[(bkg[u] * 8 + j) * g.bn + bn_[u]] : 0.0f;
            // the fp16 tiles overwrite the fp32 values: every converter must have read first (an
            // mbarrier with a bounded wait: a role that gave up must not leave the others parked)
            mbar_arrive(&readdone[s]);
            if (!mbar_wait(&readdone[s], ph, abort_flag, g.status, 15)) { ok = false; break; }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                float x[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) x[j] = __fmul_rn(va[u][j], sc_a);
                uint4 hi, lo;
                split8(x, hi, lo);
                const int off = piece_off(am, akg + 4 * u);
                *reinterpret_cast<uint4*>(st + off) = hi;
                *reinterpret_cast<uint4*>(st + a_tile + off) = lo;
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (bkg[u] < 0) continue;
                float x[8], xw[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    x[j] = __fmul_rn(vb[u][j], sc_b);
                    xw[j] = __fmul_rn(__fmul_rn(vb[u][j], wr[bkg[u] * 8 + j]), sc_b);   // the power of two is exact
                }
                uint4 hi, lo;
                uint8_t* bh = st + 2 * a_tile;
                split8(xw, hi, lo);
                int off = piece_off(bn_[u], bkg[u]);
                *reinterpret_cast<uint4*>(bh + off) = hi;
                *reinterpret_cast<uint4*>(bh + bx_tile + off) = lo;
                split8(x, hi, lo);
                off = piece_off(g.bn + bn_[u], bkg[u]);
                *reinterpret_cast<uint4*>(bh + off) = hi;
                *reinterpret_cast<uint4*>(bh + bx_tile + off) = lo;
            }
            fence_proxy_async();   // the tensor core reads these generic-proxy stores
            mbar_arrive(&full[s]);
        }
        if (k_blocks > 0) drain((k_blocks - 1) / ET_CHUNK, ok);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * g.acc_cols)
                     : "memory");
    }
}

// sums the splits in index order and undoes the operand scales
__global__ void einsum_tc_reduce_kernel(const float* __restrict__ partial, int splits, size_t len, int a, int b,
                                        const unsigned* __restrict__ maxbits, float* __restrict__ g_raw,
                                        float* __restrict__ g_ones) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= len) return;
    const int e_ab = range_exp(maxbits[0]) + range_exp(maxbits[1]) - 2 * kExpOp, e_w = range_exp(maxbits[2]);
    const size_t m = i / (size_t)b, it = (i - m * (size_t)b) * (size_t)a + m;   // partial sums hold the row innermost
    float sr = 0.0f, so = 0.0f;
    for (int k = 0; k < splits; ++k) {
        sr = __fadd_rn(sr, partial[(size_t)k * 2 * len + it]);
        so = __fadd_rn(so, partial[(size_t)k * 2 * len + len + it]);
    }
    g_raw[i] = ldexpf(sr, e_ab + e_w);
    g_ones[i] = ldexpf(so, e_ab + 1);
}

// 3-D fp32 map over (column, j, i) of a (half, r, cols) tensor with element strides (s0, s1, 1)
int make_map_cols(CUtensorMap* map, const float* base, int64_t s0, int64_t s1, int64_t half, int r, int cols,
                  int box_cols, int box_rows, int box_pairs) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return HSES_ERR_CUDA;
    }
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)r, (cuuint64_t)half};
    cuuint64_t strides[2] = {(cuuint64_t)s1 * 4, (cuuint64_t)s0 * 4};
    cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, (cuuint32_t)box_pairs};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (einsum_pair) failed with code " + std::to_string((int)rc));
        return HSES_ERR_CUDA;
    }
    return HSES_OK;
}

size_t up256e(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace

bool einsum_tc_supports(const float* a_t, int64_t a_s0, int64_t a_s1, const float* b_t, int64_t b_s0, int64_t b_s1,
                        int64_t half, int r, int a, int b) {
    // tensor maps: 16-byte aligned base and strides, strides below 2^40 bytes, positive pair stride
    auto ok_map = [](const float* p, int64_t s0, int64_t s1) {
        return ((uintptr_t)p & 15u) == 0 && s0 % 4 == 0 && s1 % 4 == 0 && s0 > 0 && s1 > 0 && s0 < (1ll << 37) &&
               s1 < (1ll << 37);
    };
    if (!ok_map(a_t, a_s0, a_s1) || !ok_map(b_t, b_s0, b_s1)) return false;
    // a k-block is 64 rows: whole pairs when r divides 64, else the rows of one pair (zero-filled past r)
    if (!(r >= 32 || 64 % r == 0)) return false;
    if (half >= (1ll << 31) || a > (1 << 20) || b > (1 << 20)) return false;
    // short contractions stay on the fp32 kernel: set-up and the three range launches would dominate
    return half * r >= 32768 && (int64_t)a * b >= 1024;
}

EinsumTcPlan plan_einsum_tc(int64_t half, int r, int a, int b) {
    EinsumTcPlan p{};
    const int tiles_n = (b + ET_MAX_BN - 1) / ET_MAX_BN;
    p.bn = ((b + tiles_n - 1) / tiles_n + 15) / 16 * 16;
    p.n_tiles = (b + p.bn - 1) / p.bn;
    p.m_tiles = (a + ET_BM - 1) / ET_BM;
    if (r < 64 && 64 % r == 0) {
        p.rb = r;
        p.ppb = 64 / r;
        p.kq = 1;
        p.blocks = (half + p.ppb - 1) / p.ppb;
    } else {
        p.rb = 64;
        p.ppb = 1;
        p.kq = (r + 63) / 64;
        p.blocks = half * p.kq;
    }
    const int tiles = p.n_tiles * p.m_tiles;
    int64_t want = plan_sm_count() / tiles;   // one CTA per SM fits: one full wave
    if (want > p.blocks / 4) want = p.blocks / 4;   // at least four k-blocks per split
    if (want > 1024) want = 1024;
    if (want < 1) want = 1;
    p.splits = (int)want;
    p.bytes = 256 + up256e((size_t)p.splits * 2 * (size_t)a * b * sizeof(float));
    return p;
}

int run_einsum_tc(hses_ctx* ctx, cudaStream_t st, const float* a_t, int64_t a_s0, int64_t a_s1, const float* b_t,
                  int64_t b_s0, int64_t b_s1, const float* scores, int64_t half, int r, int a, int b, float* g_raw,
                  float* g_ones, void* workspace, size_t workspace_bytes) {
    const EinsumTcPlan p = plan_einsum_tc(half, r, a, b);
    HSES_REQUIRE(workspace != nullptr && workspace_bytes >= p.bytes && ((uintptr_t)workspace & 255u) == 0,
                 "workspace too small or not 256-byte aligned; see hses_einsum_pair_workspace_bytes");
    unsigned* maxbits = reinterpret_cast<unsigned*>(workspace);
    float* partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + 256);
    HSES_CUDA(cudaMemsetAsync(maxbits, 0, 16, st));
    const int sms = plan_sm_count();
    {
        HSES_KERNEL(ctx, st, "einsum_abs_max");
        abs_max_kernel<<<sms * 8, 256, 0, st>>>(a_t, a_s0, a_s1, half, r, a, maxbits);
        HSES_LAUNCH_CHECK();
    }
    {
        HSES_KERNEL(ctx, st, "einsum_abs_max");
        abs_max_kernel<<<sms * 8, 256, 0, st>>>(b_t, b_s0, b_s1, half, r, b, maxbits + 1);
        HSES_LAUNCH_CHECK();
    }
    {
        HSES_KERNEL(ctx, st, "einsum_weight_max");
        const int64_t want = (half + 255) / 256;
        weight_max_kernel<<<(unsigned)(want < sms ? want : sms), 256, 0, st>>>(scores, half, maxbits + 2);
        HSES_LAUNCH_CHECK();
    }
    EtArgs g{};
    g.scores = scores;
    g.maxbits = maxbits;
    g.half = half;
    g.r = r;
    g.a = a;
    g.b = b;
    g.bn = p.bn;
    g.n_tiles = p.n_tiles;
    g.rb = p.rb;
    g.ppb = p.ppb;
    g.kq = p.kq;
    g.blocks = p.blocks;
    g.splits = p.splits;
    g.acc_cols = 2 * p.bn > 128 ? 256 : 2 * p.bn > 64 ? 128 : 2 * p.bn > 32 ? 64 : 32;
    g.partial = partial;
    g.status = ctx->t.status_word;
    const int stage_bytes = 2 * ET_BM * ET_BK * 2 + 2 * (2 * p.bn * ET_BK * 2);
    const int smem_bytes = ET_STAGES * stage_bytes + 128 + ET_STAGES * ET_BK * 4 + 1024;
    HSES_CUDA(cudaFuncSetAttribute(einsum_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    CUtensorMap tm_a, tm_b;
    int mrc = make_map_cols(&tm_a, a_t, a_s0, a_s1, half, r, a, ET_BM, p.rb, p.ppb);
    if (mrc == HSES_OK) mrc = make_map_cols(&tm_b, b_t, b_s0, b_s1, half, r, b, p.bn, p.rb, p.ppb);
    if (mrc != HSES_OK) return mrc;
    {
        dim3 grid((unsigned)(p.n_tiles * p.m_tiles), (unsigned)p.splits);
        HSES_KERNEL(ctx, st, "einsum_tc");
        einsum_tc_kernel<<<grid, ET_THREADS, smem_bytes, st>>>(tm_a, tm_b, g);
        HSES_LAUNCH_CHECK();
    }
    const size_t len = (size_t)a * b;
    HSES_KERNEL(ctx, st, "einsum_pair_reduce");
    einsum_tc_reduce_kernel<<<(unsigned)((len + 255) / 256), 256, 0, st>>>(partial, p.splits, len, a, b, maxbits, g_raw,
                                                                          g_ones);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // namespace hses
