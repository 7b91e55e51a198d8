// Perturbed linear layer y = x·Wᵀ + (x·B_i)·A_iᵀ for a whole population
// (do_mm, hyperscalees-noiser/src/eggroll.rs:419-446) with an optional fused
// LIF step (lif_step, hyperscalees-models/src/snn.rs:53-65).
//
// This file holds the dispatcher and the general fp32 SIMT path, which takes
// any shape and pitch.  The tensor-core path for tile-aligned shapes lives in
// linear_tc.cu.
#include <cuda_fp16.h>

#include "common.cuh"
#include "linear.cuh"

namespace hses {

// ---------------------------------------------------------------------------
// SIMT path, three launches:
//   1. raw factors of every antithetic pair into scratch (pair-folded: the
//      two members of a pair share one draw, eggroll.rs:60-65);
//   2. t = x·B_pair, (rows, r);
//   3. tiled fp32 GEMM x·Wᵀ whose epilogue adds t·(±sigma/sqrt(r)·A_pair)ᵀ
//      and applies the LIF step.
// ---------------------------------------------------------------------------

// scratch layout: A (pairs, a, r) | B (pairs, b, r) | t (rows, r)
struct SimtScratch {
    float* A;
    float* B;
    float* t;
    size_t bytes;
};
static SimtScratch simt_scratch(const hses_linear_args& g, void* base) {
    int64_t first_pair = g.first_thread / 2;
    int64_t last_pair = (g.first_thread + g.n_pop - 1) / 2;
    size_t pairs = (size_t)(last_pair - first_pair + 1);
    size_t rows = (size_t)g.t_steps * g.n_pop * g.bm;
    size_t na = pairs * g.a * g.rank, nb = pairs * g.k * g.rank, nt = rows * g.rank;
    auto up = [](size_t v) { return (v + 63) / 64 * 64; };
    SimtScratch s;
    s.A = reinterpret_cast<float*>(base);
    s.B = s.A + up(na);
    s.t = s.B + up(nb);
    s.bytes = (up(na) + up(nb) + up(nt)) * sizeof(float);
    return s;
}

// t[R, q] = sum_k x[R, k] * B_pair(R)[k, q]; one warp per row, lanes over k.
__global__ void lowrank_project_kernel(const float* __restrict__ x, int64_t rows, int bm,
                                       int64_t n_pop, int k, int64_t x_stride, int rank,
                                       int32_t first_thread, int32_t first_pair,
                                       const float* __restrict__ B, float* __restrict__ t) {
    int64_t R = (int64_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    int lane = threadIdx.x & 31;
    if (R >= rows) return;
    int64_t member = (R / bm) % n_pop;
    int64_t pair = (first_thread + member) / 2 - first_pair;
    const float* xr = x + (size_t)R * x_stride;
    const float* Bp = B + (size_t)pair * k * rank;
    for (int q0 = 0; q0 < rank; q0 += 8) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
        for (int kk = lane; kk < k; kk += 32) {
            float xv = xr[kk];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (q0 + j < rank) acc[j] = fmaf(xv, Bp[(size_t)kk * rank + q0 + j], acc[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float v = acc[j];
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0 && q0 + j < rank) t[(size_t)R * rank + q0 + j] = v;
        }
    }
}

constexpr int TM = 128, TK = 16, TT = 256;  // row tile, k step, threads (the column tile is 16 * NJ)

struct EpilogueArgs {
    int perturb, lif, reset;
    float base_sigma, leak, v_th, out_scale;
    const float* out_scale_ptr;
    int rank, bm;
    int64_t n_pop;
    int32_t first_thread, first_pair;
    const float* A;  // (pairs, a, r)
    const float* t;  // (rows, r)
    float* out;
    int64_t out_stride;
    float* pot;
};

// NJ = output columns per thread: 8 (a 128-column tile: columns {tc..tc+3, 64+tc..64+tc+3}) or, for
// narrow layers, 4, 2 or 1 consecutive columns (tiles of 64, 32, 16 columns), so that a 16-wide
// projection does not pay for a 128-wide tile.  The k loop of an output is the same in every form.
template <int NJ>
__global__ void __launch_bounds__(TT, 2)
linear_simt_kernel(const float* __restrict__ x, int64_t rows, int k, int64_t x_stride,
                   const float* __restrict__ w, int a, int64_t w_stride, EpilogueArgs ep) {
    constexpr int TNJ = 16 * NJ;
    __shared__ __align__(16) float sx[TK][TM + 4];
    __shared__ __align__(16) float sw[TK][TNJ + 4];
    int64_t row0 = (int64_t)blockIdx.y * TM;
    int col0 = blockIdx.x * TNJ;
    int tid = threadIdx.x;
    // a thread owns rows {tr..tr+3, 64+tr..64+tr+3} and (NJ = 8) the same pattern of
    // columns, so its shared-memory reads are two conflict-free float4 loads
    int tr = (tid / 16) * 4, tc = (tid % 16) * (NJ == 8 ? 4 : NJ);
    float acc[8][NJ];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < NJ; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < k; k0 += TK) {
        // each thread loads 8 elements of each tile: element e -> (row e/16, k e%16)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            int idx = tid + e * TT;
            int r = idx / TK, kk = idx % TK;
            int64_t gr = row0 + r;
            sx[kk][r] = (gr < rows && k0 + kk < k) ? x[(size_t)gr * x_stride + k0 + kk] : 0.0f;
            if (r < TNJ) {
                int gc = col0 + r;
                sw[kk][r] = (gc < a && k0 + kk < k) ? w[(size_t)gc * w_stride + k0 + kk] : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float xa[8], wb[NJ];
            *reinterpret_cast<float4*>(&xa[0]) = *reinterpret_cast<const float4*>(&sx[kk][tr]);
            *reinterpret_cast<float4*>(&xa[4]) = *reinterpret_cast<const float4*>(&sx[kk][64 + tr]);
            if (NJ == 8) {
                *reinterpret_cast<float4*>(&wb[0]) = *reinterpret_cast<const float4*>(&sw[kk][tc]);
                *reinterpret_cast<float4*>(&wb[NJ == 8 ? 4 : 0]) = *reinterpret_cast<const float4*>(&sw[kk][64 + tc]);
            } else {
#pragma unroll
                for (int j = 0; j < NJ; ++j) wb[j] = sw[kk][tc + j];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < NJ; ++j) acc[i][j] = fmaf(xa[i], wb[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int64_t R = row0 + (i < 4 ? tr + i : 64 + tr + i - 4);
        if (R >= rows) continue;
        const float* Ap = nullptr;
        const float* tr_ = nullptr;
        float scale = 0.0f;
        if (ep.perturb) {
            int64_t member = (R / ep.bm) % ep.n_pop;
            int32_t thread_id = ep.first_thread + (int32_t)member;
            Ap = ep.A + (size_t)(thread_id / 2 - ep.first_pair) * a * ep.rank;
            tr_ = ep.t + (size_t)R * ep.rank;
            scale = (thread_id % 2 == 0) ? ep.base_sigma : -ep.base_sigma;
        }
        // u[j] = sum_q t[R][q] * (scale * A[n_j][q]), q ascending; with a rank that is a multiple of
        // four the row of t and the rows of A are read as 16-byte pieces, once per row and column
        float u[NJ];
#pragma unroll
        for (int j = 0; j < NJ; ++j) u[j] = 0.0f;
        if (ep.perturb) {
            const bool vec = (ep.rank & 3) == 0 && (((uintptr_t)ep.A | (uintptr_t)ep.t) & 15u) == 0;
            if (vec) {
                for (int q4 = 0; q4 < ep.rank; q4 += 4) {
                    const float4 t4 = *reinterpret_cast<const float4*>(tr_ + q4);
#pragma unroll
                    for (int j = 0; j < NJ; ++j) {
                        int n = col0 + (NJ == 8 ? (j < 4 ? tc + j : 64 + tc + j - 4) : tc + j);
                        if (n >= a) n = a - 1;
                        const float4 a4 = *reinterpret_cast<const float4*>(Ap + (size_t)n * ep.rank + q4);
                        u[j] = fmaf(t4.x, __fmul_rn(a4.x, scale), u[j]);
                        u[j] = fmaf(t4.y, __fmul_rn(a4.y, scale), u[j]);
                        u[j] = fmaf(t4.z, __fmul_rn(a4.z, scale), u[j]);
                        u[j] = fmaf(t4.w, __fmul_rn(a4.w, scale), u[j]);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    int n = col0 + (NJ == 8 ? (j < 4 ? tc + j : 64 + tc + j - 4) : tc + j);
                    if (n >= a) continue;
                    for (int q = 0; q < ep.rank; ++q)
                        u[j] = fmaf(tr_[q], __fmul_rn(Ap[(size_t)n * ep.rank + q], scale), u[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            int n = col0 + (NJ == 8 ? (j < 4 ? tc + j : 64 + tc + j - 4) : tc + j);
            if (n >= a) continue;
            float y = acc[i][j];
            if (ep.perturb) y = __fadd_rn(y, u[j]);
            size_t o = (size_t)R * ep.out_stride + n;
            if (ep.lif) {
                // lif_step from v = 0: charged = 0 + ((-0) + y) * leak
                float c = __fmul_rn(y, ep.leak);
                if (ep.pot) ep.pot[o] = c;
                ep.out[o] = c >= ep.v_th ? 1.0f : 0.0f;
            } else {
                ep.out[o] = __fmul_rn(y, ep.out_scale_ptr ? *ep.out_scale_ptr : ep.out_scale);
            }
        }
    }
}

static int check_args(const hses_linear_args* g) {
    HSES_REQUIRE(g != nullptr, "args is NULL");
    HSES_REQUIRE(g->t_steps >= 1 && g->n_pop >= 1 && g->bm >= 1 && g->k >= 1 && g->a >= 1, "bad shape");
    HSES_REQUIRE(g->x_row_stride >= g->k && g->param_row_stride >= g->k && g->out_row_stride >= g->a,
                 "row stride smaller than the row");
    HSES_REQUIRE((double)g->t_steps * (double)g->n_pop * g->bm < 2147483648.0, "too many rows");
    HSES_REQUIRE(g->x != nullptr && g->param != nullptr && g->out != nullptr, "NULL pointer");
    HSES_REQUIRE(g->precision == HSES_PRECISION_FP32 || g->precision == HSES_PRECISION_BF16, "unknown precision");
    HSES_REQUIRE(g->factor_order == 0 || g->factor_order == 1, "unknown factor order");
    HSES_REQUIRE(!(g->factor_order == 1 && g->cache != nullptr), "a factor cache holds the do_mm order only");
    if (g->perturb) {
        HSES_REQUIRE(g->rank >= 1 && g->rank <= 1024, "rank out of range");
        HSES_REQUIRE(g->first_thread >= 0 && g->noise_reuse >= 0, "negative thread id or noise_reuse");
        HSES_REQUIRE((int64_t)g->first_thread + g->n_pop < (1ll << 31), "thread id overflow");
    }
    if (g->lif) {
        HSES_REQUIRE(g->tau_m != 0.0f, "tau_m must be non-zero");
        HSES_REQUIRE(g->reset_mode == HSES_RESET_HARD || g->reset_mode == HSES_RESET_SUBTRACT,
                     "bad reset mode");
    }
    HSES_REQUIRE(g->algo >= HSES_ALGO_AUTO && g->algo <= HSES_ALGO_PAIR, "unknown algo");
    return HSES_OK;
}

int resolve_factor_cache(const hses_linear_args& g, const float** A, const float** B) {
    HSES_REQUIRE(g.cache != nullptr && g.cache->data != nullptr, "factor cache is NULL");
    const hses_factor_cache& c = *g.cache;
    const int groups = g.n_groups > 1 ? g.n_groups : 1;   // grouped layout: B is (n_pairs, groups, k, rank)
    HSES_REQUIRE(c.key == g.key && c.true_epoch == true_epoch_of(g.epoch, g.noise_reuse) &&
                     c.rank == g.rank && c.a == g.a && c.b == g.k * groups,
                 "factor cache was built for another parameter, epoch bucket or shape");
    int32_t first_pair = g.first_thread / 2;
    int64_t last_pair = ((int64_t)g.first_thread + g.n_pop - 1) / 2;
    HSES_REQUIRE(first_pair >= c.first_pair && last_pair < (int64_t)c.first_pair + c.n_pairs,
                 "factor cache does not cover these members");
    size_t off = (size_t)(first_pair - c.first_pair);
    *A = c.data + off * c.a * c.rank;
    *B = c.data + (size_t)c.n_pairs * c.a * c.rank + off * c.b * c.rank;
    return HSES_OK;
}

static int run_simt(hses_ctx* ctx, cudaStream_t st, const hses_linear_args& g) {
    int64_t rows = (int64_t)g.t_steps * g.n_pop * g.bm;
    EpilogueArgs ep{};
    ep.perturb = g.perturb;
    ep.lif = g.lif;
    ep.reset = g.reset_mode;
    ep.rank = g.rank;
    ep.bm = g.bm;
    ep.n_pop = g.n_pop;
    ep.first_thread = g.first_thread;
    ep.first_pair = g.first_thread / 2;
    ep.out = g.out;
    ep.out_stride = g.out_row_stride;
    ep.pot = g.lif ? g.potentials : nullptr;
    ep.leak = g.lif ? 1.0f / g.tau_m : 0.0f;
    ep.v_th = g.v_th;
    ep.out_scale = g.out_scale;
    ep.out_scale_ptr = g.out_scale_ptr;
    if (g.perturb) {
        SimtScratch s = simt_scratch(g, g.workspace);
        HSES_REQUIRE(g.workspace != nullptr && g.workspace_bytes >= s.bytes,
                     "workspace too small; see hses_perturbed_linear_workspace_bytes");
        ep.base_sigma = g.sigma / sqrtf((float)g.rank);
        ep.t = s.t;
        const float *fa = s.A, *fb = s.B;
        if (g.cache) {
            int rc = resolve_factor_cache(g, &fa, &fb);
            if (rc != HSES_OK) return rc;
        } else {
            int64_t pairs = (g.first_thread + g.n_pop - 1) / 2 - ep.first_pair + 1;
            // do_Tmm order: the output-side rows lead the stream, the input-side rows follow
            int rc = g.factor_order == 1
                         ? launch_pair_factors(ctx, st, g.key, true_epoch_of(g.epoch, g.noise_reuse), ep.first_pair, pairs,
                                               g.rank, g.k, g.a, nullptr, s.B, s.A)
                         : launch_pair_factors(ctx, st, g.key, true_epoch_of(g.epoch, g.noise_reuse), ep.first_pair, pairs,
                                               g.rank, g.a, g.k, nullptr, s.A, s.B);
            if (rc != HSES_OK) return rc;
        }
        ep.A = fa;
        HSES_KERNEL(ctx, st, "lowrank_project");
        lowrank_project_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(
            g.x, rows, g.bm, g.n_pop, g.k, g.x_row_stride, g.rank, g.first_thread, ep.first_pair,
            fb, s.t);
        HSES_LAUNCH_CHECK();
    }
    int64_t row_tiles = (rows + TM - 1) / TM;
    HSES_REQUIRE(row_tiles <= 65535ll * 32768ll, "too many rows");
    HSES_REQUIRE(row_tiles <= 65535, "too many rows for the SIMT path (rows/128 must be <= 65535)");
    HSES_KERNEL(ctx, st, "linear_simt");
    // narrow layers take a narrower column tile
    const int nj = g.a <= 16 ? 1 : g.a <= 32 ? 2 : g.a <= 64 ? 4 : 8;
    dim3 grid((unsigned)((g.a + 16 * nj - 1) / (16 * nj)), (unsigned)row_tiles);
    if (nj == 1)
        linear_simt_kernel<1><<<grid, TT, 0, st>>>(g.x, rows, g.k, g.x_row_stride, g.param, g.a, g.param_row_stride, ep);
    else if (nj == 2)
        linear_simt_kernel<2><<<grid, TT, 0, st>>>(g.x, rows, g.k, g.x_row_stride, g.param, g.a, g.param_row_stride, ep);
    else if (nj == 4)
        linear_simt_kernel<4><<<grid, TT, 0, st>>>(g.x, rows, g.k, g.x_row_stride, g.param, g.a, g.param_row_stride, ep);
    else
        linear_simt_kernel<8><<<grid, TT, 0, st>>>(g.x, rows, g.k, g.x_row_stride, g.param, g.a, g.param_row_stride, ep);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

// spikes (0/1 in f32, pitched rows) once more as dense fp16 rows; a is a multiple of 8
__global__ void spikes_to_half_kernel(const float* __restrict__ src, int64_t rows, int a, int64_t stride,
                                      __half* __restrict__ dst) {
    const int a8 = a >> 3;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * a8) return;
    const int64_t r = i / a8;
    const int c = (int)(i - r * a8) * 8;
    const float4 v0 = *reinterpret_cast<const float4*>(src + r * stride + c);
    const float4 v1 = *reinterpret_cast<const float4*>(src + r * stride + c + 4);
    const __half2 h0 = __floats2half2_rn(v0.x, v0.y), h1 = __floats2half2_rn(v0.z, v0.w);
    const __half2 h2 = __floats2half2_rn(v1.x, v1.y), h3 = __floats2half2_rn(v1.z, v1.w);
    *reinterpret_cast<uint4*>(dst + r * a + c) =
        make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                   *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
}

// Narrow layers (at most 64 inputs and outputs) stay on the kernel that keeps W in shared memory when a
// pair owns few rows; with many rows per pair the tensor-core path, which also takes narrow outputs, is
// the faster one — by 2.4x when the factors come from a cache; when they have to be regenerated it
// regenerates the output-side factor once per 128-row tile and is the slower one, but the choice must
// not depend on the cache: a call with and without one returns the same bits.
static bool prefers_small_path(const hses_linear_args& g) {
    if (g.algo != HSES_ALGO_AUTO || g.lif == 2 || !small_path_supports(g)) return false;
    return (int64_t)2 * g.bm * g.t_steps <= 256;
}

// does the call end in the per-pair kernel with the scan inside it (the one kernel that writes out_half itself)?
static bool ends_in_pair_scan(const hses_linear_args& g) {
    if (g.lif != 2) return false;
    const bool pair_ok = pair_path_supports(g);
    const bool takes_pair = (g.algo == HSES_ALGO_PAIR && pair_ok) ||
                            (g.algo == HSES_ALGO_AUTO && !tensor_path_supports(g) && pair_ok);
    return takes_pair && pair_path_fuses_scan(g);
}

}  // namespace hses

using namespace hses;

extern "C" {

size_t hses_perturbed_linear_workspace_bytes(const hses_linear_args* g) {
    if (g == nullptr || g->t_steps < 1 || g->n_pop < 1 || g->bm < 1 || g->k < 1 || g->a < 1) return 0;
    if (g->lif == 2) {
        // the per-pair path when it finishes the scan itself, else whatever the layer without the scan takes
        const bool pair_ok2 = pair_path_supports(*g);
        const bool takes_pair = (g->algo == HSES_ALGO_PAIR && pair_ok2) ||
                                (g->algo == HSES_ALGO_AUTO && !tensor_path_supports(*g) && pair_ok2);
        if (takes_pair && pair_path_fuses_scan(*g)) return pair_path_workspace_bytes(*g);
        hses_linear_args h = *g;
        h.lif = 0;
        return hses_perturbed_linear_workspace_bytes(&h);
    }
    // the tensor path always needs room for the split weights, the general path
    // only needs scratch when it perturbs
    if (g->n_groups > 1 || g->x_op != HSES_X_NONE) return tensor_path_supports(*g) ? tensor_path_workspace_bytes(*g) : 0;
    if (prefers_small_path(*g)) return small_path_workspace_bytes(*g);
    if ((g->algo == HSES_ALGO_AUTO || g->algo == HSES_ALGO_TENSOR) && tensor_path_supports(*g))
        return tensor_path_workspace_bytes(*g);
    if (g->algo == HSES_ALGO_AUTO && small_path_supports(*g)) return small_path_workspace_bytes(*g);
    if ((g->algo == HSES_ALGO_AUTO || g->algo == HSES_ALGO_PAIR) && pair_path_supports(*g))
        return pair_path_workspace_bytes(*g);
    if (g->algo == HSES_ALGO_TENSOR || g->algo == HSES_ALGO_PAIR || !g->perturb) return 0;
    return simt_scratch(*g, nullptr).bytes;
}

int hses_perturbed_linear(hses_ctx* ctx, hses_stream stream, const hses_linear_args* g) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    int rc = check_args(g);
    if (rc != HSES_OK) return rc;
    if (g->out_half != nullptr) {
        HSES_REQUIRE(g->lif != 0, "out_half is the spike output of a layer with lif = 1 or 2");
        HSES_REQUIRE(g->a % 8 == 0 && ((uintptr_t)g->out_half & 15u) == 0 && g->out_row_stride % 4 == 0 &&
                         ((uintptr_t)g->out & 15u) == 0,
                     "out_half needs a multiple of 8 outputs and 16-byte aligned rows");
        if (!ends_in_pair_scan(*g)) {
            hses_linear_args h = *g;
            h.out_half = nullptr;
            rc = hses_perturbed_linear(ctx, stream, &h);
            if (rc != HSES_OK) return rc;
            const int64_t rows = (int64_t)g->t_steps * g->n_pop * g->bm, n8 = rows * (g->a / 8);
            HSES_KERNEL(ctx, as_stream(stream), "spikes_to_half");
            spikes_to_half_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, as_stream(stream)>>>(
                g->out, rows, g->a, g->out_row_stride, reinterpret_cast<__half*>(g->out_half));
            HSES_LAUNCH_CHECK();
            return HSES_OK;
        }
    }
    if (g->lif == 2) {
        HSES_REQUIRE(g->potentials == nullptr, "lif == 2 has no potentials output");
        // the same choice of path as below
        const bool pair_ok2 = pair_path_supports(*g);
        const bool takes_pair = (g->algo == HSES_ALGO_PAIR && pair_ok2) ||
                                (g->algo == HSES_ALGO_AUTO && !tensor_path_supports(*g) && pair_ok2);
        if (takes_pair && pair_path_fuses_scan(*g))
            return run_pair_path(ctx, as_stream(stream), *g);   // the scan runs in that kernel's last phase
        // elsewhere: the currents go to `out` and are scanned in place
        hses_linear_args h = *g;
        h.lif = 0;
        h.out_scale = 1.0f;
        h.out_scale_ptr = nullptr;
        rc = hses_perturbed_linear(ctx, stream, &h);
        if (rc != HSES_OK) return rc;
        return hses_lif_scan(ctx, stream, g->out, g->t_steps, g->n_pop * g->bm, g->a, g->out_row_stride, nullptr,
                             g->tau_m, g->v_th, g->reset_mode, g->out);
    }
    if (g->x_op != HSES_X_NONE) {
        // an activation on the input: only where the prepass of the tensor-core path can apply it on the fly
        HSES_REQUIRE(g->x_op == HSES_X_RELU_SQUARE, "unknown x_op");
        if ((g->algo != HSES_ALGO_AUTO && g->algo != HSES_ALGO_TENSOR) || !tensor_path_supports(*g)) {
            set_error("hses_perturbed_linear: x_op needs the tensor-core path with the rows prepass");
            return HSES_ERR_UNSUPPORTED;
        }
        return run_tensor_path(ctx, as_stream(stream), *g);
    }
    if (g->n_groups > 1) {
        // several parameters stacked in one call: the tensor-core path or nothing
        if ((g->algo != HSES_ALGO_AUTO && g->algo != HSES_ALGO_TENSOR) || !tensor_path_supports(*g)) {
            set_error("hses_perturbed_linear: n_groups > 1 needs the tensor-core path, a grouped factor cache and "
                      "shapes it covers");
            return HSES_ERR_UNSUPPORTED;
        }
        return run_tensor_path(ctx, as_stream(stream), *g);
    }
    if (prefers_small_path(*g)) return run_small_path(ctx, as_stream(stream), *g);
    bool tc_ok = tensor_path_supports(*g);
    if (g->algo == HSES_ALGO_TENSOR && !tc_ok) {
        set_error("hses_perturbed_linear: the tensor-core path does not cover this shape");
        return HSES_ERR_UNSUPPORTED;
    }
    if (g->algo == HSES_ALGO_TENSOR || (g->algo == HSES_ALGO_AUTO && tc_ok))
        return run_tensor_path(ctx, as_stream(stream), *g);
    if (g->algo == HSES_ALGO_AUTO && small_path_supports(*g)) return run_small_path(ctx, as_stream(stream), *g);
    bool pair_ok = pair_path_supports(*g);
    if (g->algo == HSES_ALGO_PAIR && !pair_ok) {
        set_error("hses_perturbed_linear: the per-pair path does not cover this shape");
        return HSES_ERR_UNSUPPORTED;
    }
    if (g->algo == HSES_ALGO_PAIR || (g->algo == HSES_ALGO_AUTO && pair_ok))
        return run_pair_path(ctx, as_stream(stream), *g);
    return run_simt(ctx, as_stream(stream), *g);
}

}  // extern "C"
