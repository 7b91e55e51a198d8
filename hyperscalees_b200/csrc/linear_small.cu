// Perturbed linear layer for narrow layers (k <= 64 inputs, a <= 64 outputs, rank <= 16): the
// per-head and per-token projections of the SNN-rate transformer
// (hyperscalees-models/src/snn_transformer.rs:273-297) at population scale.
//
// Such a layer is a few kilobytes of weights and a few kilobytes of factors per antithetic
// pair; the wide-tile kernels spend their time on set-up.  Here a CTA keeps W in shared memory
// for its whole life and walks over pairs: it stages the pair's factors and 32 of its rows at a
// time, forms t = x·B and y = x·Wᵀ + t·(s·A)ᵀ from shared memory and finishes the rows (gain or
// one LIF step).  Factors come from a factor cache or from scratch that pair_factors filled.
#include "common.cuh"
#include "linear.cuh"

namespace hses {

namespace {

constexpr int SP_THREADS = 256;
constexpr int SP_ROWS = 32;     // rows staged at a time
constexpr int SP_MAXK = 64, SP_MAXA = 64, SP_MAXR = 16;

struct SmallArgs {
    const float* x;
    int64_t x_stride;
    const float* w;
    int64_t w_stride;
    int t_steps, bm, k, a, rank;
    int64_t n_pop;
    int32_t first_thread;
    int64_t pairs;
    const float* A;   // raw (pairs, a, rank) from the call's first pair on
    const float* B;   // raw (pairs, k, rank)
    float base_sigma;
    float* out;
    int64_t out_stride;
    float* pot;
    int lif;
    float leak, v_th, out_scale;
    const float* out_scale_ptr;
};

__global__ void __launch_bounds__(SP_THREADS, 4)
small_pair_kernel(const SmallArgs g) {
    // pitch 68 floats: rows are 16-byte aligned and eight neighbouring rows read as 16-byte pieces
    // cover all banks once; columns k..k4-1 are zero
    __shared__ __align__(16) float ws[SP_MAXA][SP_MAXK + 4];
    __shared__ __align__(16) float xs[SP_ROWS][SP_MAXK + 4];
    __shared__ float bs[SP_MAXK][SP_MAXR];
    __shared__ float as_[SP_MAXA][SP_MAXR + 1];
    __shared__ float ts[SP_ROWS][SP_MAXR + 1];
    __shared__ int64_t row_s[SP_ROWS];
    __shared__ int odd_s[SP_ROWS];
    const int tid = threadIdx.x;
    const int k = g.k, a = g.a, rank = g.rank;
    const int k4 = (k + 3) & ~3;
    for (int e = tid; e < a * k4; e += SP_THREADS) {
        const int n = e / k4, kk = e - n * k4;
        ws[n][kk] = kk < k ? g.w[(size_t)n * g.w_stride + kk] : 0.0f;
    }
    const float gain = g.out_scale_ptr ? *g.out_scale_ptr : g.out_scale;
    const int rows_per_step = 2 * g.bm;                 // both members of a pair
    const int rows_total = rows_per_step * g.t_steps;   // rows of a pair
    for (int64_t p = blockIdx.x; p < g.pairs; p += gridDim.x) {
        __syncthreads();   // the previous pair's factors and rows are no longer read
        const float* Bp = g.B + (size_t)p * k * rank;
        const float* Ap = g.A + (size_t)p * a * rank;
        for (int e = tid; e < k4 * rank; e += SP_THREADS) bs[e / rank][e % rank] = e < k * rank ? Bp[e] : 0.0f;
        for (int e = tid; e < a * rank; e += SP_THREADS) as_[e / rank][e % rank] = __fmul_rn(Ap[e], g.base_sigma);
        const int64_t m_lo = p * 2;   // first member of the pair inside the call's population slice
        for (int r0 = 0; r0 < rows_total; r0 += SP_ROWS) {
            const int nrows = rows_total - r0 < SP_ROWS ? rows_total - r0 : SP_ROWS;
            __syncthreads();   // xs, ts of the previous chunk are no longer read
            if (tid < nrows) {
                const int lr = r0 + tid;
                const int step = lr / rows_per_step, rr = lr - step * rows_per_step;
                row_s[tid] = ((int64_t)step * g.n_pop + m_lo) * g.bm + rr;
                odd_s[tid] = (int)((g.first_thread + m_lo + rr / g.bm) & 1);
            }
            __syncthreads();
            for (int e = tid; e < SP_ROWS * k4; e += SP_THREADS) {
                const int r = e / k4, kk = e - r * k4;
                xs[r][kk] = (r < nrows && kk < k) ? g.x[(size_t)row_s[r] * g.x_stride + kk] : 0.0f;
            }
            __syncthreads();
            // t = x * B: thread -> (row, q)
            for (int e = tid; e < nrows * rank; e += SP_THREADS) {
                const int r = e / rank, q = e - r * rank;
                float acc = 0.0f;
                for (int kk = 0; kk < k4; kk += 4) {
                    const float4 xv = *reinterpret_cast<const float4*>(&xs[r][kk]);
                    acc = fmaf(xv.x, bs[kk][q], acc);
                    acc = fmaf(xv.y, bs[kk + 1][q], acc);
                    acc = fmaf(xv.z, bs[kk + 2][q], acc);
                    acc = fmaf(xv.w, bs[kk + 3][q], acc);
                }
                ts[r][q] = acc;
            }
            __syncthreads();
            // y = x * W^T + t * (s*A)^T.  Thread (rg, cg) owns rows rg, rg+16 and columns cg, cg+16,
            // cg+32, cg+48: six shared-memory reads feed eight multiply-adds, the x values are
            // broadcasts and the W values of a warp lie in different banks (odd pitch).
            {
                const int cg = tid & 15, rg = tid >> 4;
                const int nj = (a + 15) >> 4;   // column groups of 16 that exist (uniform)
                float acc[2][4];
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
                if (cg < a) {
                    for (int kk = 0; kk < k4; kk += 4) {
                        const float4 x0 = *reinterpret_cast<const float4*>(&xs[rg][kk]);
                        const float4 x1 = *reinterpret_cast<const float4*>(&xs[rg + 16][kk]);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (j >= nj) break;
                            const int n = cg + 16 * j < a ? cg + 16 * j : cg;
                            const float4 wv = *reinterpret_cast<const float4*>(&ws[n][kk]);
                            acc[0][j] = fmaf(x0.x, wv.x, acc[0][j]);
                            acc[0][j] = fmaf(x0.y, wv.y, acc[0][j]);
                            acc[0][j] = fmaf(x0.z, wv.z, acc[0][j]);
                            acc[0][j] = fmaf(x0.w, wv.w, acc[0][j]);
                            acc[1][j] = fmaf(x1.x, wv.x, acc[1][j]);
                            acc[1][j] = fmaf(x1.y, wv.y, acc[1][j]);
                            acc[1][j] = fmaf(x1.z, wv.z, acc[1][j]);
                            acc[1][j] = fmaf(x1.w, wv.w, acc[1][j]);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int r = rg + 16 * i;
                        if (r >= nrows) continue;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int n = cg + 16 * j;
                            if (n >= a) continue;
                            float u = 0.0f;
                            for (int q = 0; q < rank; ++q) u = fmaf(ts[r][q], as_[n][q], u);
                            const float y = __fadd_rn(acc[i][j], odd_s[r] ? -u : u);
                            const size_t o = (size_t)row_s[r] * g.out_stride + n;
                            if (g.lif) {
                                const float c = __fmul_rn(y, g.leak);
                                if (g.pot) g.pot[o] = c;
                                g.out[o] = c >= g.v_th ? 1.0f : 0.0f;
                            } else {
                                g.out[o] = __fmul_rn(y, gain);
                            }
                        }
                    }
                }
            }
        }
    }
}

size_t up256s(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace

bool small_path_supports(const hses_linear_args& g) {
    if (!g.perturb || g.lif == 2 || g.factor_order != 0) return false;
    if (g.k > SP_MAXK || g.a > SP_MAXA || g.rank > SP_MAXR) return false;
    if (g.first_thread % 2 != 0 || g.n_pop % 2 != 0) return false;
    // without a cache all factors of the call go to scratch at once
    if (!g.cache && (double)(g.n_pop / 2) * (g.a + g.k) * g.rank * sizeof(float) > 256.0 * 1024 * 1024) return false;
    return true;
}

size_t small_path_workspace_bytes(const hses_linear_args& g) {
    if (g.cache) return 0;
    return up256s((size_t)(g.n_pop / 2) * (g.a + g.k) * g.rank * sizeof(float));
}

int run_small_path(hses_ctx* ctx, cudaStream_t st, const hses_linear_args& g) {
    const int64_t pairs = g.n_pop / 2;
    const int32_t first_pair = g.first_thread / 2;
    const float *A = nullptr, *B = nullptr;
    if (g.cache) {
        int rc = resolve_factor_cache(g, &A, &B);
        if (rc != HSES_OK) return rc;
    } else {
        size_t need = small_path_workspace_bytes(g);
        HSES_REQUIRE(g.workspace != nullptr && g.workspace_bytes >= need && ((uintptr_t)g.workspace & 15u) == 0,
                     "workspace too small or misaligned; see hses_perturbed_linear_workspace_bytes");
        float* sa = reinterpret_cast<float*>(g.workspace);
        float* sb = sa + (size_t)pairs * g.a * g.rank;
        int rc = launch_pair_factors(ctx, st, g.key, true_epoch_of(g.epoch, g.noise_reuse), first_pair, pairs, g.rank,
                                     g.a, g.k, nullptr, sa, sb);
        if (rc != HSES_OK) return rc;
        A = sa;
        B = sb;
    }
    SmallArgs s{};
    s.x = g.x;
    s.x_stride = g.x_row_stride;
    s.w = g.param;
    s.w_stride = g.param_row_stride;
    s.t_steps = g.t_steps;
    s.bm = g.bm;
    s.k = g.k;
    s.a = g.a;
    s.rank = g.rank;
    s.n_pop = g.n_pop;
    s.first_thread = g.first_thread;
    s.pairs = pairs;
    s.A = A;
    s.B = B;
    s.base_sigma = g.sigma / sqrtf((float)g.rank);
    s.out = g.out;
    s.out_stride = g.out_row_stride;
    s.pot = g.lif ? g.potentials : nullptr;
    s.lif = g.lif;
    s.leak = g.lif ? 1.0f / g.tau_m : 0.0f;
    s.v_th = g.v_th;
    s.out_scale = g.out_scale;
    s.out_scale_ptr = g.out_scale_ptr;
    // one wave of resident CTAs: a second, partial wave would only lengthen the launch
    int per_sm = 0, sms = 0, dev = 0;
    HSES_CUDA(cudaGetDevice(&dev));
    HSES_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    HSES_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, small_pair_kernel, SP_THREADS, 0));
    const int64_t want = (int64_t)sms * (per_sm > 0 ? per_sm : 1);
    const unsigned grid = (unsigned)(pairs < want ? pairs : want);
    HSES_KERNEL(ctx, st, "small_pair");
    small_pair_kernel<<<grid, SP_THREADS, 0, st>>>(s);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // namespace hses
