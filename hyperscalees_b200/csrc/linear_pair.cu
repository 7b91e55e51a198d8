// Perturbed linear layer for populations whose antithetic pairs own only a few rows but
// carry wide factors (one sample per member, rank 64..128: the large-population
// configuration of do_mm, hyperscalees-noiser/src/eggroll.rs:419-446).
//
// With two members * bm * t_steps <= 32 rows per pair, the rank-r correction of a pair reads
// (a + k) * rank factor values for at most 32 rows of output: it is bound by the bytes of
// the factors, not by arithmetic, and nothing is shared between pairs.  The layer therefore
// runs as
//   1. the clean product x·Wᵀ of all rows through the ordinary paths (tensor cores when the
//      shape allows), written to `out`;
//   2. one CTA per pair that streams the pair's raw factors once from memory — a factor cache,
//      or a scratch chunk that pair_factors has just filled — computes t = x_rows·B (k-slices
//      in registers, reduced through shared memory), then u = t·(s·A)ᵀ, and finishes the rows
//      in place: out = f(out ± u) with f the readout gain or the LIF step.
#include <stdlib.h>

#include "common.cuh"
#include "linear.cuh"
#include "tc_common.cuh"

namespace hses {

namespace {

constexpr int PP_THREADS = 256;
constexpr int PP_CHUNK_FLOATS = 6144;   // at most 24 KB of B per pass
constexpr int PP_STAGES = 3;            // passes in flight: two are being copied while one is consumed
constexpr int PP_A_SMEM_FLOATS = 16384; // A of a pair is prefetched into shared memory up to 64 KB
constexpr size_t kPairScratchBytes = 256ull << 20;  // factor scratch per chunk when regenerating

using namespace tc;

struct PairArgs {
    const float* x;
    int64_t x_stride;
    int t_steps;
    int64_t n_pop;
    int bm, k, a, rank;
    int kc;            // rows of B per pass, a multiple of 4 * kslices
    int kslices;       // k-slices a pass is split into (threads per slice: (RMAX / 8) * (rank / 8))
    int a_in_smem;     // A of the pair is copied to shared memory while t is computed
    int32_t first_thread;
    int32_t pair0;     // absolute index of the pair handled by block 0
    const float* A;    // raw (pairs, a, rank) from pair0 on
    const float* B;    // raw (pairs, k, rank) from pair0 on
    float base_sigma;
    float* out;
    int64_t out_stride;
    float* pot;
    int lif;
    float leak, v_th, out_scale;
    const float* out_scale_ptr;
    int* status;
    unsigned long long* dbg;
};

// phase cycle counters of block 0 of the last launch when HSES_TC_DEBUG is set in the environment
__device__ unsigned long long g_pair_dbg[8];

// plain (untiled) bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// The pair's B and the matching columns of its x rows stream through a ring of PP_STAGES
// shared-memory stages filled by the copy engine, two copies per pass: the B rows of a pass are
// contiguous (one untiled bulk copy) and the pair's x rows are one box (columns, the pair's
// rows of a step, steps) of a 3-D tensor map over x.  Two passes are in flight while one is
// consumed and no thread ever waits for a global load it issued itself.  A of the pair is
// copied to shared memory in the background when it fits.
template <int RMAX>
__global__ void __launch_bounds__(PP_THREADS, 2)
pair_lowrank_kernel(const __grid_constant__ CUtensorMap tm_x, const PairArgs g) {
    extern __shared__ __align__(128) float smem[];
    __shared__ int64_t row_s[32];
    __shared__ int odd_s[32];                 // the row's member has an odd thread id: A is negated
    __shared__ uint64_t bars[PP_STAGES + 1];  // one per stage, then A
    __shared__ int abort_flag_s;
    volatile int* abort_flag = &abort_flag_s;
    const int tid = threadIdx.x;
    const long long t_start = clock64();
    auto tick = [&](int slot) {
        if (g.dbg != nullptr && blockIdx.x == 0 && tid == 0) g.dbg[slot] = (unsigned long long)(clock64() - t_start);
    };
    const int rank = g.rank, k = g.k, a = g.a, kc = g.kc;
    const int xp = kc;
    const int bbuf_floats = PP_STAGES * kc * rank;
    const int red_floats = g.kslices * RMAX * rank;
    float* xs = smem;                                   // [PP_STAGES][RMAX][xp]
    float* bbuf = smem + PP_STAGES * RMAX * xp;         // [PP_STAGES][kc][rank]; later the k-slice sums
    float* red = bbuf;                                  // [kslices][RMAX][rank]; slice 0 becomes t
    float* as = bbuf + (bbuf_floats > red_floats ? bbuf_floats : red_floats);  // [a][rank] when a_in_smem
    const int32_t pair = g.pair0 + blockIdx.x;
    int64_t m_lo = (int64_t)pair * 2 - g.first_thread, m_hi = m_lo + 2;
    if (m_lo < 0) m_lo = 0;
    if (m_hi > g.n_pop) m_hi = g.n_pop;
    const int rows_per_step = (int)(m_hi - m_lo) * g.bm;
    const int rows = rows_per_step * g.t_steps;  // <= RMAX by construction of the launch
    if (rows <= 0) return;
    if (tid < 32) {
        int lr = tid < rows ? tid : rows - 1;
        int step = lr / rows_per_step, rr = lr - step * rows_per_step;
        row_s[tid] = ((int64_t)step * g.n_pop + m_lo) * g.bm + rr;
        odd_s[tid] = (int)((g.first_thread + m_lo + rr / g.bm) & 1);
    }
    // rows this pair does not have read as zero (the copies never write them)
    if (rows < RMAX)
        for (int i = tid; i < PP_STAGES * RMAX * xp; i += (int)blockDim.x) xs[i] = 0.0f;
    const float* Bp = g.B + (size_t)blockIdx.x * k * rank;
    const float* Ap = g.A + (size_t)blockIdx.x * a * rank;
    const int chunks = (k + kc - 1) / kc;
    if (tid == 0) {
        abort_flag_s = 0;
        for (int i = 0; i <= PP_STAGES; ++i) mbar_init(&bars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // thread 0 is the producer: one pass = kn rows of B and kn columns of every x row
    auto issue = [&](int c) {
        const int s = c % PP_STAGES;
        const int k0 = c * kc;
        const int kn = k - k0 < kc ? k - k0 : kc;  // multiple of 4
        // the box is always counted in full: columns past k arrive as zeros
        mbar_expect_tx(&bars[s], (uint32_t)(kn * rank * 4 + rows * kc * 4));
        bulk_load(bbuf + (size_t)s * kc * rank, Bp + (size_t)k0 * rank, (uint32_t)(kn * rank * 4), &bars[s]);
        tma_load_3d(xs + (size_t)s * RMAX * xp, &tm_x, k0, (int)(m_lo * g.bm), 0, &bars[s]);
    };
    if (tid == 0) {
        fence_proxy_async();  // the zero fill above precedes the copy engine's writes
        if (g.a_in_smem) {
            mbar_expect_tx(&bars[PP_STAGES], (uint32_t)(a * rank * 4));
            bulk_load(as, Ap, (uint32_t)(a * rank * 4), &bars[PP_STAGES]);
        }
        for (int c = 0; c < PP_STAGES - 1 && c < chunks; ++c) issue(c);
    }

    tick(0);
    // ---- t = x_rows * B.  A thread owns an 8 x 8 tile of t for one k-slice: rows rg, rg+RG, ...
    // and the columns 4qg..4qg+3 and rank/2+4qg..+3, so that every 16-byte shared-memory load
    // feeds 8..32 multiply-adds.  The eight lanes that share a load phase have the same rows (x
    // is broadcast) and neighbouring 16-byte pieces of B (no bank conflicts).  The k-slices are
    // added through shared memory afterwards. ----
    constexpr int RG = RMAX / 8;
    const int qgroups = rank / 8;
    const int tpk = RG * qgroups;            // threads per k-slice
    const int kslices = g.kslices;
    const int tt = tid % tpk, ks = tid / tpk;
    const int qg = tt % qgroups, rg = tt / qgroups;
    const int q_lo = 4 * qg, q_hi = rank / 2 + 4 * qg;
    const bool active = ks < kslices;
    float acc[8][8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[j][i] = 0.0f;
    bool ok = true;
    for (int c = 0; c < chunks; ++c) {
        const int s = c % PP_STAGES;
        const int kn = k - c * kc < kc ? k - c * kc : kc;
        if (tid == 0 && c + PP_STAGES - 1 < chunks) {
            // that stage was last read in pass c-1, which ended with a barrier
            fence_proxy_async();
            issue(c + PP_STAGES - 1);
        }
        if (ok) ok = mbar_wait(&bars[s], (uint32_t)(c / PP_STAGES) & 1, abort_flag, g.status, 20);
        if (active && ok) {
            const float* bc = bbuf + (size_t)s * kc * rank;
            const float* xc = xs + ((size_t)s * RMAX + rg) * xp;
            for (int kk = ks * 4; kk < kn; kk += 4 * kslices) {
                float4 xv[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) xv[j] = *reinterpret_cast<const float4*>(xc + (size_t)j * RG * xp + kk);
#pragma unroll
                for (int kq = 0; kq < 4; ++kq) {
                    const float4 bl = *reinterpret_cast<const float4*>(bc + (size_t)(kk + kq) * rank + q_lo);
                    const float4 bh = *reinterpret_cast<const float4*>(bc + (size_t)(kk + kq) * rank + q_hi);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float xval = kq == 0 ? xv[j].x : kq == 1 ? xv[j].y : kq == 2 ? xv[j].z : xv[j].w;
                        acc[j][0] = fmaf(xval, bl.x, acc[j][0]);
                        acc[j][1] = fmaf(xval, bl.y, acc[j][1]);
                        acc[j][2] = fmaf(xval, bl.z, acc[j][2]);
                        acc[j][3] = fmaf(xval, bl.w, acc[j][3]);
                        acc[j][4] = fmaf(xval, bh.x, acc[j][4]);
                        acc[j][5] = fmaf(xval, bh.y, acc[j][5]);
                        acc[j][6] = fmaf(xval, bh.z, acc[j][6]);
                        acc[j][7] = fmaf(xval, bh.w, acc[j][7]);
                    }
                }
            }
        }
        __syncthreads();
    }
    tick(1);
    // k-slice sums: red[ks][row][q]
    if (active) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float* dst = red + ((size_t)ks * RMAX + rg + j * RG) * rank;
            *reinterpret_cast<float4*>(dst + q_lo) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
            *reinterpret_cast<float4*>(dst + q_hi) = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
        }
    }
    __syncthreads();
    for (int e = tid; e < RMAX * rank; e += (int)blockDim.x) {
        float sum = red[e];
        for (int p = 1; p < kslices; ++p) sum += red[(size_t)p * RMAX * rank + e];
        red[e] = sum;  // t[r][q], r = e / rank
    }
    if (g.a_in_smem && ok) ok = mbar_wait(&bars[PP_STAGES], 0, abort_flag, g.status, 21);
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out: copies that were issued still target this CTA's shared memory, give
        // them a bounded moment, then leave the rows as the clean product wrote them
        if (tid == 0)
            for (int b = 0; b <= PP_STAGES; ++b)
                for (uint32_t i = 0; i < 4096; ++i) {
                    if (mbar_try(&bars[b], 0) || mbar_try(&bars[b], 1)) break;
                    __nanosleep(256);
                }
        return;
    }
    const float* ts = red;
    tick(2);

    // ---- u = t * (s*A)ᵀ and the final transform of the rows.  A thread owns 4 rows x NC
    // consecutive output columns; the clean product of its outputs is fetched first so that its
    // latency hides behind the multiply-adds. ----
    constexpr int NC = 2;
    constexpr int RG4 = RMAX / 4;  // row groups of this phase: rows prg, prg + RG4, ...
    const float gain = g.out_scale_ptr ? *g.out_scale_ptr : g.out_scale;
    const int nq4 = rank / 4;
    const int ngroups = (a + NC - 1) / NC;
    for (int item = tid; item < ngroups * RG4; item += (int)blockDim.x) {
        const int ng = item / RG4, prg = item - ng * RG4;
        const int n0 = ng * NC;
        float u[4][NC], base[4][NC];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = prg + j * RG4;
            const float* orow = g.out + (size_t)row_s[r < rows ? r : 0] * g.out_stride;
#pragma unroll
            for (int c4 = 0; c4 < NC; ++c4) {
                u[j][c4] = 0.0f;
                base[j][c4] = (r < rows && n0 + c4 < a) ? orow[n0 + c4] : 0.0f;
            }
        }
        const float* abase = (g.a_in_smem ? as : Ap);
        // neighbouring threads start at neighbouring 16-byte pieces of their rows: the rows of A
        // and of t are rank floats apart in shared memory, and without the rotation the lanes of
        // a load phase would all hit the same banks
        int q4 = item % nq4;
        for (int i = 0; i < nq4; ++i) {
            float4 av[NC];
#pragma unroll
            for (int c4 = 0; c4 < NC; ++c4) {
                const int n = n0 + c4 < a ? n0 + c4 : a - 1;   // a ragged last group repeats the last column
                const float4* an = reinterpret_cast<const float4*>(abase + (size_t)n * rank) + q4;
                float4 v = g.a_in_smem ? *an : __ldg(an);
                av[c4] = make_float4(__fmul_rn(v.x, g.base_sigma), __fmul_rn(v.y, g.base_sigma),
                                     __fmul_rn(v.z, g.base_sigma), __fmul_rn(v.w, g.base_sigma));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 tv = *reinterpret_cast<const float4*>(ts + (size_t)(prg + j * RG4) * rank + q4 * 4);
#pragma unroll
                for (int c4 = 0; c4 < NC; ++c4) {
                    u[j][c4] = fmaf(tv.x, av[c4].x, u[j][c4]);
                    u[j][c4] = fmaf(tv.y, av[c4].y, u[j][c4]);
                    u[j][c4] = fmaf(tv.z, av[c4].z, u[j][c4]);
                    u[j][c4] = fmaf(tv.w, av[c4].w, u[j][c4]);
                }
            }
            if (++q4 == nq4) q4 = 0;
        }
        tick(3);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = prg + j * RG4;
            if (r < rows) {
                const int64_t R = row_s[r];
                const bool odd = odd_s[r] != 0;
                float* orow = g.out + (size_t)R * g.out_stride;
                float* prow = g.pot ? g.pot + (size_t)R * g.out_stride : nullptr;
#pragma unroll
                for (int c4 = 0; c4 < NC; ++c4) {
                    const int n = n0 + c4;
                    if (n < a) {
                        float y = __fadd_rn(base[j][c4], odd ? -u[j][c4] : u[j][c4]);
                        if (g.lif) {
                            float cpot = __fmul_rn(y, g.leak);
                            if (prow) prow[n] = cpot;
                            orow[n] = cpot >= g.v_th ? 1.0f : 0.0f;
                        } else {
                            orow[n] = __fmul_rn(y, gain);
                        }
                    }
                }
            }
        }
    }
    tick(4);
}

// k-slices of a pass: as many as the block has threads for, at most 64 (a pass is at most 256
// columns, the limit of a TMA box)
// threads per CTA: the 8-row tile (a pair with at most 8 rows, e.g. the readout of one sample per
// member) has too little work for 256 threads (measured: 0.25 ms with 128 threads, 0.33 ms with 256)
int threads_of(int rmax) { return rmax == 8 ? 128 : PP_THREADS; }
int kslices_of(int rmax, int rank) {
    int ks = threads_of(rmax) / ((rmax / 8) * (rank / 8));
    if (ks < 1) ks = 1;
    return ks > 64 ? 64 : ks;
}
// rows of B per pass: a multiple of 4 * kslices (every slice does the same number of steps),
// as many as fit the per-pass budget, at least one step per slice
int kc_of(int rmax, int rank) {
    int unit = 4 * kslices_of(rmax, rank);
    int m = PP_CHUNK_FLOATS / (rank * unit);
    if (m < 1) m = 1;
    if (m * unit > 256) m = 256 / unit;
    return m * unit;
}

bool a_fits(const hses_linear_args& g) { return (size_t)g.a * g.rank <= (size_t)PP_A_SMEM_FLOATS; }

int rmax_of(const hses_linear_args& g) {
    int rows = 2 * g.bm * g.t_steps;
    return rows <= 8 ? 8 : rows <= 16 ? 16 : 32;
}

size_t pair_smem_bytes(int rmax, const hses_linear_args& g) {
    int kc = kc_of(rmax, g.rank), kslices = kslices_of(rmax, g.rank);
    size_t bbuf = (size_t)PP_STAGES * kc * g.rank, red = (size_t)kslices * rmax * g.rank;
    size_t fl = (size_t)PP_STAGES * rmax * kc + (bbuf > red ? bbuf : red) +
                (a_fits(g) ? (size_t)g.a * g.rank : 0);
    return fl * sizeof(float);
}

hses_linear_args base_call(const hses_linear_args& g) {
    hses_linear_args b = g;
    b.perturb = 0;
    b.lif = 0;
    b.out_scale = 1.0f;
    b.out_scale_ptr = nullptr;
    b.potentials = nullptr;
    b.cache = nullptr;
    b.algo = HSES_ALGO_AUTO;
    return b;
}

size_t up256(size_t v) { return (v + 255) / 256 * 256; }

int64_t chunk_pairs_of(const hses_linear_args& g, int64_t pairs) {
    size_t per_pair = (size_t)(g.a + g.k) * g.rank * sizeof(float);
    int64_t fit = (int64_t)(kPairScratchBytes / per_pair);
    if (fit < 1) fit = 1;
    return pairs < fit ? pairs : fit;
}

}  // namespace

bool pair_path_supports(const hses_linear_args& g) {
    if (!g.perturb) return false;
    if (g.rank % 8 != 0 || g.rank > PP_THREADS || g.k % 4 != 0) return false;
    if ((int64_t)2 * g.bm * g.t_steps > 32) return false;
    if (g.first_thread % 2 != 0 || g.n_pop % 2 != 0) return false;
    // the bulk copies of the x rows need 16-byte aligned row starts
    if (g.x_row_stride % 4 != 0 || ((uintptr_t)g.x & 15u) != 0) return false;
    return true;
}

size_t pair_path_workspace_bytes(const hses_linear_args& g) {
    hses_linear_args b = base_call(g);
    size_t base = up256(hses_perturbed_linear_workspace_bytes(&b));
    if (g.cache) return base;
    int64_t pairs = g.n_pop / 2;
    return base + up256((size_t)chunk_pairs_of(g, pairs) * (g.a + g.k) * g.rank * sizeof(float));
}

int run_pair_path(hses_ctx* ctx, cudaStream_t st, const hses_linear_args& g) {
    // 1. clean product of all rows
    hses_linear_args b = base_call(g);
    size_t base_bytes = up256(hses_perturbed_linear_workspace_bytes(&b));
    size_t need = pair_path_workspace_bytes(g);
    HSES_REQUIRE(need == 0 || (g.workspace != nullptr && g.workspace_bytes >= need &&
                               ((uintptr_t)g.workspace & 15u) == 0),
                 "workspace too small or misaligned; see hses_perturbed_linear_workspace_bytes");
    b.workspace = base_bytes ? g.workspace : nullptr;
    b.workspace_bytes = base_bytes;
    int rc = hses_perturbed_linear(ctx, reinterpret_cast<hses_stream>(st), &b);
    if (rc != HSES_OK) return rc;

    // 2. per-pair correction
    PairArgs pa{};
    pa.x = g.x;
    pa.x_stride = g.x_row_stride;
    pa.t_steps = g.t_steps;
    pa.n_pop = g.n_pop;
    pa.bm = g.bm;
    pa.k = g.k;
    pa.a = g.a;
    pa.rank = g.rank;
    pa.first_thread = g.first_thread;
    pa.base_sigma = g.sigma / sqrtf((float)g.rank);
    pa.out = g.out;
    pa.out_stride = g.out_row_stride;
    pa.pot = g.lif ? g.potentials : nullptr;
    pa.lif = g.lif;
    pa.leak = g.lif ? 1.0f / g.tau_m : 0.0f;
    pa.v_th = g.v_th;
    pa.out_scale = g.out_scale;
    pa.out_scale_ptr = g.out_scale_ptr;
    const int rmax = rmax_of(g);
    const size_t smem = pair_smem_bytes(rmax, g);
    // x as (column, row within a step, step); a box holds the rows of one pair for one pass
    CUtensorMap tm_x;
    {
        EncodeTiledFn fn = encode_fn();
        if (!fn) {
            set_error("cuTensorMapEncodeTiled is not available from the driver");
            return HSES_ERR_CUDA;
        }
        const uint64_t rows_per_step = (uint64_t)g.n_pop * g.bm;
        cuuint64_t dims[3] = {(cuuint64_t)g.k, (cuuint64_t)rows_per_step, (cuuint64_t)g.t_steps};
        cuuint64_t strides[2] = {(cuuint64_t)g.x_row_stride * 4, (cuuint64_t)g.x_row_stride * 4 * rows_per_step};
        cuuint32_t box[3] = {(cuuint32_t)kc_of(rmax, g.rank), (cuuint32_t)(2 * g.bm), (cuuint32_t)g.t_steps};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = fn(&tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(g.x), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            set_error("cuTensorMapEncodeTiled (x rows of a pair) failed with code " + std::to_string((int)r));
            return HSES_ERR_CUDA;
        }
    }
    pa.kc = kc_of(rmax, g.rank);
    pa.kslices = kslices_of(rmax, g.rank);
    pa.a_in_smem = a_fits(g) ? 1 : 0;
    pa.status = ctx->t.status_word;
    pa.dbg = nullptr;
    if (getenv("HSES_TC_DEBUG")) {
        void* dp = nullptr;
        HSES_CUDA(cudaGetSymbolAddress(&dp, g_pair_dbg));
        pa.dbg = reinterpret_cast<unsigned long long*>(dp);
    }
    auto launch = [&](int64_t n_pairs) -> int {
        HSES_KERNEL(ctx, st, "pair_lowrank");
        switch (rmax) {
            case 8:
                HSES_CUDA(cudaFuncSetAttribute(pair_lowrank_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                pair_lowrank_kernel<8><<<(unsigned)n_pairs, threads_of(8), smem, st>>>(tm_x, pa);
                break;
            case 16:
                HSES_CUDA(cudaFuncSetAttribute(pair_lowrank_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                pair_lowrank_kernel<16><<<(unsigned)n_pairs, threads_of(16), smem, st>>>(tm_x, pa);
                break;
            default:
                HSES_CUDA(cudaFuncSetAttribute(pair_lowrank_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                pair_lowrank_kernel<32><<<(unsigned)n_pairs, threads_of(32), smem, st>>>(tm_x, pa);
                break;
        }
        HSES_LAUNCH_CHECK();
        return HSES_OK;
    };
    const int32_t first_pair = g.first_thread / 2;
    const int64_t pairs = g.n_pop / 2;
    if (g.cache) {
        const float *ca = nullptr, *cb = nullptr;
        rc = resolve_factor_cache(g, &ca, &cb);
        if (rc != HSES_OK) return rc;
        pa.pair0 = first_pair;
        pa.A = ca;
        pa.B = cb;
        return launch(pairs);
    }
    // regenerate chunk by chunk into scratch: the generator kernel runs at full occupancy
    const int64_t cp = chunk_pairs_of(g, pairs);
    float* sa = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(g.workspace) + base_bytes);
    float* sb = sa + (size_t)cp * g.a * g.rank;
    const int32_t te = true_epoch_of(g.epoch, g.noise_reuse);
    for (int64_t done = 0; done < pairs; done += cp) {
        int64_t cnt = pairs - done < cp ? pairs - done : cp;
        rc = launch_pair_factors(ctx, st, g.key, te, first_pair + (int32_t)done, cnt, g.rank, g.a, g.k, nullptr,
                                 sa, sb);
        if (rc != HSES_OK) return rc;
        pa.pair0 = first_pair + (int32_t)done;
        pa.A = sa;
        pa.B = sb;
        rc = launch(cnt);
        if (rc != HSES_OK) return rc;
    }
    return HSES_OK;
}

}  // namespace hses

// Diagnostic, not part of the declared ABI: phase cycle counters of block 0 of the last
// per-pair launch made with HSES_TC_DEBUG set (synchronises the device).
extern "C" int hses_internal_pair_cycles(unsigned long long* out8) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, hses::g_pair_dbg) != cudaSuccess) return 2;
    if (cudaMemcpy(out8, p, sizeof(unsigned long long) * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return 2;
    return 0;
}
