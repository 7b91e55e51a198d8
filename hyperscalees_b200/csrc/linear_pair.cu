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
//      in registers, reduced through shared memory), then u = (s·t)·Aᵀ, and finishes the rows
//      in place: out = f(out ± u) with f the readout gain or the LIF step.
#include <stdlib.h>

#include <cuda_fp16.h>

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
    int a_swz;         // ... as 32-column boxes with the 128-byte swizzle (tensor map tm_a)
    int32_t first_thread;
    int32_t pair0;     // absolute index of the pair handled by block 0
    const float* A;    // raw (pairs, a, rank) from pair0 on
    const float* B;    // raw (pairs, k, rank) from pair0 on
    float base_sigma;
    float* out;
    int64_t out_stride;
    float* pot;
    __half* out_half;  // dense fp16 copy of the spikes (row stride a), written by the fused scan
    int lif;           // 0: y * gain; 1: one LIF step from v = 0; 2: LIF scan over the steps (swizzled form only)
    int reset;
    float leak, v_th, out_scale;
    const float* out_scale_ptr;
    int* status;
};

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
pair_lowrank_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_a,
                    const PairArgs g) {
    extern __shared__ __align__(128) float smem[];
    __shared__ int64_t row_s[32];
    __shared__ int odd_s[32];                 // the row's member has an odd thread id: A is negated
    __shared__ uint64_t bars[PP_STAGES + 1];  // one per stage, then A
    __shared__ int abort_flag_s;
    volatile int* abort_flag = &abort_flag_s;
    const int tid = threadIdx.x;
    const int rank = g.rank, k = g.k, a = g.a, kc = g.kc;
    const int xp = kc;
    const int bbuf_floats = PP_STAGES * kc * rank;
    const int red_floats = g.kslices * RMAX * rank;
    float* xs = smem;                                   // [PP_STAGES][RMAX][xp]
    float* bbuf = smem + PP_STAGES * RMAX * xp;         // [PP_STAGES][kc][rank]; later the k-slice sums
    float* red = bbuf;                                  // [kslices][RMAX][rank]; slice 0 becomes t
    float* as = bbuf + (bbuf_floats > red_floats ? bbuf_floats : red_floats);  // [a][rank] when a_in_smem
    // swizzled form: rank/32 boxes of [a][32], each starting on a 1024-byte boundary so that the
    // 16-byte piece c of row n sits at piece c ^ (n & 7)
    const int bstride = ((a * 128 + 1023) / 1024) * 256;   // floats between boxes
    if (g.a_swz) as += ((1024u - (smem_u32(as) & 1023u)) & 1023u) / 4;
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
        if (g.a_swz) {
            mbar_expect_tx(&bars[PP_STAGES], (uint32_t)(a * rank * 4));
            for (int b = 0; b < rank / 32; ++b)
                tma_load_2d(as + (size_t)b * bstride, &tm_a, 32 * b, (int)blockIdx.x * a, &bars[PP_STAGES]);
        } else if (g.a_in_smem) {
            mbar_expect_tx(&bars[PP_STAGES], (uint32_t)(a * rank * 4));
            bulk_load(as, Ap, (uint32_t)(a * rank * 4), &bars[PP_STAGES]);
        }
        for (int c = 0; c < PP_STAGES - 1 && c < chunks; ++c) issue(c);
    }

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
    // k-slice sums: red[ks][row][q]
    if (active) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float* dst = red + ((size_t)ks * RMAX + rg + j * RG) * rank;
            *reinterpret_cast<float4*>(dst + q_lo) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
            *reinterpret_cast<float4*>(dst + q_hi) = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
        }
    }
    // clean product under this thread's outputs of the second phase (swizzled form, first round of
    // tasks): fetched here so that its latency hides behind the k-slice sums
    constexpr int RGROUPS = RMAX / 8;
    float base0[4][2];
    auto load_base = [&](int task, float (&bs)[4][2]) {
        const int rh = task & 1, rest = task >> 1;
        const int rgp = rest % RGROUPS, cb = rest / RGROUPS;
        const int nc0 = cb * 64 + (tid & 31);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int r = rgp * 8 + rh * 4 + jj;
            const float* orow = g.out + (size_t)row_s[r < rows ? r : 0] * g.out_stride;
#pragma unroll
            for (int c2 = 0; c2 < 2; ++c2) {
                const int n = nc0 + 32 * c2;
                bs[jj][c2] = (r < rows && n < a) ? orow[n] : 0.0f;
            }
        }
    };
    const int tasks2 = RGROUPS * ((a + 63) >> 6) * 2;
    if (g.a_swz && (tid >> 5) < tasks2) load_base(tid >> 5, base0);
    __syncthreads();
    {
        // 16 bytes per thread and several slices in flight: the additions of an element keep their order
        const int tot4 = RMAX * rank / 4;
        float4* red4 = reinterpret_cast<float4*>(red);
        for (int e4 = tid; e4 < tot4; e4 += (int)blockDim.x) {
            float4 sum = red4[e4];
#pragma unroll 4
            for (int p = 1; p < kslices; ++p) {
                const float4 v = red4[(size_t)p * tot4 + e4];
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            // sigma goes onto t here (rows x rank values) rather than onto A in the second phase (a x rank)
            const float sg = g.base_sigma;
            red4[e4] = make_float4(__fmul_rn(sum.x, sg), __fmul_rn(sum.y, sg), __fmul_rn(sum.z, sg), __fmul_rn(sum.w, sg));  // s*t[r][q], r = e / rank
        }
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

    if (g.a_swz) {
        // ---- u = (s*t) * Aᵀ, swizzled A.  A warp takes a task = (8 rows, 64 columns, half of the
        // rank); a lane owns columns lane and lane + 32 of the block, so the A pieces of a load are
        // 32 different rows of one box column (conflict-free through the swizzle) and the t pieces
        // are broadcasts: 10 loads feed 64 multiply-adds.  The two rank halves of a tile swap four
        // rows each through shared memory and finish four rows each. ----
        const float gain = g.out_scale_ptr ? *g.out_scale_ptr : g.out_scale;
        const int nwarps = (int)blockDim.x >> 5, wid = tid >> 5, lane = tid & 31;
        const int tasks = tasks2;
        const int halfq = rank >> 3;              // 16-byte pieces per rank half
        float* xch = red + RMAX * rank;           // [warp][lane][8]
        const bool scan = g.lif == 2;
        float* ytile = xch + nwarps * 32 * 8;     // [row][a]: currents of all steps, scanned at the end
        for (int t0 = 0; t0 < tasks; t0 += nwarps) {
            const int task = t0 + wid;
            const bool live = task < tasks;
            const int rh = task & 1, rest = task >> 1;
            const int rgp = rest % RGROUPS, cb = rest / RGROUPS;
            const int nc0 = cb * 64 + lane;       // columns nc0 and nc0 + 32
            float acc[8][2], base[4][2];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = 0.0f;
            if (live) {
                if (t0 == 0) {
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) base[jj][0] = base0[jj][0], base[jj][1] = base0[jj][1];
                } else {
                    load_base(task, base);
                }
                const int n_a = nc0 < a ? nc0 : a - 1, n_b = nc0 + 32 < a ? nc0 + 32 : a - 1;
                const float* trow = ts + (size_t)rgp * 8 * rank;
                for (int i = 0; i < halfq; ++i) {
                    const int q4 = rh * halfq + i;
                    const float* box = as + (size_t)(q4 >> 3) * bstride;
                    const int c = q4 & 7;
                    const float4 va = *reinterpret_cast<const float4*>(box + n_a * 32 + ((c ^ (n_a & 7)) << 2));
                    const float4 vb = *reinterpret_cast<const float4*>(box + n_b * 32 + ((c ^ (n_b & 7)) << 2));
                    const float4 sa4 = va, sb4 = vb;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 tv = *reinterpret_cast<const float4*>(trow + (size_t)j * rank + q4 * 4);
                        acc[j][0] = fmaf(tv.x, sa4.x, acc[j][0]);
                        acc[j][0] = fmaf(tv.y, sa4.y, acc[j][0]);
                        acc[j][0] = fmaf(tv.z, sa4.z, acc[j][0]);
                        acc[j][0] = fmaf(tv.w, sa4.w, acc[j][0]);
                        acc[j][1] = fmaf(tv.x, sb4.x, acc[j][1]);
                        acc[j][1] = fmaf(tv.y, sb4.y, acc[j][1]);
                        acc[j][1] = fmaf(tv.z, sb4.z, acc[j][1]);
                        acc[j][1] = fmaf(tv.w, sb4.w, acc[j][1]);
                    }
                }
                // hand the other half's rows over
                float4* xo = reinterpret_cast<float4*>(xch + ((size_t)wid * 32 + lane) * 8);
                float o[8];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {   // static register indices: select with the half bit
                    o[2 * jj] = rh ? acc[jj][0] : acc[4 + jj][0];
                    o[2 * jj + 1] = rh ? acc[jj][1] : acc[4 + jj][1];
                }
                xo[0] = make_float4(o[0], o[1], o[2], o[3]);
                xo[1] = make_float4(o[4], o[5], o[6], o[7]);
            }
            __syncthreads();
            if (live) {
                const float4* xi = reinterpret_cast<const float4*>(xch + ((size_t)(wid ^ 1) * 32 + lane) * 8);
                const float4 p0 = xi[0], p1 = xi[1];
                const float other[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int r = rgp * 8 + rh * 4 + jj;
                    if (r < rows) {
                        const int64_t R = row_s[r];
                        const bool odd = odd_s[r] != 0;
                        float* orow = g.out + (size_t)R * g.out_stride;
                        float* prow = g.pot ? g.pot + (size_t)R * g.out_stride : nullptr;
#pragma unroll
                        for (int c2 = 0; c2 < 2; ++c2) {
                            const int n = nc0 + 32 * c2;
                            if (n < a) {
                                const float mine = rh ? acc[4 + jj][c2] : acc[jj][c2];
                                // the lower rank half first, whichever warp finishes the row
                                const float u = rh ? __fadd_rn(other[2 * jj + c2], mine) : __fadd_rn(mine, other[2 * jj + c2]);
                                float y = __fadd_rn(base[jj][c2], odd ? -u : u);
                                if (scan) {
                                    ytile[r * a + n] = y;
                                } else if (g.lif) {
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
            if (t0 + nwarps < tasks) __syncthreads();   // the exchange buffer is reused by the next round
        }
        if (scan) {
            // run_lif over the steps (snn.rs:73-97): one thread per (row of a step, column), membrane
            // from v = 0; lanes own neighbouring columns, so every store is a full line
            __syncthreads();
            for (int idx = tid; idx < rows_per_step * a; idx += (int)blockDim.x) {
                const int rr = idx / a, n = idx - rr * a;
                float v = 0.0f;
                for (int step = 0; step < g.t_steps; ++step) {
                    const int r = step * rows_per_step + rr;
                    const float sp = lif_update(v, ytile[r * a + n], g.leak, g.v_th, g.reset);
                    g.out[(size_t)row_s[r] * g.out_stride + n] = sp;
                    if (g.out_half) g.out_half[(size_t)row_s[r] * a + n] = __float2half_rn(sp);
                }
            }
        }
        return;
    }

    // ---- u = (s*t) * Aᵀ and the final transform of the rows.  A thread owns 4 rows x NC
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
                av[c4] = v;
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

// A goes to shared memory as swizzled 32-column boxes (conflict-free column-per-lane reads in the
// second phase) when the rank is a multiple of 32, a box holds all rows (<= 256) and the
// exchange buffer of that phase fits behind t in the k-slice area
size_t a_swz_floats(const hses_linear_args& g) {
    return (size_t)(g.rank / 32) * (((size_t)g.a * 128 + 1023) / 1024 * 256);
}
bool a_swizzled(int rmax, const hses_linear_args& g) {
    if (!a_fits(g) || g.rank % 32 != 0 || g.a > 256) return false;
    int kc = kc_of(rmax, g.rank), kslices = kslices_of(rmax, g.rank);
    size_t bbuf = (size_t)PP_STAGES * kc * g.rank, red = (size_t)kslices * rmax * g.rank;
    size_t area = bbuf > red ? bbuf : red;
    return (size_t)rmax * g.rank + (size_t)threads_of(rmax) * 8 <= area && a_swz_floats(g) <= 2 * (size_t)PP_A_SMEM_FLOATS;
}

// the currents of a pair (rows x a) fit behind t and the exchange buffer in the k-slice area
bool scan_fits(int rmax, const hses_linear_args& g) {
    if (!a_swizzled(rmax, g)) return false;
    int kc = kc_of(rmax, g.rank), kslices = kslices_of(rmax, g.rank);
    size_t bbuf = (size_t)PP_STAGES * kc * g.rank, red = (size_t)kslices * rmax * g.rank;
    size_t area = bbuf > red ? bbuf : red;
    return (size_t)rmax * g.rank + (size_t)threads_of(rmax) * 8 + (size_t)rmax * g.a <= area;
}

size_t pair_smem_bytes(int rmax, const hses_linear_args& g) {
    int kc = kc_of(rmax, g.rank), kslices = kslices_of(rmax, g.rank);
    size_t bbuf = (size_t)PP_STAGES * kc * g.rank, red = (size_t)kslices * rmax * g.rank;
    size_t afl = a_swizzled(rmax, g) ? a_swz_floats(g) + 256 : (a_fits(g) ? (size_t)g.a * g.rank : 0);
    size_t fl = (size_t)PP_STAGES * rmax * kc + (bbuf > red ? bbuf : red) + afl;
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
    b.out_half = nullptr;
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

bool pair_path_fuses_scan(const hses_linear_args& g) { return g.potentials == nullptr && scan_fits(rmax_of(g), g); }

bool pair_path_supports(const hses_linear_args& g) {
    if (!g.perturb || g.factor_order != 0) return false;
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
    pa.out_half = g.lif == 2 ? reinterpret_cast<__half*>(g.out_half) : nullptr;
    pa.lif = g.lif;
    pa.reset = g.reset_mode;
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
    pa.a_swz = a_swizzled(rmax, g) ? 1 : 0;
    pa.status = ctx->t.status_word;
    auto launch = [&](int64_t n_pairs) -> int {
        // A of the launch's pairs as (rank, pairs * a); a box is 32 columns of all rows of one pair
        CUtensorMap tm_a = tm_x;   // a valid map also when the swizzled form is not used
        if (pa.a_swz) {
            EncodeTiledFn fn = encode_fn();
            cuuint64_t dims[2] = {(cuuint64_t)g.rank, (cuuint64_t)n_pairs * g.a};
            cuuint64_t strides[1] = {(cuuint64_t)g.rank * 4};
            cuuint32_t box[2] = {32, (cuuint32_t)g.a};
            cuuint32_t estr[2] = {1, 1};
            CUresult r = fn(&tm_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(pa.A), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) {
                set_error("cuTensorMapEncodeTiled (A of a pair) failed with code " + std::to_string((int)r));
                return HSES_ERR_CUDA;
            }
        }
        HSES_KERNEL(ctx, st, "pair_lowrank");
        switch (rmax) {
            case 8:
                HSES_CUDA(cudaFuncSetAttribute(pair_lowrank_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                pair_lowrank_kernel<8><<<(unsigned)n_pairs, threads_of(8), smem, st>>>(tm_x, tm_a, pa);
                break;
            case 16:
                HSES_CUDA(cudaFuncSetAttribute(pair_lowrank_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                pair_lowrank_kernel<16><<<(unsigned)n_pairs, threads_of(16), smem, st>>>(tm_x, tm_a, pa);
                break;
            default:
                HSES_CUDA(cudaFuncSetAttribute(pair_lowrank_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                pair_lowrank_kernel<32><<<(unsigned)n_pairs, threads_of(32), smem, st>>>(tm_x, tm_a, pa);
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
