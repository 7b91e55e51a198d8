// Tensor-core path of the perturbed linear layer (do_mm,
// hyperscalees-noiser/src/eggroll.rs:419-446, + lif_step, snn.rs:53-65).
//
//   launch 1  split_w         every row of W times a power of two, then fp16 hi + lo (22 bits)
//   launch 2  lowrank_t       t = x·B_pair, B regenerated from the seed stream in shared memory,
//                             never written to HBM; the same pass writes the fp16 split of x
//   launch 3  linear_tc       persistent, one CTA per SM, warp-specialised:
//       warp 0       TMA producer: x_hi, x_lo, W_hi, W_lo tiles -> 128B-swizzled smem ring
//       warp 1       MMA issuer: tcgen05.mma kind::f16, three passes per k-step
//                    (x_lo·W_hi + x_hi·W_lo + x_hi·W_hi), fp32 accumulators in TMEM, two
//                    accumulator buffers so the epilogue overlaps the next 256-column chunk
//       warps 2-9    epilogue, two per TMEM quadrant: TMEM -> registers, undo the operand
//                    scales, add t·(±s·A)ᵀ from the staged A rows (packed fp32 pairs), LIF
//                    step, store spikes
//       warps 10-25  noise generators, four per quadrant: regenerate the A rows of the
//                    quadrant's antithetic pair, sixteen output columns at a time, into a
//                    shared-memory ring of eight such items, ahead of the MMAs; an item is
//                    produced by one generator warp and consumed by one epilogue warp, so a
//                    generator always has a free slot to write while its last item is read
// Three fp16 passes on scaled hi/lo operands make every product fp32-equivalent (2^-21
// relative residue); a single pass would break the spike tolerance.  No TMA multicast and no
// cluster launch is used anywhere.  Every barrier wait is bounded: a wait that runs out
// records a code in the context's status word, all roles leave their loops, TMEM is released
// and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "linear.cuh"
#include "tc_common.cuh"

namespace hses {

namespace {

using namespace tc;

constexpr int BM_TILE = 128;      // rows per M tile (TMEM lanes)
constexpr int BK = 64;            // fp16 elements per k-block = one 128 B swizzle row
// warps: 0 TMA, 1 MMA, 2-9 epilogue (two per TMEM quadrant), 10-25 noise generators
constexpr int MAX_GENS = 4;        // generator warps per TMEM quadrant, at most
constexpr int MAX_DEPTH = 8;       // ring slots (items) per TMEM quadrant, at most
constexpr int NTHREADS = 32 * (10 + 4 * MAX_GENS);
constexpr int EPI_WARP0 = 2;
constexpr int GEN_WARP0 = 10;

// One ring item holds the A rows of ROWS consecutive output columns of one antithetic pair.
// With rank >= 8 two lanes share a row (each generates half of its rank values), an item covers 16
// columns and belongs to one epilogue warp; with rank 4 a lane owns a row, an item covers 32
// columns and both epilogue warps of the quadrant read it.  Inside a slot the value (q, n) sits
// at float (q % NPL) * 32 + (q / NPL) * ROWS + n: the lanes of a store cover 32 consecutive
// floats, and an epilogue warp reads four neighbouring columns of one q with a 16-byte broadcast.
template <int RG>
struct Item {
    static constexpr int RANK = RG * 4;
    static constexpr int LPR = RG >= 2 ? 2 : 1;      // lanes per row
    static constexpr int ROWS = 32 / LPR;
    static constexpr int NPL = RG > 0 ? RANK / LPR : 4;  // normals per lane and item
    static constexpr int SLOT_FLOATS = ROWS * RANK;
    __device__ __forceinline__ static int at(int q, int n) { return (q % NPL) * 32 + (q / NPL) * ROWS + n; }
};
inline int item_rows(int rank) { return rank >= 8 ? 16 : 32; }
inline int item_normals_per_lane(int rank) { return rank >= 8 ? rank / 2 : rank; }
struct TcArgs {
    int64_t rows;
    int k, a;
    int bm;
    int64_t n_pop;
    int perturb, lif;
    int rank;        // columns of t and of a staged A row: the factor rank rounded up to a multiple of 4
    int rank_true;   // the factor rank itself (1, 2, 3, or equal to rank)
    int one_pass;    // 1: operands rounded to bf16, a single MMA pass (no hi/lo split)
    int row_a0;      // first row of the output-side factor in a member's (a+k, rank) stream block
    uint64_t key;
    int32_t true_epoch, first_thread;
    float base_sigma, leak, v_th, out_scale;
    const float* t;       // (rows, t_stride): rank columns per group of output columns
    int t_stride;         // floats between rows of t: groups * rank
    int group_cols;       // output columns per group (several stacked parameters), 0: one parameter
    const float* out_scale_ptr;  // device gain overriding out_scale, or NULL
    const float* row_scale;  // (rows): 2^-e of the power-of-two scale applied to each x row
    const float* col_scale;  // (a):    the same for each row of the parameter
    float* out;
    int64_t out_stride;
    float* pot;
    const uint64_t* pow2; // T^(2^k) tables
    const uint64_t* hop;  // generator advance from the end of one item of a warp to its next one
    const int* x_lo_flag; // 0 when every lo half of the split x is zero (x exactly representable in fp16)
    const float* cache_a; // cached raw A rows (pair, a, rank) from the call's first pair on, or NULL
    LibmCal cal;
    int* status;
    // Ring slots (items) per TMEM quadrant and active generator warps per quadrant.  A slot must
    // always be written by the same generator warp and read by the same epilogue warp(s): waits
    // are on barrier phase parity, and a waiter that could fall two phases behind would take an
    // older phase for the one it waits for.  Hence ring_depth is a multiple of gens, and even
    // when an item belongs to one of the two epilogue warps.
    int ring_depth, gens;
    // Operand ring: stages in use and bytes per stage.  The one-pass mode loads one x tile and one W
    // tile per k-block instead of two of each, so the same shared memory holds twice the stages.
    int n_stages, stage_bytes;
};

template <int BN>
struct TcSmem {
    static constexpr int STAGES = BN == 256 ? 2 : 3;   // with both halves of both operands in a stage
    static constexpr int MAX_STAGES = 2 * STAGES;      // with one half of each (one-pass mode)
    static constexpr int X_BYTES = BM_TILE * BK * 2;
    static constexpr int W_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = 2 * X_BYTES + 2 * W_BYTES;
    static constexpr int HOP_BYTES = 0;     // the hop table is read through L1;
    static constexpr int TAB_BYTES = 1280;  // the logarithm's helper table and the thresholds as 2 x 128 bytes
    static constexpr int BAR_BYTES = 656;
    static constexpr int FIXED = STAGES * STAGE_BYTES + HOP_BYTES + TAB_BYTES + BAR_BYTES + 1024;
    static constexpr int LIMIT = 232448;  // 227 KB of dynamic shared memory per CTA
    // ring of staged A rows: 4 quadrants * depth items * rows of an item * rank floats
    static int a_bytes(int depth, int rank) { return 4 * depth * item_rows(rank) * rank * 4; }
};

// Eight consecutive floats of an output row: one 256-bit store when `wide` (p on a 32-byte boundary),
// else two 16-byte stores.  streaming: written once and not read again by this kernel.
__device__ __forceinline__ void store8(float* p, const float (&v)[8], bool wide, bool streaming) {
    if (wide) {
        if (streaming)
            asm volatile("st.global.cs.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(v[0]), "f"(v[1]),
                         "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
                         : "memory");
        else
            asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(v[0]), "f"(v[1]),
                         "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
                         : "memory");
    } else if (streaming) {
        __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
        __stcs(reinterpret_cast<float4*>(p + 4), make_float4(v[4], v[5], v[6], v[7]));
    } else {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// ----------------------------------------------------------------------- kernel
// R1: the factor rank is 1 (run as RG = 1): the epilogue leaves out the three zero columns of t and A.
// GRP: several stacked parameters (n_groups): an instance of its own, so that the reload of t per column
// group costs the other calls neither registers nor instructions (it made the rank-16 epilogue spill).
// RG = rank / 4 (0: clean product, no noise).  The rank is a template parameter so that the
// per-column dot product unrolls exactly and the epilogue loop stays small enough for the
// instruction cache.
template <int BN, int RG, bool R1 = false, bool GRP = false>
__global__ void __launch_bounds__(NTHREADS, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap tm_xhi, const __grid_constant__ CUtensorMap tm_xlo,
                 const __grid_constant__ CUtensorMap tm_whi, const __grid_constant__ CUtensorMap tm_wlo,
                 const TcArgs g) {
    using S = TcSmem<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;
    double2* log_tab_s = reinterpret_cast<double2*>(smem + S::STAGES * S::STAGE_BYTES + S::HOP_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::STAGES * S::STAGE_BYTES + S::HOP_BYTES + S::TAB_BYTES);
    float* a_stage = reinterpret_cast<float*>(smem + S::STAGES * S::STAGE_BYTES + S::HOP_BYTES + S::TAB_BYTES +
                                              S::BAR_BYTES);
    uint64_t* full = bars;                   // [STAGES] TMA landed
    uint64_t* empty = bars + S::MAX_STAGES;      // [MAX_STAGES] MMAs finished reading the stage
    uint64_t* tfull = bars + 2 * S::MAX_STAGES;  // [2] accumulator ready
    uint64_t* tempty = tfull + 2;            // [2] accumulator drained
    uint64_t* afull = tempty + 2;                     // [4][MAX_DEPTH] ring slot staged
    uint64_t* aempty = afull + 4 * MAX_DEPTH;         // [4][MAX_DEPTH] ring slot consumed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aempty + 4 * MAX_DEPTH);
    volatile int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (int)(g.rows / BM_TILE);
    const int n_chunks = (g.a + BN - 1) / BN;   // columns past a in the last chunk: zero rows of W (TMA fill), never stored
    const int k_blocks = (g.k + BK - 1) / BK;  // a ragged last block is zero-filled by TMA
    // inside a stage: x hi, (x lo,) W hi, (W lo); the one-pass mode packs the two tiles it loads
    const int w_off = g.one_pass ? TcSmem<BN>::X_BYTES : 2 * TcSmem<BN>::X_BYTES;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < S::MAX_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 256);
        }
        for (int i = 0; i < 4 * MAX_DEPTH; ++i) {
            mbar_init(&afull[i], 32);
            mbar_init(&aempty[i], Item<RG>::LPR == 2 ? 32 : 64);   // one or both epilogue warps read an item
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // small read-only tables go to shared memory: the epilogue's noise regeneration
    // looks them up for every normal
    if (RG > 0) {
        for (int i = threadIdx.x; i < 64; i += NTHREADS) log_tab_s[i] = g.cal.log_tab[i];
        // thresholds of the rounding filter as bytes (ceil(log2)), one per 1/128 of the input range
        // (the larger of the two 1/256 thresholds): 256 bytes instead of 2 KB
        uint8_t* thr_s = reinterpret_cast<uint8_t*>(log_tab_s + 64);
        for (int i = threadIdx.x; i < 128; i += NTHREADS) {
            const uint32_t tl = max(g.cal.log_delta[2 * i], g.cal.log_delta[2 * i + 1]);
            const uint32_t tc_ = max(g.cal.cos_delta[2 * i], g.cal.cos_delta[2 * i + 1]);
            thr_s[i] = pack_threshold_log2(tl);
            thr_s[128 + i] = pack_threshold_log2(tc_);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(2 * BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            // inputs that are exact in fp16 (0/1 spikes, small integers) have an all-zero lo half:
            // its tiles are neither loaded nor multiplied
            const bool skip_xlo = g.one_pass || *g.x_lo_flag == 0;
            for (int mt = blockIdx.x; mt < m_tiles && ok; mt += gridDim.x) {
                for (int c = 0; c < n_chunks && ok; ++c) {
                    for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                        int s = it % g.n_stages;
                        uint32_t ph = (it / g.n_stages) & 1;
                        if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, g.status, 1)) { ok = false; break; }
                        uint8_t* st = stage_base + s * g.stage_bytes;
                        mbar_expect_tx(&full[s], (skip_xlo ? 1 : 2) * S::X_BYTES + (g.one_pass ? 1 : 2) * S::W_BYTES);
                        tma_load_2d(st, &tm_xhi, kb * BK, mt * BM_TILE, &full[s]);
                        if (!skip_xlo) tma_load_2d(st + S::X_BYTES, &tm_xlo, kb * BK, mt * BM_TILE, &full[s]);
                        tma_load_2d(st + w_off, &tm_whi, kb * BK, c * BN, &full[s]);
                        if (!g.one_pass) tma_load_2d(st + w_off + S::W_BYTES, &tm_wlo, kb * BK, c * BN, &full[s]);
                    }
                }
            }
            if (!ok) {
                // copies already issued still land in this CTA's shared memory: give them a
                // bounded moment before the block is torn down
                for (int s = 0; s < g.n_stages; ++s)
                    for (uint32_t i = 0; i < 4096; ++i) {
                        if (mbar_try(&full[s], 0) || mbar_try(&full[s], 1)) break;
                        __nanosleep(256);
                    }
            }
        }
    } else if (warp == 1) {
        // --------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = g.one_pass ? make_idesc_bf16(BN) : make_idesc(BN);
            uint32_t it = 0, acc_it = 0;
            bool ok = true;
            const bool skip_xlo = g.one_pass || *g.x_lo_flag == 0;
            for (int mt = blockIdx.x; mt < m_tiles && ok; mt += gridDim.x) {
                for (int c = 0; c < n_chunks && ok; ++c, ++acc_it) {
                    int b = acc_it & 1;
                    if (!mbar_wait(&tempty[b], ((acc_it >> 1) & 1) ^ 1, abort_flag, g.status, 2)) { ok = false; break; }
                    tc_fence_after();
                    uint32_t d = tmem_base + (uint32_t)(b * BN);
                    for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                        int s = it % g.n_stages;
                        uint32_t ph = (it / g.n_stages) & 1;
                        if (!mbar_wait(&full[s], ph, abort_flag, g.status, 3)) { ok = false; break; }
                        tc_fence_after();
                        uint8_t* st = stage_base + s * g.stage_bytes;
                        uint64_t dxh = make_smem_desc(st), dxl = make_smem_desc(st + S::X_BYTES);
                        uint64_t dwh = make_smem_desc(st + w_off);
                        uint64_t dwl = make_smem_desc(st + w_off + S::W_BYTES);
#pragma unroll
                        for (int ks = 0; ks < BK / 16; ++ks) {
                            uint64_t off = (uint64_t)(ks * 32 >> 4);  // 16 fp16 = 32 B along K
                            if (g.one_pass) {
                                umma_f16(d, dxh + off, dwh + off, idesc, (kb | ks) != 0);
                                continue;
                            }
                            if (!skip_xlo) umma_f16(d, dxl + off, dwh + off, idesc, (kb | ks) != 0);
                            umma_f16(d, dxh + off, dwl + off, idesc, skip_xlo ? (uint32_t)((kb | ks) != 0) : 1u);
                            umma_f16(d, dxh + off, dwh + off, idesc, 1);
                        }
                        umma_commit(&empty[s]);
                    }
                    if (ok) umma_commit(&tfull[b]);
                }
            }
        }
    } else if (warp < GEN_WARP0) {
        // ----------------------------------------------- epilogue (two warps per TMEM quadrant:
        // warp (q4, eh) takes columns [16*eh, 16*eh+16) of every 32-column block, eight at a time:
        // the TMEM load of eight accumulators is issued first and waited for only after the
        // rank-r term of those columns has been summed from the staged A rows)
        using IT = Item<RG>;
        constexpr int RANK = RG * 4;
        // 8-column pieces in flight: with rank <= 4 the registers hold two, and nothing else would
        // cover the latency of the accumulator load
        constexpr int H = RG <= 1 ? 2 : 1;
        const int q4 = warp & 3;  // TMEM lane quadrant this warp may read (warp id mod 4)
        const int eh = (warp - EPI_WARP0) >> 2;
        const float out_scale = g.out_scale_ptr ? *g.out_scale_ptr : g.out_scale;
        // every 8-column piece of every output row starts on a 32-byte boundary
        const bool wide_out = (reinterpret_cast<uintptr_t>(g.out) & 31) == 0 && (g.out_stride & 7) == 0 &&
                              (!g.pot || (reinterpret_cast<uintptr_t>(g.pot) & 31) == 0);
        const int depth = g.ring_depth;
        const int items_per_tile = g.a / IT::ROWS;
        uint32_t acc_it = 0;
        uint32_t tile_no = 0;  // M tiles this CTA has finished: fixes how often each ring slot was used
        bool ok = true;
        for (int mt = blockIdx.x; mt < m_tiles && ok; mt += gridDim.x, ++tile_no) {
            const int64_t R = (int64_t)mt * BM_TILE + q4 * 32 + lane;
            f32x2 tq2[RANK > 0 ? RANK : 1];
            bool odd_member = false;
            const float rs = g.row_scale ? g.row_scale[R] : 1.0f;
            if (RG > 0) {
                int64_t member = (R / g.bm) % g.n_pop;
                int32_t thread_id = g.first_thread + (int32_t)member;
                odd_member = (thread_id & 1) != 0;  // sign -1: A of the pair is negated for this row
#pragma unroll
                for (int q = 0; q < RANK; q += 4) {
                    float4 tv = *reinterpret_cast<const float4*>(g.t + (size_t)R * (GRP ? g.t_stride : RANK) + q);
                    tq2[q] = pk2(tv.x, tv.x); tq2[q + 1] = pk2(tv.y, tv.y);
                    tq2[q + 2] = pk2(tv.z, tv.z); tq2[q + 3] = pk2(tv.w, tv.w);
                }
            }
            for (int c = 0; c < n_chunks && ok; ++c, ++acc_it) {
                int b = acc_it & 1;
                if (!mbar_wait(&tfull[b], (acc_it >> 1) & 1, abort_flag, g.status, 6)) { ok = false; break; }
                tc_fence_after();
                for (int cb = 0; cb < BN / 32 && ok; ++cb) {
                    const int n0 = c * BN + cb * 32 + eh * 16;   // first of this warp's sixteen columns
                    if (n0 >= g.a) continue;                     // ragged last chunk: no such columns, no such item
                    const float* my_a = nullptr;
                    int slot = 0;
                    if (GRP && RG > 0) {
                        // stacked parameters: these columns' group has its own t (its own B)
                        const float* tg = g.t + (size_t)R * g.t_stride + (n0 / g.group_cols) * RANK;
#pragma unroll
                        for (int q = 0; q < RANK; q += 4) {
                            float4 tv = *reinterpret_cast<const float4*>(tg + q);
                            tq2[q] = pk2(tv.x, tv.x); tq2[q + 1] = pk2(tv.y, tv.y);
                            tq2[q + 2] = pk2(tv.z, tv.z); tq2[q + 3] = pk2(tv.w, tv.w);
                        }
                    }
                    if (RG > 0) {
                        // the item that holds these columns: one generator warp staged it
                        const uint32_t item = tile_no * (uint32_t)items_per_tile +
                                              (uint32_t)(IT::LPR == 2 ? (n0 >> 4) : (n0 >> 5));
                        slot = (int)(item % (uint32_t)depth);
                        if (!mbar_wait(&afull[q4 * MAX_DEPTH + slot], (item / (uint32_t)depth) & 1, abort_flag, g.status, 7)) {
                            ok = false;
                            break;
                        }
                        my_a = a_stage + (q4 * depth + slot) * IT::SLOT_FLOATS + (IT::LPR == 2 ? 0 : eh * 16);
                    }
                    float* orow = g.out + (size_t)R * g.out_stride + n0;
                    float* prow = (g.lif && g.pot) ? g.pot + (size_t)R * g.out_stride + n0 : nullptr;
#pragma unroll 1
                    for (int j0 = 0; j0 < 16; j0 += 8 * H) {
                        uint32_t acc[H][8];
#pragma unroll
                        for (int h = 0; h < H; ++h)
                            tmem_ld8_issue(tmem_base + ((uint32_t)(q4 * 32) << 16) +
                                           (uint32_t)(b * BN + cb * 32 + eh * 16 + j0 + 8 * h), acc[h]);
                        float cs[H][8];
#pragma unroll
                        for (int h = 0; h < H; ++h) {
                            // the one-pass mode scales nothing: no loads then
                            const float4 cs0 = g.one_pass ? make_float4(1.f, 1.f, 1.f, 1.f)
                                                          : *reinterpret_cast<const float4*>(g.col_scale + n0 + j0 + 8 * h);
                            const float4 cs1 = g.one_pass ? make_float4(1.f, 1.f, 1.f, 1.f)
                                                          : *reinterpret_cast<const float4*>(g.col_scale + n0 + j0 + 8 * h + 4);
                            cs[h][0] = cs0.x; cs[h][1] = cs0.y; cs[h][2] = cs0.z; cs[h][3] = cs0.w;
                            cs[h][4] = cs1.x; cs[h][5] = cs1.y; cs[h][6] = cs1.z; cs[h][7] = cs1.w;
                        }
                        // u[j] = sum_q t[q] * (base_sigma * A[n0+j0+j][q]), q ascending, one rounding per
                        // multiply-add; two neighbouring columns advance together in one packed fma
                        f32x2 u2[H][4];
#pragma unroll
                        for (int h = 0; h < H; ++h) u2[h][0] = u2[h][1] = u2[h][2] = u2[h][3] = 0ull;
                        if (RG > 0) {
#pragma unroll
                            for (int q = 0; q < (R1 ? 1 : RANK); ++q) {   // zero columns add nothing
#pragma unroll
                                for (int h = 0; h < H; ++h) {
                                    const ulonglong2 a01 = *reinterpret_cast<const ulonglong2*>(my_a + IT::at(q, j0 + 8 * h));
                                    const ulonglong2 a23 = *reinterpret_cast<const ulonglong2*>(my_a + IT::at(q, j0 + 8 * h + 4));
                                    u2[h][0] = fma2(tq2[q], a01.x, u2[h][0]);
                                    u2[h][1] = fma2(tq2[q], a01.y, u2[h][1]);
                                    u2[h][2] = fma2(tq2[q], a23.x, u2[h][2]);
                                    u2[h][3] = fma2(tq2[q], a23.y, u2[h][3]);
                                }
                            }
                        }
                        tmem_ld_wait();
#pragma unroll
                        for (int h = 0; h < H; ++h) {
                            float u[8];
                            upk2(u2[h][0], u[0], u[1]); upk2(u2[h][1], u[2], u[3]);
                            upk2(u2[h][2], u[4], u[5]); upk2(u2[h][3], u[6], u[7]);
                            float y[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                // undo the two power-of-two operand scales (exact); the member's sign is applied to
                                // the finished sum (negating every term of a sum negates the sum exactly)
                                float v = __fmul_rn(__fmul_rn(__uint_as_float(acc[h][j]), rs), cs[h][j]);
                                if (RG > 0) v = __fadd_rn(v, odd_member ? -u[j] : u[j]);
                                y[j] = v;
                            }
                            // eight consecutive outputs of a row are one 32-byte sector: a single 256-bit store
                            // where the row starts on a sector boundary (half the store instructions and half
                            // the data-path cycles of two 16-byte stores, which is what the epilogue spends
                            // most of its time on once the product is a single pass)
                            if (g.lif) {
                                float cv[8], sv[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    cv[j] = __fmul_rn(y[j], g.leak);
                                    sv[j] = cv[j] >= g.v_th ? 1.0f : 0.0f;
                                }
                                if (prow) store8(prow + j0 + 8 * h, cv, wide_out, false);
                                store8(orow + j0 + 8 * h, sv, wide_out, true);
                            } else {
                                float o[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) o[j] = __fmul_rn(y[j], out_scale);
                                store8(orow + j0 + 8 * h, o, wide_out, false);
                            }
                        }
                    }
                    if (RG > 0) mbar_arrive(&aempty[q4 * MAX_DEPTH + slot]);  // the item's reader(s) hand the slot back
                }
                tc_fence_before();
                mbar_arrive(&tempty[b]);
            }
        }
    } else if (RG > 0 && (warp - GEN_WARP0) / 4 < g.gens) {
        // ------------------------------------------------------------ noise generators
        // Generator (gq, gi) regenerates, for TMEM quadrant gq, the A rows of every gens-th item
        // (ROWS output columns of the quadrant's antithetic pair), scaled by base_sigma, into the
        // ring slot the item maps to.  It runs ahead of the epilogue and never touches TMEM, so the
        // regeneration overlaps the MMAs.
        using IT = Item<RG>;
        constexpr int RANK = RG * 4;
        const int gq = (warp - GEN_WARP0) & 3, gi = (warp - GEN_WARP0) >> 2;
        const int depth = g.ring_depth, GENS = g.gens;
        LibmCal cal = g.cal;
        cal.log_tab = log_tab_s;
        cal.log_delta = reinterpret_cast<const uint32_t*>(log_tab_s + 64);                         // byte tables, see
        cal.cos_delta = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(log_tab_s + 64) + 128);  // next_normals4_t<true, 17>
        LibmCal cal4 = g.cal;      // the one-at-a-time generator of ranks 1..3 reads the 32-bit thresholds
        cal4.log_tab = log_tab_s;
        const int items_per_tile = g.a / IT::ROWS;
        const int n_local = lane % IT::ROWS, qoff = (lane / IT::ROWS) * IT::NPL;   // this lane's row and first rank index
        float* const lane_a = a_stage + (size_t)gq * depth * IT::SLOT_FLOATS + (lane / IT::ROWS) * IT::ROWS + n_local;
        uint32_t tile_no = 0;
        bool ok = true;
        for (int mt = blockIdx.x; mt < m_tiles && ok; mt += gridDim.x, ++tile_no) {
            // every row of this quadrant's 32-row slice belongs to one antithetic pair
            int64_t member0 = (((int64_t)mt * BM_TILE + gq * 32) / g.bm) % g.n_pop;
            int32_t pair = (g.first_thread + (int32_t)member0) / 2;
            // Items are numbered through all tiles of this CTA; this warp takes those with
            // item % GENS == gi, so that a ring slot (item % depth, depth a multiple of GENS) is
            // always written by the same warp.  it0: its first item inside this tile.
            const int it0 = (int)(((uint32_t)gi + (uint32_t)GENS - (tile_no * (uint32_t)items_per_tile) % (uint32_t)GENS) % (uint32_t)GENS);
            // cached factors: this lane's share of row (item * ROWS + n_local) of the pair, raw normals
            // (ranks 1..3 run as rank 4 with zero columns: rt values per row in the stream and in a cache)
            const int rt = g.rank_true;
            const float* src = g.cache_a ? g.cache_a + ((size_t)(pair - g.first_thread / 2) * g.a + it0 * IT::ROWS + n_local) * rt + qoff
                                         : nullptr;
            uint64_t a_state = 0;
            if (!src) {
                uint64_t s0 = noise_seed(g.key, g.true_epoch, pair) | 1ull;
                a_state = jump_by(g.pow2, s0, 2ull * ((uint64_t)rt * (uint64_t)(g.row_a0 + it0 * IT::ROWS + n_local) + (uint64_t)qoff));
            }
            for (int it = it0; it < items_per_tile; it += GENS) {
                const uint32_t item = tile_no * (uint32_t)items_per_tile + (uint32_t)it;
                const int slot = (int)(item % (uint32_t)depth);
                float4 v[IT::NPL / 4];
                if (src) {   // the loads fly while the slot is waited for
                    if (rt < 4) {
                        v[0] = make_float4(__ldg(src), rt > 1 ? __ldg(src + 1) : 0.0f, rt > 2 ? __ldg(src + 2) : 0.0f, 0.0f);
                    } else {
#pragma unroll
                        for (int c4 = 0; c4 < IT::NPL / 4; ++c4) v[c4] = __ldg(reinterpret_cast<const float4*>(src) + c4);
                    }
                    src += (size_t)GENS * IT::ROWS * rt;
                }
                if (!mbar_wait(&aempty[gq * MAX_DEPTH + slot], ((item / (uint32_t)depth) & 1) ^ 1, abort_flag, g.status, 8)) {
                    ok = false;
                    break;
                }
                float* dst = lane_a + slot * IT::SLOT_FLOATS;
#pragma unroll 1
                for (int c4 = 0; c4 < IT::NPL / 4; ++c4) {
                    float z[4];
                    if (src) {
                        z[0] = v[c4].x; z[1] = v[c4].y; z[2] = v[c4].z; z[3] = v[c4].w;
                    } else if (rt < 4) {
                        z[1] = z[2] = z[3] = 0.0f;
                        z[0] = next_normal(a_state, cal4);
                        if (rt > 1) z[1] = next_normal(a_state, cal4);
                        if (rt > 2) z[2] = next_normal(a_state, cal4);
                    } else {
                        next_normals4_t<true, 17>(a_state, cal, z);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) dst[(4 * c4 + j) * 32] = __fmul_rn(z[j], g.base_sigma);
                }
                if (!src) a_state = jump_apply(g.hop, a_state);  // on to this generator's next item
                mbar_arrive(&afull[gq * MAX_DEPTH + slot]);       // 32 arrivals publish the item
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
}

// ------------------------------------------------------------ auxiliary kernels
// Operand preparation: every row is multiplied by a power of two that brings its largest
// magnitude into [2^13, 2^14) and then split into two fp16 values, hi = fp16(v) and
// lo = fp16(v - hi).  hi + lo carries 22 significant bits of v, and three fp16 MMA passes
// (hi*hi + hi*lo + lo*hi, fp32 accumulate) give fp32-equivalent products at the fp16 tensor
// rate and with half the shared-memory traffic of a TF32 split.  The scales are undone exactly
// in the epilogue.  One warp per row; rows are multiples of four long and 16-byte aligned.
// bf16 != 0: one-pass mode, hi = bf16(v) with no scale and no lo half (bf16 has the range of fp32).
__global__ void split_f16_rows_kernel(const float* __restrict__ x, int64_t rows, int k, int64_t stride,
                                      __half* __restrict__ hi, __half* __restrict__ lo,
                                      float* __restrict__ inv_scale, int* __restrict__ lo_flag, int bf16) {
    int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (r >= rows) return;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)r * stride);
    int n4 = k >> 2;
    if (bf16) {
        if (lane == 0) inv_scale[r] = 1.0f;
        uint2* dh = reinterpret_cast<uint2*>(hi + (size_t)r * k);
        for (int i = lane; i < n4; i += 32) {
            const float4 v = src[i];
            const __nv_bfloat162 b01 = __floats2bfloat162_rn(v.x, v.y), b23 = __floats2bfloat162_rn(v.z, v.w);
            dh[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&b01), *reinterpret_cast<const uint32_t*>(&b23));
        }
        return;
    }
    float m = 0.0f;
    for (int i = lane; i < n4; i += 32) {
        float4 v = src[i];
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    // exponent of the row maximum; zero, denormal, infinite or NaN rows keep scale 1
    int ex = (int)((__float_as_uint(m) >> 23) & 0xffu) - 127;
    int e = 13 - ex;
    if (ex <= -127 || ex >= 128) e = 0;
    if (e > 100) e = 100;
    if (e < -100) e = -100;
    float s = __uint_as_float((uint32_t)(127 + e) << 23);
    if (lane == 0) inv_scale[r] = __uint_as_float((uint32_t)(127 - e) << 23);
    uint2* dh = reinterpret_cast<uint2*>(hi + (size_t)r * k);
    uint2* dl = reinterpret_cast<uint2*>(lo + (size_t)r * k);
    uint32_t nz = 0;
    for (int i = lane; i < n4; i += 32) {
        float4 v = src[i];
        float f[4] = {v.x * s, v.y * s, v.z * s, v.w * s};
        __half h[4], l[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            h[j] = __float2half_rn(f[j]);
            l[j] = __float2half_rn(f[j] - __half2float(h[j]));
        }
        dh[i] = make_uint2((uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16),
                           (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16));
        const uint2 lw = make_uint2((uint32_t)__half_as_ushort(l[0]) | ((uint32_t)__half_as_ushort(l[1]) << 16),
                                    (uint32_t)__half_as_ushort(l[2]) | ((uint32_t)__half_as_ushort(l[3]) << 16));
        dl[i] = lw;
        nz |= (lw.x | lw.y) & 0x7fff7fffu;  // a lo half of -0 is still zero
    }
    // one flag per call tells the GEMM whether any lo half is non-zero (checked first: a set flag is not set again)
    if (lo_flag != nullptr && __any_sync(0xffffffffu, nz != 0) && lane == 0 && *reinterpret_cast<volatile int*>(lo_flag) == 0)
        atomicOr(lo_flag, 1);
}

// t[R, q] = sum_k x[R, k] * B_pair[k, q].  CTA (pair, chunk) takes up to LT_ROWS of the pair's rows
// (all time steps of both members count) and, on the way, writes the fp16 hi/lo split of those
// x rows (see split_f16_rows_kernel) so that x is read from HBM once.
//
// B is produced block by block in shared memory, LT_KB rows at a time, one row per thread: either
// regenerated from the pair's stream or copied from a factor cache.  A pair with many rows is
// spread over several CTAs, each regenerating the pair's B: that costs k*rank normals per CTA
// against LT_ROWS*k*rank multiply-adds, and buys the parallelism small populations need.
//
// The product is laid out so that neither operand is the bottleneck of the load pipe: a warp owns
// a tile of 8 rows; its lanes are (k-slice, group of four q), so the B block is read with
// conflict-free 16-byte loads that are reused for all 8 rows, and x is read straight from global
// memory, 16 bytes per lane and one 128-byte line per warp.  Each lane accumulates its k-slice
// over the whole of k; the slices are added with shuffles at the end.  When the CTA has fewer
// than eight row tiles the idle warps take a share of every B block (k-parts) and the parts are
// added in a fixed order through shared memory.  RANK_G = rank / 4.
constexpr int LT_THREADS = 256;
constexpr int LT_ROWS = 64;
constexpr int LT_KB = 256;
template <int RANK_G>
__global__ void __launch_bounds__(LT_THREADS, 2)
lowrank_t_kernel(LibmCal cal, const uint64_t* __restrict__ pow2, const uint64_t* __restrict__ hop_kb,
                 uint64_t key, int32_t true_epoch, int32_t first_thread, const float* __restrict__ x,
                 int64_t x_stride, int t_steps, int64_t n_pop, int bm, int k, float* __restrict__ t,
                 __half* __restrict__ xhi, __half* __restrict__ xlo, float* __restrict__ inv_scale,
                 const float* __restrict__ cache_b, int* __restrict__ lo_flag, int bf16, int rank_true, int row_b0,
                 int skip_split) {
    constexpr int RANK = RANK_G * 4;
    constexpr int KQ = 32 / RANK_G;   // lanes along k
    constexpr int KSTEP = 4 * KQ;     // k covered by one pass of a warp
    __shared__ __align__(16) float bs[LT_KB * RANK];  // one block of B; reused for the k-part sums
    __shared__ uint64_t hop_s[kJumpWords];
    __shared__ double2 log_tab_s[64];
    __shared__ uint32_t delta_s[512];
    __shared__ int64_t row_s[LT_ROWS];  // global row of each of this CTA's rows
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (!cache_b) {
        for (int i = tid; i < kJumpWords; i += LT_THREADS) hop_s[i] = hop_kb[i];
        for (int i = tid; i < 64; i += LT_THREADS) log_tab_s[i] = cal.log_tab[i];
        for (int i = tid; i < 256; i += LT_THREADS) {
            delta_s[i] = cal.log_delta[i];
            delta_s[256 + i] = cal.cos_delta[i];
        }
        cal.log_tab = log_tab_s;
        cal.log_delta = delta_s;
        cal.cos_delta = delta_s + 256;
    }
    const int32_t first_pair = first_thread / 2;
    const int32_t pair = first_pair + blockIdx.x;
    // members of this pair inside the population slice
    int64_t m_lo = (int64_t)pair * 2 - first_thread, m_hi = m_lo + 2;
    if (m_lo < 0) m_lo = 0;
    if (m_hi > n_pop) m_hi = n_pop;
    const int rows_per_step = (int)(m_hi - m_lo) * bm;
    const int row0 = blockIdx.y * LT_ROWS;  // first of this CTA's rows among the pair's rows
    const int total_rows = min(LT_ROWS, rows_per_step * t_steps - row0);
    if (total_rows <= 0) return;
    if (tid < LT_ROWS) {
        int lr = row0 + (tid < total_rows ? tid : total_rows - 1);  // rows past the end repeat the last one
        int step = lr / rows_per_step, rr = lr - step * rows_per_step;
        row_s[tid] = ((int64_t)step * n_pop + m_lo) * bm + rr;
    }
    __syncthreads();

    // ---- operand split of this CTA's x rows (one warp per row) ----
    const int n4 = k >> 2;
    uint32_t lo_nz = 0;  // any non-zero lo half written by this thread
    auto finish_row = [&](int64_t R, float m, float& sc) {
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        int ex = (int)((__float_as_uint(m) >> 23) & 0xffu) - 127;
        int e = 13 - ex;
        if (ex <= -127 || ex >= 128) e = 0;
        if (e > 100) e = 100;
        if (e < -100) e = -100;
        if (bf16) e = 0;   // one-pass mode: no scale
        sc = __uint_as_float((uint32_t)(127 + e) << 23);
        if (lane == 0) inv_scale[R] = __uint_as_float((uint32_t)(127 - e) << 23);
    };
    auto split4 = [&](float4 v, float sc, uint2& h2, uint2& l2) {
        if (bf16) {   // hi = bf16(v), the lo half is neither written nor read
            const __nv_bfloat162 b01 = __floats2bfloat162_rn(v.x, v.y), b23 = __floats2bfloat162_rn(v.z, v.w);
            h2 = make_uint2(*reinterpret_cast<const uint32_t*>(&b01), *reinterpret_cast<const uint32_t*>(&b23));
            l2 = make_uint2(0u, 0u);
            return;
        }
        const float x0 = v.x * sc, x1 = v.y * sc, x2 = v.z * sc, x3 = v.w * sc;
        const __half2 h01 = __floats2half2_rn(x0, x1), h23 = __floats2half2_rn(x2, x3);
        const float2 b01 = __half22float2(h01), b23 = __half22float2(h23);
        const __half2 l01 = __floats2half2_rn(x0 - b01.x, x1 - b01.y), l23 = __floats2half2_rn(x2 - b23.x, x3 - b23.y);
        h2 = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
        l2 = make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
        lo_nz |= (l2.x | l2.y) & 0x7fff7fffu;  // a lo half of -0 is still zero
    };
    if (skip_split) {
        // the operand split of these rows is already in the workspace (an earlier projection of the same x)
    } else if (n4 <= 32) {
        // short rows (up to 128 values): one 16-byte piece per lane covers a row, so a warp keeps eight
        // rows in flight, one trip to memory for all of them
        for (int lr0 = warp * 8; lr0 < total_rows; lr0 += 8 * (LT_THREADS / 32)) {
            float4 v[8];
            int64_t R[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool valid = lr0 + j < total_rows;   // warp-uniform
                R[j] = row_s[valid ? lr0 + j : lr0];
                v[j] = (valid && lane < n4) ? __ldg(reinterpret_cast<const float4*>(x + (size_t)R[j] * x_stride) + lane)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (lr0 + j >= total_rows) break;
                const float m = fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w)));
                float sc;
                finish_row(R[j], m, sc);
                if (lane < n4) {
                    uint2 h2, l2;
                    split4(v[j], sc, h2, l2);
                    reinterpret_cast<uint2*>(xhi + (size_t)R[j] * k)[lane] = h2;
                    if (!bf16) reinterpret_cast<uint2*>(xlo + (size_t)R[j] * k)[lane] = l2;
                }
            }
        }
    } else if (n4 <= 256) {
        // rows of up to 1024 values stay in registers between the maximum and the conversion, and a
        // warp keeps two rows in flight: one trip to memory per row instead of two dependent ones
        for (int lr = warp; lr < total_rows; lr += 2 * (LT_THREADS / 32)) {
            const int lr1 = lr + LT_THREADS / 32;
            const bool two = lr1 < total_rows;
            const int64_t R0 = row_s[lr], R1 = row_s[two ? lr1 : lr];
            const float4* s0 = reinterpret_cast<const float4*>(x + (size_t)R0 * x_stride);
            const float4* s1 = reinterpret_cast<const float4*>(x + (size_t)R1 * x_stride);
            float4 v0[8], v1[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = lane + 32 * j;
                v0[j] = i < n4 ? __ldg(s0 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                v1[j] = (two && i < n4) ? __ldg(s1 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float m0 = 0.0f, m1 = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                m0 = fmaxf(m0, fmaxf(fmaxf(fabsf(v0[j].x), fabsf(v0[j].y)), fmaxf(fabsf(v0[j].z), fabsf(v0[j].w))));
                m1 = fmaxf(m1, fmaxf(fmaxf(fabsf(v1[j].x), fabsf(v1[j].y)), fmaxf(fabsf(v1[j].z), fabsf(v1[j].w))));
            }
            float sc0, sc1 = 1.0f;
            finish_row(R0, m0, sc0);
            if (two) finish_row(R1, m1, sc1);   // warp-uniform branch
            uint2* dh0 = reinterpret_cast<uint2*>(xhi + (size_t)R0 * k);
            uint2* dl0 = reinterpret_cast<uint2*>(xlo + (size_t)R0 * k);
            uint2* dh1 = reinterpret_cast<uint2*>(xhi + (size_t)R1 * k);
            uint2* dl1 = reinterpret_cast<uint2*>(xlo + (size_t)R1 * k);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = lane + 32 * j;
                if (i < n4) {
                    uint2 h2, l2;
                    split4(v0[j], sc0, h2, l2);
                    dh0[i] = h2;
                    if (!bf16) dl0[i] = l2;
                    if (two) {
                        split4(v1[j], sc1, h2, l2);
                        dh1[i] = h2;
                        if (!bf16) dl1[i] = l2;
                    }
                }
            }
        }
    } else {
        for (int lr = warp; lr < total_rows; lr += LT_THREADS / 32) {
            const int64_t R = row_s[lr];
            const float4* src = reinterpret_cast<const float4*>(x + (size_t)R * x_stride);
            float m = 0.0f;
            for (int i = lane; i < n4; i += 32) {
                float4 v = src[i];
                m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
            float sc;
            finish_row(R, m, sc);
            uint2* dh = reinterpret_cast<uint2*>(xhi + (size_t)R * k);
            uint2* dl = reinterpret_cast<uint2*>(xlo + (size_t)R * k);
            for (int i = lane; i < n4; i += 32) {
                uint2 h2, l2;
                split4(src[i], sc, h2, l2);
                dh[i] = h2;
                if (!bf16) dl[i] = l2;
            }
        }
    }

    // one flag per call tells the GEMM whether any lo half is non-zero (a set flag is not set again)
    if (__any_sync(0xffffffffu, lo_nz != 0) && lane == 0 && *reinterpret_cast<volatile int*>(lo_flag) == 0)
        atomicOr(lo_flag, 1);

    // ---- t = x * B ----
    const int n_tiles = (total_rows + 7) >> 3;                     // 1..8
    const int ksplit = n_tiles <= 1 ? 8 : n_tiles <= 2 ? 4 : n_tiles <= 4 ? 2 : 1;
    const bool active = warp < n_tiles * ksplit;
    const int tile = warp % n_tiles, kpart = warp / n_tiles;
    const int part_len = LT_KB / ksplit;
    const int kq = lane / RANK_G, qg = lane - kq * RANK_G;
    const float* xrow[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) xrow[r] = x + (size_t)row_s[tile * 8 + r] * x_stride;
    float acc[8][4];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.0f;

    uint64_t sb = 0;
    if (!cache_b) {
        sb = noise_seed(key, true_epoch, pair) | 1ull;
        sb = jump_by(pow2, sb, 2ull * (uint64_t)rank_true * (uint64_t)(row_b0 + tid));   // row_b0: first input-side row
    }
    // cached raw B rows of this pair, (k, rank) row-major like the block in shared memory
    // (ranks 1..3: rank_true values per row, the remaining columns of the block are zero)
    const float4* cb4 = cache_b ? reinterpret_cast<const float4*>(cache_b + (size_t)blockIdx.x * k * RANK) : nullptr;
    const float* cb1 = cache_b ? cache_b + (size_t)blockIdx.x * k * rank_true : nullptr;
    for (int k0 = 0; k0 < k; k0 += LT_KB) {
        const int kn = k - k0 < LT_KB ? k - k0 : LT_KB;  // multiple of 4
        // Row k of the block is stored at row perm(k): inside every group of KSTEP rows the rows
        // with the same k mod 4 are made neighbours, so that the lanes of a warp — which own four
        // consecutive k each — read one contiguous 512-byte stretch per load (no bank conflicts).
        if (cb4 && rank_true < 4) {
            for (int kr = tid; kr < kn; kr += LT_THREADS) {
                const int pr = (kr / KSTEP) * KSTEP + (kr & 3) * KQ + ((kr % KSTEP) >> 2);
                const float* row = cb1 + (size_t)(k0 + kr) * rank_true;
                reinterpret_cast<float4*>(bs)[pr] = make_float4(__ldg(row), rank_true > 1 ? __ldg(row + 1) : 0.0f,
                                                               rank_true > 2 ? __ldg(row + 2) : 0.0f, 0.0f);
            }
        } else if (cb4) {
            for (int i = tid; i < kn * RANK_G; i += LT_THREADS) {
                const int kr = i / RANK_G, c = i - kr * RANK_G;
                const int pr = (kr / KSTEP) * KSTEP + (kr & 3) * KQ + ((kr % KSTEP) >> 2);
                reinterpret_cast<float4*>(bs)[pr * RANK_G + c] = __ldg(cb4 + (size_t)k0 * RANK_G + i);
            }
        } else if (tid < kn) {
            const int pr = (tid / KSTEP) * KSTEP + (tid & 3) * KQ + ((tid % KSTEP) >> 2);
            if (rank_true < 4) {
                float z[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                z[0] = next_normal(sb, cal);
                if (rank_true > 1) z[1] = next_normal(sb, cal);
                if (rank_true > 2) z[2] = next_normal(sb, cal);
                *reinterpret_cast<float4*>(bs + pr * RANK) = make_float4(z[0], z[1], z[2], z[3]);
            } else {
#pragma unroll 1
                for (int q = 0; q < RANK; q += 4) {
                    float z[4];
                    next_normals4(sb, cal, z);
                    *reinterpret_cast<float4*>(bs + pr * RANK + q) = make_float4(z[0], z[1], z[2], z[3]);
                }
            }
            sb = jump_apply(hop_s, sb);
        }
        __syncthreads();
        if (active) {
            const int kend = min(kpart * part_len + part_len, kn);
            for (int kk = kpart * part_len + 4 * kq; kk < kend; kk += KSTEP) {
                // rows kk..kk+3 live at perm(kk) + {0, KQ, 2KQ, 3KQ}
                const float* bq = bs + ((kk / KSTEP) * KSTEP + ((kk % KSTEP) >> 2)) * RANK + qg * 4;
                float4 b0 = *reinterpret_cast<const float4*>(bq);
                float4 b1 = *reinterpret_cast<const float4*>(bq + KQ * RANK);
                float4 b2 = *reinterpret_cast<const float4*>(bq + 2 * KQ * RANK);
                float4 b3 = *reinterpret_cast<const float4*>(bq + 3 * KQ * RANK);
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    float4 xv = __ldg(reinterpret_cast<const float4*>(xrow[r] + k0 + kk));
                    acc[r][0] = fmaf(xv.x, b0.x, acc[r][0]); acc[r][1] = fmaf(xv.x, b0.y, acc[r][1]);
                    acc[r][2] = fmaf(xv.x, b0.z, acc[r][2]); acc[r][3] = fmaf(xv.x, b0.w, acc[r][3]);
                    acc[r][0] = fmaf(xv.y, b1.x, acc[r][0]); acc[r][1] = fmaf(xv.y, b1.y, acc[r][1]);
                    acc[r][2] = fmaf(xv.y, b1.z, acc[r][2]); acc[r][3] = fmaf(xv.y, b1.w, acc[r][3]);
                    acc[r][0] = fmaf(xv.z, b2.x, acc[r][0]); acc[r][1] = fmaf(xv.z, b2.y, acc[r][1]);
                    acc[r][2] = fmaf(xv.z, b2.z, acc[r][2]); acc[r][3] = fmaf(xv.z, b2.w, acc[r][3]);
                    acc[r][0] = fmaf(xv.w, b3.x, acc[r][0]); acc[r][1] = fmaf(xv.w, b3.y, acc[r][1]);
                    acc[r][2] = fmaf(xv.w, b3.z, acc[r][2]); acc[r][3] = fmaf(xv.w, b3.w, acc[r][3]);
                }
            }
        }
        __syncthreads();
    }
    // add the k-slices of the lanes (lanes that differ in kq), lowest lanes end up with the sums
#pragma unroll
    for (int off = RANK_G; off < 32; off <<= 1)
#pragma unroll
        for (int r = 0; r < 8; ++r)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[r][j] += __shfl_xor_sync(0xffffffffu, acc[r][j], off);
    float* part = bs;  // [warp][8 rows][RANK]
    if (active && kq == 0) {
#pragma unroll
        for (int r = 0; r < 8; ++r)
            *reinterpret_cast<float4*>(part + (warp * 8 + r) * RANK + qg * 4) =
                make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
    __syncthreads();
    for (int e = tid; e < total_rows * RANK; e += LT_THREADS) {
        int lr = e / RANK, q = e - lr * RANK;
        int tl = lr >> 3, r = lr & 7;
        float sum = 0.0f;
        for (int p = 0; p < ksplit; ++p) sum += part[((tl + n_tiles * p) * 8 + r) * RANK + q];
        t[(size_t)row_s[lr] * RANK + q] = sum;
    }
}

// x_op of hses_linear_args on a piece of x as it arrives in registers
__device__ __forceinline__ float4 apply_x_op(float4 v, int x_op) {
    if (x_op == HSES_X_RELU_SQUARE) {
        const float a = fmaxf(v.x, 0.0f), b = fmaxf(v.y, 0.0f), c = fmaxf(v.z, 0.0f), d = fmaxf(v.w, 0.0f);
        v = make_float4(__fmul_rn(a, a), __fmul_rn(b, b), __fmul_rn(c, c), __fmul_rn(d, d));
    }
    return v;
}

// The prepass for layers whose rows fit the registers of a warp (k <= 1024) and whose whole B fits
// the shared memory of a CTA (ranks 1..4, 8, 16; ranks below 4 as rank 4 with zero columns, rank_true
// values per row in the stream and in the cache).  Phase 1: the 256 threads regenerate (or copy from
// the factor cache) all k rows of the pair's B into shared memory, each thread a run of consecutive
// rows, which are consecutive in the stream.  Phase 2: a warp loads RPR x rows into registers ONCE,
// NJ 16-byte pieces per lane and row (2 rows of up to 1024 values, 4 of up to 256, 8 of up to 128:
// as many as the registers hold), and does everything with them there: the row maximum, the fp16
// operand split, and t = x * B, each lane multiplying the pieces it holds with the matching rows of
// B and the warp adding its lanes' sums with a halving exchange.  lowrank_t_kernel reads x a second
// time, 128 bytes per row and trip, for its t product and spends as long waiting for those trips as
// on the generation.
// B row kr is stored at row p = (kr / 128) * 128 + (kr % 4) * 32 + (kr % 128) / 4, its 16-byte
// chunk c at chunk (c + p / (8 / RANK_G)) % RANK_G: the lanes of a warp, which hold pieces
// 32 apart, then read consecutive rows, eight of them covering all banks.
template <int RANK_G, int NJ, int RPR, bool HALF>
__global__ void __launch_bounds__(LT_THREADS, 2)
lowrank_t_rows_kernel(LibmCal cal, const uint64_t* __restrict__ pow2,
                      uint64_t key, int32_t true_epoch, int32_t first_thread, const float* __restrict__ x,
                      int64_t x_stride, int t_steps, int64_t n_pop, int bm, int k, float* __restrict__ t,
                      __half* __restrict__ xhi, __half* __restrict__ xlo, float* __restrict__ inv_scale,
                      const float* __restrict__ cache_b, int* __restrict__ lo_flag, int bf16, int rank_true,
                      int row_b0, int skip_split, int n_groups, int x_op) {
    constexpr int RANK = RANK_G * 4;
    constexpr int RP = 8 / RANK_G;    // rows of B per 128 bytes
    constexpr int ROWS_CTA = HALF ? 2 * LT_ROWS : LT_ROWS;   // x rows per CTA
    extern __shared__ __align__(16) float bsm[];   // ceil(k / 128) * 128 rows of RANK floats
    __shared__ double2 log_tab_s[64];
    __shared__ uint32_t delta_s[512];
    __shared__ int64_t row_s[ROWS_CTA];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (!cache_b) {
        for (int i = tid; i < 64; i += LT_THREADS) log_tab_s[i] = cal.log_tab[i];
        for (int i = tid; i < 256; i += LT_THREADS) {
            delta_s[i] = cal.log_delta[i];
            delta_s[256 + i] = cal.cos_delta[i];
        }
        cal.log_tab = log_tab_s;
        cal.log_delta = delta_s;
        cal.cos_delta = delta_s + 256;
    }
    const int32_t first_pair = first_thread / 2;
    const int32_t pair = first_pair + blockIdx.x;
    int64_t m_lo = (int64_t)pair * 2 - first_thread, m_hi = m_lo + 2;
    if (m_lo < 0) m_lo = 0;
    if (m_hi > n_pop) m_hi = n_pop;
    const int rows_per_step = (int)(m_hi - m_lo) * bm;
    const int row0 = blockIdx.y * ROWS_CTA;
    const int total_rows = min(ROWS_CTA, rows_per_step * t_steps - row0);
    if (total_rows <= 0) return;
    if (tid < ROWS_CTA) {
        int lr = row0 + (tid < total_rows ? tid : total_rows - 1);  // rows past the end repeat the last one
        int step = lr / rows_per_step, rr = lr - step * rows_per_step;
        row_s[tid] = ((int64_t)step * n_pop + m_lo) * bm + rr;
    }
    __syncthreads();

    // ---- phase 1: B of this pair ----
    float4* bsm4 = reinterpret_cast<float4*>(bsm);
    auto stored_row = [](int kr) { return (kr & ~127) + (kr & 3) * 32 + ((kr & 127) >> 2); };
    // several stacked parameters (n_groups > 1, cached factors only): group g's B block sits at
    // bsm + g * gstride floats and came from cache block (pair, g)
    const int gstride = ((k + 127) & ~127) * RANK;
    if (cache_b && rank_true < 4) {
        for (int grp = 0; grp < n_groups; ++grp) {
            const float* cb1 = cache_b + ((size_t)blockIdx.x * n_groups + grp) * k * rank_true;
            float4* dst = bsm4 + grp * (gstride / 4);
            for (int kr = tid; kr < k; kr += LT_THREADS) {
                const float* row = cb1 + (size_t)kr * rank_true;
                dst[stored_row(kr)] = make_float4(__ldg(row), rank_true > 1 ? __ldg(row + 1) : 0.0f,
                                                  rank_true > 2 ? __ldg(row + 2) : 0.0f, 0.0f);
            }
        }
    } else if (cache_b) {
        for (int grp = 0; grp < n_groups; ++grp) {
            const float4* cb4 = reinterpret_cast<const float4*>(cache_b + ((size_t)blockIdx.x * n_groups + grp) * k * RANK);
            float4* dst = bsm4 + grp * (gstride / 4);
            for (int i = tid; i < k * RANK_G; i += LT_THREADS) {
                const int kr = i / RANK_G, c = i - kr * RANK_G;
                const int p = stored_row(kr);
                dst[p * RANK_G + ((c + p / RP) % RANK_G)] = __ldg(cb4 + i);
            }
        }
    } else {
        const int rpt = (k + LT_THREADS - 1) / LT_THREADS;   // rows per thread
        const int kr0 = tid * rpt, kr1 = min(kr0 + rpt, k);
        if (kr0 < k) {
            uint64_t sb = noise_seed(key, true_epoch, pair) | 1ull;
            sb = jump_by(pow2, sb, 2ull * (uint64_t)rank_true * (uint64_t)(row_b0 + kr0));   // row_b0: first input-side row
#pragma unroll 1
            for (int kr = kr0; kr < kr1; ++kr) {
                const int p = stored_row(kr);
                if (rank_true < 4) {
                    float z[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    z[0] = next_normal(sb, cal);
                    if (rank_true > 1) z[1] = next_normal(sb, cal);
                    if (rank_true > 2) z[2] = next_normal(sb, cal);
                    bsm4[p] = make_float4(z[0], z[1], z[2], z[3]);
                    continue;
                }
#pragma unroll 1
                for (int c = 0; c < RANK_G; ++c) {
                    float z[4];
                    next_normals4(sb, cal, z);
                    bsm4[p * RANK_G + ((c + p / RP) % RANK_G)] = make_float4(z[0], z[1], z[2], z[3]);
                }
            }
        }
    }
    __syncthreads();

    // ---- phase 2: split and t of RPR rows per warp and round, NJ 16-byte pieces per lane and row ----
    const int n4 = k >> 2;
    uint32_t lo_nz = 0;  // any non-zero lo half written by this thread
    // HALF: rows of up to 64 values take half a warp each, so a warp works on 2 * RPR rows at a time
    constexpr int W = HALF ? 16 : 32;              // lanes per row
    constexpr int RSTEP = HALF ? 2 : 1;            // rows between a lane's consecutive rows
    const int li = lane & (W - 1), hs = HALF ? lane >> 4 : 0;
    auto finish_row = [&](int64_t R, float m, float& sc, bool valid) {
#pragma unroll
        for (int off = W / 2; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        int ex = (int)((__float_as_uint(m) >> 23) & 0xffu) - 127;
        int e = 13 - ex;
        if (ex <= -127 || ex >= 128) e = 0;
        if (e > 100) e = 100;
        if (e < -100) e = -100;
        if (bf16) e = 0;   // one-pass mode: no scale
        sc = __uint_as_float((uint32_t)(127 + e) << 23);
        if (li == 0 && valid) inv_scale[R] = __uint_as_float((uint32_t)(127 - e) << 23);
    };
    auto split4 = [&](float4 v, float sc, uint2& h2, uint2& l2) {
        if (bf16) {   // hi = bf16(v), the lo half is neither written nor read
            const __nv_bfloat162 b01 = __floats2bfloat162_rn(v.x, v.y), b23 = __floats2bfloat162_rn(v.z, v.w);
            h2 = make_uint2(*reinterpret_cast<const uint32_t*>(&b01), *reinterpret_cast<const uint32_t*>(&b23));
            l2 = make_uint2(0u, 0u);
            return;
        }
        const float x0 = v.x * sc, x1 = v.y * sc, x2 = v.z * sc, x3 = v.w * sc;
        const __half2 h01 = __floats2half2_rn(x0, x1), h23 = __floats2half2_rn(x2, x3);
        const float2 b01 = __half22float2(h01), b23 = __half22float2(h23);
        const __half2 l01 = __floats2half2_rn(x0 - b01.x, x1 - b01.y), l23 = __floats2half2_rn(x2 - b23.x, x3 - b23.y);
        h2 = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
        l2 = make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
        lo_nz |= (l2.x | l2.y) & 0x7fff7fffu;  // a lo half of -0 is still zero
    };
    constexpr int NW = LT_THREADS / 32;
    constexpr int RW = RPR * RSTEP;   // rows of a warp and round
    constexpr int N = RPR * RANK;     // sums of a lane group and round: N[row * RANK + q]
    const ulonglong2* bsm2 = reinterpret_cast<const ulonglong2*>(bsm);
    for (int lr0 = warp * RW; lr0 < total_rows; lr0 += NW * RW) {
        float4 v[RPR][NJ];   // streaming loads: x passes once and must not push the jump tables out of L1
#pragma unroll
        for (int r = 0; r < RPR; ++r) {
            const int lr = lr0 + r * RSTEP + hs;
            const bool valid = lr < total_rows;   // the same for all lanes of a row
            const float4* src = reinterpret_cast<const float4*>(x + (size_t)row_s[valid ? lr : lr0] * x_stride);
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int i = li + 32 * j;
                v[r][j] = apply_x_op((valid && i < n4) ? __ldcs(src + i) : make_float4(0.f, 0.f, 0.f, 0.f), x_op);
            }
        }
        if (!skip_split) {
            float sc[RPR];
#pragma unroll
            for (int r = 0; r < RPR; ++r) {
                const int lr = lr0 + r * RSTEP + hs;
                float m = 0.0f;
#pragma unroll
                for (int j = 0; j < NJ; ++j)
                    m = fmaxf(m, fmaxf(fmaxf(fabsf(v[r][j].x), fabsf(v[r][j].y)), fmaxf(fabsf(v[r][j].z), fabsf(v[r][j].w))));
                finish_row(row_s[lr < total_rows ? lr : lr0], m, sc[r], lr < total_rows);
            }
#pragma unroll
            for (int r = 0; r < RPR; ++r) {
                const int lr = lr0 + r * RSTEP + hs;
                if (lr < total_rows) {
                    const int64_t R = row_s[lr];
                    uint2* dh = reinterpret_cast<uint2*>(xhi + (size_t)R * k);
                    uint2* dl = reinterpret_cast<uint2*>(xlo + (size_t)R * k);
#pragma unroll
                    for (int j = 0; j < NJ; ++j) {
                        const int i = li + 32 * j;
                        if (i < n4) {
                            uint2 h2, l2;
                            split4(v[r][j], sc[r], h2, l2);
                            dh[i] = h2;
                            if (!bf16) dl[i] = l2;
                        }
                    }
                }
            }
        }
        for (int grp = 0; grp < n_groups; ++grp) {
            const ulonglong2* bg = bsm2 + grp * (gstride / 4);
            // t of the rows, two q per packed fp32 instruction: acc2[(row * RANK + q) / 2]
            f32x2 acc2[N / 2];
#pragma unroll
            for (int i = 0; i < N / 2; ++i) acc2[i] = 0ull;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                if (li + 32 * j < n4) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int p = j * 128 + e * 32 + li;
                        f32x2 xe[RPR];
#pragma unroll
                        for (int r = 0; r < RPR; ++r) {
                            const float xv = e == 0 ? v[r][j].x : e == 1 ? v[r][j].y : e == 2 ? v[r][j].z : v[r][j].w;
                            xe[r] = pk2(xv, xv);
                        }
#pragma unroll
                        for (int c = 0; c < RANK_G; ++c) {
                            const ulonglong2 b = bg[p * RANK_G + ((c + p / RP) % RANK_G)];
#pragma unroll
                            for (int r = 0; r < RPR; ++r) {
                                acc2[r * (RANK / 2) + 2 * c] = fma2(xe[r], b.x, acc2[r * (RANK / 2) + 2 * c]);
                                acc2[r * (RANK / 2) + 2 * c + 1] = fma2(xe[r], b.y, acc2[r * (RANK / 2) + 2 * c + 1]);
                            }
                        }
                    }
                }
            }
            float acc[N];
#pragma unroll
            for (int i = 0; i < N / 2; ++i) upk2(acc2[i], acc[2 * i], acc[2 * i + 1]);
            // halving exchange over the W lanes of a row group: in the step with distance off a lane keeps
            // the half of its values that its bit `off` selects, summed with its partner's.  After the
            // steps a lane holds N / W finished sums from index li * N / W on (N >= W), or groups of W / N
            // lanes hold the sum of index li / group (N < W: the last steps add single values).
            constexpr int STEPS = HALF ? 4 : 5;
#pragma unroll
            for (int s = 0; s < STEPS; ++s) {
                const int n = N >> s, off = (W / 2) >> s;
                if (n > 1) {
                    const bool up = (lane & off) != 0;
#pragma unroll
                    for (int i = 0; i < n / 2; ++i) {
                        const float send = up ? acc[i] : acc[i + n / 2];
                        const float keep = up ? acc[i + n / 2] : acc[i];
                        acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                    }
                } else {
                    acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], off);
                }
            }
            constexpr int NF = N >= W ? N / W : 1;      // finished sums per lane
            constexpr int GROUP = N >= W ? 1 : W / N;   // lanes holding the same sum
            if (li % GROUP == 0) {
                const int idx = (li / GROUP) * NF;      // NF consecutive q of one row
                const int row = idx / RANK, q = idx - row * RANK;
                const int lr = lr0 + row * RSTEP + hs;
                if (lr < total_rows) {
                    float* dst = t + ((size_t)row_s[lr] * n_groups + grp) * RANK + q;
                    if (NF == 1) dst[0] = acc[0];
                    else if (NF == 2) *reinterpret_cast<float2*>(dst) = make_float2(acc[0], acc[1]);
                    else *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[NF > 2 ? 2 : 0], acc[NF > 3 ? 3 : 0]);
                }
            }
        }
    }
    // one flag per call tells the GEMM whether any lo half is non-zero (a set flag is not set again)
    if (__any_sync(0xffffffffu, lo_nz != 0) && lane == 0 && *reinterpret_cast<volatile int*>(lo_flag) == 0)
        atomicOr(lo_flag, 1);
}

// The rows prepass for rows longer than a warp's registers (1024 < k, B of the pair within 64 KB: rank <= 4
// up to k = 4096, rank 8 up to 2048): the row passes through the registers 1024 values at a time, once for
// the maximum (not in the one-pass mode) and once for the split and t, whose sums stay in registers over
// the pieces.  The block kernel walks such a row four values per lane and trip.
template <int RANK_G>
__global__ void __launch_bounds__(LT_THREADS, 2)
lowrank_t_long_kernel(LibmCal cal, const uint64_t* __restrict__ pow2,
                      uint64_t key, int32_t true_epoch, int32_t first_thread, const float* __restrict__ x,
                      int64_t x_stride, int t_steps, int64_t n_pop, int bm, int k, float* __restrict__ t,
                      __half* __restrict__ xhi, __half* __restrict__ xlo, float* __restrict__ inv_scale,
                      const float* __restrict__ cache_b, int* __restrict__ lo_flag, int bf16, int rank_true,
                      int row_b0, int skip_split, int n_groups, int x_op) {
    constexpr int RANK = RANK_G * 4;
    constexpr int NJ = 8, RPR = 2;   // 1024 values of two rows in flight per warp
    constexpr bool HALF = false;
    constexpr int RP = 8 / RANK_G;    // rows of B per 128 bytes
    constexpr int ROWS_CTA = HALF ? 2 * LT_ROWS : LT_ROWS;   // x rows per CTA
    extern __shared__ __align__(16) float bsm[];   // ceil(k / 128) * 128 rows of RANK floats
    __shared__ double2 log_tab_s[64];
    __shared__ uint32_t delta_s[512];
    __shared__ int64_t row_s[ROWS_CTA];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (!cache_b) {
        for (int i = tid; i < 64; i += LT_THREADS) log_tab_s[i] = cal.log_tab[i];
        for (int i = tid; i < 256; i += LT_THREADS) {
            delta_s[i] = cal.log_delta[i];
            delta_s[256 + i] = cal.cos_delta[i];
        }
        cal.log_tab = log_tab_s;
        cal.log_delta = delta_s;
        cal.cos_delta = delta_s + 256;
    }
    const int32_t first_pair = first_thread / 2;
    const int32_t pair = first_pair + blockIdx.x;
    int64_t m_lo = (int64_t)pair * 2 - first_thread, m_hi = m_lo + 2;
    if (m_lo < 0) m_lo = 0;
    if (m_hi > n_pop) m_hi = n_pop;
    const int rows_per_step = (int)(m_hi - m_lo) * bm;
    const int row0 = blockIdx.y * ROWS_CTA;
    const int total_rows = min(ROWS_CTA, rows_per_step * t_steps - row0);
    if (total_rows <= 0) return;
    if (tid < ROWS_CTA) {
        int lr = row0 + (tid < total_rows ? tid : total_rows - 1);  // rows past the end repeat the last one
        int step = lr / rows_per_step, rr = lr - step * rows_per_step;
        row_s[tid] = ((int64_t)step * n_pop + m_lo) * bm + rr;
    }
    __syncthreads();

    // ---- phase 1: B of this pair ----
    float4* bsm4 = reinterpret_cast<float4*>(bsm);
    auto stored_row = [](int kr) { return (kr & ~127) + (kr & 3) * 32 + ((kr & 127) >> 2); };
    // several stacked parameters (n_groups > 1, cached factors only): group g's B block sits at
    // bsm + g * gstride floats and came from cache block (pair, g)
    const int gstride = ((k + 127) & ~127) * RANK;
    if (cache_b && rank_true < 4) {
        for (int grp = 0; grp < n_groups; ++grp) {
            const float* cb1 = cache_b + ((size_t)blockIdx.x * n_groups + grp) * k * rank_true;
            float4* dst = bsm4 + grp * (gstride / 4);
            for (int kr = tid; kr < k; kr += LT_THREADS) {
                const float* row = cb1 + (size_t)kr * rank_true;
                dst[stored_row(kr)] = make_float4(__ldg(row), rank_true > 1 ? __ldg(row + 1) : 0.0f,
                                                  rank_true > 2 ? __ldg(row + 2) : 0.0f, 0.0f);
            }
        }
    } else if (cache_b) {
        for (int grp = 0; grp < n_groups; ++grp) {
            const float4* cb4 = reinterpret_cast<const float4*>(cache_b + ((size_t)blockIdx.x * n_groups + grp) * k * RANK);
            float4* dst = bsm4 + grp * (gstride / 4);
            for (int i = tid; i < k * RANK_G; i += LT_THREADS) {
                const int kr = i / RANK_G, c = i - kr * RANK_G;
                const int p = stored_row(kr);
                dst[p * RANK_G + ((c + p / RP) % RANK_G)] = __ldg(cb4 + i);
            }
        }
    } else {
        const int rpt = (k + LT_THREADS - 1) / LT_THREADS;   // rows per thread
        const int kr0 = tid * rpt, kr1 = min(kr0 + rpt, k);
        if (kr0 < k) {
            uint64_t sb = noise_seed(key, true_epoch, pair) | 1ull;
            sb = jump_by(pow2, sb, 2ull * (uint64_t)rank_true * (uint64_t)(row_b0 + kr0));   // row_b0: first input-side row
#pragma unroll 1
            for (int kr = kr0; kr < kr1; ++kr) {
                const int p = stored_row(kr);
                if (rank_true < 4) {
                    float z[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    z[0] = next_normal(sb, cal);
                    if (rank_true > 1) z[1] = next_normal(sb, cal);
                    if (rank_true > 2) z[2] = next_normal(sb, cal);
                    bsm4[p] = make_float4(z[0], z[1], z[2], z[3]);
                    continue;
                }
#pragma unroll 1
                for (int c = 0; c < RANK_G; ++c) {
                    float z[4];
                    next_normals4(sb, cal, z);
                    bsm4[p * RANK_G + ((c + p / RP) % RANK_G)] = make_float4(z[0], z[1], z[2], z[3]);
                }
            }
        }
    }
    __syncthreads();

    // ---- phase 2: split and t of RPR rows per warp and round, NJ 16-byte pieces per lane and row ----
    const int n4 = k >> 2;
    uint32_t lo_nz = 0;  // any non-zero lo half written by this thread
    // HALF: rows of up to 64 values take half a warp each, so a warp works on 2 * RPR rows at a time
    constexpr int W = HALF ? 16 : 32;              // lanes per row
    constexpr int RSTEP = HALF ? 2 : 1;            // rows between a lane's consecutive rows
    const int li = lane & (W - 1), hs = HALF ? lane >> 4 : 0;
    auto finish_row = [&](int64_t R, float m, float& sc, bool valid) {
#pragma unroll
        for (int off = W / 2; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        int ex = (int)((__float_as_uint(m) >> 23) & 0xffu) - 127;
        int e = 13 - ex;
        if (ex <= -127 || ex >= 128) e = 0;
        if (e > 100) e = 100;
        if (e < -100) e = -100;
        if (bf16) e = 0;   // one-pass mode: no scale
        sc = __uint_as_float((uint32_t)(127 + e) << 23);
        if (li == 0 && valid) inv_scale[R] = __uint_as_float((uint32_t)(127 - e) << 23);
    };
    auto split4 = [&](float4 v, float sc, uint2& h2, uint2& l2) {
        if (bf16) {   // hi = bf16(v), the lo half is neither written nor read
            const __nv_bfloat162 b01 = __floats2bfloat162_rn(v.x, v.y), b23 = __floats2bfloat162_rn(v.z, v.w);
            h2 = make_uint2(*reinterpret_cast<const uint32_t*>(&b01), *reinterpret_cast<const uint32_t*>(&b23));
            l2 = make_uint2(0u, 0u);
            return;
        }
        const float x0 = v.x * sc, x1 = v.y * sc, x2 = v.z * sc, x3 = v.w * sc;
        const __half2 h01 = __floats2half2_rn(x0, x1), h23 = __floats2half2_rn(x2, x3);
        const float2 b01 = __half22float2(h01), b23 = __half22float2(h23);
        const __half2 l01 = __floats2half2_rn(x0 - b01.x, x1 - b01.y), l23 = __floats2half2_rn(x2 - b23.x, x3 - b23.y);
        h2 = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
        l2 = make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
        lo_nz |= (l2.x | l2.y) & 0x7fff7fffu;  // a lo half of -0 is still zero
    };
    constexpr int NW = LT_THREADS / 32;
    constexpr int RW = RPR * RSTEP;   // rows of a warp and round
    constexpr int N = RPR * RANK;     // sums of a lane group and round: N[row * RANK + q]
    const ulonglong2* bsm2 = reinterpret_cast<const ulonglong2*>(bsm);
    for (int lr0 = warp * RW; lr0 < total_rows; lr0 += NW * RW) {
        const float4* src[RPR];
        bool valid[RPR];
        int64_t R[RPR];
#pragma unroll
        for (int r = 0; r < RPR; ++r) {
            valid[r] = lr0 + r < total_rows;   // warp-uniform
            R[r] = row_s[valid[r] ? lr0 + r : lr0];
            src[r] = reinterpret_cast<const float4*>(x + (size_t)R[r] * x_stride);
        }
        // the scale of a row needs the maximum of the whole row: one pass of its own (the one-pass mode
        // scales nothing and skips it; the second read of the row then comes from L2)
        float sc[RPR];
#pragma unroll
        for (int r = 0; r < RPR; ++r) sc[r] = 1.0f;
        if (!skip_split) {
            float m[RPR];
#pragma unroll
            for (int r = 0; r < RPR; ++r) m[r] = 0.0f;
            if (!bf16) {
                for (int c4 = 0; c4 < n4; c4 += 32 * NJ) {
                    float4 v[RPR][NJ];
#pragma unroll
                    for (int r = 0; r < RPR; ++r)
#pragma unroll
                        for (int j = 0; j < NJ; ++j) {
                            const int i = c4 + lane + 32 * j;
                            v[r][j] = apply_x_op((valid[r] && i < n4) ? __ldg(src[r] + i) : make_float4(0.f, 0.f, 0.f, 0.f), x_op);
                        }
#pragma unroll
                    for (int r = 0; r < RPR; ++r)
#pragma unroll
                        for (int j = 0; j < NJ; ++j)
                            m[r] = fmaxf(m[r], fmaxf(fmaxf(fabsf(v[r][j].x), fabsf(v[r][j].y)),
                                                     fmaxf(fabsf(v[r][j].z), fabsf(v[r][j].w))));
                }
            }
#pragma unroll
            for (int r = 0; r < RPR; ++r) finish_row(R[r], m[r], sc[r], valid[r]);
        }
        f32x2 acc2[N / 2];
#pragma unroll
        for (int i = 0; i < N / 2; ++i) acc2[i] = 0ull;
        for (int c4 = 0; c4 < n4; c4 += 32 * NJ) {
            float4 v[RPR][NJ];
#pragma unroll
            for (int r = 0; r < RPR; ++r)
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const int i = c4 + lane + 32 * j;
                    v[r][j] = apply_x_op((valid[r] && i < n4) ? __ldcs(src[r] + i) : make_float4(0.f, 0.f, 0.f, 0.f), x_op);
                }
            if (!skip_split) {
#pragma unroll
                for (int r = 0; r < RPR; ++r) {
                    if (valid[r]) {
                        uint2* dh = reinterpret_cast<uint2*>(xhi + (size_t)R[r] * k);
                        uint2* dl = reinterpret_cast<uint2*>(xlo + (size_t)R[r] * k);
#pragma unroll
                        for (int j = 0; j < NJ; ++j) {
                            const int i = c4 + lane + 32 * j;
                            if (i < n4) {
                                uint2 h2, l2;
                                split4(v[r][j], sc[r], h2, l2);
                                dh[i] = h2;
                                if (!bf16) dl[i] = l2;
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                if (c4 + lane + 32 * j < n4) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int p = 4 * c4 + j * 128 + e * 32 + lane;   // stored row of B row 4 * piece + e
                        f32x2 xe[RPR];
#pragma unroll
                        for (int r = 0; r < RPR; ++r) {
                            const float xv = e == 0 ? v[r][j].x : e == 1 ? v[r][j].y : e == 2 ? v[r][j].z : v[r][j].w;
                            xe[r] = pk2(xv, xv);
                        }
#pragma unroll
                        for (int c = 0; c < RANK_G; ++c) {
                            const ulonglong2 b = bsm2[p * RANK_G + ((c + p / RP) % RANK_G)];
#pragma unroll
                            for (int r = 0; r < RPR; ++r) {
                                acc2[r * (RANK / 2) + 2 * c] = fma2(xe[r], b.x, acc2[r * (RANK / 2) + 2 * c]);
                                acc2[r * (RANK / 2) + 2 * c + 1] = fma2(xe[r], b.y, acc2[r * (RANK / 2) + 2 * c + 1]);
                            }
                        }
                    }
                }
            }
        }
        float acc[N];
#pragma unroll
        for (int i = 0; i < N / 2; ++i) upk2(acc2[i], acc[2 * i], acc[2 * i + 1]);
        // halving exchange, see lowrank_t_rows_kernel
#pragma unroll
        for (int s = 0; s < 5; ++s) {
            const int n = N >> s, off = 16 >> s;
            if (n > 1) {
                const bool up = (lane & off) != 0;
#pragma unroll
                for (int i = 0; i < n / 2; ++i) {
                    const float send = up ? acc[i] : acc[i + n / 2];
                    const float keep = up ? acc[i + n / 2] : acc[i];
                    acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            } else {
                acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], off);
            }
        }
        constexpr int NF = N >= 32 ? N / 32 : 1;
        constexpr int GROUP = N >= 32 ? 1 : 32 / N;
        if (lane % GROUP == 0) {
            const int idx = (lane / GROUP) * NF;
            const int row = idx / RANK, q = idx - row * RANK;
            if (lr0 + row < total_rows) t[(size_t)row_s[lr0 + row] * RANK + q] = acc[0];
        }
    }
    // one flag per call tells the GEMM whether any lo half is non-zero (a set flag is not set again)
    if (__any_sync(0xffffffffu, lo_nz != 0) && lane == 0 && *reinterpret_cast<volatile int*>(lo_flag) == 0)
        atomicOr(lo_flag, 1);
}

// ------------------------------------------------------------------- host side
// 2-D fp16 map over (rows, cols) with `stride` elements between rows; box = (64, box_rows).
int make_map(CUtensorMap* map, const __half* base, int64_t rows, int cols, int64_t stride, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return HSES_ERR_CUDA;
    }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)stride * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
        return HSES_ERR_CUDA;
    }
    return HSES_OK;
}

struct TcScratch {
    __half *xhi, *xlo, *whi, *wlo;
    float *rs, *cs, *t;
    int* lo_flag;  // set by the x split when a lo half is non-zero
    size_t bytes;
};
// shared memory of one group's B in lowrank_t_rows_kernel: whole 128-row groups of the padded rank
static size_t rows_prepass_b_bytes(int k, int rank) {
    return (size_t)((k + 127) / 128) * 128 * (rank < 4 ? 4 : rank) * sizeof(float);
}

TcScratch tc_scratch(const hses_linear_args& g, void* base) {
    auto up = [](size_t v) { return (v + 63) / 64 * 64; };
    size_t rows = (size_t)g.t_steps * g.n_pop * g.bm;
    size_t nw = up((size_t)g.a * g.k), nx = up(rows * g.k);   // fp16 elements
    size_t nt = g.perturb ? up(rows * (size_t)((g.rank + 3) / 4 * 4) * (size_t)(g.n_groups > 1 ? g.n_groups : 1)) : 0;   // floats: t has the padded rank, once per group
    TcScratch s;
    s.xhi = reinterpret_cast<__half*>(base);
    s.xlo = s.xhi + nx;
    s.whi = s.xlo + nx;
    s.wlo = s.whi + nw;
    s.rs = reinterpret_cast<float*>(s.wlo + nw);
    s.cs = s.rs + up(rows);
    s.t = s.cs + up((size_t)g.a);
    s.lo_flag = reinterpret_cast<int*>(s.t + nt);
    s.bytes = (2 * nx + 2 * nw) * sizeof(__half) + (up(rows) + up((size_t)g.a) + nt + 64) * sizeof(float);
    return s;
}

template <int BN, int RG, bool R1 = false, bool GRP = false>
int launch_tc_rg(hses_ctx* ctx, cudaStream_t st, const CUtensorMap& tm_x, const CUtensorMap& tm_xlo,
                 const CUtensorMap& tm_whi, const CUtensorMap& tm_wlo, const TcArgs& ta, int grid,
                 int smem_bytes) {
    HSES_CUDA(cudaFuncSetAttribute(linear_tc_kernel<BN, RG, R1, GRP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   smem_bytes));
    HSES_KERNEL(ctx, st, "linear_tc");
    linear_tc_kernel<BN, RG, R1, GRP><<<grid, NTHREADS, smem_bytes, st>>>(tm_x, tm_xlo, tm_whi, tm_wlo, ta);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

template <int BN>
int launch_tc(hses_ctx* ctx, cudaStream_t st, const hses_linear_args& g, const TcScratch& sc, TcArgs ta) {
    // Generator warps per quadrant and ring slots: the deepest ring that fits in shared memory under
    // the rule stated at TcArgs (depth a multiple of the generator count, and even for 16-column
    // items).  More slots than generators matter more than a fourth generator: a generator needs a
    // free slot to write while the epilogue still reads its previous item.
    ta.gens = 0;
    ta.ring_depth = 0;
    if (g.perturb) {
        const int choices[][2] = {{4, 8}, {3, 6}, {4, 4}, {2, 4}, {2, 2}, {1, 2}};   // (gens, depth), best first
        for (auto& ch : choices) {
            if (TcSmem<BN>::FIXED + TcSmem<BN>::a_bytes(ch[1], ta.rank) <= TcSmem<BN>::LIMIT) {
                ta.gens = ch[0];
                ta.ring_depth = ch[1];
                break;
            }
        }
        HSES_REQUIRE(ta.gens > 0, "linear_tc: the ring of staged factor rows does not fit in shared memory");
        const uint64_t* hop = nullptr;
        // from the end of a lane's share of one item to the start of its share of the warp's next item
        const uint64_t per_lane = ta.rank_true < 4 ? (uint64_t)ta.rank_true : (uint64_t)item_normals_per_lane(ta.rank);
        int hrc = get_hop_table(ctx, 2ull * ((uint64_t)ta.rank_true * item_rows(ta.rank) * ta.gens - per_lane), &hop);
        if (hrc != HSES_OK) return hrc;
        ta.hop = hop;
    }
    CUtensorMap tm_x, tm_xlo, tm_whi, tm_wlo;
    int64_t rows = ta.rows;
    int rc = make_map(&tm_x, sc.xhi, rows, g.k, g.k, BM_TILE);
    if (rc == HSES_OK) rc = make_map(&tm_xlo, sc.xlo, rows, g.k, g.k, BM_TILE);
    if (rc == HSES_OK) rc = make_map(&tm_whi, sc.whi, g.a, g.k, g.k, BN);
    if (rc == HSES_OK) rc = make_map(&tm_wlo, sc.wlo, g.a, g.k, g.k, BN);
    if (rc != HSES_OK) return rc;
    using S = TcSmem<BN>;
    ta.n_stages = ta.one_pass ? S::MAX_STAGES : S::STAGES;
    ta.stage_bytes = ta.one_pass ? S::X_BYTES + S::W_BYTES : S::STAGE_BYTES;
    int smem_bytes = S::FIXED + (g.perturb ? S::a_bytes(ta.ring_depth, ta.rank) : 0);
    HSES_REQUIRE(smem_bytes <= S::LIMIT, "shared memory budget exceeded");
    int m_tiles = (int)(rows / BM_TILE);
    int grid = m_tiles < ctx->sm_count ? m_tiles : ctx->sm_count;
    if (ta.group_cols) {   // stacked parameters: ranks 1..4, 8, 16 (tensor_path_supports)
        switch (ta.rank / 4) {
            case 1:
                if (ta.rank_true == 1) return launch_tc_rg<BN, 1, true, true>(ctx, st, tm_x, tm_xlo, tm_whi, tm_wlo, ta, grid, smem_bytes);
                return launch_tc_rg<BN, 1, false, true>(ctx, st, tm_x, tm_xlo, tm_whi, tm_wlo, ta, grid, smem_bytes);
            case 2: return launch_tc_rg<BN, 2, false, true>(ctx, st, tm_x, tm_xlo, tm_whi, tm_wlo, ta, grid, smem_bytes);
            case 4: return launch_tc_rg<BN, 4, false, true>(ctx, st, tm_x, tm_xlo, tm_whi, tm_wlo, ta, grid, smem_bytes);
        }
    }
    switch (ta.rank / 4) {
        case 0: return launch_tc_rg<BN, 0>(ctx, st, tm_x, tm_xlo, tm_whi, tm_wlo, ta, grid, smem_bytes);
        case 1:
            if (ta.rank_true == 1) return launch_tc_rg<BN, 1, true>(ctx, st, tm_x, tm_xlo, tm_whi, tm_wlo, ta, grid, smem_bytes);
            return launch_tc_rg<BN, 1>(ctx, st, tm_x, tm_xlo, tm_whi, tm_wlo, ta, grid, smem_bytes);
        case 2: return launch_tc_rg<BN, 2>(ctx, st, tm_x, tm_xlo, tm_whi, tm_wlo, ta, grid, smem_bytes);
        case 4: return launch_tc_rg<BN, 4>(ctx, st, tm_x, tm_xlo, tm_whi, tm_wlo, ta, grid, smem_bytes);
        case 8: return launch_tc_rg<BN, 8>(ctx, st, tm_x, tm_xlo, tm_whi, tm_wlo, ta, grid, smem_bytes);
    }
    set_error("linear_tc: unsupported rank");
    return HSES_ERR_UNSUPPORTED;
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

}  // namespace

bool tensor_path_supports(const hses_linear_args& g) {
    int64_t rows = (int64_t)g.t_steps * g.n_pop * g.bm;
    if (rows % BM_TILE != 0 || g.k % 8 != 0) return false;
    // Output columns come in 16-column pieces per epilogue warp and 16- or 32-column ring items; a
    // ragged last chunk is fine as long as every ring slot keeps one reader: whole 32-column blocks,
    // or a single 16-column item per tile
    if (g.a % 32 != 0 && !(g.a == 16 && (!g.perturb || g.rank >= 8))) return false;
    if (g.x_row_stride % 4 != 0 || g.out_row_stride % 4 != 0 || g.param_row_stride % 4 != 0) return false;
    if (!aligned16(g.x) || !aligned16(g.param) || !aligned16(g.out) || (g.potentials && !aligned16(g.potentials))) return false;
    if (g.k > (1 << 20) || g.a > (1 << 20)) return false;
    if (g.perturb) {
        if (g.rank != 1 && g.rank != 2 && g.rank != 3 && g.rank != 4 && g.rank != 8 && g.rank != 16 && g.rank != 32)
            return false;
        // every 32-row slice of a tile must belong to one antithetic pair
        bool pair_rows = (g.bm % 32 == 0) || (g.bm == 16 && g.first_thread % 2 == 0 && g.n_pop % 2 == 0);
        if (!pair_rows) return false;
    }
    if (g.x_op != HSES_X_NONE) {
        // the prepasses that hold x in registers apply it there; nothing else does
        if (!g.perturb || g.lif == 2 || g.x_half != nullptr || g.x_split_valid) return false;
        const bool rows_ok = (g.rank <= 4 || g.rank == 8 || g.rank == 16) && g.k <= 1024;
        const bool long_ok = (g.rank <= 4 || g.rank == 8) && g.k > 1024 && rows_prepass_b_bytes(g.k, g.rank) <= 65536;
        if (!rows_ok && !long_ok) return false;
    }
    if (g.n_groups > 1) {
        // stacked parameters: cached factors, the rows prepass with all groups' B in shared memory, and
        // groups that are whole ring items
        if (!g.perturb || g.cache == nullptr || g.factor_order != 0 || g.a % g.n_groups != 0) return false;
        if (!(g.rank <= 4 || g.rank == 8 || g.rank == 16) || g.k > 1024) return false;
        const int gc = g.a / g.n_groups;
        if (gc % 32 != 0 && !(gc % 16 == 0 && g.rank >= 8)) return false;
        if ((size_t)g.n_groups * rows_prepass_b_bytes(g.k, g.rank) > 65536) return false;
    }
    return true;
}

size_t tensor_path_workspace_bytes(const hses_linear_args& g) { return tc_scratch(g, nullptr).bytes; }

int run_tensor_path(hses_ctx* ctx, cudaStream_t st, const hses_linear_args& g) {
    TcScratch sc = tc_scratch(g, g.workspace);
    HSES_REQUIRE(g.workspace != nullptr && g.workspace_bytes >= sc.bytes && aligned16(g.workspace),
                 "workspace too small or misaligned; see hses_perturbed_linear_workspace_bytes");
    int64_t rows = (int64_t)g.t_steps * g.n_pop * g.bm;
    const int one_pass = g.precision == HSES_PRECISION_BF16 ? 1 : 0;
    const bool reuse_split = g.x_split_valid != 0;   // x's operand split of the previous call is still in the workspace
    if (!reuse_split) HSES_CUDA(cudaMemsetAsync(sc.lo_flag, 0, sizeof(int), st));
    {
        HSES_KERNEL(ctx, st, "split_w");
        split_f16_rows_kernel<<<(unsigned)((g.a + 7) / 8), 256, 0, st>>>(g.param, g.a, g.k, g.param_row_stride,
                                                                        sc.whi, sc.wlo, sc.cs, nullptr, one_pass);
        HSES_LAUNCH_CHECK();
    }
    // a caller-provided fp16 copy of an x that is exact in fp16 is the operand as it stands
    const bool x_ready = !g.perturb && !one_pass && g.x_half != nullptr && aligned16(g.x_half);
    if (x_ready) sc.xhi = reinterpret_cast<__half*>(const_cast<void*>(g.x_half));
    if (!g.perturb && !x_ready && !reuse_split) {  // with noise the pair kernel below splits x while it computes t
        HSES_KERNEL(ctx, st, "split_x");
        split_f16_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(g.x, rows, g.k, g.x_row_stride, sc.xhi,
                                                                         sc.xlo, sc.rs, sc.lo_flag, one_pass);
        HSES_LAUNCH_CHECK();
    }
    TcArgs ta{};
    ta.rows = rows;
    ta.k = g.k;
    ta.a = g.a;
    ta.bm = g.bm;
    ta.n_pop = g.n_pop;
    ta.perturb = g.perturb;
    ta.lif = g.lif;
    ta.rank = g.perturb ? (g.rank + 3) / 4 * 4 : 0;
    ta.rank_true = g.perturb ? g.rank : 0;
    ta.one_pass = one_pass;
    ta.row_a0 = g.factor_order == 1 ? 0 : g.k;
    ta.key = g.key;
    ta.true_epoch = true_epoch_of(g.epoch, g.noise_reuse);
    ta.first_thread = g.first_thread;
    ta.base_sigma = g.perturb ? g.sigma / sqrtf((float)g.rank) : 0.0f;
    ta.leak = g.lif ? 1.0f / g.tau_m : 0.0f;
    ta.v_th = g.v_th;
    ta.out_scale = g.out_scale;
    ta.out_scale_ptr = g.out_scale_ptr;
    ta.t = sc.t;
    ta.t_stride = ta.rank * (g.n_groups > 1 ? g.n_groups : 1);
    ta.group_cols = g.n_groups > 1 ? g.a / g.n_groups : 0;
    ta.row_scale = x_ready ? nullptr : sc.rs;   // NULL: no row was scaled
    ta.col_scale = sc.cs;
    ta.out = g.out;
    ta.out_stride = g.out_row_stride;
    ta.pot = g.lif ? g.potentials : nullptr;
    ta.pow2 = ctx->t.jump_pow2;
    ta.cal = ctx->cal();
    ta.status = ctx->t.status_word;
    ta.hop = nullptr;
    const float *cache_a = nullptr, *cache_b = nullptr;
    if (g.perturb && g.cache) {
        int crc = resolve_factor_cache(g, &cache_a, &cache_b);
        if (crc != HSES_OK) return crc;
    }
    ta.cache_a = cache_a;
    ta.x_lo_flag = sc.lo_flag;
    if (g.perturb) {
        const uint64_t* hop127 = nullptr;
        int rc = get_hop_table(ctx, 2ull * g.rank * (LT_KB - 1), &hop127);   // rank values per row in the stream
        if (rc != HSES_OK) return rc;
        int64_t pairs = (g.first_thread + g.n_pop - 1) / 2 - g.first_thread / 2 + 1;
        HSES_KERNEL(ctx, st, "lowrank_t");
#define HSES_LT(RG)                                                                                          \
    lowrank_t_kernel<RG><<<lt_grid, LT_THREADS, 0, st>>>(                                            \
        ctx->cal(), ctx->t.jump_pow2, hop127, g.key, ta.true_epoch, g.first_thread, g.x, g.x_row_stride,     \
        g.t_steps, g.n_pop, g.bm, g.k, sc.t, sc.xhi, sc.xlo, sc.rs, cache_b, sc.lo_flag, one_pass, g.rank, g.factor_order == 1 ? g.a : 0, \
        reuse_split ? 1 : 0)
        dim3 lt_grid((unsigned)pairs, (unsigned)((2 * (int64_t)g.bm * g.t_steps + LT_ROWS - 1) / LT_ROWS));
        if ((g.rank <= 4 || g.rank == 8 || g.rank == 16) && g.k <= 1024) {
            // whole B of a pair in shared memory, x rows read once (see lowrank_t_rows_kernel)
            const int groups = g.n_groups > 1 ? g.n_groups : 1;
            const size_t b_bytes = groups * rows_prepass_b_bytes(g.k, g.rank);   // at most 64 KB
#define HSES_LTR(RG, NJ, RPR, HALF)                                                                               \
    do {                                                                                                      \
        HSES_CUDA(cudaFuncSetAttribute(lowrank_t_rows_kernel<RG, NJ, RPR, HALF>,                              \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));                  \
        lowrank_t_rows_kernel<RG, NJ, RPR, HALF><<<HALF ? lt_grid2 : lt_grid, LT_THREADS, b_bytes, st>>>(     \
            ctx->cal(), ctx->t.jump_pow2, g.key, ta.true_epoch, g.first_thread, g.x, g.x_row_stride,          \
            g.t_steps, g.n_pop, g.bm, g.k, sc.t, sc.xhi, sc.xlo, sc.rs, cache_b, sc.lo_flag, one_pass, g.rank, \
            g.factor_order == 1 ? g.a : 0, reuse_split ? 1 : 0, groups, g.x_op);                                      \
    } while (0)
            // rows in flight per warp: as many as the registers hold (16 pieces, 64 sums); rows of up to 64
            // values take half a warp each, and a CTA twice the rows
            dim3 lt_grid2(lt_grid.x, (lt_grid.y + 1) / 2);
#define HSES_LTR_K(RG, RPR1, RPR2)                                                                            \
    do {                                                                                                      \
        if (g.k <= 64) HSES_LTR(RG, 1, RPR1, true);                                                           \
        else if (g.k <= 128) HSES_LTR(RG, 1, RPR1, false);                                                    \
        else if (g.k <= 256) HSES_LTR(RG, 2, RPR2, false);                                                    \
        else HSES_LTR(RG, 8, 2, false);                                                                       \
    } while (0)
            switch ((g.rank + 3) / 4) {
                case 1: HSES_LTR_K(1, 8, 4); break;
                case 2: HSES_LTR_K(2, 8, 4); break;
                default: HSES_LTR_K(4, 4, 2); break;
            }
#undef HSES_LTR_K
#undef HSES_LTR
        } else if ((g.rank <= 4 || g.rank == 8) && g.k > 1024 && rows_prepass_b_bytes(g.k, g.rank) <= 65536) {
            // long rows with B still within shared memory (see lowrank_t_long_kernel)
            const size_t b_bytes = rows_prepass_b_bytes(g.k, g.rank);
#define HSES_LTL(RG)                                                                                          \
    do {                                                                                                      \
        HSES_CUDA(cudaFuncSetAttribute(lowrank_t_long_kernel<RG>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                       65536));                                                               \
        lowrank_t_long_kernel<RG><<<lt_grid, LT_THREADS, b_bytes, st>>>(                                      \
            ctx->cal(), ctx->t.jump_pow2, g.key, ta.true_epoch, g.first_thread, g.x, g.x_row_stride,          \
            g.t_steps, g.n_pop, g.bm, g.k, sc.t, sc.xhi, sc.xlo, sc.rs, cache_b, sc.lo_flag, one_pass, g.rank, \
            g.factor_order == 1 ? g.a : 0, reuse_split ? 1 : 0, 1, g.x_op);                                           \
    } while (0)
            if (g.rank <= 4) HSES_LTL(1);
            else HSES_LTL(2);
#undef HSES_LTL
        } else
        switch ((g.rank + 3) / 4) {
            case 1: HSES_LT(1); break;
            case 2: HSES_LT(2); break;
            case 4: HSES_LT(4); break;
            default: HSES_LT(8); break;
        }
#undef HSES_LT
        HSES_LAUNCH_CHECK();
    }
    if (g.a % 256 == 0) return launch_tc<256>(ctx, st, g, sc, ta);
    return launch_tc<128>(ctx, st, g, sc, ta);
}

}  // namespace hses
