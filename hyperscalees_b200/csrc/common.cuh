// Shared declarations of the library's translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <string>
#include <vector>

#include "../../include/hses.h"
#include "rng.cuh"

namespace hses {

void set_error(const std::string& msg);

struct DeviceTables {
    // libm calibration
    double2* log_tab = nullptr;
    uint32_t* log_flip = nullptr;
    uint32_t* cos_flip = nullptr;
    uint32_t* log_delta = nullptr;
    uint32_t* cos_delta = nullptr;
    float log_of_zero = 0.0f;
    uint64_t n_log_flips = 0, n_cos_flips = 0;
    // generator jump tables: entry k advances the state by 2^k steps
    uint64_t* jump_pow2 = nullptr;  // kJumpLevels matrices
    // one int per device: kernels with bounded waits record here why they gave up
    int* status_word = nullptr;
};

// Nibble table (kJumpWords uint64) that advances the generator by `distance`
// steps, built on first use and cached per device.
int get_hop_table(hses_ctx* ctx, uint64_t distance, const uint64_t** dev_tab);

constexpr int kJumpLevels = 48;

// Multiprocessor count the split-K planners size their grids for: that of the current CUDA
// device, read once (the *_workspace_bytes entry points have no context to ask).  Every device
// this library accepts is an sm_100 part, so a process sees one value.
int plan_sm_count();

// Per-context launch counters and optional CUDA-event timing of every kernel
// the library launches (hses_profile_* in the C ABI).
struct KernelStat {
    const char* name = nullptr;
    int64_t launches = 0;
    double ms = 0.0;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending;
};
struct Profiler {
    bool timing = false;
    std::vector<KernelStat> stats;
    std::vector<cudaEvent_t> pool;
    KernelStat& get(const char* name);
    cudaEvent_t event();
};
struct KernelScope {
    Profiler* prof;
    KernelStat* stat;
    cudaStream_t stream;
    cudaEvent_t start = nullptr;
    KernelScope(Profiler& p, cudaStream_t s, const char* name) : prof(&p), stat(&p.get(name)), stream(s) {
        stat->launches++;
        if (p.timing) {
            start = p.event();
            cudaEventRecord(start, s);
        }
    }
    ~KernelScope() {
        if (start) {
            cudaEvent_t stop = prof->event();
            cudaEventRecord(stop, stream);
            stat->pending.emplace_back(start, stop);
        }
    }
};

}  // namespace hses

struct hses_ctx {
    int device = 0;
    int sm_count = 0;
    hses::DeviceTables t;
    hses::Profiler prof;
    hses::LibmCal cal() const {
        hses::LibmCal c;
        c.log_tab = t.log_tab;
        c.log_flip = t.log_flip;
        c.cos_flip = t.cos_flip;
        c.log_delta = t.log_delta;
        c.cos_delta = t.cos_delta;
        c.log_of_zero = t.log_of_zero;
        return c;
    }
};

#define HSES_CUDA(call)                                                                   \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess) {                                                          \
            hses::set_error(std::string(#call) + " failed: " + cudaGetErrorString(e_));   \
            return HSES_ERR_CUDA;                                                         \
        }                                                                                 \
    } while (0)

#define HSES_REQUIRE(cond, msg)                                   \
    do {                                                          \
        if (!(cond)) {                                            \
            hses::set_error(std::string(__func__) + ": " + (msg)); \
            return HSES_ERR_INVALID;                              \
        }                                                         \
    } while (0)

// Counts (and, when profiling is on, times) the kernel launched right after it.
#define HSES_KERNEL(ctx, stream, name) hses::KernelScope hses_kernel_scope_((ctx)->prof, (stream), (name))

#define HSES_LAUNCH_CHECK()                                                                 \
    do {                                                                                    \
        cudaError_t e_ = cudaGetLastError();                                                \
        if (e_ != cudaSuccess) {                                                            \
            hses::set_error(std::string(__func__) + ": launch failed: " + cudaGetErrorString(e_)); \
            return HSES_ERR_CUDA;                                                           \
        }                                                                                   \
    } while (0)

namespace hses {
// Raw factors of `pairs` antithetic pairs starting at first_pair:
// A (pairs, a, r) and B (pairs, b, r), row-major.  When pair_weight is given
// (device, 2 floats per pair: the fitnesses of the even and the odd member),
// A is multiplied by (f_even - f_odd).  With no_alloc the launch uses no table that
// would have to be allocated on first use (slower row-to-row advance, same values).
int launch_pair_factors(hses_ctx* ctx, cudaStream_t stream, uint64_t key, int32_t true_epoch,
                        int32_t first_pair, int64_t pairs, int rank, int a, int b,
                        const float* pair_weight, float* A, float* B, bool no_alloc = false);
// One solver step (hses_solver_step's arithmetic) over several tensors in one launch; gradients
// back to back in `grads`, tensors with a NULL parameter skipped.
int solver_step_multi(hses_ctx* ctx, cudaStream_t st, const hses_solver* solver, int32_t step, int n_tensors,
                      float* const* params, float* const* m_bufs, float* const* v_bufs, const int64_t* lens,
                      const float* grads);
// lif_step (hyperscalees-models/src/snn.rs:53-65): charge, threshold, reset; returns the spike
__device__ __forceinline__ float lif_update(float& v, float cur, float leak, float v_th, int reset) {
    float d = __fadd_rn(-v, cur);
    float m = __fmul_rn(d, leak);
    float c = __fadd_rn(v, m);
    float s = c >= v_th ? 1.0f : 0.0f;
    v = reset == HSES_RESET_HARD ? __fmul_rn(c, __fadd_rn(-s, 1.0f)) : __fsub_rn(c, __fmul_rn(s, v_th));
    return s;
}


}  // namespace hses

static inline cudaStream_t as_stream(hses_stream s) { return reinterpret_cast<cudaStream_t>(s); }
