// Host side of the libm calibration: builds the fp64 helper table for the
// log candidate and turns (candidate, host libm) pairs into flip bitmaps and
// per-region filter thresholds.  See rng.cuh for the scheme.
#pragma once

#include <math.h>
#include <stdint.h>
#include <string.h>

#include <string>
#include <thread>
#include <vector>

namespace hses {

constexpr uint32_t kUnits = 1u << 24;

// 64 x {1/c, log c}; c is the centre of each sub-interval of [0.75, 1.5)
// except the two that touch 1.0, where c = 1 (log c = 0, z*1 - 1 exact).
inline void build_log_table(double* tab /* 128 doubles */) {
    for (int j = 0; j < 64; ++j) {
        double c;
        if (j == 31 || j == 32) c = 1.0;
        else if (j < 32) c = 0.75 + (j + 0.5) / 128.0;
        else c = 1.0 + (j - 32 + 0.5) / 64.0;
        tab[2 * j] = 1.0 / c;
        tab[2 * j + 1] = (c == 1.0) ? 0.0 : log(c);
    }
}

struct CalibResult {
    std::vector<uint32_t> flip;   // 2^24 bits
    uint32_t delta[256];
    uint64_t n_flips = 0;
    uint32_t max_dist = 0;        // largest distance-from-midpoint among flipped inputs
    std::string error;            // non-empty when a candidate is not a neighbour of libm
};

// bits[i] is the rounded candidate and code[i] = dist | (rounded_up << 31) as
// produced by round_candidate(); want(i) is the host libm value for input i.
// `first` skips inputs the device handles separately (i = 0 for the logarithm).
template <class Want>
inline void calibrate(const uint32_t* cand_bits, const uint32_t* cand_code, uint32_t first,
                      Want want, CalibResult& out) {
    out.flip.assign(kUnits / 32, 0u);
    for (int r = 0; r < 256; ++r) out.delta[r] = 0;
    unsigned nt = std::thread::hardware_concurrency();
    if (nt == 0) nt = 1;
    if (nt > 16) nt = 16;
    // regions (top byte of the input) are split across threads: every thread
    // owns whole 32-bit words of the bitmap and whole entries of delta.
    std::vector<std::thread> pool;
    std::vector<uint64_t> flips(nt, 0);
    std::vector<uint32_t> maxd(nt, 0);
    std::vector<std::string> errs(nt);
    for (unsigned t = 0; t < nt; ++t) {
        pool.emplace_back([&, t]() {
            for (uint32_t region = t; region < 256; region += nt) {
                uint32_t d = 0;
                for (uint32_t i = region << 16; i < ((region + 1) << 16); ++i) {
                    if (i < first) continue;
                    float w = want(i);
                    uint32_t wb;
                    memcpy(&wb, &w, 4);
                    if (wb == cand_bits[i]) continue;
                    uint32_t alt = (cand_code[i] >> 31) ? cand_bits[i] - 1u : cand_bits[i] + 1u;
                    uint32_t dist = cand_code[i] & 0x7fffffffu;
                    if (wb != alt) {
                        if (errs[t].empty())
                            errs[t] = "libm calibration: candidate for input " + std::to_string(i) +
                                      " is not adjacent to the host libm value";
                        continue;
                    }
                    out.flip[i >> 5] |= 1u << (i & 31u);
                    ++flips[t];
                    if (dist + 1 > d) d = dist + 1;
                }
                out.delta[region] = d;
                if (d > maxd[t]) maxd[t] = d;
            }
        });
    }
    for (auto& th : pool) th.join();
    for (unsigned t = 0; t < nt; ++t) {
        out.n_flips += flips[t];
        if (maxd[t] > out.max_dist) out.max_dist = maxd[t];
        if (out.error.empty() && !errs[t].empty()) out.error = errs[t];
    }
}

// The two libm expressions the reference evaluates (noiser.rs:470-476).
inline float host_logf_u24(uint32_t i) {
    float u = (float)i / 16777216.0f;
    return logf(fmaxf(u, 1e-9f));
}
inline float host_cosf_u24(uint32_t j) {
    float u = (float)j / 16777216.0f;
    return cosf(6.2831855f * u);
}

}  // namespace hses
