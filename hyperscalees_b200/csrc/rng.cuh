// Counter-style device RNG for the EggRoll noise factors.
//
// The reference draws every factor from a sequential xorshift64 stream
// (hyperscalees-noiser/src/noiser.rs:436-490) seeded by a 64-bit hash of
// (parameter key, epoch bucket, antithetic pair) (noiser.rs:495-506).  Here a
// thread lands anywhere in that stream with a GF(2) jump (the generator is a
// linear map on 64-bit states) and then regenerates normals in registers.
//
// The Box-Muller step calls the platform libm in the reference (Rust
// f32::ln / f32::cos lower to logf / cosf).  Those are not correctly rounded,
// so bit-exactness is obtained in two stages:
//   1. a deterministic fp64 "candidate" for logf(u) and cosf(TAU*u), built
//      from IEEE basic operations only (explicit fma/mul/add, no contraction),
//      rounded to fp32;
//   2. a per-context calibration that compares the candidate with the host
//      libm over all 2^24 possible uniforms and records, one bit per input,
//      where libm rounds to the other neighbour.  A cheap distance-to-midpoint
//      test on the low 29 bits of the fp64 value filters out the ~90 % of
//      inputs that cannot be affected before the bitmap is consulted.
// The functions below compile for host and device so the candidate math can
// be exercised on the CPU as well.
#pragma once

#include <stdint.h>
#include <string.h>
#include <math.h>

#if defined(__CUDACC__)
#define HSES_HD __host__ __device__ __forceinline__
#else
#define HSES_HD static inline
#endif

#if !defined(__CUDACC__)
struct double2 { double x, y; };
#endif

namespace hses {

// ---------------------------------------------------------------------------
// bit casts and strictly rounded arithmetic
// ---------------------------------------------------------------------------
HSES_HD uint32_t f2u(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
HSES_HD float u2f(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}
HSES_HD uint64_t d2u(double d) {
#if defined(__CUDA_ARCH__)
    return (uint64_t)__double_as_longlong(d);
#else
    uint64_t u; memcpy(&u, &d, 8); return u;
#endif
}
HSES_HD double dfma(double a, double b, double c) {
#if defined(__CUDA_ARCH__)
    return __fma_rn(a, b, c);
#else
    return fma(a, b, c);
#endif
}
HSES_HD double dmul(double a, double b) {
#if defined(__CUDA_ARCH__)
    return __dmul_rn(a, b);
#else
    return a * b;
#endif
}
HSES_HD double dadd(double a, double b) {
#if defined(__CUDA_ARCH__)
    return __dadd_rn(a, b);
#else
    return a + b;
#endif
}
HSES_HD float fmul(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fmul_rn(a, b);
#else
    return a * b;
#endif
}
HSES_HD float fsqrt(float a) {
#if defined(__CUDA_ARCH__)
    return __fsqrt_rn(a);
#else
    return sqrtf(a);
#endif
}
HSES_HD float d2f_rn(double d) {
#if defined(__CUDA_ARCH__)
    return __double2float_rn(d);
#else
    return (float)d;
#endif
}

// ---------------------------------------------------------------------------
// seed hash and generator (noiser.rs:444-455, 495-506)
// ---------------------------------------------------------------------------
HSES_HD uint64_t noise_seed(uint64_t key, int32_t true_epoch, int32_t true_thread) {
    uint64_t h = key ^ 0x9E3779B97F4A7C15ull;
    h *= 0xBF58476D1CE4E5B9ull;
    h ^= (uint64_t)(int64_t)true_epoch * 0x94D049BB133111EBull;
    h = ((h << 17) | (h >> 47)) ^ (uint64_t)(int64_t)true_thread;
    h ^= h >> 33;
    h *= 0xBF58476D1CE4E5B9ull;
    h ^= h >> 29;
    h *= 0x94D049BB133111EBull;
    h ^= h >> 32;
    return h;
}

// One generator step (shifts 13, 7, 17).  On the device every 64-bit shift is
// written as 32x32->64 multiplications by a power of two: the product of a word
// with 2^s holds (word << s) in its low half and (word >> (32 - s)) in its high
// half, and multiplications issue on the FMA pipe, which this code leaves idle,
// instead of the integer pipe that bounds it.
HSES_HD uint64_t xs64_step(uint64_t x) {
#if defined(__CUDA_ARCH__)
    uint32_t lo = (uint32_t)x, hi = (uint32_t)(x >> 32);
    uint64_t m = (uint64_t)lo * 8192u;                 // x ^= x << 13
    uint32_t h = hi * 8192u;
    lo ^= (uint32_t)m;
    hi ^= h ^ (uint32_t)(m >> 32);
    uint64_t mh = (uint64_t)hi * 33554432u;            // x ^= x >> 7
    uint64_t ml = (uint64_t)lo * 33554432u;
    lo ^= (uint32_t)(ml >> 32) ^ (uint32_t)mh;
    hi ^= (uint32_t)(mh >> 32);
    m = (uint64_t)lo * 131072u;                        // x ^= x << 17
    h = hi * 131072u;
    lo ^= (uint32_t)m;
    hi ^= h ^ (uint32_t)(m >> 32);
    return ((uint64_t)hi << 32) | lo;
#else
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    return x;
#endif
}

// eggroll.rs:60-65: noise_reuse==0 pins the epoch bucket to 0; members 2p and
// 2p+1 share the draw of pair p, the odd one with A negated.
HSES_HD int32_t true_epoch_of(int32_t epoch, int32_t noise_reuse) {
    return noise_reuse == 0 ? 0 : epoch / noise_reuse;
}

// ---------------------------------------------------------------------------
// GF(2) jump tables: one 64x64 matrix is stored as 16 nibble tables of 16
// entries (2 KB); applying it costs 16 lookups and xors.
// ---------------------------------------------------------------------------
constexpr int kJumpWords = 256;  // uint64 words per matrix

HSES_HD uint64_t jump_apply(const uint64_t* __restrict__ tab, uint64_t x) {
    uint64_t r = 0;
#pragma unroll
    for (int p = 0; p < 16; ++p) r ^= tab[p * 16 + (int)((x >> (4 * p)) & 15)];
    return r;
}

// tabs[k] advances the state by unit*2^k steps; n is in units.
HSES_HD uint64_t jump_by(const uint64_t* __restrict__ tabs, uint64_t x, uint64_t n) {
    for (int k = 0; n != 0; ++k, n >>= 1)
        if (n & 1) x = jump_apply(tabs + (size_t)k * kJumpWords, x);
    return x;
}

// ---------------------------------------------------------------------------
// libm-conformant logf / cosf on the 24-bit uniforms
// ---------------------------------------------------------------------------
struct LibmCal {
    const double2* log_tab;      // 64 x {1/c, log c}
    const uint32_t* log_flip;    // 2^24 bits
    const uint32_t* cos_flip;    // 2^24 bits
    const uint32_t* log_delta;   // 256 thresholds on |low29 - 2^28|, by top byte of the input
    const uint32_t* cos_delta;   // 256 thresholds
    float log_of_zero;           // host logf(1e-9f), used when the uniform is 0
};

constexpr double kLn2 = 0x1.62e42fefa39efp-1;
constexpr double kPio2Hi = 0x1.921fb54442d10p+0;   // pi/2 to 49 bits: n*hi exact for n <= 15
constexpr double kPio2Lo = 0x1.08d313198a2e0p-49;  // pi/2 - hi
constexpr float kTauF = 6.2831855f;                // std::f32::consts::TAU

// fp64 value of log(i * 2^-24), i in [1, 2^24), accurate to ~2^-38 relative.
// z*2^k = u with z in [0.75, 1.5); 64 sub-intervals uniform in the fp32 bit
// pattern, the two that touch 1.0 use c = 1 so r = z - 1 is exact there.
HSES_HD double log_candidate(uint32_t i, const double2* __restrict__ tab) {
    float uf = (float)i * 5.9604644775390625e-08f;  // exact: i < 2^24, scale 2^-24
    uint32_t ix = f2u(uf);
    uint32_t tmp = ix - 0x3f400000u;
    int j = (int)((tmp >> 17) & 63u);
    int k = (int32_t)tmp >> 23;
    float zf = u2f(ix - (tmp & 0xff800000u));
    double2 e = tab[j];
    double r = dfma((double)zf, e.x, -1.0);
    double p = dfma(r, -1.0 / 6.0, 1.0 / 5.0);
    p = dfma(r, p, -1.0 / 4.0);
    p = dfma(r, p, 1.0 / 3.0);
    p = dfma(r, p, -1.0 / 2.0);
    p = dfma(dmul(r, r), p, r);              // r - r^2/2 + ... - r^6/6
    return dfma((double)k, kLn2, dadd(e.y, p));
}

// fp64 value of cos(theta) for an fp32 theta in [0, 2*pi], ~2^-44 relative.
// cos(t) = sin(t + pi/2) = (-1)^q sin(rho), rho = t - (2q-1)*pi/2 in [-pi/2, pi/2].
HSES_HD double cos_candidate(float theta) {
    int q = (int)(fmul(theta, 0.31830987f) + 1.0f);  // any q with |rho| <~ pi/2 + 1e-6 works
    double n = (double)(2 * q - 1);
    double rho = dfma(-n, kPio2Hi, (double)theta);
    rho = dfma(-n, kPio2Lo, rho);
    double s = dmul(rho, rho);
    double p = dfma(s, 1.0 / 355687428096000.0, -1.0 / 1307674368000.0);  // 1/17!, -1/15!
    p = dfma(s, p, 1.0 / 6227020800.0);                                  // 1/13!
    p = dfma(s, p, -1.0 / 39916800.0);                                   // -1/11!
    p = dfma(s, p, 1.0 / 362880.0);                                      // 1/9!
    p = dfma(s, p, -1.0 / 5040.0);                                       // -1/7!
    p = dfma(s, p, 1.0 / 120.0);                                         // 1/5!
    p = dfma(s, p, -1.0 / 6.0);                                          // -1/3!
    double v = dfma(dmul(rho, s), p, rho);
    return (q & 1) ? -v : v;
}

// Round an fp64 candidate to fp32 and report how the rounding went:
// low29 = discarded mantissa bits, alt = the neighbour on the other side of
// the rounding midpoint.
struct Rounded {
    uint32_t bits;   // round-to-nearest result
    uint32_t alt;    // the other bracketing fp32 value: bits + step
    uint32_t dist;   // |low29 - 2^28|: 0 at the midpoint, 2^28 on an fp32 value
    int32_t step;    // +1 or -1
};
HSES_HD Rounded round_candidate(double y) {
    // The rounding itself is the hardware's fp64 -> fp32 conversion (the conversion pipe is nearly idle
    // in this code, the integer pipe is what bounds it).  The other neighbour lies one step up in
    // magnitude when the discarded bits are below the midpoint and one step down otherwise.  An exact
    // midpoint would make that rule name the wrong neighbour for an even mantissa; the candidates
    // (logarithms and cosines of fp32 arguments) never are, and the calibration would refuse a
    // context in which the host's value is neither `bits` nor `alt`.
    Rounded r;
#if defined(__CUDA_ARCH__)
    const uint32_t low = (uint32_t)__double2loint(y) & 0x1fffffffu;
#else
    const uint32_t low = (uint32_t)(d2u(y) & 0x1fffffffull);
#endif
    r.bits = f2u(d2f_rn(y));
    r.step = low >= 0x10000000u ? -1 : 1;
    r.alt = r.bits + (uint32_t)r.step;
    r.dist = low >= 0x10000000u ? low - 0x10000000u : 0x10000000u - low;
    return r;
}

// bit (i mod 32) of a bitmap word
HSES_HD uint32_t bit_of(uint32_t word, uint32_t i) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_r(word, 0u, i) & 1u;   // the funnel shift takes its count modulo 32
#else
    return (word >> (i & 31u)) & 1u;
#endif
}

HSES_HD float apply_flip(const Rounded& r, uint32_t idx, const uint32_t* __restrict__ flip,
                         const uint32_t* __restrict__ delta) {
    uint32_t bits = r.bits;
    if (r.dist < delta[idx >> 16]) {
        if ((flip[idx >> 5] >> (idx & 31u)) & 1u) bits = r.alt;
    }
    return u2f(bits);
}

// logf(max(i*2^-24, 1e-9f)) as the host libm returns it.
HSES_HD float libm_logf_u24(uint32_t i, const LibmCal& cal) {
    if (i == 0) return cal.log_of_zero;
    return apply_flip(round_candidate(log_candidate(i, cal.log_tab)), i, cal.log_flip, cal.log_delta);
}
// cosf(TAU * j*2^-24) as the host libm returns it.
HSES_HD float libm_cosf_u24(uint32_t j, const LibmCal& cal) {
    float theta = fmul(kTauF, (float)j * 5.9604644775390625e-08f);
    return apply_flip(round_candidate(cos_candidate(theta)), j, cal.cos_flip, cal.cos_delta);
}

// noiser.rs:470-477: one standard normal from two consecutive generator outputs.
HSES_HD float normal_from_draws(uint64_t x1, uint64_t x2, const LibmCal& cal) {
    float lg = libm_logf_u24((uint32_t)(x1 >> 40), cal);
    float radius = fsqrt(fmul(-2.0f, lg));
    return fmul(radius, libm_cosf_u24((uint32_t)(x2 >> 40), cal));
}

HSES_HD float next_normal(uint64_t& state, const LibmCal& cal) {
    uint64_t x1 = xs64_step(state);
    uint64_t x2 = xs64_step(x1);
    state = x2;
    return normal_from_draws(x1, x2, cal);
}

// Four consecutive normals of the stream.  Same values as four next_normal()
// calls; the work is laid out as independent chains (eight generator steps, four
// logarithms, four cosines, then all bitmap reads issued together without
// branches) so that table and bitmap latencies overlap instead of adding up.
// LOG2T: the two threshold tables are 256 bytes each holding ceil(log2(threshold)) (see
// pack_thresholds_log2): a threshold rounded up only sends a few more candidates to the bitmap,
// whose bit decides, so the values are the same; the tables then fit where 2 KB would not.
// TSHIFT: the byte tables are indexed by input >> TSHIFT (16: 256 entries; 17: 128 entries, each the
// larger of two neighbouring thresholds — again only a few more candidates for the bitmap).
template <bool LOG2T, int TSHIFT = 16>
HSES_HD void next_normals4_t(uint64_t& state, const LibmCal& cal, float (&out)[4]) {
    uint32_t iu[4], ju[4];
    uint64_t x = state;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        x = xs64_step(x);
        iu[j] = (uint32_t)(x >> 40);
        x = xs64_step(x);
        ju[j] = (uint32_t)(x >> 40);
    }
    state = x;
    Rounded rl[4], rc[4];
    bool nl[4], nc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t i = iu[j] ? iu[j] : 1u;  // the zero uniform is replaced below
        rl[j] = round_candidate(log_candidate(i, cal.log_tab));
        if (LOG2T)
            nl[j] = rl[j].dist < (1u << reinterpret_cast<const uint8_t*>(cal.log_delta)[i >> TSHIFT]);
        else
            nl[j] = rl[j].dist < cal.log_delta[i >> 16];
        float theta = fmul(kTauF, (float)ju[j] * 5.9604644775390625e-08f);
        rc[j] = round_candidate(cos_candidate(theta));
        if (LOG2T)
            nc[j] = rc[j].dist < (1u << reinterpret_cast<const uint8_t*>(cal.cos_delta)[ju[j] >> TSHIFT]);
        else
            nc[j] = rc[j].dist < cal.cos_delta[ju[j] >> 16];
    }
    uint32_t wl[4], wc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t i = iu[j] ? iu[j] : 1u;
        wl[j] = nl[j] ? cal.log_flip[i >> 5] : 0u;
        wc[j] = nc[j] ? cal.cos_flip[ju[j] >> 5] : 0u;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t i = iu[j] ? iu[j] : 1u;
        // the bitmap's bit times the step to the other neighbour: a multiply-add (FMA pipe) instead of
        // a compare and a select (integer pipe, the one that bounds this code)
        uint32_t lb = rl[j].bits + (uint32_t)((int32_t)bit_of(wl[j], i) * rl[j].step);
        uint32_t cb = rc[j].bits + (uint32_t)((int32_t)bit_of(wc[j], ju[j]) * rc[j].step);
        float lg = iu[j] ? u2f(lb) : cal.log_of_zero;
        out[j] = fmul(fsqrt(fmul(-2.0f, lg)), u2f(cb));
    }
}

HSES_HD void next_normals4(uint64_t& state, const LibmCal& cal, float (&out)[4]) {
    next_normals4_t<false>(state, cal, out);
}
// ceil(log2(t)) of a 32-bit threshold as a byte (0 for t <= 1): dist < t implies dist < 2^byte
HSES_HD uint8_t pack_threshold_log2(uint32_t t) {
    uint8_t e = 0;
    while (e < 31 && (1u << e) < t) ++e;
    return e;
}

}  // namespace hses
