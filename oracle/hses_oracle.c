/*
 * CPU oracle for the EggRoll population step.  TEST INFRASTRUCTURE ONLY —
 * see hses_oracle.h for scope and parity status.  Each function cites the
 * reference source (paths relative to the reference's burn_impl/ directory)
 * that it restates.  Compile with -ffp-contract=off: every fp32 operation is
 * rounded on its own, as an op-by-op tensor backend does.
 */
#include "hses_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* A launcher may pin OMP_NUM_THREADS to 1 for every rank; the timed CPU baseline asks for the
 * cores the process may run on instead. */
void hso_set_num_threads(int n) {
    if (n >= 1) omp_set_num_threads(n);
}

int hso_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* RNG contract                                                             */
/* ------------------------------------------------------------------------ */

/* hyperscalees-noiser/src/noiser.rs:495-506 (noise_seed).  The i32 arguments
 * are converted with `as u64`, i.e. sign-extended. */
uint64_t hso_noise_seed(uint64_t key, int32_t true_epoch, int32_t true_thread) {
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

/* noiser.rs:444-455 (DeterministicNoise::new / next_u64). */
static inline uint64_t xs64_next(uint64_t *s) {
    uint64_t x = *s;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    *s = x;
    return x;
}

/* noiser.rs:457-460 (next_unit): 24 fractional bits, exact in fp32. */
static inline float xs64_unit(uint64_t *s) {
    return (float)(xs64_next(s) >> 40) / 16777216.0f;
}

/* noiser.rs:470-477 (standard_normal): Box-Muller, cosine branch only. */
static inline float xs64_normal(uint64_t *s) {
    float u1 = fmaxf(xs64_unit(s), 1e-9f);
    float u2 = xs64_unit(s);
    float radius = sqrtf(-2.0f * logf(u1));
    float theta = 6.2831855f * u2; /* std::f32::consts::TAU */
    return radius * cosf(theta);
}

void hso_xorshift64_stream(uint64_t seed, uint64_t *out, size_t n) {
    uint64_t s = seed | 1ull;
    for (size_t i = 0; i < n; ++i) out[i] = xs64_next(&s);
}

void hso_units(uint64_t seed, float *out, size_t n) {
    uint64_t s = seed | 1ull;
    for (size_t i = 0; i < n; ++i) out[i] = xs64_unit(&s);
}

/* noiser.rs:481-490 (normal_tensor): row-major fill. */
void hso_normals(uint64_t seed, float *out, size_t n) {
    uint64_t s = seed | 1ull;
    for (size_t i = 0; i < n; ++i) out[i] = xs64_normal(&s);
}

/* hyperscalees-noiser/src/eggroll.rs:60-65 (epoch_thread_sign). */
void hso_epoch_thread_sign(int32_t epoch, int32_t thread_id, int32_t noise_reuse,
                           int32_t *true_epoch, int32_t *true_thread, float *sign) {
    *true_epoch = noise_reuse == 0 ? 0 : epoch / noise_reuse;
    *true_thread = thread_id / 2;
    *sign = (thread_id % 2 == 0) ? 1.0f : -1.0f;
}

/* eggroll.rs:86-103 (get_lora_update_params): one (a+b, r) normal tensor,
 * rows [0,b) are B, rows [b,a+b) are A; A is scaled by sign*base_sigma. */
void hso_lora_params(float base_sigma, uint64_t key, int rank, int32_t epoch,
                     int32_t thread_id, int a, int b, int32_t noise_reuse,
                     float *A, float *B) {
    int32_t te, tt;
    float sign;
    hso_epoch_thread_sign(epoch, thread_id, noise_reuse, &te, &tt, &sign);
    uint64_t s = hso_noise_seed(key, te, tt) | 1ull;
    size_t nb = (size_t)b * rank, na = (size_t)a * rank;
    for (size_t i = 0; i < nb; ++i) {
        float z = xs64_normal(&s);
        if (B) B[i] = z;
    }
    float sc = sign * base_sigma;
    for (size_t i = 0; i < na; ++i) {
        float z = xs64_normal(&s);
        if (A) A[i] = z * sc;
    }
}

/* eggroll.rs:312-324 (get_nonlora_update_params). */
void hso_nonlora_params(float base_sigma, uint64_t key, int32_t epoch,
                        int32_t thread_id, int rows, int cols,
                        int32_t noise_reuse, float *out) {
    int32_t te, tt;
    float sign;
    hso_epoch_thread_sign(epoch, thread_id, noise_reuse, &te, &tt, &sign);
    uint64_t s = hso_noise_seed(key, te, tt) | 1ull;
    float sc = sign * base_sigma;
    size_t n = (size_t)rows * cols;
    for (size_t i = 0; i < n; ++i) out[i] = xs64_normal(&s) * sc;
}

/* ------------------------------------------------------------------------ */
/* Perturbed linear                                                         */
/* ------------------------------------------------------------------------ */

static inline float dot_f32(const float *p, const float *q, int n, int sp, int sq) {
    float acc = 0.0f;
    for (int i = 0; i < n; ++i) acc += p[(size_t)i * sp] * q[(size_t)i * sq];
    return acc;
}
static inline float dot_f64(const float *p, const float *q, int n, int sp, int sq) {
    double acc = 0.0;
    for (int i = 0; i < n; ++i) acc += (double)p[(size_t)i * sp] * (double)q[(size_t)i * sq];
    return (float)acc;
}

/* Baseline-timing variant of the dot product: sixteen independent partial
 * sums so the compiler can keep SIMD lanes busy (a tuned CPU GEMM, which the
 * reference's CPU backend uses, does not accumulate strictly in index order
 * either).  Selected with acc mode 2; parity checks use modes 0 and 1. */
__attribute__((target_clones("avx512f", "avx2", "default")))
static float dot_fast(const float *p, const float *q, int n) {
    float acc[16] = {0};
    int i = 0;
    for (; i + 16 <= n; i += 16)
        for (int j = 0; j < 16; ++j) acc[j] += p[i + j] * q[i + j];
    float s = 0.0f;
    for (int j = 0; j < 16; ++j) s += acc[j];
    for (; i < n; ++i) s += p[i] * q[i];
    return s;
}

/* Baseline-timing variant of the base product: a 4 x 4 block of outputs (four rows of x against
 * four rows of the parameter) with sixteen SIMD accumulators, so that every loaded vector feeds
 * four multiply-adds — the register blocking a tuned CPU GEMM such as the reference's backend
 * applies.  Fused multiply-adds, lane-wise partial sums: for timing (acc mode 2) only. */
__attribute__((target_clones("avx512f", "avx2,fma", "default")))
static void base_block4x4(const float *x, const float *w, int b, float *y, int ystride) {
    float acc[16][16];
    for (int e = 0; e < 16; ++e)
        for (int l = 0; l < 16; ++l) acc[e][l] = 0.0f;
    int i = 0;
    for (; i + 16 <= b; i += 16)
        for (int r = 0; r < 4; ++r)
            for (int c = 0; c < 4; ++c)
                for (int l = 0; l < 16; ++l)
                    acc[r * 4 + c][l] = __builtin_fmaf(x[(size_t)r * b + i + l], w[(size_t)c * b + i + l], acc[r * 4 + c][l]);
    for (int r = 0; r < 4; ++r)
        for (int c = 0; c < 4; ++c) {
            float s = 0.0f;
            for (int l = 0; l < 16; ++l) s += acc[r * 4 + c][l];
            for (int k = i; k < b; ++k) s += x[(size_t)r * b + k] * w[(size_t)c * b + k];
            y[(size_t)r * ystride + c] = s;
        }
}

/* y = x·paramᵀ + (x·B)·Aᵀ with pre-generated factors; evaluation order of
 * eggroll.rs:427,443: base first, then t = x·B, u = t·Aᵀ, y = base + u. */
static void mm_with_factors(const float *x, int bm, const float *param, int a, int b,
                            int rank, const float *A, const float *B, int acc64,
                            float *y) {
    float *t = A ? (float *)malloc(sizeof(float) * (size_t)bm * rank) : NULL;
    if (A) {
        for (int m = 0; m < bm; ++m)
            for (int q = 0; q < rank; ++q)
                t[(size_t)m * rank + q] =
                    acc64 == 1 ? dot_f64(x + (size_t)m * b, B + q, b, 1, rank)
                               : dot_f32(x + (size_t)m * b, B + q, b, 1, rank);
    }
    if (acc64 == 2 && bm % 4 == 0 && a % 4 == 0) {
        /* blocked base product, then the rank-r term per output */
        for (int m = 0; m < bm; m += 4)
            for (int n = 0; n < a; n += 4)
                base_block4x4(x + (size_t)m * b, param + (size_t)n * b, b, y + (size_t)m * a + n, a);
        if (A)
            for (int m = 0; m < bm; ++m)
                for (int n = 0; n < a; ++n)
                    y[(size_t)m * a + n] += dot_f32(t + (size_t)m * rank, A + (size_t)n * rank, rank, 1, 1);
        free(t);
        return;
    }
    for (int m = 0; m < bm; ++m) {
        for (int n = 0; n < a; ++n) {
            float base = acc64 == 2 ? dot_fast(x + (size_t)m * b, param + (size_t)n * b, b)
                         : acc64 ? dot_f64(x + (size_t)m * b, param + (size_t)n * b, b, 1, 1)
                                 : dot_f32(x + (size_t)m * b, param + (size_t)n * b, b, 1, 1);
            if (A) {
                float u = acc64 == 1 ? dot_f64(t + (size_t)m * rank, A + (size_t)n * rank, rank, 1, 1)
                                     : dot_f32(t + (size_t)m * rank, A + (size_t)n * rank, rank, 1, 1);
                base = base + u;
            }
            y[(size_t)m * a + n] = base;
        }
    }
    free(t);
}

/* eggroll.rs:419-446 (do_mm_impl). */
void hso_do_mm(const float *x, int bm, const float *param, int a, int b,
               float sigma, int rank, uint64_t key, int has_iter, int32_t epoch,
               int32_t thread_id, int32_t noise_reuse, int acc64, float *y) {
    if (!has_iter) {
        mm_with_factors(x, bm, param, a, b, rank, NULL, NULL, acc64, y);
        return;
    }
    float *A = (float *)malloc(sizeof(float) * (size_t)a * rank);
    float *B = (float *)malloc(sizeof(float) * (size_t)b * rank);
    float base_sigma = sigma / sqrtf((float)rank);
    hso_lora_params(base_sigma, key, rank, epoch, thread_id, a, b, noise_reuse, A, B);
    mm_with_factors(x, bm, param, a, b, rank, A, B, acc64, y);
    free(A);
    free(B);
}

/* ------------------------------------------------------------------------ */
/* LIF                                                                      */
/* ------------------------------------------------------------------------ */

/* hyperscalees-models/src/snn.rs:53-65 (lif_step): leak -> charge -> fire ->
 * reset, each op rounded.  Hard reset is the reference behaviour; the
 * subtractive reset (charged - spike*v_th) has no reference counterpart and
 * is defined here only. */
static inline float lif_one(float *v, float cur, float leak, float v_th, int reset_mode) {
    float d = (-*v) + cur;
    float m = d * leak;
    float c = *v + m;
    float s = (c >= v_th) ? 1.0f : 0.0f;
    if (reset_mode == HSO_RESET_HARD)
        *v = c * ((-s) + 1.0f);
    else
        *v = c - s * v_th;
    return s;
}

/* snn.rs:73-97 (run_lif). */
void hso_run_lif(const float *cur, int T, size_t nh, float tau_m, float v_th,
                 int reset_mode, float *v, float *spikes) {
    float leak = 1.0f / tau_m;
    for (int t = 0; t < T; ++t)
        for (size_t i = 0; i < nh; ++i)
            spikes[(size_t)t * nh + i] = lif_one(&v[i], cur[(size_t)t * nh + i], leak, v_th, reset_mode);
}

/* ------------------------------------------------------------------------ */
/* Poisson encode                                                           */
/* ------------------------------------------------------------------------ */

/* hyperscalees-kernels/src/poisson_encode_fused_oxide.rs:36-52,84-105: one
 * xorshift32 stream per element, seeded 1000000007*idx + (s0^s1^s2^s3) +
 * 0x9E3779B9; u = ((x>>9)+1)/8388609; spike = u < p.  Rows are pitched. */
void hso_poisson_encode(const float *probs, size_t batch, size_t in_dim,
                        size_t row_stride, int T, const uint32_t seeds[4],
                        float *out) {
    uint32_t mix = seeds[0] ^ seeds[1] ^ seeds[2] ^ seeds[3];
    size_t out_step = batch * row_stride;
    for (size_t row = 0; row < batch; ++row) {
        for (size_t col = 0; col < in_dim; ++col) {
            uint32_t idx = (uint32_t)(row * in_dim + col);
            size_t base = row * row_stride + col;
            float p = probs[base];
            uint32_t x = 1000000007u * idx + mix + 0x9E3779B9u;
            for (int t = 0; t < T; ++t) {
                x ^= x << 13;
                x ^= x >> 17;
                x ^= x << 5;
                float u = ((float)(x >> 9) + 1.0f) / 8388609.0f;
                out[(size_t)t * out_step + base] = (u < p) ? 1.0f : 0.0f;
            }
        }
    }
}

/* ------------------------------------------------------------------------ */
/* Fitness                                                                  */
/* ------------------------------------------------------------------------ */

/* hyperscalees-envs/src/snn_mnist.rs:180-201 (fitness_from_logits_reward);
 * the max-shifted log_softmax is the form spelled out in the reference's own
 * test (snn_mnist.rs:373-401). */
void hso_fitness(const float *logits, size_t n, int classes, const int32_t *labels,
                 int reward, float *out) {
    for (size_t i = 0; i < n; ++i) {
        const float *row = logits + i * (size_t)classes;
        float mx = row[0];
        int arg = 0;
        for (int c = 1; c < classes; ++c)
            if (row[c] > mx) { mx = row[c]; arg = c; }
        if (reward == HSO_REWARD_BINARY) {
            out[i] = (arg == labels[i]) ? 1.0f : 0.0f;
        } else {
            float sum = 0.0f;
            for (int c = 0; c < classes; ++c) sum += expf(row[c] - mx);
            out[i] = row[labels[i]] - mx - logf(sum);
        }
    }
}

/* hyperscalees-noiser/src/noiser.rs:517-537 (convert_fitnesses_impl): global
 * mean/var, std = sqrt(var + 1e-5); per-group centring uses the global std. */
void hso_convert_fitnesses(const float *raw, size_t n, int group_size, float *out) {
    float sum = 0.0f, sumsq = 0.0f;
    for (size_t i = 0; i < n; ++i) sum += raw[i];
    for (size_t i = 0; i < n; ++i) sumsq += raw[i] * raw[i];
    float mean = sum / (float)n;
    float var = sumsq / (float)n - mean * mean;
    float std = sqrtf(var + 1e-5f);
    float inv = 1.0f / std;
    if (group_size == 0) {
        for (size_t i = 0; i < n; ++i) out[i] = (raw[i] + (-mean)) * inv;
    } else {
        size_t gs = (size_t)group_size, ng = n / gs;
        for (size_t g = 0; g < ng; ++g) {
            float gsum = 0.0f;
            for (size_t j = 0; j < gs; ++j) gsum += raw[g * gs + j];
            float gmean = gsum / (float)gs;
            for (size_t j = 0; j < gs; ++j) out[g * gs + j] = (raw[g * gs + j] - gmean) * inv;
        }
    }
}

/* EggRollBS::convert_fitnesses, hyperscalees-noiser/src/eggroll_bs.rs:226-250: raw scores as
 * (Q, G) rows; baseline = first column; Z = (S - b) / (row std + 1e-8), row var = E[x^2] - E[x]^2;
 * columns 0 and 1 are zeroed; result = mean over rows (length G). */
void hso_convert_fitnesses_bs(const float *raw, size_t n, int group_size, float *out) {
    size_t g = (size_t)group_size, q = n / g;
    for (size_t j = 0; j < g; ++j) out[j] = 0.0f;
    for (size_t r = 0; r < q; ++r) {
        const float *s = raw + r * g;
        float sum = 0.0f, sumsq = 0.0f;
        for (size_t j = 0; j < g; ++j) sum += s[j];
        for (size_t j = 0; j < g; ++j) sumsq += s[j] * s[j];
        float mean = sum / (float)g;
        float std = sqrtf(sumsq / (float)g - mean * mean);
        float den = std + 1e-8f;
        for (size_t j = 2; j < g; ++j) out[j] += (s[j] - s[0]) / den;
    }
    for (size_t j = 0; j < g; ++j) out[j] = out[j] / (float)q;
}

/* ------------------------------------------------------------------------ */
/* SNN forward for one member                                               */
/* ------------------------------------------------------------------------ */

/* snn.rs:253-282 (SnnModel::forward) with the noise closure of
 * hyperscalees/src/snn_mnist_train.rs:186-214, generalised to any number of
 * hidden layers; noise keys are per parameter index.  Dense (PARAM-class)
 * leaves such as out_gain stay clean in the forward (snn.rs:280-281). */
void hso_snn_forward(const hso_snn_t *m, const float *spikes_in, int T, int bm,
                     int has_iter, int32_t epoch, int32_t thread_id, int acc64,
                     float *logits, float *hidden_spikes) {
    int L = m->n_layers;
    float base_sigma = m->sigma / sqrtf((float)m->rank);
    const float *cur_in = spikes_in;
    float *owned = NULL;
    for (int l = 0; l < L - 1; ++l) {
        int b = m->dims[l], a = m->dims[l + 1];
        float *A = NULL, *B = NULL;
        if (has_iter) {
            A = (float *)malloc(sizeof(float) * (size_t)a * m->rank);
            B = (float *)malloc(sizeof(float) * (size_t)b * m->rank);
            hso_lora_params(base_sigma, m->keys[l], m->rank, epoch, thread_id, a, b,
                            m->noise_reuse, A, B);
        }
        float *cur = (float *)malloc(sizeof(float) * (size_t)T * bm * a);
        for (int t = 0; t < T; ++t)
            mm_with_factors(cur_in + (size_t)t * bm * b, bm, m->w[l], a, b, m->rank, A, B,
                            acc64, cur + (size_t)t * bm * a);
        free(A);
        free(B);
        float *v = (float *)calloc((size_t)bm * a, sizeof(float));
        float *sp = (float *)malloc(sizeof(float) * (size_t)T * bm * a);
        float vth = m->v_th_layer ? m->v_th_layer[l] : m->v_th;
        hso_run_lif(cur, T, (size_t)bm * a, m->tau_m, vth, m->reset_mode, v, sp);
        free(v);
        free(cur);
        free(owned);
        owned = sp;
        cur_in = sp;
    }
    int h = m->dims[L - 1], c = m->dims[L];
    if (hidden_spikes && owned) memcpy(hidden_spikes, owned, sizeof(float) * (size_t)T * bm * h);
    /* rate = mean over T (snn.rs:278) */
    float *rate = (float *)malloc(sizeof(float) * (size_t)bm * h);
    for (int i = 0; i < bm * h; ++i) {
        float s = 0.0f;
        for (int t = 0; t < T; ++t) s += cur_in[(size_t)t * bm * h + i];
        rate[i] = s / (float)T;
    }
    float *A = NULL, *B = NULL;
    if (has_iter) {
        A = (float *)malloc(sizeof(float) * (size_t)c * m->rank);
        B = (float *)malloc(sizeof(float) * (size_t)h * m->rank);
        hso_lora_params(base_sigma, m->keys[L - 1], m->rank, epoch, thread_id, c, h,
                        m->noise_reuse, A, B);
    }
    mm_with_factors(rate, bm, m->w[L - 1], c, h, m->rank, A, B, acc64, logits);
    for (int i = 0; i < bm * c; ++i) logits[i] = logits[i] * m->out_gain;
    free(A);
    free(B);
    free(rate);
    free(owned);
}

/* ------------------------------------------------------------------------ */
/* ES update                                                                */
/* ------------------------------------------------------------------------ */

/* eggroll.rs:353-373 (simple_lora_update) followed by the -g*sqrt(N) of
 * do_update_with (eggroll.rs:384-404).  acc += (A_i·B_iᵀ)·f_i in member
 * order; the rank-r dot product is rounded before the fitness scale. */
static void lora_grad_impl(float sigma, uint64_t key, int a, int b, int rank,
                           const float *scores, const int32_t *epochs,
                           const int32_t *thread_ids, size_t n, int32_t noise_reuse,
                           int sign_factors, float *out) {
    float base_sigma = sigma / sqrtf((float)rank);
    size_t ab = (size_t)a * b;
    int nthreads = hso_num_threads();
    float *partial = (float *)calloc(ab * (size_t)nthreads, sizeof(float));
    /* members are summed in index order inside a thread's contiguous range;
     * the per-thread partials are then added in thread order (the reference's
     * accumulation order across members is a plain loop; fp32 results agree
     * to rounding). */
#pragma omp parallel
    {
#ifdef _OPENMP
        int tid = omp_get_thread_num(), nt = omp_get_num_threads();
#else
        int tid = 0, nt = 1;
#endif
        float *acc = partial + ab * (size_t)tid;
        float *A = (float *)malloc(sizeof(float) * (size_t)a * rank);
        float *B = (float *)malloc(sizeof(float) * (size_t)b * rank);
        size_t lo = n * (size_t)tid / nt, hi = n * (size_t)(tid + 1) / nt;
        for (size_t i = lo; i < hi; ++i) {
            hso_lora_params(base_sigma, key, rank, epochs[i], thread_ids[i], a, b, noise_reuse, A, B);
            if (sign_factors) {
                /* alteggroll.rs:65-90: A_new = sign(A) * (sigma * f / sqrt(rank)), B_new = sign(B);
                 * the fitness is folded in below, after the dot product, which is exact here
                 * because every product is +-base_sigma or 0 */
                for (int e = 0; e < a * rank; ++e) A[e] = (A[e] > 0.0f ? 1.0f : A[e] < 0.0f ? -1.0f : 0.0f) * base_sigma;
                for (int e = 0; e < b * rank; ++e) B[e] = B[e] > 0.0f ? 1.0f : B[e] < 0.0f ? -1.0f : 0.0f;
            }
            float f = scores[i];
            for (int p = 0; p < a; ++p)
                for (int q = 0; q < b; ++q) {
                    float d = dot_f32(A + (size_t)p * rank, B + (size_t)q * rank, rank, 1, 1);
                    acc[(size_t)p * b + q] += d * f;
                }
        }
        free(A);
        free(B);
    }
    float inv_n = 1.0f / (float)n, rootn = sqrtf((float)n);
    for (size_t j = 0; j < ab; ++j) {
        float s = 0.0f;
        for (int t = 0; t < nthreads; ++t) s += partial[ab * (size_t)t + j];
        out[j] = -((s * inv_n) * rootn);
    }
    free(partial);
}

void hso_lora_grad(float sigma, uint64_t key, int a, int b, int rank,
                   const float *scores, const int32_t *epochs,
                   const int32_t *thread_ids, size_t n, int32_t noise_reuse,
                   float *out) {
    lora_grad_impl(sigma, key, a, b, rank, scores, epochs, thread_ids, n, noise_reuse, 0, out);
}

/* The sub-block out[m0..m1) x [n0..n1) of hso_lora_grad, for populations too large to contract
 * whole on the CPU: the same stream positions and the same sum (eggroll.rs:353-373, 384-404),
 * with the normals of the rows outside the block stepped over in the integer stream instead of
 * evaluated, and the member sum kept in fp64 (a yardstick for fp32 sums of 10^4..10^5 terms). */
void hso_lora_grad_block(float sigma, uint64_t key, int a, int b, int rank,
                         const float *scores, const int32_t *epochs,
                         const int32_t *thread_ids, size_t n, int32_t noise_reuse,
                         int m0, int m1, int n0, int n1, float *out) {
    (void)a;
    float base_sigma = sigma / sqrtf((float)rank);
    int bm = m1 - m0, bn = n1 - n0;
    size_t blk = (size_t)bm * bn;
    int nthreads = hso_num_threads();
    double *partial = (double *)calloc(blk * (size_t)nthreads, sizeof(double));
#pragma omp parallel num_threads(nthreads)
    {
        int t = 0;
#ifdef _OPENMP
        t = omp_get_thread_num();
#endif
        double *acc = partial + blk * (size_t)t;
        float *A = (float *)malloc(sizeof(float) * (size_t)bm * rank);
        float *B = (float *)malloc(sizeof(float) * (size_t)bn * rank);
#pragma omp for schedule(static)
        for (long i = 0; i < (long)n; ++i) {
            int32_t te, tt;
            float sign;
            hso_epoch_thread_sign(epochs[i], thread_ids[i], noise_reuse, &te, &tt, &sign);
            uint64_t s = hso_noise_seed(key, te, tt) | 1ull;
            /* every normal consumes two generator outputs */
            for (size_t k = 0; k < 2 * (size_t)rank * (size_t)n0; ++k) xs64_next(&s);
            for (int e = 0; e < bn * rank; ++e) B[e] = xs64_normal(&s);
            for (size_t k = 0; k < 2 * (size_t)rank * (size_t)(b - n1 + m0); ++k) xs64_next(&s);
            float sc = sign * base_sigma;
            for (int e = 0; e < bm * rank; ++e) A[e] = xs64_normal(&s) * sc;
            float f = scores[i];
            for (int p = 0; p < bm; ++p)
                for (int q = 0; q < bn; ++q) {
                    float d = dot_f32(A + (size_t)p * rank, B + (size_t)q * rank, rank, 1, 1);
                    acc[(size_t)p * bn + q] += (double)(d * f);
                }
        }
        free(A);
        free(B);
    }
    float inv_n = 1.0f / (float)n, rootn = sqrtf((float)n);
    for (size_t j = 0; j < blk; ++j) {
        double sum = 0.0;
        for (int t = 0; t < nthreads; ++t) sum += partial[blk * (size_t)t + j];
        out[j] = -(((float)sum * inv_n) * rootn);
    }
    free(partial);
}

/* AltEggRoll (hyperscalees-noiser/src/alteggroll.rs:65-90 + do_update_with): the same update
 * with every factor entry replaced by its sign. */
void hso_alt_lora_grad(float sigma, uint64_t key, int a, int b, int rank,
                       const float *scores, const int32_t *epochs,
                       const int32_t *thread_ids, size_t n, int32_t noise_reuse,
                       float *out) {
    lora_grad_impl(sigma, key, a, b, rank, scores, epochs, thread_ids, n, noise_reuse, 1, out);
}

/* eggroll.rs:331-350 (simple_full_update) + do_update_with. */
void hso_full_grad(float sigma, uint64_t key, int rows, int cols,
                   const float *scores, const int32_t *epochs,
                   const int32_t *thread_ids, size_t n, int32_t noise_reuse,
                   int freeze_nonlora, float *out) {
    size_t len = (size_t)rows * cols;
    float *acc = (float *)calloc(len, sizeof(float));
    float *up = (float *)malloc(sizeof(float) * len);
    if (!freeze_nonlora) {
        for (size_t i = 0; i < n; ++i) {
            hso_nonlora_params(sigma, key, epochs[i], thread_ids[i], rows, cols, noise_reuse, up);
            for (size_t j = 0; j < len; ++j) acc[j] += up[j] * scores[i];
        }
    }
    float inv_n = 1.0f / (float)n, rootn = sqrtf((float)n);
    for (size_t j = 0; j < len; ++j) out[j] = -((acc[j] * inv_n) * rootn);
    free(acc);
    free(up);
}

/* eggroll.rs:726-738 (lora_einsum_raw): Σ_n f_n Σ_r A'[n,r,i] B'[n,r,j]. */
void hso_lora_einsum_raw(const float *a_t, const float *b_t, const float *scores,
                         size_t n, int r, int a, int b, float *out) {
    for (int i = 0; i < a; ++i)
        for (int j = 0; j < b; ++j) {
            float acc = 0.0f;
            for (size_t k = 0; k < n * (size_t)r; ++k) {
                float w = scores ? a_t[k * a + i] * scores[k / r] : a_t[k * a + i];
                acc += w * b_t[k * b + j];
            }
            out[(size_t)i * b + j] = acc;
        }
}

/* eggroll.rs:741-748 (lora_einsum_ones). */
void hso_lora_einsum_ones(const float *a_t, const float *b_t, size_t n, int r,
                          int a, int b, float *out) {
    hso_lora_einsum_raw(a_t, b_t, NULL, n, r, a, b, out);
}

/* eggroll.rs:820-850 (lora_einsum_pair_half): f_pair = f_i + f_{half+i};
 * g_raw = Σ f_pair A'_i⊗B'_i ; g_ones = 2 Σ A'_i⊗B'_i. */
void hso_lora_einsum_pair_half(const float *a_half, const float *b_half,
                               const float *scores, size_t half, int r, int a,
                               int b, float *g_raw, float *g_ones) {
    float *fp = (float *)malloc(sizeof(float) * half);
    for (size_t i = 0; i < half; ++i) fp[i] = scores[i] + scores[half + i];
    hso_lora_einsum_raw(a_half, b_half, fp, half, r, a, b, g_raw);
    hso_lora_einsum_raw(a_half, b_half, NULL, half, r, a, b, g_ones);
    for (size_t j = 0; j < (size_t)a * b; ++j) g_ones[j] = g_ones[j] * 2.0f;
    free(fp);
}

/* eggroll.rs:902-915 (combine_affine_grads). */
void hso_combine_affine(const float *grad_acc, const float *ones_acc, size_t len,
                        float mean, float std, size_t batch, float *out) {
    float scale = -1.0f / (std * sqrtf((float)batch));
    for (size_t j = 0; j < len; ++j) out[j] = (grad_acc[j] - ones_acc[j] * mean) * scale;
}

/* ------------------------------------------------------------------------ */
/* Solver                                                                   */
/* ------------------------------------------------------------------------ */

/* noiser.rs:155-224 (Solver::update).  AdamW adds +wd*param, unscaled by lr,
 * exactly as the reference writes it (noiser.rs:207-212). */
void hso_solver_update(const hso_solver_t *s, int32_t step, float *param,
                       const float *grad, float *m, float *v, size_t len) {
    if (s->kind == HSO_SGD) {
        for (size_t i = 0; i < len; ++i) param[i] = param[i] - grad[i] * s->lr;
        return;
    }
    float t = (float)step;
    float bc1 = 1.0f - powf(s->beta1, t);
    float bc2 = 1.0f - powf(s->beta2, t);
    float wd = s->kind == HSO_ADAMW ? s->weight_decay : 0.0f;
    float omb1 = 1.0f - s->beta1, omb2 = 1.0f - s->beta2;
    float ibc1 = 1.0f / bc1, ibc2 = 1.0f / bc2;
    float nlr = -s->lr;
    for (size_t i = 0; i < len; ++i) {
        float g = grad[i];
        float mn = m[i] * s->beta1 + g * omb1;
        float vn = v[i] * s->beta2 + powf(g, 2.0f) * omb2;
        m[i] = mn;
        v[i] = vn;
        float mh = mn * ibc1, vh = vn * ibc2;
        float denom = sqrtf(vh) + s->eps;
        float term = (mh / denom) * nlr;
        if (wd == 0.0f)
            param[i] = param[i] + term;
        else
            param[i] = (param[i] + term) + param[i] * wd;
    }
}

/* noiser.rs:232-244 (clip_grads_global_norm): returns the factor every
 * gradient is multiplied by (1 when no clipping applies). */
float hso_clip_scale(const float *const *grads, const size_t *lens, int n,
                     float max_norm) {
    float global_sq = 0.0f;
    for (int k = 0; k < n; ++k) {
        float s = 0.0f;
        for (size_t i = 0; i < lens[k]; ++i) s += powf(grads[k][i], 2.0f);
        global_sq += s;
    }
    float norm = sqrtf(global_sq);
    if (norm > max_norm && norm > 0.0f) return max_norm / norm;
    return 1.0f;
}

/* ------------------------------------------------------------------------ */
/* Perturbed linear + one LIF step over a population                        */
/* ------------------------------------------------------------------------ */

/* Composition of do_mm (eggroll.rs:419-446) and lif_step (snn.rs:53-65) from
 * v0 = 0 for every member of a population; member i uses thread id
 * first_thread + i.  Members are independent, so they are spread over the
 * host threads. */
void hso_perturbed_linear_lif(const float *x, size_t n_pop, int bm, int k,
                              const float *param, int a, float sigma, int rank,
                              uint64_t key, int32_t epoch, int32_t first_thread,
                              int32_t noise_reuse, float tau_m, float v_th,
                              int reset_mode, int acc64, float *spikes,
                              float *potentials) {
    float leak = 1.0f / tau_m;
#pragma omp parallel
    {
        float *y = (float *)malloc(sizeof(float) * (size_t)bm * a);
#pragma omp for schedule(dynamic, 1)
        for (long long i = 0; i < (long long)n_pop; ++i) {
            hso_do_mm(x + (size_t)i * bm * k, bm, param, a, k, sigma, rank, key, 1, epoch,
                      first_thread + (int32_t)i, noise_reuse, acc64, y);
            for (int j = 0; j < bm * a; ++j) {
                float v = 0.0f;
                /* charged potential (before the reset) for tolerance checks */
                float d = (-v) + y[j];
                float c = v + d * leak;
                if (potentials) potentials[(size_t)i * bm * a + j] = c;
                spikes[(size_t)i * bm * a + j] = lif_one(&v, y[j], leak, v_th, reset_mode);
            }
        }
        free(y);
    }
}

/* ------------------------------------------------------------------------ */
/* GPU-path noise stream                                                    */
/* ------------------------------------------------------------------------ */

/* hyperscalees-kernels/src/lib.rs:26-101: three Tausworthe steps and one LCG
 * step per uniform, two uniforms per Box-Muller pair, cos and sin both kept. */
static inline uint32_t taus(uint32_t z, int s1, int s2, int s3, uint32_t m) {
    uint32_t b = ((z << s1) ^ z) >> s2;
    return ((z & m) << s3) ^ b;
}
static inline float taus_unit(uint32_t st[4]) {
    st[0] = taus(st[0], 13, 19, 12, 4294967294u);
    st[1] = taus(st[1], 2, 25, 4, 4294967288u);
    st[2] = taus(st[2], 3, 11, 17, 4294967280u);
    st[3] = st[3] * 1664525u + 1013904223u;
    uint32_t r = st[0] ^ st[1] ^ st[2] ^ st[3];
    return ((float)(r >> 9) + 1.0f) / 8388609.0f;
}

/* lib.rs:123-143 (prng_normal_half_kernel): thread t fills out[128t..128t+128). */
void hso_prng_normal_half(float *out, size_t total_threads, float mean, float std,
                          const uint32_t seeds[4]) {
    for (size_t t = 0; t < total_threads; ++t) {
        uint32_t s = 1000000007u * (uint32_t)t;
        uint32_t st[4] = {s + seeds[0], s + seeds[1], s + seeds[2], s + seeds[3]};
        for (int i = 0; i < 128; i += 2) {
            float u0 = taus_unit(st), u1 = taus_unit(st);
            float coeff = sqrtf(logf(u0) * -2.0f) * std;
            float arg = (2.0f * 3.14159274f) * u1;
            out[t * 128 + i] = cosf(arg) * coeff + mean;
            out[t * 128 + i + 1] = sinf(arg) * coeff + mean;
        }
    }
}

/* ------------------------------------------------------------------------ */
/* RWKV-7 state recurrence                                                  */
/* ------------------------------------------------------------------------ */

/* hyperscalees-models/src/llm.rs:235-296 (rwkv7_inner_loop): decay
 * w = exp(-exp(w)); sa = S·a; S = S⊙w + v kᵀ + sa bᵀ; out = S·r. */
void hso_wkv7(const float *r, const float *w, const float *k, const float *v,
              const float *a, const float *b, const uint8_t *new_starts, int T,
              int H, int S, float *state, float *out) {
    float *sa = (float *)malloc(sizeof(float) * (size_t)S);
    for (int t = 0; t < T; ++t) {
        if (new_starts && new_starts[t]) memset(state, 0, sizeof(float) * (size_t)H * S * S);
        for (int h = 0; h < H; ++h) {
            size_t o = ((size_t)t * H + h) * S;
            float *st = state + (size_t)h * S * S;
            for (int i = 0; i < S; ++i) {
                float acc = 0.0f;
                for (int j = 0; j < S; ++j) acc += st[(size_t)i * S + j] * a[o + j];
                sa[i] = acc;
            }
            for (int i = 0; i < S; ++i)
                for (int j = 0; j < S; ++j) {
                    float dec = expf(-expf(w[o + j]));
                    float s0 = st[(size_t)i * S + j] * dec;
                    float s1 = s0 + v[o + i] * k[o + j];
                    st[(size_t)i * S + j] = s1 + sa[i] * b[o + j];
                }
            for (int i = 0; i < S; ++i) {
                float acc = 0.0f;
                for (int j = 0; j < S; ++j) acc += st[(size_t)i * S + j] * r[o + j];
                out[o + i] = acc;
            }
        }
    }
    free(sa);
}

/* ------------------------------------------------------------------------ */
/* Spiking self-attention core                                              */
/* ------------------------------------------------------------------------ */

/* src/hyperscalees/models/snn_self_attention.py:45-98 (row_softmax_lif,
 * self_attention_lif) for one head: Q, K, V are (tokens, d) firing rates.
 * mode 0 is the spike product without softmax, O = (beta Q K^T) V, which has no
 * reference counterpart beyond the two matmuls (mode 3: the same with the scores of keys
 * j > i set to zero, for next-token models); mode 1 is the LIF-count row
 * softmax: each row of beta*QK^T divided by (max|row| + 1e-6), n_iter LIF steps
 * (hard reset, lif_step of snn_attention.py) driven by row - g_inh*sum(counts),
 * weights = counts / (sum(counts) + 1e-6). */
void hso_spiking_attention(const float *Q, const float *K, const float *V, int tokens, int d,
                           int mode, float beta, float tau_m, float v_th, float g_inh, int n_iter,
                           float *O, float *A) {
    float *row = (float *)malloc(sizeof(float) * (size_t)tokens * 3);
    float *u = row + tokens, *cnt = row + 2 * tokens;
    for (int i = 0; i < tokens; ++i) {
        float amax = 0.0f;
        for (int j = 0; j < tokens; ++j) {
            float acc = 0.0f;
            for (int c = 0; c < d; ++c) acc += Q[(size_t)i * d + c] * K[(size_t)j * d + c];
            row[j] = beta * acc;
            if (mode == 3 && j > i) row[j] = 0.0f; /* causal spike product: keys after the query are masked */
            if (fabsf(row[j]) > amax) amax = fabsf(row[j]);
        }
        if (mode == 1) {
            float inv = amax + 1e-6f, leak = 1.0f / tau_m;
            for (int j = 0; j < tokens; ++j) { row[j] = row[j] / inv; u[j] = 0.0f; cnt[j] = 0.0f; }
            for (int it = 0; it < n_iter; ++it) {
                float G = 0.0f;
                for (int j = 0; j < tokens; ++j) G += cnt[j];
                float inh = g_inh * G;
                for (int j = 0; j < tokens; ++j) {
                    float s = lif_one(&u[j], row[j] - inh, leak, v_th, HSO_RESET_HARD);
                    cnt[j] += s;
                }
            }
            float tot = 0.0f;
            for (int j = 0; j < tokens; ++j) tot += cnt[j];
            tot += 1e-6f;
            for (int j = 0; j < tokens; ++j) row[j] = cnt[j] / tot;
        }
        if (mode == 2) {
            /* continuous_attention, hyperscalees-models/src/snn_transformer.rs:80-102: Hopfield
             * relaxation u <- u + (1/tau)(-u + H - g*mean_key(u)) from u = H, n_iter steps, then
             * a stable softmax along the keys with 1e-6 added to the denominator */
            float one_over_tau = 1.0f / tau_m;
            for (int j = 0; j < tokens; ++j) u[j] = row[j];
            for (int it = 0; it < n_iter; ++it) {
                float m = 0.0f;
                for (int j = 0; j < tokens; ++j) m += u[j];
                m = m / (float)tokens;
                for (int j = 0; j < tokens; ++j) u[j] = u[j] + ((-u[j] + row[j]) - m * g_inh) * one_over_tau;
            }
            float mx = u[0];
            for (int j = 1; j < tokens; ++j) if (u[j] > mx) mx = u[j];
            float tot = 0.0f;
            for (int j = 0; j < tokens; ++j) { cnt[j] = expf(u[j] - mx); tot += cnt[j]; }
            tot += 1e-6f;
            for (int j = 0; j < tokens; ++j) row[j] = cnt[j] / tot;
        }
        if (A) memcpy(A + (size_t)i * tokens, row, sizeof(float) * (size_t)tokens);
        for (int c = 0; c < d; ++c) {
            float acc = 0.0f;
            for (int j = 0; j < tokens; ++j) acc += row[j] * V[(size_t)j * d + c];
            O[(size_t)i * d + c] = acc;
        }
    }
    free(row);
}

/* ------------------------------------------------------------------------ */
/* RWKV-7 block pieces around the WKV recurrence                             */
/* ------------------------------------------------------------------------ */

/* layer_norm, hyperscalees-models/src/llm.rs:64-84: per row over the last axis,
 * var = E[x^2] - E[x]^2, (x - mean) / sqrt(var + eps) * weight + bias. */
void hso_layer_norm(const float *x, size_t rows, int c, const float *weight, const float *bias,
                    float eps, float *out) {
    for (size_t r = 0; r < rows; ++r) {
        const float *xr = x + r * (size_t)c;
        float sum = 0.0f, sumsq = 0.0f;
        for (int j = 0; j < c; ++j) sum += xr[j];
        for (int j = 0; j < c; ++j) sumsq += xr[j] * xr[j];
        float mean = sum / (float)c;
        float var = sumsq / (float)c - mean * mean;
        float std = sqrtf(var + eps);
        for (int j = 0; j < c; ++j) out[r * (size_t)c + j] = (xr[j] - mean) / std * weight[j] + bias[j];
    }
}

/* GroupNorm::forward, llm.rs:90-145: x (n, c, l) (l = 1 for the rank-2 form), channels split
 * into `groups`; statistics over the (c / groups) * l values of a group; gamma/beta per channel. */
void hso_group_norm(const float *x, size_t n, int c, int l, int groups, const float *weight,
                    const float *bias, float eps, float *out) {
    int inner = c / groups;
    size_t cnt = (size_t)inner * l;
    for (size_t i = 0; i < n; ++i)
        for (int g = 0; g < groups; ++g) {
            const float *xg = x + (i * (size_t)c + (size_t)g * inner) * l;
            float sum = 0.0f, sumsq = 0.0f;
            for (size_t j = 0; j < cnt; ++j) sum += xg[j];
            for (size_t j = 0; j < cnt; ++j) sumsq += xg[j] * xg[j];
            float mean = sum / (float)cnt;
            float var = sumsq / (float)cnt - mean * mean;
            float std = sqrtf(var + eps);
            for (int ch = 0; ch < inner; ++ch)
                for (int t = 0; t < l; ++t) {
                    size_t o = (i * (size_t)c + (size_t)g * inner + ch) * l + t;
                    out[o] = weight[g * inner + ch] * ((x[o] - mean) / std) + bias[g * inner + ch];
                }
        }
}

/* The token shift of ChannelMixing / TimeMixing, llm.rs:192-206: sx = previous row (row 0: the
 * carried state), zero where a new sequence starts, minus x; out = x + sx * coef. */
void hso_token_shift_mix(const float *x, int T, int c, const float *state, const uint8_t *new_starts,
                         const float *coef, float *out) {
    for (int t = 0; t < T; ++t)
        for (int j = 0; j < c; ++j) {
            float prev = t == 0 ? state[j] : x[(size_t)(t - 1) * c + j];
            if (new_starts && new_starts[t]) prev = 0.0f;
            float sx = prev - x[(size_t)t * c + j];
            out[(size_t)t * c + j] = x[(size_t)t * c + j] + sx * coef[j];
        }
}

/* ChannelMixing::forward, llm.rs:192-213 with bias-free Linear layers (x @ W^T, common.rs:123-127):
 * xk = token shift; k = relu(xk @ Wk^T)^2 (Wk: (f, c)); out = k @ Wv^T (Wv: (c, f));
 * state_out = x[length - 1]. */
void hso_channel_mix(const float *x, int T, int c, int f, const float *state, const uint8_t *new_starts,
                     const float *x_k, const float *wk, const float *wv, int length, float *out,
                     float *state_out) {
    float *xk = (float *)malloc(sizeof(float) * (size_t)T * c);
    float *k = (float *)malloc(sizeof(float) * (size_t)T * f);
    hso_token_shift_mix(x, T, c, state, new_starts, x_k, xk);
    for (int t = 0; t < T; ++t)
        for (int j = 0; j < f; ++j) {
            float d = dot_f32(xk + (size_t)t * c, wk + (size_t)j * c, c, 1, 1);
            d = d > 0.0f ? d : 0.0f;
            k[(size_t)t * f + j] = d * d;
        }
    for (int t = 0; t < T; ++t)
        for (int j = 0; j < c; ++j) out[(size_t)t * c + j] = dot_f32(k + (size_t)t * f, wv + (size_t)j * f, f, 1, 1);
    for (int j = 0; j < c; ++j) state_out[j] = x[(size_t)(length - 1) * c + j];
    free(xk);
    free(k);
}

/* rate_encode, snn_transformer.rs:109-116: sigmoid(gain * p / (1 + |p|)). */
void hso_rate_encode(const float *p, size_t n, float gain, float *out) {
    for (size_t i = 0; i < n; ++i) {
        float ss = p[i] / (fabsf(p[i]) + 1.0f);
        out[i] = 1.0f / (1.0f + expf(-(ss * gain)));
    }
}
