/*
 * CPU oracle for the EggRoll population step.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference algorithm (HyperscaleES,
 * burn_impl/ Rust crates).  It exists so that the CUDA path can be checked
 * against an independent implementation and so that a CPU baseline can be
 * timed.  Nothing in the shipped library links, loads or calls it; only the
 * test suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Parity status: the reference cannot be compiled or imported on the build
 * machine (no Rust toolchain, no JAX), so this restatement is pinned against
 *   (a) the hand-computed expectations inside the reference's own unit tests
 *       (transcribed under tests/golden/ with file:line citations), and
 *   (b) an independent pure-integer Python restatement of the RNG contract
 *       (tests/golden/gen_rng_kat.py).
 * The reference holds no absolute known-answer vector for its RNG output, so
 * the float normals are pinned by source reading plus the host libm
 * (logf/cosf/sqrtf of glibc on x86-64), which is what the Rust code calls.
 * Accumulation order inside matmuls is owned by a third-party crate
 * (burn-flex 0.21.0 / gemm 0.19.0) and is NOT pinned: matmul results are
 * compared with tolerances, never bitwise.
 *
 * Every step is individually rounded in fp32 (compile with
 * -ffp-contract=off), matching an op-by-op tensor backend.
 */
#ifndef HSES_ORACLE_H
#define HSES_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- RNG contract (hyperscalees-noiser/src/noiser.rs:436-506) ---------- */
uint64_t hso_noise_seed(uint64_t key, int32_t true_epoch, int32_t true_thread);
void hso_xorshift64_stream(uint64_t seed, uint64_t *out, size_t n);
void hso_units(uint64_t seed, float *out, size_t n);
void hso_normals(uint64_t seed, float *out, size_t n);
/* hyperscalees-noiser/src/eggroll.rs:60-65 */
void hso_epoch_thread_sign(int32_t epoch, int32_t thread_id, int32_t noise_reuse,
                           int32_t *true_epoch, int32_t *true_thread, float *sign);
/* eggroll.rs:86-103: A is (a,r) scaled by sign*base_sigma, B is (b,r) raw. */
void hso_lora_params(float base_sigma, uint64_t key, int rank, int32_t epoch,
                     int32_t thread_id, int a, int b, int32_t noise_reuse,
                     float *A, float *B);
/* eggroll.rs:312-324 */
void hso_nonlora_params(float base_sigma, uint64_t key, int32_t epoch,
                        int32_t thread_id, int rows, int cols,
                        int32_t noise_reuse, float *out);

/* ---- perturbed linear (eggroll.rs:419-446) ----------------------------- */
/* y(bm,a) = x(bm,b)·paramᵀ + (x·B)·Aᵀ ; iter==0 -> clean.  acc64 selects the
 * accumulation of the dot products: 0 = fp32 in index order, 1 = double (used
 * to locate near-threshold elements), 2 = fp32 with SIMD-friendly partial sums
 * for the base product (CPU-baseline timing only). */
void hso_do_mm(const float *x, int bm, const float *param, int a, int b,
               float sigma, int rank, uint64_t key, int has_iter, int32_t epoch,
               int32_t thread_id, int32_t noise_reuse, int acc64, float *y);

/* ---- LIF (hyperscalees-models/src/snn.rs:53-97) ------------------------ */
enum { HSO_RESET_HARD = 0, HSO_RESET_SUBTRACT = 1 };
/* cur,(T,n,h) contiguous; v in/out (n,h); spikes (T,n,h). */
void hso_run_lif(const float *cur, int T, size_t nh, float tau_m, float v_th,
                 int reset_mode, float *v, float *spikes);

/* ---- Poisson encode, xorshift32 stream
 *      (hyperscalees-kernels/src/poisson_encode_fused_oxide.rs:36-105) ---- */
void hso_poisson_encode(const float *probs, size_t batch, size_t in_dim,
                        size_t row_stride, int T, const uint32_t seeds[4],
                        float *out /* (T,batch,row_stride) */);

/* ---- fitness (hyperscalees-envs/src/snn_mnist.rs:180-201) -------------- */
enum { HSO_REWARD_LOGLIK = 0, HSO_REWARD_BINARY = 1 };
void hso_fitness(const float *logits, size_t n, int classes, const int32_t *labels,
                 int reward, float *out);
/* noiser.rs:517-537 */
void hso_convert_fitnesses(const float *raw, size_t n, int group_size, float *out);
void hso_convert_fitnesses_bs(const float *raw, size_t n, int group_size, float *out);

/* ---- SNN forward for one member
 *      (snn.rs:253-282 generalised to a list of hidden layers) ------------ */
typedef struct {
    int n_layers;            /* hidden layers + readout */
    const int *dims;         /* n_layers+1 entries: in, h1, ..., classes */
    const float *const *w;   /* n_layers matrices, (out,in) row-major */
    const uint64_t *keys;    /* n_layers base keys */
    float out_gain;
    float tau_m, v_th;       /* shared by all hidden layers ... */
    const float *v_th_layer; /* ... unless non-NULL: one threshold per hidden layer */
    int reset_mode;
    float sigma;
    int rank;
    int32_t noise_reuse;
} hso_snn_t;
/* spikes_in (T,bm,in); logits (bm,classes).  has_iter==0 -> clean forward.
 * hidden_spikes, if non-NULL, receives the spikes of the last hidden layer
 * (T,bm,h_last). */
void hso_snn_forward(const hso_snn_t *m, const float *spikes_in, int T, int bm,
                     int has_iter, int32_t epoch, int32_t thread_id, int acc64,
                     float *logits, float *hidden_spikes);

/* ---- ES update (eggroll.rs:331-404) ------------------------------------ */
/* g = (1/N) Σ f_i A_i B_iᵀ, returns grad = -(g*sqrt(N)) in out (a,b). */
void hso_lora_grad(float sigma, uint64_t key, int a, int b, int rank,
                   const float *scores, const int32_t *epochs,
                   const int32_t *thread_ids, size_t n, int32_t noise_reuse,
                   float *out);
/* rows [m0,m1) x columns [n0,n1) of the same gradient, member sum in fp64 */
void hso_lora_grad_block(float sigma, uint64_t key, int a, int b, int rank,
                         const float *scores, const int32_t *epochs,
                         const int32_t *thread_ids, size_t n, int32_t noise_reuse,
                         int m0, int m1, int n0, int n1, float *out);
void hso_alt_lora_grad(float sigma, uint64_t key, int a, int b, int rank,
                   const float *scores, const int32_t *epochs,
                   const int32_t *thread_ids, size_t n, int32_t noise_reuse,
                   float *out);
void hso_full_grad(float sigma, uint64_t key, int rows, int cols,
                   const float *scores, const int32_t *epochs,
                   const int32_t *thread_ids, size_t n, int32_t noise_reuse,
                   int freeze_nonlora, float *out);
/* einsum helpers on materialised (n,r,a)/(n,r,b) noise (eggroll.rs:726-915) */
void hso_lora_einsum_raw(const float *a_t, const float *b_t, const float *scores,
                         size_t n, int r, int a, int b, float *out);
void hso_lora_einsum_ones(const float *a_t, const float *b_t, size_t n, int r,
                          int a, int b, float *out);
void hso_lora_einsum_pair_half(const float *a_half, const float *b_half,
                               const float *scores, size_t half, int r, int a,
                               int b, float *g_raw, float *g_ones);
void hso_combine_affine(const float *grad_acc, const float *ones_acc, size_t len,
                        float mean, float std, size_t batch, float *out);

/* ---- solver (noiser.rs:155-244) ---------------------------------------- */
enum { HSO_SGD = 0, HSO_ADAM = 1, HSO_ADAMW = 2 };
typedef struct {
    int kind;
    float lr, beta1, beta2, eps, weight_decay;
} hso_solver_t;
/* step is the value AFTER the increment for Adam/AdamW (ignored for SGD). */
void hso_solver_update(const hso_solver_t *s, int32_t step, float *param,
                       const float *grad, float *m, float *v, size_t len);
float hso_clip_scale(const float *const *grads, const size_t *lens, int n,
                     float max_norm);

/* ---- perturbed-linear + one LIF step over a population (microbench) ---- */
/* x (n_pop,bm,k); param (a,k); spikes (n_pop,bm,a); potentials optional
 * (charged membrane before reset).  thread ids = first_thread + member. */
void hso_perturbed_linear_lif(const float *x, size_t n_pop, int bm, int k,
                              const float *param, int a, float sigma, int rank,
                              uint64_t key, int32_t epoch, int32_t first_thread,
                              int32_t noise_reuse, float tau_m, float v_th,
                              int reset_mode, int acc64, float *spikes,
                              float *potentials);

/* ---- GPU-path noise stream (hyperscalees-kernels/src/lib.rs:26-143) ---- */
void hso_prng_normal_half(float *out, size_t total_threads, float mean, float std,
                          const uint32_t seeds[4]);

/* ---- RWKV-7 inner loop (hyperscalees-models/src/llm.rs:235-296) -------- */
/* r,w,k,v,a,b: (T,H,S); state in/out (H,S,S) indexed [h][i][j]; out (T,H,S).
 * new_starts (T) optional: state is zeroed before step t when non-zero. */
void hso_wkv7(const float *r, const float *w, const float *k, const float *v,
              const float *a, const float *b, const uint8_t *new_starts, int T,
              int H, int S, float *state, float *out);

/* ---- spiking self-attention core for one head
 *      (src/hyperscalees/models/snn_self_attention.py:45-98) ------------------ */
void hso_spiking_attention(const float *Q, const float *K, const float *V, int tokens, int d,
                           int mode, float beta, float tau_m, float v_th, float g_inh, int n_iter,
                           float *O, float *A);

void hso_layer_norm(const float *x, size_t rows, int c, const float *weight, const float *bias,
                    float eps, float *out);
void hso_group_norm(const float *x, size_t n, int c, int l, int groups, const float *weight,
                    const float *bias, float eps, float *out);
void hso_token_shift_mix(const float *x, int T, int c, const float *state, const uint8_t *new_starts,
                         const float *coef, float *out);
void hso_channel_mix(const float *x, int T, int c, int f, const float *state, const uint8_t *new_starts,
                     const float *x_k, const float *wk, const float *wv, int length, float *out,
                     float *state_out);
void hso_rate_encode(const float *p, size_t n, float gain, float *out);
int hso_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
