/*
 * hses.h — C ABI of the B200-native EggRoll population step.
 *
 * Conventions (they follow the raw-pointer seam the reference already uses
 * for its native kernels, hyperscalees/src/oxide.rs:96-146):
 *   - every pointer marked "device" is a CUDA device pointer owned by the
 *     caller; outputs are caller-allocated, nothing here frees caller memory;
 *   - matrices are row-major fp32 with an explicit row stride in ELEMENTS
 *     (Burn pitches rows to 256 B, oxide.rs:225-232), unless stated otherwise;
 *   - work is enqueued on the caller's stream and never synchronised inside
 *     an entry point (oxide.rs:119-125); the only blocking call is
 *     hses_ctx_create;
 *   - every entry point returns an hses_status; on failure
 *     hses_last_error() gives a message for the calling thread.  Shape
 *     violations are reported, not aborted on;
 *   - a context belongs to one device and is not thread-safe; distinct
 *     contexts are independent.
 *
 * There is no CPU fallback: every compute entry point launches CUDA kernels
 * built for sm_100a and fails if that is impossible.
 */
#ifndef HSES_H
#define HSES_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct hses_ctx hses_ctx;
typedef void* hses_stream; /* cudaStream_t */

enum hses_status {
    HSES_OK = 0,
    HSES_ERR_INVALID = 1,     /* bad argument / unsupported shape */
    HSES_ERR_CUDA = 2,        /* a CUDA runtime call failed */
    HSES_ERR_CALIBRATION = 3, /* libm calibration found a non-adjacent value */
    HSES_ERR_UNSUPPORTED = 4, /* requested algorithm cannot run this shape */
    HSES_ERR_COMM = 5         /* a collective or its communicator failed (a peer left, transport error) */
};

enum hses_reset_mode { HSES_RESET_HARD = 0, HSES_RESET_SUBTRACT = 1 };
enum hses_reward { HSES_REWARD_LOGLIK = 0, HSES_REWARD_BINARY = 1 };
enum hses_solver_kind { HSES_SGD = 0, HSES_ADAM = 1, HSES_ADAMW = 2 };
enum hses_factor_layout {
    HSES_LAYOUT_NAR = 0, /* A (n,a,r), B (n,b,r): batched_lora_noise, eggroll.rs:116-130 */
    HSES_LAYOUT_NRA = 1  /* A (n,r,a), B (n,r,b): batched forward / einsum layout, snn.rs:472-476 */
};
enum hses_linear_algo { HSES_ALGO_AUTO = 0, HSES_ALGO_SIMT = 1, HSES_ALGO_TENSOR = 2, HSES_ALGO_PAIR = 3 };
enum hses_precision { HSES_PRECISION_FP32 = 0, HSES_PRECISION_BF16 = 1 };
enum hses_x_op { HSES_X_NONE = 0, HSES_X_RELU_SQUARE = 1 };

const char* hses_last_error(void);
int hses_version(void);

/* ---- context: replaces hyperscalees-core default_device()/is_gpu()
 *      (hyperscalees-core/src/lib.rs:6-23) and the process-global kernel
 *      caches of oxide.rs:197-202.  Creation uploads the generator's jump
 *      tables and calibrates the device logf/cosf against the host libm over
 *      all 2^24 uniforms (blocking, well under a second). ------------------- */
int hses_ctx_create(int device, hses_ctx** out);
int hses_ctx_destroy(hses_ctx* ctx);
/* How many of the 2^24 inputs the host libm rounds away from the correctly
 * rounded value (diagnostic; tests compare it with their own count). */
int hses_ctx_calibration_info(const hses_ctx* ctx, uint64_t* log_flips, uint64_t* cos_flips);

/* ---- device-side status.  Kernels that wait on barriers do so with an
 *      iteration limit; one that gives up records a non-zero code here and
 *      returns instead of hanging.  This call synchronises (it copies one int
 *      back), reports the code and clears it; 0 means no kernel gave up.
 *      The reference has no counterpart (its launches cannot time out). ----- */
int hses_ctx_device_status(hses_ctx* ctx, int* status);

/* ---- launch accounting.  Every kernel the library launches is counted per
 *      context; with timing on, each launch is also bracketed by CUDA events
 *      on the launching stream.  hses_profile_enable clears the counters;
 *      hses_profile_read waits for the recorded events of entry `index`
 *      (0 .. hses_profile_count()-1) and returns its name, launch count and
 *      summed device time.  The reference's closest facility is the
 *      ACC_TIMING / ACC_PHASE wall-clock switches of
 *      hyperscalees/src/bin/accumulate_train.rs:722-768. -------------------- */
int hses_profile_enable(hses_ctx* ctx, int timing);
int hses_profile_count(hses_ctx* ctx);
int hses_profile_read(hses_ctx* ctx, int index, const char** name, int64_t* launches,
                      double* total_ms);

/* ---- seed hash: noise_seed, hyperscalees-noiser/src/noiser.rs:495-506 ---- */
uint64_t hses_noise_seed(uint64_t key, int32_t true_epoch, int32_t true_thread);

/* ---- DeterministicNoise::normal_tensor, noiser.rs:481-490: n standard
 *      normals of the stream seeded by `seed`, in stream order. ------------ */
int hses_normal_fill(hses_ctx* ctx, hses_stream stream, uint64_t seed, float* out /*device*/,
                     size_t n);

/* ---- get_lora_update_params / batched_lora_noise, eggroll.rs:86-130.
 *      Member i uses thread id thread_ids[i] (device int32) or, when
 *      thread_ids is NULL, first_thread + i.  A is scaled by sign*base_sigma
 *      (sign = -1 for odd thread ids), B is the raw normal block.  Either
 *      output may be NULL. -------------------------------------------------- */
int hses_lora_factors(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                      int32_t noise_reuse, const int32_t* thread_ids /*device or NULL*/,
                      int32_t first_thread, int64_t n_members, int32_t rank, int32_t a, int32_t b,
                      float base_sigma, int32_t layout, float* A /*device*/, float* B /*device*/);

/* ---- get_nonlora_update_params, eggroll.rs:312-324: sign*base_sigma*N(0,1)
 *      of shape (rows, cols) per member, out is (n, rows, cols). ----------- */
int hses_dense_noise(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                     int32_t noise_reuse, const int32_t* thread_ids /*device or NULL*/,
                     int32_t first_thread, int64_t n_members, int32_t rows, int32_t cols,
                     float base_sigma, float* out /*device*/);

/* ---- prng_normal_half, oxide.rs:233-275 / kernel hyperscalees-kernels/src/lib.rs:26-143: the
 *      hybrid Tausworthe + LCG stream of the GPU trainer's half-noise buffers.  out holds
 *      total_threads * 128 values (N_VALUES_PER_THREAD, lib.rs:19); reference thread t fills
 *      out[128t, 128t+128) from states 1000000007*t + seeds[j].  Unlike the reference wrapper
 *      (wall-clock seeds, oxide.rs:205-223) the four seed words are explicit.  The integer
 *      stream and the uniforms are bit-exact; ln/sqrt/cos/sin are device functions. ---- */
int hses_prng_normal_half(hses_ctx* ctx, hses_stream stream, float* out /*device*/, int64_t total_threads,
                          float mean, float std, const uint32_t seeds[4]);

/* ---- poisson_encode_fused, oxide.rs:573-625 /
 *      hyperscalees-kernels/src/poisson_encode_fused_oxide.rs:61-106.
 *      probs (batch, in_dim) pitched; out (T, batch, in_dim) with the same
 *      pitch.  Unlike the reference wrapper (wall-clock seeds, oxide.rs:205-223)
 *      the four seed words are explicit, so the spikes are reproducible. ---- */
int hses_poisson_encode(hses_ctx* ctx, hses_stream stream, const float* probs /*device*/,
                        int64_t batch, int32_t in_dim, int64_t row_stride, int32_t T,
                        const uint32_t seeds[4], float* out /*device*/);
/* The same kernel, writing in the same pass a second copy of the spikes as fp16 0/1 in dense rows
 * (T, batch, in_dim): the operand format of the tensor-core layer that follows (x_half of
 * hses_linear_args), so that the layer does not have to read and convert the f32 spikes again.
 * out_half NULL gives hses_poisson_encode. */
int hses_poisson_encode_dual(hses_ctx* ctx, hses_stream stream, const float* probs /*device*/,
                             int64_t batch, int32_t in_dim, int64_t row_stride, int32_t T,
                             const uint32_t seeds[4], float* out /*device*/, void* out_half /*device or NULL*/);

/* ---- lif_fused, oxide.rs:489-543 / lif_fused_oxide.rs:37-70, run_lif
 *      snn.rs:73-97.  cur and spikes are (T, n, h) pitched; v is (n, h)
 *      pitched, read as v0 and overwritten with the final potential, or NULL
 *      for v0 = 0 with no write-back.  spikes may be the same buffer as cur
 *      (the scan then replaces the currents by the spikes). ------------------ */
int hses_lif_scan(hses_ctx* ctx, hses_stream stream, const float* cur /*device*/, int32_t T,
                  int64_t n, int32_t h, int64_t row_stride, float* v /*device or NULL*/,
                  float tau_m, float v_th, int32_t reset_mode, float* spikes /*device*/);

/* ---- LoraNoiseCache / build_lora_noise_cache, eggroll.rs:229-309: the raw
 *      factors of a contiguous range of antithetic pairs of one parameter,
 *      generated once and kept in device memory, so that the forward pass and
 *      the update of a step (and, while the epoch bucket does not change, of
 *      later steps) read them instead of regenerating them.  Reading a factor
 *      costs 4 bytes of HBM traffic, regenerating it about 150 instructions.
 *      Layout of `data`: A (n_pairs, a, rank) then B (n_pairs, b, rank), both
 *      raw N(0,1): neither the member's sign nor sigma/sqrt(rank) is applied, so
 *      one cache serves both members of a pair and any sigma.  The reference
 *      keeps its cache in host memory, one entry per member, and only for
 *      noise_reuse == 0; this one is valid for the epoch bucket it was built
 *      for and is checked against key and bucket by every call that takes it. */
typedef struct {
    const float* data; /* device, hses_factor_cache_bytes() */
    uint64_t key;
    int32_t true_epoch; /* epoch bucket: 0 when noise_reuse == 0, else epoch / noise_reuse */
    int32_t first_pair; /* = thread id / 2 of the first member covered */
    int64_t n_pairs;
    int32_t rank;
    int32_t a;
    int32_t b;
} hses_factor_cache;
size_t hses_factor_cache_bytes(int64_t n_pairs, int32_t rank, int32_t a, int32_t b);
/* Fills `data` and writes the descriptor to *cache. */
int hses_factor_cache_build(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                            int32_t noise_reuse, int32_t first_pair, int64_t n_pairs,
                            int32_t rank, int32_t a, int32_t b, float* data /*device*/,
                            hses_factor_cache* cache /*host, out*/);

/* ---- do_mm, eggroll.rs:419-446, for a whole population in one call, with
 *      an optional fused lif_step (snn.rs:53-65) from v0 = 0.
 *      x is (t_steps, n_pop, bm, k): row R belongs to member (R / bm) % n_pop,
 *      whose thread id is first_thread + member.  param is (a, k).
 *      out is (t_steps*n_pop*bm, a): y = x·paramᵀ + (x·B)·Aᵀ when lif == 0,
 *      else the 0/1 spikes of one LIF step applied to y.  potentials
 *      (optional, same shape) receives the charged membrane before reset. --- */
typedef struct {
    const float* x; /* device */
    int32_t t_steps;
    int64_t n_pop;
    int32_t bm;
    int32_t k;
    int64_t x_row_stride;
    const float* param; /* device, (a, k) */
    int32_t a;
    int64_t param_row_stride;
    float sigma; /* EggRoll sigma; the kernel uses sigma / sqrt(rank) */
    int32_t rank;
    uint64_t key;
    int32_t epoch;
    int32_t first_thread;
    int32_t noise_reuse;
    int32_t perturb; /* 0: clean x·paramᵀ (iterinfo = None) */
    int32_t lif;     /* 0: write y; 1: write spikes of one LIF step; 2: write the spikes of a LIF scan over
                        the t_steps from v0 = 0 (run_lif, snn.rs:73-97): row p of step t hands its membrane
                        to row p of step t+1; potentials must be NULL */
    float tau_m;
    float v_th;
    int32_t reset_mode;
    float out_scale; /* lif == 0 only: y is multiplied by this (readout gain, snn.rs:280-281) */
    const float* out_scale_ptr; /* device or NULL: when set, the gain is read from here instead
                                   (a trained out_gain can stay on the device between steps) */
    float* out; /* device */
    int64_t out_row_stride;
    float* potentials; /* device or NULL */
    int32_t algo;      /* hses_linear_algo */
    void* workspace;   /* device scratch, hses_perturbed_linear_workspace_bytes() */
    size_t workspace_bytes;
    const hses_factor_cache* cache; /* host pointer or NULL: take the factors from this cache
                                       instead of regenerating them (same results, bit for bit) */
    int32_t precision; /* hses_precision of the base product x·paramᵀ: FP32 (default) keeps products
                          fp32-equivalent (three fp16 passes on hi/lo halves); BF16 rounds x and param
                          to bf16 and multiplies once with fp32 accumulation — the arithmetic of a
                          model held in bf16 (the RWKV LM).  The rank-r term is fp32 in both.  Only the
                          tensor-core path has the BF16 form; with HSES_ALGO_AUTO a shape it does not
                          cover is computed in fp32 */
    int32_t factor_order; /* 0: do_mm, the parameter is (a = out, k = in) and the factor rows of the
                             input side come first in the member's stream (eggroll.rs:86-103, 419-446).
                             1: do_Tmm (eggroll.rs:450-477): the reference parameter is stored (in, out)
                             and its factor block puts the `out` rows first, then the `in` rows scaled by
                             sign*sigma/sqrt(rank); `param` is still handed over as (a = out, k = in), i.e.
                             transposed, and the call returns x·param_refᵀᵀ + (x·A)·Bᵀ.  Not combinable
                             with a factor cache */
    const void* x_half; /* device or NULL: the matrix x once more as dense fp16 rows (rows, k), for
                           callers whose x is exact in fp16 and who have that copy anyway (the 0/1
                           spikes hses_poisson_encode_dual writes).  The tensor-core path then takes
                           it as its operand instead of converting x; x itself is still required */
    void* out_half;     /* device or NULL: with lif = 1 or 2, the spikes once more as dense fp16 rows
                           (rows, a), written by the kernel that finishes the layer where it can (the
                           per-pair kernel with the fused scan), else by one conversion pass: the
                           x_half of the layer that follows.  a must be a multiple of 8 */
    int32_t x_split_valid; /* 1: the previous call on this workspace had the same x, the same shapes
                           (t_steps, n_pop, bm, k, a, rank, perturb, precision) and took the tensor-core
                           path, and nothing else has written the workspace since: its fp16 operand
                           split of x is still there and is not computed again (several projections of
                           one activation, e.g. the per-head Q/K/V of a block).  Ignored by the other
                           paths */
    int32_t n_groups;   /* 0 or 1: one parameter.  G >= 2: `param` holds G parameters of a / G rows each,
                           stacked along the rows, every one with its own noise (the per-head projections of
                           one activation in one call: x is read once instead of G times).  The factors come
                           from `cache`, which the caller assembles in the grouped layout: A (n_pairs, a, rank)
                           with the groups' A blocks stacked like the parameter, then B (n_pairs, G, k, rank);
                           its descriptor has b = G * k and the key the call passes as `key`.  Tensor-core
                           path only (k <= 1024, rank 1..4, 8 or 16, a / G a multiple of 32, or of 16 with
                           rank >= 8, the G blocks of B within 64 KB); other shapes return
                           HSES_ERR_UNSUPPORTED.  Column c of the result belongs to group c / (a / G) */
    int32_t x_op;       /* 0: x as it is.  HSES_X_RELU_SQUARE: the layer's input is relu(x)^2 (ChannelMixing's
                           k = relu(key(x))^2, llm.rs:208), applied where the tensor-core path's prepass reads x,
                           so that the activation costs no pass of its own.  Calls with noise whose prepass keeps
                           B in shared memory only (rank 1..4, 8, 16 and k within its limits); other calls return
                           HSES_ERR_UNSUPPORTED and the caller applies hses_relu_square first */
} hses_linear_args;
/* Scratch the call needs for these shapes and this algo (0 is possible). */
size_t hses_perturbed_linear_workspace_bytes(const hses_linear_args* args);
int hses_perturbed_linear(hses_ctx* ctx, hses_stream stream, const hses_linear_args* args);

/* ---- mean firing rate over the time axis, spikes.mean_dim(0) of snn.rs:278:
 *      x (T, n, h) pitched -> out (n, h) with its own pitch. ---------------- */
int hses_time_mean(hses_ctx* ctx, hses_stream stream, const float* x /*device*/, int32_t T,
                   int64_t n, int32_t h, int64_t row_stride, float* out /*device*/,
                   int64_t out_row_stride);

/* ---- fitness_from_logits_reward, hyperscalees-envs/src/snn_mnist.rs:180-201.
 *      logits (n, classes) dense; labels device int32; out (n). ------------- */
int hses_fitness(hses_ctx* ctx, hses_stream stream, const float* logits /*device*/, int64_t n,
                 int32_t classes, const int32_t* labels /*device*/, int32_t reward,
                 float* out /*device*/);

/* ---- mean over each member's bm consecutive samples: (n_pop*bm) -> (n_pop) */
int hses_member_mean(hses_ctx* ctx, hses_stream stream, const float* per_sample /*device*/,
                     int64_t n_pop, int32_t bm, float* out /*device*/);

/* ---- convert_fitnesses, eggroll.rs:967-992 / noiser.rs:517-537.  stats
 *      (optional, device, 2 floats) receives {mean, std}. ------------------- */
int hses_convert_fitnesses(hses_ctx* ctx, hses_stream stream, const float* raw /*device*/,
                           int64_t n, int32_t group_size, float* out /*device*/,
                           float* stats /*device or NULL*/);

/* ---- EggRollBS::convert_fitnesses, hyperscalees-noiser/src/eggroll_bs.rs:226-250: the raw
 *      scores as (Q = n / group_size, G = group_size) rows; the first column of a row is its
 *      baseline, Z = (S - baseline) / (row std + 1e-8), columns 0 and 1 are zeroed, and the
 *      result is the mean of Z over the rows: G values in `out`.  row_den: device scratch of Q
 *      floats. -------------------------------------------------------------- */
int hses_convert_fitnesses_bs(hses_ctx* ctx, hses_stream stream, const float* raw /*device*/,
                              int64_t n, int32_t group_size, float* out /*device, G*/,
                              float* row_den /*device, Q*/);
/* out[i] = a[i] * b[i]: applies EggRollBS's member mask (eggroll_bs.rs:73-80) to a fitness vector. */
int hses_vector_mul(hses_ctx* ctx, hses_stream stream, const float* a /*device*/,
                    const float* b /*device*/, float* out /*device*/, int64_t n);

/* ---- simple_lora_update + do_update_with, eggroll.rs:353-404:
 *      grad(a,b) = -sqrt(N) * (1/N) * sum_i f_i A_i B_iᵀ with the factors
 *      regenerated from seeds.  Members are first_thread .. first_thread+n-1
 *      (n even, first_thread even: antithetic pairs are folded).  `fitness`
 *      holds the n converted fitnesses.  n_total is the N of the formula
 *      (= n unless the caller splits the population and sums partial grads).
 *      workspace: device scratch of hses_es_update_workspace_bytes(). ------- */
size_t hses_es_update_workspace_bytes(int32_t a, int32_t b, int32_t rank, int64_t n);
int hses_es_update(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                   int32_t noise_reuse, int32_t first_thread, int64_t n, int64_t n_total,
                   int32_t rank, int32_t a, int32_t b, float sigma,
                   const float* fitness /*device*/, float* grad /*device (a,b) dense*/,
                   void* workspace /*device*/, size_t workspace_bytes);

/* ---- The same contraction with two more choices, for the trainer's chunked
 *      accumulation (accumulated_update / accumulated_update_cached,
 *      eggroll.rs:550-702):
 *        cache  when not NULL the factors are read from it, not regenerated;
 *        mode   HSES_UPDATE_GRAD: what hses_es_update computes;
 *               HSES_UPDATE_RAW_ACC: grad += sum_i s_i A_i B_iᵀ with A_i scaled
 *               by sign*sigma/sqrt(rank) (lora_einsum_raw, eggroll.rs:726-738),
 *               `fitness` holding raw scores; chunks of one step add up in
 *               grad, and combine_affine_grads (eggroll.rs:902-915) turns the
 *               sums into the gradient once mean and std are known.  The
 *               companion sum of lora_einsum_ones over whole antithetic pairs
 *               is exactly zero (A_2p+1 = -A_2p), so it needs no kernel. ---- */
enum { HSES_UPDATE_GRAD = 0, HSES_UPDATE_RAW_ACC = 1 };
typedef struct {
    uint64_t key;
    int32_t epoch;
    int32_t noise_reuse;
    int32_t first_thread;
    int64_t n;
    int64_t n_total;
    int32_t rank;
    int32_t a;
    int32_t b;
    float sigma;
    const float* fitness; /* device, n */
    float* grad;          /* device (a,b) dense */
    void* workspace;      /* device, hses_es_update_workspace_bytes() */
    size_t workspace_bytes;
    const hses_factor_cache* cache; /* host pointer or NULL */
    int32_t mode;
    int32_t sign_factors; /* 1: AltEggRoll's update, every factor entry replaced by its sign
                             (hyperscalees-noiser/src/alteggroll.rs:65-90) */
    int32_t algo;         /* hses_linear_algo: AUTO takes the tcgen05 contraction when rank is a
                             multiple of 64, else the general fp32 kernel; SIMT / TENSOR force
                             one of them */
} hses_update_args;
int hses_es_update_ex(hses_ctx* ctx, hses_stream stream, const hses_update_args* args);

/* ---- hses_es_update for callers that cannot hand over a workspace.  It has
 *      no counterpart in the reference.  Some hosts of this library never get
 *      to call cudaMalloc themselves: a plugin running inside another runtime's
 *      memory pool, a process whose device memory is fully pre-partitioned, or a
 *      step that must not touch the allocator because it would synchronise the
 *      device.  For them the scratch (factor chunk + split-K partial sums) is a
 *      fixed array of hses_es_update_static_scratch_bytes() = 16 MiB that is
 *      part of the library's device image, so every GPU that loads the library
 *      carries it until the process exits.  The call allocates nothing and
 *      frees nothing.  Limits and rules:
 *        - the partial sums (a*b floats per split) plus the factors of at least
 *          one antithetic pair ((a+b)*rank floats) must fit in the array,
 *          otherwise HSES_ERR_INVALID is returned with a message;
 *        - the first call on a device looks up the array's device address (the
 *          context's device must be current); make that first call before any
 *          stream capture begins;
 *        - all calls share the one array: it keeps whatever the last call left,
 *          nothing in it needs clearing beforehand (the first chunk overwrites
 *          the partial sums), and two calls that overlap on the GPU (different
 *          streams, or different contexts on one device) race on it.
 *      Results equal hses_es_update up to the fp32 summation order. --------- */
size_t hses_es_update_static_scratch_bytes(void);
int hses_es_update_static(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                          int32_t noise_reuse, int32_t first_thread, int64_t n, int64_t n_total,
                          int32_t rank, int32_t a, int32_t b, float sigma,
                          const float* fitness /*device*/, float* grad /*device (a,b) dense*/);

/* ---- einsum_pair_fused, hyperscalees/src/oxide.rs:318-462 (kernel parameter list
 *      hyperscalees-kernels/src/einsum_pair_fused_oxide.rs:96-113), for callers that bring
 *      their own half-population factors instead of letting the library regenerate them:
 *      a_t (half, r, a) and b_t (half, r, b) with element strides of dim 0 and dim 1 given
 *      (innermost stride 1; padded row pitches allowed), row (i, j) shared by members i and
 *      i + half; scores: n = 2*half raw scores.
 *      g_raw = sum_k (s_i + s_{i+half}) a_t[k] (x) b_t[k], g_ones = 2 * sum_k a_t[k] (x) b_t[k],
 *      both (a, b) dense, overwritten (no zero-initialisation needed, no 2a <= 256 limit).
 *      Contractions of 32768 rows and more whose bases and strides are multiples of 16 bytes (r
 *      from 32 up, or a divisor of 64) and whose workspace is 256-byte aligned run on the tensor
 *      cores with fp32-equivalent three-pass fp16 products (each operand scaled by a power of two
 *      found from its largest magnitude); all others on an fp32 kernel.  Both add their split-K
 *      partial sums in a fixed order: the same inputs give the same bits on every call. -- */
size_t hses_einsum_pair_workspace_bytes(int64_t half, int32_t r, int32_t a, int32_t b);
int hses_einsum_pair(hses_ctx* ctx, hses_stream stream, const float* a_t /*device*/, int64_t a_stride0,
                     int64_t a_stride1, const float* b_t /*device*/, int64_t b_stride0, int64_t b_stride1,
                     const float* scores /*device*/, int64_t half, int32_t r, int32_t a, int32_t b,
                     float* g_raw /*device*/, float* g_ones /*device*/, void* workspace /*device*/,
                     size_t workspace_bytes);

/* ---- simple_full_update + do_update_with, eggroll.rs:331-350, 384-404, for
 *      dense (PARAM-class) leaves of `len` = rows*cols elements. ----------- */
int hses_es_update_dense(hses_ctx* ctx, hses_stream stream, uint64_t key, int32_t epoch,
                         int32_t noise_reuse, int32_t first_thread, int64_t n, int64_t n_total,
                         int32_t len, float sigma, const float* fitness /*device*/,
                         float* grad /*device*/);

/* ---- Solver::update, noiser.rs:155-224.  step is the counter value after
 *      the increment (1 on the first Adam step).  m, v may be NULL for SGD.
 *      grad_scale multiplies the gradient first (clip_by_global_norm). ----- */
typedef struct {
    int32_t kind; /* hses_solver_kind */
    float lr, beta1, beta2, eps, weight_decay;
} hses_solver;
int hses_solver_step(hses_ctx* ctx, hses_stream stream, const hses_solver* solver, int32_t step,
                     float grad_scale, float* param /*device*/, const float* grad /*device*/,
                     float* m /*device*/, float* v /*device*/, int64_t len);

/* ---- SNN population step as two calls around the (optional) fitness all-gather.
 *      The model is the reference's SnnModel / TrainableVthSnn generalised to a list of layer
 *      widths (hyperscalees-models/src/snn.rs:188-282, 388-416): per hidden layer a perturbed
 *      linear over all T steps followed by the LIF scan, then the mean firing rate, the
 *      perturbed readout and the clean out_gain.  Arrays inside hses_snn_model are HOST arrays;
 *      weights[l] are device pointers to (dims[l+1], dims[l]) matrices with weight_strides[l]. */
typedef struct {
    int32_t n_layers;              /* hidden layers + readout */
    const int32_t* dims;           /* n_layers + 1 entries: in, h1, ..., classes */
    const float* const* weights;   /* n_layers device pointers */
    const int64_t* weight_strides; /* n_layers row strides (elements) */
    const uint64_t* keys;          /* n_layers base keys (one per parameter index) */
    float out_gain;
    const float* out_gain_dev;     /* device or NULL: overrides out_gain (the (1,1) parameter tensor) */
    float tau_m;
    const float* v_th;             /* n_layers - 1 thresholds, one per hidden layer */
    int32_t reset_mode;
    const hses_factor_cache* const* caches; /* NULL, or n_layers host pointers (NULL entries allowed):
                                               factor caches the perturbed layers read instead of
                                               regenerating; hses_population_update uses an entry
                                               only when it covers the whole population */
} hses_snn_model;

typedef struct {
    int32_t T;
    int64_t n_pop;
    int32_t bm;                    /* samples per member */
    int32_t perturb;               /* 0: clean forward (iterinfo = None) */
    float sigma;
    int32_t rank;
    int32_t epoch;
    int32_t first_thread;          /* thread id of member 0 of this shard */
    int32_t noise_reuse;
} hses_pop_args;

/* spikes_in: (T, n_pop*bm, dims[0]) with row stride in_stride -> logits (n_pop*bm, classes) dense. */
size_t hses_snn_forward_workspace_bytes(const hses_snn_model* m, const hses_pop_args* p);
int hses_snn_forward(hses_ctx* ctx, hses_stream stream, const hses_snn_model* m, const hses_pop_args* p,
                     const float* spikes_in /*device*/, int64_t in_stride, float* logits /*device*/,
                     void* workspace /*device*/, size_t workspace_bytes);

/* First half of a step, the composition of hyperscalees/src/snn_mnist_train.rs:159-216 for a
 * shard of the population: Poisson-encode images (n_pop*bm, dims[0]) with the given seed words,
 * run the perturbed forward, score it (reward per sample, mean over each member's bm samples).
 * raw_fitness receives n_pop values; logits_out (optional) the (n_pop*bm, classes) logits. */
size_t hses_population_eval_workspace_bytes(const hses_snn_model* m, const hses_pop_args* p);
int hses_population_eval(hses_ctx* ctx, hses_stream stream, const hses_snn_model* m, const hses_pop_args* p,
                         const float* images /*device*/, int64_t image_stride,
                         const int32_t* labels /*device*/, const uint32_t seeds[4], int32_t reward,
                         float* raw_fitness /*device*/, float* logits_out /*device or NULL*/,
                         void* workspace /*device*/, size_t workspace_bytes);

/* Second half (snn_mnist_train.rs:218-232, EggRoll::convert_fitnesses + do_updates): z-score the
 * FULL raw fitness vector (n_total values, thread ids 0..n_total-1, after any all-gather), build
 * every layer's gradient from the regenerated noise, the dense-noise gradient of out_gain, and
 * apply one solver step in place.  params: n_layers weight matrices (dense, device, updated in
 * place) followed by the (1,1) out_gain tensor; m/v: matching moment buffers or NULL for SGD.
 * step is the solver counter after the increment. */
size_t hses_population_update_workspace_bytes(const hses_snn_model* m, int32_t rank, int64_t n_total);
int hses_population_update(hses_ctx* ctx, hses_stream stream, const hses_snn_model* m, float sigma,
                           int32_t rank, int32_t epoch, int32_t noise_reuse, int32_t group_size,
                           int32_t freeze_nonlora, uint64_t gain_key, const float* raw_fitness /*device*/,
                           int64_t n_total, const hses_solver* solver, int32_t step,
                           float* const* params /*host array of device pointers*/,
                           float* const* m_bufs, float* const* v_bufs, void* workspace /*device*/,
                           size_t workspace_bytes);

/* The same second half in two calls, for ranks that split the update as well as the forward
 * pass (the reference's multi-GPU script replicates the update,
 * snn_mnist_train_multi_gpu.py:225-234; this is the partial-sum alternative): hses_population_grads z-scores the FULL fitness vector and
 * writes the gradient contribution of members first_thread .. first_thread+n_local-1 (whole
 * pairs) of every parameter, scaled for a population of n_total, into `grads` — the weight
 * matrices back to back in layer order, dense, then one float for out_gain
 * (hses_population_grads_elems() floats).  The caller sums `grads` over the ranks (one
 * all-reduce) and hands the sum to hses_population_apply, which runs the solver step on every
 * parameter.  With first_thread = 0 and n_local = n_total the pair equals
 * hses_population_update. */
size_t hses_population_grads_elems(const hses_snn_model* m);
int hses_population_grads(hses_ctx* ctx, hses_stream stream, const hses_snn_model* m, float sigma,
                          int32_t rank, int32_t epoch, int32_t noise_reuse, int32_t group_size,
                          int32_t freeze_nonlora, uint64_t gain_key,
                          const float* raw_fitness /*device, n_total*/, int64_t n_total,
                          int32_t first_thread, int64_t n_local, float* grads /*device*/,
                          void* workspace /*device, hses_population_update_workspace_bytes()*/,
                          size_t workspace_bytes);
int hses_population_apply(hses_ctx* ctx, hses_stream stream, const hses_snn_model* m,
                          const hses_solver* solver, int32_t step, float* const* params /*device*/,
                          float* const* m_bufs, float* const* v_bufs, const float* grads /*device*/);

/* ---- rwkv7_inner_loop, hyperscalees-models/src/llm.rs:235-296, for a batch of sequences.
 *      r, w, k, v, a, b, out: (n_seq, T, H, S) dense; state (n_seq, H, S, S) is read and left
 *      holding the final state; new_starts (n_seq, T) bytes or NULL zeroes the state before a
 *      step.  S is 32 or 64. ------------------------------------------------------------ */
int hses_wkv7(hses_ctx* ctx, hses_stream stream, const float* r, const float* w, const float* k,
              const float* v, const float* a, const float* b, const uint8_t* new_starts /*device or NULL*/,
              int64_t n_seq, int32_t T, int32_t H, int32_t S, float* state, float* out);

/* ---- spiking self-attention core on firing rates (src/hyperscalees/models/snn_self_attention.py:45-98;
 *      the Rust port keeps a continuous variant, hyperscalees-models/src/snn_transformer.rs:80-102).
 *      Q, K, V, O: (n_seq, tokens, heads*head_dim) with row_stride; mode 0: O = (beta Q K^T) V,
 *      the spike product without softmax; mode 3: the same with a causal mask (the score of key
 *      j is zero for j > i: a token of a next-token model does not see later ones); mode 1: LIF-count row softmax (n_iter LIF steps with
 *      global inhibition g_inh); mode 2: the Rust port's continuous form — n_iter Hopfield
 *      relaxations u <- u + (1/tau_m)(-u + H - g_inh * mean_key(u)) from u = H, then a stable
 *      softmax along the keys (snn_transformer.rs:80-102).  beta_per_seq (optional): n_seq scales
 *      that replace beta, one per sequence (the per-member beta of forward_batched,
 *      snn_transformer.rs:366-371).  A_out (optional): (n_seq, heads, tokens, tokens) weights. ---------------------------------------------------------- */
int hses_spiking_attention(hses_ctx* ctx, hses_stream stream, const float* Q, const float* K, const float* V,
                           int64_t n_seq, int32_t tokens, int32_t heads, int32_t head_dim, int64_t row_stride,
                           int32_t mode, float beta, const float* beta_per_seq /*device or NULL*/, float tau_m,
                           float v_th, float g_inh, int32_t n_iter, float* O, float* A_out /*device or NULL*/);

/* ---- RWKV-7 block pieces around the recurrence, hyperscalees-models/src/llm.rs:64-213.
 *      layer_norm (64-84): per row of c values, var = E[x^2] - E[x]^2, then weight and bias.
 *      GroupNorm::forward (90-145): x (n, c, l) dense (l = 1 for the rank-2 form), statistics
 *      over the (c / groups) * l values of a group, gamma and beta per channel.
 *      token_shift_mix (192-206, and the same step of TimeMixing): out = x + (prev - x) * coef
 *      with prev the previous row (row 0: the carried state, c values) and 0 where new_starts
 *      (T bytes or NULL) marks the start of a sequence; not in place.
 *      relu_square: k = relu(x)^2 of ChannelMixing (208).  ChannelMixing::forward is
 *      token_shift_mix -> hses_perturbed_linear (key) -> relu_square -> hses_perturbed_linear
 *      (value); the new state is row length-1 of x. ------------------------------------- */
int hses_layer_norm(hses_ctx* ctx, hses_stream stream, const float* x /*device*/, int64_t rows,
                    int32_t c, const float* weight, const float* bias, float eps, float* out);
int hses_group_norm(hses_ctx* ctx, hses_stream stream, const float* x /*device*/, int64_t n, int32_t c,
                    int32_t l, int32_t groups, const float* weight, const float* bias, float eps,
                    float* out);
int hses_token_shift_mix(hses_ctx* ctx, hses_stream stream, const float* x /*device (T,c)*/, int32_t T,
                         int32_t c, const float* state /*device (c)*/,
                         const uint8_t* new_starts /*device or NULL*/, const float* coef /*device (c)*/,
                         float* out /*device (T,c)*/);
/* hses_token_shift_mix for n_mix (at most 8) coefficient vectors of one x: coefs and outs are host arrays of
 * device pointers; x and its previous rows are read once (the six mixes of TimeMixing, llm.rs:381-392). */
int hses_token_shift_mix_multi(hses_ctx* ctx, hses_stream stream, const float* x /*device (T,c)*/, int32_t T, int32_t c,
                               const float* state, const uint8_t* new_starts /*or NULL*/, int32_t n_mix,
                               const float* const* coefs /*host*/, float* const* outs /*host*/);
/* The element-wise work of TimeMixing::forward around the recurrence (llm.rs:396-440 and 462-472), all
 * tensors (rows, H*S) dense, parameters H*S values:
 *   prepare: w = -softplus(-(w0 + w_lin)) - 0.5;  v = v_raw in layer 0 (v_lin NULL), else
 *            v_raw + (v_first - v_raw) * sigmoid(v0 + v_lin);  a = sigmoid(a0 + a_lin);
 *            kk = k_raw * k_k normalised per head (L2, floor 1e-12);  k = k_raw * (k_a * (a - 1) + 1);
 *            outputs w, v, k, -kk, kk * a (the decay, value, key, a and b inputs of hses_wkv7);
 *   finish:  out = (y_norm + (sum over the head of r * k * r_k) * v) * gate.
 * Head size 32, 64 or 128; every pointer 16-byte aligned. */
int hses_rwkv_mix_prepare(hses_ctx* ctx, hses_stream stream, int64_t rows, int32_t H, int32_t S, const float* w_lin,
                          const float* v_raw, const float* v_lin /*or NULL*/, const float* v_first /*or NULL*/,
                          const float* a_lin, const float* k_raw, const float* w0, const float* v0 /*or NULL*/,
                          const float* a0, const float* k_k, const float* k_a, float* w_out, float* v_out,
                          float* k_out, float* nkk_out, float* kka_out);
int hses_rwkv_mix_finish(hses_ctx* ctx, hses_stream stream, int64_t rows, int32_t H, int32_t S, const float* y_norm,
                         const float* r, const float* k, const float* v, const float* gate, const float* r_k,
                         float* out);
int hses_relu_square(hses_ctx* ctx, hses_stream stream, const float* x /*device*/, int64_t n,
                     float* out /*device*/);
/* rate_encode, hyperscalees-models/src/snn_transformer.rs:109-116: sigmoid(gain * p / (1 + |p|)). */
int hses_rate_encode(hses_ctx* ctx, hses_stream stream, const float* p /*device*/, int64_t n, float gain,
                     float* out /*device*/);

/* ---- pieces of the token-level spiking transformer (BASELINE's next-token form of the spiking
 *      self-attention model; the reference has the LIF-coded Q/K/V of
 *      src/hyperscalees/models/snn_self_attention.py:114-131 and the block structure of
 *      hyperscalees-models/src/snn_transformer.rs:345-413, but no token embedding: do_emb is
 *      unimplemented in both noisers, src/hyperscalees/noiser/eggroll.py:93 and
 *      hyperscalees-noiser/src/eggroll.rs:943-954, whose comment gives the clean form param[x]).
 *      hses_embedding: out[row] = table[ids[row]] + A_m[ids[row], :] B_m^T + pos[row % L]; A
 *      (n, vocab, rank) already scaled by sign*sigma/sqrt(rank) and B (n, d, rank) as
 *      hses_lora_factors writes them for a parameter of shape (a = vocab, b = d); member m owns
 *      rows [m*rows_per_member, (m+1)*rows_per_member); A = B = NULL gives the clean gather, pos
 *      NULL leaves the position term out.  An id outside [0, vocab) yields a row of zeros and sets
 *      bit 15 of the context's device status word.
 *      hses_lif_rate: out[i] = (1/T) * sum of the T spikes of lif_step (snn.rs:53-65) driven by
 *      the constant current cur[i] from v = 0.
 *      hses_swish: x * sigmoid(x) (snn_transformer.rs:404).  hses_add_inplace: acc += y.
 *      hses_token_fitness: per member the mean over its seqs sequences and positions 0..L-2 of
 *      log_softmax(gain * logits[s, t])[ids[s, t+1]]; per_token (n_members*seqs*L) is scratch that
 *      ends up holding the per-position terms. ------------------------------------------------- */
int hses_embedding(hses_ctx* ctx, hses_stream stream, const int32_t* ids /*device (rows)*/, int64_t rows,
                   const float* table /*device (vocab,d)*/, int64_t table_stride, int32_t vocab, int32_t d,
                   const float* pos /*device (L,d) or NULL*/, int32_t L, const float* A /*device or NULL*/,
                   const float* B /*device or NULL*/, int32_t rank, int64_t rows_per_member,
                   float* out /*device (rows,d)*/, int64_t out_stride);
int hses_lif_rate(hses_ctx* ctx, hses_stream stream, const float* cur /*device*/, int64_t n, int32_t T,
                  float tau_m, float v_th, int32_t reset_mode, float* out /*device*/);
int hses_swish(hses_ctx* ctx, hses_stream stream, const float* x /*device*/, int64_t n, float* out /*device*/);
int hses_add_inplace(hses_ctx* ctx, hses_stream stream, float* acc /*device*/, const float* y /*device*/, int64_t n);
int hses_token_fitness(hses_ctx* ctx, hses_stream stream, const float* logits /*device (n*seqs*L, vocab)*/,
                       int64_t logits_stride, const int32_t* ids /*device (n*seqs*L)*/, int64_t n_members,
                       int32_t seqs, int32_t L, int32_t vocab, float gain, float* per_token /*device scratch*/,
                       float* fitness /*device (n_members)*/);

/* ---- collectives of the sharded population step.  The reference's product crates hold no
 *      multi-GPU code; its recipe is the Python trainer
 *      llm_experiments/snn_mnist_train_multi_gpu.py:187-234 (sharded forward, the fitness of all
 *      shards on every device, replicated update), and the only NCCL plumbing in its tree is the
 *      vendored runtime's (burn_impl/vendor/cubecl-cuda/src/compute/server.rs:277-388:
 *      comm_init_rank from a unique id, all_reduce on a stream).  These entry points give a Rust
 *      trainer the same two calls: one communicator per rank (= per process and GPU), built from
 *      a 128-byte id that rank 0 creates and hands to the others out of band; an all-gather of
 *      equally long fitness shards into thread-id order; an in-place sum of the flat gradient
 *      buffer of hses_population_grads (every rank receives the same bits, so the ranks'
 *      parameters stay identical after hses_population_apply).  Both are enqueued on the caller's
 *      stream and return at once.  NCCL is loaded at run time (libnccl.so.2, or the library the
 *      environment variable HSES_NCCL_LIBRARY names).  ctx may be NULL (no launch accounting).
 *      Failures: a call that NCCL refuses, or hses_comm_async_error() reporting a failed
 *      collective (a peer that left, a transport error), returns HSES_ERR_COMM and marks the
 *      communicator broken; every later collective on it fails at once and hses_comm_destroy
 *      aborts it instead of waiting for work that cannot finish.  A rank may leave only between
 *      steps; the others should poll hses_comm_async_error (or their own heartbeat) before the
 *      next launch. ------------------------------------------------------------------------ */
#define HSES_COMM_ID_BYTES 128
typedef struct hses_comm hses_comm;
int hses_comm_unique_id(uint8_t* id /*host, HSES_COMM_ID_BYTES*/);
int hses_comm_init(hses_ctx* ctx, const uint8_t* id /*host*/, int32_t rank, int32_t world, hses_comm** out);
int hses_comm_rank(const hses_comm* comm);
int hses_comm_world(const hses_comm* comm);
int hses_comm_async_error(hses_comm* comm);
int hses_comm_destroy(hses_comm* comm);
int hses_comm_abort(hses_comm* comm);
int hses_allgather_fitness(hses_comm* comm, hses_stream stream, const float* local /*device (n_local)*/,
                           int64_t n_local, float* all /*device (world * n_local)*/);
int hses_allreduce_grads(hses_comm* comm, hses_stream stream, float* grads /*device, in place*/, int64_t count);

/* ---- the fitness exchange without a library collective: peer memory over NVLink.
 *      Every rank owns a WINDOW of device memory (two copies of the population's raw-fitness
 *      vector, steps alternate between them, and one flag word per rank and copy) that the other
 *      ranks of the node map through a CUDA IPC handle.  hses_fitness_publish (one kernel) stores
 *      this rank's shard into every rank's window and then raises this rank's flag there with the
 *      step's tag; hses_fitness_wait (one kernel) waits until all `world` flags of its own window
 *      carry the tag and copies the vector to `out`.  The wait is bounded (about a second): when a
 *      shard does not arrive it sets bit 9 of the context's device status word, leaves `out`
 *      untouched and returns — read hses_ctx_device_status before trusting `out`.  Tags are the
 *      step number (>= 1, increasing by one); all ranks use the same tag in the same step.  Plain
 *      stores and loads only (no multicast).  world <= 16.  The reference exchanges the vector
 *      through the host (llm_experiments/snn_mnist_train_multi_gpu.py:225-234, 291). --------- */
size_t hses_peer_window_bytes(int64_t n_total);
/* allocates and clears this rank's window; `handle` (64 bytes) is what the other ranks open */
int hses_peer_alloc(hses_ctx* ctx, int64_t n_total, void** window /*device, out*/, uint8_t handle[64] /*out*/);
int hses_peer_open(hses_ctx* ctx, const uint8_t handle[64], void** window /*peer device memory, out*/);
int hses_peer_close(void* window /*from hses_peer_open*/);
int hses_peer_free(void* window /*from hses_peer_alloc*/);
/* windows: HOST array of `world` device pointers, entry r = rank r's window (own one included) */
int hses_fitness_publish(hses_ctx* ctx, hses_stream stream, const float* local /*device*/, int64_t n_local,
                         int64_t offset, int64_t n_total, void* const* windows /*host*/, int32_t rank,
                         int32_t world, uint32_t tag);
int hses_fitness_wait(hses_ctx* ctx, hses_stream stream, const void* own_window /*device*/, int64_t n_total,
                      int32_t world, uint32_t tag, float* out /*device, n_total*/);
/* both in one launch: the step's usual call (a rank's stores are under way while it waits for the others') */
int hses_fitness_exchange(hses_ctx* ctx, hses_stream stream, const float* local /*device*/, int64_t n_local,
                          int64_t offset, int64_t n_total, void* const* windows /*host*/, int32_t rank,
                          int32_t world, uint32_t tag, float* out /*device, n_total*/);

#ifdef __cplusplus
}
#endif
#endif /* HSES_H */
