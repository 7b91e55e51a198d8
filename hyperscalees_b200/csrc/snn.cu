// Composite entry points of the SNN population step: they only sequence the kernels of the
// other translation units on the caller's stream, with all intermediates in caller scratch.
//   forward   SnnModel::forward, hyperscalees-models/src/snn.rs:253-282 (any number of hidden layers)
//   eval      encode -> forward -> fitness, hyperscalees/src/snn_mnist_train.rs:159-216
//   update    convert_fitnesses + do_updates, hyperscalees-noiser/src/eggroll.rs:967-1005
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "linear.cuh"
#include "update_tc.cuh"

namespace hses {

namespace {

size_t up64(size_t v) { return (v + 63) / 64 * 64; }

struct FwdPlan {
    size_t rows, maxh, cur, spk, rate, half, lin_bytes, bytes;
};

hses_linear_args layer_args(const hses_snn_model* m, const hses_pop_args* p, int l, bool readout) {
    hses_linear_args g{};
    g.t_steps = readout ? 1 : p->T;
    g.n_pop = p->n_pop;
    g.bm = p->bm;
    g.k = m->dims[l];
    g.x_row_stride = m->dims[l];
    g.param = m->weights ? m->weights[l] : nullptr;
    g.a = m->dims[l + 1];
    g.param_row_stride = m->weight_strides ? m->weight_strides[l] : m->dims[l];
    g.sigma = p->sigma;
    g.rank = p->rank;
    g.key = m->keys ? m->keys[l] : 0;
    g.epoch = p->epoch;
    g.first_thread = p->first_thread;
    g.noise_reuse = p->noise_reuse;
    g.perturb = p->perturb;
    g.lif = 0;
    g.tau_m = m->tau_m;
    g.reset_mode = m->reset_mode;
    g.out_scale = readout ? m->out_gain : 1.0f;
    g.out_scale_ptr = readout ? m->out_gain_dev : nullptr;
    g.out_row_stride = m->dims[l + 1];
    g.algo = HSES_ALGO_AUTO;
    g.cache = (p->perturb && m->caches) ? m->caches[l] : nullptr;
    return g;
}

// Alignment the tensor path asks of its operands is known only with real pointers; for sizing,
// stand-ins with 16-byte alignment are used (every scratch sub-buffer is 256-byte aligned).
FwdPlan plan_forward(const hses_snn_model* m, const hses_pop_args* p) {
    FwdPlan f{};
    f.rows = (size_t)p->n_pop * p->bm;
    for (int l = 1; l < m->n_layers; ++l) f.maxh = std::max(f.maxh, (size_t)m->dims[l]);
    f.cur = up64((size_t)p->T * f.rows * f.maxh);
    f.spk = f.cur;
    f.rate = up64(f.rows * (size_t)m->dims[m->n_layers - 1]);
    for (int l = 0; l < m->n_layers; ++l) {
        hses_linear_args g = layer_args(m, p, l, l == m->n_layers - 1);
        g.x = reinterpret_cast<const float*>(0x100);
        g.param = reinterpret_cast<const float*>(0x100);
        g.out = reinterpret_cast<float*>(0x100);
        if (l == 0) g.x_row_stride = (m->dims[0] + 3) / 4 * 4;
        if (l < m->n_layers - 1) g.lif = 2;   // hidden layers run with the fused scan (same choice of path as the call)
        f.lin_bytes = std::max(f.lin_bytes, hses_perturbed_linear_workspace_bytes(&g));
        // the first layer may arrive with another pitch: leave room for the general path too
        g.algo = HSES_ALGO_SIMT;
        f.lin_bytes = std::max(f.lin_bytes, hses_perturbed_linear_workspace_bytes(&g));
    }
    f.lin_bytes = up64(f.lin_bytes);
    // hidden layers hand their spikes to the next hidden layer as fp16 as well (its tensor-core
    // operand): two buffers of half the size of a spike buffer, when there is such a hand-over
    f.half = m->n_layers > 2 ? up64((f.spk + 1) / 2) : 0;
    f.bytes = (f.cur + 2 * f.spk + f.rate + 2 * f.half) * sizeof(float) + f.lin_bytes;
    return f;
}

int check_model(const hses_snn_model* m, const hses_pop_args* p) {
    HSES_REQUIRE(m != nullptr && p != nullptr, "NULL model or arguments");
    HSES_REQUIRE(m->n_layers >= 1 && m->dims != nullptr, "bad layer list");
    for (int l = 0; l <= m->n_layers; ++l) HSES_REQUIRE(m->dims[l] >= 1, "layer width must be positive");
    HSES_REQUIRE(p->T >= 1 && p->n_pop >= 1 && p->bm >= 1, "bad population shape");
    HSES_REQUIRE(m->n_layers == 1 || m->v_th != nullptr, "v_th is NULL");
    HSES_REQUIRE(m->tau_m != 0.0f, "tau_m must be non-zero");
    return HSES_OK;
}

}  // namespace

}  // namespace hses

using namespace hses;

extern "C" {

size_t hses_snn_forward_workspace_bytes(const hses_snn_model* m, const hses_pop_args* p) {
    if (check_model(m, p) != HSES_OK) return 0;
    return plan_forward(m, p).bytes;
}

// spikes_half: optional dense fp16 copy of the input spikes (T*rows, in) for the first layer's
// tensor-core product.
static int snn_forward_impl(hses_ctx* ctx, hses_stream stream, const hses_snn_model* m, const hses_pop_args* p,
                            const float* spikes_in, int64_t in_stride, const void* spikes_half, float* logits,
                            void* workspace, size_t workspace_bytes) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    int rc = check_model(m, p);
    if (rc != HSES_OK) return rc;
    HSES_REQUIRE(m->weights != nullptr && m->weight_strides != nullptr, "weights are NULL");
    HSES_REQUIRE(!p->perturb || m->keys != nullptr, "keys are NULL");
    HSES_REQUIRE(spikes_in != nullptr && logits != nullptr, "NULL pointer");
    HSES_REQUIRE(in_stride >= m->dims[0], "in_stride smaller than the input width");
    FwdPlan f = plan_forward(m, p);
    HSES_REQUIRE(workspace != nullptr && workspace_bytes >= f.bytes && ((uintptr_t)workspace & 255u) == 0,
                 "workspace too small or not 256-byte aligned; see hses_snn_forward_workspace_bytes");
    float* cur = reinterpret_cast<float*>(workspace);
    float* spk[2] = {cur + f.cur, cur + f.cur + f.spk};
    float* rate = cur + f.cur + 2 * f.spk;
    float* half_buf[2] = {rate + f.rate, rate + f.rate + f.half};
    void* lin_ws = rate + f.rate + 2 * f.half;

    const float* layer_in = spikes_in;
    int64_t layer_in_stride = in_stride;
    const int L = m->n_layers;
    const void* next_half = nullptr;
    for (int l = 0; l < L - 1; ++l) {
        hses_linear_args g = layer_args(m, p, l, false);
        g.x = layer_in;
        g.x_row_stride = layer_in_stride;
        if (l == 0) g.x_half = spikes_half;
        // a hidden layer that feeds another hidden layer writes its spikes as fp16 too, and the
        // layer after it takes that copy as the operand of its tensor-core product
        const void* in_half = l > 0 ? next_half : nullptr;
        if (l > 0) g.x_half = in_half;
        next_half = nullptr;
        if (l + 1 < L - 1 && m->dims[l + 1] % 8 == 0 && f.half) {
            // only when the next layer's clean product is the unperturbed tensor-core one (the per-pair
            // path's first launch, or a clean forward): the other kernels read the f32 spikes
            hses_linear_args n = layer_args(m, p, l + 1, false);
            n.x = spk[l & 1];
            n.out = spk[(l + 1) & 1];
            n.lif = 2;
            hses_linear_args nc = n;
            nc.perturb = 0;
            nc.lif = 0;
            const bool clean_tc = tensor_path_supports(nc);
            const bool wants = n.perturb ? (!tensor_path_supports(n) && pair_path_supports(n) && clean_tc) : clean_tc;
            if (wants) {
                g.out_half = half_buf[l & 1];
                next_half = half_buf[l & 1];
            }
        }
        // currents and the LIF scan over the T steps in one call: the per-pair path finishes the scan
        // inside its kernel (the currents never reach memory), the other paths scan `out` in place
        float* out_spk = spk[l & 1];
        g.out = out_spk;
        g.lif = 2;
        g.v_th = m->v_th[l];
        g.workspace = lin_ws;
        g.workspace_bytes = f.lin_bytes;
        rc = hses_perturbed_linear(ctx, stream, &g);
        if (rc != HSES_OK) return rc;
        layer_in = out_spk;
        layer_in_stride = m->dims[l + 1];
    }
    const float* readout_in = layer_in;
    int64_t readout_stride = layer_in_stride;
    hses_pop_args pr = *p;
    if (L > 1) {
        // mean firing rate over T (snn.rs:278); a model without hidden layers reads the input of step 0..T-1 averaged
        rc = hses_time_mean(ctx, stream, layer_in, p->T, (int64_t)f.rows, m->dims[L - 1], layer_in_stride, rate,
                            m->dims[L - 1]);
        if (rc != HSES_OK) return rc;
        readout_in = rate;
        readout_stride = m->dims[L - 1];
    } else {
        rc = hses_time_mean(ctx, stream, spikes_in, p->T, (int64_t)f.rows, m->dims[0], in_stride, rate, m->dims[0]);
        if (rc != HSES_OK) return rc;
        readout_in = rate;
        readout_stride = m->dims[0];
    }
    hses_linear_args g = layer_args(m, &pr, L - 1, true);
    g.x = readout_in;
    g.x_row_stride = readout_stride;
    g.out = logits;
    g.workspace = lin_ws;
    g.workspace_bytes = f.lin_bytes;
    return hses_perturbed_linear(ctx, stream, &g);
}

int hses_snn_forward(hses_ctx* ctx, hses_stream stream, const hses_snn_model* m, const hses_pop_args* p,
                     const float* spikes_in, int64_t in_stride, float* logits, void* workspace,
                     size_t workspace_bytes) {
    return snn_forward_impl(ctx, stream, m, p, spikes_in, in_stride, nullptr, logits, workspace, workspace_bytes);
}

// The encoder can hand the first layer an fp16 copy of the spikes when a dense fp16 row is a
// valid tensor-map row (16-byte pitch) and a valid vector store of the encoder.
static bool eval_writes_half(const hses_snn_model* m) { return m->n_layers > 1 && m->dims[0] % 8 == 0; }

size_t hses_population_eval_workspace_bytes(const hses_snn_model* m, const hses_pop_args* p) {
    if (check_model(m, p) != HSES_OK) return 0;
    FwdPlan f = plan_forward(m, p);
    size_t in_stride = (size_t)(m->dims[0] + 3) / 4 * 4;
    size_t extra = up64((size_t)p->T * f.rows * in_stride) + up64(f.rows * (size_t)m->dims[m->n_layers]) +
                   up64(f.rows);
    size_t half = eval_writes_half(m) ? up64((size_t)p->T * f.rows * m->dims[0] / 2) : 0;   // in floats
    return f.bytes + (extra + half) * sizeof(float);
}

int hses_population_eval(hses_ctx* ctx, hses_stream stream, const hses_snn_model* m, const hses_pop_args* p,
                         const float* images, int64_t image_stride, const int32_t* labels,
                         const uint32_t seeds[4], int32_t reward, float* raw_fitness, float* logits_out,
                         void* workspace, size_t workspace_bytes) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    int rc = check_model(m, p);
    if (rc != HSES_OK) return rc;
    HSES_REQUIRE(images != nullptr && labels != nullptr && raw_fitness != nullptr && seeds != nullptr,
                 "NULL pointer");
    size_t need = hses_population_eval_workspace_bytes(m, p);
    HSES_REQUIRE(workspace != nullptr && workspace_bytes >= need && ((uintptr_t)workspace & 255u) == 0,
                 "workspace too small or not 256-byte aligned; see hses_population_eval_workspace_bytes");
    FwdPlan f = plan_forward(m, p);
    const int in = m->dims[0], classes = m->dims[m->n_layers];
    // the encoder writes with the pitch of its input; a dense copy of the images would cost a pass,
    // so the spike buffer simply takes the image pitch when it fits the reserved width
    size_t reserved = (size_t)(in + 3) / 4 * 4;
    HSES_REQUIRE((size_t)image_stride <= reserved || image_stride == in,
                 "image row stride must be the input width or its 4-element round-up");
    uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
    float* spikes = reinterpret_cast<float*>(base + f.bytes);
    float* logits = spikes + up64((size_t)p->T * f.rows * reserved);
    float* per_sample = logits + up64(f.rows * (size_t)classes);
    // the encoder writes the spikes twice in one pass: f32 (the layout every path reads) and, when
    // the first layer's tensor-core product can take it, fp16 as that product's operand
    void* spikes_half = eval_writes_half(m) ? static_cast<void*>(per_sample + up64(f.rows)) : nullptr;
    rc = hses_poisson_encode_dual(ctx, stream, images, (int64_t)f.rows, in, image_stride, p->T, seeds, spikes,
                                  spikes_half);
    if (rc != HSES_OK) return rc;
    float* lg = logits_out ? logits_out : logits;
    rc = snn_forward_impl(ctx, stream, m, p, spikes, image_stride, spikes_half, lg, workspace, f.bytes);
    if (rc != HSES_OK) return rc;
    rc = hses_fitness(ctx, stream, lg, (int64_t)f.rows, classes, labels, reward, per_sample);
    if (rc != HSES_OK) return rc;
    return hses_member_mean(ctx, stream, per_sample, p->n_pop, p->bm, raw_fitness);
}

size_t hses_population_update_workspace_bytes(const hses_snn_model* m, int32_t rank, int64_t n_total) {
    if (m == nullptr || m->n_layers < 1 || m->dims == nullptr || n_total < 2) return 0;
    size_t grad = 0, upd = 0;
    for (int l = 0; l < m->n_layers; ++l) {
        grad = std::max(grad, (size_t)m->dims[l + 1] * m->dims[l]);
        upd = std::max(upd, hses_es_update_workspace_bytes(m->dims[l + 1], m->dims[l], rank, n_total));
    }
    return (up64((size_t)n_total) + up64(grad)) * sizeof(float) + up64(upd);
}

int hses_population_update(hses_ctx* ctx, hses_stream stream, const hses_snn_model* m, float sigma, int32_t rank,
                           int32_t epoch, int32_t noise_reuse, int32_t group_size, int32_t freeze_nonlora,
                           uint64_t gain_key, const float* raw_fitness, int64_t n_total,
                           const hses_solver* solver, int32_t step, float* const* params, float* const* m_bufs,
                           float* const* v_bufs, void* workspace, size_t workspace_bytes) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(m != nullptr && m->n_layers >= 1 && m->dims != nullptr && m->keys != nullptr, "bad model");
    HSES_REQUIRE(raw_fitness != nullptr && solver != nullptr && params != nullptr, "NULL pointer");
    HSES_REQUIRE(n_total >= 2 && n_total % 2 == 0, "the population must consist of whole antithetic pairs");
    size_t need = hses_population_update_workspace_bytes(m, rank, n_total);
    HSES_REQUIRE(workspace != nullptr && workspace_bytes >= need && ((uintptr_t)workspace & 255u) == 0,
                 "workspace too small or not 256-byte aligned; see hses_population_update_workspace_bytes");
    size_t grad_elems = 0;
    for (int l = 0; l < m->n_layers; ++l) grad_elems = std::max(grad_elems, (size_t)m->dims[l + 1] * m->dims[l]);
    float* fit = reinterpret_cast<float*>(workspace);
    float* grad = fit + up64((size_t)n_total);
    void* upd_ws = grad + up64(grad_elems);
    size_t upd_bytes = workspace_bytes - (up64((size_t)n_total) + up64(grad_elems)) * sizeof(float);
    int rc = hses_convert_fitnesses(ctx, stream, raw_fitness, n_total, group_size, fit, nullptr);
    if (rc != HSES_OK) return rc;
    const bool moments = solver->kind != HSES_SGD;
    HSES_REQUIRE(!moments || (m_bufs != nullptr && v_bufs != nullptr), "Adam needs moment buffers");
    bool range_valid = false;
    for (int l = 0; l < m->n_layers; ++l) {
        int a = m->dims[l + 1], b = m->dims[l];
        hses_update_args u{};
        u.key = m->keys[l];
        u.epoch = epoch;
        u.noise_reuse = noise_reuse;
        u.first_thread = 0;
        u.n = n_total;
        u.n_total = n_total;
        u.rank = rank;
        u.a = a;
        u.b = b;
        u.sigma = sigma;
        u.fitness = fit;
        u.grad = grad;
        u.workspace = upd_ws;
        u.workspace_bytes = upd_bytes;
        u.mode = HSES_UPDATE_GRAD;
        const hses_factor_cache* c = m->caches ? m->caches[l] : nullptr;
        if (c && c->first_pair == 0 && c->n_pairs >= n_total / 2) u.cache = c;
        // the layers share the fitness vector and the workspace: the pair-weight range that the
        // first tensor-core layer leaves at the start of the workspace serves the following ones
        bool took_tc = false;
        rc = es_update_ex_impl(ctx, stream, &u, range_valid, &took_tc);
        if (rc != HSES_OK) return rc;
        range_valid = took_tc;
        rc = hses_solver_step(ctx, stream, solver, step, 1.0f, params[l], grad, moments ? m_bufs[l] : nullptr,
                              moments ? v_bufs[l] : nullptr, (int64_t)a * b);
        if (rc != HSES_OK) return rc;
    }
    // out_gain: PARAM-class leaf of shape (1,1), dense noise (eggroll.rs:331-350); frozen -> zero gradient
    if (params[m->n_layers] != nullptr) {
        if (freeze_nonlora) {
            HSES_CUDA(cudaMemsetAsync(grad, 0, sizeof(float), as_stream(stream)));
        } else {
            rc = hses_es_update_dense(ctx, stream, gain_key, epoch, noise_reuse, 0, n_total, n_total, 1, sigma, fit,
                                      grad);
            if (rc != HSES_OK) return rc;
        }
        rc = hses_solver_step(ctx, stream, solver, step, 1.0f, params[m->n_layers], grad,
                              moments ? m_bufs[m->n_layers] : nullptr, moments ? v_bufs[m->n_layers] : nullptr, 1);
        if (rc != HSES_OK) return rc;
    }
    return HSES_OK;
}

size_t hses_population_grads_elems(const hses_snn_model* m) {
    if (m == nullptr || m->n_layers < 1 || m->dims == nullptr) return 0;
    size_t n = 1;  // out_gain
    for (int l = 0; l < m->n_layers; ++l) n += (size_t)m->dims[l + 1] * m->dims[l];
    return n;
}

int hses_population_grads(hses_ctx* ctx, hses_stream stream, const hses_snn_model* m, float sigma, int32_t rank,
                          int32_t epoch, int32_t noise_reuse, int32_t group_size, int32_t freeze_nonlora,
                          uint64_t gain_key, const float* raw_fitness, int64_t n_total, int32_t first_thread,
                          int64_t n_local, float* grads, void* workspace, size_t workspace_bytes) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(m != nullptr && m->n_layers >= 1 && m->dims != nullptr && m->keys != nullptr, "bad model");
    HSES_REQUIRE(raw_fitness != nullptr && grads != nullptr, "NULL pointer");
    HSES_REQUIRE(n_total >= 2 && n_total % 2 == 0, "the population must consist of whole antithetic pairs");
    HSES_REQUIRE(first_thread >= 0 && first_thread % 2 == 0 && n_local >= 2 && n_local % 2 == 0 &&
                     (int64_t)first_thread + n_local <= n_total,
                 "the shard must consist of whole antithetic pairs inside the population");
    size_t need = hses_population_update_workspace_bytes(m, rank, n_total);
    HSES_REQUIRE(workspace != nullptr && workspace_bytes >= need && ((uintptr_t)workspace & 255u) == 0,
                 "workspace too small or not 256-byte aligned; see hses_population_update_workspace_bytes");
    size_t grad_elems = 0;
    for (int l = 0; l < m->n_layers; ++l) grad_elems = std::max(grad_elems, (size_t)m->dims[l + 1] * m->dims[l]);
    float* fit = reinterpret_cast<float*>(workspace);
    void* upd_ws = fit + up64((size_t)n_total) + up64(grad_elems);
    size_t upd_bytes = workspace_bytes - (up64((size_t)n_total) + up64(grad_elems)) * sizeof(float);
    int rc = hses_convert_fitnesses(ctx, stream, raw_fitness, n_total, group_size, fit, nullptr);
    if (rc != HSES_OK) return rc;
    float* g = grads;
    bool range_valid = false;
    for (int l = 0; l < m->n_layers; ++l) {
        int a = m->dims[l + 1], b = m->dims[l];
        hses_update_args u{};
        u.key = m->keys[l];
        u.epoch = epoch;
        u.noise_reuse = noise_reuse;
        u.first_thread = first_thread;
        u.n = n_local;
        u.n_total = n_total;
        u.rank = rank;
        u.a = a;
        u.b = b;
        u.sigma = sigma;
        u.fitness = fit + first_thread;
        u.grad = g;
        u.workspace = upd_ws;
        u.workspace_bytes = upd_bytes;
        u.mode = HSES_UPDATE_GRAD;
        const hses_factor_cache* c = m->caches ? m->caches[l] : nullptr;
        if (c && c->first_pair <= first_thread / 2 &&
            (int64_t)c->first_pair + c->n_pairs >= (int64_t)first_thread / 2 + n_local / 2)
            u.cache = c;
        bool took_tc = false;
        rc = es_update_ex_impl(ctx, stream, &u, range_valid, &took_tc);
        if (rc != HSES_OK) return rc;
        range_valid = took_tc;
        g += (size_t)a * b;
    }
    // out_gain: PARAM-class leaf of shape (1,1), dense noise (eggroll.rs:331-350); frozen -> zero gradient
    if (freeze_nonlora) {
        HSES_CUDA(cudaMemsetAsync(g, 0, sizeof(float), as_stream(stream)));
    } else {
        rc = hses_es_update_dense(ctx, stream, gain_key, epoch, noise_reuse, first_thread, n_local, n_total, 1, sigma,
                                  fit + first_thread, g);
        if (rc != HSES_OK) return rc;
    }
    return HSES_OK;
}

int hses_population_apply(hses_ctx* ctx, hses_stream stream, const hses_snn_model* m, const hses_solver* solver,
                          int32_t step, float* const* params, float* const* m_bufs, float* const* v_bufs,
                          const float* grads) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(m != nullptr && m->n_layers >= 1 && m->dims != nullptr, "bad model");
    HSES_REQUIRE(solver != nullptr && params != nullptr && grads != nullptr, "NULL pointer");
    const bool moments = solver->kind != HSES_SGD;
    HSES_REQUIRE(!moments || (m_bufs != nullptr && v_bufs != nullptr), "Adam needs moment buffers");
    // every leaf in one launch: the step's cost is launches, not arithmetic
    std::vector<int64_t> lens((size_t)m->n_layers + 1);
    for (int l = 0; l <= m->n_layers; ++l) lens[l] = l < m->n_layers ? (int64_t)m->dims[l + 1] * m->dims[l] : 1;
    return solver_step_multi(ctx, as_stream(stream), solver, step, m->n_layers + 1, params, m_bufs, v_bufs,
                             lens.data(), grads);
}

}  // extern "C"
