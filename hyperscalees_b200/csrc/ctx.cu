// Context management: error strings, generator jump tables, libm calibration.
#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "calib.hpp"
#include "common.cuh"

namespace hses {

static thread_local std::string g_last_error;
void set_error(const std::string& msg) { g_last_error = msg; }

KernelStat& Profiler::get(const char* name) {
    for (auto& k : stats)
        if (k.name == name || strcmp(k.name, name) == 0) return k;
    stats.reserve(64);  // KernelStat references stay valid for the few dozen kernels that exist
    stats.emplace_back();
    stats.back().name = name;
    return stats.back();
}
cudaEvent_t Profiler::event() {
    if (!pool.empty()) {
        cudaEvent_t e = pool.back();
        pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

// ---------------------------------------------------------------------------
// xorshift64 as a linear map on GF(2)^64 (noiser.rs:449-455): column j of a
// matrix is the image of the state with only bit j set.
// ---------------------------------------------------------------------------
struct BitMat {
    uint64_t col[64];
    uint64_t apply(uint64_t x) const {
        uint64_t r = 0;
        for (int j = 0; j < 64; ++j)
            if ((x >> j) & 1) r ^= col[j];
        return r;
    }
};
static BitMat step_matrix() {
    BitMat m;
    for (int j = 0; j < 64; ++j) m.col[j] = xs64_step(1ull << j);
    return m;
}
static BitMat compose(const BitMat& a, const BitMat& b) {  // a after b
    BitMat m;
    for (int j = 0; j < 64; ++j) m.col[j] = a.apply(b.col[j]);
    return m;
}
static void nibble_table(const BitMat& m, uint64_t* tab /* kJumpWords */) {
    for (int p = 0; p < 16; ++p)
        for (int v = 0; v < 16; ++v) tab[p * 16 + v] = m.apply((uint64_t)v << (4 * p));
}

// ---------------------------------------------------------------------------
// calibration kernel: rounded candidates for every 24-bit uniform
// ---------------------------------------------------------------------------
__global__ void candidates_kernel(const double2* __restrict__ log_tab, int which,
                                  uint32_t* __restrict__ bits, uint32_t* __restrict__ code) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= kUnits) return;
    Rounded r;
    if (which == 0) {
        if (i == 0) { bits[0] = 0; code[0] = 0; return; }
        r = round_candidate(log_candidate(i, log_tab));
    } else {
        float theta = fmul(kTauF, (float)i * 5.9604644775390625e-08f);
        r = round_candidate(cos_candidate(theta));
    }
    bits[i] = r.bits;
    code[i] = r.dist | ((r.alt < r.bits) ? 0x80000000u : 0u);
}

int plan_sm_count() {
    static int cached = 0;
    if (cached > 0) return cached;
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
        cached = n;
    else
        return 148;  // no device visible (size queries on a host without a GPU): the B200's count
    return cached;
}

static std::mutex g_tables_mutex;
static std::map<int, std::shared_ptr<DeviceTables>> g_tables;

// host copies of T^(2^k) and the per-device cache of composed hop tables
static std::vector<BitMat> g_pow2_host;
static std::mutex g_hop_mutex;
static std::map<std::pair<int, uint64_t>, uint64_t*> g_hop_tables;

static void ensure_pow2_host() {
    if (!g_pow2_host.empty()) return;
    BitMat m = step_matrix();
    for (int k = 0; k < kJumpLevels; ++k) {
        g_pow2_host.push_back(m);
        m = compose(m, m);
    }
}

int get_hop_table(hses_ctx* ctx, uint64_t distance, const uint64_t** dev_tab) {
    std::lock_guard<std::mutex> lock(g_hop_mutex);
    auto key = std::make_pair(ctx->device, distance);
    auto it = g_hop_tables.find(key);
    if (it != g_hop_tables.end()) {
        *dev_tab = it->second;
        return HSES_OK;
    }
    HSES_REQUIRE(distance < (1ull << kJumpLevels), "hop distance too large");
    ensure_pow2_host();
    BitMat m;
    for (int j = 0; j < 64; ++j) m.col[j] = 1ull << j;  // identity
    for (int k = 0; k < kJumpLevels; ++k)
        if ((distance >> k) & 1) m = compose(g_pow2_host[k], m);
    uint64_t host[kJumpWords];
    nibble_table(m, host);
    uint64_t* dev = nullptr;
    HSES_CUDA(cudaMalloc(&dev, sizeof(host)));
    HSES_CUDA(cudaMemcpy(dev, host, sizeof(host), cudaMemcpyHostToDevice));
    g_hop_tables[key] = dev;
    *dev_tab = dev;
    return HSES_OK;
}

static int build_tables(DeviceTables& t) {
    // log helper table
    double host_tab[128];
    build_log_table(host_tab);
    HSES_CUDA(cudaMalloc(&t.log_tab, sizeof(host_tab)));
    HSES_CUDA(cudaMemcpy(t.log_tab, host_tab, sizeof(host_tab), cudaMemcpyHostToDevice));

    HSES_CUDA(cudaMalloc(&t.status_word, sizeof(int)));
    HSES_CUDA(cudaMemset(t.status_word, 0, sizeof(int)));

    // jump tables T^(2^k)
    {
        std::vector<uint64_t> host((size_t)kJumpLevels * kJumpWords);
        BitMat m = step_matrix();
        for (int k = 0; k < kJumpLevels; ++k) {
            nibble_table(m, host.data() + (size_t)k * kJumpWords);
            m = compose(m, m);
        }
        HSES_CUDA(cudaMalloc(&t.jump_pow2, host.size() * sizeof(uint64_t)));
        HSES_CUDA(cudaMemcpy(t.jump_pow2, host.data(), host.size() * sizeof(uint64_t),
                             cudaMemcpyHostToDevice));
    }

    // candidates on the device, libm on the host
    uint32_t *d_bits = nullptr, *d_code = nullptr;
    HSES_CUDA(cudaMalloc(&d_bits, (size_t)kUnits * 4));
    HSES_CUDA(cudaMalloc(&d_code, (size_t)kUnits * 4));
    std::vector<uint32_t> h_bits(kUnits), h_code(kUnits);
    CalibResult res[2];
    for (int which = 0; which < 2; ++which) {
        candidates_kernel<<<kUnits / 256, 256>>>(t.log_tab, which, d_bits, d_code);
        HSES_LAUNCH_CHECK();
        HSES_CUDA(cudaMemcpy(h_bits.data(), d_bits, (size_t)kUnits * 4, cudaMemcpyDeviceToHost));
        HSES_CUDA(cudaMemcpy(h_code.data(), d_code, (size_t)kUnits * 4, cudaMemcpyDeviceToHost));
        if (which == 0)
            calibrate(h_bits.data(), h_code.data(), 1u, host_logf_u24, res[0]);
        else
            calibrate(h_bits.data(), h_code.data(), 0u, host_cosf_u24, res[1]);
        if (!res[which].error.empty()) {
            set_error(res[which].error);
            cudaFree(d_bits);
            cudaFree(d_code);
            return HSES_ERR_CALIBRATION;
        }
    }
    HSES_CUDA(cudaFree(d_bits));
    HSES_CUDA(cudaFree(d_code));

    uint32_t** flips[2] = {&t.log_flip, &t.cos_flip};
    uint32_t** deltas[2] = {&t.log_delta, &t.cos_delta};
    for (int which = 0; which < 2; ++which) {
        HSES_CUDA(cudaMalloc(flips[which], (size_t)kUnits / 8));
        HSES_CUDA(cudaMemcpy(*flips[which], res[which].flip.data(), (size_t)kUnits / 8,
                             cudaMemcpyHostToDevice));
        HSES_CUDA(cudaMalloc(deltas[which], 256 * 4));
        HSES_CUDA(cudaMemcpy(*deltas[which], res[which].delta, 256 * 4, cudaMemcpyHostToDevice));
    }
    t.n_log_flips = res[0].n_flips;
    t.n_cos_flips = res[1].n_flips;
    t.log_of_zero = logf(1e-9f);
    return HSES_OK;
}

}  // namespace hses

using namespace hses;

extern "C" {

const char* hses_last_error(void) { return g_last_error.c_str(); }
int hses_version(void) { return 1; }

uint64_t hses_noise_seed(uint64_t key, int32_t true_epoch, int32_t true_thread) {
    return noise_seed(key, true_epoch, true_thread);
}

int hses_ctx_create(int device, hses_ctx** out) {
    HSES_REQUIRE(out != nullptr, "out is NULL");
    *out = nullptr;
    int count = 0;
    HSES_CUDA(cudaGetDeviceCount(&count));
    HSES_REQUIRE(device >= 0 && device < count, "no such CUDA device");
    HSES_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    HSES_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("hses_ctx_create: this library is built for sm_100a only; device is sm_" +
                  std::to_string(prop.major) + std::to_string(prop.minor));
        return HSES_ERR_UNSUPPORTED;
    }
    std::shared_ptr<DeviceTables> tables;
    {
        std::lock_guard<std::mutex> lock(g_tables_mutex);
        auto it = g_tables.find(device);
        if (it == g_tables.end()) {
            auto fresh = std::make_shared<DeviceTables>();
            int rc = build_tables(*fresh);
            if (rc != HSES_OK) return rc;
            g_tables[device] = fresh;
            tables = fresh;
        } else {
            tables = it->second;
        }
    }
    hses_ctx* ctx = new hses_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->t = *tables;  // device pointers are shared; the cache keeps them alive
    *out = ctx;
    return HSES_OK;
}

int hses_ctx_destroy(hses_ctx* ctx) {
    delete ctx;
    return HSES_OK;
}

int hses_ctx_device_status(hses_ctx* ctx, int* status) {
    HSES_REQUIRE(ctx != nullptr && status != nullptr, "NULL pointer");
    HSES_CUDA(cudaMemcpy(status, ctx->t.status_word, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status != 0) HSES_CUDA(cudaMemset(ctx->t.status_word, 0, sizeof(int)));
    return HSES_OK;
}

int hses_profile_enable(hses_ctx* ctx, int timing) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    for (auto& k : ctx->prof.stats) {
        for (auto& pr : k.pending) {
            cudaEventSynchronize(pr.second);
            ctx->prof.pool.push_back(pr.first);
            ctx->prof.pool.push_back(pr.second);
        }
        k.pending.clear();
        k.launches = 0;
        k.ms = 0.0;
    }
    ctx->prof.timing = timing != 0;
    return HSES_OK;
}

int hses_profile_count(hses_ctx* ctx) { return ctx ? (int)ctx->prof.stats.size() : 0; }

int hses_profile_read(hses_ctx* ctx, int index, const char** name, int64_t* launches,
                      double* total_ms) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    HSES_REQUIRE(index >= 0 && index < (int)ctx->prof.stats.size(), "index out of range");
    KernelStat& k = ctx->prof.stats[index];
    for (auto& pr : k.pending) {
        HSES_CUDA(cudaEventSynchronize(pr.second));
        float ms = 0.0f;
        HSES_CUDA(cudaEventElapsedTime(&ms, pr.first, pr.second));
        k.ms += ms;
        ctx->prof.pool.push_back(pr.first);
        ctx->prof.pool.push_back(pr.second);
    }
    k.pending.clear();
    if (name) *name = k.name;
    if (launches) *launches = k.launches;
    if (total_ms) *total_ms = k.ms;
    return HSES_OK;
}

int hses_ctx_calibration_info(const hses_ctx* ctx, uint64_t* log_flips, uint64_t* cos_flips) {
    HSES_REQUIRE(ctx != nullptr, "ctx is NULL");
    if (log_flips) *log_flips = ctx->t.n_log_flips;
    if (cos_flips) *cos_flips = ctx->t.n_cos_flips;
    return HSES_OK;
}

}  // extern "C"
