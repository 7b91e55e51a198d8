// The fitness exchange of the sharded population step over peer memory (NVLink): every rank's
// kernel stores its shard of the raw-fitness vector straight into every rank's copy of the whole
// vector and then raises a flag there; a second kernel waits, with an iteration limit, until all
// shards of the step have arrived.  No library collective, no host round trip, plain stores and
// loads (no multicast), so the exchange can sit between the forward and the update on one stream.
//
// A rank's window (hses_peer_alloc) holds two copies of the vector — steps alternate between
// them, so a rank that runs ahead never writes into a copy a slower rank still reads — and one
// flag word per rank and copy.  The window is ordinary device memory shared through CUDA IPC
// handles (hses_peer_open maps a peer's window).
#include <cstring>

#include "common.cuh"

namespace hses {

namespace {

constexpr int kPeerMaxWorld = 16;
constexpr uint32_t kPeerSpin = 1u << 21;   // polls of about half a microsecond: gives up after about a second

struct PeerTable {
    float* base[kPeerMaxWorld];
};

__host__ __device__ inline size_t window_floats(int64_t n_total) { return 2 * (size_t)((n_total + 63) / 64 * 64); }

// one CTA: the shard goes to every rank's copy (16 bytes per thread and store where the alignment
// allows), then, once every thread's stores are ordered before it, the flags go up
__device__ __forceinline__ void publish_body(const PeerTable& peers, const float* __restrict__ local, int64_t n_local,
                                             int64_t offset, int64_t n_total, int rank, int world, uint32_t tag) {
    const size_t copy = (size_t)(tag & 1u) * (window_floats(n_total) / 2);
    const bool vec = ((offset | n_local) & 3) == 0 && ((uintptr_t)local & 15u) == 0;   // windows are 256-byte aligned
    for (int p = 0; p < world; ++p) {
        float* dst = peers.base[p] + copy + offset;
        if (vec) {
            for (int64_t i = threadIdx.x; i < n_local / 4; i += blockDim.x)
                reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(local)[i];
        } else {
            for (int64_t i = threadIdx.x; i < n_local; i += blockDim.x) dst[i] = local[i];
        }
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < world) {
        uint32_t* flags = reinterpret_cast<uint32_t*>(peers.base[threadIdx.x] + window_floats(n_total));
        uint32_t* f = flags + (tag & 1u) * kPeerMaxWorld + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(tag) : "memory");
    }
}

// waits until every rank's flag of this copy carries the step's tag, then copies the vector out
__device__ __forceinline__ void wait_body(const float* __restrict__ own, int64_t n_total, int world, uint32_t tag,
                                          float* __restrict__ out, int* __restrict__ status) {
    __shared__ int failed;
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    if ((int)threadIdx.x < world) {
        const uint32_t* f = reinterpret_cast<const uint32_t*>(own + window_floats(n_total)) + (tag & 1u) * kPeerMaxWorld +
                            threadIdx.x;
        bool ok = false;
        for (uint32_t i = 0; i < kPeerSpin; ++i) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (v == tag) { ok = true; break; }
            if (i > 4096) __nanosleep(500);   // the shards of a step arrive within microseconds of each other
        }
        if (!ok) {
            failed = 1;
            atomicOr(status, 1 << 9);   // bit 9: a shard of the fitness exchange did not arrive
        }
    }
    __syncthreads();
    if (failed) return;   // `out` keeps what it held: the caller reads the status before using it
    const float* src = own + (size_t)(tag & 1u) * (window_floats(n_total) / 2);
    // written by other GPUs: not through L1
    if ((n_total & 3) == 0 && ((uintptr_t)out & 15u) == 0) {
        for (int64_t i = threadIdx.x; i < n_total / 4; i += blockDim.x)
            reinterpret_cast<float4*>(out)[i] = __ldcg(reinterpret_cast<const float4*>(src) + i);
    } else {
        for (int64_t i = threadIdx.x; i < n_total; i += blockDim.x) out[i] = __ldcg(src + i);
    }
}

__global__ void __launch_bounds__(1024)
fitness_publish_kernel(PeerTable peers, const float* __restrict__ local, int64_t n_local, int64_t offset,
                       int64_t n_total, int rank, int world, uint32_t tag) {
    publish_body(peers, local, n_local, offset, n_total, rank, world, tag);
}

__global__ void __launch_bounds__(1024)
fitness_wait_kernel(const float* __restrict__ own, int64_t n_total, int world, uint32_t tag, float* __restrict__ out,
                    int* __restrict__ status) {
    wait_body(own, n_total, world, tag, out, status);
}

// both halves in one launch: a rank's stores are under way while it starts to wait for the others'
__global__ void __launch_bounds__(1024)
fitness_exchange_kernel(PeerTable peers, const float* __restrict__ local, int64_t n_local, int64_t offset,
                        int64_t n_total, int rank, int world, uint32_t tag, float* __restrict__ out,
                        int* __restrict__ status) {
    publish_body(peers, local, n_local, offset, n_total, rank, world, tag);
    wait_body(peers.base[rank], n_total, world, tag, out, status);
}

}  // namespace

}  // namespace hses

using namespace hses;

extern "C" {

size_t hses_peer_window_bytes(int64_t n_total) {
    if (n_total < 1) return 0;
    return window_floats(n_total) * sizeof(float) + 2 * kPeerMaxWorld * sizeof(uint32_t);
}

int hses_peer_alloc(hses_ctx* ctx, int64_t n_total, void** window, uint8_t handle[64]) {
    HSES_REQUIRE(ctx != nullptr && window != nullptr && handle != nullptr, "NULL pointer");
    HSES_REQUIRE(n_total >= 1, "empty population");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* p = nullptr;
    const size_t bytes = hses_peer_window_bytes(n_total);
    HSES_CUDA(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        set_error(std::string("hses_peer_alloc: ") + cudaGetErrorString(e));
        return HSES_ERR_CUDA;
    }
    memcpy(handle, &h, 64);
    *window = p;
    return HSES_OK;
}

int hses_peer_open(hses_ctx* ctx, const uint8_t handle[64], void** window) {
    HSES_REQUIRE(ctx != nullptr && window != nullptr && handle != nullptr, "NULL pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    HSES_CUDA(cudaIpcOpenMemHandle(window, h, cudaIpcMemLazyEnablePeerAccess));
    return HSES_OK;
}

int hses_peer_close(void* window) {
    if (window) HSES_CUDA(cudaIpcCloseMemHandle(window));
    return HSES_OK;
}

int hses_peer_free(void* window) {
    if (window) HSES_CUDA(cudaFree(window));
    return HSES_OK;
}

int hses_fitness_publish(hses_ctx* ctx, hses_stream stream, const float* local, int64_t n_local, int64_t offset,
                         int64_t n_total, void* const* windows, int32_t rank, int32_t world, uint32_t tag) {
    HSES_REQUIRE(ctx != nullptr && local != nullptr && windows != nullptr, "NULL pointer");
    HSES_REQUIRE(world >= 1 && world <= kPeerMaxWorld && rank >= 0 && rank < world, "bad rank or world size");
    HSES_REQUIRE(n_local >= 0 && offset >= 0 && offset + n_local <= n_total, "shard outside the population");
    HSES_REQUIRE(tag != 0, "tag 0 is the cleared state of the flags");
    PeerTable t{};
    for (int p = 0; p < world; ++p) {
        HSES_REQUIRE(windows[p] != nullptr, "NULL window");
        t.base[p] = reinterpret_cast<float*>(windows[p]);
    }
    HSES_KERNEL(ctx, as_stream(stream), "fitness_publish");
    fitness_publish_kernel<<<1, 1024, 0, as_stream(stream)>>>(t, local, n_local, offset, n_total, rank, world, tag);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_fitness_exchange(hses_ctx* ctx, hses_stream stream, const float* local, int64_t n_local, int64_t offset,
                          int64_t n_total, void* const* windows, int32_t rank, int32_t world, uint32_t tag, float* out) {
    HSES_REQUIRE(ctx != nullptr && local != nullptr && windows != nullptr && out != nullptr, "NULL pointer");
    HSES_REQUIRE(world >= 1 && world <= kPeerMaxWorld && rank >= 0 && rank < world, "bad rank or world size");
    HSES_REQUIRE(n_local >= 0 && offset >= 0 && offset + n_local <= n_total, "shard outside the population");
    HSES_REQUIRE(tag != 0, "tag 0 is the cleared state of the flags");
    PeerTable t{};
    for (int p = 0; p < world; ++p) {
        HSES_REQUIRE(windows[p] != nullptr, "NULL window");
        t.base[p] = reinterpret_cast<float*>(windows[p]);
    }
    HSES_KERNEL(ctx, as_stream(stream), "fitness_exchange");
    fitness_exchange_kernel<<<1, 1024, 0, as_stream(stream)>>>(t, local, n_local, offset, n_total, rank, world, tag, out,
                                                             ctx->t.status_word);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

int hses_fitness_wait(hses_ctx* ctx, hses_stream stream, const void* own_window, int64_t n_total, int32_t world,
                      uint32_t tag, float* out) {
    HSES_REQUIRE(ctx != nullptr && own_window != nullptr && out != nullptr, "NULL pointer");
    HSES_REQUIRE(world >= 1 && world <= kPeerMaxWorld && n_total >= 1 && tag != 0, "bad arguments");
    HSES_KERNEL(ctx, as_stream(stream), "fitness_wait");
    fitness_wait_kernel<<<1, 1024, 0, as_stream(stream)>>>(reinterpret_cast<const float*>(own_window), n_total, world, tag,
                                                         out, ctx->t.status_word);
    HSES_LAUNCH_CHECK();
    return HSES_OK;
}

}  // extern "C"
