// Collectives of the sharded population step behind the C ABI: one communicator per rank,
// an all-gather of the raw fitness shards and an in-place sum of the flat gradient buffer,
// both enqueued on the caller's stream.  The population step has no other exchange: every
// rank regenerates its own members' noise from (key, epoch, thread id), the rule of the
// reference's multi-GPU recipe (llm_experiments/snn_mnist_train_multi_gpu.py:187-234).
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy the process already holds when
// there is one), through the handful of public entry points declared below, so the library
// has no link-time dependency on it and a host process with its own NCCL keeps a single copy.
// HSES_NCCL_LIBRARY names another shared object with the same entry points (the CPU tests use
// a stand-in whose calls can be made to fail).
#include <dlfcn.h>
#include <stdlib.h>

#include <mutex>

#include "common.cuh"

namespace hses {
namespace {

// The public NCCL ABI used here (nccl.h): result codes, the 128-byte unique id, the float
// data type and the sum operator.
typedef int nccl_result_t;  // 0 = ncclSuccess, 7 = ncclInProgress
typedef struct { char internal[128]; } nccl_unique_id;
typedef void* nccl_comm_t;
constexpr int kNcclFloat32 = 7;
constexpr int kNcclSum = 0;

struct NcclApi {
    void* handle = nullptr;
    nccl_result_t (*GetUniqueId)(nccl_unique_id*) = nullptr;
    nccl_result_t (*CommInitRank)(nccl_comm_t*, int, nccl_unique_id, int) = nullptr;
    nccl_result_t (*CommDestroy)(nccl_comm_t) = nullptr;
    nccl_result_t (*CommAbort)(nccl_comm_t) = nullptr;
    nccl_result_t (*CommGetAsyncError)(nccl_comm_t, nccl_result_t*) = nullptr;
    nccl_result_t (*AllGather)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t) = nullptr;
    nccl_result_t (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(nccl_result_t) = nullptr;
    std::string error;
};

std::mutex g_api_mutex;
NcclApi g_api;

int load_api() {
    std::lock_guard<std::mutex> lock(g_api_mutex);
    if (g_api.handle) return HSES_OK;
    const char* override_path = getenv("HSES_NCCL_LIBRARY");
    void* h = nullptr;
    if (override_path && *override_path) {
        h = dlopen(override_path, RTLD_NOW | RTLD_LOCAL);
    } else {
        h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy already in the process, if any
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    }
    if (!h) {
        const char* e = dlerror();
        set_error(std::string("NCCL could not be loaded: ") + (e ? e : "unknown error"));
        return HSES_ERR_UNSUPPORTED;
    }
    NcclApi api;
    api.handle = h;
#define HSES_SYM(field, name)                                                        \
    *reinterpret_cast<void**>(&api.field) = dlsym(h, name);                           \
    if (!api.field) {                                                                 \
        set_error(std::string("NCCL library lacks ") + name);                         \
        dlclose(h);                                                                   \
        return HSES_ERR_UNSUPPORTED;                                                  \
    }
    HSES_SYM(GetUniqueId, "ncclGetUniqueId")
    HSES_SYM(CommInitRank, "ncclCommInitRank")
    HSES_SYM(CommDestroy, "ncclCommDestroy")
    HSES_SYM(CommAbort, "ncclCommAbort")
    HSES_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
    HSES_SYM(AllGather, "ncclAllGather")
    HSES_SYM(AllReduce, "ncclAllReduce")
    HSES_SYM(GetErrorString, "ncclGetErrorString")
#undef HSES_SYM
    g_api = api;
    return HSES_OK;
}

int nccl_fail(const char* what, nccl_result_t r) {
    const char* s = g_api.GetErrorString ? g_api.GetErrorString(r) : nullptr;
    set_error(std::string(what) + " failed: " + (s ? s : "NCCL error") + " (code " + std::to_string(r) + ")");
    return HSES_ERR_COMM;
}

}  // namespace
}  // namespace hses

struct hses_comm {
    hses::nccl_comm_t comm = nullptr;
    hses_ctx* ctx = nullptr;  // optional: launch accounting of the collectives
    int rank = 0, world = 1;
    bool broken = false;      // a collective or the async-error poll reported a failure
};

using namespace hses;

extern "C" {

int hses_comm_unique_id(uint8_t* id) {
    HSES_REQUIRE(id != nullptr, "id is NULL");
    int rc = load_api();
    if (rc != HSES_OK) return rc;
    nccl_unique_id u;
    nccl_result_t r = g_api.GetUniqueId(&u);
    if (r != 0) return nccl_fail("ncclGetUniqueId", r);
    memcpy(id, u.internal, HSES_COMM_ID_BYTES);
    return HSES_OK;
}

int hses_comm_init(hses_ctx* ctx, const uint8_t* id, int32_t rank, int32_t world, hses_comm** out) {
    HSES_REQUIRE(out != nullptr, "out is NULL");
    *out = nullptr;
    HSES_REQUIRE(id != nullptr, "id is NULL");
    HSES_REQUIRE(world >= 1 && rank >= 0 && rank < world, "rank must be in [0, world)");
    int rc = load_api();
    if (rc != HSES_OK) return rc;
    if (ctx != nullptr) {
        int current = -1;
        HSES_CUDA(cudaGetDevice(&current));
        HSES_REQUIRE(current == ctx->device, "the context's device must be the current CUDA device");
    }
    nccl_unique_id u;
    memcpy(u.internal, id, HSES_COMM_ID_BYTES);
    nccl_comm_t c = nullptr;
    nccl_result_t r = g_api.CommInitRank(&c, world, u, rank);
    if (r != 0) return nccl_fail("ncclCommInitRank", r);
    hses_comm* h = new hses_comm();
    h->comm = c;
    h->ctx = ctx;
    h->rank = rank;
    h->world = world;
    *out = h;
    return HSES_OK;
}

int hses_comm_rank(const hses_comm* comm) { return comm ? comm->rank : -1; }
int hses_comm_world(const hses_comm* comm) { return comm ? comm->world : 0; }

int hses_comm_async_error(hses_comm* comm) {
    HSES_REQUIRE(comm != nullptr, "comm is NULL");
    if (comm->broken) {
        set_error("hses_comm_async_error: an earlier call on this communicator failed");
        return HSES_ERR_COMM;
    }
    nccl_result_t state = 0;
    nccl_result_t r = g_api.CommGetAsyncError(comm->comm, &state);
    if (r != 0) {
        comm->broken = true;
        return nccl_fail("ncclCommGetAsyncError", r);
    }
    if (state != 0 && state != 7 /* ncclInProgress */) {
        comm->broken = true;
        return nccl_fail("a collective on this communicator", state);
    }
    return HSES_OK;
}

int hses_comm_destroy(hses_comm* comm) {
    if (comm == nullptr) return HSES_OK;
    // a communicator that has seen a failure (a peer that left, a transport error) is aborted:
    // ncclCommDestroy would wait for collectives that can no longer finish
    nccl_result_t r = comm->broken ? g_api.CommAbort(comm->comm) : g_api.CommDestroy(comm->comm);
    delete comm;
    if (r != 0) return nccl_fail("ncclCommDestroy", r);
    return HSES_OK;
}

int hses_comm_abort(hses_comm* comm) {
    if (comm == nullptr) return HSES_OK;
    comm->broken = true;
    return hses_comm_destroy(comm);
}

int hses_allgather_fitness(hses_comm* comm, hses_stream stream, const float* local, int64_t n_local, float* all) {
    HSES_REQUIRE(comm != nullptr, "comm is NULL");
    HSES_REQUIRE(n_local >= 1, "n_local must be positive");
    HSES_REQUIRE(local != nullptr && all != nullptr, "NULL pointer");
    if (comm->broken) {
        set_error("hses_allgather_fitness: the communicator is in an error state; destroy it");
        return HSES_ERR_COMM;
    }
    cudaStream_t st = as_stream(stream);
    nccl_result_t r;
    if (comm->ctx) {
        HSES_KERNEL(comm->ctx, st, "allgather_fitness");
        r = g_api.AllGather(local, all, (size_t)n_local, kNcclFloat32, comm->comm, st);
    } else {
        r = g_api.AllGather(local, all, (size_t)n_local, kNcclFloat32, comm->comm, st);
    }
    if (r != 0) {
        comm->broken = true;
        return nccl_fail("ncclAllGather", r);
    }
    return HSES_OK;
}

int hses_allreduce_grads(hses_comm* comm, hses_stream stream, float* grads, int64_t count) {
    HSES_REQUIRE(comm != nullptr, "comm is NULL");
    HSES_REQUIRE(count >= 1 && grads != nullptr, "nothing to reduce");
    if (comm->broken) {
        set_error("hses_allreduce_grads: the communicator is in an error state; destroy it");
        return HSES_ERR_COMM;
    }
    cudaStream_t st = as_stream(stream);
    nccl_result_t r;
    if (comm->ctx) {
        HSES_KERNEL(comm->ctx, st, "allreduce_grads");
        r = g_api.AllReduce(grads, grads, (size_t)count, kNcclFloat32, kNcclSum, comm->comm, st);
    } else {
        r = g_api.AllReduce(grads, grads, (size_t)count, kNcclFloat32, kNcclSum, comm->comm, st);
    }
    if (r != 0) {
        comm->broken = true;
        return nccl_fail("ncclAllReduce", r);
    }
    return HSES_OK;
}

}  // extern "C"
