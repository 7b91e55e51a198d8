/* Stand-in for the NCCL entry points the library binds at run time, for CPU tests of the
 * communicator wrapper (no GPU, one rank).  Buffers are host memory.  Failures are injected
 * through the environment:
 *   FAKE_NCCL_FAIL=init|allgather|allreduce   the named call returns ncclSystemError (2)
 *   FAKE_NCCL_ASYNC=<code>                    ncclCommGetAsyncError reports <code> (6 = remote error)
 * Calls are counted in the file FAKE_NCCL_LOG names (one line per call), so a test can tell
 * ncclCommAbort from ncclCommDestroy. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct { char internal[128]; } fake_id_t;
typedef struct { int rank, world; } fake_comm_t;

static void note(const char* what) {
    const char* path = getenv("FAKE_NCCL_LOG");
    if (!path) return;
    FILE* f = fopen(path, "a");
    if (!f) return;
    fprintf(f, "%s\n", what);
    fclose(f);
}
static int fails(const char* what) {
    const char* f = getenv("FAKE_NCCL_FAIL");
    return f && strcmp(f, what) == 0;
}

int ncclGetUniqueId(fake_id_t* id) {
    note("ncclGetUniqueId");
    for (int i = 0; i < 128; ++i) id->internal[i] = (char)(i * 7 + 1);
    return 0;
}
int ncclCommInitRank(void** comm, int world, fake_id_t id, int rank) {
    note("ncclCommInitRank");
    if (fails("init")) return 2;
    if (id.internal[1] != 8) return 4; /* ncclInvalidArgument: not the id handed out above */
    fake_comm_t* c = (fake_comm_t*)malloc(sizeof(fake_comm_t));
    c->rank = rank;
    c->world = world;
    *comm = c;
    return 0;
}
int ncclCommDestroy(void* comm) { note("ncclCommDestroy"); free(comm); return 0; }
int ncclCommAbort(void* comm) { note("ncclCommAbort"); free(comm); return 0; }
int ncclCommGetAsyncError(void* comm, int* state) {
    (void)comm;
    const char* a = getenv("FAKE_NCCL_ASYNC");
    *state = a ? atoi(a) : 0;
    return 0;
}
int ncclAllGather(const void* src, void* dst, size_t count, int dtype, void* comm, void* stream) {
    (void)stream;
    note("ncclAllGather");
    if (fails("allgather")) return 2;
    fake_comm_t* c = (fake_comm_t*)comm;
    if (dtype != 7) return 4;
    /* one rank: every slot of the output is this rank's shard */
    for (int r = 0; r < c->world; ++r) memcpy((char*)dst + (size_t)r * count * 4, src, count * 4);
    return 0;
}
int ncclAllReduce(const void* src, void* dst, size_t count, int dtype, int op, void* comm, void* stream) {
    (void)stream;
    note("ncclAllReduce");
    if (fails("allreduce")) return 2;
    fake_comm_t* c = (fake_comm_t*)comm;
    if (dtype != 7 || op != 0) return 4;
    /* every rank is taken to hold the same values: the sum is world times the input */
    const float* s = (const float*)src;
    float* d = (float*)dst;
    for (size_t i = 0; i < count; ++i) d[i] = s[i] * (float)c->world;
    return 0;
}
const char* ncclGetErrorString(int code) {
    switch (code) {
        case 0: return "no error";
        case 2: return "unhandled system error";
        case 4: return "invalid argument";
        case 6: return "remote process exited or there was a network error";
        default: return "error";
    }
}
