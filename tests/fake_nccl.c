/* fake_nccl.c - a stand-in for libnccl, for the failure tests of the gradient exchange on
 * machines without a GPU.  Test infrastructure only.
 *
 * It plays a world of two ranks inside one process: this process is rank 0 and the "peer" is
 * whatever FAKE_NCCL_MODE says:
 *   ok            the peer joins and contributes the same values as this rank (a float sum
 *                 doubles every element); to the bucket-length agreement it contributes
 *                 FAKE_NCCL_PEER_COUNT when that is set (a peer with a different bucket size)
 *   never_joins   ncclCommInitRankConfig answers "in progress" and the state never changes
 *   init_error    joining ends in ncclSystemError
 *   peer_dies     joining works, the first float all-reduce is never accepted ("in progress")
 *   call_error    joining works, a float all-reduce fails with ncclInternalError
 * Buffers are host memory.  boat_fake_nccl marks the library as a stand-in; the fake_nccl_*
 * getters let a test see what was called. */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define EXPORT __attribute__((visibility("default")))

typedef enum { ncclSuccess = 0, ncclSystemError = 2, ncclInternalError = 3, ncclInProgress = 7 } ncclResult_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef struct fake_comm { int world, rank; } *ncclComm_t;
enum { ncclInt64 = 4, ncclFloat32 = 7 };
enum { ncclSum = 0, ncclMax = 2 };

EXPORT int boat_fake_nccl = 1;

static struct fake_comm g_comm_storage;
static ncclResult_t g_state = ncclSuccess;
static int g_aborts, g_destroys, g_float_reduces, g_group_depth;

static const char* mode(void) {
    const char* m = getenv("FAKE_NCCL_MODE");
    return m ? m : "ok";
}

EXPORT int fake_nccl_abort_count(void) { return g_aborts; }
EXPORT int fake_nccl_destroy_count(void) { return g_destroys; }
EXPORT int fake_nccl_float_reduce_count(void) { return g_float_reduces; }

EXPORT ncclResult_t ncclGetUniqueId(ncclUniqueId* id) {
    memset(id, 0x5a, sizeof *id);
    return ncclSuccess;
}

EXPORT ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, void* config) {
    (void)id;
    (void)config;
    g_comm_storage.world = nranks;
    g_comm_storage.rank = rank;
    *comm = &g_comm_storage;
    if (!strcmp(mode(), "never_joins")) return g_state = ncclInProgress;
    if (!strcmp(mode(), "init_error")) {
        g_state = ncclSystemError;
        return ncclInProgress;
    }
    return g_state = ncclSuccess;
}

EXPORT ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* state) {
    (void)comm;
    *state = g_state;
    return ncclSuccess;
}

EXPORT ncclResult_t ncclCommAbort(ncclComm_t comm) {
    (void)comm;
    ++g_aborts;
    g_state = ncclSuccess;
    return ncclSuccess;
}

EXPORT ncclResult_t ncclCommFinalize(ncclComm_t comm) {
    (void)comm;
    return ncclSuccess;
}

EXPORT ncclResult_t ncclCommDestroy(ncclComm_t comm) {
    (void)comm;
    ++g_destroys;
    return ncclSuccess;
}

EXPORT ncclResult_t ncclGroupStart(void) {
    ++g_group_depth;
    return ncclSuccess;
}

EXPORT ncclResult_t ncclGroupEnd(void) {
    --g_group_depth;
    return g_state;
}

EXPORT ncclResult_t ncclAllReduce(const void* send, void* recv, size_t count, int dtype, int op, ncclComm_t comm,
                                  void* stream) {
    (void)comm;
    (void)stream;
    if (dtype == ncclInt64 && op == ncclMax) {
        /* the bucket-length agreement: elements {n, -n}; the peer brings {m, -m} */
        const int64_t* in = (const int64_t*)send;
        int64_t* out = (int64_t*)recv;
        const char* peer = getenv("FAKE_NCCL_PEER_COUNT");
        for (size_t i = 0; i < count; ++i) {
            int64_t mine = in[i], theirs = mine;
            if (peer && count == 2) {
                int64_t m = atoll(peer);
                if (in[0] < 0) m = -m;            /* the overlapped sums agree on minus the total */
                theirs = i == 0 ? m : -m;
            }
            out[i] = mine > theirs ? mine : theirs;
        }
        return ncclSuccess;
    }
    if (dtype == ncclFloat32 && op == ncclSum) {
        ++g_float_reduces;
        if (!strcmp(mode(), "peer_dies")) return g_state = ncclInProgress;
        if (!strcmp(mode(), "call_error")) return ncclInternalError;
        const float* in = (const float*)send;
        float* out = (float*)recv;
        for (size_t i = 0; i < count; ++i) out[i] = in[i] + in[i];
        return ncclSuccess;
    }
    return ncclInternalError;
}

EXPORT const char* ncclGetErrorString(ncclResult_t r) {
    switch (r) {
        case ncclSuccess: return "no error";
        case ncclSystemError: return "unhandled system error";
        case ncclInternalError: return "internal error";
        case ncclInProgress: return "in progress";
        default: return "unknown";
    }
}
