// comm.cu - the one collective of the data-parallel attention step: an in-place FP32 sum of
// (pieces of) the flat gradient bucket over all ranks, through NCCL on NVLink/NVSwitch.  One
// process per GPU.  The reference has no counterpart (it is a single-process CPU library).
//
// Overlap: sums can be started on a stream of their own (allreduce_begin) as soon as the
// kernels that produce a piece have been launched, and are joined to the library stream later
// (allreduce_join), so that the transfer of the output projection's gradients runs under the
// attention-core backward and that of the input projections' gradients under the input-
// gradient GEMMs.
//
// Failure handling: the communicator is non-blocking.  Every NCCL call may answer "in
// progress"; the host then polls ncclCommGetAsyncError under a deadline.  A rank that never
// joins, a peer that died or an error reported by NCCL ends in ncclCommAbort and an error
// status - never in a host thread stuck inside NCCL.  Before the first sum of a given length
// the ranks agree on that length through the communicator itself (a two-element maximum), so a
// rank that brings a bucket of another size gets an error instead of a hang or silent garbage.
//
// NCCL is loaded at first use with dlopen (BOAT_NCCL_LIB names the library, default
// libnccl.so.2) so that single-GPU users need no NCCL at all and a host program that already
// loaded one shares that copy.  A library that exports `boat_fake_nccl` is a stand-in used by
// the failure tests on machines without a GPU: with it no CUDA call is made here (buffers are
// host memory, there are no streams).
#include "common.cuh"
#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

namespace boatcu {

static struct {
    void* lib;
    bool fake;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*);
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*);
    ncclResult_t (*CommAbort)(ncclComm_t);
    ncclResult_t (*CommFinalize)(ncclComm_t);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    const char* (*GetErrorString)(ncclResult_t);
} g_nccl;

static ncclComm_t g_comm = nullptr;
static int g_world = 1;
static cudaStream_t g_comm_stream = nullptr;     // the overlapped sums run here
static cudaEvent_t g_ev_ready = nullptr, g_ev_done = nullptr;
static bool g_pending = false;                   // sums started and not yet joined
static int64_t g_agreed[8];                      // bucket lengths the ranks have agreed on
static int g_n_agreed = 0;

static double env_seconds(const char* name, double dflt) {
    const char* e = getenv(name);
    if (!e || !*e) return dflt;
    double v = atof(e);
    return v > 0 ? v : dflt;
}
// BOAT_COMM_INIT_TIMEOUT_S: how long every rank may take to join (default 120 s).
// BOAT_COMM_TIMEOUT_S: how long NCCL may take to accept a collective (default 30 s).
static double init_deadline() { return env_seconds("BOAT_COMM_INIT_TIMEOUT_S", 120.0); }
static double call_deadline() { return env_seconds("BOAT_COMM_TIMEOUT_S", 30.0); }

static double now_s() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

static int load_nccl() {
    if (g_nccl.lib) return 0;
    const char* forced = getenv("BOAT_NCCL_LIB");
    const char* names[] = {forced && *forced ? forced : "libnccl.so.2", "libnccl.so"};
    void* lib = nullptr;
    for (const char* n : names) {
        lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (lib || (forced && *forced)) break;
    }
    if (!lib) return set_error(20, "NCCL library not found: %s", dlerror());
#define LOAD(field, sym)                                                     \
    *(void**)(&g_nccl.field) = dlsym(lib, sym);                              \
    if (!g_nccl.field) return set_error(20, "NCCL symbol %s missing", sym);
    LOAD(GetUniqueId, "ncclGetUniqueId")
    LOAD(CommInitRankConfig, "ncclCommInitRankConfig")
    LOAD(CommGetAsyncError, "ncclCommGetAsyncError")
    LOAD(CommAbort, "ncclCommAbort")
    LOAD(CommFinalize, "ncclCommFinalize")
    LOAD(CommDestroy, "ncclCommDestroy")
    LOAD(AllReduce, "ncclAllReduce")
    LOAD(GroupStart, "ncclGroupStart")
    LOAD(GroupEnd, "ncclGroupEnd")
    LOAD(GetErrorString, "ncclGetErrorString")
#undef LOAD
    g_nccl.fake = dlsym(lib, "boat_fake_nccl") != nullptr;
    g_nccl.lib = lib;
    return 0;
}

// Gives the communicator up for good: abort it and fall back to a world of one.
static void abandon() {
    if (g_comm) g_nccl.CommAbort(g_comm);
    g_comm = nullptr;
    g_world = 1;
    g_pending = false;
    g_n_agreed = 0;
}

// After an NCCL call answered `first`: wait until the communicator has left "in progress".
// Past the deadline, or on an error state, the communicator is aborted.
static int settle(const char* what, ncclResult_t first, double deadline_s) {
    if (first != ncclSuccess && first != ncclInProgress) {
        int rc = set_error(2000 + (int)first, "%s failed: %s; communicator aborted", what, g_nccl.GetErrorString(first));
        abandon();
        return rc;
    }
    const double t0 = now_s();
    for (;;) {
        ncclResult_t state = ncclSuccess;
        ncclResult_t q = g_nccl.CommGetAsyncError(g_comm, &state);
        if (q != ncclSuccess) state = q;
        if (state == ncclSuccess) return 0;
        if (state != ncclInProgress) {
            int rc = set_error(2000 + (int)state, "%s: NCCL reports %s; communicator aborted", what,
                               g_nccl.GetErrorString(state));
            abandon();
            return rc;
        }
        if (now_s() - t0 > deadline_s) {
            int rc = set_error(23, "%s: not complete after %.1f s (a rank that never joined or has gone); "
                                   "communicator aborted", what, deadline_s);
            abandon();
            return rc;
        }
        struct timespec nap = {0, 200000};      // 0.2 ms
        nanosleep(&nap, nullptr);
    }
}

// Device memory for the length agreement - or host memory with the stand-in library.
static void* small_alloc(size_t bytes) {
    if (g_nccl.fake) return malloc(bytes);
    void* p = nullptr;
    return boat_cuda_malloc(&p, bytes) == 0 ? p : nullptr;
}
static void small_free(void* p) {
    if (g_nccl.fake) free(p);
    else boat_cuda_free(p);
}
static int small_put(void* dst, const void* src, size_t bytes) {
    if (g_nccl.fake) return memcpy(dst, src, bytes), 0;
    return boat_cuda_memcpy_h2d(dst, src, bytes);
}
static int small_get(void* dst, const void* src, size_t bytes) {
    if (g_nccl.fake) return memcpy(dst, src, bytes), 0;
    return boat_cuda_memcpy_d2h(dst, src, bytes);
}

// All ranks must bring the same element count: max(n) == -max(-n) over the ranks.
static int agree_on_length(int64_t n) {
    for (int i = 0; i < g_n_agreed; ++i)
        if (g_agreed[i] == n) return 0;
    int64_t* d = (int64_t*)small_alloc(2 * sizeof(int64_t));
    if (!d) return set_error(24, "all-reduce: no memory for the bucket-length agreement (%s)", boat_cuda_last_error());
    int64_t h[2] = {n, -n};
    int rc = small_put(d, h, sizeof h);
    if (rc == 0)
        rc = settle("bucket-length agreement",
                    g_nccl.AllReduce(d, d, 2, ncclInt64, ncclMax, g_comm, g_nccl.fake ? (cudaStream_t)0 : stream()),
                    call_deadline());
    if (rc == 0) rc = small_get(h, d, sizeof h);
    small_free(d);
    if (rc != 0) return rc;
    if (h[0] != n || h[1] != -n)
        return set_error(25, "all-reduce: this rank brings %lld elements, another rank %lld: the ranks must "
                             "reduce buckets of one size", (long long)n, (long long)(h[0] != n ? h[0] : -h[1]));
    if (g_n_agreed < 8) g_agreed[g_n_agreed++] = n;
    return 0;
}

static int comm_streams() {
    if (g_comm_stream || g_nccl.fake) return 0;
    int lo = 0, hi = 0;
    BOATCU_CHECK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    // highest priority: a few communication CTAs should get their SMs ahead of the next compute wave
    BOATCU_CHECK(cudaStreamCreateWithPriority(&g_comm_stream, cudaStreamNonBlocking, hi));
    BOATCU_CHECK(cudaEventCreateWithFlags(&g_ev_ready, cudaEventDisableTiming));
    BOATCU_CHECK(cudaEventCreateWithFlags(&g_ev_done, cudaEventDisableTiming));
    return 0;
}

// Called by boat_cuda_sync(): nothing of ours may still be running when it returns.
int comm_stream_sync() {
    if (g_comm_stream && g_pending) BOATCU_CHECK(cudaStreamSynchronize(g_comm_stream));
    return 0;
}

}  // namespace boatcu

using namespace boatcu;

extern "C" {

int boat_cuda_comm_unique_id(void* id_out) {
    if (!id_out) return set_error(21, "boat_cuda_comm_unique_id: NULL buffer");
    if (int rc = load_nccl()) return rc;
    ncclUniqueId id;
    ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) return set_error(2000 + (int)r, "ncclGetUniqueId failed: %s", g_nccl.GetErrorString(r));
    memcpy(id_out, &id, sizeof id);
    return 0;
}

int boat_cuda_comm_init(int rank, int world, const void* id_in) {
    if (world < 1 || rank < 0 || rank >= world || !id_in) return set_error(21, "boat_cuda_comm_init: bad arguments");
    if (g_comm) return set_error(21, "boat_cuda_comm_init: a communicator already exists");
    if (world == 1) {
        g_world = 1;
        return 0;
    }
    if (int rc = load_nccl()) return rc;
    if (!g_nccl.fake) {
        if (int rc = ensure_init()) return rc;
        if (int rc = comm_streams()) return rc;
    }
    ncclUniqueId id;
    memcpy(&id, id_in, sizeof id);
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 0;
    ncclResult_t r = g_nccl.CommInitRankConfig(&g_comm, world, id, rank, &cfg);
    if (!g_comm && r != ncclSuccess && r != ncclInProgress)
        return set_error(2000 + (int)r, "ncclCommInitRankConfig failed: %s", g_nccl.GetErrorString(r));
    g_n_agreed = 0;
    if (int rc = settle("joining the communicator", r, init_deadline())) return rc;
    g_world = world;
    return 0;
}

int boat_cuda_comm_world(void) { return g_world; }

int boat_cuda_allreduce_sum_f32(float* buf, int64_t n) {
    if (g_world <= 1 || n <= 0) return 0;
    if (!g_comm) return set_error(22, "boat_cuda_allreduce_sum_f32: no communicator");
    if (int rc = agree_on_length(n)) return rc;
    return settle("gradient all-reduce",
                  g_nccl.AllReduce(buf, buf, (size_t)n, ncclFloat32, ncclSum, g_comm,
                                   g_nccl.fake ? (cudaStream_t)0 : stream()),
                  call_deadline());
}

int boat_cuda_allreduce_begin(float* const* bufs, const int64_t* counts, int pieces) {
    if (g_world <= 1 || pieces <= 0) return 0;
    if (!g_comm) return set_error(22, "boat_cuda_allreduce_begin: no communicator");
    if (!bufs || !counts) return set_error(21, "boat_cuda_allreduce_begin: NULL arguments");
    int64_t total = 0;
    for (int i = 0; i < pieces; ++i) {
        if (counts[i] < 0 || (counts[i] > 0 && !bufs[i])) return set_error(21, "boat_cuda_allreduce_begin: bad piece %d", i);
        total += counts[i];
    }
    if (total == 0) return 0;
    // one agreement per distinct combination is enough: the total stands for it
    if (int rc = agree_on_length(-total)) return rc;
    cudaStream_t s = g_nccl.fake ? (cudaStream_t)0 : g_comm_stream;
    if (!g_nccl.fake) {
        // the pieces are final once everything launched so far on the library stream has run
        BOATCU_CHECK(cudaEventRecord(g_ev_ready, stream()));
        BOATCU_CHECK(cudaStreamWaitEvent(g_comm_stream, g_ev_ready, 0));
    }
    ncclResult_t r = g_nccl.GroupStart();
    if (r != ncclSuccess && r != ncclInProgress) return settle("ncclGroupStart", r, call_deadline());
    for (int i = 0; i < pieces; ++i) {
        if (counts[i] == 0) continue;
        r = g_nccl.AllReduce(bufs[i], bufs[i], (size_t)counts[i], ncclFloat32, ncclSum, g_comm, s);
        if (r != ncclSuccess && r != ncclInProgress) {
            g_nccl.GroupEnd();
            return settle("gradient all-reduce (piece)", r, call_deadline());
        }
    }
    if (int rc = settle("gradient all-reduce (overlapped)", g_nccl.GroupEnd(), call_deadline())) return rc;
    g_pending = true;
    return 0;
}

int boat_cuda_allreduce_join(void) {
    if (!g_pending) return 0;
    if (!g_nccl.fake) {
        BOATCU_CHECK(cudaEventRecord(g_ev_done, g_comm_stream));
        BOATCU_CHECK(cudaStreamWaitEvent(stream(), g_ev_done, 0));
    }
    g_pending = false;
    return 0;
}

int boat_cuda_allreduce_pending(void) { return g_pending ? 1 : 0; }

int boat_cuda_comm_destroy(void) {
    if (g_comm) {
        if (g_comm_stream && g_pending) cudaStreamSynchronize(g_comm_stream);
        g_pending = false;
        ncclComm_t c = g_comm;
        // A non-blocking communicator is finalized first (flushes what was issued; completes in
        // the background, polled under the usual deadline) and destroyed afterwards.
        ncclResult_t r = g_nccl.CommFinalize(c);
        if (r == ncclInProgress) {
            const double t0 = now_s();
            ncclResult_t state = ncclInProgress;
            while (state == ncclInProgress && now_s() - t0 < call_deadline()) {
                if (g_nccl.CommGetAsyncError(c, &state) != ncclSuccess) break;
                struct timespec nap = {0, 200000};
                nanosleep(&nap, nullptr);
            }
            r = state == ncclInProgress ? ncclSuccess : state;
        }
        if (r == ncclSuccess) r = g_nccl.CommDestroy(c);
        else g_nccl.CommAbort(c);
        g_comm = nullptr;
        g_world = 1;
        g_n_agreed = 0;
        if (r != ncclSuccess) return set_error(2000 + (int)r, "ncclCommDestroy failed: %s", g_nccl.GetErrorString(r));
    }
    g_world = 1;
    return 0;
}

}  // extern "C"
