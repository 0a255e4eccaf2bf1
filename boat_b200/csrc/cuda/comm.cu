// comm.cu - the one collective of the data-parallel attention step: an in-place FP32 sum of
// the flat gradient bucket over all ranks, through NCCL on NVLink/NVSwitch.  One process
// per GPU.  The reference has no counterpart (it is a single-process CPU library).
//
// NCCL is loaded at first use with dlopen so that single-GPU users need no NCCL at all and
// so that a host program which already loaded a libnccl.so.2 shares that copy.
#include "common.cuh"
#include <dlfcn.h>
#include <string.h>

namespace boatcu {

// Just enough of NCCL's C interface to call it through function pointers.
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;                   // 0 == ncclSuccess
enum { kNcclFloat32 = 7, kNcclSum = 0 };    // ncclFloat32, ncclSum in nccl.h

static struct {
    void* lib;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    const char* (*GetErrorString)(ncclResult_t);
} g_nccl;

static ncclComm_t g_comm = nullptr;
static int g_world = 1;

static int load_nccl() {
    if (g_nccl.lib) return 0;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    void* lib = nullptr;
    for (const char* n : names) {
        lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (lib) break;
    }
    if (!lib) return set_error(20, "NCCL library not found: %s", dlerror());
#define LOAD(field, sym)                                                     \
    *(void**)(&g_nccl.field) = dlsym(lib, sym);                              \
    if (!g_nccl.field) return set_error(20, "NCCL symbol %s missing", sym);
    LOAD(GetUniqueId, "ncclGetUniqueId")
    LOAD(CommInitRank, "ncclCommInitRank")
    LOAD(AllReduce, "ncclAllReduce")
    LOAD(CommDestroy, "ncclCommDestroy")
    LOAD(GetErrorString, "ncclGetErrorString")
#undef LOAD
    g_nccl.lib = lib;
    return 0;
}

#define NCCL_OK(call)                                                                        \
    do {                                                                                     \
        ncclResult_t r__ = (call);                                                           \
        if (r__ != 0) return set_error(2000 + r__, "%s failed: %s", #call, g_nccl.GetErrorString(r__)); \
    } while (0)

}  // namespace boatcu

using namespace boatcu;

extern "C" {

int boat_cuda_comm_unique_id(void* id_out) {
    if (!id_out) return set_error(21, "boat_cuda_comm_unique_id: NULL buffer");
    if (int rc = load_nccl()) return rc;
    ncclUniqueId id;
    NCCL_OK(g_nccl.GetUniqueId(&id));
    memcpy(id_out, &id, sizeof id);
    return 0;
}

int boat_cuda_comm_init(int rank, int world, const void* id_in) {
    if (world < 1 || rank < 0 || rank >= world || !id_in) return set_error(21, "boat_cuda_comm_init: bad arguments");
    if (g_comm) return set_error(21, "boat_cuda_comm_init: a communicator already exists");
    if (int rc = ensure_init()) return rc;
    if (world == 1) {
        g_world = 1;
        return 0;
    }
    if (int rc = load_nccl()) return rc;
    ncclUniqueId id;
    memcpy(&id, id_in, sizeof id);
    NCCL_OK(g_nccl.CommInitRank(&g_comm, world, id, rank));
    g_world = world;
    return 0;
}

int boat_cuda_comm_world(void) { return g_world; }

int boat_cuda_allreduce_sum_f32(float* buf, int64_t n) {
    if (g_world <= 1 || n <= 0) return 0;
    if (!g_comm) return set_error(22, "boat_cuda_allreduce_sum_f32: no communicator");
    NCCL_OK(g_nccl.AllReduce(buf, buf, (size_t)n, kNcclFloat32, kNcclSum, g_comm, stream()));
    return 0;
}

int boat_cuda_comm_destroy(void) {
    if (g_comm) {
        NCCL_OK(g_nccl.CommDestroy(g_comm));
        g_comm = nullptr;
    }
    g_world = 1;
    return 0;
}

}  // extern "C"
