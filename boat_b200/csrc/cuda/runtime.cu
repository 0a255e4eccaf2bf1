// runtime.cu - device selection, the library stream, stream-ordered HBM allocation and
// host<->HBM copies.  Stands in for the device stubs of the reference's memory layer
// (src/core/memory.c:174-186 allocate_device/free_device and :230-247 copy/set, which were
// malloc/memcpy/memset regardless of the device argument).
#include "tc_common.cuh"
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>
#include <atomic>
#include <mutex>
#include <unordered_map>
#include <vector>
#include <string>
#include <map>

namespace boatcu {

static thread_local char g_err[512] = "";
static std::mutex g_mu;
static bool g_ready = false;
static int g_device = -1;                       // the one device this process's library is bound to
static int g_sm_count = 0;
static cudaStream_t g_stream = 0;
static std::atomic<uint64_t> g_launches{0};
static std::unordered_map<void*, size_t>* g_live = nullptr;
static size_t g_live_bytes = 0;
static unsigned int* g_status_host = nullptr;   // kernel status word, host view
static unsigned int* g_status_dev = nullptr;    // the same word as kernels see it

int set_error(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return status;
}

cudaStream_t stream() { return g_stream; }
bool ready() { return g_ready; }
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

static int pick_device(int requested) {
    if (requested >= 0) return requested;
    const char* e = getenv("BOAT_CUDA_DEVICE");
    if (e && *e) return atoi(e);
    e = getenv("LOCAL_RANK");
    if (e && *e) return atoi(e);
    return 0;
}

static int init_locked(int device) {
    if (g_ready) {
        // The library serves one device per process (one process per GPU); a later request for
        // another one is an error, not a silent no-op.
        if (device >= 0 && device != g_device)
            return set_error(6, "boat_cuda_init(%d): the library is already bound to device %d", device, g_device);
        return 0;
    }
    int n = 0;
    cudaError_t err = cudaGetDeviceCount(&n);
    if (err != cudaSuccess || n == 0) {
        cudaGetLastError();
        return set_error(2, "no CUDA device available: %s",
                         err == cudaSuccess ? "device count is 0" : cudaGetErrorString(err));
    }
    int dev = pick_device(device);
    if (dev < 0 || dev >= n) return set_error(2, "device index %d out of range: %d device(s) visible", dev, n);
    BOATCU_CHECK(cudaSetDevice(dev));
    cudaDeviceProp prop;
    BOATCU_CHECK(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10) {
        return set_error(3, "device %d is sm_%d%d; this library contains sm_100a code only",
                         dev, prop.major, prop.minor);
    }
    // Keep freed blocks in the pool instead of returning them to the driver: a training
    // step allocates and frees the same sizes every iteration.
    cudaMemPool_t pool;
    BOATCU_CHECK(cudaDeviceGetDefaultMemPool(&pool, dev));
    uint64_t keep = UINT64_MAX;
    BOATCU_CHECK(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
    if (!g_live) g_live = new std::unordered_map<void*, size_t>();
    BOATCU_CHECK(cudaHostAlloc((void**)&g_status_host, sizeof(unsigned int), cudaHostAllocMapped));
    *g_status_host = 0;
    BOATCU_CHECK(cudaHostGetDevicePointer((void**)&g_status_dev, g_status_host, 0));
    g_device = dev;
    g_sm_count = prop.multiProcessorCount;
    g_ready = true;
    return 0;
}

int bound_device() { return g_device; }
int sm_count() { return g_sm_count > 0 ? g_sm_count : 1; }

// ---- kernel status word ---------------------------------------------------------------------
// One 32-bit word in mapped pinned host memory.  Kernels write a code there when a bounded
// wait gives up; the host reads it after a synchronisation without any copy.
unsigned int* kernel_status_ptr() { return g_status_dev; }

unsigned int take_kernel_status() {
    if (!g_status_host) return 0;
    unsigned int v = *(volatile unsigned int*)g_status_host;
    if (v) *(volatile unsigned int*)g_status_host = 0;
    return v;
}

static int report_kernel_status(const char* where) {
    unsigned int v = take_kernel_status();
    if (v == 0) return 0;
    return set_error(30, "%s: a tensor-core kernel gave up waiting (role code %u); its results are invalid", where, v);
}

// ---- tensor maps -------------------------------------------------------------------------------
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static encode_tiled_fn g_encode = nullptr;

int make_tensor_map_2d(CUtensorMap* map, const void* base, int esize, uint64_t rows, uint64_t cols, uint64_t ld,
                       uint32_t box_rows, uint32_t box_cols, bool atom32) {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        BOATCU_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (!fn || q != cudaDriverEntryPointSuccess) return set_error(31, "cuTensorMapEncodeTiled is not available");
        g_encode = (encode_tiled_fn)fn;
    }
    if (((uintptr_t)base & 15) != 0 || ((ld * (uint64_t)esize) & 15) != 0)
        return set_error(31, "tensor map: base or row pitch not 16-byte aligned");
    if (box_cols * (uint32_t)esize != 128 || box_rows > 256 || box_rows == 0)
        return set_error(31, "tensor map: box must be 128 bytes wide and at most 256 rows");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * (uint64_t)esize};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt = esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    CUresult r = g_encode(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(31, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return 0;
}

// ---- per-kernel timing ---------------------------------------------------------------------
struct ProfileEntry {
    const char* name;
    cudaEvent_t start, stop;
};
static bool g_profiling = false;
static std::vector<ProfileEntry>* g_profile = nullptr;

ProfileScope::ProfileScope(const char* name) : slot(-1) {
    if (!g_profiling) return;
    ProfileEntry e;
    e.name = name;
    if (cudaEventCreate(&e.start) != cudaSuccess || cudaEventCreate(&e.stop) != cudaSuccess) return;
    cudaEventRecord(e.start, g_stream);
    g_profile->push_back(e);
    slot = (int)g_profile->size() - 1;
}

ProfileScope::~ProfileScope() {
    if (slot >= 0) cudaEventRecord((*g_profile)[slot].stop, g_stream);
}

// The current device is a per-thread setting of the CUDA runtime: a thread that enters the
// library for the first time is switched to the bound device, so that its launches and the
// pointers it is handed belong to the same GPU.
static thread_local bool t_on_bound_device = false;

int ensure_init() {
    if (!g_ready) {
        std::lock_guard<std::mutex> lk(g_mu);
        if (int rc = init_locked(-1)) return rc;
    }
    if (!t_on_bound_device) {
        BOATCU_CHECK(cudaSetDevice(g_device));
        t_on_bound_device = true;
    }
    return 0;
}

}  // namespace boatcu

using namespace boatcu;

extern "C" {

int boat_cuda_init(int device) {
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (int rc = init_locked(device)) return rc;
    }
    return ensure_init();
}

int boat_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

const char* boat_cuda_last_error(void) { return g_err; }

void* boat_cuda_stream(void) { return (void*)g_stream; }

int boat_cuda_set_stream(void* s) {
    g_stream = (cudaStream_t)s;
    return 0;
}

// ---- copies that overlap kernels -----------------------------------------------------------------
// One extra stream per direction (non-blocking: the library stream may be the legacy default
// stream).  Ordering against the library stream is by events: the copy streams see buffers
// allocated or written on the library stream after boat_cuda_copies_after_compute(), uploads
// become visible to later kernels through boat_cuda_join_uploads(), and a download starts after
// the kernels launched before it.
static cudaStream_t g_up = nullptr, g_down = nullptr;
static cudaEvent_t g_up_done = nullptr, g_compute_done = nullptr;
static bool g_copy_pending = false;

static int copy_streams() {
    if (g_up) return 0;
    BOATCU_CHECK(cudaStreamCreateWithFlags(&g_up, cudaStreamNonBlocking));
    BOATCU_CHECK(cudaStreamCreateWithFlags(&g_down, cudaStreamNonBlocking));
    BOATCU_CHECK(cudaEventCreateWithFlags(&g_up_done, cudaEventDisableTiming));
    BOATCU_CHECK(cudaEventCreateWithFlags(&g_compute_done, cudaEventDisableTiming));
    return 0;
}

int boat_cuda_copies_after_compute(void) {
    if (int rc = ensure_init()) return rc;
    if (int rc = copy_streams()) return rc;
    BOATCU_CHECK(cudaEventRecord(g_compute_done, g_stream));
    BOATCU_CHECK(cudaStreamWaitEvent(g_up, g_compute_done, 0));
    BOATCU_CHECK(cudaStreamWaitEvent(g_down, g_compute_done, 0));
    return 0;
}

int boat_cuda_upload_async(void* dst, const void* src, size_t bytes) {
    if (bytes == 0) return 0;
    if (int rc = ensure_init()) return rc;
    if (int rc = copy_streams()) return rc;
    BOATCU_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, g_up));
    g_copy_pending = true;
    return 0;
}

int boat_cuda_join_uploads(void) {
    if (!g_up) return 0;
    BOATCU_CHECK(cudaEventRecord(g_up_done, g_up));
    BOATCU_CHECK(cudaStreamWaitEvent(g_stream, g_up_done, 0));
    return 0;
}

int boat_cuda_download_async(void* dst, const void* src, size_t bytes) {
    if (bytes == 0) return 0;
    if (int rc = ensure_init()) return rc;
    if (int rc = copy_streams()) return rc;
    BOATCU_CHECK(cudaEventRecord(g_compute_done, g_stream));
    BOATCU_CHECK(cudaStreamWaitEvent(g_down, g_compute_done, 0));
    BOATCU_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, g_down));
    g_copy_pending = true;
    return 0;
}

int boat_cuda_sync(void) {
    if (int rc = ensure_init()) return rc;
    BOATCU_CHECK(cudaStreamSynchronize(g_stream));
    if (g_copy_pending) {
        BOATCU_CHECK(cudaStreamSynchronize(g_up));
        BOATCU_CHECK(cudaStreamSynchronize(g_down));
        g_copy_pending = false;
    }
    if (int rc = comm_stream_sync()) return rc;
    return report_kernel_status("boat_cuda_sync");
}

int boat_cuda_malloc(void** ptr, size_t bytes) {
    if (!ptr) return set_error(4, "boat_cuda_malloc: NULL out pointer");
    *ptr = nullptr;
    if (bytes == 0) return 0;
    if (int rc = ensure_init()) return rc;
    BOATCU_CHECK(cudaMallocAsync(ptr, bytes, g_stream));
    std::lock_guard<std::mutex> lk(g_mu);
    (*g_live)[*ptr] = bytes;
    g_live_bytes += bytes;
    return 0;
}

int boat_cuda_free(void* ptr) {
    if (!ptr) return 0;
    if (int rc = ensure_init()) return rc;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_live->find(ptr);
        if (it == g_live->end()) return set_error(5, "boat_cuda_free: %p was not allocated here", ptr);
        g_live_bytes -= it->second;
        g_live->erase(it);
    }
    BOATCU_CHECK(cudaFreeAsync(ptr, g_stream));
    return 0;
}

size_t boat_cuda_bytes_in_use(void) { return g_live_bytes; }
uint64_t boat_cuda_launch_count(void) { return g_launches.load(); }

int boat_cuda_memcpy_h2d(void* dst, const void* src, size_t bytes) {
    if (bytes == 0) return 0;
    if (int rc = ensure_init()) return rc;
    BOATCU_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, g_stream));
    BOATCU_CHECK(cudaStreamSynchronize(g_stream));
    return 0;
}

int boat_cuda_memcpy_d2h(void* dst, const void* src, size_t bytes) {
    if (bytes == 0) return 0;
    if (int rc = ensure_init()) return rc;
    BOATCU_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, g_stream));
    BOATCU_CHECK(cudaStreamSynchronize(g_stream));
    return report_kernel_status("boat_cuda_memcpy_d2h");
}

int boat_cuda_memcpy_d2d(void* dst, const void* src, size_t bytes) {
    if (bytes == 0) return 0;
    if (int rc = ensure_init()) return rc;
    BOATCU_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, g_stream));
    return 0;
}

int boat_cuda_memset(void* dst, int value, size_t bytes) {
    if (bytes == 0) return 0;
    if (int rc = ensure_init()) return rc;
    BOATCU_CHECK(cudaMemsetAsync(dst, value, bytes, g_stream));
    return 0;
}

// ---- pinned host blocks ---------------------------------------------------------------------
// Large host tensors are the source and destination of every upload and download of the
// host-tensor path.  Page-locked memory makes those copies several times faster, but locking
// pages costs milliseconds per allocation, so freed blocks are kept and handed out again.
// Freed blocks stay page-locked for re-use up to a cap (BOAT_PINNED_POOL_MB, default 4096); beyond
// it a freed block is unlocked and returned to the system at once.
// A plain host allocation never starts the GPU: before boat_cuda_init (explicit, or implicit in the
// first compute call) host_alloc declines and the caller uses ordinary memory.
static std::multimap<size_t, void*>* g_pinned_free = nullptr;
static std::unordered_map<void*, size_t>* g_pinned_size = nullptr;
static size_t g_pinned_free_bytes = 0;

static size_t pinned_pool_cap() {
    static size_t cap = 0;
    if (cap == 0) {
        const char* e = getenv("BOAT_PINNED_POOL_MB");
        long long mb = e && *e ? atoll(e) : 4096;
        if (mb < 0) mb = 0;
        cap = (size_t)mb << 20;
        if (cap == 0) cap = 1;      // "0" = keep nothing
    }
    return cap;
}

void* boat_cuda_host_alloc(size_t bytes) {
    if (bytes == 0 || !g_ready) return nullptr;
    if (ensure_init() != 0) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_pinned_free) {
        g_pinned_free = new std::multimap<size_t, void*>();
        g_pinned_size = new std::unordered_map<void*, size_t>();
    }
    auto it = g_pinned_free->lower_bound(bytes);
    if (it != g_pinned_free->end() && it->first <= bytes + bytes / 4) {
        void* p = it->second;
        g_pinned_free_bytes -= it->first;
        g_pinned_free->erase(it);
        return p;
    }
    void* p = nullptr;
    if (cudaHostAlloc(&p, bytes, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    (*g_pinned_size)[p] = bytes;
    return p;
}

int boat_cuda_host_free(void* ptr) {
    if (!ptr) return 0;
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_pinned_size ? g_pinned_size->find(ptr) : std::unordered_map<void*, size_t>::iterator();
    if (!g_pinned_size || it == g_pinned_size->end()) return set_error(5, "boat_cuda_host_free: %p is not a pinned block", ptr);
    if (g_pinned_free_bytes + it->second > pinned_pool_cap()) {
        g_pinned_size->erase(it);
        if (cudaFreeHost(ptr) != cudaSuccess) cudaGetLastError();
        return 0;
    }
    g_pinned_free_bytes += it->second;
    g_pinned_free->insert({it->second, ptr});
    return 0;
}

int boat_cuda_profile_enable(int on) {
    if (int rc = ensure_init()) return rc;
    if (!g_profile) g_profile = new std::vector<ProfileEntry>();
    g_profiling = on != 0;
    return 0;
}

// Waits for the stream, then writes one line per kernel family into `out`:
// "<name> <launch scopes> <total milliseconds>\n".  Clears the record.
int boat_cuda_profile_report(char* out, size_t out_bytes) {
    if (!out || out_bytes == 0) return set_error(4, "boat_cuda_profile_report: no buffer");
    out[0] = 0;
    if (!g_profile) return 0;
    BOATCU_CHECK(cudaStreamSynchronize(g_stream));
    std::map<std::string, std::pair<int, double>> acc;
    for (auto& e : *g_profile) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, e.start, e.stop) == cudaSuccess) {
            auto& a = acc[e.name];
            a.first += 1;
            a.second += ms;
        }
        cudaEventDestroy(e.start);
        cudaEventDestroy(e.stop);
    }
    g_profile->clear();
    size_t used = 0;
    for (auto& kv : acc) {
        int n = snprintf(out + used, out_bytes - used, "%s %d %.6f\n", kv.first.c_str(), kv.second.first, kv.second.second);
        if (n < 0 || (size_t)n >= out_bytes - used) break;
        used += (size_t)n;
    }
    return 0;
}

int boat_cuda_host_register(void* host, size_t bytes) {
    if (int rc = ensure_init()) return rc;
    BOATCU_CHECK(cudaHostRegister(host, bytes, cudaHostRegisterDefault));
    return 0;
}

int boat_cuda_host_unregister(void* host) {
    if (int rc = ensure_init()) return rc;
    BOATCU_CHECK(cudaHostUnregister(host));
    return 0;
}

}  // extern "C"
