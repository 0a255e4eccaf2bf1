// attn_bwd_static.cu - attention-core backward for callers that must not allocate.
//
// boat_cuda_attn_bwd needs scratch memory from its caller (the per-row delta and, on the
// tensor-core path, the FP32 buffer in which dQ contributions are summed).  Some callers have
// nowhere to get it from: code running inside a region where the CUDA allocator may not be
// entered (a latency-critical serving loop that forbids cudaMalloc because it can synchronise
// the whole device, a host program whose memory budget is fixed up front, a plugin called
// from a framework that owns all device memory).  For them this file keeps one fixed scratch
// block inside the library image and offers an entry point that uses it.
//
// The block is a file-scope __device__ array: every GPU whose context loads this library
// holds kStaticScratchBytes of HBM for it until the process exits, used or not.
#include "common.cuh"

namespace boatcu {
namespace {

constexpr size_t kStaticScratchBytes = (size_t)16 << 20;      // 16 MiB, the stated maximum
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code the name g_static_scratch is only a handle for the runtime, not an address a
// kernel can use; the device address has to be asked for, once per device, with that device
// current.
void* g_scratch_addr[kMaxDevices];

int scratch_address(void** out) {
    // ensure_init() has made the library's device current for this thread; anything else here
    // would hand out another GPU's copy of the block.
    int dev = -1;
    BOATCU_CHECK(cudaGetDevice(&dev));
    if (dev != bound_device())
        return set_error(40, "boat_cuda_attn_bwd_static: current device %d is not the library's device %d", dev,
                         bound_device());
    if (dev < 0 || dev >= kMaxDevices) return set_error(40, "device index %d out of range", dev);
    if (!g_scratch_addr[dev]) {
        void* ptr = nullptr;
        BOATCU_CHECK(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (!ptr) return set_error(40, "cudaGetSymbolAddress gave no address for the static scratch block");
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace
}  // namespace boatcu

using namespace boatcu;

extern "C" {

size_t boat_cuda_attn_bwd_static_capacity(void) { return kStaticScratchBytes; }

int boat_cuda_attn_bwd_static(int mma, int64_t units, int64_t S, int64_t hs, int causal, float scale,
                              const void* Q, const void* K, const void* V, const void* O, const void* dO,
                              const float* lse, int io_type, void* dQ, void* dK, void* dV) {
    if (!ready())
        return set_error(41, "boat_cuda_attn_bwd_static: call boat_cuda_init first - this entry point never "
                             "initialises the library, because initialising allocates");
    if (int rc = ensure_init()) return rc;     // already initialised: only makes the bound device current
    if (units < 0 || S < 0 || hs < 0) return set_error(41, "boat_cuda_attn_bwd_static: negative size");
    const size_t need = boat_cuda_attn_bwd_scratch_bytes(mma, units, S, hs);
    if (need > kStaticScratchBytes)
        return set_error(42, "boat_cuda_attn_bwd_static: this problem needs %zu bytes of scratch, the built-in "
                             "block holds %zu; use boat_cuda_attn_bwd with your own scratch",
                         need, kStaticScratchBytes);
    void* scratch = nullptr;
    if (int rc = scratch_address(&scratch)) return rc;
    // Everything the kernels expect to start from zero (the dQ sum) is cleared by the call
    // below on the library stream before it is used; the delta part is fully rewritten.
    return boat_cuda_attn_bwd(mma, units, S, hs, causal, scale, Q, K, V, O, dO, lse, io_type, dQ, dK, dV, scratch,
                              kStaticScratchBytes);
}

}  // extern "C"
