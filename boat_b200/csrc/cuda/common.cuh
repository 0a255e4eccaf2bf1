// common.cuh - shared helpers for the sm_100a kernels: status handling, launch accounting,
// storage-type helpers.  Internal to the CUDA backend.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include "boat_cuda.h"

namespace boatcu {

// Records a failure text for boat_cuda_last_error() and returns the status to hand back.
int set_error(int status, const char* fmt, ...);
cudaStream_t stream();
void count_launch(int n = 1);
int ensure_init();
bool ready();          // has boat_cuda_init (or a first call) bound the library to a device yet?
int bound_device();    // index of that device, -1 before
int sm_count();        // its number of SMs (grid sizing); 1 before the library is bound
int comm_stream_sync();   // waits for gradient sums still running on the communication stream

// Optional per-kernel timing (boat_cuda_profile_*): while enabled, a scope records a CUDA
// event pair on the library stream around the launches it encloses.
struct ProfileScope {
    explicit ProfileScope(const char* name);
    ~ProfileScope();
    int slot;
};

#define BOATCU_CHECK(expr)                                                          \
    do {                                                                            \
        cudaError_t err__ = (expr);                                                 \
        if (err__ != cudaSuccess)                                                   \
            return boatcu::set_error(1000 + (int)err__, "%s failed: %s (%s:%d)",   \
                                     #expr, cudaGetErrorString(err__), __FILE__, __LINE__); \
    } while (0)

// After a kernel launch: catches bad launch configurations without synchronising.
#define BOATCU_LAUNCH_OK(name)                                                      \
    do {                                                                            \
        cudaError_t err__ = cudaGetLastError();                                     \
        if (err__ != cudaSuccess)                                                   \
            return boatcu::set_error(1000 + (int)err__, "launch of %s failed: %s", \
                                     name, cudaGetErrorString(err__));              \
        boatcu::count_launch();                                                     \
    } while (0)

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

inline size_t type_size(int t) { return t == BOAT_CUDA_BF16 ? 2 : 4; }

// FP32 value rounded to the nearest TF32 number (ties away from zero), still an FP32 bit pattern.
__device__ __forceinline__ float round_to_tf32(float v) {
    uint32_t t;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(v));
    return __uint_as_float(t);
}
// Output element of BOAT_CUDA_F32_TF32: stored as float, rounded on conversion.
struct f32_tf32 { float v; };
template <> __device__ __forceinline__ f32_tf32 from_f32<f32_tf32>(float v) { return f32_tf32{round_to_tf32(v)}; }

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// out[r] = sum_d A[r,d]*B[r,d] over [rows, cols] row-major buffers of storage type `type`.
int rowdot(const void* A, const void* B, int type, int64_t rows, int64_t cols, float* out);
// The same pass emitting what the BF16 tensor-core backward reads per row:
// delta2_out[r] = -scale * sum_d dO[r,d]*O[r,d] and lse2_out[r] = -lse[r] * log2(e).
int rowdot_stats(const void* dO, const void* O, int type, int64_t rows, int64_t cols, const float* lse, float scale,
                 float* delta2_out, float* lse2_out);

// CUDA-core (exact FP32 accumulate) implementations, any shape.
int gemm_simt(int trans_a, int trans_b, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
              const void* B, int64_t ldb, int in_type, void* C, int64_t ldc, int out_type, const float* bias);
int attn_fwd_simt(int64_t units, int64_t S, int64_t hs, int causal, float scale, const void* Q, const void* K,
                  const void* V, int io_type, void* O, float* lse);
int attn_bwd_simt(int64_t units, int64_t S, int64_t hs, int causal, float scale, const void* Q, const void* K,
                  const void* V, const void* dO, const float* lse, const float* delta, int io_type,
                  void* dQ, void* dK, void* dV);

// tcgen05 implementations; return -1 (without setting an error) when the shape is outside
// what the tensor-core kernels cover, so that the dispatcher can say so.
bool gemm_tc_supported(int mma, int trans_a, int trans_b, int64_t M, int64_t N, int64_t K, const void* A,
                       int64_t lda, const void* B, int64_t ldb, int in_type, const void* C, int64_t ldc,
                       int out_type);
int gemm_tc(int mma, int trans_a, int trans_b, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
            const void* B, int64_t ldb, int in_type, void* C, int64_t ldc, int out_type, const float* bias);
void gemm_tc_set_yielding(bool on);
// `groups` (1..4) problems of one shape, layout and type in one launch; bias may be NULL or hold NULLs.
int gemm_tc_grouped(int mma, int trans_a, int trans_b, int groups, int64_t M, int64_t N, int64_t K,
                    const void* const* A, int64_t lda, const void* const* B, int64_t ldb, void* const* C,
                    int64_t ldc, int out_type, const float* const* bias);

}  // namespace boatcu
