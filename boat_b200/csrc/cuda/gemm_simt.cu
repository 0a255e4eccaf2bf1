// gemm_simt.cu - CUDA-core GEMM with FP32 accumulation for shapes the tensor-core kernels do
// not take (tiny or ragged problems) and for the exact-FP32 mode.  64x64 output tile per
// 256-thread CTA, 4x4 outputs per thread, K in steps of 16 through shared memory.
// Stands in for boat_matmul's triple loop (reference src/ops/linear.c:116-130).
#include "common.cuh"

namespace boatcu {

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(int ta, int tb, int64_t M, int64_t N, int64_t K, const TI* __restrict__ A, int64_t lda,
                 const TI* __restrict__ B, int64_t ldb, TO* __restrict__ C, int64_t ldc,
                 const float* __restrict__ bias) {
    __shared__ float As[16][64 + 4];
    __shared__ float Bs[16][64 + 4];
    const int tid = threadIdx.x;
    const int64_t m0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
    const int tr = (tid / 16) * 4, tc = (tid % 16) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int64_t k0 = 0; k0 < K; k0 += 16) {
        // 64x16 elements of each operand, 4 per thread.  The index split follows the
        // contiguous direction of the operand so that global reads coalesce.
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int idx = tid + e * 256;
            int mm, kk;
            if (ta) { mm = idx % 64; kk = idx / 64; } else { kk = idx % 16; mm = idx / 16; }
            int64_t gm = m0 + mm, gk = k0 + kk;
            float v = 0.f;
            if (gm < M && gk < K) v = to_f32(ta ? A[gk * lda + gm] : A[gm * lda + gk]);
            As[kk][mm] = v;
            int nn;
            if (tb) { kk = idx % 16; nn = idx / 16; } else { nn = idx % 64; kk = idx / 64; }
            int64_t gn = n0 + nn;
            gk = k0 + kk;
            v = 0.f;
            if (gn < N && gk < K) v = to_f32(tb ? B[gn * ldb + gk] : B[gk * ldb + gn]);
            Bs[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][tr + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tc + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int64_t gm = m0 + tr + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int64_t gn = n0 + tc + j;
            if (gn < N) C[gm * ldc + gn] = from_f32<TO>(acc[i][j] + (bias ? bias[gn] : 0.f));
        }
    }
}

int gemm_simt(int ta, int tb, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda, const void* B,
              int64_t ldb, int in_type, void* C, int64_t ldc, int out_type, const float* bias) {
    if (M <= 0 || N <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    dim3 grid((unsigned)ceil_div(N, 64), (unsigned)ceil_div(M, 64));
    if (grid.y > 65535) return set_error(7, "gemm_simt: M=%lld too large for this kernel", (long long)M);
    cudaStream_t s = stream();
    typedef __nv_bfloat16 bf;
    if (in_type != BOAT_CUDA_BF16 && out_type == BOAT_CUDA_F32_TF32)
        gemm_simt_kernel<float, f32_tf32><<<grid, 256, 0, s>>>(ta, tb, M, N, K, (const float*)A, lda, (const float*)B, ldb, (f32_tf32*)C, ldc, bias);
    else if (out_type == BOAT_CUDA_F32_TF32)
        gemm_simt_kernel<bf, f32_tf32><<<grid, 256, 0, s>>>(ta, tb, M, N, K, (const bf*)A, lda, (const bf*)B, ldb, (f32_tf32*)C, ldc, bias);
    else if (in_type != BOAT_CUDA_BF16 && out_type == BOAT_CUDA_F32)
        gemm_simt_kernel<float, float><<<grid, 256, 0, s>>>(ta, tb, M, N, K, (const float*)A, lda, (const float*)B, ldb, (float*)C, ldc, bias);
    else if (in_type != BOAT_CUDA_BF16)
        gemm_simt_kernel<float, bf><<<grid, 256, 0, s>>>(ta, tb, M, N, K, (const float*)A, lda, (const float*)B, ldb, (bf*)C, ldc, bias);
    else if (out_type == BOAT_CUDA_F32)
        gemm_simt_kernel<bf, float><<<grid, 256, 0, s>>>(ta, tb, M, N, K, (const bf*)A, lda, (const bf*)B, ldb, (float*)C, ldc, bias);
    else
        gemm_simt_kernel<bf, bf><<<grid, 256, 0, s>>>(ta, tb, M, N, K, (const bf*)A, lda, (const bf*)B, ldb, (bf*)C, ldc, bias);
    BOATCU_LAUNCH_OK("gemm_simt");
    return 0;
}

}  // namespace boatcu
