// norm_act.cu - LayerNorm forward/backward and GELU forward/backward: the HBM-bound kernels
// of the pre-LN encoder block around the attention layer.
//
// LayerNorm forward restates boat_layernorm_forward (reference src/layers/norm.c:231-317):
// per row, mean = sum/H, biased variance = sum((x-mean)^2)/H, y = (x-mean)/sqrt(var+eps)*w + b.
// The reference has no LayerNorm backward (norm.c:397-402 is a stub) and no GELU
// (src/ops/activation.c:298-302 is a stub); those follow the textbook formulas, with the
// exact erf form of GELU.  One CTA per row keeps the row in shared memory, so a row is read
// from HBM once per kernel; 128-bit accesses where the row length allows.
#include "common.cuh"

namespace boatcu {

static const int kNormThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
    // red: 32 floats of shared memory.  Returns the sum over the CTA in every thread.
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                       // protects `red` against the previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

template <typename T>
__device__ __forceinline__ void load_row(float* dst, const T* src, int cols) {
    if (sizeof(T) == 2 && (cols & 7) == 0) {
        for (int i = threadIdx.x; i < cols / 8; i += blockDim.x) {
            uint4 v = reinterpret_cast<const uint4*>(src)[i];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float2 f = __bfloat1622float2(h[k]);
                dst[8 * i + 2 * k] = f.x;
                dst[8 * i + 2 * k + 1] = f.y;
            }
        }
    } else if (sizeof(T) == 4 && (cols & 3) == 0) {
        for (int i = threadIdx.x; i < cols / 4; i += blockDim.x)
            reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < cols; i += blockDim.x) dst[i] = to_f32(src[i]);
    }
}

template <typename T>
__device__ __forceinline__ void store_row(T* dst, const float* src, int cols) {
    if (sizeof(T) == 2 && (cols & 7) == 0) {
        for (int i = threadIdx.x; i < cols / 8; i += blockDim.x) {
            uint4 o;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(src[8 * i], src[8 * i + 1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(src[8 * i + 2], src[8 * i + 3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(src[8 * i + 4], src[8 * i + 5]);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(src[8 * i + 6], src[8 * i + 7]);
            o.x = *reinterpret_cast<uint32_t*>(&h0);
            o.y = *reinterpret_cast<uint32_t*>(&h1);
            o.z = *reinterpret_cast<uint32_t*>(&h2);
            o.w = *reinterpret_cast<uint32_t*>(&h3);
            reinterpret_cast<uint4*>(dst)[i] = o;
        }
    } else if (sizeof(T) == 4 && (cols & 3) == 0) {
        for (int i = threadIdx.x; i < cols / 4; i += blockDim.x)
            reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < cols; i += blockDim.x) dst[i] = from_f32<T>(src[i]);
    }
}

// y = (x - mean) * rstd * gamma + beta, row statistics saved for the backward
template <typename T>
__global__ void __launch_bounds__(kNormThreads)
layernorm_fwd_kernel(const T* __restrict__ x, int cols, const float* __restrict__ gamma, const float* __restrict__ beta,
                     float eps, T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out) {
    extern __shared__ float row[];          // [cols] + 32
    float* red = row + cols;
    const int64_t r = blockIdx.x;
    load_row(row, x + r * cols, cols);
    __syncthreads();
    float s = 0.f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) s += row[i];
    const float mean = block_sum(s, red) / (float)cols;
    float v = 0.f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float d = row[i] - mean;
        v += d * d;
    }
    const float var = block_sum(v, red) / (float)cols;
    const float rstd = 1.0f / sqrtf(var + eps);
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float n = (row[i] - mean) * rstd;
        if (gamma) n = n * gamma[i];
        if (beta) n = n + beta[i];
        row[i] = n;
    }
    __syncthreads();
    store_row(y + r * cols, row, cols);
    if (threadIdx.x == 0) {
        if (mean_out) mean_out[r] = mean;
        if (rstd_out) rstd_out[r] = rstd;
    }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)),  g = dy * gamma,  xhat = (x - mean) * rstd
template <typename T>
__global__ void __launch_bounds__(kNormThreads)
layernorm_bwd_dx_kernel(const T* __restrict__ dy, const T* __restrict__ x, int cols, const float* __restrict__ gamma,
                        const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx) {
    extern __shared__ float smem[];         // g[cols], xhat[cols], 32
    float* g = smem;
    float* xh = smem + cols;
    float* red = xh + cols;
    const int64_t r = blockIdx.x;
    load_row(g, dy + r * cols, cols);
    load_row(xh, x + r * cols, cols);
    __syncthreads();
    const float m = mean[r], rs = rstd[r];
    float s1 = 0.f, s2 = 0.f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float gi = g[i] * (gamma ? gamma[i] : 1.f);
        float xi = (xh[i] - m) * rs;
        g[i] = gi;
        xh[i] = xi;
        s1 += gi;
        s2 += gi * xi;
    }
    const float mg = block_sum(s1, red) / (float)cols;
    const float mgx = block_sum(s2, red) / (float)cols;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) g[i] = rs * (g[i] - mg - xh[i] * mgx);
    __syncthreads();
    store_row(dx + r * cols, g, cols);
}

// dgamma[j] += sum_r dy[r,j] * xhat[r,j],  dbeta[j] += sum_r dy[r,j]   (outputs zeroed by the caller)
template <typename T>
__global__ void layernorm_bwd_params_kernel(const T* __restrict__ dy, const T* __restrict__ x, int64_t rows, int cols,
                                            const float* __restrict__ mean, const float* __restrict__ rstd,
                                            float* __restrict__ dgamma, float* __restrict__ dbeta) {
    __shared__ float pg[8][33], pb[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + tx;
    float ag = 0.f, ab = 0.f;
    if (col < cols) {
        for (int64_t r = (int64_t)blockIdx.y * 8 + ty; r < rows; r += (int64_t)gridDim.y * 8) {
            float d = to_f32(dy[r * cols + col]);
            float xh = (to_f32(x[r * cols + col]) - mean[r]) * rstd[r];
            ag += d * xh;
            ab += d;
        }
    }
    pg[ty][tx] = ag;
    pb[ty][tx] = ab;
    __syncthreads();
    if (ty == 0 && col < cols) {
        float sg = 0.f, sb = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            sg += pg[k][tx];
            sb += pb[k][tx];
        }
        if (dgamma) atomicAdd(dgamma + col, sg);
        if (dbeta) atomicAdd(dbeta + col, sb);
    }
}

// ---- GELU, exact erf form ------------------------------------------------------------------------
__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_grad_f(float x) {
    return 0.5f * (1.0f + erff(x * 0.70710678118654752f)) + x * 0.3989422804014327f * expf(-0.5f * x * x);
}

template <typename T, bool BWD>
__global__ void gelu_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ dy, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += step) {
        float v = to_f32(x[i]);
        out[i] = from_f32<T>(BWD ? to_f32(dy[i]) * gelu_grad_f(v) : gelu_f(v));
    }
}

// 8 BF16 or 4 FP32 per thread per access
template <typename T, bool BWD>
__global__ void gelu_vec_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ dy, int64_t nvec) {
    constexpr int V = 16 / sizeof(T);
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (; i < nvec; i += step) {
        uint4 xv = reinterpret_cast<const uint4*>(x)[i];
        uint4 dv = BWD ? reinterpret_cast<const uint4*>(dy)[i] : make_uint4(0, 0, 0, 0);
        const T* xe = reinterpret_cast<const T*>(&xv);
        const T* de = reinterpret_cast<const T*>(&dv);
        uint4 ov;
        T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
        for (int k = 0; k < V; ++k) {
            float v = to_f32(xe[k]);
            oe[k] = from_f32<T>(BWD ? to_f32(de[k]) * gelu_grad_f(v) : gelu_f(v));
        }
        reinterpret_cast<uint4*>(out)[i] = ov;
    }
}

static inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

template <typename T, bool BWD>
static int launch_gelu(void* out, const void* x, const void* dy, int64_t n) {
    constexpr int V = 16 / sizeof(T);
    const bool vec = (n % V) == 0 && aligned16(out) && aligned16(x) && (!BWD || aligned16(dy));
    int64_t items = vec ? n / V : n;
    int64_t blocks = ceil_div(items, 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    ProfileScope prof(BWD ? "gelu_bwd" : "gelu_fwd");
    if (vec)
        gelu_vec_kernel<T, BWD><<<(unsigned)blocks, 256, 0, stream()>>>((T*)out, (const T*)x, (const T*)dy, items);
    else
        gelu_kernel<T, BWD><<<(unsigned)blocks, 256, 0, stream()>>>((T*)out, (const T*)x, (const T*)dy, n);
    BOATCU_LAUNCH_OK("gelu");
    return 0;
}

}  // namespace boatcu

using namespace boatcu;

extern "C" {

int boat_cuda_layernorm_fwd(const void* x, int type, int64_t rows, int64_t cols, const float* gamma, const float* beta,
                            float eps, void* y, float* mean_out, float* rstd_out) {
    if (rows <= 0 || cols <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    if (cols > 12000) return set_error(50, "layernorm: row length %lld exceeds 12000", (long long)cols);
    if (rows > 0x7fffffffLL) return set_error(50, "layernorm: too many rows");
    size_t smem = ((size_t)cols + 32) * sizeof(float);
    ProfileScope prof("layernorm_fwd");
    if (type == BOAT_CUDA_BF16) {
        auto k = layernorm_fwd_kernel<__nv_bfloat16>;
        BOATCU_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<(unsigned)rows, kNormThreads, smem, stream()>>>((const __nv_bfloat16*)x, (int)cols, gamma, beta, eps,
                                                            (__nv_bfloat16*)y, mean_out, rstd_out);
    } else {
        auto k = layernorm_fwd_kernel<float>;
        BOATCU_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<(unsigned)rows, kNormThreads, smem, stream()>>>((const float*)x, (int)cols, gamma, beta, eps, (float*)y,
                                                            mean_out, rstd_out);
    }
    BOATCU_LAUNCH_OK("layernorm_fwd");
    return 0;
}

int boat_cuda_layernorm_bwd(const void* dy, const void* x, int type, int64_t rows, int64_t cols, const float* gamma,
                            const float* mean, const float* rstd, void* dx, float* dgamma, float* dbeta) {
    if (rows <= 0 || cols <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    if (cols > 12000) return set_error(50, "layernorm: row length %lld exceeds 12000", (long long)cols);
    size_t smem = (2 * (size_t)cols + 32) * sizeof(float);
    ProfileScope prof("layernorm_bwd");
    if (dgamma) BOATCU_CHECK(cudaMemsetAsync(dgamma, 0, (size_t)cols * sizeof(float), stream()));
    if (dbeta) BOATCU_CHECK(cudaMemsetAsync(dbeta, 0, (size_t)cols * sizeof(float), stream()));
    dim3 pgrid((unsigned)ceil_div(cols, 32), 1);
    int64_t want = 148 * 8 / pgrid.x, max_y = ceil_div(rows, 8);
    pgrid.y = (unsigned)(want < 1 ? 1 : (want > max_y ? max_y : want));
    if (type == BOAT_CUDA_BF16) {
        typedef __nv_bfloat16 bf;
        auto k = layernorm_bwd_dx_kernel<bf>;
        BOATCU_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<(unsigned)rows, kNormThreads, smem, stream()>>>((const bf*)dy, (const bf*)x, (int)cols, gamma, mean, rstd, (bf*)dx);
        BOATCU_LAUNCH_OK("layernorm_bwd_dx");
        if (dgamma || dbeta) {
            layernorm_bwd_params_kernel<bf><<<pgrid, 256, 0, stream()>>>((const bf*)dy, (const bf*)x, rows, (int)cols, mean, rstd, dgamma, dbeta);
            BOATCU_LAUNCH_OK("layernorm_bwd_params");
        }
    } else {
        auto k = layernorm_bwd_dx_kernel<float>;
        BOATCU_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<(unsigned)rows, kNormThreads, smem, stream()>>>((const float*)dy, (const float*)x, (int)cols, gamma, mean, rstd, (float*)dx);
        BOATCU_LAUNCH_OK("layernorm_bwd_dx");
        if (dgamma || dbeta) {
            layernorm_bwd_params_kernel<float><<<pgrid, 256, 0, stream()>>>((const float*)dy, (const float*)x, rows, (int)cols, mean, rstd, dgamma, dbeta);
            BOATCU_LAUNCH_OK("layernorm_bwd_params");
        }
    }
    return 0;
}

int boat_cuda_gelu_fwd(void* y, const void* x, int type, int64_t n) {
    if (n <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    return type == BOAT_CUDA_BF16 ? launch_gelu<__nv_bfloat16, false>(y, x, nullptr, n) : launch_gelu<float, false>(y, x, nullptr, n);
}

int boat_cuda_gelu_bwd(void* dx, const void* dy, const void* x, int type, int64_t n) {
    if (n <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    return type == BOAT_CUDA_BF16 ? launch_gelu<__nv_bfloat16, true>(dx, x, dy, n) : launch_gelu<float, true>(dx, x, dy, n);
}

}  // extern "C"
