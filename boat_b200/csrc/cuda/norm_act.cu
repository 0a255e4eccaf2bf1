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

// ---- one warp per row ------------------------------------------------------------------------------
// For rows of up to 2048 elements whose length is a multiple of 32 vectors of 16 bytes: a lane
// holds NV vectors of the row in registers, the row statistics are shuffle reductions, and a
// row costs no shared memory and no CTA barrier.  Lane l owns vectors l, l+32, l+64, ... so that
// every access of the warp is one contiguous run of 512 bytes.
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& v, float* f) {
    if (sizeof(T) == 2) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 t = __bfloat1622float2(h[k]);
            f[2 * k] = t.x;
            f[2 * k + 1] = t.y;
        }
    } else {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
}

template <typename T>
__device__ __forceinline__ uint4 pack16(const float* f) {
    uint4 o;
    if (sizeof(T) == 2) {
        __nv_bfloat162 h0 = __floats2bfloat162_rn(f[0], f[1]), h1 = __floats2bfloat162_rn(f[2], f[3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(f[4], f[5]), h3 = __floats2bfloat162_rn(f[6], f[7]);
        o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
        o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
    } else {
        o.x = __float_as_uint(f[0]); o.y = __float_as_uint(f[1]); o.z = __float_as_uint(f[2]); o.w = __float_as_uint(f[3]);
    }
    return o;
}

// V (4 or 8) consecutive floats of a parameter vector, 16-byte loads
template <int V>
__device__ __forceinline__ void load_param(const float* __restrict__ p, int c0, float* f) {
#pragma unroll
    for (int k = 0; k < V; k += 4) {
        const float4 t = *reinterpret_cast<const float4*>(p + c0 + k);
        f[k] = t.x; f[k + 1] = t.y; f[k + 2] = t.z; f[k + 3] = t.w;
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

constexpr int kNormRowsPerWarp = 4;          // consecutive rows per warp: gamma and beta are loaded once for them

template <typename T, int NV>
__global__ void __launch_bounds__(kNormThreads)
layernorm_fwd_warp_kernel(const T* __restrict__ x, int64_t rows, const float* __restrict__ gamma,
                          const float* __restrict__ beta, float eps, T* __restrict__ y, float* __restrict__ mean_out,
                          float* __restrict__ rstd_out) {
    constexpr int V = Vec16<T>::N, COLS = NV * 32 * V;
    const int lane = threadIdx.x & 31;
    const int64_t r0 = ((int64_t)blockIdx.x * (kNormThreads / 32) + (threadIdx.x >> 5)) * kNormRowsPerWarp;
    if (r0 >= rows) return;
    float gm[NV][V], bt[NV][V];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c0 = (i * 32 + lane) * V;
        if (gamma) load_param<V>(gamma, c0, gm[i]);
        if (beta) load_param<V>(beta, c0, bt[i]);
    }
#pragma unroll 1
    for (int rr = 0; rr < kNormRowsPerWarp; ++rr) {
        const int64_t r = r0 + rr;
        if (r >= rows) break;
        const uint4* src = reinterpret_cast<const uint4*>(x + r * COLS);
        float f[NV][V];
#pragma unroll
        for (int i = 0; i < NV; ++i) unpack16<T>(src[i * 32 + lane], f[i]);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
            for (int k = 0; k < V; ++k) s += f[i][k];
        const float mean = warp_sum(s) / (float)COLS;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const float d = f[i][k] - mean;
                q += d * d;
            }
        const float rstd = 1.0f / sqrtf(warp_sum(q) / (float)COLS + eps);
        uint4* dst = reinterpret_cast<uint4*>(y + r * COLS);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
#pragma unroll
            for (int k = 0; k < V; ++k) {
                float n = (f[i][k] - mean) * rstd;
                if (gamma) n = n * gm[i][k];
                if (beta) n = n + bt[i][k];
                f[i][k] = n;
            }
            dst[i * 32 + lane] = pack16<T>(f[i]);
        }
        if (lane == 0) {
            if (mean_out) mean_out[r] = mean;
            if (rstd_out) rstd_out[r] = rstd;
        }
    }
}

// dx as in layernorm_bwd_dx_kernel; in the same pass every warp sums dy*xhat and dy over the
// rows it walks (a grid-stride loop), per column, in registers; warps of a CTA combine in
// shared memory and CTAs by atomicAdd into the zeroed dgamma / dbeta - dy and x are read once.
template <typename T, int NV>
__global__ void __launch_bounds__(kNormThreads)
layernorm_bwd_warp_kernel(const T* __restrict__ dy, const T* __restrict__ x, int64_t rows,
                          const float* __restrict__ gamma, const float* __restrict__ mean,
                          const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dgamma,
                          float* __restrict__ dbeta) {
    constexpr int V = Vec16<T>::N, COLS = NV * 32 * V;
    extern __shared__ float part[];                 // [2][COLS] when parameter gradients are wanted
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool params = dgamma != nullptr || dbeta != nullptr;
    if (params) {
        for (int i = threadIdx.x; i < 2 * COLS; i += blockDim.x) part[i] = 0.f;
        __syncthreads();
    }
    float ag[NV][V], ab[NV][V];
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int k = 0; k < V; ++k) ag[i][k] = ab[i][k] = 0.f;
    const int64_t stride = (int64_t)gridDim.x * (kNormThreads / 32);
    for (int64_t r = (int64_t)blockIdx.x * (kNormThreads / 32) + warp; r < rows; r += stride) {
        const uint4* gsrc = reinterpret_cast<const uint4*>(dy + r * COLS);
        const uint4* xsrc = reinterpret_cast<const uint4*>(x + r * COLS);
        float g[NV][V], xh[NV][V];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            unpack16<T>(gsrc[i * 32 + lane], g[i]);
            unpack16<T>(xsrc[i * 32 + lane], xh[i]);
        }
        const float m = mean[r], rs = rstd[r];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            float gm[V];
            if (gamma) load_param<V>(gamma, (i * 32 + lane) * V, gm);
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const float xi = (xh[i][k] - m) * rs;
                const float d = g[i][k];
                ag[i][k] += d * xi;
                ab[i][k] += d;
                const float gi = gamma ? d * gm[k] : d;
                g[i][k] = gi;
                xh[i][k] = xi;
                s1 += gi;
                s2 += gi * xi;
            }
        }
        const float mg = warp_sum(s1) / (float)COLS, mgx = warp_sum(s2) / (float)COLS;
        uint4* dst = reinterpret_cast<uint4*>(dx + r * COLS);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
#pragma unroll
            for (int k = 0; k < V; ++k) g[i][k] = rs * (g[i][k] - mg - xh[i][k] * mgx);
            dst[i * 32 + lane] = pack16<T>(g[i]);
        }
    }
    if (!params) return;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c0 = (i * 32 + lane) * V;
#pragma unroll
        for (int k = 0; k < V; ++k) {
            atomicAdd(part + c0 + k, ag[i][k]);
            atomicAdd(part + COLS + c0 + k, ab[i][k]);
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < COLS; c += blockDim.x) {
        if (dgamma) atomicAdd(dgamma + c, part[c]);
        if (dbeta) atomicAdd(dbeta + c, part[COLS + c]);
    }
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
// Phi(x) = (1 + erf(x/sqrt 2))/2 and e = exp(-x^2/2) from one exponential: erf by Abramowitz &
// Stegun 7.1.26, erf(z) = 1 - (a1 t + ... + a5 t^5) exp(-z^2), t = 1/(1 + p z), |error| <= 1.5e-7,
// whose exponential at z = |x|/sqrt 2 is the exp(-x^2/2) that the derivative needs anyway.
// erff + expf cost ~40 instructions per element and made these kernels instruction-bound
// (55 % of HBM bandwidth); this form needs one ex2, one rcp and a dozen FMAs.
__device__ __forceinline__ void gelu_parts(float x, float& phi, float& e) {
    const float z = fabsf(x) * 0.70710678118654752f;
    // one MUFU instruction each (relative error ~2^-22, far inside the 1.5e-7 of the formula)
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-0.72134752044448170f * x * x));   // exp(-x^2/2)
    float t;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.0f)));
    float poly = fmaf(1.061405429f, t, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    const float half_erfc = 0.5f * poly * t * e;                   // (1 - erf(z)) / 2
    phi = x >= 0.f ? 1.0f - half_erfc : half_erfc;
}
__device__ __forceinline__ float gelu_f(float x) {
    float phi, e;
    gelu_parts(x, phi, e);
    return x * phi;
}
__device__ __forceinline__ float gelu_grad_f(float x) {
    float phi, e;
    gelu_parts(x, phi, e);
    return fmaf(x * 0.3989422804014327f, e, phi);
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

// 8 BF16 or 4 FP32 per 16-byte access; a thread issues the loads of kGeluUnroll accesses (a CTA
// covers kGeluUnroll consecutive runs of 256 vectors) before it computes, to keep enough bytes in
// flight with one or two input streams.
constexpr int kGeluUnroll = 4;
template <typename T, bool BWD>
__global__ void __launch_bounds__(256)
gelu_vec_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ dy, int64_t nvec) {
    constexpr int V = 16 / sizeof(T);
    const int64_t chunk = (int64_t)gridDim.x * 256 * kGeluUnroll;
    for (int64_t base = (int64_t)blockIdx.x * 256 * kGeluUnroll + threadIdx.x; base < nvec; base += chunk) {
        uint4 xv[kGeluUnroll], dv[kGeluUnroll];
#pragma unroll
        for (int u = 0; u < kGeluUnroll; ++u) {
            const int64_t i = base + u * 256;
            if (i < nvec) {
                xv[u] = reinterpret_cast<const uint4*>(x)[i];
                if (BWD) dv[u] = reinterpret_cast<const uint4*>(dy)[i];
            }
        }
#pragma unroll
        for (int u = 0; u < kGeluUnroll; ++u) {
            const int64_t i = base + u * 256;
            if (i >= nvec) break;
            const T* xe = reinterpret_cast<const T*>(&xv[u]);
            const T* de = reinterpret_cast<const T*>(&dv[u]);
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
}

static inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

template <typename T, bool BWD>
static int launch_gelu(void* out, const void* x, const void* dy, int64_t n) {
    constexpr int V = 16 / sizeof(T);
    const bool vec = (n % V) == 0 && aligned16(out) && aligned16(x) && (!BWD || aligned16(dy));
    int64_t items = vec ? n / V : n;
    int64_t blocks = ceil_div(items, vec ? 256 * kGeluUnroll : 256);   // the loops are grid-stride
    if (blocks > 0x7fffffffLL) blocks = 0x7fffffffLL;
    ProfileScope prof(BWD ? "gelu_bwd" : "gelu_fwd");
    if (vec)
        gelu_vec_kernel<T, BWD><<<(unsigned)blocks, 256, 0, stream()>>>((T*)out, (const T*)x, (const T*)dy, items);
    else
        gelu_kernel<T, BWD><<<(unsigned)blocks, 256, 0, stream()>>>((T*)out, (const T*)x, (const T*)dy, n);
    BOATCU_LAUNCH_OK("gelu");
    return 0;
}

// Warp-per-row dispatch.  Returns 0 when the shape is not covered (the caller falls back to
// the CTA-per-row kernels), -1 after a successful launch, an error status otherwise.
template <typename T, int NV>
static int fwd_warp_launch(const void* x, int64_t rows, const float* gamma, const float* beta, float eps, void* y,
                           float* mean_out, float* rstd_out) {
    const int64_t blocks = ceil_div(rows, (kNormThreads / 32) * kNormRowsPerWarp);
    layernorm_fwd_warp_kernel<T, NV><<<(unsigned)blocks, kNormThreads, 0, stream()>>>((const T*)x, rows, gamma, beta, eps,
                                                                                       (T*)y, mean_out, rstd_out);
    BOATCU_LAUNCH_OK("layernorm_fwd_warp");
    return -1;
}

template <typename T, int NV>
static int bwd_warp_launch(const void* dy, const void* x, int64_t rows, const float* gamma, const float* mean,
                           const float* rstd, void* dx, float* dgamma, float* dbeta) {
    constexpr int COLS = NV * 32 * (16 / (int)sizeof(T));
    int64_t blocks = ceil_div(rows, kNormThreads / 32);
    if (blocks > sm_count() * 4) blocks = sm_count() * 4;         // persistent: the column sums live in registers across rows
    const size_t smem = (dgamma || dbeta) ? 2 * COLS * sizeof(float) : 0;
    layernorm_bwd_warp_kernel<T, NV><<<(unsigned)blocks, kNormThreads, smem, stream()>>>(
        (const T*)dy, (const T*)x, rows, gamma, mean, rstd, (T*)dx, dgamma, dbeta);
    BOATCU_LAUNCH_OK("layernorm_bwd_warp");
    return -1;
}

static int warp_nv(int type, int64_t cols, const void* a, const void* b, const void* c) {
    const int v = type == BOAT_CUDA_BF16 ? 8 : 4;
    if (cols % (32 * v) != 0) return 0;
    const int64_t nv = cols / (32 * v);
    if (nv != 1 && nv != 2 && nv != 4 && nv != 8) return 0;
    if ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) != 0) return 0;
    return (int)nv;
}

static int layernorm_fwd_warp(const void* x, int type, int64_t rows, int64_t cols, const float* gamma, const float* beta,
                              float eps, void* y, float* mean_out, float* rstd_out) {
    typedef __nv_bfloat16 bf;
    const int nv = warp_nv(type, cols, x, y, nullptr);
#define BOAT_LN_FWD(T, NV) case NV: return fwd_warp_launch<T, NV>(x, rows, gamma, beta, eps, y, mean_out, rstd_out)
    if (type == BOAT_CUDA_BF16) {
        switch (nv) { BOAT_LN_FWD(bf, 1); BOAT_LN_FWD(bf, 2); BOAT_LN_FWD(bf, 4); BOAT_LN_FWD(bf, 8); default: return 0; }
    }
    switch (nv) { BOAT_LN_FWD(float, 1); BOAT_LN_FWD(float, 2); BOAT_LN_FWD(float, 4); BOAT_LN_FWD(float, 8); default: return 0; }
#undef BOAT_LN_FWD
}

static int layernorm_bwd_warp(const void* dy, const void* x, int type, int64_t rows, int64_t cols, const float* gamma,
                              const float* mean, const float* rstd, void* dx, float* dgamma, float* dbeta) {
    typedef __nv_bfloat16 bf;
    const int nv = warp_nv(type, cols, dy, x, dx);
    if (nv > 4) return 0;                           // 8 vectors x 4 live arrays would spill
#define BOAT_LN_BWD(T, NV) case NV: return bwd_warp_launch<T, NV>(dy, x, rows, gamma, mean, rstd, dx, dgamma, dbeta)
    if (type == BOAT_CUDA_BF16) {
        switch (nv) { BOAT_LN_BWD(bf, 1); BOAT_LN_BWD(bf, 2); BOAT_LN_BWD(bf, 4); default: return 0; }
    }
    switch (nv) { BOAT_LN_BWD(float, 1); BOAT_LN_BWD(float, 2); BOAT_LN_BWD(float, 4); default: return 0; }
#undef BOAT_LN_BWD
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
    if (int done = layernorm_fwd_warp(x, type, rows, cols, gamma, beta, eps, y, mean_out, rstd_out)) return done < 0 ? 0 : done;
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
    if (int done = layernorm_bwd_warp(dy, x, type, rows, cols, gamma, mean, rstd, dx, dgamma, dbeta)) return done < 0 ? 0 : done;
    dim3 pgrid((unsigned)ceil_div(cols, 32), 1);
    int64_t want = (int64_t)sm_count() * 8 / pgrid.x, max_y = ceil_div(rows, 8);
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
