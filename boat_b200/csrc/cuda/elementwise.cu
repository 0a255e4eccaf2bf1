// elementwise.cu - the HBM-bound tail of the attention step: bias/grad element-wise work,
// column sums for bias gradients, FP32<->BF16 casts, the row dot product delta = sum(dO*O)
// and a tiled transpose.  Every kernel moves 128 bits per thread per access when the
// pointers and sizes allow it and falls back to scalar accesses otherwise; reductions use
// warp shuffles.  Reference counterparts are named per function in boat_cuda.h.
#include "common.cuh"

namespace boatcu {

static const int kThreads = 256;

// One CTA per 256 work items, no persistent cap: for these streaming kernels the hardware's
// CTA scheduler balances better than a grid-stride loop over 8 CTAs per SM (measured on the
// Adam step: 6.3 TB/s against 5.3 TB/s).  The kernels keep their grid-stride loops, so the
// limit of the grid's x dimension only matters beyond 2^31 * 256 items.
static inline int grid_for(int64_t work_items, int per_block) {
    int64_t blocks = ceil_div(work_items, per_block);
    if (blocks > 0x7fffffffLL) blocks = 0x7fffffffLL;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

static inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// Rounded product, then rounded sum - deliberately not an FMA: the reference's SGD step is
// p - fl(g*lr) (boat_mul_scalar then boat_sub_), and with alpha = -lr this reproduces it
// bit for bit.
__device__ __forceinline__ float mul_add(float alpha, float x, float y) { return __fadd_rn(__fmul_rn(alpha, x), y); }

// ---- y = alpha*x (+ y), 4 floats per access -------------------------------------------
template <bool ACCUM>
__global__ void axpy_vec4(float* __restrict__ y, const float* __restrict__ x, float alpha, int64_t n4) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t step = (int64_t)gridDim.x * blockDim.x;
    float4* y4 = reinterpret_cast<float4*>(y);
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (; i < n4; i += step) {
        float4 a = x4[i];
        float4 r;
        if (ACCUM) {
            float4 b = y4[i];
            r = make_float4(mul_add(alpha, a.x, b.x), mul_add(alpha, a.y, b.y), mul_add(alpha, a.z, b.z), mul_add(alpha, a.w, b.w));
        } else {
            r = make_float4(alpha * a.x, alpha * a.y, alpha * a.z, alpha * a.w);
        }
        y4[i] = r;
    }
}

template <bool ACCUM>
__global__ void axpy_scalar(float* __restrict__ y, const float* __restrict__ x, float alpha, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += step) y[i] = ACCUM ? mul_add(alpha, x[i], y[i]) : alpha * x[i];
}

template <bool ACCUM>
static int launch_axpy(float* y, const float* x, float alpha, int64_t n) {
    if (n <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    if (aligned16(y) && aligned16(x) && (n % 4) == 0) {
        axpy_vec4<ACCUM><<<grid_for(n / 4, kThreads), kThreads, 0, stream()>>>(y, x, alpha, n / 4);
    } else {
        axpy_scalar<ACCUM><<<grid_for(n, kThreads), kThreads, 0, stream()>>>(y, x, alpha, n);
    }
    BOATCU_LAUNCH_OK("axpy");
    return 0;
}

// ---- y = a * b -------------------------------------------------------------------------------
__global__ void mul_kernel(float* __restrict__ y, const float* __restrict__ a, const float* __restrict__ b,
                           int64_t n, int vec) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t step = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        int64_t n4 = n / 4;
        for (; i < n4; i += step) {
            float4 p = reinterpret_cast<const float4*>(a)[i];
            float4 q = reinterpret_cast<const float4*>(b)[i];
            reinterpret_cast<float4*>(y)[i] = make_float4(p.x * q.x, p.y * q.y, p.z * q.z, p.w * q.w);
        }
    } else {
        for (; i < n; i += step) y[i] = a[i] * b[i];
    }
}

// ---- y[i,j] = x[i,j] + bias[j] ---------------------------------------------------------------
__global__ void add_bias_kernel(float* __restrict__ y, const float* __restrict__ x,
                                const float* __restrict__ bias, int64_t rows, int64_t cols, int vec) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t step = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        int64_t c4 = cols / 4, n4 = rows * c4;
        for (; i < n4; i += step) {
            float4 v = reinterpret_cast<const float4*>(x)[i];
            float4 b = reinterpret_cast<const float4*>(bias)[i % c4];
            reinterpret_cast<float4*>(y)[i] = make_float4(v.x + b.x, v.y + b.y, v.z + b.z, v.w + b.w);
        }
    } else {
        int64_t n = rows * cols;
        for (; i < n; i += step) y[i] = x[i] + bias[i % cols];
    }
}

// ---- y = alpha*a + beta*b on FP32 or BF16 storage (residual adds, differences, MSE gradient) ----
template <typename T>
__global__ void lincomb_kernel(T* __restrict__ y, const T* __restrict__ a, float alpha, const T* __restrict__ b,
                               float beta, int64_t n, int vec) {
    constexpr int V = 16 / sizeof(T);
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        const int64_t nv = n / V;
        for (; i < nv; i += step) {
            uint4 av = reinterpret_cast<const uint4*>(a)[i], bv = reinterpret_cast<const uint4*>(b)[i], ov;
            const T* ae = reinterpret_cast<const T*>(&av);
            const T* be = reinterpret_cast<const T*>(&bv);
            T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
            for (int k = 0; k < V; ++k) oe[k] = from_f32<T>(alpha * to_f32(ae[k]) + beta * to_f32(be[k]));
            reinterpret_cast<uint4*>(y)[i] = ov;
        }
    } else {
        for (; i < n; i += step) y[i] = from_f32<T>(alpha * to_f32(a[i]) + beta * to_f32(b[i]));
    }
}

// ---- casts -----------------------------------------------------------------------------------
__global__ void cast_f32_to_bf16(__nv_bfloat16* __restrict__ dst, const float* __restrict__ src, int64_t n, int vec) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t step = (int64_t)gridDim.x * blockDim.x;
    if (vec) {   // 8 elements: two 128-bit loads, one 128-bit store
        int64_t n8 = n / 8;
        for (; i < n8; i += step) {
            float4 a = reinterpret_cast<const float4*>(src)[2 * i];
            float4 b = reinterpret_cast<const float4*>(src)[2 * i + 1];
            __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
            uint4 o;
            o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
            o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
            reinterpret_cast<uint4*>(dst)[i] = o;
        }
    } else {
        for (; i < n; i += step) dst[i] = __float2bfloat16_rn(src[i]);
    }
}

__global__ void cast_bf16_to_f32(float* __restrict__ dst, const __nv_bfloat16* __restrict__ src, int64_t n, int vec) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t step = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        int64_t n8 = n / 8;
        for (; i < n8; i += step) {
            uint4 v = reinterpret_cast<const uint4*>(src)[i];
            __nv_bfloat162 p0 = *reinterpret_cast<__nv_bfloat162*>(&v.x), p1 = *reinterpret_cast<__nv_bfloat162*>(&v.y);
            __nv_bfloat162 p2 = *reinterpret_cast<__nv_bfloat162*>(&v.z), p3 = *reinterpret_cast<__nv_bfloat162*>(&v.w);
            float2 f0 = __bfloat1622float2(p0), f1 = __bfloat1622float2(p1);
            float2 f2 = __bfloat1622float2(p2), f3 = __bfloat1622float2(p3);
            reinterpret_cast<float4*>(dst)[2 * i] = make_float4(f0.x, f0.y, f1.x, f1.y);
            reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(f2.x, f2.y, f3.x, f3.y);
        }
    } else {
        for (; i < n; i += step) dst[i] = __bfloat162float(src[i]);
    }
}

// ---- y = x rounded to the nearest TF32 value (10-bit mantissa), still stored as FP32 -------------
// tcgen05 kind::tf32 drops the low 13 mantissa bits of its operands; a chain of contractions
// then drifts by a systematic ~2^-11 per stage.  Rounding operands to nearest beforehand
// makes the truncation exact and the error unbiased.
__device__ __forceinline__ float round_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

__global__ void round_tf32_kernel(float* __restrict__ y, const float* __restrict__ x, int64_t n, int vec) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t step = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        int64_t n4 = n / 4;
        for (; i < n4; i += step) {
            float4 v = reinterpret_cast<const float4*>(x)[i];
            reinterpret_cast<float4*>(y)[i] = make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
        }
    } else {
        for (; i < n; i += step) y[i] = round_tf32(x[i]);
    }
}

// ---- several FP32 tensors to BF16 or to TF32-valued FP32, one launch ----------------------------
constexpr int kMaxConvert = 8;
struct ConvertTable {
    const float* src[kMaxConvert];
    void* dst[kMaxConvert];
    int64_t n[kMaxConvert];
};

// blockIdx.y = tensor; vec: every tensor is 16-byte aligned with a multiple of 8 elements
template <bool TO_BF16>
__global__ void convert_multi_kernel(const ConvertTable t, int vec) {
    const float* __restrict__ src = t.src[blockIdx.y];
    const int64_t n = t.n[blockIdx.y];
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        const int64_t n8 = n / 8;
        for (; i < n8; i += step) {
            const float4 a = reinterpret_cast<const float4*>(src)[2 * i];
            const float4 b = reinterpret_cast<const float4*>(src)[2 * i + 1];
            if (TO_BF16) {
                __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
                uint4 o;
                o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
                o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
                reinterpret_cast<uint4*>(t.dst[blockIdx.y])[i] = o;
            } else {
                float4* d = reinterpret_cast<float4*>(t.dst[blockIdx.y]);
                d[2 * i] = make_float4(round_tf32(a.x), round_tf32(a.y), round_tf32(a.z), round_tf32(a.w));
                d[2 * i + 1] = make_float4(round_tf32(b.x), round_tf32(b.y), round_tf32(b.z), round_tf32(b.w));
            }
        }
    } else {
        for (; i < n; i += step) {
            if (TO_BF16) ((__nv_bfloat16*)t.dst[blockIdx.y])[i] = __float2bfloat16_rn(src[i]);
            else         ((float*)t.dst[blockIdx.y])[i] = round_tf32(src[i]);
        }
    }
}

// ---- column sums: out[j] += sum_i X[i,j] -----------------------------------------------------
// Block = 32 column lanes x 8 row lanes; a column lane owns VEC adjacent columns.  Row lanes
// are combined through shared memory, blocks through atomicAdd into a zeroed output.
// blockIdx.z selects one of several matrices of the same shape.
constexpr int kMaxColsum = 4;
struct ColsumTable {
    const void* x[kMaxColsum];
    float* out[kMaxColsum];
};

template <typename T, int VEC>
__global__ void colsum_kernel(const ColsumTable t, int64_t rows, int64_t cols) {
    const T* __restrict__ X = (const T*)t.x[blockIdx.z];
    float* __restrict__ out = t.out[blockIdx.z];
    __shared__ float part[8][32 * VEC + 1];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t col0 = ((int64_t)blockIdx.x * 32 + tx) * VEC;
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
    if (col0 < cols) {
        for (int64_t r = (int64_t)blockIdx.y * 8 + ty; r < rows; r += (int64_t)gridDim.y * 8) {
            const T* p = X + r * cols + col0;
            if (VEC == 1) {
                acc[0] += to_f32(p[0]);
            } else if (sizeof(T) == 4) {      // VEC == 4
                float4 v = *reinterpret_cast<const float4*>(p);
                acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
            } else {                          // bf16, VEC == 8
                uint4 v = *reinterpret_cast<const uint4*>(p);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float2 f = __bfloat1622float2(h[k]);
                    acc[2 * k] += f.x; acc[2 * k + 1] += f.y;
                }
            }
        }
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) part[ty][tx * VEC + v] = acc[v];
    __syncthreads();
    // 256 threads fold the 8 row lanes of 32*VEC columns
    for (int c = threadIdx.x; c < 32 * VEC; c += blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) s += part[k][c];
        int64_t col = (int64_t)blockIdx.x * 32 * VEC + c;
        if (col < cols) atomicAdd(out + col, s);
    }
}

// ---- delta[r] = sum_d dO[r,d] * O[r,d]: one warp per row, shuffle reduction --------------------
// With `lse2_out` the kernel emits the two per-row statistics in the form the BF16 backward's inner
// loops consume them (one FMA each): out[r] = -delta[r] * scale and lse2_out[r] = -lse[r] * log2(e).
struct RowStats {
    const float* lse;
    float* lse2_out;
    float scale;
};
__device__ __forceinline__ void emit_row(float* __restrict__ out, const RowStats& st, int64_t row, float s) {
    if (st.lse2_out) {
        out[row] = s * -st.scale;
        st.lse2_out[row] = st.lse[row] * -1.4426950408889634f;
    } else {
        out[row] = s;
    }
}

template <typename T>
__global__ void rowdot_kernel(const T* __restrict__ A, const T* __restrict__ B, int64_t rows, int cols,
                              float* __restrict__ out, const RowStats st) {
    const int lane = threadIdx.x & 31;
    int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t step = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (; row < rows; row += step) {
        const T* a = A + row * cols;
        const T* b = B + row * cols;
        float s = 0.f;
        for (int d = lane; d < cols; d += 32) s += to_f32(a[d]) * to_f32(b[d]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) emit_row(out, st, row, s);
    }
}

// 128-bit variant: 8 bf16 (or 4 floats) per lane per access; cols must divide accordingly.
template <typename T, int VEC>
__global__ void rowdot_vec_kernel(const T* __restrict__ A, const T* __restrict__ B, int64_t rows, int cols,
                                  float* __restrict__ out, const RowStats st) {
    const int lanes_per_row = cols / VEC;            // power of two <= 32 checked by the launcher
    const int rows_per_warp = 32 / lanes_per_row;
    const int lane = threadIdx.x & 31;
    const int sub = lane / lanes_per_row, l = lane % lanes_per_row;
    int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t base = warp * rows_per_warp; base < rows; base += nwarps * rows_per_warp) {
        int64_t row = base + sub;
        float s = 0.f;
        if (row < rows) {
            const uint4 va = *reinterpret_cast<const uint4*>(A + row * cols + l * VEC);
            const uint4 vb = *reinterpret_cast<const uint4*>(B + row * cols + l * VEC);
            if (sizeof(T) == 4) {
                const float* fa = reinterpret_cast<const float*>(&va);
                const float* fb = reinterpret_cast<const float*>(&vb);
#pragma unroll
                for (int k = 0; k < 4; ++k) s += fa[k] * fb[k];
            } else {
                const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&va);
                const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&vb);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float2 x = __bfloat1622float2(ha[k]), y = __bfloat1622float2(hb[k]);
                    s += x.x * y.x + x.y * y.y;
                }
            }
        }
        for (int o = lanes_per_row >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (l == 0 && row < rows) emit_row(out, st, row, s);
    }
}

static int rowdot_launch(const void* A, const void* B, int type, int64_t rows, int64_t cols, float* out, const RowStats st) {
    if (rows <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    const int vec = type == BOAT_CUDA_BF16 ? 8 : 4;
    int64_t lpr = cols / vec;
    bool pow2 = lpr > 0 && (lpr & (lpr - 1)) == 0;
    if (cols % vec == 0 && pow2 && lpr <= 32 && aligned16(A) && aligned16(B)) {
        int rows_per_block = (kThreads / 32) * (int)(32 / lpr);
        int grid = grid_for(rows, rows_per_block);
        if (type == BOAT_CUDA_BF16)
            rowdot_vec_kernel<__nv_bfloat16, 8><<<grid, kThreads, 0, stream()>>>(
                (const __nv_bfloat16*)A, (const __nv_bfloat16*)B, rows, (int)cols, out, st);
        else
            rowdot_vec_kernel<float, 4><<<grid, kThreads, 0, stream()>>>((const float*)A, (const float*)B, rows, (int)cols, out, st);
    } else {
        int grid = grid_for(rows, kThreads / 32);
        if (type == BOAT_CUDA_BF16)
            rowdot_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream()>>>(
                (const __nv_bfloat16*)A, (const __nv_bfloat16*)B, rows, (int)cols, out, st);
        else
            rowdot_kernel<float><<<grid, kThreads, 0, stream()>>>((const float*)A, (const float*)B, rows, (int)cols, out, st);
    }
    BOATCU_LAUNCH_OK("rowdot");
    return 0;
}

int rowdot(const void* A, const void* B, int type, int64_t rows, int64_t cols, float* out) {
    return rowdot_launch(A, B, type, rows, cols, out, RowStats{nullptr, nullptr, 0.f});
}

int rowdot_stats(const void* dO, const void* O, int type, int64_t rows, int64_t cols, const float* lse, float scale,
                 float* delta2_out, float* lse2_out) {
    return rowdot_launch(dO, O, type, rows, cols, delta2_out, RowStats{lse, lse2_out, scale});
}

// ---- out[b, j, i] = in[b, i, j], 32x32 shared-memory tiles --------------------------------------
__global__ void transpose_kernel(float* __restrict__ out, const float* __restrict__ in, int64_t rows, int64_t cols) {
    __shared__ float tile[32][33];
    const float* src = in + (int64_t)blockIdx.z * rows * cols;
    float* dst = out + (int64_t)blockIdx.z * rows * cols;
    int64_t c = (int64_t)blockIdx.x * 32 + threadIdx.x;
    for (int k = threadIdx.y; k < 32; k += 8) {
        int64_t r = (int64_t)blockIdx.y * 32 + k;
        if (r < rows && c < cols) tile[k][threadIdx.x] = src[r * cols + c];
    }
    __syncthreads();
    int64_t r2 = (int64_t)blockIdx.y * 32 + threadIdx.x;   // becomes the column of out
    for (int k = threadIdx.y; k < 32; k += 8) {
        int64_t c2 = (int64_t)blockIdx.x * 32 + k;         // becomes the row of out
        if (c2 < cols && r2 < rows) dst[c2 * rows + r2] = tile[threadIdx.x][k];
    }
}

}  // namespace boatcu

using namespace boatcu;

extern "C" {

int boat_cuda_axpy(float* y, const float* x, float alpha, int64_t n) { return launch_axpy<true>(y, x, alpha, n); }
int boat_cuda_scale(float* y, const float* x, float alpha, int64_t n) { return launch_axpy<false>(y, x, alpha, n); }

int boat_cuda_mul(float* y, const float* a, const float* b, int64_t n) {
    if (n <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    int vec = aligned16(y) && aligned16(a) && aligned16(b) && (n % 4) == 0;
    mul_kernel<<<grid_for(vec ? n / 4 : n, kThreads), kThreads, 0, stream()>>>(y, a, b, n, vec);
    BOATCU_LAUNCH_OK("mul");
    return 0;
}

int boat_cuda_add_bias(float* y, const float* x, const float* bias, int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    int vec = aligned16(y) && aligned16(x) && aligned16(bias) && (cols % 4) == 0;
    int64_t n = rows * cols;
    add_bias_kernel<<<grid_for(vec ? n / 4 : n, kThreads), kThreads, 0, stream()>>>(y, x, bias, rows, cols, vec);
    BOATCU_LAUNCH_OK("add_bias");
    return 0;
}

int boat_cuda_cast(void* dst, int dst_type, const void* src, int src_type, int64_t n) {
    if (n <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    if (dst_type == src_type) return boat_cuda_memcpy_d2d(dst, src, (size_t)n * type_size(dst_type));
    int vec = aligned16(dst) && aligned16(src) && (n % 8) == 0;
    int grid = grid_for(vec ? n / 8 : n, kThreads);
    ProfileScope prof("cast");
    if (dst_type == BOAT_CUDA_BF16)
        cast_f32_to_bf16<<<grid, kThreads, 0, stream()>>>((__nv_bfloat16*)dst, (const float*)src, n, vec);
    else
        cast_bf16_to_f32<<<grid, kThreads, 0, stream()>>>((float*)dst, (const __nv_bfloat16*)src, n, vec);
    BOATCU_LAUNCH_OK("cast");
    return 0;
}

int boat_cuda_lincomb(void* y, const void* a, float alpha, const void* b, float beta, int type, int64_t n) {
    if (n <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    const int V = type == BOAT_CUDA_BF16 ? 8 : 4;
    int vec = aligned16(y) && aligned16(a) && aligned16(b) && (n % V) == 0;
    int grid = grid_for(vec ? n / V : n, kThreads);
    ProfileScope prof("lincomb");
    if (type == BOAT_CUDA_BF16)
        lincomb_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream()>>>((__nv_bfloat16*)y, (const __nv_bfloat16*)a, alpha,
                                                                       (const __nv_bfloat16*)b, beta, n, vec);
    else
        lincomb_kernel<float><<<grid, kThreads, 0, stream()>>>((float*)y, (const float*)a, alpha, (const float*)b, beta, n, vec);
    BOATCU_LAUNCH_OK("lincomb");
    return 0;
}

int boat_cuda_round_tf32(float* y, const float* x, int64_t n) {
    if (n <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    int vec = aligned16(y) && aligned16(x) && (n % 4) == 0;
    ProfileScope prof("round_tf32");
    round_tf32_kernel<<<grid_for(vec ? n / 4 : n, kThreads), kThreads, 0, stream()>>>(y, x, n, vec);
    BOATCU_LAUNCH_OK("round_tf32");
    return 0;
}

int boat_cuda_colsum_multi(const void* const* X, int x_type, int64_t rows, int64_t cols, float* const* out, int count) {
    if (cols <= 0 || count <= 0) return 0;
    if (count > kMaxColsum) return set_error(11, "boat_cuda_colsum_multi: %d matrices (1 to %d)", count, kMaxColsum);
    if (!X || !out) return set_error(11, "boat_cuda_colsum_multi: NULL table");
    if (int rc = ensure_init()) return rc;
    ProfileScope prof("colsum");
    ColsumTable t;
    const int vec = x_type == BOAT_CUDA_BF16 ? 8 : 4;
    bool can_vec = (cols % vec) == 0;
    for (int i = 0; i < kMaxColsum; ++i) {
        const int s = i < count ? i : 0;
        if (!X[s] || !out[s]) return set_error(11, "boat_cuda_colsum_multi: NULL operand");
        t.x[i] = X[s];
        t.out[i] = out[s];
        can_vec = can_vec && aligned16(X[s]);
    }
    // one clear per output: neighbouring outputs may still be separate allocations, which a single
    // clear must not span
    for (int i = 0; i < count; ++i) BOATCU_CHECK(cudaMemsetAsync(out[i], 0, (size_t)cols * sizeof(float), stream()));
    if (rows <= 0) return 0;
    const int cols_per_block = 32 * (can_vec ? vec : 1);
    dim3 grid((unsigned)ceil_div(cols, cols_per_block), 1, (unsigned)count);
    int64_t want = (int64_t)sm_count() * 8 / ((int64_t)grid.x * count);
    int64_t max_y = ceil_div(rows, 8);
    grid.y = (unsigned)(want < 1 ? 1 : (want > max_y ? max_y : want));
    if (grid.y > 65535) grid.y = 65535;
    if (x_type == BOAT_CUDA_BF16) {
        if (can_vec) colsum_kernel<__nv_bfloat16, 8><<<grid, kThreads, 0, stream()>>>(t, rows, cols);
        else         colsum_kernel<__nv_bfloat16, 1><<<grid, kThreads, 0, stream()>>>(t, rows, cols);
    } else {
        if (can_vec) colsum_kernel<float, 4><<<grid, kThreads, 0, stream()>>>(t, rows, cols);
        else         colsum_kernel<float, 1><<<grid, kThreads, 0, stream()>>>(t, rows, cols);
    }
    BOATCU_LAUNCH_OK("colsum");
    return 0;
}

int boat_cuda_colsum(const void* X, int x_type, int64_t rows, int64_t cols, float* out) {
    if (cols <= 0) return 0;
    return boat_cuda_colsum_multi(&X, x_type, rows, cols, &out, 1);
}

int boat_cuda_convert_multi(void* const* dst, int dst_type, const float* const* src, const int64_t* n, int count) {
    if (count <= 0) return 0;
    if (count > kMaxConvert) return set_error(11, "boat_cuda_convert_multi: %d tensors (1 to %d)", count, kMaxConvert);
    if (dst_type != BOAT_CUDA_BF16 && dst_type != BOAT_CUDA_F32_TF32)
        return set_error(10, "boat_cuda_convert_multi: target type %d (BF16 or TF32-valued FP32)", dst_type);
    if (!dst || !src || !n) return set_error(11, "boat_cuda_convert_multi: NULL table");
    if (int rc = ensure_init()) return rc;
    ConvertTable t;
    int vec = 1;
    int64_t longest = 0;
    for (int i = 0; i < kMaxConvert; ++i) {
        const int s = i < count ? i : 0;
        if (n[s] < 0 || (n[s] > 0 && (!dst[s] || !src[s]))) return set_error(11, "boat_cuda_convert_multi: bad entry %d", s);
        t.src[i] = src[s];
        t.dst[i] = dst[s];
        t.n[i] = n[s];
        vec = vec && aligned16(dst[s]) && aligned16(src[s]) && (n[s] % 8) == 0;
        if (n[s] > longest) longest = n[s];
    }
    if (longest == 0) return 0;
    // the blocks of all tensors together fill the GPU a few times over
    int64_t per_tensor = ceil_div(vec ? longest / 8 : longest, kThreads);
    const int64_t cap = ceil_div((int64_t)sm_count() * 16, count);
    if (per_tensor > cap) per_tensor = cap;
    dim3 grid((unsigned)per_tensor, (unsigned)count, 1);
    ProfileScope prof("cast");
    if (dst_type == BOAT_CUDA_BF16) convert_multi_kernel<true><<<grid, kThreads, 0, stream()>>>(t, vec);
    else                            convert_multi_kernel<false><<<grid, kThreads, 0, stream()>>>(t, vec);
    BOATCU_LAUNCH_OK("convert_multi");
    return 0;
}

int boat_cuda_transpose(float* out, const float* in, int64_t batch, int64_t rows, int64_t cols) {
    if (batch <= 0 || rows <= 0 || cols <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    if (batch > 65535) return set_error(6, "boat_cuda_transpose: batch %lld exceeds 65535", (long long)batch);
    dim3 grid((unsigned)ceil_div(cols, 32), (unsigned)ceil_div(rows, 32), (unsigned)batch);
    transpose_kernel<<<grid, dim3(32, 8, 1), 0, stream()>>>(out, in, rows, cols);
    BOATCU_LAUNCH_OK("transpose");
    return 0;
}

}  // extern "C"
