// attn_simt.cu - CUDA-core attention core, forward and backward, FP32 arithmetic, any
// sequence length and head size up to 128.  One thread owns one query row (forward, dQ) or
// one key row (dK, dV); the other side streams through shared memory in tiles that every
// thread reads as a broadcast, so no cross-thread reduction is needed.  The S x S matrices
// are never written to memory: probabilities are rebuilt from the saved log-sum-exp.
//
// Restates scaled_dot_product_attention_impl (reference src/layers/attention.c:997-1073)
// and attention_backward (attention.c:1421-1526) for the exact-FP32 mode and for shapes
// outside the tensor-core kernels.
#include "common.cuh"
#include <float.h>

namespace boatcu {

static const int ROWS = 64;   // rows owned by a CTA = threads per CTA

template <int TILE, typename T>
__device__ __forceinline__ void load_tile(float* dst, const T* src, int64_t row0, int64_t S, int hs, int tid) {
    // dst[r*hs + d] = src[(row0+r)*hs + d] for r < TILE, zero past the end of the sequence
    for (int idx = tid; idx < TILE * hs; idx += ROWS) {
        int r = idx / hs;
        dst[idx] = (row0 + r < S) ? to_f32(src[row0 * hs + idx]) : 0.f;
    }
}

// ---- forward -----------------------------------------------------------------------------------
template <int HS_MAX, int TILE, typename T>
__global__ void __launch_bounds__(ROWS)
attn_fwd_simt_kernel(int64_t S, int hs, int causal, float scale, const T* __restrict__ Q,
                     const T* __restrict__ K, const T* __restrict__ V, T* __restrict__ O,
                     float* __restrict__ lse) {
    extern __shared__ float smem[];
    float* q_s = smem;                       // [hs][ROWS]   column = thread
    float* k_s = q_s + (size_t)hs * ROWS;    // [TILE][hs]
    float* v_s = k_s + (size_t)TILE * hs;    // [TILE][hs]
    const int tid = threadIdx.x;
    const int64_t unit = blockIdx.y;
    const int64_t i0 = (int64_t)blockIdx.x * ROWS;
    const int64_t i = i0 + tid;
    const T* Qu = Q + unit * S * hs;
    const T* Ku = K + unit * S * hs;
    const T* Vu = V + unit * S * hs;
    const bool live = i < S;

    for (int idx = tid; idx < ROWS * hs; idx += ROWS) {
        int r = idx / hs, d = idx % hs;
        q_s[d * ROWS + r] = (i0 + r < S) ? to_f32(Qu[i0 * hs + idx]) : 0.f;
    }
    float o[HS_MAX];
#pragma unroll
    for (int d = 0; d < HS_MAX; ++d) o[d] = 0.f;
    float m = -FLT_MAX, l = 0.f;

    const int64_t j_end = causal ? min(S, i0 + ROWS) : S;
    for (int64_t j0 = 0; j0 < j_end; j0 += TILE) {
        __syncthreads();
        load_tile<TILE>(k_s, Ku, j0, S, hs, tid);
        load_tile<TILE>(v_s, Vu, j0, S, hs, tid);
        __syncthreads();
        float s[TILE];
        float tmax = -FLT_MAX;
#pragma unroll
        for (int t = 0; t < TILE; ++t) {
            float acc = 0.f;
            for (int d = 0; d < hs; ++d) acc = fmaf(q_s[d * ROWS + tid], k_s[t * hs + d], acc);
            acc *= scale;
            int64_t j = j0 + t;
            bool ok = j < S && (!causal || j <= i);
            s[t] = ok ? acc : -FLT_MAX;
            tmax = fmaxf(tmax, s[t]);
        }
        if (tmax == -FLT_MAX) continue;          // nothing visible for this row in this tile
        float m_new = fmaxf(m, tmax);
        float corr = (m == -FLT_MAX) ? 0.f : expf(m - m_new);
        l *= corr;
#pragma unroll
        for (int d = 0; d < HS_MAX; ++d) o[d] *= corr;
#pragma unroll
        for (int t = 0; t < TILE; ++t) {
            float p = (s[t] == -FLT_MAX) ? 0.f : expf(s[t] - m_new);
            l += p;
#pragma unroll
            for (int d = 0; d < HS_MAX; ++d)
                if (d < hs) o[d] = fmaf(p, v_s[t * hs + d], o[d]);
        }
        m = m_new;
    }
    if (live) {
        float inv = 1.f / l;
        T* Ou = O + unit * S * hs + i * hs;
#pragma unroll
        for (int d = 0; d < HS_MAX; ++d)
            if (d < hs) Ou[d] = from_f32<T>(o[d] * inv);
        lse[unit * S + i] = m + logf(l);
    }
}

// ---- backward, dQ: thread = query row ------------------------------------------------------------
template <int HS_MAX, int TILE, typename T>
__global__ void __launch_bounds__(ROWS)
attn_bwd_dq_simt_kernel(int64_t S, int hs, int causal, float scale, const T* __restrict__ Q,
                        const T* __restrict__ K, const T* __restrict__ V, const T* __restrict__ dO,
                        const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dQ) {
    extern __shared__ float smem[];
    float* q_s = smem;                        // [hs][ROWS]
    float* do_s = q_s + (size_t)hs * ROWS;    // [hs][ROWS]
    float* k_s = do_s + (size_t)hs * ROWS;    // [TILE][hs]
    float* v_s = k_s + (size_t)TILE * hs;     // [TILE][hs]
    const int tid = threadIdx.x;
    const int64_t unit = blockIdx.y;
    const int64_t i0 = (int64_t)blockIdx.x * ROWS;
    const int64_t i = i0 + tid;
    const int64_t base = unit * S * hs;
    const bool live = i < S;
    for (int idx = tid; idx < ROWS * hs; idx += ROWS) {
        int r = idx / hs, d = idx % hs;
        bool in = i0 + r < S;
        q_s[d * ROWS + r] = in ? to_f32(Q[base + i0 * hs + idx]) : 0.f;
        do_s[d * ROWS + r] = in ? to_f32(dO[base + i0 * hs + idx]) : 0.f;
    }
    const float lse_i = live ? lse[unit * S + i] : 0.f;
    const float delta_i = live ? delta[unit * S + i] : 0.f;
    float acc[HS_MAX];
#pragma unroll
    for (int d = 0; d < HS_MAX; ++d) acc[d] = 0.f;

    const int64_t j_end = causal ? min(S, i0 + ROWS) : S;
    for (int64_t j0 = 0; j0 < j_end; j0 += TILE) {
        __syncthreads();
        load_tile<TILE>(k_s, K + base, j0, S, hs, tid);
        load_tile<TILE>(v_s, V + base, j0, S, hs, tid);
        __syncthreads();
#pragma unroll 1
        for (int t = 0; t < TILE; ++t) {
            int64_t j = j0 + t;
            if (!(live && j < S && (!causal || j <= i))) continue;
            float s = 0.f, dp = 0.f;
            for (int d = 0; d < hs; ++d) {
                s = fmaf(q_s[d * ROWS + tid], k_s[t * hs + d], s);
                dp = fmaf(do_s[d * ROWS + tid], v_s[t * hs + d], dp);
            }
            float p = expf(s * scale - lse_i);
            float ds = p * (dp - delta_i) * scale;
#pragma unroll
            for (int d = 0; d < HS_MAX; ++d)
                if (d < hs) acc[d] = fmaf(ds, k_s[t * hs + d], acc[d]);
        }
    }
    if (live) {
        T* out = dQ + base + i * hs;
#pragma unroll
        for (int d = 0; d < HS_MAX; ++d)
            if (d < hs) out[d] = from_f32<T>(acc[d]);
    }
}

// ---- backward, dK (WANT_K) or dV: thread = key row -------------------------------------------------
template <int HS_MAX, int TILE, typename T, bool WANT_K>
__global__ void __launch_bounds__(ROWS)
attn_bwd_kv_simt_kernel(int64_t S, int hs, int causal, float scale, const T* __restrict__ Q,
                        const T* __restrict__ K, const T* __restrict__ V, const T* __restrict__ dO,
                        const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dOut) {
    extern __shared__ float smem[];
    float* k_s = smem;                        // [hs][ROWS]
    float* v_s = k_s + (size_t)hs * ROWS;     // [hs][ROWS]
    float* q_s = v_s + (size_t)hs * ROWS;     // [TILE][hs]
    float* do_s = q_s + (size_t)TILE * hs;    // [TILE][hs]
    float* lse_s = do_s + (size_t)TILE * hs;  // [TILE]
    float* delta_s = lse_s + TILE;            // [TILE]
    const int tid = threadIdx.x;
    const int64_t unit = blockIdx.y;
    const int64_t j0 = (int64_t)blockIdx.x * ROWS;
    const int64_t j = j0 + tid;
    const int64_t base = unit * S * hs;
    const bool live = j < S;
    for (int idx = tid; idx < ROWS * hs; idx += ROWS) {
        int r = idx / hs, d = idx % hs;
        bool in = j0 + r < S;
        k_s[d * ROWS + r] = in ? to_f32(K[base + j0 * hs + idx]) : 0.f;
        v_s[d * ROWS + r] = in ? to_f32(V[base + j0 * hs + idx]) : 0.f;
    }
    float acc[HS_MAX];
#pragma unroll
    for (int d = 0; d < HS_MAX; ++d) acc[d] = 0.f;

    const int64_t i_begin = causal ? (j0 / TILE) * TILE : 0;
    for (int64_t i0 = i_begin; i0 < S; i0 += TILE) {
        __syncthreads();
        load_tile<TILE>(q_s, Q + base, i0, S, hs, tid);
        load_tile<TILE>(do_s, dO + base, i0, S, hs, tid);
        if (tid < TILE) {
            bool in = i0 + tid < S;
            lse_s[tid] = in ? lse[unit * S + i0 + tid] : 0.f;
            delta_s[tid] = in ? delta[unit * S + i0 + tid] : 0.f;
        }
        __syncthreads();
#pragma unroll 1
        for (int t = 0; t < TILE; ++t) {
            int64_t i = i0 + t;
            if (!(live && i < S && (!causal || j <= i))) continue;
            float s = 0.f, dp = 0.f;
            for (int d = 0; d < hs; ++d) {
                s = fmaf(q_s[t * hs + d], k_s[d * ROWS + tid], s);
                if (WANT_K) dp = fmaf(do_s[t * hs + d], v_s[d * ROWS + tid], dp);
            }
            float p = expf(s * scale - lse_s[t]);
            if (WANT_K) {
                float ds = p * (dp - delta_s[t]) * scale;
#pragma unroll
                for (int d = 0; d < HS_MAX; ++d)
                    if (d < hs) acc[d] = fmaf(ds, q_s[t * hs + d], acc[d]);
            } else {
#pragma unroll
                for (int d = 0; d < HS_MAX; ++d)
                    if (d < hs) acc[d] = fmaf(p, do_s[t * hs + d], acc[d]);
            }
        }
    }
    if (live) {
        T* out = dOut + base + j * hs;
#pragma unroll
        for (int d = 0; d < HS_MAX; ++d)
            if (d < hs) out[d] = from_f32<T>(acc[d]);
    }
}

static const int TILE = 16;

template <int HS_MAX, typename T>
static int launch_fwd(int64_t units, int64_t S, int hs, int causal, float scale, const void* Q, const void* K,
                      const void* V, void* O, float* lse) {
    size_t smem = ((size_t)hs * ROWS + 2 * (size_t)TILE * hs) * sizeof(float);
    auto kern = attn_fwd_simt_kernel<HS_MAX, TILE, T>;
    BOATCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)ceil_div(S, ROWS), (unsigned)units);
    kern<<<grid, ROWS, smem, stream()>>>(S, hs, causal, scale, (const T*)Q, (const T*)K, (const T*)V, (T*)O, lse);
    BOATCU_LAUNCH_OK("attn_fwd_simt");
    return 0;
}

template <int HS_MAX, typename T>
static int launch_bwd(int64_t units, int64_t S, int hs, int causal, float scale, const void* Q, const void* K,
                      const void* V, const void* dO, const float* lse, const float* delta, void* dQ, void* dK,
                      void* dV) {
    dim3 grid((unsigned)ceil_div(S, ROWS), (unsigned)units);
    {
        size_t smem = (2 * (size_t)hs * ROWS + 2 * (size_t)TILE * hs) * sizeof(float);
        auto kern = attn_bwd_dq_simt_kernel<HS_MAX, TILE, T>;
        BOATCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, ROWS, smem, stream()>>>(S, hs, causal, scale, (const T*)Q, (const T*)K, (const T*)V,
                                            (const T*)dO, lse, delta, (T*)dQ);
        BOATCU_LAUNCH_OK("attn_bwd_dq_simt");
    }
    size_t smem = (2 * (size_t)hs * ROWS + 2 * (size_t)TILE * hs + 2 * TILE) * sizeof(float);
    {
        auto kern = attn_bwd_kv_simt_kernel<HS_MAX, TILE, T, true>;
        BOATCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, ROWS, smem, stream()>>>(S, hs, causal, scale, (const T*)Q, (const T*)K, (const T*)V,
                                            (const T*)dO, lse, delta, (T*)dK);
        BOATCU_LAUNCH_OK("attn_bwd_dk_simt");
    }
    {
        auto kern = attn_bwd_kv_simt_kernel<HS_MAX, TILE, T, false>;
        BOATCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, ROWS, smem, stream()>>>(S, hs, causal, scale, (const T*)Q, (const T*)K, (const T*)V,
                                            (const T*)dO, lse, delta, (T*)dV);
        BOATCU_LAUNCH_OK("attn_bwd_dv_simt");
    }
    return 0;
}

#define DISPATCH_HS(FN, ...)                                                                  \
    do {                                                                                      \
        if (io_type == BOAT_CUDA_BF16) {                                                      \
            if (hs <= 16) return FN<16, __nv_bfloat16>(__VA_ARGS__);                          \
            if (hs <= 64) return FN<64, __nv_bfloat16>(__VA_ARGS__);                          \
            return FN<128, __nv_bfloat16>(__VA_ARGS__);                                       \
        } else {                                                                              \
            if (hs <= 16) return FN<16, float>(__VA_ARGS__);                                  \
            if (hs <= 64) return FN<64, float>(__VA_ARGS__);                                  \
            return FN<128, float>(__VA_ARGS__);                                               \
        }                                                                                     \
    } while (0)

static int check_shape(int64_t units, int64_t S, int64_t hs) {
    if (hs > 128) return set_error(8, "attention: head size %lld > 128 is not supported", (long long)hs);
    if (units > 65535) return set_error(8, "attention: %lld (batch x heads) units exceed 65535", (long long)units);
    (void)S;
    return 0;
}

int attn_fwd_simt(int64_t units, int64_t S, int64_t hs, int causal, float scale, const void* Q, const void* K,
                  const void* V, int io_type, void* O, float* lse) {
    if (units <= 0 || S <= 0 || hs <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    if (int rc = check_shape(units, S, hs)) return rc;
    DISPATCH_HS(launch_fwd, units, S, (int)hs, causal, scale, Q, K, V, O, lse);
}

int attn_bwd_simt(int64_t units, int64_t S, int64_t hs, int causal, float scale, const void* Q, const void* K,
                  const void* V, const void* dO, const float* lse, const float* delta, int io_type, void* dQ,
                  void* dK, void* dV) {
    if (units <= 0 || S <= 0 || hs <= 0) return 0;
    if (int rc = ensure_init()) return rc;
    if (int rc = check_shape(units, S, hs)) return rc;
    DISPATCH_HS(launch_bwd, units, S, (int)hs, causal, scale, Q, K, V, dO, lse, delta, dQ, dK, dV);
}

}  // namespace boatcu
