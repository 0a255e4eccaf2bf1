// optim.cu - the Adam step on the device, one launch for a whole list of parameter tensors.
//
// Counterpart: adam_update_parameter in the reference's src/optimizers/adam.c (lines
// 156-193), which walks one tensor at a time on the host.  The arithmetic below keeps the
// reference's order of rounded FP32 operations (no fused multiply-add, IEEE division and
// square root), so that a step gives the same bits as the reference gives on the host:
//
//     m  = fl(fl(b1*m) + fl(fl(1-b1)*g))
//     v  = fl(fl(b2*v) + fl(fl(fl(1-b2)*g)*g))
//     mh = fl(m / fl(1-b1^t))        vh = fl(v / fl(1-b2^t))
//     p  = fl(p - fl(fl(lr*mh) / fl(sqrt(vh) + eps)))
//
// The kernel is HBM-bound: per element it reads p, g, m, v and writes p, m, v (28 bytes).
// Work is cut into fixed chunks; a table in constant-bank kernel arguments maps each chunk
// to its tensor, so small bias vectors and large weight matrices share one grid.  One CTA
// per 1024-element chunk, one 128-bit access per thread and array: measured on B200 this
// simple shape moves 6.3 TB/s, against 5.3 TB/s for a persistent grid and 4.9 TB/s for four
// accesses per thread (84 registers, fewer resident warps, a coarser tail).
#include "common.cuh"

namespace boatcu {

static const int kAdamThreads = 256;
static const int kAdamChunk = kAdamThreads * 4;
static const int kAdamMaxTensors = 24;         // per launch; longer lists take several launches

struct AdamTable {
    float* p[kAdamMaxTensors];
    const float* g[kAdamMaxTensors];
    float* m[kAdamMaxTensors];
    float* v[kAdamMaxTensors];
    long long n[kAdamMaxTensors];
    int first_chunk[kAdamMaxTensors + 1];      // prefix sum of chunks per tensor
    int count;
};

struct AdamConst {
    float lr, b1, b2, eps;
    float one_minus_b1, one_minus_b2;          // fl(1-b1), fl(1-b2)
    float corr1, corr2;                        // fl(1-b1^t), fl(1-b2^t)
};

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const AdamConst& c) {
    m = __fadd_rn(__fmul_rn(c.b1, m), __fmul_rn(c.one_minus_b1, g));
    v = __fadd_rn(__fmul_rn(c.b2, v), __fmul_rn(__fmul_rn(c.one_minus_b2, g), g));
    float mh = __fdiv_rn(m, c.corr1);
    float vh = __fdiv_rn(v, c.corr2);
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(c.lr, mh), __fadd_rn(__fsqrt_rn(vh), c.eps)));
}

__global__ void __launch_bounds__(kAdamThreads) adam_multi_kernel(const __grid_constant__ AdamTable tab,
                                                                  const AdamConst c, int total_chunks) {
    for (int chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
        // which tensor owns this chunk (the table is short: linear scan, uniform per CTA)
        int t = 0;
        while (t + 1 < tab.count && chunk >= tab.first_chunk[t + 1]) ++t;
        const long long base = (long long)(chunk - tab.first_chunk[t]) * kAdamChunk;
        const long long n = tab.n[t];
        float* __restrict__ p = tab.p[t] + base;
        const float* __restrict__ g = tab.g[t] + base;
        float* __restrict__ m = tab.m[t] + base;
        float* __restrict__ v = tab.v[t] + base;
        const long long left = n - base;
        const bool vec = ((((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15) == 0);
        if (vec && left >= kAdamChunk) {
            const int i = threadIdx.x;
            float4 P = reinterpret_cast<const float4*>(p)[i];
            float4 G = __ldcs(reinterpret_cast<const float4*>(g) + i);
            float4 M = reinterpret_cast<const float4*>(m)[i];
            float4 V = reinterpret_cast<const float4*>(v)[i];
            adam_one(P.x, G.x, M.x, V.x, c);
            adam_one(P.y, G.y, M.y, V.y, c);
            adam_one(P.z, G.z, M.z, V.z, c);
            adam_one(P.w, G.w, M.w, V.w, c);
            reinterpret_cast<float4*>(p)[i] = P;
            reinterpret_cast<float4*>(m)[i] = M;
            reinterpret_cast<float4*>(v)[i] = V;
        } else {
            const int lim = left < kAdamChunk ? (int)left : kAdamChunk;
            for (int i = threadIdx.x; i < lim; i += kAdamThreads) {
                float pi = p[i], mi = m[i], vi = v[i];
                adam_one(pi, g[i], mi, vi, c);
                p[i] = pi;
                m[i] = mi;
                v[i] = vi;
            }
        }
    }
}

}  // namespace boatcu

using namespace boatcu;

extern "C" int boat_cuda_adam_step(int count, float* const* params, const float* const* grads, float* const* m,
                                   float* const* v, const int64_t* nelements, float lr, float beta1, float beta2,
                                   float epsilon, float corr1, float corr2) {
    if (count < 0 || (count > 0 && (!params || !grads || !m || !v || !nelements)))
        return set_error(2, "boat_cuda_adam_step: bad argument list");
    if (count == 0) return 0;
    if (int rc = ensure_init()) return rc;
    ProfileScope scope("adam_step");
    AdamConst c;
    c.lr = lr; c.b1 = beta1; c.b2 = beta2; c.eps = epsilon;
    c.one_minus_b1 = 1.0f - beta1;
    c.one_minus_b2 = 1.0f - beta2;
    c.corr1 = corr1; c.corr2 = corr2;
    int done = 0;
    while (done < count) {
        AdamTable tab;
        tab.count = 0;
        tab.first_chunk[0] = 0;
        int64_t chunks = 0;
        while (done < count && tab.count < kAdamMaxTensors) {
            const int64_t n = nelements[done];
            if (n < 0 || (n > 0 && (!params[done] || !grads[done] || !m[done] || !v[done])))
                return set_error(2, "boat_cuda_adam_step: tensor %d has a null pointer or a negative size", done);
            const int64_t mine = ceil_div(n, kAdamChunk);
            if (chunks + mine > 0x7fffffff) {
                if (tab.count == 0) return set_error(2, "boat_cuda_adam_step: tensor %d is too large", done);
                break;
            }
            if (n > 0) {
                const int t = tab.count++;
                tab.p[t] = params[done]; tab.g[t] = grads[done]; tab.m[t] = m[done]; tab.v[t] = v[done];
                tab.n[t] = n;
                chunks += mine;
                tab.first_chunk[t + 1] = (int)chunks;
            }
            ++done;
        }
        if (tab.count == 0) continue;
        adam_multi_kernel<<<(int)chunks, kAdamThreads, 0, stream()>>>(tab, c, (int)chunks);
        BOATCU_LAUNCH_OK("adam_multi_kernel");
    }
    return 0;
}
