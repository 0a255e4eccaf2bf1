// attn_tc.cu - host side of the tcgen05 attention-core kernels: shape support, tensor maps,
// launches.  The kernels themselves are in attn_fwd_tc.cuh, attn_bwd_tc.cuh (BF16 storage) and
// attn_bwd_tf32_tc.cuh (FP32 storage).
#include "attn_bwd_tc.cuh"
#include "attn_bwd_tf32_tc.cuh"
#include <stdlib.h>

namespace boatcu {

using namespace attn_tc;

namespace {

template <typename T, int HS>
int launch_fwd(int64_t units, int64_t S, int causal, float scale, const void* Q, const void* K, const void* V,
               void* O, float* lse) {
    using C = FwdCfg<T, HS>;
    CUtensorMap mq, mk, mv;
    const uint64_t rows = (uint64_t)units * (uint64_t)S;
    if (int rc = make_tensor_map_2d(&mq, Q, C::ES, rows, HS, HS, kTile, C::BOXC)) return rc;
    if (int rc = make_tensor_map_2d(&mk, K, C::ES, rows, HS, HS, kTile, C::BOXC)) return rc;
    // V is read by the tensor core along its contiguous head dimension: FP32 needs the
    // 32-byte-unit swizzle for that
    if (int rc = make_tensor_map_2d(&mv, V, C::ES, rows, HS, HS, kTile, C::BOXC, C::TF32)) return rc;
    FwdParams p;
    p.O = O;
    p.lse = lse;
    p.S = (int)S;
    p.units = (int)units;
    p.causal = causal;
    p.scale = scale;
    p.status = kernel_status_ptr();
    // units whose K and V (2 * S * hs elements each) together take about a third of L2
    const int64_t group = (40ll << 20) / (2 * S * HS * (int64_t)C::ES);
    p.group = (int)(group < 1 ? 1 : (group > units ? units : group));
    {
        // BOAT_FWD_GROUP=n in the environment overrides the group size; it is read at every launch so
        // that a test can run a small problem in several groups, the first of them short
        const char* e = getenv("BOAT_FWD_GROUP");
        const int n = e ? atoi(e) : 0;
        if (n >= 1) p.group = n > (int)units ? (int)units : n;
    }
    auto kern = attn_fwd_tc_kernel<T, HS>;
    static bool configured = false;
    if (!configured) {
        BOATCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured = true;
    }
    const int64_t grid = units * ((S / kTile + 1) / 2);      // one CTA per pair of query tiles
    ProfileScope prof("attn_fwd_tc");
    kern<<<(unsigned)grid, kFwdThreads, C::SMEM, stream()>>>(mq, mk, mv, p);
    BOATCU_LAUNCH_OK("attn_fwd_tc");
    return 0;
}

}  // namespace

bool attn_tc_supported(int mma, int64_t units, int64_t S, int64_t hs, int io_type) {
    if (S < kTile || S % kTile != 0) return false;
    if (units * (S / kTile) > 0x7fffffffLL || units * S > 0x7fffffffLL) return false;
    if (mma == BOAT_MMA_BF16) return io_type == BOAT_CUDA_BF16 && (hs == 64 || hs == 128);
    if (mma == BOAT_MMA_TF32) return io_type == BOAT_CUDA_F32 && hs == 64;
    return false;
}

int attn_fwd_tc(int mma, int64_t units, int64_t S, int64_t hs, int causal, float scale, const void* Q, const void* K,
                const void* V, int io_type, void* O, float* lse) {
    (void)io_type;
    if (int rc = ensure_init()) return rc;
    if (mma == BOAT_MMA_BF16) {
        if (hs == 64) return launch_fwd<__nv_bfloat16, 64>(units, S, causal, scale, Q, K, V, O, lse);
        return launch_fwd<__nv_bfloat16, 128>(units, S, causal, scale, Q, K, V, O, lse);
    }
    return launch_fwd<float, 64>(units, S, causal, scale, Q, K, V, O, lse);
}

namespace {

template <int HS>
int launch_bwd(int64_t units, int64_t S, int causal, float scale, const void* Q, const void* K, const void* V,
               const void* O, const void* dO, const float* lse, void* dQ, void* dK, void* dV, float* dq_accum,
               float* stats2) {
    using C = BwdCfg<HS>;
    CUtensorMap mq, mk, mv, mdo, mdq;
    const uint64_t rows = (uint64_t)units * (uint64_t)S;
    if (int rc = make_tensor_map_2d(&mq, Q, 2, rows, HS, HS, kTile, 64)) return rc;
    if (int rc = make_tensor_map_2d(&mk, K, 2, rows, HS, HS, kTile, 64)) return rc;
    if (int rc = make_tensor_map_2d(&mv, V, 2, rows, HS, HS, kTile, 64)) return rc;
    if (int rc = make_tensor_map_2d(&mdo, dO, 2, rows, HS, HS, kTile, 64)) return rc;
    if (int rc = make_tensor_map_2d(&mdq, dq_accum, 4, rows, HS, HS, kTile, 32)) return rc;   // FP32 reduce-add target
    const size_t n = (size_t)units * (size_t)S * HS;
    BwdParams p;
    p.lse2 = stats2;
    p.delta2 = stats2 + rows;
    p.dq_accum = dq_accum;
    p.dK = dK;
    p.dV = dV;
    p.S = (int)S;
    p.units = (int)units;
    p.causal = causal;
    // units whose dQ (FP32), Q, dO, K and V - 16 bytes per element of the unit - share L2 at a time
    const int64_t unit_bytes = S * HS * 16;
    int64_t group = (64ll << 20) / unit_bytes;
    p.group = (int)(group < 1 ? 1 : (group > units ? units : group));
    // Two walks per CTA halve what a CTA pays once (start-up, the last tile's read-out, exit) and
    // equalise the CTAs when causal: 5-10 % at 8- and 16-tile walks.  With equal CTAs the last
    // wave is a loss that many short CTAs would fill, and at 64-tile walks the per-CTA cost is
    // small anyway (measured: no gain at 64 tiles, 10 % slower when only 3.5 waves of pairs exist).
    const int64_t n_tiles = S / kTile;
    p.pair = (n_tiles <= 32 && units * ((n_tiles + 1) / 2) >= 8 * (int64_t)sm_count()) ? 1 : 0;
    {
        // BOAT_BWD_PAIR=0/1 in the environment overrides the rule; it is read at every launch so
        // that one test process can run both schedules on the same problem
        const char* e = getenv("BOAT_BWD_PAIR");
        if (e && (e[0] == '0' || e[0] == '1')) p.pair = e[0] - '0';
    }
    p.scale = scale;
    p.status = kernel_status_ptr();
    auto kern = attn_bwd_tc_kernel<HS>;
    static bool configured = false;
    if (!configured) {
        BOATCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured = true;
    }
    {
        // the per-row statistics in the form the kernel's inner loops consume them:
        // -lse * log2(e) and -scale * rowsum(dO o O)
        ProfileScope prof("attn_delta");
        if (int rc = rowdot_stats(dO, O, BOAT_CUDA_BF16, (int64_t)rows, HS, lse, scale, stats2 + rows, stats2)) return rc;
    }
    {
        ProfileScope prof("attn_bwd_tc");
        BOATCU_CHECK(cudaMemsetAsync(dq_accum, 0, n * sizeof(float), stream()));
        const int64_t grid = units * (p.pair ? (S / kTile + 1) / 2 : S / kTile);
        kern<<<(unsigned)grid, kBwdThreads, C::SMEM, stream()>>>(mq, mk, mv, mdo, mdq, p);
        BOATCU_LAUNCH_OK("attn_bwd_tc");
        // the summed FP32 contributions become the BF16 output
        if (int rc = boat_cuda_cast(dQ, BOAT_CUDA_BF16, dq_accum, BOAT_CUDA_F32, (int64_t)n)) return rc;
    }
    return 0;
}

// FP32 storage, TF32 arithmetic, head size 64: a dQ kernel over query tiles and a dK/dV kernel over
// key tiles; no scratch beyond delta.
int launch_bwd_tf32(int64_t units, int64_t S, int causal, float scale, const void* Q, const void* K, const void* V,
                    const void* dO, const float* lse, const float* delta, void* dQ, void* dK, void* dV) {
    using C = Bwd32Cfg;
    constexpr int HS = kBwd32HS;
    CUtensorMap mq, mq_mn, mk, mk_mn, mv, mdo, mdo_mn;
    const uint64_t rows = (uint64_t)units * (uint64_t)S;
    // the same matrices with both shared-memory layouts: 16-byte swizzle units for operands read
    // along hs, 32-byte units for operands read along their rows
    if (int rc = make_tensor_map_2d(&mq, Q, 4, rows, HS, HS, kTile, 32)) return rc;
    if (int rc = make_tensor_map_2d(&mq_mn, Q, 4, rows, HS, HS, kTile, 32, true)) return rc;
    if (int rc = make_tensor_map_2d(&mk, K, 4, rows, HS, HS, kTile, 32)) return rc;
    if (int rc = make_tensor_map_2d(&mk_mn, K, 4, rows, HS, HS, kTile, 32, true)) return rc;
    if (int rc = make_tensor_map_2d(&mv, V, 4, rows, HS, HS, kTile, 32)) return rc;
    if (int rc = make_tensor_map_2d(&mdo, dO, 4, rows, HS, HS, kTile, 32)) return rc;
    if (int rc = make_tensor_map_2d(&mdo_mn, dO, 4, rows, HS, HS, kTile, 32, true)) return rc;
    Bwd32Params p;
    p.lse = lse;
    p.delta = delta;
    p.dQ = (float*)dQ;
    p.dK = (float*)dK;
    p.dV = (float*)dV;
    p.S = (int)S;
    p.units = (int)units;
    p.causal = causal;
    p.scale = scale;
    p.status = kernel_status_ptr();
    static bool configured = false;     // per process = per device: the library binds to one device
    if (!configured) {
        BOATCU_CHECK(cudaFuncSetAttribute(attn_bwd_dq_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_DQ));
        BOATCU_CHECK(cudaFuncSetAttribute(attn_bwd_dkv_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_DKV));
        configured = true;
    }
    const unsigned grid = (unsigned)(units * (S / kTile));
    ProfileScope prof("attn_bwd_tc");
    attn_bwd_dkv_tf32_kernel<<<grid, kBwd32Threads, C::SMEM_DKV, stream()>>>(mq, mq_mn, mk, mv, mdo, mdo_mn, p);
    BOATCU_LAUNCH_OK("attn_bwd_dkv_tf32");
    attn_bwd_dq_tf32_kernel<<<grid, kBwd32Threads, C::SMEM_DQ, stream()>>>(mq, mk, mk_mn, mv, mdo, p);
    BOATCU_LAUNCH_OK("attn_bwd_dq_tf32");
    return 0;
}

}  // namespace

// Scratch of the BF16 tensor-core backward: the FP32 accumulation buffer of dQ, then the two
// pre-scaled statistics per row.  (units*S is a multiple of 128, so both parts are 512-byte multiples.)
size_t attn_bwd_tc_scratch_bytes(int mma, int64_t units, int64_t S, int64_t hs) {
    if (mma != BOAT_MMA_BF16) return 0;
    return (size_t)units * (size_t)S * (size_t)hs * sizeof(float) + 2 * (size_t)units * (size_t)S * sizeof(float);
}

int attn_bwd_tc(int mma, int64_t units, int64_t S, int64_t hs, int causal, float scale, const void* Q, const void* K,
                const void* V, const void* O, const void* dO, const float* lse, const float* delta, int io_type, void* dQ,
                void* dK, void* dV, void* scratch, size_t scratch_bytes) {
    if (int rc = ensure_init()) return rc;
    if (mma == BOAT_MMA_BF16) {
        if (scratch_bytes < attn_bwd_tc_scratch_bytes(mma, units, S, hs))
            return set_error(12, "attention backward: scratch too small for the dQ accumulation buffer");
        float* stats2 = (float*)scratch + (size_t)units * (size_t)S * (size_t)hs;
        if (hs == 64)
            return launch_bwd<64>(units, S, causal, scale, Q, K, V, O, dO, lse, dQ, dK, dV, (float*)scratch, stats2);
        return launch_bwd<128>(units, S, causal, scale, Q, K, V, O, dO, lse, dQ, dK, dV, (float*)scratch, stats2);
    }
    (void)io_type;
    return launch_bwd_tf32(units, S, causal, scale, Q, K, V, dO, lse, delta, dQ, dK, dV);
}

}  // namespace boatcu
