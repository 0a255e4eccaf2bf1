// attn_bwd_tf32_tc.cuh - fused attention backward on tcgen05 for FP32 storage (kind::tf32, FP32
// accumulation), head size 64.
//
// Replaces attention_backward (reference src/layers/attention.c:1388-1534) for FP32 tensors:
// the probabilities are rebuilt from the saved log-sum-exp tile by tile, and P and dS stay in
// TF32 (never BF16), so the result holds the 5e-3 tolerance of TF32 arithmetic.
//
// Two kernels instead of one.  The BF16 backward keeps dS^T in shared memory because dQ = dS.K
// wants dS with queries on the M side while dK = dS^T.Q wants it with keys on the M side; an
// FP32 dS^T tile is 64 KB and does not fit beside double-staged FP32 Q/dO tiles.  Splitting the
// work by output removes the tile altogether - each product then takes its left operand
// straight from tensor memory, exactly where the softmax warps wrote it:
//
//   dq kernel   CTA = one 128-row query tile, walks the key tiles (like the forward)
//       S  = Q.K^T, dP = dO.V^T             both operands from shared memory
//       dS = P*(dP - delta)/sqrt(hs)        softmax warps, thread = query row, written over S
//       dQ += dS.K                          A = dS from tensor memory, B = K with hs on the N side
//   dkv kernel  CTA = one 128-row key tile, walks the query tiles that see it
//       S^T = K.Q^T, dP^T = V.dO^T
//       P^T over S^T, dS^T over dP^T        softmax warps, thread = key row
//       dV += P^T.dO,  dK += dS^T.Q         A from tensor memory, B = dO / Q with hs on the N side
// dQ, dK, dV leave the kernels rounded to TF32: they feed the TF32 projection GEMMs.
//
// No scratch memory, no atomics, no reduction between CTAs: every output row is produced by one
// CTA, so the results are deterministic.  The price is that S and dP are computed twice (7
// products per tile pair instead of 5); this path serves FP32 tensors, whose problems are small.
//
// An FP32 operand that the tensor core reads along M or N must lie in shared memory with the
// 128-byte swizzle in 32-byte units, one that it reads along K with the usual 16-byte units.
// K (dq kernel) and Q, dO (dkv kernel) are needed both ways, so those tiles are loaded twice,
// once per tensor map; the second copy comes from L2.
// Warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: softmax and epilogue.
#pragma once
#include "attn_bwd_tc.cuh"

namespace boatcu {
namespace attn_tc {

constexpr int kBwd32Threads = 192;
constexpr int kBwd32HS = 64;
constexpr int kBwd32Tile = 2 * kBoxBytes;          // one 128 x 64 FP32 tile: two boxes of 128 rows x 128 bytes

struct Bwd32Cfg {
    // resident tiles + one stage + (lse, delta) buffers + barriers
    static constexpr int SMEM_DQ = 2 * kBwd32Tile + 3 * kBwd32Tile + 1024 + 256;
    static constexpr int SMEM_DKV = 2 * kBwd32Tile + 4 * kBwd32Tile + 2048 + 1024 + 256;
    static constexpr uint32_t COL_S = 0, COL_DP = 128;
    static constexpr uint32_t COL_DQ = 256;                     // dq kernel
    static constexpr uint32_t COL_DV = 256, COL_DK = 320;       // dkv kernel
    static constexpr uint32_t TMEM_COLS = 512;
};

struct Bwd32Params {
    const float* lse;      // [units*S]
    const float* delta;    // [units*S]
    float* dQ;             // dq kernel
    float* dK;             // dkv kernel
    float* dV;
    int S, units, causal;
    float scale;
    unsigned int* status;
};

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t t;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(x));
    return t;
}

// ------------------------------------------------------------------------------------------------
// dQ: one query tile per CTA
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kBwd32Threads, 1)
attn_bwd_dq_tf32_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_k_mn, const __grid_constant__ CUtensorMap map_v,
                        const __grid_constant__ CUtensorMap map_do, const Bwd32Params p) {
    using C = Bwd32Cfg;
    constexpr int HS = kBwd32HS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = smem;
    uint8_t* do_smem = q_smem + kBwd32Tile;
    uint8_t* k_smem = do_smem + kBwd32Tile;          // K read along hs (scores)
    uint8_t* kmn_smem = k_smem + kBwd32Tile;         // K read along the key rows (dQ)
    uint8_t* v_smem = kmn_smem + kBwd32Tile;
    uint64_t* bars = (uint64_t*)(v_smem + kBwd32Tile);
    uint64_t* q_full = bars;            // Q and dO landed
    uint64_t* kv_full = bars + 1;       // K, K (second layout) and V of the tile landed
    uint64_t* kv_empty = bars + 2;      // the tile's MMAs are complete
    uint64_t* s_full = bars + 3;        // S and dP complete
    uint64_t* ds_full = bars + 4;       // dS written (128 arrivals)
    uint64_t* dq_done = bars + 5;       // last dQ MMA complete
    uint32_t* tmem_slot = (uint32_t*)(bars + 6);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = p.S / kTile;
    const int unit = blockIdx.x % p.units;
    const int qt = n_tiles - 1 - blockIdx.x / p.units;       // long (late) rows first when causal
    const int n_kv = p.causal ? qt + 1 : n_tiles;
    const int row_base = unit * p.S;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(kv_full, 1);
        mbar_init(kv_empty, 1);
        mbar_init(s_full, 1);
        mbar_init(ds_full, 128);
        mbar_init(dq_done, 1);
        fence_barrier_init();
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_k_mn);
        tma_prefetch_desc(&map_v);
        tma_prefetch_desc(&map_do);
    }
    if (warp == 1) tmem_alloc(tmem_slot, C::TMEM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base + C::COL_S, tmem_dp = tmem_base + C::COL_DP, tmem_dq = tmem_base + C::COL_DQ;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            mbar_arrive_expect_tx(q_full, 2 * kBwd32Tile);
            for (int b = 0; b < 2; ++b) {
                tma_load_2d(q_smem + b * kBoxBytes, &map_q, q_full, b * 32, row_base + qt * kTile);
                tma_load_2d(do_smem + b * kBoxBytes, &map_do, q_full, b * 32, row_base + qt * kTile);
            }
            for (int j = 0; j < n_kv && ok; ++j) {
                if (!mbar_wait(kv_empty, (j & 1) ^ 1, p.status, kTimeoutProducer)) { ok = false; break; }
                mbar_arrive_expect_tx(kv_full, 3 * kBwd32Tile);
                const int y = row_base + j * kTile;
                for (int b = 0; b < 2; ++b) {
                    tma_load_2d(k_smem + b * kBoxBytes, &map_k, kv_full, b * 32, y);
                    tma_load_2d(kmn_smem + b * kBoxBytes, &map_k_mn, kv_full, b * 32, y);
                    tma_load_2d(v_smem + b * kBoxBytes, &map_v, kv_full, b * 32, y);
                }
            }
            if (!ok)
                for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(kTF32, false, false, kTile, kTile);   // S = Q.K^T, dP = dO.V^T
            constexpr uint32_t idesc_o = make_idesc(kTF32, false, true, kTile, HS);       // dQ += dS.K
            const uint32_t q_addr = smem_u32(q_smem), do_addr = smem_u32(do_smem), k_addr = smem_u32(k_smem);
            const uint32_t kmn_addr = smem_u32(kmn_smem), v_addr = smem_u32(v_smem);
            bool ok = mbar_wait(q_full, 0, p.status, kTimeoutMma);
            for (int j = 0; j < n_kv && ok; ++j) {
                if (!mbar_wait(kv_full, j & 1, p.status, kTimeoutMma)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < HS * 4 / 32; ++kk) {
                    const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
                    mma_ss<true>(tmem_s, smem_desc_sw128(q_addr + off, 16, 1024), smem_desc_sw128(k_addr + off, 16, 1024),
                                 idesc_s, kk > 0);
                }
#pragma unroll
                for (int kk = 0; kk < HS * 4 / 32; ++kk) {
                    const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
                    mma_ss<true>(tmem_dp, smem_desc_sw128(do_addr + off, 16, 1024), smem_desc_sw128(v_addr + off, 16, 1024),
                                 idesc_s, kk > 0);
                }
                mma_commit(s_full);
                if (!mbar_wait(ds_full, j & 1, p.status, kTimeoutMma)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < kTile / 8; ++kk)
                    mma_ts<true>(tmem_dq, tmem_s + kk * 8, smem_desc_mn(kmn_addr + kk * 8 * 128, kBoxBytes, true), idesc_o,
                                 j > 0 || kk > 0);
                mma_commit(kv_empty);
            }
            if (ok) mma_commit(dq_done);
        }
    } else {
        // softmax warps: thread = query row
        const int lane_group = warp & 3;
        const int r_in_tile = lane_group * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
        const int64_t grow = (int64_t)row_base + (int64_t)qt * kTile + r_in_tile;
        const float sl2 = p.scale * 1.4426950408889634f;
        const float neg_lse2 = -p.lse[grow] * 1.4426950408889634f;
        const float neg_delta_s = -p.delta[grow] * p.scale;
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            if (!mbar_wait(s_full, j & 1, p.status, kTimeoutSoftmax)) { ok = false; break; }
            tc_fence_after_sync();
            const bool diag = p.causal && j == qt;
#pragma unroll 1
            for (int c = 0; c < kTile / 32; ++c) {
                uint32_t s[32], d[32];
                tmem_ld32(tmem_s + lane_addr + c * 32, s);
                tmem_ld32(tmem_dp + lane_addr + c * 32, d);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float pr = fast_exp2(fmaf(__uint_as_float(s[i]), sl2, neg_lse2));
                    if (diag && c * 32 + i > r_in_tile) pr = 0.f;
                    // P * (dP - delta) / sqrt(hs)
                    s[i] = to_tf32(pr * fmaf(__uint_as_float(d[i]), p.scale, neg_delta_s));
                }
                tmem_st32(tmem_s + lane_addr + c * 32, s);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(ds_full);
        }
        if (ok && mbar_wait(dq_done, 0, p.status, kTimeoutEpilogue)) {
            tc_fence_after_sync();
            float* out = p.dQ + grow * HS;
#pragma unroll 1
            for (int c = 0; c < HS / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_dq + lane_addr + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(out + c * 32 + i) =
                        make_float4(round_to_tf32(__uint_as_float(r[i])), round_to_tf32(__uint_as_float(r[i + 1])),
                                    round_to_tf32(__uint_as_float(r[i + 2])), round_to_tf32(__uint_as_float(r[i + 3])));
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// dK, dV: one key tile per CTA
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kBwd32Threads, 1)
attn_bwd_dkv_tf32_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_q_mn,
                         const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_do_mn,
                         const Bwd32Params p) {
    using C = Bwd32Cfg;
    constexpr int HS = kBwd32HS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* k_smem = smem;
    uint8_t* v_smem = k_smem + kBwd32Tile;
    uint8_t* q_smem = v_smem + kBwd32Tile;           // Q read along hs (scores)
    uint8_t* qmn_smem = q_smem + kBwd32Tile;         // Q read along the query rows (dK)
    uint8_t* do_smem = qmn_smem + kBwd32Tile;        // dO read along hs (dP)
    uint8_t* domn_smem = do_smem + kBwd32Tile;       // dO read along the query rows (dV)
    float* stat_s = (float*)(domn_smem + kBwd32Tile);    // [2][-lse*log2e [128], -delta/sqrt(hs) [128]]
    uint64_t* bars = (uint64_t*)(stat_s + 512);
    uint64_t* kv_full = bars;
    uint64_t* q_full = bars + 1;        // the four Q / dO tiles landed
    uint64_t* q_empty = bars + 2;       // the tile's MMAs are complete
    uint64_t* s_full = bars + 3;        // S^T and dP^T complete
    uint64_t* p_full = bars + 4;        // P^T and dS^T written (128 arrivals)
    uint64_t* acc_done = bars + 5;      // last dV, dK MMAs complete
    uint32_t* tmem_slot = (uint32_t*)(bars + 6);
    volatile uint32_t* wait_ok = tmem_slot + 1;      // [2] outcome of the bounded wait, by tile parity

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = p.S / kTile;
    const int unit = blockIdx.x % p.units;
    const int jt = blockIdx.x / p.units;                     // early key tiles have the long walks when causal
    const int i0 = p.causal ? jt : 0;
    const int n_q = n_tiles - i0;
    const int row_base = unit * p.S;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        mbar_init(s_full, 1);
        mbar_init(p_full, 128);
        mbar_init(acc_done, 1);
        fence_barrier_init();
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_q_mn);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        tma_prefetch_desc(&map_do);
        tma_prefetch_desc(&map_do_mn);
    }
    if (warp == 1) tmem_alloc(tmem_slot, C::TMEM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_st = tmem_base + C::COL_S, tmem_dpt = tmem_base + C::COL_DP;
    const uint32_t tmem_dv = tmem_base + C::COL_DV, tmem_dk = tmem_base + C::COL_DK;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            mbar_arrive_expect_tx(kv_full, 2 * kBwd32Tile);
            for (int b = 0; b < 2; ++b) {
                tma_load_2d(k_smem + b * kBoxBytes, &map_k, kv_full, b * 32, row_base + jt * kTile);
                tma_load_2d(v_smem + b * kBoxBytes, &map_v, kv_full, b * 32, row_base + jt * kTile);
            }
            for (int t = 0; t < n_q && ok; ++t) {
                if (!mbar_wait(q_empty, (t & 1) ^ 1, p.status, kTimeoutProducer)) { ok = false; break; }
                mbar_arrive_expect_tx(q_full, 4 * kBwd32Tile);
                const int y = row_base + (i0 + t) * kTile;
                for (int b = 0; b < 2; ++b) {
                    tma_load_2d(q_smem + b * kBoxBytes, &map_q, q_full, b * 32, y);
                    tma_load_2d(qmn_smem + b * kBoxBytes, &map_q_mn, q_full, b * 32, y);
                    tma_load_2d(do_smem + b * kBoxBytes, &map_do, q_full, b * 32, y);
                    tma_load_2d(domn_smem + b * kBoxBytes, &map_do_mn, q_full, b * 32, y);
                }
            }
            if (!ok)
                for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(kTF32, false, false, kTile, kTile);   // S^T = K.Q^T, dP^T = V.dO^T
            constexpr uint32_t idesc_o = make_idesc(kTF32, false, true, kTile, HS);       // dV += P^T.dO, dK += dS^T.Q
            const uint32_t k_addr = smem_u32(k_smem), v_addr = smem_u32(v_smem), q_addr = smem_u32(q_smem);
            const uint32_t qmn_addr = smem_u32(qmn_smem), do_addr = smem_u32(do_smem), domn_addr = smem_u32(domn_smem);
            bool ok = mbar_wait(kv_full, 0, p.status, kTimeoutMma);
            for (int t = 0; t < n_q && ok; ++t) {
                if (!mbar_wait(q_full, t & 1, p.status, kTimeoutMma)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < HS * 4 / 32; ++kk) {
                    const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
                    mma_ss<true>(tmem_st, smem_desc_sw128(k_addr + off, 16, 1024), smem_desc_sw128(q_addr + off, 16, 1024),
                                 idesc_s, kk > 0);
                }
#pragma unroll
                for (int kk = 0; kk < HS * 4 / 32; ++kk) {
                    const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
                    mma_ss<true>(tmem_dpt, smem_desc_sw128(v_addr + off, 16, 1024), smem_desc_sw128(do_addr + off, 16, 1024),
                                 idesc_s, kk > 0);
                }
                mma_commit(s_full);
                if (!mbar_wait(p_full, t & 1, p.status, kTimeoutMma)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < kTile / 8; ++kk)
                    mma_ts<true>(tmem_dv, tmem_st + kk * 8, smem_desc_mn(domn_addr + kk * 8 * 128, kBoxBytes, true), idesc_o,
                                 t > 0 || kk > 0);
#pragma unroll
                for (int kk = 0; kk < kTile / 8; ++kk)
                    mma_ts<true>(tmem_dk, tmem_dpt + kk * 8, smem_desc_mn(qmn_addr + kk * 8 * 128, kBoxBytes, true), idesc_o,
                                 t > 0 || kk > 0);
                mma_commit(q_empty);
            }
            if (ok) mma_commit(acc_done);
        }
    } else {
        // softmax warps: thread = key row; the statistics belong to the query columns
        const int lane_group = warp & 3;
        const int r = lane_group * 32 + lane;
        const int tid = (warp - 2) * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
        const float sl2 = p.scale * 1.4426950408889634f;
        bool ok = true;
        for (int t = 0; t < n_q; ++t) {
            const int i = i0 + t;
            // -lse (log2 domain) and -delta/sqrt(hs) of the 128 queries of this tile, one per thread.
            // Two buffers by tile parity: a thread that is already in tile t+1 writes the other
            // buffer, and it cannot reach tile t+2 before every thread has passed the barrier of t+1.
            float* lse_s = stat_s + (t & 1) * 256;
            float* delta_s = lse_s + 128;
            const int64_t qrow = (int64_t)row_base + (int64_t)i * kTile + tid;
            lse_s[tid] = p.lse[qrow] * -1.4426950408889634f;
            delta_s[tid] = p.delta[qrow] * -p.scale;
            // One thread does the bounded wait and publishes the outcome, so that all 128 take the
            // same branch and nobody is left alone at the named barrier of the next tile.  The flag
            // of this parity is rewritten two tiles later, after the barrier of the tile in between.
            if (tid == 0) wait_ok[t & 1] = mbar_wait(s_full, t & 1, p.status, kTimeoutSoftmax) ? 1u : 0u;
            named_barrier_sync(1, 128);
            if (wait_ok[t & 1] == 0u) { ok = false; break; }
            tc_fence_after_sync();
            const bool diag = p.causal && i == jt;
#pragma unroll 1
            for (int c = 0; c < kTile / 32; ++c) {
                uint32_t s[32], d[32];
                tmem_ld32(tmem_st + lane_addr + c * 32, s);
                tmem_ld32(tmem_dpt + lane_addr + c * 32, d);
                tmem_wait_ld();
#pragma unroll
                for (int x = 0; x < 32; x += 4) {
                    const float4 l4 = *reinterpret_cast<const float4*>(lse_s + c * 32 + x);
                    const float4 d4 = *reinterpret_cast<const float4*>(delta_s + c * 32 + x);
                    const float nl[4] = {l4.x, l4.y, l4.z, l4.w}, nd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float pr = fast_exp2(fmaf(__uint_as_float(s[x + e]), sl2, nl[e]));
                        if (diag && c * 32 + x + e < r) pr = 0.f;        // query q sees key r only when q >= r
                        s[x + e] = to_tf32(pr);
                        d[x + e] = to_tf32(pr * fmaf(__uint_as_float(d[x + e]), p.scale, nd[e]));
                    }
                }
                tmem_st32(tmem_st + lane_addr + c * 32, s);
                tmem_st32(tmem_dpt + lane_addr + c * 32, d);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(p_full);
        }
        // every thread waits for itself here: no barrier follows
        if (ok && mbar_wait(acc_done, 0, p.status, kTimeoutEpilogue)) {
            tc_fence_after_sync();
            const int64_t grow = (int64_t)row_base + (int64_t)jt * kTile + r;
#pragma unroll 1
            for (int which = 0; which < 2; ++which) {
                float* out = (which ? p.dK : p.dV) + grow * HS;
                const uint32_t col = which ? tmem_dk : tmem_dv;
#pragma unroll 1
                for (int c = 0; c < HS / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(col + lane_addr + c * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int x = 0; x < 32; x += 4)
                        *reinterpret_cast<float4*>(out + c * 32 + x) =
                            make_float4(round_to_tf32(__uint_as_float(v[x])), round_to_tf32(__uint_as_float(v[x + 1])),
                                        round_to_tf32(__uint_as_float(v[x + 2])), round_to_tf32(__uint_as_float(v[x + 3])));
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

}  // namespace attn_tc
}  // namespace boatcu
