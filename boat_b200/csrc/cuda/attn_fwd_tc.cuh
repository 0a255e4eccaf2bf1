// attn_fwd_tc.cuh - fused attention forward on tcgen05: scaled QK^T, causal mask, online
// softmax and PV in one kernel; the S x S matrix lives only in tensor memory, only the
// log-sum-exp per row is saved for the backward.
//
// Replaces scaled_dot_product_attention_impl (reference src/layers/attention.c:997-1073),
// which materialises scores and probabilities as [B,nh,S,S] FP32 tensors.
//
// One CTA = one 128-row query tile of one (batch,head) unit; it walks the key/value tiles of
// 128 rows.  Per key tile:
//     S  = Q . K^T            tcgen05.mma, both operands from shared memory, S in tensor memory
//     P  = exp2(S*c - m*c)    4 softmax warps, one thread per query row (TMEM lane = row):
//                             tcgen05.ld, running max m and sum l in registers, P written
//                             back over S in tensor memory (BF16 pairs, or FP32 for TF32)
//     O += P . V              tcgen05.mma, A = P from tensor memory, B = V from shared memory
//                             read along its contiguous head dimension (no transpose)
// The accumulator O is rescaled in tensor memory only when the running max has grown by more
// than 2^8 (the warp votes), the exact correction is folded into the final 1/l.
// Two CTAs share an SM (<= 112 KB shared memory, <= 256 TMEM columns each), so one CTA's
// softmax overlaps the other's MMAs.  Warp 0: TMA producer, warp 1: MMA issuer,
// warps 2-5: softmax and epilogue.
#pragma once
#include "tc_common.cuh"
#include <float.h>

namespace boatcu {
namespace attn_tc {

using namespace tc;

constexpr int kTile = 128;            // query rows per CTA and key rows per step
constexpr int kBoxBytes = kTile * 128;   // one TMA box: 128 rows x 128 bytes
constexpr int kFwdThreads = 192;

template <typename T, int HS>
struct FwdCfg {
    static constexpr int ES = sizeof(T);
    static constexpr bool TF32 = ES == 4;
    static constexpr int ROWB = HS * ES;                 // bytes per row of Q/K/V
    static constexpr int NBOX = ROWB / 128;              // boxes per 128-row tile
    static constexpr int BOXC = 128 / ES;                // elements per box row
    static constexpr int UK = 32 / ES;                   // K extent of one MMA
    static constexpr int TILE_BYTES = NBOX * kBoxBytes;
    static constexpr int KV_STAGES = TILE_BYTES <= 16384 ? 2 : 1;
    static constexpr int SMEM = TILE_BYTES * (1 + 2 * KV_STAGES) + 1024 + 256;
    static constexpr uint32_t S_COLS = kTile;            // FP32 scores, later P in place
    static constexpr uint32_t TMEM_COLS = (S_COLS + HS) <= 128 ? 128 : 256;
    static_assert(S_COLS + HS <= 256, "tensor memory budget");
    static_assert(ROWB % 128 == 0, "row must be whole 128-byte boxes");
};

struct FwdParams {
    void* O;
    float* lse;
    int S;             // sequence length (multiple of 128)
    int units;
    int causal;
    float scale;       // 1/sqrt(hs)
    unsigned int* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename T, int HS>
__global__ void __launch_bounds__(kFwdThreads, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
    using C = FwdCfg<T, HS>;
    constexpr bool TF32 = C::TF32;
    constexpr int ST = C::KV_STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = smem;
    uint8_t* k_smem = q_smem + C::TILE_BYTES;
    uint8_t* v_smem = k_smem + ST * C::TILE_BYTES;
    uint64_t* bars = (uint64_t*)(v_smem + ST * C::TILE_BYTES);
    uint64_t* q_full = bars;              // 1
    uint64_t* k_full = bars + 1;          // [ST]
    uint64_t* k_empty = k_full + ST;      // [ST]
    uint64_t* v_full = k_empty + ST;      // [ST]
    uint64_t* v_empty = v_full + ST;      // [ST]
    uint64_t* s_full = v_empty + ST;      // 1: S tile complete in TMEM
    uint64_t* p_full = s_full + 1;        // 1: P written (128 arrivals)
    uint64_t* o_done = p_full + 1;        // 1: last PV complete
    uint32_t* tmem_slot = (uint32_t*)(o_done + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_tiles = p.S / kTile;
    const int unit = blockIdx.x % p.units;
    const int qt = q_tiles - 1 - blockIdx.x / p.units;     // long (late) rows first when causal
    const int n_kv = p.causal ? qt + 1 : q_tiles;
    const int row_base = unit * p.S;                       // first row of this unit in [units*S, hs]

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < ST; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(p_full, 128);
        mbar_init(o_done, 1);
        fence_barrier_init();
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
    }
    if (warp == 1) tmem_alloc(tmem_slot, C::TMEM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base;                 // S / P
    const uint32_t tmem_o = tmem_base + C::S_COLS;     // O accumulator, HS columns

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            bool ok = true;
            mbar_arrive_expect_tx(q_full, C::TILE_BYTES);
            for (int b = 0; b < C::NBOX; ++b)
                tma_load_2d(q_smem + b * kBoxBytes, &map_q, q_full, b * C::BOXC, row_base + qt * kTile);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int s = j % ST;
                const uint32_t par = ((j / ST) & 1) ^ 1;
                const int y = row_base + j * kTile;
                if (!mbar_wait(&k_empty[s], par, p.status, kTimeoutProducer)) { ok = false; break; }
                mbar_arrive_expect_tx(&k_full[s], C::TILE_BYTES);
                for (int b = 0; b < C::NBOX; ++b)
                    tma_load_2d(k_smem + s * C::TILE_BYTES + b * kBoxBytes, &map_k, &k_full[s], b * C::BOXC, y);
                if (!mbar_wait(&v_empty[s], par, p.status, kTimeoutProducer)) { ok = false; break; }
                mbar_arrive_expect_tx(&v_full[s], C::TILE_BYTES);
                for (int b = 0; b < C::NBOX; ++b)
                    tma_load_2d(v_smem + s * C::TILE_BYTES + b * kBoxBytes, &map_v, &v_full[s], b * C::BOXC, y);
            }
            if (!ok)
                for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t fmt = TF32 ? kTF32 : kBF16;
            constexpr uint32_t idesc_s = make_idesc(fmt, false, false, kTile, kTile);   // S = Q K^T
            constexpr uint32_t idesc_o = make_idesc(fmt, false, true, kTile, HS);       // O = P V
            bool ok = mbar_wait(q_full, 0, p.status, kTimeoutMma);
            const uint32_t q_addr = smem_u32(q_smem);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int s = j % ST;
                const uint32_t par = (j / ST) & 1;
                if (!mbar_wait(&k_full[s], par, p.status, kTimeoutMma)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t k_addr = smem_u32(k_smem + s * C::TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < C::ROWB / 32; ++kk) {
                    const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
                    mma_ss<TF32>(tmem_s, smem_desc_sw128(q_addr + off, 16, 1024), smem_desc_sw128(k_addr + off, 16, 1024),
                                 idesc_s, kk > 0);
                }
                mma_commit(&k_empty[s]);
                mma_commit(s_full);
                // wait for the softmax warps to turn S into P, then accumulate P.V
                if (!mbar_wait(p_full, j & 1, p.status, kTimeoutMma)) { ok = false; break; }
                if (!mbar_wait(&v_full[s], par, p.status, kTimeoutMma)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t v_addr = smem_u32(v_smem + s * C::TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < kTile / C::UK; ++kk) {
                    mma_ts<TF32>(tmem_o, tmem_s + kk * 8, smem_desc_mn(v_addr + kk * C::UK * 128, kBoxBytes, TF32),
                                 idesc_o, j > 0 || kk > 0);
                }
                mma_commit(&v_empty[s]);
            }
            if (ok) mma_commit(o_done);
        }
    } else {
        // ---------------- softmax + epilogue: warps 2..5, thread = query row ----------------
        const int lane_group = warp & 3;
        const int r_in_tile = lane_group * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
        const float sl2 = p.scale * 1.4426950408889634f;      // scores -> log2 domain
        float m_ref = -FLT_MAX;      // max the exponentials are taken against
        float l = 0.f;               // running sum of exp
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            if (!mbar_wait(s_full, j & 1, p.status, kTimeoutSoftmax)) { ok = false; break; }
            tc_fence_after_sync();
            const bool diag = p.causal && j == qt;
            // pass 1: row maximum of the visible scores (the mask only exists on the diagonal tile).
            // The 32-column chunks are double-buffered in registers: the load of the next chunk is
            // in flight while this one is reduced, and four running maxima keep the chain short.
            float tmax;
            {
                uint32_t rr[2][32];
                float t4[4] = {-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX};
                tmem_ld32(tmem_s + lane_addr, rr[0]);
#pragma unroll
                for (int c = 0; c < kTile / 32; ++c) {
                    tmem_wait_ld();
                    if (c + 1 < kTile / 32) tmem_ld32(tmem_s + lane_addr + (c + 1) * 32, rr[(c + 1) & 1]);
                    const uint32_t(&r)[32] = rr[c & 1];
                    if (diag) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c * 32 + i <= r_in_tile) t4[i & 3] = fmaxf(t4[i & 3], __uint_as_float(r[i]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i += 2)
                            t4[(i >> 1) & 3] = fmaxf(t4[(i >> 1) & 3], fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
                    }
                }
                tmax = fmaxf(fmaxf(t4[0], t4[1]), fmaxf(t4[2], t4[3]));
            }
            const float m_new = fmaxf(m_ref, tmax);
            const bool need = (j == 0) || (m_new - m_ref) * sl2 > 8.0f;
            if (__any_sync(0xffffffffu, need)) {
                float alpha = 1.f;
                if (need) {
                    alpha = (j == 0) ? 0.f : fast_exp2((m_ref - m_new) * sl2);
                    m_ref = m_new;
                    l *= alpha;
                }
                if (j > 0) {
                    // S_j is complete, so every earlier P.V has completed too (in-order pipe)
#pragma unroll 1
                    for (int c = 0; c < HS / 32; ++c) {
                        uint32_t r[32];
                        tmem_ld32(tmem_o + lane_addr + c * 32, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st32(tmem_o + lane_addr + c * 32, r);
                    }
                    tmem_wait_st();
                }
            }
            // pass 2: P = exp2(s*sl2 - m*sl2), written over S; same double buffering.  P of chunk c
            // lands in columns that belong to chunks already loaded (BF16: [16c, 16c+16), TF32: the
            // chunk's own), never in those of the chunk in flight.
            const float neg_m = -m_ref * sl2;
            float lsum;
            {
                uint32_t rr[2][32];
                float l4[4] = {0.f, 0.f, 0.f, 0.f};
                tmem_ld32(tmem_s + lane_addr, rr[0]);
#pragma unroll
                for (int c = 0; c < kTile / 32; ++c) {
                    tmem_wait_ld();
                    if (c + 1 < kTile / 32) tmem_ld32(tmem_s + lane_addr + (c + 1) * 32, rr[(c + 1) & 1]);
                    uint32_t(&r)[32] = rr[c & 1];
                    float pv[32];
                    if (diag) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            float e = fast_exp2(fmaf(__uint_as_float(r[i]), sl2, neg_m));
                            pv[i] = (c * 32 + i > r_in_tile) ? 0.f : e;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) pv[i] = fast_exp2(fmaf(__uint_as_float(r[i]), sl2, neg_m));
                    }
                    if (TF32) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            // round to the nearest TF32 value: the MMA would otherwise truncate
                            uint32_t t32;
                            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t32) : "f"(pv[i]));
                            l4[i & 3] += __uint_as_float(t32);
                            r[i] = t32;
                        }
                        tmem_st32(tmem_s + lane_addr + c * 32, r);
                    } else {
                        uint32_t h[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            __nv_bfloat162 b2 = __floats2bfloat162_rn(pv[2 * i], pv[2 * i + 1]);
                            l4[i & 3] += pv[2 * i] + pv[2 * i + 1];
                            h[i] = *reinterpret_cast<uint32_t*>(&b2);
                        }
                        tmem_st16(tmem_s + lane_addr + c * 16, h);
                    }
                }
                lsum = (l4[0] + l4[1]) + (l4[2] + l4[3]);
            }
            l += lsum;
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(p_full);
        }
        // epilogue: O / l -> global, lse = m*scale + ln(l)
        if (ok && mbar_wait(o_done, 0, p.status, kTimeoutEpilogue)) {
            tc_fence_after_sync();
            const float inv = 1.f / l;
            const int64_t grow = (int64_t)row_base + (int64_t)qt * kTile + r_in_tile;
            T* out = (T*)p.O + grow * HS;
#pragma unroll 1
            for (int c = 0; c < HS / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_o + lane_addr + c * 32, r);
                tmem_wait_ld();
                if (TF32) {
#pragma unroll
                    // TF32-valued output: it feeds the TF32 output projection
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>((float*)out + c * 32 + i) =
                            make_float4(round_to_tf32(__uint_as_float(r[i]) * inv), round_to_tf32(__uint_as_float(r[i + 1]) * inv),
                                        round_to_tf32(__uint_as_float(r[i + 2]) * inv), round_to_tf32(__uint_as_float(r[i + 3]) * inv));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 o;
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                        __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
                        __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
                        o.x = *reinterpret_cast<uint32_t*>(&h0);
                        o.y = *reinterpret_cast<uint32_t*>(&h1);
                        o.z = *reinterpret_cast<uint32_t*>(&h2);
                        o.w = *reinterpret_cast<uint32_t*>(&h3);
                        *reinterpret_cast<uint4*>((__nv_bfloat16*)out + c * 32 + i) = o;
                    }
                }
            }
            p.lse[grow] = m_ref * p.scale + logf(l);
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
