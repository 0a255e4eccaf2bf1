// attn_fwd_tc.cuh - fused attention forward on tcgen05: scaled QK^T, causal mask, online
// softmax and PV in one kernel; the S x S matrix lives only in tensor memory, only the
// log-sum-exp per row is saved for the backward.
//
// Replaces scaled_dot_product_attention_impl (reference src/layers/attention.c:997-1073),
// which materialises scores and probabilities as [B,nh,S,S] FP32 tensors.
//
// One CTA owns an SM and two adjacent 128-row query tiles A and B of one (batch, head) unit and
// walks the key/value tiles of 128 rows.  Per key tile and query tile:
//     S  = Q . K^T            tcgen05.mma, both operands from shared memory, S in tensor memory
//     P  = exp2(S*c - m*c)    4 softmax warps per query tile, one thread per query row (TMEM lane =
//                             row): the row of 128 scores comes into registers with one
//                             tcgen05.ld wait, running max m and sum l stay in registers, P is
//                             written back over S (BF16 pairs, or TF32-valued FP32)
//     O += P . V              tcgen05.mma, A = P from tensor memory, B = V from shared memory
//                             read along its contiguous head dimension (no transpose)
// The accumulator O is rescaled in tensor memory only when the running max has grown by more
// than 2^8 (the warp votes), the exact correction is folded into the final 1/l.
//
// One thread issues the MMAs of both query tiles in a fixed order,
//     S_A(0) S_B(0) | P.V_A(0) S_A(1) | P.V_B(0) S_B(1) | P.V_A(1) S_A(2) | ...
// so that the exponentials of tile A's step run under the MMAs of tile B and the other way
// round (with one query tile per CTA and two CTAs per SM nothing orders the two, and they
// drift into doing their exponentials at the same time on the SM's one special-function unit).
// K and V tiles are loaded once for both query tiles; CTAs of a few units at a time are scheduled
// together so that those tiles stay in L2.
//
// Warp 0: TMA producer; warp 1: MMA issuer; warps 2-5: softmax and epilogue of tile A;
// warps 6-9: of tile B.  Tensor memory: S/P of A and B in columns [0,128) and [128,256), the
// two O accumulators behind them.
#pragma once
#include "tc_common.cuh"
#include <float.h>

namespace boatcu {
namespace attn_tc {

using namespace tc;

constexpr int kTile = 128;            // query rows per CTA and key rows per step
constexpr int kBoxBytes = kTile * 128;   // one TMA box: 128 rows x 128 bytes
constexpr int kFwdThreads = 320;     // producer, MMA issuer, 2 x 4 softmax warps

template <typename T, int HS>
struct FwdCfg {
    static constexpr int ES = sizeof(T);
    static constexpr bool TF32 = ES == 4;
    static constexpr int ROWB = HS * ES;                 // bytes per row of Q/K/V
    static constexpr int NBOX = ROWB / 128;              // boxes per 128-row tile
    static constexpr int BOXC = 128 / ES;                // elements per box row
    static constexpr int UK = 32 / ES;                   // K extent of one MMA
    static constexpr int TILE_BYTES = NBOX * kBoxBytes;
    static constexpr int KV_STAGES = TILE_BYTES <= 16384 ? 3 : 2;
    static constexpr int SMEM = TILE_BYTES * (2 + 2 * KV_STAGES) + 1024 + 256;   // Q of both tiles, K and V rings
    static constexpr uint32_t COL_O = 2 * kTile;         // S/P of tiles A and B, then O of A, then O of B
    static constexpr uint32_t TMEM_COLS = 512;           // 2 x (128 + HS) rounded up to a power of two
    static_assert(2 * (kTile + HS) <= 512, "tensor memory budget");
    static_assert(SMEM <= 227 * 1024, "shared memory budget");
    static_assert(ROWB % 128 == 0, "row must be whole 128-byte boxes");
};

struct FwdParams {
    void* O;
    float* lse;
    int S;             // sequence length (multiple of 128)
    int units;
    int causal;
    float scale;       // 1/sqrt(hs)
    int group;         // units whose CTAs are scheduled together (their K and V share L2)
    unsigned int* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One row of 128 scores in registers -> probabilities exp2(s*sl2 + neg_m) in place (BF16: packed
// pairs in sc[0..63]; TF32: TF32-valued floats in sc[0..127]); returns their sum.  Columns beyond
// `last` are masked (DIAG only).  DIAG is a template parameter so that the loop body is one
// straight-line block: a branch per element pair would keep the compiler from overlapping the
// pairs' FMA -> exp2 -> convert chains, and a lone warp would then run at the chain's latency.
template <bool TF32, bool DIAG>
__device__ __forceinline__ float exp_row(uint32_t (&sc)[kTile], float sl2, float neg_m, int last) {
    const uint64_t sl2_2 = pack_f32x2(sl2, sl2), neg_m2 = pack_f32x2(neg_m, neg_m);
    uint64_t l2[4] = {0ull, 0ull, 0ull, 0ull};          // four chains of (even, odd) partial sums
#pragma unroll
    for (int i = 0; i < kTile; i += 2) {
        float x0, x1;
        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sc[i]), __uint_as_float(sc[i + 1])), sl2_2, neg_m2), x0, x1);
        float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
        if (DIAG) {
            e0 = i > last ? 0.f : e0;
            e1 = i + 1 > last ? 0.f : e1;
        }
        if (TF32) {
            // round to the nearest TF32 value: the MMA would otherwise truncate
            e0 = round_to_tf32(e0);
            e1 = round_to_tf32(e1);
            sc[i] = __float_as_uint(e0);
            sc[i + 1] = __float_as_uint(e1);
        } else {
            __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
            sc[i >> 1] = *reinterpret_cast<uint32_t*>(&b2);
        }
        l2[(i >> 1) & 3] = add_f32x2(l2[(i >> 1) & 3], pack_f32x2(e0, e1));
    }
    float a0, a1;
    unpack_f32x2(add_f32x2(add_f32x2(l2[0], l2[1]), add_f32x2(l2[2], l2[3])), a0, a1);
    return a0 + a1;
}

template <typename T, int HS>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
    using C = FwdCfg<T, HS>;
    constexpr bool TF32 = C::TF32;
    constexpr int ST = C::KV_STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = smem;                               // tile A, then tile B
    uint8_t* k_smem = q_smem + 2 * C::TILE_BYTES;
    uint8_t* v_smem = k_smem + ST * C::TILE_BYTES;
    uint64_t* bars = (uint64_t*)(v_smem + ST * C::TILE_BYTES);
    uint64_t* q_full = bars;              // 1
    uint64_t* k_full = bars + 1;          // [ST]
    uint64_t* k_empty = k_full + ST;      // [ST]
    uint64_t* v_full = k_empty + ST;      // [ST]
    uint64_t* v_empty = v_full + ST;      // [ST]
    uint64_t* s_full = v_empty + ST;      // [2]: S of tile A / B complete in tensor memory
    uint64_t* p_full = s_full + 2;        // [2]: P of tile A / B written (128 arrivals each)
    uint64_t* o_done = p_full + 2;        // 1: every MMA complete
    uint32_t* tmem_slot = (uint32_t*)(o_done + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_tiles = p.S / kTile;
    const int n_pairs = (q_tiles + 1) / 2;
    // CTA order: units in groups of p.group, so that the K and V tiles which the CTAs running at one
    // time stream through shared memory (every CTA of a unit reads all of the unit's K and V) stay
    // in L2; inside a group the tile pair is the slow index, long (late) rows first when causal.
    // When the units do not divide into whole groups the short group goes first: the launch then ends
    // with the short CTAs of a full group, which fill the SMs evenly.
    const int per_group = p.group * n_pairs;
    const int short_group = p.units % p.group;             // 0: all groups are whole
    const int short_ctas = short_group * n_pairs;
    int unit0, in_group, rem;
    if ((int)blockIdx.x < short_ctas) {
        unit0 = 0;
        in_group = short_group;
        rem = blockIdx.x;
    } else {
        const int b = blockIdx.x - short_ctas;
        const int grp = b / per_group;
        unit0 = short_group + grp * p.group;
        in_group = p.group;
        rem = b - grp * per_group;
    }
    const int unit = unit0 + rem % in_group;
    const int pt = n_pairs - 1 - rem / in_group;
    const int qt_a = 2 * pt, qt_b = 2 * pt + 1;
    const bool has_b = qt_b < q_tiles;                     // an odd tile count leaves the last CTA one tile
    const int n_a = p.causal ? qt_a + 1 : q_tiles;
    const int n_b = has_b ? (p.causal ? qt_b + 1 : q_tiles) : 0;
    const int n_kv = n_a > n_b ? n_a : n_b;
    const int row_base = unit * p.S;                       // first row of this unit in [units*S, hs]

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < ST; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int g = 0; g < 2; ++g) {
            mbar_init(&s_full[g], 1);
            mbar_init(&p_full[g], 128);
        }
        mbar_init(o_done, 1);
        fence_barrier_init();
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        // This thread is also the producer: the loads that wait for nothing - both query tiles and the
        // first ring-full of key and value tiles - start here, under the tensor-memory allocation
        // and the CTA's first barrier.
        mbar_arrive_expect_tx(q_full, (has_b ? 2 : 1) * C::TILE_BYTES);
        for (int g = 0; g < (has_b ? 2 : 1); ++g)
            for (int b = 0; b < C::NBOX; ++b)
                tma_load_2d(q_smem + g * C::TILE_BYTES + b * kBoxBytes, &map_q, q_full, b * C::BOXC,
                            row_base + (qt_a + g) * kTile);
        for (int j = 0; j < n_kv && j < ST; ++j) {
            const int y = row_base + j * kTile;
            mbar_arrive_expect_tx(&k_full[j], C::TILE_BYTES);
            for (int b = 0; b < C::NBOX; ++b)
                tma_load_2d(k_smem + j * C::TILE_BYTES + b * kBoxBytes, &map_k, &k_full[j], b * C::BOXC, y);
            mbar_arrive_expect_tx(&v_full[j], C::TILE_BYTES);
            for (int b = 0; b < C::NBOX; ++b)
                tma_load_2d(v_smem + j * C::TILE_BYTES + b * kBoxBytes, &map_v, &v_full[j], b * C::BOXC, y);
        }
    }
    if (warp == 1) tmem_alloc(tmem_slot, C::TMEM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            bool ok = true;
            for (int j = ST; j < n_kv && ok; ++j) {               // the first ST tiles are on their way
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
            tc_fence_after_sync();
            // S of tile g against key tile j (already waited for) into the tile's S columns
            auto issue_s = [&](int g, int j) {
                const uint32_t q_addr = smem_u32(q_smem + g * C::TILE_BYTES);
                const uint32_t k_addr = smem_u32(k_smem + (j % ST) * C::TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < C::ROWB / 32; ++kk) {
                    const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
                    mma_ss<TF32>(tmem_base + g * kTile, smem_desc_sw128(q_addr + off, 16, 1024),
                                 smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, kk > 0);
                }
                mma_commit(&s_full[g]);
            };
            // O of tile g += P (over the tile's S columns) . V_j
            auto issue_pv = [&](int g, int j) {
                const uint32_t v_addr = smem_u32(v_smem + (j % ST) * C::TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < kTile / C::UK; ++kk) {
                    mma_ts<TF32>(tmem_base + C::COL_O + g * HS, tmem_base + g * kTile + kk * 8,
                                 smem_desc_mn(v_addr + kk * C::UK * 128, kBoxBytes, TF32), idesc_o, j > 0 || kk > 0);
                }
            };
            if (ok && mbar_wait(&k_full[0], 0, p.status, kTimeoutMma)) {
                tc_fence_after_sync();
                issue_s(0, 0);
                if (has_b) issue_s(1, 0);
                mma_commit(&k_empty[0]);
            } else {
                ok = false;
            }
            for (int j = 0; j < n_kv && ok; ++j) {
                const uint32_t par = (j / ST) & 1;
                const bool next = j + 1 < n_kv;
                const uint32_t par_next = ((j + 1) / ST) & 1;
                bool v_waited = false, k_waited = false;
                for (int g = 0; g < 2 && ok; ++g) {
                    const int n_g = g ? n_b : n_a;
                    if (j < n_g) {
                        if (!mbar_wait(&p_full[g], j & 1, p.status, kTimeoutMma)) { ok = false; break; }
                        if (!v_waited && !mbar_wait(&v_full[j % ST], par, p.status, kTimeoutMma)) { ok = false; break; }
                        v_waited = true;
                        tc_fence_after_sync();
                        issue_pv(g, j);
                    }
                    if (j + 1 < n_g) {
                        if (!k_waited && !mbar_wait(&k_full[(j + 1) % ST], par_next, p.status, kTimeoutMma)) { ok = false; break; }
                        k_waited = true;
                        tc_fence_after_sync();
                        issue_s(g, j + 1);
                    }
                }
                if (!ok) break;
                mma_commit(&v_empty[j % ST]);                    // both tiles' P.V of this step are issued
                if (next) mma_commit(&k_empty[(j + 1) % ST]);   // and both S of the next
            }
            if (ok) mma_commit(o_done);
        }
    } else {
        // ---------------- softmax + epilogue: warps 2..5 tile A, 6..9 tile B; thread = query row ----------------
        const int g = (warp - 2) >> 2;
        const int n_g = g ? n_b : n_a;
        const int qt = g ? qt_b : qt_a;
        const int lane_group = warp & 3;
        const int r_in_tile = lane_group * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
        const uint32_t tmem_s = tmem_base + g * kTile;
        const uint32_t tmem_o = tmem_base + C::COL_O + g * HS;
        const float sl2 = p.scale * 1.4426950408889634f;      // scores -> log2 domain
        float m_ref = -FLT_MAX;      // max the exponentials are taken against
        float l = 0.f;               // running sum of exp
        bool ok = true;
        for (int j = 0; j < n_g; ++j) {
            if (!mbar_wait(&s_full[g], j & 1, p.status, kTimeoutSoftmax)) { ok = false; break; }
            tc_fence_after_sync();
            const bool diag = p.causal && j == qt;
            // The whole row of scores (128 columns) comes into registers with one wait; the maximum and
            // the exponentials both work from there.
            uint32_t sc[kTile];
#pragma unroll
            for (int c = 0; c < kTile / 32; ++c)
                tmem_ld32(tmem_s + lane_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(sc + c * 32));
            tmem_wait_ld();
            // row maximum of the visible scores (the mask only exists on the diagonal tile)
            float tmax;
            {
                float t8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) t8[i] = -FLT_MAX;
                if (diag) {
#pragma unroll
                    for (int i = 0; i < kTile; ++i)
                        t8[i & 7] = fmaxf(t8[i & 7], i <= r_in_tile ? __uint_as_float(sc[i]) : -FLT_MAX);
                } else {
#pragma unroll
                    for (int i = 0; i < kTile; i += 2)
                        t8[(i >> 1) & 7] = max3_f32(t8[(i >> 1) & 7], __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
                }
                tmax = fmaxf(max3_f32(t8[0], t8[1], t8[2]), max3_f32(t8[3], t8[4], t8[5]));
                tmax = max3_f32(tmax, t8[6], t8[7]);
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
                    // S_j of this tile is complete, so its earlier P.V have completed too (the MMA
                    // thread issues S_j behind P.V_(j-1) and the pipe is in order)
#pragma unroll 1
                    for (int c = 0; c < HS / 16; ++c) {
                        uint32_t r[16];
                        tmem_ld16(tmem_o + lane_addr + c * 16, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st16(tmem_o + lane_addr + c * 16, r);
                    }
                    tmem_wait_st();
                }
            }
            // P = exp2(s*sl2 - m*sl2) in place in the registers (BF16: packed pairs in the first 64),
            // two elements per FMA-pipe instruction, then written over S
            const float neg_m = -m_ref * sl2;
            float lsum;
            {
                lsum = diag ? exp_row<TF32, true>(sc, sl2, neg_m, r_in_tile) : exp_row<TF32, false>(sc, sl2, neg_m, r_in_tile);
                constexpr int P_CHUNKS = TF32 ? kTile / 32 : kTile / 64;
#pragma unroll
                for (int c = 0; c < P_CHUNKS; ++c)
                    tmem_st32(tmem_s + lane_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(sc + c * 32));
            }
            l += lsum;
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&p_full[g]);
        }
        // epilogue: O / l -> global, lse = m*scale + ln(l)
        if (n_g > 0 && ok && mbar_wait(o_done, 0, p.status, kTimeoutEpilogue)) {
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
