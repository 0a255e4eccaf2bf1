// attn_bwd_tc.cuh - fused attention backward on tcgen05 (BF16 storage, FP32 accumulation).
//
// Replaces attention_backward (reference src/layers/attention.c:1421-1526), which keeps the
// probabilities of the forward and builds four more [B,nh,S,S] tensors.  Here P is rebuilt
// from the saved log-sum-exp, tile by tile, and nothing of size S x S touches HBM.
//
// A walk: one 128-row key/value tile of one (batch,head) unit against the query tiles that see
// it (all of them, or those at or below the diagonal when causal).  K and V stay in shared
// memory, dK and dV accumulate in tensor memory for the whole walk.  A CTA does two walks of
// its unit back to back (when causal, tile j and tile n-1-j: n+1 query tiles for every CTA).
// Per query tile, with everything transposed so that key rows sit on the TMEM lanes:
//
//   S^T  = K . Q^T                                              SS MMA into region R0
//   P^T  = exp2(S^T*c - lse)        phase A, 8 softmax warps, written over S^T in R0 (BF16)
//   dV  += P^T . dO                 A = P^T in tensor memory
//   dP^T = V . dO^T                 SS MMA into R0 again, behind dV on the in-order tensor pipe
//   dS^T = P^T * (dP^T - delta) / sqrt(hs)    phase B; P^T is kept in registers, dS^T goes to smem
//   dK  += dS^T . Q                 A = dS^T from shared memory (K-major view)
//   dQ_i = dS . K                   A = the same shared-memory tile read along M (MN-major view)
//
// Tensor memory (512 columns): R0 = S^T / P^T (128), dQ (HS), dV (HS), dK (HS); with head size
// 128 that is all of it and dP^T borrows the dQ columns: the dQ warps take a tile's dQ into
// registers and shared memory within a few hundred cycles of its completion, and the next dQ
// product only comes after the softmax warps have consumed dP^T.  With head size 64 dP^T has 128
// columns of its own.  In both cases dP^T is issued a tile ahead, S^T of tile t+1 follows dV of
// tile t on the pipe, and the softmax warps - the critical resource - go from the exponentials
// (A) straight to dS^T (B) without waiting for the tensor pipe.
//
// dQ of a query tile gets one contribution per key tile; CTAs add theirs into an FP32 buffer
// with TMA reduce-add (cp.reduce.async.bulk.tensor), and a cast kernel turns the sum into the
// output type afterwards.  Four dedicated warps move the dQ tile out of tensor memory through
// the tile's dO stage, which is idle once the tile's MMAs are complete, half a tile at a time;
// the thread that issues the reductions then loads the dO tile two steps ahead into it.  An SM
// gets reductions out at only about 20 bytes per clock (measured alike for TMA reduce-add and
// for red.global.add.v4.f32, which also stalls the softmax warps' shared memory traffic), so
// the read-out of a tile takes most of a tile period - off the critical path.
// The softmax warps synchronise only through the mbarriers of the pipeline - no barrier among
// themselves inside a walk: the per-row statistics of a query tile (-lse*log2e and
// -delta/sqrt(hs), pre-scaled by a small kernel) are brought in by the producer with two bulk
// copies per tile.
// Warp 0: TMA producer (K, V, Q, statistics), warp 1: MMA issuer, warps 2-9: softmax + final dK/dV store
// (two warps per TMEM lane group, 64 query columns each), warps 10-13: dQ reduction.
#pragma once
#include <type_traits>
#include "attn_fwd_tc.cuh"

namespace boatcu {
namespace attn_tc {

constexpr int kBwdThreads = 448;

template <int HS>
struct BwdCfg {
    static constexpr int ROWB = HS * 2;
    static constexpr int NBOX = ROWB / 128;
    static constexpr int TILE_BYTES = NBOX * kBoxBytes;       // one 128 x HS BF16 tile
    static constexpr int DS_BYTES = 2 * kBoxBytes;             // dS^T: 128 x 128 BF16
    // Q / dO stages: three when they fit (head size 64), so that the dO tile loaded behind a
    // dQ read-out is not needed before the tile after next
    static constexpr int Q_STAGES = HS == 64 ? 3 : 2;
    // K,V + Q,dO stages + dS^T + two (lse, delta) buffers + barriers.  With head size 128 this
    // is 231,680 of the 232,448 bytes a CTA may have, so the base must come 1024-byte aligned
    // from the launch (checked at kernel entry) - there is no room for manual alignment slack.
    static constexpr int SMEM = 2 * TILE_BYTES + Q_STAGES * 2 * TILE_BYTES + DS_BYTES + 2048 + 256;
    // tensor memory columns
    // R0 (columns 0..127) holds S^T, then P^T.  With head size 64 dP^T has 128 columns of its
    // own.  With head size 128 nothing is left (R0 + dQ + dV + dK = 512), and dP^T borrows the dQ
    // columns: they are idle from the moment the dQ warps hold a tile's dQ in registers and
    // shared memory until the next tile's dQ product, which needs dS^T and therefore comes after
    // the softmax warps have read dP^T anyway.  Either way dP^T of a tile is issued before the
    // softmax warps ask for it, and they go from the exponentials straight on to dS^T.
    static constexpr bool DP_OWN = 256 + 3 * HS <= 512;
    static constexpr uint32_t COL_S = 0;
    static constexpr uint32_t COL_DQ = DP_OWN ? 256 : 128, COL_DV = COL_DQ + HS, COL_DK = COL_DQ + 2 * HS;
    static constexpr uint32_t COL_DP = DP_OWN ? 128 : COL_DQ;
    static constexpr uint32_t TMEM_COLS = 512;
};

struct BwdParams {
    const float* lse2;     // [units*S]  -lse * log2(e): the exponent offset in the log2 domain
    const float* delta2;   // [units*S]  -delta / sqrt(hs)
    float* dq_accum;       // [units*S, hs] FP32, zeroed before the launch
    void* dK;
    void* dV;
    int S, units, causal;
    int group;             // units scheduled together, see the kernel
    int pair;              // 1: a CTA walks two key tiles of its unit, 0: one
    float scale;
    unsigned int* status;
};

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int HS>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                 const __grid_constant__ CUtensorMap map_dq, const BwdParams p) {
    using C = BwdCfg<HS>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    if ((smem_u32(smem) & 1023u) != 0) {         // uniform for the whole CTA; nothing to undo yet
        if (threadIdx.x == 0) atomicCAS(p.status, 0u, (unsigned int)kTimeoutOther + 100u);
        return;
    }
    uint8_t* k_smem = smem;
    uint8_t* v_smem = k_smem + C::TILE_BYTES;
    uint8_t* q_smem = v_smem + C::TILE_BYTES;                          // [Q_STAGES]
    uint8_t* do_smem = q_smem + C::Q_STAGES * C::TILE_BYTES;           // [Q_STAGES]
    uint8_t* ds_smem = do_smem + C::Q_STAGES * C::TILE_BYTES;
    float* stat_s = (float*)(ds_smem + C::DS_BYTES);                   // [2][-lse*log2e[128], -delta/sqrt(hs)[128]]
    uint64_t* bars = (uint64_t*)(stat_s + 512);
    uint64_t* kv_full = bars;                   // 1
    uint64_t* q_full = bars + 16;               // [Q_STAGES] Q tile landed
    uint64_t* s_full = bars + 5;                // S^T complete
    uint64_t* ds_full = bars + 6;               // dS^T in smem (256 arrivals)
    uint64_t* dq_full = bars + 7;               // all MMAs of the tile complete
    uint64_t* dq_empty = bars + 8;              // dQ is out of its TMEM columns
    uint64_t* all_done = bars + 9;
    uint64_t* dp_full = bars + 10;              // dP^T complete
    uint64_t* do_full = bars + 19;              // [Q_STAGES] dO tile landed
    uint64_t* q_empty = bars + 22;              // [Q_STAGES] S^T and dK of the tile are complete: its Q stage is free
    uint64_t* p_full = bars + 3;                // P^T in TMEM (256 arrivals)
    uint64_t* kv_empty = bars + 1;              // the first walk's MMAs are complete: K and V may be replaced
    uint64_t* acc_free = bars + 2;              // dK, dV of the first walk are stored (256 arrivals)
    uint64_t* stat_full = bars + 11;            // [2] the tile's statistics landed
    uint64_t* stat_empty = bars + 13;           // [2] phase B of the tile is over (256 arrivals)
    uint32_t* tmem_slot = (uint32_t*)(bars + 25);
    volatile uint32_t* drain_ok = tmem_slot + 3;       // same idea for the dQ warps

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = p.S / kTile;
    // CTA order: units in groups of p.group; inside a group the key-tile pair is the slow index.
    // The CTAs that run at the same time then belong to a few (batch, head) units, so the FP32 dQ
    // rows they reduce into (S*HS*4 bytes per unit) and the unit's Q and dO stay in L2 - with
    // key tiles as the slow index over all units, the dQ buffer of a large problem (268 MB at 64
    // units x 8192 x 128) no longer fits and every reduction misses to HBM.
    // A CTA walks two key tiles of its unit, one after the other: with a causal mask tile pj and
    // tile n_tiles-1-pj, whose walks together are n_tiles+1 query tiles for every pj, so all CTAs
    // carry the same load; without a mask two neighbouring tiles.  Start-up, the last tile's
    // read-out and the exit of a CTA are paid once per pair, and the second walk starts while the
    // first one's dQ is still draining.
    // (p.pair == 0: one walk per CTA - better when the walks are long or the CTAs few, see the
    // launcher.)
    const int n_pairs = p.pair ? (n_tiles + 1) / 2 : n_tiles;
    const int per_group = p.group * n_pairs;
    const int grp = blockIdx.x / per_group;
    const int rem = blockIdx.x - grp * per_group;
    const int in_group = min(p.group, p.units - grp * p.group);
    const int pj = rem / in_group;
    const int unit = grp * p.group + rem % in_group;
    const int jtA = !p.pair || p.causal ? pj : 2 * pj;
    const int jtB = p.causal ? n_tiles - 1 - pj : 2 * pj + 1;
    const bool has_b = p.pair && jtB != jtA && jtB < n_tiles;
    const int ibA = p.causal ? jtA : 0, ibB = p.causal ? jtB : 0;
    const int nA = n_tiles - ibA;                       // query tiles of the first walk
    const int n_q = nA + (has_b ? n_tiles - ibB : 0);   // of both
    const int row_base = unit * p.S;
    // query tile and key tile of step gt of the combined walk
    auto qtile = [&](int gt) { return gt < nA ? ibA + gt : ibB + gt - nA; };

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        for (int s = 0; s < C::Q_STAGES; ++s) {
            mbar_init(&q_full[s], 1);
            mbar_init(&do_full[s], 1);
            mbar_init(&q_empty[s], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(ds_full, 256);
        mbar_init(p_full, 256);
        mbar_init(dp_full, 1);
        mbar_init(dq_full, 1);
        mbar_init(dq_empty, 1);
        mbar_init(all_done, 1);
        mbar_init(kv_empty, 1);
        mbar_init(acc_free, 256);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&stat_full[b], 1);
            mbar_init(&stat_empty[b], 256);
        }
        fence_barrier_init();
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        tma_prefetch_desc(&map_do);
        tma_prefetch_desc(&map_dq);
        // This thread is also the producer: the loads that wait for nothing - K and V of the first
        // walk, dO of the first Q_STAGES query tiles (later ones are loaded by the dQ warps, which
        // stage dQ through the dO buffers and know when one is free again) - start here, under the
        // tensor-memory allocation and the CTA's first barrier.
        mbar_arrive_expect_tx(kv_full, 2 * C::TILE_BYTES);
        for (int b = 0; b < C::NBOX; ++b) {
            tma_load_2d(k_smem + b * kBoxBytes, &map_k, kv_full, b * 64, row_base + jtA * kTile);
            tma_load_2d(v_smem + b * kBoxBytes, &map_v, kv_full, b * 64, row_base + jtA * kTile);
        }
        for (int t = 0; t < n_q && t < C::Q_STAGES; ++t) {
            mbar_arrive_expect_tx(&do_full[t], C::TILE_BYTES);
            for (int b = 0; b < C::NBOX; ++b)
                tma_load_2d(do_smem + t * C::TILE_BYTES + b * kBoxBytes, &map_do, &do_full[t], b * 64,
                            row_base + qtile(t) * kTile);
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
            auto load_kv = [&](int jt) {
                mbar_arrive_expect_tx(kv_full, 2 * C::TILE_BYTES);
                for (int b = 0; b < C::NBOX; ++b) {
                    tma_load_2d(k_smem + b * kBoxBytes, &map_k, kv_full, b * 64, row_base + jt * kTile);
                    tma_load_2d(v_smem + b * kBoxBytes, &map_v, kv_full, b * 64, row_base + jt * kTile);
                }
            };
            for (int t = 0; t < n_q; ++t) {
                if (t == nA) {                  // second walk: its K and V, once the first walk's MMAs are done
                    if (!mbar_wait(kv_empty, 0, p.status, kTimeoutProducer)) break;
                    load_kv(jtB);
                }
                const int s = t % C::Q_STAGES;
                if (!mbar_wait(&q_empty[s], ((t / C::Q_STAGES) & 1) ^ 1, p.status, kTimeoutProducer)) break;
                mbar_arrive_expect_tx(&q_full[s], C::TILE_BYTES);
                for (int b = 0; b < C::NBOX; ++b)
                    tma_load_2d(q_smem + s * C::TILE_BYTES + b * kBoxBytes, &map_q, &q_full[s], b * 64,
                                row_base + qtile(t) * kTile);
                // the tile's 128 exponent offsets and 128 deltas, into the buffer of its parity once
                // the tile before last has left it
                if (!mbar_wait(&stat_empty[t & 1], ((t >> 1) & 1) ^ 1, p.status, kTimeoutProducer)) break;
                mbar_arrive_expect_tx(&stat_full[t & 1], 1024);
                bulk_load_1d(stat_s + (t & 1) * 256, p.lse2 + row_base + qtile(t) * kTile, 512, &stat_full[t & 1]);
                bulk_load_1d(stat_s + (t & 1) * 256 + 128, p.delta2 + row_base + qtile(t) * kTile, 512, &stat_full[t & 1]);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_st = make_idesc(kBF16, false, false, kTile, kTile);   // K.Q^T, V.dO^T
            constexpr uint32_t idesc_acc = make_idesc(kBF16, false, true, kTile, HS);      // dV, dK
            constexpr uint32_t idesc_dq = make_idesc(kBF16, true, true, kTile, HS);        // dQ
            const uint32_t k_addr = smem_u32(k_smem), v_addr = smem_u32(v_smem), ds_addr = smem_u32(ds_smem);
            // Issue order on the (in-order) tensor pipe, per tile t:
            //   dV(t) S(t+1) | dQ(t) dK(t) | dP(t+1)
            // dV follows phase A; S^T of the next tile overwrites R0 right behind it (dV, ahead on
            // the pipe, is the only reader of P^T).  dK and dQ need dS^T from phase B.  dP^T of the
            // next tile follows them: into its own columns (head size 64), or into the dQ columns
            // once the dQ warps have taken this tile's dQ out of them (head size 128) - in both
            // cases long before phase B of the next tile asks for it.
            auto issue_s = [&](int t) -> bool {
                const int s = t % C::Q_STAGES;
                if (!mbar_wait(&q_full[s], (t / C::Q_STAGES) & 1, p.status, kTimeoutMma)) return false;
                tc_fence_after_sync();
                const uint32_t q_addr = smem_u32(q_smem + s * C::TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < C::ROWB / 32; ++kk) {
                    const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
                    mma_ss<false>(tmem_base + C::COL_S, smem_desc_sw128(k_addr + off, 16, 1024),
                                  smem_desc_sw128(q_addr + off, 16, 1024), idesc_st, kk > 0);
                }
                mma_commit(s_full);
                return true;
            };
            auto issue_dp = [&](int t) -> bool {        // dP^T = V . dO^T
                const int s = t % C::Q_STAGES;
                if (!mbar_wait(&do_full[s], (t / C::Q_STAGES) & 1, p.status, kTimeoutMma)) return false;
                tc_fence_after_sync();
                const uint32_t do_addr = smem_u32(do_smem + s * C::TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < C::ROWB / 32; ++kk) {
                    const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
                    mma_ss<false>(tmem_base + C::COL_DP, smem_desc_sw128(v_addr + off, 16, 1024),
                                  smem_desc_sw128(do_addr + off, 16, 1024), idesc_st, kk > 0);
                }
                mma_commit(dp_full);
                return true;
            };
            bool ok = mbar_wait(kv_full, 0, p.status, kTimeoutMma);
            ok = ok && issue_s(0);
            ok = ok && issue_dp(0);
            for (int t = 0; t < n_q && ok; ++t) {
                const int s = t % C::Q_STAGES;
                const bool first = t == 0 || t == nA;           // first tile of a walk: dK, dV start over
                const bool early_next = t + 1 < n_q && t + 1 != nA;   // the next tile belongs to the same walk
                const uint32_t q_addr = smem_u32(q_smem + s * C::TILE_BYTES);
                const uint32_t do_addr = smem_u32(do_smem + s * C::TILE_BYTES);
                if (t == nA) {
                    // second walk: wait for its K and V, then the MMAs a walk begins with.  R0 (and with
                    // head size 64 the dP^T columns) are free: phase B of the previous tile is over.
                    if (!mbar_wait(kv_full, 1, p.status, kTimeoutMma)) { ok = false; break; }
                    if (!issue_s(t)) { ok = false; break; }
                    // the first walk's last dQ must be out of the columns dP^T borrows
                    if (!C::DP_OWN && !mbar_wait(dq_empty, (t - 1) & 1, p.status, kTimeoutMma)) { ok = false; break; }
                    if (!issue_dp(t)) { ok = false; break; }
                }
                if (!mbar_wait(p_full, t & 1, p.status, kTimeoutMma)) { ok = false; break; }
                if (!mbar_wait(&do_full[s], (t / C::Q_STAGES) & 1, p.status, kTimeoutMma)) { ok = false; break; }
                if (t == nA && !mbar_wait(acc_free, 0, p.status, kTimeoutMma)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk)      // dV += P^T . dO      (K = 128 query rows)
                    mma_ts<false>(tmem_base + C::COL_DV, tmem_base + C::COL_S + (kk / 4) * 64 + (kk % 4) * 8,
                                  smem_desc_mn(do_addr + kk * 2048, kBoxBytes, false), idesc_acc, !first || kk > 0);
                // R0 is free as soon as dV, ahead on the pipe, has read P^T
                if (early_next && !issue_s(t + 1)) { ok = false; break; }
                if (!mbar_wait(ds_full, t & 1, p.status, kTimeoutMma)) { ok = false; break; }
                if (t > 0) {
                    // the previous dQ must have left its TMEM columns
                    if (!mbar_wait(dq_empty, (t - 1) & 1, p.status, kTimeoutMma)) { ok = false; break; }
                }
                tc_fence_after_sync();
                // dQ first: its completion starts the read-out, whose first step (tensor memory ->
                // registers) gates the next tile's dP^T when that borrows the dQ columns; dK runs
                // on the pipe meanwhile.  This tile's dO stage was last read by dV and dP^T, which
                // are ahead of dQ on the pipe, so it is free for the read-out's staging at dq_full.
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk)      // dQ_i = dS . K        (K = 128 key rows)
                    mma_ss<false>(tmem_base + C::COL_DQ, smem_desc_mn(ds_addr + kk * 2048, kBoxBytes, false),
                                  smem_desc_mn(k_addr + kk * 2048, kBoxBytes, false), idesc_dq, kk > 0);
                mma_commit(dq_full);
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk) {    // dK += dS^T . Q
                    const uint32_t off = (kk / 4) * kBoxBytes + (kk % 4) * 32;
                    mma_ss<false>(tmem_base + C::COL_DK, smem_desc_sw128(ds_addr + off, 16, 1024),
                                  smem_desc_mn(q_addr + kk * 2048, kBoxBytes, false), idesc_acc, !first || kk > 0);
                }
                mma_commit(&q_empty[s]);  // also: the dS^T tile is no longer read
                if (t == nA - 1 && has_b) {
                    mma_commit(kv_empty);                   // K and V of the first walk are no longer read
                    mma_commit(all_done);                   // and its dK, dV are complete
                }
                // dS^T of tile t is in shared memory, so the softmax warps are done with dP^T(t)
                if (early_next) {
                    // borrowed columns: this tile's dQ, just issued, has to complete and leave them first
                    if (!C::DP_OWN && !mbar_wait(dq_empty, t & 1, p.status, kTimeoutMma)) { ok = false; break; }
                    if (!issue_dp(t + 1)) { ok = false; break; }
                }
            }
            if (ok) mma_commit(all_done);
        }
    } else if (warp < 10) {
        // ---------------- softmax / dS: warps 2..9 ----------------
        // thread = (key row r, half h of the 128 query columns); the two warps that share a
        // TMEM lane group each own 64 columns.
        const int w = warp - 2;
        const int lane_group = warp & 3;
        const int half = w >> 2;
        const int r = lane_group * 32 + lane;                       // key row inside the tile
        const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
        const uint32_t col0 = 64u * half;                           // first query column of this thread
        const float sl2 = p.scale * 1.4426950408889634f;
        const uint64_t sl2_2 = pack_f32x2(sl2, sl2), scale_2 = pack_f32x2(p.scale, p.scale);
        uint8_t* ds_row = ds_smem + half * kBoxBytes + r * 128;     // box `half` holds query columns 64h..64h+63
        const int swz = r & 7;
        bool ok = true;
        // Every thread does its own (bounded) waits; there is no barrier among the softmax warps
        // inside the walk, so a thread that is done with a tile moves on at once.  When a wait
        // gives up, the thread leaves the loop; the others see the status word at their next wait
        // and follow.
        // dK, dV of a finished walk: the first four warps store dV, the other four dK.
        auto store_dkdv = [&](int jt, uint32_t phase) -> bool {
            if (!mbar_wait_warp(all_done, phase, p.status, kTimeoutEpilogue)) return false;
            tc_fence_after_sync();
            const int64_t grow = (int64_t)row_base + (int64_t)jt * kTile + r;
            __nv_bfloat16* out = (__nv_bfloat16*)(half ? p.dK : p.dV) + grow * HS;
            const uint32_t col = half ? C::COL_DK : C::COL_DV;
#pragma unroll 1
            for (int c = 0; c < HS / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + col + lane_addr + c * 32, v);
                tmem_wait_ld();
#pragma unroll
                for (int x = 0; x < 32; x += 8) {
                    uint4 o;
                    o.x = pack_bf16(__uint_as_float(v[x]), __uint_as_float(v[x + 1]));
                    o.y = pack_bf16(__uint_as_float(v[x + 2]), __uint_as_float(v[x + 3]));
                    o.z = pack_bf16(__uint_as_float(v[x + 4]), __uint_as_float(v[x + 5]));
                    o.w = pack_bf16(__uint_as_float(v[x + 6]), __uint_as_float(v[x + 7]));
                    *reinterpret_cast<uint4*>(out + c * 32 + x) = o;
                }
            }
            return true;
        };
        for (int t = 0; t < n_q; ++t) {
            const int i = qtile(t);
            // -lse*log2e and -delta/sqrt(hs) of this query tile, put into the buffer of this tile's
            // parity by the producer
            const float* lse_s = stat_s + (t & 1) * 256;
            const float* delta_s = lse_s + 128;
            if (!mbar_wait_warp(&stat_full[t & 1], (t >> 1) & 1, p.status, kTimeoutSoftmax)) { ok = false; break; }
            if (!mbar_wait_warp(s_full, t & 1, p.status, kTimeoutSoftmax)) { ok = false; break; }
            tc_fence_after_sync();
            const bool diag = p.causal && i == (t < nA ? jtA : jtB);
            // ---- phase A: P^T = exp2(S^T*c - lse) for this thread's 64 columns ----
            uint32_t ph[32];                                        // 64 probabilities as BF16 pairs
            {
                uint32_t s0[32], s1[32];
                tmem_ld32(tmem_base + C::COL_S + lane_addr + col0, s0);
                tmem_ld32(tmem_base + C::COL_S + lane_addr + col0 + 32, s1);
                tmem_wait_ld();
                // The mask test is a compile-time flag of the loop body: a branch per group of
                // columns would end the compiler's scheduling region there and leave the warp
                // running each group's FMA -> exp2 -> convert chain at its latency.
                auto phase_a = [&](auto diag_c) {
                constexpr bool kDiag = decltype(diag_c)::value;
#pragma unroll
                for (int x = 0; x < 32; x += 4) {
                    // four consecutive query columns from each 32-column chunk; their -lse come
                    // as one 16-byte shared-memory load (a broadcast: all threads ask for the same)
                    const int q0 = col0 + x, q1 = col0 + 32 + x;
                    const float4 la = *reinterpret_cast<const float4*>(lse_s + q0);
                    const float4 lb = *reinterpret_cast<const float4*>(lse_s + q1);
                    float a[4], b[4];
                    // s*c - lse for two columns per FMA-pipe instruction
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s0[x]), __uint_as_float(s0[x + 1])), sl2_2, pack_f32x2(la.x, la.y)), a[0], a[1]);
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s0[x + 2]), __uint_as_float(s0[x + 3])), sl2_2, pack_f32x2(la.z, la.w)), a[2], a[3]);
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s1[x]), __uint_as_float(s1[x + 1])), sl2_2, pack_f32x2(lb.x, lb.y)), b[0], b[1]);
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s1[x + 2]), __uint_as_float(s1[x + 3])), sl2_2, pack_f32x2(lb.z, lb.w)), b[2], b[3]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        a[e] = fast_exp2(a[e]);
                        b[e] = fast_exp2(b[e]);
                    }
                    if (kDiag) {                     // query q sees key r only when q >= r
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            a[e] = q0 + e < r ? 0.f : a[e];
                            b[e] = q1 + e < r ? 0.f : b[e];
                        }
                    }
                    ph[x >> 1] = pack_bf16(a[0], a[1]);
                    ph[(x >> 1) + 1] = pack_bf16(a[2], a[3]);
                    ph[16 + (x >> 1)] = pack_bf16(b[0], b[1]);
                    ph[16 + (x >> 1) + 1] = pack_bf16(b[2], b[3]);
                }
                };
                if (diag) phase_a(std::true_type{});
                else      phase_a(std::false_type{});
                // P^T over this thread's own S^T columns: 64 BF16 = 32 columns starting at col0
                tmem_st32(tmem_base + C::COL_S + lane_addr + col0, ph);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(p_full);
            // ---- phase B: dS^T = P^T * (dP^T - delta) / sqrt(hs) ----
            if (!mbar_wait_warp(dp_full, t & 1, p.status, kTimeoutSoftmax)) { ok = false; break; }
            tc_fence_after_sync();
            {
                uint32_t d0[32], d1[32];
                tmem_ld32(tmem_base + C::COL_DP + lane_addr + col0, d0);
                tmem_ld32(tmem_base + C::COL_DP + lane_addr + col0 + 32, d1);
                tmem_wait_ld();
#pragma unroll
                for (int half32 = 0; half32 < 2; ++half32) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {            // one 16-byte unit = 8 query columns
                        const int x = u * 8;                                  // index inside the 32-column chunk
                        const int q = col0 + half32 * 32 + x;
                        const float4 da = *reinterpret_cast<const float4*>(delta_s + q);
                        const float4 db = *reinterpret_cast<const float4*>(delta_s + q + 4);
                        const float nd[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
                        uint32_t o[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t pk = ph[half32 * 16 + (x >> 1) + e];        // two probabilities, BF16
                            const float dp0 = __uint_as_float(half32 ? d1[x + 2 * e] : d0[x + 2 * e]);
                            const float dp1 = __uint_as_float(half32 ? d1[x + 2 * e + 1] : d0[x + 2 * e + 1]);
                            // (dP - delta) / sqrt(hs) for both columns in one FP32 FMA, rounded to BF16 and
                            // multiplied with the BF16 probabilities in one packed BF16 multiply
                            float t0, t1;
                            unpack_f32x2(fma_f32x2(pack_f32x2(dp0, dp1), scale_2, pack_f32x2(nd[2 * e], nd[2 * e + 1])), t0, t1);
                            o[e] = mul_bf16x2(pk, pack_bf16(t0, t1));
                        }
                        const int unit16 = half32 * 4 + u;
                        *reinterpret_cast<uint4*>(ds_row + ((unit16 ^ swz) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
            }
            fence_proxy_async_smem();
            mbar_arrive(ds_full);
            mbar_arrive(&stat_empty[t & 1]);                 // this tile's statistics are no longer read
            if (t == nA - 1 && has_b) {
                // end of the first walk: its dK, dV leave tensor memory before the second walk's first
                // dV and dK MMAs start them over
                if (!store_dkdv(jtA, 0u)) { ok = false; break; }
                tc_fence_before_sync();
                mbar_arrive(acc_free);
            }
        }
        // final: dK, dV of the walk that ended last
        if (ok) store_dkdv(has_b ? jtB : jtA, has_b ? 1u : 0u);
    } else {
        // ---------------- dQ reduction: warps 10..13, thread = query row ----------------
        // The FP32 dQ tile is HS/32 boxes of 128 rows x 128 bytes (16 KB each), twice what the tile's
        // dO stage holds - the stage is idle once the tile's MMAs are complete and serves as the
        // staging area, one box per slot.  The first half of the boxes goes straight through their
        // slots; the second half is taken into registers at once (which frees the tensor-memory
        // columns) and follows box by box, each as soon as the reduction that used its slot has
        // been read out - so the TMA unit always has the next box queued behind the one it is
        // reading.  The dO tile two steps ahead is then loaded slot by slot on the same terms.
        const int lane_group = warp & 3;
        const int r = lane_group * 32 + lane;
        const int tid128 = (warp - 10) * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
        const int swz = r & 7;
        // all but the most recent n reduction groups of this thread have been read out of shared memory
        auto wait_read = [](int n) {
            if (n == 0) tma_wait_group_read0();
            else tma_wait_group_read1();
        };
        for (int t = 0; t < n_q; ++t) {
            const int s = t % C::Q_STAGES;
            if (tid128 == 0) drain_ok[0] = mbar_wait(dq_full, t & 1, p.status, kTimeoutOther) ? 1u : 0u;
            named_barrier_sync(2, 128);
            if (drain_ok[0] == 0u) break;
            tc_fence_after_sync();
            const int y = row_base + qtile(t) * kTile;
            uint8_t* stage = do_smem + s * C::TILE_BYTES;
            auto stage_box = [&](const uint32_t (&v)[32], int slot) {
                uint8_t* row = stage + slot * kBoxBytes + r * 128;
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    *reinterpret_cast<uint4*>(row + ((u ^ swz) << 4)) = make_uint4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
            };
            uint32_t v[C::NBOX][32];
            // boxes 0 .. NBOX-1: tensor memory -> registers -> their slots -> one reduction group each
#pragma unroll
            for (int b = 0; b < C::NBOX; ++b) tmem_ld32(tmem_base + C::COL_DQ + lane_addr + b * 32, v[b]);
            tmem_wait_ld();
#pragma unroll
            for (int b = 0; b < C::NBOX; ++b) stage_box(v[b], b);
            fence_proxy_async_smem();
            named_barrier_sync(2, 128);
            if (tid128 == 0) {
                for (int b = 0; b < C::NBOX; ++b) {
                    tma_reduce_add_2d(&map_dq, stage + b * kBoxBytes, b * 32, y);
                    tma_commit_group();
                }
            }
            // boxes NBOX .. 2*NBOX-1 wait in registers; the TMEM columns are free as soon as they are loaded
#pragma unroll
            for (int b = 0; b < C::NBOX; ++b)
                tmem_ld32(tmem_base + C::COL_DQ + lane_addr + (C::NBOX + b) * 32, v[b]);
            tmem_wait_ld();
            tc_fence_before_sync();
            named_barrier_sync(2, 128);                     // everybody holds the second half
            if (tid128 == 0) mbar_arrive(dq_empty);         // the dQ columns are free
#pragma unroll
            for (int b = 0; b < C::NBOX; ++b) {
                // slot b was last used by the group issued NBOX groups ago
                if (tid128 == 0) wait_read(C::NBOX - 1);
                named_barrier_sync(2, 128);                 // slot b has been read
                stage_box(v[b], b);
                fence_proxy_async_smem();
                named_barrier_sync(2, 128);
                if (tid128 == 0) {
                    tma_reduce_add_2d(&map_dq, stage + b * kBoxBytes, (C::NBOX + b) * 32, y);
                    tma_commit_group();
                }
            }
            if (tid128 == 0 && t + C::Q_STAGES < n_q) {
                mbar_arrive_expect_tx(&do_full[s], C::TILE_BYTES);
                for (int b = 0; b < C::NBOX; ++b) {
                    wait_read(C::NBOX - 1 - b);             // the last group that used slot b has been read
                    tma_load_2d(stage + b * kBoxBytes, &map_do, &do_full[s], b * 64,
                                row_base + qtile(t + C::Q_STAGES) * kTile);
                }
            }
        }
        // The CTA may end once the reductions have read their shared-memory source; that they have
        // landed in global memory by the time the next kernel runs is the grid's completion.
        if (tid128 == 0) tma_wait_group_read0();
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
