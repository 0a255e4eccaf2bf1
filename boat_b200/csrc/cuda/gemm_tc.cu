// gemm_tc.cu - the projection GEMMs of the attention layer on Blackwell tensor cores.
//
//   C[M,N] = op(A) . op(B) (+ bias)      BF16 storage (kind::f16) or FP32 storage (kind::tf32),
//                                         FP32 accumulation in tensor memory
//
// Replaces boat_matmul (reference src/ops/linear.c:116-130) inside linear_projection
// (src/layers/attention.c:247-308) and linear_projection_backward (attention.c:1186-1293).
// The three products of a projection differ only in which operand is stored transposed;
// instead of materialising transposes as the reference does (linear.c:306-334), the shared
// memory descriptors tell the tensor core which way each operand lies:
//
//   Y  = X . W      A = X  [M,K] K-major      B = W  [K,N] N-major
//   dX = dY . W^T   A = dY [M,K] K-major      B = W  [N,K] K-major
//   dW = X^T . dY   A = X  [K,M] M-major      B = dY [K,N] N-major
//
// Kernel shape: persistent, one 192-thread CTA per SM.  Warp 0 feeds a 4-stage shared-memory
// ring with TMA (128-byte swizzle, no multicast); one thread of warp 1 issues tcgen05.mma
// 128 x BN x (32 bytes of K) and commits stages back to the producer; warps 2-5 drain the
// accumulator from tensor memory (tcgen05.ld), add the bias, convert and store.  The
// accumulator is double-buffered in tensor memory (2 x BN columns) so that the epilogue of one
// tile overlaps the main loop of the next.  Weight gradients have few output tiles and a
// very long K: they are split along K over several CTAs that add into a zeroed output.
//
// Up to kMaxGroups problems of one shape and layout (the Q, K and V projections of a layer, their
// weight gradients, their input gradients) run as one launch: the persistent CTAs walk the tiles of
// all groups, group index fastest, so CTAs at work at the same time read the operand the groups
// share (X for self-attention) from L2.
#include "tc_common.cuh"

namespace boatcu {

using namespace tc;

namespace {

constexpr int BM = 128;
constexpr int STAGES = 4;
constexpr int kThreads = 192;

template <typename T, int BN>
struct Cfg {
    static constexpr int ES = sizeof(T);
    static constexpr int BK = 128 / ES;             // one 128-byte swizzle row of K (or of M/N)
    static constexpr int UK = 32 / ES;              // K extent of one tcgen05.mma
    static constexpr int A_BYTES = BM * 128;
    static constexpr int B_BYTES = BN * 128;
    static constexpr int CHUNK_BYTES = BK * 128;    // one [BK rows x 128 B] box of an MN-major operand
    static constexpr int SMEM = STAGES * (A_BYTES + B_BYTES) + 1024 /*alignment*/ + 256 /*barriers*/;
    static constexpr uint32_t TMEM_COLS = 2 * BN;   // two accumulators
};

constexpr int kMaxGroups = 4;

struct GroupMaps {
    CUtensorMap a[kMaxGroups], b[kMaxGroups];
};

struct Params {
    void* C[kMaxGroups];
    const float* bias[kMaxGroups];
    int groups;
    int64_t ldc;
    int M, N, K;
    int out_type;
    int split_k;
    unsigned int* status;
};

template <typename T, bool A_MN, bool B_MN, int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ GroupMaps maps, const __grid_constant__ Params p) {
    using C = Cfg<T, BN>;
    constexpr bool TF32 = sizeof(T) == 4;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* a_smem = smem;
    uint8_t* b_smem = smem + STAGES * C::A_BYTES;
    uint64_t* bars = (uint64_t*)(smem + STAGES * (C::A_BYTES + C::B_BYTES));
    uint64_t* full = bars;                 // [STAGES] TMA -> MMA
    uint64_t* empty = bars + STAGES;       // [STAGES] MMA -> TMA
    uint64_t* acc_full = bars + 2 * STAGES;       // [2] MMA -> epilogue
    uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2] epilogue -> MMA
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
    const int k_blocks = (p.K + C::BK - 1) / C::BK;
    const int work_items = m_tiles * n_tiles * p.groups * p.split_k;      // w = ((tile * groups) + g) * split_k + split

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 128);
        }
        fence_barrier_init();
        for (int g = 0; g < p.groups; ++g) {
            tma_prefetch_desc(&maps.a[g]);
            tma_prefetch_desc(&maps.b[g]);
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
            uint32_t it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < work_items && ok; w += gridDim.x) {
                const int split = w % p.split_k, gt = w / p.split_k;
                const int g = gt % p.groups, tile = gt / p.groups;
                const CUtensorMap* map_a = &maps.a[g];
                const CUtensorMap* map_b = &maps.b[g];
                const int m0 = (tile / n_tiles) * BM, n0 = (tile % n_tiles) * BN;
                const int kb0 = (int)((int64_t)split * k_blocks / p.split_k);
                const int kb1 = (int)((int64_t)(split + 1) * k_blocks / p.split_k);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, p.status, kTimeoutProducer)) { ok = false; break; }
                    mbar_arrive_expect_tx(&full[s], C::A_BYTES + C::B_BYTES);
                    const int k0 = kb * C::BK;
                    uint8_t* a_dst = a_smem + s * C::A_BYTES;
                    uint8_t* b_dst = b_smem + s * C::B_BYTES;
                    if (A_MN) {
                        for (int c = 0; c < BM / C::BK; ++c)
                            tma_load_2d(a_dst + c * C::CHUNK_BYTES, map_a, &full[s], m0 + c * C::BK, k0);
                    } else {
                        tma_load_2d(a_dst, map_a, &full[s], k0, m0);
                    }
                    if (B_MN) {
                        for (int c = 0; c < BN / C::BK; ++c)
                            tma_load_2d(b_dst + c * C::CHUNK_BYTES, map_b, &full[s], n0 + c * C::BK, k0);
                    } else {
                        tma_load_2d(b_dst, map_b, &full[s], k0, n0);
                    }
                }
            }
            if (!ok) {
                // give loads already in flight time to land before the CTA's memory goes away
                for (int i = 0; i < 1000; ++i) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(TF32 ? kTF32 : kBF16, A_MN, B_MN, BM, BN);
            uint32_t it = 0, acc_it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < work_items && ok; w += gridDim.x, ++acc_it) {
                const int split = w % p.split_k;
                const int kb0 = (int)((int64_t)split * k_blocks / p.split_k);
                const int kb1 = (int)((int64_t)(split + 1) * k_blocks / p.split_k);
                const int buf = acc_it & 1;
                if (!mbar_wait(&acc_empty[buf], ((acc_it >> 1) & 1) ^ 1, p.status, kTimeoutMma)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full[s], (it / STAGES) & 1, p.status, kTimeoutMma)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(a_smem + s * C::A_BYTES);
                    const uint32_t b_addr = smem_u32(b_smem + s * C::B_BYTES);
#pragma unroll
                    for (int kk = 0; kk < C::BK / C::UK; ++kk) {
                        const uint64_t a_desc = A_MN ? smem_desc_mn(a_addr + kk * C::UK * 128, C::CHUNK_BYTES, TF32)
                                                     : smem_desc_sw128(a_addr + kk * 32, 16, 1024);
                        const uint64_t b_desc = B_MN ? smem_desc_mn(b_addr + kk * C::UK * 128, C::CHUNK_BYTES, TF32)
                                                     : smem_desc_sw128(b_addr + kk * 32, 16, 1024);
                        mma_ss<TF32>(d_tmem, a_desc, b_desc, idesc, kb > kb0 || kk > 0);
                    }
                    mma_commit(&empty[s]);            // stage reusable once these MMAs have read it
                }
                if (ok) mma_commit(&acc_full[buf]);   // accumulator complete
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 ----------------
        const int lane_group = warp & 3;              // TMEM lanes this warp may touch
        uint32_t acc_it = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < work_items && ok; w += gridDim.x, ++acc_it) {
            const int split = w % p.split_k, gt = w / p.split_k;
            const int g = gt % p.groups, tile = gt / p.groups;
            const int m0 = (tile / n_tiles) * BM, n0 = (tile % n_tiles) * BN;
            void* const out = p.C[g];
            const float* const bias = p.bias[g];
            const int buf = acc_it & 1;
            if (!mbar_wait(&acc_full[buf], (acc_it >> 1) & 1, p.status, kTimeoutEpilogue)) { ok = false; break; }
            tc_fence_after_sync();
            const int row = m0 + lane_group * 32 + lane;
            const uint32_t t_addr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + buf * BN;
            const bool add_bias = bias != nullptr && split == 0;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(t_addr + c * 32, r);
                tmem_wait_ld();
                const int col0 = n0 + c * 32;
                if (row < p.M && col0 < p.N) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (add_bias) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < p.N) v[j] += __ldg(bias + col0 + j);
                    }
                    if (p.split_k > 1) {
                        float* dst = (float*)out + (int64_t)row * p.ldc + col0;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < p.N) atomicAdd(dst + j, v[j]);
                    } else if (p.out_type != BOAT_CUDA_BF16) {
                        if (p.out_type == BOAT_CUDA_F32_TF32) {        // feeds another TF32 contraction
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = round_to_tf32(v[j]);
                        }
                        float* dst = (float*)out + (int64_t)row * p.ldc + col0;
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            if (col0 + j < p.N)       // N is a multiple of 4 on this path
                                *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
                        __nv_bfloat16* dst = (__nv_bfloat16*)out + (int64_t)row * p.ldc + col0;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            if (col0 + j < p.N) {     // N is a multiple of 8 on this path
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]);
                                __nv_bfloat162 h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
                                __nv_bfloat162 h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                uint4 o;
                                o.x = *reinterpret_cast<uint32_t*>(&h0);
                                o.y = *reinterpret_cast<uint32_t*>(&h1);
                                o.z = *reinterpret_cast<uint32_t*>(&h2);
                                o.w = *reinterpret_cast<uint32_t*>(&h3);
                                *reinterpret_cast<uint4*>(dst + j) = o;
                            }
                        }
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

bool g_yielding = false;

template <typename T, bool A_MN, bool B_MN, int BN>
int launch(int groups, int64_t M, int64_t N, int64_t K, const void* const* A, int64_t lda, const void* const* B,
           int64_t ldb, void* const* Cp, int64_t ldc, int out_type, const float* const* bias, int split_k) {
    using C = Cfg<T, BN>;
    GroupMaps maps;
    Params p;
    for (int g = 0; g < kMaxGroups; ++g) {
        const int s = g < groups ? g : 0;       // unused slots repeat group 0: valid descriptors, never walked
        // A: K-major -> matrix [M rows, K cols], box [BM, BK].  M-major -> stored [K rows, M cols], box [BK, BK].
        if (int rc = A_MN ? make_tensor_map_2d(&maps.a[g], A[s], C::ES, (uint64_t)K, (uint64_t)M, (uint64_t)lda, C::BK, C::BK, C::ES == 4)
                          : make_tensor_map_2d(&maps.a[g], A[s], C::ES, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, C::BK))
            return rc;
        if (int rc = B_MN ? make_tensor_map_2d(&maps.b[g], B[s], C::ES, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, C::BK, C::BK, C::ES == 4)
                          : make_tensor_map_2d(&maps.b[g], B[s], C::ES, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, BN, C::BK))
            return rc;
        p.C[g] = Cp[s];
        p.bias[g] = bias ? bias[s] : nullptr;
    }
    const int tiles = (int)(ceil_div(M, BM) * ceil_div(N, BN)) * groups;
    if (split_k > 1) {
        for (int g = 0; g < groups; ++g) {
            if (ldc == N) {
                BOATCU_CHECK(cudaMemsetAsync(Cp[g], 0, (size_t)M * N * sizeof(float), stream()));
            } else {
                BOATCU_CHECK(cudaMemset2DAsync(Cp[g], (size_t)ldc * sizeof(float), 0, (size_t)N * sizeof(float), (size_t)M, stream()));
            }
        }
    }
    p.groups = groups;
    p.ldc = ldc;
    p.M = (int)M;
    p.N = (int)N;
    p.K = (int)K;
    p.out_type = out_type;
    p.split_k = split_k;
    p.status = kernel_status_ptr();
    auto kern = gemm_tc_kernel<T, A_MN, B_MN, BN>;
    static bool configured = false;     // per process = per device: the library binds to one device
    if (!configured) {
        BOATCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured = true;
    }
    const int work = tiles * split_k;
    // Persistent by default: one CTA per SM walks the tiles.  A yielding launch has one CTA per tile
    // instead, so that SMs come free all along and the CTAs of a collective started beside it (whose
    // stream has priority) get placed while the GEMM runs, not after it.
    const int grid = (g_yielding || work < sm_count()) ? work : sm_count();
    ProfileScope prof(A_MN ? "gemm_tc_tn" : (B_MN ? "gemm_tc_nn" : "gemm_tc_nt"));
    kern<<<grid, kThreads, C::SMEM, stream()>>>(maps, p);
    BOATCU_LAUNCH_OK("gemm_tc");
    return 0;
}

template <typename T, int BN>
int dispatch_layout_bn(int ta, int tb, int groups, int64_t M, int64_t N, int64_t K, const void* const* A, int64_t lda,
                       const void* const* B, int64_t ldb, void* const* C, int64_t ldc, int out_type,
                       const float* const* bias, int split_k) {
    // trans_a: A stored [K,M] (M-major).  trans_b == 0: B stored [K,N] (N-major).
    if (!ta && !tb) return launch<T, false, true, BN>(groups, M, N, K, A, lda, B, ldb, C, ldc, out_type, bias, split_k);
    if (!ta && tb) return launch<T, false, false, BN>(groups, M, N, K, A, lda, B, ldb, C, ldc, out_type, bias, split_k);
    if (ta && !tb) return launch<T, true, true, BN>(groups, M, N, K, A, lda, B, ldb, C, ldc, out_type, bias, split_k);
    return launch<T, true, false, BN>(groups, M, N, K, A, lda, B, ldb, C, ldc, out_type, bias, split_k);
}

template <typename T>
int dispatch_layout(int ta, int tb, int groups, int64_t M, int64_t N, int64_t K, const void* const* A, int64_t lda,
                    const void* const* B, int64_t ldb, void* const* C, int64_t ldc, int out_type,
                    const float* const* bias) {
    const int64_t sms = sm_count();
    const int64_t tiles = ceil_div(M, BM) * ceil_div(N, 256) * groups;
    const int64_t k_blocks = ceil_div(K, (int64_t)(128 / sizeof(T)));
    // Few output tiles and a long K (weight gradients): spread K over the idle SMs, at least 8
    // K-blocks per piece; the pieces add into a zeroed FP32 output.
    int64_t split_k = 1;
    if (out_type == BOAT_CUDA_F32 && tiles * 2 <= sms) {
        split_k = sms / tiles;
        if (split_k > k_blocks / 8) split_k = k_blocks / 8;
        if (split_k < 1) split_k = 1;
    }
    // 128 x 256 tiles by default.  A problem with fewer such tiles than SMs (and no long K to split
    // instead) gets 128 x 128 tiles when those still fit in one wave: twice the CTAs at work, half
    // the main loop per CTA.  (More narrow tiles than SMs would only add a second, partly empty wave.)
    const int64_t narrow_tiles = ceil_div(M, BM) * ceil_div(N, 128) * groups;
    if (tiles < sms && narrow_tiles <= sms && split_k == 1 && N > 128)
        return dispatch_layout_bn<T, 128>(ta, tb, groups, M, N, K, A, lda, B, ldb, C, ldc, out_type, bias, 1);
    return dispatch_layout_bn<T, 256>(ta, tb, groups, M, N, K, A, lda, B, ldb, C, ldc, out_type, bias, (int)split_k);
}

}  // namespace

bool gemm_tc_supported(int mma, int ta, int tb, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                       const void* B, int64_t ldb, int in_type, const void* C, int64_t ldc, int out_type) {
    (void)ta;
    (void)tb;
    if (mma != BOAT_MMA_BF16 && mma != BOAT_MMA_TF32) return false;
    const int es = mma == BOAT_MMA_BF16 ? 2 : 4;
    if ((mma == BOAT_MMA_BF16) != (in_type == BOAT_CUDA_BF16)) return false;
    const int oes = out_type == BOAT_CUDA_BF16 ? 2 : 4;
    if (M < 128 || N < 64 || K < 128 / es) return false;               // small problems: CUDA cores
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return false;
    if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) return false;
    if ((lda * es) % 16 || (ldb * es) % 16 || (ldc * oes) % 16) return false;
    if (N % (16 / oes)) return false;
    return true;
}

int gemm_tc_grouped(int mma, int ta, int tb, int groups, int64_t M, int64_t N, int64_t K, const void* const* A,
                    int64_t lda, const void* const* B, int64_t ldb, void* const* C, int64_t ldc, int out_type,
                    const float* const* bias) {
    if (groups < 1 || groups > kMaxGroups) return set_error(11, "gemm_tc_grouped: %d groups (1..%d)", groups, kMaxGroups);
    if (int rc = ensure_init()) return rc;
    if (mma == BOAT_MMA_BF16)
        return dispatch_layout<__nv_bfloat16>(ta, tb, groups, M, N, K, A, lda, B, ldb, C, ldc, out_type, bias);
    return dispatch_layout<float>(ta, tb, groups, M, N, K, A, lda, B, ldb, C, ldc, out_type, bias);
}

void gemm_tc_set_yielding(bool on) { g_yielding = on; }

int gemm_tc(int mma, int ta, int tb, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda, const void* B,
            int64_t ldb, int in_type, void* C, int64_t ldc, int out_type, const float* bias) {
    (void)in_type;
    return gemm_tc_grouped(mma, ta, tb, 1, M, N, K, &A, lda, &B, ldb, &C, ldc, out_type, &bias);
}

}  // namespace boatcu
