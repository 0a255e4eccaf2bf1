// dispatch.cu - the extern "C" contraction and attention-core entry points: argument checks
// and the choice between the tcgen05 kernels and the CUDA-core kernels.  The choice is by
// shape only: a TF32 or BF16 request whose shape the tensor-core kernels do not cover
// (sequence not a multiple of 128, head size other than 64 / 128, tiny or unaligned GEMMs)
// runs on the CUDA cores with the same storage types and FP32 FMA arithmetic - at least as
// accurate as what was asked for, never less.
#include "common.cuh"

using namespace boatcu;

namespace boatcu {
bool attn_tc_supported(int mma, int64_t units, int64_t S, int64_t hs, int io_type);
int attn_fwd_tc(int mma, int64_t units, int64_t S, int64_t hs, int causal, float scale, const void* Q,
                const void* K, const void* V, int io_type, void* O, float* lse);
size_t attn_bwd_tc_scratch_bytes(int mma, int64_t units, int64_t S, int64_t hs);
int attn_bwd_tc(int mma, int64_t units, int64_t S, int64_t hs, int causal, float scale, const void* Q,
                const void* K, const void* V, const void* O, const void* dO, const float* lse, const float* delta,
                int io_type, void* dQ, void* dK, void* dV, void* scratch, size_t scratch_bytes);
}

static int check_types(const char* who, int mma, int in_type) {
    if (mma < BOAT_MMA_FP32 || mma > BOAT_MMA_BF16) return set_error(10, "%s: unknown arithmetic %d", who, mma);
    if (in_type != BOAT_CUDA_F32 && in_type != BOAT_CUDA_BF16 && in_type != BOAT_CUDA_F32_TF32)
        return set_error(10, "%s: unknown storage type %d", who, in_type);
    if (mma == BOAT_MMA_BF16 && in_type != BOAT_CUDA_BF16) return set_error(10, "%s: BF16 arithmetic needs BF16 storage", who);
    if (mma == BOAT_MMA_TF32 && in_type == BOAT_CUDA_BF16) return set_error(10, "%s: TF32 arithmetic needs FP32 storage", who);
    return 0;
}

extern "C" {

int boat_cuda_gemm(int mma, int ta, int tb, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                   const void* B, int64_t ldb, int in_type, void* C, int64_t ldc, int out_type, const float* bias) {
    if (int rc = check_types("boat_cuda_gemm", mma, in_type)) return rc;
    if (in_type == BOAT_CUDA_F32_TF32) in_type = BOAT_CUDA_F32;          // rounded or not, the storage is FP32
    if (out_type < BOAT_CUDA_F32 || out_type > BOAT_CUDA_F32_TF32) return set_error(10, "boat_cuda_gemm: unknown output type %d", out_type);
    if (M < 0 || N < 0 || K < 0) return set_error(11, "boat_cuda_gemm: negative size");
    if (M == 0 || N == 0) return 0;
    if (!A || !B || !C) return set_error(11, "boat_cuda_gemm: NULL operand");
    if (mma != BOAT_MMA_FP32) {
        if (gemm_tc_supported(mma, ta, tb, M, N, K, A, lda, B, ldb, in_type, C, ldc, out_type))
            return gemm_tc(mma, ta, tb, M, N, K, A, lda, B, ldb, in_type, C, ldc, out_type, bias);
        // Small or unaligned problems: same storage types, FP32 FMA arithmetic (more
        // accurate than the requested tensor-core format, never less).
    }
    ProfileScope prof("gemm_simt");
    return gemm_simt(ta, tb, M, N, K, A, lda, B, ldb, in_type, C, ldc, out_type, bias);
}

int boat_cuda_gemm_set_yielding(int on) {
    gemm_tc_set_yielding(on != 0);
    return 0;
}

int boat_cuda_gemm_grouped(int mma, int ta, int tb, int groups, int64_t M, int64_t N, int64_t K, const void* const* A,
                           int64_t lda, const void* const* B, int64_t ldb, int in_type, void* const* C, int64_t ldc,
                           int out_type, const float* const* bias) {
    if (groups < 1 || groups > 4) return set_error(11, "boat_cuda_gemm_grouped: %d groups (1 to 4)", groups);
    if (!A || !B || !C) return set_error(11, "boat_cuda_gemm_grouped: NULL operand table");
    if (int rc = check_types("boat_cuda_gemm_grouped", mma, in_type)) return rc;
    const int store = in_type == BOAT_CUDA_F32_TF32 ? BOAT_CUDA_F32 : in_type;
    bool one_launch = mma != BOAT_MMA_FP32 && out_type >= BOAT_CUDA_F32 && out_type <= BOAT_CUDA_F32_TF32 && M > 0 && N > 0 && K >= 0;
    for (int g = 0; g < groups && one_launch; ++g)
        one_launch = A[g] && B[g] && C[g] && gemm_tc_supported(mma, ta, tb, M, N, K, A[g], lda, B[g], ldb, store, C[g], ldc, out_type);
    if (one_launch) return gemm_tc_grouped(mma, ta, tb, groups, M, N, K, A, lda, B, ldb, C, ldc, out_type, bias);
    // shapes the tensor-core kernel does not cover (or bad arguments, reported by the single call)
    for (int g = 0; g < groups; ++g)
        if (int rc = boat_cuda_gemm(mma, ta, tb, M, N, K, A[g], lda, B[g], ldb, in_type, C[g], ldc, out_type, bias ? bias[g] : nullptr))
            return rc;
    return 0;
}

int boat_cuda_attn_fwd(int mma, int64_t units, int64_t S, int64_t hs, int causal, float scale, const void* Q,
                       const void* K, const void* V, int io_type, void* O, float* lse) {
    if (int rc = check_types("boat_cuda_attn_fwd", mma, io_type)) return rc;
    if (io_type == BOAT_CUDA_F32_TF32) io_type = BOAT_CUDA_F32;
    if (units < 0 || S < 0 || hs < 0) return set_error(11, "boat_cuda_attn_fwd: negative size");
    if (units == 0 || S == 0 || hs == 0) return 0;
    if (!Q || !K || !V || !O || !lse) return set_error(11, "boat_cuda_attn_fwd: NULL operand");
    if (mma != BOAT_MMA_FP32 && attn_tc_supported(mma, units, S, hs, io_type))
        return attn_fwd_tc(mma, units, S, hs, causal, scale, Q, K, V, io_type, O, lse);
    {
        ProfileScope prof("attn_fwd_simt");
        if (int rc = attn_fwd_simt(units, S, hs, causal, scale, Q, K, V, io_type, O, lse)) return rc;
    }
    // TF32 contract: O is TF32-valued whichever kernel produced it
    if (mma == BOAT_MMA_TF32) return boat_cuda_round_tf32((float*)O, (const float*)O, units * S * hs);
    return 0;
}

size_t boat_cuda_attn_bwd_scratch_bytes(int mma, int64_t units, int64_t S, int64_t hs) {
    size_t delta = (size_t)units * (size_t)S * sizeof(float);
    delta = (delta + 255) & ~(size_t)255;
    size_t extra = 0;
    if (mma != BOAT_MMA_FP32 && attn_tc_supported(mma, units, S, hs, mma == BOAT_MMA_BF16 ? BOAT_CUDA_BF16 : BOAT_CUDA_F32))
        extra = attn_bwd_tc_scratch_bytes(mma, units, S, hs);
    return delta + extra;
}

int boat_cuda_attn_bwd(int mma, int64_t units, int64_t S, int64_t hs, int causal, float scale, const void* Q,
                       const void* K, const void* V, const void* O, const void* dO, const float* lse,
                       int io_type, void* dQ, void* dK, void* dV, void* scratch, size_t scratch_bytes) {
    if (int rc = check_types("boat_cuda_attn_bwd", mma, io_type)) return rc;
    if (io_type == BOAT_CUDA_F32_TF32) io_type = BOAT_CUDA_F32;
    if (units < 0 || S < 0 || hs < 0) return set_error(11, "boat_cuda_attn_bwd: negative size");
    if (units == 0 || S == 0 || hs == 0) return 0;
    if (!Q || !K || !V || !O || !dO || !lse || !dQ || !dK || !dV) return set_error(11, "boat_cuda_attn_bwd: NULL operand");
    size_t need = boat_cuda_attn_bwd_scratch_bytes(mma, units, S, hs);
    if (!scratch || scratch_bytes < need)
        return set_error(12, "boat_cuda_attn_bwd: scratch of %zu bytes given, %zu needed", scratch_bytes, need);
    if (((uintptr_t)scratch & 255) != 0) return set_error(12, "boat_cuda_attn_bwd: scratch must be 256-byte aligned");
    float* delta = (float*)scratch;
    size_t delta_bytes = ((size_t)units * (size_t)S * sizeof(float) + 255) & ~(size_t)255;
    const bool tensor_cores = mma != BOAT_MMA_FP32 && attn_tc_supported(mma, units, S, hs, io_type);
    if (!(tensor_cores && mma == BOAT_MMA_BF16)) {      // the BF16 kernel's launcher makes its own, pre-scaled
        ProfileScope prof("attn_delta");
        if (int rc = rowdot(dO, O, io_type, units * S, hs, delta)) return rc;
    }
    if (tensor_cores)
        return attn_bwd_tc(mma, units, S, hs, causal, scale, Q, K, V, O, dO, lse, delta, io_type, dQ, dK, dV,
                           (char*)scratch + delta_bytes, scratch_bytes - delta_bytes);
    {
        ProfileScope prof("attn_bwd_simt");
        if (int rc = attn_bwd_simt(units, S, hs, causal, scale, Q, K, V, dO, lse, delta, io_type, dQ, dK, dV)) return rc;
    }
    if (mma == BOAT_MMA_TF32) {
        const int64_t n = units * S * hs;
        if (int rc = boat_cuda_round_tf32((float*)dQ, (const float*)dQ, n)) return rc;
        if (int rc = boat_cuda_round_tf32((float*)dK, (const float*)dK, n)) return rc;
        return boat_cuda_round_tf32((float*)dV, (const float*)dV, n);
    }
    return 0;
}

}  // extern "C"
