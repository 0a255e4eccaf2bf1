/* boat_cuda.h - the extern "C" surface between the C host layer and the sm_100a kernels.
 *
 * Plain pointers and sizes only; every function returns 0 on success and a non-zero
 * status otherwise (boat_cuda_last_error() has the text), never exits, and launches on the
 * library stream (boat_cuda_stream()).  All pointers are DEVICE pointers unless a
 * parameter says "host".
 *
 * Each entry names the piece of the reference it stands in for; paths are relative to the
 * reference tree (xiaoshaoning/boat).
 */
#ifndef BOAT_CUDA_H
#define BOAT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#pragma GCC visibility push(default)

/* Storage type of a device buffer.  BOAT_CUDA_F32_TF32 is FP32 storage whose values have been
 * rounded to the nearest TF32 number (10 mantissa bits): accepted as the OUTPUT type of
 * boat_cuda_gemm for results that feed another TF32 contraction - the tensor core truncates
 * FP32 operands, so rounding in the producing epilogue keeps the pipeline unbiased without a
 * separate rounding pass.  As an input type it is the same as BOAT_CUDA_F32. */
enum { BOAT_CUDA_F32 = 0, BOAT_CUDA_BF16 = 1, BOAT_CUDA_F32_TF32 = 2 };

/* Arithmetic used by the contraction kernels.
 *   FP32: CUDA-core FMA, any shape (the exact path; reference numerics are IEEE FP32).
 *   TF32: tcgen05 kind::tf32 on FP32 storage, FP32 accumulate in tensor memory.
 *   BF16: tcgen05 kind::f16 on BF16 storage, FP32 accumulate in tensor memory. */
enum { BOAT_MMA_FP32 = 0, BOAT_MMA_TF32 = 1, BOAT_MMA_BF16 = 2 };

/* ---- runtime: replaces the host-only device stubs of src/core/memory.c:174-186,
 *      :230-247 (allocate / copy / set "on device" were malloc/memcpy/memset) ---------- */
int         boat_cuda_init(int device);          /* idempotent; device < 0: env BOAT_CUDA_DEVICE or LOCAL_RANK or 0 */
int         boat_cuda_device_count(void);        /* 0 when no usable GPU / driver */
const char* boat_cuda_last_error(void);
void*       boat_cuda_stream(void);              /* cudaStream_t the library launches on */
int         boat_cuda_set_stream(void* stream);
int         boat_cuda_sync(void);                /* wait for the library stream and the copy streams */
int         boat_cuda_malloc(void** ptr, size_t bytes);   /* stream-ordered pool allocation */
int         boat_cuda_free(void* ptr);
int         boat_cuda_memcpy_h2d(void* dst, const void* src_host, size_t bytes);  /* returns after arrival */
int         boat_cuda_memcpy_d2h(void* dst_host, const void* src, size_t bytes);  /* returns after arrival */
int         boat_cuda_memcpy_d2d(void* dst, const void* src, size_t bytes);       /* asynchronous on the stream */
/* Copies on their own streams, one per direction, so that PCIe traffic overlaps kernels.
 * copies_after_compute: both copy streams wait for what has been launched (and allocated) on
 * the library stream so far - call it after allocating the buffers the copies will touch.
 * upload_async: host -> device on the upload stream, in issue order, overlapping later launches.
 * join_uploads: every later launch on the library stream waits for the uploads issued so far.
 * download_async: device -> host on the download stream, after the kernels launched before it.
 * boat_cuda_sync() also waits for these copies - call it before the host reads a download and
 * before freeing a buffer a copy may still touch.  Page-locked host memory
 * (boat_cuda_host_alloc / _register) is needed for real overlap. */
int         boat_cuda_copies_after_compute(void);
int         boat_cuda_upload_async(void* dst, const void* src_host, size_t bytes);
int         boat_cuda_join_uploads(void);
int         boat_cuda_download_async(void* dst_host, const void* src, size_t bytes);
int         boat_cuda_memset(void* dst, int value, size_t bytes);
void*       boat_cuda_host_alloc(size_t bytes);          /* page-locked host block from a re-use pool; NULL on failure */
int         boat_cuda_host_free(void* ptr);              /* back to the pool (never unlocked until exit) */
int         boat_cuda_host_register(void* host, size_t bytes);   /* pin a caller buffer for fast copies */
int         boat_cuda_host_unregister(void* host);
size_t      boat_cuda_bytes_in_use(void);        /* bytes handed out by boat_cuda_malloc and not yet freed */
uint64_t    boat_cuda_launch_count(void);        /* kernels of this library launched so far */
/* Per-kernel timing for benchmarks: while enabled, every kernel family is bracketed by CUDA
 * events on the library stream; report() synchronises and writes "<name> <scopes> <ms>" lines. */
int         boat_cuda_profile_enable(int on);
int         boat_cuda_profile_report(char* out, size_t out_bytes);

/* Self-test of the kernels' bounded waits (no counterpart in the reference).  Launches a
 * one-block kernel that waits, for at most limit_ns (<= 1 s), on a barrier nobody completes:
 * the wait gives up, records role code 9 in the kernel status word and the kernel returns
 * normally.  The next boat_cuda_sync() / boat_cuda_memcpy_d2h() then fails with status 30 and
 * clears the word; the call after that succeeds again.  Nothing hangs and nothing faults. */
int         boat_cuda_selftest_wait_timeout(uint64_t limit_ns);

/* ---- contraction: replaces boat_matmul (src/ops/linear.c:12-170) as used by
 *      linear_projection (src/layers/attention.c:247-308) and
 *      linear_projection_backward (attention.c:1186-1293), including the materialised
 *      boat_transpose calls (linear.c:238-406) that those make --------------------------
 * C[M,N] = op(A) . op(B) (+ bias[N] broadcast over rows), row-major, leading dimensions in
 * elements.  trans_a: A is stored [K,M];  trans_b: B is stored [N,K].
 *   forward projection   Y  = X . W + b      trans_a=0 trans_b=0
 *   input gradient       dX = dY . W^T       trans_a=0 trans_b=1
 *   weight gradient      dW = X^T . dY       trans_a=1 trans_b=0
 * in_type is the storage type of A and B (F32 for mma FP32/TF32, BF16 for mma BF16);
 * out_type the storage type of C; bias is FP32 or NULL. */
int boat_cuda_gemm(int mma, int trans_a, int trans_b, int64_t M, int64_t N, int64_t K,
                   const void* A, int64_t lda, const void* B, int64_t ldb, int in_type,
                   void* C, int64_t ldc, int out_type, const float* bias);

/* While on, tensor-core GEMM launches use one CTA per output tile instead of one persistent CTA per
 * SM: SMs come free all along the launch, so a collective started beside it on another stream gets
 * placed while the GEMM runs.  The attention backward switches it on around the input-gradient GEMMs
 * when it has just started a gradient sum (overlap mode 1). */
int boat_cuda_gemm_set_yielding(int on);

/* `groups` (1 to 4) contractions of one shape, layout and type as one launch: the Q, K and V
 * projections of a layer (attention.c:363-365 makes three linear_projection calls), their three
 * weight gradients, their three input gradients.  A, B, C are tables of `groups` pointers (entries
 * may repeat: self-attention passes the same X three times); bias is NULL or a table whose
 * entries may be NULL.  Results equal `groups` calls of boat_cuda_gemm, to which shapes outside
 * the tensor-core kernel fall back one by one. */
int boat_cuda_gemm_grouped(int mma, int trans_a, int trans_b, int groups, int64_t M, int64_t N, int64_t K,
                           const void* const* A, int64_t lda, const void* const* B, int64_t ldb, int in_type,
                           void* const* C, int64_t ldc, int out_type, const float* const* bias);

/* ---- attention core: replaces scaled_dot_product_attention_impl
 *      (src/layers/attention.c:882-1079) ------------------------------------------------
 * Q,K,V,O are [units, S, hs] contiguous: unit u = (b*nh + h) is the block at element
 * u*S*hs - the reference's reshape-only head split (attention.c:393-397).
 * O = softmax(scale * Q K^T, causal: j>i masked) V.  The S x S probabilities are never
 * stored; lse[units*S] (FP32) receives max + log(sum exp) of the scaled scores per row,
 * which is all the backward needs.  With mma = BOAT_MMA_TF32 the values of O are rounded to
 * TF32 (they feed the TF32 output projection); likewise dQ, dK, dV of the backward. */
int boat_cuda_attn_fwd(int mma, int64_t units, int64_t S, int64_t hs, int causal, float scale,
                       const void* Q, const void* K, const void* V, int io_type,
                       void* O, float* lse);

/* ---- attention core backward: replaces attention_backward
 *      (src/layers/attention.c:1388-1534) -----------------------------------------------
 * Recomputes P = exp(scale*QK^T - lse) tile by tile and produces
 *   dV = P^T dO, dP = dO V^T, dS = P * (dP - delta) * scale, dQ = dS K, dK = dS^T Q
 * with delta_i = sum_d dO[i,d]*O[i,d] (equal to the reference's sum_j dP_ij P_ij,
 * attention.c:1472-1488).  `scratch` is device memory the kernels may use freely:
 * boat_cuda_attn_bwd_scratch_bytes() gives the size needed for a problem. */
size_t boat_cuda_attn_bwd_scratch_bytes(int mma, int64_t units, int64_t S, int64_t hs);
int boat_cuda_attn_bwd(int mma, int64_t units, int64_t S, int64_t hs, int causal, float scale,
                       const void* Q, const void* K, const void* V, const void* O,
                       const void* dO, const float* lse, int io_type,
                       void* dQ, void* dK, void* dV, void* scratch, size_t scratch_bytes);

/* ---- attention core backward without caller scratch (no counterpart in the reference) -----
 * Same computation and arguments as boat_cuda_attn_bwd, for callers that cannot provide
 * scratch because they may not allocate device memory where they call from: serving loops
 * that ban cudaMalloc (it can stall every stream of the device), programs with a device
 * memory budget fixed at start-up, plugins inside a host framework that owns all HBM.
 * The scratch is a fixed 16 MiB block inside the library image (capacity() returns the
 * size); each GPU that loads the library holds it until the process exits.  Problems whose
 * boat_cuda_attn_bwd_scratch_bytes() exceeds it are refused with a clear error.
 * The call makes no cudaMalloc/cudaFree and no allocating library call - with one exception:
 * while boat_cuda_profile_enable(1) is in force, the timing scopes create CUDA events, so
 * keep profiling off where allocation is banned.  It never
 * initialises the library: call boat_cuda_init() once beforehand (that does allocate).
 * The first call on a device looks up the block's device address; make that first call
 * outside any stream capture.  All calls share the one block and it keeps the previous
 * call's contents - the kernels clear what they sum into - so two calls whose GPU work
 * overlaps (different streams, different threads) race on it: keep them on one stream. */
size_t boat_cuda_attn_bwd_static_capacity(void);
int boat_cuda_attn_bwd_static(int mma, int64_t units, int64_t S, int64_t hs, int causal, float scale,
                              const void* Q, const void* K, const void* V, const void* O,
                              const void* dO, const float* lse, int io_type,
                              void* dQ, void* dK, void* dV);

/* ---- element-wise / reduction tail ----------------------------------------------------
 * colsum:  out[j] = sum_i X[i,j]     bias gradient loop, attention.c:1271-1284
 * axpy:    y += alpha * x            boat_add_ (arithmetic.c:362-391) with alpha = 1 for
 *                                    gradient accumulation (autodiff.c:2495-2525);
 *                                    alpha = -lr for the SGD step, i.e. boat_mul_scalar +
 *                                    boat_sub_ (attention.c:745-812)
 * scale:   y = alpha * x             boat_mul_scalar (arithmetic.c:425-484)
 * add_bias: y[i,j] = x[i,j] + b[j]   boat_add bias broadcast (arithmetic.c:199-203)
 * mul:     y = a * b                 boat_mul, equal shapes (arithmetic.c:240-285)
 * lincomb: y = alpha*a + beta*b on FP32 or BF16 storage - boat_add / boat_sub of equal shapes
 *          (arithmetic.c:157-285), the residual adds of the encoder block, the MSE gradient
 * cast:    FP32 <-> BF16, round to nearest even
 * round_tf32: y = x rounded to the nearest TF32 value, stored as FP32 (in place allowed);
 *          operands prepared this way make the tensor core's own truncation exact
 * transpose: out[b, j, i] = in[b, i, j]   boat_transpose of the last two dims (linear.c:238-406) */
int boat_cuda_colsum(const void* X, int x_type, int64_t rows, int64_t cols, float* out);
/* colsum of `count` (1 to 4) matrices of one shape and type in one launch: the bias gradients of
 * the Q, K and V projections. */
int boat_cuda_colsum_multi(const void* const* X, int x_type, int64_t rows, int64_t cols, float* const* out, int count);
int boat_cuda_axpy(float* y, const float* x, float alpha, int64_t n);
int boat_cuda_scale(float* y, const float* x, float alpha, int64_t n);
int boat_cuda_add_bias(float* y, const float* x, const float* bias, int64_t rows, int64_t cols);
int boat_cuda_mul(float* y, const float* a, const float* b, int64_t n);
int boat_cuda_lincomb(void* y, const void* a, float alpha, const void* b, float beta, int type, int64_t n);
int boat_cuda_cast(void* dst, int dst_type, const void* src, int src_type, int64_t n);
int boat_cuda_round_tf32(float* y, const float* x, int64_t n);
/* `count` (1 to 8) FP32 tensors converted in one launch: to BF16 (dst_type BOAT_CUDA_BF16) or to
 * TF32-valued FP32 (BOAT_CUDA_F32_TF32) - the per-step copies of a layer's FP32 weights in the
 * form the tensor cores read. */
int boat_cuda_convert_multi(void* const* dst, int dst_type, const float* const* src, const int64_t* n, int count);
int boat_cuda_transpose(float* out, const float* in, int64_t batch, int64_t rows, int64_t cols);

/* ---- LayerNorm and GELU (the pre-LN encoder block around the attention layer) --------------
 * layernorm_fwd: per row of [rows, cols]: y = (x - mean) / sqrt(var + eps) * gamma + beta with
 *   the biased variance - boat_layernorm_forward, src/layers/norm.c:231-317.  gamma/beta FP32
 *   or NULL; mean_out / rstd_out [rows] FP32 (or NULL) are what the backward needs.
 * layernorm_bwd: dx, and dgamma / dbeta [cols] FP32 (overwritten; NULL to skip).  The
 *   reference's backward is a stub (norm.c:397-402); this is the analytic gradient.
 * gelu_fwd / gelu_bwd: y = x/2 (1 + erf(x/sqrt 2)), dx = dy * dGELU(x).  The reference's
 *   boat_gelu is a stub (src/ops/activation.c:298-302); the exact erf form is used. */
int boat_cuda_layernorm_fwd(const void* x, int type, int64_t rows, int64_t cols, const float* gamma,
                            const float* beta, float eps, void* y, float* mean_out, float* rstd_out);
int boat_cuda_layernorm_bwd(const void* dy, const void* x, int type, int64_t rows, int64_t cols,
                            const float* gamma, const float* mean, const float* rstd,
                            void* dx, float* dgamma, float* dbeta);
int boat_cuda_gelu_fwd(void* y, const void* x, int type, int64_t n);
int boat_cuda_gelu_bwd(void* dx, const void* dy, const void* x, int type, int64_t n);

/* ---- Adam step over a list of FP32 tensors (adam_update_parameter, src/optimizers/adam.c:156-193) ----
 * For tensor t in [0,count) and each of its nelements[t] elements, in the reference's order of
 * rounded FP32 operations:  m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g;
 * p -= lr*(m/corr1) / (sqrt(v/corr2) + eps),  corr1 = 1-b1^t, corr2 = 1-b2^t computed by the
 * caller on the host (the reference uses powf there).  The pointer arrays live in host memory;
 * the tensors they point to live on the device.  One launch covers up to 24 tensors. */
int boat_cuda_adam_step(int count, float* const* params, const float* const* grads, float* const* m,
                        float* const* v, const int64_t* nelements, float lr, float beta1, float beta2,
                        float epsilon, float corr1, float corr2);

/* ---- gradient exchange between GPUs (nothing in the reference: it is single-process) ---
 * One process per GPU.  Rank 0 makes an id (128 bytes) and hands it to the others by any
 * host channel; every rank then calls comm_init.  allreduce sums an FP32 buffer in place
 * across ranks on the library stream.
 *
 * allreduce_begin / _join overlap the sums with later kernels: begin starts the in-place sums of
 * `pieces` buffers (bufs[i], counts[i] floats) on a communication stream of the library, ordered
 * after everything launched on the library stream so far; join makes the library stream wait
 * for all sums begun since the last join.  Nothing may write the pieces in between.
 *
 * Failures end in an error status, not in a stuck host thread: the communicator is
 * non-blocking, every NCCL call is polled under a deadline (BOAT_COMM_INIT_TIMEOUT_S, default
 * 120 s, for joining; BOAT_COMM_TIMEOUT_S, default 30 s, for a collective to be accepted), and
 * on a deadline or an NCCL error the communicator is aborted (status 23 / 2000+ncclResult) and
 * comm_world() is 1 again.  Before the first sum of a given length the ranks agree on that
 * length through the communicator; a rank with another bucket size gets status 25.
 * BOAT_NCCL_LIB names the NCCL library to load (default libnccl.so.2). */
int boat_cuda_comm_unique_id(void* id_out_host_128B);
int boat_cuda_comm_init(int rank, int world, const void* id_host_128B);
int boat_cuda_comm_world(void);                 /* 1 when no communicator exists */
int boat_cuda_allreduce_sum_f32(float* buf, int64_t n);
int boat_cuda_allreduce_begin(float* const* bufs, const int64_t* counts, int pieces);
int boat_cuda_allreduce_join(void);
int boat_cuda_allreduce_pending(void);          /* 1 between a begin and its join */
int boat_cuda_comm_destroy(void);

#pragma GCC visibility pop
#ifdef __cplusplus
}
#endif
#endif /* BOAT_CUDA_H */
