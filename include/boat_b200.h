/* boat_b200.h - additions to Boat's C API that only make sense with a GPU behind it.
 *
 * None of these has a counterpart in the reference (its layer is host-only and FP32-only);
 * they add capability and never change the meaning of a reference entry point.  A program
 * that ignores this header gets the reference's behaviour with the arithmetic done on the
 * GPU: host tensors in, host tensors out. */
#ifndef BOAT_B200_H
#define BOAT_B200_H

#include "boat/tensor.h"
#include "boat/layers/attention.h"
#include "boat/layers/norm.h"
#include "boat/layers.h"
#include "boat/optimizers.h"
#include "boat_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Move the layer's eight parameters (and from then on its gradients) to `device`.
 * With BOAT_DEVICE_CUDA the accessors hand out CUDA tensors, nothing is uploaded per call
 * and forward/backward accept CUDA inputs without host traffic.  Returns 0 on success. */
BOAT_API int boat_attention_to_device(boat_attention_t* attention, boat_device_t device);

/* Choose the arithmetic: BOAT_MMA_FP32 (exact CUDA-core path, any shape), BOAT_MMA_TF32
 * or BOAT_MMA_BF16 (tcgen05 tensor-core paths; need seq_len % 128 == 0 and head size 64 or
 * 128, other shapes run on the CUDA cores with the same storage), or -1 for automatic:
 * BF16 tensors -> BF16, FP32 tensors -> exact FP32 whatever the shape, so that a reference
 * program's numbers never depend on the sequence length; TF32 is always an explicit choice.
 * The default is taken from the environment variable BOAT_MMA (fp32 | tf32 | bf16 | auto),
 * else automatic.  Returns 0 on success. */
BOAT_API int boat_attention_set_precision(boat_attention_t* attention, int mma);
BOAT_API int boat_attention_get_precision(const boat_attention_t* attention);

/* Forward for a contiguous range of (batch, head) units of a larger [B, seq_len, H] problem,
 * given only the token rows that range owns - the entry that lets one problem be split over
 * GPUs by batch x heads.  Boat's head split is a reshape (src/layers/attention.c:393-397), so
 * with the head count dividing seq_len, unit u = b*heads + h of the flattened [B*seq_len, H]
 * input is exactly its rows [u*seq_len/heads, (u+1)*seq_len/heads): n consecutive units are
 * n*seq_len/heads consecutive rows and need nothing else.  query, key, value: [R, H] with R a
 * multiple of seq_len/heads; returns [R, H] - the same rows of the full problem's output.
 * boat_attention_backward then takes the [R, H] upstream gradient of those rows and returns
 * their [R, H] input gradients; the parameter gradients it leaves are this range's share, and
 * their sum over all ranges (boat_attention_allreduce_grads) is the full problem's gradient.
 * NULL when seq_len is not a multiple of the head count or the shapes do not fit. */
BOAT_API boat_tensor_t* boat_attention_forward_units(boat_attention_t* attention, const boat_tensor_t* query,
                                                     const boat_tensor_t* key, const boat_tensor_t* value,
                                                     int64_t seq_len);

/* The layer keeps its eight gradients back to back in one FP32 buffer, in the order
 * dWq dWk dWv dWo dbq dbk dbv dbo; the accessor tensors are windows into it.  Gives its
 * address (device memory for a CUDA layer, host memory otherwise) and element count;
 * NULL / 0 before the first backward. */
BOAT_API int boat_attention_grad_bucket(const boat_attention_t* attention, float** data, size_t* nelements);

/* Sum the gradient bucket over all ranks of the communicator made with
 * boat_cuda_comm_init (data-parallel training: every rank holds the same weights and a
 * different slice of the batch).  No-op with a single rank.  Returns 0 on success. */
BOAT_API int boat_attention_allreduce_grads(boat_attention_t* attention);

/* Overlap that sum with the backward (a CUDA layer, more than one rank).  mode 0 (default): nothing
 * is summed before boat_attention_allreduce_grads.  mode 1: boat_attention_backward itself starts,
 * on a communication stream, the sum of dWo | dbo as soon as the output projection's gradients are
 * final - it then runs under the attention-core backward - and the sum of dWq dWk dWv | dbq dbk dbv
 * before the three input-gradient GEMMs, which are then launched with one CTA per tile so that the
 * collective's CTAs are placed while they run.  mode 2: only the first of these is started by the
 * backward; the second is started by boat_attention_allreduce_grads (with two ranks the sum is short
 * and the one-CTA-per-tile GEMMs of mode 1 cost about what hiding it saves).  In modes 1
 * and 2 boat_attention_allreduce_grads joins the sums: call it, as before, after the backward and
 * before anything reads or updates the gradients. */
BOAT_API int boat_attention_get_grad_overlap(const boat_attention_t* attention);
BOAT_API int boat_attention_set_grad_overlap(boat_attention_t* attention, int mode);

/* Register the layer's parameters with an optimizer (boat/optimizers.h), each with its
 * gradient tensor.  The reference's layer makes new gradient tensors on every backward
 * (src/layers/attention.c:653-654, :702-703), which leaves an optimizer's registered pointers
 * dangling; here the gradient tensors are fixed windows into the bucket above and are created
 * (zeroed) by this call if no backward has run yet.  They are re-made when the layer moves to
 * another device, so call boat_attention_to_device first.  Returns 0 on success. */
BOAT_API int boat_attention_add_to_optimizer(boat_attention_t* attention, boat_optimizer_t* optimizer);

/* A pre-LN transformer encoder block step composed from borrowed layers:
 *   y = x + attention(LN1(x));  out = y + dense2(GELU(dense1(LN2(y))))
 * forward returns out for x [B,S,d]; backward takes dL/dout and returns dL/dx, leaving the
 * parameter gradients in the layers (dense gradients accumulate, as in the reference).  The
 * reference has the layers but no such composition; this is the chain of layer calls a caller
 * would write, issued from C.  free() releases the block's own state, not the layers. */
typedef struct boat_encoder_block_t boat_encoder_block_t;
BOAT_API boat_encoder_block_t* boat_encoder_block_create(boat_layernorm_t* norm1, boat_attention_t* attention,
                                                         boat_layernorm_t* norm2, boat_dense_layer_t* dense1,
                                                         boat_dense_layer_t* dense2);
BOAT_API boat_tensor_t* boat_encoder_block_forward(boat_encoder_block_t* block, const boat_tensor_t* x);
BOAT_API boat_tensor_t* boat_encoder_block_backward(boat_encoder_block_t* block, const boat_tensor_t* grad_output);
BOAT_API void boat_encoder_block_free(boat_encoder_block_t* block);
/* Data-parallel training of the block: sum every parameter gradient it left in its layers (the
 * attention bucket, both LayerNorms, both dense layers) over the ranks of the communicator, in
 * place; joins sums the attention backward started itself (boat_attention_set_grad_overlap).
 * The layers must be on BOAT_DEVICE_CUDA.  Returns 0 on success. */
BOAT_API int boat_encoder_block_allreduce_grads(boat_encoder_block_t* block);

/* Fill the layer's parameters from a safetensors checkpoint image (or file).  The reference
 * detects attention tensors by name in src/format/huggingface.c:917-932 and stops there (TODO);
 * this completes that step with the same name test: among the tensors whose name starts with
 * `prefix` (NULL or "" for any) and contains "attention", the one containing "query" / "key" /
 * "value" / "output" with a 2-D ".weight" becomes Wq / Wk / Wv / Wo - transposed, because
 * checkpoints store [out, in] and Boat [in, out] - and a 1-D ".bias" the matching bias.  F32, BF16
 * and F16 tensors are accepted.  Missing biases keep their values.  Returns 0, or 1 bad
 * argument / unreadable file, 2 malformed image, 3 a projection matrix is missing, 4 wrong
 * shape or type or an ambiguous name match, 5 device error. */
BOAT_API int boat_attention_load_safetensors(boat_attention_t* attention, const void* image, size_t size,
                                             const char* prefix);
BOAT_API int boat_attention_load_safetensors_file(boat_attention_t* attention, const char* path, const char* prefix);

/* alpha*a + beta*b for equal shapes, FP32 or BF16, host or device: one kernel for residual
 * adds, differences and the mean-squared-error gradient 2(o - t)/n. */
BOAT_API boat_tensor_t* boat_lincomb(const boat_tensor_t* a, float alpha, const boat_tensor_t* b, float beta);

/* dx = dy * dGELU/dx(input), the backward of boat_gelu (the reference has neither). */
BOAT_API boat_tensor_t* boat_gelu_backward(const boat_tensor_t* grad_output, const boat_tensor_t* input);

/* Parameter access and placement for the layers around attention, as for the attention layer. */
BOAT_API boat_tensor_t* boat_layernorm_get_weight(const boat_layernorm_t* norm);
BOAT_API boat_tensor_t* boat_layernorm_get_bias(const boat_layernorm_t* norm);
BOAT_API boat_tensor_t* boat_layernorm_get_grad_weight(const boat_layernorm_t* norm);   /* NULL before backward */
BOAT_API boat_tensor_t* boat_layernorm_get_grad_bias(const boat_layernorm_t* norm);
BOAT_API int boat_layernorm_to_device(boat_layernorm_t* norm, boat_device_t device);
BOAT_API int boat_dense_layer_to_device(boat_dense_layer_t* layer, boat_device_t device);

#ifdef __cplusplus
}
#endif
#endif /* BOAT_B200_H */
