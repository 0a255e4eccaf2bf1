/* attention.h - multi-head attention layer: forward, backward, SGD update.
 *
 * Same entry points, argument meaning and error behaviour as the reference's
 * include/boat/layers/attention.h:19-107 (implementation there:
 * src/layers/attention.c).  What the layer computes, per call:
 *
 *   forward   Qp = q.Wq+bq, Kp = k.Wk+bk, Vp = v.Wv+bv            (attention.c:247-308, :363-365)
 *             heads: [B,S,H] is VIEWED as [B,nh,S,hs] - a reshape, not a transpose, so
 *             head (b,h) is the contiguous S*hs block at element (b*nh+h)*S*hs
 *                                                                  (attention.c:393-397)
 *             O = softmax(Qp.Kp^T / sqrt(hs) [causal: j>i -> -1e9]) . Vp   (:882-1079)
 *             out = O.Wo + bo                                      (:460-465)
 *   backward  dWo, dbo, dO;  dV = P^T dO, dP = dO V^T, dS = P*(dP - rowsum(dP*P)) / sqrt(hs),
 *             dQ = dS K, dK = dS^T Q;  then dW*, db*, dq, dk, dv   (:468-732, :1186-1534)
 *   update    p -= lr * g for the 8 parameters, gradients kept     (:734-815)
 *
 * attention_mask, dropout_prob and use_rotary are accepted and ignored exactly as in the
 * reference (attention.c:1022-1025, :1061-1062, :419-421).
 *
 * All arithmetic runs on the GPU; there is no host fallback.  CPU tensors are uploaded
 * for the call and results are written back to host tensors, CUDA tensors are used in
 * place. */
#ifndef BOAT_ATTENTION_H
#define BOAT_ATTENTION_H

#include "../tensor.h"
#include "../export.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct boat_attention_t boat_attention_t;

typedef struct {
    size_t hidden_size;    /* d_model                                            */
    size_t num_heads;
    size_t head_size;      /* 0 -> hidden_size / num_heads                       */
    float  dropout_prob;   /* stored, never applied                              */
    bool   causal_mask;    /* scores[i][j>i] = -1e9 before the softmax           */
    bool   use_bias;
    bool   use_rotary;     /* stored, never applied                              */
    float  rotary_theta;
} boat_attention_config_t;

/* NULL if config is NULL, a size is 0, or hidden_size % num_heads != 0
 * (attention.c:126-134).  Weights [in,out] ~ U(+-sqrt(2/(in+out))) from rand(), biases 0. */
BOAT_API boat_attention_t* BOAT_CALL boat_attention_create(const boat_attention_config_t* config);
BOAT_API void BOAT_CALL boat_attention_free(boat_attention_t* attention);

/* Returns a new [B,S,H] tensor (refcount 1) or NULL.  The three inputs are referenced by
 * the layer until the next forward or boat_attention_free. */
BOAT_API boat_tensor_t* BOAT_CALL boat_attention_forward(boat_attention_t* attention,
                                                         const boat_tensor_t* query,
                                                         const boat_tensor_t* key,
                                                         const boat_tensor_t* value,
                                                         const boat_tensor_t* attention_mask);

/* false if there is no cached forward.  Each non-NULL out-parameter receives a new
 * tensor owned by the caller.  Parameter gradients are stored in the layer and read
 * through the accessors; each backward overwrites them (no accumulation). */
BOAT_API bool BOAT_CALL boat_attention_backward(boat_attention_t* attention,
                                                const boat_tensor_t* grad_output,
                                                boat_tensor_t** grad_query,
                                                boat_tensor_t** grad_key,
                                                boat_tensor_t** grad_value);

BOAT_API void BOAT_CALL boat_attention_update(boat_attention_t* attention, float learning_rate);
BOAT_API void BOAT_CALL boat_attention_set_dropout(boat_attention_t* attention, float dropout_prob);
BOAT_API void BOAT_CALL boat_attention_set_causal(boat_attention_t* attention, bool causal);

/* Self-attention through a temporary layer with fresh random weights (attention.c:830-879). */
BOAT_API boat_tensor_t* BOAT_CALL boat_multihead_attention(const boat_tensor_t* input,
                                                           size_t num_heads,
                                                           float dropout_prob,
                                                           bool causal_mask,
                                                           const boat_tensor_t* attention_mask);

/* softmax(scale * Q K^T [causal]) V on [B,nh,S,hs] FP32 tensors.  Inputs with ndim 3 or
 * >4 give a copy of `value`, ndim < 3 gives NULL (attention.c:899-917). */
BOAT_API boat_tensor_t* BOAT_CALL boat_scaled_dot_product_attention(const boat_tensor_t* query,
                                                                    const boat_tensor_t* key,
                                                                    const boat_tensor_t* value,
                                                                    float scale_factor,
                                                                    const boat_tensor_t* attention_mask,
                                                                    bool causal_mask,
                                                                    float dropout_prob);

/* Placeholders kept for link compatibility: return NULL / do nothing (attention.c:1094-1117). */
BOAT_API boat_tensor_t* BOAT_CALL boat_rotary_position_encoding(const boat_tensor_t* tensor,
                                                                size_t seq_len, size_t head_size,
                                                                float theta);
BOAT_API void BOAT_CALL boat_apply_rotary_embedding(boat_tensor_t* query, boat_tensor_t* key,
                                                    size_t seq_len, size_t head_size, float theta);

/* Parameter / gradient accessors (attention.c:1537-1631).  The returned tensor is the
 * layer's own (no reference is taken); gradients are NULL before the first backward. */
#define BOAT_ATTN_ACCESSOR(name) \
    BOAT_API boat_tensor_t* BOAT_CALL boat_attention_get_##name(const boat_attention_t* attention)
BOAT_ATTN_ACCESSOR(weight_q);      BOAT_ATTN_ACCESSOR(weight_k);
BOAT_ATTN_ACCESSOR(weight_v);      BOAT_ATTN_ACCESSOR(weight_o);
BOAT_ATTN_ACCESSOR(bias_q);        BOAT_ATTN_ACCESSOR(bias_k);
BOAT_ATTN_ACCESSOR(bias_v);        BOAT_ATTN_ACCESSOR(bias_o);
BOAT_ATTN_ACCESSOR(grad_weight_q); BOAT_ATTN_ACCESSOR(grad_weight_k);
BOAT_ATTN_ACCESSOR(grad_weight_v); BOAT_ATTN_ACCESSOR(grad_weight_o);
BOAT_ATTN_ACCESSOR(grad_bias_q);   BOAT_ATTN_ACCESSOR(grad_bias_k);
BOAT_ATTN_ACCESSOR(grad_bias_v);   BOAT_ATTN_ACCESSOR(grad_bias_o);
#undef BOAT_ATTN_ACCESSOR

#ifdef __cplusplus
}
#endif
#endif /* BOAT_ATTENTION_H */
