/* layers.h - the generic-layer entry points of the attention path and of the two layers the
 * encoder block puts around it (dense, LayerNorm).
 *
 * The reference's include/boat/layers.h declares adapters for every layer type; the
 * attention layer's five are at layers.h:82-92 (implementation:
 * src/layers/attention.c:1119-1175).  boat_attention_layer_t is the same object as
 * boat_attention_t. */
#ifndef BOAT_LAYERS_H
#define BOAT_LAYERS_H

#include "tensor.h"
#include "export.h"
#include "layers/attention.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef boat_attention_t boat_attention_layer_t;
typedef struct boat_dense_layer_t boat_dense_layer_t;
typedef struct boat_norm_layer_t boat_norm_layer_t;

/* Fully connected layer y = x.W + b for 2-D input [rows, in] (reference layers.h:23-35,
 * src/layers/dense.c): weight [in,out] Xavier-uniform from rand(), zero bias; backward
 * returns dX and ACCUMULATES dW, db; update is p -= lr*g and then clears the gradients. */
BOAT_API boat_dense_layer_t* BOAT_CALL boat_dense_layer_create(size_t input_features, size_t output_features, bool use_bias);
BOAT_API void BOAT_CALL boat_dense_layer_free(boat_dense_layer_t* layer);
BOAT_API boat_tensor_t* BOAT_CALL boat_dense_layer_forward(boat_dense_layer_t* layer, const boat_tensor_t* input);
BOAT_API boat_tensor_t* BOAT_CALL boat_dense_layer_backward(boat_dense_layer_t* layer, const boat_tensor_t* grad_output);
BOAT_API void BOAT_CALL boat_dense_layer_update(boat_dense_layer_t* layer, float learning_rate);
BOAT_API void BOAT_CALL boat_dense_layer_set_weight(boat_dense_layer_t* layer, boat_tensor_t* weight);
BOAT_API void BOAT_CALL boat_dense_layer_set_bias(boat_dense_layer_t* layer, boat_tensor_t* bias);
BOAT_API boat_tensor_t* BOAT_CALL boat_dense_layer_get_weight(const boat_dense_layer_t* layer);
BOAT_API boat_tensor_t* BOAT_CALL boat_dense_layer_get_bias(const boat_dense_layer_t* layer);
BOAT_API boat_tensor_t* BOAT_CALL boat_dense_layer_get_grad_weight(const boat_dense_layer_t* layer);
BOAT_API boat_tensor_t* BOAT_CALL boat_dense_layer_get_grad_bias(const boat_dense_layer_t* layer);

/* LayerNorm through the generic-layer names (reference layers.h:75-79, declared only). */
BOAT_API boat_norm_layer_t* BOAT_CALL boat_norm_layer_create(size_t normalized_shape, float eps, bool elementwise_affine);
BOAT_API void BOAT_CALL boat_norm_layer_free(boat_norm_layer_t* layer);
BOAT_API boat_tensor_t* BOAT_CALL boat_norm_layer_forward(boat_norm_layer_t* layer, const boat_tensor_t* input);
BOAT_API boat_tensor_t* BOAT_CALL boat_norm_layer_backward(boat_norm_layer_t* layer, const boat_tensor_t* grad_output);
BOAT_API void BOAT_CALL boat_norm_layer_update(boat_norm_layer_t* layer, float learning_rate);

/* use_bias = true, no rotary; head_size = hidden/num_heads (attention.c:1122-1140). */
BOAT_API boat_attention_layer_t* BOAT_CALL boat_attention_layer_create(size_t hidden_size,
                                                                       size_t num_heads,
                                                                       float dropout_prob,
                                                                       bool causal_mask);
BOAT_API void BOAT_CALL boat_attention_layer_free(boat_attention_layer_t* layer);
BOAT_API boat_tensor_t* BOAT_CALL boat_attention_layer_forward(boat_attention_layer_t* layer,
                                                               const boat_tensor_t* query,
                                                               const boat_tensor_t* key,
                                                               const boat_tensor_t* value,
                                                               const boat_tensor_t* attention_mask);
/* Returns the gradient w.r.t. query; the key/value gradients are dropped (attention.c:1158-1171). */
BOAT_API boat_tensor_t* BOAT_CALL boat_attention_layer_backward(boat_attention_layer_t* layer,
                                                                const boat_tensor_t* grad_output);
BOAT_API void BOAT_CALL boat_attention_layer_update(boat_attention_layer_t* layer, float learning_rate);

#ifdef __cplusplus
}
#endif
#endif /* BOAT_LAYERS_H */
