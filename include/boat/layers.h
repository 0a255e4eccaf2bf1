/* layers.h - the generic-layer adapter of the attention layer.
 *
 * The reference's include/boat/layers.h declares adapters for every layer type; the
 * attention path only needs the five at layers.h:82-92 (implementation:
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
