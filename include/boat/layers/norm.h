/* norm.h - LayerNorm layer.
 *
 * The LayerNorm part of the reference's include/boat/layers/norm.h:22-38, :74-76 (RMSNorm and
 * the functional forms, which the reference declares and leaves as stubs returning NULL -
 * src/layers/norm.c:414-478 - are not on the attention path and are not provided).
 * Forward matches boat_layernorm_forward (norm.c:231-317).  The reference's
 * boat_layernorm_backward and boat_layernorm_update are stubs (norm.c:397-412); here they do
 * the work: backward returns the input gradient and stores d(weight), d(bias) in the layer. */
#ifndef BOAT_NORM_H
#define BOAT_NORM_H

#include "../tensor.h"
#include "../export.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct boat_layernorm_t boat_layernorm_t;

typedef struct {
    size_t normalized_shape;   /* length of the last dimension                     */
    float  eps;                /* added to the variance inside the square root     */
    bool   elementwise_affine; /* learnable weight (ones) ...                      */
    bool   use_bias;           /* ... and bias (zeros)                             */
} boat_layernorm_config_t;

BOAT_API boat_layernorm_t* boat_layernorm_create(const boat_layernorm_config_t* config);
BOAT_API void boat_layernorm_free(boat_layernorm_t* norm);
/* Any rank >= 1 whose last dimension equals normalized_shape; FP32 or BF16; host or device. */
BOAT_API boat_tensor_t* boat_layernorm_forward(boat_layernorm_t* norm, const boat_tensor_t* input);
BOAT_API boat_tensor_t* boat_layernorm_backward(boat_layernorm_t* norm, const boat_tensor_t* grad_output);
BOAT_API void boat_layernorm_update(boat_layernorm_t* norm, float learning_rate);
/* The layer takes its own reference on the tensor (norm.c:481-517). */
BOAT_API void boat_layernorm_set_weight(boat_layernorm_t* norm, boat_tensor_t* weight);
BOAT_API void boat_layernorm_set_bias(boat_layernorm_t* norm, boat_tensor_t* bias);

#ifdef __cplusplus
}
#endif
#endif /* BOAT_NORM_H */
