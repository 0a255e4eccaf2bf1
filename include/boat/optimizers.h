/* boat/optimizers.h - the optimizer that follows the attention training step.
 *
 * Same names, arguments and behaviour as the reference's include/boat/optimizers.h for the
 * Adam optimizer (src/optimizers/adam.c) and the type-dispatching entry points
 * (src/optimizers/optimizer_common.c).  The update runs on the GPU in the reference's order
 * of FP32 operations and gives the same bits.  Parameters may be host tensors (uploaded,
 * updated and written back on every step, as a drop-in needs) or CUDA tensors (updated in
 * place, nothing crosses PCIe).  The moment estimates always live on the GPU.
 *
 * Not provided: RMSprop and Adagrad (outside the attention path), and SGD, whose create
 * function is a stub returning NULL in the reference (optimizer_common.c:77-82) - kept so. */
#ifndef BOAT_OPTIMIZERS_H
#define BOAT_OPTIMIZERS_H

#include "export.h"
#include "tensor.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    BOAT_OPTIMIZER_SGD,
    BOAT_OPTIMIZER_ADAM,
    BOAT_OPTIMIZER_RMSPROP,
    BOAT_OPTIMIZER_ADAGRAD
} boat_optimizer_type_t;

typedef struct boat_optimizer_t boat_optimizer_t;

/* NULL, as in the reference. */
BOAT_API boat_optimizer_t* boat_sgd_optimizer_create(float learning_rate, float momentum);
/* NULL unless learning_rate > 0 and 0 < beta1, beta2 < 1 (adam.c:37-49). */
BOAT_API boat_optimizer_t* boat_adam_optimizer_create(float learning_rate, float beta1, float beta2, float epsilon);

/* One update of every registered parameter from its gradient tensor, then timestep += 1
 * (adam.c:196-209).  Bias corrections use powf(beta, timestep + 1) as the reference does. */
BOAT_API void boat_optimizer_step(boat_optimizer_t* optimizer);
/* Sets every registered gradient tensor to zero (adam.c:211-231). */
BOAT_API void boat_optimizer_zero_grad(boat_optimizer_t* optimizer);
/* Frees the optimizer and its moment estimates; parameters and gradients stay the caller's. */
BOAT_API void boat_optimizer_free(boat_optimizer_t* optimizer);

/* Registers a (parameter, gradient) pair; both are borrowed, not referenced, and must
 * outlive the optimizer, be FP32, and have the same number of elements (adam.c:87-128). */
BOAT_API void boat_optimizer_add_parameter(boat_optimizer_t* optimizer, boat_tensor_t* param, boat_tensor_t* grad);

BOAT_API float boat_optimizer_get_learning_rate(const boat_optimizer_t* optimizer);
BOAT_API void boat_optimizer_set_learning_rate(boat_optimizer_t* optimizer, float learning_rate);

#ifdef __cplusplus
}
#endif
#endif /* BOAT_OPTIMIZERS_H */
