/* autodiff.h - variables and reverse-mode differentiation, attention op only.
 *
 * Subset of the reference's include/boat/autodiff.h:25-66 that reaches the attention
 * layer: variable create/free/accessors, boat_var_attention and boat_variable_backward
 * (reference implementation: src/autodiff.c:138-463, :569-572, :2388-2532).  The
 * reference keeps op nodes in a generic graph library; here a variable simply points at
 * the op record that produced it, which is all reverse mode needs for this path.  The
 * other 17 op types of the reference are outside this path and are not provided. */
#ifndef BOAT_AUTODIFF_H
#define BOAT_AUTODIFF_H

#include "tensor.h"
#include "export.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct boat_variable_t boat_variable_t;
struct boat_attention_t;

/* The variable takes its own reference on `tensor` (autodiff.c:152-153). */
BOAT_API boat_variable_t* boat_variable_create(boat_tensor_t* tensor, bool requires_grad);
BOAT_API boat_variable_t* boat_variable_create_with_shape(const int64_t* shape, size_t ndim,
                                                          boat_dtype_t dtype, bool requires_grad);
BOAT_API void boat_variable_free(const boat_variable_t* variable);

BOAT_API boat_tensor_t* boat_variable_data(const boat_variable_t* variable);
BOAT_API boat_tensor_t* boat_variable_grad(const boat_variable_t* variable);   /* NULL until backward */
BOAT_API bool boat_variable_requires_grad(const boat_variable_t* variable);
BOAT_API void boat_variable_set_requires_grad(boat_variable_t* variable, bool requires_grad);
BOAT_API void boat_variable_zero_grad(boat_variable_t* variable);              /* drops the grad tensor */

/* grad_output == NULL means a gradient of ones (autodiff.c:311-338).  Leaves accumulate
 * into .grad; an attention output runs boat_attention_backward and adds dq, dk, dv into
 * the .grad of the query, key and value variables - the same variable passed three times
 * ends with dq+dk+dv (autodiff.c:2482-2526). */
BOAT_API void boat_variable_backward(boat_variable_t* variable, boat_tensor_t* grad_output);
BOAT_API void boat_variable_backward_full(const boat_variable_t* variable);

/* Forward through `attention` with gradient tracking.  The layer stays owned by the
 * caller: freeing variables never frees the layer (the reference's op-node destructor
 * did, autodiff.c:775-777 with :2418; that hazard is deliberately not reproduced). */
BOAT_API boat_variable_t* boat_var_attention(const boat_variable_t* query,
                                             const boat_variable_t* key,
                                             const boat_variable_t* value,
                                             const struct boat_attention_t* attention,
                                             const boat_tensor_t* attention_mask);

#ifdef __cplusplus
}
#endif
#endif /* BOAT_AUTODIFF_H */
