/* autodiff.h - variables and reverse-mode differentiation for the attention path.
 *
 * Subset of the reference's include/boat/autodiff.h:25-66: variable create/free/accessors,
 * boat_variable_backward, the attention op and the ops an encoder block puts next to it -
 * add, sub, mul, matmul and the dense-layer op (reference implementation:
 * src/autodiff.c:138-572, :1002-1180, :1454-1496, :2388-2672).  Every op accepts host or
 * CUDA tensors; with CUDA tensors the graph never leaves the GPU.  The reference keeps op
 * nodes in a generic graph library; here a variable simply points at the op record that
 * produced it, which is all reverse mode needs.  The reference's other op types (div, dot,
 * relu, sigmoid, tanh, softmax, reductions, conv, pool, flatten) are outside this path and
 * are not provided. */
#ifndef BOAT_AUTODIFF_H
#define BOAT_AUTODIFF_H

#include "tensor.h"
#include "export.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct boat_variable_t boat_variable_t;
struct boat_attention_t;
struct boat_dense_layer_t;

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

/* Element-wise ops on equal shapes and the 2-D matrix product, with gradient tracking
 * (autodiff.c:466-499).  Backward: add da=db=g; sub da=g, db=-g; mul da=g*b, db=g*a;
 * matmul dA=g.B^T, dB=A^T.g. */
BOAT_API boat_variable_t* boat_var_add(const boat_variable_t* a, const boat_variable_t* b);
BOAT_API boat_variable_t* boat_var_sub(const boat_variable_t* a, const boat_variable_t* b);
BOAT_API boat_variable_t* boat_var_mul(const boat_variable_t* a, const boat_variable_t* b);
BOAT_API boat_variable_t* boat_var_matmul(const boat_variable_t* a, const boat_variable_t* b);

/* Forward through a dense layer ([N, in] input); backward runs boat_dense_layer_backward,
 * which accumulates the layer's dW and db, and adds dx to the input's gradient
 * (autodiff.c:563-567, :2640-2672).  The layer stays owned by the caller. */
BOAT_API boat_variable_t* boat_var_dense(const boat_variable_t* input, const struct boat_dense_layer_t* layer);

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
