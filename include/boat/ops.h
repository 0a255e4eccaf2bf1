/* ops.h - the stateless tensor operations the attention path and its callers use.
 *
 * Subset of the reference's include/boat/ops.h: the functions src/layers/attention.c and
 * src/autodiff.c call on this path (boat_matmul linear.c:12-170, boat_transpose
 * linear.c:238-406, boat_add/boat_mul arithmetic.c:157-285, boat_add_/boat_sub_
 * arithmetic.c:362-422, boat_mul_scalar arithmetic.c:425-484).  FP32 only, computed on
 * the GPU; CPU tensors are staged through HBM for the call. */
#ifndef BOAT_OPS_H
#define BOAT_OPS_H

#include "tensor.h"
#include "export.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Element-wise with the broadcast forms the path uses: equal shapes, or `b` equal to the
 * trailing dimensions of `a` (bias [H] added to [B,S,H]).  Other shape pairs give NULL. */
BOAT_API boat_tensor_t* boat_add(const boat_tensor_t* a, const boat_tensor_t* b);
BOAT_API boat_tensor_t* boat_mul(const boat_tensor_t* a, const boat_tensor_t* b);
/* Equal shapes only; FP32 or BF16 (boat_add of equal shapes accepts BF16 as well). */
BOAT_API boat_tensor_t* boat_sub(const boat_tensor_t* a, const boat_tensor_t* b);

/* In place, equal element counts required (arithmetic.c:362-422); otherwise no-op. */
BOAT_API void boat_add_(boat_tensor_t* a, const boat_tensor_t* b);
BOAT_API void boat_sub_(boat_tensor_t* a, const boat_tensor_t* b);

BOAT_API boat_tensor_t* boat_mul_scalar(const boat_tensor_t* a, double scalar);

/* GELU, exact erf form x/2 (1 + erf(x/sqrt 2)).  A stub returning NULL in the reference
 * (src/ops/activation.c:298-302); FP32 or BF16 tensors. */
BOAT_API boat_tensor_t* boat_gelu(const boat_tensor_t* a);

/* 2-D..4-D, leading (batch) dimensions must match exactly (linear.c:32-36). */
BOAT_API boat_tensor_t* boat_matmul(const boat_tensor_t* a, const boat_tensor_t* b);
/* Materialised swap of two dimensions. */
BOAT_API boat_tensor_t* boat_transpose(const boat_tensor_t* a, int dim0, int dim1);

#ifdef __cplusplus
}
#endif
#endif /* BOAT_OPS_H */
