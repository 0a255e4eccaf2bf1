/* tensor.h - dense row-major tensor handle used by the attention path.
 *
 * ABI-compatible with the reference's include/boat/tensor.h: the enum values, the opaque
 * handle and every function below keep the reference's name, argument order and meaning
 * (tensor.h:22-104 there).  Two things are new:
 *   - BOAT_DEVICE_CUDA tensors really live in B200 HBM (the reference silently gave host
 *     memory for them, src/core/tensor.c:55-57 -> src/core/memory.c:46-74).  For such a
 *     tensor boat_tensor_data() is a DEVICE pointer; move bytes with boat_memory_copy().
 *   - BOAT_DTYPE_BFLOAT16 is appended directly before BOAT_DTYPE_COUNT, so every
 *     existing dtype keeps its number.
 * Functions the reference declares but never defines (clone, contiguous, transpose,
 * concatenate, stack, print, to_string, equal, allclose) are not part of this path and
 * are not declared; boat_tensor_to_device (declared-only in the reference, tensor.h:92)
 * is implemented because host<->HBM movement is this library's job. */
#ifndef BOAT_TENSOR_H
#define BOAT_TENSOR_H

#include <stddef.h>
#include <stdint.h>
#include <stdbool.h>
#include "export.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct boat_tensor_t boat_tensor_t;

/* Element types.  Numbering follows the reference (FLOAT64 = 0, FLOAT32 = 1, ...). */
typedef enum {
    BOAT_DTYPE_FLOAT64,
    BOAT_DTYPE_FLOAT32,
    BOAT_DTYPE_FLOAT16,
    BOAT_DTYPE_FLOAT8,
    BOAT_DTYPE_FLOAT4,
    BOAT_DTYPE_INT64,
    BOAT_DTYPE_INT32,
    BOAT_DTYPE_UINT8,
    BOAT_DTYPE_BITS2,
    BOAT_DTYPE_BITS1,
    BOAT_DTYPE_BOOL,
    BOAT_DTYPE_BFLOAT16,   /* extension: 16-bit brain float, device activations/shadows */
    BOAT_DTYPE_COUNT
} boat_dtype_t;

#ifndef BOAT_DEVICE_T_DEFINED
#define BOAT_DEVICE_T_DEFINED
enum boat_device_enum {
    BOAT_DEVICE_CPU,       /* host memory                               */
    BOAT_DEVICE_CUDA,      /* HBM of the current CUDA device (B200)     */
    BOAT_DEVICE_COUNT
};
typedef enum boat_device_enum boat_device_t;
#endif

#define BOAT_MAX_DIMS 8

/* Lifetime.  Every returned tensor has reference count 1 and is owned by the caller;
 * boat_tensor_free and boat_tensor_unref are the same operation (reference:
 * src/core/tensor.c:164-191).  New tensors are zero-filled (tensor.c:132). */
BOAT_API boat_tensor_t* boat_tensor_create(const int64_t* shape, size_t ndim,
                                           boat_dtype_t dtype, boat_device_t device);
BOAT_API boat_tensor_t* boat_tensor_create_like(const boat_tensor_t* other);
BOAT_API boat_tensor_t* boat_tensor_from_data(const int64_t* shape, size_t ndim,
                                              boat_dtype_t dtype, const void* data);
BOAT_API void boat_tensor_free(boat_tensor_t* tensor);
BOAT_API void boat_tensor_ref(boat_tensor_t* tensor);
BOAT_API void boat_tensor_unref(boat_tensor_t* tensor);

/* Properties.  A NULL handle yields the reference's defaults (NULL / 0 / FLOAT32 / CPU /
 * false), never a crash (tensor.c:193-227). */
BOAT_API const int64_t* boat_tensor_shape(const boat_tensor_t* tensor);
BOAT_API size_t         boat_tensor_ndim(const boat_tensor_t* tensor);
BOAT_API boat_dtype_t   boat_tensor_dtype(const boat_tensor_t* tensor);
BOAT_API boat_device_t  boat_tensor_device(const boat_tensor_t* tensor);
BOAT_API size_t         boat_tensor_nbytes(const boat_tensor_t* tensor);
BOAT_API size_t         boat_tensor_nelements(const boat_tensor_t* tensor);
BOAT_API bool           boat_tensor_is_contiguous(const boat_tensor_t* tensor);
BOAT_API void*          boat_tensor_data(const boat_tensor_t* tensor);
BOAT_API const void*    boat_tensor_const_data(const boat_tensor_t* tensor);

/* Views.  A reshape shares the parent's bytes and keeps the parent alive
 * (tensor.c:253-300); a slice is a unit-step window of a contiguous parent
 * (tensor.c:302-456). */
BOAT_API boat_tensor_t* boat_tensor_reshape(const boat_tensor_t* tensor,
                                            const int64_t* new_shape, size_t new_ndim);
BOAT_API boat_tensor_t* boat_tensor_slice(const boat_tensor_t* tensor, const size_t* start,
                                          const size_t* end, const size_t* step);

/* Copy a tensor to the other memory space (host <-> HBM).  Returns a new tensor. */
BOAT_API boat_tensor_t* boat_tensor_to_device(const boat_tensor_t* tensor, boat_device_t dev);

BOAT_API size_t      boat_dtype_size(boat_dtype_t dtype);
BOAT_API const char* boat_dtype_name(boat_dtype_t dtype);

#ifdef __cplusplus
}
#endif
#endif /* BOAT_TENSOR_H */
