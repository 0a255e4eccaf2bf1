/* boat_internal.h - declarations shared by the C host layer (not installed). */
#ifndef BOAT_INTERNAL_H
#define BOAT_INTERNAL_H

#include <boat/tensor.h>
#include <boat/memory.h>
#include <boat_cuda.h>

/* Same information as the reference's tensor record (src/core/tensor.c:14-26); for a CUDA
 * tensor `data` is a device pointer. */
struct boat_tensor_t {
    int64_t*       shape;
    size_t         ndim;
    boat_dtype_t   dtype;
    boat_device_t  device;
    void*          data;
    size_t         nbytes;
    size_t         nelements;
    bool           is_contiguous;
    size_t         ref_count;
    boat_tensor_t* parent;     /* kept alive while this view exists */
    bool           is_view;
};

/* boat_tensor_create without the zero fill, for outputs a kernel overwrites completely. */
boat_tensor_t* boat_tensor_create_uninit(const int64_t* shape, size_t ndim, boat_dtype_t dtype,
                                         boat_device_t device);
/* A CUDA tensor around a buffer from boat_cuda_malloc; the tensor owns the buffer from then on. */
boat_tensor_t* boat_tensor_adopt_device(const int64_t* shape, size_t ndim, boat_dtype_t dtype, void* device_data);
/* A view of `bytes` bytes starting `offset_bytes` into `parent` with its own shape. */
boat_tensor_t* boat_tensor_window(boat_tensor_t* parent, size_t offset_bytes, const int64_t* shape,
                                  size_t ndim);

/* Prints "boat: <what>: <device error text>" to stderr; returns rc unchanged. */
int boat_report(const char* what, int rc);

#endif
