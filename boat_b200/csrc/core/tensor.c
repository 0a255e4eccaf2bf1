/* tensor.c - reference-counted dense tensors in host memory or B200 HBM.
 *
 * Behaviour follows the reference (src/core/tensor.c): create zero-fills (:132), free and
 * unref are one operation (:164-191), a reshape is a view that pins its parent (:253-300),
 * a slice is a unit-step window of a contiguous parent (:302-456), accessors answer NULL
 * handles with defaults (:193-227).  Difference: the data of a BOAT_DEVICE_CUDA tensor is
 * allocated in HBM through the CUDA runtime layer instead of malloc (reference :55-62). */
#include "boat_internal.h"
#include <string.h>

static size_t element_size(boat_dtype_t dtype) {
    switch (dtype) {
        case BOAT_DTYPE_FLOAT64:  return 8;
        case BOAT_DTYPE_FLOAT32:  return 4;
        case BOAT_DTYPE_FLOAT16:  return 2;
        case BOAT_DTYPE_BFLOAT16: return 2;
        case BOAT_DTYPE_INT64:    return 8;
        case BOAT_DTYPE_INT32:    return 4;
        case BOAT_DTYPE_FLOAT8:
        case BOAT_DTYPE_FLOAT4:
        case BOAT_DTYPE_UINT8:
        case BOAT_DTYPE_BITS2:
        case BOAT_DTYPE_BITS1:    return 1;
        case BOAT_DTYPE_BOOL:     return sizeof(bool);
        default:                  return 0;
    }
}

static size_t packed_bytes(boat_dtype_t dtype, size_t n) {
    switch (dtype) {               /* sub-byte types share bytes (tensor.c:105-115) */
        case BOAT_DTYPE_FLOAT4: return (n + 1) / 2;
        case BOAT_DTYPE_BITS2:  return (n + 3) / 4;
        case BOAT_DTYPE_BITS1:  return (n + 7) / 8;
        default:                return n * element_size(dtype);
    }
}

static boat_tensor_t* new_record(const int64_t* shape, size_t ndim) {
    boat_tensor_t* t = (boat_tensor_t*)boat_calloc(sizeof(boat_tensor_t), BOAT_DEVICE_CPU);
    if (!t) return NULL;
    if (ndim > 0) {
        t->shape = (int64_t*)boat_malloc(sizeof(int64_t) * ndim, BOAT_DEVICE_CPU);
        if (!t->shape) {
            boat_free(t);
            return NULL;
        }
        memcpy(t->shape, shape, sizeof(int64_t) * ndim);
    }
    t->ndim = ndim;
    t->ref_count = 1;
    return t;
}

static boat_tensor_t* create_impl(const int64_t* shape, size_t ndim, boat_dtype_t dtype,
                                  boat_device_t device, bool zero) {
    if ((!shape && ndim > 0) || ndim > BOAT_MAX_DIMS) return NULL;
    size_t n = 1;
    for (size_t i = 0; i < ndim; ++i) {
        if (shape[i] < 0) return NULL;
        n *= (size_t)shape[i];
    }
    size_t nbytes = packed_bytes(dtype, n);
    if (nbytes == 0) return NULL;          /* the reference's allocator refuses 0 bytes (memory.c:48-50) */
    boat_tensor_t* t = new_record(shape, ndim);
    if (!t) return NULL;
    t->dtype = dtype;
    t->device = device;
    t->nelements = n;
    t->nbytes = nbytes;
    t->is_contiguous = true;
    t->data = boat_memory_allocate_device(nbytes, device, NULL, 0);
    if (!t->data) {
        boat_free(t->shape);
        boat_free(t);
        return NULL;
    }
    if (zero) boat_memory_set(t->data, 0, nbytes, device);
    return t;
}

boat_tensor_t* boat_tensor_adopt_device(const int64_t* shape, size_t ndim, boat_dtype_t dtype, void* device_data) {
    if (!device_data || (!shape && ndim > 0) || ndim > BOAT_MAX_DIMS) return NULL;
    size_t n = 1;
    for (size_t i = 0; i < ndim; ++i) {
        if (shape[i] < 0) return NULL;
        n *= (size_t)shape[i];
    }
    boat_tensor_t* t = new_record(shape, ndim);
    if (!t) return NULL;
    t->dtype = dtype;
    t->device = BOAT_DEVICE_CUDA;
    t->nelements = n;
    t->nbytes = packed_bytes(dtype, n);
    t->is_contiguous = true;
    t->data = device_data;
    return t;
}

boat_tensor_t* boat_tensor_create(const int64_t* shape, size_t ndim, boat_dtype_t dtype, boat_device_t device) {
    return create_impl(shape, ndim, dtype, device, true);
}

boat_tensor_t* boat_tensor_create_uninit(const int64_t* shape, size_t ndim, boat_dtype_t dtype,
                                         boat_device_t device) {
    return create_impl(shape, ndim, dtype, device, false);
}

boat_tensor_t* boat_tensor_from_data(const int64_t* shape, size_t ndim, boat_dtype_t dtype, const void* data) {
    boat_tensor_t* t = create_impl(shape, ndim, dtype, BOAT_DEVICE_CPU, data == NULL);
    if (t && data) memcpy(t->data, data, t->nbytes);
    return t;
}

boat_tensor_t* boat_tensor_create_like(const boat_tensor_t* other) {
    if (!other) return NULL;
    return boat_tensor_create(other->shape, other->ndim, other->dtype, other->device);
}

void boat_tensor_ref(boat_tensor_t* t) {
    if (t) t->ref_count++;
}

void boat_tensor_free(boat_tensor_t* t) {
    if (!t) return;
    if (--t->ref_count != 0) return;
    boat_tensor_t* parent = t->parent;
    if (!t->is_view && t->data) boat_memory_free_device(t->data, t->device);
    boat_free(t->shape);
    boat_free(t);
    if (parent) boat_tensor_free(parent);
}

void boat_tensor_unref(boat_tensor_t* t) { boat_tensor_free(t); }

const int64_t* boat_tensor_shape(const boat_tensor_t* t) { return t ? t->shape : NULL; }
size_t boat_tensor_ndim(const boat_tensor_t* t) { return t ? t->ndim : 0; }
boat_dtype_t boat_tensor_dtype(const boat_tensor_t* t) { return t ? t->dtype : BOAT_DTYPE_FLOAT32; }
boat_device_t boat_tensor_device(const boat_tensor_t* t) { return t ? t->device : BOAT_DEVICE_CPU; }
size_t boat_tensor_nbytes(const boat_tensor_t* t) { return t ? t->nbytes : 0; }
size_t boat_tensor_nelements(const boat_tensor_t* t) { return t ? t->nelements : 0; }
bool boat_tensor_is_contiguous(const boat_tensor_t* t) { return t ? t->is_contiguous : false; }
void* boat_tensor_data(const boat_tensor_t* t) { return t ? t->data : NULL; }
const void* boat_tensor_const_data(const boat_tensor_t* t) { return t ? t->data : NULL; }

size_t boat_dtype_size(boat_dtype_t dtype) { return element_size(dtype); }

const char* boat_dtype_name(boat_dtype_t dtype) {
    static const char* names[BOAT_DTYPE_COUNT] = {
        "float64", "float32", "float16", "float8", "float4", "int64", "int32", "uint8",
        "bits2", "bits1", "bool", "bfloat16"};
    return ((int)dtype >= 0 && dtype < BOAT_DTYPE_COUNT) ? names[dtype] : "unknown";
}

static boat_tensor_t* make_view(boat_tensor_t* parent, void* data, const int64_t* shape, size_t ndim,
                                size_t nelements, size_t nbytes) {
    boat_tensor_t* v = new_record(shape, ndim);
    if (!v) return NULL;
    v->dtype = parent->dtype;
    v->device = parent->device;
    v->data = data;
    v->nelements = nelements;
    v->nbytes = nbytes;
    v->is_contiguous = false;      /* the reference marks every view so (tensor.c:291, :436) */
    v->is_view = true;
    v->parent = parent;
    boat_tensor_ref(parent);
    return v;
}

boat_tensor_t* boat_tensor_reshape(const boat_tensor_t* tensor, const int64_t* new_shape, size_t new_ndim) {
    if (!tensor || !new_shape || new_ndim > BOAT_MAX_DIMS) return NULL;
    size_t n = 1;
    for (size_t i = 0; i < new_ndim; ++i) n *= (size_t)new_shape[i];
    if (n != tensor->nelements) {
        fprintf(stderr, "Error: Reshape element count mismatch: %zu != %zu\n", n, tensor->nelements);
        return NULL;
    }
    return make_view((boat_tensor_t*)tensor, tensor->data, new_shape, new_ndim, n, tensor->nbytes);
}

boat_tensor_t* boat_tensor_window(boat_tensor_t* parent, size_t offset_bytes, const int64_t* shape, size_t ndim) {
    if (!parent || !shape) return NULL;
    size_t n = 1;
    for (size_t i = 0; i < ndim; ++i) n *= (size_t)shape[i];
    size_t nbytes = n * element_size(parent->dtype);
    if (offset_bytes + nbytes > parent->nbytes) return NULL;
    boat_tensor_t* v = make_view(parent, (char*)parent->data + offset_bytes, shape, ndim, n, nbytes);
    if (v) v->is_contiguous = true;
    return v;
}

boat_tensor_t* boat_tensor_slice(const boat_tensor_t* tensor, const size_t* start, const size_t* end,
                                 const size_t* step) {
    if (!tensor || !start || !end) return NULL;
    size_t ndim = tensor->ndim;
    if (ndim == 0) {
        fprintf(stderr, "Error: Cannot slice scalar tensor\n");
        return NULL;
    }
    int64_t shape[BOAT_MAX_DIMS];
    for (size_t i = 0; i < ndim; ++i) {
        size_t st = step ? step[i] : 1, dim = (size_t)tensor->shape[i];
        if (st == 0) {
            fprintf(stderr, "Error: Step cannot be zero\n");
            return NULL;
        }
        if (start[i] >= dim || end[i] > dim || start[i] >= end[i]) {
            fprintf(stderr, "Error: Invalid slice range for dimension %zu: [%zu, %zu) (dim size: %zu)\n",
                    i, start[i], end[i], dim);
            return NULL;
        }
        if (st != 1) {
            fprintf(stderr, "Error: Non-unit step slicing not yet implemented\n");
            return NULL;
        }
        shape[i] = (int64_t)(end[i] - start[i]);
    }
    if (!tensor->is_contiguous) {
        fprintf(stderr, "Error: Slicing non-contiguous tensors not supported\n");
        return NULL;
    }
    size_t offset = 0, stride = 1, n = 1;
    for (size_t k = ndim; k-- > 0;) {
        offset += start[k] * stride;
        stride *= (size_t)tensor->shape[k];
        n *= (size_t)shape[k];
    }
    size_t es = element_size(tensor->dtype);
    return make_view((boat_tensor_t*)tensor, (char*)tensor->data + offset * es, shape, ndim, n, n * es);
}

boat_tensor_t* boat_tensor_to_device(const boat_tensor_t* tensor, boat_device_t dev) {
    if (!tensor) return NULL;
    boat_tensor_t* out = create_impl(tensor->shape, tensor->ndim, tensor->dtype, dev, false);
    if (!out) return NULL;
    boat_memory_copy(out->data, tensor->data, tensor->nbytes, dev, tensor->device);
    return out;
}
