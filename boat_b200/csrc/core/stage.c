/* stage.c - see stage.h. */
#include "stage.h"
#include <stdlib.h>
#include <strings.h>

int boat_storage_of(boat_dtype_t dt) { return dt == BOAT_DTYPE_BFLOAT16 ? BOAT_CUDA_BF16 : BOAT_CUDA_F32; }
size_t boat_storage_size(int type) { return type == BOAT_CUDA_BF16 ? 2 : 4; }
bool boat_dtype_supported(boat_dtype_t dt) { return dt == BOAT_DTYPE_FLOAT32 || dt == BOAT_DTYPE_BFLOAT16; }

void* boat_dev_alloc(size_t bytes) {
    void* p = NULL;
    if (boat_report("device allocation", boat_cuda_malloc(&p, bytes)) != 0) return NULL;
    return p;
}

void boat_dev_free(void* p) {
    if (p) boat_report("device free", boat_cuda_free(p));
}

void* boat_stage_in(const boat_tensor_t* t, int type, bool* owned) {
    int have = boat_storage_of(t->dtype);
    size_t n = t->nelements;
    *owned = false;
    if (t->device == BOAT_DEVICE_CUDA && have == type) return t->data;
    *owned = true;
    void* raw = t->data;
    void* tmp = NULL;
    if (t->device != BOAT_DEVICE_CUDA) {
        tmp = boat_dev_alloc(n * boat_storage_size(have));
        if (!tmp) return NULL;
        if (boat_report("upload", boat_cuda_memcpy_h2d(tmp, t->data, n * boat_storage_size(have))) != 0) {
            boat_dev_free(tmp);
            return NULL;
        }
        if (have == type) return tmp;
        raw = tmp;
    }
    void* out = boat_dev_alloc(n * boat_storage_size(type));
    if (out && boat_report("cast", boat_cuda_cast(out, type, raw, have, (int64_t)n)) != 0) {
        boat_dev_free(out);
        out = NULL;
    }
    boat_dev_free(tmp);
    return out;
}

boat_tensor_t* boat_emit_out(const int64_t* shape, size_t ndim, const boat_tensor_t* like, void* src, int type) {
    boat_tensor_t* out = boat_tensor_create_uninit(shape, ndim, like->dtype, like->device);
    if (!out) return NULL;
    int want = boat_storage_of(like->dtype);
    size_t n = out->nelements;
    int rc;
    if (like->device == BOAT_DEVICE_CUDA) {
        rc = boat_cuda_cast(out->data, want, src, type, (int64_t)n);
    } else if (want == type) {
        rc = boat_cuda_memcpy_d2h(out->data, src, n * boat_storage_size(type));
    } else {
        void* tmp = boat_dev_alloc(n * boat_storage_size(want));
        rc = tmp ? boat_cuda_cast(tmp, want, src, type, (int64_t)n) : 1;
        if (rc == 0) rc = boat_cuda_memcpy_d2h(out->data, tmp, n * boat_storage_size(want));
        boat_dev_free(tmp);
    }
    if (boat_report("result transfer", rc) != 0) {
        boat_tensor_free(out);
        return NULL;
    }
    return out;
}

boat_tensor_t* boat_emit_out_take(const int64_t* shape, size_t ndim, const boat_tensor_t* like, void** src, int type) {
    if (like->device == BOAT_DEVICE_CUDA && boat_storage_of(like->dtype) == type && *src) {
        boat_tensor_t* out = boat_tensor_adopt_device(shape, ndim, like->dtype, *src);
        if (out) *src = NULL;
        return out;
    }
    return boat_emit_out(shape, ndim, like, *src, type);
}

int boat_default_mma(boat_dtype_t dt) {
    if (dt == BOAT_DTYPE_BFLOAT16) return BOAT_MMA_BF16;
    const char* e = getenv("BOAT_MMA");
    if (e && !strcasecmp(e, "tf32")) return BOAT_MMA_TF32;
    return BOAT_MMA_FP32;
}
