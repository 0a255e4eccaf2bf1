/* ops.c - the stateless FP32 tensor operations around the attention layer, on the GPU.
 *
 * Covers what the reference's layer and autodiff call on this path: boat_matmul
 * (src/ops/linear.c:12-170), boat_transpose of the last two dimensions (linear.c:238-406),
 * boat_add / boat_mul for equal shapes and trailing-dimension broadcast
 * (src/ops/arithmetic.c:157-285), boat_add_ / boat_sub_ (arithmetic.c:362-422) and
 * boat_mul_scalar (arithmetic.c:425-484).  Operands on the host are staged through HBM
 * for the call; the result lives where the first operand lives. */
#include "../core/boat_internal.h"
#include <boat/ops.h>
#include <string.h>

typedef struct {
    float* p;
    bool owned;
} dev_buf_t;

static dev_buf_t to_dev(const boat_tensor_t* t) {
    dev_buf_t b = {NULL, false};
    if (t->device == BOAT_DEVICE_CUDA) {
        b.p = (float*)t->data;
        return b;
    }
    void* p = NULL;
    if (boat_report("device allocation", boat_cuda_malloc(&p, t->nbytes)) != 0) return b;
    if (boat_report("upload", boat_cuda_memcpy_h2d(p, t->data, t->nbytes)) != 0) {
        boat_cuda_free(p);
        return b;
    }
    b.p = (float*)p;
    b.owned = true;
    return b;
}

static dev_buf_t out_dev(const boat_tensor_t* t) {
    dev_buf_t b = {NULL, false};
    if (t->device == BOAT_DEVICE_CUDA) {
        b.p = (float*)t->data;
        return b;
    }
    void* p = NULL;
    if (boat_report("device allocation", boat_cuda_malloc(&p, t->nbytes)) == 0) {
        b.p = (float*)p;
        b.owned = true;
    }
    return b;
}

static void drop(dev_buf_t* b) {
    if (b->owned && b->p) boat_cuda_free(b->p);
    b->p = NULL;
}

/* Copies a device result back into a host tensor when needed, releases staging, and gives
 * back `out` or NULL (freeing it) according to rc. */
static boat_tensor_t* finish(boat_tensor_t* out, dev_buf_t* o, int rc, const char* what) {
    if (rc == 0 && o->owned) rc = boat_cuda_memcpy_d2h(out->data, o->p, out->nbytes);
    drop(o);
    if (boat_report(what, rc) != 0) {
        boat_tensor_free(out);
        return NULL;
    }
    return out;
}

static bool f32_pair(const boat_tensor_t* a, const boat_tensor_t* b) {
    return a && b && a->dtype == BOAT_DTYPE_FLOAT32 && b->dtype == BOAT_DTYPE_FLOAT32;
}

/* b equals a, or b's shape is the trailing part of a's shape. */
static bool trailing_match(const boat_tensor_t* a, const boat_tensor_t* b) {
    if (b->ndim > a->ndim) return false;
    for (size_t i = 0; i < b->ndim; ++i)
        if (b->shape[b->ndim - 1 - i] != a->shape[a->ndim - 1 - i]) return false;
    return true;
}

boat_tensor_t* boat_lincomb(const boat_tensor_t* a, float alpha, const boat_tensor_t* b, float beta);

static boat_tensor_t* binary(const boat_tensor_t* a, const boat_tensor_t* b, bool is_add) {
    if (is_add && a && b && a->dtype == BOAT_DTYPE_BFLOAT16 && b->dtype == BOAT_DTYPE_BFLOAT16 &&
        a->nelements == b->nelements)
        return boat_lincomb(a, 1.0f, b, 1.0f);
    if (!f32_pair(a, b)) return NULL;
    if (b->nelements > a->nelements) {           /* the larger operand leads; both ops commute */
        const boat_tensor_t* t = a;
        a = b;
        b = t;
    }
    if (!trailing_match(a, b)) return NULL;
    if (boat_report("CUDA start-up", boat_cuda_init(-1)) != 0) return NULL;
    boat_tensor_t* out = boat_tensor_create_uninit(a->shape, a->ndim, a->dtype, a->device);
    if (!out) return NULL;
    dev_buf_t da = to_dev(a), db = to_dev(b), dout = out_dev(out);
    int rc = 1;
    if (da.p && db.p && dout.p) {
        int64_t n = (int64_t)a->nelements, cols = (int64_t)b->nelements;
        if (cols == n)
            rc = is_add ? (boat_cuda_memcpy_d2d(dout.p, da.p, a->nbytes) || boat_cuda_axpy(dout.p, db.p, 1.0f, n))
                        : boat_cuda_mul(dout.p, da.p, db.p, n);
        else if (is_add)
            rc = boat_cuda_add_bias(dout.p, da.p, db.p, n / cols, cols);
        else {
            rc = 1;                              /* broadcast product is not on this path */
            fprintf(stderr, "boat_mul: broadcast shapes are not supported\n");
        }
    }
    drop(&da);
    drop(&db);
    return finish(out, &dout, rc, is_add ? "boat_add" : "boat_mul");
}

boat_tensor_t* boat_add(const boat_tensor_t* a, const boat_tensor_t* b) { return binary(a, b, true); }
boat_tensor_t* boat_mul(const boat_tensor_t* a, const boat_tensor_t* b) { return binary(a, b, false); }

static void inplace(boat_tensor_t* a, const boat_tensor_t* b, float alpha, const char* what) {
    if (!f32_pair(a, b) || a->nelements != b->nelements) return;   /* silently, as the reference */
    if (boat_report("CUDA start-up", boat_cuda_init(-1)) != 0) return;
    dev_buf_t da = to_dev(a), db = to_dev(b);
    int rc = 1;
    if (da.p && db.p) {
        rc = boat_cuda_axpy(da.p, db.p, alpha, (int64_t)a->nelements);
        if (rc == 0 && da.owned) rc = boat_cuda_memcpy_d2h(a->data, da.p, a->nbytes);
    }
    boat_report(what, rc);
    drop(&da);
    drop(&db);
}

void boat_add_(boat_tensor_t* a, const boat_tensor_t* b) { inplace(a, b, 1.0f, "boat_add_"); }
void boat_sub_(boat_tensor_t* a, const boat_tensor_t* b) { inplace(a, b, -1.0f, "boat_sub_"); }

boat_tensor_t* boat_mul_scalar(const boat_tensor_t* a, double scalar) {
    if (!a || a->dtype != BOAT_DTYPE_FLOAT32) return NULL;
    if (boat_report("CUDA start-up", boat_cuda_init(-1)) != 0) return NULL;
    boat_tensor_t* out = boat_tensor_create_uninit(a->shape, a->ndim, a->dtype, a->device);
    if (!out) return NULL;
    dev_buf_t da = to_dev(a), dout = out_dev(out);
    int rc = (da.p && dout.p) ? boat_cuda_scale(dout.p, da.p, (float)scalar, (int64_t)a->nelements) : 1;
    drop(&da);
    return finish(out, &dout, rc, "boat_mul_scalar");
}

boat_tensor_t* boat_matmul(const boat_tensor_t* a, const boat_tensor_t* b) {
    if (!f32_pair(a, b)) return NULL;
    if (a->ndim < 2 || a->ndim > 4 || b->ndim != a->ndim) return NULL;
    size_t nb = a->ndim - 2;
    int64_t batch = 1, shape[4];
    for (size_t i = 0; i < nb; ++i) {
        if (a->shape[i] != b->shape[i]) return NULL;
        batch *= a->shape[i];
        shape[i] = a->shape[i];
    }
    int64_t m = a->shape[nb], k = a->shape[nb + 1], n = b->shape[nb + 1];
    if (b->shape[nb] != k) return NULL;
    shape[nb] = m;
    shape[nb + 1] = n;
    if (boat_report("CUDA start-up", boat_cuda_init(-1)) != 0) return NULL;
    boat_tensor_t* out = boat_tensor_create_uninit(shape, a->ndim, a->dtype, a->device);
    if (!out) return NULL;
    dev_buf_t da = to_dev(a), db = to_dev(b), dout = out_dev(out);
    int rc = (da.p && db.p && dout.p) ? 0 : 1;
    for (int64_t i = 0; rc == 0 && i < batch; ++i)
        rc = boat_cuda_gemm(BOAT_MMA_FP32, 0, 0, m, n, k, da.p + i * m * k, k, db.p + i * k * n, n, BOAT_CUDA_F32,
                            dout.p + i * m * n, n, BOAT_CUDA_F32, NULL);
    drop(&da);
    drop(&db);
    return finish(out, &dout, rc, "boat_matmul");
}

boat_tensor_t* boat_transpose(const boat_tensor_t* a, int dim0, int dim1) {
    if (!a || a->dtype != BOAT_DTYPE_FLOAT32) return NULL;
    int nd = (int)a->ndim;
    if (dim0 < 0 || dim1 < 0 || dim0 >= nd || dim1 >= nd) return NULL;
    int lo = dim0 < dim1 ? dim0 : dim1, hi = dim0 < dim1 ? dim1 : dim0;
    if (lo != hi && !(lo == nd - 2 && hi == nd - 1)) {
        fprintf(stderr, "boat_transpose: only the last two dimensions can be swapped\n");
        return NULL;
    }
    int64_t shape[BOAT_MAX_DIMS];
    memcpy(shape, a->shape, sizeof(int64_t) * a->ndim);
    shape[dim0] = a->shape[dim1];
    shape[dim1] = a->shape[dim0];
    if (boat_report("CUDA start-up", boat_cuda_init(-1)) != 0) return NULL;
    boat_tensor_t* out = boat_tensor_create_uninit(shape, a->ndim, a->dtype, a->device);
    if (!out) return NULL;
    dev_buf_t da = to_dev(a), dout = out_dev(out);
    int rc = 1;
    if (da.p && dout.p) {
        if (lo == hi) {
            rc = boat_cuda_memcpy_d2d(dout.p, da.p, a->nbytes);
        } else {
            int64_t rows = a->shape[nd - 2], cols = a->shape[nd - 1];
            int64_t batch = (int64_t)a->nelements / (rows * cols);
            rc = 0;
            for (int64_t b0 = 0; rc == 0 && b0 < batch; b0 += 65535) {
                int64_t nbatch = batch - b0 < 65535 ? batch - b0 : 65535;
                rc = boat_cuda_transpose(dout.p + b0 * rows * cols, da.p + b0 * rows * cols, nbatch, rows, cols);
            }
        }
    }
    drop(&da);
    return finish(out, &dout, rc, "boat_transpose");
}

/* ---- GELU (exact erf form).  The reference declares boat_gelu and leaves it a stub returning
 * NULL (src/ops/activation.c:298-302); FP32 and BF16 tensors, host or device. ---- */
#include "../core/stage.h"
#include <boat_b200.h>

static boat_tensor_t* gelu_impl(const boat_tensor_t* x, const boat_tensor_t* grad) {
    if (!x || !boat_dtype_supported(x->dtype)) return NULL;
    if (grad && (grad->nelements != x->nelements || grad->dtype != x->dtype)) return NULL;
    if (boat_report("CUDA start-up", boat_cuda_init(-1)) != 0) return NULL;
    const int type = boat_storage_of(x->dtype);
    bool xo = false, go = false;
    void* dx = boat_stage_in(x, type, &xo);
    void* dg = grad ? boat_stage_in(grad, type, &go) : NULL;
    void* dy = boat_dev_alloc(x->nelements * boat_storage_size(type));
    boat_tensor_t* out = NULL;
    if (dx && dy && (!grad || dg)) {
        int rc = grad ? boat_cuda_gelu_bwd(dy, dg, dx, type, (int64_t)x->nelements)
                      : boat_cuda_gelu_fwd(dy, dx, type, (int64_t)x->nelements);
        if (boat_report("GELU", rc) == 0) out = boat_emit_out_take(x->shape, x->ndim, x, &dy, type);
    }
    boat_dev_free(dy);
    if (xo) boat_dev_free(dx);
    if (go) boat_dev_free(dg);
    return out;
}

boat_tensor_t* boat_lincomb(const boat_tensor_t* a, float alpha, const boat_tensor_t* b, float beta) {
    if (!a || !b || a->dtype != b->dtype || a->nelements != b->nelements || !boat_dtype_supported(a->dtype)) return NULL;
    if (boat_report("CUDA start-up", boat_cuda_init(-1)) != 0) return NULL;
    const int type = boat_storage_of(a->dtype);
    bool ao = false, bo = false;
    void* da = boat_stage_in(a, type, &ao);
    void* db = boat_stage_in(b, type, &bo);
    void* dy = boat_dev_alloc(a->nelements * boat_storage_size(type));
    boat_tensor_t* out = NULL;
    if (da && db && dy &&
        boat_report("lincomb", boat_cuda_lincomb(dy, da, alpha, db, beta, type, (int64_t)a->nelements)) == 0)
        out = boat_emit_out_take(a->shape, a->ndim, a, &dy, type);
    boat_dev_free(dy);
    if (ao) boat_dev_free(da);
    if (bo) boat_dev_free(db);
    return out;
}

boat_tensor_t* boat_sub(const boat_tensor_t* a, const boat_tensor_t* b) {
    if (!a || !b || a->ndim != b->ndim) return NULL;
    for (size_t i = 0; i < a->ndim; ++i)
        if (a->shape[i] != b->shape[i]) return NULL;
    return boat_lincomb(a, 1.0f, b, -1.0f);
}

boat_tensor_t* boat_gelu(const boat_tensor_t* a) { return gelu_impl(a, NULL); }

boat_tensor_t* boat_gelu_backward(const boat_tensor_t* grad_output, const boat_tensor_t* input) {
    if (!grad_output) return NULL;
    return gelu_impl(input, grad_output);
}
