/* autodiff.c - reverse-mode differentiation through the attention layer.
 *
 * The slice of the reference's src/autodiff.c that the attention path uses: variables
 * (:24-31, :138-253), boat_variable_backward (:299-455) and the attention op
 * (:2388-2532).  The reference records ops in a general graph container; reverse mode
 * over this path only ever walks from an output to the op that made it, so a variable
 * here carries a pointer to that op record and nothing else.  Input variables are
 * borrowed, as in the reference: keep them alive until backward has run. */
#include "core/boat_internal.h"
#include <boat/autodiff.h>
#include <boat/ops.h>
#include <boat/layers/attention.h>

typedef struct {
    boat_variable_t* inputs[3];       /* query, key, value */
    boat_attention_t* layer;          /* borrowed: never freed from here */
} attention_op_t;

struct boat_variable_t {
    boat_tensor_t* data;
    boat_tensor_t* grad;
    bool requires_grad;
    attention_op_t* producer;         /* NULL for leaves; owned by this variable */
};

boat_variable_t* boat_variable_create(boat_tensor_t* tensor, bool requires_grad) {
    if (!tensor) return NULL;
    boat_variable_t* v = (boat_variable_t*)boat_calloc(sizeof *v, BOAT_DEVICE_CPU);
    if (!v) return NULL;
    v->data = tensor;
    boat_tensor_ref(tensor);
    v->requires_grad = requires_grad;
    return v;
}

boat_variable_t* boat_variable_create_with_shape(const int64_t* shape, size_t ndim, boat_dtype_t dtype,
                                                 bool requires_grad) {
    boat_tensor_t* t = boat_tensor_create(shape, ndim, dtype, BOAT_DEVICE_CPU);
    if (!t) return NULL;
    boat_variable_t* v = boat_variable_create(t, requires_grad);
    boat_tensor_unref(t);      /* the variable's own reference keeps it (the reference leaked this one) */
    return v;
}

void boat_variable_free(const boat_variable_t* variable) {
    boat_variable_t* v = (boat_variable_t*)variable;
    if (!v) return;
    if (v->grad) boat_tensor_unref(v->grad);
    if (v->data) boat_tensor_unref(v->data);
    if (v->producer) boat_free(v->producer);
    boat_free(v);
}

boat_tensor_t* boat_variable_data(const boat_variable_t* v) { return v ? v->data : NULL; }
boat_tensor_t* boat_variable_grad(const boat_variable_t* v) { return v ? v->grad : NULL; }
bool boat_variable_requires_grad(const boat_variable_t* v) { return v ? v->requires_grad : false; }

void boat_variable_set_requires_grad(boat_variable_t* v, bool requires_grad) {
    if (v) v->requires_grad = requires_grad;
}

void boat_variable_zero_grad(boat_variable_t* v) {
    if (v && v->grad) {
        boat_tensor_unref(v->grad);
        v->grad = NULL;
    }
}

/* grad += g, creating a zero grad of the data's shape first (autodiff.c:2482-2494). */
static bool accumulate(boat_variable_t* v, const boat_tensor_t* g) {
    if (!v->grad) {
        v->grad = boat_tensor_create_like(v->data);
        if (!v->grad) return false;
    }
    boat_add_(v->grad, g);
    return true;
}

static void backward_attention(attention_op_t* op, const boat_tensor_t* grad_output) {
    boat_tensor_t* g[3] = {NULL, NULL, NULL};
    if (!boat_attention_backward(op->layer, grad_output, &g[0], &g[1], &g[2])) return;
    for (int i = 0; i < 3; ++i)
        if (g[i] && op->inputs[i] && op->inputs[i]->requires_grad && !accumulate(op->inputs[i], g[i])) break;
    for (int i = 0; i < 3; ++i)
        if (g[i]) boat_tensor_unref(g[i]);
}

void boat_variable_backward(boat_variable_t* v, boat_tensor_t* grad_output) {
    if (!v || !v->requires_grad) return;
    boat_tensor_t* seed = grad_output;
    if (!seed) {
        /* no upstream gradient: ones of the output's shape (autodiff.c:311-338) */
        if (v->data->dtype != BOAT_DTYPE_FLOAT32) return;
        boat_tensor_t* host = boat_tensor_create(v->data->shape, v->data->ndim, BOAT_DTYPE_FLOAT32, BOAT_DEVICE_CPU);
        if (!host) return;
        float* p = (float*)host->data;
        for (size_t i = 0; i < host->nelements; ++i) p[i] = 1.0f;
        seed = host;
        if (v->data->device == BOAT_DEVICE_CUDA) {
            seed = boat_tensor_to_device(host, BOAT_DEVICE_CUDA);
            boat_tensor_unref(host);
            if (!seed) return;
        }
    }
    if (!v->producer) {
        accumulate(v, seed);                                   /* leaf (autodiff.c:346-361) */
    } else {
        backward_attention(v->producer, seed);
        /* continue into inputs that were themselves computed (autodiff.c:431-450) */
        for (int i = 0; i < 3; ++i) {
            boat_variable_t* in = v->producer->inputs[i];
            bool seen = false;
            for (int j = 0; j < i; ++j) seen = seen || v->producer->inputs[j] == in;
            if (in && !seen && in->requires_grad && in->grad && in->producer) {
                boat_tensor_ref(in->grad);
                boat_variable_backward(in, in->grad);
                boat_tensor_unref(in->grad);
            }
        }
    }
    if (seed != grad_output) boat_tensor_unref(seed);
}

void boat_variable_backward_full(const boat_variable_t* v) { boat_variable_backward((boat_variable_t*)v, NULL); }

boat_variable_t* boat_var_attention(const boat_variable_t* query, const boat_variable_t* key,
                                    const boat_variable_t* value, const struct boat_attention_t* attention,
                                    const boat_tensor_t* attention_mask) {
    if (!query || !key || !value || !attention) return NULL;
    bool requires_grad = query->requires_grad || key->requires_grad || value->requires_grad;
    boat_tensor_t* out = boat_attention_forward((boat_attention_t*)attention, query->data, key->data, value->data,
                                                attention_mask);
    if (!out) return NULL;
    boat_variable_t* v = boat_variable_create(out, requires_grad);
    boat_tensor_unref(out);                       /* the variable holds the only reference now */
    if (!v) return NULL;
    if (requires_grad) {
        attention_op_t* op = (attention_op_t*)boat_calloc(sizeof *op, BOAT_DEVICE_CPU);
        if (!op) {
            boat_variable_free(v);
            return NULL;
        }
        op->inputs[0] = (boat_variable_t*)query;
        op->inputs[1] = (boat_variable_t*)key;
        op->inputs[2] = (boat_variable_t*)value;
        op->layer = (boat_attention_t*)attention;
        v->producer = op;
    }
    return v;
}
