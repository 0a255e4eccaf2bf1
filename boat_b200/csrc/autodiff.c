/* autodiff.c - reverse-mode differentiation through the attention layer and the ops next to it.
 *
 * The slice of the reference's src/autodiff.c that an encoder block uses: variables
 * (:24-31, :138-253), boat_variable_backward (:299-455), the element-wise ops add / sub / mul
 * (:466-485, backward :1002-1180), matmul (:494-499, :1454-1496), the dense-layer op (:563-567,
 * :2640-2672) and the attention op (:569-572, :2388-2532).  Every op works on whatever device
 * its tensors live on: with CUDA tensors a whole graph stays in HBM between layers.
 * The reference records ops in a general graph container; reverse mode over these ops only
 * ever walks from an output to the op that made it, so a variable here carries a pointer to
 * that op record and nothing else.  Input variables are borrowed, as in the reference: keep
 * them alive until backward has run. */
#include "core/boat_internal.h"
#include <boat/autodiff.h>
#include <boat/ops.h>
#include <boat/layers.h>
#include <boat/layers/attention.h>

typedef enum { OP_ADD, OP_SUB, OP_MUL, OP_MATMUL, OP_DENSE, OP_ATTENTION } op_type_t;

typedef struct {
    op_type_t type;
    boat_variable_t* inputs[3];       /* a, b | input | query, key, value */
    int n_inputs;
    void* layer;                      /* dense or attention layer; borrowed, never freed from here */
} op_record_t;

struct boat_variable_t {
    boat_tensor_t* data;
    boat_tensor_t* grad;
    bool requires_grad;
    op_record_t* producer;            /* NULL for leaves; owned by this variable */
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

/* grad += g where g is a fresh tensor this function consumes; the first contribution becomes
 * the gradient itself, as compute_backward_matmul does (autodiff.c:1470-1475). */
static void accumulate_owned(boat_variable_t* v, boat_tensor_t* g) {
    if (!g) return;
    if (!v->grad && g->nelements == v->data->nelements) {
        v->grad = g;
        return;
    }
    accumulate(v, g);
    boat_tensor_unref(g);
}

static void backward_attention(op_record_t* op, const boat_tensor_t* grad_output) {
    boat_tensor_t* g[3] = {NULL, NULL, NULL};
    if (!boat_attention_backward((boat_attention_t*)op->layer, grad_output, &g[0], &g[1], &g[2])) return;
    for (int i = 0; i < 3; ++i)
        if (g[i] && op->inputs[i] && op->inputs[i]->requires_grad && !accumulate(op->inputs[i], g[i])) break;
    for (int i = 0; i < 3; ++i)
        if (g[i]) boat_tensor_unref(g[i]);
}

static void backward_op(op_record_t* op, const boat_tensor_t* g) {
    boat_variable_t *a = op->inputs[0], *b = op->inputs[1];
    switch (op->type) {
    case OP_ADD:                                   /* da = g, db = g (autodiff.c:1002-1064) */
        if (a->requires_grad) accumulate(a, g);
        if (b->requires_grad) accumulate(b, g);
        break;
    case OP_SUB:                                   /* da = g, db = -g (autodiff.c:1066-1113) */
        if (a->requires_grad) accumulate(a, g);
        if (b->requires_grad) accumulate_owned(b, boat_mul_scalar(g, -1.0));
        break;
    case OP_MUL:                                   /* da = g*b, db = g*a (autodiff.c:1115-1180) */
        if (a->requires_grad) accumulate_owned(a, boat_mul(g, b->data));
        if (b->requires_grad) accumulate_owned(b, boat_mul(g, a->data));
        break;
    case OP_MATMUL:                                /* dA = g.B^T, dB = A^T.g (autodiff.c:1454-1496) */
        if (a->requires_grad) {
            boat_tensor_t* bt = boat_transpose(b->data, 0, 1);
            if (bt) {
                accumulate_owned(a, boat_matmul(g, bt));
                boat_tensor_unref(bt);
            }
        }
        if (b->requires_grad) {
            boat_tensor_t* at = boat_transpose(a->data, 0, 1);
            if (at) {
                accumulate_owned(b, boat_matmul(at, g));
                boat_tensor_unref(at);
            }
        }
        break;
    case OP_DENSE: {                               /* the layer keeps dW, db; dx comes back (autodiff.c:2640-2672) */
        boat_tensor_t* gi = boat_dense_layer_backward((boat_dense_layer_t*)op->layer, g);
        if (gi && a->requires_grad) accumulate_owned(a, gi);
        else if (gi) boat_tensor_unref(gi);
        break;
    }
    case OP_ATTENTION:
        backward_attention(op, g);
        break;
    }
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
        backward_op(v->producer, seed);
        /* Continue into inputs that were themselves computed (autodiff.c:431-450), with the
         * gradient they have accumulated so far.  The reference walks the input list as it is,
         * so a computed variable that is passed twice to one op is walked twice; here each
         * distinct input is walked once. */
        for (int i = 0; i < v->producer->n_inputs; ++i) {
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

/* Output variable of an op over `out` (consumed); records the op when a gradient is wanted
 * (create_operation, autodiff.c:2070-2160). */
static boat_variable_t* make_result(boat_tensor_t* out, op_type_t type, const boat_variable_t* const* inputs,
                                    int n_inputs, const void* layer) {
    if (!out) return NULL;
    bool requires_grad = false;
    for (int i = 0; i < n_inputs; ++i) requires_grad = requires_grad || inputs[i]->requires_grad;
    boat_variable_t* v = boat_variable_create(out, requires_grad);
    boat_tensor_unref(out);                       /* the variable holds the only reference now */
    if (!v || !requires_grad) return v;
    op_record_t* op = (op_record_t*)boat_calloc(sizeof *op, BOAT_DEVICE_CPU);
    if (!op) {
        boat_variable_free(v);
        return NULL;
    }
    op->type = type;
    op->n_inputs = n_inputs;
    for (int i = 0; i < n_inputs; ++i) op->inputs[i] = (boat_variable_t*)inputs[i];
    op->layer = (void*)layer;
    v->producer = op;
    return v;
}

boat_variable_t* boat_var_add(const boat_variable_t* a, const boat_variable_t* b) {
    if (!a || !b) return NULL;
    const boat_variable_t* in[2] = {a, b};
    return make_result(boat_add(a->data, b->data), OP_ADD, in, 2, NULL);
}

boat_variable_t* boat_var_sub(const boat_variable_t* a, const boat_variable_t* b) {
    if (!a || !b) return NULL;
    const boat_variable_t* in[2] = {a, b};
    return make_result(boat_sub(a->data, b->data), OP_SUB, in, 2, NULL);
}

boat_variable_t* boat_var_mul(const boat_variable_t* a, const boat_variable_t* b) {
    if (!a || !b) return NULL;
    const boat_variable_t* in[2] = {a, b};
    return make_result(boat_mul(a->data, b->data), OP_MUL, in, 2, NULL);
}

boat_variable_t* boat_var_matmul(const boat_variable_t* a, const boat_variable_t* b) {
    if (!a || !b) return NULL;
    const boat_variable_t* in[2] = {a, b};
    return make_result(boat_matmul(a->data, b->data), OP_MATMUL, in, 2, NULL);
}

boat_variable_t* boat_var_dense(const boat_variable_t* input, const struct boat_dense_layer_t* layer) {
    if (!input || !layer) return NULL;
    const boat_variable_t* in[1] = {input};
    return make_result(boat_dense_layer_forward((boat_dense_layer_t*)layer, input->data), OP_DENSE, in, 1, layer);
}

boat_variable_t* boat_var_attention(const boat_variable_t* query, const boat_variable_t* key,
                                    const boat_variable_t* value, const struct boat_attention_t* attention,
                                    const boat_tensor_t* attention_mask) {
    if (!query || !key || !value || !attention) return NULL;
    const boat_variable_t* in[3] = {query, key, value};
    return make_result(boat_attention_forward((boat_attention_t*)attention, query->data, key->data, value->data,
                                              attention_mask),
                       OP_ATTENTION, in, 3, attention);
}
