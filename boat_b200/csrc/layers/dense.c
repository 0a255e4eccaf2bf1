/* dense.c - fully connected layer y = x.W + b on the GPU, the MLP half of the encoder block.
 *
 * Same behaviour as the reference's src/layers/dense.c: weight [in,out] Xavier-uniform from
 * rand() (:57-63), zero bias, gradient tensors created zeroed with the layer (:82-112);
 * forward takes 2-D input only and keeps a reference to it (:135-185); backward returns
 * dX = dY.W^T and ACCUMULATES dW += X^T.dY, db += sum_rows dY (:187-297); update is
 * p -= lr*g followed by clearing the gradients (:299-327).  The contractions are the same
 * tcgen05 / CUDA-core GEMMs the attention projections use. */
#include "../core/stage.h"
#include <boat/layers.h>
#include <boat/ops.h>
#include <boat_b200.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

struct boat_dense_layer_t {
    size_t in_features, out_features;
    bool use_bias;
    boat_tensor_t *weight, *bias, *grad_weight, *grad_bias;
    boat_tensor_t* cache_input;
};

boat_dense_layer_t* boat_dense_layer_create(size_t input_features, size_t output_features, bool use_bias) {
    if (input_features == 0 || output_features == 0) return NULL;
    boat_dense_layer_t* l = (boat_dense_layer_t*)boat_calloc(sizeof *l, BOAT_DEVICE_CPU);
    if (!l) return NULL;
    l->in_features = input_features;
    l->out_features = output_features;
    l->use_bias = use_bias;
    const int64_t wshape[2] = {(int64_t)input_features, (int64_t)output_features}, bshape[1] = {(int64_t)output_features};
    l->weight = boat_tensor_create(wshape, 2, BOAT_DTYPE_FLOAT32, BOAT_DEVICE_CPU);
    l->grad_weight = boat_tensor_create(wshape, 2, BOAT_DTYPE_FLOAT32, BOAT_DEVICE_CPU);
    if (use_bias) {
        l->bias = boat_tensor_create(bshape, 1, BOAT_DTYPE_FLOAT32, BOAT_DEVICE_CPU);
        l->grad_bias = boat_tensor_create(bshape, 1, BOAT_DTYPE_FLOAT32, BOAT_DEVICE_CPU);
    }
    if (!l->weight || !l->grad_weight || (use_bias && (!l->bias || !l->grad_bias))) {
        boat_dense_layer_free(l);
        return NULL;
    }
    float* w = (float*)l->weight->data;
    float bound = sqrtf(2.0f / (float)(input_features + output_features));
    for (size_t i = 0; i < l->weight->nelements; ++i) w[i] = ((float)rand() / RAND_MAX) * 2.0f * bound - bound;
    return l;
}

void boat_dense_layer_free(boat_dense_layer_t* l) {
    if (!l) return;
    boat_tensor_t* all[5] = {l->weight, l->bias, l->grad_weight, l->grad_bias, l->cache_input};
    for (int i = 0; i < 5; ++i)
        if (all[i]) boat_tensor_free(all[i]);
    boat_free(l);
}

boat_tensor_t* boat_dense_layer_forward(boat_dense_layer_t* l, const boat_tensor_t* input) {
    if (!l || !input) return NULL;
    boat_tensor_ref((boat_tensor_t*)input);
    if (l->cache_input) boat_tensor_unref(l->cache_input);
    l->cache_input = (boat_tensor_t*)input;
    if (input->ndim != 2 || input->shape[1] != (int64_t)l->in_features || !boat_dtype_supported(input->dtype)) return NULL;
    if (boat_report("CUDA start-up", boat_cuda_init(-1)) != 0) return NULL;
    const int mma = boat_default_mma(input->dtype), type = boat_storage_of(input->dtype);
    const int64_t N = input->shape[0], I = (int64_t)l->in_features, O = (int64_t)l->out_features;
    bool xo = false, wo = false, bo = false;
    void* dx = boat_stage_in(input, type, &xo);
    void* dw = boat_stage_in(l->weight, type, &wo);
    float* db = l->bias ? (float*)boat_stage_in(l->bias, BOAT_CUDA_F32, &bo) : NULL;
    void* dy = boat_dev_alloc((size_t)N * O * boat_storage_size(type));
    boat_tensor_t* out = NULL;
    const int64_t oshape[2] = {N, O};
    if (dx && dw && dy && (!l->bias || db) &&
        boat_report("dense forward", boat_cuda_gemm(mma, 0, 0, N, O, I, dx, I, dw, O, type, dy, O, type, db)) == 0)
        out = boat_emit_out_take(oshape, 2, input, &dy, type);
    boat_dev_free(dy);
    if (xo) boat_dev_free(dx);
    if (wo) boat_dev_free(dw);
    if (bo) boat_dev_free(db);
    return out;
}

BOAT_NOINLINE boat_tensor_t* boat_dense_layer_backward(boat_dense_layer_t* l, const boat_tensor_t* grad_output) {
    if (!l || !grad_output || !l->cache_input) return NULL;
    const boat_tensor_t* x = l->cache_input;
    if (x->ndim != 2 || grad_output->ndim != 2) {
        fprintf(stderr, "Error: Dense layer backward expects 2D tensors\n");
        return NULL;
    }
    const int64_t N = x->shape[0], I = (int64_t)l->in_features, O = (int64_t)l->out_features;
    if (x->shape[1] != I || grad_output->shape[1] != O || grad_output->shape[0] != N ||
        !boat_dtype_supported(grad_output->dtype)) {
        fprintf(stderr, "Error: Dense layer backward shape mismatch\n");
        return NULL;
    }
    const int mma = boat_default_mma(x->dtype), type = boat_storage_of(x->dtype);
    bool xo = false, go = false, wo = false;
    void* dx = boat_stage_in(x, type, &xo);
    void* dg = boat_stage_in(grad_output, type, &go);
    void* dw = boat_stage_in(l->weight, type, &wo);
    void* d_dx = boat_dev_alloc((size_t)N * I * boat_storage_size(type));
    float* d_dw = (float*)boat_dev_alloc((size_t)I * O * sizeof(float));
    float* d_db = l->bias ? (float*)boat_dev_alloc((size_t)O * sizeof(float)) : NULL;
    boat_tensor_t* out = NULL;
    if (dx && dg && dw && d_dx && d_dw && (!l->bias || d_db) &&
        boat_report("dense dX", boat_cuda_gemm(mma, 0, 1, N, I, O, dg, O, dw, O, type, d_dx, I, type, NULL)) == 0 &&
        boat_report("dense dW", boat_cuda_gemm(mma, 1, 0, I, O, N, dx, I, dg, O, type, d_dw, O, BOAT_CUDA_F32, NULL)) == 0 &&
        (!l->bias || boat_report("dense db", boat_cuda_colsum(dg, type, N, O, d_db)) == 0)) {
        /* accumulate into the layer's gradients, wherever they live */
        boat_tensor_t* grads[2] = {l->grad_weight, l->grad_bias};
        float* fresh[2] = {d_dw, d_db};
        int rc = 0;
        for (int i = 0; i < 2 && rc == 0; ++i) {
            boat_tensor_t* g = grads[i];
            if (!g || !fresh[i]) continue;
            if (g->device == BOAT_DEVICE_CUDA) {
                rc = boat_cuda_axpy((float*)g->data, fresh[i], 1.0f, (int64_t)g->nelements);
            } else {
                float* acc = (float*)boat_dev_alloc(g->nbytes);
                rc = acc ? boat_cuda_memcpy_h2d(acc, g->data, g->nbytes) : 1;
                if (rc == 0) rc = boat_cuda_axpy(acc, fresh[i], 1.0f, (int64_t)g->nelements);
                if (rc == 0) rc = boat_cuda_memcpy_d2h(g->data, acc, g->nbytes);
                boat_dev_free(acc);
            }
        }
        if (boat_report("dense gradient accumulation", rc) == 0) out = boat_emit_out_take(x->shape, 2, x, &d_dx, type);
    }
    boat_dev_free(d_db);
    boat_dev_free(d_dw);
    boat_dev_free(d_dx);
    if (xo) boat_dev_free(dx);
    if (go) boat_dev_free(dg);
    if (wo) boat_dev_free(dw);
    return out;
}

BOAT_NOINLINE void boat_dense_layer_update(boat_dense_layer_t* l, float learning_rate) {
    if (!l) return;
    boat_tensor_t* pairs[2][2] = {{l->weight, l->grad_weight}, {l->bias, l->grad_bias}};
    for (int i = 0; i < 2; ++i) {
        boat_tensor_t *w = pairs[i][0], *g = pairs[i][1];
        if (!w || !g) continue;
        boat_tensor_t* step = boat_mul_scalar(g, learning_rate);
        if (step) {
            boat_sub_(w, step);
            boat_tensor_unref(step);
        }
        boat_memory_set(g->data, 0, g->nbytes, g->device);      /* the reference clears after the step */
    }
}

static void replace(boat_tensor_t** slot, boat_tensor_t* t) {
    if (!t) return;
    boat_tensor_ref(t);
    if (*slot) boat_tensor_free(*slot);
    *slot = t;
}

void boat_dense_layer_set_weight(boat_dense_layer_t* l, boat_tensor_t* weight) {
    if (l && weight && weight->ndim == 2 && weight->shape[0] == (int64_t)l->in_features &&
        weight->shape[1] == (int64_t)l->out_features)
        replace(&l->weight, weight);
}

void boat_dense_layer_set_bias(boat_dense_layer_t* l, boat_tensor_t* bias) {
    if (l && bias && bias->nelements == l->out_features) {
        replace(&l->bias, bias);
        l->use_bias = true;
    }
}

boat_tensor_t* boat_dense_layer_get_weight(const boat_dense_layer_t* l) { return l ? l->weight : NULL; }
boat_tensor_t* boat_dense_layer_get_bias(const boat_dense_layer_t* l) { return l ? l->bias : NULL; }
boat_tensor_t* boat_dense_layer_get_grad_weight(const boat_dense_layer_t* l) { return l ? l->grad_weight : NULL; }
boat_tensor_t* boat_dense_layer_get_grad_bias(const boat_dense_layer_t* l) { return l ? l->grad_bias : NULL; }

int boat_dense_layer_to_device(boat_dense_layer_t* l, boat_device_t device) {
    if (!l) return 1;
    boat_tensor_t** slots[4] = {&l->weight, &l->bias, &l->grad_weight, &l->grad_bias};
    for (int i = 0; i < 4; ++i) {
        boat_tensor_t* t = *slots[i];
        if (!t || t->device == device) continue;
        boat_tensor_t* moved = boat_tensor_to_device(t, device);
        if (!moved) return 2;
        boat_tensor_free(t);
        *slots[i] = moved;
    }
    return 0;
}
