/* norm.c - LayerNorm layer on the GPU.
 *
 * Forward follows the reference's boat_layernorm_forward (src/layers/norm.c:231-317): the
 * last dimension is normalised with the biased variance, eps inside the square root, then
 * weight and bias.  Create/free/set_weight/set_bias as norm.c:73-131, :481-517 (weight ones,
 * bias zeros, FP32 host tensors).  The reference's backward and update are stubs
 * (norm.c:397-412); here backward returns the input gradient and keeps d(weight), d(bias) in
 * the layer, and update is the SGD step the other layers use.  RMSNorm is not on the path. */
#include "../core/stage.h"
#include <boat/layers/norm.h>
#include <boat/layers.h>
#include <boat/ops.h>
#include <boat_b200.h>
#include <string.h>

struct boat_layernorm_t {
    boat_layernorm_config_t config;
    boat_tensor_t* weight;          /* gamma, FP32 [H] or NULL */
    boat_tensor_t* bias;            /* beta */
    boat_tensor_t* grad_weight;     /* NULL until the first backward */
    boat_tensor_t* grad_bias;
    boat_tensor_t* cache_input;     /* referenced until the next forward */
    float* d_mean;                  /* [rows] device */
    float* d_rstd;
    int64_t rows;
};

static boat_tensor_t* filled(size_t n, float v) {
    const int64_t shape[1] = {(int64_t)n};
    boat_tensor_t* t = boat_tensor_create(shape, 1, BOAT_DTYPE_FLOAT32, BOAT_DEVICE_CPU);
    if (t && v != 0.0f) {
        float* p = (float*)t->data;
        for (size_t i = 0; i < n; ++i) p[i] = v;
    }
    return t;
}

boat_layernorm_t* boat_layernorm_create(const boat_layernorm_config_t* config) {
    if (!config || config->normalized_shape == 0) return NULL;
    boat_layernorm_t* n = (boat_layernorm_t*)boat_calloc(sizeof *n, BOAT_DEVICE_CPU);
    if (!n) return NULL;
    n->config = *config;
    if (config->elementwise_affine) {
        n->weight = filled(config->normalized_shape, 1.0f);
        if (config->use_bias) n->bias = filled(config->normalized_shape, 0.0f);
        if (!n->weight || (config->use_bias && !n->bias)) {
            boat_layernorm_free(n);
            return NULL;
        }
    }
    return n;
}

static void drop_cache(boat_layernorm_t* n) {
    if (n->cache_input) boat_tensor_unref(n->cache_input);
    n->cache_input = NULL;
    boat_dev_free(n->d_mean);
    boat_dev_free(n->d_rstd);
    n->d_mean = n->d_rstd = NULL;
}

void boat_layernorm_free(boat_layernorm_t* n) {
    if (!n) return;
    drop_cache(n);
    if (n->weight) boat_tensor_free(n->weight);
    if (n->bias) boat_tensor_free(n->bias);
    if (n->grad_weight) boat_tensor_free(n->grad_weight);
    if (n->grad_bias) boat_tensor_free(n->grad_bias);
    boat_free(n);
}

boat_tensor_t* boat_layernorm_forward(boat_layernorm_t* n, const boat_tensor_t* input) {
    if (!n || !input || input->ndim < 1 || !boat_dtype_supported(input->dtype)) return NULL;
    const int64_t H = (int64_t)n->config.normalized_shape;
    if (input->shape[input->ndim - 1] != H) return NULL;
    if (boat_report("CUDA start-up", boat_cuda_init(-1)) != 0) return NULL;
    boat_tensor_ref((boat_tensor_t*)input);
    drop_cache(n);
    n->cache_input = (boat_tensor_t*)input;
    const int type = boat_storage_of(input->dtype);
    const int64_t rows = (int64_t)input->nelements / H;
    bool xo = false, go = false, bo = false;
    void* dx = boat_stage_in(input, type, &xo);
    float* dg = n->weight ? (float*)boat_stage_in(n->weight, BOAT_CUDA_F32, &go) : NULL;
    float* db = n->bias ? (float*)boat_stage_in(n->bias, BOAT_CUDA_F32, &bo) : NULL;
    void* dy = boat_dev_alloc(input->nelements * boat_storage_size(type));
    n->d_mean = (float*)boat_dev_alloc((size_t)rows * sizeof(float));
    n->d_rstd = (float*)boat_dev_alloc((size_t)rows * sizeof(float));
    n->rows = rows;
    boat_tensor_t* out = NULL;
    if (dx && dy && n->d_mean && n->d_rstd && (!n->weight || dg) && (!n->bias || db) &&
        boat_report("LayerNorm forward", boat_cuda_layernorm_fwd(dx, type, rows, H, dg, db, n->config.eps, dy,
                                                                 n->d_mean, n->d_rstd)) == 0)
        out = boat_emit_out_take(input->shape, input->ndim, input, &dy, type);
    boat_dev_free(dy);
    if (xo) boat_dev_free(dx);
    if (go) boat_dev_free(dg);
    if (bo) boat_dev_free(db);
    return out;
}

static boat_tensor_t* grad_like(boat_tensor_t** slot, const boat_tensor_t* param) {
    if (!*slot || (*slot)->device != param->device) {
        if (*slot) boat_tensor_free(*slot);
        *slot = boat_tensor_create(param->shape, param->ndim, BOAT_DTYPE_FLOAT32, param->device);
    }
    return *slot;
}

boat_tensor_t* boat_layernorm_backward(boat_layernorm_t* n, const boat_tensor_t* grad_output) {
    if (!n || !grad_output || !n->cache_input || !n->d_mean) return NULL;
    const boat_tensor_t* x = n->cache_input;
    if (grad_output->nelements != x->nelements || !boat_dtype_supported(grad_output->dtype)) return NULL;
    const int64_t H = (int64_t)n->config.normalized_shape, rows = n->rows;
    const int type = boat_storage_of(x->dtype);
    bool xo = false, yo = false, go = false;
    void* dx_in = boat_stage_in(x, type, &xo);
    void* dy = boat_stage_in(grad_output, type, &yo);
    float* dg = n->weight ? (float*)boat_stage_in(n->weight, BOAT_CUDA_F32, &go) : NULL;
    void* dx = boat_dev_alloc(x->nelements * boat_storage_size(type));
    /* Each parameter gradient lives where its parameter lives, and the two need not agree (a
     * host bias set on a CUDA layer, a bias without a weight): the kernel writes a CUDA
     * gradient in place and a host gradient through a device temporary that is then copied down. */
    float *d_dgamma = NULL, *d_dbeta = NULL;
    bool gamma_tmp = false, beta_tmp = false;
    boat_tensor_t* out = NULL;
    if (n->weight && grad_like(&n->grad_weight, n->weight)) {
        gamma_tmp = n->grad_weight->device != BOAT_DEVICE_CUDA;
        d_dgamma = gamma_tmp ? (float*)boat_dev_alloc((size_t)H * 4) : (float*)n->grad_weight->data;
    }
    if (n->bias && grad_like(&n->grad_bias, n->bias)) {
        beta_tmp = n->grad_bias->device != BOAT_DEVICE_CUDA;
        d_dbeta = beta_tmp ? (float*)boat_dev_alloc((size_t)H * 4) : (float*)n->grad_bias->data;
    }
    if (dx_in && dy && dx && (!n->weight || (dg && d_dgamma)) && (!n->bias || d_dbeta) &&
        boat_report("LayerNorm backward", boat_cuda_layernorm_bwd(dy, dx_in, type, rows, H, dg, n->d_mean, n->d_rstd,
                                                                  dx, d_dgamma, d_dbeta)) == 0) {
        int rc = 0;
        if (gamma_tmp && d_dgamma) rc = boat_cuda_memcpy_d2h(n->grad_weight->data, d_dgamma, (size_t)H * 4);
        if (rc == 0 && beta_tmp && d_dbeta) rc = boat_cuda_memcpy_d2h(n->grad_bias->data, d_dbeta, (size_t)H * 4);
        if (boat_report("gradient download", rc) == 0) out = boat_emit_out_take(x->shape, x->ndim, x, &dx, type);
    }
    if (gamma_tmp) boat_dev_free(d_dgamma);
    if (beta_tmp) boat_dev_free(d_dbeta);
    boat_dev_free(dx);
    if (xo) boat_dev_free(dx_in);
    if (yo) boat_dev_free(dy);
    if (go) boat_dev_free(dg);
    return out;
}

void boat_layernorm_update(boat_layernorm_t* n, float learning_rate) {
    if (!n) return;
    boat_tensor_t* pairs[2][2] = {{n->weight, n->grad_weight}, {n->bias, n->grad_bias}};
    for (int i = 0; i < 2; ++i) {
        boat_tensor_t *w = pairs[i][0], *g = pairs[i][1];
        if (!w || !g) continue;
        boat_tensor_t* step = boat_mul_scalar(g, learning_rate);     /* p -= lr * g, as the other layers do */
        if (step) {
            boat_sub_(w, step);
            boat_tensor_unref(step);
        }
    }
}

static void replace_param(boat_tensor_t** slot, boat_tensor_t* t, size_t want, const char* what) {
    if (!t) return;
    if (t->ndim < 1 || t->shape[0] != (int64_t)want) {
        fprintf(stderr, "Error: %s shape [%lld] does not match normalized_shape %zu\n", what,
                t->ndim ? (long long)t->shape[0] : 0LL, want);
        return;
    }
    boat_tensor_ref(t);
    if (*slot) boat_tensor_free(*slot);
    *slot = t;
}

void boat_layernorm_set_weight(boat_layernorm_t* n, boat_tensor_t* weight) {
    if (n) replace_param(&n->weight, weight, n->config.normalized_shape, "Weight");
}

void boat_layernorm_set_bias(boat_layernorm_t* n, boat_tensor_t* bias) {
    if (n) replace_param(&n->bias, bias, n->config.normalized_shape, "Bias");
}

boat_tensor_t* boat_layernorm_get_weight(const boat_layernorm_t* n) { return n ? n->weight : NULL; }
boat_tensor_t* boat_layernorm_get_bias(const boat_layernorm_t* n) { return n ? n->bias : NULL; }
boat_tensor_t* boat_layernorm_get_grad_weight(const boat_layernorm_t* n) { return n ? n->grad_weight : NULL; }
boat_tensor_t* boat_layernorm_get_grad_bias(const boat_layernorm_t* n) { return n ? n->grad_bias : NULL; }

int boat_layernorm_to_device(boat_layernorm_t* n, boat_device_t device) {
    if (!n) return 1;
    boat_tensor_t** slots[2] = {&n->weight, &n->bias};
    for (int i = 0; i < 2; ++i) {
        boat_tensor_t* t = *slots[i];
        if (!t || t->device == device) continue;
        boat_tensor_t* moved = boat_tensor_to_device(t, device);
        if (!moved) return 2;
        boat_tensor_free(t);
        *slots[i] = moved;
    }
    return 0;
}

/* generic-layer adapter (reference include/boat/layers.h:75-79; the reference never defines
 * these): weight and bias both on when elementwise_affine */
boat_norm_layer_t* boat_norm_layer_create(size_t normalized_shape, float eps, bool elementwise_affine) {
    boat_layernorm_config_t cfg = {normalized_shape, eps, elementwise_affine, elementwise_affine};
    return (boat_norm_layer_t*)boat_layernorm_create(&cfg);
}
void boat_norm_layer_free(boat_norm_layer_t* l) { boat_layernorm_free((boat_layernorm_t*)l); }
boat_tensor_t* boat_norm_layer_forward(boat_norm_layer_t* l, const boat_tensor_t* x) {
    return boat_layernorm_forward((boat_layernorm_t*)l, x);
}
boat_tensor_t* boat_norm_layer_backward(boat_norm_layer_t* l, const boat_tensor_t* g) {
    return boat_layernorm_backward((boat_layernorm_t*)l, g);
}
void boat_norm_layer_update(boat_norm_layer_t* l, float lr) { boat_layernorm_update((boat_layernorm_t*)l, lr); }
