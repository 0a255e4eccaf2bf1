/* adam.c - host side of the Adam optimizer; the arithmetic is boat_cuda_adam_step.
 *
 * Follows the reference's src/optimizers/adam.c (state record :19-39, create :42-86,
 * registration :87-128, step :156-209, zero_grad :211-231, free :233-262, learning-rate
 * access :264-283) and the type dispatch of src/optimizers/optimizer_common.c.  Differences,
 * all on this side of the API: the moment estimates are device buffers; every registered
 * tensor of a step goes to the GPU in one launch; a parameter that already is a CUDA tensor
 * is updated where it lies. */
#include <boat/optimizers.h>
#include "../core/stage.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

struct boat_optimizer_t {
    boat_optimizer_type_t type;        /* first, as the reference's dispatch expects */
    float          learning_rate, beta1, beta2, epsilon;
    int64_t        timestep;
    boat_tensor_t** params;            /* borrowed */
    boat_tensor_t** grads;             /* borrowed */
    float**        m;                  /* device, zero at registration */
    float**        v;
    size_t         count, capacity;
};

boat_optimizer_t* boat_sgd_optimizer_create(float learning_rate, float momentum) {
    (void)learning_rate;
    (void)momentum;
    return NULL;
}

boat_optimizer_t* boat_adam_optimizer_create(float learning_rate, float beta1, float beta2, float epsilon) {
    if (!(learning_rate > 0.0f)) return NULL;
    if (!(beta1 > 0.0f && beta1 < 1.0f) || !(beta2 > 0.0f && beta2 < 1.0f)) return NULL;
    boat_optimizer_t* o = (boat_optimizer_t*)calloc(1, sizeof *o);
    if (!o) return NULL;
    o->type = BOAT_OPTIMIZER_ADAM;
    o->learning_rate = learning_rate;
    o->beta1 = beta1;
    o->beta2 = beta2;
    o->epsilon = epsilon;
    return o;
}

static bool grow(boat_optimizer_t* o) {
    size_t cap = o->capacity ? o->capacity * 2 : 16;
    boat_tensor_t** p = (boat_tensor_t**)realloc(o->params, cap * sizeof *p);
    if (p) o->params = p;
    boat_tensor_t** g = (boat_tensor_t**)realloc(o->grads, cap * sizeof *g);
    if (g) o->grads = g;
    float** m = (float**)realloc(o->m, cap * sizeof *m);
    if (m) o->m = m;
    float** v = (float**)realloc(o->v, cap * sizeof *v);
    if (v) o->v = v;
    if (!p || !g || !m || !v) return false;
    o->capacity = cap;
    return true;
}

void boat_optimizer_add_parameter(boat_optimizer_t* o, boat_tensor_t* param, boat_tensor_t* grad) {
    if (!o || o->type != BOAT_OPTIMIZER_ADAM || !param || !grad) return;
    if (param->dtype != BOAT_DTYPE_FLOAT32 || grad->dtype != BOAT_DTYPE_FLOAT32 ||
        param->nelements != grad->nelements) {
        fprintf(stderr, "boat: optimizer parameters and gradients must be FP32 tensors of equal size\n");
        return;
    }
    if (o->count == o->capacity && !grow(o)) return;
    size_t bytes = param->nelements * sizeof(float);
    float* m = bytes ? (float*)boat_dev_alloc(bytes) : NULL;
    float* v = bytes ? (float*)boat_dev_alloc(bytes) : NULL;
    if (bytes && (!m || !v || boat_report("moment reset", boat_cuda_memset(m, 0, bytes)) != 0 ||
                  boat_report("moment reset", boat_cuda_memset(v, 0, bytes)) != 0)) {
        boat_dev_free(m);
        boat_dev_free(v);
        return;
    }
    o->params[o->count] = param;
    o->grads[o->count] = grad;
    o->m[o->count] = m;
    o->v[o->count] = v;
    o->count++;
}

void boat_optimizer_step(boat_optimizer_t* o) {
    if (!o || o->type != BOAT_OPTIMIZER_ADAM) return;
    const size_t n = o->count;
    if (n) {
        float** p = (float**)calloc(n, sizeof *p);
        const float** g = (const float**)calloc(n, sizeof *g);
        int64_t* len = (int64_t*)calloc(n, sizeof *len);
        bool* own_p = (bool*)calloc(n, sizeof *own_p);
        bool* own_g = (bool*)calloc(n, sizeof *own_g);
        bool ok = p && g && len && own_p && own_g;
        for (size_t i = 0; ok && i < n; ++i) {
            len[i] = (int64_t)o->params[i]->nelements;
            if (!len[i]) continue;
            p[i] = (float*)boat_stage_in(o->params[i], BOAT_CUDA_F32, &own_p[i]);
            g[i] = (const float*)boat_stage_in(o->grads[i], BOAT_CUDA_F32, &own_g[i]);
            ok = p[i] && g[i];
        }
        if (ok) {
            /* float powers of a float exponent, as adam.c:173-174 computes them */
            float t = (float)(o->timestep + 1);
            float corr1 = 1.0f - powf(o->beta1, t);
            float corr2 = 1.0f - powf(o->beta2, t);
            ok = boat_report("Adam step",
                             boat_cuda_adam_step((int)n, (float* const*)p, (const float* const*)g, (float* const*)o->m,
                                                 (float* const*)o->v, len, o->learning_rate, o->beta1,
                                                 o->beta2, o->epsilon, corr1, corr2)) == 0;
        }
        for (size_t i = 0; p && g && own_p && own_g && i < n; ++i) {
            if (ok && own_p[i])
                boat_report("parameter download",
                            boat_cuda_memcpy_d2h(o->params[i]->data, p[i], o->params[i]->nbytes));
            if (own_p[i]) boat_dev_free(p[i]);
            if (own_g[i]) boat_dev_free((void*)g[i]);
        }
        free(p);
        free((void*)g);
        free(len);
        free(own_p);
        free(own_g);
    }
    o->timestep++;
}

void boat_optimizer_zero_grad(boat_optimizer_t* o) {
    if (!o || o->type != BOAT_OPTIMIZER_ADAM) return;
    for (size_t i = 0; i < o->count; ++i) {
        boat_tensor_t* g = o->grads[i];
        if (!g || !g->nbytes) continue;
        if (g->device == BOAT_DEVICE_CUDA)
            boat_report("gradient reset", boat_cuda_memset(g->data, 0, g->nbytes));
        else
            memset(g->data, 0, g->nbytes);
    }
}

void boat_optimizer_free(boat_optimizer_t* o) {
    if (!o) return;
    for (size_t i = 0; i < o->count; ++i) {
        boat_dev_free(o->m[i]);
        boat_dev_free(o->v[i]);
    }
    free(o->params);
    free(o->grads);
    free(o->m);
    free(o->v);
    free(o);
}

float boat_optimizer_get_learning_rate(const boat_optimizer_t* o) {
    return (o && o->type == BOAT_OPTIMIZER_ADAM) ? o->learning_rate : 0.0f;
}

void boat_optimizer_set_learning_rate(boat_optimizer_t* o, float learning_rate) {
    if (o && o->type == BOAT_OPTIMIZER_ADAM) o->learning_rate = learning_rate;
}
