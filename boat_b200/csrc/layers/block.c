/* block.c - one pre-LN transformer encoder block step, composed in C from the layers.
 *
 *   y   = x + attention(LN1(x))
 *   out = y + dense2(GELU(dense1(LN2(y))))
 *
 * The reference has the pieces (boat_layernorm_forward src/layers/norm.c:231-317, the dense layer
 * src/layers/dense.c:135-297, the attention layer) but no block object and no test that chains
 * them; this is the chaining a caller would write with the layer API, kept inside the library so
 * that a step is two calls and the sixty-odd kernel launches of a step are issued back to back.
 * The layers are borrowed: create, fill, place (to_device) and free them with their own API.
 * Works on host or CUDA tensors like the layers it calls. */
#include "../core/boat_internal.h"
#include <boat_b200.h>
#include <boat/ops.h>

#include <stdlib.h>

struct boat_encoder_block_t {
    boat_layernorm_t *ln1, *ln2;
    boat_attention_t* attn;
    boat_dense_layer_t *fc1, *fc2;
    boat_tensor_t* u;                 /* dense1 output before GELU, kept for the backward */
    int64_t shape[3];                 /* [B, S, d] of the last forward */
    bool sums_begun;                  /* the last backward started the gradient sums of the dense and
                                         LayerNorm layers itself, all of them */
    bool sums_in_flight;              /* some were started and nobody has waited for them yet */
};

/* In-place sum over the ranks of the gradients of up to four tensors, started on the communication
 * stream behind what the library stream has queued so far.  false when a tensor is not FP32 on the
 * GPU or the start fails. */
static bool begin_sums(boat_tensor_t* const t[], int n) {
    float* piece[4];
    int64_t count[4];
    int k = 0;
    for (int i = 0; i < n && k < 4; ++i) {
        if (!t[i]) continue;
        if (t[i]->device != BOAT_DEVICE_CUDA || t[i]->dtype != BOAT_DTYPE_FLOAT32) return false;
        piece[k] = (float*)t[i]->data;
        count[k++] = (int64_t)t[i]->nelements;
    }
    return k == 0 || boat_report("block gradient all-reduce", boat_cuda_allreduce_begin(piece, count, k)) == 0;
}

boat_encoder_block_t* boat_encoder_block_create(boat_layernorm_t* norm1, boat_attention_t* attention,
                                                boat_layernorm_t* norm2, boat_dense_layer_t* dense1,
                                                boat_dense_layer_t* dense2) {
    if (!norm1 || !attention || !norm2 || !dense1 || !dense2) return NULL;
    boat_encoder_block_t* b = (boat_encoder_block_t*)calloc(1, sizeof *b);
    if (!b) return NULL;
    b->ln1 = norm1;
    b->attn = attention;
    b->ln2 = norm2;
    b->fc1 = dense1;
    b->fc2 = dense2;
    return b;
}

void boat_encoder_block_free(boat_encoder_block_t* b) {
    if (!b) return;
    if (b->u) boat_tensor_unref(b->u);
    free(b);
}

/* Frees `t` (when not NULL) and returns `keep`: lets a chain of temporaries read top to bottom. */
static boat_tensor_t* drop(boat_tensor_t* t, boat_tensor_t* keep) {
    if (t) boat_tensor_unref(t);
    return keep;
}

boat_tensor_t* boat_encoder_block_forward(boat_encoder_block_t* b, const boat_tensor_t* x) {
    if (!b || !x || x->ndim != 3) return NULL;
    const int64_t T = x->shape[0] * x->shape[1], d = x->shape[2];
    const int64_t flat[2] = {T, d};
    boat_tensor_t *h1 = NULL, *att = NULL, *r1 = NULL, *h2 = NULL, *h2f = NULL, *u = NULL, *act = NULL, *m = NULL,
                  *m3 = NULL, *out = NULL;
    if (b->u) b->u = drop(b->u, NULL);
    for (int i = 0; i < 3; ++i) b->shape[i] = x->shape[i];
    h1 = boat_layernorm_forward(b->ln1, x);
    att = h1 ? boat_attention_forward(b->attn, h1, h1, h1, NULL) : NULL;
    r1 = att ? boat_lincomb(x, 1.0f, att, 1.0f) : NULL;
    h2 = r1 ? boat_layernorm_forward(b->ln2, r1) : NULL;
    h2f = h2 ? boat_tensor_reshape(h2, flat, 2) : NULL;
    u = h2f ? boat_dense_layer_forward(b->fc1, h2f) : NULL;
    act = u ? boat_gelu(u) : NULL;
    m = act ? boat_dense_layer_forward(b->fc2, act) : NULL;
    m3 = m ? boat_tensor_reshape(m, x->shape, 3) : NULL;
    out = m3 ? boat_lincomb(r1, 1.0f, m3, 1.0f) : NULL;
    if (out) {
        b->u = u;
        u = NULL;
    }
    drop(h1, NULL); drop(att, NULL); drop(r1, NULL); drop(h2f, NULL); drop(h2, NULL); drop(u, NULL);
    drop(act, NULL); drop(m3, NULL); drop(m, NULL);
    return out;
}

boat_tensor_t* boat_encoder_block_backward(boat_encoder_block_t* b, const boat_tensor_t* grad_output) {
    if (!b || !grad_output || !b->u) return NULL;
    const int64_t T = b->shape[0] * b->shape[1], d = b->shape[2];
    if ((int64_t)grad_output->nelements != T * d) return NULL;
    const int64_t flat[2] = {T, d};
    boat_tensor_t *g2 = NULL, *da = NULL, *du = NULL, *dh2 = NULL, *dh2_3 = NULL, *dln2 = NULL, *dr1 = NULL,
                  *gq = NULL, *gk = NULL, *gv = NULL, *s1 = NULL, *dh1 = NULL, *dln1 = NULL, *dx = NULL;
    /* Data parallel with overlap (the attention layer's setting decides): a layer's gradients are
     * final when its backward has been issued, long before the step ends - their sums over the ranks
     * start right there and run under the kernels that follow. */
    const bool overlap = boat_cuda_comm_world() > 1 && boat_attention_get_grad_overlap(b->attn) != 0;
    bool begun = overlap;
    if (b->sums_in_flight) {
        /* sums of a step whose boat_encoder_block_allreduce_grads never came still read and write the
         * gradients this backward is about to add to */
        b->sums_in_flight = false;
        if (boat_report("block gradient all-reduce", boat_cuda_allreduce_join()) != 0) return NULL;
    }
    b->sums_begun = false;
    /* MLP branch: out = r1 + dense2(GELU(dense1(LN2(r1)))) */
    g2 = boat_tensor_reshape(grad_output, flat, 2);
    da = g2 ? boat_dense_layer_backward(b->fc2, g2) : NULL;
    if (da && begun) {
        boat_tensor_t* const t[2] = {boat_dense_layer_get_grad_weight(b->fc2), boat_dense_layer_get_grad_bias(b->fc2)};
        begun = begin_sums(t, 2);
        b->sums_in_flight = begun;
    }
    du = da ? boat_gelu_backward(da, b->u) : NULL;
    dh2 = du ? boat_dense_layer_backward(b->fc1, du) : NULL;
    if (dh2 && begun) {
        boat_tensor_t* const t[2] = {boat_dense_layer_get_grad_weight(b->fc1), boat_dense_layer_get_grad_bias(b->fc1)};
        begun = begin_sums(t, 2);
    }
    dh2_3 = dh2 ? boat_tensor_reshape(dh2, b->shape, 3) : NULL;
    dln2 = dh2_3 ? boat_layernorm_backward(b->ln2, dh2_3) : NULL;
    dr1 = dln2 ? boat_lincomb(grad_output, 1.0f, dln2, 1.0f) : NULL;
    /* attention branch: r1 = x + attention(LN1(x)), query = key = value */
    if (dr1 && boat_attention_backward(b->attn, dr1, &gq, &gk, &gv)) {
        s1 = boat_lincomb(gq, 1.0f, gk, 1.0f);
        dh1 = s1 ? boat_lincomb(s1, 1.0f, gv, 1.0f) : NULL;
        dln1 = dh1 ? boat_layernorm_backward(b->ln1, dh1) : NULL;
        dx = dln1 ? boat_lincomb(dr1, 1.0f, dln1, 1.0f) : NULL;
        if (dx && begun) {
            /* the four small LayerNorm gradients as one group */
            boat_tensor_t* const t[4] = {boat_layernorm_get_grad_weight(b->ln1), boat_layernorm_get_grad_bias(b->ln1),
                                         boat_layernorm_get_grad_weight(b->ln2), boat_layernorm_get_grad_bias(b->ln2)};
            begun = begin_sums(t, 4);
            b->sums_begun = begun;
        }
    }
    drop(g2, NULL); drop(da, NULL); drop(du, NULL); drop(dh2_3, NULL); drop(dh2, NULL); drop(dln2, NULL);
    drop(dr1, NULL); drop(gq, NULL); drop(gk, NULL); drop(gv, NULL); drop(s1, NULL); drop(dh1, NULL); drop(dln1, NULL);
    return dx;
}

/* Data-parallel step: every rank holds the same parameters and its own rows.  Sums all parameter
 * gradients of the block over the ranks - the attention layer's bucket, both LayerNorms' and both
 * dense layers' weight and bias gradients - as one group of in-place sums, and makes the library
 * stream wait for them. */
int boat_encoder_block_allreduce_grads(boat_encoder_block_t* b) {
    if (!b) return 1;
    if (boat_cuda_comm_world() <= 1) return 0;
    if (b->sums_begun) {
        /* the backward started the dense and LayerNorm sums; the attention layer starts what it still
         * owes and makes the library stream wait for all of them */
        b->sums_begun = false;
        b->sums_in_flight = false;
        return boat_attention_allreduce_grads(b->attn);
    }
    if (b->sums_in_flight) {
        /* a backward that failed half-way started some sums: wait for them, report the step as lost */
        b->sums_in_flight = false;
        boat_report("block gradient all-reduce", boat_cuda_allreduce_join());
        fprintf(stderr, "boat: the block's last backward did not complete; its gradients are not summed\n");
        return 4;
    }
    boat_tensor_t* t[8] = {boat_layernorm_get_grad_weight(b->ln1), boat_layernorm_get_grad_bias(b->ln1),
                           boat_layernorm_get_grad_weight(b->ln2), boat_layernorm_get_grad_bias(b->ln2),
                           boat_dense_layer_get_grad_weight(b->fc1), boat_dense_layer_get_grad_bias(b->fc1),
                           boat_dense_layer_get_grad_weight(b->fc2), boat_dense_layer_get_grad_bias(b->fc2)};
    float* piece[8];
    int64_t count[8];
    int n = 0;
    for (int i = 0; i < 8; ++i) {
        if (!t[i]) continue;
        if (t[i]->device != BOAT_DEVICE_CUDA || t[i]->dtype != BOAT_DTYPE_FLOAT32) {
            fprintf(stderr, "boat: gradient all-reduce needs the block's layers on BOAT_DEVICE_CUDA\n");
            return 2;
        }
        piece[n] = (float*)t[i]->data;
        count[n++] = (int64_t)t[i]->nelements;
    }
    if (boat_report("block gradient all-reduce", boat_cuda_allreduce_begin(piece, count, n)) != 0) return 3;
    /* the attention bucket: what its backward has not started yet; then the library stream waits for
     * every sum under way */
    return boat_attention_allreduce_grads(b->attn);
}
