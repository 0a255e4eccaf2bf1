/* attention.c - host orchestration of the multi-head attention layer on the GPU.
 *
 * Same public behaviour as the reference layer (src/layers/attention.c): create/free
 * (:126-244), forward (:310-466), backward (:468-732), SGD update (:734-815), the
 * functional wrappers (:830-879, :1082-1117), the generic-layer adapter (:1119-1175) and
 * the accessors (:1537-1631).  The arithmetic is not here: every contraction, softmax and
 * reduction is a kernel behind boat_cuda.h.  This file decides what lives where:
 *
 *   - Parameters are FP32 tensors on the layer's device (host after create, HBM after
 *     boat_attention_to_device).  Host parameters may be edited by the caller through
 *     boat_tensor_data() at any time without notice (the reference's finite-difference
 *     test does), so they are uploaded for every call; device parameters are used in place.
 *   - Activations kept for backward are device buffers in the storage type of the chosen
 *     arithmetic: the three projections, the pre-projection attention output and one
 *     log-sum-exp per (unit,row).  The reference's [B,nh,S,S] probability cache
 *     (:941-949) does not exist.
 *   - The eight parameter gradients are windows into one flat FP32 bucket so that the
 *     multi-GPU path reduces them with a single collective; each backward overwrites it
 *     (the reference replaces the tensors, :653-654, :702-703 - same "no accumulation").
 */
#include "../core/boat_internal.h"
#include <boat/layers.h>
#include <boat_b200.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>

enum { WQ, WK, WV, WO, BQ, BK, BV, BO, NPARAM };

struct boat_attention_t {
    boat_attention_config_t config;
    boat_tensor_t* param[NPARAM];       /* biases NULL without use_bias            */
    boat_tensor_t* grad[NPARAM];        /* windows into grad_bucket                */
    boat_tensor_t* grad_bucket;         /* FP32, on `device`                       */
    boat_device_t  device;              /* where the parameters live               */
    int            precision;           /* -1 automatic, else BOAT_MMA_*           */
    int            grad_overlap;        /* 0: sums only in allreduce_grads; 1: backward starts both groups
                                           itself; 2: backward starts dWo|dbo, the rest waits for allreduce_grads */
    bool           rest_pending;        /* mode 2: dWq dWk dWv | dbq dbk dbv still to be summed */
    bool           sums_begun;          /* the last backward started sums of this layer's bucket that nobody
                                           has joined yet */

    /* state of the last forward, consumed by backward */
    boat_tensor_t* cache_in[3];         /* query, key, value - referenced          */
    bool           cached;
    int            mma, type;           /* arithmetic and storage type it used     */
    int64_t        T, S;                /* token rows and sequence length of the call        */
    int64_t        units;               /* (batch, head) units = T * nh / S                  */
    int64_t        gran;                /* units per indivisible piece when the work is cut
                                           into chunks: nh (a whole batch entry) for [B,S,H]
                                           inputs, 1 for a unit range (see forward_units)    */
    void*          d_in[3];             /* inputs on device in `type`              */
    bool           d_in_owned[3];
    void*          d_proj[3];           /* Qp, Kp, Vp [B*S, H]                     */
    void*          d_ctx;               /* attention output before Wo              */
    float*         d_lse;               /* [B*nh*S]                                */

    /* The four FP32 weights of a CUDA layer in the form the tensor cores read (BF16, or TF32-valued
     * FP32), made by one launch in forward and used again by the backward of the same step.
     * `shadow_fresh` holds only from a forward to the end of the next backward, and every call
     * that hands out or changes a weight clears it; a caller that overwrites a weight through a
     * raw device pointer between forward and backward is not seen. */
    void*          shadow_w;            /* 4 * H * H elements                      */
    int            shadow_form;         /* BOAT_CUDA_BF16 or BOAT_CUDA_F32_TF32    */
    bool           shadow_fresh;
};

/* ---- small helpers ---------------------------------------------------------------------- */

static int storage_of(boat_dtype_t dt) { return dt == BOAT_DTYPE_BFLOAT16 ? BOAT_CUDA_BF16 : BOAT_CUDA_F32; }
static size_t storage_size(int type) { return type == BOAT_CUDA_BF16 ? 2 : 4; }
static bool dtype_ok(boat_dtype_t dt) { return dt == BOAT_DTYPE_FLOAT32 || dt == BOAT_DTYPE_BFLOAT16; }

static void* dev_alloc(size_t bytes) {
    void* p = NULL;
    if (boat_report("device allocation", boat_cuda_malloc(&p, bytes)) != 0) return NULL;
    return p;
}

static void dev_free(void* p) {
    if (p) boat_report("device free", boat_cuda_free(p));
}

/* Device buffer holding tensor `t` in storage type `type`.  *owned says whether the caller
 * must release it (false: it is the tensor's own HBM). */
static void* stage_in(const boat_tensor_t* t, int type, bool* owned) {
    int have = storage_of(t->dtype);
    size_t n = t->nelements;
    *owned = false;
    if (t->device == BOAT_DEVICE_CUDA && have == type) return t->data;
    *owned = true;
    void* raw = t->data;
    void* tmp = NULL;
    if (t->device != BOAT_DEVICE_CUDA) {
        tmp = dev_alloc(n * storage_size(have));
        if (!tmp) return NULL;
        if (boat_report("upload", boat_cuda_memcpy_h2d(tmp, t->data, n * storage_size(have))) != 0) {
            dev_free(tmp);
            return NULL;
        }
        if (have == type) return tmp;
        raw = tmp;
    }
    void* out = dev_alloc(n * storage_size(type));
    if (out && boat_report("cast", boat_cuda_cast(out, type, raw, have, (int64_t)n)) != 0) {
        dev_free(out);
        out = NULL;
    }
    dev_free(tmp);
    return out;
}

/* Operand for arithmetic `mma`: like stage_in, and for TF32 the values are additionally
 * rounded to the nearest TF32 number (in a private copy - the caller's tensor is never
 * modified), so that the tensor core's truncation of FP32 operands is exact. */
static void* stage_operand(const boat_tensor_t* t, int mma, int type, bool* owned) {
    void* p = stage_in(t, type, owned);
    if (!p || mma != BOAT_MMA_TF32) return p;
    void* dst = p;
    if (!*owned) {
        dst = dev_alloc(t->nelements * sizeof(float));
        if (!dst) return NULL;
        *owned = true;
    }
    if (boat_report("TF32 rounding", boat_cuda_round_tf32((float*)dst, (const float*)p, (int64_t)t->nelements)) != 0) {
        dev_free(dst);
        *owned = false;
        return NULL;
    }
    return dst;
}

/* Output type for a GEMM whose result feeds another contraction of arithmetic `mma`: in TF32 mode
 * the epilogue rounds to TF32 (the attention kernels do the same for their outputs), so no
 * separate rounding pass runs between kernels. */
static int feed_type(int mma, int type) { return mma == BOAT_MMA_TF32 ? BOAT_CUDA_F32_TF32 : type; }

/* New tensor with the dtype/device of `like`, filled from device buffer `src` (storage
 * `type`): a cast on the device for a CUDA result, a download (after a cast when the types
 * differ) for a host result.  `src` stays the caller's. */
static boat_tensor_t* emit_out(const int64_t* shape, size_t ndim, const boat_tensor_t* like, void* src,
                               int type) {
    boat_tensor_t* out = boat_tensor_create_uninit(shape, ndim, like->dtype, like->device);
    if (!out) return NULL;
    int want = storage_of(like->dtype);
    size_t n = out->nelements;
    int rc = 0;
    if (like->device == BOAT_DEVICE_CUDA) {
        rc = boat_cuda_cast(out->data, want, src, type, (int64_t)n);
    } else if (want == type) {
        rc = boat_cuda_memcpy_d2h(out->data, src, n * storage_size(type));
    } else {
        void* tmp = dev_alloc(n * storage_size(want));
        rc = tmp ? boat_cuda_cast(tmp, want, src, type, (int64_t)n) : 1;
        if (rc == 0) rc = boat_cuda_memcpy_d2h(out->data, tmp, n * storage_size(want));
        dev_free(tmp);
    }
    if (boat_report("result transfer", rc) != 0) {
        boat_tensor_free(out);
        return NULL;
    }
    return out;
}

static int env_precision(void) {
    const char* e = getenv("BOAT_MMA");
    if (!e) return -1;
    if (!strcasecmp(e, "fp32")) return BOAT_MMA_FP32;
    if (!strcasecmp(e, "tf32")) return BOAT_MMA_TF32;
    if (!strcasecmp(e, "bf16")) return BOAT_MMA_BF16;
    return -1;
}

/* Arithmetic for a call: the explicit setting (boat_attention_set_precision, or BOAT_MMA in the
 * environment at create time), else by the input's storage type alone: BF16 tensors use BF16
 * tensor cores, FP32 tensors the exact FP32 kernels - the numerics of a reference program never
 * change with the sequence length.  TF32 is always an explicit choice. */
static int pick_mma(const boat_attention_t* a, const boat_tensor_t* q) {
    if (a->precision >= 0) return a->precision;
    return q->dtype == BOAT_DTYPE_BFLOAT16 ? BOAT_MMA_BF16 : BOAT_MMA_FP32;
}

static void drop_forward_state(boat_attention_t* a) {
    for (int i = 0; i < 3; ++i) {
        if (a->d_in_owned[i]) {
            /* the same staged buffer may serve several inputs (self-attention) */
            for (int j = i + 1; j < 3; ++j)
                if (a->d_in[j] == a->d_in[i]) a->d_in_owned[j] = false;
            dev_free(a->d_in[i]);
        }
        a->d_in[i] = NULL;
        a->d_in_owned[i] = false;
        dev_free(a->d_proj[i]);
        a->d_proj[i] = NULL;
        if (a->cache_in[i]) boat_tensor_unref(a->cache_in[i]);
        a->cache_in[i] = NULL;
    }
    dev_free(a->d_ctx);
    a->d_ctx = NULL;
    dev_free(a->d_lse);
    a->d_lse = NULL;
    a->cached = false;
}

/* Device copies of the parameters for one call: weights in storage `type`, biases FP32. */
typedef struct {
    void* w[4];
    float* b[4];
    bool w_owned[4], b_owned[4];
    void* raw_w[4];             /* chunked host paths: where a weight lands before its conversion */
    bool late[4];               /* ... and whether it still has to be brought up */
} staged_params_t;

static void release_params(staged_params_t* p) {
    for (int i = 0; i < 4; ++i) {
        if (p->w_owned[i]) dev_free(p->w[i]);
        if (p->b_owned[i]) dev_free(p->b[i]);
        dev_free(p->raw_w[i]);
    }
    memset(p, 0, sizeof *p);
}

/* The weights of a CUDA layer as tensor-core operands, from the layer's shadow block: converted
 * by one launch, or - in the backward that follows a forward - not at all. */
static bool shadow_weights(boat_attention_t* a, int form, bool backward, staged_params_t* p) {
    const size_t H = a->config.hidden_size, n = H * H, es = form == BOAT_CUDA_BF16 ? 2 : 4;
    if (a->shadow_w && a->shadow_form != form) {
        dev_free(a->shadow_w);
        a->shadow_w = NULL;
    }
    if (!a->shadow_w) {
        a->shadow_w = dev_alloc(4 * n * es);
        if (!a->shadow_w) return false;
        a->shadow_form = form;
        a->shadow_fresh = false;
    }
    void* dst[4];
    const float* src[4];
    int64_t count[4];
    for (int i = 0; i < 4; ++i) {
        dst[i] = (char*)a->shadow_w + (size_t)i * n * es;
        src[i] = (const float*)a->param[WQ + i]->data;
        count[i] = (int64_t)n;
        p->w[i] = dst[i];
        p->w_owned[i] = false;
    }
    if (backward && a->shadow_fresh) return true;
    a->shadow_fresh = false;
    if (boat_report("weight conversion", boat_cuda_convert_multi(dst, form, src, count, 4)) != 0) return false;
    a->shadow_fresh = !backward;
    return true;
}

static bool stage_params(boat_attention_t* a, int mma, int type, bool backward, staged_params_t* p) {
    memset(p, 0, sizeof *p);
    bool shadow = a->device == BOAT_DEVICE_CUDA && (type == BOAT_CUDA_BF16 || mma == BOAT_MMA_TF32);
    for (int i = 0; i < 4 && shadow; ++i) {
        const boat_tensor_t* w = a->param[WQ + i];
        shadow = w->device == BOAT_DEVICE_CUDA && w->dtype == BOAT_DTYPE_FLOAT32 &&
                 w->nelements == a->config.hidden_size * a->config.hidden_size;
    }
    if (shadow && !shadow_weights(a, mma == BOAT_MMA_TF32 ? BOAT_CUDA_F32_TF32 : BOAT_CUDA_BF16, backward, p)) return false;
    for (int i = 0; i < 4; ++i) {
        if (!shadow) p->w[i] = stage_operand(a->param[WQ + i], mma, type, &p->w_owned[i]);
        if (!p->w[i]) goto fail;
        if (a->param[BQ + i]) {
            p->b[i] = (float*)stage_in(a->param[BQ + i], BOAT_CUDA_F32, &p->b_owned[i]);
            if (!p->b[i]) goto fail;
        }
    }
    return true;
fail:
    release_params(p);
    return false;
}


/* The chunked host-tensor paths bring a host layer's parameters up on the upload stream, behind the
 * first chunk of input and each group just before the first kernel that reads it, so that this
 * kernel waits for nothing else.  The device buffers are allocated up front, before the copy
 * streams are tied to the library stream: a buffer allocated later could only be written once the
 * kernels queued before its allocation have run, which would hold up every later upload. */
static bool prepare_late_params(boat_attention_t* a, int mma, int type, bool with_bias, staged_params_t* p) {
    memset(p, 0, sizeof *p);
    const size_t n = a->config.hidden_size * a->config.hidden_size;
    const bool convert = type == BOAT_CUDA_BF16 || mma == BOAT_MMA_TF32;
    for (int i = 0; i < 4; ++i) {
        const boat_tensor_t* w = a->param[WQ + i];
        if (w->device == BOAT_DEVICE_CUDA || w->dtype != BOAT_DTYPE_FLOAT32 || w->nelements != n) goto fail;
        p->w[i] = dev_alloc(n * storage_size(type));
        p->w_owned[i] = p->w[i] != NULL;
        if (!p->w[i]) goto fail;
        if (convert) {
            p->raw_w[i] = dev_alloc(n * sizeof(float));
            if (!p->raw_w[i]) goto fail;
        }
        p->late[i] = true;
        const boat_tensor_t* b = a->param[BQ + i];
        if (with_bias && b) {
            if (b->device == BOAT_DEVICE_CUDA || b->dtype != BOAT_DTYPE_FLOAT32) goto fail;
            p->b[i] = (float*)dev_alloc(b->nelements * sizeof(float));
            p->b_owned[i] = p->b[i] != NULL;
            if (!p->b[i]) goto fail;
        }
    }
    return true;
fail:
    release_params(p);
    return false;
}

/* Uploads and converts weights lo..hi (with their biases) prepared by prepare_late_params; a no-op
 * for parameters that were staged up front. */
static bool stage_param_range(boat_attention_t* a, int type, staged_params_t* p, int lo, int hi) {
    const int64_t n = (int64_t)(a->config.hidden_size * a->config.hidden_size);
    for (int i = lo; i <= hi; ++i) {
        if (!p->late[i]) continue;
        p->late[i] = false;
        void* land = p->raw_w[i] ? p->raw_w[i] : p->w[i];
        int rc = boat_cuda_upload_async(land, a->param[WQ + i]->data, (size_t)n * sizeof(float));
        if (rc == 0 && p->b[i]) rc = boat_cuda_upload_async(p->b[i], a->param[BQ + i]->data, a->param[BQ + i]->nbytes);
        if (rc == 0) rc = boat_cuda_join_uploads();
        if (rc == 0 && type == BOAT_CUDA_BF16) rc = boat_cuda_cast(p->w[i], BOAT_CUDA_BF16, land, BOAT_CUDA_F32, n);
        else if (rc == 0 && p->raw_w[i]) rc = boat_cuda_round_tf32((float*)p->w[i], (const float*)land, n);
        if (boat_report("parameter upload", rc) != 0) return false;
    }
    return true;
}

/* ---- host tensors: transfers overlapped with the arithmetic ------------------------------------
 * With host tensors a step moves about a gigabyte over PCIe (inputs and parameters up, outputs
 * and gradients down), more time than the kernels take.  Everything that is computed per token
 * row or per (batch, head) unit - projections, attention core, input gradients - is therefore
 * done in chunks of whole batch entries: while chunk c is computed, chunk c+1 is uploaded and
 * chunk c-1 downloaded, on the copy streams of boat_cuda_upload_async / _download_async.  Only
 * the weight and bias gradients, which sum over all rows, run once at the end.  The arithmetic
 * per row is the same as in the one-piece path.  A host layer's parameters go up on the upload
 * stream as well, behind the first chunk and in the order the kernels need them. */
enum { MAX_CHUNKS = 8 };

static bool on_host(const boat_tensor_t* t) { return t->device != BOAT_DEVICE_CUDA; }

/* BOAT_HOST_PIPELINE=0 in the environment selects the one-piece path for host tensors too. */
static bool pipeline_enabled(void) {
    static int enabled = -1;
    if (enabled < 0) {
        const char* e = getenv("BOAT_HOST_PIPELINE");
        enabled = !(e && e[0] == '0');
    }
    return enabled != 0;
}

/* First batch entry of chunk c when B entries are cut into n chunks. */
static int64_t chunk_begin(int64_t B, int n, int c) { return B * c / n; }

/* Rows [r0, r0+nr) of host tensor `t` (row length H) into the same rows of `dst` (device,
 * storage `type`): upload, then cast through `raw` (device, the tensor's own storage) when the
 * types differ, then TF32 rounding when the arithmetic wants it.  Everything after the upload
 * is ordered behind it on the library stream. */
static int stage_rows(const boat_tensor_t* t, int mma, int type, void* dst, void* raw, int64_t r0, int64_t nr,
                      int64_t H) {
    const int have = storage_of(t->dtype);
    const size_t hsz = storage_size(have), tsz = storage_size(type);
    const int64_t n = nr * H;
    char* d = (char*)dst + (size_t)(r0 * H) * tsz;
    const char* src = (const char*)t->data + (size_t)(r0 * H) * hsz;
    int rc;
    if (have == type) {
        rc = boat_cuda_upload_async(d, src, (size_t)n * hsz);
        if (rc == 0) rc = boat_cuda_join_uploads();
    } else {
        char* r = (char*)raw + (size_t)(r0 * H) * hsz;
        rc = boat_cuda_upload_async(r, src, (size_t)n * hsz);
        if (rc == 0) rc = boat_cuda_join_uploads();
        if (rc == 0) rc = boat_cuda_cast(d, type, r, have, n);
    }
    if (rc == 0 && mma == BOAT_MMA_TF32) rc = boat_cuda_round_tf32((float*)d, (const float*)d, n);
    return boat_report("chunk upload", rc);
}

/* Forward for host inputs cut into at least two chunks.  Fills the layer's forward state like the
 * one-piece path.  A chunk is a run of whole pieces of a->gran units, i.e. of gran*S/nh token rows. */
static boat_tensor_t* forward_pipelined(boat_attention_t* a, const boat_tensor_t* const in[3], int mma, int type,
                                        staged_params_t* p) {
    const int64_t H = (int64_t)a->config.hidden_size, nh = (int64_t)a->config.num_heads;
    const int64_t hs = (int64_t)a->config.head_size, S = a->S, T = a->T;
    const int64_t G = a->units / a->gran, grows = a->gran * S / nh;      /* pieces, token rows per piece */
    const size_t tsz = storage_size(type), act_bytes = (size_t)T * (size_t)H * tsz;
    const int out_type = storage_of(in[0]->dtype);
    const size_t osz = storage_size(out_type);
    const int nchunk = (int)(G < MAX_CHUNKS ? G : MAX_CHUNKS);
    void* raw[3] = {NULL, NULL, NULL};
    void* d_out = NULL;
    bool ok = false;
    boat_tensor_t* result = boat_tensor_create_uninit(in[0]->shape, in[0]->ndim, in[0]->dtype, BOAT_DEVICE_CPU);
    if (!result) return NULL;

    for (int i = 0; i < 3; ++i) {
        int same = -1;
        for (int j = 0; j < i; ++j)
            if (in[j] == in[i]) same = j;
        if (same >= 0) {
            a->d_in[i] = a->d_in[same];
            a->d_in_owned[i] = false;
            continue;
        }
        a->d_in[i] = dev_alloc(act_bytes);
        a->d_in_owned[i] = a->d_in[i] != NULL;
        if (!a->d_in[i]) goto done;
        if (storage_of(in[i]->dtype) != type) {
            raw[i] = dev_alloc((size_t)T * (size_t)H * storage_size(storage_of(in[i]->dtype)));
            if (!raw[i]) goto done;
        }
    }
    for (int i = 0; i < 3; ++i) {
        a->d_proj[i] = dev_alloc(act_bytes);
        if (!a->d_proj[i]) goto done;
    }
    a->d_ctx = dev_alloc(act_bytes);
    a->d_lse = (float*)dev_alloc((size_t)a->units * S * sizeof(float));
    d_out = dev_alloc((size_t)T * (size_t)H * osz);
    if (!a->d_ctx || !a->d_lse || !d_out) goto done;
    if (boat_report("copy streams", boat_cuda_copies_after_compute()) != 0) goto done;

    for (int c = 0; c < nchunk; ++c) {
        const int64_t b0 = chunk_begin(G, nchunk, c), b1 = chunk_begin(G, nchunk, c + 1);
        const int64_t r0 = b0 * grows, nr = (b1 - b0) * grows;
        const size_t off = (size_t)(r0 * H) * tsz, ooff = (size_t)(r0 * H) * osz;
        for (int i = 0; i < 3; ++i)
            if (a->d_in_owned[i] && stage_rows(in[i], mma, type, a->d_in[i], raw[i], r0, nr, H) != 0) goto done;
        if (c == 0 && !stage_param_range(a, type, p, WQ, WV)) goto done;
        for (int i = 0; i < 3; ++i) {
            if (boat_report("projection", boat_cuda_gemm(mma, 0, 0, nr, H, H, (char*)a->d_in[i] + off, H, p->w[i], H, type,
                                                         (char*)a->d_proj[i] + off, H, feed_type(mma, type), p->b[i])) != 0)
                goto done;
        }
        if (boat_report("attention core",
                        boat_cuda_attn_fwd(mma, (b1 - b0) * a->gran, S, hs, a->config.causal_mask, 1.0f / sqrtf((float)hs),
                                           (char*)a->d_proj[0] + off, (char*)a->d_proj[1] + off, (char*)a->d_proj[2] + off,
                                           type, (char*)a->d_ctx + off, a->d_lse + b0 * a->gran * S)) != 0)
            goto done;
        if (c == 0 && !stage_param_range(a, type, p, WO, WO)) goto done;
        if (boat_report("output projection", boat_cuda_gemm(mma, 0, 0, nr, H, H, (char*)a->d_ctx + off, H, p->w[WO], H, type,
                                                            (char*)d_out + ooff, H, out_type, p->b[WO])) != 0)
            goto done;
        if (boat_report("chunk download", boat_cuda_download_async((char*)result->data + ooff, (char*)d_out + ooff,
                                                                   (size_t)(nr * H) * osz)) != 0)
            goto done;
    }
    ok = true;
done:
    if (boat_report("forward", boat_cuda_sync()) != 0) ok = false;     /* copies done before anything is freed */
    for (int i = 0; i < 3; ++i) dev_free(raw[i]);
    dev_free(d_out);
    if (!ok) {
        boat_tensor_free(result);
        result = NULL;
    }
    return result;
}


/* Backward for a host grad_output and host inputs in at least two chunks: dOut up, d(ctx),
 * attention core and the three input gradients per chunk, input gradients down while the next
 * chunk is computed; weight and bias gradients over all rows at the end. */
static bool backward_pipelined(boat_attention_t* a, const boat_tensor_t* grad_output, int mma, int type,
                               staged_params_t* p, float* const d_dw[4], float* const d_db[4],
                               boat_tensor_t* gin[3]) {
    const int64_t H = (int64_t)a->config.hidden_size, nh = (int64_t)a->config.num_heads;
    const int64_t hs = (int64_t)a->config.head_size, S = a->S, T = a->T;
    /* The backward moves three times as much down as up and its kernels have time to spare, so its
     * pieces may be finer than the forward's: halves of a piece as long as those are still whole
     * units owning whole token rows, until there are MAX_CHUNKS chunks - a shorter wait for the first
     * download and a shorter last one. */
    int64_t gran = a->gran;
    while (a->units / gran < MAX_CHUNKS && gran % 2 == 0 && ((gran / 2) * S) % nh == 0) gran /= 2;
    const int64_t G = a->units / gran, grows = gran * S / nh;
    const size_t tsz = storage_size(type), act_bytes = (size_t)T * (size_t)H * tsz;
    const bool bias = a->param[BQ] != NULL;
    const int nchunk = (int)(G < MAX_CHUNKS ? G : MAX_CHUNKS);
    void *d_go = NULL, *raw_go = NULL, *d_dctx = NULL, *scratch = NULL;
    void *d_dproj[3] = {NULL, NULL, NULL}, *d_dx[3] = {NULL, NULL, NULL};
    int out_type[3];
    bool ok = false;
    size_t scratch_bytes = 0;

    d_go = dev_alloc(act_bytes);
    d_dctx = dev_alloc(act_bytes);
    if (!d_go || !d_dctx) goto done;
    if (storage_of(grad_output->dtype) != type) {
        raw_go = dev_alloc((size_t)T * (size_t)H * storage_size(storage_of(grad_output->dtype)));
        if (!raw_go) goto done;
    }
    for (int i = 0; i < 3; ++i) {
        const boat_tensor_t* x = a->cache_in[i];
        out_type[i] = storage_of(x->dtype);
        d_dproj[i] = dev_alloc(act_bytes);
        d_dx[i] = dev_alloc((size_t)T * (size_t)H * storage_size(out_type[i]));
        gin[i] = boat_tensor_create_uninit(x->shape, x->ndim, x->dtype, BOAT_DEVICE_CPU);
        if (!d_dproj[i] || !d_dx[i] || !gin[i]) goto done;
    }
    for (int c = 0; c < nchunk; ++c) {              /* the largest chunk decides the scratch size */
        const int64_t nb = chunk_begin(G, nchunk, c + 1) - chunk_begin(G, nchunk, c);
        const size_t need = boat_cuda_attn_bwd_scratch_bytes(mma, nb * gran, S, hs);
        if (need > scratch_bytes) scratch_bytes = need;
    }
    scratch = dev_alloc(scratch_bytes ? scratch_bytes : 256);
    if (!scratch) goto done;
    if (boat_report("copy streams", boat_cuda_copies_after_compute()) != 0) goto done;

    for (int c = 0; c < nchunk; ++c) {
        const int64_t b0 = chunk_begin(G, nchunk, c), b1 = chunk_begin(G, nchunk, c + 1);
        const int64_t r0 = b0 * grows, nr = (b1 - b0) * grows;
        const size_t off = (size_t)(r0 * H) * tsz;
        if (stage_rows(grad_output, mma, type, d_go, raw_go, r0, nr, H) != 0) goto done;
        /* Wo behind the first chunk of dOut; the other weights behind it, needed only after the
         * attention-core backward of that chunk */
        if (c == 0 && !stage_param_range(a, type, p, WO, WO)) goto done;
        /* d(ctx) = dOut . Wo^T */
        if (boat_report("dOut.Wo^T", boat_cuda_gemm(mma, 0, 1, nr, H, H, (char*)d_go + off, H, p->w[WO], H, type,
                                                    (char*)d_dctx + off, H, feed_type(mma, type), NULL)) != 0)
            goto done;
        if (boat_report("attention core backward",
                        boat_cuda_attn_bwd(mma, (b1 - b0) * gran, S, hs, a->config.causal_mask, 1.0f / sqrtf((float)hs),
                                           (char*)a->d_proj[0] + off, (char*)a->d_proj[1] + off, (char*)a->d_proj[2] + off,
                                           (char*)a->d_ctx + off, (char*)d_dctx + off, a->d_lse + b0 * gran * S, type,
                                           (char*)d_dproj[0] + off, (char*)d_dproj[1] + off, (char*)d_dproj[2] + off,
                                           scratch, scratch_bytes)) != 0)
            goto done;
        if (c == 0 && !stage_param_range(a, type, p, WQ, WV)) goto done;
        for (int i = 0; i < 3; ++i) {
            const size_t osz = storage_size(out_type[i]), ooff = (size_t)(r0 * H) * osz;
            /* dX = dP . W^T */
            if (boat_report("dX", boat_cuda_gemm(mma, 0, 1, nr, H, H, (char*)d_dproj[i] + off, H, p->w[i], H, type,
                                                 (char*)d_dx[i] + ooff, H, out_type[i], NULL)) != 0)
                goto done;
            if (boat_report("chunk download", boat_cuda_download_async((char*)gin[i]->data + ooff, (char*)d_dx[i] + ooff,
                                                                       (size_t)(nr * H) * osz)) != 0)
                goto done;
        }
    }
    /* sums over all rows: dWo = ctx^T . dOut, dbo = colsum(dOut), dW = X^T . dP, db = colsum(dP) */
    if (boat_report("dWo", boat_cuda_gemm(mma, 1, 0, H, H, T, a->d_ctx, H, d_go, H, type, d_dw[WO], H, BOAT_CUDA_F32, NULL)) != 0) goto done;
    if (bias && boat_report("dbo", boat_cuda_colsum(d_go, type, T, H, d_db[WO])) != 0) goto done;
    for (int i = 0; i < 3; ++i) {
        if (boat_report("dW", boat_cuda_gemm(mma, 1, 0, H, H, T, a->d_in[i], H, d_dproj[i], H, type, d_dw[i], H, BOAT_CUDA_F32, NULL)) != 0) goto done;
        if (bias && boat_report("db", boat_cuda_colsum(d_dproj[i], type, T, H, d_db[i])) != 0) goto done;
    }
    if (a->device != BOAT_DEVICE_CUDA &&
        boat_report("gradient download", boat_cuda_download_async(a->grad_bucket->data, d_dw[0], a->grad_bucket->nbytes)) != 0)
        goto done;
    ok = true;
done:
    if (boat_report("backward", boat_cuda_sync()) != 0) ok = false;    /* copies done before anything is freed */
    dev_free(scratch);
    for (int i = 0; i < 3; ++i) {
        dev_free(d_dproj[i]);
        dev_free(d_dx[i]);
    }
    dev_free(d_dctx);
    dev_free(raw_go);
    dev_free(d_go);
    return ok;
}

/* ---- create / free ------------------------------------------------------------------------ */

static boat_tensor_t* new_weight(size_t in, size_t out) {
    const int64_t shape[2] = {(int64_t)in, (int64_t)out};
    boat_tensor_t* w = boat_tensor_create(shape, 2, BOAT_DTYPE_FLOAT32, BOAT_DEVICE_CPU);
    if (!w) return NULL;
    /* Xavier/Glorot uniform from rand(), element order and formula of the reference
     * (attention.c:100-104), so a seeded caller sees the same initial weights. */
    float* v = (float*)w->data;
    float bound = sqrtf(2.0f / (float)(in + out));
    for (size_t i = 0; i < w->nelements; ++i) v[i] = ((float)rand() / RAND_MAX) * 2.0f * bound - bound;
    return w;
}

boat_attention_t* boat_attention_create(const boat_attention_config_t* config) {
    if (!config || config->hidden_size == 0 || config->num_heads == 0) return NULL;
    if (config->hidden_size % config->num_heads != 0) return NULL;
    boat_attention_t* a = (boat_attention_t*)boat_calloc(sizeof *a, BOAT_DEVICE_CPU);
    if (!a) return NULL;
    a->config = *config;
    if (config->head_size == 0) a->config.head_size = config->hidden_size / config->num_heads;
    a->device = BOAT_DEVICE_CPU;
    a->precision = env_precision();
    size_t H = config->hidden_size;
    for (int i = 0; i < 4; ++i) {
        a->param[WQ + i] = new_weight(H, H);
        if (!a->param[WQ + i]) goto fail;
    }
    if (config->use_bias) {
        const int64_t shape[1] = {(int64_t)H};
        for (int i = 0; i < 4; ++i) {
            a->param[BQ + i] = boat_tensor_create(shape, 1, BOAT_DTYPE_FLOAT32, BOAT_DEVICE_CPU);
            if (!a->param[BQ + i]) goto fail;
        }
    }
    return a;
fail:
    boat_attention_free(a);
    return NULL;
}

static void drop_shadow(boat_attention_t* a) {
    dev_free(a->shadow_w);
    a->shadow_w = NULL;
    a->shadow_fresh = false;
}

void boat_attention_free(boat_attention_t* a) {
    if (!a) return;
    drop_forward_state(a);
    drop_shadow(a);
    for (int i = 0; i < NPARAM; ++i) {
        if (a->param[i]) boat_tensor_free(a->param[i]);
        if (a->grad[i]) boat_tensor_free(a->grad[i]);
    }
    if (a->grad_bucket) boat_tensor_free(a->grad_bucket);
    boat_free(a);
}

/* ---- forward ------------------------------------------------------------------------------- */

/* The step itself, for T token rows holding `units` (batch, head) units of sequence length S; `gran`
 * units form one indivisible piece when host tensors are moved in chunks.  Inputs are [.., H]
 * tensors of T*H elements each; the result has the query's shape. */
static boat_tensor_t* forward_rows(boat_attention_t* a, const boat_tensor_t* query, const boat_tensor_t* key,
                                   const boat_tensor_t* value, int64_t T, int64_t S, int64_t units, int64_t gran) {
    const boat_tensor_t* in[3] = {query, key, value};
    const int64_t H = (int64_t)a->config.hidden_size, hs = (int64_t)a->config.head_size;
    if (boat_report("CUDA start-up", boat_cuda_init(-1)) != 0) return NULL;

    /* Take the new inputs before releasing the old ones: they may be the same tensors. */
    for (int i = 0; i < 3; ++i) boat_tensor_ref((boat_tensor_t*)in[i]);
    drop_forward_state(a);
    for (int i = 0; i < 3; ++i) a->cache_in[i] = (boat_tensor_t*)in[i];

    const int mma = pick_mma(a, query);
    const int type = mma == BOAT_MMA_BF16 ? BOAT_CUDA_BF16 : BOAT_CUDA_F32;
    const size_t act_bytes = (size_t)T * (size_t)H * storage_size(type);
    a->mma = mma;
    a->type = type;
    a->T = T;
    a->S = S;
    a->units = units;
    a->gran = gran;

    staged_params_t p;
    void* d_out = NULL;
    boat_tensor_t* result = NULL;
    const bool pipelined = units / gran >= 2 && pipeline_enabled() && on_host(query) && on_host(key) && on_host(value);
    /* a host layer's parameters of a chunked call are brought up inside it, behind the first chunk */
    if (!(pipelined && a->device != BOAT_DEVICE_CUDA && prepare_late_params(a, mma, type, true, &p)) &&
        !stage_params(a, mma, type, false, &p))
        goto done;
    if (pipelined) {
        result = forward_pipelined(a, in, mma, type, &p);
        if (result) a->cached = true;
        goto done;
    }

    for (int i = 0; i < 3; ++i) {
        int same = -1;
        for (int j = 0; j < i; ++j)
            if (in[j] == in[i]) same = j;
        if (same >= 0) {
            a->d_in[i] = a->d_in[same];
            a->d_in_owned[i] = false;
        } else {
            a->d_in[i] = stage_operand(in[i], mma, type, &a->d_in_owned[i]);
            if (!a->d_in[i]) goto done;
        }
    }
    for (int i = 0; i < 3; ++i) {
        a->d_proj[i] = dev_alloc(act_bytes);
        if (!a->d_proj[i]) goto done;
    }
    /* the three projections (attention.c:363-365) as one launch */
    if (boat_report("projections", boat_cuda_gemm_grouped(mma, 0, 0, 3, T, H, H, (const void* const*)a->d_in, H,
                                                          (const void* const*)p.w, H, type, a->d_proj, H,
                                                          feed_type(mma, type), (const float* const*)p.b)) != 0)
        goto done;
    a->d_ctx = dev_alloc(act_bytes);
    a->d_lse = (float*)dev_alloc((size_t)units * S * sizeof(float));
    if (!a->d_ctx || !a->d_lse) goto done;
    /* [B,S,H] viewed as [B*nh, S, hs]: the head split is a reshape (attention.c:393-397). */
    if (boat_report("attention core", boat_cuda_attn_fwd(mma, units, S, hs, a->config.causal_mask,
                                                         1.0f / sqrtf((float)hs), a->d_proj[0], a->d_proj[1],
                                                         a->d_proj[2], type, a->d_ctx, a->d_lse)) != 0)
        goto done;
    /* The output projection writes the caller's dtype directly when that is a device
     * storage type the GEMM can emit. */
    {
        int out_type = storage_of(query->dtype);
        if (query->device == BOAT_DEVICE_CUDA) {
            /* a CUDA result is the GEMM's own output buffer: no copy */
            result = boat_tensor_create_uninit(query->shape, query->ndim, query->dtype, BOAT_DEVICE_CUDA);
            if (!result) goto done;
            if (boat_report("output projection", boat_cuda_gemm(mma, 0, 0, T, H, H, a->d_ctx, H, p.w[WO], H, type,
                                                                result->data, H, out_type, p.b[WO])) != 0) {
                boat_tensor_free(result);
                result = NULL;
                goto done;
            }
        } else {
            d_out = dev_alloc((size_t)T * H * storage_size(out_type));
            if (!d_out) goto done;
            if (boat_report("output projection", boat_cuda_gemm(mma, 0, 0, T, H, H, a->d_ctx, H, p.w[WO], H, type,
                                                                d_out, H, out_type, p.b[WO])) != 0)
                goto done;
            result = emit_out(query->shape, query->ndim, query, d_out, out_type);
        }
    }
    if (result) a->cached = true;
done:
    dev_free(d_out);
    release_params(&p);
    if (!result) {
        /* keep the input references (the reference does, attention.c:355-372) but no
         * half-built device state */
        boat_tensor_t* keep[3] = {a->cache_in[0], a->cache_in[1], a->cache_in[2]};
        for (int i = 0; i < 3; ++i) a->cache_in[i] = NULL;
        drop_forward_state(a);
        for (int i = 0; i < 3; ++i) a->cache_in[i] = keep[i];
    }
    return result;
}

boat_tensor_t* boat_attention_forward(boat_attention_t* a, const boat_tensor_t* query, const boat_tensor_t* key,
                                      const boat_tensor_t* value, const boat_tensor_t* attention_mask) {
    (void)attention_mask;                       /* ignored, as in the reference (attention.c:1022-1025) */
    if (!a || !query || !key || !value) return NULL;
    const boat_tensor_t* in[3] = {query, key, value};
    const int64_t H = (int64_t)a->config.hidden_size, nh = (int64_t)a->config.num_heads;
    const int64_t hs = (int64_t)a->config.head_size;
    if (query->ndim != 3 || nh * hs != H) return NULL;
    const int64_t B = query->shape[0], S = query->shape[1];
    for (int i = 0; i < 3; ++i) {
        if (!dtype_ok(in[i]->dtype) || in[i]->ndim != 3 || in[i]->shape[0] != B || in[i]->shape[1] != S ||
            in[i]->shape[2] != H)
            return NULL;
    }
    return forward_rows(a, query, key, value, B * S, S, B * nh, nh);
}

/* A contiguous range of (batch, head) units of a larger [B,S,H] problem, given only the token rows
 * that range touches.  The head split is a reshape (reference attention.c:393-397): with nh
 * dividing S, unit u of the flattened [B*S, H] input is exactly its token rows
 * [u*S/nh, (u+1)*S/nh), so n consecutive units are n*S/nh consecutive rows, and the projections
 * (row-wise maps) shard the same way. */
boat_tensor_t* boat_attention_forward_units(boat_attention_t* a, const boat_tensor_t* query, const boat_tensor_t* key,
                                            const boat_tensor_t* value, int64_t seq_len) {
    if (!a || !query || !key || !value || seq_len <= 0) return NULL;
    const boat_tensor_t* in[3] = {query, key, value};
    const int64_t H = (int64_t)a->config.hidden_size, nh = (int64_t)a->config.num_heads;
    const int64_t hs = (int64_t)a->config.head_size;
    if (nh * hs != H) return NULL;
    if (seq_len % nh != 0) {
        fprintf(stderr, "boat_attention_forward_units: the sequence length (%lld) must be a multiple of the head "
                        "count (%lld) for units to own whole token rows\n", (long long)seq_len, (long long)nh);
        return NULL;
    }
    const int64_t unit_rows = seq_len / nh;
    if (query->ndim != 2 || query->shape[1] != H || query->shape[0] <= 0 || query->shape[0] % unit_rows != 0) return NULL;
    const int64_t R = query->shape[0];
    for (int i = 0; i < 3; ++i)
        if (!dtype_ok(in[i]->dtype) || in[i]->ndim != 2 || in[i]->shape[0] != R || in[i]->shape[1] != H) return NULL;
    return forward_rows(a, query, key, value, R, seq_len, R / unit_rows, 1);
}

/* ---- backward ------------------------------------------------------------------------------ */

static bool ensure_grads(boat_attention_t* a) {
    if (a->grad_bucket && a->grad_bucket->device == a->device) return true;
    for (int i = 0; i < NPARAM; ++i) {
        if (a->grad[i]) boat_tensor_free(a->grad[i]);
        a->grad[i] = NULL;
    }
    if (a->grad_bucket) boat_tensor_free(a->grad_bucket);
    const int64_t H = (int64_t)a->config.hidden_size;
    const bool bias = a->param[BQ] != NULL;
    const int64_t total[1] = {4 * H * H + (bias ? 4 * H : 0)};
    a->grad_bucket = boat_tensor_create(total, 1, BOAT_DTYPE_FLOAT32, a->device);
    if (!a->grad_bucket) return false;
    const int64_t wshape[2] = {H, H}, bshape[1] = {H};
    for (int i = 0; i < 4; ++i) {
        a->grad[WQ + i] = boat_tensor_window(a->grad_bucket, (size_t)i * H * H * 4, wshape, 2);
        if (!a->grad[WQ + i]) return false;
        if (bias) {
            a->grad[BQ + i] = boat_tensor_window(a->grad_bucket, (size_t)(4 * H * H + i * H) * 4, bshape, 1);
            if (!a->grad[BQ + i]) return false;
        }
    }
    return true;
}

bool boat_attention_backward(boat_attention_t* a, const boat_tensor_t* grad_output, boat_tensor_t** grad_query,
                             boat_tensor_t** grad_key, boat_tensor_t** grad_value) {
    if (!a || !grad_output) {
        printf("[ERROR] boat_attention_backward: invalid arguments\n");
        return false;
    }
    if (!a->cached) {
        printf("[ERROR] boat_attention_backward: missing cached tensors\n");
        return false;
    }
    const int64_t H = (int64_t)a->config.hidden_size;
    const int64_t hs = (int64_t)a->config.head_size, S = a->S, T = a->T, units = a->units;
    if (!dtype_ok(grad_output->dtype) || (int64_t)grad_output->nelements != T * H) {
        printf("[ERROR] boat_attention_backward: grad_output does not match the cached forward\n");
        return false;
    }
    const int mma = a->mma, type = a->type;
    const size_t act_bytes = (size_t)T * (size_t)H * storage_size(type);
    const bool bias = a->param[BQ] != NULL;
    bool ok = false, go_owned = false;
    staged_params_t p;
    memset(&p, 0, sizeof p);
    void *d_go = NULL, *d_dctx = NULL, *d_dproj[3] = {NULL, NULL, NULL}, *scratch = NULL, *d_dx = NULL;
    float* d_bucket = NULL;
    boat_tensor_t* gin[3] = {NULL, NULL, NULL};
    size_t scratch_bytes;

    if (!ensure_grads(a)) goto done;
    /* gradient sums of this layer's previous step still on the communication stream read the bucket
     * this step is about to overwrite.  (Sums other layers have under way - an encoder block starts
     * its dense layers' before this call - are not waited for.) */
    if (a->sums_begun && boat_cuda_allreduce_pending() &&
        boat_report("gradient all-reduce", boat_cuda_allreduce_join()) != 0)
        goto done;
    a->sums_begun = false;
    const bool pipelined = units / a->gran >= 2 && pipeline_enabled() && on_host(grad_output) && on_host(a->cache_in[0]) &&
                           on_host(a->cache_in[1]) && on_host(a->cache_in[2]);
    if (!(pipelined && a->device != BOAT_DEVICE_CUDA && prepare_late_params(a, mma, type, false, &p))) {
        /* (a host layer's parameters of a chunked call are brought up inside it, behind the first chunk) */
        const bool staged = stage_params(a, mma, type, true, &p);
        a->shadow_fresh = false;                /* one backward per forward may trust the forward's copies */
        if (!staged) goto done;
    }
    /* gradients are produced in HBM; a host layer receives them with one copy at the end */
    d_bucket = a->device == BOAT_DEVICE_CUDA ? (float*)a->grad_bucket->data
                                             : (float*)dev_alloc(a->grad_bucket->nbytes);
    if (!d_bucket) goto done;
    float* d_dw[4];
    float* d_db[4];
    for (int i = 0; i < 4; ++i) {
        d_dw[i] = d_bucket + (size_t)i * H * H;
        d_db[i] = bias ? d_bucket + (size_t)4 * H * H + (size_t)i * H : NULL;
    }
    if (pipelined) {
        ok = backward_pipelined(a, grad_output, mma, type, &p, d_dw, d_db, gin);
        goto done;
    }
    d_go = stage_operand(grad_output, mma, type, &go_owned);
    if (!d_go) goto done;

    /* output projection: d(ctx) = dOut . Wo^T,  dWo = ctx^T . dOut,  dbo = colsum(dOut) */
    d_dctx = dev_alloc(act_bytes);
    if (!d_dctx) goto done;
    if (boat_report("dOut.Wo^T", boat_cuda_gemm(mma, 0, 1, T, H, H, d_go, H, p.w[WO], H, type, d_dctx, H, feed_type(mma, type), NULL)) != 0) goto done;
    if (boat_report("dWo", boat_cuda_gemm(mma, 1, 0, H, H, T, a->d_ctx, H, d_go, H, type, d_dw[WO], H, BOAT_CUDA_F32, NULL)) != 0) goto done;
    if (bias && boat_report("dbo", boat_cuda_colsum(d_go, type, T, H, d_db[WO])) != 0) goto done;
    /* Data parallel with overlap: dWo and dbo are final here, long before the step ends - their
     * sum over the ranks runs under the attention-core backward. */
    const bool overlap = a->grad_overlap != 0 && a->device == BOAT_DEVICE_CUDA && boat_cuda_comm_world() > 1;
    a->rest_pending = false;
    if (overlap) {
        float* piece[2] = {d_dw[WO], d_db[WO]};
        const int64_t count[2] = {H * H, bias ? H : 0};
        if (boat_report("gradient all-reduce", boat_cuda_allreduce_begin(piece, count, 2)) != 0) goto done;
        a->sums_begun = true;
    }

    /* attention core */
    for (int i = 0; i < 3; ++i) {
        d_dproj[i] = dev_alloc(act_bytes);
        if (!d_dproj[i]) goto done;
    }
    scratch_bytes = boat_cuda_attn_bwd_scratch_bytes(mma, units, S, hs);
    scratch = dev_alloc(scratch_bytes);
    if (!scratch) goto done;
    if (boat_report("attention core backward",
                    boat_cuda_attn_bwd(mma, units, S, hs, a->config.causal_mask, 1.0f / sqrtf((float)hs),
                                       a->d_proj[0], a->d_proj[1], a->d_proj[2], a->d_ctx, d_dctx, a->d_lse, type,
                                       d_dproj[0], d_dproj[1], d_dproj[2], scratch, scratch_bytes)) != 0)
        goto done;

    /* input projections: dW = X^T . dP and db = colsum(dP) first - with overlap their sum over
     * the ranks then runs under the three dX = dP . W^T GEMMs that follow */
    if (boat_report("dW", boat_cuda_gemm_grouped(mma, 1, 0, 3, H, H, T, (const void* const*)a->d_in, H,
                                                 (const void* const*)d_dproj, H, type, (void* const*)d_dw, H,
                                                 BOAT_CUDA_F32, NULL)) != 0)
        goto done;
    if (bias && boat_report("db", boat_cuda_colsum_multi((const void* const*)d_dproj, type, T, H, d_db, 3)) != 0) goto done;
    if (overlap && a->grad_overlap == 1) {
        float* piece[2] = {d_dw[WQ], d_db[WQ]};            /* dWq|dWk|dWv and dbq|dbk|dbv are contiguous */
        const int64_t count[2] = {3 * H * H, bias ? 3 * H : 0};
        if (boat_report("gradient all-reduce", boat_cuda_allreduce_begin(piece, count, 2)) != 0) goto done;
    } else if (overlap) {
        a->rest_pending = true;
    }
    const bool yield = overlap && a->grad_overlap == 1;      /* a sum was just started beside these GEMMs */
    if (yield) boat_cuda_gemm_set_yielding(1);
    {
        /* dX = dP . W^T for the three inputs: one launch when they share device and dtype */
        const boat_tensor_t* x0 = a->cache_in[0];
        bool together = x0->device == BOAT_DEVICE_CUDA;
        for (int i = 1; i < 3; ++i)
            together = together && a->cache_in[i]->device == BOAT_DEVICE_CUDA && a->cache_in[i]->dtype == x0->dtype;
        if (together) {
            void* target[3];
            for (int i = 0; i < 3; ++i) {
                const boat_tensor_t* x = a->cache_in[i];
                /* a CUDA gradient is the GEMM's own output buffer: no copy */
                gin[i] = boat_tensor_create_uninit(x->shape, x->ndim, x->dtype, BOAT_DEVICE_CUDA);
                if (!gin[i]) goto done;
                target[i] = gin[i]->data;
            }
            if (boat_report("dX", boat_cuda_gemm_grouped(mma, 0, 1, 3, T, H, H, (const void* const*)d_dproj, H,
                                                         (const void* const*)p.w, H, type, target, H,
                                                         storage_of(x0->dtype), NULL)) != 0)
                goto done;
        } else {
            for (int i = 0; i < 3; ++i) {
                const boat_tensor_t* x = a->cache_in[i];
                int out_type = storage_of(x->dtype);
                void* dx_target;
                if (x->device == BOAT_DEVICE_CUDA) {
                    gin[i] = boat_tensor_create_uninit(x->shape, x->ndim, x->dtype, BOAT_DEVICE_CUDA);
                    if (!gin[i]) goto done;
                    dx_target = gin[i]->data;
                } else {
                    d_dx = dev_alloc((size_t)T * H * storage_size(out_type));
                    if (!d_dx) goto done;
                    dx_target = d_dx;
                }
                if (boat_report("dX", boat_cuda_gemm(mma, 0, 1, T, H, H, d_dproj[i], H, p.w[i], H, type, dx_target, H, out_type, NULL)) != 0) goto done;
                if (x->device != BOAT_DEVICE_CUDA) {
                    gin[i] = emit_out(x->shape, x->ndim, x, d_dx, out_type);
                    dev_free(d_dx);
                    d_dx = NULL;
                    if (!gin[i]) goto done;
                }
            }
        }
    }
    if (a->device != BOAT_DEVICE_CUDA &&
        boat_report("gradient download", boat_cuda_memcpy_d2h(a->grad_bucket->data, d_bucket, a->grad_bucket->nbytes)) != 0)
        goto done;
    ok = true;
done:
    boat_cuda_gemm_set_yielding(0);
    dev_free(d_dx);
    dev_free(scratch);
    for (int i = 0; i < 3; ++i) dev_free(d_dproj[i]);
    dev_free(d_dctx);
    if (a->device != BOAT_DEVICE_CUDA) dev_free(d_bucket);
    if (go_owned) dev_free(d_go);
    release_params(&p);
    if (!ok) {
        for (int i = 0; i < 3; ++i)
            if (gin[i]) boat_tensor_free(gin[i]);
        return false;
    }
    boat_tensor_t** outp[3] = {grad_query, grad_key, grad_value};
    for (int i = 0; i < 3; ++i) {
        if (outp[i]) *outp[i] = gin[i];
        else boat_tensor_free(gin[i]);
    }
    return true;
}

/* ---- update / setters ------------------------------------------------------------------------ */

void boat_attention_update(boat_attention_t* a, float learning_rate) {
    if (!a || !a->grad_bucket) return;
    a->shadow_fresh = false;
    for (int i = 0; i < NPARAM; ++i) {
        boat_tensor_t *w = a->param[i], *g = a->grad[i];
        if (!w || !g) continue;
        int64_t n = (int64_t)w->nelements;
        if (a->device == BOAT_DEVICE_CUDA) {
            boat_report("SGD step", boat_cuda_axpy((float*)w->data, (const float*)g->data, -learning_rate, n));
            continue;
        }
        bool wo, go;
        float* dw = (float*)stage_in(w, BOAT_CUDA_F32, &wo);
        float* dg = (float*)stage_in(g, BOAT_CUDA_F32, &go);
        if (dw && dg && boat_report("SGD step", boat_cuda_axpy(dw, dg, -learning_rate, n)) == 0)
            boat_report("parameter download", boat_cuda_memcpy_d2h(w->data, dw, w->nbytes));
        if (wo) dev_free(dw);
        if (go) dev_free(dg);
    }
}

BOAT_NOINLINE void boat_attention_set_dropout(boat_attention_t* a, float dropout_prob) {
    if (a) a->config.dropout_prob = dropout_prob;
}

BOAT_NOINLINE void boat_attention_set_causal(boat_attention_t* a, bool causal) {
    if (a) a->config.causal_mask = causal;
}

/* ---- functional wrappers ----------------------------------------------------------------------- */

boat_tensor_t* boat_multihead_attention(const boat_tensor_t* input, size_t num_heads, float dropout_prob,
                                        bool causal_mask, const boat_tensor_t* attention_mask) {
    if (!input || input->ndim != 3 || num_heads == 0) return NULL;
    size_t H = (size_t)input->shape[2];
    if (H % num_heads != 0) return NULL;
    boat_attention_config_t cfg = {H, num_heads, H / num_heads, dropout_prob, causal_mask, true, false, 10000.0f};
    boat_attention_t* a = boat_attention_create(&cfg);
    if (!a) return NULL;
    boat_tensor_t* out = boat_attention_forward(a, input, input, input, attention_mask);
    boat_attention_free(a);
    return out;
}

boat_tensor_t* boat_scaled_dot_product_attention(const boat_tensor_t* query, const boat_tensor_t* key,
                                                 const boat_tensor_t* value, float scale_factor,
                                                 const boat_tensor_t* attention_mask, bool causal_mask,
                                                 float dropout_prob) {
    (void)attention_mask;
    (void)dropout_prob;
    if (!query || !key || !value) return NULL;
    if (query->ndim < 3 || key->ndim < 3 || value->ndim < 3) return NULL;
    if (query->ndim != 4 || key->ndim != 4 || value->ndim != 4) {
        /* the reference answers anything but 4-D with a copy of `value` (attention.c:905-917) */
        boat_tensor_t* copy = boat_tensor_create_uninit(value->shape, value->ndim, value->dtype, value->device);
        if (copy) boat_memory_copy(copy->data, value->data, value->nbytes, copy->device, value->device);
        return copy;
    }
    for (int d = 0; d < 4; ++d)
        if (key->shape[d] != query->shape[d] || value->shape[d] != query->shape[d]) return NULL;
    if (query->dtype != BOAT_DTYPE_FLOAT32 || key->dtype != BOAT_DTYPE_FLOAT32 || value->dtype != BOAT_DTYPE_FLOAT32)
        return NULL;                                 /* FP32 only (attention.c:934-938) */
    if (boat_report("CUDA start-up", boat_cuda_init(-1)) != 0) return NULL;
    const int64_t units = query->shape[0] * query->shape[1], S = query->shape[2], hs = query->shape[3];
    const boat_tensor_t* in[3] = {query, key, value};
    void* d[3] = {NULL, NULL, NULL};
    bool owned[3] = {false, false, false};
    boat_tensor_t* out = NULL;
    void* d_o = NULL;
    float* d_lse = NULL;
    for (int i = 0; i < 3; ++i) {
        d[i] = stage_in(in[i], BOAT_CUDA_F32, &owned[i]);
        if (!d[i]) goto done;
    }
    d_o = dev_alloc(query->nbytes);
    d_lse = (float*)dev_alloc((size_t)units * S * sizeof(float));
    if (!d_o || !d_lse) goto done;
    if (boat_report("attention core", boat_cuda_attn_fwd(BOAT_MMA_FP32, units, S, hs, causal_mask, scale_factor,
                                                         d[0], d[1], d[2], BOAT_CUDA_F32, d_o, d_lse)) != 0)
        goto done;
    out = emit_out(value->shape, 4, value, d_o, BOAT_CUDA_F32);
done:
    for (int i = 0; i < 3; ++i)
        if (owned[i]) dev_free(d[i]);
    dev_free(d_o);
    dev_free(d_lse);
    return out;
}

boat_tensor_t* boat_rotary_position_encoding(const boat_tensor_t* tensor, size_t seq_len, size_t head_size, float theta) {
    (void)tensor; (void)seq_len; (void)head_size; (void)theta;
    return NULL;
}

void boat_apply_rotary_embedding(boat_tensor_t* query, boat_tensor_t* key, size_t seq_len, size_t head_size, float theta) {
    (void)query; (void)key; (void)seq_len; (void)head_size; (void)theta;
}

/* ---- generic-layer adapter ---------------------------------------------------------------------- */

boat_attention_layer_t* boat_attention_layer_create(size_t hidden_size, size_t num_heads, float dropout_prob,
                                                    bool causal_mask) {
    if (num_heads == 0) return NULL;
    boat_attention_config_t cfg = {hidden_size, num_heads, hidden_size / num_heads, dropout_prob, causal_mask,
                                   true, false, 10000.0f};
    return boat_attention_create(&cfg);   /* rejects hidden_size % num_heads != 0 */
}

void boat_attention_layer_free(boat_attention_layer_t* layer) { boat_attention_free(layer); }

BOAT_NOINLINE boat_tensor_t* boat_attention_layer_forward(boat_attention_layer_t* layer, const boat_tensor_t* query,
                                                          const boat_tensor_t* key, const boat_tensor_t* value,
                                                          const boat_tensor_t* attention_mask) {
    return boat_attention_forward(layer, query, key, value, attention_mask);
}

BOAT_NOINLINE boat_tensor_t* boat_attention_layer_backward(boat_attention_layer_t* layer,
                                                           const boat_tensor_t* grad_output) {
    boat_tensor_t *gq = NULL, *gk = NULL, *gv = NULL;
    if (!boat_attention_backward(layer, grad_output, &gq, &gk, &gv)) return NULL;
    if (gk) boat_tensor_free(gk);
    if (gv) boat_tensor_free(gv);
    return gq;
}

BOAT_NOINLINE void boat_attention_layer_update(boat_attention_layer_t* layer, float learning_rate) {
    boat_attention_update(layer, learning_rate);
}

/* ---- accessors ------------------------------------------------------------------------------------ */

#define ACCESSOR(name, field, idx) \
    BOAT_NOINLINE boat_tensor_t* boat_attention_get_##name(const boat_attention_t* a) { return a ? a->field[idx] : NULL; }
/* a caller holding a weight tensor may write it: the converted copies are no longer trusted */
#define WEIGHT_ACCESSOR(name, idx)                                                         \
    BOAT_NOINLINE boat_tensor_t* boat_attention_get_##name(const boat_attention_t* a) {    \
        if (!a) return NULL;                                                               \
        ((boat_attention_t*)a)->shadow_fresh = false;                                      \
        return a->param[idx];                                                              \
    }
WEIGHT_ACCESSOR(weight_q, WQ) WEIGHT_ACCESSOR(weight_k, WK) WEIGHT_ACCESSOR(weight_v, WV) WEIGHT_ACCESSOR(weight_o, WO)
ACCESSOR(bias_q, param, BQ) ACCESSOR(bias_k, param, BK) ACCESSOR(bias_v, param, BV) ACCESSOR(bias_o, param, BO)
ACCESSOR(grad_weight_q, grad, WQ) ACCESSOR(grad_weight_k, grad, WK) ACCESSOR(grad_weight_v, grad, WV)
ACCESSOR(grad_weight_o, grad, WO) ACCESSOR(grad_bias_q, grad, BQ) ACCESSOR(grad_bias_k, grad, BK)
ACCESSOR(grad_bias_v, grad, BV) ACCESSOR(grad_bias_o, grad, BO)

/* ---- GPU-only additions ------------------------------------------------------------------------------ */

int boat_attention_to_device(boat_attention_t* a, boat_device_t device) {
    if (!a || (device != BOAT_DEVICE_CPU && device != BOAT_DEVICE_CUDA)) return 1;
    if (a->device == device) return 0;
    drop_shadow(a);
    boat_tensor_t* moved[NPARAM] = {0};
    for (int i = 0; i < NPARAM; ++i) {
        if (!a->param[i]) continue;
        moved[i] = boat_tensor_to_device(a->param[i], device);
        if (!moved[i]) {
            for (int j = 0; j < i; ++j)
                if (moved[j]) boat_tensor_free(moved[j]);
            return 2;
        }
    }
    boat_tensor_t* old_bucket = a->grad_bucket;
    for (int i = 0; i < NPARAM; ++i) {
        if (a->param[i]) boat_tensor_free(a->param[i]);
        a->param[i] = moved[i];
    }
    a->device = device;
    if (old_bucket) {
        /* carry the gradient values over to the new place */
        boat_tensor_ref(old_bucket);
        if (ensure_grads(a))
            boat_memory_copy(a->grad_bucket->data, old_bucket->data, old_bucket->nbytes, device, old_bucket->device);
        boat_tensor_free(old_bucket);
    }
    return 0;
}

int boat_attention_add_to_optimizer(boat_attention_t* a, boat_optimizer_t* optimizer) {
    if (!a || !optimizer) return 1;
    if (!ensure_grads(a)) return 2;          /* a new bucket starts out zero */
    for (int i = 0; i < NPARAM; ++i)
        if (a->param[i] && a->grad[i]) boat_optimizer_add_parameter(optimizer, a->param[i], a->grad[i]);
    return 0;
}

int boat_attention_set_precision(boat_attention_t* a, int mma) {
    if (!a || mma < -1 || mma > BOAT_MMA_BF16) return 1;
    a->precision = mma;
    return 0;
}

int boat_attention_get_precision(const boat_attention_t* a) { return a ? a->precision : -1; }

int boat_attention_grad_bucket(const boat_attention_t* a, float** data, size_t* nelements) {
    if (!a) return 1;
    if (data) *data = a->grad_bucket ? (float*)a->grad_bucket->data : NULL;
    if (nelements) *nelements = a->grad_bucket ? a->grad_bucket->nelements : 0;
    return 0;
}

int boat_attention_get_grad_overlap(const boat_attention_t* a) { return a ? a->grad_overlap : 0; }

int boat_attention_set_grad_overlap(boat_attention_t* a, int mode) {
    if (!a || mode < 0 || mode > 2) return 1;
    a->grad_overlap = mode;
    return 0;
}

int boat_attention_allreduce_grads(boat_attention_t* a) {
    if (!a || !a->grad_bucket) return 1;
    if (boat_cuda_comm_world() <= 1) return 0;
    if (a->device != BOAT_DEVICE_CUDA) {
        fprintf(stderr, "boat: gradient all-reduce needs the layer on BOAT_DEVICE_CUDA\n");
        return 2;
    }
    const int64_t H = (int64_t)a->config.hidden_size;
    const bool bias = a->param[BQ] != NULL;
    float* bucket = (float*)a->grad_bucket->data;
    if (a->rest_pending) {
        /* the backward started dWo|dbo itself and left the other group for now (mode 2) */
        float* piece[2] = {bucket, bucket + 4 * H * H};
        const int64_t count[2] = {3 * H * H, bias ? 3 * H : 0};
        a->rest_pending = false;
        if (boat_report("gradient all-reduce", boat_cuda_allreduce_begin(piece, count, 2)) != 0) return 3;
    } else if (!a->sums_begun) {
        /* nothing of this bucket is under way: all of it now, behind whatever other layers started */
        float* piece[1] = {bucket};
        const int64_t count[1] = {(int64_t)a->grad_bucket->nelements};
        if (boat_report("gradient all-reduce", boat_cuda_allreduce_begin(piece, count, 1)) != 0) return 3;
    }
    a->sums_begun = false;
    /* the library stream waits for every sum under way */
    return boat_report("gradient all-reduce", boat_cuda_allreduce_join());
}
