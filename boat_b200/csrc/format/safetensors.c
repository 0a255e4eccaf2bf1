/* safetensors.c - fill an attention layer's parameters from a safetensors image.
 *
 * The reference reads safetensors headers in src/format/huggingface.c (:619-680 header,
 * :680-850 tensor walk) but stops at the attention layer: create_layer_from_config only prints
 * "Detected attention layer ... Query weight" and returns NULL (:917-932, a TODO).  This file is
 * that missing step for the one layer this library is about, keeping the reference's way of
 * recognising the tensors: a name that contains "attention" and one of "query", "key", "value",
 * "output".
 *
 * File layout (the published safetensors format): u64 little-endian header length N, N bytes of
 * JSON {"name": {"dtype": "F32", "shape": [..], "data_offsets": [begin, end]}, ...,
 * "__metadata__": {...}}, then the tensor bytes; offsets are relative to the end of the header.
 * Checkpoints store a projection as [out, in] (y = x W^T + b); Boat stores [in, out]
 * (src/layers/attention.c:90), so weights are transposed on the way in - on the GPU, with the
 * kernels that exist anyway: upload the raw bytes, cast to FP32, transpose into place.
 * Note that a checkpoint trained with column-split heads is not made Boat-compatible by this:
 * Boat splits heads by reshaping [B,S,H] to [B,nh,S,hs] without a transpose. */
#include "../core/stage.h"
#include <boat_b200.h>

#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

enum { ST_F32, ST_BF16, ST_F16, ST_OTHER };

typedef struct {
    const char* name;     /* not terminated: name_len bytes inside the header */
    size_t name_len;
    int dtype;
    int64_t shape[4];
    int ndim;
    uint64_t begin, end;  /* relative to the data section */
} st_entry_t;

/* ---- a JSON reader for exactly this header shape ------------------------------------------------ */

typedef struct {
    const char* p;
    const char* end;
} cur_t;

static void skip_ws(cur_t* c) {
    while (c->p < c->end && (*c->p == ' ' || *c->p == '\n' || *c->p == '\t' || *c->p == '\r')) c->p++;
}

static bool eat(cur_t* c, char ch) {
    skip_ws(c);
    if (c->p < c->end && *c->p == ch) {
        c->p++;
        return true;
    }
    return false;
}

/* A string without escape processing (tensor names and dtype tags never need any); a backslash
 * escapes the next character for the purpose of finding the end. */
static bool read_string(cur_t* c, const char** s, size_t* len) {
    if (!eat(c, '"')) return false;
    *s = c->p;
    while (c->p < c->end && *c->p != '"') {
        if (*c->p == '\\') c->p++;
        c->p++;
    }
    if (c->p >= c->end) return false;
    *len = (size_t)(c->p - *s);
    c->p++;
    return true;
}

static bool read_uint(cur_t* c, uint64_t* v) {
    skip_ws(c);
    if (c->p >= c->end || *c->p < '0' || *c->p > '9') return false;
    uint64_t x = 0;
    while (c->p < c->end && *c->p >= '0' && *c->p <= '9') {
        if (x > (UINT64_MAX - 9) / 10) return false;
        x = x * 10 + (uint64_t)(*c->p - '0');
        c->p++;
    }
    *v = x;
    return true;
}

/* Skips any JSON value (used for "__metadata__" and unknown keys). */
static bool skip_value(cur_t* c, int depth) {
    if (depth > 16) return false;
    skip_ws(c);
    if (c->p >= c->end) return false;
    if (*c->p == '"') {
        const char* s;
        size_t n;
        return read_string(c, &s, &n);
    }
    if (*c->p == '{' || *c->p == '[') {
        const char close = *c->p == '{' ? '}' : ']';
        const bool object = *c->p == '{';
        c->p++;
        if (eat(c, close)) return true;
        do {
            if (object) {
                const char* s;
                size_t n;
                if (!read_string(c, &s, &n) || !eat(c, ':')) return false;
            }
            if (!skip_value(c, depth + 1)) return false;
        } while (eat(c, ','));
        return eat(c, close);
    }
    while (c->p < c->end && *c->p != ',' && *c->p != '}' && *c->p != ']') c->p++;   /* number, true, false, null */
    return true;
}

static bool key_is(const char* s, size_t n, const char* lit) { return strlen(lit) == n && memcmp(s, lit, n) == 0; }

static bool read_entry(cur_t* c, st_entry_t* e) {
    bool have_dtype = false, have_shape = false, have_off = false;
    if (!eat(c, '{')) return false;
    if (eat(c, '}')) return false;
    do {
        const char* k;
        size_t kn;
        if (!read_string(c, &k, &kn) || !eat(c, ':')) return false;
        if (key_is(k, kn, "dtype")) {
            const char* d;
            size_t dn;
            if (!read_string(c, &d, &dn)) return false;
            e->dtype = key_is(d, dn, "F32") ? ST_F32 : key_is(d, dn, "BF16") ? ST_BF16 : key_is(d, dn, "F16") ? ST_F16 : ST_OTHER;
            have_dtype = true;
        } else if (key_is(k, kn, "shape")) {
            if (!eat(c, '[')) return false;
            e->ndim = 0;
            if (!eat(c, ']')) {
                do {
                    uint64_t v;
                    if (e->ndim >= 4) {                       /* more dimensions than any parameter here has */
                        if (!read_uint(c, &v)) return false;
                        e->ndim = 5;
                        continue;
                    }
                    if (!read_uint(c, &v) || v > INT64_MAX) return false;
                    e->shape[e->ndim++] = (int64_t)v;
                } while (eat(c, ','));
                if (!eat(c, ']')) return false;
            }
            have_shape = true;
        } else if (key_is(k, kn, "data_offsets")) {
            if (!eat(c, '[') || !read_uint(c, &e->begin) || !eat(c, ',') || !read_uint(c, &e->end) || !eat(c, ']'))
                return false;
            have_off = true;
        } else if (!skip_value(c, 0)) {
            return false;
        }
    } while (eat(c, ','));
    return eat(c, '}') && have_dtype && have_shape && have_off;
}

/* ---- tensor names ------------------------------------------------------------------------------------- */

static bool contains(const char* s, size_t n, const char* lit) {
    const size_t m = strlen(lit);
    for (size_t i = 0; i + m <= n; ++i)
        if (memcmp(s + i, lit, m) == 0) return true;
    return false;
}

static bool ends_with(const char* s, size_t n, const char* lit) {
    const size_t m = strlen(lit);
    return n >= m && memcmp(s + n - m, lit, m) == 0;
}

/* 0..3 = Wq Wk Wv Wo, 4..7 = bq bk bv bo, -1 = not a parameter of the attention layer.
 * Same tests as huggingface.c:917-932 plus what tells weights from biases and keeps the
 * LayerNorm that lives under "attention.output" in BERT-style checkpoints out. */
static int classify(const st_entry_t* e, const char* prefix) {
    const size_t pn = prefix ? strlen(prefix) : 0;
    if (pn && (e->name_len < pn || memcmp(e->name, prefix, pn) != 0)) return -1;
    if (!contains(e->name, e->name_len, "attention")) return -1;
    if (contains(e->name, e->name_len, "norm") || contains(e->name, e->name_len, "Norm")) return -1;
    int which = contains(e->name, e->name_len, "query") ? 0 : contains(e->name, e->name_len, "key") ? 1
              : contains(e->name, e->name_len, "value") ? 2 : contains(e->name, e->name_len, "output") ? 3 : -1;
    if (which < 0) return -1;
    if (ends_with(e->name, e->name_len, ".weight") && e->ndim == 2) return which;
    if (ends_with(e->name, e->name_len, ".bias") && e->ndim == 1) return 4 + which;
    return -1;
}

/* ---- moving one tensor into a parameter ------------------------------------------------------------------ */

static float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {                                   /* subnormal: normalise */
            exp = 127 - 15 + 1;
            while (!(man & 0x400u)) {
                man <<= 1;
                exp--;
            }
            bits = sign | (exp << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, sizeof f);
    return f;
}

/* FP32 copy of the entry on the device; NULL on failure.  `n` elements. */
static float* entry_on_device(const st_entry_t* e, const uint8_t* data, size_t n) {
    const uint8_t* src = data + e->begin;
    float* out = NULL;
    if (e->dtype == ST_F32) {
        out = (float*)boat_dev_alloc(n * 4);
        if (out && boat_report("checkpoint upload", boat_cuda_memcpy_h2d(out, src, n * 4)) != 0) {
            boat_dev_free(out);
            out = NULL;
        }
    } else if (e->dtype == ST_BF16) {
        void* raw = boat_dev_alloc(n * 2);
        out = raw ? (float*)boat_dev_alloc(n * 4) : NULL;
        if (!out || boat_report("checkpoint upload", boat_cuda_memcpy_h2d(raw, src, n * 2)) != 0 ||
            boat_report("checkpoint cast", boat_cuda_cast(out, BOAT_CUDA_F32, raw, BOAT_CUDA_BF16, (int64_t)n)) != 0) {
            boat_dev_free(out);
            out = NULL;
        }
        boat_dev_free(raw);
    } else {                                       /* F16: widened on the host, there is no FP16 kernel here */
        float* host = (float*)malloc(n * 4);
        if (!host) return NULL;
        for (size_t i = 0; i < n; ++i) {
            uint16_t h;
            memcpy(&h, src + 2 * i, 2);
            host[i] = half_to_float(h);
        }
        out = (float*)boat_dev_alloc(n * 4);
        if (out && boat_report("checkpoint upload", boat_cuda_memcpy_h2d(out, host, n * 4)) != 0) {
            boat_dev_free(out);
            out = NULL;
        }
        free(host);
    }
    return out;
}

static int store_param(boat_tensor_t* param, const st_entry_t* e, const uint8_t* data, bool transpose) {
    const size_t n = param->nelements;
    float* dev = entry_on_device(e, data, n);
    if (!dev) return 5;
    int rc = 0;
    float* result = dev;
    float* tmp = NULL;
    if (transpose) {
        /* checkpoint [out, in] -> Boat [in, out] */
        result = param->device == BOAT_DEVICE_CUDA ? (float*)param->data : (tmp = (float*)boat_dev_alloc(n * 4));
        if (!result || boat_report("checkpoint transpose", boat_cuda_transpose(result, dev, 1, e->shape[0], e->shape[1])) != 0)
            rc = 5;
    }
    if (rc == 0 && param->device != BOAT_DEVICE_CUDA)
        rc = boat_report("parameter download", boat_cuda_memcpy_d2h(param->data, result, n * 4)) ? 5 : 0;
    else if (rc == 0 && !transpose)
        rc = boat_report("parameter copy", boat_cuda_memcpy_d2d(param->data, dev, n * 4)) ? 5 : 0;
    if (rc == 0) rc = boat_report("checkpoint load", boat_cuda_sync()) ? 5 : 0;    /* `data` may go away after return */
    boat_dev_free(tmp);
    boat_dev_free(dev);
    return rc;
}

/* ---- entry points ------------------------------------------------------------------------------------------ */

int boat_attention_load_safetensors(boat_attention_t* attention, const void* image, size_t size, const char* prefix) {
    if (!attention || !image) return 1;
    const uint8_t* bytes = (const uint8_t*)image;
    if (size < 8) return 2;
    uint64_t header_len = 0;
    for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | bytes[i];
    if (header_len > size - 8 || header_len < 2) return 2;
    const uint8_t* data = bytes + 8 + header_len;
    const uint64_t data_size = size - 8 - header_len;

    boat_tensor_t* params[8] = {
        boat_attention_get_weight_q(attention), boat_attention_get_weight_k(attention),
        boat_attention_get_weight_v(attention), boat_attention_get_weight_o(attention),
        boat_attention_get_bias_q(attention),   boat_attention_get_bias_k(attention),
        boat_attention_get_bias_v(attention),   boat_attention_get_bias_o(attention)};
    st_entry_t found[8];
    bool have[8] = {false};

    cur_t c = {(const char*)bytes + 8, (const char*)bytes + 8 + header_len};
    if (!eat(&c, '{')) return 2;
    if (!eat(&c, '}')) {
        do {
            st_entry_t e;
            memset(&e, 0, sizeof e);
            if (!read_string(&c, &e.name, &e.name_len) || !eat(&c, ':')) return 2;
            if (key_is(e.name, e.name_len, "__metadata__")) {
                if (!skip_value(&c, 0)) return 2;
                continue;
            }
            if (!read_entry(&c, &e)) return 2;
            if (e.begin > e.end || e.end > data_size) return 2;
            const int slot = classify(&e, prefix);
            if (slot < 0 || !params[slot]) continue;       /* not ours, or a bias the layer does not have */
            if (have[slot]) {
                fprintf(stderr, "boat: several tensors in the checkpoint match one attention parameter; give a name prefix\n");
                return 4;
            }
            found[slot] = e;
            have[slot] = true;
        } while (eat(&c, ','));
        if (!eat(&c, '}')) return 2;
    }

    for (int slot = 0; slot < 8; ++slot) {
        if (!params[slot]) continue;
        if (!have[slot]) {
            if (slot < 4) return 3;                         /* a projection matrix is missing */
            continue;                                       /* a missing bias keeps its value */
        }
        const st_entry_t* e = &found[slot];
        const boat_tensor_t* p = params[slot];
        if (e->dtype == ST_OTHER || p->dtype != BOAT_DTYPE_FLOAT32) return 4;
        const size_t esize = e->dtype == ST_F32 ? 4 : 2;
        bool shape_ok = slot < 4 ? (e->shape[0] == p->shape[1] && e->shape[1] == p->shape[0])
                                 : (e->shape[0] == p->shape[0]);
        if (!shape_ok || e->end - e->begin != (uint64_t)p->nelements * esize) return 4;
    }
    for (int slot = 0; slot < 8; ++slot) {
        if (!params[slot] || !have[slot]) continue;
        int rc = store_param(params[slot], &found[slot], data, slot < 4);
        if (rc) return rc;
    }
    return 0;
}

int boat_attention_load_safetensors_file(boat_attention_t* attention, const char* path, const char* prefix) {
    if (!attention || !path) return 1;
    FILE* f = fopen(path, "rb");
    if (!f) return 1;
    int rc = 2;
    void* buf = NULL;
    if (fseek(f, 0, SEEK_END) == 0) {
        long n = ftell(f);
        if (n >= 8 && fseek(f, 0, SEEK_SET) == 0 && (buf = malloc((size_t)n)) != NULL && fread(buf, 1, (size_t)n, f) == (size_t)n)
            rc = boat_attention_load_safetensors(attention, buf, (size_t)n, prefix);
    }
    free(buf);
    fclose(f);
    return rc;
}
