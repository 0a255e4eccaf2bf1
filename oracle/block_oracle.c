/* block_oracle.c - CPU restatement of the layers the encoder block puts around attention.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT (same rules as attention_oracle.c).
 *
 *   layernorm forward   restates boat_layernorm_forward, reference src/layers/norm.c:178-202,
 *                       :231-317, keeping its float accumulation order - PINNED: bit-identical
 *                       to the reference library and to the committed golden vectors.
 *   dense forward/backward  restates src/layers/dense.c:135-297 (matmul of linear.c:116-130,
 *                       bias add, dW/db accumulation) - PINNED the same way.
 *   layernorm backward, GELU forward/backward - PARITY UNPINNED: the reference has stubs only
 *                       (norm.c:397-402, src/ops/activation.c:298-302).  These are the analytic
 *                       formulas in double precision, checked against central differences of
 *                       the forward by the CPU tests.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

API void oracle_layernorm_forward(const float* x, int64_t rows, int64_t H, const float* w, const float* b, float eps,
                                  float* y) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* in = x + r * H;
        float sum = 0.0f;
        for (int64_t h = 0; h < H; ++h) sum += in[h];
        float m = sum / H;
        float var_sum = 0.0f;
        for (int64_t h = 0; h < H; ++h) {
            float diff = in[h] - m;
            var_sum += diff * diff;
        }
        float v = var_sum / H;
        float scale = 1.0f / sqrtf(v + eps);
        for (int64_t h = 0; h < H; ++h) {
            float n = (in[h] - m) * scale;
            if (w) n = n * w[h];
            if (b) n = n + b[h];
            y[r * H + h] = n;
        }
    }
}

/* dx, dgamma, dbeta of y = (x-mean)/sqrt(var+eps)*w + b, all sums in double */
API void oracle_layernorm_backward(const float* dy, const float* x, int64_t rows, int64_t H, const float* w, float eps,
                                   float* dx, float* dgamma, float* dbeta) {
    double* dg = calloc((size_t)H, sizeof(double));
    double* db = calloc((size_t)H, sizeof(double));
    for (int64_t r = 0; r < rows; ++r) {
        const float* in = x + r * H;
        double m = 0, v = 0;
        for (int64_t h = 0; h < H; ++h) m += in[h];
        m /= H;
        for (int64_t h = 0; h < H; ++h) v += (in[h] - m) * (in[h] - m);
        v /= H;
        double rs = 1.0 / sqrt(v + eps), s1 = 0, s2 = 0;
        for (int64_t h = 0; h < H; ++h) {
            double xh = (in[h] - m) * rs, g = (double)dy[r * H + h] * (w ? w[h] : 1.0);
            s1 += g;
            s2 += g * xh;
            dg[h] += dy[r * H + h] * xh;
            db[h] += dy[r * H + h];
        }
        s1 /= H;
        s2 /= H;
        for (int64_t h = 0; h < H; ++h) {
            double xh = (in[h] - m) * rs, g = (double)dy[r * H + h] * (w ? w[h] : 1.0);
            dx[r * H + h] = (float)(rs * (g - s1 - xh * s2));
        }
    }
    for (int64_t h = 0; h < H; ++h) {
        if (dgamma) dgamma[h] = (float)dg[h];
        if (dbeta) dbeta[h] = (float)db[h];
    }
    free(dg);
    free(db);
}

API void oracle_gelu_forward(const float* x, float* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = (float)(0.5 * x[i] * (1.0 + erf(x[i] / sqrt(2.0))));
}

API void oracle_gelu_backward(const float* dy, const float* x, float* dx, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        double v = x[i];
        double d = 0.5 * (1.0 + erf(v / sqrt(2.0))) + v * exp(-0.5 * v * v) / sqrt(2.0 * 3.14159265358979323846);
        dx[i] = (float)(dy[i] * d);
    }
}

static void matmul(const float* a, const float* b, float* out, int64_t m, int64_t k, int64_t n) {
    for (int64_t i = 0; i < m; ++i) {
        float* o = out + i * n;
        for (int64_t j = 0; j < n; ++j) o[j] = 0.0f;
        for (int64_t l = 0; l < k; ++l) {
            const float av = a[i * k + l];
            for (int64_t j = 0; j < n; ++j) o[j] += av * b[l * n + j];
        }
    }
}

/* y = x.W (+ b), dense.c:135-185 */
API void oracle_dense_forward(const float* x, const float* w, const float* bias, float* y, int64_t N, int64_t I, int64_t O) {
    matmul(x, w, y, N, I, O);
    if (bias)
        for (int64_t i = 0; i < N; ++i)
            for (int64_t j = 0; j < O; ++j) y[i * O + j] += bias[j];
}

/* dx = dy.W^T; dw += x^T.dy; db += sum_rows dy   (dense.c:187-297: gradients accumulate) */
API int oracle_dense_backward(const float* x, const float* w, const float* dy, float* dx, float* dw_acc, float* db_acc,
                              int64_t N, int64_t I, int64_t O) {
    float* wt = malloc(sizeof(float) * (size_t)I * (size_t)O);
    float* xt = malloc(sizeof(float) * (size_t)N * (size_t)I);
    float* fresh = malloc(sizeof(float) * (size_t)I * (size_t)O);
    if (!wt || !xt || !fresh) {
        free(wt); free(xt); free(fresh);
        return 1;
    }
    for (int64_t i = 0; i < I; ++i)
        for (int64_t j = 0; j < O; ++j) wt[j * I + i] = w[i * O + j];
    for (int64_t i = 0; i < N; ++i)
        for (int64_t j = 0; j < I; ++j) xt[j * N + i] = x[i * I + j];
    matmul(dy, wt, dx, N, O, I);
    matmul(xt, dy, fresh, I, N, O);
    for (int64_t i = 0; i < I * O; ++i) dw_acc[i] = dw_acc[i] + fresh[i];
    if (db_acc)
        for (int64_t b = 0; b < N; ++b)
            for (int64_t j = 0; j < O; ++j) db_acc[j] += dy[b * O + j];
    free(wt); free(xt); free(fresh);
    return 0;
}
