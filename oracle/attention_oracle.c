/* attention_oracle.c - CPU restatement of Boat's multi-head attention forward + backward.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT.  This file exists to check the CUDA path: only the
 * tests, the smoke check and the benchmark's CPU-baseline legs may call it.  Nothing in the
 * library (boat_b200/) links or loads it.
 *
 * It follows the reference (xiaoshaoning/boat) operation by operation and keeps the
 * reference's FP32 accumulation order per output element, so that on the same inputs it
 * agrees with the reference's own build bit for bit (checked by the CPU tests against
 * oracle/_ref/libboat_ref.so and against the committed golden vectors):
 *
 *   matmul          out[i,j] = sum_l a[i,l]*b[l,j], float accumulator, l ascending
 *                                                   src/ops/linear.c:116-130
 *   projection      Y = X.W, then + bias            src/layers/attention.c:247-308
 *   head split      [B,S,H] viewed as [B,nh,S,hs]   attention.c:393-397  (reshape only)
 *   scores          sum_d q[i,d]*k[j,d], then *scale attention.c:997-1009
 *   causal mask     scores[i][j>i] = -1e9f          attention.c:1012-1020
 *   softmax         max-subtract, expf, divide by the float sum if != 0
 *                                                   attention.c:1028-1046
 *   P.V             sum_j p[i,j]*v[j,d]             attention.c:1065-1073
 *   dV = P^T.dO, dP = dO.V^T                        attention.c:1423-1441
 *   dS = P*(dP - sum_j dP*P), row sum in double, the subtraction in double
 *                                                   attention.c:1472-1488
 *   dS *= scale (float)                             attention.c:1497
 *   dQ = dS.K, dK = dS^T.Q                          attention.c:1505-1526
 *   dX = dY.W^T, dW = X^T.dY, db = sum rows dY      attention.c:1213-1284
 *
 * Loops over independent output rows are OpenMP-parallel; that changes which core computes
 * an element, never the order of the additions inside it.  Build without -ffast-math and
 * without FMA contraction (the Makefile passes -ffp-contract=off).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define API __attribute__((visibility("default")))

API int oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

API void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* out[m,n] = a[m,k] . b[k,n]; each element accumulates l = 0..k-1 in a float, as the
 * reference does.  The j loop is innermost only in memory order: acc[j] is still one
 * running float sum per output. */
static void matmul(const float* a, const float* b, float* out, int64_t m, int64_t k, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i) {
        float* o = out + i * n;
        for (int64_t j = 0; j < n; ++j) o[j] = 0.0f;
        for (int64_t l = 0; l < k; ++l) {
            const float av = a[i * k + l];
            const float* br = b + l * n;
            for (int64_t j = 0; j < n; ++j) o[j] += av * br[j];
        }
    }
}

static float* transpose(const float* a, int64_t rows, int64_t cols) {
    float* t = (float*)malloc(sizeof(float) * (size_t)rows * (size_t)cols);
    if (!t) return NULL;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < rows; ++i)
        for (int64_t j = 0; j < cols; ++j) t[j * rows + i] = a[i * cols + j];
    return t;
}

/* y = x.W (+ b): linear_projection */
static void project(const float* x, const float* w, const float* bias, float* y, int64_t T, int64_t H) {
    matmul(x, w, y, T, H, H);
    if (bias) {
#pragma omp parallel for schedule(static)
        for (int64_t t = 0; t < T; ++t)
            for (int64_t h = 0; h < H; ++h) y[t * H + h] = y[t * H + h] + bias[h];
    }
}

/* linear_projection_backward: dx = dy.W^T, dw = x^T.dy, db = sum_t dy */
static int project_backward(const float* x, const float* w, const float* dy, float* dx, float* dw, float* db,
                            int64_t T, int64_t H) {
    float* wt = transpose(w, H, H);
    float* xt = transpose(x, T, H);
    if (!wt || !xt) {
        free(wt);
        free(xt);
        return 1;
    }
    matmul(dy, wt, dx, T, H, H);
    matmul(xt, dy, dw, H, T, H);
    free(wt);
    free(xt);
    if (db) {
        for (int64_t h = 0; h < H; ++h) db[h] = 0.0f;
        for (int64_t t = 0; t < T; ++t)          /* row order of the reference's b,s loops */
            for (int64_t h = 0; h < H; ++h) db[h] += dy[t * H + h];
    }
    return 0;
}

/* Attention core of one unit (b,h): q,k,v,o are [S,hs]; p receives the [S,S] probabilities. */
static void core_forward(const float* q, const float* k, const float* v, float* o, float* p, int64_t S, int64_t hs,
                         float scale, int causal) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < S; ++i) {
        float* row = p + i * S;
        for (int64_t j = 0; j < S; ++j) {
            float sum = 0.0f;
            for (int64_t d = 0; d < hs; ++d) sum += q[i * hs + d] * k[j * hs + d];
            row[j] = sum * scale;
        }
        if (causal)
            for (int64_t j = i + 1; j < S; ++j) row[j] = -1e9f;
        float mx = row[0];
        for (int64_t j = 1; j < S; ++j)
            if (row[j] > mx) mx = row[j];
        float se = 0.0f;
        for (int64_t j = 0; j < S; ++j) {
            row[j] = expf(row[j] - mx);
            se += row[j];
        }
        if (se != 0.0f)
            for (int64_t j = 0; j < S; ++j) row[j] /= se;
        for (int64_t d = 0; d < hs; ++d) {
            float sum = 0.0f;
            for (int64_t j = 0; j < S; ++j) sum += row[j] * v[j * hs + d];
            o[i * hs + d] = sum;
        }
    }
}

/* attention_backward for one unit.  p is overwritten with dS*scale. */
static int core_backward(const float* q, const float* k, const float* v, float* p, const float* go, float* dq, float* dk,
                         float* dv, int64_t S, int64_t hs, float scale) {
    float* pt = transpose(p, S, S);
    float* vt = transpose(v, S, hs);
    float* dp = (float*)malloc(sizeof(float) * (size_t)S * (size_t)S);
    if (!pt || !vt || !dp) {
        free(pt);
        free(vt);
        free(dp);
        return 1;
    }
    matmul(pt, go, dv, S, S, hs);          /* dV = P^T dO */
    matmul(go, vt, dp, S, hs, S);          /* dP = dO V^T */
    free(pt);
    free(vt);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < S; ++i) {
        double sum = 0.0;
        for (int64_t j = 0; j < S; ++j) sum += (double)dp[i * S + j] * (double)p[i * S + j];
        for (int64_t j = 0; j < S; ++j) {
            float ds = (float)(p[i * S + j] * (dp[i * S + j] - sum));   /* float*(double) -> double -> float */
            p[i * S + j] = ds * scale;
        }
    }
    free(dp);
    matmul(p, k, dq, S, S, hs);            /* dQ = dS K */
    float* dst = transpose(p, S, S);
    if (!dst) return 1;
    matmul(dst, q, dk, S, S, hs);          /* dK = dS^T Q */
    free(dst);
    return 0;
}

/* One training step of the layer: forward, then backward from `dout`.
 *
 * q,k,v,dout,out,dq,dk,dv: [B,S,H].  w[4] = Wq,Wk,Wv,Wo as [H,H] ([in,out]); b[4] = biases
 * or all NULL.  dw[4], db[4] receive the parameter gradients (db may be NULL when there is
 * no bias).  Any of dout/dq/dk/dv/dw may be NULL to run the forward only.  `lse`, when not
 * NULL, receives max + log(sum exp) per (unit,row) [B*nh*S] for checks of the saved
 * statistics.  Returns 0, or 1 when memory runs out. */
API int oracle_attention_step(int64_t B, int64_t S, int64_t H, int64_t nh, int causal,
                              const float* q, const float* k, const float* v,
                              const float* const w[4], const float* const b[4],
                              const float* dout, float* out,
                              float* dq, float* dk, float* dv,
                              float* const dw[4], float* const db[4], float* lse) {
    const int64_t T = B * S, hs = H / nh, units = B * nh;
    const float scale = 1.0f / sqrtf((float)hs);
    const size_t act = sizeof(float) * (size_t)T * (size_t)H;
    int rc = 1;
    float *qp = malloc(act), *kp = malloc(act), *vp = malloc(act), *ctx = malloc(act);
    float* p = malloc(sizeof(float) * (size_t)S * (size_t)S);
    float *dctx = NULL, *dqp = NULL, *dkp = NULL, *dvp = NULL;
    if (!qp || !kp || !vp || !ctx || !p) goto done;
    project(q, w[0], b ? b[0] : NULL, qp, T, H);
    project(k, w[1], b ? b[1] : NULL, kp, T, H);
    project(v, w[2], b ? b[2] : NULL, vp, T, H);
    const int backward = dout != NULL;
    if (backward) {
        dctx = malloc(act);
        dqp = malloc(act);
        dkp = malloc(act);
        dvp = malloc(act);
        if (!dctx || !dqp || !dkp || !dvp) goto done;
        /* dctx needs only dout and Wo; do it first so that the unit loop can run forward
         * and backward of a unit back to back without keeping B*nh probability matrices. */
        float* wt = transpose(w[3], H, H);
        if (!wt) goto done;
        matmul(dout, wt, dctx, T, H, H);
        free(wt);
    }
    for (int64_t u = 0; u < units; ++u) {
        const int64_t off = u * S * hs;
        core_forward(qp + off, kp + off, vp + off, ctx + off, p, S, hs, scale, causal);
        if (lse) {
            /* statistics of the scaled, masked scores, recomputed the plain way */
            for (int64_t i = 0; i < S; ++i) {
                float mx = -INFINITY;
                int64_t jn = causal ? i + 1 : S;
                float* sc = (float*)malloc(sizeof(float) * (size_t)jn);
                if (!sc) goto done;
                for (int64_t j = 0; j < jn; ++j) {
                    float sum = 0.0f;
                    for (int64_t d = 0; d < hs; ++d) sum += qp[off + i * hs + d] * kp[off + j * hs + d];
                    sc[j] = sum * scale;
                    if (sc[j] > mx) mx = sc[j];
                }
                double se = 0.0;
                for (int64_t j = 0; j < jn; ++j) se += exp((double)sc[j] - (double)mx);
                lse[u * S + i] = (float)((double)mx + log(se));
                free(sc);
            }
        }
        if (backward && core_backward(qp + off, kp + off, vp + off, p, dctx + off, dqp + off, dkp + off, dvp + off, S,
                                      hs, scale))
            goto done;
    }
    project(ctx, w[3], b ? b[3] : NULL, out, T, H);
    if (backward) {
        float* scratch_dx = malloc(act);
        if (!scratch_dx) goto done;
        int bad = project_backward(ctx, w[3], dout, scratch_dx, dw[3], db ? db[3] : NULL, T, H);
        free(scratch_dx);
        bad |= project_backward(q, w[0], dqp, dq, dw[0], db ? db[0] : NULL, T, H);
        bad |= project_backward(k, w[1], dkp, dk, dw[1], db ? db[1] : NULL, T, H);
        bad |= project_backward(v, w[2], dvp, dv, dw[2], db ? db[2] : NULL, T, H);
        if (bad) goto done;
    }
    rc = 0;
done:
    free(qp); free(kp); free(vp); free(ctx); free(p);
    free(dctx); free(dqp); free(dkp); free(dvp);
    return rc;
}

/* Attention core alone on [units,S,hs] buffers: O and (optionally) dQ,dK,dV for given dO.
 * Used to check single (batch,head) units of problems whose full step is too large for a
 * CPU run. */
API int oracle_attention_core(int64_t units, int64_t S, int64_t hs, int causal, float scale,
                              const float* q, const float* k, const float* v, const float* go,
                              float* o, float* dq, float* dk, float* dv) {
    float* p = malloc(sizeof(float) * (size_t)S * (size_t)S);
    if (!p) return 1;
    int rc = 0;
    for (int64_t u = 0; u < units && rc == 0; ++u) {
        const int64_t off = u * S * hs;
        core_forward(q + off, k + off, v + off, o + off, p, S, hs, scale, causal);
        if (go) rc = core_backward(q + off, k + off, v + off, p, go + off, dq + off, dk + off, dv + off, S, hs, scale);
    }
    free(p);
    return rc;
}

/* SGD step of boat_attention_update (attention.c:745-812): p -= fl(g * lr). */
API void oracle_sgd(float* param, const float* grad, float lr, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        float t = grad[i] * lr;
        param[i] = param[i] - t;
    }
}
