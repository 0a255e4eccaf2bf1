/* optimizer_oracle.c - CPU restatement of the reference's Adam step.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT (same rules as attention_oracle.c).
 *
 * Restates adam_update_parameter / adam_optimizer_step, reference src/optimizers/adam.c
 * :156-209: every operation is a rounded FP32 operation in the reference's order, the bias
 * corrections use powf with a float exponent.  PINNED: bit-identical to the reference library
 * over many steps and to the committed golden vectors (tests/golden).  Build without floating
 * point contraction (the Makefile passes -ffp-contract=off).
 */
#include <math.h>
#include <stdint.h>

#define API __attribute__((visibility("default")))

/* One step over one tensor; `timestep` is the number of steps taken before this one. */
API void oracle_adam_step(float* param, const float* grad, float* m, float* v, int64_t n, float lr, float beta1,
                          float beta2, float eps, int64_t timestep) {
    float beta1_pow = powf(beta1, (float)(timestep + 1));
    float beta2_pow = powf(beta2, (float)(timestep + 1));
    for (int64_t i = 0; i < n; ++i) {
        float g = grad[i];
        m[i] = beta1 * m[i] + (1.0f - beta1) * g;
        v[i] = beta2 * v[i] + (1.0f - beta2) * g * g;
        float m_hat = m[i] / (1.0f - beta1_pow);
        float v_hat = v[i] / (1.0f - beta2_pow);
        param[i] -= lr * m_hat / (sqrtf(v_hat) + eps);
    }
}
