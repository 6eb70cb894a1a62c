/*
 * CPU restatement of Volta's optimizer arithmetic (Adam, SGD, Muon).
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is the checker the CUDA path is compared
 * against and the timed CPU baseline of the benchmark; the product library never
 * links, loads or calls it.
 *
 * Every function follows one function of the reference (rlarson20/Volta 0.3.0), cited
 * by path:line inside that project.  Rust never contracts or reassociates floating
 * point, `f32::mul_add` is a correctly rounded fused multiply-add, and `/`, `sqrt` are
 * IEEE; this file is therefore compiled with -ffp-contract=off and without fast-math,
 * uses fmaf() exactly where the reference writes mul_add, and keeps the reference's
 * pass structure (grad copy, weight-decay pass, moment pass, parameter pass).
 *
 * Pinned: Adam and SGD arithmetic, against the hand-computed known-answer tests the
 * reference holds (tests/test_optimizers.rs:13-140,168-223; tests/coverage_fill.rs:45-67;
 * src/lib.rs:3102-3119).
 * PARITY UNPINNED: Muon's Newton-Schulz.  The reference has no numeric test for it
 * (src/nn/optim/muon.rs:172-192 only checks "changed and < 2.0") and its contraction
 * is the third-party crate matrixmultiply 0.3.10 (Cargo.lock:694-695), whose source is
 * not part of the reference tree.  vo_sgemm() restates that crate's published blocking
 * scheme (k split in blocks of 256, one fused multiply-add chain per block, block
 * results added into C); vo_sgemm_f64acc() is a second opinion with f64 accumulation.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* f32::powi(a, b): Rust lowers to the llvm.powi intrinsic, which compiler-rt implements
 * as __powisf2: square-and-multiply over the exponent bits, least significant first,
 * every product rounded to f32.  Used by src/nn/optim/adam.rs:188-189. */
float vo_powi_f32(float a, int b)
{
    const int recip = b < 0;
    float r = 1.0f;
    for (;;) {
        if (b & 1) r *= a;
        b /= 2;
        if (b == 0) break;
        a *= a;
    }
    return recip ? 1.0f / r : r;
}

/* Bias-correction scales, src/nn/optim/adam.rs:188-189. */
void vo_adam_bias_scales(float beta1, float beta2, int t, float *m_hat_scale, float *v_hat_scale)
{
    *m_hat_scale = 1.0f / (1.0f - vo_powi_f32(beta1, t));
    *v_hat_scale = 1.0f / (1.0f - vo_powi_f32(beta2, t));
}

/* Adam::step_cpu_param, src/nn/optim/adam.rs:139-205, for one tensor.
 * `t` is the already-incremented time step (adam.rs:71).  `scratch` (n floats) takes
 * the place of the reference's gradient clone (adam.rs:143-149). */
void vo_adam_step(float *p, const float *g, float *m, float *v, size_t n,
                  float lr, float beta1, float beta2, float eps, float weight_decay, int t,
                  float *scratch)
{
    float *ag = scratch;
    memcpy(ag, g, n * sizeof(float)); /* adam.rs:143-149 */
    if (weight_decay != 0.0f) {       /* adam.rs:150-154 */
        for (size_t j = 0; j < n; ++j) ag[j] += weight_decay * p[j];
    }
    for (size_t j = 0; j < n; ++j) { /* adam.rs:172-185 */
        float gv = ag[j];
        m[j] = fmaf(beta1, m[j], (1.0f - beta1) * gv);
        v[j] = fmaf(beta2, v[j], (1.0f - beta2) * (gv * gv)); /* powi(2) == gv*gv */
    }
    float s1, s2; /* adam.rs:188-189 */
    vo_adam_bias_scales(beta1, beta2, t, &s1, &s2);
    for (size_t j = 0; j < n; ++j) { /* adam.rs:196-204 */
        float m_hat = m[j] * s1;
        float v_hat = v[j] * s2;
        p[j] -= lr * m_hat / (sqrtf(v_hat) + eps);
    }
}

/* SGD::step_cpu_param, src/nn/optim/sgd.rs:189-238.  `vel` may be NULL when
 * momentum <= 0 (sgd.rs:30: velocity exists only if momentum > 0.0). */
void vo_sgd_step(float *p, const float *g, float *vel, size_t n,
                 float lr, float momentum, float weight_decay, float *scratch)
{
    float *ag = scratch;
    memcpy(ag, g, n * sizeof(float)); /* sgd.rs:194-199 */
    if (weight_decay != 0.0f) {       /* sgd.rs:201-205 */
        for (size_t j = 0; j < n; ++j) ag[j] += weight_decay * p[j];
    }
    if (momentum > 0.0f) {
        for (size_t j = 0; j < n; ++j) vel[j] = fmaf(momentum, vel[j], -(lr * ag[j])); /* sgd.rs:216-218 */
        for (size_t j = 0; j < n; ++j) p[j] += vel[j];                                /* sgd.rs:225-227 */
    } else {
        for (size_t j = 0; j < n; ++j) p[j] -= lr * ag[j]; /* sgd.rs:234-236 */
    }
}

/* optimizer_step.wgsl:25-65 restated as plain arithmetic (secondary, informational:
 * the reference holds it to 1e-4 of the CPU path, src/lib.rs:3872-3877).  WGSL leaves
 * contraction and pow() precision to the implementation; this uses unfused f32
 * operations and powf. */
void vo_wgsl_optimizer_step(float *params, const float *grads, float *state1, float *state2,
                            size_t n, uint32_t op, float lr, float beta1, float beta2, float t,
                            float eps, float weight_decay)
{
    for (size_t i = 0; i < n; ++i) {
        float grad = grads[i];
        if (weight_decay != 0.0f) grad = grad + weight_decay * params[i];
        if (op == 0u) {
            params[i] = params[i] - lr * grad;
        } else if (op == 1u) {
            state1[i] = beta1 * state1[i] - lr * grad;
            params[i] = params[i] + state1[i];
        } else {
            state1[i] = beta1 * state1[i] + (1.0f - beta1) * grad;
            state2[i] = beta2 * state2[i] + (1.0f - beta2) * grad * grad;
            float m_hat_scale = 1.0f / (1.0f - powf(beta1, t));
            float v_hat_scale = 1.0f / (1.0f - powf(beta2, t));
            float m_hat = state1[i] * m_hat_scale;
            float v_hat = state2[i] * v_hat_scale;
            params[i] = params[i] - lr * m_hat / (sqrtf(v_hat) + eps);
        }
    }
}

/* RawTensor::transpose_2d, src/ops/matmul.rs:34-49. */
void vo_transpose_2d(const float *src, float *dst, size_t m, size_t n)
{
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) dst[j * m + i] = src[i * n + j];
}

/* RawTensor::matmul_raw, src/ops/matmul.rs:56-124: C[m,n] = A[m,k] B[k,n], row-major,
 * alpha 1, beta 0, through matrixmultiply::sgemm.  Restated blocking of that crate:
 * k is cut in blocks of KC = 256; within a block every C element is one chain of
 * fused multiply-adds in k order starting from 0; the first block's result is stored,
 * later blocks are added.  Rows are independent, so the OpenMP split changes nothing. */
#define VO_KC 256
void vo_sgemm(const float *a, const float *b, float *c, size_t m, size_t k, size_t n)
{
#pragma omp parallel
    {
        float *acc = (float *)malloc(n * sizeof(float));
#pragma omp for schedule(static)
        for (ptrdiff_t i = 0; i < (ptrdiff_t)m; ++i) {
            float *ci = c + (size_t)i * n;
            if (k == 0)
                for (size_t j = 0; j < n; ++j) ci[j] = 0.0f;
            for (size_t k0 = 0; k0 < k; k0 += VO_KC) {
                size_t k1 = k0 + VO_KC < k ? k0 + VO_KC : k;
                for (size_t j = 0; j < n; ++j) acc[j] = 0.0f;
                for (size_t kk = k0; kk < k1; ++kk) {
                    const float aik = a[(size_t)i * k + kk];
                    const float *bk = b + kk * n;
                    for (size_t j = 0; j < n; ++j) acc[j] = fmaf(aik, bk[j], acc[j]);
                }
                if (k0 == 0)
                    for (size_t j = 0; j < n; ++j) ci[j] = acc[j];
                else
                    for (size_t j = 0; j < n; ++j) ci[j] = ci[j] + acc[j];
            }
        }
        free(acc);
    }
}

/* Same contraction with every C element accumulated in f64 and rounded once. */
void vo_sgemm_f64acc(const float *a, const float *b, float *c, size_t m, size_t k, size_t n)
{
#pragma omp parallel
    {
        double *acc = (double *)malloc(n * sizeof(double));
#pragma omp for schedule(static)
        for (ptrdiff_t i = 0; i < (ptrdiff_t)m; ++i) {
            for (size_t j = 0; j < n; ++j) acc[j] = 0.0;
            for (size_t kk = 0; kk < k; ++kk) {
                const double aik = a[(size_t)i * k + kk];
                const float *bk = b + kk * n;
                for (size_t j = 0; j < n; ++j) acc[j] += aik * (double)bk[j];
            }
            for (size_t j = 0; j < n; ++j) c[(size_t)i * n + j] = (float)acc[j];
        }
        free(acc);
    }
}

/* Sequential f32 sum of squares, src/nn/optim/muon.rs:58
 * (`g.iter().map(|x| x * x).sum()` is a left fold in element order). */
float vo_sum_sq_sequential(const float *x, size_t n)
{
    float s = 0.0f;
    for (size_t i = 0; i < n; ++i) s += x[i] * x[i];
    return s;
}

/* Muon::newton_schulz, src/nn/optim/muon.rs:49-104.  gemm_mode 0: vo_sgemm,
 * 1: vo_sgemm_f64acc. */
void vo_newton_schulz(float *g, size_t rows, size_t cols, int steps, int gemm_mode)
{
    const size_t n = rows * cols;
    void (*gemm)(const float *, const float *, float *, size_t, size_t, size_t) =
        gemm_mode == 1 ? vo_sgemm_f64acc : vo_sgemm;
    float sum_sq = vo_sum_sq_sequential(g, n); /* muon.rs:58 */
    float norm = sqrtf(sum_sq + 1e-8f);        /* muon.rs:59 */
    if (norm > 1e-8f)                          /* muon.rs:60-64 */
        for (size_t i = 0; i < n; ++i) g[i] /= norm;

    float *xt = (float *)malloc(n * sizeof(float));
    float *xtx = (float *)malloc(cols * cols * sizeof(float));
    float *cm = (float *)malloc(cols * cols * sizeof(float));
    float *next = (float *)malloc(n * sizeof(float));
    for (int s = 0; s < steps; ++s) {       /* muon.rs:67-100 */
        vo_transpose_2d(g, xt, rows, cols); /* muon.rs:69 */
        gemm(xt, g, xtx, cols, rows, cols); /* muon.rs:73 */
        for (size_t i = 0; i < cols; ++i)   /* muon.rs:76-89 */
            for (size_t j = 0; j < cols; ++j) {
                float val = xtx[i * cols + j];
                cm[i * cols + j] = (i == j) ? 3.0f - val : -val;
            }
        gemm(g, cm, next, rows, cols, cols);                /* muon.rs:93 */
        for (size_t i = 0; i < n; ++i) g[i] = next[i] * 0.5f; /* muon.rs:95-99 */
    }
    free(xt);
    free(xtx);
    free(cm);
    free(next);
}

/* Muon::step for one parameter, src/nn/optim/muon.rs:108-163.  (rows, cols) is the
 * caller's flattening of the shape per muon.rs:117-130.  `update_out` (n floats)
 * receives the orthogonalised update (the reference's local `update`), so tests can
 * compare the Newton-Schulz output itself. */
void vo_muon_step(float *w, const float *grad, float *velocity, size_t rows, size_t cols,
                  float lr, float momentum, int nesterov, int ns_steps, int gemm_mode,
                  float *update_out)
{
    const size_t n = rows * cols;
    for (size_t i = 0; i < n; ++i) velocity[i] = fmaf(momentum, velocity[i], grad[i]); /* muon.rs:133-136 */
    if (nesterov) {
        for (size_t i = 0; i < n; ++i) update_out[i] = momentum * velocity[i] + grad[i]; /* muon.rs:139-147 */
    } else {
        memcpy(update_out, velocity, n * sizeof(float)); /* muon.rs:148-150 */
    }
    if (rows > 1 && cols > 1) vo_newton_schulz(update_out, rows, cols, ns_steps, gemm_mode); /* muon.rs:153-155 */
    for (size_t i = 0; i < n; ++i) w[i] -= lr * update_out[i] * 0.1f; /* muon.rs:158-160 */
}

int vo_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void vo_set_threads(int n)
{
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
