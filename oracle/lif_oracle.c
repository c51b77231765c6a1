/*
 * CPU oracle for the LIF "fire" forward recurrence and its BPTT backward pass.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA kernels are compared
 * against (tests, the smoke check, and the CPU-baseline leg of the benchmark). Nothing
 * in the shipped package links, loads or calls it.
 *
 * It restates, in plain C, the arithmetic of the reference project
 * (liangling76/snn_gpu_training_bptt):
 *   forward   snnlib/cuda/snn_kernel_fp.cu:37-52   (fire_s_fp_kernel hot loop)
 *             snnlib/cuda/snn_kernel_bp.cu:34-51   (fire_u_fp_kernel: same recurrence, emits u)
 *   backward  snnlib/cuda/snn_kernel_bp.cu:117-138 (fire_bp_kernel hot loop)
 * and of the reference's pure-PyTorch twin snnlib/example/gold_op.py:17-44, whose
 * rounding it reproduces bit for bit (every product and sum is rounded separately:
 * compile with -ffp-contract=off).
 *
 * Parity pinning: checked against golden vectors produced by importing the reference's
 * gold_op.py (tests/golden/make_golden.py), see tests/test_oracle.py.
 *
 * Layout: time-major [T, N] contiguous, element (t, n) at t*N + n, where N = B*C*H*W is
 * the flattened neuron axis (neurons are independent, so the reference's separate B and
 * CHW loops collapse into one).
 */
#include <stdint.h>
#include <stddef.h>
#include <math.h>
#include <stdlib.h>

#define ORACLE_MAX_T 4096

/* u_t = (alpha*u_{t-1})*(1-s_{t-1}) + x_t ; s_t = u_t > thresh.  u_{-1} = s_{-1} = 0. */
void oracle_lif_fwd_f32(const float *x, float *spike, float *mem, int64_t T, int64_t N,
                        float alpha, float thresh)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float u = 0.0f;
        int s = 0;
        for (int64_t t = 0; t < T; ++t) {
            float leak = alpha * u;          /* rounded product */
            leak = leak * (float)(1 - s);    /* gate: times 1.0 or 0.0 */
            u = leak + x[t * N + n];
            s = u > thresh;
            if (spike) spike[t * N + n] = (float)s;
            if (mem) mem[t * N + n] = u;
        }
    }
}

/*
 * Reverse-time pass (snn_kernel_bp.cu:117-138). With gu the gradient w.r.t. u_{t+1}
 * (0 past the end):
 *   inside  = (u_t - thresh < interval) && (thresh - u_t < interval)
 *   gs      = inside ? g_t - (gu*alpha)*u_t : 0
 *   gu      = gs*beta + (gu*alpha)*(u_t <= thresh)
 *   grad_x_t = gu
 */
void oracle_lif_bwd_f32(const float *x, const float *grad_spike, float *grad_x, int64_t T,
                        int64_t N, float alpha, float thresh, float beta, float interval)
{
    if (T > ORACLE_MAX_T) return;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float ubuf[ORACLE_MAX_T];
        float u = 0.0f;
        int s = 0;
        for (int64_t t = 0; t < T; ++t) {
            float leak = alpha * u;
            leak = leak * (float)(1 - s);
            u = leak + x[t * N + n];
            s = u > thresh;
            ubuf[t] = u;
        }
        float gu = 0.0f;
        for (int64_t t = T - 1; t >= 0; --t) {
            float ut = ubuf[t];
            float ga = gu * alpha;
            float gs = 0.0f;
            if ((ut - thresh) < interval && (thresh - ut) < interval) {
                float r = ga * ut;
                gs = grad_spike[t * N + n] - r;
            }
            float a = gs * beta;
            float b = ga * (float)(ut <= thresh);
            gu = a + b;
            grad_x[t * N + n] = gu;
        }
    }
}

/* Same recurrences in double precision (the reference dispatches double as well;
 * alpha/thresh/beta/interval stay float arguments and are promoted). */
void oracle_lif_fwd_f64(const double *x, double *spike, double *mem, int64_t T, int64_t N,
                        float alpha, float thresh)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        double u = 0.0;
        int s = 0;
        for (int64_t t = 0; t < T; ++t) {
            double leak = (double)alpha * u;
            leak = leak * (double)(1 - s);
            u = leak + x[t * N + n];
            s = u > (double)thresh;
            if (spike) spike[t * N + n] = (double)s;
            if (mem) mem[t * N + n] = u;
        }
    }
}

void oracle_lif_bwd_f64(const double *x, const double *grad_spike, double *grad_x, int64_t T,
                        int64_t N, float alpha, float thresh, float beta, float interval)
{
    if (T > ORACLE_MAX_T) return;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        double ubuf[ORACLE_MAX_T];
        double u = 0.0;
        int s = 0;
        for (int64_t t = 0; t < T; ++t) {
            double leak = (double)alpha * u;
            leak = leak * (double)(1 - s);
            u = leak + x[t * N + n];
            s = u > (double)thresh;
            ubuf[t] = u;
        }
        double gu = 0.0;
        for (int64_t t = T - 1; t >= 0; --t) {
            double ut = ubuf[t];
            double ga = gu * (double)alpha;
            double gs = 0.0;
            if ((ut - (double)thresh) < (double)interval && ((double)thresh - ut) < (double)interval)
                gs = grad_spike[t * N + n] - ga * ut;
            gu = gs * (double)beta + ga * (double)(ut <= (double)thresh);
            grad_x[t * N + n] = gu;
        }
    }
}

/*
 * Packed spike words: bit t of word n is spike (t, n); one 32-bit word per neuron
 * covers T <= 32 time steps. Not part of the reference; it is the compact form the
 * CUDA forward can emit, restated here so tests can check it.
 */
void oracle_lif_fwd_bits_f32(const float *x, uint32_t *bits, int64_t T, int64_t N, float alpha,
                             float thresh)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float u = 0.0f;
        int s = 0;
        uint32_t w = 0;
        for (int64_t t = 0; t < T && t < 32; ++t) {
            float leak = alpha * u;
            leak = leak * (float)(1 - s);
            u = leak + x[t * N + n];
            s = u > thresh;
            w |= (uint32_t)s << t;
        }
        bits[n] = w;
    }
}

/* =========================================================================================
 * Batch-norm family (reference: snnlib/cuda/snn_kernel_fp.cu:80-122 bn_fp_kernel, :157-210
 * bn_fire_s_fp_kernel; snnlib/cuda/snn_kernel_bp.cu:175-285 bn_bp_*_kernel, :432-479
 * bn_fire_u_fp_kernel, :533-610 bn_fire_bp_wb_kernel, :613-677 bn_fire_bp_x_kernel).
 * Layout [T, B, C, HW] contiguous. fire != 0: BN folded into the LIF input; fire == 0: plain BN.
 * ======================================================================================= */

/* forward: w' = weight/sqrt(var+eps), ivar = w'/weight, current = (x-mean)*w' + bias.
 * If var == NULL, ivar_io is an input and w' = weight*ivar (the backward-time rebuild). */
void oracle_bn_lif_fwd_f32(const float *x, const float *var, const float *mean, const float *weight,
                           const float *bias, float eps, float *out, float *mem, float *ivar_io,
                           int64_t T, int64_t B, int64_t C, int64_t HW, int fire, float alpha,
                           float thresh)
{
    const int64_t CHW = C * HW, N = B * CHW;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < CHW; ++i) {
        const int64_t c = i / HW;
        const float m = mean[c], b = bias[c];
        float w;
        if (var) {
            w = weight[c] / sqrtf(var[c] + eps);
            if (i % HW == 0) ivar_io[c] = w / weight[c];
        } else {
            w = weight[c] * ivar_io[c];
        }
        for (int64_t bb = 0; bb < B; ++bb) {
            float u = 0.0f;
            int s = 0;
            for (int64_t t = 0; t < T; ++t) {
                const int64_t k = t * N + bb * CHW + i;
                float cur = (x[k] - m) * w;
                if (fire) {
                    float leak = alpha * u;
                    leak = leak * (float)(1 - s);
                    u = leak + cur;
                    u = u + b;
                    s = u > thresh;
                    if (out) out[k] = (float)s;
                    if (mem) mem[k] = u;
                } else {
                    out[k] = cur + b;
                }
            }
        }
    }
}

/* backward. Outputs: grad_x [T,B,C,HW]; grad_weight, grad_bias, gxhat, gxhatx [C].
 * If use_given_means != 0, gxhat/gxhatx are inputs (the second half of the sync-BN split). */
void oracle_bn_lif_bwd_f32(const float *x, const float *grad, const float *ivar, const float *mean,
                           const float *weight, const float *bias, float *grad_x, float *grad_weight,
                           float *grad_bias, float *gxhat, float *gxhatx, int use_given_means,
                           int64_t T, int64_t B, int64_t C, int64_t HW, int fire, float alpha,
                           float thresh, float beta, float interval)
{
    const int64_t CHW = C * HW, N = B * CHW;
    if (T > ORACLE_MAX_T) return;
    /* pass 1: per-position sums in float (as the reference kernel accumulates them), combined
     * over the positions of a channel in double */
    double *acc = (double *)calloc((size_t)C * 4, sizeof(double));
    for (int64_t i = 0; i < CHW; ++i) {
        const int64_t c = i / HW;
        const float m = mean[c], w = weight[c], iv = ivar[c], b = fire ? bias[c] : 0.0f;
        const float wiv = w * iv;
        float sb = 0.0f, sw = 0.0f, sx = 0.0f, sxx = 0.0f;
        for (int64_t bb = 0; bb < B; ++bb) {
            float ubuf[ORACLE_MAX_T];
            if (fire) {
                float u = 0.0f;
                int s = 0;
                for (int64_t t = 0; t < T; ++t) {
                    const int64_t k = t * N + bb * CHW + i;
                    float leak = alpha * u;
                    leak = leak * (float)(1 - s);
                    u = leak + (x[k] - m) * wiv;
                    u = u + b;
                    s = u > thresh;
                    ubuf[t] = u;
                }
            }
            float gu = 0.0f;
            for (int64_t t = T - 1; t >= 0; --t) {
                const int64_t k = t * N + bb * CHW + i;
                if (fire) {
                    const float ut = ubuf[t];
                    const float ga = gu * alpha;
                    float gs = 0.0f;
                    if ((ut - thresh) < interval && (thresh - ut) < interval) gs = grad[k] - ga * ut;
                    gu = gs * beta + ga * (float)(ut <= thresh);
                } else {
                    gu = grad[k];
                }
                const float xh = (x[k] - m) * iv;
                sb += gu;
                sw += gu * xh;
                sx += gu * w;
                sxx += gu * w * xh;
            }
        }
        acc[c * 4 + 0] += sb;
        acc[c * 4 + 1] += sw;
        acc[c * 4 + 2] += (double)(sx / (float)(T * B));
        acc[c * 4 + 3] += (double)(sxx / (float)(T * B));
    }
    for (int64_t c = 0; c < C; ++c) {
        grad_bias[c] = (float)acc[c * 4 + 0];
        grad_weight[c] = (float)acc[c * 4 + 1];
        if (!use_given_means) {
            gxhat[c] = (float)(acc[c * 4 + 2] / (double)HW);
            gxhatx[c] = (float)(acc[c * 4 + 3] / (double)HW);
        }
    }
    free(acc);
    /* pass 2: input gradient */
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < CHW; ++i) {
        const int64_t c = i / HW;
        const float m = mean[c], w = weight[c], iv = ivar[c], b = fire ? bias[c] : 0.0f;
        const float wiv = w * iv, gh = gxhat[c], ghx = gxhatx[c];
        for (int64_t bb = 0; bb < B; ++bb) {
            float ubuf[ORACLE_MAX_T];
            if (fire) {
                float u = 0.0f;
                int s = 0;
                for (int64_t t = 0; t < T; ++t) {
                    const int64_t k = t * N + bb * CHW + i;
                    float leak = alpha * u;
                    leak = leak * (float)(1 - s);
                    u = leak + (x[k] - m) * wiv;
                    u = u + b;
                    s = u > thresh;
                    ubuf[t] = u;
                }
            }
            float gu = 0.0f;
            for (int64_t t = T - 1; t >= 0; --t) {
                const int64_t k = t * N + bb * CHW + i;
                if (fire) {
                    const float ut = ubuf[t];
                    const float ga = gu * alpha;
                    float gs = 0.0f;
                    if ((ut - thresh) < interval && (thresh - ut) < interval) gs = grad[k] - ga * ut;
                    gu = gs * beta + ga * (float)(ut <= thresh);
                } else {
                    gu = grad[k];
                }
                const float xh = (x[k] - m) * iv;
                grad_x[k] = gu * w * iv - iv * (xh * ghx + gh);
            }
        }
    }
}
