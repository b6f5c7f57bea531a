/*
 * CPU oracle for the dense-contraction path of CrusaderBackend's seblas library.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA kernels are compared against and the
 * timed CPU baseline of the benchmark. Nothing in the shipped library calls it.
 *
 * Parity status: the reference ships no golden vectors, fixtures or known-answer tests for this path
 * (its validation/UnitTestTools.cu compares kernels with cuDNN by hand); the restatement below is pinned
 * instead against outputs of the reference's own seblas kernels, rebuilt for sm_100 and run on a B200,
 * stored under tests/golden/ together with the script that produced them.
 *
 * Every *_f64 function accumulates in double from fp32 inputs and returns doubles: it is the ground
 * truth. Every *_f32 function is the same loop in fp32 with OpenMP and is what the benchmark times.
 * All tensors are dense row-major / NCHW as in seblas/tensor/Tensor.cuh:48-99.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef long long i64;

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the timed baseline asks for the cores it is meant to use. */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------------------------ GEMM
 * C = op(A) * op(B): semantics of seblas::sgemm / sgemmTN / sgemmNT (seblas/operations/cuGEMM.cu:1649-1699).
 * transA: A is stored K x M; transB: B is stored N x K. */
static inline float a_at(const float* A, int lda, int transA, int m, int k) {
    return transA ? A[(i64)k * lda + m] : A[(i64)m * lda + k];
}
static inline float b_at(const float* B, int ldb, int transB, int k, int n) {
    return transB ? B[(i64)n * ldb + k] : B[(i64)k * ldb + n];
}

void orc_gemm_f64(int transA, int transB, int M, int N, int K, const float* A, int lda, const float* B, int ldb,
                  double* C, int ldc) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        double* row = C + (i64)m * ldc;
        for (int n = 0; n < N; ++n) row[n] = 0.0;
        for (int k = 0; k < K; ++k) {
            const double a = (double)a_at(A, lda, transA, m, k);
            if (!transB) {
                const float* b = B + (i64)k * ldb;
                for (int n = 0; n < N; ++n) row[n] += a * (double)b[n];
            } else {
                for (int n = 0; n < N; ++n) row[n] += a * (double)B[(i64)n * ldb + k];
            }
        }
    }
}

/* Selected rows of C only (fp64), for sampled checks of large products: out is nrows x N. */
void orc_gemm_f64_rows(int transA, int transB, int M, int N, int K, const float* A, int lda, const float* B,
                       int ldb, const int* rows, int nrows, double* out) {
    (void)M;
#pragma omp parallel for schedule(dynamic)
    for (int r = 0; r < nrows; ++r) {
        const int m = rows[r];
        double* row = out + (i64)r * N;
        for (int n = 0; n < N; ++n) row[n] = 0.0;
        for (int k = 0; k < K; ++k) {
            const double a = (double)a_at(A, lda, transA, m, k);
            for (int n = 0; n < N; ++n) row[n] += a * (double)b_at(B, ldb, transB, k, n);
        }
    }
}

/* Selected columns of C only (fp64): out is M x ncols. */
void orc_gemm_f64_cols(int transA, int transB, int M, int N, int K, const float* A, int lda, const float* B,
                       int ldb, const int* cols, int ncols, double* out) {
    (void)N;
#pragma omp parallel for schedule(dynamic)
    for (int m = 0; m < M; ++m) {
        for (int c = 0; c < ncols; ++c) {
            const int n = cols[c];
            double s = 0.0;
            for (int k = 0; k < K; ++k) s += (double)a_at(A, lda, transA, m, k) * (double)b_at(B, ldb, transB, k, n);
            out[(i64)m * ncols + c] = s;
        }
    }
}

/* fp32 OpenMP GEMM (timed CPU baseline). Cache-blocked i-k-j; accumulate != 0 adds to C as seblas::sgemmNTA
 * does (seblas/operations/cuGEMM.cu:1701-1714). */
void orc_gemm_f32(int transA, int transB, int M, int N, int K, const float* A, int lda, const float* B, int ldb,
                  float* C, int ldc, int accumulate) {
    const int BM = 64, BKc = 256;
    float* Bt = NULL;
    const float* Bn = B;
    int ldbn = ldb;
    if (transB) { /* make B K x N once so the inner loop streams unit-stride */
        Bt = (float*)malloc((size_t)K * N * sizeof(float));
#pragma omp parallel for schedule(static)
        for (int k = 0; k < K; ++k)
            for (int n = 0; n < N; ++n) Bt[(i64)k * N + n] = B[(i64)n * ldb + k];
        Bn = Bt;
        ldbn = N;
    }
#pragma omp parallel for schedule(dynamic)
    for (int m0 = 0; m0 < M; m0 += BM) {
        const int m1 = m0 + BM < M ? m0 + BM : M;
        if (!accumulate)
            for (int m = m0; m < m1; ++m) memset(C + (i64)m * ldc, 0, (size_t)N * sizeof(float));
        for (int k0 = 0; k0 < K; k0 += BKc) {
            const int k1 = k0 + BKc < K ? k0 + BKc : K;
            for (int m = m0; m < m1; ++m) {
                float* row = C + (i64)m * ldc;
                for (int k = k0; k < k1; ++k) {
                    const float a = a_at(A, lda, transA, m, k);
                    const float* b = Bn + (i64)k * ldbn;
                    for (int n = 0; n < N; ++n) row[n] += a * b[n];
                }
            }
        }
    }
    free(Bt);
}

/* ------------------------------------------------------------------------------------------ convolution
 * Forward: index map of gemmImplicit4D (seblas/operations/cuConv.cu:105-115): ih = oh*sH - pH + fh,
 * iw = ow*sW - pW + fw, out-of-range taps read zero; bias added per output channel (:235-239).
 * W: OC x IC x FH x FW, X: N x IC x IH x IW, Y: N x OC x OH x OW, OH = (IH - FH + 2 pH)/sH + 1 (cuConv.cu:731-755). */
#define CONV_FWD_BODY(ACC_T, OUT_T)                                                                              \
    const int OH = (IH - FH + 2 * pH) / sH + 1, OW = (IW - FW + 2 * pW) / sW + 1;                                \
    _Pragma("omp parallel for collapse(2) schedule(static)") for (int n = 0; n < N; ++n) for (int oc = 0; oc < OC; \
                                                                                            ++oc) {              \
        for (int oh = 0; oh < OH; ++oh)                                                                          \
            for (int ow = 0; ow < OW; ++ow) {                                                                    \
                ACC_T acc = bias ? (ACC_T)bias[oc] : (ACC_T)0;                                                   \
                for (int ic = 0; ic < IC; ++ic)                                                                  \
                    for (int fh = 0; fh < FH; ++fh) {                                                            \
                        const int ih = oh * sH - pH + fh;                                                        \
                        if (ih < 0 || ih >= IH) continue;                                                        \
                        for (int fw = 0; fw < FW; ++fw) {                                                        \
                            const int iw = ow * sW - pW + fw;                                                    \
                            if (iw < 0 || iw >= IW) continue;                                                    \
                            acc += (ACC_T)W[(((i64)oc * IC + ic) * FH + fh) * FW + fw] *                         \
                                   (ACC_T)X[(((i64)n * IC + ic) * IH + ih) * IW + iw];                           \
                        }                                                                                        \
                    }                                                                                            \
                Y[(((i64)n * OC + oc) * OH + oh) * OW + ow] = (OUT_T)acc;                                        \
            }                                                                                                    \
    }

void orc_conv_fwd_f64(const float* W, const float* X, const float* bias, double* Y, int N, int IC, int IH, int IW,
                      int OC, int FH, int FW, int sH, int sW, int pH, int pW) {
    CONV_FWD_BODY(double, double)
}
void orc_conv_fwd_f32(const float* W, const float* X, const float* bias, float* Y, int N, int IC, int IH, int IW,
                      int OC, int FH, int FW, int sH, int sW, int pH, int pW) {
    CONV_FWD_BODY(float, float)
}

/* Data gradient (seblas::convDerive, cuConv.cu:774-791; kernel :262-486): dX[n,ic,ih,iw] = sum over (oc,fh,fw)
 * of W[oc,ic,fh,fw] * dY[n,oc,oh,ow] for the (oh,ow) with ih = oh*sH - pH + fh, iw = ow*sW - pW + fw.
 * The reference reaches the same sum by rotating the filter 180 degrees (:321-326), inserting zeros between
 * the dY samples (ih % stride == 0, :347-352) and padding by newPad = (IH + FH - 1 - OH*s)/2 (:780-781), which
 * equals FH - 1 - pH for every shape whose forward geometry is exact. */
#define CONV_DGRAD_BODY(ACC_T, OUT_T)                                                                            \
    const int OH = (IH - FH + 2 * pH) / sH + 1, OW = (IW - FW + 2 * pW) / sW + 1;                                \
    _Pragma("omp parallel for collapse(2) schedule(static)") for (int n = 0; n < N; ++n) for (int ic = 0; ic < IC; \
                                                                                            ++ic) {              \
        for (int ih = 0; ih < IH; ++ih)                                                                          \
            for (int iw = 0; iw < IW; ++iw) {                                                                    \
                ACC_T acc = (ACC_T)0;                                                                            \
                for (int fh = 0; fh < FH; ++fh) {                                                                \
                    const int th = ih + pH - fh;                                                                 \
                    if (th < 0 || th % sH) continue;                                                             \
                    const int oh = th / sH;                                                                      \
                    if (oh >= OH) continue;                                                                      \
                    for (int fw = 0; fw < FW; ++fw) {                                                            \
                        const int tw = iw + pW - fw;                                                             \
                        if (tw < 0 || tw % sW) continue;                                                         \
                        const int ow = tw / sW;                                                                  \
                        if (ow >= OW) continue;                                                                  \
                        for (int oc = 0; oc < OC; ++oc)                                                          \
                            acc += (ACC_T)W[(((i64)oc * IC + ic) * FH + fh) * FW + fw] *                         \
                                   (ACC_T)dY[(((i64)n * OC + oc) * OH + oh) * OW + ow];                          \
                    }                                                                                            \
                }                                                                                                \
                dX[(((i64)n * IC + ic) * IH + ih) * IW + iw] = (OUT_T)acc;                                       \
            }                                                                                                    \
    }

void orc_conv_dgrad_f64(const float* W, const float* dY, double* dX, int N, int IC, int IH, int IW, int OC, int FH,
                        int FW, int sH, int sW, int pH, int pW) {
    CONV_DGRAD_BODY(double, double)
}
void orc_conv_dgrad_f32(const float* W, const float* dY, float* dX, int N, int IC, int IH, int IW, int OC, int FH,
                        int FW, int sH, int sW, int pH, int pW) {
    CONV_DGRAD_BODY(float, float)
}

/* Weight gradient (seblas::convError, cuConv.cu:793-806; kernel :488-707): dW[oc,ic,fh,fw] (+)= sum over
 * (n,oh,ow) of dY[n,oc,oh,ow] * X[n,ic,oh*sH - pH + fh,ow*sW - pW + fw]. The reference accumulates into dW
 * (:702-703). Its kernel computes ih = fh*stride - pad + oh*stride (:570-571), which is only right for
 * stride 1; this restatement uses the mathematically correct map for every stride. */
#define CONV_WGRAD_BODY(ACC_T)                                                                                   \
    const int OH = (IH - FH + 2 * pH) / sH + 1, OW = (IW - FW + 2 * pW) / sW + 1;                                \
    _Pragma("omp parallel for collapse(2) schedule(static)") for (int oc = 0; oc < OC; ++oc) for (int ic = 0;    \
                                                                                                ic < IC; ++ic) { \
        for (int fh = 0; fh < FH; ++fh)                                                                          \
            for (int fw = 0; fw < FW; ++fw) {                                                                    \
                ACC_T acc = (ACC_T)0;                                                                            \
                for (int n = 0; n < N; ++n)                                                                      \
                    for (int oh = 0; oh < OH; ++oh) {                                                            \
                        const int ih = oh * sH - pH + fh;                                                        \
                        if (ih < 0 || ih >= IH) continue;                                                        \
                        for (int ow = 0; ow < OW; ++ow) {                                                        \
                            const int iw = ow * sW - pW + fw;                                                    \
                            if (iw < 0 || iw >= IW) continue;                                                    \
                            acc += (ACC_T)dY[(((i64)n * OC + oc) * OH + oh) * OW + ow] *                         \
                                   (ACC_T)X[(((i64)n * IC + ic) * IH + ih) * IW + iw];                           \
                        }                                                                                        \
                    }                                                                                            \
                const i64 o = (((i64)oc * IC + ic) * FH + fh) * FW + fw;                                         \
                dW[o] = accumulate ? dW[o] + acc : acc;                                                          \
            }                                                                                                    \
    }

void orc_conv_wgrad_f64(const float* dY, const float* X, double* dW, int N, int IC, int IH, int IW, int OC, int FH,
                        int FW, int sH, int sW, int pH, int pW, int accumulate) {
    CONV_WGRAD_BODY(double)
}
void orc_conv_wgrad_f32(const float* dY, const float* X, float* dW, int N, int IC, int IH, int IW, int OC, int FH,
                        int FW, int sH, int sW, int pH, int pW, int accumulate) {
    CONV_WGRAD_BODY(float)
}

/* The weight-gradient index map exactly as the reference kernel evaluates it (cuConv.cu:570-571):
 * ih = fh*sH - pH + oh*sH. Kept so the golden vectors of the reference can be explained at stride > 1. */
void orc_conv_wgrad_refmap_f64(const float* dY, const float* X, double* dW, int N, int IC, int IH, int IW, int OC,
                               int FH, int FW, int sH, int sW, int pH, int pW) {
    const int OH = (IH - FH + 2 * pH) / sH + 1, OW = (IW - FW + 2 * pW) / sW + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int oc = 0; oc < OC; ++oc)
        for (int ic = 0; ic < IC; ++ic)
            for (int fh = 0; fh < FH; ++fh)
                for (int fw = 0; fw < FW; ++fw) {
                    double acc = 0.0;
                    for (int n = 0; n < N; ++n)
                        for (int oh = 0; oh < OH; ++oh) {
                            const int ih = fh * sH - pH + oh * sH;
                            if (ih < 0 || ih >= IH) continue;
                            for (int ow = 0; ow < OW; ++ow) {
                                const int iw = fw * sW - pW + ow * sW;
                                if (iw < 0 || iw >= IW) continue;
                                acc += (double)dY[(((i64)n * OC + oc) * OH + oh) * OW + ow] *
                                       (double)X[(((i64)n * IC + ic) * IH + ih) * IW + iw];
                            }
                        }
                    dW[(((i64)oc * IC + ic) * FH + fh) * FW + fw] = acc;
                }
}

/* Bias gradient of a convolution: db[c] = sum over (n,h,w) of dY (cuDNN backward-bias as called by
 * seann/operands/cudnn/cuConv2D.cu:69). */
void orc_conv_bias_grad_f64(const float* dY, double* db, int N, int C, int HW) {
    for (int c = 0; c < C; ++c) {
        double s = 0.0;
        for (int n = 0; n < N; ++n)
            for (int i = 0; i < HW; ++i) s += (double)dY[((i64)n * C + c) * HW + i];
        db[c] = s;
    }
}

/* ------------------------------------------------------------------------------------------ Linear
 * seblas::linear (cuLinear.cu:1052-1072; kernel :33-222): Y[n,m] = sum_k W[m,k] X[n,k] + b[m].
 * X: batch x IN, W: OUT x IN, b: OUT, Y: batch x OUT. */
void orc_linear_f64(const float* X, const float* W, const float* b, double* Y, int batch, int IN, int OUT) {
    for (int n = 0; n < batch; ++n)
        for (int m = 0; m < OUT; ++m) {
            double s = b ? (double)b[m] : 0.0;
            for (int k = 0; k < IN; ++k) s += (double)W[(i64)m * IN + k] * (double)X[(i64)n * IN + k];
            Y[(i64)n * OUT + m] = s;
        }
}
/* seblas::linearXGrad (cuLinear.cu:1075-1095): dX[n,k] = sum_m W[m,k] dY[n,m]. */
void orc_linear_xgrad_f64(const float* dY, const float* W, double* dX, int batch, int IN, int OUT) {
    for (int n = 0; n < batch; ++n)
        for (int k = 0; k < IN; ++k) {
            double s = 0.0;
            for (int m = 0; m < OUT; ++m) s += (double)W[(i64)m * IN + k] * (double)dY[(i64)n * OUT + m];
            dX[(i64)n * IN + k] = s;
        }
}
/* seblas::linearParamGrad (cuLinear.cu:1098-1115; kernel :872-1049): dW[m,k] += sum_n dY[n,m] X[n,k];
 * db[m] += sum_n dY[n,m], each counted once (the reference kernel adds db from every thread column,
 * cuLinear.cu:1037-1040, so its db is not a usable oracle). dW/db hold the values to accumulate onto. */
void orc_linear_paramgrad_f64(const float* dY, const float* X, double* dW, double* db, int batch, int IN, int OUT) {
    for (int m = 0; m < OUT; ++m) {
        for (int k = 0; k < IN; ++k) {
            double s = 0.0;
            for (int n = 0; n < batch; ++n) s += (double)dY[(i64)n * OUT + m] * (double)X[(i64)n * IN + k];
            dW[(i64)m * IN + k] += s;
        }
        if (db) {
            double s = 0.0;
            for (int n = 0; n < batch; ++n) s += (double)dY[(i64)n * OUT + m];
            db[m] += s;
        }
    }
}

/* ------------------------------------------------------------------------------------------ BatchNorm
 * seblas::batchNorm (cuBatchNorm.cu:14-61): statistics per (c,h,w) position over the batch only,
 * biased variance, eps = 1e-8 inside the square root. P = C*H*W positions. */
void orc_bn_fwd_f64(const float* X, const float* beta, const float* gamma, double* mean, double* var, double* Y,
                    double* xhat, int N, int P) {
#pragma omp parallel for schedule(static)
    for (int p = 0; p < P; ++p) {
        double m = 0.0, v = 0.0;
        for (int n = 0; n < N; ++n) m += (double)X[(i64)n * P + p];
        m /= (double)N;
        for (int n = 0; n < N; ++n) {
            const double d = (double)X[(i64)n * P + p] - m;
            v += d * d;
        }
        v /= (double)N;
        const double inv = 1.0 / sqrt(v + 1e-8);
        for (int n = 0; n < N; ++n) {
            const double xh = ((double)X[(i64)n * P + p] - m) * inv;
            if (xhat) xhat[(i64)n * P + p] = xh;
            Y[(i64)n * P + p] = xh * (double)gamma[p] + (double)beta[p];
        }
        if (mean) mean[p] = m;
        if (var) var[p] = v;
    }
}
/* seblas::batchNormGrad (cuBatchNorm.cu:64-125): statistics recomputed from X, then
 *   dxhat = dy*gamma; dvar = sum dxhat (x-mean) (-1/2)(var+eps)^(-3/2);
 *   dmean = sum -dxhat/sqrt(var+eps) + dvar * sum(-2 (x-mean)) / N;
 *   dx = dxhat/sqrt(var+eps) + dvar 2 (x-mean)/N + dmean/N. */
void orc_bn_bwd_f64(const float* dY, const float* gamma, const float* X, double* dX, int N, int P) {
#pragma omp parallel for schedule(static)
    for (int p = 0; p < P; ++p) {
        double m = 0.0, v = 0.0;
        for (int n = 0; n < N; ++n) m += (double)X[(i64)n * P + p];
        m /= (double)N;
        for (int n = 0; n < N; ++n) {
            const double d = (double)X[(i64)n * P + p] - m;
            v += d * d;
        }
        v /= (double)N;
        const double g = (double)gamma[p];
        const double inv = 1.0 / sqrt(v + 1e-8);
        double dvar = 0.0, dmean = 0.0, temp = 0.0;
        for (int n = 0; n < N; ++n) {
            const double xc = (double)X[(i64)n * P + p] - m;
            const double dxh = (double)dY[(i64)n * P + p] * g;
            dvar += dxh * xc * -0.5 * pow(v + 1e-8, -1.5);
            dmean += -dxh * inv;
            temp += -2.0 * xc;
        }
        dmean += dvar * temp / (double)N;
        for (int n = 0; n < N; ++n) {
            const double xc = (double)X[(i64)n * P + p] - m;
            const double dxh = (double)dY[(i64)n * P + p] * g;
            dX[(i64)n * P + p] = dxh * inv + dvar * xc * 2.0 / (double)N + dmean / (double)N;
        }
    }
}
/* seblas::batchNormParamGrads (cuBatchNorm.cu:128-147): dgamma[p] = sum_n dy*xhat, dbeta[p] = sum_n dy
 * (assigned, not accumulated). */
void orc_bn_paramgrad_f64(const float* dY, const float* xhat, double* dgamma, double* dbeta, int N, int P) {
#pragma omp parallel for schedule(static)
    for (int p = 0; p < P; ++p) {
        double g = 0.0, b = 0.0;
        for (int n = 0; n < N; ++n) {
            const double dy = (double)dY[(i64)n * P + p];
            b += dy;
            g += dy * (double)xhat[(i64)n * P + p];
        }
        dgamma[p] = g;
        dbeta[p] = b;
    }
}

/* ------------------------------------------------------------------------------------------ activations / pooling
 * seblas::relu (cuActivation.cu:268) and reluGradFast (:296): y = max(x,0); dx = x > 0 ? dy : 0. */
void orc_relu_f64(const float* X, double* Y, i64 n) {
    for (i64 i = 0; i < n; ++i) Y[i] = X[i] > 0.f ? (double)X[i] : 0.0;
}
void orc_relu_grad_f64(const float* X, const float* dY, double* dX, i64 n) {
    for (i64 i = 0; i < n; ++i) dX[i] = X[i] > 0.f ? (double)dY[i] : 0.0;
}
/* seblas::avgPool / avgPoolBack (cuPool.cu:75-119,153-169): non-overlapping windows (range == stride),
 * mean of the window; the gradient is spread evenly over the window. X: NC x H x W, Y: NC x H/r x W/r. */
void orc_avgpool_f64(const float* X, double* Y, int NC, int H, int W, int rH, int rW) {
    const int OH = H / rH, OW = W / rW;
    for (int c = 0; c < NC; ++c)
        for (int oh = 0; oh < OH; ++oh)
            for (int ow = 0; ow < OW; ++ow) {
                double s = 0.0;
                for (int i = 0; i < rH; ++i)
                    for (int j = 0; j < rW; ++j) s += (double)X[((i64)c * H + oh * rH + i) * W + ow * rW + j];
                Y[((i64)c * OH + oh) * OW + ow] = s / (double)(rH * rW);
            }
}
void orc_avgpool_back_f64(const float* dY, double* dX, int NC, int H, int W, int rH, int rW) {
    const int OH = H / rH, OW = W / rW;
    for (i64 i = 0; i < (i64)NC * H * W; ++i) dX[i] = 0.0;
    for (int c = 0; c < NC; ++c)
        for (int oh = 0; oh < OH; ++oh)
            for (int ow = 0; ow < OW; ++ow) {
                const double g = (double)dY[((i64)c * OH + oh) * OW + ow] / (double)(rH * rW);
                for (int i = 0; i < rH; ++i)
                    for (int j = 0; j < rW; ++j) dX[((i64)c * H + oh * rH + i) * W + ow * rW + j] = g;
            }
}
/* seblas::globalAvgPool / globalAvgPoolBack (cuPool.cu:121-133,171-184): mean over H*W per (n,c). */
void orc_gap_f64(const float* X, double* Y, int NC, int HW) {
    for (int c = 0; c < NC; ++c) {
        double s = 0.0;
        for (int i = 0; i < HW; ++i) s += (double)X[(i64)c * HW + i];
        Y[c] = s / (double)HW;
    }
}
void orc_gap_back_f64(const float* dY, double* dX, int NC, int HW) {
    for (int c = 0; c < NC; ++c)
        for (int i = 0; i < HW; ++i) dX[(i64)c * HW + i] = (double)dY[c] / (double)HW;
}

/* ------------------------------------------------------------------------------------------ loss / optimizer
 * seblas::softmax, single-block path (cuReduce.cu:98-147): y = exp(x - max) / (sum + 1e-10) per row of `step`. */
void orc_softmax_f64(const float* X, double* Y, int rows, int step) {
    for (int r = 0; r < rows; ++r) {
        double mx = -1e300;
        for (int i = 0; i < step; ++i) mx = X[(i64)r * step + i] > mx ? X[(i64)r * step + i] : mx;
        double s = 0.0;
        for (int i = 0; i < step; ++i) s += exp((double)X[(i64)r * step + i] - mx);
        for (int i = 0; i < step; ++i) Y[(i64)r * step + i] = exp((double)X[(i64)r * step + i] - mx) / (s + 1e-10);
    }
}
/* seblas::crossEntropyLoss (cuLoss.cu:231-234): dY = Y - labels; crossEntropyCalc (:31-37,220-229):
 * loss = sum over all elements of -log(y + 1e-10) * label. Returns the loss. */
double orc_cross_entropy_f64(const float* Y, const float* labels, double* dY, i64 n) {
    double loss = 0.0;
    for (i64 i = 0; i < n; ++i) {
        if (dY) dY[i] = (double)Y[i] - (double)labels[i];
        loss += -log((double)Y[i] + 1e-10) * (double)labels[i];
    }
    return loss;
}
/* seann::Momentum::apply (seann/optimizers/Optimizers.cu:17-22) over seblas::momentumApply
 * (cuOptim.cu:38-46): w *= (1 - l2) for weight tensors, m = beta m + (1 - beta) g, w -= lr m, g = 0.
 * Updates w, m, g in place (doubles). */
void orc_momentum_f64(double* w, double* g, double* m, i64 n, double lr, double beta, double l2, int is_weight) {
    for (i64 i = 0; i < n; ++i) {
        if (is_weight) w[i] *= (1.0 - l2);
        const double mv = beta * m[i] + (1.0 - beta) * g[i];
        w[i] -= lr * mv;
        m[i] = mv;
        g[i] = 0.0;
    }
}
/* Same update in fp32, operation by operation as the reference kernels perform it. */
void orc_momentum_f32(float* w, float* g, float* m, i64 n, float lr, float beta, float l2, int is_weight) {
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; ++i) {
        float wv = w[i];
        if (is_weight) wv = wv * (1.0f - l2);
        const float mv = beta * m[i] + (1.0f - beta) * g[i];
        wv -= lr * mv;
        w[i] = wv;
        m[i] = mv;
        g[i] = 0.0f;
    }
}

/* ---- fp32 OpenMP BatchNorm (timed CPU baseline only; the checker uses the fp64 versions above) ------------------
 * Same arithmetic as seblas::batchNorm / batchNormGrad / batchNormParamGrads (seblas/operations/cuBatchNorm.cu:14-147):
 * statistics per position p over the batch, eps = 1e-8, the backward pass recomputes them from X. Optional tail of the
 * forward pass: + res (shortcut add), then ReLU. */
void orc_bn_fwd_f32(const float* X, const float* beta, const float* gamma, const float* res, float* Y, int N, long long P,
                    int relu) {
#pragma omp parallel for schedule(static)
    for (long long p = 0; p < P; ++p) {
        float m = 0.f, v = 0.f;
        for (int n = 0; n < N; ++n) m += X[n * P + p];
        m /= (float)N;
        for (int n = 0; n < N; ++n) { const float d = X[n * P + p] - m; v += d * d; }
        v /= (float)N;
        const float inv = 1.0f / sqrtf(v + 1e-8f);
        for (int n = 0; n < N; ++n) {
            float y = (X[n * P + p] - m) * inv * gamma[p] + beta[p];
            if (res) y += res[n * P + p];
            if (relu && y < 0.f) y = 0.f;
            Y[n * P + p] = y;
        }
    }
}

void orc_bn_bwd_f32(const float* dY, const float* gamma, const float* X, float* dX, float* dgamma, float* dbeta, int N,
                    long long P) {
    const float invN = 1.0f / (float)N;
#pragma omp parallel for schedule(static)
    for (long long p = 0; p < P; ++p) {
        float m = 0.f, v = 0.f;
        for (int n = 0; n < N; ++n) m += X[n * P + p];
        m *= invN;
        float sdx = 0.f, sd = 0.f, sxc = 0.f;
        for (int n = 0; n < N; ++n) {
            const float xc = X[n * P + p] - m, dy = dY[n * P + p];
            v += xc * xc; sdx += dy * xc; sd += dy; sxc += xc;
        }
        const float inv = 1.0f / sqrtf(v * invN + 1e-8f);
        const float g = gamma[p];
        const float dvar = g * sdx * -0.5f * inv * inv * inv;
        const float dmean = -g * sd * inv + dvar * (-2.0f * sxc) * invN;
        for (int n = 0; n < N; ++n)
            dX[n * P + p] = dY[n * P + p] * g * inv + dvar * (X[n * P + p] - m) * 2.0f * invN + dmean * invN;
        dbeta[p] = sd;
        dgamma[p] = sdx * inv;
    }
}
