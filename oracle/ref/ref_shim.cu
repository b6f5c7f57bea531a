// C entry points over the REFERENCE's own seblas kernels (compiled from the reference tree by build_ref.sh into
// oracle/_ref/libseblas_ref.so). Test infrastructure: used to record golden vectors from the reference itself
// and to time it beside the new kernels. Every function takes device pointers; the seblas::Tensor headers the
// reference kernels dereference are created in pinned host memory exactly as the reference does
// (seblas/tensor/Tensor.cuh:97-110).
#include "seblas/operations/cuOperations.cuh"

using namespace seblas;

namespace {
Tensor* view(float* p, uint32 n, uint32 c, uint32 h, uint32 w) {
    return Tensor::declare(shape4(n, c, h, w))->attach(p, 0);
}
void drop(Tensor* t) {
    cudnnDestroyTensorDescriptor(t->cudnnDesc);
    cudaFreeHost(t);
}
template <typename F>
int guarded(F f) {
    try {
        f();
    } catch (const std::exception& e) {
        fprintf(stderr, "[ref] exception: %s\n", e.what());
        return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
}  // namespace

extern "C" {

// form 0: sgemm (C[b] = A B[b]); 1: sgemmTN (A stored K x M); 2: sgemmNT (B stored N x K, batch must be 1)
int ref_gemm(int form, float* A, float* B, float* C, int M, int N, int K, int batch) {
    return guarded([&] {
        Tensor* a = form == 1 ? view(A, 1, 1, K, M) : view(A, 1, 1, M, K);
        Tensor* b = form == 2 ? view(B, 1, 1, N, K) : view(B, batch, 1, K, N);
        Tensor* c = view(C, batch, 1, M, N);
        if (form == 0) sgemm(a, b, c);
        else if (form == 1) sgemmTN(a, b, c);
        else sgemmNT(a, b, c);
        drop(a); drop(b); drop(c);
    });
}

// sgemmNTA: C += sum over n of A[n] * B[n]^T (A batch x M x K, B batch x N x K, C M x N)
int ref_gemm_nta(float* A, float* B, float* C, int M, int N, int K, int batch) {
    return guarded([&] {
        Tensor* a = view(A, batch, 1, M, K);
        Tensor* b = view(B, batch, 1, N, K);
        Tensor* c = view(C, 1, 1, M, N);
        sgemmNTA(a, b, c);
        drop(a); drop(b); drop(c);
    });
}

int ref_conv(float* W, float* X, float* Y, float* bias, int N, int IC, int IH, int IW, int OC, int FH, int FW, int sH,
             int sW, int pH, int pW) {
    return guarded([&] {
        const int OH = (IH - FH + 2 * pH) / sH + 1, OW = (IW - FW + 2 * pW) / sW + 1;
        Tensor* w = view(W, OC, IC, FH, FW);
        Tensor* x = view(X, N, IC, IH, IW);
        Tensor* y = view(Y, N, OC, OH, OW);
        Tensor* b = bias ? view(bias, 1, 1, OC, 1) : nullptr;
        conv(w, x, y, sH, sW, pH, pW, b);
        drop(w); drop(x); drop(y);
        if (b) drop(b);
    });
}

int ref_conv_derive(float* W, float* dY, float* dX, int N, int IC, int IH, int IW, int OC, int FH, int FW, int sH,
                    int sW, int pH, int pW) {
    return guarded([&] {
        const int OH = (IH - FH + 2 * pH) / sH + 1, OW = (IW - FW + 2 * pW) / sW + 1;
        Tensor* w = view(W, OC, IC, FH, FW);
        Tensor* dy = view(dY, N, OC, OH, OW);
        Tensor* dx = view(dX, N, IC, IH, IW);
        convDerive(w, dy, dx, sH, sW, pH, pW);
        drop(w); drop(dy); drop(dx);
    });
}

int ref_conv_error(float* dY, float* X, float* dW, int N, int IC, int IH, int IW, int OC, int FH, int FW, int sH,
                   int sW, int pH, int pW) {
    return guarded([&] {
        const int OH = (IH - FH + 2 * pH) / sH + 1, OW = (IW - FW + 2 * pW) / sW + 1;
        Tensor* dy = view(dY, N, OC, OH, OW);
        Tensor* x = view(X, N, IC, IH, IW);
        Tensor* dw = view(dW, OC, IC, FH, FW);
        convError(dy, x, dw, sH, sW, pH, pW);
        drop(dy); drop(x); drop(dw);
    });
}

int ref_linear(float* X, float* W, float* B, float* Y, int batch, int IN, int OUT) {
    return guarded([&] {
        Tensor* x = view(X, batch, 1, IN, 1);
        Tensor* w = view(W, 1, 1, OUT, IN);
        Tensor* b = view(B, 1, 1, OUT, 1);
        Tensor* y = view(Y, batch, 1, OUT, 1);
        linear(x, w, b, y);
        drop(x); drop(w); drop(b); drop(y);
    });
}

int ref_linear_xgrad(float* dY, float* W, float* dX, int batch, int IN, int OUT) {
    return guarded([&] {
        Tensor* dy = view(dY, batch, 1, OUT, 1);
        Tensor* w = view(W, 1, 1, OUT, IN);
        Tensor* dx = view(dX, batch, 1, IN, 1);
        linearXGrad(dy, w, dx);
        drop(dy); drop(w); drop(dx);
    });
}

int ref_linear_paramgrad(float* dY, float* X, float* dW, float* dB, int batch, int IN, int OUT) {
    return guarded([&] {
        Tensor* dy = view(dY, batch, 1, OUT, 1);
        Tensor* x = view(X, batch, 1, IN, 1);
        Tensor* dw = view(dW, 1, 1, OUT, IN);
        Tensor* db = view(dB, 1, 1, OUT, 1);
        linearParamGrad(dy, x, dw, db);
        drop(dy); drop(x); drop(dw); drop(db);
    });
}

// Batch size must not exceed 96 (seblas/operations/cuBatchNorm.cu:155).
int ref_batchnorm(float* X, float* beta, float* gamma, float* mean, float* var, float* Y, float* xhat, int N, int C,
                  int H, int W) {
    return guarded([&] {
        Tensor* x = view(X, N, C, H, W);
        Tensor* y = view(Y, N, C, H, W);
        Tensor* xh = view(xhat, N, C, H, W);
        Tensor* b = view(beta, 1, C, H, W);
        Tensor* g = view(gamma, 1, C, H, W);
        Tensor* m = view(mean, 1, C, H, W);
        Tensor* v = view(var, 1, C, H, W);
        batchNorm(x, b, g, m, v, y, xh);
        drop(x); drop(y); drop(xh); drop(b); drop(g); drop(m); drop(v);
    });
}

int ref_batchnorm_grad(float* dY, float* gamma, float* X, float* dX, int N, int C, int H, int W) {
    return guarded([&] {
        Tensor* dy = view(dY, N, C, H, W);
        Tensor* g = view(gamma, 1, C, H, W);
        Tensor* x = view(X, N, C, H, W);
        Tensor* dx = view(dX, N, C, H, W);
        batchNormGrad(dy, g, x, dx);
        drop(dy); drop(g); drop(x); drop(dx);
    });
}

int ref_batchnorm_paramgrads(float* dY, float* xhat, float* dGamma, float* dBeta, int N, int C, int H, int W) {
    return guarded([&] {
        Tensor* dy = view(dY, N, C, H, W);
        Tensor* xh = view(xhat, N, C, H, W);
        Tensor* dg = view(dGamma, 1, C, H, W);
        Tensor* db = view(dBeta, 1, C, H, W);
        batchNormParamGrads(dy, xh, dg, db);
        drop(dy); drop(xh); drop(dg); drop(db);
    });
}

int ref_relu(float* X, float* Y, int n) {
    return guarded([&] {
        Tensor* x = view(X, 1, 1, 1, n);
        Tensor* y = view(Y, 1, 1, 1, n);
        relu(x, y);
        drop(x); drop(y);
    });
}

int ref_relu_grad(float* X, float* dY, float* dX, int n) {
    return guarded([&] {
        Tensor* x = view(X, 1, 1, 1, n);
        Tensor* dy = view(dY, 1, 1, 1, n);
        Tensor* dx = view(dX, 1, 1, 1, n);
        reluGradFast(x, dy, dx);
        drop(x); drop(dy); drop(dx);
    });
}

int ref_avgpool(float* X, float* Y, int N, int C, int H, int W, int r) {
    return guarded([&] {
        Tensor* x = view(X, N, C, H, W);
        Tensor* y = view(Y, N, C, H / r, W / r);
        avgPool(x, y, r, r, r, r);
        drop(x); drop(y);
    });
}

int ref_avgpool_back(float* dX, float* dY, int N, int C, int H, int W, int r) {
    return guarded([&] {
        Tensor* dx = view(dX, N, C, H, W);
        Tensor* dy = view(dY, N, C, H / r, W / r);
        avgPoolBack(dx, dy, r, r, r, r);
        drop(dx); drop(dy);
    });
}

int ref_global_avgpool(float* X, float* Y, int N, int C, int H, int W) {
    return guarded([&] {
        Tensor* x = view(X, N, C, H, W);
        Tensor* y = view(Y, N, C, 1, 1);
        globalAvgPool(x, y, nullptr);  // H*W <= 1024: the single-block reduction needs no buffer
        drop(x); drop(y);
    });
}

int ref_global_avgpool_back(float* dX, float* dY, int N, int C, int H, int W) {
    return guarded([&] {
        Tensor* dx = view(dX, N, C, H, W);
        Tensor* dy = view(dY, N, C, 1, 1);
        globalAvgPoolBack(dx, dy);
        drop(dx); drop(dy);
    });
}

int ref_softmax(float* X, float* Y, int rows, int step) {
    return guarded([&] {
        Tensor* x = view(X, rows, 1, step, 1);
        Tensor* y = view(Y, rows, 1, step, 1);
        softmax(x, y, nullptr, step);
        cudaDeviceSynchronize();
        drop(x); drop(y);
    });
}

int ref_momentum(float* W, float* G, float* M, int n, float lr, float beta) {
    return guarded([&] {
        Tensor* w = view(W, 1, 1, 1, n);
        Tensor* g = view(G, 1, 1, 1, n);
        Tensor* m = view(M, 1, 1, 1, n);
        momentumApply(w, g, m, lr, beta);
        drop(w); drop(g); drop(m);
    });
}

int ref_scale(float* W, int n, float s) {
    return guarded([&] {
        Tensor* w = view(W, 1, 1, 1, n);
        *w * s;
        cudaDeviceSynchronize();
        drop(w);
    });
}

}  // extern "C"
