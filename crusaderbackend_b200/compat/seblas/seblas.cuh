// Header shim with the reference's seblas interface, written fresh on top of the crusader_b200 C ABI.
//
// It mirrors, for the dense-contraction path and its neighbours, the names, argument order, return values and
// error behaviour of
//   seblas/tensor/Tensor.cuh:48-208, seblas/tensor/Parameter.cuh:11-77,
//   seblas/operations/cuGEMM.cuh:12-21, cuConv.cuh:20-42, cuLinear.cuh:14-18, cuBatchNorm.cuh:12-16,
//   cuPool.cuh:13-27 (average / global average), cuActivation.cuh:13-18 (ReLU), cuReduce.cuh:44 (softmax),
//   cuLoss.cuh:18-20 (cross entropy), cuOptim.cuh:12-25 (SGD / Momentum), seblas/assist/CudaAssert.cuh,
// so that operand code written against those headers compiles against this one and runs on the sm_100a kernels.
// Every operation returns after the device finished it (the reference ends each op with cudaDeviceSynchronize),
// shape errors throw std::invalid_argument, device errors throw std::runtime_error.
// The functions the operands never reach on this path (dropout, YOLO loss, AdaGrad / AdaDelta / Adam, max-pool, leaky
// ReLU and the other activations) are declared with the reference's signatures, so that the whole of seann compiles,
// and throw std::runtime_error when called. Random fills draw from a seeded host generator (the reference seeds from
// the clock); cuDNN is not used: cudnnHandle_t is an opaque stand-in so that seann/operands/OperandBase.cuh compiles.
#pragma once
#include <cuda_runtime.h>

#include <cassert>
#include <cmath>
#include <cstdio>
#include <fstream>
#include <iostream>
#include <random>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "../../../include/crusader_b200.h"
#include "../seio/logging/LogUtils.cuh"

// seblas/tensor/Tensor.cuh:24 leaks `using namespace std` into every file that includes it, and the operand sources
// rely on it (string, fstream, to_string without qualification).
using namespace std;

// Stand-in for the one cuDNN name the operand base class touches (seann/operands/OperandBase.cuh:13,27-31).
#if !defined(CUDNN_H_) && !defined(CUDNN_VERSION)
struct cbCudnnStandIn;
typedef cbCudnnStandIn* cudnnHandle_t;
inline int cudnnCreate(cudnnHandle_t* h) {
    static char token;
    *h = reinterpret_cast<cudnnHandle_t>(&token);
    return 0;
}
#endif

#define CPU_THREADS 20

// seblas/assist/CudaAssert.cuh:10 and seblas/tensor/Tensor.cuh:26 open these namespaces at global scope as well.
namespace seutil {}
using namespace seutil;
using namespace seio;

namespace seblas {

typedef unsigned int uint32;
typedef unsigned long long uint64;
const uint32 WARP_SIZE = 32;
const uint32 REDUCE_BLOCK = 1024;
const uint32 REDUCE_WARPS = 32;
const dim3 CUDA_BLOCK_SIZE = {16, 16};
const dim3 CUDA_BLOCK_SIZE_3D = {16, 16, 4};

[[noreturn]] inline void offPath(const char* what) {
    throw std::runtime_error(std::string(what) + " is outside the dense-contraction path this library replaces");
}

struct index4 {
    uint32 n = 0, c = 0, h = 0, w = 0;
    index4(uint32 n, uint32 c, uint32 h, uint32 w) : n(n), c(c), h(h), w(w) {}
    index4(uint32 c, uint32 h, uint32 w) : c(c), h(h), w(w) {}
    index4(uint32 h, uint32 w) : h(h), w(w) {}
    index4 operator+(index4 o) const { return {n + o.n, c + o.c, h + o.h, w + o.w}; }
    index4 operator-(index4 o) const { return {n - o.n, c - o.c, h - o.h, w - o.w}; }
    bool operator==(index4 o) const { return n == o.n && c == o.c && h == o.h && w == o.w; }
    bool operator>(index4 o) const { return n > o.n && c > o.c && h > o.h && w > o.w; }
    bool operator<(index4 o) const { return n < o.n && c < o.c && h < o.h && w < o.w; }
    // same value as seblas/tensor/Tensor.cu:345-347 (the conditional chain parses right to left)
    uint32 getOffset() const { return n == 0 ? 1 : n * c == 0 ? 1 : c * h == 0 ? 1 : h * w; }
    std::string toString() const {
        return "(" + std::to_string(n) + "," + std::to_string(c) + "," + std::to_string(h) + "," + std::to_string(w) + ")";
    }
};

struct shape4 : public index4 {
    uint32 size;
    shape4(uint32 n, uint32 c, uint32 h, uint32 w) : index4(n, c, h, w) { size = n * c * h * w; }
    shape4(uint32 c, uint32 h, uint32 w) : index4(1, c, h, w) { size = c * h * w; }
    shape4(uint32 h, uint32 w) : index4(1, 1, h, w) { size = h * w; }
};

// ---- library context shared by every operation (the reference's only global is its cudnn handle)
inline cb_ctx*& context_slot() {
    static cb_ctx* ctx = nullptr;
    return ctx;
}
inline cb_ctx* context() {
    cb_ctx*& ctx = context_slot();
    if (!ctx) {
        if (cb_create(&ctx, 0, nullptr) != CB_OK) throw std::runtime_error("crusader_b200: cb_create failed (no B200?)");
        cb_set_sync(ctx, 1);
        cb_set_math(ctx, CB_MATH_3XTF32);
    }
    return ctx;
}
inline void setMathMode(int cb_math_mode) { cb_set_math(context(), cb_math_mode); }
inline void check(int rc, const char* file, int line) {
    if (rc == CB_OK) return;
    const std::string msg = std::string(cb_last_error(context())) + "  line: " + std::to_string(line) + "  file: " + file;
    if (rc == CB_EINVAL) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}
#define SEBLAS_CB(call) ::seblas::check((call), __FILE__, __LINE__)

inline void assertCuda(const char* file, int line) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        throw std::runtime_error(std::string("Device error encountered: ") + cudaGetErrorString(e) + "  line: " +
                                 std::to_string(line) + "  file: " + file);
}

// Seed of the host generator behind Tensor::randNormal / randUniform; every fill advances it, so a fixed seed gives a
// reproducible initialisation of a whole model.
inline std::mt19937_64& randEngine() {
    static std::mt19937_64 e(0x5eb1a5ull);
    return e;
}
inline void setRandSeed(uint64 seed) { randEngine().seed(seed); }

class Tensor {
public:
    shape4 dims;
    float* elements = nullptr;
    int deviceId = 0;  // -1 host, otherwise GPU

    static Tensor* declare(shape4 dims) {
        Tensor* t = static_cast<Tensor*>(::operator new(sizeof(Tensor)));
        new (t) Tensor(dims);
        return t;
    }
    template <typename... Args> static Tensor* declare(Args&&... a) { return declare(shape4(std::forward<Args>(a)...)); }
    static Tensor* create(shape4 dims) { return declare(dims)->instantiate(); }
    template <typename... Args> static Tensor* create(Args&&... a) { return create(shape4(std::forward<Args>(a)...)); }
    static Tensor* createHost(shape4 dims) { return declare(dims)->instantiateHost(); }
    template <typename... Args> static Tensor* createHost(Args... a) { return createHost(shape4(a...)); }

    Tensor* reshape(shape4 d) { assert(d.size == dims.size); dims = d; return this; }
    template <typename... Args> Tensor* reshape(Args&&... a) { return reshape(shape4(std::forward<Args>(a)...)); }
    Tensor* instantiate() {
        cudaMalloc(&elements, sizeof(float) * dims.size);
        assertCuda(__FILE__, __LINE__);
        cudaMemset(elements, 0, sizeof(float) * dims.size);
        deviceId = 0;
        return this;
    }
    Tensor* instantiateHost() { cudaMallocHost(&elements, sizeof(float) * dims.size); deviceId = -1; return this; }
    Tensor* destroy() { cudaFree(elements); return this; }
    Tensor* destroyHost() { cudaFreeHost(elements); return this; }
    void eliminate() { destroy(); ::operator delete(this); }
    void eliminateHost() { destroyHost(); ::operator delete(this); }
    Tensor* attach(Tensor* o) { assert(dims.size <= o->dims.size); elements = o->elements; deviceId = o->deviceId; return this; }
    Tensor* attach(float* e, int dev) { elements = e; deviceId = dev; return this; }
    Tensor* copyToH2D(Tensor* d) const { cudaMemcpy(d->elements, elements, sizeof(float) * dims.size, cudaMemcpyHostToDevice); return d; }
    Tensor* copyToD2H(Tensor* h) const { cudaMemcpy(h->elements, elements, sizeof(float) * dims.size, cudaMemcpyDeviceToHost); return h; }
    Tensor* copyToD2D(Tensor* d) const { cudaMemcpy(d->elements, elements, sizeof(float) * dims.size, cudaMemcpyDeviceToDevice); return d; }
    Tensor* copyToH2H(Tensor* h) const { cudaMemcpy(h->elements, elements, sizeof(float) * dims.size, cudaMemcpyHostToHost); return h; }
    Tensor* toDevice() {
        float* h = elements;
        instantiate();
        cudaMemcpy(elements, h, sizeof(float) * dims.size, cudaMemcpyHostToDevice);
        cudaFreeHost(h);
        return this;
    }
    Tensor* toHost() {
        float* d = elements;
        instantiateHost();
        cudaMemcpy(elements, d, sizeof(float) * dims.size, cudaMemcpyDeviceToHost);
        cudaFree(d);
        return this;
    }
    Tensor* ripOffDevice() const { Tensor* h = createHost(dims); copyToD2H(h); return h; }
    Tensor* ripOffHost() const { Tensor* d = create(dims); copyToH2D(d); return d; }
    Tensor* ripOffHost(float* src) { Tensor* d = create(dims); cudaMemcpy(d->elements, src, sizeof(float) * dims.size, cudaMemcpyHostToDevice); return d; }
    // in-place arithmetic (GPU tensors): seblas/tensor/Tensor.cu:462-660
    Tensor* operator+(Tensor* o) { assert(dims.size == o->dims.size); SEBLAS_CB(cb_tensor_op(context(), CB_OP_ADD, elements, o->elements, 0.f, dims.size)); return this; }
    Tensor* operator-(Tensor* o) { assert(dims.size == o->dims.size); SEBLAS_CB(cb_tensor_op(context(), CB_OP_SUB, elements, o->elements, 0.f, dims.size)); return this; }
    Tensor* operator*(Tensor* o) { assert(dims.size == o->dims.size); SEBLAS_CB(cb_tensor_op(context(), CB_OP_MUL, elements, o->elements, 0.f, dims.size)); return this; }
    Tensor* operator/(Tensor* o) { assert(dims.size == o->dims.size); SEBLAS_CB(cb_tensor_op(context(), CB_OP_DIV, elements, o->elements, 0.f, dims.size)); return this; }
    Tensor* operator+(float s) { SEBLAS_CB(cb_tensor_op(context(), CB_OP_ADD_SCALAR, elements, nullptr, s, dims.size)); return this; }
    Tensor* operator-(float s) { SEBLAS_CB(cb_tensor_op(context(), CB_OP_SUB_SCALAR, elements, nullptr, s, dims.size)); return this; }
    Tensor* operator*(float s) { SEBLAS_CB(cb_tensor_op(context(), CB_OP_MUL_SCALAR, elements, nullptr, s, dims.size)); return this; }
    Tensor* operator/(float s) { SEBLAS_CB(cb_tensor_op(context(), CB_OP_DIV_SCALAR, elements, nullptr, s, dims.size)); return this; }
    Tensor* constFill(float v) { SEBLAS_CB(cb_tensor_op(context(), CB_OP_FILL, elements, nullptr, v, dims.size)); return this; }
    // Random fills: seeded host draws copied to the device (seblas/tensor/Tensor.cu:659-686 seeds curand from the clock).
    Tensor* randUniform(float lo, float hi) {
        std::uniform_real_distribution<float> d(lo, hi);
        return fillFromHost([&] { return d(randEngine()); });
    }
    Tensor* randNormal(float mean, float stddev) {
        std::normal_distribution<float> d(mean, stddev);
        return fillFromHost([&] { return d(randEngine()); });
    }
    float get(uint32 offset) const { float v; cudaMemcpy(&v, elements + offset, sizeof(float), deviceId == -1 ? cudaMemcpyHostToHost : cudaMemcpyDeviceToHost); return v; }

private:
    explicit Tensor(shape4 d) : dims(d) {}
    template <typename F> Tensor* fillFromHost(F draw) {
        if (deviceId == -1) {
            for (uint32 i = 0; i < dims.size; ++i) elements[i] = draw();
            return this;
        }
        std::vector<float> h(dims.size);
        for (float& v : h) v = draw();
        cudaMemcpy(elements, h.data(), sizeof(float) * dims.size, cudaMemcpyHostToDevice);
        assertCuda(__FILE__, __LINE__);
        return this;
    }
};

class Parameter {
public:
    Tensor* A;
    Tensor* dA;
    Tensor* dAReserve;
    static Parameter* create(shape4 dims) {
        Parameter* p = new Parameter();
        p->A = Tensor::create(dims); p->dA = Tensor::create(dims); p->dAReserve = Tensor::create(dims);
        return p;
    }
    template <typename... Args> static Parameter* create(Args&&... a) { return create(shape4(std::forward<Args>(a)...)); }
    static Parameter* create(Tensor* src) {
        Parameter* p = new Parameter();
        p->A = src; p->dA = Tensor::create(src->dims); p->dAReserve = Tensor::create(src->dims);
        return p;
    }
    static Parameter* declare(shape4 dims) {
        Parameter* p = new Parameter();
        p->A = Tensor::declare(dims); p->dA = Tensor::declare(dims); p->dAReserve = Tensor::declare(dims);
        return p;
    }
    template <typename... Args> static Parameter* declare(Args&&... a) { return declare(shape4(std::forward<Args>(a)...)); }
    Parameter* instantiate() { A->instantiate(); dA->instantiate(); dAReserve->instantiate(); return this; }
    Parameter* inherit(Parameter* s) { assert(s->A->dims.size == A->dims.size); A->attach(s->A); dA->attach(s->dA); dAReserve->attach(s->dAReserve); return this; }
    void eliminate() const { A->eliminate(); dA->eliminate(); dAReserve->eliminate(); }
};

// ------------------------------------------------------------------ cuGEMM.cuh
inline Tensor* sgemm(Tensor* A, Tensor* B, Tensor* C) {  // C[b] = A * B[b] over B->dims.n
    assert(A->dims.w == B->dims.h && A->dims.h == C->dims.h && B->dims.w == C->dims.w);
    const int M = A->dims.h, K = A->dims.w, N = B->dims.w;
    SEBLAS_CB(cb_gemm(context(), 0, 0, M, N, K, A->elements, K, B->elements, N, C->elements, N, (int)B->dims.n, 0,
                      (long long)K * N, (long long)M * N, 0));
    return C;
}
inline Tensor* sgemmTN(Tensor* A, Tensor* B, Tensor* C) {  // A stored K x M
    assert(A->dims.h == B->dims.h && A->dims.w == C->dims.h && B->dims.w == C->dims.w);
    const int K = A->dims.h, M = A->dims.w, N = B->dims.w;
    SEBLAS_CB(cb_gemm(context(), 1, 0, M, N, K, A->elements, M, B->elements, N, C->elements, N, (int)B->dims.n, 0,
                      (long long)K * N, (long long)M * N, 0));
    return C;
}
inline Tensor* sgemmNT(Tensor* A, Tensor* B, Tensor* C) {  // B stored N x K
    assert(A->dims.w == B->dims.w && A->dims.h == C->dims.h && B->dims.h == C->dims.w);
    const int M = A->dims.h, K = A->dims.w, N = B->dims.h;
    SEBLAS_CB(cb_gemm(context(), 0, 1, M, N, K, A->elements, K, B->elements, K, C->elements, N, 1, 0, 0, 0, 0));
    return C;
}
inline Tensor* sgemmNTA(Tensor* A, Tensor* B, Tensor* C) {  // C += sum over A->dims.n of A[n] * B[n]^T
    assert(A->dims.w == B->dims.w && A->dims.h == C->dims.h && B->dims.h == C->dims.w);
    const int M = A->dims.h, K = A->dims.w, N = B->dims.h;
    SEBLAS_CB(cb_gemm_batch_reduce(context(), 0, 1, M, N, K, A->elements, K, B->elements, K, C->elements, N, (int)A->dims.n,
                                   (long long)M * K, (long long)N * K, 1));
    return C;
}

// ------------------------------------------------------------------ cuConv.cuh
inline void assertConv(Tensor* filters, Tensor* features, Tensor* out, uint32 sH, uint32 sW, uint32 pH, uint32 pW) {
    if (out->dims.h != (features->dims.h - filters->dims.h + 2 * pH) / sH + 1)
        throw std::invalid_argument("assertConv: rows (h) relationship did not satisfy");
    if (out->dims.w != (features->dims.w - filters->dims.w + 2 * pW) / sW + 1)
        throw std::invalid_argument("assertConv: cols (w) relationship did not satisfy");
    if (out->dims.c != filters->dims.n || features->dims.c != filters->dims.c)
        throw std::invalid_argument("assertConv: channels relationship did not satisfy");
    if (out->dims.n != features->dims.n) throw std::invalid_argument("assertConv: batch relationship did not satisfy");
}
inline Tensor* conv(Tensor* A, Tensor* B, Tensor* C, int sH, int sW, int pH, int pW, Tensor* biases) {
    assertConv(A, B, C, sH, sW, pH, pW);
    SEBLAS_CB(cb_conv_fwd(context(), A->elements, B->elements, C->elements, biases ? biases->elements : nullptr, B->dims.n,
                          B->dims.c, B->dims.h, B->dims.w, A->dims.n, A->dims.h, A->dims.w, sH, sW, pH, pW, 0));
    return C;
}
inline Tensor* convDerive(Tensor* A, Tensor* B, Tensor* C, int sH, int sW, int pH, int pW) {
    assertConv(A, C, B, sH, sW, pH, pW);
    SEBLAS_CB(cb_conv_dgrad(context(), A->elements, B->elements, C->elements, C->dims.n, C->dims.c, C->dims.h, C->dims.w,
                            A->dims.n, A->dims.h, A->dims.w, sH, sW, pH, pW));
    return C;
}
inline Tensor* convError(Tensor* A, Tensor* B, Tensor* C, int sH, int sW, int pH, int pW) {
    assertConv(C, B, A, sH, sW, pH, pW);
    SEBLAS_CB(cb_conv_wgrad(context(), A->elements, B->elements, C->elements, B->dims.n, B->dims.c, B->dims.h, B->dims.w,
                            C->dims.n, C->dims.h, C->dims.w, sH, sW, pH, pW, 1));
    return A;  // the reference returns its first argument (seblas/operations/cuConv.cu:805)
}
inline Tensor* convBias(Tensor* Y, Tensor* biases) {
    assert(biases->dims.size == Y->dims.c);
    SEBLAS_CB(cb_conv_bias(context(), Y->elements, biases->elements, Y->dims.n, Y->dims.c, Y->dims.h * Y->dims.w));
    return Y;
}

// ------------------------------------------------------------------ cuLinear.cuh
inline Tensor* linear(Tensor* X, Tensor* W, Tensor* B, Tensor* Y) {
    assert(W->dims.w == X->dims.h && B->dims.h == Y->dims.h && X->dims.n == Y->dims.n);
    SEBLAS_CB(cb_linear_fwd(context(), X->elements, W->elements, B->elements, Y->elements, X->dims.n, W->dims.w, W->dims.h));
    return Y;
}
inline Tensor* linearXGrad(Tensor* dY, Tensor* W, Tensor* dX) {
    assert(W->dims.h == dY->dims.h && dX->dims.n == dY->dims.n && W->dims.w == dX->dims.h);
    SEBLAS_CB(cb_linear_xgrad(context(), dY->elements, W->elements, dX->elements, dX->dims.n, W->dims.w, W->dims.h));
    return dX;
}
inline Tensor* linearParamGrad(Tensor* dY, Tensor* X, Tensor* dW, Tensor* dB) {
    assert(X->dims.h == dW->dims.w && dY->dims.h == dW->dims.h && X->dims.n == dY->dims.n);
    SEBLAS_CB(cb_linear_paramgrad(context(), dY->elements, X->elements, dW->elements, dB ? dB->elements : nullptr,
                                  X->dims.n, dW->dims.w, dW->dims.h));
    return dW;
}

// ------------------------------------------------------------------ cuBatchNorm.cuh (any batch size)
inline Tensor* batchNorm(Tensor* X, Tensor* beta, Tensor* gamma, Tensor* mean, Tensor* var, Tensor* Y, Tensor* xHat) {
    assert(X->dims.n == Y->dims.n && X->dims.size == Y->dims.size);
    SEBLAS_CB(cb_bn_fwd(context(), X->elements, beta->elements, gamma->elements, mean ? mean->elements : nullptr,
                        var ? var->elements : nullptr, Y->elements, xHat ? xHat->elements : nullptr, X->dims.n,
                        X->dims.size / X->dims.n));
    return Y;
}
inline Tensor* batchNormGrad(Tensor* dY, Tensor* gamma, Tensor* X, Tensor* dX) {
    assert(dY->dims.n == X->dims.n && dY->dims.size == X->dims.size);
    SEBLAS_CB(cb_bn_bwd(context(), dY->elements, gamma->elements, X->elements, dX->elements, X->dims.n, X->dims.size / X->dims.n));
    return dX;
}
inline void batchNormParamGrads(Tensor* dY, Tensor* xHat, Tensor* dGamma, Tensor* dBeta) {
    assert(dY->dims.n == xHat->dims.n && dY->dims.size == xHat->dims.size);
    SEBLAS_CB(cb_bn_paramgrad(context(), dY->elements, xHat->elements, dGamma->elements, dBeta->elements, dY->dims.n,
                              dY->dims.size / dY->dims.n));
}

// ------------------------------------------------------------------ cuActivation.cuh / cuPool.cuh / cuReduce.cuh / cuLoss.cuh
inline Tensor* relu(Tensor* X, Tensor* Y) { SEBLAS_CB(cb_relu(context(), X->elements, Y->elements, X->dims.size)); return Y; }
inline Tensor* reluGradFast(Tensor* X, Tensor* dY, Tensor* dX) {
    SEBLAS_CB(cb_relu_grad(context(), X->elements, dY->elements, dX->elements, X->dims.size));
    return dX;
}
inline void avgPool(Tensor* X, Tensor* Y, uint32 sH, uint32 sW, uint32 rH, uint32 rW) {
    assert(sH == rH && sW == rW);  // the reference kernels index as if window == stride (seblas/operations/cuPool.cu:27-28)
    SEBLAS_CB(cb_avgpool(context(), X->elements, Y->elements, (long long)X->dims.n * X->dims.c, X->dims.h, X->dims.w, rH, rW));
}
inline void avgPoolBack(Tensor* dX, Tensor* dY, uint32 sH, uint32 sW, uint32 rH, uint32 rW) {
    assert(sH == rH && sW == rW);
    SEBLAS_CB(cb_avgpool_back(context(), dX->elements, dY->elements, (long long)dX->dims.n * dX->dims.c, dX->dims.h, dX->dims.w, rH, rW));
}
inline void globalAvgPool(Tensor* X, Tensor* Y, Tensor* /*buffer*/) {
    SEBLAS_CB(cb_global_avgpool(context(), X->elements, Y->elements, (long long)X->dims.n * X->dims.c, X->dims.h * X->dims.w));
}
inline void globalAvgPoolBack(Tensor* dX, Tensor* dY) {
    SEBLAS_CB(cb_global_avgpool_back(context(), dX->elements, dY->elements, (long long)dX->dims.n * dX->dims.c, dX->dims.h * dX->dims.w));
}
inline Tensor* softmax(Tensor* A, Tensor* out, Tensor* /*buffer*/, uint32 step) {
    assert(A->dims.size % step == 0 && out->dims.size == A->dims.size);
    SEBLAS_CB(cb_softmax(context(), A->elements, out->elements, A->dims.size / step, step));
    return out;
}
inline void crossEntropyLoss(Parameter* Y, Tensor* labels) {  // Y->dA = Y->A - labels
    SEBLAS_CB(cb_cross_entropy(context(), Y->A->elements, labels->elements, Y->dA->elements, nullptr, Y->A->dims.size));
}
inline float crossEntropyCalc(Parameter* Y, Tensor* labels, Tensor* buf) {  // sum(-log(y + 1e-10) * label)
    assert(buf && buf->dims.size >= 1);
    SEBLAS_CB(cb_cross_entropy(context(), Y->A->elements, labels->elements, nullptr, buf->elements, Y->A->dims.size));
    return buf->get(0);
}
typedef void (*LossFunc)(Parameter*, Tensor*);
typedef float (*LossFuncCalc)(Parameter*, Tensor*, Tensor* buf);

// ------------------------------------------------------------------ cuOptim.cuh
inline void SGDApply(Tensor* X, Tensor* Xgrad, float lr) {  // x -= lr * g; g = 0: Momentum with beta = 0 and a throw-away buffer
    Tensor* m = Tensor::create(X->dims);
    SEBLAS_CB(cb_momentum(context(), X->elements, Xgrad->elements, m->elements, X->dims.size, lr, 0.f, 0.f, 0));
    m->eliminate();
}
inline void momentumApply(Tensor* X, Tensor* Xgrad, Tensor* V, float lr, float beta) {
    SEBLAS_CB(cb_momentum(context(), X->elements, Xgrad->elements, V->elements, X->dims.size, lr, beta, 0.f, 0));
}


inline void adaGradApply(Tensor*, Tensor*, Tensor*, float, float) { offPath("adaGradApply"); }
inline void adaDeltaApply(Tensor*, Tensor*, Tensor*, Tensor*, float, float) { offPath("adaDeltaApply"); }
inline void adamApply(Tensor*, Tensor*, Tensor*, Tensor*, float, float, float, float, float) { offPath("adamApply"); }

// ------------------------------------------------------------------ cuReduce.cuh (sums; the softmax is above)
// out[r] = sum of the r-th run of `step` consecutive elements of A (seblas/operations/cuReduce.cu:235-272); the
// buffer the reference needs for runs above 1024 elements is accepted and left untouched.
inline Tensor* reduce(Tensor* A, Tensor* out, Tensor* /*buffer*/, uint32 step) {
    assert(A->dims.size % step == 0 && out->dims.size == A->dims.size / step);
    SEBLAS_CB(cb_conv_bias_grad(context(), A->elements, out->elements, 1, (int)(A->dims.size / step), (int)step, 0));
    return out;
}
inline float reduce(Tensor* A, Tensor* buffer) {
    Tensor* t = Tensor::create(shape4(1, 1));
    reduce(A, t, buffer, A->dims.size);
    const float v = t->get(0);
    t->eliminate();
    return v;
}
inline Tensor* rowReduce(Tensor* A, Tensor* out, Tensor* buffer) { return reduce(A, out, buffer, A->dims.w); }
inline Tensor* channelReduce(Tensor* A, Tensor* out, Tensor* buffer) { return reduce(A, out, buffer, A->dims.h * A->dims.w); }
inline Tensor* colReduce(Tensor*, Tensor*, Tensor*) { offPath("colReduce"); }
inline Tensor* rowSoftmax(Tensor* A, Tensor* out, Tensor* buffer) { return softmax(A, out, buffer, A->dims.w); }
inline Tensor* colSoftmax(Tensor*, Tensor*, Tensor*) { offPath("colSoftmax"); }

// ------------------------------------------------------------------ cuConcat.cuh
// Y = [Xs[0] ; Xs[1] ; ...] along the channel axis, and its gradient, which ADDS each slice of Y->dA into the
// matching Xs[i]->dAReserve (seblas/operations/cuConcat.cu:9-83).
inline Parameter* concat(Parameter** Xs, uint32 paramCount, Parameter* Y) {
    std::vector<const float*> src(paramCount);
    std::vector<int> ch(paramCount);
    uint32 c = 0;
    for (uint32 i = 0; i < paramCount; ++i) {
        assert(Xs[i]->A->dims.n == Y->A->dims.n && Xs[i]->A->dims.h == Y->A->dims.h && Xs[i]->A->dims.w == Y->A->dims.w);
        src[i] = Xs[i]->A->elements;
        ch[i] = (int)Xs[i]->A->dims.c;
        c += Xs[i]->A->dims.c;
    }
    assert(c == Y->A->dims.c);
    SEBLAS_CB(cb_concat_channels(context(), (int)paramCount, src.data(), ch.data(), Y->A->elements, (int)Y->A->dims.n,
                                 (int)(Y->A->dims.h * Y->A->dims.w)));
    return Y;
}
inline void concatGrads(Parameter* Y, Parameter** Xs, uint32 paramCount) {
    std::vector<float*> dst(paramCount);
    std::vector<int> ch(paramCount);
    for (uint32 i = 0; i < paramCount; ++i) {
        dst[i] = Xs[i]->dAReserve->elements;
        ch[i] = (int)Xs[i]->A->dims.c;
    }
    SEBLAS_CB(cb_concat_grads(context(), (int)paramCount, dst.data(), ch.data(), Y->dA->elements, (int)Y->A->dims.n,
                              (int)(Y->A->dims.h * Y->A->dims.w)));
}

// ------------------------------------------------------------------ declared for completeness, not on the path
inline Tensor* dropout(Tensor*, Tensor*, Tensor*, float) { offPath("dropout"); }
inline Tensor* dropoutGrad(Tensor*, Tensor*, Tensor*, float) { offPath("dropoutGrad"); }
inline Tensor* dropoutInfer(Tensor*, Tensor*, float) { offPath("dropoutInfer"); }
inline void maxPool(Tensor*, Tensor*, Tensor*, uint32, uint32, uint32, uint32) { offPath("maxPool"); }
inline void maxPoolBack(Tensor*, Tensor*, Tensor*, uint32, uint32, uint32, uint32) { offPath("maxPoolBack"); }
inline Tensor* reluGrad(Tensor*, Tensor*) { offPath("reluGrad"); }
inline Tensor* lRelu(Tensor*, Tensor*, float) { offPath("lRelu"); }
inline Tensor* lReluGrad(Tensor*, Tensor*, float) { offPath("lReluGrad"); }
inline Tensor* lReluGradFast(Tensor*, Tensor*, Tensor*, float) { offPath("lReluGradFast"); }
inline Tensor* elu(Tensor*, Tensor*, float) { offPath("elu"); }
inline Tensor* eluGrad(Tensor*, Tensor*, float) { offPath("eluGrad"); }
inline Tensor* sigmoid(Tensor*, Tensor*) { offPath("sigmoid"); }
inline Tensor* sigmoidGrad(Tensor*, Tensor*) { offPath("sigmoidGrad"); }
inline Tensor* tanh(Tensor*, Tensor*) { offPath("tanh"); }
inline Tensor* tanhGrad(Tensor*, Tensor*) { offPath("tanhGrad"); }
inline void Yolo1CompositeLoss(Parameter*, Tensor*) { offPath("Yolo1CompositeLoss"); }
inline float Yolo1CompositeCalc(Parameter*, Tensor*, Tensor*) { offPath("Yolo1CompositeCalc"); }

// ------------------------------------------------------------------ assist/Inspections.cuh
inline void inspect(Tensor* t) {
    std::vector<float> h(t->dims.size);
    cudaMemcpy(h.data(), t->elements, sizeof(float) * t->dims.size,
               t->deviceId == -1 ? cudaMemcpyHostToHost : cudaMemcpyDeviceToHost);
    size_t i = 0;
    for (uint32 n = 0; n < t->dims.n; ++n, printf("\n"))
        for (uint32 c = 0; c < t->dims.c; ++c, printf("\n"))
            for (uint32 y = 0; y < t->dims.h; ++y, printf("\n"))
                for (uint32 x = 0; x < t->dims.w; ++x) printf("%f, ", h[i++]);
}

}  // namespace seblas
