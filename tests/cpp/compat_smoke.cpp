// Exercises the header shim the way the reference's hand-run validation does (validation/UnitTestTools.cu:130-170
// compares linearParamGrad with sgemmNTA on the same data): the seblas-named calls must agree with each other and
// with a host loop. Exit code 0 = pass.
#include <cmath>
#include <cstdio>
#include <vector>

#include "seblas/operations/cuOperations.cuh"

using namespace seblas;

static float lcg(unsigned& s) { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xFFFF) / 32768.0f - 1.0f; }

int main() {
    unsigned seed = 1;
    const int batch = 16, IN = 64, OUT = 24;
    std::vector<float> hX(batch * IN), hdY(batch * OUT), hW(OUT * IN);
    for (auto& v : hX) v = lcg(seed);
    for (auto& v : hdY) v = lcg(seed);
    for (auto& v : hW) v = lcg(seed);
    Tensor* X = Tensor::declare(batch, 1, IN, 1)->ripOffHost(hX.data());
    Tensor* dY = Tensor::declare(batch, 1, OUT, 1)->ripOffHost(hdY.data());
    Tensor* dW = Tensor::create(OUT, IN);
    Tensor* dB = Tensor::create(OUT, 1);
    linearParamGrad(dY, X, dW, dB);
    // same contraction through sgemmTN: dW = dY^T (batch x OUT stored K x M) * X (batch x IN)
    Tensor* dW2 = Tensor::create(OUT, IN);
    sgemmTN(dY->reshape(shape4(batch, OUT)), X->reshape(shape4(batch, IN)), dW2);
    std::vector<float> a(OUT * IN), b(OUT * IN);
    cudaMemcpy(a.data(), dW->elements, a.size() * 4, cudaMemcpyDeviceToHost);
    cudaMemcpy(b.data(), dW2->elements, b.size() * 4, cudaMemcpyDeviceToHost);
    double worst = 0;
    for (int m = 0; m < OUT; ++m)
        for (int k = 0; k < IN; ++k) {
            double ref = 0;
            for (int n = 0; n < batch; ++n) ref += (double)hdY[n * OUT + m] * hX[n * IN + k];
            worst = std::fmax(worst, std::fabs(a[m * IN + k] - ref));
            worst = std::fmax(worst, std::fabs(b[m * IN + k] - ref));
        }
    printf("linearParamGrad / sgemmTN vs host loop: max abs err %.3g\n", worst);
    if (worst > 1e-3) return 1;  // the reference's own tolerance for this test (UnitTestTools.cu:152)
    // a bad convolution shape must throw std::invalid_argument like assertConv
    bool threw = false;
    try {
        Tensor* f = Tensor::create(4, 3, 3, 3); Tensor* x = Tensor::create(1, 3, 8, 8); Tensor* y = Tensor::create(1, 4, 7, 7);
        conv(f, x, y, 1, 1, 1, 1, nullptr);
    } catch (const std::invalid_argument&) { threw = true; }
    if (!threw) { printf("assertConv did not throw\n"); return 2; }
    // in-place tensor arithmetic and constFill
    Tensor* t = Tensor::create(1000, 1)->constFill(2.0f);
    *t * 3.0f;
    *t + t;
    if (std::fabs(t->get(999) - 12.0f) > 1e-6) { printf("tensor arithmetic wrong: %f\n", t->get(999)); return 3; }
    printf("compat smoke ok\n");
    return 0;
}
