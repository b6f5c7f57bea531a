// Dense-layer entry points lowered onto the GEMM core. Shapes follow seblas::linear / linearXGrad /
// linearParamGrad (seblas/operations/cuLinear.cu:1052-1115): X is batch x IN, W is OUT x IN, Y is batch x OUT.
#include "cb_internal.h"

namespace cb {
namespace {

// db[m] += sum_n dY[n,m]: one warp per 32 columns, rows strided over the warps of a block, each term counted once
// (the reference kernel adds its partial from every thread column, seblas/operations/cuLinear.cu:1037-1040).
__global__ void __launch_bounds__(256) colsum_add_kernel(const float* __restrict__ dY, float* __restrict__ db,
                                                         int batch, int OUT) {
    __shared__ float part[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m = blockIdx.x * 32 + lane;
    float s = 0.f;
    if (m < OUT)
        for (int n = warp; n < batch; n += 8) s += dY[(long long)n * OUT + m];
    part[warp][lane] = s;
    __syncthreads();
    if (warp == 0 && m < OUT) {
        float v = 0.f;
        for (int w = 0; w < 8; ++w) v += part[w][lane];
        db[m] += v;
    }
}

int run_gemm(cb_ctx* ctx, const GemmCall& g) {
    if (ctx->math != CB_MATH_FP32 && umma_gemm_eligible(g)) return launch_umma_gemm(ctx, g, ctx->math == CB_MATH_3XTF32);
    return launch_simt_gemm(ctx, g);
}

}  // namespace
}  // namespace cb

using namespace cb;

extern "C" {

int cb_linear_fwd(cb_ctx* ctx, const float* X, const float* W, const float* b, float* Y, int batch, int IN, int OUT) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (batch < 0 || IN < 0 || OUT < 0) return fail(ctx, CB_EINVAL, "cb_linear_fwd: negative extent");
    if (batch == 0 || OUT == 0) return CB_OK;
    if (!X || !W || !Y) return fail(ctx, CB_EINVAL, "cb_linear_fwd: null operand");
    if (IN == 0) return fail(ctx, CB_EINVAL, "cb_linear_fwd: IN == 0");
    // D[i = out][j = sample] = sum_k W[i,k] X[j,k]; both operands have k contiguous; Y[j*OUT + i]
    GemmCall g;
    g.I = OUT; g.J = batch; g.K = IN;
    g.P = W; g.ldp = IN; g.p_mn = 0;
    g.Q = X; g.ldq = IN; g.q_mn = 0;
    g.C = Y; g.ldc = OUT; g.out_mode = 0;
    g.ep.bias_i = b;
    int rc = run_gemm(ctx, g);
    return rc == CB_OK ? finish(ctx, "cb_linear_fwd") : rc;
}

int cb_linear_xgrad(cb_ctx* ctx, const float* dY, const float* W, float* dX, int batch, int IN, int OUT) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (batch < 0 || IN < 0 || OUT < 0) return fail(ctx, CB_EINVAL, "cb_linear_xgrad: negative extent");
    if (batch == 0 || IN == 0) return CB_OK;
    if (!dY || !W || !dX) return fail(ctx, CB_EINVAL, "cb_linear_xgrad: null operand");
    if (OUT == 0) return fail(ctx, CB_EINVAL, "cb_linear_xgrad: OUT == 0");
    // D[i = in][j = sample] = sum_m W[m,i] dY[j,m]: W is read with i contiguous (MN-major), dY with m contiguous
    GemmCall g;
    g.I = IN; g.J = batch; g.K = OUT;
    g.P = W; g.ldp = IN; g.p_mn = 1;
    g.Q = dY; g.ldq = OUT; g.q_mn = 0;
    g.C = dX; g.ldc = IN; g.out_mode = 0;
    int rc = run_gemm(ctx, g);
    return rc == CB_OK ? finish(ctx, "cb_linear_xgrad") : rc;
}

int cb_linear_paramgrad(cb_ctx* ctx, const float* dY, const float* X, float* dW, float* db, int batch, int IN,
                        int OUT) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (batch < 0 || IN < 0 || OUT < 0) return fail(ctx, CB_EINVAL, "cb_linear_paramgrad: negative extent");
    if (OUT == 0 || batch == 0) return CB_OK;
    if (!dY || !X || !dW) return fail(ctx, CB_EINVAL, "cb_linear_paramgrad: null operand");
    if (IN > 0) {
        // D[i = in][j = out] += sum_n X[n,i] dY[n,j]: both operands are read with the output index contiguous
        GemmCall g;
        g.I = IN; g.J = OUT; g.K = batch;
        g.P = X; g.ldp = IN; g.p_mn = 1;
        g.Q = dY; g.ldq = OUT; g.q_mn = 1;
        g.C = dW; g.ldc = IN; g.out_mode = 0;
        g.accumulate = 1;
        int rc = run_gemm(ctx, g);
        if (rc != CB_OK) return rc;
    }
    if (db) {
        colsum_add_kernel<<<(OUT + 31) / 32, 256, 0, ctx->stream>>>(dY, db, batch, OUT);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return check_cuda(ctx, e, "cb_linear_paramgrad: bias gradient");
        ctx->launches += 1;
    }
    return finish(ctx, "cb_linear_paramgrad");
}

}  // extern "C"
