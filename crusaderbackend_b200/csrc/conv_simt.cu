// CUDA-core fp32 convolution kernels (any filter size, stride and padding) and the cb_conv_* dispatchers.
// These serve CB_MATH_FP32 and every geometry the tensor-core implicit-GEMM kernels do not cover; they compute
// exact fp32 FMAs. Index maps follow seblas/operations/cuConv.cu:105-115 (forward) and the adjoint of it for the
// two gradients (the reference's weight-gradient map at :570-571 is wrong for stride > 1 and is not reproduced).
#include <cstdlib>

#include "cb_internal.h"

namespace cb {
namespace {

struct ConvGeo {
    int N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, OH, OW;
    long long x_batch, y_batch;  // elements between consecutive images of the input-side / output-side tensor
};

constexpr int kOcTile = 8;

__device__ __forceinline__ float apply_epilogue(const ConvEpilogue& ep, float v, int oc, long long pos_idx, float old) {
    if (ep.scale) {
        const long long si = ep.per_position ? pos_idx : (long long)oc;
        v = fmaf(v, ep.scale[si], ep.shift[si]);
    }
    if (ep.bias) v += ep.bias[oc];
    if (ep.accumulate) v += old;
    if (ep.relu) v = fmaxf(v, 0.f);
    return v;
}

// Forward: one thread per output pixel, kOcTile output channels in registers; consecutive threads walk ow, so
// X loads are coalesced and every weight load is a warp-wide broadcast.
__global__ void __launch_bounds__(256) conv_fwd_simt(const float* __restrict__ W, const float* __restrict__ X,
                                                     float* __restrict__ Y, const ConvGeo g, const ConvEpilogue ep) {
    const long long pix = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long npix = (long long)g.N * g.OH * g.OW;
    if (pix >= npix) return;
    const int oc0 = blockIdx.y * kOcTile;
    const int ow = (int)(pix % g.OW);
    const long long t = pix / g.OW;
    const int oh = (int)(t % g.OH);
    const int n = (int)(t / g.OH);
    float acc[kOcTile];
#pragma unroll
    for (int o = 0; o < kOcTile; ++o) acc[o] = 0.f;
    const float* Xn = X + (long long)n * g.x_batch;
    const long long wstride = (long long)g.IC * g.FH * g.FW;
    for (int ic = 0; ic < g.IC; ++ic) {
        for (int fh = 0; fh < g.FH; ++fh) {
            const int ih = oh * g.sH - g.pH + fh;
            if (ih < 0 || ih >= g.IH) continue;
            for (int fw = 0; fw < g.FW; ++fw) {
                const int iw = ow * g.sW - g.pW + fw;
                if (iw < 0 || iw >= g.IW) continue;
                const float x = Xn[((long long)ic * g.IH + ih) * g.IW + iw];
                const float* wp = W + ((long long)oc0 * g.IC + ic) * g.FH * g.FW + fh * g.FW + fw;
#pragma unroll
                for (int o = 0; o < kOcTile; ++o)
                    if (oc0 + o < g.OC) acc[o] = fmaf(__ldg(wp + o * wstride), x, acc[o]);
            }
        }
    }
    float* Yn = Y + (long long)n * g.y_batch;
#pragma unroll
    for (int o = 0; o < kOcTile; ++o)
        if (oc0 + o < g.OC) {
            const long long idx = ((long long)(oc0 + o) * g.OH + oh) * g.OW + ow;
            Yn[idx] = apply_epilogue(ep, acc[o], oc0 + o, idx, ep.accumulate ? Yn[idx] : 0.f);
        }
}

// Data gradient: one thread per dX pixel, kOcTile input channels in registers. x_batch is dX's stride, y_batch dY's.
__global__ void __launch_bounds__(256) conv_dgrad_simt(const float* __restrict__ W, const float* __restrict__ dY,
                                                       float* __restrict__ dX, const ConvGeo g, int accumulate) {
    const long long pix = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long npix = (long long)g.N * g.IH * g.IW;
    if (pix >= npix) return;
    const int ic0 = blockIdx.y * kOcTile;
    const int iw = (int)(pix % g.IW);
    const long long t = pix / g.IW;
    const int ih = (int)(t % g.IH);
    const int n = (int)(t / g.IH);
    float acc[kOcTile];
#pragma unroll
    for (int o = 0; o < kOcTile; ++o) acc[o] = 0.f;
    const float* dYn = dY + (long long)n * g.y_batch;
    const int taps = g.FH * g.FW;
    for (int fh = 0; fh < g.FH; ++fh) {
        const int th = ih + g.pH - fh;
        if (th < 0 || th % g.sH) continue;
        const int oh = th / g.sH;
        if (oh >= g.OH) continue;
        for (int fw = 0; fw < g.FW; ++fw) {
            const int tw = iw + g.pW - fw;
            if (tw < 0 || tw % g.sW) continue;
            const int ow = tw / g.sW;
            if (ow >= g.OW) continue;
            for (int oc = 0; oc < g.OC; ++oc) {
                const float d = dYn[((long long)oc * g.OH + oh) * g.OW + ow];
                const float* wp = W + ((long long)oc * g.IC + ic0) * taps + fh * g.FW + fw;
#pragma unroll
                for (int o = 0; o < kOcTile; ++o)
                    if (ic0 + o < g.IC) acc[o] = fmaf(__ldg(wp + o * taps), d, acc[o]);
            }
        }
    }
    float* dXn = dX + (long long)n * g.x_batch;
#pragma unroll
    for (int o = 0; o < kOcTile; ++o)
        if (ic0 + o < g.IC) {
            float* dst = dXn + ((long long)(ic0 + o) * g.IH + ih) * g.IW + iw;
            *dst = accumulate ? *dst + acc[o] : acc[o];
        }
}

// Weight gradient: one block per (oc, ic) pair and batch slice; threads stride over the output pixels and keep up
// to 9 filter taps in registers, then reduce across the block with warp shuffles.
constexpr int kTapGroup = 9;
__global__ void __launch_bounds__(256) conv_wgrad_simt(const float* __restrict__ dY, const float* __restrict__ X,
                                                       float* __restrict__ dW, const ConvGeo g, int n_per_split,
                                                       int mode /*0 store, 1 add, 2 atomic*/) {
    __shared__ float part[8][kTapGroup];
    const int oc = blockIdx.x, ic = blockIdx.y;
    const int n0 = blockIdx.z * n_per_split;
    const int n1 = min(g.N, n0 + n_per_split);
    const int taps = g.FH * g.FW;
    const int opix = g.OH * g.OW;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int t0 = 0; t0 < taps; t0 += kTapGroup) {
        float acc[kTapGroup];
#pragma unroll
        for (int t = 0; t < kTapGroup; ++t) acc[t] = 0.f;
        for (int n = n0; n < n1; ++n) {
            const float* dyp = dY + (long long)n * g.y_batch + (long long)oc * opix;
            const float* xp = X + (long long)n * g.x_batch + (long long)ic * g.IH * g.IW;
            for (int q = threadIdx.x; q < opix; q += blockDim.x) {
                const int oh = q / g.OW, ow = q - oh * g.OW;
                const float d = dyp[q];
#pragma unroll
                for (int t = 0; t < kTapGroup; ++t) {
                    const int tap = t0 + t;
                    if (tap < taps) {
                        const int fh = tap / g.FW, fw = tap - fh * g.FW;
                        const int ih = oh * g.sH - g.pH + fh, iw = ow * g.sW - g.pW + fw;
                        if (ih >= 0 && ih < g.IH && iw >= 0 && iw < g.IW) acc[t] = fmaf(d, xp[ih * g.IW + iw], acc[t]);
                    }
                }
            }
        }
#pragma unroll
        for (int t = 0; t < kTapGroup; ++t) {
            float v = acc[t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) part[warp][t] = v;
        }
        __syncthreads();
        if (threadIdx.x < kTapGroup && t0 + threadIdx.x < taps) {
            float v = 0.f;
            for (int w = 0; w < 8; ++w) v += part[w][threadIdx.x];
            float* dst = dW + ((long long)oc * g.IC + ic) * taps + t0 + threadIdx.x;
            if (mode == 2) atomicAdd(dst, v);
            else if (mode == 1) *dst += v;
            else *dst = v;
        }
        __syncthreads();
    }
}

int make_geo(cb_ctx* ctx, ConvGeo& g, int N, int IC, int IH, int IW, int OC, int FH, int FW, int sH, int sW, int pH,
             int pW, long long x_batch, long long y_batch, const char* who) {
    if (N < 0 || IC < 0 || OC < 0 || IH < 0 || IW < 0) return fail(ctx, CB_EINVAL, std::string(who) + ": negative extent");
    if (FH < 1 || FW < 1 || sH < 1 || sW < 1 || pH < 0 || pW < 0)
        return fail(ctx, CB_EINVAL, std::string(who) + ": filter, stride must be >= 1 and padding >= 0");
    if (IH + 2 * pH < FH || IW + 2 * pW < FW) return fail(ctx, CB_EINVAL, std::string(who) + ": filter larger than the padded input");
    g = ConvGeo{N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, (IH - FH + 2 * pH) / sH + 1, (IW - FW + 2 * pW) / sW + 1, 0, 0};
    const long long x_dense = (long long)IC * IH * IW, y_dense = (long long)OC * g.OH * g.OW;
    if ((x_batch && x_batch < x_dense) || (y_batch && y_batch < y_dense))
        return fail(ctx, CB_EINVAL, std::string(who) + ": batch stride smaller than one image");
    g.x_batch = x_batch ? x_batch : x_dense;
    g.y_batch = y_batch ? y_batch : y_dense;
    return CB_OK;
}

int after_launch(cb_ctx* ctx, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, what);
    ctx->launches += 1;
    ctx->last_kernel = "simt_fp32";
    return finish(ctx, what);
}

// ---- 3xTF32 composition: x = hi + lo with hi = the 19 bits the tensor core reads, lo = rna_tf32(x - hi).
// lo[n][i] = lo part of x[n*x_batch + i], written densely (per elements per image)
__global__ void tf32_lo_kernel(const float* __restrict__ x, float* __restrict__ lo, long long n, long long per,
                               long long x_batch) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long img = i / per;
        const float v = x[img * x_batch + (i - img * per)];
        const float hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
        uint32_t r;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v - hi));
        lo[i] = __uint_as_float(r);
    }
}
// out = epilogue((a + b) + c): the sum of the three tensor-core passes (the two small cross terms first), dense
// temporaries in, (possibly strided) output tensor out
__global__ void sum3_kernel(float* __restrict__ out, const float* __restrict__ lead, const float* __restrict__ a,
                            const float* __restrict__ b, const ConvEpilogue ep, long long n, long long per, long long plane,
                            long long out_batch) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long img = i / per, r = i - img * per;
        float* dst = out + img * out_batch + r;
        const float v = (a[i] + b[i]) + lead[i];
        *dst = apply_epilogue(ep, v, (int)(r / plane), r, ep.accumulate ? *dst : 0.f);
    }
}

int grid_el(const cb_ctx* ctx, long long n) {
    long long g = (n + 255) / 256;
    const long long cap = (long long)ctx->sm_count * 16;
    return (int)(g > cap ? cap : (g < 1 ? 1 : g));
}

}  // namespace

// 3xTF32 forward / data gradient on the tensor cores: out = pass(W_hi, In_lo) + pass(W_lo, In_hi) + pass(W_hi, In_hi),
// where every pass is the TF32 kernel (it reads the hi parts by truncation). The dropped lo*lo term is < 2^-20 relative.
// Scratch (workspace3): In_lo, W_lo and the three partial outputs, all densely packed; the last kernel adds them and
// applies the epilogue while writing the caller's output. Returns CB_EUNSUPPORTED when the TF32 kernel does not cover the
// geometry, before any work was queued.
static int conv_3xtf32(cb_ctx* ctx, const float* W, const float* In, float* Out, const ConvEpilogue& ep, int N, int IC,
                       int IH, int IW, int OC, int FH, int FW, int sH, int sW, int pH, int pW, bool dgrad_of,
                       long long in_per, long long out_per, long long out_plane, long long in_batch, long long out_batch) {
    static const int one_pass = [] {
        const char* e = std::getenv("CB_CONV_X3_ONEPASS");  // development switch, default on
        return e ? std::atoi(e) : 1;
    }();
    if (one_pass && sH == 1 && sW == 1) {
        // one pass of the tensor-core kernel over three channel groups, when the tripled filter fits
        const int rc1 = umma_conv_fwd_x3(ctx, W, In, Out, ep, N, IC, IH, IW, OC, FH, FW, pH, pW, dgrad_of, in_batch, out_batch);
        if (rc1 != CB_EUNSUPPORTED) return rc1;
    }
    const long long w_elems = (long long)OC * IC * FH * FW;
    const long long in_elems = in_per * N, out_elems = out_per * N;
    auto up = [](long long n) { return (n + 63) & ~63LL; };
    const size_t need = (size_t)(up(in_elems) + up(w_elems) + 3 * up(out_elems)) * sizeof(float);
    int rc = ensure_workspace3(ctx, need);
    if (rc != CB_OK) return rc;
    float* in_lo = static_cast<float*>(ctx->workspace3);
    float* w_lo = in_lo + up(in_elems);
    float* t0 = w_lo + up(w_elems);
    float* t1 = t0 + up(out_elems);
    float* t2 = t1 + up(out_elems);
    const ConvEpilogue plain{};
    // leading term first: it also tells whether the geometry is covered
    rc = umma_conv_fwd(ctx, W, In, t0, plain, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, dgrad_of, in_batch, 0);
    if (rc != CB_OK) return rc;
    tf32_lo_kernel<<<grid_el(ctx, in_elems), 256, 0, ctx->stream>>>(In, in_lo, in_elems, in_per, in_batch ? in_batch : in_per);
    tf32_lo_kernel<<<grid_el(ctx, w_elems), 256, 0, ctx->stream>>>(W, w_lo, w_elems, w_elems, w_elems);
    rc = umma_conv_fwd(ctx, W, in_lo, t1, plain, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, dgrad_of, 0, 0);
    if (rc == CB_OK) {
        // w_lo is a temporary whose address recurs with different contents: it must not enter the packed-filter cache
        const int cache_on = ctx->filter_cache_on;
        ctx->filter_cache_on = 0;
        rc = umma_conv_fwd(ctx, w_lo, In, t2, plain, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, dgrad_of, in_batch, 0);
        ctx->filter_cache_on = cache_on;
    }
    if (rc != CB_OK) return rc;
    sum3_kernel<<<grid_el(ctx, out_elems), 256, 0, ctx->stream>>>(Out, t0, t1, t2, ep, out_elems, out_per, out_plane,
                                                                 out_batch ? out_batch : out_per);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "3xTF32 convolution");
    ctx->launches += 3;
    ctx->last_kernel = "umma_3xtf32";
    return CB_OK;
}

// 3xTF32 weight gradient: the products dY_hi X_hi, dY_hi X_lo, dY_lo X_hi in ONE launch of the tensor-core kernel
// (it walks the pixels three times into one accumulator), or, with that switched off, as three accumulating launches
// (dense tensors only).
static int wgrad_3xtf32(cb_ctx* ctx, const float* dY, const float* X, float* dW, int N, int IC, int IH, int IW, int OC, int FH,
                        int FW, int sH, int sW, int pH, int pW, int accumulate, long long x_elems, long long dy_elems,
                        long long dy_batch, long long x_batch) {
    static const int onepass = [] {
        const char* e = std::getenv("CB_WGRAD_X3_ONEPASS");  // development switch, default on
        return e ? std::atoi(e) : 1;
    }();
    if (onepass) {
        const int rc1 = umma_conv_wgrad(ctx, dY, X, dW, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, accumulate, dy_batch, x_batch, true);
        if (rc1 == CB_OK) ctx->last_kernel = "umma_3xtf32";
        return rc1;
    }
    if (dy_batch || x_batch) return CB_EUNSUPPORTED;
    auto up = [](long long n) { return (n + 63) & ~63LL; };
    int rc = ensure_workspace3(ctx, (size_t)(up(x_elems) + up(dy_elems)) * sizeof(float));
    if (rc != CB_OK) return rc;
    float* x_lo = static_cast<float*>(ctx->workspace3);
    float* dy_lo = x_lo + up(x_elems);
    rc = umma_conv_wgrad(ctx, dY, X, dW, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, accumulate, 0, 0);
    if (rc != CB_OK) return rc;
    tf32_lo_kernel<<<grid_el(ctx, x_elems), 256, 0, ctx->stream>>>(X, x_lo, x_elems, x_elems, x_elems);
    tf32_lo_kernel<<<grid_el(ctx, dy_elems), 256, 0, ctx->stream>>>(dY, dy_lo, dy_elems, dy_elems, dy_elems);
    rc = umma_conv_wgrad(ctx, dY, x_lo, dW, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, 1, 0, 0);
    if (rc == CB_OK) rc = umma_conv_wgrad(ctx, dy_lo, X, dW, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, 1, 0, 0);
    if (rc != CB_OK) return rc;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "3xTF32 weight gradient");
    ctx->launches += 2;
    ctx->last_kernel = "umma_3xtf32";
    return CB_OK;
}

}  // namespace cb

using namespace cb;

static int conv_fwd_impl(cb_ctx* ctx, const float* W, const float* X, float* Y, int N, int IC, int IH, int IW, int OC, int FH,
                         int FW, int sH, int sW, int pH, int pW, const cb_epilogue* cep, const char* who) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    ConvEpilogue ep{};
    long long xb = 0, yb = 0;
    if (cep) {
        ep.bias = cep->bias; ep.scale = cep->scale; ep.shift = cep->shift;
        ep.per_position = cep->per_position ? 1 : 0; ep.relu = cep->relu ? 1 : 0; ep.accumulate = cep->accumulate ? 1 : 0;
        xb = cep->x_batch_stride; yb = cep->y_batch_stride;
        if ((ep.scale == nullptr) != (ep.shift == nullptr)) return fail(ctx, CB_EINVAL, std::string(who) + ": scale and shift go together");
    }
    ConvGeo g;
    int rc = make_geo(ctx, g, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, xb, yb, who);
    if (rc != CB_OK) return rc;
    const long long npix = (long long)N * g.OH * g.OW;
    if (npix == 0 || OC == 0) return CB_OK;
    if (!W || !X || !Y) return fail(ctx, CB_EINVAL, std::string(who) + ": null operand");
    if (ctx->math == CB_MATH_TF32) {  // tensor cores; 3xTF32 = three such passes; FP32 (and uncovered geometries) = CUDA cores
        rc = umma_conv_fwd(ctx, W, X, Y, ep, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, false, xb, yb);
        if (rc != CB_EUNSUPPORTED) return rc == CB_OK ? finish(ctx, who) : rc;
    } else if (ctx->math == CB_MATH_3XTF32) {
        rc = conv_3xtf32(ctx, W, X, Y, ep, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, false, (long long)IC * IH * IW,
                         (long long)OC * g.OH * g.OW, (long long)g.OH * g.OW, xb, yb);
        if (rc != CB_EUNSUPPORTED) return rc == CB_OK ? finish(ctx, who) : rc;
    }
    dim3 grid((unsigned)((npix + 255) / 256), (unsigned)((OC + kOcTile - 1) / kOcTile));
    conv_fwd_simt<<<grid, 256, 0, ctx->stream>>>(W, X, Y, g, ep);
    return after_launch(ctx, who);
}

static int conv_dgrad_impl(cb_ctx* ctx, const float* W, const float* dY, float* dX, int N, int IC, int IH, int IW, int OC,
                           int FH, int FW, int sH, int sW, int pH, int pW, int accumulate, long long dy_batch, long long dx_batch,
                           const char* who) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    ConvGeo g;
    int rc = make_geo(ctx, g, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, dx_batch, dy_batch, who);
    if (rc != CB_OK) return rc;
    const long long npix = (long long)N * IH * IW;
    if (npix == 0 || IC == 0) return CB_OK;
    if (!W || !dY || !dX) return fail(ctx, CB_EINVAL, std::string(who) + ": null operand");
    ConvEpilogue ep{};
    ep.accumulate = accumulate ? 1 : 0;
    if (ctx->math == CB_MATH_TF32) {
        rc = umma_conv_fwd(ctx, W, dY, dX, ep, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, true, dy_batch, dx_batch);
        if (rc != CB_EUNSUPPORTED) return rc == CB_OK ? finish(ctx, who) : rc;
    } else if (ctx->math == CB_MATH_3XTF32) {
        rc = conv_3xtf32(ctx, W, dY, dX, ep, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, true, (long long)OC * g.OH * g.OW,
                         (long long)IC * IH * IW, (long long)IH * IW, dy_batch, dx_batch);
        if (rc != CB_EUNSUPPORTED) return rc == CB_OK ? finish(ctx, who) : rc;
    }
    dim3 grid((unsigned)((npix + 255) / 256), (unsigned)((IC + kOcTile - 1) / kOcTile));
    conv_dgrad_simt<<<grid, 256, 0, ctx->stream>>>(W, dY, dX, g, accumulate ? 1 : 0);
    return after_launch(ctx, who);
}

extern "C" {

int cb_conv_fwd(cb_ctx* ctx, const float* W, const float* X, float* Y, const float* bias, int N, int IC, int IH,
                int IW, int OC, int FH, int FW, int sH, int sW, int pH, int pW, int relu) {
    cb_epilogue ep{};
    ep.bias = bias;
    ep.relu = relu;
    return conv_fwd_impl(ctx, W, X, Y, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, &ep, "cb_conv_fwd");
}

int cb_conv_fwd_ex(cb_ctx* ctx, const float* W, const float* X, float* Y, int N, int IC, int IH, int IW, int OC, int FH,
                   int FW, int sH, int sW, int pH, int pW, const cb_epilogue* ep) {
    return conv_fwd_impl(ctx, W, X, Y, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, ep, "cb_conv_fwd_ex");
}

int cb_conv_dgrad(cb_ctx* ctx, const float* W, const float* dY, float* dX, int N, int IC, int IH, int IW, int OC,
                  int FH, int FW, int sH, int sW, int pH, int pW) {
    return conv_dgrad_impl(ctx, W, dY, dX, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, 0, 0, 0, "cb_conv_dgrad");
}

int cb_conv_dgrad_ex(cb_ctx* ctx, const float* W, const float* dY, float* dX, int N, int IC, int IH, int IW, int OC,
                     int FH, int FW, int sH, int sW, int pH, int pW, int accumulate, long long dy_batch_stride,
                     long long dx_batch_stride) {
    return conv_dgrad_impl(ctx, W, dY, dX, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, accumulate, dy_batch_stride,
                           dx_batch_stride, "cb_conv_dgrad_ex");
}

int cb_conv_cache_filters(cb_ctx* ctx, int on) {
    if (!ctx) return CB_EINVAL;
    ctx->filter_cache_on = on ? 1 : 0;
    ctx->filter_version += 1;
    return CB_OK;
}

int cb_filters_changed(cb_ctx* ctx) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    const int rc = filter_cache_repack_all(ctx);
    return rc == CB_OK ? finish(ctx, "cb_filters_changed") : rc;
}

}  // extern "C"

static int conv_wgrad_impl(cb_ctx* ctx, const float* dY, const float* X, float* dW, int N, int IC, int IH, int IW, int OC,
                           int FH, int FW, int sH, int sW, int pH, int pW, int accumulate, long long dy_batch, long long x_batch,
                           const char* who) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    ConvGeo g;
    int rc = make_geo(ctx, g, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, x_batch, dy_batch, who);
    if (rc != CB_OK) return rc;
    if (OC == 0 || IC == 0) return CB_OK;
    if (!dW) return fail(ctx, CB_EINVAL, std::string(who) + ": null operand");
    const size_t wbytes = (size_t)OC * IC * FH * FW * sizeof(float);
    if ((long long)N * g.OH * g.OW == 0) {
        if (!accumulate) {
            cudaError_t e = cudaMemsetAsync(dW, 0, wbytes, ctx->stream);
            if (e != cudaSuccess) return check_cuda(ctx, e, "convolution weight gradient: clear");
        }
        return finish(ctx, who);
    }
    if (!dY || !X) return fail(ctx, CB_EINVAL, std::string(who) + ": null operand");
    if (ctx->math == CB_MATH_TF32) {
        rc = umma_conv_wgrad(ctx, dY, X, dW, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, accumulate, dy_batch, x_batch);
        if (rc != CB_EUNSUPPORTED) return rc == CB_OK ? finish(ctx, who) : rc;
    } else if (ctx->math == CB_MATH_3XTF32) {
        rc = wgrad_3xtf32(ctx, dY, X, dW, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, accumulate,
                          (long long)N * IC * IH * IW, (long long)N * OC * g.OH * g.OW, dy_batch, x_batch);
        if (rc != CB_EUNSUPPORTED) return rc == CB_OK ? finish(ctx, who) : rc;
    }
    if (OC > 65535 || IC > 65535) return fail(ctx, CB_EUNSUPPORTED, std::string(who) + ": more than 65535 channels");
    int splits = 1;
    if (!ctx->deterministic) {
        const long long pairs = (long long)OC * IC;
        splits = (int)((4LL * ctx->sm_count + pairs - 1) / pairs);
        if (splits > N) splits = N;
        if (splits < 1) splits = 1;
    }
    const int nps = (N + splits - 1) / splits;
    splits = (N + nps - 1) / nps;
    int mode = accumulate ? 1 : 0;
    if (splits > 1) {
        mode = 2;
        if (!accumulate) {
            cudaError_t e = cudaMemsetAsync(dW, 0, wbytes, ctx->stream);
            if (e != cudaSuccess) return check_cuda(ctx, e, "convolution weight gradient: clear");
        }
    }
    conv_wgrad_simt<<<dim3(OC, IC, splits), 256, 0, ctx->stream>>>(dY, X, dW, g, nps, mode);
    return after_launch(ctx, who);
}

extern "C" {

int cb_conv_wgrad(cb_ctx* ctx, const float* dY, const float* X, float* dW, int N, int IC, int IH, int IW, int OC,
                  int FH, int FW, int sH, int sW, int pH, int pW, int accumulate) {
    return conv_wgrad_impl(ctx, dY, X, dW, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, accumulate, 0, 0, "cb_conv_wgrad");
}

int cb_conv_wgrad_ex(cb_ctx* ctx, const float* dY, const float* X, float* dW, int N, int IC, int IH, int IW, int OC,
                     int FH, int FW, int sH, int sW, int pH, int pW, int accumulate, long long dy_batch_stride,
                     long long x_batch_stride) {
    return conv_wgrad_impl(ctx, dY, X, dW, N, IC, IH, IW, OC, FH, FW, sH, sW, pH, pW, accumulate, dy_batch_stride,
                           x_batch_stride, "cb_conv_wgrad_ex");
}

}  // extern "C"
