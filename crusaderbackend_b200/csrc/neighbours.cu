// Memory-bound neighbours of the contraction path: per-(c,h,w) BatchNorm, ReLU, average / global-average
// pooling, softmax + cross-entropy, bias add / bias gradient, Momentum-SGD and the in-place tensor arithmetic of
// seblas::Tensor. All kernels stream HBM with 128-bit accesses where alignment allows, use grid-stride loops
// sized to the SM count, and reduce with warp shuffles.
#include <vector>

#include "cb_internal.h"
#include "cb_ptx.cuh"

namespace cb {
namespace {

constexpr int kThreads = 256;

inline int grid_for(const cb_ctx* ctx, long long work_items, int per_block = kThreads) {
    long long blocks = (work_items + per_block - 1) / per_block;
    const long long cap = (long long)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ------------------------------------------------------------------ BatchNorm over the batch, per position
// One thread owns VEC consecutive positions p (a float4 when VEC == 4) and walks the batch with stride P, so a
// warp reads 512 contiguous bytes per sample. Two passes over X for mean / variance, third pass writes Y, xhat.
template <int VEC>
__global__ void bn_fwd_kernel(const float* __restrict__ X, const float* __restrict__ beta,
                              const float* __restrict__ gamma, float* __restrict__ mean, float* __restrict__ var,
                              float* __restrict__ Y, float* __restrict__ xhat, int N, long long P) {
    const long long nvec = P / VEC;
    for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec;
         v += (long long)gridDim.x * blockDim.x) {
        const long long p = v * VEC;
        float m[VEC], s[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) { m[e] = 0.f; s[e] = 0.f; }
        for (int n = 0; n < N; ++n) {
            float x[VEC];
            if (VEC == 4) *reinterpret_cast<float4*>(x) = *reinterpret_cast<const float4*>(X + n * P + p);
            else x[0] = X[n * P + p];
#pragma unroll
            for (int e = 0; e < VEC; ++e) m[e] += x[e];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) m[e] /= (float)N;
        for (int n = 0; n < N; ++n) {
            float x[VEC];
            if (VEC == 4) *reinterpret_cast<float4*>(x) = *reinterpret_cast<const float4*>(X + n * P + p);
            else x[0] = X[n * P + p];
#pragma unroll
            for (int e = 0; e < VEC; ++e) s[e] += (x[e] - m[e]) * (x[e] - m[e]);
        }
        float inv[VEC], g[VEC], b[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            s[e] /= (float)N;
            inv[e] = 1.0f / sqrtf(s[e] + 1e-8f);
            g[e] = gamma[p + e];
            b[e] = beta[p + e];
        }
        for (int n = 0; n < N; ++n) {
            float x[VEC], y[VEC], h[VEC];
            if (VEC == 4) *reinterpret_cast<float4*>(x) = *reinterpret_cast<const float4*>(X + n * P + p);
            else x[0] = X[n * P + p];
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                h[e] = (x[e] - m[e]) * inv[e];
                y[e] = h[e] * g[e] + b[e];
            }
            if (VEC == 4) {
                *reinterpret_cast<float4*>(Y + n * P + p) = *reinterpret_cast<float4*>(y);
                if (xhat) *reinterpret_cast<float4*>(xhat + n * P + p) = *reinterpret_cast<float4*>(h);
            } else {
                Y[n * P + p] = y[0];
                if (xhat) xhat[n * P + p] = h[0];
            }
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            if (mean) mean[p + e] = m[e];
            if (var) var[p + e] = s[e];
        }
    }
}

template <int VEC>
__global__ void bn_bwd_kernel(const float* __restrict__ dY, const float* __restrict__ gamma,
                              const float* __restrict__ X, float* __restrict__ dX, int N, long long P) {
    const long long nvec = P / VEC;
    const float invN = 1.0f / (float)N;
    for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec;
         v += (long long)gridDim.x * blockDim.x) {
        const long long p = v * VEC;
        float m[VEC], s[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) { m[e] = 0.f; s[e] = 0.f; }
        for (int n = 0; n < N; ++n) {
            float x[VEC];
            if (VEC == 4) *reinterpret_cast<float4*>(x) = *reinterpret_cast<const float4*>(X + n * P + p);
            else x[0] = X[n * P + p];
#pragma unroll
            for (int e = 0; e < VEC; ++e) m[e] += x[e];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) m[e] *= invN;
        // one pass gathers sum(dxhat * xc), sum(dxhat), sum(xc) and sum(xc^2)
        float sdx[VEC], sd[VEC], sxc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) { sdx[e] = 0.f; sd[e] = 0.f; sxc[e] = 0.f; }
        float g[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) g[e] = gamma[p + e];
        for (int n = 0; n < N; ++n) {
            float x[VEC], dy[VEC];
            if (VEC == 4) {
                *reinterpret_cast<float4*>(x) = *reinterpret_cast<const float4*>(X + n * P + p);
                *reinterpret_cast<float4*>(dy) = *reinterpret_cast<const float4*>(dY + n * P + p);
            } else {
                x[0] = X[n * P + p];
                dy[0] = dY[n * P + p];
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float xc = x[e] - m[e];
                const float dxh = dy[e] * g[e];
                s[e] += xc * xc;
                sdx[e] += dxh * xc;
                sd[e] += dxh;
                sxc[e] += xc;
            }
        }
        float inv[VEC], dvar[VEC], dmean[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float varv = s[e] * invN + 1e-8f;
            inv[e] = 1.0f / sqrtf(varv);
            dvar[e] = sdx[e] * -0.5f * inv[e] * inv[e] * inv[e];
            dmean[e] = -sd[e] * inv[e] + dvar[e] * (-2.0f * sxc[e]) * invN;
        }
        for (int n = 0; n < N; ++n) {
            float x[VEC], dy[VEC], o[VEC];
            if (VEC == 4) {
                *reinterpret_cast<float4*>(x) = *reinterpret_cast<const float4*>(X + n * P + p);
                *reinterpret_cast<float4*>(dy) = *reinterpret_cast<const float4*>(dY + n * P + p);
            } else {
                x[0] = X[n * P + p];
                dy[0] = dY[n * P + p];
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                o[e] = dy[e] * g[e] * inv[e] + dvar[e] * (x[e] - m[e]) * 2.0f * invN + dmean[e] * invN;
            if (VEC == 4) *reinterpret_cast<float4*>(dX + n * P + p) = *reinterpret_cast<float4*>(o);
            else dX[n * P + p] = o[0];
        }
    }
}

template <int VEC>
__global__ void bn_paramgrad_kernel(const float* __restrict__ dY, const float* __restrict__ xhat,
                                    float* __restrict__ dgamma, float* __restrict__ dbeta, int N, long long P) {
    const long long nvec = P / VEC;
    for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec;
         v += (long long)gridDim.x * blockDim.x) {
        const long long p = v * VEC;
        float sg[VEC], sb[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) { sg[e] = 0.f; sb[e] = 0.f; }
        for (int n = 0; n < N; ++n) {
            float h[VEC], dy[VEC];
            if (VEC == 4) {
                *reinterpret_cast<float4*>(h) = *reinterpret_cast<const float4*>(xhat + n * P + p);
                *reinterpret_cast<float4*>(dy) = *reinterpret_cast<const float4*>(dY + n * P + p);
            } else {
                h[0] = xhat[n * P + p];
                dy[0] = dY[n * P + p];
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) { sb[e] += dy[e]; sg[e] += dy[e] * h[e]; }
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) { dgamma[p + e] = sg[e]; dbeta[p + e] = sb[e]; }
    }
}


// ------------------------------------------------------------------ BatchNorm, batch-parallel form
// Block = 16 float4 position vectors (64 positions, 256 contiguous bytes per sample) x 16 batch groups. Every thread
// keeps its SPT samples (n = group, group + 16, ...) in registers, so X (and dY) are read from HBM exactly once;
// the per-position sums are combined across the 16 groups through shared memory in a fixed order. This fills the GPU
// where the one-thread-per-position form leaves it with P/4 threads (4096 for a 16x32x32 map).
__device__ __forceinline__ float4 f4_add(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 f4_zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }

// sum over the 16 batch groups of the block; every thread returns the total of its position vector
__device__ __forceinline__ float4 bn_group_sum(float4 v, float4 (*red)[16]) {
    red[threadIdx.y][threadIdx.x] = v;
    __syncthreads();
    float4 t = f4_zero();
#pragma unroll
    for (int g = 0; g < 16; ++g) t = f4_add(t, red[g][threadIdx.x]);
    __syncthreads();
    return t;
}

// Sums, over the G batch groups of a block, of Q float4 quantities per position vector; every thread returns the totals
// of its position. The G x (Q float4) values go through shared memory once: thread (x, g) with g < 4 Q adds component
// g & 3 of quantity g >> 2 over the groups in group order (a fixed order: deterministic), and everyone reads the
// totals back. red: Q * 1024 floats, tot: Q * (1024 / G) floats.
template <int Q, int G>
__device__ __forceinline__ void bn_block_sums(float4 (&v)[Q], float* red, float* tot) {
    constexpr int W = (256 / G) * 4;  // floats per group row: the block's positions
    static_assert(G >= 4 * Q, "one summing thread per (quantity, component)");
    const int x = threadIdx.x, g = threadIdx.y;
#pragma unroll
    for (int q = 0; q < Q; ++q) *reinterpret_cast<float4*>(red + (q * G + g) * W + x * 4) = v[q];
    __syncthreads();
    if (g < 4 * Q) {
        const float* src = red + (g >> 2) * G * W + x * 4 + (g & 3);
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < G; ++k) t += src[k * W];
        tot[(g >> 2) * W + x * 4 + (g & 3)] = t;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < Q; ++q) v[q] = *reinterpret_cast<const float4*>(tot + q * W + x * 4);
}

// Block = 256 / G float4 position vectors x G batch groups (G = 16, 32 or 64: more groups for small maps, so that the
// grid still covers the GPU); thread (x, g) keeps samples n = g, g + G, ... (SPT of them) in registers.
template <int SPT, int G>
__global__ void __launch_bounds__(256) bn_fwd_par_kernel(const float* __restrict__ X, const float* __restrict__ beta,
                                                         const float* __restrict__ gamma, float* __restrict__ mean,
                                                         float* __restrict__ var, float* __restrict__ Y,
                                                         float* __restrict__ xhat, const float* __restrict__ res, int N,
                                                         long long P, int relu, long long xs) {
    // xs: floats between consecutive samples of X (P when dense; larger for a channel-prefix view of a wider tensor)
    constexpr int PB = 256 / G;
    __shared__ __align__(16) float red[1024];
    __shared__ __align__(16) float tot[PB * 4];
    griddep_wait();
    griddep_launch();
    const long long p = ((long long)blockIdx.x * PB + threadIdx.x) * 4;
    const bool live = p < P;
    const int g = threadIdx.y;
    float4 x[SPT];
    float4 s[1] = {f4_zero()};
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        const int n = g + G * i;
        x[i] = (live && n < N) ? *reinterpret_cast<const float4*>(X + (long long)n * xs + p) : f4_zero();
        s[0] = f4_add(s[0], x[i]);
    }
    const float invN = 1.0f / (float)N;
    bn_block_sums<1, G>(s, red, tot);
    const float4 m = make_float4(s[0].x * invN, s[0].y * invN, s[0].z * invN, s[0].w * invN);
    float4 q[1] = {f4_zero()};
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        if (g + G * i < N) {
            const float a = x[i].x - m.x, b = x[i].y - m.y, c = x[i].z - m.z, d = x[i].w - m.w;
            q[0] = f4_add(q[0], make_float4(a * a, b * b, c * c, d * d));
        }
    }
    bn_block_sums<1, G>(q, red, tot);
    const float4 v = make_float4(q[0].x * invN, q[0].y * invN, q[0].z * invN, q[0].w * invN);
    if (!live) return;
    const float4 inv = make_float4(1.0f / sqrtf(v.x + 1e-8f), 1.0f / sqrtf(v.y + 1e-8f), 1.0f / sqrtf(v.z + 1e-8f),
                                   1.0f / sqrtf(v.w + 1e-8f));
    const float4 ga = *reinterpret_cast<const float4*>(gamma + p), be = *reinterpret_cast<const float4*>(beta + p);
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        const int n = g + G * i;
        if (n < N) {
            const float4 h = make_float4((x[i].x - m.x) * inv.x, (x[i].y - m.y) * inv.y, (x[i].z - m.z) * inv.z,
                                         (x[i].w - m.w) * inv.w);
            float4 y = make_float4(h.x * ga.x + be.x, h.y * ga.y + be.y, h.z * ga.z + be.z, h.w * ga.w + be.w);
            if (res) y = f4_add(y, *reinterpret_cast<const float4*>(res + (long long)n * P + p));  // shortcut add
            if (relu) y = make_float4(fmaxf(y.x, 0.f), fmaxf(y.y, 0.f), fmaxf(y.z, 0.f), fmaxf(y.w, 0.f));
            *reinterpret_cast<float4*>(Y + (long long)n * P + p) = y;
            if (xhat) *reinterpret_cast<float4*>(xhat + (long long)n * P + p) = h;
        }
    }
    if (g == 0) {
        if (mean) *reinterpret_cast<float4*>(mean + p) = m;
        if (var) *reinterpret_cast<float4*>(var + p) = v;
    }
}

// Data gradient (statistics recomputed from X as seblas::batchNormGrad does) and, when dgamma / dbeta are given, the
// parameter gradients dbeta = sum dy, dgamma = sum dy * xhat of seblas::batchNormParamGrads in the same pass.
template <int SPT, int G>
__global__ void __launch_bounds__(256, SPT <= 4 ? 4 : 1) bn_bwd_par_kernel(const float* __restrict__ dY, const float* __restrict__ gamma,
                                                         const float* __restrict__ X, float* __restrict__ dX,
                                                         float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                         const float* __restrict__ relu_out, float* __restrict__ dres,
                                                         int dres_add, int pg_add, int N, long long P, long long xs,
                                                         long long dxs, int dx_add) {
    // xs / dxs: floats between consecutive samples of X / dX (P when dense); dx_add: dX += instead of dX =
    constexpr int PB = 256 / G;
    __shared__ __align__(16) float red[4 * 1024];
    __shared__ __align__(16) float tot[4 * PB * 4];
    griddep_wait();
    griddep_launch();
    const long long p = ((long long)blockIdx.x * PB + threadIdx.x) * 4;
    const bool live = p < P;
    const int g = threadIdx.y;
    float4 x[SPT], dy[SPT];
    float4 s[1] = {f4_zero()};
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        const int n = g + G * i;
        const bool on = live && n < N;
        x[i] = on ? *reinterpret_cast<const float4*>(X + (long long)n * xs + p) : f4_zero();
        dy[i] = on ? *reinterpret_cast<const float4*>(dY + (long long)n * P + p) : f4_zero();
        if (relu_out && on) {  // the ReLU that followed this layer in the forward pass: dy passes where its output is > 0
            const float4 r = *reinterpret_cast<const float4*>(relu_out + (long long)n * P + p);
            dy[i] = make_float4(r.x > 0.f ? dy[i].x : 0.f, r.y > 0.f ? dy[i].y : 0.f, r.z > 0.f ? dy[i].z : 0.f,
                                r.w > 0.f ? dy[i].w : 0.f);
        }
        if (dres && on) {  // the shortcut that was added before that ReLU receives the same masked gradient
            float4* d = reinterpret_cast<float4*>(dres + (long long)n * P + p);
            *d = dres_add ? f4_add(*d, dy[i]) : dy[i];
        }
        s[0] = f4_add(s[0], x[i]);
    }
    const float invN = 1.0f / (float)N;
    bn_block_sums<1, G>(s, red, tot);
    const float4 m = make_float4(s[0].x * invN, s[0].y * invN, s[0].z * invN, s[0].w * invN);
    const float4 ga = live ? *reinterpret_cast<const float4*>(gamma + p) : f4_zero();
    // sums of xc^2, dy * xc (dxhat = dy * gamma is factored out below), dy and xc, in one exchange
    float4 sums[4] = {f4_zero(), f4_zero(), f4_zero(), f4_zero()};
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        if (g + G * i < N) {
            const float4 xc = make_float4(x[i].x - m.x, x[i].y - m.y, x[i].z - m.z, x[i].w - m.w);
            x[i] = xc;  // keep the centred value
            sums[0] = f4_add(sums[0], make_float4(xc.x * xc.x, xc.y * xc.y, xc.z * xc.z, xc.w * xc.w));
            sums[1] = f4_add(sums[1], make_float4(dy[i].x * xc.x, dy[i].y * xc.y, dy[i].z * xc.z, dy[i].w * xc.w));
            sums[2] = f4_add(sums[2], dy[i]);
            sums[3] = f4_add(sums[3], xc);
        }
    }
    bn_block_sums<4, G>(sums, red, tot);
    const float4 sq = sums[0], sdx = sums[1], sd = sums[2], sxc = sums[3];
    if (!live) return;
    float o_inv[4], o_dvar[4], o_dmean[4];
    const float sqv[4] = {sq.x, sq.y, sq.z, sq.w}, sdxv[4] = {sdx.x, sdx.y, sdx.z, sdx.w}, sdv[4] = {sd.x, sd.y, sd.z, sd.w},
                sxcv[4] = {sxc.x, sxc.y, sxc.z, sxc.w}, gav[4] = {ga.x, ga.y, ga.z, ga.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float inv = 1.0f / sqrtf(sqv[e] * invN + 1e-8f);
        o_inv[e] = inv;
        o_dvar[e] = gav[e] * sdxv[e] * -0.5f * inv * inv * inv;
        o_dmean[e] = -gav[e] * sdv[e] * inv + o_dvar[e] * (-2.0f * sxcv[e]) * invN;
    }
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        const int n = g + G * i;
        if (n < N) {
            float4 o;
            o.x = dy[i].x * gav[0] * o_inv[0] + o_dvar[0] * x[i].x * 2.0f * invN + o_dmean[0] * invN;
            o.y = dy[i].y * gav[1] * o_inv[1] + o_dvar[1] * x[i].y * 2.0f * invN + o_dmean[1] * invN;
            o.z = dy[i].z * gav[2] * o_inv[2] + o_dvar[2] * x[i].z * 2.0f * invN + o_dmean[2] * invN;
            o.w = dy[i].w * gav[3] * o_inv[3] + o_dvar[3] * x[i].w * 2.0f * invN + o_dmean[3] * invN;
            float4* dst = reinterpret_cast<float4*>(dX + (long long)n * dxs + p);
            *dst = dx_add ? f4_add(*dst, o) : o;
        }
    }
    if (g == 0 && dgamma && dbeta) {
        float4 gb = sd;
        float4 gg = make_float4(sdx.x * o_inv[0], sdx.y * o_inv[1], sdx.z * o_inv[2], sdx.w * o_inv[3]);  // sum dy * xhat
        if (pg_add) {  // a later group of a batch whose statistics are taken per group
            gb = f4_add(gb, *reinterpret_cast<const float4*>(dbeta + p));
            gg = f4_add(gg, *reinterpret_cast<const float4*>(dgamma + p));
        }
        *reinterpret_cast<float4*>(dbeta + p) = gb;
        *reinterpret_cast<float4*>(dgamma + p) = gg;
    }
}

// Parameter gradients alone (seblas::batchNormParamGrads): one pass over dY and xhat, batch-parallel.
__global__ void __launch_bounds__(256) bn_paramgrad_par_kernel(const float* __restrict__ dY, const float* __restrict__ xhat,
                                                               float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                               int N, long long P) {
    __shared__ float4 red[16][16];
    const long long p = ((long long)blockIdx.x * 16 + threadIdx.x) * 4;
    const bool live = p < P;
    float4 sg = f4_zero(), sb = f4_zero();
    if (live) {
        for (int n = threadIdx.y; n < N; n += 16) {
            const float4 h = *reinterpret_cast<const float4*>(xhat + (long long)n * P + p);
            const float4 d = *reinterpret_cast<const float4*>(dY + (long long)n * P + p);
            sb = f4_add(sb, d);
            sg = f4_add(sg, make_float4(d.x * h.x, d.y * h.y, d.z * h.z, d.w * h.w));
        }
    }
    sg = bn_group_sum(sg, red);
    sb = bn_group_sum(sb, red);
    if (live && threadIdx.y == 0) {
        *reinterpret_cast<float4*>(dgamma + p) = sg;
        *reinterpret_cast<float4*>(dbeta + p) = sb;
    }
}

// Eligibility of the batch-parallel kernels: non-zero when N <= 256 (16 samples per thread at 16 groups).
inline int bn_spt(int N) { return N <= 256 ? 1 : 0; }

// Batch groups per block: 32 when every group still gets two samples, else 16 (measured on the ResNet-56 step at
// batch 128 / 64 / 16: 32 groups beat 16 and 64 on every map size once N >= 64); then the samples per thread, the
// smallest power of two >= ceil(N / groups).
struct BnShape { int groups, spt; unsigned grid; };
inline BnShape bn_shape(const cb_ctx* ctx, int N, long long P) {
    static const int forced = [] {
        const char* e = std::getenv("CB_BN_GROUPS");  // development override: 16, 32 or 64
        return e ? std::atoi(e) : 0;
    }();
    int G = N >= 64 ? 32 : 16;
    static const int small64 = [] {
        const char* e = std::getenv("CB_BN_SMALL64");  // development switch, default on
        return e ? std::atoi(e) : 1;
    }();
    if (small64 && G == 32 && N >= 128 && (P / 4 + 7) / 8 < ctx->sm_count) G = 64;  // maps too small to fill the GPU at 32
    if (forced == 16 || forced == 32 || forced == 64) G = forced;
    const int need = (N + G - 1) / G;
    int spt = 1;
    while (spt < need) spt <<= 1;
    const int pb = 256 / G;
    return BnShape{G, spt, (unsigned)((P / 4 + pb - 1) / pb)};
}

#define BN_DISPATCH(shape, KERNEL, ...)                                                                        \
    do {                                                                                                       \
        const dim3 blk_((unsigned)(256 / (shape).groups), (unsigned)(shape).groups);                            \
        switch ((shape).groups * 100 + (shape).spt) {                                                          \
            case 1601: launch_dep(ctx, KERNEL<1, 16>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;        \
            case 1602: launch_dep(ctx, KERNEL<2, 16>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;        \
            case 1604: launch_dep(ctx, KERNEL<4, 16>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;        \
            case 1608: launch_dep(ctx, KERNEL<8, 16>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;        \
            case 1616: launch_dep(ctx, KERNEL<16, 16>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;       \
            case 3201: launch_dep(ctx, KERNEL<1, 32>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;        \
            case 3202: launch_dep(ctx, KERNEL<2, 32>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;        \
            case 3204: launch_dep(ctx, KERNEL<4, 32>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;        \
            case 3208: launch_dep(ctx, KERNEL<8, 32>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;        \
            case 6401: launch_dep(ctx, KERNEL<1, 64>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;        \
            case 6402: launch_dep(ctx, KERNEL<2, 64>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;        \
            default: launch_dep(ctx, KERNEL<4, 64>, dim3((shape).grid), blk_, 0, __VA_ARGS__); break;          \
        }                                                                                                      \
    } while (0)

void launch_bn_fwd_par(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, float* mean, float* var, float* Y,
                       float* xhat, const float* res, int N, long long P, int relu, long long xs = 0) {
    const BnShape sh = bn_shape(ctx, N, P);
    if (xs == 0) xs = P;
    BN_DISPATCH(sh, bn_fwd_par_kernel, X, beta, gamma, mean, var, Y, xhat, res, N, P, relu, xs);
}
void launch_bn_bwd_par(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, float* dgamma,
                       float* dbeta, const float* relu_out, float* dres, int dres_add, int pg_add, int N, long long P,
                       long long xs = 0, long long dxs = 0, int dx_add = 0) {
    const BnShape sh = bn_shape(ctx, N, P);
    if (xs == 0) xs = P;
    if (dxs == 0) dxs = P;
    BN_DISPATCH(sh, bn_bwd_par_kernel, dY, gamma, X, dX, dgamma, dbeta, relu_out, dres, dres_add, pg_add, N, P, xs, dxs, dx_add);
}

// ------------------------------------------------------------------ elementwise
enum { OP_RELU, OP_RELU_GRAD, OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_ADDS, OP_SUBS, OP_MULS, OP_DIVS, OP_FILL,
       OP_ADD_ZERO_B, OP_ADD_RELU };

template <int OP>
__device__ __forceinline__ float ew(float a, float b, float c, float s) {
    switch (OP) {
        case OP_RELU: return fmaxf(a, 0.f);
        case OP_RELU_GRAD: return a > 0.f ? b : 0.f;
        case OP_ADD: case OP_ADD_ZERO_B: return a + b;
        case OP_ADD_RELU: return fmaxf(a + b, 0.f);
        case OP_SUB: return a - b;
        case OP_MUL: return a * b;
        case OP_DIV: return a / b;
        case OP_ADDS: return a + s;
        case OP_SUBS: return a - s;
        case OP_MULS: return a * s;
        case OP_DIVS: return a / s;
        default: return s;
    }
}

// out[i] = f(a[i], b[i], s). OP_ADD_ZERO_B additionally clears b (gradient hand-over in the backward pass).
template <int OP, bool VEC>
__global__ void eltwise_kernel(const float* __restrict__ a, float* __restrict__ b, float* __restrict__ out, float s,
                               long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (VEC) {
        const long long nv = n >> 2;
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += stride) {
            float4 x = a ? reinterpret_cast<const float4*>(a)[i] : make_float4(0, 0, 0, 0);
            float4 y = b ? reinterpret_cast<const float4*>(b)[i] : make_float4(0, 0, 0, 0);
            float4 r;
            r.x = ew<OP>(x.x, y.x, 0, s); r.y = ew<OP>(x.y, y.y, 0, s);
            r.z = ew<OP>(x.z, y.z, 0, s); r.w = ew<OP>(x.w, y.w, 0, s);
            reinterpret_cast<float4*>(out)[i] = r;
            if (OP == OP_ADD_ZERO_B) reinterpret_cast<float4*>(b)[i] = make_float4(0, 0, 0, 0);
        }
    } else {
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
            const float x = a ? a[i] : 0.f, y = b ? b[i] : 0.f;
            out[i] = ew<OP>(x, y, 0, s);
            if (OP == OP_ADD_ZERO_B) b[i] = 0.f;
        }
    }
}

template <int OP>
int launch_eltwise(cb_ctx* ctx, const float* a, float* b, float* out, float s, long long n, const char* what) {
    if (n == 0) return CB_OK;
    const bool vec = (n % 4 == 0) && aligned16(a) && aligned16(b) && aligned16(out);
    const int grid = grid_for(ctx, vec ? n / 4 : n);
    if (vec) eltwise_kernel<OP, true><<<grid, kThreads, 0, ctx->stream>>>(a, b, out, s, n);
    else eltwise_kernel<OP, false><<<grid, kThreads, 0, ctx->stream>>>(a, b, out, s, n);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, what);
    ctx->launches += 1;
    return finish(ctx, what);
}

// ------------------------------------------------------------------ pooling
// Non-overlapping rH x rW windows; one thread per output element, consecutive threads -> consecutive ow.
// C / ys: channels per sample and floats between consecutive samples of the pooled tensor (ys == 0: dense)
__global__ void avgpool_kernel(const float* __restrict__ X, float* __restrict__ Y, long long total, int H, int W,
                               int rH, int rW, int C, long long ys) {
    const int OH = H / rH, OW = W / rW;
    const float inv = 1.0f / (float)(rH * rW);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int ow = (int)(i % OW);
        const long long t = i / OW;
        const int oh = (int)(t % OH);
        const long long c = t / OH;
        const float* src = X + (c * H + (long long)oh * rH) * W + (long long)ow * rW;
        float s = 0.f;
        for (int a = 0; a < rH; ++a)
            for (int b = 0; b < rW; ++b) s += src[a * W + b];
        long long o = i;
        if (ys) {
            const long long n = c / C;
            o = n * ys + ((c - n * C) * OH + oh) * (long long)OW + ow;
        }
        Y[o] = s * inv;
    }
}
// One thread per INPUT element: every dX element of a covered window gets dY / (rH*rW), the rest zero.
__global__ void avgpool_back_kernel(float* __restrict__ dX, const float* __restrict__ dY, long long total, int H,
                                    int W, int rH, int rW, int C, long long ys) {
    const int OH = H / rH, OW = W / rW;
    const float inv = 1.0f / (float)(rH * rW);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int w = (int)(i % W);
        const long long t = i / W;
        const int h = (int)(t % H);
        const long long c = t / H;
        const int oh = h / rH, ow = w / rW;
        long long o = (c * OH + oh) * OW + ow;
        if (ys) {
            const long long n = c / C;
            o = n * ys + ((c - n * C) * OH + oh) * (long long)OW + ow;
        }
        dX[i] = (oh < OH && ow < OW) ? dY[o] * inv : 0.f;
    }
}
// Global average pool: one warp per (n,c) plane.
__global__ void gap_kernel(const float* __restrict__ X, float* __restrict__ Y, long long planes, int HW) {
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long pl = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; pl < planes; pl += warps) {
        const float* src = X + pl * HW;
        float s = 0.f;
        for (int i = lane; i < HW; i += 32) s += src[i];
        s = warp_sum(s);
        if (lane == 0) Y[pl] = s / (float)HW;
    }
}
__global__ void gap_back_kernel(float* __restrict__ dX, const float* __restrict__ dY, long long total, int HW) {
    const float inv = 1.0f / (float)HW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        dX[i] = dY[i / HW] * inv;
}

// ------------------------------------------------------------------ softmax / cross entropy
// One warp per row of `step` elements: y = exp(x - max) / (sum + 1e-10).
__global__ void softmax_kernel(const float* __restrict__ X, float* __restrict__ Y, int rows, int step) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const float* x = X + (long long)r * step;
        float mx = -1e15f;
        for (int i = lane; i < step; i += 32) mx = fmaxf(mx, x[i]);
        mx = warp_max(mx);
        float s = 0.f;
        for (int i = lane; i < step; i += 32) s += expf(x[i] - mx);
        s = warp_sum(s);
        const float inv = 1.0f / (s + 1e-10f);
        for (int i = lane; i < step; i += 32) Y[(long long)r * step + i] = expf(x[i] - mx) * inv;
    }
}
// dY = Y - labels and loss += sum(-log(Y + 1e-10) * labels); one atomic per block.
__global__ void cross_entropy_kernel(const float* __restrict__ Y, const float* __restrict__ labels,
                                     float* __restrict__ dY, float* __restrict__ loss, long long n) {
    __shared__ float part[kThreads / 32];
    float s = 0.f;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const float y = Y[i], l = labels[i];
        if (dY) dY[i] = y - l;
        s += -logf(y + 1e-10f) * l;
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < kThreads / 32 ? part[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0 && loss) atomicAdd(loss, v);
    }
}

// ------------------------------------------------------------------ bias
__global__ void bias_add_kernel(float* __restrict__ Y, const float* __restrict__ bias, long long total, int C,
                                int HW) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        Y[i] += bias[(i / HW) % C];
}
// db[c] (+)= sum over (n, hw) of dY[n,c,hw]; one block per channel.
__global__ void bias_grad_kernel(const float* __restrict__ dY, float* __restrict__ db, int N, int C, int HW,
                                 int accumulate) {
    __shared__ float part[kThreads / 32];
    const int c = blockIdx.x;
    float s = 0.f;
    const long long per = (long long)N * HW;
    for (long long i = threadIdx.x; i < per; i += blockDim.x) {
        const long long n = i / HW, r = i - n * HW;
        s += dY[(n * C + c) * HW + r];
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < kThreads / 32 ? part[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) db[c] = accumulate ? db[c] + v : v;
    }
}

// ------------------------------------------------------------------ Momentum-SGD over many tensors in one launch
struct MomentumTensor {
    float* w; float* g; float* m;
    long long n;
    int is_weight;
};
// blockIdx.y = tensor. w *= (1 - l2) for weight tensors, m = beta m + (1 - beta) g, w -= lr m, g = 0.
__global__ void momentum_multi_kernel(const MomentumTensor* __restrict__ ts, float lr, float beta, float l2) {
    griddep_wait();
    griddep_launch();
    const MomentumTensor t = ts[blockIdx.y];
    const float decay = t.is_weight ? (1.0f - l2) : 1.0f;
    const float omb = 1.0f - beta;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const bool vec = (t.n % 4 == 0) && (((uintptr_t)t.w | (uintptr_t)t.g | (uintptr_t)t.m) & 15u) == 0;
    if (vec) {
        const long long nv = t.n >> 2;
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += stride) {
            float4 w = reinterpret_cast<float4*>(t.w)[i];
            const float4 g = reinterpret_cast<float4*>(t.g)[i];
            float4 m = reinterpret_cast<float4*>(t.m)[i];
            m.x = beta * m.x + omb * g.x; m.y = beta * m.y + omb * g.y;
            m.z = beta * m.z + omb * g.z; m.w = beta * m.w + omb * g.w;
            w.x = w.x * decay - lr * m.x; w.y = w.y * decay - lr * m.y;
            w.z = w.z * decay - lr * m.z; w.w = w.w * decay - lr * m.w;
            reinterpret_cast<float4*>(t.w)[i] = w;
            reinterpret_cast<float4*>(t.m)[i] = m;
            reinterpret_cast<float4*>(t.g)[i] = make_float4(0, 0, 0, 0);
        }
    } else {
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < t.n; i += stride) {
            const float m = beta * t.m[i] + omb * t.g[i];
            t.w[i] = t.w[i] * decay - lr * m;
            t.m[i] = m;
            t.g[i] = 0.f;
        }
    }
}

// dA[i] = dB[i] = (Y[i] > 0 ? dY[i] : 0): the gradient of out = relu(a + b) for both addends (dB may be null)
__global__ void relu_grad2_kernel(const float* __restrict__ Y, const float* __restrict__ dY, float* __restrict__ dA,
                                  float* __restrict__ dB, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float g = Y[i] > 0.f ? dY[i] : 0.f;
        dA[i] = g;
        if (dB) dB[i] = g;
    }
}

// dst[n][c][hw] += src[n][c0 + c][hw]: one channel slice of a concatenated gradient added into its source's buffer
__global__ void slice_add_kernel(float* __restrict__ dst, const float* __restrict__ src, long long total, long long per_n,
                                 long long src_per_n, long long src_off) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / per_n, r = i - n * per_n;
        dst[i] += src[n * src_per_n + src_off + r];
    }
}

// ------------------------------------------------------------------ classifier head in one kernel per direction
// Forward, one CTA per sample: global average pooling over the H*W plane of every channel, the dense layer
// logits = W pooled + b, the softmax y = exp(x - max) / (sum + 1e-10), the loss gradient y - label and the sample's
// loss -sum(log(y + 1e-10) * label): what GlobalAvgPool, Linear, Softmax and the cross-entropy pair do in four launches.
__global__ void __launch_bounds__(256) head_fwd_kernel(const float* __restrict__ X, const float* __restrict__ W,
                                                       const float* __restrict__ b, const float* __restrict__ labels,
                                                       float* __restrict__ pooled, float* __restrict__ logits,
                                                       float* __restrict__ probs, float* __restrict__ dlogits,
                                                       float* __restrict__ loss_n, int C, int HW, int M) {
    griddep_wait();
    griddep_launch();
    extern __shared__ float sh[];  // pooled[C], then logits[32]
    float* shl = sh + C;
    const int n = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* Xn = X + (long long)n * C * HW;
    // pooling: a warp takes four channels at a time so that their loads are in flight together; each channel is summed
    // lane-strided, then across the lanes
    for (int c0 = warp * 4; c0 < C; c0 += 32) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        for (int i = lane; i < HW; i += 32) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c0 + j < C) s[j] += Xn[(long long)(c0 + j) * HW + i];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float t = warp_sum(s[j]);
            if (lane == 0 && c0 + j < C) {
                sh[c0 + j] = t / (float)HW;
                pooled[(long long)n * C + c0 + j] = sh[c0 + j];
            }
        }
    }
    __syncthreads();
    // logits: one warp per class, lanes stride the channels (coalesced weight rows), summed across the lanes
    for (int m = warp; m < M; m += 8) {
        float a = 0.f;
        for (int c = lane; c < C; c += 32) a = fmaf(W[(long long)m * C + c], sh[c], a);
        a = warp_sum(a);
        if (lane == 0) shl[m] = a + (b ? b[m] : 0.f);
    }
    __syncthreads();
    if (warp != 0) return;
    float logit = -1e15f;
    if (lane < M) {
        logit = shl[lane];
        logits[(long long)n * M + lane] = logit;
    }
    const float mx = warp_max(logit);
    const float e = lane < M ? expf(logit - mx) : 0.f;
    const float sum = warp_sum(e);
    const float y = e * (1.0f / (sum + 1e-10f));
    float l = 0.f;
    if (lane < M) {
        const float lab = labels[(long long)n * M + lane];
        probs[(long long)n * M + lane] = y;
        dlogits[(long long)n * M + lane] = y - lab;
        l = -logf(y + 1e-10f) * lab;
    }
    l = warp_sum(l);
    if (lane == 0) loss_n[n] = l;
}

// Backward. CTA n < N: dX[n][c][:] = (sum_m W[m][c] dlogits[n][m]) / HW (dense-layer data gradient and the pooling
// gradient). The next ceil(M C / 256) CTAs: dW[m][c] += sum_n dlogits[n][m] pooled[n][c], one output per thread. The
// last CTA: db[m] += sum_n dlogits[n][m] and the batch's summed loss. Every sum runs in sample order (deterministic).
__global__ void __launch_bounds__(256) head_bwd_kernel(const float* __restrict__ dlogits, const float* __restrict__ pooled,
                                                       const float* __restrict__ W, float* __restrict__ dX,
                                                       float* __restrict__ dW, float* __restrict__ db,
                                                       const float* __restrict__ loss_n, float* __restrict__ loss_sum, int N,
                                                       int C, int HW, int M) {
    griddep_wait();
    griddep_launch();
    extern __shared__ float sh[];  // dpooled[C]
    const int n = blockIdx.x;
    if (n < N) {
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            float a = 0.f;
            for (int m = 0; m < M; ++m) a = fmaf(W[(long long)m * C + c], dlogits[(long long)n * M + m], a);
            sh[c] = a / (float)HW;
        }
        __syncthreads();
        float* out = dX + (long long)n * C * HW;
        for (int i = threadIdx.x; i < C * HW; i += blockDim.x) out[i] = sh[i / HW];
        return;
    }
    const int w_ctas = (M * C + 255) / 256;
    if (n < N + w_ctas) {
        const int i = (n - N) * 256 + (int)threadIdx.x;
        if (i >= M * C) return;
        const int m = i / C, c = i - m * C;
        float a = 0.f;
        int k = 0;
        for (; k + 8 <= N; k += 8) {  // eight samples' loads in flight, added in sample order
            float d[8], q[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                d[u] = dlogits[(long long)(k + u) * M + m];
                q[u] = pooled[(long long)(k + u) * C + c];
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) a = fmaf(d[u], q[u], a);
        }
        for (; k < N; ++k) a = fmaf(dlogits[(long long)k * M + m], pooled[(long long)k * C + c], a);
        dW[i] += a;
        return;
    }
    if (db && (int)threadIdx.x < M) {
        const int m = threadIdx.x;
        float a = 0.f;
        int k = 0;
        for (; k + 8 <= N; k += 8) {
            float d[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) d[u] = dlogits[(long long)(k + u) * M + m];
#pragma unroll
            for (int u = 0; u < 8; ++u) a += d[u];
        }
        for (; k < N; ++k) a += dlogits[(long long)k * M + m];
        db[m] += a;
    }
    if (threadIdx.x == 32 && loss_sum) {
        float a = 0.f;
        int k = 0;
        for (; k + 16 <= N; k += 16) {
            float d[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) d[u] = loss_n[k + u];
#pragma unroll
            for (int u = 0; u < 16; ++u) a += d[u];
        }
        for (; k < N; ++k) a += loss_n[k];
        *loss_sum = a;
    }
}

int done(cb_ctx* ctx, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, what);
    ctx->launches += 1;
    return finish(ctx, what);
}

}  // namespace
}  // namespace cb

using namespace cb;

extern "C" {

int cb_bn_fwd(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, float* mean, float* var, float* Y,
              float* xhat, int N, long long P) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (N < 0 || P < 0) return fail(ctx, CB_EINVAL, "cb_bn_fwd: negative extent");
    if (N == 0 || P == 0) return CB_OK;
    if (!X || !beta || !gamma || !Y) return fail(ctx, CB_EINVAL, "cb_bn_fwd: null operand");
    const bool vec = (P % 4 == 0) && aligned16(X) && aligned16(Y) && (!xhat || aligned16(xhat));
    const int spt = bn_spt(N);
    if (vec && spt > 0 && aligned16(beta) && aligned16(gamma) && (!mean || aligned16(mean)) && (!var || aligned16(var))) {
        launch_bn_fwd_par(ctx, X, beta, gamma, mean, var, Y, xhat, nullptr, N, P, 0);
        return done(ctx, "cb_bn_fwd");
    }
    if (vec) bn_fwd_kernel<4><<<grid_for(ctx, P / 4, 128), 128, 0, ctx->stream>>>(X, beta, gamma, mean, var, Y, xhat, N, P);
    else bn_fwd_kernel<1><<<grid_for(ctx, P, 128), 128, 0, ctx->stream>>>(X, beta, gamma, mean, var, Y, xhat, N, P);
    return done(ctx, "cb_bn_fwd");
}

int cb_bn_bwd(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, int N, long long P) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (N < 0 || P < 0) return fail(ctx, CB_EINVAL, "cb_bn_bwd: negative extent");
    if (N == 0 || P == 0) return CB_OK;
    if (!dY || !gamma || !X || !dX) return fail(ctx, CB_EINVAL, "cb_bn_bwd: null operand");
    const bool vec = (P % 4 == 0) && aligned16(X) && aligned16(dY) && aligned16(dX);
    const int spt = bn_spt(N);
    if (vec && spt > 0 && aligned16(gamma)) {
        launch_bn_bwd_par(ctx, dY, gamma, X, dX, nullptr, nullptr, nullptr, nullptr, 0, 0, N, P);
        return done(ctx, "cb_bn_bwd");
    }
    if (vec) bn_bwd_kernel<4><<<grid_for(ctx, P / 4, 128), 128, 0, ctx->stream>>>(dY, gamma, X, dX, N, P);
    else bn_bwd_kernel<1><<<grid_for(ctx, P, 128), 128, 0, ctx->stream>>>(dY, gamma, X, dX, N, P);
    return done(ctx, "cb_bn_bwd");
}

int cb_bn_paramgrad(cb_ctx* ctx, const float* dY, const float* xhat, float* dgamma, float* dbeta, int N, long long P) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (N < 0 || P < 0) return fail(ctx, CB_EINVAL, "cb_bn_paramgrad: negative extent");
    if (P == 0) return CB_OK;
    if (!dY || !xhat || !dgamma || !dbeta) return fail(ctx, CB_EINVAL, "cb_bn_paramgrad: null operand");
    const bool vec = (P % 4 == 0) && aligned16(xhat) && aligned16(dY);
    if (vec && aligned16(dgamma) && aligned16(dbeta)) {
        bn_paramgrad_par_kernel<<<(unsigned)((P / 4 + 15) / 16), dim3(16, 16), 0, ctx->stream>>>(dY, xhat, dgamma, dbeta, N, P);
        return done(ctx, "cb_bn_paramgrad");
    }
    if (vec) bn_paramgrad_kernel<4><<<grid_for(ctx, P / 4, 128), 128, 0, ctx->stream>>>(dY, xhat, dgamma, dbeta, N, P);
    else bn_paramgrad_kernel<1><<<grid_for(ctx, P, 128), 128, 0, ctx->stream>>>(dY, xhat, dgamma, dbeta, N, P);
    return done(ctx, "cb_bn_paramgrad");
}

static int bn_bwd_fused_impl(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, float* dgamma,
                             float* dbeta, const float* relu_out, float* dres, int dres_add, int pg_add, int N, long long P,
                             long long xs = 0, long long dxs = 0, int dx_add = 0) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (N < 0 || P < 0) return fail(ctx, CB_EINVAL, "cb_bn_bwd_fused: negative extent");
    if (N == 0 || P == 0) return CB_OK;
    if (!dY || !gamma || !X || !dX || !dgamma || !dbeta) return fail(ctx, CB_EINVAL, "cb_bn_bwd_fused: null operand");
    const int spt = bn_spt(N);
    const bool ok = (P % 4 == 0) && spt > 0 && aligned16(X) && aligned16(dY) && aligned16(dX) && aligned16(gamma) &&
                    aligned16(dgamma) && aligned16(dbeta) && (!relu_out || aligned16(relu_out)) && (!dres || aligned16(dres));
    if (!ok) return fail(ctx, CB_EUNSUPPORTED, "cb_bn_bwd_fused: needs N <= 256, P % 4 == 0 and 16-byte aligned tensors");
    if ((xs && (xs < P || (xs & 3))) || (dxs && (dxs < P || (dxs & 3))))
        return fail(ctx, CB_EINVAL, "cb_bn_bwd_fused: a batch stride must be at least P and a multiple of 4 floats");
    launch_bn_bwd_par(ctx, dY, gamma, X, dX, dgamma, dbeta, relu_out, dres, dres_add, pg_add, N, P, xs, dxs, dx_add);
    return done(ctx, "cb_bn_bwd_fused");
}
int cb_bn_bwd_fused_ex(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, float* dgamma,
                       float* dbeta, const float* relu_out, int N, long long P, long long x_batch_stride,
                       long long dx_batch_stride, int accumulate_dx) {
    return bn_bwd_fused_impl(ctx, dY, gamma, X, dX, dgamma, dbeta, relu_out, nullptr, 0, 0, N, P, x_batch_stride, dx_batch_stride,
                             accumulate_dx ? 1 : 0);
}
int cb_bn_bwd_fused(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, float* dgamma,
                    float* dbeta, const float* relu_out, int N, long long P) {
    return bn_bwd_fused_impl(ctx, dY, gamma, X, dX, dgamma, dbeta, relu_out, nullptr, 0, 0, N, P);
}
int cb_bn_bwd_fused_res(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, float* dgamma,
                        float* dbeta, const float* relu_out, float* dR, int accumulate_dR, int N, long long P) {
    if (ctx && (!relu_out || !dR)) return fail(ctx, CB_EINVAL, "cb_bn_bwd_fused_res: null ReLU output or shortcut gradient");
    return bn_bwd_fused_impl(ctx, dY, gamma, X, dX, dgamma, dbeta, relu_out, dR, accumulate_dR ? 1 : 0, 0, N, P);
}
}  // extern "C"

extern "C" {
static int bn_fwd_relu_impl(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, const float* R, float* Y, int N,
                            long long P, long long xs = 0);
}

namespace cb {
// One group of a batch whose BatchNorm statistics are taken per group of samples (the executor's model of per-GPU
// statistics in data-parallel training): the group's slices of the tensors, parameter gradients added onto what the
// earlier groups left when `add_param_grads`.
int bn_bwd_group(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, float* dgamma, float* dbeta,
                 const float* relu_out, float* dR, int accumulate_dR, int add_param_grads, int N, long long P) {
    return bn_bwd_fused_impl(ctx, dY, gamma, X, dX, dgamma, dbeta, relu_out, dR, accumulate_dR, add_param_grads, N, P);
}
int bn_fwd_group(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, const float* R, float* Y, int relu, int N,
                 long long P) {
    if (relu) return bn_fwd_relu_impl(ctx, X, beta, gamma, R, Y, N, P);
    return cb_bn_fwd(ctx, X, beta, gamma, nullptr, nullptr, Y, nullptr, N, P);
}
}  // namespace cb

extern "C" {

static int bn_fwd_relu_impl(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, const float* R, float* Y, int N,
                            long long P, long long xs) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (N < 0 || P < 0) return fail(ctx, CB_EINVAL, "cb_bn_fwd_relu: negative extent");
    if (N == 0 || P == 0) return CB_OK;
    if (!X || !beta || !gamma || !Y) return fail(ctx, CB_EINVAL, "cb_bn_fwd_relu: null operand");
    const int spt = bn_spt(N);
    if (!((P % 4 == 0) && spt > 0 && aligned16(X) && aligned16(Y) && aligned16(beta) && aligned16(gamma) && (!R || aligned16(R))))
        return fail(ctx, CB_EUNSUPPORTED, "cb_bn_fwd_relu: needs N <= 256, P % 4 == 0 and 16-byte aligned tensors");
    if (xs && (xs < P || (xs & 3))) return fail(ctx, CB_EINVAL, "cb_bn_fwd_relu: the batch stride must be at least P and a multiple of 4 floats");
    launch_bn_fwd_par(ctx, X, beta, gamma, nullptr, nullptr, Y, nullptr, R, N, P, 1, xs);
    return done(ctx, "cb_bn_fwd_relu");
}
int cb_bn_fwd_relu_ex(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, float* Y, int N, long long P,
                      long long x_batch_stride) {
    return bn_fwd_relu_impl(ctx, X, beta, gamma, nullptr, Y, N, P, x_batch_stride);
}
int cb_bn_fwd_relu(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, float* Y, int N, long long P) {
    return bn_fwd_relu_impl(ctx, X, beta, gamma, nullptr, Y, N, P);
}
int cb_bn_fwd_add_relu(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, const float* R, float* Y, int N,
                       long long P) {
    if (ctx && !R) return fail(ctx, CB_EINVAL, "cb_bn_fwd_add_relu: null addend");
    return bn_fwd_relu_impl(ctx, X, beta, gamma, R, Y, N, P);
}

int cb_add_relu(cb_ctx* ctx, const float* A, const float* B, float* Out, long long n) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (n < 0 || (n > 0 && (!A || !B || !Out))) return fail(ctx, CB_EINVAL, "cb_add_relu: bad argument");
    return launch_eltwise<OP_ADD_RELU>(ctx, A, const_cast<float*>(B), Out, 0.f, n, "cb_add_relu");
}

int cb_relu_grad2(cb_ctx* ctx, const float* Y, const float* dY, float* dA, float* dB, long long n) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (n < 0 || (n > 0 && (!Y || !dY || !dA))) return fail(ctx, CB_EINVAL, "cb_relu_grad2: bad argument");
    if (n == 0) return CB_OK;
    relu_grad2_kernel<<<grid_for(ctx, n), kThreads, 0, ctx->stream>>>(Y, dY, dA, dB, n);
    return done(ctx, "cb_relu_grad2");
}

int cb_relu(cb_ctx* ctx, const float* X, float* Y, long long n) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (n < 0 || (n > 0 && (!X || !Y))) return fail(ctx, CB_EINVAL, "cb_relu: bad argument");
    return launch_eltwise<OP_RELU>(ctx, X, nullptr, Y, 0.f, n, "cb_relu");
}

int cb_relu_grad(cb_ctx* ctx, const float* X, const float* dY, float* dX, long long n) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (n < 0 || (n > 0 && (!X || !dY || !dX))) return fail(ctx, CB_EINVAL, "cb_relu_grad: bad argument");
    return launch_eltwise<OP_RELU_GRAD>(ctx, X, const_cast<float*>(dY), dX, 0.f, n, "cb_relu_grad");
}

int cb_tensor_op(cb_ctx* ctx, int op, float* A, const float* B, float scalar, long long n) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    ctx->filter_version += 1;  // A may be a convolution filter: cached packed copies are stale from here on
    if (n < 0 || (n > 0 && !A)) return fail(ctx, CB_EINVAL, "cb_tensor_op: bad argument");
    if (op >= CB_OP_ADD && op <= CB_OP_DIV && n > 0 && !B) return fail(ctx, CB_EINVAL, "cb_tensor_op: null B");
    float* b = const_cast<float*>(B);
    switch (op) {
        case CB_OP_ADD: return launch_eltwise<OP_ADD>(ctx, A, b, A, 0.f, n, "cb_tensor_op(add)");
        case CB_OP_SUB: return launch_eltwise<OP_SUB>(ctx, A, b, A, 0.f, n, "cb_tensor_op(sub)");
        case CB_OP_MUL: return launch_eltwise<OP_MUL>(ctx, A, b, A, 0.f, n, "cb_tensor_op(mul)");
        case CB_OP_DIV: return launch_eltwise<OP_DIV>(ctx, A, b, A, 0.f, n, "cb_tensor_op(div)");
        case CB_OP_ADD_SCALAR: return launch_eltwise<OP_ADDS>(ctx, A, nullptr, A, scalar, n, "cb_tensor_op(add scalar)");
        case CB_OP_SUB_SCALAR: return launch_eltwise<OP_SUBS>(ctx, A, nullptr, A, scalar, n, "cb_tensor_op(sub scalar)");
        case CB_OP_MUL_SCALAR: return launch_eltwise<OP_MULS>(ctx, A, nullptr, A, scalar, n, "cb_tensor_op(mul scalar)");
        case CB_OP_DIV_SCALAR: return launch_eltwise<OP_DIVS>(ctx, A, nullptr, A, scalar, n, "cb_tensor_op(div scalar)");
        case CB_OP_FILL: return launch_eltwise<OP_FILL>(ctx, nullptr, nullptr, A, scalar, n, "cb_tensor_op(fill)");
        default: return fail(ctx, CB_EINVAL, "cb_tensor_op: unknown op");
    }
}

int cb_grad_handover(cb_ctx* ctx, float* dA, float* dA_reserve, long long n) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (n < 0 || (n > 0 && (!dA || !dA_reserve))) return fail(ctx, CB_EINVAL, "cb_grad_handover: bad argument");
    return launch_eltwise<OP_ADD_ZERO_B>(ctx, dA, dA_reserve, dA, 0.f, n, "cb_grad_handover");
}

int cb_avgpool(cb_ctx* ctx, const float* X, float* Y, long long NC, int H, int W, int rH, int rW) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (NC < 0 || H < 0 || W < 0 || rH < 1 || rW < 1) return fail(ctx, CB_EINVAL, "cb_avgpool: bad extent");
    const long long total = NC * (H / rH) * (W / rW);
    if (total == 0) return CB_OK;
    if (!X || !Y) return fail(ctx, CB_EINVAL, "cb_avgpool: null operand");
    avgpool_kernel<<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>(X, Y, total, H, W, rH, rW, 1, 0);
    return done(ctx, "cb_avgpool");
}

int cb_avgpool_ex(cb_ctx* ctx, const float* X, float* Y, int N, int C, int H, int W, int rH, int rW, long long y_batch_stride) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (N < 0 || C < 1 || H < 0 || W < 0 || rH < 1 || rW < 1) return fail(ctx, CB_EINVAL, "cb_avgpool_ex: bad extent");
    const long long total = (long long)N * C * (H / rH) * (W / rW);
    if (total == 0) return CB_OK;
    if (!X || !Y) return fail(ctx, CB_EINVAL, "cb_avgpool_ex: null operand");
    if (y_batch_stride && y_batch_stride < (long long)C * (H / rH) * (W / rW))
        return fail(ctx, CB_EINVAL, "cb_avgpool_ex: batch stride smaller than one pooled sample");
    avgpool_kernel<<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>(X, Y, total, H, W, rH, rW, C, y_batch_stride);
    return done(ctx, "cb_avgpool_ex");
}

int cb_avgpool_back_ex(cb_ctx* ctx, float* dX, const float* dY, int N, int C, int H, int W, int rH, int rW,
                       long long dy_batch_stride) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (N < 0 || C < 1 || H < 0 || W < 0 || rH < 1 || rW < 1) return fail(ctx, CB_EINVAL, "cb_avgpool_back_ex: bad extent");
    const long long total = (long long)N * C * H * W;
    if (total == 0) return CB_OK;
    if (!dX || !dY) return fail(ctx, CB_EINVAL, "cb_avgpool_back_ex: null operand");
    if (dy_batch_stride && dy_batch_stride < (long long)C * (H / rH) * (W / rW))
        return fail(ctx, CB_EINVAL, "cb_avgpool_back_ex: batch stride smaller than one pooled sample");
    avgpool_back_kernel<<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>(dX, dY, total, H, W, rH, rW, C, dy_batch_stride);
    return done(ctx, "cb_avgpool_back_ex");
}

int cb_avgpool_back(cb_ctx* ctx, float* dX, const float* dY, long long NC, int H, int W, int rH, int rW) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (NC < 0 || H < 0 || W < 0 || rH < 1 || rW < 1) return fail(ctx, CB_EINVAL, "cb_avgpool_back: bad extent");
    const long long total = NC * H * W;
    if (total == 0) return CB_OK;
    if (!dX || !dY) return fail(ctx, CB_EINVAL, "cb_avgpool_back: null operand");
    avgpool_back_kernel<<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>(dX, dY, total, H, W, rH, rW, 1, 0);
    return done(ctx, "cb_avgpool_back");
}

int cb_global_avgpool(cb_ctx* ctx, const float* X, float* Y, long long NC, int HW) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (NC < 0 || HW < 1) return fail(ctx, CB_EINVAL, "cb_global_avgpool: bad extent");
    if (NC == 0) return CB_OK;
    if (!X || !Y) return fail(ctx, CB_EINVAL, "cb_global_avgpool: null operand");
    gap_kernel<<<grid_for(ctx, NC * 32), kThreads, 0, ctx->stream>>>(X, Y, NC, HW);
    return done(ctx, "cb_global_avgpool");
}

int cb_global_avgpool_back(cb_ctx* ctx, float* dX, const float* dY, long long NC, int HW) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (NC < 0 || HW < 1) return fail(ctx, CB_EINVAL, "cb_global_avgpool_back: bad extent");
    if (NC == 0) return CB_OK;
    if (!dX || !dY) return fail(ctx, CB_EINVAL, "cb_global_avgpool_back: null operand");
    gap_back_kernel<<<grid_for(ctx, NC * HW), kThreads, 0, ctx->stream>>>(dX, dY, NC * HW, HW);
    return done(ctx, "cb_global_avgpool_back");
}

int cb_softmax(cb_ctx* ctx, const float* X, float* Y, int rows, int step) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (rows < 0 || step < 1) return fail(ctx, CB_EINVAL, "cb_softmax: bad extent");
    if (rows == 0) return CB_OK;
    if (!X || !Y) return fail(ctx, CB_EINVAL, "cb_softmax: null operand");
    softmax_kernel<<<grid_for(ctx, (long long)rows * 32), kThreads, 0, ctx->stream>>>(X, Y, rows, step);
    return done(ctx, "cb_softmax");
}

int cb_cross_entropy(cb_ctx* ctx, const float* Y, const float* labels, float* dY, float* loss_sum, long long n) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (n < 0) return fail(ctx, CB_EINVAL, "cb_cross_entropy: negative extent");
    if (!Y || !labels) return fail(ctx, CB_EINVAL, "cb_cross_entropy: null operand");
    if (loss_sum) {
        cudaError_t e = cudaMemsetAsync(loss_sum, 0, sizeof(float), ctx->stream);
        if (e != cudaSuccess) return check_cuda(ctx, e, "cb_cross_entropy: clear of the loss word");
    }
    if (n == 0) return CB_OK;
    cross_entropy_kernel<<<grid_for(ctx, n), kThreads, 0, ctx->stream>>>(Y, labels, dY, loss_sum, n);
    return done(ctx, "cb_cross_entropy");
}

int cb_head_fwd(cb_ctx* ctx, const float* X, const float* W, const float* b, const float* labels, float* pooled, float* logits,
                float* probs, float* dlogits, float* loss_per_sample, int N, int C, int HW, int M) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (N < 0 || C < 1 || HW < 1 || M < 1) return fail(ctx, CB_EINVAL, "cb_head_fwd: bad extent");
    if (M > 32 || C > 8192) return fail(ctx, CB_EUNSUPPORTED, "cb_head_fwd: at most 32 classes and 8192 channels");
    if (N == 0) return CB_OK;
    if (!X || !W || !labels || !pooled || !logits || !probs || !dlogits || !loss_per_sample)
        return fail(ctx, CB_EINVAL, "cb_head_fwd: null operand");
    launch_dep(ctx, head_fwd_kernel, dim3((unsigned)N), dim3(256), (size_t)(C + 32) * sizeof(float), X, W, b, labels, pooled, logits, probs,
               dlogits, loss_per_sample, C, HW, M);
    return done(ctx, "cb_head_fwd");
}

int cb_head_bwd(cb_ctx* ctx, const float* dlogits, const float* pooled, const float* W, float* dX, float* dW, float* db,
                const float* loss_per_sample, float* loss_sum, int N, int C, int HW, int M) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (N < 0 || C < 1 || HW < 1 || M < 1) return fail(ctx, CB_EINVAL, "cb_head_bwd: bad extent");
    if (C > 8192) return fail(ctx, CB_EUNSUPPORTED, "cb_head_bwd: at most 8192 channels");
    if (N == 0) return CB_OK;
    if (!dlogits || !pooled || !W || !dX || !dW || (loss_sum && !loss_per_sample)) return fail(ctx, CB_EINVAL, "cb_head_bwd: null operand");
    launch_dep(ctx, head_bwd_kernel, dim3((unsigned)(N + (M * C + 255) / 256 + 1)), dim3(256), (size_t)C * sizeof(float), dlogits, pooled, W, dX, dW, db,
               loss_per_sample, loss_sum, N, C, HW, M);
    return done(ctx, "cb_head_bwd");
}

int cb_conv_bias(cb_ctx* ctx, float* Y, const float* bias, int N, int C, int HW) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (N < 0 || C < 0 || HW < 0) return fail(ctx, CB_EINVAL, "cb_conv_bias: negative extent");
    const long long total = (long long)N * C * HW;
    if (total == 0) return CB_OK;
    if (!Y || !bias) return fail(ctx, CB_EINVAL, "cb_conv_bias: null operand");
    bias_add_kernel<<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>(Y, bias, total, C, HW);
    return done(ctx, "cb_conv_bias");
}

int cb_conv_bias_grad(cb_ctx* ctx, const float* dY, float* db, int N, int C, int HW, int accumulate) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (N < 0 || C < 0 || HW < 0) return fail(ctx, CB_EINVAL, "cb_conv_bias_grad: negative extent");
    if (C == 0) return CB_OK;
    if (!dY || !db) return fail(ctx, CB_EINVAL, "cb_conv_bias_grad: null operand");
    bias_grad_kernel<<<C, kThreads, 0, ctx->stream>>>(dY, db, N, C, HW, accumulate ? 1 : 0);
    return done(ctx, "cb_conv_bias_grad");
}

int cb_concat_channels(cb_ctx* ctx, int count, const float* const* X, const int* channels, float* Y, int N, int HW) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (count < 0 || N < 0 || HW < 0 || (count > 0 && (!X || !channels || !Y))) return fail(ctx, CB_EINVAL, "cb_concat_channels: bad argument");
    long long ctot = 0;
    for (int i = 0; i < count; ++i) {
        if (channels[i] < 0 || (channels[i] > 0 && !X[i])) return fail(ctx, CB_EINVAL, "cb_concat_channels: bad source");
        ctot += channels[i];
    }
    if (N == 0 || HW == 0 || ctot == 0) return CB_OK;
    long long c0 = 0;
    for (int i = 0; i < count; ++i) {
        if (channels[i] == 0) continue;
        const size_t row = (size_t)channels[i] * HW * sizeof(float);
        cudaError_t e = cudaMemcpy2DAsync(Y + c0 * HW, (size_t)ctot * HW * sizeof(float), X[i], row, row, (size_t)N,
                                          cudaMemcpyDeviceToDevice, ctx->stream);
        if (e != cudaSuccess) return check_cuda(ctx, e, "cb_concat_channels");
        c0 += channels[i];
    }
    return finish(ctx, "cb_concat_channels");
}

int cb_concat_grads(cb_ctx* ctx, int count, float* const* dX, const int* channels, const float* dY, int N, int HW) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (count < 0 || N < 0 || HW < 0 || (count > 0 && (!dX || !channels || !dY))) return fail(ctx, CB_EINVAL, "cb_concat_grads: bad argument");
    long long ctot = 0;
    for (int i = 0; i < count; ++i) {
        if (channels[i] < 0 || (channels[i] > 0 && !dX[i])) return fail(ctx, CB_EINVAL, "cb_concat_grads: bad destination");
        ctot += channels[i];
    }
    if (N == 0 || HW == 0 || ctot == 0) return CB_OK;
    long long c0 = 0;
    for (int i = 0; i < count; ++i) {
        if (channels[i] == 0) continue;
        const long long per_n = (long long)channels[i] * HW, total = per_n * N;
        slice_add_kernel<<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>(dX[i], dY, total, per_n, ctot * HW, c0 * HW);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return check_cuda(ctx, e, "cb_concat_grads");
        ctx->launches += 1;
        c0 += channels[i];
    }
    return finish(ctx, "cb_concat_grads");
}

int cb_momentum_multi(cb_ctx* ctx, int ntensors, float* const* w, float* const* g, float* const* m,
                      const long long* sizes, const unsigned char* is_weight, float lr, float beta, float l2) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (ntensors < 0) return fail(ctx, CB_EINVAL, "cb_momentum_multi: negative tensor count");
    ctx->filter_version += 1;  // the updated tensors may be convolution filters: cached packed copies are stale
    if (ntensors == 0) return CB_OK;
    if (!w || !g || !m || !sizes) return fail(ctx, CB_EINVAL, "cb_momentum_multi: null table");
    if (ntensors > 65535) return fail(ctx, CB_EUNSUPPORTED, "cb_momentum_multi: more than 65535 tensors");
    // descriptor table: staged through the context workspace (pinned-free path: small synchronous copy)
    const size_t bytes = sizeof(MomentumTensor) * (size_t)ntensors;
    int rc = ensure_workspace(ctx, bytes);
    if (rc != CB_OK) return rc;
    MomentumTensor* host = new MomentumTensor[ntensors];
    long long biggest = 1;
    for (int i = 0; i < ntensors; ++i) {
        if (sizes[i] < 0 || (sizes[i] > 0 && (!w[i] || !g[i] || !m[i]))) {
            delete[] host;
            return fail(ctx, CB_EINVAL, "cb_momentum_multi: bad tensor entry");
        }
        host[i] = MomentumTensor{w[i], g[i], m[i], sizes[i], is_weight ? (int)is_weight[i] : 0};
        if (sizes[i] > biggest) biggest = sizes[i];
    }
    cudaError_t e = cudaMemcpyAsync(ctx->workspace, host, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);  // host table is freed below
    delete[] host;
    if (e != cudaSuccess) return check_cuda(ctx, e, "cb_momentum_multi: descriptor upload");
    int gx = (int)((biggest / 4 + kThreads - 1) / kThreads);
    if (gx < 1) gx = 1;
    if (gx > 64) gx = 64;
    launch_dep(ctx, momentum_multi_kernel, dim3((unsigned)gx, (unsigned)ntensors), dim3(kThreads), 0,
               static_cast<const MomentumTensor*>(ctx->workspace), lr, beta, l2);
    return done(ctx, "cb_momentum_multi");
}

}  // extern "C"

namespace cb {
// Descriptor table kept on the device by long-lived callers (the training-step executor), so that the update is a
// single kernel launch with no host copy or synchronisation in the step.
int momentum_table_build(cb_ctx* ctx, int ntensors, float* const* w, float* const* g, float* const* m,
                         const long long* sizes, const unsigned char* is_weight, void** dev_table, long long* biggest) {
    std::vector<MomentumTensor> host((size_t)ntensors);
    *biggest = 1;
    for (int i = 0; i < ntensors; ++i) {
        host[i] = MomentumTensor{w[i], g[i], m[i], sizes[i], is_weight ? (int)is_weight[i] : 0};
        if (sizes[i] > *biggest) *biggest = sizes[i];
    }
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, sizeof(MomentumTensor) * (size_t)(ntensors > 0 ? ntensors : 1));
    if (e == cudaSuccess) e = cudaMemcpy(d, host.data(), sizeof(MomentumTensor) * (size_t)ntensors, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return check_cuda(ctx, e, "momentum table upload");
    *dev_table = d;
    return CB_OK;
}
int momentum_table_launch(cb_ctx* ctx, const void* dev_table, int ntensors, long long biggest, float lr, float beta,
                          float l2) {
    if (ntensors <= 0) return CB_OK;
    int gx = (int)((biggest / 4 + kThreads - 1) / kThreads);
    if (gx < 1) gx = 1;
    if (gx > 64) gx = 64;
    launch_dep(ctx, momentum_multi_kernel, dim3((unsigned)gx, (unsigned)ntensors), dim3(kThreads), 0,
               static_cast<const MomentumTensor*>(dev_table), lr, beta, l2);
    int rc = done(ctx, "momentum step");
    if (rc != CB_OK) return rc;
    return filter_cache_repack_all(ctx);  // the filters just changed: one launch re-packs every cached copy
}
}  // namespace cb

extern "C" {

int cb_momentum(cb_ctx* ctx, float* w, float* g, float* m, long long n, float lr, float beta, float l2,
                int is_weight) {
    unsigned char flag = is_weight ? 1 : 0;
    return cb_momentum_multi(ctx, 1, &w, &g, &m, &n, &flag, lr, beta, l2);
}

}  // extern "C"
