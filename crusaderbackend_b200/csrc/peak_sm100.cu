// Measured ceiling of the TF32 tensor pipe: a kernel that does nothing but issue tcgen05.mma on operands that stay
// resident in shared memory (no global traffic, no epilogue), on every SM. What it reaches is the denominator the
// GEMM and convolution kernels are held against: no kernel that also has to feed and drain the tensor core can be
// faster than this loop.
#include <cstdlib>

#include "cb_internal.h"
#include "cb_ptx.cuh"

namespace cb {
namespace {

struct __align__(8) PeakSmem {
    uint64_t done;
    uint32_t tmem_base;
    int abort_flag;
};

// Each CTA: `iters` groups of 4 UMMAs (M = 128, N = n, K = 8 each: one 32-wide k block) onto one accumulator, the
// operands a [128][32] and an [n][32] fp32 tile of shared memory in the layout the flags name (K-major: 128-byte rows,
// 128-byte swizzle; MN-major: 32-row boxes, 32-byte-atom swizzle), contents irrelevant (zeroed).
__global__ void __launch_bounds__(128, 1) umma_peak_kernel(int n, int p_mn, int q_mn, int iters, int* status, int table) {
    __shared__ uint2 tab[4];  // development variant: operand offsets read from shared memory before every UMMA
    extern __shared__ uint8_t smem_raw[];
    __shared__ PeakSmem ps;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t p_bytes = 128u * 32u * 4u, q_bytes = (uint32_t)n * 32u * 4u;
    for (uint32_t v = threadIdx.x; v < (table >= 2 ? 4u : 1u) * (p_bytes + q_bytes) / 16u; v += blockDim.x)
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(base + v * 16u), "r"(0u) : "memory");
    if (threadIdx.x == 0) {
        ps.abort_flag = 0;
        mbar_init(smem_u32(&ps.done), 1);
        mbar_fence_init();
    }
    fence_proxy_async_smem();
    __syncthreads();
    int cols = 32;
    while (cols < n) cols <<= 1;
    if (warp == 0) {
        tmem_alloc(smem_u32(&ps.tmem_base), (uint32_t)cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) {
        if (table == 4) {
            // development variant: the whole warp runs the loop, one elected lane issues; operand set changes per group
            const uint32_t idesc = umma_idesc_tf32(128, (uint32_t)n, p_mn ? 1u : 0u, q_mn ? 1u : 0u);
            const uint64_t dP = p_mn ? umma_smem_desc(base, 4096u, 512u, UMMA_SW_128B_BASE32B)
                                     : umma_smem_desc(base, 16u, 1024u, UMMA_SW_128B);
            const uint64_t dQ = q_mn ? umma_smem_desc(base + p_bytes, 4096u, 512u, UMMA_SW_128B_BASE32B)
                                     : umma_smem_desc(base + p_bytes, 16u, 1024u, UMMA_SW_128B);
            const uint64_t stepP = p_mn ? (1024u >> 4) : (32u >> 4), stepQ = q_mn ? (1024u >> 4) : (32u >> 4);
            const uint32_t d = ps.tmem_base;
            const uint32_t set_units = (p_bytes + q_bytes) >> 4;
            for (int it = 0; it < iters; ++it) {
                const uint64_t o = (uint64_t)((uint32_t)(it & 3) * set_units);
                umma_tf32_elect(d, dP + o, dQ + o, idesc, it ? 1u : 0u);
                umma_tf32_elect(d, dP + o + stepP, dQ + o + stepQ, idesc, 1u);
                umma_tf32_elect(d, dP + o + 2 * stepP, dQ + o + 2 * stepQ, idesc, 1u);
                umma_tf32_elect(d, dP + o + 3 * stepP, dQ + o + 3 * stepQ, idesc, 1u);
            }
            if (lane == 0) {
                tc_commit(smem_u32(&ps.done));
                mbar_wait(smem_u32(&ps.done), 0, &ps.abort_flag, status, CBK_TIMEOUT_TMEM_FULL);
            }
        } else if (lane == 0) {
            const uint32_t idesc = umma_idesc_tf32(128, (uint32_t)n, p_mn ? 1u : 0u, q_mn ? 1u : 0u);
            const uint64_t dP = p_mn ? umma_smem_desc(base, 4096u, 512u, UMMA_SW_128B_BASE32B)
                                     : umma_smem_desc(base, 16u, 1024u, UMMA_SW_128B);
            const uint64_t dQ = q_mn ? umma_smem_desc(base + p_bytes, 4096u, 512u, UMMA_SW_128B_BASE32B)
                                     : umma_smem_desc(base + p_bytes, 16u, 1024u, UMMA_SW_128B);
            const uint64_t stepP = p_mn ? (1024u >> 4) : (32u >> 4), stepQ = q_mn ? (1024u >> 4) : (32u >> 4);
            const uint32_t d = ps.tmem_base;
            if (table) {
                for (int k = 0; k < 4; ++k) tab[k] = make_uint2((uint32_t)(k * stepP), (uint32_t)(k * stepQ));
                for (int it = 0; it < iters; ++it) {
#pragma unroll 2
                    for (int k = 0; k < 4; ++k) {
                        uint2 off;
                        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(off.x), "=r"(off.y) : "r"(smem_u32(&tab[k])));
                        umma_tf32(d, dP + off.x, dQ + off.y, idesc, (it | k) ? 1u : 0u);
                    }
                }
            } else if (table >= 2) {
                // development variant: every group of four UMMAs reads another of four operand sets (as a pipeline's
                // stages would), all zero-filled
                const uint32_t set_units = table == 2 ? (p_bytes + q_bytes) >> 4 : 0u;  // 3: same addresses, still computed per group
                for (int it = 0; it < iters; ++it) {
                    const uint64_t o = (uint64_t)((uint32_t)(it & 3) * set_units);
                    umma_tf32(d, dP + o, dQ + o, idesc, it ? 1u : 0u);
                    umma_tf32(d, dP + o + stepP, dQ + o + stepQ, idesc, 1u);
                    umma_tf32(d, dP + o + 2 * stepP, dQ + o + 2 * stepQ, idesc, 1u);
                    umma_tf32(d, dP + o + 3 * stepP, dQ + o + 3 * stepQ, idesc, 1u);
                }
            } else
            for (int it = 0; it < iters; ++it) {
                umma_tf32(d, dP, dQ, idesc, it ? 1u : 0u);
                umma_tf32(d, dP + stepP, dQ + stepQ, idesc, 1u);
                umma_tf32(d, dP + 2 * stepP, dQ + 2 * stepQ, idesc, 1u);
                umma_tf32(d, dP + 3 * stepP, dQ + 3 * stepQ, idesc, 1u);
            }
            tc_commit(smem_u32(&ps.done));
            mbar_wait(smem_u32(&ps.done), 0, &ps.abort_flag, status, CBK_TIMEOUT_TMEM_FULL);
        }
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(ps.tmem_base, (uint32_t)cols);
    }
}

}  // namespace
}  // namespace cb

using namespace cb;

extern "C" int cb_measure_umma_peak(cb_ctx* ctx, int n, int p_mn, int q_mn, int iters, float* tflops) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (!tflops || iters < 1 || n < 16 || n > 256 || (n & 15)) return fail(ctx, CB_EINVAL, "cb_measure_umma_peak: n must be a multiple of 16 in 16..256");
    if ((p_mn || q_mn) && (n & 31)) return fail(ctx, CB_EINVAL, "cb_measure_umma_peak: MN-major operands come in 32-row boxes");
    const size_t smem = 4 * (128 * 128 + (size_t)n * 128) + 1024;
    cudaError_t e = cudaFuncSetAttribute(umma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return check_cuda(ctx, e, "umma_peak_kernel attribute");
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    static const int table = [] { const char* e = std::getenv("CB_PEAK_TABLE"); return e ? std::atoi(e) : 0; }();  // development variant
    umma_peak_kernel<<<ctx->sm_count, 128, smem, ctx->stream>>>(n, p_mn, q_mn, iters / 8 + 1, ctx->d_status, table);  // warm-up
    cudaEventRecord(e0, ctx->stream);
    umma_peak_kernel<<<ctx->sm_count, 128, smem, ctx->stream>>>(n, p_mn, q_mn, iters, ctx->d_status, table);
    cudaEventRecord(e1, ctx->stream);
    e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess) return check_cuda(ctx, e, "cb_measure_umma_peak");
    ctx->launches += 2;
    const double flops = 2.0 * 128.0 * n * 32.0 * (double)iters * ctx->sm_count;
    *tflops = (float)(flops / (ms * 1e-3) / 1e12);
    return cb_synchronize(ctx);
}
