// Tensor-core implicit-GEMM convolution for sm_100a (TF32 mode), NCHW fp32, no materialised im2col.
//
// Forward and data-gradient run the same kernel: D[pixel][oc] = sum over (tap, c) of In[n, c, oh+fh-pH, ow+fw-pW]
// * Wp[tap][oc][c]. The 128 TMEM lanes of an accumulator are 128 output pixels (UMMA M), the columns are the output
// channels (UMMA N = OC rounded up to 16), K walks 8 input channels of one filter tap per tcgen05.mma.
//
//  * Pixels are grouped in "lines" of 32 consecutive floats of one channel plane (32/W image rows of a W-wide map,
//    W in {8,16,32}); a CTA tile is 4 lines. For each filter row fh and line, one TMA box (W, 32/W rows, 8 channels)
//    of the NCHW input lands as an [8 channels][128 bytes] block — exactly the MN-major operand layout the tensor
//    core reads (128-byte swizzle with 32-byte atoms). Rows above / below the image are out of bounds for the
//    tensor map and arrive as zeros, which is the vertical padding.
//  * A TMA box may not start at an odd column (its innermost coordinate must be 16-byte aligned), so the
//    horizontal taps cannot be fetched as shifted boxes. Four "shift" warps build the fw = 0 and fw = 2 copies of
//    every block in shared memory from the centre copy (a register rotate by one float per 128-byte row, with
//    zeros entering at the row edges = the horizontal padding) and hand them to the MMA warp through an mbarrier.
//  * The filter is packed once per call into [tap][32-channel group][oc][32 channels] (K-major rows of 128 bytes,
//    zero padded) in the context workspace and stays resident in shared memory for the whole persistent CTA.
//    For the data gradient the pack transposes the channel roles and rotates the filter by 180 degrees
//    (seblas/operations/cuConv.cu:321-326 does the same rotation on the fly).
//  * Epilogue: tcgen05.ld, + bias, ReLU, and stores in which the 32 lanes of a warp write 128 contiguous bytes.
//
// Covered geometry: stride 1, filter 1x1 (pad 0) or 3x3 (pad 1) per axis, W in {8,16,32}, (32/W) | H,
// OC <= 256, packed filter <= ~150 KB. Everything else is served by the CUDA-core kernels in conv_simt.cu.
#include "cb_internal.h"
#include "cb_ptx.cuh"

namespace cb {
namespace {

constexpr int kCB = 8;          // input channels per pipeline stage (= one UMMA K step per tap)
constexpr int kMaxStages = 6;
constexpr int kRowBytes = 128;  // one line of 32 floats

struct ConvParams {
    int N, Cin, H, W, Cout;   // "input" and "output" of this pass (forward: X -> Y, dgrad: dY -> dX)
    int FH, FW, pH;           // vertical taps, horizontal taps, vertical padding
    int OCp;                  // Cout rounded up to 16 (UMMA N)
    int CG;                   // 32-channel groups of the packed filter
    int NCB;                  // ceil(Cin / 8) pipeline stages per tile
    int L;                    // image rows per line (32 / W)
    int LPI;                  // lines per image (H / L)
    long long total_lines;    // N * LPI
    int tiles;                // ceil(total_lines / 4)
    int stages;
    int tmem_cols;
    uint32_t w_bytes;         // resident packed filter
    uint32_t stage_bytes;     // FW * FH * 4 lines * 8 channels * 128 B
    float* Out;
    const float* bias;
    int relu;
    int* status;
};

struct __align__(8) ConvSmem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t xf[kMaxStages];
    uint64_t tfull[2];
    uint64_t tempty[2];
    uint64_t wbar;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, int lane, volatile int* abort_flag,
                                          int* status, int code) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, status, code) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Physical byte address of the 16-byte chunk `q` (0..7) of the 128-byte row at `row_addr` under the 128-byte
// swizzle with 32-byte atoms: the 32-byte chunk index is XORed with bits [7,9) of the address.
__device__ __forceinline__ uint32_t sw32_chunk(uint32_t row_addr, int q) {
    const uint32_t phase = (row_addr >> 7) & 3u;
    return row_addr + ((((uint32_t)q >> 1) ^ phase) << 5) + (((uint32_t)q & 1u) << 4);
}

template <int W>
__device__ __forceinline__ void shift_row(uint32_t src_row, uint32_t left_row, uint32_t right_row) {
    float v[32];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(v[4 * q]), "=f"(v[4 * q + 1]), "=f"(v[4 * q + 2]), "=f"(v[4 * q + 3])
                     : "r"(sw32_chunk(src_row, q)));
    }
    // left tap (fw = 0): out[x] = in[x - 1], zero where the column would be -1
    // right tap (fw = 2): out[x] = in[x + 1], zero where the column would be W
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        float l[4], r[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int x = 4 * q + e;
            const int col = x % W;
            l[e] = (col >= 1) ? v[(x + 31) & 31] : 0.f;
            r[e] = (col < W - 1) ? v[(x + 1) & 31] : 0.f;
        }
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(sw32_chunk(left_row, q)), "f"(l[0]), "f"(l[1]),
                     "f"(l[2]), "f"(l[3])
                     : "memory");
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(sw32_chunk(right_row, q)), "f"(r[0]), "f"(r[1]),
                     "f"(r[2]), "f"(r[3])
                     : "memory");
    }
}

__global__ void __launch_bounds__(320, 1)
    umma_conv_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmW,
                     const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ ConvSmem cs;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int* abort_flag = &cs.abort_flag;

    const uint32_t w_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t st_base = w_base + p.w_bytes;
    const uint32_t set_bytes = (uint32_t)p.FH * 4u * kCB * kRowBytes;  // one horizontal tap: FH x 4 lines x 8 rows
    const int taps = p.FH * p.FW;
    const int centre = p.FW >> 1;  // set index of the unshifted copy

    if (threadIdx.x == 0) {
        cs.abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&cs.full[s]), 1);
            mbar_init(smem_u32(&cs.empty[s]), 1);
            mbar_init(smem_u32(&cs.xf[s]), 128);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&cs.tfull[a]), 1);
            mbar_init(smem_u32(&cs.tempty[a]), 128);
        }
        mbar_init(smem_u32(&cs.wbar), 1);
        mbar_fence_init();
        tma_prefetch_desc(&tmIn);
        tma_prefetch_desc(&tmW);
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc(smem_u32(&cs.tmem_base), (uint32_t)p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = cs.tmem_base;
    const uint32_t acc_stride = (uint32_t)p.tmem_cols >> 1;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // resident filter: one box [OCp rows][32 channels] per (tap, channel group)
            const uint32_t wbar = smem_u32(&cs.wbar);
            mbar_expect_tx(wbar, p.w_bytes);
            const int boxes = taps * p.CG;
            for (int b = 0; b < boxes; ++b)
                tma_load_3d(w_base + (uint32_t)b * p.OCp * kRowBytes, &tmW, wbar, 0, b * p.OCp, 0);
        }
        __syncwarp();
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x) {
            for (int cb = 0; cb < p.NCB; ++cb) {
                ok = warp_wait(smem_u32(&cs.empty[s]), ph ^ 1u, lane, abort_flag, p.status, CBK_TIMEOUT_EMPTY);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t full = smem_u32(&cs.full[s]);
                    const uint32_t dst0 = st_base + s * p.stage_bytes + (uint32_t)centre * set_bytes;
                    mbar_expect_tx(full, set_bytes);
                    for (int fh = 0; fh < p.FH; ++fh) {
                        for (int j = 0; j < 4; ++j) {
                            const long long g = 4LL * tile + j;
                            // lines past the end use an image index >= N: the whole box is zero-filled
                            const int n = (int)(g / p.LPI);
                            const int h0 = (int)(g - (long long)n * p.LPI) * p.L;
                            tma_load_4d(dst0 + (uint32_t)((fh * 4 + j) * kCB) * kRowBytes, &tmIn, full, 0,
                                        h0 + fh - p.pH, cb * kCB, n);
                        }
                    }
                }
                __syncwarp();
                if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ UMMA issuer
        const uint32_t idesc = umma_idesc_tf32(128, (uint32_t)p.OCp, 1u, 0u);
        uint32_t s = 0, ph = 0, lt = 0;
        bool ok = warp_wait(smem_u32(&cs.wbar), 0, lane, abort_flag, p.status, CBK_TIMEOUT_FULL);
        for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++lt) {
            const uint32_t a = lt & 1u;
            ok = warp_wait(smem_u32(&cs.tempty[a]), ((lt >> 1) & 1u) ^ 1u, lane, abort_flag, p.status,
                           CBK_TIMEOUT_TMEM_EMPTY);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + a * acc_stride;
            for (int cb = 0; cb < p.NCB; ++cb) {
                ok = warp_wait(smem_u32(&cs.full[s]), ph, lane, abort_flag, p.status, CBK_TIMEOUT_FULL);
                if (!ok) break;
                if (p.FW > 1) {
                    ok = warp_wait(smem_u32(&cs.xf[s]), ph, lane, abort_flag, p.status, CBK_TIMEOUT_XFORM);
                    if (!ok) break;
                }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t stg = st_base + s * p.stage_bytes;
                    const uint32_t wq = w_base + (uint32_t)(cb >> 2) * p.OCp * kRowBytes + (uint32_t)(cb & 3) * 32u;
                    for (int fh = 0; fh < p.FH; ++fh) {
                        for (int fw = 0; fw < p.FW; ++fw) {
                            const int t = fh * p.FW + fw;
                            // P: 4 lines x [8 channels][128 B], MN-major, 1024 B between lines, 512 B per 4 rows
                            const uint64_t dP = umma_smem_desc(stg + (uint32_t)fw * set_bytes +
                                                                   (uint32_t)fh * 4u * kCB * kRowBytes,
                                                               1024u, 512u, UMMA_SW_128B_BASE32B);
                            // Q: packed filter rows [oc][32 channels], K-major, 8 channels of this stage
                            const uint64_t dQ = umma_smem_desc(wq + (uint32_t)t * p.CG * p.OCp * kRowBytes, 16u, 1024u,
                                                               UMMA_SW_128B);
                            umma_tf32(d_tmem, dP, dQ, idesc, (cb == 0 && t == 0) ? 0u : 1u);
                        }
                    }
                    tc_commit(smem_u32(&cs.empty[s]));
                    if (cb == p.NCB - 1) tc_commit(smem_u32(&cs.tfull[a]));
                }
                __syncwarp();
                if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;
        uint32_t lt = 0;
        bool ok = true;
        const long long plane = (long long)p.H * p.W;
        for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++lt) {
            const uint32_t a = lt & 1u;
            ok = mbar_wait(smem_u32(&cs.tfull[a]), (lt >> 1) & 1u, abort_flag, p.status, CBK_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const long long g = 4LL * tile + quarter;
            const bool valid = g < p.total_lines;
            const int n = (int)(g / p.LPI);
            const int h0 = (int)(g - (long long)n * p.LPI) * p.L;
            // lane x of the line is pixel (h0 + x / W, x % W): 32 consecutive floats of the output plane
            float* out = p.Out + ((long long)n * p.Cout * p.H + h0) * p.W + lane;
            const uint32_t t_row = tmem_base + a * acc_stride + ((uint32_t)(32 * quarter) << 16);
            for (int c = 0; c < p.OCp; c += 16) {
                uint32_t r[16];
                tmem_ld16(t_row + (uint32_t)c, r);
                tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int oc = c + e;
                        if (oc < p.Cout) {
                            float v = __uint_as_float(r[e]);
                            if (p.bias) v += __ldg(p.bias + oc);
                            if (p.relu) v = fmaxf(v, 0.f);
                            out[(long long)oc * plane] = v;
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&cs.tempty[a]));
        }
    } else {
        // ------------------------------------------------------------ shift warps (horizontal taps)
        if (p.FW > 1) {
            const int t = threadIdx.x - 192;  // 0..127
            const int rows = p.FH * 4 * kCB;  // centre rows per stage (<= 96)
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x) {
                for (int cb = 0; cb < p.NCB; ++cb) {
                    ok = mbar_wait(smem_u32(&cs.full[s]), ph, abort_flag, p.status, CBK_TIMEOUT_XFORM_FULL);
                    if (!ok) break;
                    if (t < rows) {
                        const uint32_t stg = st_base + s * p.stage_bytes;
                        const uint32_t src = stg + set_bytes + (uint32_t)t * kRowBytes;
                        const uint32_t lft = stg + (uint32_t)t * kRowBytes;
                        const uint32_t rgt = stg + 2u * set_bytes + (uint32_t)t * kRowBytes;
                        if (p.W == 32) shift_row<32>(src, lft, rgt);
                        else if (p.W == 16) shift_row<16>(src, lft, rgt);
                        else shift_row<8>(src, lft, rgt);
                    }
                    fence_proxy_async_smem();
                    mbar_arrive(smem_u32(&cs.xf[s]));
                    if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
}

// Packs the filter for the kernel above. Wp row index = (tap * CG + cg) * OCp + o, 32 floats per row.
//   forward:  Wp[tap=(fh,fw)][cg][o][c] = W[o][cg*32 + c][fh][fw]                 (W is OC x IC x FH x FW)
//   dgrad:    Wp[tap=(fh,fw)][cg][o][c] = W[cg*32 + c][o][FH-1-fh][FW-1-fw]       (o = input channel of the conv)
__global__ void pack_filter_kernel(const float* __restrict__ W, float* __restrict__ Wp, int OC, int IC, int FH, int FW,
                                   int OCp, int CG, int dgrad, long long total) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i & 31);
        long long r = i >> 5;
        const int o = (int)(r % OCp);
        r /= OCp;
        const int cg = (int)(r % CG);
        const int tap = (int)(r / CG);
        const int fh = tap / FW, fw = tap - fh * FW;
        const int ch = cg * 32 + c;
        float v = 0.f;
        if (!dgrad) {
            if (o < OC && ch < IC) v = W[(((long long)o * IC + ch) * FH + fh) * FW + fw];
        } else {
            if (o < IC && ch < OC) v = W[(((long long)ch * IC + o) * FH + (FH - 1 - fh)) * FW + (FW - 1 - fw)];
        }
        Wp[i] = v;
    }
}

}  // namespace

int umma_conv_fwd(cb_ctx* ctx, const float* W, const float* X, float* Y, const float* bias, int N, int IC, int IH,
                  int IW, int OC, int FH, int FW, int sH, int sW, int pH, int pW, int relu, bool dgrad_of) {
    // geometry covered by the tensor-core path
    if (sH != 1 || sW != 1) return CB_EUNSUPPORTED;
    if (!((FH == 1 && pH == 0) || (FH == 3 && pH == 1))) return CB_EUNSUPPORTED;
    if (!((FW == 1 && pW == 0) || (FW == 3 && pW == 1))) return CB_EUNSUPPORTED;
    if (IW != 8 && IW != 16 && IW != 32) return CB_EUNSUPPORTED;
    const int L = 32 / IW;
    if (IH % L) return CB_EUNSUPPORTED;
    // roles: forward reads X (IC channels) and writes OC planes; the data gradient reads dY (OC) and writes IC
    const int Cin = dgrad_of ? OC : IC;
    const int Cout = dgrad_of ? IC : OC;
    const int OCp = (Cout + 15) / 16 * 16;
    if (OCp > 256 || Cin < 1) return CB_EUNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(X) & 15u) != 0) return CB_EUNSUPPORTED;
    const int CG = (Cin + 31) / 32;
    const int taps = FH * FW;
    const size_t w_bytes = (size_t)taps * CG * OCp * kRowBytes;
    const uint32_t stage_bytes = (uint32_t)FW * FH * 4 * kCB * kRowBytes;
    const long long smem_cap = (long long)ctx->max_smem_optin - 2048;
    long long stages = (smem_cap - (long long)w_bytes) / stage_bytes;
    if (stages < 2) return CB_EUNSUPPORTED;
    if (stages > kMaxStages) stages = kMaxStages;

    int rc = ensure_workspace(ctx, w_bytes);
    if (rc != CB_OK) return rc;
    float* Wp = static_cast<float*>(ctx->workspace);
    {
        const long long total = (long long)w_bytes / 4;
        int grid = (int)((total + 255) / 256);
        if (grid > ctx->sm_count * 8) grid = ctx->sm_count * 8;
        pack_filter_kernel<<<grid, 256, 0, ctx->stream>>>(W, Wp, OC, IC, FH, FW, OCp, CG, dgrad_of ? 1 : 0, total);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return check_cuda(ctx, e, "pack_filter_kernel launch");
        ctx->launches += 1;
    }

    ConvParams p{};
    p.N = N; p.Cin = Cin; p.H = IH; p.W = IW; p.Cout = Cout;
    p.FH = FH; p.FW = FW; p.pH = pH;
    p.OCp = OCp; p.CG = CG; p.NCB = (Cin + kCB - 1) / kCB;
    p.L = L; p.LPI = IH / L;
    p.total_lines = (long long)N * p.LPI;
    p.tiles = (int)((p.total_lines + 3) / 4);
    p.stages = (int)stages;
    int cols = 32;
    while (cols < 2 * OCp) cols <<= 1;
    p.tmem_cols = cols;
    p.w_bytes = (uint32_t)w_bytes;
    p.stage_bytes = stage_bytes;
    p.Out = Y; p.bias = bias; p.relu = relu;
    p.status = ctx->d_status;

    CUtensorMap tmIn, tmW;
    {
        // input planes: (W, H, C, N); box = one line of 8 channels; rows and channels out of range read as zero
        uint64_t dims[4] = {(uint64_t)IW, (uint64_t)IH, (uint64_t)Cin, (uint64_t)N};
        uint64_t str[3] = {(uint64_t)IW * 4, (uint64_t)IH * IW * 4, (uint64_t)Cin * IH * IW * 4};
        uint32_t box[4] = {(uint32_t)IW, (uint32_t)L, (uint32_t)kCB, 1u};
        rc = encode_tmap(ctx, &tmIn, X, 4, dims, str, box, nullptr, 129);
        if (rc != CB_OK) return rc;
    }
    {
        uint64_t dims[3] = {32, (uint64_t)taps * CG * OCp, 1};
        uint64_t str[2] = {128, (uint64_t)taps * CG * OCp * 128};
        uint32_t box[3] = {32, (uint32_t)OCp, 1};
        rc = encode_tmap(ctx, &tmW, Wp, 3, dims, str, box, nullptr, 128);
        if (rc != CB_OK) return rc;
    }
    const size_t smem = w_bytes + (size_t)p.stages * stage_bytes + 1024;
    cudaError_t e = cudaFuncSetAttribute(umma_conv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return check_cuda(ctx, e, "umma_conv_kernel attribute");
    const int grid = p.tiles < ctx->sm_count ? p.tiles : ctx->sm_count;
    umma_conv_kernel<<<grid, 320, smem, ctx->stream>>>(tmIn, tmW, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "umma_conv_kernel launch");
    ctx->launches += 1;
    ctx->last_kernel = "umma_tf32";
    return CB_OK;
}

int umma_conv_wgrad(cb_ctx*, const float*, const float*, float*, int, int, int, int, int, int, int, int, int, int,
                    int, int) {
    return CB_EUNSUPPORTED;
}

}  // namespace cb
