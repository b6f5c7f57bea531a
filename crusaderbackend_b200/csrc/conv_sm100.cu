// Tensor-core implicit-GEMM convolution for sm_100a (TF32 mode), NCHW fp32, no materialised im2col.
//
// Forward and data-gradient run the same kernel: D[pixel][oc] = sum over (tap, c) of In[n, c, oh+fh-pH, ow+fw-pW]
// * Wp[tap][oc][c]. The 128 TMEM lanes of an accumulator are 128 output pixels (UMMA M), the columns are the output
// channels (UMMA N), K walks 8 input channels of one filter tap per tcgen05.mma.
//
//  * Pixels are grouped in "lines" of 32 consecutive floats of one channel plane (32/W image rows of a W-wide map,
//    W in {8,16,32}); a CTA tile is 4 lines. For each filter row fh and line, one TMA box (32 pixels of the
//    flattened H*W plane, 8*KS channels) of the NCHW input lands as [channels][128 bytes] — exactly the MN-major
//    operand layout the tensor core reads (128-byte swizzle with 32-byte atoms). Rows above / below the image are out
//    of bounds for the tensor map and arrive as zeros, which is the vertical padding.
//  * A TMA box may not start at an odd column (its innermost coordinate must be 16-byte aligned), so the
//    horizontal taps cannot be fetched as shifted boxes. They are not shifted on the input side at all: the three
//    horizontal taps of a filter row are folded into the UMMA N dimension (accumulator column fw*OCs + oc holds the
//    partial sum of tap fw evaluated at the UNSHIFTED pixel), and the epilogue adds D0[x-1] + D1[x] + D2[x+1] with
//    two warp shuffles per value; lanes at a row edge take zero instead, which is the horizontal padding.
//  * The filter reaches the kernel already packed as [fh][32-channel group][fw][oc][32 channels] (K-major rows of
//    128 bytes, zero padded) in global memory and is fetched once per CTA by TMA into 128-byte-swizzled shared
//    memory, where it stays for the whole persistent CTA. The packing is a separate small kernel
//    (pack_filter_kernel); with the context's filter cache on it runs once per weight update instead of once per call
//    (cb_conv_cache_filters / cb_filters_changed). For the data gradient the pack transposes the channel roles and
//    rotates the filter by 180 degrees (seblas/operations/cuConv.cu:321-326 does the same rotation on the fly).
//  * When a layer has fewer pixel tiles than the GPU has CTA slots, the output channels are split over 2 or 4 CTAs
//    per tile (each fetches only its slice of the packed filter and runs a narrower UMMA), so that small feature maps
//    still occupy the whole GPU.
//  * Epilogue (4 or 2 warps per TMEM lane quarter): tcgen05.ld, tap combine, then optional per-channel or
//    per-position scale / shift, bias, accumulation onto the output, ReLU, and stores in which the 32 lanes of a warp
//    write 128 contiguous bytes.
//
// Covered geometry: stride 1, filter 1x1 (pad 0) or 3x3 (pad 1) per axis, W in {8,16,32}, (32/W) | H,
// FW * OC(rounded to 16) <= 256 per CTA, packed filter slice <= ~150 KB; stride 2 through the phase split below.
// Everything else is served by the CUDA-core kernels in conv_simt.cu.
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "conv_common.cuh"

namespace cb {
namespace {

struct ConvParams {
    int N, Cin, H, W, Cout;   // "input" and "output" of this pass (forward: X -> Y, dgrad: dY -> dX)
    int FH, FW, pH, pW;       // taps and padding: tap (fh, fw) reads the input at offset (fh - pH, fw - pW), each in [-1, 1]
    int OCs;                  // output channels one CTA computes (a multiple of 16)
    int nsplit;               // CTAs sharing a pixel tile, CTA b taking channels [(b % nsplit) * OCs, +OCs)
    int NQ;                   // UMMA N = FW * OCs
    int CG;                   // 32-channel groups of the packed filter
    int KS;                   // UMMA K steps (8 channels each) per pipeline stage
    int NCB;                  // ceil(Cin / (8 * KS)) pipeline stages per tile
    int L;                    // image rows per line (32 / W)
    int LPI;                  // lines per image (H / L)
    int shared_rows;          // 1: the FH taps of a tile share FH + 3 row blocks (W == 32); 0: FH * 4 blocks
    int nblocks;              // row blocks per stage
    long long total_lines;    // N * LPI
    int tiles;                // ceil(total_lines / 4)
    int stages;
    int tmem_cols;
    uint32_t w_bytes;         // resident slice of the packed filter
    uint32_t block_bytes;     // one line of a stage: 8 * KS channels x 128 B
    uint32_t stage_bytes;     // nblocks * block_bytes
    int tma_out;              // 1: results leave through TMA stores (2: TMA reduce-adds) staged in shared memory
    float* Out;
    long long out_batch;      // elements between consecutive images of the output
    ConvEpilogue ep;
    int c_wrap;         // > 0: input channels from c_wrap on are read again from channel (c - c_wrap) (3xTF32 form)
    int issue_uniform;  // the MMA warp issues as a whole with an elected lane (wide accumulators) instead of from lane 0
    int* status;
    long long* trace;
    int dbg;       // development probes of the trace build
};

struct __align__(8) ConvSmem {
    uint64_t full[kConvMaxStages];
    uint64_t empty[kConvMaxStages];
    uint64_t tfull[2];
    uint64_t tempty[2];
    uint64_t wbar;
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
};

enum { PACK_FWD = 0, PACK_DGRAD = 1, PACK_S2_FWD = 2, PACK_S2_DGRAD = 3, PACK_FWD_X3 = 4, PACK_DGRAD_X3 = 5 };
constexpr int kMaxTileUmmas = 256;  // most UMMAs of one tile (filter rows x 8-channel steps) a plan may need

// Horizontal tap sets the kernel is instantiated for: the taps' column offsets fw - pW.
enum { TAPS_1 = 0 /* {0} */, TAPS_3 = 1 /* {-1, 0, +1} */, TAPS_2L = 2 /* {-1, 0} */, TAPS_2R = 3 /* {0, +1} */ };

// One chunk of 8 output channels of a tile's epilogue: the horizontal taps were accumulated at the unshifted pixel in
// column blocks fw*OCs + c; the tap with column offset d holds its partial sum d lanes away, and lanes that would read
// across a row edge take zero instead (the horizontal padding). The epilogue is bound by latency and instruction issue (an SM
// runs up to 16 epilogue warps of two CTAs), so the tap set is a template parameter and the plain forms take a branch-free path.
// The 8 x 32 results leave either through one TMA store of the [8 channels][32 pixels] block, staged in this warp's
// shared-memory slot `stage` (eight direct stores per thread land in eight different 4 KB-apart lines and were the
// slowest part of the kernel), or, for the epilogue forms TMA cannot express (accumulate followed by ReLU), directly.
template <int TAPS>
__device__ __forceinline__ void conv_epilogue_chunk(const ConvParams& p, const CUtensorMap* tmOut, uint32_t t_row, int c,
                                                    int oc0, float* img, long long plane, int pix, int n, bool valid,
                                                    bool has_left, bool has_right, uint32_t stage, int lane, bool traced) {
    uint32_t r0[8], r1[8], r2[8];
    tmem_ld8(t_row + (uint32_t)c, r0);
    if (TAPS != TAPS_1) tmem_ld8(t_row + (uint32_t)(p.OCs + c), r1);
    if (TAPS == TAPS_3) tmem_ld8(t_row + (uint32_t)(2 * p.OCs + c), r2);
    tmem_ld_wait();
    if (traced) CB_TRACE_EVENT(p.trace, 13);
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        if (TAPS == TAPS_1) {
            v[e] = __uint_as_float(r0[e]);
        } else if (TAPS == TAPS_3) {
            const float up = __shfl_up_sync(0xffffffffu, __uint_as_float(r0[e]), 1);
            const float dn = __shfl_down_sync(0xffffffffu, __uint_as_float(r2[e]), 1);
            v[e] = ((has_left ? up : 0.f) + __uint_as_float(r1[e])) + (has_right ? dn : 0.f);
        } else if (TAPS == TAPS_2L) {
            const float up = __shfl_up_sync(0xffffffffu, __uint_as_float(r0[e]), 1);
            v[e] = (has_left ? up : 0.f) + __uint_as_float(r1[e]);
        } else {
            const float dn = __shfl_down_sync(0xffffffffu, __uint_as_float(r1[e]), 1);
            v[e] = __uint_as_float(r0[e]) + (has_right ? dn : 0.f);
        }
    }
    if (traced) CB_TRACE_EVENT(p.trace, 14);
    const bool plain = p.ep.scale == nullptr && p.ep.bias == nullptr;
    if (p.tma_out) {
        // the store issued two chunks ago from this slot must have finished reading it
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        const uint32_t mine = stage + (uint32_t)(lane * 4);
        if (plain) {
            const bool relu = p.ep.relu != 0;
#pragma unroll
            for (int e = 0; e < 8; ++e)
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(mine + (uint32_t)(e * 128)), "f"(relu ? fmaxf(v[e], 0.f) : v[e])
                             : "memory");
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int oc = oc0 + c + e;
                float y = v[e];
                if (oc < p.Cout) {
                    if (p.ep.scale) {
                        const long long si = p.ep.per_position ? (long long)oc * plane + pix : (long long)oc;
                        y = fmaf(y, __ldg(p.ep.scale + si), __ldg(p.ep.shift + si));
                    }
                    if (p.ep.bias) y += __ldg(p.ep.bias + oc);
                    if (p.ep.relu) y = fmaxf(y, 0.f);
                }
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(mine + (uint32_t)(e * 128)), "f"(y) : "memory");
            }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && valid) {
            if (p.tma_out == 2) tma_reduce_add_3d(tmOut, stage, pix, oc0 + c, n);
            else tma_store_3d(tmOut, stage, pix, oc0 + c, n);
            tma_store_commit();
        }
    } else if (valid) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int oc = oc0 + c + e;
            if (oc < p.Cout) {
                float y = v[e];
                const long long idx = (long long)oc * plane + pix;
                if (p.ep.scale) {
                    const long long si = p.ep.per_position ? idx : (long long)oc;
                    y = fmaf(y, __ldg(p.ep.scale + si), __ldg(p.ep.shift + si));
                }
                if (p.ep.bias) y += __ldg(p.ep.bias + oc);
                if (p.ep.accumulate) y += img[idx];
                if (p.ep.relu) y = fmaxf(y, 0.f);
                img[idx] = y;
            }
        }
    }
    if (traced) CB_TRACE_EVENT(p.trace, 15);
}

// Epilogue warps are a template parameter of the kernel (8 = 2 per TMEM lane quarter is what the planner picks; 16 is
// kept for experiments). Outputs of at most 32 channels per CTA with a small filter run two CTAs per SM so that their
// UMMA chains overlap.
template <int kEpiWarps, int TAPS>
__global__ void __launch_bounds__(64 + 32 * kEpiWarps, kEpiWarps <= 8 ? 2 : 1)
    umma_conv_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmW,
                     const __grid_constant__ CUtensorMap tmOut, const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ ConvSmem cs;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int* abort_flag = &cs.abort_flag;

    const uint32_t w_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t st_base = w_base + p.w_bytes;
    const uint32_t out_base = st_base + (uint32_t)p.stages * p.stage_bytes;  // epilogue staging: 2 KB per epilogue warp
    // this CTA's slice of the output channels and its walk over the pixel tiles
    const int split = (int)blockIdx.x % p.nsplit;
    const int tile0 = (int)blockIdx.x / p.nsplit;
    const int tile_step = (int)gridDim.x / p.nsplit;
    const int oc0 = split * p.OCs;

    if (threadIdx.x == 0) {
        CB_TRACE_WALL(p.trace, 0);
        CB_TRACE_EVENT(p.trace, 1);
        cs.abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&cs.full[s]), 1);
            mbar_init(smem_u32(&cs.empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&cs.tfull[a]), 1);
            mbar_init(smem_u32(&cs.tempty[a]), 32 * kEpiWarps);
        }
        mbar_init(smem_u32(&cs.wbar), 1);
        mbar_init(smem_u32(&cs.drain), 1);
        mbar_fence_init();
        tma_prefetch_desc(&tmIn);
        tma_prefetch_desc(&tmW);
        if (p.tma_out) tma_prefetch_desc(&tmOut);
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc(smem_u32(&cs.tmem_base), (uint32_t)p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Up to here nothing has touched global memory (barriers, descriptor prefetch of kernel parameters, TMEM): the
    // kernel before this one may still be running. From here on its results are complete, and the kernel after this
    // one may begin its own preamble.
    griddep_wait();
    griddep_launch();
    const uint32_t tmem_base = cs.tmem_base;
    const uint32_t acc_stride = (uint32_t)p.tmem_cols >> 1;
    uint32_t armed = 0, armed_parity = 0;  // producer lane: stages armed at least once / parity of their last arming
    if (threadIdx.x == 0) CB_TRACE_EVENT(p.trace, 2);

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // resident filter slice: one box [FW taps][OCs rows][32 channels] per (filter row, channel group)
            const uint32_t wbar = smem_u32(&cs.wbar);
            mbar_expect_tx(wbar, p.w_bytes);
            const int boxes = p.FH * p.CG;
            for (int b = 0; b < boxes; ++b)
                tma_load_3d(w_base + (uint32_t)b * p.NQ * kRowBytes, &tmW, wbar, 0, oc0, b * p.FW);
        }
        __syncwarp();
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (int tile = tile0; tile < p.tiles && ok; tile += tile_step) {
            for (int cb = 0; cb < p.NCB; ++cb) {
                ok = conv_warp_wait(smem_u32(&cs.empty[s]), ph ^ 1u, lane, abort_flag, p.status, CBK_TIMEOUT_EMPTY);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t full = smem_u32(&cs.full[s]);
                    const uint32_t dst0 = st_base + s * p.stage_bytes;
                    mbar_expect_tx(full, p.stage_bytes);
                    armed |= 1u << s;
                    armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
                    int c0 = cb * p.KS * kCB;
                    if (p.c_wrap && c0 >= p.c_wrap) c0 -= p.c_wrap;  // third channel group of the 3xTF32 form: x_hi again
                    if (p.shared_rows) {
                        // W == 32: the tile is 4 consecutive rows of one image; ONE box (32 px, 8*KS channels, FH+3
                        // rows) lands as [row][channel][128 B]; rows above / below the image are zero-filled
                        const int g = 4 * tile;  // 32-bit: a 64-bit division costs ~100 cycles on this path
                        const int n = g / p.LPI;
                        const int h0 = g - n * p.LPI;
                        tma_load_4d(dst0, &tmIn, full, 0, c0, h0 - p.pH, n);
                    } else {
                        for (int fh = 0; fh < p.FH; ++fh) {
                            for (int j = 0; j < 4; ++j) {
                                const int g = 4 * tile + j;
                                // lines past the end use an image index >= N: the whole box is zero-filled
                                const int n = g / p.LPI;
                                const int h0 = (g - n * p.LPI) * p.L;
                                tma_load_3d(dst0 + (uint32_t)(fh * 4 + j) * p.block_bytes, &tmIn, full,
                                            (h0 + fh - p.pH) * p.W, c0, n);
                            }
                        }
                    }
                }
                __syncwarp();
                if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ UMMA issuer
        // One thread feeds the tensor core, and what it spends per tcgen05.mma bounds the kernel (a 128 x 48 x 8 UMMA is
        // ~50 cycles of tensor pipe). The operand descriptors are advanced by plain integer arithmetic on values that
        // come from kernel parameters and loop counters only: a descriptor offset fetched from a shared-memory table
        // costs ~113 cycles per UMMA whatever its size (measured with the UMMA-only loop of peak_sm100.cu: 52 -> 113
        // cycles at N = 64, 103 -> 124 at N = 192), one computed with divisions ~150 instructions.
        const uint32_t idesc = umma_idesc_tf32(128, (uint32_t)p.NQ, 1u, 0u);
        // P: 4 lines x [8 channels][128 B], MN-major: block_bytes between lines (LBO), 512 B per 4 channel rows (SBO)
        const uint64_t descP0 = umma_smem_desc(0, p.block_bytes, 512u, UMMA_SW_128B_BASE32B);
        // Q: packed filter rows [(fw, oc)][32 channels], K-major 128-byte rows
        const uint64_t descQ0 = umma_smem_desc(w_base, 16u, 1024u, UMMA_SW_128B);
        const uint32_t blk_units = p.block_bytes >> 4;                     // descriptor address units (16 B) per line block
        const uint32_t fh_units = (p.shared_rows ? 1u : 4u) * blk_units;  // between consecutive filter rows of P
        const uint32_t q_group_units = (uint32_t)p.NQ * (kRowBytes >> 4);  // one (filter row, 32-channel group) of Q
        const uint32_t q_fh_units = (uint32_t)p.CG * q_group_units;        // between consecutive filter rows of Q
        uint32_t s = 0, ph = 0, lt = 0;
        bool ok = conv_warp_wait(smem_u32(&cs.wbar), 0, lane, abort_flag, p.status, CBK_TIMEOUT_FULL);
        if (lane == 0) CB_TRACE_EVENT(p.trace, 4);
#ifdef CB_TRACE
        long long t_tempty = 0, t_full = 0, t_issue = 0;
#endif
        for (int tile = tile0; tile < p.tiles && ok; tile += tile_step, ++lt) {
            const uint32_t a = lt & 1u;
#ifdef CB_TRACE
            const long long c_t0 = clock64();
#endif
            ok = conv_warp_wait(smem_u32(&cs.tempty[a]), ((lt >> 1) & 1u) ^ 1u, lane, abort_flag, p.status,
                                CBK_TIMEOUT_TMEM_EMPTY);
            if (!ok) break;
            tc_fence_after();
#ifdef CB_TRACE
            t_tempty += clock64() - c_t0;
#endif
            const uint32_t d_tmem = tmem_base + a * acc_stride;
            int ti = 0;
            for (int cb = 0; cb < p.NCB; ++cb) {
#ifdef CB_TRACE
                const long long c_f0 = clock64();
#endif
                ok = conv_warp_wait(smem_u32(&cs.full[s]), ph, lane, abort_flag, p.status, CBK_TIMEOUT_FULL);
                if (!ok) break;
                tc_fence_after();
#ifdef CB_TRACE
                const long long c_f1 = clock64();
                t_full += c_f1 - c_f0;
#endif
                if (lane == 0 && lt == 0 && cb == 0) CB_TRACE_EVENT(p.trace, 5);
                const uint64_t pbase = descP0 + (uint64_t)(((st_base + s * p.stage_bytes) >> 4) & 0x3FFFu);
                const uint32_t ks0 = (uint32_t)(cb * p.KS);  // first K step of the stage: channels [8 ks0, ..)
                if (p.issue_uniform) {
                    // Wide accumulators (long MMA phases): the whole warp runs the loop with the same values and one
                    // elected lane issues, so that the descriptors stay in uniform registers — from a one-lane branch a
                    // descriptor that changes between UMMAs costs ~110 cycles of issue, more than a 128 x 192 x 8 UMMA
                    // takes (measured with the UMMA-only loop of peak_sm100.cu). Narrow accumulators measured slower
                    // this way and keep the one-lane form.
                    for (int fh = 0; fh < p.FH; ++fh) {
                        const uint64_t prow = pbase + (uint64_t)((uint32_t)fh * fh_units);
                        const uint64_t qrow = descQ0 + (uint64_t)((uint32_t)fh * q_fh_units);
                        for (int kk = 0; kk < p.KS; ++kk, ++ti) {
                            const uint32_t ks = ks0 + (uint32_t)kk;
                            umma_tf32_elect(d_tmem, prow + (uint64_t)((uint32_t)kk * 64u),
                                            qrow + (uint64_t)((ks >> 2) * q_group_units + (ks & 3u) * 2u), idesc, ti != 0 ? 1u : 0u);
                        }
                    }
                    tc_commit_elect(smem_u32(&cs.empty[s]));
                    if (cb == p.NCB - 1) tc_commit_elect(smem_u32(&cs.tfull[a]));
                } else if (lane == 0) {
                    for (int fh = 0; fh < p.FH; ++fh) {
                        const uint64_t prow = pbase + (uint64_t)((uint32_t)fh * fh_units);
                        const uint64_t qrow = descQ0 + (uint64_t)((uint32_t)fh * q_fh_units);
                        for (int kk = 0; kk < p.KS; ++kk, ++ti) {
                            const uint32_t ks = ks0 + (uint32_t)kk;
                            umma_tf32(d_tmem, prow + (uint64_t)((uint32_t)kk * 64u),
                                      qrow + (uint64_t)((ks >> 2) * q_group_units + (ks & 3u) * 2u), idesc, ti != 0 ? 1u : 0u);
                        }
                    }
                    tc_commit(smem_u32(&cs.empty[s]));
                    if (cb == p.NCB - 1) tc_commit(smem_u32(&cs.tfull[a]));
                }
                if (lane == 0 && lt == 0 && cb == p.NCB - 1) CB_TRACE_EVENT(p.trace, 6);
                __syncwarp();
#ifdef CB_TRACE
                t_issue += clock64() - c_f1;
#endif
                if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
            }
        }
#ifdef CB_TRACE
        if (lane == 0 && p.trace) {
            // behind the 1024 x 16 event slots: per-CTA sums of the issuer's waits and issue time
            long long* sums = p.trace + 1024 * 16 + (long long)blockIdx.x * 4;
            sums[0] = t_tempty;
            sums[1] = t_full;
            sums[2] = t_issue;
            sums[3] = (long long)p.stages * 10000 + p.KS * 1000 + p.NCB * 100 + p.nsplit;
        }
#endif
    } else {
        // ------------------------------------------------------------ epilogue (warps 2 ..)
        // One scheduler cannot hide the shuffle and store latencies of a single warp, so every TMEM lane quarter is
        // served by several warps that split the channel chunks between them.
        const int quarter = warp & 3;
        const int slot = (warp - 2) >> 2;
        const uint32_t my_stage = out_base + (uint32_t)(warp - 2) * 2048u;
        uint32_t buf = 0;
        uint32_t lt = 0;
        bool ok = true;
        const long long plane = (long long)p.H * p.W;
        const int col = lane & (p.W - 1);
        const bool has_left = col > 0, has_right = col < p.W - 1;
        for (int tile = tile0; tile < p.tiles && ok; tile += tile_step, ++lt) {
            const uint32_t a = lt & 1u;
            ok = mbar_wait(smem_u32(&cs.tfull[a]), (lt >> 1) & 1u, abort_flag, p.status, CBK_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (threadIdx.x == 64 && lt == 0) CB_TRACE_EVENT(p.trace, 7);
            if (threadIdx.x == 64 && lt == 1) CB_TRACE_EVENT(p.trace, 9);
            const int g = 4 * tile + quarter;
            const bool valid = g < (int)p.total_lines;
            const int n = g / p.LPI;
            const int h0 = (g - n * p.LPI) * p.L;
            // lane x of the line is pixel (h0 + x / W, x % W): 32 consecutive floats of the output plane
            float* img = p.Out + (long long)n * p.out_batch;
            const int pix = h0 * p.W + lane;
            const uint32_t t_row = tmem_base + a * acc_stride + ((uint32_t)(32 * quarter) << 16);
#ifdef CB_TRACE
            if (p.dbg & 1) {  // development probe: leave the accumulator unread (how fast is the MMA phase alone?)
                tc_fence_before();
                mbar_arrive(smem_u32(&cs.tempty[a]));
                continue;
            }
#endif
            for (int c = slot * 8; c < p.OCs; c += 8 * (kEpiWarps / 4), buf ^= 1u)
                conv_epilogue_chunk<TAPS>(p, &tmOut, t_row, c, oc0, img, plane, pix, n, valid, has_left, has_right,
                                    my_stage + buf * 1024u, lane, threadIdx.x == 64 && lt == 0 && c == 0);
            tc_fence_before();
            mbar_arrive(smem_u32(&cs.tempty[a]));
            if (threadIdx.x == 64 && lt == 0) CB_TRACE_EVENT(p.trace, 8);
            if (threadIdx.x == 64) CB_TRACE_EVENT(p.trace, 10);
        }
        // this warp's stores must be complete before its staging memory is released with the CTA
        if (p.tma_out && lane == 0) tma_store_wait_all<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (cs.abort_flag) {
        // A bounded wait gave up somewhere in this CTA. Copies armed before that may still be in flight towards this
        // CTA's shared memory and issued MMAs may still be running on its accumulators: give both a bounded chance to
        // finish before the shared memory and TMEM are released.
        if (warp == 0 && lane == 0) {
            mbar_drain(smem_u32(&cs.wbar), 0, p.status);
            for (int st = 0; st < p.stages; ++st)
                if ((armed >> st) & 1u) mbar_drain(smem_u32(&cs.full[st]), (armed_parity >> st) & 1u, p.status);
        }
        if (warp == 1) {  // the commit comes from the lane that issued the MMAs
            if (p.issue_uniform) tc_commit_elect(smem_u32(&cs.drain));
            else if (lane == 0) tc_commit(smem_u32(&cs.drain));
            if (lane == 0) mbar_drain(smem_u32(&cs.drain), 0, p.status);
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
    if (threadIdx.x == 0) {
        CB_TRACE_EVENT(p.trace, 11);
        CB_TRACE_WALL(p.trace, 12);
    }
}

// What one packed filter is made from: W is the caller's OC x IC x FHs x FWs filter, (FHc, FWc) the taps of the
// convolution the kernel runs. Row index = ((fh * CG + cg) * FWc + fw) * OCp + o, 32 floats per row.
//   PACK_FWD:      row[c] = W[o][cg*32 + c][fh][fw]
//   PACK_DGRAD:    row[c] = W[cg*32 + c][o][FH-1-fh][FW-1-fw]          (o = input channel of the convolution)
//   PACK_S2_FWD:   the stride-2 3x3 convolution as a 2x2 convolution over the 4 input phases stacked as channels
//                  c' = phase*IC + c: row[c'] = W[o][c][s2_tap(ph, fh)][s2_tap(pw, fw)] (zero where no tap lands)
//   PACK_S2_DGRAD: its adjoint: input channels are the OC planes of dY, output o' = out_first + o indexes (phase, c),
//                  taps flipped: row[oc] = W[oc][c][s2_tap(ph, 1-fh)][s2_tap(pw, 1-fw)]
struct PackJob {
    const float* W;
    float* Wp;
    int OC, IC, FHs, FWs, FHc, FWc, OCp, CG, mode, out_first, out_count;
    long long total;  // floats of the packed filter
};

__device__ __forceinline__ float pack_value(const PackJob& j, long long i) {
    const int c = (int)(i & 31);
    long long r = i >> 5;
    const int o = (int)(r % j.OCp);
    r /= j.OCp;
    const int fw = (int)(r % j.FWc);
    r /= j.FWc;
    const int cg = (int)(r % j.CG);
    const int fh = (int)(r / j.CG);
    const int ch = cg * 32 + c;
    const float* W = j.W;
    const int OC = j.OC, IC = j.IC, FHs = j.FHs, FWs = j.FWs;
    if (j.mode == PACK_FWD_X3 || j.mode == PACK_DGRAD_X3) {
        // 3xTF32 in one pass: the convolution runs over three groups of input channels [x ; x_lo ; x] against
        // [w ; w ; w_lo] (the tensor core reads the hi part of whatever it is given), all into one accumulator
        const int cin = j.mode == PACK_FWD_X3 ? IC : OC;   // input channels of the convolution the kernel runs
        const int cout = j.mode == PACK_FWD_X3 ? OC : IC;
        if (o >= cout || ch >= 3 * cin) return 0.f;
        const int grp = ch / cin, cc = ch - grp * cin;
        const float w = j.mode == PACK_FWD_X3 ? W[(((long long)o * IC + cc) * FHs + fh) * FWs + fw]
                                               : W[(((long long)cc * IC + o) * FHs + (FHs - 1 - fh)) * FWs + (FWs - 1 - fw)];
        if (grp < 2) return w;
        const float hi = __uint_as_float(__float_as_uint(w) & 0xFFFFE000u);
        uint32_t r;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(w - hi));
        return __uint_as_float(r);
    }
    if (j.mode == PACK_FWD) {
        if (o < OC && ch < IC) return W[(((long long)o * IC + ch) * FHs + fh) * FWs + fw];
    } else if (j.mode == PACK_DGRAD) {
        if (o < IC && ch < OC) return W[(((long long)ch * IC + o) * FHs + (FHs - 1 - fh)) * FWs + (FWs - 1 - fw)];
    } else if (j.mode == PACK_S2_FWD) {
        if (o < OC && ch < 4 * IC) {
            const int phase = ch / IC, cc = ch - phase * IC;
            const int sh = s2_tap(phase >> 1, fh), sw = s2_tap(phase & 1, fw);
            if (sh >= 0 && sw >= 0) return W[(((long long)o * IC + cc) * FHs + sh) * FWs + sw];
        }
    } else {
        if (o < j.out_count && ch < OC) {
            const int og = j.out_first + o;
            const int phase = og / IC, cc = og - phase * IC;
            const int sh = s2_tap(phase >> 1, 1 - fh), sw = s2_tap(phase & 1, 1 - fw);
            if (sh >= 0 && sw >= 0) return W[(((long long)ch * IC + cc) * FHs + sh) * FWs + sw];
        }
    }
    return 0.f;
}

__global__ void pack_filter_kernel(const PackJob j) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < j.total; i += (long long)gridDim.x * blockDim.x)
        j.Wp[i] = pack_value(j, i);
}
// Every cached filter of a context in one launch: blockIdx.y indexes a device table of jobs.
__global__ void pack_filter_table_kernel(const PackJob* __restrict__ jobs) {
    griddep_wait();
    griddep_launch();
    const PackJob j = jobs[blockIdx.y];
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < j.total; i += (long long)gridDim.x * blockDim.x)
        j.Wp[i] = pack_value(j, i);
}

// ---- re-layout kernels of the stride-2 path (memory-bound, one element per thread, coalesced on the write side)
// Xs[n][phase*C + c][i][j] = X[n][c][2i + (phase >> 1)][2j + (phase & 1)]
__global__ void space_to_depth2_kernel(const float* __restrict__ X, float* __restrict__ Xs, int C, int H, int W,
                                       long long total) {
    griddep_wait();
    griddep_launch();
    const int H2 = H / 2, W2 = W / 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int j = (int)(i % W2);
        long long r = i / W2;
        const int ii = (int)(r % H2);
        r /= H2;
        const int cp = (int)(r % (4 * C));
        const long long n = r / (4 * C);
        const int phase = cp / C, c = cp - phase * C;
        Xs[i] = X[((n * C + c) * H + 2 * ii + (phase >> 1)) * W + 2 * j + (phase & 1)];
    }
}
// dX[n][c][y][x] (+)= dXs[group][n][o][y/2][x/2] with phase*C + c = group*per_group + o
__global__ void depth_to_space2_kernel(const float* __restrict__ dXs, float* __restrict__ dX, int N, int C, int H, int W,
                                       int per_group, long long total, int accumulate) {
    griddep_wait();
    griddep_launch();
    const int H2 = H / 2, W2 = W / 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int x = (int)(i % W);
        long long r = i / W;
        const int y = (int)(r % H);
        r /= H;
        const int c = (int)(r % C);
        const long long n = r / C;
        const int og = ((y & 1) * 2 + (x & 1)) * C + c;
        const int g = og / per_group, o = og - g * per_group;
        const float v = dXs[((((long long)g * N + n) * per_group + o) * H2 + (y >> 1)) * W2 + (x >> 1)];
        dX[i] = accumulate ? dX[i] + v : v;
    }
}
// Xsub[nc][i][j] = X[nc][2i][2j]
__global__ void subsample2_kernel(const float* __restrict__ X, float* __restrict__ Xsub, long long NC, int H, int W,
                                  long long total) {
    griddep_wait();
    griddep_launch();
    const int H2 = H / 2, W2 = W / 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int j = (int)(i % W2);
        const long long r = i / W2;
        const int ii = (int)(r % H2);
        const long long nc = r / H2;
        Xsub[i] = X[(nc * H + 2 * ii) * W + 2 * j];
    }
}
// dX[nc][y][x] (+)= (y, x both even) ? dXsub[nc][y/2][x/2] : 0
__global__ void upsample2_zero_kernel(const float* __restrict__ dXsub, float* __restrict__ dX, int H, int W,
                                      long long total, int accumulate) {
    griddep_wait();
    griddep_launch();
    const int H2 = H / 2, W2 = W / 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int x = (int)(i % W);
        const long long r = i / W;
        const int y = (int)(r % H);
        const long long nc = r / H;
        const float v = ((x | y) & 1) ? 0.f : dXsub[(nc * H2 + (y >> 1)) * W2 + (x >> 1)];
        if (accumulate) {
            if (!((x | y) & 1)) dX[i] += v;
        } else {
            dX[i] = v;
        }
    }
}

// Vector forms of the four re-layout kernels for 16-byte aligned tensors with W % 4 == 0: one thread moves four
// consecutive pixels of an input row (a 16-byte access on the full-resolution side, two 8-byte accesses on the
// half-resolution side), so every access is coalesced.
__global__ void space_to_depth2_vec_kernel(const float* __restrict__ X, float* __restrict__ Xs, int C, int H, int W,
                                           long long items) {
    griddep_wait();
    griddep_launch();
    const int H2 = H / 2, W2 = W / 2, WQ = W / 4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < items;
         i += (long long)gridDim.x * blockDim.x) {
        const int q = (int)(i % WQ);
        long long r = i / WQ;
        const int y = (int)(r % H);
        r /= H;
        const int c = (int)(r % C);
        const long long n = r / C;
        const float4 v = *reinterpret_cast<const float4*>(X + ((n * C + c) * H + y) * W + 4 * q);
        const int row = y & 1;
        float* d0 = Xs + (((n * 4 + 2 * row) * C + c) * H2 + (y >> 1)) * W2 + 2 * q;  // phase (row, 0)
        float* d1 = d0 + (long long)C * H2 * W2;                                       // phase (row, 1)
        *reinterpret_cast<float2*>(d0) = make_float2(v.x, v.z);
        *reinterpret_cast<float2*>(d1) = make_float2(v.y, v.w);
    }
}
__global__ void depth_to_space2_vec_kernel(const float* __restrict__ dXs, float* __restrict__ dX, int N, int C, int H, int W,
                                           int per_group, long long items, int accumulate) {
    griddep_wait();
    griddep_launch();
    const int H2 = H / 2, W2 = W / 2, WQ = W / 4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < items;
         i += (long long)gridDim.x * blockDim.x) {
        const int q = (int)(i % WQ);
        long long r = i / WQ;
        const int y = (int)(r % H);
        r /= H;
        const int c = (int)(r % C);
        const long long n = r / C;
        float2 ph[2];
#pragma unroll
        for (int col = 0; col < 2; ++col) {
            const int og = ((y & 1) * 2 + col) * C + c;
            const int g = og / per_group, o = og - g * per_group;
            ph[col] = *reinterpret_cast<const float2*>(dXs + ((((long long)g * N + n) * per_group + o) * H2 + (y >> 1)) * W2 + 2 * q);
        }
        float4* dst = reinterpret_cast<float4*>(dX + ((n * C + c) * H + y) * W + 4 * q);
        float4 v = make_float4(ph[0].x, ph[1].x, ph[0].y, ph[1].y);
        if (accumulate) {
            const float4 old = *dst;
            v = make_float4(old.x + v.x, old.y + v.y, old.z + v.z, old.w + v.w);
        }
        *dst = v;
    }
}
__global__ void subsample2_vec_kernel(const float* __restrict__ X, float* __restrict__ Xsub, long long NC, int H, int W,
                                      long long items) {
    griddep_wait();
    griddep_launch();
    const int H2 = H / 2, W2 = W / 2, WQ = W / 4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < items;
         i += (long long)gridDim.x * blockDim.x) {
        const int q = (int)(i % WQ);
        const long long r = i / WQ;
        const int ii = (int)(r % H2);
        const long long nc = r / H2;
        const float4 v = *reinterpret_cast<const float4*>(X + (nc * H + 2 * ii) * W + 4 * q);
        *reinterpret_cast<float2*>(Xsub + (nc * H2 + ii) * W2 + 2 * q) = make_float2(v.x, v.z);
    }
}
__global__ void upsample2_zero_vec_kernel(const float* __restrict__ dXsub, float* __restrict__ dX, int H, int W,
                                          long long items, int accumulate) {
    griddep_wait();
    griddep_launch();
    const int H2 = H / 2, W2 = W / 2, WQ = W / 4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < items;
         i += (long long)gridDim.x * blockDim.x) {
        const int q = (int)(i % WQ);
        const long long r = i / WQ;
        const int y = (int)(r % H);
        const long long nc = r / H;
        float4* dst = reinterpret_cast<float4*>(dX + (nc * H + y) * W + 4 * q);
        if (y & 1) {
            if (!accumulate) *dst = make_float4(0.f, 0.f, 0.f, 0.f);
            continue;
        }
        const float2 a = *reinterpret_cast<const float2*>(dXsub + (nc * H2 + (y >> 1)) * W2 + 2 * q);
        if (accumulate) {
            const float4 old = *dst;
            *dst = make_float4(old.x + a.x, old.y, old.z + a.y, old.w);
        } else {
            *dst = make_float4(a.x, 0.f, a.y, 0.f);
        }
    }
}
static bool vec_ok(const void* a, const void* b, int W) {
    return (W & 3) == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15u) == 0;
}

// 3xTF32 in one pass: X2[n][c] = X[n][c] and X2[n][C + c] = lo part of X[n][c] (x = hi + lo with hi the 19 bits the
// tensor core reads, lo = rna_tf32(x - hi)), four pixels per thread; X may be batch-strided, X2 is dense.
__global__ void tf32_split2_kernel(const float* __restrict__ X, float* __restrict__ X2, long long per4, long long x_batch,
                                   long long items) {
    griddep_wait();
    griddep_launch();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < items; i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / per4, r = i - n * per4;
        const float4 v = *reinterpret_cast<const float4*>(X + n * x_batch + 4 * r);
        float4 lo;
        const float in[4] = {v.x, v.y, v.z, v.w};
        float out[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float hi = __uint_as_float(__float_as_uint(in[e]) & 0xFFFFE000u);
            uint32_t q;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(q) : "f"(in[e] - hi));
            out[e] = __uint_as_float(q);
        }
        lo = make_float4(out[0], out[1], out[2], out[3]);
        float* dst = X2 + n * 8 * per4 + 4 * r;   // a sample of X2 holds 2 * per elements = 8 * per4 floats
        *reinterpret_cast<float4*>(dst) = v;
        *reinterpret_cast<float4*>(dst + 4 * per4) = lo;
    }
}

int relayout_grid(const cb_ctx* ctx, long long n) {
    long long g = (n + 255) / 256;
    const long long cap = (long long)ctx->sm_count * 16;
    return (int)(g > cap ? cap : (g < 1 ? 1 : g));
}

// Where a launch takes its stream, scratch and status word from: a cb_ctx or the static arrays of the allocation-free
// entry point.
struct ConvEnv {
    cudaStream_t stream;
    int sm_count, smem_optin;
    int* status;
};

// Geometry the tensor-core forward / data-gradient kernel covers; fills the derived sizes.
struct ConvPlan {
    int Cin, Cout, OCp, OCs, nsplit, NQ, CG, L, KS, shared_rows, nblocks, stages;
    int ew;      // epilogue warps of the kernel instantiation: 8 or 16
    int c_wrap = 0;  // set by the caller before planning: input-channel wrap of the 3xTF32 form (0 = none)
    int ks_max = 4;  // set by the caller before planning: most K steps a stage may carry
    int per_sm;  // CTAs the plan expects to share an SM (2 for narrow outputs with a small filter, else 1)
    size_t w_bytes;       // one CTA's slice of the packed filter
    size_t w_total_bytes; // the whole packed filter
    uint32_t block_bytes, stage_bytes;
};

// Development override of the output-channel split (1, 2 or 4); 0 = choose from the tile count.
int forced_nsplit() {
    static const int v = [] {
        const char* e = std::getenv("CB_CONV_NSPLIT");
        return e ? std::atoi(e) : 0;
    }();
    return v;
}

// Development override of the epilogue warp count (8 or 16); 0 = choose from the output width.
int forced_ew() {
    static const int v = [] {
        const char* e = std::getenv("CB_CONV_EW");
        return e ? std::atoi(e) : 0;
    }();
    return v;
}

int plan_conv(ConvPlan& q, int smem_optin, int sm_count, const float* X, int N, int Cin, int Cout, int IH, int IW, int FH,
              int FW, int pH, int pW) {
    // every tap must read within one pixel of the output position: offsets fh - pH and fw - pW in [-1, 1]
    if (FH < 1 || FH > 3 || FW < 1 || FW > 3 || pH < 0 || pH > 1 || pW < 0 || pW > 1) return CB_EUNSUPPORTED;
    if (FH - 1 - pH > 1 || FW - 1 - pW > 1) return CB_EUNSUPPORTED;
    if (FW == 1 && pW != 0) return CB_EUNSUPPORTED;  // the kernel's one-tap form reads the output's own column
    if (IW != 8 && IW != 16 && IW != 32) return CB_EUNSUPPORTED;
    q.L = 32 / IW;
    if (IH % q.L) return CB_EUNSUPPORTED;
    q.Cin = Cin;
    q.Cout = Cout;
    q.OCp = (q.Cout + 15) / 16 * 16;
    if (q.Cin < 1) return CB_EUNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(X) & 15u) != 0) return CB_EUNSUPPORTED;
    q.CG = (q.Cin + 31) / 32;
    q.w_total_bytes = (size_t)FH * q.CG * FW * q.OCp * kRowBytes;
    q.shared_rows = (q.L == 1 && IH % 4 == 0) ? 1 : 0;
    q.nblocks = q.shared_rows ? FH + 3 : FH * 4;
    const long long tiles = ((long long)N * (IH / q.L) + 3) / 4;
    const int cin8 = (q.Cin + 7) / 8;
    // Candidate splits of the output channels over 1, 2 or 4 CTAs per pixel tile: the widest split that still fits the
    // resident CTA slots in one wave wins (small feature maps then fill the GPU); each candidate must be launchable.
    int best = 0;
    ConvPlan bestq{};
    bool forced_hit = false;
    for (int ns = 1; ns <= 4 && !forced_hit; ns <<= 1) {
        // a four-way split only when forced or when nothing narrower fits the 256 accumulator columns (very wide outputs)
        if (ns == 4 && forced_nsplit() != 4 && best != 0) break;
        // a split that needs extra padding channels only when no narrower split fits at all
        if (q.OCp % (16 * ns) != 0 && best != 0) break;
        ConvPlan c = q;
        c.nsplit = ns;
        // the packed filter is padded to a whole number of 16-channel groups per CTA; channels past Cout are zero rows
        // and their outputs are dropped by the store
        c.OCp = (q.Cout + 16 * ns - 1) / (16 * ns) * (16 * ns);
        c.w_total_bytes = (size_t)FH * q.CG * FW * c.OCp * kRowBytes;
        c.OCs = c.OCp / ns;
        c.NQ = FW * c.OCs;
        if (c.NQ > 256) continue;
        c.w_bytes = (size_t)FH * c.CG * c.NQ * kRowBytes;
        // Two epilogue warps per TMEM lane quarter: with four, the waiting and draining warps took issue slots from the
        // one thread that feeds the tensor core and the wide layers ran 15 % slower. Narrow outputs with a small filter
        // are sized so that two CTAs fit one SM (shared memory and TMEM halves).
        c.ew = 8;
        if (forced_ew() == 8 || forced_ew() == 16) c.ew = forced_ew();
        const bool two_per_sm = c.OCs <= 32 && c.w_bytes <= 40 * 1024 && c.ew <= 8;
        const long long avail = two_per_sm ? (long long)(smem_optin < 113 * 1024 ? smem_optin : 113 * 1024) : (long long)smem_optin;
        const long long cap = avail - 4096 - (long long)c.w_bytes - 2048LL * c.ew;  // static shared memory, alignment slack;  // 2 KB of store staging per epilogue warp
        // as many K steps per stage as leaves at least 2 stages: fewer, larger TMA boxes measured faster than a deeper
        // pipeline of small ones
        c.KS = 0;
        for (int ks = 4; ks >= 1; ks >>= 1) {
            if (ks > cin8 && ks > 1) continue;
            if (ks > q.ks_max) continue;
            const long long st = cap / ((long long)c.nblocks * ks * kCB * kRowBytes);
            if (st >= 2) {
                c.KS = ks;
                c.stages = (int)(st > kConvMaxStages ? kConvMaxStages : st);
                break;
            }
        }
        if (c.KS == 0) continue;
        if ((cin8 + c.KS - 1) / c.KS * c.KS * FH > kMaxTileUmmas) continue;
        c.block_bytes = (uint32_t)c.KS * kCB * kRowBytes;
        c.stage_bytes = (uint32_t)c.nblocks * c.block_bytes;
        c.per_sm = two_per_sm ? 2 : 1;
        const long long slots = (long long)sm_count * c.per_sm;
        forced_hit = forced_nsplit() == ns;
        if (best == 0 || tiles * ns <= slots || forced_hit) {
            best = ns;
            bestq = c;
        }
    }
    if (best == 0) return CB_EUNSUPPORTED;
    q = bestq;
    return CB_OK;
}

// How the caller's filter becomes the packed filter of the convolution the kernel runs.
struct PackSpec {
    int mode, OC, IC, FHs, FWs, out_first, out_count;
};

PackJob make_job(const PackSpec& ps, const ConvPlan& q, const float* W, float* dst, int FH, int FW) {
    PackJob j{};
    j.W = W; j.Wp = dst;
    j.OC = ps.OC; j.IC = ps.IC; j.FHs = ps.FHs; j.FWs = ps.FWs; j.FHc = FH; j.FWc = FW;
    j.OCp = q.OCp; j.CG = q.CG; j.mode = ps.mode; j.out_first = ps.out_first; j.out_count = ps.out_count;
    j.total = (long long)q.w_total_bytes / 4;
    return j;
}

int launch_pack(cb_ctx* err_ctx, const ConvEnv& env, const PackJob& j) {
    int grid = (int)((j.total + 255) / 256);
    if (grid > env.sm_count * 8) grid = env.sm_count * 8;
    pack_filter_kernel<<<grid, 256, 0, env.stream>>>(j);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(err_ctx, e, "pack_filter_kernel launch");
    return CB_OK;
}

// Launches the kernel on an already packed filter: Y (N x q.Cout x IH x IW) = taps (FH, FW, pH, pW) over
// X (N x q.Cin x IH x IW). in_batch / out_batch: elements between consecutive images (0 = densely packed).
int launch_conv(cb_ctx* err_ctx, const ConvEnv& env, const ConvPlan& q, const float* packed, const float* X, float* Y,
                const ConvEpilogue& ep, int N, int IH, int IW, int FH, int FW, int pH, int pW, long long in_batch,
                long long out_batch) {
    ConvParams p{};
    p.N = N; p.Cin = q.Cin; p.H = IH; p.W = IW; p.Cout = q.Cout;
    p.FH = FH; p.FW = FW; p.pH = pH; p.pW = pW;
    p.OCs = q.OCs; p.nsplit = q.nsplit; p.NQ = q.NQ; p.CG = q.CG; p.KS = q.KS;
    p.c_wrap = q.c_wrap;
    p.NCB = (q.Cin + q.KS * kCB - 1) / (q.KS * kCB);
    p.L = q.L; p.LPI = IH / q.L;
    p.shared_rows = q.shared_rows; p.nblocks = q.nblocks;
    p.total_lines = (long long)N * p.LPI;
    if (p.total_lines > (1LL << 29)) return fail(err_ctx, CB_EUNSUPPORTED, "convolution: more than 2^29 lines of 32 pixels");
    p.tiles = (int)((p.total_lines + 3) / 4);
    p.stages = q.stages;
    int cols = 32;
    while (cols < 2 * q.NQ) cols <<= 1;
    p.tmem_cols = cols;
    p.w_bytes = (uint32_t)q.w_bytes;
    p.block_bytes = q.block_bytes;
    p.stage_bytes = q.stage_bytes;
    const uint64_t plane = (uint64_t)IH * IW;
    p.Out = Y;
    p.out_batch = out_batch ? out_batch : (long long)q.Cout * (long long)plane;
    p.ep = ep;
    p.status = env.status;
    {
        static const int forced = [] {
            const char* e = std::getenv("CB_CONV_ISSUE");  // development override: 0 one lane, 1 whole warp
            return e ? std::atoi(e) : -1;
        }();
        p.issue_uniform = forced >= 0 ? forced : (q.NQ >= 160 ? 1 : 0);
    }
    p.trace = err_ctx ? err_ctx->trace : nullptr;
#ifdef CB_TRACE
    {
        const char* e = std::getenv("CB_DBG");
        p.dbg = e ? std::atoi(e) : 0;
    }
#endif
    const uint64_t in_stride = (uint64_t)(in_batch ? in_batch : (long long)q.Cin * (long long)plane) * 4;
    if (in_stride & 15u) return fail(err_ctx, CB_EUNSUPPORTED, "convolution: the input batch stride must be a multiple of 4 floats");

    CUtensorMap tmIn, tmW;
    int rc;
    if (q.shared_rows) {
        // 32-wide maps: (w, channel, row, image) so that one box of FH+3 rows lands as [row][channel][128 B]
        uint64_t dims[4] = {32, (uint64_t)q.Cin, (uint64_t)IH, (uint64_t)N};
        uint64_t str[3] = {plane * 4, 128, in_stride};
        uint32_t box[4] = {32u, (uint32_t)(q.KS * kCB), (uint32_t)q.nblocks, 1u};
        rc = encode_tmap(err_ctx, &tmIn, X, 4, dims, str, box, nullptr, 129);
    } else {
        // planes flattened to (H*W, C, N): a box is 32 consecutive floats of 8*KS channel planes, starting at pixel
        // (row * W) — a multiple of 4 floats, as TMA requires of the innermost coordinate. Pixels before the plane's
        // first row or after its last one, and channels >= C, are out of bounds and read as zero. (A box whose inner
        // extent is below the 128-byte swizzle span would be padded to 128 bytes per inner row in shared memory, so
        // the (W, H) plane is never used as two tensor-map dimensions when W < 32.)
        uint64_t dims[3] = {plane, (uint64_t)q.Cin, (uint64_t)N};
        uint64_t str[2] = {plane * 4, in_stride};
        uint32_t box[3] = {32u, (uint32_t)(q.KS * kCB), 1u};
        rc = encode_tmap(err_ctx, &tmIn, X, 3, dims, str, box, nullptr, 129);
    }
    if (rc != CB_OK) return rc;
    {
        // packed filter as (32 channels, OCp rows, (fh, channel group, fw) planes): a box is FW planes of OCs rows
        const uint64_t planes = (uint64_t)FH * q.CG * FW;
        uint64_t dims[3] = {32, (uint64_t)q.OCp, planes};
        uint64_t str[2] = {128, (uint64_t)q.OCp * 128};
        uint32_t box[3] = {32, (uint32_t)q.OCs, (uint32_t)FW};
        rc = encode_tmap(err_ctx, &tmW, packed, 3, dims, str, box, nullptr, 128);
        if (rc != CB_OK) return rc;
    }
    // Results leave through TMA unless the epilogue needs the old output before a ReLU, or the output is not 16-byte
    // aligned in every plane and image (TMA's base and stride rules).
    const long long out_stride_b = p.out_batch * 4;
    p.tma_out = (ep.accumulate && ep.relu) ? 0 : (ep.accumulate ? 2 : 1);
    if ((reinterpret_cast<uintptr_t>(Y) & 15u) || (out_stride_b & 15)) p.tma_out = 0;
    CUtensorMap tmOut = tmIn;  // placeholder when unused
    if (p.tma_out) {
        uint64_t dims[3] = {plane, (uint64_t)q.Cout, (uint64_t)N};
        uint64_t str[2] = {plane * 4, (uint64_t)out_stride_b};
        uint32_t box[3] = {32u, 8u, 1u};
        rc = encode_tmap(err_ctx, &tmOut, Y, 3, dims, str, box, nullptr, 0);
        if (rc != CB_OK) return rc;
    }
    const size_t smem = q.w_bytes + (size_t)p.stages * q.stage_bytes + 2048u * (size_t)q.ew + 1024;
    // per device: the opt-in shared-memory size is raised to the maximum once (several host threads may race here)
    static std::once_flag attr_once[64];
    static cudaError_t attr_error[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const ConvParams);
    static const KernelFn kernels[2][4] = {
        {umma_conv_kernel<8, TAPS_1>, umma_conv_kernel<8, TAPS_3>, umma_conv_kernel<8, TAPS_2L>, umma_conv_kernel<8, TAPS_2R>},
        {umma_conv_kernel<16, TAPS_1>, umma_conv_kernel<16, TAPS_3>, umma_conv_kernel<16, TAPS_2L>, umma_conv_kernel<16, TAPS_2R>}};
    auto raise_limits = [&]() -> cudaError_t {
        for (int a = 0; a < 2; ++a)
            for (int b = 0; b < 4; ++b) {
                cudaError_t e = cudaFuncSetAttribute(kernels[a][b], cudaFuncAttributeMaxDynamicSharedMemorySize, env.smem_optin - 3072);
                if (e != cudaSuccess) return e;
            }
        return cudaSuccess;
    };
    cudaError_t attr_e;
    if (dev >= 0 && dev < 64) {
        std::call_once(attr_once[dev], [&] { attr_error[dev] = raise_limits(); });
        attr_e = attr_error[dev];
    } else {
        attr_e = raise_limits();
    }
    if (attr_e != cudaSuccess) return check_cuda(err_ctx, attr_e, "umma_conv_kernel attribute");
    const int slots = env.sm_count * q.per_sm;  // resident CTAs
    int per_split = slots / q.nsplit;
    if (per_split < 1) per_split = 1;
    if (per_split > p.tiles) per_split = p.tiles;
    const int grid = per_split * q.nsplit;
    const int taps = FW == 1 ? TAPS_1 : (FW == 3 ? TAPS_3 : (pW == 1 ? TAPS_2L : TAPS_2R));
    cudaError_t e = launch_dep_on(env.stream, err_ctx && err_ctx->pdl, kernels[q.ew == 8 ? 0 : 1][taps], dim3((unsigned)grid),
                                  dim3((unsigned)(64 + 32 * q.ew)), smem, tmIn, tmW, tmOut, p);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(err_ctx, e, "umma_conv_kernel launch");
    return CB_OK;
}

}  // namespace

int launch_space_to_depth2(cb_ctx* ctx, const float* X, float* Xs, int N, int C, int H, int W) {
    const long long n_el = (long long)N * C * H * W;
    cudaError_t e = vec_ok(X, Xs, W)
                        ? launch_dep(ctx, space_to_depth2_vec_kernel, dim3((unsigned)relayout_grid(ctx, n_el / 4)), dim3(256), 0, X, Xs, C, H, W, n_el / 4)
                        : launch_dep(ctx, space_to_depth2_kernel, dim3((unsigned)relayout_grid(ctx, n_el)), dim3(256), 0, X, Xs, C, H, W, n_el);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "space_to_depth2_kernel launch");
    ctx->launches += 1;
    return CB_OK;
}
int launch_subsample2(cb_ctx* ctx, const float* X, float* Xsub, long long NC, int H, int W) {
    const long long n_sub = NC * (H / 2) * (W / 2);
    const long long n_items = NC * (H / 2) * (W / 4);
    cudaError_t e = vec_ok(X, Xsub, W)
                        ? launch_dep(ctx, subsample2_vec_kernel, dim3((unsigned)relayout_grid(ctx, n_items)), dim3(256), 0, X, Xsub, NC, H, W, n_items)
                        : launch_dep(ctx, subsample2_kernel, dim3((unsigned)relayout_grid(ctx, n_sub)), dim3(256), 0, X, Xsub, NC, H, W, n_sub);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "subsample2_kernel launch");
    ctx->launches += 1;
    return CB_OK;
}

// ------------------------------------------------------------------------------------------ packed-filter cache
// With the cache on (cb_conv_cache_filters), a context keeps one packed copy per (filter pointer, geometry, pass) it
// has seen and re-packs it only after the caller announced a weight update: cb_filters_changed re-packs every cached
// filter in ONE launch, so a training step pays one pack launch instead of two per convolution. Filters the context's
// own update calls may have touched (cb_momentum*, cb_tensor_op) are re-packed lazily by the next convolution that
// uses them.
struct FilterCacheEntry {
    PackJob job;
    long long version;  // value of cb_ctx::filter_version when the packed copy was last written
};
struct FilterCache {
    std::vector<FilterCacheEntry> entries;
    PackJob* dev_table = nullptr;
    size_t dev_table_entries = 0;
    long long biggest = 0;
};

static bool same_job(const PackJob& a, const PackJob& b) {
    return a.W == b.W && a.OC == b.OC && a.IC == b.IC && a.FHs == b.FHs && a.FWs == b.FWs && a.FHc == b.FHc &&
           a.FWc == b.FWc && a.OCp == b.OCp && a.CG == b.CG && a.mode == b.mode && a.out_first == b.out_first &&
           a.out_count == b.out_count;
}

void filter_cache_destroy(cb_ctx* ctx) {
    FilterCache* fc = static_cast<FilterCache*>(ctx->filter_cache);
    if (!fc) return;
    for (FilterCacheEntry& e : fc->entries) cudaFree(e.job.Wp);
    if (fc->dev_table) cudaFree(fc->dev_table);
    delete fc;
    ctx->filter_cache = nullptr;
}

// Packed filter for this call: from the cache (packing it now if it is new or stale) or, with the cache off, packed
// into the context workspace.
static int packed_filter(cb_ctx* ctx, const ConvEnv& env, const ConvPlan& q, const PackSpec& ps, const float* W, int FH,
                         int FW, const float** out) {
    if (!ctx->filter_cache_on) {
        int rc = ensure_workspace(ctx, q.w_total_bytes);
        if (rc != CB_OK) return rc;
        const PackJob j = make_job(ps, q, W, static_cast<float*>(ctx->workspace), FH, FW);
        rc = launch_pack(ctx, env, j);
        if (rc != CB_OK) return rc;
        ctx->launches += 1;
        *out = j.Wp;
        return CB_OK;
    }
    if (!ctx->filter_cache) ctx->filter_cache = new FilterCache();
    FilterCache* fc = static_cast<FilterCache*>(ctx->filter_cache);
    PackJob want = make_job(ps, q, W, nullptr, FH, FW);
    FilterCacheEntry* hit = nullptr;
    for (FilterCacheEntry& e : fc->entries)
        if (same_job(e.job, want)) { hit = &e; break; }
    if (!hit) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(ctx->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return fail(ctx, CB_ENOMEM, "a convolution filter was seen for the first time while the stream is being captured: "
                                        "run the same calls once before the capture so that its packed copy exists");
        void* d = nullptr;
        cudaError_t e = cudaMalloc(&d, q.w_total_bytes);
        if (e != cudaSuccess) {
            check_cuda(ctx, e, "packed filter cudaMalloc");
            return CB_ENOMEM;
        }
        want.Wp = static_cast<float*>(d);
        fc->entries.push_back(FilterCacheEntry{want, -1});
        hit = &fc->entries.back();
    }
    if (hit->version != ctx->filter_version) {
        int rc = launch_pack(ctx, env, hit->job);
        if (rc != CB_OK) return rc;
        ctx->launches += 1;
        hit->version = ctx->filter_version;
    }
    *out = hit->job.Wp;
    return CB_OK;
}

// Re-packs every cached filter in one launch and marks them current.
int filter_cache_repack_all(cb_ctx* ctx) {
    ctx->filter_version += 1;
    FilterCache* fc = static_cast<FilterCache*>(ctx->filter_cache);
    if (!ctx->filter_cache_on || !fc || fc->entries.empty()) return CB_OK;
    if (fc->dev_table_entries != fc->entries.size()) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(ctx->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return CB_OK;  // filters first seen after the last table build: they re-pack lazily at their next use
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) return check_cuda(ctx, e, "filter table rebuild");
        if (fc->dev_table) cudaFree(fc->dev_table);
        fc->dev_table = nullptr;
        std::vector<PackJob> host(fc->entries.size());
        fc->biggest = 0;
        for (size_t i = 0; i < host.size(); ++i) {
            host[i] = fc->entries[i].job;
            if (host[i].total > fc->biggest) fc->biggest = host[i].total;
        }
        void* d = nullptr;
        e = cudaMalloc(&d, sizeof(PackJob) * host.size());
        if (e == cudaSuccess) e = cudaMemcpy(d, host.data(), sizeof(PackJob) * host.size(), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) return check_cuda(ctx, e, "filter table upload");
        fc->dev_table = static_cast<PackJob*>(d);
        fc->dev_table_entries = host.size();
    }
    int gx = (int)((fc->biggest + 255) / 256);
    if (gx > 64) gx = 64;
    if (gx < 1) gx = 1;
    cudaError_t e = launch_dep(ctx, pack_filter_table_kernel, dim3((unsigned)gx, (unsigned)fc->dev_table_entries), dim3(256), 0,
                               (const PackJob*)fc->dev_table);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "pack_filter_table_kernel launch");
    ctx->launches += 1;
    for (FilterCacheEntry& en : fc->entries) en.version = ctx->filter_version;
    return CB_OK;
}

static int conv_on_packed(cb_ctx* ctx, const ConvEnv& env, const ConvPlan& q, const PackSpec& ps, const float* W,
                          const float* X, float* Y, const ConvEpilogue& ep, int N, int IH, int IW, int FH, int FW, int pH,
                          int pW, long long in_batch, long long out_batch) {
    const float* packed = nullptr;
    int rc = packed_filter(ctx, env, q, ps, W, FH, FW, &packed);
    if (rc != CB_OK) return rc;
    rc = launch_conv(ctx, env, q, packed, X, Y, ep, N, IH, IW, FH, FW, pH, pW, in_batch, out_batch);
    if (rc != CB_OK) return rc;
    ctx->launches += 1;
    return CB_OK;
}

// 3xTF32 forward / data gradient in ONE pass of the tensor-core kernel (stride 1): x = x_hi + x_lo, w = w_hi + w_lo and
// y = x_hi w_hi + x_lo w_hi + x_hi w_lo are a single convolution over three groups of input channels, [x ; x_lo ; x]
// against [w ; w ; w_lo], because the tensor core itself takes the hi part of what it reads. One small pass writes
// X2 = [x ; x_lo] (dense scratch), the packed filter carries the three weight groups (cached like any other), and the
// kernel's producer reads channels [0, cin) a second time for the third group. Everything accumulates in one TMEM
// accumulator and leaves through the ordinary epilogue. CB_EUNSUPPORTED (nothing queued) when the channel count is not
// a multiple of 8 or the tripled filter does not fit; the caller then composes three passes.
int umma_conv_fwd_x3(cb_ctx* ctx, const float* W, const float* X, float* Y, const ConvEpilogue& ep, int N, int IC, int IH,
                     int IW, int OC, int FH, int FW, int pH, int pW, bool dgrad_of, long long in_batch, long long out_batch) {
    if (!((FH == 1 && pH == 0) || (FH == 3 && pH == 1))) return CB_EUNSUPPORTED;
    if (!((FW == 1 && pW == 0) || (FW == 3 && pW == 1))) return CB_EUNSUPPORTED;
    const int cin = dgrad_of ? OC : IC, cout = dgrad_of ? IC : OC;
    if (cin % 8 || ((long long)IH * IW) % 4) return CB_EUNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(X) & 15u) || (in_batch & 3)) return CB_EUNSUPPORTED;
    ConvEnv env{ctx->stream, ctx->sm_count, ctx->max_smem_optin, ctx->d_status};
    ConvPlan q{};
    q.c_wrap = 2 * cin;
    q.ks_max = (cin % 32 == 0) ? 4 : ((cin % 16 == 0) ? 2 : 1);  // a stage's channels stay inside one group
    int rc = plan_conv(q, ctx->max_smem_optin, ctx->sm_count, nullptr /* the scratch copy is aligned */, N, 3 * cin, cout, IH, IW,
                       FH, FW, pH, pW);
    if (rc != CB_OK) return rc;
    // A tripled 64-channel filter only fits when the output channels are split four ways; every CTA then re-reads the
    // input tile for 16 output channels, which pays on small maps (64->64 @8x8: 21 us against 36 composed) and not on
    // large ones (64->64 @32x32: 207 us against 141).
    if (q.nsplit > 2 && ((long long)N * (IH / q.L) + 3) / 4 > ctx->sm_count) return CB_EUNSUPPORTED;
    const long long per = (long long)cin * IH * IW;
    rc = ensure_workspace3(ctx, (size_t)N * 2 * per * sizeof(float));
    if (rc != CB_OK) return rc;
    float* X2 = static_cast<float*>(ctx->workspace3);
    const long long items = (long long)N * (per / 4);
    cudaError_t e = launch_dep(ctx, tf32_split2_kernel, dim3((unsigned)relayout_grid(ctx, items)), dim3(256), 0, X, X2, per / 4,
                               in_batch ? in_batch : per, items);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "tf32_split2_kernel launch");
    ctx->launches += 1;
    const PackSpec ps{dgrad_of ? PACK_DGRAD_X3 : PACK_FWD_X3, OC, IC, FH, FW, 0, 0};
    rc = conv_on_packed(ctx, env, q, ps, W, X2, Y, ep, N, IH, IW, FH, FW, pH, pW, 2 * per, out_batch);
    if (rc != CB_OK) return rc;
    ctx->last_kernel = "umma_3xtf32";
    return CB_OK;
}

// Forward (dgrad_of = false: Y = conv(W, X), full epilogue) or data gradient (dgrad_of = true: X is dY, Y is dX; of the
// epilogue only `accumulate` applies). Returns CB_EUNSUPPORTED, before any work is queued, for geometries outside the
// tensor-core kernel.
int umma_conv_fwd(cb_ctx* ctx, const float* W, const float* X, float* Y, const ConvEpilogue& ep, int N, int IC, int IH,
                  int IW, int OC, int FH, int FW, int sH, int sW, int pH, int pW, bool dgrad_of, long long in_batch,
                  long long out_batch) {
    ConvEnv env{ctx->stream, ctx->sm_count, ctx->max_smem_optin, ctx->d_status};
    ConvPlan q{};
    int rc;
    if (sH == 1 && sW == 1) {
        // ---- stride 1: 1x1 (pad 0) or 3x3 (pad 1) per axis
        if (!((FH == 1 && pH == 0) || (FH == 3 && pH == 1))) return CB_EUNSUPPORTED;
        if (!((FW == 1 && pW == 0) || (FW == 3 && pW == 1))) return CB_EUNSUPPORTED;
        rc = plan_conv(q, ctx->max_smem_optin, ctx->sm_count, X, N, dgrad_of ? OC : IC, dgrad_of ? IC : OC, IH, IW, FH, FW, pH, pW);
        if (rc != CB_OK) return rc;
        const PackSpec ps{dgrad_of ? PACK_DGRAD : PACK_FWD, OC, IC, FH, FW, 0, 0};
        rc = conv_on_packed(ctx, env, q, ps, W, X, Y, ep, N, IH, IW, FH, FW, pH, pW, in_batch, out_batch);
        if (rc != CB_OK) return rc;
        ctx->last_kernel = "umma_tf32";
        return CB_OK;
    }
    // ---- stride 2 (square): 3x3 pad 1 through the 4 input phases, 1x1 pad 0 through phase (0,0); dense tensors only
    if (sH != 2 || sW != 2 || FH != FW || pH != pW || (IH & 1) || (IW & 1)) return CB_EUNSUPPORTED;
    if (!((FH == 3 && pH == 1) || (FH == 1 && pH == 0))) return CB_EUNSUPPORTED;
    if (in_batch || out_batch) return CB_EUNSUPPORTED;
    const int H2 = IH / 2, W2 = IW / 2;
    const long long plane2 = (long long)H2 * W2;
    const ConvEpilogue plain{};
    if (FH == 1) {
        // Y = W * X[:, :, ::2, ::2]  /  dX[:, :, ::2, ::2] = W^T dY, zero elsewhere
        rc = plan_conv(q, ctx->max_smem_optin, ctx->sm_count, dgrad_of ? X : nullptr /* the sub-sampled copy is aligned */, N,
                       dgrad_of ? OC : IC, dgrad_of ? IC : OC, H2, W2, 1, 1, 0, 0);
        if (rc != CB_OK) return rc;
        const size_t sub_bytes = (size_t)N * IC * plane2 * sizeof(float);
        rc = ensure_workspace2(ctx, sub_bytes);
        if (rc != CB_OK) return rc;
        float* sub = static_cast<float*>(ctx->workspace2);
        const PackSpec ps{dgrad_of ? PACK_DGRAD : PACK_FWD, OC, IC, 1, 1, 0, 0};
        if (!dgrad_of) {
            rc = launch_subsample2(ctx, X, sub, (long long)N * IC, IH, IW);
            if (rc == CB_OK) rc = conv_on_packed(ctx, env, q, ps, W, sub, Y, ep, N, H2, W2, 1, 1, 0, 0, 0, 0);
        } else {
            rc = conv_on_packed(ctx, env, q, ps, W, X /* = dY */, sub, plain, N, H2, W2, 1, 1, 0, 0, 0, 0);
            const long long n_full = (long long)N * IC * IH * IW;
            if (rc == CB_OK) {
                if (vec_ok(sub, Y, IW))
                    launch_dep(ctx, upsample2_zero_vec_kernel, dim3((unsigned)relayout_grid(ctx, n_full / 4)), dim3(256), 0,
                               (const float*)sub, Y /* = dX */, IH, IW, n_full / 4, ep.accumulate ? 1 : 0);
                else
                    launch_dep(ctx, upsample2_zero_kernel, dim3((unsigned)relayout_grid(ctx, n_full)), dim3(256), 0, (const float*)sub,
                               Y /* = dX */, IH, IW, n_full, ep.accumulate ? 1 : 0);
                ctx->launches += 1;
            }
        }
        if (rc != CB_OK) return rc;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return check_cuda(ctx, e, "stride-2 1x1 convolution");
        ctx->last_kernel = "umma_tf32";
        return CB_OK;
    }
    const int C4 = 4 * IC;
    const size_t s2d_bytes = (size_t)N * C4 * plane2 * sizeof(float);
    if (!dgrad_of) {
        // Xs[n][phase*IC + c] = X[n][c][phase rows / cols]; Y = 2x2 convolution (taps at -1, 0) over the 4*IC planes
        rc = ensure_workspace2(ctx, s2d_bytes);
        if (rc != CB_OK) return rc;
        float* Xs = static_cast<float*>(ctx->workspace2);
        rc = plan_conv(q, ctx->max_smem_optin, ctx->sm_count, Xs, N, C4, OC, H2, W2, 2, 2, 1, 1);
        if (rc != CB_OK) return rc;
        rc = launch_space_to_depth2(ctx, X, Xs, N, IC, IH, IW);
        if (rc != CB_OK) return rc;
        const PackSpec ps{PACK_S2_FWD, OC, IC, 3, 3, 0, 0};
        rc = conv_on_packed(ctx, env, q, ps, W, Xs, Y, ep, N, H2, W2, 2, 2, 1, 1, 0, 0);
        if (rc != CB_OK) return rc;
        ctx->last_kernel = "umma_tf32";
        return CB_OK;
    }
    // data gradient: dXs (4*IC phase planes) = adjoint 2x2 convolution (taps at 0, +1) over dY, in channel groups small
    // enough for the accumulator (FW * roundup16(channels) <= 256), then interleaved back into dX
    int groups = 1;
    while (groups <= 4 && 2 * ((C4 / groups + 15) / 16 * 16) > 256) groups *= 2;
    if (groups > 4) return CB_EUNSUPPORTED;
    const int per_group = C4 / groups;
    rc = ensure_workspace2(ctx, s2d_bytes);
    if (rc != CB_OK) return rc;
    float* dXs = static_cast<float*>(ctx->workspace2);
    rc = plan_conv(q, ctx->max_smem_optin, ctx->sm_count, X /* = dY */, N, OC, per_group, H2, W2, 2, 2, 0, 0);
    if (rc != CB_OK) return rc;
    for (int g = 0; g < groups; ++g) {
        const PackSpec ps{PACK_S2_DGRAD, OC, IC, 3, 3, g * per_group, per_group};
        rc = conv_on_packed(ctx, env, q, ps, W, X /* = dY */, dXs + (size_t)g * N * per_group * plane2, plain, N, H2, W2, 2, 2,
                            0, 0, 0, 0);
        if (rc != CB_OK) return rc;
    }
    const long long n_full = (long long)N * IC * IH * IW;
    cudaError_t e = vec_ok(dXs, Y, IW)
                        ? launch_dep(ctx, depth_to_space2_vec_kernel, dim3((unsigned)relayout_grid(ctx, n_full / 4)), dim3(256), 0,
                                     (const float*)dXs, Y /* = dX */, N, IC, IH, IW, per_group, n_full / 4, ep.accumulate ? 1 : 0)
                        : launch_dep(ctx, depth_to_space2_kernel, dim3((unsigned)relayout_grid(ctx, n_full)), dim3(256), 0,
                                     (const float*)dXs, Y /* = dX */, N, IC, IH, IW, per_group, n_full, ep.accumulate ? 1 : 0);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "depth_to_space2_kernel launch");
    ctx->launches += 1;
    ctx->last_kernel = "umma_tf32";
    return CB_OK;
}

// ------------------------------------------------------------------------------------------ allocation-free forward
// cb_conv_fwd_noalloc: the tensor-core forward convolution for callers that must not allocate device memory —
// code running under a memory manager that has already claimed the whole GPU (so cudaMalloc would fail), code
// on a latency-critical path where cudaMalloc's implicit device synchronisation is unacceptable, and code that
// runs while a stream is being captured (allocation calls are not allowed there). The ordinary entry point keeps
// its packed filter in a context workspace that grows with cudaMalloc; this one keeps it in the fixed array below,
// which every GPU that loads the library holds from load to exit (160 KiB + one status word).
namespace {

constexpr int kNoAllocPackFloats = 40960;  // 160 KiB: enough for a 64 -> 64 channel 3x3 filter (147 456 bytes)
static __device__ __align__(256) float g_noalloc_pack[kNoAllocPackFloats];
static __device__ __align__(16) int g_noalloc_status;

struct NoAllocDevice {
    std::once_flag once;
    cudaError_t init_error = cudaSuccess;
    int major = 0;
    float* pack = nullptr;  // device address of g_noalloc_pack on this GPU (the symbol itself is a host stand-in)
    int* status = nullptr;
    int sm_count = 0;
    int smem_optin = 0;
};
constexpr int kNoAllocMaxDevices = 64;
NoAllocDevice g_noalloc_dev[kNoAllocMaxDevices];

int noalloc_fail(char* err, int err_len, int code, const char* msg) {
    if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s", msg);
    return code;
}

// Makes `device` current for the duration of a call and puts the caller's device back on every return path.
struct DeviceScope {
    int prev = -1;
    cudaError_t error;
    explicit DeviceScope(int device) {
        error = cudaGetDevice(&prev);
        if (error == cudaSuccess && prev != device) error = cudaSetDevice(device);
    }
    ~DeviceScope() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

// Once per device, with that device current: resolves the device addresses of the static arrays and reads the
// attributes the launch needs. Safe when several host threads make their first call at the same time.
NoAllocDevice* noalloc_device(int device, char* err, int err_len, int* rc) {
    NoAllocDevice& d = g_noalloc_dev[device];
    std::call_once(d.once, [&] {
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.pack), g_noalloc_pack);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status), g_noalloc_status);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, device);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
        d.init_error = e;
    });
    if (d.init_error != cudaSuccess) {
        *rc = noalloc_fail(err, err_len, CB_ECUDA, cudaGetErrorString(d.init_error));
        return nullptr;
    }
    if (d.major != 10) {
        *rc = noalloc_fail(err, err_len, CB_EUNSUPPORTED, "this library only carries sm_100a code");
        return nullptr;
    }
    return &d;
}

}  // namespace
}  // namespace cb

extern "C" int cb_conv_fwd_noalloc(int device, void* cuda_stream, const float* W, const float* X, float* Y,
                                   const float* bias, int N, int IC, int IH, int IW, int OC, int FH, int FW, int sH,
                                   int sW, int pH, int pW, int relu, char* err, int err_len) {
    using namespace cb;
    if (err && err_len > 0) err[0] = 0;
    if (device < 0 || device >= kNoAllocMaxDevices) return noalloc_fail(err, err_len, CB_EINVAL, "device index out of range");
    if (N < 0 || IC < 1 || OC < 1 || IH < 1 || IW < 1) return noalloc_fail(err, err_len, CB_EINVAL, "bad extent");
    if (!W || !X || !Y) return noalloc_fail(err, err_len, CB_EINVAL, "null operand");
    if (sH != 1 || sW != 1 || !((FH == 1 && pH == 0) || (FH == 3 && pH == 1)) ||
        !((FW == 1 && pW == 0) || (FW == 3 && pW == 1)) || (IW != 8 && IW != 16 && IW != 32) || (IH % (32 / IW)) ||
        (reinterpret_cast<uintptr_t>(X) & 15u))
        return noalloc_fail(err, err_len, CB_EUNSUPPORTED,
                            "cb_conv_fwd_noalloc covers stride 1, 1x1 (pad 0) / 3x3 (pad 1) filters, map width 8, 16 or 32 "
                            "and a 16-byte aligned input");
    const size_t w_need = (size_t)FH * ((IC + 31) / 32) * FW * ((OC + 15) / 16 * 16) * kRowBytes;
    if (FW * ((OC + 15) / 16 * 16) > 256) return noalloc_fail(err, err_len, CB_EUNSUPPORTED, "FW * OC (rounded up to 16) exceeds 256");
    if (w_need > sizeof(float) * (size_t)kNoAllocPackFloats) {
        char msg[200];
        snprintf(msg, sizeof(msg), "packed filter needs %zu bytes; the static scratch of cb_conv_fwd_noalloc holds %zu",
                 w_need, sizeof(float) * (size_t)kNoAllocPackFloats);
        return noalloc_fail(err, err_len, CB_EINVAL, msg);
    }
    if (N == 0) return CB_OK;

    DeviceScope scope(device);
    if (scope.error != cudaSuccess) return noalloc_fail(err, err_len, CB_ECUDA, cudaGetErrorString(scope.error));
    int rc = CB_OK;
    NoAllocDevice* d = noalloc_device(device, err, err_len, &rc);
    if (!d) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    ConvPlan q{};
    if (plan_conv(q, d->smem_optin, d->sm_count, X, N, IC, OC, IH, IW, FH, FW, pH, pW) != CB_OK)
        return noalloc_fail(err, err_len, CB_EUNSUPPORTED, "geometry outside the tensor-core convolution kernel");
    // The scratch keeps the previous call's contents: the pack kernel rewrites all w_bytes (padding included). The
    // status word is NOT cleared here, so that a device-side timeout of an earlier call stays visible until
    // cb_conv_fwd_noalloc_status reads (and clears) it.
    ConvEnv env{stream, d->sm_count, d->smem_optin, d->status};
    const PackSpec ps{PACK_FWD, OC, IC, FH, FW, 0, 0};
    cb_ctx messages;  // host-side only: collects the text of a CUDA / tensor-map error; owns no device memory
    messages.device = device;
    ConvEpilogue ep{};
    ep.bias = bias;
    ep.relu = relu ? 1 : 0;
    rc = launch_pack(&messages, env, make_job(ps, q, W, d->pack, FH, FW));
    if (rc == CB_OK) rc = launch_conv(&messages, env, q, d->pack, X, Y, ep, N, IH, IW, FH, FW, pH, pW, 0, 0);
    if (rc != CB_OK)
        return noalloc_fail(err, err_len, rc, messages.last_error.empty() ? "kernel launch or tensor map encoding failed"
                                                                          : messages.last_error.c_str());
    return CB_OK;
}

extern "C" int cb_conv_fwd_noalloc_status(int device, void* cuda_stream, char* err, int err_len) {
    using namespace cb;
    if (err && err_len > 0) err[0] = 0;
    if (device < 0 || device >= kNoAllocMaxDevices) return noalloc_fail(err, err_len, CB_EINVAL, "device index out of range");
    DeviceScope scope(device);
    if (scope.error != cudaSuccess) return noalloc_fail(err, err_len, CB_ECUDA, cudaGetErrorString(scope.error));
    int rc = CB_OK;
    NoAllocDevice* d = noalloc_device(device, err, err_len, &rc);
    if (!d) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    cudaError_t e = cudaStreamSynchronize(stream);
    int st = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&st, d->status, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return noalloc_fail(err, err_len, CB_ECUDA, cudaGetErrorString(e));
    if (st != 0) {
        e = cudaMemsetAsync(d->status, 0, sizeof(int), stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        char msg[160];
        snprintf(msg, sizeof(msg), "a bounded device-side wait of cb_conv_fwd_noalloc expired: device status %d (%s)", st,
                 status_name(st));
        return noalloc_fail(err, err_len, CB_ETIMEOUT, msg);
    }
    return CB_OK;
}
