// Tensor-core implicit-GEMM convolution for sm_100a (TF32 mode), NCHW fp32, no materialised im2col.
//
// Forward and data-gradient run the same kernel: D[pixel][oc] = sum over (tap, c) of In[n, c, oh+fh-pH, ow+fw-pW]
// * Wp[tap][oc][c]. The 128 TMEM lanes of an accumulator are 128 output pixels (UMMA M), the columns are the output
// channels (UMMA N = OC rounded up to 16), K walks 8 input channels of one filter tap per tcgen05.mma.
//
//  * Pixels are grouped in "lines" of 32 consecutive floats of one channel plane (32/W image rows of a W-wide map,
//    W in {8,16,32}); a CTA tile is 4 lines. For each filter row fh and line, one TMA box (32 pixels of the
//    flattened H*W plane, 8 channels) of the NCHW input lands as an [8 channels][128 bytes] block — exactly the MN-major operand layout the tensor
//    core reads (128-byte swizzle with 32-byte atoms). Rows above / below the image are out of bounds for the
//    tensor map and arrive as zeros, which is the vertical padding.
//  * A TMA box may not start at an odd column (its innermost coordinate must be 16-byte aligned), so the
//    horizontal taps cannot be fetched as shifted boxes. They are not shifted on the input side at all: the three
//    horizontal taps of a filter row are folded into the UMMA N dimension (N = 3 x OC, accumulator column
//    fw*OCp + oc holds the partial sum of tap fw evaluated at the UNSHIFTED pixel), and the epilogue adds
//    D0[x-1] + D1[x] + D2[x+1] with two warp shuffles per value; lanes at a row edge take zero instead, which is
//    the horizontal padding. A pipeline stage is therefore only the centre copy of the input rows.
//  * The filter is packed once per CTA into [fh][32-channel group][fw][oc][32 channels] (K-major rows of 128 bytes,
//    zero padded, 128-byte swizzle) and stays resident in shared memory for the whole persistent CTA. The sixteen
//    epilogue warps, idle until the first tile completes, build it straight from the caller's filter (coalesced
//    reads, scattered 4-byte shared-memory writes), so forward and data gradient need no scratch buffer. (The
//    allocation-free entry point keeps the older route: a pack kernel writes a scratch copy that TMA then loads.)
//    For the data gradient the pack transposes the channel roles and rotates the filter by 180 degrees
//    (seblas/operations/cuConv.cu:321-326 does the same rotation on the fly).
//  * Epilogue (16 warps, 4 per TMEM lane quarter): tcgen05.ld, tap combine, + bias, ReLU, and stores in which the 32
//    lanes of a warp write 128 contiguous bytes.
//
// Covered geometry: stride 1, filter 1x1 (pad 0) or 3x3 (pad 1) per axis, W in {8,16,32}, (32/W) | H,
// FW * OC(rounded to 16) <= 256, packed filter <= ~150 KB. Everything else is served by the CUDA-core kernels in conv_simt.cu.
#include <cstdio>

#include "cb_internal.h"
#include "cb_ptx.cuh"

namespace cb {
namespace {

constexpr int kCB = 8;          // input channels per UMMA K step
constexpr int kMaxStages = 8;
constexpr int kRowBytes = 128;  // one line of 32 floats

struct ConvParams {
    int N, Cin, H, W, Cout;   // "input" and "output" of this pass (forward: X -> Y, dgrad: dY -> dX)
    int FH, FW, pH, pW;       // taps and padding: tap (fh, fw) reads the input at offset (fh - pH, fw - pW), each in [-1, 1]
    int OCp;                  // Cout rounded up to 16
    int NQ;                   // UMMA N = FW * OCp
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
    uint32_t w_bytes;         // resident packed filter
    uint32_t block_bytes;     // one line of a stage: 8 * KS channels x 128 B
    uint32_t stage_bytes;     // nblocks * block_bytes
    float* Out;
    const float* bias;
    int relu;
    int* status;
    // filter packing done by the CTA itself (0: the packed filter is fetched by TMA from a scratch buffer)
    int pack_in_kernel, pack_mode, OCs, ICs, FHs, FWs, out_first, out_count;
    const float* Wsrc;
    long long* trace;
};

struct __align__(8) ConvSmem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tfull[2];
    uint64_t tempty[2];
    uint64_t wbar;
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, int lane, volatile int* abort_flag,
                                          int* status, int code) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, status, code) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Source filter tap of the stride-2 convolution that lands on (input phase, tap of the 2x2 phase convolution):
// with ih = 2 oh + fh - 1, tap fh = 0 reads phase 1 at row oh - 1, fh = 1 phase 0 at row oh, fh = 2 phase 1 at row oh.
__device__ __forceinline__ int s2_tap(int phase, int t) { return phase == 1 ? (t == 0 ? 0 : 2) : (t == 1 ? 1 : -1); }

enum { PACK_FWD = 0, PACK_DGRAD = 1, PACK_S2_FWD = 2, PACK_S2_DGRAD = 3 };

// Inverse of s2_tap: source tap f of the 3x3 stride-2 filter -> (input phase, tap of the 2x2 phase convolution).
__device__ __forceinline__ void s2_untap(int f, int& phase, int& t) {
    phase = (f == 1) ? 0 : 1;
    t = (f == 0) ? 0 : 1;
}

// Epilogue warps are a template parameter of the kernel: 16 (4 per TMEM lane quarter) for wide outputs, 8 for outputs
// of at most 32 channels, where two such CTAs share an SM so that their UMMA chains (each serial on its accumulator)
// overlap.

template <int CH>
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[CH]) {
    if constexpr (CH == 32) tmem_ld32(taddr, r);
    else if constexpr (CH == 16) tmem_ld16(taddr, r);
    else tmem_ld8(taddr, r);
}

// One chunk of CH output channels of a tile's epilogue: the FW horizontal taps were accumulated at the unshifted
// pixel in column blocks fw*OCp + oc; tap fw reads column ow + (fw - pW), so its partial sum sits (fw - pW) lanes
// away. Lanes that would read across a row edge take zero instead (the horizontal padding).
template <int CH>
__device__ __forceinline__ void conv_epilogue_chunk(const ConvParams& p, uint32_t t_row, int c, float* out,
                                                    long long plane, bool valid, bool has_left, bool has_right) {
    uint32_t r0[CH], r1[CH], r2[CH];
    tmem_ld_n<CH>(t_row + (uint32_t)c, r0);
    if (p.FW > 1) tmem_ld_n<CH>(t_row + (uint32_t)(p.OCp + c), r1);
    if (p.FW > 2) tmem_ld_n<CH>(t_row + (uint32_t)(2 * p.OCp + c), r2);
    tmem_ld_wait();
    float v[CH];
#pragma unroll
    for (int e = 0; e < CH; ++e) v[e] = 0.f;
    for (int fw = 0; fw < p.FW; ++fw) {
        const int d = fw - p.pW;  // warp-uniform
#pragma unroll
        for (int e = 0; e < CH; ++e) {
            const float x = __uint_as_float(fw == 0 ? r0[e] : (fw == 1 ? r1[e] : r2[e]));
            if (d == 0) {
                v[e] += x;
            } else if (d < 0) {
                const float up = __shfl_up_sync(0xffffffffu, x, 1);
                v[e] += has_left ? up : 0.f;
            } else {
                const float dn = __shfl_down_sync(0xffffffffu, x, 1);
                v[e] += has_right ? dn : 0.f;
            }
        }
    }
    if (valid) {
#pragma unroll
        for (int e = 0; e < CH; ++e) {
            const int oc = c + e;
            if (oc < p.Cout) {
                float y = v[e];
                if (p.bias) y += __ldg(p.bias + oc);
                if (p.relu) y = fmaxf(y, 0.f);
                out[(long long)oc * plane] = y;
            }
        }
    }
}

template <int kEpiWarps>
__global__ void __launch_bounds__(64 + 32 * kEpiWarps, kEpiWarps == 8 ? 2 : 1)
    umma_conv_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmW,
                     const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ ConvSmem cs;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int* abort_flag = &cs.abort_flag;

    const uint32_t w_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t st_base = w_base + p.w_bytes;

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
        mbar_init(smem_u32(&cs.wbar), p.pack_in_kernel ? 32 * kEpiWarps : 1);
        mbar_init(smem_u32(&cs.drain), 1);
        mbar_fence_init();
        tma_prefetch_desc(&tmIn);
        if (!p.pack_in_kernel) tma_prefetch_desc(&tmW);
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
    uint32_t armed = 0, armed_parity = 0;  // producer lane: stages armed at least once / parity of their last arming
    if (threadIdx.x == 0) CB_TRACE_EVENT(p.trace, 2);

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0 && !p.pack_in_kernel) {
            // resident filter: one box [FW*OCp rows][32 channels] per (filter row, channel group)
            const uint32_t wbar = smem_u32(&cs.wbar);
            mbar_expect_tx(wbar, p.w_bytes);
            const int boxes = p.FH * p.CG;
            for (int b = 0; b < boxes; ++b)
                tma_load_3d(w_base + (uint32_t)b * p.NQ * kRowBytes, &tmW, wbar, 0, b * p.NQ, 0);
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
                    const uint32_t dst0 = st_base + s * p.stage_bytes;
                    mbar_expect_tx(full, p.stage_bytes);
                    armed |= 1u << s;
                    armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
                    const int c0 = cb * p.KS * kCB;
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
        // One thread feeds the tensor core: descriptor constants are hoisted and each UMMA costs a few integer adds.
        const uint32_t idesc = umma_idesc_tf32(128, (uint32_t)p.NQ, 1u, 0u);
        // P: 4 lines x [8 channels][128 B], MN-major: block_bytes between lines (LBO), 512 B per 4 channel rows (SBO)
        const uint64_t descP0 = umma_smem_desc(0, p.block_bytes, 512u, UMMA_SW_128B_BASE32B);
        // Q: packed filter rows [(fw, oc)][32 channels], K-major 128-byte rows
        const uint64_t descQ0 = umma_smem_desc(w_base, 16u, 1024u, UMMA_SW_128B);
        const uint32_t blk_units = p.block_bytes >> 4;               // descriptor address units (16 B) per line block
        const uint32_t fh_blocks = p.shared_rows ? 1u : 4u;          // blocks between consecutive filter rows
        const uint32_t q_group_units = (uint32_t)p.NQ * (kRowBytes >> 4);  // one (filter row, 32-channel group) of Q
        uint32_t s = 0, ph = 0, lt = 0;
        bool ok = warp_wait(smem_u32(&cs.wbar), 0, lane, abort_flag, p.status, CBK_TIMEOUT_FULL);
        if (lane == 0) CB_TRACE_EVENT(p.trace, 4);
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
                tc_fence_after();
                if (lane == 0 && lt == 0 && cb == 0) CB_TRACE_EVENT(p.trace, 5);
                if (lane == 0) {
                    const uint64_t pbase = descP0 + (uint64_t)(((st_base + s * p.stage_bytes) >> 4) & 0x3FFFu);
                    uint32_t accumulate = cb == 0 ? 0u : 1u;
                    for (int fh = 0; fh < p.FH; ++fh) {
                        const uint64_t dPf = pbase + (uint64_t)((uint32_t)fh * fh_blocks * blk_units);
                        const uint32_t q_fh = (uint32_t)(fh * p.CG) * q_group_units;
                        for (int kk = 0; kk < p.KS; ++kk) {
                            const uint32_t ks = (uint32_t)(cb * p.KS + kk);  // global K step: channels [8 ks, 8 ks + 8)
                            umma_tf32(d_tmem, dPf + (uint64_t)(kk * 64), descQ0 + (uint64_t)(q_fh + (ks >> 2) * q_group_units + (ks & 3u) * 2u),
                                      idesc, accumulate);
                            accumulate = 1u;
                        }
                    }
                    tc_commit(smem_u32(&cs.empty[s]));
                    if (cb == p.NCB - 1) tc_commit(smem_u32(&cs.tfull[a]));
                    if (lt == 0 && cb == p.NCB - 1) CB_TRACE_EVENT(p.trace, 6);
                }
                __syncwarp();
                if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..17)
        // One scheduler cannot hide the shuffle and store latencies of a single warp, so every TMEM lane quarter is
        // served by four warps that split the channel chunks between them.
        const int quarter = warp & 3;
        const int slot = (warp - 2) >> 2;
        if (p.pack_in_kernel) {
            // The epilogue warps are idle until the first tile completes: they build the resident packed filter
            // straight from the caller's OC x IC x FH x FW filter (coalesced reads, scattered 4-byte writes into the
            // 128-byte-swizzled K-major rows), so no separate pack kernel or scratch buffer is needed.
            const int te = threadIdx.x - 64, ne = 32 * kEpiWarps;
            for (uint32_t v = (uint32_t)te; v < (p.w_bytes >> 4); v += (uint32_t)ne)
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(w_base + v * 16u), "r"(0u) : "memory");
            asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
            const int taps_s = p.FHs * p.FWs;
            const int total_src = p.OCs * p.ICs * taps_s;
#pragma unroll 4
            for (int j = te; j < total_src; j += ne) {
                const int tap = j % taps_s, r = j / taps_s;
                const int ch_s = r % p.ICs, o_s = r / p.ICs;
                const int fh_s = tap / p.FWs, fw_s = tap - fh_s * p.FWs;
                int fh, fw, o, ch;
                bool keep = true;
                if (p.pack_mode == PACK_FWD) {
                    fh = fh_s; fw = fw_s; o = o_s; ch = ch_s;
                } else if (p.pack_mode == PACK_DGRAD) {
                    fh = p.FHs - 1 - fh_s; fw = p.FWs - 1 - fw_s; o = ch_s; ch = o_s;
                } else {
                    int ph, pw, th, tw;
                    s2_untap(fh_s, ph, th);
                    s2_untap(fw_s, pw, tw);
                    const int og = (ph * 2 + pw) * p.ICs + ch_s;
                    if (p.pack_mode == PACK_S2_FWD) {
                        fh = th; fw = tw; o = o_s; ch = og;
                    } else {
                        fh = 1 - th; fw = 1 - tw; o = og - p.out_first; ch = o_s;
                        keep = o >= 0 && o < p.out_count;
                    }
                }
                if (keep) {
                    const uint32_t R = (uint32_t)(((fh * p.CG + (ch >> 5)) * p.FW + fw) * p.OCp + o);
                    const uint32_t c = (uint32_t)ch & 31u;
                    const uint32_t addr = w_base + R * kRowBytes + (((c >> 2) ^ (R & 7u)) << 4) + ((c & 3u) << 2);
                    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(__ldg(p.Wsrc + j)) : "memory");
                }
            }
            fence_proxy_async_smem();
            mbar_arrive(smem_u32(&cs.wbar));
            if (threadIdx.x == 64) CB_TRACE_EVENT(p.trace, 3);
        }
        uint32_t lt = 0;
        bool ok = true;
        const long long plane = (long long)p.H * p.W;
        const int col = lane & (p.W - 1);
        const bool has_left = col > 0, has_right = col < p.W - 1;
        for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++lt) {
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
            float* out = p.Out + ((long long)n * p.Cout * p.H + h0) * p.W + lane;
            const uint32_t t_row = tmem_base + a * acc_stride + ((uint32_t)(32 * quarter) << 16);
            for (int c = slot * 8; c < p.OCp; c += 8 * (kEpiWarps / 4))
                conv_epilogue_chunk<8>(p, t_row, c, out, plane, valid, has_left, has_right);
            tc_fence_before();
            mbar_arrive(smem_u32(&cs.tempty[a]));
            if (threadIdx.x == 64 && lt == 0) CB_TRACE_EVENT(p.trace, 8);
            if (threadIdx.x == 64) CB_TRACE_EVENT(p.trace, 10);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (cs.abort_flag) {
        // A bounded wait gave up somewhere in this CTA. Copies armed before that may still be in flight towards this
        // CTA's shared memory and issued MMAs may still be running on its accumulators: give both a bounded chance to
        // finish before the shared memory and TMEM are released.
        if (warp == 0 && lane == 0) {
            if (!p.pack_in_kernel) mbar_drain(smem_u32(&cs.wbar), 0, p.status);
            for (int st = 0; st < p.stages; ++st)
                if ((armed >> st) & 1u) mbar_drain(smem_u32(&cs.full[st]), (armed_parity >> st) & 1u, p.status);
        }
        if (warp == 1 && lane == 0) {
            tc_commit(smem_u32(&cs.drain));
            mbar_drain(smem_u32(&cs.drain), 0, p.status);
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

// Packs the filter for the kernel above. Row index = ((fh * CG + cg) * FWc + fw) * OCp + o, 32 floats per row; W is the
// caller's OC x IC x FHs x FWs filter, (FHc, FWc) the taps of the convolution the kernel runs.
//   PACK_FWD:      row[c] = W[o][cg*32 + c][fh][fw]
//   PACK_DGRAD:    row[c] = W[cg*32 + c][o][FH-1-fh][FW-1-fw]          (o = input channel of the convolution)
//   PACK_S2_FWD:   the stride-2 3x3 convolution as a 2x2 convolution over the 4 input phases stacked as channels
//                  c' = phase*IC + c: row[c'] = W[o][c][s2_tap(ph, fh)][s2_tap(pw, fw)] (zero where no tap lands)
//   PACK_S2_DGRAD: its adjoint: input channels are the OC planes of dY, output o' = out_first + o indexes (phase, c),
//                  taps flipped: row[oc] = W[oc][c][s2_tap(ph, 1-fh)][s2_tap(pw, 1-fw)]
__global__ void pack_filter_kernel(const float* __restrict__ W, float* __restrict__ Wp, int OC, int IC, int FHs, int FWs,
                                   int FHc, int FWc, int OCp, int CG, int mode, int out_first, int out_count,
                                   long long total) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i & 31);
        long long r = i >> 5;
        const int o = (int)(r % OCp);
        r /= OCp;
        const int fw = (int)(r % FWc);
        r /= FWc;
        const int cg = (int)(r % CG);
        const int fh = (int)(r / CG);
        const int ch = cg * 32 + c;
        float v = 0.f;
        if (mode == PACK_FWD) {
            if (o < OC && ch < IC) v = W[(((long long)o * IC + ch) * FHs + fh) * FWs + fw];
        } else if (mode == PACK_DGRAD) {
            if (o < IC && ch < OC) v = W[(((long long)ch * IC + o) * FHs + (FHs - 1 - fh)) * FWs + (FWs - 1 - fw)];
        } else if (mode == PACK_S2_FWD) {
            if (o < OC && ch < 4 * IC) {
                const int phase = ch / IC, cc = ch - phase * IC;
                const int sh = s2_tap(phase >> 1, fh), sw = s2_tap(phase & 1, fw);
                if (sh >= 0 && sw >= 0) v = W[(((long long)o * IC + cc) * FHs + sh) * FWs + sw];
            }
        } else {
            if (o < out_count && ch < OC) {
                const int og = out_first + o;
                const int phase = og / IC, cc = og - phase * IC;
                const int sh = s2_tap(phase >> 1, 1 - fh), sw = s2_tap(phase & 1, 1 - fw);
                if (sh >= 0 && sw >= 0) v = W[(((long long)ch * IC + cc) * FHs + sh) * FWs + sw];
            }
        }
        Wp[i] = v;
    }
}

// ---- re-layout kernels of the stride-2 path (memory-bound, one element per thread, coalesced on the write side)
// Xs[n][phase*C + c][i][j] = X[n][c][2i + (phase >> 1)][2j + (phase & 1)]
__global__ void space_to_depth2_kernel(const float* __restrict__ X, float* __restrict__ Xs, int C, int H, int W,
                                       long long total) {
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
// dX[n][c][y][x] = dXs[group][n][o][y/2][x/2] with phase*C + c = group*per_group + o
__global__ void depth_to_space2_kernel(const float* __restrict__ dXs, float* __restrict__ dX, int N, int C, int H, int W,
                                       int per_group, long long total) {
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
        dX[i] = dXs[((((long long)g * N + n) * per_group + o) * H2 + (y >> 1)) * W2 + (x >> 1)];
    }
}
// Xsub[nc][i][j] = X[nc][2i][2j]
__global__ void subsample2_kernel(const float* __restrict__ X, float* __restrict__ Xsub, long long NC, int H, int W,
                                  long long total) {
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
// dX[nc][y][x] = (y, x both even) ? dXsub[nc][y/2][x/2] : 0
__global__ void upsample2_zero_kernel(const float* __restrict__ dXsub, float* __restrict__ dX, int H, int W,
                                      long long total) {
    const int H2 = H / 2, W2 = W / 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int x = (int)(i % W);
        const long long r = i / W;
        const int y = (int)(r % H);
        const long long nc = r / H;
        dX[i] = ((x | y) & 1) ? 0.f : dXsub[(nc * H2 + (y >> 1)) * W2 + (x >> 1)];
    }
}

// Where a launch takes its stream, scratch and status word from: a cb_ctx (workspace grown with cudaMalloc) or the
// static arrays of the allocation-free entry point.
struct ConvEnv {
    cudaStream_t stream;
    int sm_count, smem_optin;
    float* pack;   // scratch for the packed filter (>= pack_bytes)
    int* status;
};

// Geometry the tensor-core forward / data-gradient kernel covers; fills the derived sizes.
struct ConvPlan {
    int Cin, Cout, OCp, NQ, CG, L, KS, shared_rows, nblocks, stages;
    int ew;   // epilogue warps of the kernel instantiation: 8 (two CTAs per SM) or 16
    size_t w_bytes;
    uint32_t block_bytes, stage_bytes;
};

static int plan_conv(ConvPlan& q, int smem_optin, const float* X, int Cin, int Cout, int IH, int IW, int FH, int FW,
                     int pH, int pW) {
    // every tap must read within one pixel of the output position: offsets fh - pH and fw - pW in [-1, 1]
    if (FH < 1 || FH > 3 || FW < 1 || FW > 3 || pH < 0 || pH > 1 || pW < 0 || pW > 1) return CB_EUNSUPPORTED;
    if (FH - 1 - pH > 1 || FW - 1 - pW > 1) return CB_EUNSUPPORTED;
    if (IW != 8 && IW != 16 && IW != 32) return CB_EUNSUPPORTED;
    q.L = 32 / IW;
    if (IH % q.L) return CB_EUNSUPPORTED;
    q.Cin = Cin;
    q.Cout = Cout;
    q.OCp = (q.Cout + 15) / 16 * 16;
    q.NQ = FW * q.OCp;
    if (q.NQ > 256 || q.Cin < 1) return CB_EUNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(X) & 15u) != 0) return CB_EUNSUPPORTED;
    q.CG = (q.Cin + 31) / 32;
    q.w_bytes = (size_t)FH * q.CG * q.NQ * kRowBytes;
    q.shared_rows = (q.L == 1 && IH % 4 == 0) ? 1 : 0;
    q.nblocks = q.shared_rows ? FH + 3 : FH * 4;
    // narrow outputs: the 8-epilogue-warp instantiation, sized so that two CTAs fit one SM (shared memory and TMEM halves)
    q.ew = (q.OCp <= 32 && q.w_bytes <= 40 * 1024) ? 8 : 16;
    const long long budget = q.ew == 8 ? (long long)(smem_optin < 113 * 1024 ? smem_optin : 113 * 1024) : (long long)smem_optin;
    const long long cap = budget - 2048 - (long long)q.w_bytes;
    // as many K steps per stage as leaves a pipeline of at least 4 stages (fewer, larger TMA boxes)
    const int cin8 = (q.Cin + 7) / 8;
    q.KS = 0;
    for (int ks = 4; ks >= 1; ks >>= 1) {
        if (ks > cin8 && ks > 1) continue;
        const long long st = cap / ((long long)q.nblocks * ks * kCB * kRowBytes);
        if (st >= 4 || (ks == 1 && st >= 2)) {
            q.KS = ks;
            q.stages = (int)(st > kMaxStages ? kMaxStages : st);
            break;
        }
    }
    if (q.KS == 0) return CB_EUNSUPPORTED;
    q.block_bytes = (uint32_t)q.KS * kCB * kRowBytes;
    q.stage_bytes = (uint32_t)q.nblocks * q.block_bytes;
    return CB_OK;
}

// How the caller's filter becomes the packed filter of the convolution the kernel runs.
struct PackSpec {
    int mode, OC, IC, FHs, FWs, out_first, out_count;
};

// Packs the filter into env.pack and launches the kernel: Y (N x q.Cout x IH x IW) = taps (FH, FW, pH, pW) over
// X (N x q.Cin x IH x IW). `err_ctx` may be null (allocation-free entry point).
static int launch_conv(cb_ctx* err_ctx, const ConvEnv& env, const ConvPlan& q, const PackSpec& ps, const float* W,
                       const float* X, float* Y, const float* bias, int N, int IH, int IW, int FH, int FW, int pH, int pW,
                       int relu) {
    const bool in_kernel = env.pack == nullptr;  // no scratch given: the CTAs pack the filter themselves
    if (!in_kernel) {
        const long long total = (long long)q.w_bytes / 4;
        int grid = (int)((total + 255) / 256);
        if (grid > env.sm_count * 8) grid = env.sm_count * 8;
        pack_filter_kernel<<<grid, 256, 0, env.stream>>>(W, env.pack, ps.OC, ps.IC, ps.FHs, ps.FWs, FH, FW, q.OCp, q.CG,
                                                         ps.mode, ps.out_first, ps.out_count, total);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return check_cuda(err_ctx, e, "pack_filter_kernel launch");
    }
    ConvParams p{};
    p.N = N; p.Cin = q.Cin; p.H = IH; p.W = IW; p.Cout = q.Cout;
    p.FH = FH; p.FW = FW; p.pH = pH; p.pW = pW;
    p.OCp = q.OCp; p.NQ = q.NQ; p.CG = q.CG; p.KS = q.KS;
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
    p.Out = Y; p.bias = bias; p.relu = relu;
    p.status = env.status;
    p.pack_in_kernel = in_kernel ? 1 : 0;
    p.pack_mode = ps.mode; p.OCs = ps.OC; p.ICs = ps.IC; p.FHs = ps.FHs; p.FWs = ps.FWs;
    p.out_first = ps.out_first; p.out_count = ps.out_count;
    p.Wsrc = W;
    p.trace = err_ctx ? err_ctx->trace : nullptr;

    CUtensorMap tmIn, tmW;
    int rc;
    const uint64_t plane = (uint64_t)IH * IW;
    if (q.shared_rows) {
        // 32-wide maps: (w, channel, row, image) so that one box of FH+3 rows lands as [row][channel][128 B]
        uint64_t dims[4] = {32, (uint64_t)q.Cin, (uint64_t)IH, (uint64_t)N};
        uint64_t str[3] = {plane * 4, 128, (uint64_t)q.Cin * plane * 4};
        uint32_t box[4] = {32u, (uint32_t)(q.KS * kCB), (uint32_t)q.nblocks, 1u};
        rc = encode_tmap(err_ctx, &tmIn, X, 4, dims, str, box, nullptr, 129);
    } else {
        // planes flattened to (H*W, C, N): a box is 32 consecutive floats of 8*KS channel planes, starting at pixel
        // (row * W) — a multiple of 4 floats, as TMA requires of the innermost coordinate. Pixels before the plane's
        // first row or after its last one, and channels >= C, are out of bounds and read as zero. (A box whose inner
        // extent is below the 128-byte swizzle span would be padded to 128 bytes per inner row in shared memory, so
        // the (W, H) plane is never used as two tensor-map dimensions when W < 32.)
        uint64_t dims[3] = {plane, (uint64_t)q.Cin, (uint64_t)N};
        uint64_t str[2] = {plane * 4, (uint64_t)q.Cin * plane * 4};
        uint32_t box[3] = {32u, (uint32_t)(q.KS * kCB), 1u};
        rc = encode_tmap(err_ctx, &tmIn, X, 3, dims, str, box, nullptr, 129);
    }
    if (rc != CB_OK) return rc;
    if (in_kernel) {
        tmW = tmIn;  // unused by the kernel in this mode; any valid map will do
    } else {
        const uint64_t rows = (uint64_t)FH * q.CG * q.NQ;
        uint64_t dims[3] = {32, rows, 1};
        uint64_t str[2] = {128, rows * 128};
        uint32_t box[3] = {32, (uint32_t)q.NQ, 1};
        rc = encode_tmap(err_ctx, &tmW, env.pack, 3, dims, str, box, nullptr, 128);
        if (rc != CB_OK) return rc;
    }
    const size_t smem = q.w_bytes + (size_t)p.stages * q.stage_bytes + 1024;
    static bool attr_set[64] = {};  // per device: the opt-in shared-memory size is raised to the maximum once
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(umma_conv_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, env.smem_optin - 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(umma_conv_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, env.smem_optin - 1024);
        if (e != cudaSuccess) return check_cuda(err_ctx, e, "umma_conv_kernel attribute");
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const int slots = env.sm_count * (q.ew == 8 ? 2 : 1);  // resident CTAs
    const int grid = p.tiles < slots ? p.tiles : slots;
    if (q.ew == 8) umma_conv_kernel<8><<<grid, 64 + 32 * 8, smem, env.stream>>>(tmIn, tmW, p);
    else umma_conv_kernel<16><<<grid, 64 + 32 * 16, smem, env.stream>>>(tmIn, tmW, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(err_ctx, e, "umma_conv_kernel launch");
    return CB_OK;
}

}  // namespace

// Small filters are packed by the CTAs themselves (no extra launch, no scratch); large ones (a CTA would spend longer
// packing than computing its first tile) by the pack kernel into the context workspace, fetched by TMA.
static int launch_conv_auto(cb_ctx* ctx, ConvEnv env, const ConvPlan& q, const PackSpec& ps, const float* W, const float* X,
                            float* Y, const float* bias, int N, int IH, int IW, int FH, int FW, int pH, int pW, int relu) {
    const long long src = (long long)ps.OC * ps.IC * ps.FHs * ps.FWs;
    env.pack = nullptr;
    if (src > 12288) {
        int rc = ensure_workspace(ctx, q.w_bytes);
        if (rc != CB_OK) return rc;
        env.pack = static_cast<float*>(ctx->workspace);
        ctx->launches += 1;
    }
    return launch_conv(ctx, env, q, ps, W, X, Y, bias, N, IH, IW, FH, FW, pH, pW, relu);
}

int umma_conv_fwd(cb_ctx* ctx, const float* W, const float* X, float* Y, const float* bias, int N, int IC, int IH,
                  int IW, int OC, int FH, int FW, int sH, int sW, int pH, int pW, int relu, bool dgrad_of) {
    ConvEnv env{ctx->stream, ctx->sm_count, ctx->max_smem_optin, nullptr, ctx->d_status};
    ConvPlan q{};
    int rc;
    if (sH == 1 && sW == 1) {
        // ---- stride 1: 1x1 (pad 0) or 3x3 (pad 1) per axis
        if (!((FH == 1 && pH == 0) || (FH == 3 && pH == 1))) return CB_EUNSUPPORTED;
        if (!((FW == 1 && pW == 0) || (FW == 3 && pW == 1))) return CB_EUNSUPPORTED;
        rc = plan_conv(q, ctx->max_smem_optin, X, dgrad_of ? OC : IC, dgrad_of ? IC : OC, IH, IW, FH, FW, pH, pW);
        if (rc != CB_OK) return rc;
        const PackSpec ps{dgrad_of ? PACK_DGRAD : PACK_FWD, OC, IC, FH, FW, 0, 0};
        rc = launch_conv_auto(ctx, env, q, ps, W, X, Y, bias, N, IH, IW, FH, FW, pH, pW, relu);
        if (rc != CB_OK) return rc;
        ctx->launches += 1;
        ctx->last_kernel = "umma_tf32";
        return CB_OK;
    }
    // ---- stride 2 (square): 3x3 pad 1 through the 4 input phases, 1x1 pad 0 through phase (0,0)
    if (sH != 2 || sW != 2 || FH != FW || pH != pW || (IH & 1) || (IW & 1)) return CB_EUNSUPPORTED;
    if (!((FH == 3 && pH == 1) || (FH == 1 && pH == 0))) return CB_EUNSUPPORTED;
    const int H2 = IH / 2, W2 = IW / 2;
    const long long plane2 = (long long)H2 * W2;
    const int launch_threads = 256;
    auto grid_of = [&](long long n) {
        long long g = (n + launch_threads - 1) / launch_threads;
        const long long cap = (long long)ctx->sm_count * 16;
        return (int)(g > cap ? cap : (g < 1 ? 1 : g));
    };
    if (FH == 1) {
        // Y = W * X[:, :, ::2, ::2]  /  dX[:, :, ::2, ::2] = W^T dY, zero elsewhere
        rc = plan_conv(q, ctx->max_smem_optin, dgrad_of ? X : nullptr /* the sub-sampled copy is aligned */, dgrad_of ? OC : IC,
                       dgrad_of ? IC : OC, H2, W2, 1, 1, 0, 0);
        if (rc != CB_OK) return rc;
        const size_t sub_bytes = (size_t)N * IC * plane2 * sizeof(float);
        rc = ensure_workspace2(ctx, sub_bytes);
        if (rc != CB_OK) return rc;
        float* sub = static_cast<float*>(ctx->workspace2);
        const PackSpec ps{dgrad_of ? PACK_DGRAD : PACK_FWD, OC, IC, 1, 1, 0, 0};
        const long long n_sub = (long long)N * IC * plane2;
        if (!dgrad_of) {
            subsample2_kernel<<<grid_of(n_sub), launch_threads, 0, ctx->stream>>>(X, sub, (long long)N * IC, IH, IW, n_sub);
            rc = launch_conv_auto(ctx, env, q, ps, W, sub, Y, bias, N, H2, W2, 1, 1, 0, 0, relu);
        } else {
            rc = launch_conv_auto(ctx, env, q, ps, W, X /* = dY */, sub, nullptr, N, H2, W2, 1, 1, 0, 0, 0);
            const long long n_full = (long long)N * IC * IH * IW;
            if (rc == CB_OK)
                upsample2_zero_kernel<<<grid_of(n_full), launch_threads, 0, ctx->stream>>>(sub, Y /* = dX */, IH, IW, n_full);
        }
        if (rc != CB_OK) return rc;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return check_cuda(ctx, e, "stride-2 1x1 convolution");
        ctx->launches += 2;
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
        rc = plan_conv(q, ctx->max_smem_optin, Xs, C4, OC, H2, W2, 2, 2, 1, 1);
        if (rc != CB_OK) return rc;
        const long long n_el = (long long)N * C4 * plane2;
        space_to_depth2_kernel<<<grid_of(n_el), launch_threads, 0, ctx->stream>>>(X, Xs, IC, IH, IW, n_el);
        const PackSpec ps{PACK_S2_FWD, OC, IC, 3, 3, 0, 0};
        rc = launch_conv_auto(ctx, env, q, ps, W, Xs, Y, bias, N, H2, W2, 2, 2, 1, 1, relu);
        if (rc != CB_OK) return rc;
        ctx->launches += 2;
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
    rc = plan_conv(q, ctx->max_smem_optin, X /* = dY */, OC, per_group, H2, W2, 2, 2, 0, 0);
    if (rc != CB_OK) return rc;
    for (int g = 0; g < groups; ++g) {
        const PackSpec ps{PACK_S2_DGRAD, OC, IC, 3, 3, g * per_group, per_group};
        rc = launch_conv_auto(ctx, env, q, ps, W, X /* = dY */, dXs + (size_t)g * N * per_group * plane2, nullptr, N, H2, W2, 2, 2,
                         0, 0, 0);
        if (rc != CB_OK) return rc;
    }
    const long long n_full = (long long)N * IC * IH * IW;
    depth_to_space2_kernel<<<grid_of(n_full), launch_threads, 0, ctx->stream>>>(dXs, Y /* = dX */, N, IC, IH, IW, per_group,
                                                                                 n_full);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "depth_to_space2_kernel launch");
    ctx->launches += groups + 1;
    ctx->last_kernel = "umma_tf32";
    return CB_OK;
}

namespace {

// ------------------------------------------------------------------------------------------ weight gradient
// dW[oc][c][fh][fw] = sum over output pixels of dY[oc][pix] * X[c][pix shifted by (fh-pH, fw-pW)]: a contraction
// over pixels, so both operands are K-major (32 pixels of one channel plane = one 128-byte row, standard 128-byte
// swizzle). Per line of 32 output pixels a stage holds
//   A: FH blocks [Cp channel rows][32 px] of X, fetched at the vertically shifted pixel offsets (UMMA M side,
//      rows stacked as (fh, c); 128 rows per M tile), and
//   B: the dY line [OCp rows][32 px] three times, as (fw, oc) rows of the UMMA N side: the centre copy comes from
//      TMA, the copies for fw = 0 / fw = 2 are the same rows rotated by one pixel (zeros entering at the image row
//      edges), written by eight shift warps — shifting dY by -d is the same sum as shifting X by +d.
// Every CTA walks its share of the lines accumulating D[(fh,c)][(fw,oc)] in TMEM (the whole K split across CTAs),
// writes its partial to the workspace, and a second kernel adds the partials in a fixed order (deterministic).
struct WgradParams {
    int N, Cin, H, W, OC;
    int FH, FW, pH, pW;
    int Cp, OCp, NQ, mtiles, rowsA;  // rowsA = FH * Cp valid accumulator rows
    int L, LPI;
    long long total_lines;
    int stages, tmem_cols;
    uint32_t stage_bytes, a_bytes;
    float* partial;                  // [gridDim.x][mtiles * 128][NQ]
    int* status;
};

struct __align__(8) WgradSmem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t xf[kMaxStages];
    uint64_t tfull;
    uint32_t tmem_base;
    int abort_flag;
};

// 16-byte chunk q of the 128-byte row at row_addr under the standard 128-byte swizzle (chunk ^= row index mod 8)
__device__ __forceinline__ uint32_t sw128_chunk(uint32_t row_addr, int q) {
    return row_addr + ((((uint32_t)q) ^ ((row_addr >> 7) & 7u)) << 4);
}

constexpr int kShiftWarps = 8;  // one scheduler cannot hide the shared-memory latencies of a single warp

// One 16-byte chunk (pixels 4q .. 4q+3) of the horizontally shifted copies of a dY row: row_m1 (tap offset -1: pairs
// X[px] with dY[px + 1]) and row_p1 (tap offset +1: pairs X[px] with dY[px - 1]); zeros enter at the edges of the
// W-wide image rows packed in the line; an address of 0 skips that copy.
__device__ __forceinline__ void shift_dy_chunk(uint32_t src_row, uint32_t row_m1, uint32_t row_p1, int q, int W) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(sw128_chunk(src_row, q)));
    float left = 0.f, right = 0.f;
    if (q > 0) asm volatile("ld.shared.f32 %0, [%1];" : "=f"(left) : "r"(sw128_chunk(src_row, q - 1) + 12u));
    if (q < 7) asm volatile("ld.shared.f32 %0, [%1];" : "=f"(right) : "r"(sw128_chunk(src_row, q + 1)));
    const int x0 = 4 * q, wm = W - 1;
    if (row_m1) {
        const float a0 = ((x0 & wm) < wm) ? v.y : 0.f, a1 = (((x0 + 1) & wm) < wm) ? v.z : 0.f;
        const float a2 = (((x0 + 2) & wm) < wm) ? v.w : 0.f, a3 = (((x0 + 3) & wm) < wm) ? right : 0.f;
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(sw128_chunk(row_m1, q)), "f"(a0), "f"(a1), "f"(a2), "f"(a3) : "memory");
    }
    if (row_p1) {
        const float b0 = ((x0 & wm) >= 1) ? left : 0.f, b1 = (((x0 + 1) & wm) >= 1) ? v.x : 0.f;
        const float b2 = (((x0 + 2) & wm) >= 1) ? v.y : 0.f, b3 = (((x0 + 3) & wm) >= 1) ? v.z : 0.f;
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(sw128_chunk(row_p1, q)), "f"(b0), "f"(b1), "f"(b2), "f"(b3) : "memory");
    }
}

__global__ void __launch_bounds__(192 + 32 * kShiftWarps, 1)
    umma_wgrad_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmdY,
                      const WgradParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ WgradSmem ws;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int* abort_flag = &ws.abort_flag;
    const uint32_t st_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t set_bytes = (uint32_t)p.OCp * kRowBytes;
    const int centre = p.pW;  // (fw, oc) rows of the N side: the unshifted copy is the tap with fw - pW == 0

    if (threadIdx.x == 0) {
        ws.abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&ws.full[s]), 1);
            mbar_init(smem_u32(&ws.empty[s]), 1);
            mbar_init(smem_u32(&ws.xf[s]), 32 * kShiftWarps);
        }
        mbar_init(smem_u32(&ws.tfull), 1);
        mbar_fence_init();
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmdY);
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc(smem_u32(&ws.tmem_base), (uint32_t)p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ws.tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (long long g = blockIdx.x; g < p.total_lines && ok; g += gridDim.x) {
            ok = warp_wait(smem_u32(&ws.empty[s]), ph ^ 1u, lane, abort_flag, p.status, CBK_TIMEOUT_EMPTY);
            if (!ok) break;
            if (lane == 0) {
                const uint32_t full = smem_u32(&ws.full[s]);
                const uint32_t stg = st_base + s * p.stage_bytes;
                const int gi = (int)g;  // total_lines < 2^29 (checked on the host)
                const int n = gi / p.LPI;
                const int h0 = (gi - n * p.LPI) * p.L;
                mbar_expect_tx(full, p.a_bytes + set_bytes);
                for (int fh = 0; fh < p.FH; ++fh)
                    tma_load_3d(stg + (uint32_t)fh * p.Cp * kRowBytes, &tmX, full, (h0 + fh - p.pH) * p.W, 0, n);
                tma_load_3d(stg + p.a_bytes + (uint32_t)centre * set_bytes, &tmdY, full, h0 * p.W, 0, n);
            }
            __syncwarp();
            if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ UMMA issuer
        const uint32_t idesc = umma_idesc_tf32(128, (uint32_t)p.NQ, 0u, 0u);
        const uint64_t desc0 = umma_smem_desc(0, 16u, 1024u, UMMA_SW_128B);  // K-major 128-byte rows; address added per stage
        uint32_t s = 0, ph = 0;
        bool ok = true;
        bool first_line = true;
        for (long long g = blockIdx.x; g < p.total_lines && ok; g += gridDim.x) {
            ok = warp_wait(smem_u32(&ws.full[s]), ph, lane, abort_flag, p.status, CBK_TIMEOUT_FULL);
            if (!ok) break;
            if (p.FW > 1) {
                ok = warp_wait(smem_u32(&ws.xf[s]), ph, lane, abort_flag, p.status, CBK_TIMEOUT_XFORM);
                if (!ok) break;
            }
            tc_fence_after();
            if (lane == 0) {
                const uint32_t stg = st_base + s * p.stage_bytes;
                const uint64_t dA0 = desc0 + (uint64_t)((stg >> 4) & 0x3FFFu);
                const uint64_t dB0 = desc0 + (uint64_t)(((stg + p.a_bytes) >> 4) & 0x3FFFu);
                const uint32_t first = first_line ? 0u : 1u;
                for (int m = 0; m < p.mtiles; ++m) {
                    const uint64_t dA = dA0 + (uint64_t)(m * (16384 >> 4));
                    const uint32_t d = tmem_base + (uint32_t)m * p.NQ;
                    umma_tf32(d, dA, dB0, idesc, first);
                    umma_tf32(d, dA + 2, dB0 + 2, idesc, 1u);
                    umma_tf32(d, dA + 4, dB0 + 4, idesc, 1u);
                    umma_tf32(d, dA + 6, dB0 + 6, idesc, 1u);
                }
                tc_commit(smem_u32(&ws.empty[s]));
                if (g + gridDim.x >= p.total_lines) tc_commit(smem_u32(&ws.tfull));
            }
            __syncwarp();
            first_line = false;
            if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue: partial sums to the workspace
        const int quarter = warp & 3;
        bool ok = mbar_wait(smem_u32(&ws.tfull), 0, abort_flag, p.status, CBK_TIMEOUT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
            const int rows_tot = p.mtiles * 128;
            for (int m = 0; m < p.mtiles; ++m) {
                const int r = m * 128 + 32 * quarter + lane;
                float* dst = p.partial + ((long long)blockIdx.x * rows_tot + r) * p.NQ;
                const uint32_t t_row = tmem_base + (uint32_t)m * p.NQ + ((uint32_t)(32 * quarter) << 16);
                for (int c = 0; c < p.NQ; c += 16) {
                    uint32_t v[16];
                    tmem_ld16(t_row + (uint32_t)c, v);
                    tmem_ld_wait();
                    if (r < p.rowsA) {
#pragma unroll
                        for (int e = 0; e < 16; e += 4)
                            *reinterpret_cast<float4*>(dst + c + e) =
                                make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]), __uint_as_float(v[e + 2]),
                                            __uint_as_float(v[e + 3]));
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ shift warps: fw = 0 and fw = 2 copies of dY
        if (p.FW > 1) {
            const int t = threadIdx.x - 192;
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (long long g = blockIdx.x; g < p.total_lines && ok; g += gridDim.x) {
                ok = mbar_wait(smem_u32(&ws.full[s]), ph, abort_flag, p.status, CBK_TIMEOUT_XFORM_FULL);
                if (!ok) break;
                for (int item = t; item < p.OCp * 8; item += 32 * kShiftWarps) {
                    const int row = item >> 3, q = item & 7;
                    const uint32_t b0 = st_base + s * p.stage_bytes + p.a_bytes + (uint32_t)row * kRowBytes;
                    const uint32_t src = b0 + (uint32_t)centre * set_bytes;
                    const uint32_t m1 = centre >= 1 ? src - set_bytes : 0u;             // tap fw = pW - 1
                    const uint32_t p1 = centre + 1 < p.FW ? src + set_bytes : 0u;       // tap fw = pW + 1
                    shift_dy_chunk(src, m1, p1, q, p.W);
                }
                fence_proxy_async_smem();
                mbar_arrive(smem_u32(&ws.xf[s]));
                if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
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

// dW[oc][c][fh][fw] (+)= sum over CTAs of partial[cta][fh*Cp + c][fw*OCp + oc], summed in CTA order.
// s2 != 0: the rows are (tap of the 2x2 phase convolution, phase*IC + c) and map back to the 3x3 stride-2 filter.
__global__ void __launch_bounds__(256) wgrad_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dW,
                                                           int nparts, int rows_tot, int rowsA, int NQ, int Cp, int Cin,
                                                           int OC, int OCp, int FH, int FW, int accumulate, int s2,
                                                           int IC_src) {
    // block = 32 consecutive accumulator elements x 8 groups of partials; each thread sums its group's partials in
    // order, the 8 group sums are added in order in shared memory: a fixed summation order (deterministic)
    __shared__ float red[8][33];
    const long long total = (long long)rowsA * NQ;
    const long long i = (long long)blockIdx.x * 32 + threadIdx.x;
    const int grp = threadIdx.y;
    float s = 0.f;
    if (i < total) {
        const long long pstride = (long long)rows_tot * NQ;
        const float* src = partial + i;  // (r, col) of the partial layout is exactly element i
#pragma unroll 4
        for (int q = grp; q < nparts; q += 8) s += __ldg(src + q * pstride);
    }
    red[grp][threadIdx.x] = s;
    __syncthreads();
    if (grp != 0 || i >= total) return;
    float sum = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) sum += red[g][threadIdx.x];
    const int col = (int)(i % NQ);
    const int r = (int)(i / NQ);
    const int fh = r / Cp, c = r - fh * Cp;
    const int fw = col / OCp, oc = col - fw * OCp;
    if (c >= Cin || oc >= OC) return;
    float* dst;
    if (!s2) {
        dst = dW + (((long long)oc * Cin + c) * FH + fh) * FW + fw;
    } else {
        const int phase = c / IC_src, cc = c - phase * IC_src;
        const int sh = s2_tap(phase >> 1, fh), sw = s2_tap(phase & 1, fw);
        if (sh < 0 || sw < 0) return;
        dst = dW + (((long long)oc * IC_src + cc) * 3 + sh) * 3 + sw;
    }
    *dst = accumulate ? *dst + sum : sum;
}

}  // namespace

// dW (+)= contraction over the pixels of N x Cin x IH x IW planes `X` and N x OC x IH x IW planes `dY` with taps
// (FH, FW, pH, pW) in the same-size convention of the forward kernel. s2 / IC_src: see wgrad_reduce_kernel.
static int wgrad_core(cb_ctx* ctx, const float* dY, const float* X, float* dW, int N, int Cin, int IH, int IW, int OC, int FH,
                      int FW, int pH, int pW, int accumulate, int s2, int IC_src) {
    if (FH < 1 || FH > 3 || FW < 1 || FW > 3 || pH < 0 || pH > 1 || pW < 0 || pW > 1) return CB_EUNSUPPORTED;
    if (FH - 1 - pH > 1 || FW - 1 - pW > 1) return CB_EUNSUPPORTED;
    if (IW != 8 && IW != 16 && IW != 32) return CB_EUNSUPPORTED;
    const int L = 32 / IW;
    if (IH % L) return CB_EUNSUPPORTED;
    const int Cp = (Cin + 7) / 8 * 8;
    const int OCp = (OC + 15) / 16 * 16;
    const int NQ = FW * OCp;
    const int rowsA = FH * Cp;
    const int mtiles = (rowsA + 127) / 128;
    if (NQ > 256 || Cp > 256 || OCp > 128 || mtiles * NQ > 512) return CB_EUNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(X) & 15u) || (reinterpret_cast<uintptr_t>(dY) & 15u)) return CB_EUNSUPPORTED;
    int rows_stage = rowsA + NQ;
    if (rows_stage < mtiles * 128) rows_stage = mtiles * 128;
    const uint32_t stage_bytes = ((uint32_t)rows_stage * kRowBytes + 1023u) & ~1023u;
    long long stages = ((long long)ctx->max_smem_optin - 2048) / stage_bytes;
    if (stages < 2) return CB_EUNSUPPORTED;
    if (stages > kMaxStages) stages = kMaxStages;

    WgradParams p{};
    p.N = N; p.Cin = Cin; p.H = IH; p.W = IW; p.OC = OC;
    p.FH = FH; p.FW = FW; p.pH = pH; p.pW = pW;
    p.Cp = Cp; p.OCp = OCp; p.NQ = NQ; p.mtiles = mtiles; p.rowsA = rowsA;
    p.L = L; p.LPI = IH / L;
    p.total_lines = (long long)N * p.LPI;
    if (p.total_lines > (1LL << 29)) return CB_EUNSUPPORTED;
    p.stages = (int)stages;
    int cols = 32;
    while (cols < mtiles * NQ) cols <<= 1;
    p.tmem_cols = cols;
    p.stage_bytes = stage_bytes;
    p.a_bytes = (uint32_t)rowsA * kRowBytes;
    p.status = ctx->d_status;
    const int grid = (int)(p.total_lines < ctx->sm_count ? p.total_lines : ctx->sm_count);
    const size_t part_bytes = (size_t)grid * mtiles * 128 * NQ * sizeof(float);
    int rc = ensure_workspace(ctx, part_bytes);
    if (rc != CB_OK) return rc;
    p.partial = static_cast<float*>(ctx->workspace);

    CUtensorMap tmX, tmdY;
    {
        uint64_t dims[3] = {(uint64_t)IH * IW, (uint64_t)Cin, (uint64_t)N};
        uint64_t str[2] = {(uint64_t)IH * IW * 4, (uint64_t)Cin * IH * IW * 4};
        uint32_t box[3] = {32u, (uint32_t)Cp, 1u};
        rc = encode_tmap(ctx, &tmX, X, 3, dims, str, box, nullptr, 128);
        if (rc != CB_OK) return rc;
    }
    {
        uint64_t dims[3] = {(uint64_t)IH * IW, (uint64_t)OC, (uint64_t)N};
        uint64_t str[2] = {(uint64_t)IH * IW * 4, (uint64_t)OC * IH * IW * 4};
        uint32_t box[3] = {32u, (uint32_t)OCp, 1u};
        rc = encode_tmap(ctx, &tmdY, dY, 3, dims, str, box, nullptr, 128);
        if (rc != CB_OK) return rc;
    }
    const size_t smem = (size_t)p.stages * stage_bytes + 1024;
    cudaError_t e = cudaFuncSetAttribute(umma_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return check_cuda(ctx, e, "umma_wgrad_kernel attribute");
    umma_wgrad_kernel<<<grid, 192 + 32 * kShiftWarps, smem, ctx->stream>>>(tmX, tmdY, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "umma_wgrad_kernel launch");
    const long long total = (long long)rowsA * NQ;
    int rgrid = (int)((total + 31) / 32);
    wgrad_reduce_kernel<<<rgrid, dim3(32, 8), 0, ctx->stream>>>(p.partial, dW, grid, mtiles * 128, rowsA, NQ, Cp, Cin, OC, OCp, FH, FW,
                                                         accumulate ? 1 : 0, s2, IC_src);
    e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "wgrad_reduce_kernel launch");
    ctx->launches += 2;
    ctx->last_kernel = "umma_tf32";
    return CB_OK;
}

int umma_conv_wgrad(cb_ctx* ctx, const float* dY, const float* X, float* dW, int N, int IC, int IH, int IW, int OC,
                    int FH, int FW, int sH, int sW, int pH, int pW, int accumulate) {
    if (sH == 1 && sW == 1) {
        if (!((FH == 1 && pH == 0) || (FH == 3 && pH == 1))) return CB_EUNSUPPORTED;
        if (!((FW == 1 && pW == 0) || (FW == 3 && pW == 1))) return CB_EUNSUPPORTED;
        return wgrad_core(ctx, dY, X, dW, N, IC, IH, IW, OC, FH, FW, pH, pW, accumulate, 0, IC);
    }
    if (sH != 2 || sW != 2 || FH != FW || pH != pW || (IH & 1) || (IW & 1)) return CB_EUNSUPPORTED;
    if (!((FH == 3 && pH == 1) || (FH == 1 && pH == 0))) return CB_EUNSUPPORTED;
    const int H2 = IH / 2, W2 = IW / 2;
    if (W2 != 8 && W2 != 16 && W2 != 32) return CB_EUNSUPPORTED;
    const long long plane2 = (long long)H2 * W2;
    auto grid_of = [&](long long n) {
        long long g = (n + 255) / 256;
        const long long cap = (long long)ctx->sm_count * 16;
        return (int)(g > cap ? cap : (g < 1 ? 1 : g));
    };
    if (FH == 1) {
        const long long n_sub = (long long)N * IC * plane2;
        int rc = ensure_workspace2(ctx, (size_t)n_sub * sizeof(float));
        if (rc != CB_OK) return rc;
        float* sub = static_cast<float*>(ctx->workspace2);
        subsample2_kernel<<<grid_of(n_sub), 256, 0, ctx->stream>>>(X, sub, (long long)N * IC, IH, IW, n_sub);
        ctx->launches += 1;
        return wgrad_core(ctx, dY, sub, dW, N, IC, H2, W2, OC, 1, 1, 0, 0, accumulate, 0, IC);
    }
    if (4 * IC > 256) return CB_EUNSUPPORTED;
    const long long n_el = (long long)N * 4 * IC * plane2;
    int rc = ensure_workspace2(ctx, (size_t)n_el * sizeof(float));
    if (rc != CB_OK) return rc;
    float* Xs = static_cast<float*>(ctx->workspace2);
    space_to_depth2_kernel<<<grid_of(n_el), 256, 0, ctx->stream>>>(X, Xs, IC, IH, IW, n_el);
    ctx->launches += 1;
    return wgrad_core(ctx, dY, Xs, dW, N, 4 * IC, H2, W2, OC, 2, 2, 1, 1, accumulate, 1, IC);
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
    bool ready = false;
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

    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return noalloc_fail(err, err_len, CB_ECUDA, cudaGetErrorString(e));
    NoAllocDevice& d = g_noalloc_dev[device];
    if (!d.ready) {
        // once per device, with that device current: resolve the device addresses of the static arrays
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.pack), g_noalloc_pack);
        if (e != cudaSuccess) return noalloc_fail(err, err_len, CB_ECUDA, cudaGetErrorString(e));
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status), g_noalloc_status);
        if (e != cudaSuccess) return noalloc_fail(err, err_len, CB_ECUDA, cudaGetErrorString(e));
        int major = 0;
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (major != 10) return noalloc_fail(err, err_len, CB_EUNSUPPORTED, "this library only carries sm_100a code");
        cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device);
        cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
        d.ready = true;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    ConvPlan q{};
    if (plan_conv(q, d.smem_optin, X, IC, OC, IH, IW, FH, FW, pH, pW) != CB_OK)
        return noalloc_fail(err, err_len, CB_EUNSUPPORTED, "geometry outside the tensor-core convolution kernel");
    // the scratch keeps the previous call's contents: the pack kernel rewrites all w_bytes (padding included) and
    // the status word is cleared, both in stream order
    e = cudaMemsetAsync(d.status, 0, sizeof(int), stream);
    if (e != cudaSuccess) return noalloc_fail(err, err_len, CB_ECUDA, cudaGetErrorString(e));
    ConvEnv env{stream, d.sm_count, d.smem_optin, d.pack, d.status};
    const PackSpec ps{PACK_FWD, OC, IC, FH, FW, 0, 0};
    if (launch_conv(nullptr, env, q, ps, W, X, Y, bias, N, IH, IW, FH, FW, pH, pW, relu) != CB_OK)
        return noalloc_fail(err, err_len, CB_ECUDA, "kernel launch or tensor map encoding failed");
    return CB_OK;
}
