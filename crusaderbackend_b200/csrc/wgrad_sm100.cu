// Tensor-core weight gradient of the convolution for sm_100a (TF32 mode), NCHW fp32.
#include <cstdlib>

#include "conv_common.cuh"

namespace cb {
namespace {

// ------------------------------------------------------------------------------------------ weight gradient
// dW[oc][c][fh][fw] = sum over output pixels of dY[oc][pix] * X[c][pix shifted by (fh-pH, fw-pW)]: a contraction
// over pixels, so both operands are K-major (32 pixels of one channel plane = one 128-byte row, standard 128-byte
// swizzle). Per line of 32 output pixels a stage holds
//   A: FH blocks [Cp channel rows][32 px] of X, fetched at the vertically shifted pixel offsets (UMMA M side,
//      rows stacked as (fh, c); 128 rows per M tile) — on 32-pixel-wide maps as one box [Cp][FH image rows][32 px],
//      rows stacked as (c, fh) — and
//   B: the dY line [OCp rows][32 px] three times, as (fw, oc) rows of the UMMA N side: the centre copy comes from
//      TMA, the copies for fw = 0 / fw = 2 are the same rows rotated by one pixel (zeros entering at the image row
//      edges), written by eight shift warps — shifting dY by -d is the same sum as shifting X by +d.
// A pipeline stage carries `lps` such lines (1, 2 or 4: as many as leave at least three stages), so that the per-stage
// hand-offs between the producer, the shift warps and the MMA issuer are paid once per 32*lps pixels. Every CTA walks
// its share of the line groups accumulating D[(fh,c)][(fw,oc)] in TMEM (the whole K split across CTAs). Its tile then
// leaves in one of two ways: laid out in filter order in the (by then idle) pipeline stages and added into dW with
// vector atomics by the whole CTA (`direct`, the default: one launch), or written to the workspace as a partial, column
// by column (the 32 lanes of a warp hold 32 consecutive rows: full 128-byte lines), for a second kernel that adds the
// partials in a fixed order (deterministic contexts).
struct WgradParams {
    int N, Cin, H, W, OC;
    int FH, FW, pH, pW;
    int Cp, OCp, NQ, mtiles, rowsA;  // rowsA = FH * Cp valid accumulator rows
    int L, LPI;
    long long total_lines;
    int lps;                         // lines per pipeline stage
    int groups;                      // ceil(total_lines / lps)
    // 3xTF32 in one launch: the line groups are walked three times, as (lo part of X, dY), (X, lo part of dY) and
    // (X, dY) — the tensor core reads the hi part of whatever it is given — and all of it lands in one accumulator
    int vgroups;                     // groups, or 3 * groups
    int stages, tmem_cols;
    uint32_t line_bytes, stage_bytes, a_bytes;  // one line slot of a stage / lps of them / the A part of a line slot
    float* partial;                  // [gridDim.x][NQ][mtiles * 128]; with `atomic`: ONE such tile that every CTA adds into
    int atomic;
    // direct != 0: no second kernel. The CTA lays its tile out in the idle pipeline stages in the order of the filter
    // block it belongs to (`OC` runs of `run` floats) and adds the runs into dW with coalesced atomics:
    // dW[base_off + oc * oc_stride + j] += tile[oc * run + j]. dW must already hold what the sums are added to.
    int direct, vec4, run, s2, IC_src;
    // rows_cf != 0 (32-pixel-wide maps): a line is one image row, so the FH vertically shifted X blocks of a line are
    // FH consecutive image rows and arrive as ONE 4-D box [channel][fh][32 px]: the accumulator rows are then ordered
    // (c, fh) instead of (fh, c), and a line costs two TMA boxes instead of FH + 1.
    int rows_cf;
    long long oc_stride, base_off;
    float* dW;
    int issue_uniform;               // the MMA warp issues as a whole with an elected lane instead of from lane 0
    int* status;
    long long* trace;
};

struct __align__(8) WgradSmem {
    uint64_t full[kConvMaxStages];
    uint64_t empty[kConvMaxStages];
    uint64_t xf[kConvMaxStages];
    uint64_t tfull;
    uint64_t drain;
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
                      const __grid_constant__ CUtensorMap tmXlo, const __grid_constant__ CUtensorMap tmdYlo,
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
        CB_TRACE_WALL(p.trace, 0);
        CB_TRACE_EVENT(p.trace, 1);
        ws.abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&ws.full[s]), 1);
            mbar_init(smem_u32(&ws.empty[s]), 1);
            mbar_init(smem_u32(&ws.xf[s]), 32 * kShiftWarps);
        }
        mbar_init(smem_u32(&ws.tfull), 1);
        mbar_init(smem_u32(&ws.drain), 1);
        mbar_fence_init();
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmdY);
        if (p.vgroups > p.groups) {
            tma_prefetch_desc(&tmXlo);
            tma_prefetch_desc(&tmdYlo);
        }
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc(smem_u32(&ws.tmem_base), (uint32_t)p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // nothing above touches global memory: the kernel before this one may still be running until here
    griddep_wait();
    griddep_launch();
    const uint32_t tmem_base = ws.tmem_base;
    if (threadIdx.x == 0) CB_TRACE_EVENT(p.trace, 2);

    uint32_t armed = 0, armed_parity = 0;  // producer lane: stages armed at least once / parity of their last arming
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (int g = blockIdx.x; g < p.vgroups && ok; g += gridDim.x) {
            ok = conv_warp_wait(smem_u32(&ws.empty[s]), ph ^ 1u, lane, abort_flag, p.status, CBK_TIMEOUT_EMPTY);
            if (!ok) break;
            if (lane == 0) {
                const uint32_t full = smem_u32(&ws.full[s]);
                mbar_expect_tx(full, (uint32_t)p.lps * (p.a_bytes + set_bytes));
                armed |= 1u << s;
                armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
                // 3xTF32 form: the two small cross terms first, while the accumulator is small (the tensor core's
                // fp32 accumulation error is relative to what the accumulator holds), the hi x hi products last
                const int pass = g / p.groups, gg = g - pass * p.groups;
                const bool x3 = p.vgroups > p.groups;
                const CUtensorMap* mx = (x3 && pass == 0) ? &tmXlo : &tmX;
                const CUtensorMap* my = (x3 && pass == 1) ? &tmdYlo : &tmdY;
                for (int l = 0; l < p.lps; ++l) {
                    const uint32_t stg = st_base + s * p.stage_bytes + (uint32_t)l * p.line_bytes;
                    // lines past the end use an image index >= N: their boxes are zero-filled and add nothing
                    const int gi = gg * p.lps + l;  // total_lines < 2^29 (checked on the host)
                    const int n = gi / p.LPI;
                    const int h0 = (gi - n * p.LPI) * p.L;
                    if (p.rows_cf) {
                        tma_load_4d(stg, mx, full, 0, h0 - p.pH, 0, n);
                    } else {
                        for (int fh = 0; fh < p.FH; ++fh)
                            tma_load_3d(stg + (uint32_t)fh * p.Cp * kRowBytes, mx, full, (h0 + fh - p.pH) * p.W, 0, n);
                    }
                    tma_load_3d(stg + p.a_bytes + (uint32_t)centre * set_bytes, my, full, h0 * p.W, 0, n);
                }
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
#ifdef CB_TRACE
        long long t_full = 0, t_xf = 0, t_issue = 0;
#endif
        for (int g = blockIdx.x; g < p.vgroups && ok; g += gridDim.x) {
#ifdef CB_TRACE
            const long long c0 = clock64();
#endif
            ok = conv_warp_wait(smem_u32(&ws.full[s]), ph, lane, abort_flag, p.status, CBK_TIMEOUT_FULL);
            if (!ok) break;
#ifdef CB_TRACE
            const long long c1 = clock64();
#endif
            if (p.FW > 1) {
                ok = conv_warp_wait(smem_u32(&ws.xf[s]), ph, lane, abort_flag, p.status, CBK_TIMEOUT_XFORM);
                if (!ok) break;
            }
            tc_fence_after();
#ifdef CB_TRACE
            const long long c2 = clock64();
            t_full += c1 - c0;
            t_xf += c2 - c1;
#endif
            if (lane == 0 && first_line) CB_TRACE_EVENT(p.trace, 5);
            if (p.issue_uniform) {
                // the whole warp runs the loop with the same values, one elected lane issues: descriptors that change
                // from UMMA to UMMA cost ~110 cycles of issue each from a one-lane branch (see umma_tf32_elect)
                for (int l = 0; l < p.lps; ++l) {
                    const uint32_t stg = st_base + s * p.stage_bytes + (uint32_t)l * p.line_bytes;
                    const uint64_t dA0 = desc0 + (uint64_t)((stg >> 4) & 0x3FFFu);
                    const uint64_t dB0 = desc0 + (uint64_t)(((stg + p.a_bytes) >> 4) & 0x3FFFu);
                    const uint32_t first = (first_line && l == 0) ? 0u : 1u;
                    for (int m = 0; m < p.mtiles; ++m) {
                        const uint64_t dA = dA0 + (uint64_t)(m * (16384 >> 4));
                        const uint32_t d = tmem_base + (uint32_t)m * p.NQ;
                        umma_tf32_elect(d, dA, dB0, idesc, first);
                        umma_tf32_elect(d, dA + 2, dB0 + 2, idesc, 1u);
                        umma_tf32_elect(d, dA + 4, dB0 + 4, idesc, 1u);
                        umma_tf32_elect(d, dA + 6, dB0 + 6, idesc, 1u);
                    }
                }
                tc_commit_elect(smem_u32(&ws.empty[s]));
                if (g + (int)gridDim.x >= p.vgroups) tc_commit_elect(smem_u32(&ws.tfull));
                if (lane == 0 && first_line) CB_TRACE_EVENT(p.trace, 6);
                if (lane == 0 && g + (int)gridDim.x >= p.vgroups) CB_TRACE_EVENT(p.trace, 7);
            } else if (lane == 0) {
                for (int l = 0; l < p.lps; ++l) {
                    const uint32_t stg = st_base + s * p.stage_bytes + (uint32_t)l * p.line_bytes;
                    const uint64_t dA0 = desc0 + (uint64_t)((stg >> 4) & 0x3FFFu);
                    const uint64_t dB0 = desc0 + (uint64_t)(((stg + p.a_bytes) >> 4) & 0x3FFFu);
                    const uint32_t first = (first_line && l == 0) ? 0u : 1u;
                    for (int m = 0; m < p.mtiles; ++m) {
                        const uint64_t dA = dA0 + (uint64_t)(m * (16384 >> 4));
                        const uint32_t d = tmem_base + (uint32_t)m * p.NQ;
                        umma_tf32(d, dA, dB0, idesc, first);
                        umma_tf32(d, dA + 2, dB0 + 2, idesc, 1u);
                        umma_tf32(d, dA + 4, dB0 + 4, idesc, 1u);
                        umma_tf32(d, dA + 6, dB0 + 6, idesc, 1u);
                    }
                }
                tc_commit(smem_u32(&ws.empty[s]));
                if (first_line) CB_TRACE_EVENT(p.trace, 6);
                if (g + (int)gridDim.x >= p.vgroups) {
                    tc_commit(smem_u32(&ws.tfull));
                    CB_TRACE_EVENT(p.trace, 7);
                }
            }
            __syncwarp();
#ifdef CB_TRACE
            t_issue += clock64() - c2;
#endif
            first_line = false;
            if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
        }
#ifdef CB_TRACE
        if (lane == 0 && p.trace) {
            p.trace[(long long)blockIdx.x * 16 + 13] = t_full;
            p.trace[(long long)blockIdx.x * 16 + 14] = t_xf;
            p.trace[(long long)blockIdx.x * 16 + 15] = t_issue;
        }
#endif
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue: partial sums to the workspace
        const int quarter = warp & 3;
        bool ok = mbar_wait(smem_u32(&ws.tfull), 0, abort_flag, p.status, CBK_TIMEOUT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (threadIdx.x == 64) CB_TRACE_EVENT(p.trace, 8);
        if (ok) {
            tc_fence_after();
            const int rows_tot = p.mtiles * 128;
            for (int m = 0; m < p.mtiles && p.direct; ++m) {
                const int r = m * 128 + 32 * quarter + lane;
                if (m * 128 + 32 * quarter >= p.rowsA) continue;  // warp-uniform: no valid row in this quarter
                // Every UMMA of this CTA has completed (tfull), so nothing reads or writes the pipeline stages any more:
                // they take the tile in filter order. Consecutive lanes are consecutive channels, FH*FW words apart
                // (9 for a 3x3 filter): odd strides spread over the banks.
                const int fh = p.rows_cf ? r % p.FH : r / p.Cp;
                const int c = p.rows_cf ? r / p.FH : r - fh * p.Cp;
                bool row_ok = r < p.rowsA && c < p.Cin;
                int roff, pw = 0;
                if (!p.s2) {
                    roff = (c * p.FH + fh) * p.FW;
                } else {
                    const int phase = c / p.IC_src, cc = c - phase * p.IC_src;
                    const int sh = s2_tap(phase >> 1, fh);
                    row_ok = row_ok && sh >= 0;
                    roff = (cc * 3 + sh) * 3;
                    pw = phase & 1;
                }
                const uint32_t t_row = tmem_base + (uint32_t)m * p.NQ + ((uint32_t)(32 * quarter) << 16);
                for (int c0 = 0; c0 < p.NQ; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(t_row + (uint32_t)c0, v);
                    tmem_ld_wait();
                    const int fw = c0 / p.OCp, oc0 = c0 - fw * p.OCp;  // OCp is a multiple of 16: one fw per chunk
                    const int sw = p.s2 ? s2_tap(pw, fw) : fw;
                    if (row_ok && sw >= 0) {
                        const uint32_t dst = st_base + 4u * (uint32_t)(oc0 * p.run + roff + sw);
#pragma unroll
                        for (int e = 0; e < 16; ++e)
                            if (oc0 + e < p.OC)
                                asm volatile("st.shared.f32 [%0], %1;" ::"r"(dst + 4u * (uint32_t)(e * p.run)), "f"(__uint_as_float(v[e])) : "memory");
                    }
                    __syncwarp();  // the next tcgen05.ld is warp-wide
                }
            }
            for (int m = 0; m < p.mtiles && !p.direct; ++m) {
                const int r = m * 128 + 32 * quarter + lane;
                if (m * 128 + 32 * quarter >= p.rowsA) continue;  // warp-uniform: no valid row in this quarter
                // partial[cta][col][row]: for one column the warp's 32 rows are 128 contiguous bytes
                float* dst = p.partial + (p.atomic ? 0LL : (long long)blockIdx.x * p.NQ * rows_tot) + r;
                const uint32_t t_row = tmem_base + (uint32_t)m * p.NQ + ((uint32_t)(32 * quarter) << 16);
                for (int c = 0; c < p.NQ; c += 16) {
                    uint32_t v[16];
                    tmem_ld16(t_row + (uint32_t)c, v);
                    tmem_ld_wait();
                    if (r < p.rowsA) {
                        if (p.atomic) {
#pragma unroll
                            for (int e = 0; e < 16; ++e) atomicAdd(dst + (long long)(c + e) * rows_tot, __uint_as_float(v[e]));
                        } else {
#pragma unroll
                            for (int e = 0; e < 16; ++e) dst[(long long)(c + e) * rows_tot] = __uint_as_float(v[e]);
                        }
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
            const int per_line = p.OCp * 8;
            for (int g = blockIdx.x; g < p.vgroups && ok; g += gridDim.x) {
                ok = mbar_wait(smem_u32(&ws.full[s]), ph, abort_flag, p.status, CBK_TIMEOUT_XFORM_FULL);
                if (!ok) break;
                for (int item = t; item < p.lps * per_line; item += 32 * kShiftWarps) {
                    const int l = item / per_line, rem = item - l * per_line;
                    const int row = rem >> 3, q = rem & 7;
                    const uint32_t b0 = st_base + s * p.stage_bytes + (uint32_t)l * p.line_bytes + p.a_bytes + (uint32_t)row * kRowBytes;
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

    if (threadIdx.x == 64) CB_TRACE_EVENT(p.trace, 10);
    tc_fence_before();
    __syncthreads();
    if (ws.abort_flag) {
        // A bounded wait gave up somewhere in this CTA: copies armed before that may still be in flight towards its
        // shared memory and issued MMAs may still run on its accumulator; both get a bounded chance to finish before
        // the shared memory and TMEM are released.
        if (warp == 0 && lane == 0) {
            for (int st = 0; st < p.stages; ++st)
                if ((armed >> st) & 1u) mbar_drain(smem_u32(&ws.full[st]), (armed_parity >> st) & 1u, p.status);
        }
        if (warp == 1) {  // the commit comes from the lane that issued the MMAs
            if (p.issue_uniform) tc_commit_elect(smem_u32(&ws.drain));
            else if (lane == 0) tc_commit(smem_u32(&ws.drain));
            if (lane == 0) mbar_drain(smem_u32(&ws.drain), 0, p.status);
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
    if (p.direct && !ws.abort_flag) {
        // the whole CTA adds the staged tile into dW: consecutive threads, consecutive addresses within a run
        const int total = p.OC * p.run;
        float* out = p.dW + p.base_off;
        if (p.vec4) {  // runs start on 16-byte boundaries and are whole float4s: one vector add per four weights
            for (int i = 4 * (int)threadIdx.x; i < total; i += 4 * (int)blockDim.x) {
                const int oc = i / p.run, j = i - oc * p.run;
                float4 v;
                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(st_base + 4u * (uint32_t)i));
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + (long long)oc * p.oc_stride + j), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
            }
        } else {
            for (int i = threadIdx.x; i < total; i += blockDim.x) {
                const int oc = i / p.run, j = i - oc * p.run;
                float v;
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(st_base + 4u * (uint32_t)i));
                atomicAdd(out + (long long)oc * p.oc_stride + j, v);
            }
        }
    }
    if (threadIdx.x == 0) {
        CB_TRACE_EVENT(p.trace, 11);
        CB_TRACE_WALL(p.trace, 12);
    }
}

// dW[oc][c][fh][fw] (+)= sum over CTAs of partial[cta][fw*OCp + oc][fh*Cp + c], summed in CTA order.
// s2 != 0: the rows are (tap of the 2x2 phase convolution, phase*IC + c) and map back to the 3x3 stride-2 filter.
template <int kReduceGroups>
__global__ void __launch_bounds__(32 * kReduceGroups) wgrad_reduce_kernel(float* __restrict__ partial, float* __restrict__ dW,
                                                           int nparts, int rows_tot, int rowsA, int NQ, int Cp, int Cin,
                                                           int OC, int OCp, int FH, int FW, int accumulate, int s2,
                                                           int IC_src, int clear, int IC_total, int c_off, int oc_off,
                                                           int rows_cf) {
    // Per-CTA partials (clear == 0): block = 32 consecutive valid accumulator rows of one column x kReduceGroups groups
    // of partials; each thread sums its group's partials in order, the group sums are added in order in shared memory:
    // a fixed summation order (deterministic). One shared accumulator tile (clear != 0): every thread row of the block
    // takes its own 32 rows, reads the sum and leaves zero behind for the next call.
    __shared__ float red[kReduceGroups][33];
    griddep_wait();
    griddep_launch();
    const long long total = (long long)rows_tot * NQ;
    const int row_blocks = (rowsA + 31) / 32;
    const int grp = threadIdx.y;
    const int unit = clear ? (int)blockIdx.x * kReduceGroups + grp : (int)blockIdx.x;
    const int col = unit / row_blocks;
    const int r = (unit - col * row_blocks) * 32 + (int)threadIdx.x;
    const bool live = col < NQ && r < rowsA;
    float sum = 0.f;
    if (clear) {
        if (!live) return;
        float* src = partial + (long long)col * rows_tot + r;  // element of the [col][row] tile layout
        sum = *src;
        *src = 0.f;
    } else {
        float s = 0.f;
        if (live) {
            const float* src = partial + (long long)col * rows_tot + r;
#pragma unroll 4
            for (int q = grp; q < nparts; q += kReduceGroups) s += __ldg(src + q * total);
        }
        red[grp][threadIdx.x] = s;
        __syncthreads();
        if (grp != 0 || !live) return;
#pragma unroll
        for (int g = 0; g < kReduceGroups; ++g) sum += red[g][threadIdx.x];
    }
    const int fh = rows_cf ? r % FH : r / Cp;  // accumulator rows are (c, fh) or (fh, c): see WgradParams::rows_cf
    const int c = rows_cf ? r / FH : r - fh * Cp;
    const int fw = col / OCp, oc = col - fw * OCp;
    if (c >= Cin || oc >= OC) return;
    float* dst;
    if (!s2) {
        // this launch may cover a block (oc_off.., c_off..) of a wider filter with IC_total input channels
        dst = dW + (((long long)(oc_off + oc) * IC_total + c_off + c) * FH + fh) * FW + fw;
    } else {
        const int phase = c / IC_src, cc = c - phase * IC_src;
        const int sh = s2_tap(phase >> 1, fh), sw = s2_tap(phase & 1, fw);
        if (sh < 0 || sw < 0) return;
        dst = dW + (((long long)oc * IC_src + cc) * 3 + sh) * 3 + sw;
    }
    *dst = accumulate ? *dst + sum : sum;
}

// lo[n][i] = rna_tf32(x - hi(x)) of x[n * x_batch + i], hi = the 19 bits the tensor core reads; four elements per
// thread, lo dense with `per4` float4 per image.
__global__ void tf32_lo4_kernel(const float* __restrict__ x, float* __restrict__ lo, long long per4, long long x_batch,
                                long long items) {
    griddep_wait();
    griddep_launch();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < items; i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / per4, r = i - n * per4;
        const float4 v = *reinterpret_cast<const float4*>(x + n * x_batch + 4 * r);
        const float in[4] = {v.x, v.y, v.z, v.w};
        float out[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float hi = __uint_as_float(__float_as_uint(in[e]) & 0xFFFFE000u);
            uint32_t q;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(q) : "f"(in[e] - hi));
            out[e] = __uint_as_float(q);
        }
        reinterpret_cast<float4*>(lo)[i] = make_float4(out[0], out[1], out[2], out[3]);
    }
}

int launch_lo(cb_ctx* ctx, const float* x, float* lo, long long images, long long per, long long x_batch) {
    const long long items = images * (per / 4);
    long long g = (items + 255) / 256;
    const long long cap = (long long)ctx->sm_count * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    cudaError_t e = launch_dep(ctx, tf32_lo4_kernel, dim3((unsigned)g), dim3(256), 0, x, lo, per / 4, x_batch ? x_batch : per, items);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "tf32_lo4_kernel launch");
    ctx->launches += 1;
    return CB_OK;
}

// lo parts of X and dY for the one-launch 3xTF32 form (dense scratch; batch strides 0 = dense)
struct LoParts {
    const float* x = nullptr;
    const float* dy = nullptr;
    long long x_batch = 0, dy_batch = 0;
};

// Development override of the lines per stage (1, 2 or 4); 0 = choose from the stage size.
int forced_lps() {
    static const int v = [] {
        const char* e = std::getenv("CB_WGRAD_LPS");
        return e ? std::atoi(e) : 0;
    }();
    return v;
}
// Development override of the fewest line groups a CTA takes; 0 = from the 256-pixel rule.
int forced_min_groups() {
    static const int v = [] {
        const char* e = std::getenv("CB_WGRAD_MINGROUPS");
        return e ? std::atoi(e) : 0;
    }();
    return v;
}

}  // namespace

// dW (+)= contraction over the pixels of N x Cin x IH x IW planes `X` and N x OC x IH x IW planes `dY` with taps
// (FH, FW, pH, pW) in the same-size convention of the forward kernel. s2 / IC_src: see wgrad_reduce_kernel.
static int wgrad_core(cb_ctx* ctx, const float* dY, const float* X, float* dW, int N, int Cin, int IH, int IW, int OC, int FH,
                      int FW, int pH, int pW, int accumulate, int s2, int IC_src, long long dy_batch, long long x_batch,
                      int IC_total = 0, int c_off = 0, int oc_off = 0, const LoParts& lo = LoParts()) {
    if (IC_total == 0) IC_total = Cin;
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
    const uint32_t line_bytes = ((uint32_t)rows_stage * kRowBytes + 1023u) & ~1023u;
    const long long smem_cap = (long long)ctx->max_smem_optin - 2048;
    if (smem_cap / line_bytes < 2) return CB_EUNSUPPORTED;
    int lps = 1;
    for (int cand = 4; cand >= 2; cand >>= 1)
        if (smem_cap / ((long long)cand * line_bytes) >= 3) { lps = cand; break; }
    if (forced_lps() && smem_cap / ((long long)forced_lps() * line_bytes) >= 2) lps = forced_lps();
    const uint32_t stage_bytes = (uint32_t)lps * line_bytes;
    long long stages = smem_cap / stage_bytes;
    if (stages > kConvMaxStages) stages = kConvMaxStages;

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
    p.line_bytes = line_bytes;
    p.stage_bytes = stage_bytes;
    p.a_bytes = (uint32_t)rowsA * kRowBytes;
    p.lps = lps;
    p.groups = (int)((p.total_lines + lps - 1) / lps);
    p.vgroups = lo.x ? 3 * p.groups : p.groups;
    p.status = ctx->d_status;
    p.trace = ctx->trace;
    // One CTA per line group up to the SM count: fewer, longer CTAs (fewer partial sums to write and reduce) measured
    // slower on every layer shape of the models.
    int min_groups = forced_min_groups() ? forced_min_groups() : 1;
    int grid = p.vgroups / min_groups;
    if (grid < 1) grid = 1;
    if (grid > ctx->sm_count) grid = ctx->sm_count;
    static const int max_grid = [] {
        const char* e = std::getenv("CB_WGRAD_MAXGRID");  // development override
        return e ? std::atoi(e) : 0;
    }();
    if (max_grid > 0 && grid > max_grid) grid = max_grid;
    else if (max_grid == 0 && ctx->wgrad_grid_cap > 0 && grid > ctx->wgrad_grid_cap) grid = ctx->wgrad_grid_cap;
    // Partial sums: one tile per CTA added in a fixed order by the second kernel (deterministic contexts), or one
    // zero-filled tile that every CTA adds into with atomics and the second kernel moves into dW and clears again.
    static const int allow_atomic = [] {
        const char* e = std::getenv("CB_WGRAD_ATOMIC");  // development switch, default on
        return e ? std::atoi(e) : 1;
    }();
    p.atomic = (!ctx->deterministic && allow_atomic) ? 1 : 0;
    static const int issue_mode = [] {
        // development override: 0 one lane (default: with back-to-back UMMAs the tensor core's operand fetches starve
        // the shift warps' shared-memory traffic and every layer shape measured 5-20 % slower), 1 whole warp
        const char* e = std::getenv("CB_WGRAD_ISSUE");
        return e ? std::atoi(e) : 0;
    }();
    p.issue_uniform = issue_mode;
    static const int allow_direct = [] {
        const char* e = std::getenv("CB_WGRAD_DIRECT");  // development switch, default on
        return e ? std::atoi(e) : 1;
    }();
    p.s2 = s2; p.IC_src = IC_src;
    static const int allow_cf = [] {
        const char* e = std::getenv("CB_WGRAD_ROWBOX");  // development switch, default on
        return e ? std::atoi(e) : 1;
    }();
    p.rows_cf = (allow_cf && IW == 32 && FH > 1 && !s2) ? 1 : 0;
    p.run = s2 ? IC_src * 9 : Cin * FH * FW;
    p.oc_stride = s2 ? (long long)IC_src * 9 : (long long)IC_total * FH * FW;
    p.base_off = s2 ? 0 : ((long long)oc_off * IC_total + c_off) * FH * FW;
    p.dW = dW;
    static const long long direct_limit = [] {
        const char* e = std::getenv("CB_WGRAD_DIRECT_LIMIT");  // development override: most weights of a direct launch
        return e ? std::atoll(e) : 1LL << 30;
    }();
    p.direct = (p.atomic && allow_direct && (long long)OC * p.run * 4 <= stages * (long long)stage_bytes &&
                (long long)OC * p.run <= direct_limit) ? 1 : 0;
    p.vec4 = ((p.run & 3) == 0 && (p.oc_stride & 3) == 0 && (p.base_off & 3) == 0 &&
              (reinterpret_cast<uintptr_t>(dW) & 15u) == 0) ? 1 : 0;
    int rc;
    if (p.direct) {
        if (!accumulate) {
            cudaError_t em = cudaMemset2DAsync(dW + p.base_off, (size_t)p.oc_stride * 4, 0, (size_t)p.run * 4, (size_t)OC, ctx->stream);
            if (em != cudaSuccess) return check_cuda(ctx, em, "cudaMemset2DAsync(weight gradient)");
        }
    } else if (p.atomic) {
        rc = ensure_wgrad_acc(ctx, (size_t)mtiles * 128 * NQ * sizeof(float));
        if (rc != CB_OK) return rc;
        p.partial = static_cast<float*>(ctx->wgrad_acc);
    } else {
        rc = ensure_workspace(ctx, (size_t)grid * mtiles * 128 * NQ * sizeof(float));
        if (rc != CB_OK) return rc;
        p.partial = static_cast<float*>(ctx->workspace);
    }

    CUtensorMap tmX, tmdY;
    // X as (32 px, image row, channel, image) with a box of FH rows, or as (pixel, channel, image) with a box per tap
    auto encode_x = [&](CUtensorMap* tm, const float* base, long long batch) -> int {
        const uint64_t bstride = (uint64_t)(batch ? batch : (long long)Cin * IH * IW) * 4;
        if (bstride & 15u) return CB_EUNSUPPORTED;
        if (p.rows_cf) {
            uint64_t dims[4] = {32u, (uint64_t)IH, (uint64_t)Cin, (uint64_t)N};
            uint64_t str[3] = {128u, (uint64_t)IH * IW * 4, bstride};
            uint32_t box[4] = {32u, (uint32_t)FH, (uint32_t)Cp, 1u};
            return encode_tmap(ctx, tm, base, 4, dims, str, box, nullptr, 128);
        }
        uint64_t dims[3] = {(uint64_t)IH * IW, (uint64_t)Cin, (uint64_t)N};
        uint64_t str[2] = {(uint64_t)IH * IW * 4, bstride};
        uint32_t box[3] = {32u, (uint32_t)Cp, 1u};
        return encode_tmap(ctx, tm, base, 3, dims, str, box, nullptr, 128);
    };
    rc = encode_x(&tmX, X, x_batch);
    if (rc != CB_OK) return rc;
    {
        uint64_t dims[3] = {(uint64_t)IH * IW, (uint64_t)OC, (uint64_t)N};
        uint64_t str[2] = {(uint64_t)IH * IW * 4, (uint64_t)(dy_batch ? dy_batch : (long long)OC * IH * IW) * 4};
        if (str[1] & 15u) return CB_EUNSUPPORTED;
        uint32_t box[3] = {32u, (uint32_t)OCp, 1u};
        rc = encode_tmap(ctx, &tmdY, dY, 3, dims, str, box, nullptr, 128);
        if (rc != CB_OK) return rc;
    }
    CUtensorMap tmXlo = tmX, tmdYlo = tmdY;
    if (lo.x) {
        rc = encode_x(&tmXlo, lo.x, lo.x_batch);
        if (rc != CB_OK) return rc;
        uint64_t dimsy[3] = {(uint64_t)IH * IW, (uint64_t)OC, (uint64_t)N};
        uint64_t stry[2] = {(uint64_t)IH * IW * 4, (uint64_t)(lo.dy_batch ? lo.dy_batch : (long long)OC * IH * IW) * 4};
        uint32_t boxy[3] = {32u, (uint32_t)OCp, 1u};
        rc = encode_tmap(ctx, &tmdYlo, lo.dy, 3, dimsy, stry, boxy, nullptr, 128);
        if (rc != CB_OK) return rc;
    }
    const size_t smem = (size_t)p.stages * stage_bytes + 1024;
    int smem_bound = 0;
    cudaError_t e = raise_dynamic_smem_once(umma_wgrad_kernel, ctx->device, ctx->max_smem_optin, &smem_bound);
    if (e != cudaSuccess) return check_cuda(ctx, e, "umma_wgrad_kernel attribute");
    if ((int)smem > smem_bound) return CB_EUNSUPPORTED;
    e = launch_dep(ctx, umma_wgrad_kernel, dim3((unsigned)grid), dim3(192 + 32 * kShiftWarps), smem, tmX, tmdY, tmXlo, tmdYlo, p);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "umma_wgrad_kernel launch");
    if (p.direct) {
        ctx->launches += 1;
        ctx->last_kernel = "umma_tf32";
        return CB_OK;
    }
    const int rgrid = NQ * ((rowsA + 31) / 32);
    static const int groups = [] {
        const char* env = std::getenv("CB_WGRAD_REDUCE_GROUPS");  // development override: 2, 4 or 8
        const int v = env ? std::atoi(env) : 8;
        return v == 2 || v == 4 ? v : 8;
    }();
    auto* reduce = groups == 2 ? wgrad_reduce_kernel<2> : (groups == 4 ? wgrad_reduce_kernel<4> : wgrad_reduce_kernel<8>);
    if (p.atomic)
        e = launch_dep(ctx, wgrad_reduce_kernel<8>, dim3((unsigned)((rgrid + 7) / 8)), dim3(32, 8), 0, p.partial, dW, 1, mtiles * 128,
                       rowsA, NQ, Cp, Cin, OC, OCp, FH, FW, accumulate ? 1 : 0, s2, IC_src, 1, IC_total, c_off, oc_off, p.rows_cf);
    else
        e = launch_dep(ctx, reduce, dim3((unsigned)rgrid), dim3(32, (unsigned)groups), 0, p.partial, dW, grid, mtiles * 128,
                       rowsA, NQ, Cp, Cin, OC, OCp, FH, FW, accumulate ? 1 : 0, s2, IC_src, 0, IC_total, c_off, oc_off, p.rows_cf);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "wgrad_reduce_kernel launch");
    ctx->launches += 2;
    ctx->last_kernel = "umma_tf32";
    return CB_OK;
}

int umma_conv_wgrad(cb_ctx* ctx, const float* dY, const float* X, float* dW, int N, int IC, int IH, int IW, int OC,
                    int FH, int FW, int sH, int sW, int pH, int pW, int accumulate, long long dy_batch, long long x_batch,
                    bool x3) {
    // 3xTF32: lo parts of the two operands (as the kernel will read them: after the stride-2 re-layout) in scratch
    auto make_lo = [&](const float* Xsrc, long long x_per, long long xb, const float* dYsrc, long long dy_per, long long yb,
                       LoParts& lo) -> int {
        auto up = [](long long n) { return (n + 63) & ~63LL; };
        const long long xe = (long long)N * x_per, ye = (long long)N * dy_per;
        int rc = ensure_workspace3(ctx, (size_t)(up(xe) + up(ye)) * sizeof(float));
        if (rc != CB_OK) return rc;
        float* xl = static_cast<float*>(ctx->workspace3);
        float* yl = xl + up(xe);
        rc = launch_lo(ctx, Xsrc, xl, N, x_per, xb);
        if (rc == CB_OK) rc = launch_lo(ctx, dYsrc, yl, N, dy_per, yb);
        lo.x = xl; lo.dy = yl; lo.x_batch = x_per; lo.dy_batch = dy_per;
        return rc;
    };
    if (N < 1 || ((long long)IH * IW & 3)) return CB_EUNSUPPORTED;
    if (sH == 1 && sW == 1) {
        if (!((FH == 1 && pH == 0) || (FH == 3 && pH == 1))) return CB_EUNSUPPORTED;
        if (!((FW == 1 && pW == 0) || (FW == 3 && pW == 1))) return CB_EUNSUPPORTED;
        // Filters wider than one launch covers (256 input channels, 128 output channels, 512 accumulator columns) are
        // cut into blocks of input x output channels: each block is its own launch pair on channel slices of X and dY
        // (same batch strides) that writes its block of dW.
        const int OCp_all = (OC + 15) / 16 * 16;
        int oc_max = (256 / FW) & ~15;
        if (oc_max > 128) oc_max = 128;
        const int oc_blocks = (OCp_all + oc_max - 1) / oc_max;
        const int oc_step = ((OC + oc_blocks - 1) / oc_blocks + 15) & ~15;
        const int nq = FW * (oc_blocks > 1 ? oc_step : OCp_all);
        int c_max = ((512 / nq) * 128 / FH) & ~7;
        if (c_max > 256) c_max = 256;
        if (c_max < 8) return CB_EUNSUPPORTED;
        const int c_blocks = (IC + c_max - 1) / c_max;
        const int c_step = ((IC + c_blocks - 1) / c_blocks + 7) & ~7;
        if (IW != 8 && IW != 16 && IW != 32) return CB_EUNSUPPORTED;  // before the lo parts are queued
        const long long plane = (long long)IH * IW;
        LoParts lo;
        if (x3) {
            const int rc = make_lo(X, (long long)IC * plane, x_batch, dY, (long long)OC * plane, dy_batch, lo);
            if (rc != CB_OK) return rc;
        }
        if (oc_blocks == 1 && c_blocks == 1)
            return wgrad_core(ctx, dY, X, dW, N, IC, IH, IW, OC, FH, FW, pH, pW, accumulate, 0, IC, dy_batch, x_batch, 0, 0, 0, lo);
        const long long xb = x_batch ? x_batch : (long long)IC * plane, yb = dy_batch ? dy_batch : (long long)OC * plane;
        for (int o0 = 0; o0 < OC; o0 += oc_step) {
            const int on = OC - o0 < oc_step ? OC - o0 : oc_step;
            for (int c0 = 0; c0 < IC; c0 += c_step) {
                const int cn = IC - c0 < c_step ? IC - c0 : c_step;
                LoParts lc = lo;
                if (x3) { lc.x = lo.x + c0 * plane; lc.dy = lo.dy + o0 * plane; }
                const int rc = wgrad_core(ctx, dY + o0 * plane, X + c0 * plane, dW, N, cn, IH, IW, on, FH, FW, pH, pW, accumulate, 0, cn,
                                          yb, xb, IC, c0, o0, lc);
                if (rc != CB_OK) return rc;
            }
        }
        return CB_OK;
    }
    if (sH != 2 || sW != 2 || FH != FW || pH != pW || (IH & 1) || (IW & 1)) return CB_EUNSUPPORTED;
    if (!((FH == 3 && pH == 1) || (FH == 1 && pH == 0))) return CB_EUNSUPPORTED;
    if (dy_batch || x_batch) return CB_EUNSUPPORTED;  // the stride-2 path re-lays dense tensors out
    const int H2 = IH / 2, W2 = IW / 2;
    if (W2 != 8 && W2 != 16 && W2 != 32) return CB_EUNSUPPORTED;
    const long long plane2 = (long long)H2 * W2;
    if (FH == 1) {
        const long long n_sub = (long long)N * IC * plane2;
        int rc = ensure_workspace2(ctx, (size_t)n_sub * sizeof(float));
        if (rc != CB_OK) return rc;
        float* sub = static_cast<float*>(ctx->workspace2);
        rc = launch_subsample2(ctx, X, sub, (long long)N * IC, IH, IW);
        if (rc != CB_OK) return rc;
        LoParts lo;
        if (x3) {
            rc = make_lo(sub, (long long)IC * plane2, 0, dY, (long long)OC * plane2, 0, lo);
            if (rc != CB_OK) return rc;
        }
        return wgrad_core(ctx, dY, sub, dW, N, IC, H2, W2, OC, 1, 1, 0, 0, accumulate, 0, IC, 0, 0, 0, 0, 0, lo);
    }
    if (4 * IC > 256) return CB_EUNSUPPORTED;
    const long long n_el = (long long)N * 4 * IC * plane2;
    int rc = ensure_workspace2(ctx, (size_t)n_el * sizeof(float));
    if (rc != CB_OK) return rc;
    float* Xs = static_cast<float*>(ctx->workspace2);
    rc = launch_space_to_depth2(ctx, X, Xs, N, IC, IH, IW);
    if (rc != CB_OK) return rc;
    LoParts lo;
    if (x3) {
        rc = make_lo(Xs, 4LL * IC * plane2, 0, dY, (long long)OC * plane2, 0, lo);
        if (rc != CB_OK) return rc;
    }
    return wgrad_core(ctx, dY, Xs, dW, N, 4 * IC, H2, W2, OC, 2, 2, 1, 1, accumulate, 1, IC, 0, 0, 0, 0, 0, lo);
}

}  // namespace cb
