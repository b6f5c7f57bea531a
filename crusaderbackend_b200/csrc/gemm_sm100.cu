// fp32 GEMM for sm_100a on the 5th-generation tensor cores.
//
// One persistent, warp-specialised kernel computes D[i][j] = sum_k P[i][k] * Q[j][k]:
//   warp 0      TMA producer: cp.async.bulk.tensor tiles into 128B-swizzled shared memory, mbarrier pipeline
//   warp 1      UMMA issuer: one lane issues tcgen05.mma kind::tf32 (M=128, N=bn, K=8), accumulators in TMEM
//   warps 2..17 epilogue: tcgen05.ld -> registers -> bias/ReLU -> global stores (four warps per TMEM lane quarter)
//   warps 18..21 (3xTF32 only) split warps: write lo = a - tf32(a) beside each stage
// P is the operand on the UMMA M side (128 TMEM lanes), Q the one on the N side (TMEM columns). Each operand
// is either K-major (k contiguous in memory) or MN-major (i / j contiguous); both are fed by TMA without
// a transpose: K-major tiles are [rows][32 k] boxes (128B swizzle), MN-major tiles are [32 k][32 rows] boxes
// (128B swizzle with 32-byte atoms, the one layout the tensor core takes for MN-major tf32), and the UMMA
// shared-memory descriptor names the layout.
//
// The row-major product C = op(A) * op(B) of the seblas GEMMs (seblas/operations/cuGEMM.cu:1649-1714) maps to
// P = op(B)^T (i = column of C) and Q = op(A) (j = row of C), so that the 32 lanes of an epilogue warp hold 32
// consecutive columns of one row of C and every store instruction writes one full 128-byte line.
//
// 3xTF32: a = hi + lo with hi = the 19 high bits the tensor core reads from the fp32 word, lo = a - hi
// (exact), rounded to TF32. D = P_hi*Q_lo + P_lo*Q_hi + P_hi*Q_hi; the dropped lo*lo term is < 2^-20 |p q|.
#include <utility>

#include <cstdlib>

#include "cb_internal.h"
#include "cb_ptx.cuh"

namespace cb {

namespace {

constexpr int kMaxStages = 8;
constexpr int kEpiWarps = 16;     // epilogue warps (4 per TMEM lane quarter)
constexpr int kBK = 32;            // fp32 elements per k-block = one 128-byte swizzle row
constexpr int kPTileBytes = 128 * kBK * 4;

struct GemmParams {
    int I, J, K, batch;
    int tiles_i, tiles_j;  // tile counts (tile = 128*mi rows of i, bn of j)
    int mi, bn;            // P sub-tiles per CTA tile, UMMA N
    int stages;
    int num_kb, splits, kb_per_split;
    int kb_per_fold;       // > 0: the k-blocks walk `kfold` operand pairs of kb_per_fold blocks each (their products are summed)
    int kc;                // k-blocks per accumulation chunk: the accumulator is drained to C every kc blocks
    int tmem_cols;         // allocated TMEM columns (power of two >= 2*bn)
    int p_batched, q_batched;
    int p_wide, q_wide;    // MN-major operand whose extent is a multiple of 32: all 32-wide slices of a tile in ONE TMA box
    float* C;
    long long ldc, strideC;
    int out_mode, accumulate, atomic_out;
    const float* bias_i;
    const float* bias_j;
    int relu;
    int* status;
};

struct __align__(8) PipeSmem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t xf[kMaxStages];
    uint64_t tfull[2];
    uint64_t tempty[2];
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

// K-major tile: rows of 128 bytes (32 k), 8-row groups 1024 bytes apart, 16-byte chunks swizzled (SW128).
__device__ __forceinline__ uint64_t desc_k(uint32_t addr) { return umma_smem_desc(addr, 16u, 1024u, UMMA_SW_128B); }
// MN-major tile: one [32 k][128 bytes of i/j] box per 32 rows of the operand, boxes 4096 bytes apart (LBO),
// 4-row groups 512 bytes apart (SBO), 32-byte chunks swizzled (SW128 base 32B).
__device__ __forceinline__ uint64_t desc_mn(uint32_t addr) {
    return umma_smem_desc(addr, 4096u, 512u, UMMA_SW_128B_BASE32B);
}

struct WorkItem {
    int b, i0, j0, kb0, kb1, split;
};

__device__ __forceinline__ WorkItem decode_work(const GemmParams& p, int w) {
    WorkItem it;
    const int tile = w / p.splits;
    it.split = w - tile * p.splits;
    const int per_batch = p.tiles_i * p.tiles_j;
    it.b = tile / per_batch;
    int r = tile - it.b * per_batch;
    // groups of 8 j-tiles, i fastest inside a group: concurrent CTAs share a near-square footprint in L2
    const int gw = 8;
    const int group = r / (gw * p.tiles_i);
    const int rg = r - group * gw * p.tiles_i;
    const int jw = min(gw, p.tiles_j - group * gw);
    const int ti = rg / jw;
    const int tj = group * gw + (rg - ti * jw);
    it.i0 = ti * 128 * p.mi;
    it.j0 = tj * p.bn;
    it.kb0 = it.split * p.kb_per_split;
    it.kb1 = min(p.num_kb, it.kb0 + p.kb_per_split);
    return it;
}

template <bool P_MN, bool Q_MN, bool X3>
__global__ void __launch_bounds__(X3 ? 64 + 32 * kEpiWarps + 128 : 64 + 32 * kEpiWarps, 1)
    umma_gemm_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
                     const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ PipeSmem ps;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int* abort_flag = &ps.abort_flag;

    const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t p_bytes = (uint32_t)p.mi * kPTileBytes;
    const uint32_t q_bytes = (uint32_t)p.bn * kBK * 4;
    const uint32_t hi_bytes = p_bytes + q_bytes;
    const uint32_t stage_bytes = X3 ? 2 * hi_bytes : hi_bytes;

    if (threadIdx.x == 0) {
        ps.abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&ps.full[s]), 1);
            mbar_init(smem_u32(&ps.empty[s]), 1);
            mbar_init(smem_u32(&ps.xf[s]), 128);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&ps.tfull[a]), 1);
            mbar_init(smem_u32(&ps.tempty[a]), 32 * kEpiWarps);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmP);
        tma_prefetch_desc(&tmQ);
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc(smem_u32(&ps.tmem_base), (uint32_t)p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ps.tmem_base;
    const uint32_t acc_stride = (uint32_t)p.tmem_cols >> 1;  // column offset of accumulator 1

    const int total_work = p.batch * p.tiles_i * p.tiles_j * p.splits;
    uint32_t armed = 0, armed_parity = 0;  // producer lane: stages armed at least once / parity of their last arming

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
            const WorkItem it = decode_work(p, w);
            for (int kb = it.kb0; kb < it.kb1; ++kb) {
                // operand pair and k-offset of this block: the batch index of the work item, or, with the batch folded
                // into K, the pair the block falls in (the tail of every pair is zero-filled by TMA)
                int pair = it.b, kk = kb;
                if (p.kb_per_fold) {
                    pair = kb / p.kb_per_fold;
                    kk = kb - pair * p.kb_per_fold;
                }
                const int bp = p.p_batched ? pair : 0;
                const int bq = p.q_batched ? pair : 0;
                ok = warp_wait(smem_u32(&ps.empty[s]), ph ^ 1u, lane, abort_flag, p.status, CBK_TIMEOUT_EMPTY);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t full = smem_u32(&ps.full[s]);
                    const uint32_t sP = tiles_base + s * stage_bytes;
                    const uint32_t sQ = sP + p_bytes;
                    mbar_expect_tx(full, hi_bytes);
                    armed |= 1u << s;
                    armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
                    const int k0 = kk * kBK;
                    if (P_MN) {
                        if (p.p_wide) {
                            tma_load_4d(sP, &tmP, full, 0, k0, it.i0 >> 5, bp);
                        } else {
                            for (int bx = 0; bx < 4 * p.mi; ++bx)
                                tma_load_3d(sP + bx * 4096u, &tmP, full, it.i0 + 32 * bx, k0, bp);
                        }
                    } else {
                        for (int m = 0; m < p.mi; ++m)
                            tma_load_3d(sP + m * kPTileBytes, &tmP, full, k0, it.i0 + 128 * m, bp);
                    }
                    if (Q_MN) {
                        if (p.q_wide) {
                            tma_load_4d(sQ, &tmQ, full, 0, k0, it.j0 >> 5, bq);
                        } else {
                            for (int bx = 0; bx < (p.bn >> 5); ++bx)
                                tma_load_3d(sQ + bx * 4096u, &tmQ, full, it.j0 + 32 * bx, k0, bq);
                        }
                    } else {
                        tma_load_3d(sQ, &tmQ, full, k0, it.j0, bq);
                    }
                }
                __syncwarp();
                if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ UMMA issuer
        // One thread feeds the tensor core, so the instructions it spends per tcgen05.mma bound the whole kernel:
        // the descriptors of a stage are built once and advanced by constant adds, the chunk position is a counter
        // (no division), and everything that is not an UMMA stays outside the unrolled k-step loop.
        const uint32_t idesc = umma_idesc_tf32(128, (uint32_t)p.bn, P_MN ? 1u : 0u, Q_MN ? 1u : 0u);
        constexpr uint64_t kStepP = P_MN ? (1024u >> 4) : (32u >> 4);  // descriptor address units (16 B) per k-step
        constexpr uint64_t kStepQ = Q_MN ? (1024u >> 4) : (32u >> 4);
        const uint64_t descP0 = P_MN ? desc_mn(0) : desc_k(0);  // layout bits; the start address is added below
        const uint64_t descQ0 = Q_MN ? desc_mn(0) : desc_k(0);
        const uint64_t lo_units = (uint64_t)(hi_bytes >> 4);
        uint32_t s = 0, ph = 0;
        uint32_t sub = 0;  // running accumulator sub-tile counter
        bool ok = true;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
            const WorkItem it = decode_work(p, w);
            int kc_pos = 0;
            for (int kb = it.kb0; kb < it.kb1 && ok; ++kb) {
                ok = warp_wait(smem_u32(&ps.full[s]), ph, lane, abort_flag, p.status, CBK_TIMEOUT_FULL);
                if (!ok) break;
                if (X3) {
                    ok = warp_wait(smem_u32(&ps.xf[s]), ph, lane, abort_flag, p.status, CBK_TIMEOUT_XFORM);
                    if (!ok) break;
                }
                tc_fence_after();
                const bool chunk_first = kc_pos == 0;
                const bool chunk_last = kc_pos == p.kc - 1 || kb == it.kb1 - 1;
                kc_pos = chunk_last ? 0 : kc_pos + 1;
                const uint32_t sP = tiles_base + s * stage_bytes;
                if (chunk_first) {
                    // first product into these accumulators: the epilogue must have drained their last use
                    for (int m = 0; m < p.mi && ok; ++m) {
                        const uint32_t u = sub + (uint32_t)m;
                        ok = warp_wait(smem_u32(&ps.tempty[u & 1u]), ((u >> 1) & 1u) ^ 1u, lane, abort_flag, p.status,
                                       CBK_TIMEOUT_TMEM_EMPTY);
                    }
                    if (!ok) break;
                    tc_fence_after();
                }
                // TF32: the whole warp runs this block with the same values and one elected lane issues — in a one-lane
                // branch a descriptor that changes from UMMA to UMMA costs ~110 cycles of issue each (measured with the
                // UMMA-only loop of peak_sm100.cu), most of a 128 x 256 x 8 UMMA's 137 cycles. 3xTF32 keeps the one-lane
                // form: with back-to-back UMMAs the tensor core's operand fetches starve the split warps' shared-memory
                // traffic and the whole pipeline ran 20-35 % slower.
                constexpr bool kElect = !X3;
                if (kElect || lane == 0) {
                    const uint64_t dQ = descQ0 + (uint64_t)(((sP + p_bytes) >> 4) & 0x3FFFu);
                    const uint32_t first = chunk_first ? 0u : 1u;
                    for (int m = 0; m < p.mi; ++m) {
                        const uint32_t d_tmem = tmem_base + ((sub + (uint32_t)m) & 1u) * acc_stride;
                        const uint64_t dP = descP0 + (uint64_t)(((sP + (uint32_t)m * (uint32_t)kPTileBytes) >> 4) & 0x3FFFu);
                        if (X3) {
#pragma unroll
                            for (int kk = 0; kk < kBK / 8; ++kk) {
                                const uint64_t a = dP + kk * kStepP, b = dQ + kk * kStepQ;
                                umma_tf32_sel<kElect>(d_tmem, a, b + lo_units, idesc, kk == 0 ? first : 1u);
                                umma_tf32_sel<kElect>(d_tmem, a + lo_units, b, idesc, 1u);
                                umma_tf32_sel<kElect>(d_tmem, a, b, idesc, 1u);
                            }
                        } else {
                            umma_tf32_sel<kElect>(d_tmem, dP, dQ, idesc, first);
                            umma_tf32_sel<kElect>(d_tmem, dP + kStepP, dQ + kStepQ, idesc, 1u);
                            umma_tf32_sel<kElect>(d_tmem, dP + 2 * kStepP, dQ + 2 * kStepQ, idesc, 1u);
                            umma_tf32_sel<kElect>(d_tmem, dP + 3 * kStepP, dQ + 3 * kStepQ, idesc, 1u);
                        }
                    }
                    tc_commit_sel<kElect>(smem_u32(&ps.empty[s]));  // stage reusable once these MMAs retire
                    if (chunk_last)
                        for (int m = 0; m < p.mi; ++m) tc_commit_sel<kElect>(smem_u32(&ps.tfull[(sub + m) & 1u]));
                }
                __syncwarp();
                if (chunk_last) sub += (uint32_t)p.mi;
                if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp < 2 + kEpiWarps) {
        // ------------------------------------------------------------ epilogue (TMEM -> global)
        // One warp per scheduler cannot hide the latencies of the epilogue's loads and stores (in 3xTF32 mode the
        // read-modify-write drains sit on the critical path), so each TMEM lane quarter is served by four warps that
        // split the column chunks between them.
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are visible to this warp
        const int slot = (warp - 2) >> 2;
        uint32_t sub = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
            const WorkItem it = decode_work(p, w);
            float* Cb = p.C + (long long)it.b * p.strideC;
            const int nchunks = (it.kb1 - it.kb0 + p.kc - 1) / p.kc;
            for (int ch = 0; ch < nchunks && ok; ++ch) {
                const bool add_bias = (it.split == 0 && ch == 0);
                const bool add_old = p.accumulate || ch > 0;      // later chunks add onto what this thread wrote
                const bool relu_now = p.relu && ch == nchunks - 1;
                for (int m = 0; m < p.mi && ok; ++m, ++sub) {
                    const uint32_t a = sub & 1u;
                    ok = mbar_wait_warp(smem_u32(&ps.tfull[a]), (sub >> 1) & 1u, lane, abort_flag, p.status,
                                        CBK_TIMEOUT_TMEM_FULL, 512);
                    if (!ok) break;
                    tc_fence_after();
                    const int i = it.i0 + 128 * m + 32 * quarter + lane;
                    const bool i_ok = i < p.I;
                    float bi = 0.f;
                    if (p.bias_i != nullptr && i_ok && add_bias) bi = p.bias_i[i];
                    const uint32_t t_row = tmem_base + a * acc_stride + ((uint32_t)(32 * quarter) << 16);
                    for (int c = slot * 16; c < p.bn; c += 16 * (kEpiWarps / 4)) {
                        if (it.j0 + c >= p.J) break;  // warp-uniform
                        uint32_t r[16];
                        tmem_ld16(t_row + (uint32_t)c, r);
                        tmem_ld_wait();
                        if (!i_ok) continue;
                        if (p.out_mode == 0) {
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                const int j = it.j0 + c + e;
                                if (j < p.J) {
                                    float v = __uint_as_float(r[e]) + bi;
                                    if (p.bias_j != nullptr && add_bias) v += p.bias_j[j];
                                    float* dst = Cb + (long long)j * p.ldc + i;
                                    if (p.atomic_out) {
                                        atomicAdd(dst, v);
                                    } else {
                                        if (add_old) v += *dst;
                                        if (relu_now) v = fmaxf(v, 0.f);
                                        *dst = v;
                                    }
                                }
                            }
                        } else {
                            float* row = Cb + (long long)i * p.ldc + it.j0 + c;
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                const int j = it.j0 + c + e;
                                if (j < p.J) {
                                    float v = __uint_as_float(r[e]) + bi;
                                    if (p.bias_j != nullptr && add_bias) v += p.bias_j[j];
                                    if (p.atomic_out) {
                                        atomicAdd(row + e, v);
                                    } else {
                                        if (add_old) v += row[e];
                                        if (relu_now) v = fmaxf(v, 0.f);
                                        row[e] = v;
                                    }
                                }
                            }
                        }
                    }
                    tc_fence_before();
                    mbar_arrive(smem_u32(&ps.tempty[a]));
                }
            }
        }
    } else {
        // ------------------------------------------------------------ split warps (3xTF32 only)
        if (X3) {
            const int t = threadIdx.x - (64 + 32 * kEpiWarps);  // 0..127
            uint32_t s = 0, ph = 0;
            bool ok = true;
            const uint32_t n_vec = hi_bytes >> 4;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
                const WorkItem it = decode_work(p, w);
                for (int kb = it.kb0; kb < it.kb1; ++kb) {
                    ok = mbar_wait_warp(smem_u32(&ps.full[s]), ph, lane, abort_flag, p.status, CBK_TIMEOUT_XFORM_FULL, 64);
                    if (!ok) break;
                    const uint32_t src = tiles_base + s * stage_bytes;
                    const uint32_t dst = src + hi_bytes;
                    for (uint32_t v = (uint32_t)t; v < n_vec; v += 128u) {
                        float4 x;
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w)
                                     : "r"(src + v * 16u));
                        uint32_t l0, l1, l2, l3;
                        {
                            const float h0 = __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u);
                            const float h1 = __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
                            const float h2 = __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u);
                            const float h3 = __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
                            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l0) : "f"(x.x - h0));
                            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l1) : "f"(x.y - h1));
                            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l2) : "f"(x.z - h2));
                            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l3) : "f"(x.w - h3));
                        }
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + v * 16u), "r"(l0), "r"(l1),
                                     "r"(l2), "r"(l3)
                                     : "memory");
                    }
                    fence_proxy_async_smem();
                    mbar_arrive(smem_u32(&ps.xf[s]));
                    if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (ps.abort_flag) {
        // A bounded wait gave up somewhere in this CTA: copies armed before that may still be in flight towards its
        // shared memory and issued MMAs may still run on its accumulators; both get a bounded chance to finish before
        // the shared memory and TMEM are released.
        if (warp == 0 && lane == 0) {
            for (int st = 0; st < p.stages; ++st)
                if ((armed >> st) & 1u) mbar_drain(smem_u32(&ps.full[st]), (armed_parity >> st) & 1u, p.status);
        }
        if (warp == 1) {  // the commit comes from the lane that issued the MMAs
            if (!X3) tc_commit_elect(smem_u32(&ps.drain));
            else if (lane == 0) tc_commit(smem_u32(&ps.drain));
            if (lane == 0) mbar_drain(smem_u32(&ps.drain), 0, p.status);
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
}

// ------------------------------------------------------------------ CUDA-core fp32 kernel (any shape / alignment)
// 64x64 tile, 16-deep k slices, 256 threads x (4x4) outputs. Exact fp32 FMA in k order.
struct SimtParams {
    int I, J, K, batch;
    const float* P; long long ldp, strideP; int p_mn;
    const float* Q; long long ldq, strideQ; int q_mn;
    float* C; long long ldc, strideC; int out_mode, accumulate, atomic_out;
    const float* bias_i; const float* bias_j; int relu;
    int splits, k_per_split;
};

__global__ void __launch_bounds__(256) simt_gemm_kernel(const SimtParams p) {
    __shared__ float sP[16][64 + 4];
    __shared__ float sQ[16][64 + 4];
    const int b = blockIdx.z / p.splits;
    const int split = blockIdx.z - b * p.splits;
    const int i0 = blockIdx.x * 64, j0 = blockIdx.y * 64;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const float* Pb = p.P + (long long)b * p.strideP;
    const float* Qb = p.Q + (long long)b * p.strideQ;
    const int k_begin = split * p.k_per_split;
    const int k_end = min(p.K, k_begin + p.k_per_split);
    float acc[4][4] = {};
    for (int k0 = k_begin; k0 < k_end; k0 += 16) {
        for (int e = threadIdx.x; e < 16 * 64; e += 256) {
            int kk, r;
            if (p.p_mn) { r = e & 63; kk = e >> 6; } else { kk = e & 15; r = e >> 4; }
            const int i = i0 + r, k = k0 + kk;
            float v = 0.f;
            if (i < p.I && k < k_end) v = p.p_mn ? Pb[(long long)k * p.ldp + i] : Pb[(long long)i * p.ldp + k];
            sP[kk][r] = v;
        }
        for (int e = threadIdx.x; e < 16 * 64; e += 256) {
            int kk, r;
            if (p.q_mn) { r = e & 63; kk = e >> 6; } else { kk = e & 15; r = e >> 4; }
            const int j = j0 + r, k = k0 + kk;
            float v = 0.f;
            if (j < p.J && k < k_end) v = p.q_mn ? Qb[(long long)k * p.ldq + j] : Qb[(long long)j * p.ldq + k];
            sQ[kk][r] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], c[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) { a[x] = sP[kk][tx + 16 * x]; c[x] = sQ[kk][ty + 16 * x]; }
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(a[x], c[y], acc[x][y]);
        }
        __syncthreads();
    }
    float* Cb = p.C + (long long)b * p.strideC;
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            const int i = i0 + tx + 16 * x, j = j0 + ty + 16 * y;
            if (i < p.I && j < p.J) {
                float v = acc[x][y];
                if (split == 0) {
                    if (p.bias_i) v += p.bias_i[i];
                    if (p.bias_j) v += p.bias_j[j];
                }
                float* dst = p.out_mode == 0 ? Cb + (long long)j * p.ldc + i : Cb + (long long)i * p.ldc + j;
                if (p.atomic_out) {
                    atomicAdd(dst, v);
                } else {
                    if (p.accumulate) v += *dst;
                    if (p.relu) v = fmaxf(v, 0.f);
                    *dst = v;
                }
            }
        }
}

// Thin products (I <= 16, e.g. the 128 x 10 x 4096 dense-layer shape): HBM/latency-bound, so K is split over many CTAs,
// one warp per output row j with lanes striding k (128-bit-coalesced reads of Q when it is K-major), the I thin
// outputs per lane reduced with warp shuffles and added atomically into C (or stored when K is not split).
__global__ void __launch_bounds__(256) skinny_gemm_kernel(const SimtParams p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = blockIdx.x * 8 + warp;
    if (j >= p.J) return;
    const int split = blockIdx.y;
    const int k0 = split * p.k_per_split, k1 = min(p.K, k0 + p.k_per_split);
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (int k = k0 + lane; k < k1; k += 32) {
        const float q = p.q_mn ? p.Q[(long long)k * p.ldq + j] : p.Q[(long long)j * p.ldq + k];
        if (p.p_mn) {
            const float* pr = p.P + (long long)k * p.ldp;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (i < p.I) acc[i] = fmaf(q, pr[i], acc[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (i < p.I) acc[i] = fmaf(q, p.P[(long long)i * p.ldp + k], acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float v = acc[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[i] = v;
    }
    if (lane < p.I) {
        float v = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (i == lane) v = acc[i];
        if (split == 0) {
            if (p.bias_i) v += p.bias_i[lane];
            if (p.bias_j) v += p.bias_j[j];
        }
        float* dst = p.out_mode == 0 ? p.C + (long long)j * p.ldc + lane : p.C + (long long)lane * p.ldc + j;
        if (p.atomic_out) {
            atomicAdd(dst, v);
        } else {
            if (p.accumulate) v += *dst;
            if (p.relu) v = fmaxf(v, 0.f);
            *dst = v;
        }
    }
}

int zero_output(cb_ctx* ctx, const GemmCall& g) {
    // rows of the output as laid out in memory: out_mode 0 -> J rows of I floats, 1 -> I rows of J floats
    const size_t width = (size_t)(g.out_mode == 0 ? g.I : g.J) * 4;
    const size_t height = (size_t)(g.out_mode == 0 ? g.J : g.I);
    for (int b = 0; b < g.batch; ++b) {
        cudaError_t e = cudaMemset2DAsync(g.C + (long long)b * g.strideC, (size_t)g.ldc * 4, 0, width, height,
                                          ctx->stream);
        if (e != cudaSuccess) return check_cuda(ctx, e, "cudaMemset2DAsync(split-K output)");
    }
    return CB_OK;
}

template <bool P_MN, bool Q_MN>
cudaError_t launch_variant(cb_ctx* ctx, bool x3, dim3 grid, size_t smem, const CUtensorMap& tp, const CUtensorMap& tq,
                           const GemmParams& gp) {
    int bound = 0;
    cudaError_t e;
    if (x3) {
        e = raise_dynamic_smem_once(umma_gemm_kernel<P_MN, Q_MN, true>, ctx->device, ctx->max_smem_optin, &bound);
        if (e != cudaSuccess) return e;
        if ((int)smem > bound) return cudaErrorInvalidValue;
        umma_gemm_kernel<P_MN, Q_MN, true><<<grid, 64 + 32 * kEpiWarps + 128, smem, ctx->stream>>>(tp, tq, gp);
    } else {
        e = raise_dynamic_smem_once(umma_gemm_kernel<P_MN, Q_MN, false>, ctx->device, ctx->max_smem_optin, &bound);
        if (e != cudaSuccess) return e;
        if ((int)smem > bound) return cudaErrorInvalidValue;
        umma_gemm_kernel<P_MN, Q_MN, false><<<grid, 64 + 32 * kEpiWarps, smem, ctx->stream>>>(tp, tq, gp);
    }
    return cudaGetLastError();
}

}  // namespace

bool umma_gemm_eligible(const GemmCall& g) {
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (!aligned16(g.P) || !aligned16(g.Q)) return false;
    if ((g.ldp & 3) || (g.ldq & 3)) return false;
    if ((g.batch > 1 || g.kfold > 1) && ((g.strideP & 3) || (g.strideQ & 3))) return false;
    if (g.kfold > 1 && g.batch != 1) return false;
    if (g.I < 1 || g.J < 1 || g.K < 1) return false;
    return true;
}

int launch_umma_gemm(cb_ctx* ctx, const GemmCall& g, bool x3) {
    // ---- tile configuration
    const int kfold = g.kfold > 1 ? g.kfold : 1;
    const int num_kb = kfold * ((g.K + kBK - 1) / kBK);
    const int smem_cap = ctx->max_smem_optin - 2048;  // static barriers + 1 KB alignment slack
    int best_mi = 1, best_bn = 16, best_stages = 2, best_splits = 1;
    double best_cost = 1e300;
    const int j_gran = g.q_mn ? 32 : 16;
    for (int mi = 1; mi <= 2; ++mi) {
        if (mi == 2 && g.I <= 128) continue;
        for (int bn = 256; bn >= 16; bn >>= 1) {
            int bn_eff = bn;
            if (g.J <= bn) {  // single j tile: shrink to the granule that covers J
                bn_eff = ((g.J + j_gran - 1) / j_gran) * j_gran;
                if (bn_eff > 256) continue;
            }
            if (bn_eff < j_gran) continue;
            const int hi = mi * kPTileBytes + bn_eff * kBK * 4;
            const int stage = x3 ? 2 * hi : hi;
            int stages = smem_cap / stage;
            if (stages > kMaxStages) stages = kMaxStages;
            if (stages < 2) continue;
            const long long tiles = (long long)g.batch * ((g.I + 128 * mi - 1) / (128 * mi)) *
                                    ((g.J + bn_eff - 1) / bn_eff);
            int splits = 1;
            // split K across CTAs (atomic adds into C) only for outputs up to split_limit elements: atomics on a large C
            // cost more than the idle SMs they would fill
            static const long long split_limit = [] {
                const char* e = std::getenv("CB_GEMM_SPLIT_LIMIT");  // development override
                return e ? std::atoll(e) : 300000LL;
            }();
            if (!ctx->deterministic && g.ep.relu == 0 && tiles * 2 <= ctx->sm_count && num_kb >= 8 &&
                (long long)g.I * g.J * g.batch <= split_limit) {
                splits = (int)(ctx->sm_count / tiles);
                // at least four k-blocks per split, one for outputs so small that the atomic adds cost nothing
                const int min_kb = (long long)g.I * g.J * g.batch <= 4096 ? 1 : 4;
                if (splits > num_kb / min_kb) splits = num_kb / min_kb;
                if (splits < 1) splits = 1;
            }
            const long long work = tiles * splits;
            const long long waves = (work + ctx->sm_count - 1) / ctx->sm_count;
            const double kb_here = (double)((num_kb + splits - 1) / splits);
            // cycles per k-block: tensor pipe (128 x bn x 8 per ~bn/2 cycles) against ~40 B/clk of L2 feed
            const double mma_cyc = (x3 ? 3.0 : 1.0) * mi * 4.0 * (bn_eff / 2.0);
            const double feed_cyc = hi / 40.0 + (x3 ? hi / 48.0 : 0.0);
            const double epi_cyc = mi * bn_eff * 6.0 + 2000.0;
            const double cost = (double)waves * (kb_here * (mma_cyc > feed_cyc ? mma_cyc : feed_cyc) + epi_cyc);
            if (cost < best_cost) {
                best_cost = cost; best_mi = mi; best_bn = bn_eff; best_stages = stages; best_splits = splits;
            }
            if (g.J <= bn) break;  // smaller bn would only repeat bn_eff
        }
    }
    if (best_cost >= 1e300) return fail(ctx, CB_EUNSUPPORTED, "umma gemm: no tile configuration fits");

    GemmParams gp{};
    gp.I = g.I; gp.J = g.J; gp.K = g.K; gp.batch = g.batch;
    gp.mi = best_mi; gp.bn = best_bn; gp.stages = best_stages;
    gp.tiles_i = (g.I + 128 * gp.mi - 1) / (128 * gp.mi);
    gp.tiles_j = (g.J + gp.bn - 1) / gp.bn;
    gp.num_kb = num_kb;
    gp.splits = best_splits;
    gp.kb_per_split = (num_kb + gp.splits - 1) / gp.splits;
    gp.splits = (num_kb + gp.kb_per_split - 1) / gp.kb_per_split;  // no empty split
    // 3xTF32: the tensor core's fp32 accumulation error grows with the number of accumulated products, so the
    // accumulator is drained into C (round-to-nearest fp32 adds) every 512 k
    gp.kc = x3 ? 16 : (1 << 30);
    int cols = 32;
    while (cols < 2 * gp.bn) cols <<= 1;
    gp.tmem_cols = cols;
    gp.kb_per_fold = kfold > 1 ? (g.K + kBK - 1) / kBK : 0;
    const int pairs = kfold > 1 ? kfold : g.batch;  // extent of the operands' batch dimension
    gp.p_batched = (pairs > 1 && g.strideP != 0) ? 1 : 0;
    gp.q_batched = (pairs > 1 && g.strideQ != 0) ? 1 : 0;
    gp.C = g.C; gp.ldc = g.ldc; gp.strideC = g.strideC;
    gp.out_mode = g.out_mode;
    gp.accumulate = g.accumulate;
    gp.atomic_out = gp.splits > 1 ? 1 : 0;
    gp.bias_i = g.ep.bias_i; gp.bias_j = g.ep.bias_j; gp.relu = g.ep.relu;
    gp.status = ctx->d_status;

    // ---- tensor maps (innermost dimension first)
    CUtensorMap tp, tq;
    {
        const uint64_t nb = gp.p_batched ? (uint64_t)pairs : 1;
        const uint64_t bstride = gp.p_batched ? (uint64_t)g.strideP * 4 : (uint64_t)g.ldp * 4 * (g.p_mn ? g.K : g.I);
        int rc;
        gp.p_wide = (g.p_mn && (g.I & 31) == 0) ? 1 : 0;
        if (gp.p_wide) {
            // view the i extent as (32, I / 32): one box [slices of the tile][32 k][32 i] is the tile's MN-major layout
            uint64_t dims[4] = {32, (uint64_t)g.K, (uint64_t)g.I / 32, nb};
            uint64_t str[3] = {(uint64_t)g.ldp * 4, 128, bstride};
            uint32_t box[4] = {32, (uint32_t)kBK, (uint32_t)(4 * gp.mi), 1};
            rc = encode_tmap(ctx, &tp, g.P, 4, dims, str, box, nullptr, 129);
        } else {
            uint64_t dims[3], str[2];
            uint32_t box[3];
            if (g.p_mn) { dims[0] = g.I; dims[1] = g.K; box[0] = 32; box[1] = kBK; }
            else        { dims[0] = g.K; dims[1] = g.I; box[0] = kBK; box[1] = 128; }
            dims[2] = nb; box[2] = 1;
            str[0] = (uint64_t)g.ldp * 4; str[1] = bstride;
            rc = encode_tmap(ctx, &tp, g.P, 3, dims, str, box, nullptr, g.p_mn ? 129 : 128);
        }
        if (rc != CB_OK) return rc;
    }
    {
        const uint64_t nb = gp.q_batched ? (uint64_t)pairs : 1;
        const uint64_t bstride = gp.q_batched ? (uint64_t)g.strideQ * 4 : (uint64_t)g.ldq * 4 * (g.q_mn ? g.K : g.J);
        int rc;
        gp.q_wide = (g.q_mn && (g.J & 31) == 0) ? 1 : 0;
        if (gp.q_wide) {
            uint64_t dims[4] = {32, (uint64_t)g.K, (uint64_t)g.J / 32, nb};
            uint64_t str[3] = {(uint64_t)g.ldq * 4, 128, bstride};
            uint32_t box[4] = {32, (uint32_t)kBK, (uint32_t)(gp.bn >> 5), 1};
            rc = encode_tmap(ctx, &tq, g.Q, 4, dims, str, box, nullptr, 129);
        } else {
            uint64_t dims[3], str[2];
            uint32_t box[3];
            if (g.q_mn) { dims[0] = g.J; dims[1] = g.K; box[0] = 32; box[1] = kBK; }
            else        { dims[0] = g.K; dims[1] = g.J; box[0] = kBK; box[1] = (uint32_t)gp.bn; }
            dims[2] = nb; box[2] = 1;
            str[0] = (uint64_t)g.ldq * 4; str[1] = bstride;
            rc = encode_tmap(ctx, &tq, g.Q, 3, dims, str, box, nullptr, g.q_mn ? 129 : 128);
        }
        if (rc != CB_OK) return rc;
    }

    if (gp.atomic_out && !g.accumulate) {
        int rc = zero_output(ctx, g);
        if (rc != CB_OK) return rc;
    }

    const long long work = (long long)gp.batch * gp.tiles_i * gp.tiles_j * gp.splits;
    const int grid = (int)(work < ctx->sm_count ? work : ctx->sm_count);
    const int hi = gp.mi * kPTileBytes + gp.bn * kBK * 4;
    const size_t smem = (size_t)gp.stages * (x3 ? 2 * hi : hi) + 1024;
    cudaError_t e;
    if (g.p_mn && g.q_mn)       e = launch_variant<true, true>(ctx, x3, dim3(grid), smem, tp, tq, gp);
    else if (g.p_mn && !g.q_mn) e = launch_variant<true, false>(ctx, x3, dim3(grid), smem, tp, tq, gp);
    else if (!g.p_mn && g.q_mn) e = launch_variant<false, true>(ctx, x3, dim3(grid), smem, tp, tq, gp);
    else                        e = launch_variant<false, false>(ctx, x3, dim3(grid), smem, tp, tq, gp);
    if (e != cudaSuccess) return check_cuda(ctx, e, "umma_gemm_kernel launch");
    ctx->launches += 1;
    ctx->last_kernel = x3 ? "umma_3xtf32" : "umma_tf32";
    return CB_OK;
}

int launch_simt_gemm(cb_ctx* ctx, const GemmCall& g_in) {
    GemmCall g = g_in;
    if (g.J <= 16 && g.I > 16) {  // put the thin extent on the I side: D'[j][i] with the operands' roles swapped
        std::swap(g.I, g.J);
        std::swap(g.P, g.Q); std::swap(g.ldp, g.ldq); std::swap(g.strideP, g.strideQ); std::swap(g.p_mn, g.q_mn);
        std::swap(g.ep.bias_i, g.ep.bias_j);
        g.out_mode ^= 1;
    }
    if (g.I <= 16 && g.batch == 1 && g.J >= 32 && g.K >= 256) {
        SimtParams sp{};
        sp.I = g.I; sp.J = g.J; sp.K = g.K; sp.batch = 1;
        sp.P = g.P; sp.ldp = g.ldp; sp.p_mn = g.p_mn;
        sp.Q = g.Q; sp.ldq = g.ldq; sp.q_mn = g.q_mn;
        sp.C = g.C; sp.ldc = g.ldc; sp.out_mode = g.out_mode; sp.accumulate = g.accumulate;
        sp.bias_i = g.ep.bias_i; sp.bias_j = g.ep.bias_j; sp.relu = g.ep.relu;
        const int jblocks = (g.J + 7) / 8;
        int splits = 1;
        if (!ctx->deterministic && g.ep.relu == 0) {
            splits = (2 * ctx->sm_count + jblocks - 1) / jblocks;
            if (splits > g.K / 128) splits = g.K / 128;
            if (splits < 1) splits = 1;
        }
        int kps = (g.K + splits - 1) / splits;
        kps = ((kps + 31) / 32) * 32;
        splits = (g.K + kps - 1) / kps;
        sp.splits = splits; sp.k_per_split = kps;
        sp.atomic_out = splits > 1 ? 1 : 0;
        if (sp.atomic_out && !g.accumulate) {
            int rc = zero_output(ctx, g);
            if (rc != CB_OK) return rc;
        }
        skinny_gemm_kernel<<<dim3(jblocks, splits), 256, 0, ctx->stream>>>(sp);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return check_cuda(ctx, e, "skinny_gemm_kernel launch");
        ctx->launches += 1;
        ctx->last_kernel = "simt_fp32";
        return CB_OK;
    }
    SimtParams sp{};
    sp.I = g.I; sp.J = g.J; sp.K = g.K; sp.batch = g.batch;
    sp.P = g.P; sp.ldp = g.ldp; sp.strideP = g.strideP; sp.p_mn = g.p_mn;
    sp.Q = g.Q; sp.ldq = g.ldq; sp.strideQ = g.strideQ; sp.q_mn = g.q_mn;
    sp.C = g.C; sp.ldc = g.ldc; sp.strideC = g.strideC; sp.out_mode = g.out_mode;
    sp.accumulate = g.accumulate;
    sp.bias_i = g.ep.bias_i; sp.bias_j = g.ep.bias_j; sp.relu = g.ep.relu;
    const int ti = (g.I + 63) / 64, tj = (g.J + 63) / 64;
    long long tiles = (long long)ti * tj * g.batch;
    int splits = 1;
    if (!ctx->deterministic && g.ep.relu == 0 && tiles * 2 <= ctx->sm_count && g.K >= 512) {
        splits = (int)(2LL * ctx->sm_count / tiles);
        if (splits > g.K / 128) splits = g.K / 128;
        if (splits < 1) splits = 1;
    }
    int kps = (g.K + splits - 1) / splits;
    kps = ((kps + 15) / 16) * 16;
    splits = (g.K + kps - 1) / kps;
    sp.splits = splits; sp.k_per_split = kps;
    sp.atomic_out = splits > 1 ? 1 : 0;
    if ((long long)g.batch * splits > 65535) return fail(ctx, CB_EUNSUPPORTED, "simt gemm: batch*splits > 65535");
    if (sp.atomic_out && !g.accumulate) {
        int rc = zero_output(ctx, g);
        if (rc != CB_OK) return rc;
    }
    dim3 grid(ti, tj, g.batch * splits);
    simt_gemm_kernel<<<grid, 256, 0, ctx->stream>>>(sp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "simt_gemm_kernel launch");
    ctx->launches += 1;
    ctx->last_kernel = "simt_fp32";
    return CB_OK;
}

}  // namespace cb
