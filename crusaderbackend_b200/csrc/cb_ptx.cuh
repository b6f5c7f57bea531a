// Inline-PTX building blocks for the sm_100a kernels: mbarrier, TMA (cp.async.bulk.tensor),
// tcgen05 (TMEM allocation, UMMA issue/commit, TMEM loads) and the UMMA descriptors.
//
// Conventions used throughout:
//  * every wait on an mbarrier is bounded (mbar_wait): after CB_WAIT_LIMIT_NS of polling the
//    waiter raises the CTA-wide abort flag, records a status code in global memory and returns
//    false; callers leave their loops; the producer then waits (bounded, mbar_drain) for the copies it
//    armed, the MMA issuer commits and waits for the MMAs it issued, and only then is TMEM freed.
//  * shared-memory addresses handed to PTX are 32-bit shared::cta window addresses.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef CB_WAIT_LIMIT_NS
#define CB_WAIT_LIMIT_NS 2000000000ull
#endif

// Development aid, compiled out unless the library is built with -DCB_TRACE: per-CTA time stamps (SM clock) of the
// pipeline roles' milestones, 16 slots per CTA, written to a buffer the caller hands in through cb_debug_set_trace.
#ifdef CB_TRACE
#define CB_TRACE_EVENT(buf, slot)                                                      \
    do {                                                                               \
        if (buf) (buf)[(long long)blockIdx.x * 16 + (slot)] = (long long)clock64();    \
    } while (0)
#define CB_TRACE_WALL(buf, slot)                                                       \
    do {                                                                               \
        if (buf) (buf)[(long long)blockIdx.x * 16 + (slot)] = (long long)cb::globaltimer_ns(); \
    } while (0)
#else
#define CB_TRACE_EVENT(buf, slot) do {} while (0)
#define CB_TRACE_WALL(buf, slot) do {} while (0)
#endif

namespace cb {

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// Status codes a kernel may leave in the context's device status word.
enum : int {
    CBK_OK = 0,
    CBK_TIMEOUT_EMPTY = 101,      // producer waited for a free pipeline stage
    CBK_TIMEOUT_FULL = 102,       // MMA issuer waited for operands
    CBK_TIMEOUT_XFORM = 103,      // MMA issuer waited for the split (lo) stage
    CBK_TIMEOUT_TMEM_EMPTY = 104, // MMA issuer waited for the epilogue to drain an accumulator
    CBK_TIMEOUT_TMEM_FULL = 105,  // epilogue waited for an accumulator
    CBK_TIMEOUT_XFORM_FULL = 106, // split warps waited for operands
    CBK_TIMEOUT_DRAIN = 107       // drain of in-flight copies after an abort
};

// Bounded wait: gives up after CB_WAIT_LIMIT_NS of wall time (or when another role raised the abort
// flag). Returns true when the phase completed, false on abort/timeout.
// Programmatic dependent launch. A kernel launched with the programmatic-serialization attribute may start while
// the kernel before it on the stream is still running: griddep_wait returns once that kernel has completed and its
// writes are visible (immediately for a kernel launched without the attribute), so everything before it must touch
// no global memory another kernel produces; griddep_launch lets the kernel after this one begin the same way.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ bool mbar_wait_for(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                              int code, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > limit_ns) break;
        }
    }
    *abort_flag = 1;
    atomicCAS(status, 0, code);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
    return mbar_wait_for(bar, parity, abort_flag, status, code, CB_WAIT_LIMIT_NS);
}

// Whole-warp wait for the roles that wait long and in numbers (epilogue warps waiting for a tile's accumulator, the
// transform warps waiting for a stage): only lane 0 polls, and with max_sleep_ns != 0 it sleeps between polls (32 ns,
// doubling up to max_sleep_ns), so that hundreds of waiting threads do not take issue slots from the one thread that
// feeds the tensor core; the other lanes then read the completed phase themselves. Sleeping pays in the GEMM's long
// main loops (+1..6 %); the convolution kernels' short ones lose to the wake-up latency and keep mbar_wait.
// Same bound and abort behaviour as mbar_wait.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int lane, volatile int* abort_flag,
                                               int* status, int code, uint32_t max_sleep_ns) {
    int ok = 1;
    if (lane == 0 && !mbar_try_wait(bar, parity)) {
        const uint64_t t0 = globaltimer_ns();
        uint32_t ns = 32;
        for (;;) {
            if (max_sleep_ns) {
                __nanosleep(ns);
                if (ns < max_sleep_ns) ns <<= 1;
            }
            if (mbar_try_wait(bar, parity)) break;
            if (*abort_flag) { ok = 0; break; }
            if (globaltimer_ns() - t0 > CB_WAIT_LIMIT_NS) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                ok = 0;
                break;
            }
        }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (ok)
        for (int i = 0; i < 1024 && !mbar_try_wait(bar, parity); ++i) {}
    return ok != 0;
}

// After an abort: gives work that is still in flight a bounded chance to land before the CTA releases what it targets.
// Waits (at most ~1 ms) for the given phase of `bar`; records CBK_TIMEOUT_DRAIN when it does not complete.
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity, int* status) {
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return;
        if ((it & 63u) == 63u && globaltimer_ns() - t0 > 1000000ull) break;
    }
    atomicCAS(status, 0, 107 /* CBK_TIMEOUT_DRAIN */);
}

// generic-proxy writes (st.shared) -> visible to the async proxy (TMA / tcgen05 operand reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- TMA tile loads (issued per CTA)
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1,
                                            int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
        "[%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// ---------------------------------------------------------------- TMA tile stores (shared -> global, bulk-group completion)
// One thread. The box described by `tm` is read from dense shared memory at `src` and written (or added, for the
// reduce form) at the given coordinates; parts of the box outside the tensor's extents are dropped. The innermost
// coordinate must be a multiple of 4 floats and no coordinate may be negative.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tm, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tm)),
                 "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* tm, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tm)),
                 "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's committed store groups are still READING their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Waits until at most N of this thread's committed store groups are still incomplete.
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
// Whole-warp, convergent. Writes the TMEM base address to *dst_smem.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// One thread. Arrives once on `bar` when every tcgen05.mma issued earlier by this thread retired.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
// Whole warp, converged: the lane umma_tf32_elect elects (the same one every time for the full mask) arrives once on
// `bar` when every tcgen05.mma it issued earlier retired.
__device__ __forceinline__ void tc_commit_elect(uint32_t bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n" ::"r"(bar)
        : "memory");
}
// One thread. D[tmem] (+)= A[smem desc] * B[smem desc], kind::tf32, fp32 accumulate.
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Whole warp, converged, every lane with the same arguments: one elected lane issues the UMMA. Keeping the issuing loop
// warp-uniform lets the compiler hold the descriptors in uniform registers; in a one-lane branch a descriptor that
// changes from one UMMA to the next costs ~110 cycles of issue each (measured with the UMMA-only loop of peak_sm100.cu).
__device__ __forceinline__ void umma_tf32_elect(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// kElect: called by the whole converged warp (elected lane issues); otherwise by the one issuing thread.
template <bool kElect>
__device__ __forceinline__ void umma_tf32_sel(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
    if (kElect) umma_tf32_elect(d_tmem, desc_a, desc_b, idesc, accumulate);
    else umma_tf32(d_tmem, desc_a, desc_b, idesc, accumulate);
}
template <bool kElect>
__device__ __forceinline__ void tc_commit_sel(uint32_t bar) {
    if (kElect) tc_commit_elect(bar);
    else tc_commit(bar);
}
// Whole-warp: 32 lanes x 16 consecutive fp32 columns starting at taddr (lane field = warp's quarter).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
        "%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// Whole-warp: 32 lanes x 8 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
// Whole-warp: 32 lanes x 32 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- UMMA descriptors
// Shared-memory matrix descriptor (64 bit): start address, leading/stride byte offsets in 16-byte
// units, descriptor version 1, swizzle mode in bits [61,64).
// UMMA_SW_128B_BASE32B (32-byte chunks swizzled inside a 128-byte row, 4-row period) is the only layout the
// tensor core accepts for MN-major 32-bit (tf32) operands; K-major tf32 operands use UMMA_SW_128B.
enum : uint32_t { UMMA_SW_NONE = 0, UMMA_SW_128B_BASE32B = 1, UMMA_SW_128B = 2, UMMA_SW_64B = 4, UMMA_SW_32B = 6 };

__host__ __device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes, uint32_t swizzle) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;  // descriptor version (Blackwell)
    d |= static_cast<uint64_t>(swizzle & 7u) << 61;
    return d;
}

// Instruction descriptor for kind::tf32 with fp32 accumulation.
// a_mn / b_mn: 0 = operand is K-major in shared memory, 1 = MN-major.
__host__ __device__ __forceinline__ uint32_t umma_idesc_tf32(uint32_t m, uint32_t n, uint32_t a_mn,
                                                             uint32_t b_mn) {
    uint32_t d = 0;
    d |= 1u << 4;   // D format: F32
    d |= 2u << 7;   // A format: TF32
    d |= 2u << 10;  // B format: TF32
    d |= (a_mn & 1u) << 15;
    d |= (b_mn & 1u) << 16;
    d |= ((n >> 3) & 0x3Fu) << 17;
    d |= ((m >> 4) & 0x1Fu) << 24;
    return d;
}

}  // namespace cb
