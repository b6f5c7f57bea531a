// C-ABI entry points: context management, error reporting and the GEMM dispatcher.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <cstring>
#include <new>

#include "cb_internal.h"
#include "cb_ptx.cuh"

namespace cb {

int fail(cb_ctx* ctx, int code, const std::string& msg) {
    if (ctx) ctx->last_error = msg;
    return code;
}

int check_cuda(cb_ctx* ctx, cudaError_t e, const char* what) {
    if (e == cudaSuccess) return CB_OK;
    return fail(ctx, CB_ECUDA, std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
}

const char* status_name(int s) {
    switch (s) {
        case CBK_TIMEOUT_EMPTY: return "producer timed out waiting for a free stage";
        case CBK_TIMEOUT_FULL: return "MMA issuer timed out waiting for operands";
        case CBK_TIMEOUT_XFORM: return "MMA issuer timed out waiting for the split stage";
        case CBK_TIMEOUT_TMEM_EMPTY: return "MMA issuer timed out waiting for a drained accumulator";
        case CBK_TIMEOUT_TMEM_FULL: return "epilogue timed out waiting for an accumulator";
        case CBK_TIMEOUT_XFORM_FULL: return "split warps timed out waiting for operands";
        case CBK_TIMEOUT_DRAIN: return "drain after abort timed out";
        default: return "unknown device status";
    }
}

static int read_status(cb_ctx* ctx, const char* what) {
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return check_cuda(ctx, e, what);
    int st = 0;
    e = cudaMemcpy(&st, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return check_cuda(ctx, e, "status readback");
    if (st != 0) {
        cudaMemset(ctx->d_status, 0, sizeof(int));
        char buf[160];
        snprintf(buf, sizeof(buf), "%s: device status %d (%s)", what, st, status_name(st));
        return fail(ctx, CB_ETIMEOUT, buf);
    }
    return CB_OK;
}

int finish(cb_ctx* ctx, const char* what) {
    if (!ctx->sync) return CB_OK;
    return read_status(ctx, what);
}

// Growth of one of the three scratch blocks. The old block is released only after the whole device is idle (work queued
// on a stream the context used earlier may still read it), and never while the workspace is frozen or the stream is
// being captured: a captured graph keeps the addresses of the blocks it was recorded with, so a later free would leave
// it reading released memory.
static int grow_block(cb_ctx* ctx, void** block, size_t* have, size_t bytes, size_t slack) {
    if (bytes <= *have) return CB_OK;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(ctx->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
        return fail(ctx, CB_ENOMEM, "workspace growth requested while the stream is being captured: run the same calls once "
                                    "before the capture so that the scratch is already large enough");
    if (ctx->workspace_frozen)
        return fail(ctx, CB_ENOMEM, "workspace is frozen (cb_freeze_workspace) and this call needs a larger scratch block");
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return check_cuda(ctx, e, "workspace growth sync");
    if (*block) cudaFree(*block);
    *block = nullptr;
    *have = 0;
    size_t want = (bytes + slack + 255) & ~size_t(255);
    e = cudaMalloc(block, want);
    if (e != cudaSuccess) {
        check_cuda(ctx, e, "workspace cudaMalloc");
        return CB_ENOMEM;
    }
    *have = want;
    return CB_OK;
}

int ensure_workspace(cb_ctx* ctx, size_t bytes) { return grow_block(ctx, &ctx->workspace, &ctx->workspace_bytes, bytes, bytes >> 2); }
int ensure_workspace2(cb_ctx* ctx, size_t bytes) { return grow_block(ctx, &ctx->workspace2, &ctx->workspace2_bytes, bytes, 0); }
int ensure_workspace3(cb_ctx* ctx, size_t bytes) { return grow_block(ctx, &ctx->workspace3, &ctx->workspace3_bytes, bytes, 0); }

int ensure_wgrad_acc(cb_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->wgrad_acc_bytes) return CB_OK;
    int rc = grow_block(ctx, &ctx->wgrad_acc, &ctx->wgrad_acc_bytes, bytes, bytes);
    if (rc != CB_OK) return rc;
    // kept all zero from here on: every call that adds into it also clears what it read
    cudaError_t e = cudaMemset(ctx->wgrad_acc, 0, ctx->wgrad_acc_bytes);
    if (e != cudaSuccess) return check_cuda(ctx, e, "weight-gradient accumulator clear");
    return CB_OK;
}

// Entry check of every context call: the context must exist and its device must be the current one (launches go to the
// current device; scratch and tensor maps belong to the context's).
int enter(cb_ctx* ctx) {
    if (!ctx) return CB_EINVAL;
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess) return fail(ctx, CB_ECUDA, "cudaGetDevice failed");
    if (cur != ctx->device) {
        char buf[128];
        snprintf(buf, sizeof(buf), "this context was created on device %d but device %d is current", ctx->device, cur);
        return fail(ctx, CB_EINVAL, buf);
    }
    return CB_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn resolve_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int encode_tmap(cb_ctx* ctx, CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, const uint32_t* elem_strides,
                int swizzle_bytes) {
    EncodeTiledFn fn = resolve_encode();
    if (!fn) return fail(ctx, CB_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if (rank < 1 || rank > 5) return fail(ctx, CB_EINVAL, "tensor map rank outside 1..5");
    cuuint64_t gd[5] = {};
    cuuint64_t gs[4] = {};
    cuuint32_t bd[5] = {}, es[5] = {};
    for (int i = 0; i < rank; ++i) {
        gd[i] = dims[i];
        bd[i] = box[i];
        es[i] = elem_strides ? elem_strides[i] : 1;
    }
    for (int i = 0; i + 1 < rank; ++i) gs[i] = strides_bytes[i];
    // The encoding is a pure function of these values: a context keeps what it has encoded (bounded: a caller that
    // walks through ever new addresses starts over at 4096 entries).
    struct Key {
        const void* base;
        cuuint64_t gd[5], gs[4];
        cuuint32_t bd[5], es[5];
        int rank, swizzle;
    } key{};  // value-initialised: padding bytes are zero, the bytes are the hash key
    std::string kbytes;
    if (ctx) {
        key.base = base; key.rank = rank; key.swizzle = swizzle_bytes;
        for (int i = 0; i < 5; ++i) { key.gd[i] = gd[i]; key.bd[i] = bd[i]; key.es[i] = es[i]; }
        for (int i = 0; i < 4; ++i) key.gs[i] = gs[i];
        kbytes.assign(reinterpret_cast<const char*>(&key), sizeof(key));
        auto it = ctx->tmap_cache.find(kbytes);
        if (it != ctx->tmap_cache.end()) {
            *out = it->second;
            ++ctx->tmap_hits;
            return CB_OK;
        }
    }
    CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
    if (swizzle_bytes == 32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
    else if (swizzle_bytes == 64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
    else if (swizzle_bytes == 128) sw = CU_TENSOR_MAP_SWIZZLE_128B;
    else if (swizzle_bytes == 129) sw = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void*>(base), gd, gs, bd, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[256];
        snprintf(buf, sizeof(buf),
                 "cuTensorMapEncodeTiled failed (CUresult %d): rank %d dims [%llu %llu %llu %llu] box [%u %u %u %u]",
                 (int)r, rank, (unsigned long long)gd[0], (unsigned long long)(rank > 1 ? gd[1] : 0),
                 (unsigned long long)(rank > 2 ? gd[2] : 0), (unsigned long long)(rank > 3 ? gd[3] : 0), bd[0],
                 rank > 1 ? bd[1] : 0, rank > 2 ? bd[2] : 0, rank > 3 ? bd[3] : 0);
        return fail(ctx, CB_ECUDA, buf);
    }
    if (ctx) {
        if (ctx->tmap_cache.size() >= 4096) ctx->tmap_cache.clear();
        ctx->tmap_cache.emplace(std::move(kbytes), *out);
        ++ctx->tmap_misses;
    }
    return CB_OK;
}

}  // namespace cb

using namespace cb;

namespace cb {
cudaError_t raise_dynamic_smem_once(const void* kernel, int device, int smem_optin, int* max_dynamic) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, int> done;
    std::lock_guard<std::mutex> lock(mu);
    auto it = done.find({kernel, device});
    if (it == done.end()) {
        cudaFuncAttributes fa;
        cudaError_t e = cudaFuncGetAttributes(&fa, kernel);
        if (e != cudaSuccess) return e;
        const int bound = smem_optin - (int)fa.sharedSizeBytes;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bound);
        if (e != cudaSuccess) return e;
        it = done.emplace(std::make_pair(kernel, device), bound).first;
    }
    if (max_dynamic) *max_dynamic = it->second;
    return cudaSuccess;
}
}  // namespace cb

extern "C" {

const char* cb_version(void) { return "crusader_b200 0.1 (sm_100a)"; }

int cb_create(cb_ctx** out, int device, void* cuda_stream) {
    if (!out) return CB_EINVAL;
    *out = nullptr;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) return CB_ECUDA;
    if (device < 0 || device >= ndev) return CB_EINVAL;
    if (cudaSetDevice(device) != cudaSuccess) return CB_ECUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return CB_ECUDA;
    if (prop.major != 10) {
        fprintf(stderr, "crusader_b200: device %d is sm_%d%d; this library only carries sm_100a code\n", device,
                prop.major, prop.minor);
        return CB_EUNSUPPORTED;
    }
    cb_ctx* ctx = new (std::nothrow) cb_ctx();
    if (!ctx) return CB_ENOMEM;
    ctx->device = device;
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    ctx->sm_count = prop.multiProcessorCount;
    ctx->max_smem_optin = (int)prop.sharedMemPerBlockOptin;
    if (const char* e = std::getenv("CB_PDL")) ctx->pdl = std::atoi(e) != 0;  // development switch, default on
    if (cudaMalloc(&ctx->d_status, sizeof(int)) != cudaSuccess || cudaMemset(ctx->d_status, 0, sizeof(int)) != cudaSuccess) {
        delete ctx;
        return CB_ENOMEM;
    }
    *out = ctx;
    return CB_OK;
}

int cb_destroy(cb_ctx* ctx) {
    if (!ctx) return CB_EINVAL;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->workspace) cudaFree(ctx->workspace);
    if (ctx->workspace2) cudaFree(ctx->workspace2);
    if (ctx->workspace3) cudaFree(ctx->workspace3);
    if (ctx->wgrad_acc) cudaFree(ctx->wgrad_acc);
    if (ctx->d_status) cudaFree(ctx->d_status);
    filter_cache_destroy(ctx);
    delete ctx;
    return CB_OK;
}

int cb_set_stream(cb_ctx* ctx, void* cuda_stream) {
    if (!ctx) return CB_EINVAL;
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    return CB_OK;
}

int cb_set_math(cb_ctx* ctx, int mode) {
    if (!ctx) return CB_EINVAL;
    if (mode != CB_MATH_TF32 && mode != CB_MATH_3XTF32 && mode != CB_MATH_FP32)
        return fail(ctx, CB_EINVAL, "cb_set_math: unknown mode");
    ctx->math = mode;
    return CB_OK;
}

int cb_get_math(const cb_ctx* ctx) { return ctx ? ctx->math : CB_EINVAL; }

int cb_set_sync(cb_ctx* ctx, int on) {
    if (!ctx) return CB_EINVAL;
    ctx->sync = on ? 1 : 0;
    return CB_OK;
}

int cb_freeze_workspace(cb_ctx* ctx, int on) {
    if (!ctx) return CB_EINVAL;
    ctx->workspace_frozen = on ? 1 : 0;
    return CB_OK;
}

int cb_set_deterministic(cb_ctx* ctx, int on) {
    if (!ctx) return CB_EINVAL;
    ctx->deterministic = on ? 1 : 0;
    return CB_OK;
}

int cb_synchronize(cb_ctx* ctx) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    return read_status(ctx, "cb_synchronize");
}

// Development aid: how often this context reused / had to make an encoded tensor map.
int cb_debug_tmap_stats(cb_ctx* ctx, long long* hits, long long* misses) {
    if (!ctx) return CB_EINVAL;
    if (hits) *hits = ctx->tmap_hits;
    if (misses) *misses = ctx->tmap_misses;
    return CB_OK;
}

#ifdef CB_TRACE
// Development builds only: the next tensor-core convolution kernels write 16 time stamps per CTA into `buf`, and the
// forward / data-gradient kernel four more words per CTA (issuer wait and issue sums) behind the first 1024 x 16:
// `buf` holds at least 1024 * 20 words.
int cb_debug_set_trace(cb_ctx* ctx, long long* buf) {
    if (!ctx) return CB_EINVAL;
    ctx->trace = buf;
    return CB_OK;
}
#endif

namespace {
// Waits on a barrier that nothing ever arrives at, with a limit of limit_ns: the bounded wait gives up, records its
// status and the kernel returns normally.
__global__ void wait_timeout_kernel(int* status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait_for(smem_u32(&bar), 0, &abort_flag, status, CBK_TIMEOUT_FULL, limit_ns);
}
}  // namespace

int cb_selftest_wait_timeout(cb_ctx* ctx, int limit_ms) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (limit_ms < 1 || limit_ms > 1000) return fail(ctx, CB_EINVAL, "cb_selftest_wait_timeout: limit must be 1..1000 ms");
    wait_timeout_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_status, (unsigned long long)limit_ms * 1000000ull);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, "cb_selftest_wait_timeout");
    ctx->launches += 1;
    return finish(ctx, "cb_selftest_wait_timeout");
}

const char* cb_last_error(const cb_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }
long long cb_launch_count(const cb_ctx* ctx) { return ctx ? ctx->launches : 0; }
const char* cb_last_kernel(const cb_ctx* ctx) { return ctx ? ctx->last_kernel : "none"; }

int cb_gemm(cb_ctx* ctx, int transA, int transB, int M, int N, int K, const float* A, int lda, const float* B,
            int ldb, float* C, int ldc, int batch, long long strideA, long long strideB, long long strideC,
            int accumulate) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (M < 0 || N < 0 || K < 0 || batch < 0) return fail(ctx, CB_EINVAL, "cb_gemm: negative extent");
    if (M == 0 || N == 0 || batch == 0) return CB_OK;
    if (!A || !B || !C) return fail(ctx, CB_EINVAL, "cb_gemm: null operand");
    if (lda < (transA ? M : K) || ldb < (transB ? K : N) || ldc < N)
        return fail(ctx, CB_EINVAL, "cb_gemm: leading dimension smaller than the row length");
    if (K == 0) {
        if (!accumulate) {
            for (int b = 0; b < batch; ++b) {
                cudaError_t e = cudaMemset2DAsync(C + (long long)b * strideC, (size_t)ldc * 4, 0, (size_t)N * 4, M,
                                                  ctx->stream);
                if (e != cudaSuccess) return check_cuda(ctx, e, "cb_gemm: clear of C for K == 0");
            }
        }
        return finish(ctx, "cb_gemm");
    }
    GemmCall g;
    g.I = N; g.J = M; g.K = K; g.batch = batch;
    g.P = B; g.ldp = ldb; g.strideP = strideB; g.p_mn = transB ? 0 : 1;
    g.Q = A; g.ldq = lda; g.strideQ = strideA; g.q_mn = transA ? 1 : 0;
    g.C = C; g.ldc = ldc; g.strideC = strideC; g.out_mode = 0;
    g.accumulate = accumulate ? 1 : 0;
    int rc;
    if (ctx->math != CB_MATH_FP32 && umma_gemm_eligible(g))
        rc = launch_umma_gemm(ctx, g, ctx->math == CB_MATH_3XTF32);
    else
        rc = launch_simt_gemm(ctx, g);
    if (rc != CB_OK) return rc;
    return finish(ctx, "cb_gemm");
}

// C (+)= sum over `count` operand pairs of op(A[b]) * op(B[b]): the batch is folded into the contraction, one launch on
// the tensor-core path (the k-blocks walk the pairs); the CUDA-core fp32 path adds the pairs one after the other.
int cb_gemm_batch_reduce(cb_ctx* ctx, int transA, int transB, int M, int N, int K, const float* A, int lda, const float* B,
                         int ldb, float* C, int ldc, int count, long long strideA, long long strideB, int accumulate) {
    if (int rc_enter = enter(ctx)) return rc_enter;
    if (M < 0 || N < 0 || K < 0 || count < 0) return fail(ctx, CB_EINVAL, "cb_gemm_batch_reduce: negative extent");
    if (M == 0 || N == 0) return CB_OK;
    if (!A || !B || !C) return fail(ctx, CB_EINVAL, "cb_gemm_batch_reduce: null operand");
    if (lda < (transA ? M : K) || ldb < (transB ? K : N) || ldc < N)
        return fail(ctx, CB_EINVAL, "cb_gemm_batch_reduce: leading dimension smaller than the row length");
    if (K == 0 || count == 0) {
        if (!accumulate) {
            cudaError_t e = cudaMemset2DAsync(C, (size_t)ldc * 4, 0, (size_t)N * 4, M, ctx->stream);
            if (e != cudaSuccess) return check_cuda(ctx, e, "cb_gemm_batch_reduce: clear of C");
        }
        return finish(ctx, "cb_gemm_batch_reduce");
    }
    GemmCall g;
    g.I = N; g.J = M; g.K = K; g.batch = 1;
    g.P = B; g.ldp = ldb; g.strideP = strideB; g.p_mn = transB ? 0 : 1;
    g.Q = A; g.ldq = lda; g.strideQ = strideA; g.q_mn = transA ? 1 : 0;
    g.C = C; g.ldc = ldc; g.strideC = 0; g.out_mode = 0;
    g.accumulate = accumulate ? 1 : 0;
    g.kfold = count;
    int rc = CB_OK;
    if (ctx->math != CB_MATH_FP32 && umma_gemm_eligible(g)) {
        rc = launch_umma_gemm(ctx, g, ctx->math == CB_MATH_3XTF32);
    } else {
        g.kfold = 1;
        for (int b = 0; b < count && rc == CB_OK; ++b) {
            g.P = B + (long long)b * strideB;
            g.Q = A + (long long)b * strideA;
            g.accumulate = (accumulate || b > 0) ? 1 : 0;
            rc = launch_simt_gemm(ctx, g);
        }
    }
    if (rc != CB_OK) return rc;
    return finish(ctx, "cb_gemm_batch_reduce");
}

}  // extern "C"
