// Host-side internals shared by the C-ABI translation units: the context object, error helpers,
// tensor-map encoding (cuTensorMapEncodeTiled resolved at run time through the CUDA runtime, so the
// library does not link against libcuda) and the launch wrappers of each kernel family.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../../include/crusader_b200.h"

struct cb_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int math = CB_MATH_TF32;
    int sync = 0;
    int deterministic = 0;
    int* d_status = nullptr;       // device status word (0 = ok, CBK_* otherwise)
    void* workspace = nullptr;     // scratch: split-K partials, packed filters
    size_t workspace_bytes = 0;
    void* workspace2 = nullptr;    // scratch: re-laid-out activations / gradients of the stride-2 convolutions
    size_t workspace2_bytes = 0;
    void* workspace3 = nullptr;    // scratch: lo parts and partial results of the 3xTF32 convolutions
    size_t workspace3_bytes = 0;
    int workspace_frozen = 0;      // 1: a call that would need a larger scratch block fails instead of reallocating
    long long launches = 0;
    int sm_count = 148;
    int max_smem_optin = 0;
    std::string last_error;
    const char* last_kernel = "none";
    long long* trace = nullptr;    // device buffer for per-CTA time stamps (builds with -DCB_TRACE only)
    int filter_cache_on = 0;       // packed convolution filters are kept between calls (cb_conv_cache_filters)
    long long filter_version = 0;  // bumped by every call that may have changed a filter's values
    void* filter_cache = nullptr;  // the cache itself (conv_sm100.cu)
    int pdl = 1;                   // launch kernels that call griddep_wait with programmatic stream serialization
    void* wgrad_acc = nullptr;     // weight-gradient accumulator [column][row], all zero between calls (wgrad_sm100.cu)
    size_t wgrad_acc_bytes = 0;
    int wgrad_grid_cap = 0;        // > 0: most CTAs a weight-gradient kernel uses (contexts that run beside another stream)
    // Encoded tensor maps by (base pointer, extents, strides, box, swizzle): a training loop presents the same few
    // hundred (tensor, tiling) pairs every step, so the encode runs once per pair (encode_tmap, cb_abi.cu).
    std::unordered_map<std::string, CUtensorMap> tmap_cache;
    long long tmap_hits = 0, tmap_misses = 0;
};

namespace cb {

int fail(cb_ctx* ctx, int code, const std::string& msg);
int check_cuda(cb_ctx* ctx, cudaError_t e, const char* what);
// Text for a CBK_* code a kernel left in a status word.
const char* status_name(int s);
// Returns after an optional sync; maps a non-zero device status word to CB_ETIMEOUT.
int finish(cb_ctx* ctx, const char* what);
// Launches `kernel` on the context's stream; with ctx->pdl the launch carries the programmatic-stream-serialization
// attribute, so ONLY for kernels whose every thread calls griddep_wait() before its first access to global memory
// that an earlier kernel may have written or may still read.
template <typename... KArgs, typename... Args>
cudaError_t launch_dep_on(cudaStream_t stream, bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1u : 0u;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_dep(cb_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
    return launch_dep_on(ctx->stream, ctx->pdl != 0, kernel, grid, block, smem, std::forward<Args>(args)...);
}

// Raises cudaFuncAttributeMaxDynamicSharedMemorySize of `kernel` to the most this device allows (opt-in limit minus
// the kernel's static shared memory), once per (kernel, device) instead of on every launch; *max_dynamic receives that
// bound. Thread-safe.
cudaError_t raise_dynamic_smem_once(const void* kernel, int device, int smem_optin, int* max_dynamic);
template <typename... KArgs>
cudaError_t raise_dynamic_smem_once(void (*kernel)(KArgs...), int device, int smem_optin, int* max_dynamic) {
    return raise_dynamic_smem_once(reinterpret_cast<const void*>(kernel), device, smem_optin, max_dynamic);
}

// CB_OK when ctx is non-null and its device is the current one.
int enter(cb_ctx* ctx);
// Grows one of the context's scratch blocks to at least `bytes`; growth waits for the whole device before the old
// block is freed, and is refused (CB_ENOMEM) while the workspace is frozen or the stream is being captured.
int ensure_workspace(cb_ctx* ctx, size_t bytes);
int ensure_workspace2(cb_ctx* ctx, size_t bytes);
int ensure_workspace3(cb_ctx* ctx, size_t bytes);
// The zero-filled accumulator of the weight-gradient kernels, at least `bytes` large (same growth rules).
int ensure_wgrad_acc(cb_ctx* ctx, size_t bytes);

// Encodes a tiled fp32 tensor map. dims/box are innermost-first; strides_bytes has rank-1 entries
// (the innermost stride is 4 bytes). swizzle_bytes in {0, 32, 64, 128}, or 129 for
// the 128-byte swizzle with 32-byte atoms. elem_strides may be null (all 1).
int encode_tmap(cb_ctx* ctx, CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, const uint32_t* elem_strides,
                int swizzle_bytes);

// Fused per-element tail applied while the accumulator is written out.
struct Epilogue {
    const float* bias_i = nullptr;  // added per UMMA-M index (null = none)
    const float* bias_j = nullptr;  // added per UMMA-N index (null = none)
    int relu = 0;
};

// D[i][j] = sum_k P[i][k] * Q[j][k]; i < I tiles of 128 (UMMA M), j < J (UMMA N).
// p_mn / q_mn: operand stored with the i / j index contiguous (MN-major) instead of k (K-major).
// out_mode 0: C[j*ldc + i]; out_mode 1: C[i*ldc + j].
struct GemmCall {
    int I = 0, J = 0, K = 0, batch = 1;
    const float* P = nullptr; long long ldp = 0, strideP = 0; int p_mn = 0;
    const float* Q = nullptr; long long ldq = 0, strideQ = 0; int q_mn = 0;
    float* C = nullptr; long long ldc = 0, strideC = 0; int out_mode = 0;
    int accumulate = 0;
    Epilogue ep;
    int kfold = 1;  // > 1 (with batch == 1): C (+)= sum over kfold operand pairs, strideP / strideQ apart, of P Q^T
};
// Per-element tail of a convolution, applied in this order while the accumulator is written out:
// y = conv; y = y * scale + shift (if scale); y += bias[oc] (if bias); y += out (if accumulate); y = max(y, 0) (if relu).
struct ConvEpilogue {
    const float* bias = nullptr;
    const float* scale = nullptr;   // with shift: Cout values, or Cout*H*W values when per_position
    const float* shift = nullptr;
    int per_position = 0;
    int relu = 0;
    int accumulate = 0;
};
// Tensor-core convolution paths. Each returns CB_EUNSUPPORTED, before any work is queued, when the geometry is outside
// what it covers. in/out batch strides: elements between consecutive images, 0 = densely packed.
int umma_conv_fwd(cb_ctx* ctx, const float* W, const float* X, float* Y, const ConvEpilogue& ep, int N, int IC, int IH,
                  int IW, int OC, int FH, int FW, int sH, int sW, int pH, int pW, bool dgrad_of, long long in_batch,
                  long long out_batch);
// 3xTF32 forward / data gradient in one tensor-core pass (stride 1; conv_sm100.cu), else CB_EUNSUPPORTED.
int umma_conv_fwd_x3(cb_ctx* ctx, const float* W, const float* X, float* Y, const ConvEpilogue& ep, int N, int IC, int IH,
                     int IW, int OC, int FH, int FW, int pH, int pW, bool dgrad_of, long long in_batch, long long out_batch);
// x3: 3xTF32 in one launch (the kernel walks (lo of X, dY), (X, lo of dY), (X, dY) into one accumulator).
int umma_conv_wgrad(cb_ctx* ctx, const float* dY, const float* X, float* dW, int N, int IC, int IH, int IW, int OC,
                    int FH, int FW, int sH, int sW, int pH, int pW, int accumulate, long long dy_batch, long long x_batch,
                    bool x3 = false);
// Packed-filter cache of a context (conv_sm100.cu).
int filter_cache_repack_all(cb_ctx* ctx);
void filter_cache_destroy(cb_ctx* ctx);

bool umma_gemm_eligible(const GemmCall& g);
int launch_umma_gemm(cb_ctx* ctx, const GemmCall& g, bool x3);
int launch_simt_gemm(cb_ctx* ctx, const GemmCall& g);

// BatchNorm on one group of samples of a batch (statistics per group; neighbours.cu).
int bn_fwd_group(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, const float* R, float* Y, int relu, int N,
                 long long P);
int bn_bwd_group(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, float* dgamma, float* dbeta,
                 const float* relu_out, float* dR, int accumulate_dR, int add_param_grads, int N, long long P);

// One operand of a parsed .crseq file (crseq.cu): its id, the words of its info record, and for convolutions the sizes
// of its parameter blobs (filter, bias). Branch operands of a ShortcutEndpoint follow their endpoint with in_branch set.
struct CrseqOperand {
    uint32_t id = 0;
    uint32_t info[9] = {};
    uint64_t param_floats[2] = {};
    int in_branch = 0;
};
struct CrseqModel {
    uint32_t epoch = 0;
    std::vector<CrseqOperand> operands;
    size_t params_begin = 0, param_bytes = 0;
};
bool crseq_parse(const std::vector<uint8_t>& file, CrseqModel& out, std::string& err);

// Momentum descriptor table resident on the device (see neighbours.cu).
int momentum_table_build(cb_ctx* ctx, int ntensors, float* const* w, float* const* g, float* const* m,
                         const long long* sizes, const unsigned char* is_weight, void** dev_table, long long* biggest);
int momentum_table_launch(cb_ctx* ctx, const void* dev_table, int ntensors, long long biggest, float lr, float beta,
                          float l2);

}  // namespace cb
