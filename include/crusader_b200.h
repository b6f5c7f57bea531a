/*
 * crusader_b200 — C ABI of the B200 (sm_100a) dense-contraction library.
 *
 * Every entry point takes raw DEVICE pointers (fp32, row-major matrices / NCHW feature maps, the
 * layout of the reference's seblas::Tensor, seblas/tensor/Tensor.cuh:48-99) plus plain integers.
 * Calls are asynchronous on the context's stream unless cb_set_sync(ctx, 1) was requested, in which
 * case each call returns only after the device finished it (the reference's convention: every
 * seblas operation ends in cudaDeviceSynchronize, seblas/operations/cuGEMM.cu:1657-1663).
 *
 * Return value: CB_OK or a negative CB_E* code; cb_last_error() describes the last failure.
 * The caller owns every tensor. A context owns a small device status word and a scratch workspace.
 * A context is used by one host thread at a time; create one per GPU. cb_create makes its device current and leaves
 * it current; every later call on the context requires that device to be the current one (CB_EINVAL otherwise).
 */
#ifndef CRUSADER_B200_H
#define CRUSADER_B200_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cb_ctx cb_ctx;

enum {
    CB_OK = 0,
    CB_EINVAL = -1,       /* bad shape, null pointer, misaligned operand */
    CB_ECUDA = -2,        /* CUDA runtime / driver error, see cb_last_error */
    CB_ETIMEOUT = -3,     /* a bounded device-side wait expired; the status word names which */
    CB_EUNSUPPORTED = -4, /* valid request this build has no kernel for */
    CB_ENOMEM = -5
};

enum {
    CB_MATH_TF32 = 0,   /* operands truncated to TF32 by the tensor core, fp32 accumulate */
    CB_MATH_3XTF32 = 1, /* hi/lo split, three tensor-core products per term: fp32-class accuracy */
    CB_MATH_FP32 = 2    /* CUDA-core fp32 FMA kernels (exact fp32; used for shapes TMA cannot address) */
};

/* ---- context ------------------------------------------------------------------------------- */

/* Creates a context on `device`. `cuda_stream` is a cudaStream_t (NULL = legacy default stream, the
 * stream every reference seblas kernel is launched on). */
int cb_create(cb_ctx** out, int device, void* cuda_stream);
int cb_destroy(cb_ctx* ctx);
int cb_set_stream(cb_ctx* ctx, void* cuda_stream);
int cb_set_math(cb_ctx* ctx, int mode);
int cb_get_math(const cb_ctx* ctx);
/* 1: synchronise after every call and surface device-side status (reference-compatible). 0: async. */
int cb_set_sync(cb_ctx* ctx, int sync_every_call);
/* 1: from now on a call that would need a larger scratch block than the context holds fails with CB_ENOMEM instead of
 * reallocating. A CUDA graph captured over cb_* calls keeps the addresses of the scratch blocks it was recorded with:
 * freeze the workspace after the warm-up calls and before (or right after) the capture, and keep it frozen for as long
 * as the graph is replayed. Growth is also refused while the context's stream is being captured. */
int cb_freeze_workspace(cb_ctx* ctx, int on);
/* 1: never split a reduction across CTAs with atomics (bit-reproducible results). Default 0. */
int cb_set_deterministic(cb_ctx* ctx, int on);
/* Waits for the stream, then reads and clears the device status word. CB_OK or CB_ETIMEOUT/CB_ECUDA. */
int cb_synchronize(cb_ctx* ctx);
/* Exercises the bounded-wait path without faulting the GPU: launches a one-CTA kernel whose only act is to wait, for
 * at most limit_ms (1..1000) milliseconds, on a barrier that nothing ever arrives at. The wait gives up, the kernel
 * records its status and returns normally; the next cb_synchronize (or this call, in sync mode) reports CB_ETIMEOUT
 * and clears the status, after which the context is usable as before. */
int cb_selftest_wait_timeout(cb_ctx* ctx, int limit_ms);
const char* cb_last_error(const cb_ctx* ctx);
/* Number of kernels this context has launched since creation (for launch accounting). */
long long cb_launch_count(const cb_ctx* ctx);
const char* cb_version(void);

/* ---- GEMM ---------------------------------------------------------------------------------- */

/*
 * C[b] = op(A[b]) * op(B[b]) (+ C[b] if accumulate), b = 0..batch-1, all row-major fp32.
 *   op(A) is M x K: transA == 0 -> A stored M x K with leading dimension lda,
 *                   transA != 0 -> A stored K x M with leading dimension lda.
 *   op(B) is K x N: transB == 0 -> B stored K x N (ldb); transB != 0 -> B stored N x K (ldb).
 *   strideA/B/C are the element distances between consecutive batch matrices (0 = shared operand).
 * Replaces seblas::sgemm (NN, batched over B.n with A shared; seblas/operations/cuGEMM.cu:1649),
 * sgemmTN (:1667) and sgemmNT (:1685); sgemmNTA (:1701) is cb_gemm_batch_reduce.
 */
int cb_gemm(cb_ctx* ctx, int transA, int transB, int M, int N, int K, const float* A, int lda, const float* B,
            int ldb, float* C, int ldc, int batch, long long strideA, long long strideB, long long strideC,
            int accumulate);

/*
 * C (+)= sum over b = 0..count-1 of op(A[b]) * op(B[b]): cb_gemm's operand conventions, one M x N result. Replaces
 * seblas::sgemmNTA (seblas/operations/cuGEMM.cu:1701-1714 with its kernels :1370-1640: C += A[n] * B[n]^T summed over
 * A->dims.n) with transA = 0, transB = 1, accumulate = 1. On the tensor-core paths the batch is folded into the
 * contraction: ONE launch whose k-blocks walk the pairs.
 */
int cb_gemm_batch_reduce(cb_ctx* ctx, int transA, int transB, int M, int N, int K, const float* A, int lda, const float* B,
                         int ldb, float* C, int ldc, int count, long long strideA, long long strideB, int accumulate);

/* Measured ceiling of the TF32 tensor pipe on this GPU: runs, on every SM, a loop that only issues
 * tcgen05.mma.kind::tf32 (M = 128, N = n, K = 8) on operands resident in shared memory — no global traffic, no
 * epilogue — `iters` groups of four per SM, timed with CUDA events, and returns the rate in TFLOP/s. p_mn / q_mn select
 * the operand layouts (0 = K-major, 1 = MN-major), which the rate depends on. Used as the roofline denominator of the
 * GEMM and convolution kernels. Synchronous. */
int cb_measure_umma_peak(cb_ctx* ctx, int n, int p_mn, int q_mn, int iters, float* tflops);

/* Name of the kernel family the last cb_gemm / cb_conv_* call dispatched to ("umma_tf32",
 * "umma_3xtf32", "simt_fp32"); for tests and launch accounting. */
const char* cb_last_kernel(const cb_ctx* ctx);

/* ---- convolution (NCHW fp32) ------------------------------------------------------------------ */

/*
 * Geometry shared by the three passes: X is N x IC x IH x IW, W is OC x IC x FH x FW, Y is N x OC x OH x OW with
 * OH = (IH - FH + 2 pH)/sH + 1 and OW likewise (the relation seblas::assertConv enforces,
 * seblas/operations/cuConv.cu:731-755).
 */

/* Y = conv(W, X) (+ bias[oc]) (then ReLU if relu != 0). Replaces seblas::conv (seblas/operations/cuConv.cu:757). */
int cb_conv_fwd(cb_ctx* ctx, const float* W, const float* X, float* Y, const float* bias, int N, int IC, int IH,
                int IW, int OC, int FH, int FW, int sH, int sW, int pH, int pW, int relu);
/* dX = data gradient of the same convolution. Replaces seblas::convDerive (seblas/operations/cuConv.cu:774). */
int cb_conv_dgrad(cb_ctx* ctx, const float* W, const float* dY, float* dX, int N, int IC, int IH, int IW, int OC,
                  int FH, int FW, int sH, int sW, int pH, int pW);
/* dW (+)= weight gradient; the reference always accumulates (accumulate = 1). Uses the correct index map
 * ih = oh*sH - pH + fh for every stride. Replaces seblas::convError (seblas/operations/cuConv.cu:793). */
int cb_conv_wgrad(cb_ctx* ctx, const float* dY, const float* X, float* dW, int N, int IC, int IH, int IW, int OC,
                  int FH, int FW, int sH, int sW, int pH, int pW, int accumulate);
/*
 * Extended forms. cb_conv_fwd_ex applies, while the accumulator is written out and in this order:
 *   y = conv(W, X);  y = y * scale + shift (if scale != NULL);  y += bias[oc] (if bias);  y += Y (if accumulate);
 *   y = max(y, 0) (if relu).
 * scale / shift hold OC values, or OC*OH*OW values (one per output position, the shape of the reference's BatchNorm
 * parameters, seann/operands/seblas/BatchNorm.cuh:27-33) when per_position != 0: a BatchNorm whose statistics are
 * already known folds into the convolution this way. x_batch_stride / y_batch_stride are the element distances between
 * consecutive images of X and Y (0 = densely packed): a convolution can read a channel prefix of, or write a channel
 * slice of, a wider N x C_total x H x W buffer without a copy, which is how a DenseNet block's channel concatenation
 * (seblas::concat, seblas/operations/cuConcat.cu:33-49) is avoided. The reference has no counterpart of these forms;
 * with ep == NULL cb_conv_fwd_ex is cb_conv_fwd without bias and ReLU.
 * cb_conv_dgrad_ex / cb_conv_wgrad_ex: `accumulate` adds the result onto dX / dW — the dA += dAReserve hand-over every
 * operand's xGrads begins with (seann/operands/seblas/Conv2D.cu:19-21) folded into the kernel — and the strides as above.
 */
typedef struct cb_epilogue {
    const float* bias;
    const float* scale;
    const float* shift;
    int per_position;
    int relu;
    int accumulate;
    long long x_batch_stride;
    long long y_batch_stride;
} cb_epilogue;
int cb_conv_fwd_ex(cb_ctx* ctx, const float* W, const float* X, float* Y, int N, int IC, int IH, int IW, int OC, int FH,
                   int FW, int sH, int sW, int pH, int pW, const cb_epilogue* ep);
int cb_conv_dgrad_ex(cb_ctx* ctx, const float* W, const float* dY, float* dX, int N, int IC, int IH, int IW, int OC,
                     int FH, int FW, int sH, int sW, int pH, int pW, int accumulate, long long dy_batch_stride,
                     long long dx_batch_stride);
int cb_conv_wgrad_ex(cb_ctx* ctx, const float* dY, const float* X, float* dW, int N, int IC, int IH, int IW, int OC,
                     int FH, int FW, int sH, int sW, int pH, int pW, int accumulate, long long dy_batch_stride,
                     long long x_batch_stride);

/*
 * Packed-filter cache. The tensor-core forward and data-gradient kernels read the filter in a packed, padded layout
 * that a small kernel produces from W before every call. With the cache on, the context keeps the packed copy of every
 * (filter pointer, geometry, pass) it has seen and reuses it until the filter's values change:
 *   - cb_momentum, cb_momentum_multi and cb_tensor_op on the same context mark every cached copy stale (each is
 *     re-packed by the next convolution that uses it);
 *   - after writing to a filter by any other route the caller must call cb_filters_changed, which re-packs every cached
 *     filter in ONE launch on the context's stream (a training step then pays one pack launch instead of two per
 *     convolution).
 * Packed copies are device allocations made at a filter's first use (do that before capturing a CUDA graph) and
 * released by cb_destroy. Default: off — every call packs its filter into the context workspace.
 */
int cb_conv_cache_filters(cb_ctx* ctx, int on);
int cb_filters_changed(cb_ctx* ctx);

/* Y[n,c,:,:] += bias[c]. Replaces seblas::convBias (seblas/operations/cuConv.cu:808). */
int cb_conv_bias(cb_ctx* ctx, float* Y, const float* bias, int N, int C, int HW);
/* db[c] (+)= sum over (n,h,w) of dY: the bias gradient cuConv2D takes from cuDNN
 * (seann/operands/cudnn/cuConv2D.cu:69). */
int cb_conv_bias_grad(cb_ctx* ctx, const float* dY, float* db, int N, int C, int HW, int accumulate);

/* ---- Linear (dense layer) ------------------------------------------------------------------------ */

/* Y[n,m] = sum_k W[m,k] X[n,k] + b[m]; X: batch x IN, W: OUT x IN, b: OUT (nullable), Y: batch x OUT.
 * Replaces seblas::linear (seblas/operations/cuLinear.cu:1052). */
int cb_linear_fwd(cb_ctx* ctx, const float* X, const float* W, const float* b, float* Y, int batch, int IN, int OUT);
/* dX[n,k] = sum_m W[m,k] dY[n,m]. Replaces seblas::linearXGrad (seblas/operations/cuLinear.cu:1075). */
int cb_linear_xgrad(cb_ctx* ctx, const float* dY, const float* W, float* dX, int batch, int IN, int OUT);
/* dW[m,k] += sum_n dY[n,m] X[n,k]; db[m] += sum_n dY[n,m] (db nullable; each term counted once).
 * Replaces seblas::linearParamGrad (seblas/operations/cuLinear.cu:1098). */
int cb_linear_paramgrad(cb_ctx* ctx, const float* dY, const float* X, float* dW, float* db, int batch, int IN,
                        int OUT);

/* ---- memory-bound neighbours ------------------------------------------------------------------- */

/* BatchNorm with statistics per (c,h,w) position over the batch (P = C*H*W positions), eps = 1e-8, any batch
 * size. mean, var and xhat may be NULL. Replaces seblas::batchNorm / batchNormGrad / batchNormParamGrads
 * (seblas/operations/cuBatchNorm.cu:150,167,180). */
int cb_bn_fwd(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, float* mean, float* var, float* Y,
              float* xhat, int N, long long P);
int cb_bn_bwd(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, int N, long long P);
int cb_bn_paramgrad(cb_ctx* ctx, const float* dY, const float* xhat, float* dgamma, float* dbeta, int N, long long P);
/* batchNormGrad and batchNormParamGrads (seblas/operations/cuBatchNorm.cu:64-147) in one pass over X and dY: dX,
 * dgamma = sum dy * xhat and dbeta = sum dy (assigned), with xhat recomputed from X so it need not be stored.
 * relu_out (nullable): output of a ReLU that followed this layer in the forward pass; dY is then masked by
 * relu_out > 0 first (reluGradFast folded in). Needs N <= 256, P % 4 == 0 and 16-byte aligned tensors
 * (CB_EUNSUPPORTED otherwise: use the separate calls). */
int cb_bn_bwd_fused(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, float* dgamma,
                    float* dbeta, const float* relu_out, int N, long long P);
/* Y = relu(batchNorm(X)) in one pass (the BatchNorm -> ReLU pair of the operand graph, seann/operands/seblas/BatchNorm.cu:14
 * followed by activate/ReLU.cu:8); same limits as cb_bn_bwd_fused. */
int cb_bn_fwd_relu(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, float* Y, int N, long long P);
/*
 * Batch-strided forms for tensors that are a channel prefix of a wider NCHW tensor (a DenseNet block buffer that later
 * layers append their feature maps to, so that concatenation costs no copy; the reference's concat copies,
 * seblas/operations/cuConcat.cu:9-60): the N samples of X (and of dX) are x_batch_stride (dx_batch_stride) floats
 * apart instead of P; 0 = dense. cb_bn_fwd_relu_ex reads X strided and writes a dense Y. cb_bn_bwd_fused_ex reads X
 * strided, writes dX strided, and with accumulate_dx adds onto what dX already holds (the gradient of the shared
 * buffer collects contributions from every layer that read it). cb_avgpool_ex / cb_avgpool_back_ex: the pooled tensor
 * (Y resp. dY) is the strided one. Strides are at least one sample and multiples of 4 floats.
 */
int cb_bn_fwd_relu_ex(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, float* Y, int N, long long P,
                      long long x_batch_stride);
int cb_bn_bwd_fused_ex(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, float* dgamma,
                       float* dbeta, const float* relu_out, int N, long long P, long long x_batch_stride,
                       long long dx_batch_stride, int accumulate_dx);
int cb_avgpool_ex(cb_ctx* ctx, const float* X, float* Y, int N, int C, int H, int W, int rH, int rW, long long y_batch_stride);
int cb_avgpool_back_ex(cb_ctx* ctx, float* dX, const float* dY, int N, int C, int H, int W, int rH, int rW,
                       long long dy_batch_stride);

/* Y = relu(batchNorm(X) + R): the BatchNorm that ends a residual block, the shortcut add
 * (seann/operands/controlling/ShortcutEndpoint.cu:57-74) and the ReLU after it (archive/Resnet56:14-15) in one pass; and
 * the matching backward pass: dY is masked by relu_out > 0, the masked gradient is written (or, with accumulate_dR,
 * added) to the shortcut's gradient dR — what ShortcutEndpoint::xGrads routes to the skip path
 * (ShortcutEndpoint.cu:76-99) — and goes on through the BatchNorm as in cb_bn_bwd_fused. Same limits as cb_bn_bwd_fused. */
int cb_bn_fwd_add_relu(cb_ctx* ctx, const float* X, const float* beta, const float* gamma, const float* R, float* Y, int N,
                       long long P);
int cb_bn_bwd_fused_res(cb_ctx* ctx, const float* dY, const float* gamma, const float* X, float* dX, float* dgamma,
                        float* dbeta, const float* relu_out, float* dR, int accumulate_dR, int N, long long P);

/* seblas::relu / reluGradFast (seblas/operations/cuActivation.cu:268,296). */
int cb_relu(cb_ctx* ctx, const float* X, float* Y, long long n);
int cb_relu_grad(cb_ctx* ctx, const float* X, const float* dY, float* dX, long long n);
/* Out = relu(A + B): the shortcut add (seann/operands/controlling/ShortcutEndpoint.cu:57-74) and the ReLU after it in one
 * pass; and its gradient for both addends, dA = dB = (Y > 0 ? dY : 0) (dB nullable). */
int cb_add_relu(cb_ctx* ctx, const float* A, const float* B, float* Out, long long n);
int cb_relu_grad2(cb_ctx* ctx, const float* Y, const float* dY, float* dA, float* dB, long long n);

/* In-place tensor arithmetic of seblas::Tensor (operator+ - * / with a tensor or a scalar, constFill;
 * seblas/tensor/Tensor.cu:462-660): A = A op B or A = A op scalar. */
enum {
    CB_OP_ADD = 0, CB_OP_SUB = 1, CB_OP_MUL = 2, CB_OP_DIV = 3,
    CB_OP_ADD_SCALAR = 4, CB_OP_SUB_SCALAR = 5, CB_OP_MUL_SCALAR = 6, CB_OP_DIV_SCALAR = 7, CB_OP_FILL = 8
};
int cb_tensor_op(cb_ctx* ctx, int op, float* A, const float* B, float scalar, long long n);
/* dA += dA_reserve; dA_reserve = 0 in one pass: the step every operand's xGrads begins with
 * (e.g. seann/operands/seblas/Conv2D.cu:19-21). */
int cb_grad_handover(cb_ctx* ctx, float* dA, float* dA_reserve, long long n);

/* Channel concatenation Y = [X[0] ; X[1] ; ...] of `count` N x channels[i] x HW tensors (seblas::concat,
 * seblas/operations/cuConcat.cu:33-49) and its gradient, which ADDS each channel slice of dY into dX[i]
 * (seblas::concatGrads, cuConcat.cu:51-82, adds into the sources' dAReserve). X / dX / channels are host arrays. */
int cb_concat_channels(cb_ctx* ctx, int count, const float* const* X, const int* channels, float* Y, int N, int HW);
int cb_concat_grads(cb_ctx* ctx, int count, float* const* dX, const int* channels, const float* dY, int N, int HW);

/* Non-overlapping average pooling over NC planes of H x W and its gradient (seblas::avgPool / avgPoolBack,
 * seblas/operations/cuPool.cu:153-169); global average pooling and its gradient (cuPool.cu:171-184). */
int cb_avgpool(cb_ctx* ctx, const float* X, float* Y, long long NC, int H, int W, int rH, int rW);
int cb_avgpool_back(cb_ctx* ctx, float* dX, const float* dY, long long NC, int H, int W, int rH, int rW);
int cb_global_avgpool(cb_ctx* ctx, const float* X, float* Y, long long NC, int HW);
int cb_global_avgpool_back(cb_ctx* ctx, float* dX, const float* dY, long long NC, int HW);

/* Row softmax y = exp(x - max)/(sum + 1e-10) (seblas::softmax, seblas/operations/cuReduce.cu:296), and the
 * softmax cross-entropy pair: dY = Y - labels (seblas::crossEntropyLoss, cuLoss.cu:231) with the summed loss
 * -sum(log(Y + 1e-10) * labels) written to the device word *loss_sum (crossEntropyCalc, cuLoss.cu:220).
 * dY and loss_sum may be NULL. */
int cb_softmax(cb_ctx* ctx, const float* X, float* Y, int rows, int step);
int cb_cross_entropy(cb_ctx* ctx, const float* Y, const float* labels, float* dY, float* loss_sum, long long n);

/* The classifier head of the models as one kernel per direction. Forward: global average pooling of X (N x C x HW)
 * (seblas::globalAvgPool, seblas/operations/cuPool.cu:171-176), the dense layer logits = W pooled + b with W M x C
 * (seblas::linear, cuLinear.cu:1052), the softmax (cuReduce.cu:296), the loss gradient dlogits = softmax - labels
 * (cuLoss.cu:231) and each sample's loss -sum(log(y + 1e-10) * label) (cuLoss.cu:220) — four launches of the operand
 * graph (GlobalAvgPool, Linear, Softmax, crossEntropyLoss / crossEntropyCalc). Backward: dX = pooling gradient of the
 * dense layer's data gradient, dW += dlogits^T pooled, db += column sums (accumulated like every seblas parameter
 * gradient; db nullable), and loss_sum (nullable) = sum of the per-sample losses. M <= 32 classes. */
int cb_head_fwd(cb_ctx* ctx, const float* X, const float* W, const float* b, const float* labels, float* pooled, float* logits,
                float* probs, float* dlogits, float* loss_per_sample, int N, int C, int HW, int M);
int cb_head_bwd(cb_ctx* ctx, const float* dlogits, const float* pooled, const float* W, float* dX, float* dW, float* db,
                const float* loss_per_sample, float* loss_sum, int N, int C, int HW, int M);

/* Momentum step of seann (seann/optimizers/Optimizers.cu:17-22 over seblas::momentumApply,
 * seblas/operations/cuOptim.cu:38-46): w *= (1 - l2) if is_weight; m = beta m + (1 - beta) g; w -= lr m; g = 0.
 * The multi form updates every tensor of a model in one launch. */
int cb_momentum(cb_ctx* ctx, float* w, float* g, float* m, long long n, float lr, float beta, float l2,
                int is_weight);
int cb_momentum_multi(cb_ctx* ctx, int ntensors, float* const* w, float* const* g, float* const* m,
                      const long long* sizes, const unsigned char* is_weight, float lr, float beta, float l2);

/* ---- allocation-free variant ---------------------------------------------------------------------- */

/*
 * Forward convolution for callers that must not allocate device memory: code that runs under a memory manager
 * which has already claimed the whole GPU (cudaMalloc would fail), code on a latency-critical path that cannot
 * afford cudaMalloc's implicit device synchronisation, and code that runs while a stream is being captured
 * (allocation calls are not permitted there). It needs no cb_ctx and calls no cudaMalloc / cudaFree or any
 * allocating library routine: the packed filter the tensor-core kernel reads lives in a fixed 160 KiB array (plus
 * one status word) that every GPU holding this library keeps from load until exit.
 * This entry point has no counterpart in the reference.
 *
 *  - Same arithmetic as cb_conv_fwd in CB_MATH_TF32 mode; Y (+ bias, then ReLU if relu != 0) is written
 *    asynchronously on `cuda_stream` of `device`.
 *  - Geometry: stride 1; 1x1 filters with padding 0 or 3x3 with padding 1 (per axis); map width 8, 16 or 32 with
 *    (32 / width) dividing the height; FW * OC (OC rounded up to 16) <= 256; X 16-byte aligned. The packed filter,
 *    FH * ceil(IC / 32) * FW * roundup16(OC) * 128 bytes, must fit in 163 840 bytes (a 64 -> 64 channel 3x3 filter
 *    needs 147 456); larger requests are rejected with CB_EINVAL and a message, other geometries with
 *    CB_EUNSUPPORTED.
 *  - The first call on a device resolves the device address of the static array (cudaGetSymbolAddress) and reads
 *    the device attributes; make that first call before any stream capture begins.
 *  - Every call on a device shares the one array (it keeps the previous call's contents; each call rewrites the
 *    part it uses). Calls that overlap on the GPU — different streams, or different host threads — race on it: issue
 *    them on one stream. Several host threads may make their first call at the same time.
 *  - The caller's current device is unchanged on return (the call makes `device` current only while it runs).
 *  - `err` (nullable) receives a message of at most err_len bytes when the return value is not CB_OK.
 *  - The call is asynchronous and returns CB_OK once the work is queued. Whether a bounded device-side wait expired
 *    while it ran is reported by cb_conv_fwd_noalloc_status, which waits for `cuda_stream`, reads the static status
 *    word (no allocation either) and returns CB_OK, or CB_ETIMEOUT with the reason in `err` after clearing the word.
 */
int cb_conv_fwd_noalloc(int device, void* cuda_stream, const float* W, const float* X, float* Y, const float* bias,
                        int N, int IC, int IH, int IW, int OC, int FH, int FW, int sH, int sW, int pH, int pW,
                        int relu, char* err, int err_len);
int cb_conv_fwd_noalloc_status(int device, void* cuda_stream, char* err, int err_len);

/*
 * Host-only readers of a .crseq model file (seio/modelcache/codec.cuh:14-70 file layout): operand count (branch
 * operands of shortcut endpoints included), epoch id and the number of parameter floats; and the parameter section as
 * the file stores it (operand order; BatchNorm beta before gamma). No GPU is touched. CB_EINVAL with a message in
 * `err` for a file that is not .crseq, is truncated, or names an operand outside the supported vocabulary.
 */
int cb_crseq_inspect(const char* path, unsigned* operand_count, unsigned* epoch, unsigned long long* param_floats,
                     char* err, int err_len);
int cb_crseq_read_params(const char* path, float* out, unsigned long long count, char* err, int err_len);

#ifdef __cplusplus
}
#endif
#endif /* CRUSADER_B200_H */
