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
 * A context is used by one host thread at a time; create one per GPU.
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
/* 1: never split a reduction across CTAs with atomics (bit-reproducible results). Default 0. */
int cb_set_deterministic(cb_ctx* ctx, int on);
/* Waits for the stream, then reads and clears the device status word. CB_OK or CB_ETIMEOUT/CB_ECUDA. */
int cb_synchronize(cb_ctx* ctx);
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
 * sgemmTN (:1667), sgemmNT (:1685) and, with accumulate=1 and the batch folded by the caller,
 * sgemmNTA (:1701).
 */
int cb_gemm(cb_ctx* ctx, int transA, int transB, int M, int N, int K, const float* A, int lda, const float* B,
            int ldb, float* C, int ldc, int batch, long long strideA, long long strideB, long long strideC,
            int accumulate);

/* Name of the kernel family the last cb_gemm / cb_conv_* call dispatched to ("umma_tf32",
 * "umma_3xtf32", "simt_fp32"); for tests and launch accounting. */
const char* cb_last_kernel(const cb_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* CRUSADER_B200_H */
