// Pieces shared by the tensor-core convolution translation units (conv_sm100.cu: forward / data gradient,
// wgrad_sm100.cu: weight gradient): pipeline constants, the warp-level bounded wait, the stride-2 tap maps, and the
// host launchers of the re-layout kernels of the stride-2 path.
#pragma once
#include "cb_internal.h"
#include "cb_ptx.cuh"

namespace cb {

constexpr int kCB = 8;          // input channels per UMMA K step
constexpr int kConvMaxStages = 8;
constexpr int kRowBytes = 128;  // one line of 32 floats

__device__ __forceinline__ bool conv_warp_wait(uint32_t bar, uint32_t parity, int lane, volatile int* abort_flag,
                                               int* status, int code) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, status, code) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Source filter tap of the stride-2 convolution that lands on (input phase, tap of the 2x2 phase convolution):
// with ih = 2 oh + fh - 1, tap fh = 0 reads phase 1 at row oh - 1, fh = 1 phase 0 at row oh, fh = 2 phase 1 at row oh.
__host__ __device__ __forceinline__ int s2_tap(int phase, int t) { return phase == 1 ? (t == 0 ? 0 : 2) : (t == 1 ? 1 : -1); }

// Re-layout passes of the stride-2 path (memory-bound, one element per thread, coalesced on the write side), launched
// on the context's stream; each counts one launch.
//   space_to_depth2: Xs[n][phase*C + c][i][j] = X[n][c][2i + (phase >> 1)][2j + (phase & 1)]
//   subsample2:      Xsub[nc][i][j] = X[nc][2i][2j]
int launch_space_to_depth2(cb_ctx* ctx, const float* X, float* Xs, int N, int C, int H, int W);
int launch_subsample2(cb_ctx* ctx, const float* X, float* Xsub, long long NC, int H, int W);

}  // namespace cb
