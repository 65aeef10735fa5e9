// Internal launch interface between the C ABI (abi.cu), the fused forward (fused.cu) and the kernel
// translation units.  Every function enqueues work on `st` and returns an MTA_* status.
#pragma once

#include "common.cuh"
#include "dropout.cuh"

namespace mta {

// Depthwise causal conv over planes; computes output rows [row_begin,row_end) of every plane.
// When `write_upper` the entries above the diagonal of those rows are written as 0, otherwise they
// are left untouched (internal scratch whose upper triangle nobody reads).
// `x_rows_stored` = rows each plane of x holds (from xv.row0 on).
int conv2d_launch(const void* x, PlaneView xv, long x_rows_stored, const void* w, int w_dtype, void* y, PlaneView yv,
                  long planes, int C, int H, int W, int R, int S, int causal, int row_begin, int row_end,
                  bool write_upper, int dtype, cudaStream_t st);
// Tensor-core version (conv2d_mma.cu): 16-bit dtypes, S <= 17, W a multiple of 8, 16-byte aligned planes.
bool conv2d_mma_supported(const void* x, PlaneView xv, const void* y, PlaneView yv, int W, int R, int S, int dtype);
int conv2d_mma_launch(const void* x, PlaneView xv, long x_rows_stored, const void* w, int w_dtype, void* y, PlaneView yv,
                      long planes, int C, int H, int W, int R, int S, int causal, int row_begin, int row_end,
                      bool write_upper, int dtype, cudaStream_t st);

// Head mix over groups of C planes; rows [row_begin,row_end).  `write_upper` as above (value `fill`).
// `w_transposed`: y[o] = sum_h Wm[h,o] x[h] (the gradient with respect to the head mix's input).
int head_linear_launch(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N,
                       int C, int P, int Q, int causal, float fill, int row_begin, int row_end, bool write_upper,
                       int dtype, cudaStream_t st, bool w_transposed = false);

// Gradients of the two stand-alone ops (backward.cu, conv2d.cu).  dx of the conv: layout of x, zeros above the diagonal
// when causal.  The weight gradients are float32, reduced in a fixed order through a caller workspace of the given size.
int conv2d_bwd_input_launch(const void* dy, const void* w, int w_dtype, void* dx, long planes, int C, int H, int W, int R,
                            int S, int causal, int dtype, cudaStream_t st);
size_t conv2d_bwd_weight_workspace(int N, int C, int H, int W, int R, int S);
int conv2d_bwd_weight_launch(const void* x, const void* dy, float* dw, void* workspace, int N, int C, int H, int W, int R,
                             int S, int causal, int dtype, cudaStream_t st);
size_t head_linear_bwd_weight_workspace(int C);
int head_linear_bwd_weight_launch(const void* x, const void* dy, float* dW, void* workspace, int N, int C, int P, int Q,
                                  int causal, int dtype, cudaStream_t st);

// Head mix followed by the causal row softmax of the mixed logits, in one pass (16-bit dtypes, C <= 32, causal);
// entries above the diagonal of y are written as 0 when `write_upper`, else left untouched.
bool head_mix_softmax_supported(const void* x, PlaneView xv, const void* y, PlaneView yv, int C, int Q, int causal, int dtype,
                                int w_dtype);
int head_mix_softmax_launch(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C,
                            int Q, int row_begin, int row_end, bool write_upper, int dtype, cudaStream_t st);

// The same on tcgen05 (head_mix_tc05.cu): C a power of two in 8..128, weights in the activations' 16-bit dtype; entries
// above the diagonal are written as 0 up to the end of the diagonal's 128-key tile, and up to Q when `write_upper`.
bool head_mix_softmax_tc05_supported(const void* x, PlaneView xv, const void* y, PlaneView yv, int C, int Q, int causal, int dtype,
                                     int w_dtype);
int head_mix_softmax_tc05_launch(const void* x, PlaneView xv, const void* Wm, void* y, PlaneView yv, int N, int C, int Q,
                                 int row_begin, int row_end, bool write_upper, int dtype, cudaStream_t st);

// The plain head mix on the same kernel (one pass): y = Wm x over the head axis (Wm read transposed when `wt`), `fill`
// above the diagonal when causal (written up to the end of the diagonal's key tile, and up to Q when `write_upper`).
bool head_linear_tc05_supported(const void* x, PlaneView xv, const void* y, PlaneView yv, int C, int Q, int dtype, int w_dtype);
int head_linear_tc05_launch(const void* x, PlaneView xv, const void* Wm, void* y, PlaneView yv, int N, int C, int Q, int causal,
                            float fill, int row_begin, int row_end, bool write_upper, bool wt, int dtype, cudaStream_t st);

// Causal row softmax of pre_scale * x; rows [row_begin,row_end).
int softmax_launch(const void* x, PlaneView xv, void* y, PlaneView yv, long planes, int P, int Q, int causal,
                   int row_begin, int row_end, bool write_upper, float pre_scale, int dtype, cudaStream_t st);

// s = round(round(Q K^T) * scale) for rows [row_begin,row_end), keys k <= q when causal.
int qk_scores_launch(const void* q, const void* k, void* s, PlaneView sv, int B, int H, int S, int D, float scale,
                     int round_scale, int causal, int row_begin, int row_end, int dtype, cudaStream_t st);

// o[rows] = p[rows, k<=q] V.  `p_rows_stored` = number of rows each plane of p holds (from pview.row0 on).
// `drop`: dropout on the weights as they are read (dropout.cuh); the default leaves them as they are.
int pv_launch(const void* p, PlaneView pview, long p_rows_stored, const void* v, void* o, int B, int H, int S, int D,
              int causal, int row_begin, int row_end, int dtype, cudaStream_t st, DropoutSpec drop = DropoutSpec());

// CUDA-core versions of the two contractions (gemm_simt.cu).
int qk_scores_simt_launch(const void* q, const void* k, void* s, PlaneView sv, int B, int H, int S, int D, float scale,
                          int round_scale, int causal, int row_begin, int row_end, int dtype, cudaStream_t st);
int pv_simt_launch(const void* p, PlaneView pview, const void* v, void* o, int B, int H, int S, int D, int causal,
                   int row_begin, int row_end, int dtype, cudaStream_t st, DropoutSpec drop = DropoutSpec());

// tcgen05 version of the conv (conv2d_tc05.cu): 16-bit dtypes, S <= 17, W a multiple of 8, R small enough for its
// shared-memory rings (R <= 13 with 16-bit weights).
bool conv2d_tc05_supported(const void* x, PlaneView xv, const void* y, PlaneView yv, int W, int R, int S, int dtype,
                           int w_dtype);
// `grad_input` (odd S): the same kernel evaluates the gradient with respect to the conv's input - taps reversed, rows
// looking forward - with x = dy and y = dx.
int conv2d_tc05_launch(const void* x, PlaneView xv, long x_rows_stored, const void* w, int w_dtype, void* y, PlaneView yv,
                       long planes, int C, int H, int W, int R, int S, int causal, int row_begin, int row_end,
                       bool write_upper, int dtype, cudaStream_t st, bool grad_input = false);

// tcgen05 tensor-core versions (gemm_tc05.cu): 16-bit dtypes, D in {64,128}, S a multiple of 8.
bool tc05_contractions_supported(int S, int D, int dtype, const void* a, const void* b, const void* c, PlaneView view);
int pv_tc05_launch(const void* p, PlaneView pview, long p_rows_stored, const void* v, void* o, int B, int H, int S, int D,
                   int causal, int row_begin, int row_end, int dtype, cudaStream_t st, DropoutSpec drop = DropoutSpec());
// Persistent, warp-specialised score-tile kernel (qk_persistent.cu); same domain as the kernels above.
// NI = 1: c = scale * a b^T.  mode 0: all tiles with keys <= query; 1 / 2: the band of a (band_cq x (2 band_pw + 1))
// conv / the tiles wholly below it.
int qk_persistent_launch(const void* a, const void* b, void* c, PlaneView cv, int B, int H, int S, int D, int NI, float scale,
                         int round_scale, int causal, int mode, int band_cq, int band_pw, int row_begin, int row_end, int dtype,
                         cudaStream_t st);
// Scaled scores Q K^T and the causal conv of them in one kernel (qk_conv_tc05.cu): y = conv(round(round(Q K^T) scale)),
// rows [row_begin,row_end); the score planes never reach memory.  16-bit dtypes, D in {64,128}, odd key extent <= 17.
bool qk_conv_supported(const void* q, const void* k, const void* y, PlaneView yv, int S, int D, int R, int KS, int causal, int dtype,
                       int w_dtype);
int qk_conv_launch(const void* q, const void* k, const void* w, int w_dtype, void* y, PlaneView yv, int B, int H, int S, int D,
                   int R, int KS, float scale, int row_begin, int row_end, int dtype, cudaStream_t st);
// The conv attention forward softmax(sm_scale * conv(round(Q K^T * score_scale))) V in one kernel with no score plane
// anywhere (conv_attn_tc05.cu); output rows [row_begin,row_end).  16-bit dtypes, D in {64,128}, odd key extent <= 17,
// causal, any S.
bool conv_attn_fused_shape_ok(int S, int D, int R, int KS, int causal, int dtype, int w_dtype);
bool conv_attn_fused_supported(const void* q, const void* k, const void* v, const void* o, int S, int D, int R, int KS, int causal,
                               int dtype, int w_dtype);
int conv_attn_fused_launch(const void* q, const void* k, const void* v, const void* w, int w_dtype, void* o, int B, int H, int S, int D,
                           int R, int KS, float score_scale, float sm_scale, int row_begin, int row_end, int dtype, cudaStream_t st);
// Reads and clears the flag raised by a device-side bounded wait that gave up (synchronises `st`).
int device_wait_status(cudaStream_t st, int* timed_out);
// True when such a wait has given up on the current device since the last device_wait_status; reads the flag's mirror in
// host memory, no synchronisation.
bool wait_flag_raised();
// Raises the flag from the host as a timed-out wait would.
int wait_flag_inject(cudaStream_t st);

}  // namespace mta
