/*
 * mta_b200 — C ABI of the B200 (sm_100a) Multi-Token-Attention forward library.
 *
 * Every pointer named x, w, y, q, k, v, o, workspace is a DEVICE pointer owned by the caller.
 * Unless a function says otherwise nothing here allocates or frees memory, every launch is
 * asynchronous on the cudaStream_t passed as `stream` (a void* so that this header needs no CUDA
 * include), and the return value is a status code:
 *     0 ok, 1 invalid argument / unsupported shape, 2 CUDA runtime error, 3 device is not sm_100,
 *     4 a device-side bounded wait ran out.
 * After a non-zero return mta_last_error() gives a thread-local, human-readable reason.
 * The functions never throw and never abort the process.
 *
 * dtype codes: 0 float32, 1 bfloat16, 2 float16.  Weights may be float32 or the activation dtype.
 *
 * Each entry point names the interface of the reference project that it stands in for
 * (paths relative to that project).
 */
#ifndef MTA_B200_H
#define MTA_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { MTA_OK = 0, MTA_ERR_INVALID = 1, MTA_ERR_CUDA = 2, MTA_ERR_ARCH = 3, MTA_ERR_TIMEOUT = 4 };
enum { MTA_F32 = 0, MTA_BF16 = 1, MTA_F16 = 2 };

/* Version of this ABI; bumped on any signature change. */
int mta_abi_version(void);

/* Thread-local description of the last failure on the calling thread ("" if none). */
const char* mta_last_error(void);

/*
 * Depthwise causal 2-D convolution over a score plane.
 * Replaces Conv2dTritonFunction.forward + conv_fwd_kernel (convolution_2d_trit.py:301-333, :52-135).
 *   x, y: (N,C,H,W) contiguous, dtype x_dtype.  w: (C,R,S), dtype w_dtype.
 *   y[n,c,q,k] = sum_{i<R,j<S} w[c,i,j] * xh[n,c,q+i-(R-1),k+j-(S-1)/2], fp32 accumulation;
 *   xh is x inside the plane and 0 outside; when causal, xh is 0 where k' > q' (input above the
 *   diagonal is never read) and y is written as 0 where k > q.  The whole of y is written.
 */
int mta_conv2d_fwd(const void* x, const void* w, void* y, int N, int C, int H, int W, int R, int S,
                   int causal, int x_dtype, int w_dtype, void* stream);

/*
 * Head-mixing linear across the channel (head) axis of a score plane, without a transpose.
 * Replaces TritonLinearHeadFunction.forward + linear_head_kernel_forward
 * (triton_linear_head.py:283-319, :76-139).
 *   x, y: (N,C,P,Q) contiguous.  Wm: (C,C) in nn.Linear orientation: y[n,o,p,q] = sum_h Wm[o,h] x[n,h,p,q]
 *   for q <= p (everywhere if not causal); y = fill where q > p (the reference pre-fills the output
 *   with `output_value`, :294-297).  fill may be -inf.  The whole of y is written.
 */
int mta_head_linear_fwd(const void* x, const void* Wm, void* y, int N, int C, int P, int Q, int causal,
                        float fill, int x_dtype, int w_dtype, void* stream);

/*
 * Row softmax over keys q <= p (causal) or all keys, computed in fp32, output in the input dtype;
 * entries above the diagonal are written as 0.  Stands in for the F.softmax(scores.float(), -1)
 * .type_as(xq) step of MTAAttentionTriton.forward (mta_attention_triton.py:79) reading only the
 * lower triangle.  x, y: (N,C,P,Q) contiguous; x may equal y.
 */
int mta_softmax_fwd(const void* x, void* y, int N, int C, int P, int Q, int causal, int dtype, void* stream);

/*
 * Causal head mix followed by the row softmax of the mixed logits, in one pass over the planes:
 *   y[n,o,p,q] = softmax_q( sum_h Wm[o,h] * x[n,h,p,q] over q <= p ),  0 for q > p.
 * The mixed logits are rounded to the dtype of x before the softmax, as the two reference stages do
 * (head mix with output_value = -inf, then F.softmax(scores.float(), -1).type_as(xq):
 * mta_attention_triton.py:76-79).  x, y: (N,C,P,Q) contiguous, x != y; Wm: (C,C).
 */
int mta_head_linear_softmax_fwd(const void* x, const void* Wm, void* y, int N, int C, int P, int Q, int x_dtype,
                                int w_dtype, void* stream);

/*
 * Scaled scores Q K^T * scale for keys k <= q (entries above the diagonal are never written when
 * causal) and P V over keys k <= q.  They stand in for the two torch.matmul calls of
 * MTAAttentionTriton.forward (mta_attention_triton.py:68-71, :89).  q,k,v,o: (B,H,S,D); s,p: (B,H,S,S).
 * `round_scale` != 0 reproduces the reference's 16-bit rounding (matmul result rounded, then
 * multiplied by the rounded scale and rounded again).
 */
int mta_qk_scores_fwd(const void* q, const void* k, void* s, int B, int H, int S, int D, float scale,
                      int round_scale, int causal, int dtype, void* stream);
int mta_pv_fwd(const void* p, const void* v, void* o, int B, int H, int S, int D, int causal, int dtype,
               void* stream);

/*
 * Fused conv attention forward: softmax(scale * conv(Q K^T)) V with the causal conv of
 * mta_conv2d_fwd applied to the unscaled scores.
 * Replaces TritonAttention.forward + _attn_fwd (conv_attention_triton.py:362-452, :167-356);
 * oracle ConvAttention.forward (conv_attention_pytorch.py:36-91).
 *   q,k,v,o: (B,H,S,D) contiguous; w: (H,cq,ck).
 * Causal 16-bit problems with D in {64,128} and an odd key extent <= 17 run as ONE kernel (scores, conv, online
 * softmax and P V per key tile, as _attn_fwd_inner does, conv_attention_triton.py:21-147): no S x S tensor exists and
 * mta_conv_attn_workspace_bytes(...) is 0 (workspace may be NULL).  Other problems (float32, non-causal, wider
 * kernels) run stage by stage and need that many bytes of caller-provided scratch (two score planes; contents
 * undefined on entry and exit).
 */
size_t mta_conv_attn_workspace_bytes(int B, int H, int S, int D, int cq, int ck, int causal, int dtype, int w_dtype);
int mta_conv_attn_fwd(const void* q, const void* k, const void* v, const void* w, void* o, void* workspace,
                      size_t workspace_bytes, int B, int H, int S, int D, int cq, int ck, int causal,
                      float scale, int dtype, int w_dtype, void* stream);

/*
 * mta_conv_attn_fwd without a caller workspace (this entry point has no counterpart in the reference), for callers
 * that must not or cannot allocate device memory: a serving loop with a frozen memory pool, code running inside an
 * allocator callback, a binding with no device buffers of its own.  Problems that mta_conv_attn_fwd runs as one kernel
 * need no scratch here either; for the rest the two scratch score planes live in a 64 MiB array built into the library
 * (MTA_STATIC_SCRATCH_BYTES, also returned by mta_static_scratch_bytes()).  Same arguments and results as
 * mta_conv_attn_fwd; returns 1 with a message when mta_conv_attn_workspace_bytes(...) exceeds the array.
 * It allocates nothing.  Looking up the array's device address is what makes the CUDA runtime place the 64 MiB on
 * that device: mta_static_scratch_prepare() does that lookup for the current device and belongs at start-up, before
 * the memory pool is frozen and before any stream capture (a first mta_conv_attn_fwd_static call would do it
 * otherwise).  All calls share the array: calls that overlap on the GPU race.
 */
#define MTA_STATIC_SCRATCH_BYTES ((size_t)64 << 20)
size_t mta_static_scratch_bytes(void);
int mta_static_scratch_prepare(void);
int mta_conv_attn_fwd_static(const void* q, const void* k, const void* v, const void* w, void* o, int B, int H, int S,
                             int D, int cq, int ck, int causal, float scale, int dtype, int w_dtype, void* stream);

/*
 * Gradients of the two stand-alone ops (the reference's autograd backward of Conv2dTritonFunction,
 * convolution_2d_trit.py:335-378, and of TritonLinearHeadFunction, triton_linear_head.py:321-370).
 *
 * mta_conv2d_bwd_input   dx[n,c,q,k] = sum_{i,j} w[c,i,j] * dyh[n,c,q-i+(R-1),k-j+(S-1)/2] for k <= q (everywhere if not
 *                        causal), 0 above the diagonal; dyh = dy inside the plane and (causal) where key <= query, else 0
 *                        (conv_bwd_input_kernel, :143-218).  dy, dx: (N,C,H,W) in `dtype`, the whole of dx is written.
 * mta_conv2d_bwd_weight  dw[c,i,j] = sum_{n,q,k} xh[n,c,q+i-(R-1),k+j-(S-1)/2] * dyh[n,c,q,k] (conv_bwd_weight_kernel,
 *                        :226-295).  dw: (C,R,S) float32 (the reference returns float64).  Partial sums go through the
 *                        workspace and are added in a fixed order in double precision.
 * mta_head_linear_bwd_input   dx[n,h,p,q] = sum_o Wm[o,h] * dy[n,o,p,q] for q <= p, 0 above the diagonal (the reference
 *                        leaves those entries uninitialised; linear_head_kernel_backward_input, :142-207).
 * mta_head_linear_bwd_weight  dW[o,h] = sum_{n,p,q<=p} dy[n,o,p,q] * x[n,h,p,q] (linear_head_kernel_backward_weight,
 *                        :210-278).  dW: (C,C) float32; workspace as above.
 */
int mta_conv2d_bwd_input(const void* dy, const void* w, void* dx, int N, int C, int H, int W, int R, int S, int causal,
                         int dtype, int w_dtype, void* stream);
size_t mta_conv2d_bwd_weight_workspace_bytes(int N, int C, int H, int W, int R, int S);
int mta_conv2d_bwd_weight(const void* x, const void* dy, float* dw, void* workspace, size_t workspace_bytes, int N, int C,
                          int H, int W, int R, int S, int causal, int dtype, void* stream);
int mta_head_linear_bwd_input(const void* dy, const void* Wm, void* dx, int N, int C, int P, int Q, int causal, int dtype,
                              int w_dtype, void* stream);
size_t mta_head_linear_bwd_weight_workspace_bytes(int C);
int mta_head_linear_bwd_weight(const void* x, const void* dy, float* dW, void* workspace, size_t workspace_bytes, int N,
                               int C, int P, int Q, int causal, int dtype, void* stream);

/*
 * Full four-stage MTA forward: QK^T/sqrt(D) -> conv (w1) -> head mix (W1) -> softmax -> conv (w2) ->
 * head mix (W2) -> @V, for batch elements [0,B) and query rows [q_row_begin, q_row_end).
 * Replaces the body of MTAAttentionTriton.forward (mta_attention_triton.py:61-92) with use_mask=False;
 * oracle MTAAttention.forward (mta_attention_pytorch.py:58-83).
 *   q,k,v,o: (B,H,S,D) contiguous (the Python module returns o.transpose(1,2) as the reference does);
 *   only rows [q_row_begin,q_row_end) of o are written.  w1 (H,cq,ck), W1 (H,H), w2 (H,cq2,ck2), W2 (H,H).
 *   ck and ck2 must be odd.  Needs mta_workspace_bytes(...) bytes of scratch.
 * The row range is what a caller sharding query rows over several GPUs passes: rows before
 * q_row_begin that the two convs reach back to ((cq-1)+(cq2-1) of them) are recomputed internally.
 */
size_t mta_workspace_bytes(int B, int H, int S, int D, int cq, int ck, int cq2, int ck2, int q_row_begin,
                           int q_row_end, int dtype);
int mta_fused_fwd(const void* q, const void* k, const void* v, const void* w1, const void* W1, const void* w2,
                  const void* W2, void* o, void* workspace, size_t workspace_bytes, int B, int H, int S, int D,
                  int cq, int ck, int cq2, int ck2, int q_row_begin, int q_row_end, int causal, int dtype,
                  int w_dtype, void* stream);

/*
 * mta_fused_fwd with dropout on the attention weights between the second head mix and the product with V, where
 * MTAAttentionTriton.forward applies F.dropout(scores, p=self.dropout, training=self.training)
 * (mta_attention_triton.py:87).  No mask tensor exists: whether weight (batch, head, query, key) is kept is a function
 * of (dropout_seed, batch * H + head, query, key) - one Philox4x32-10 block per 8 consecutive keys, counter
 * (key / 8, query, plane, 0), key = the seed, a key kept when its 16-bit field is below round((1 - p) * 65536) - so
 * the result does not depend on tiling or on the row range and can be reproduced on the host.  Kept weights are scaled
 * by 1 / (1 - p) and rounded to the dtype.  0 <= dropout_p < 1; dropout_p = 0 is mta_fused_fwd.
 */
int mta_fused_fwd_dropout(const void* q, const void* k, const void* v, const void* w1, const void* W1, const void* w2,
                          const void* W2, void* o, void* workspace, size_t workspace_bytes, int B, int H, int S, int D,
                          int cq, int ck, int cq2, int ck2, int q_row_begin, int q_row_end, int causal, int dtype,
                          int w_dtype, float dropout_p, unsigned long long dropout_seed, void* stream);

/*
 * mta_fused_fwd (all query rows) for a caller whose q, k, v and o live in HOST memory (page-locked memory lets the
 * copies overlap; pageable memory works but serialises them): the batch is cut into chunks of `chunk_batch` batch
 * elements (0 = choose) and three internal CUDA streams overlap the host->device copy of chunk c+1, the forward
 * of chunk c and the device->host copy of chunk c-1.  Stands in for .cuda() / MTAAttentionTriton.forward
 * (mta_attention_triton.py:61-92) / .cpu() done back to back.  w1, W1, w2, W2 are DEVICE pointers on the current
 * device.  Blocks until o is complete.  Staging and scratch memory are allocated on the first call per device,
 * reused and grown by later calls, and freed by mta_host_pipeline_release() (current device).
 */
int mta_fused_fwd_host(const void* q, const void* k, const void* v, const void* w1, const void* W1, const void* w2,
                       const void* W2, void* o, int B, int H, int S, int D, int cq, int ck, int cq2, int ck2,
                       int causal, int dtype, int w_dtype, int chunk_batch);
int mta_host_pipeline_release(void);

/*
 * Stage tracing of mta_fused_fwd (calling thread): after mta_set_stage_trace(1) every forward records a CUDA event
 * on its stream before each stage and after the last.  mta_stage_times_ms waits for the latest forward and writes
 * the device time of each of its stages (milliseconds) and, if `names` is not NULL, a static name per stage;
 * returns the number of stages written (at most `capacity`), or -1 on a CUDA error.
 */
int mta_set_stage_trace(int on);
int mta_stage_times_ms(float* ms, const char** names, int capacity);

/*
 * Synchronises `stream` and reports whether any kernel launched on this device since the last call gave
 * up a bounded device-side wait (returns 4 and clears the flag) - kernels never spin without limit.
 * The condition is sticky until this call: the kernel that gave up also writes a word of page-locked host memory, and
 * every compute entry point reads that word on entry (no synchronisation) and returns 4 without launching while it is
 * set, so a forward issued after a timeout has reached the host cannot pass garbage off as a result.
 */
int mta_device_status(void* stream);

/* Fault injection on the host, for tests of the path above: marks the current device exactly as a kernel's timed-out
 * wait would (no kernel is made to wait).  Until mta_device_status() clears it, kernels of this library return without
 * computing and every compute entry point returns 4 (MTA_ERR_TIMEOUT) without launching. */
int mta_inject_wait_timeout(void* stream);

/* Number of kernel launches issued by this library on the calling thread since the last reset
 * (what a benchmark reports as its launch count). */
long mta_launch_count(void);
void mta_reset_launch_count(void);

/* Selects implementation variants for A/B measurement (process-wide, atomically updated, read on every launch):
 * key "head_linear" -> 0 auto, 1 CUDA-core, 2 mma.sync tensor-core, 3 tcgen05 tensor-core; key "conv2d" -> 0 auto, 1 CUDA-core, 2 mma.sync tensor-core,
 * 3 tcgen05 tensor-core; key "gemm" (the two contractions) -> 0 auto, 1 CUDA-core, 2 tcgen05 tensor-core; key "fused"
 * -> 0 auto (mta_fused_fwd: Q K^T inside the first conv's kernel, the first head mix and the softmax as one kernel;
 * mta_conv_attn_fwd: one kernel), 1 strictly one kernel per stage, 2 the conv attention as three launches over score
 * planes (needs the workspace), 3 Q K^T and the first conv as two kernels; key "mix_softmax" (the head mix + softmax
 * kernel) -> 0 auto (tcgen05 where it applies: 16-bit activations and weights of one dtype, 8/16/32/64/128 heads),
 * 1 the mma.sync kernel, 2 tcgen05 or an error.  Returns 0, or 1 for an unknown key/value. */
int mta_set_variant(const char* key, int value);

#ifdef __cplusplus
}
#endif
#endif /* MTA_B200_H */
