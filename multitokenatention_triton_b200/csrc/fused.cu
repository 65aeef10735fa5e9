// The two composite forwards of the C ABI.
//
//   mta_fused_fwd      QK^T/sqrt(D) -> conv(w1) -> head mix(W1) -> softmax -> conv(w2) -> head mix(W2) -> @V
//                      (body of MTAAttentionTriton.forward, mta_attention_triton.py:61-92, use_mask=False)
//   mta_conv_attn_fwd  softmax(scale * conv(Q K^T)) V   (TritonAttention.forward, conv_attention_triton.py:362-452)
//
// Both keep two score-plane scratch buffers in the caller's workspace, indexed by absolute query row
// relative to the first row the request needs, so a query-row range [q_row_begin, q_row_end) costs
// memory and work proportional to that range (plus the rows the convs reach back to).  Nothing above
// the diagonal of a scratch plane is ever written or read.
#include "kernels.cuh"

namespace mta {
namespace {

struct Plan {
    int ra, rb, r0, r1;      // first score row, first softmax row, first and one-past-last output row
    size_t buf_bytes;        // one scratch buffer
    size_t total() const { return 2 * buf_bytes; }
};

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

Plan make_plan(int B, int H, int S, int cq, int cq2, int r0, int r1, int dtype) {
    Plan p;
    p.r0 = r0;
    p.r1 = r1;
    p.rb = r0 - (cq2 - 1) > 0 ? r0 - (cq2 - 1) : 0;
    p.ra = p.rb - (cq - 1) > 0 ? p.rb - (cq - 1) : 0;
    p.buf_bytes = round_up((size_t)B * H * (size_t)(r1 - p.ra) * S * dtype_size(dtype), 256);
    return p;
}

// Stage tracing of mta_fused_fwd: when switched on, the forward records a CUDA event on its stream before every stage
// and after the last, and mta_stage_times_ms turns the latest forward's events into per-stage device times.
constexpr int MAX_STAGES = 8;
thread_local bool g_trace_on = false;
thread_local cudaEvent_t g_trace_ev[MAX_STAGES + 1] = {};
thread_local const char* g_trace_name[MAX_STAGES] = {};
thread_local int g_trace_n = 0;

int trace_mark(const char* name, cudaStream_t st) {
    if (!g_trace_on || g_trace_n >= MAX_STAGES) return MTA_OK;
    if (!g_trace_ev[g_trace_n]) MTA_CUDA_OK(cudaEventCreate(&g_trace_ev[g_trace_n]));
    MTA_CUDA_OK(cudaEventRecord(g_trace_ev[g_trace_n], st));
    g_trace_name[g_trace_n++] = name;
    return MTA_OK;
}
int trace_end(cudaStream_t st) {
    if (!g_trace_on) return MTA_OK;
    if (!g_trace_ev[g_trace_n]) MTA_CUDA_OK(cudaEventCreate(&g_trace_ev[g_trace_n]));
    MTA_CUDA_OK(cudaEventRecord(g_trace_ev[g_trace_n], st));
    return MTA_OK;
}

}  // namespace
}  // namespace mta

using namespace mta;

extern "C" {

int mta_set_stage_trace(int on) {
    g_trace_on = on != 0;
    g_trace_n = 0;
    return MTA_OK;
}

int mta_stage_times_ms(float* ms, const char** names, int capacity) {
    if (!ms || capacity < 0) return -1;
    const int n = g_trace_n < capacity ? g_trace_n : capacity;
    if (g_trace_n == 0) return 0;
    if (cudaEventSynchronize(g_trace_ev[g_trace_n]) != cudaSuccess) return -1;
    for (int i = 0; i < n; ++i) {
        if (cudaEventElapsedTime(&ms[i], g_trace_ev[i], g_trace_ev[i + 1]) != cudaSuccess) return -1;
        if (names) names[i] = g_trace_name[i];
    }
    return n;
}

size_t mta_workspace_bytes(int B, int H, int S, int D, int cq, int ck, int cq2, int ck2, int q_row_begin,
                           int q_row_end, int dtype) {
    (void)D; (void)ck; (void)ck2;
    if (B <= 0 || H <= 0 || S <= 0 || cq < 1 || cq2 < 1 || q_row_begin < 0 || q_row_end > S ||
        q_row_end <= q_row_begin || !dtype_ok(dtype))
        return 0;
    return make_plan(B, H, S, cq, cq2, q_row_begin, q_row_end, dtype).total();
}

int mta_fused_fwd(const void* q, const void* k, const void* v, const void* w1, const void* W1, const void* w2,
                  const void* W2, void* o, void* workspace, size_t workspace_bytes, int B, int H, int S, int D, int cq,
                  int ck, int cq2, int ck2, int q_row_begin, int q_row_end, int causal, int dtype, int w_dtype,
                  void* stream) {
    return mta_fused_fwd_dropout(q, k, v, w1, W1, w2, W2, o, workspace, workspace_bytes, B, H, S, D, cq, ck, cq2, ck2, q_row_begin,
                                 q_row_end, causal, dtype, w_dtype, 0.0f, 0ull, stream);
}

int mta_fused_fwd_dropout(const void* q, const void* k, const void* v, const void* w1, const void* W1, const void* w2,
                          const void* W2, void* o, void* workspace, size_t workspace_bytes, int B, int H, int S, int D, int cq,
                          int ck, int cq2, int ck2, int q_row_begin, int q_row_end, int causal, int dtype, int w_dtype,
                          float dropout_p, unsigned long long dropout_seed, void* stream) {
    set_error("%s", "");
    MTA_REQUIRE(dropout_p >= 0.0f && dropout_p < 1.0f, "fused_fwd: dropout probability %g outside [0, 1)", (double)dropout_p);
    DropoutSpec drop;
    drop.p = dropout_p;
    drop.seed = dropout_seed;
    MTA_REQUIRE(dtype_ok(dtype) && dtype_ok(w_dtype), "fused_fwd: unknown dtype code (%d, %d)", dtype, w_dtype);
    MTA_REQUIRE(B >= 0 && H >= 1 && S >= 0 && D >= 1, "fused_fwd: bad shape B=%d H=%d S=%d D=%d", B, H, S, D);
    MTA_REQUIRE(cq >= 1 && ck >= 1 && cq2 >= 1 && ck2 >= 1, "fused_fwd: kernel sizes must be positive");
    MTA_REQUIRE(ck % 2 == 1 && ck2 % 2 == 1, "fused_fwd: key kernel sizes %d and %d must be odd (pad_key=\"both\")", ck, ck2);
    MTA_REQUIRE(q_row_begin >= 0 && q_row_end <= S && q_row_begin <= q_row_end, "fused_fwd: row range [%d,%d) outside [0,%d)",
                q_row_begin, q_row_end, S);
    if ((long)B * S == 0 || q_row_begin == q_row_end) return MTA_OK;
    MTA_REQUIRE(q && k && v && w1 && W1 && w2 && W2 && o, "fused_fwd: null pointer");
    MTA_REQUIRE((long)B * H <= 65535, "fused_fwd: B*H = %ld exceeds 65535", (long)B * H);
    const Plan pl = make_plan(B, H, S, cq, cq2, q_row_begin, q_row_end, dtype);
    MTA_REQUIRE(workspace && workspace_bytes >= pl.total(), "fused_fwd: workspace of %zu bytes is smaller than the %zu needed",
                workspace_bytes, pl.total());
    MTA_REQUIRE(aligned16(workspace), "fused_fwd: workspace must be 16-byte aligned");
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char* ws = static_cast<char*>(workspace);
    void* bufA = ws;
    void* bufB = ws + pl.buf_bytes;
    const PlaneView pv{(long)(pl.r1 - pl.ra) * S, pl.ra, S};
    const long planes = (long)B * H;
    const float scale = 1.0f / sqrtf((float)D);
    const int round16 = dtype != MTA_F32;
    int rc;
    g_trace_n = 0;
    // Default for 16-bit dtypes: the scores are computed inside the first conv's kernel and never stored
    // (mta_set_variant("fused", 3) keeps the two kernels apart, as do the "gemm" and "conv2d" variants).
    const bool qk_in_conv = variant("fused") == 0 && variant("gemm") == 0 && variant("conv2d") == 0 && planes <= 65535 &&
                            qk_conv_supported(q, k, bufB, pv, S, D, cq, ck, causal, dtype, w_dtype);
    if (qk_in_conv) {
        if ((rc = trace_mark("qk_scores+conv1", st))) return rc;
        if ((rc = qk_conv_launch(q, k, w1, w_dtype, bufB, pv, B, H, S, D, cq, ck, scale, pl.rb, pl.r1, dtype, st))) return rc;
    } else {
    if ((rc = trace_mark("qk_scores", st))) return rc;
    if ((rc = qk_scores_launch(q, k, bufA, pv, B, H, S, D, scale, round16, causal, pl.ra, pl.r1, dtype, st))) return rc;
    }
    if (!qk_in_conv) {
        if ((rc = trace_mark("conv1", st))) return rc;
        if ((rc = conv2d_launch(bufA, pv, pl.r1 - pl.ra, w1, w_dtype, bufB, pv, planes, H, S, S, cq, ck, causal, pl.rb, pl.r1, !causal, dtype, st))) return rc;
    }
    // the first head mix and the softmax run as one kernel where it applies (mta_set_variant("fused", 1) keeps them apart)
    if (variant("fused") != 1 && head_mix_softmax_supported(bufB, pv, bufA, pv, H, S, causal, dtype, w_dtype)) {
        if ((rc = trace_mark("head_mix1+softmax", st))) return rc;
        if ((rc = head_mix_softmax_launch(bufB, pv, W1, w_dtype, bufA, pv, B, H, S, pl.rb, pl.r1, false, dtype, st))) return rc;
    } else {
        if ((rc = trace_mark("head_mix1", st))) return rc;
        if ((rc = head_linear_launch(bufB, pv, W1, w_dtype, bufA, pv, B, H, S, S, causal, 0.0f, pl.rb, pl.r1, false, dtype, st))) return rc;
        if ((rc = trace_mark("softmax", st))) return rc;
        if ((rc = softmax_launch(bufA, pv, bufA, pv, planes, S, S, causal, pl.rb, pl.r1, false, 1.0f, dtype, st))) return rc;
    }
    if ((rc = trace_mark("conv2", st))) return rc;
    if ((rc = conv2d_launch(bufA, pv, pl.r1 - pl.ra, w2, w_dtype, bufB, pv, planes, H, S, S, cq2, ck2, causal, pl.r0, pl.r1, !causal, dtype, st))) return rc;
    if ((rc = trace_mark("head_mix2", st))) return rc;
    if ((rc = head_linear_launch(bufB, pv, W2, w_dtype, bufA, pv, B, H, S, S, causal, 0.0f, pl.r0, pl.r1, false, dtype, st))) return rc;
    if ((rc = trace_mark("pv", st))) return rc;
    if ((rc = pv_launch(bufA, pv, pl.r1 - pl.ra, v, o, B, H, S, D, causal, pl.r0, pl.r1, dtype, st, drop))) return rc;
    return trace_end(st);
}

// One kernel, no scratch: 16-bit dtypes the fused kernel takes (mta_set_variant("fused", 2) keeps the three-launch path).
static bool conv_attn_one_kernel(int S, int D, int cq, int ck, int causal, int dtype, int w_dtype) {
    return variant("fused") == 0 && variant("gemm") == 0 && variant("conv2d") == 0 &&
           conv_attn_fused_shape_ok(S, D, cq, ck, causal, dtype, w_dtype);
}

size_t mta_conv_attn_workspace_bytes(int B, int H, int S, int D, int cq, int ck, int causal, int dtype, int w_dtype) {
    if (B <= 0 || H <= 0 || S <= 0 || cq < 1 || !dtype_ok(dtype) || !dtype_ok(w_dtype)) return 0;
    if (conv_attn_one_kernel(S, D, cq, ck, causal, dtype, w_dtype)) return 0;
    return 2 * make_plan(B, H, S, cq, 1, 0, S, dtype).buf_bytes;      // this path uses the two score planes only
}

int mta_conv_attn_fwd(const void* q, const void* k, const void* v, const void* w, void* o, void* workspace,
                      size_t workspace_bytes, int B, int H, int S, int D, int cq, int ck, int causal, float scale,
                      int dtype, int w_dtype, void* stream) {
    set_error("%s", "");
    MTA_REQUIRE(dtype_ok(dtype) && dtype_ok(w_dtype), "conv_attn_fwd: unknown dtype code (%d, %d)", dtype, w_dtype);
    MTA_REQUIRE(B >= 0 && H >= 1 && S >= 0 && D >= 1, "conv_attn_fwd: bad shape B=%d H=%d S=%d D=%d", B, H, S, D);
    MTA_REQUIRE(cq >= 1 && ck >= 1 && ck % 2 == 1, "conv_attn_fwd: kernel size %dx%d needs an odd key extent", cq, ck);
    if ((long)B * S == 0) return MTA_OK;
    MTA_REQUIRE(q && k && v && w && o, "conv_attn_fwd: null pointer");
    MTA_REQUIRE((long)B * H <= 65535, "conv_attn_fwd: B*H = %ld exceeds 65535", (long)B * H);
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (conv_attn_one_kernel(S, D, cq, ck, causal, dtype, w_dtype)) {
        MTA_REQUIRE(conv_attn_fused_supported(q, k, v, o, S, D, cq, ck, causal, dtype, w_dtype),
                    "conv_attn_fwd: q, k, v and o must be 16-byte aligned");
        // raw scores into the conv (score scale 1), the softmax scale after it, as the reference orders them
        return conv_attn_fused_launch(q, k, v, w, w_dtype, o, B, H, S, D, cq, ck, 1.0f, scale, 0, S, dtype, st);
    }
    const Plan pl = make_plan(B, H, S, cq, 1, 0, S, dtype);
    MTA_REQUIRE(workspace && workspace_bytes >= 2 * pl.buf_bytes, "conv_attn_fwd: workspace of %zu bytes is smaller than the %zu needed",
                workspace_bytes, 2 * pl.buf_bytes);
    MTA_REQUIRE(aligned16(workspace), "conv_attn_fwd: workspace must be 16-byte aligned");
    void* bufA = workspace;
    void* bufB = static_cast<char*>(workspace) + pl.buf_bytes;
    const PlaneView pv{(long)S * S, 0, S};
    const long planes = (long)B * H;
    int rc;
    // 16-bit dtypes: the raw scores are computed inside the conv's kernel (scale 1: the conv attention scales after its conv)
    if ((variant("fused") == 0 || variant("fused") == 2) && variant("gemm") == 0 && variant("conv2d") == 0 && planes <= 65535 &&
        qk_conv_supported(q, k, bufB, pv, S, D, cq, ck, causal, dtype, w_dtype)) {
        if ((rc = qk_conv_launch(q, k, w, w_dtype, bufB, pv, B, H, S, D, cq, ck, 1.0f, 0, S, dtype, st))) return rc;
    } else {
        if ((rc = qk_scores_launch(q, k, bufA, pv, B, H, S, D, 1.0f, 0, causal, 0, S, dtype, st))) return rc;
        if ((rc = conv2d_launch(bufA, pv, S, w, w_dtype, bufB, pv, planes, H, S, S, cq, ck, causal, 0, S, !causal, dtype, st))) return rc;
    }
    if ((rc = softmax_launch(bufB, pv, bufB, pv, planes, S, S, causal, 0, S, false, scale, dtype, st))) return rc;
    return pv_launch(bufB, pv, S, v, o, B, H, S, D, causal, 0, S, dtype, st);
}

}  // extern "C"
