// C ABI of the library: argument validation, error text, and dispatch to the kernel launchers.
// See include/mta_b200.h for the contract of every entry point.
#include <atomic>
#include <cstring>
#include <string>

#include "kernels.cuh"

namespace mta {
namespace {
thread_local char g_error[512] = "";
thread_local long g_launches = 0;
// Kernel selection for tests and measurements: process-wide, read on every launch, written by mta_set_variant from any
// thread (relaxed atomics: a launch sees either the old or the new value of each key, never a torn one).
std::atomic<int> g_variant_head_linear{0}, g_variant_conv2d{0}, g_variant_gemm{0}, g_variant_fused{0}, g_variant_mix_softmax{0};
}  // namespace

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

void count_launch(int n) { g_launches += n; }

int variant(const char* key) {
    if (!strcmp(key, "head_linear")) return g_variant_head_linear.load(std::memory_order_relaxed);
    if (!strcmp(key, "conv2d")) return g_variant_conv2d.load(std::memory_order_relaxed);
    if (!strcmp(key, "gemm")) return g_variant_gemm.load(std::memory_order_relaxed);
    if (!strcmp(key, "fused")) return g_variant_fused.load(std::memory_order_relaxed);
    if (!strcmp(key, "mix_softmax")) return g_variant_mix_softmax.load(std::memory_order_relaxed);
    return 0;
}

int check_device() {
    int dev = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    int major = 0;
    MTA_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) {
        set_error("device %d has compute capability %d.x; this library is built for sm_100a only", dev, major);
        return MTA_ERR_ARCH;
    }
    if (wait_flag_raised()) {
        set_error("a bounded wait of an earlier kernel on device %d gave up: every kernel since then has returned without "
                  "computing; mta_device_status() reports and clears the condition", dev);
        return MTA_ERR_TIMEOUT;
    }
    return MTA_OK;
}

PlaneView full_view(int rows, int cols) { return PlaneView{(long)rows * cols, 0, cols}; }

}  // namespace mta

using namespace mta;

extern "C" {

int mta_abi_version(void) { return 2; }

const char* mta_last_error(void) { return g_error; }

long mta_launch_count(void) { return g_launches; }
void mta_reset_launch_count(void) { g_launches = 0; }

int mta_set_variant(const char* key, int value) {
    if (!key || value < 0 || value > 3) return MTA_ERR_INVALID;
    if (!strcmp(key, "head_linear")) g_variant_head_linear.store(value, std::memory_order_relaxed);
    else if (!strcmp(key, "conv2d")) g_variant_conv2d.store(value, std::memory_order_relaxed);
    else if (!strcmp(key, "gemm")) g_variant_gemm.store(value, std::memory_order_relaxed);
    else if (!strcmp(key, "fused")) g_variant_fused.store(value, std::memory_order_relaxed);
    else if (!strcmp(key, "mix_softmax")) g_variant_mix_softmax.store(value, std::memory_order_relaxed);
    else return MTA_ERR_INVALID;
    return MTA_OK;
}

int mta_conv2d_fwd(const void* x, const void* w, void* y, int N, int C, int H, int W, int R, int S, int causal,
                   int x_dtype, int w_dtype, void* stream) {
    g_error[0] = 0;
    MTA_REQUIRE(dtype_ok(x_dtype) && dtype_ok(w_dtype), "conv2d: unknown dtype code (x %d, w %d)", x_dtype, w_dtype);
    MTA_REQUIRE(N >= 0 && C >= 1 && H >= 0 && W >= 0, "conv2d: bad shape N=%d C=%d H=%d W=%d", N, C, H, W);
    MTA_REQUIRE(R >= 1 && S >= 1, "conv2d: kernel size %dx%d must be positive", R, S);
    if ((long)N * H * W == 0) return MTA_OK;
    MTA_REQUIRE(x && w && y, "conv2d: null pointer");
    MTA_REQUIRE(x != y, "conv2d: in-place operation is not supported");
    if (int rc = check_device()) return rc;
    const PlaneView v = full_view(H, W);
    return conv2d_launch(x, v, H, w, w_dtype, y, v, (long)N * C, C, H, W, R, S, causal ? 1 : 0, 0, H, true, x_dtype,
                         static_cast<cudaStream_t>(stream));
}

int mta_head_linear_fwd(const void* x, const void* Wm, void* y, int N, int C, int P, int Q, int causal, float fill,
                        int x_dtype, int w_dtype, void* stream) {
    g_error[0] = 0;
    MTA_REQUIRE(dtype_ok(x_dtype) && dtype_ok(w_dtype), "head_linear: unknown dtype code (x %d, w %d)", x_dtype, w_dtype);
    MTA_REQUIRE(N >= 0 && C >= 1 && P >= 0 && Q >= 0, "head_linear: bad shape N=%d C=%d P=%d Q=%d", N, C, P, Q);
    if ((long)N * P * Q == 0) return MTA_OK;
    MTA_REQUIRE(x && Wm && y, "head_linear: null pointer");
    MTA_REQUIRE(x != y, "head_linear: in-place operation is not supported");
    if (int rc = check_device()) return rc;
    const PlaneView v = full_view(P, Q);
    return head_linear_launch(x, v, Wm, w_dtype, y, v, N, C, P, Q, causal ? 1 : 0, fill, 0, P, true, x_dtype,
                              static_cast<cudaStream_t>(stream));
}

int mta_softmax_fwd(const void* x, void* y, int N, int C, int P, int Q, int causal, int dtype, void* stream) {
    g_error[0] = 0;
    MTA_REQUIRE(dtype_ok(dtype), "softmax: unknown dtype code %d", dtype);
    MTA_REQUIRE(N >= 0 && C >= 1 && P >= 0 && Q >= 0, "softmax: bad shape N=%d C=%d P=%d Q=%d", N, C, P, Q);
    if ((long)N * P * Q == 0) return MTA_OK;
    MTA_REQUIRE(x && y, "softmax: null pointer");
    if (int rc = check_device()) return rc;
    const PlaneView v = full_view(P, Q);
    return softmax_launch(x, v, y, v, (long)N * C, P, Q, causal ? 1 : 0, 0, P, true, 1.0f, dtype,
                          static_cast<cudaStream_t>(stream));
}

int mta_head_linear_softmax_fwd(const void* x, const void* Wm, void* y, int N, int C, int P, int Q, int x_dtype, int w_dtype,
                                void* stream) {
    g_error[0] = 0;
    MTA_REQUIRE(dtype_ok(x_dtype) && dtype_ok(w_dtype), "head_linear_softmax: unknown dtype code (x %d, w %d)", x_dtype, w_dtype);
    MTA_REQUIRE(N >= 0 && C >= 1 && P >= 0 && Q >= 0, "head_linear_softmax: bad shape N=%d C=%d P=%d Q=%d", N, C, P, Q);
    if ((long)N * P * Q == 0) return MTA_OK;
    MTA_REQUIRE(x && Wm && y, "head_linear_softmax: null pointer");
    MTA_REQUIRE(x != y, "head_linear_softmax: in-place operation is not supported");
    if (int rc = check_device()) return rc;
    const PlaneView v = full_view(P, Q);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (variant("fused") != 1 && head_mix_softmax_supported(x, v, y, v, C, Q, 1, x_dtype, w_dtype))
        return head_mix_softmax_launch(x, v, Wm, w_dtype, y, v, N, C, Q, 0, P, true, x_dtype, st);
    // shapes the one-pass kernel does not take: the two stages, the softmax in place
    if (int rc = head_linear_launch(x, v, Wm, w_dtype, y, v, N, C, P, Q, 1, 0.0f, 0, P, false, x_dtype, st)) return rc;
    return softmax_launch(y, v, y, v, (long)N * C, P, Q, 1, 0, P, true, 1.0f, x_dtype, st);
}

int mta_conv2d_bwd_input(const void* dy, const void* w, void* dx, int N, int C, int H, int W, int R, int S, int causal,
                         int dtype, int w_dtype, void* stream) {
    g_error[0] = 0;
    MTA_REQUIRE(dtype_ok(dtype) && dtype_ok(w_dtype), "conv2d_bwd_input: unknown dtype code (dy %d, w %d)", dtype, w_dtype);
    MTA_REQUIRE(N >= 0 && C >= 1 && H >= 0 && W >= 0, "conv2d_bwd_input: bad shape N=%d C=%d H=%d W=%d", N, C, H, W);
    MTA_REQUIRE(R >= 1 && S >= 1, "conv2d_bwd_input: kernel size %dx%d must be positive", R, S);
    if ((long)N * H * W == 0) return MTA_OK;
    MTA_REQUIRE(dy && w && dx, "conv2d_bwd_input: null pointer");
    MTA_REQUIRE(dy != dx, "conv2d_bwd_input: in-place operation is not supported");
    if (int rc = check_device()) return rc;
    return conv2d_bwd_input_launch(dy, w, w_dtype, dx, (long)N * C, C, H, W, R, S, causal ? 1 : 0, dtype,
                                   static_cast<cudaStream_t>(stream));
}

size_t mta_conv2d_bwd_weight_workspace_bytes(int N, int C, int H, int W, int R, int S) {
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || R < 1 || S < 1) return 0;
    return conv2d_bwd_weight_workspace(N, C, H, W, R, S);
}

int mta_conv2d_bwd_weight(const void* x, const void* dy, float* dw, void* workspace, size_t workspace_bytes, int N, int C,
                          int H, int W, int R, int S, int causal, int dtype, void* stream) {
    g_error[0] = 0;
    MTA_REQUIRE(dtype_ok(dtype), "conv2d_bwd_weight: unknown dtype code %d", dtype);
    MTA_REQUIRE(N >= 0 && C >= 1 && H >= 0 && W >= 0, "conv2d_bwd_weight: bad shape N=%d C=%d H=%d W=%d", N, C, H, W);
    MTA_REQUIRE(R >= 1 && S >= 1, "conv2d_bwd_weight: kernel size %dx%d must be positive", R, S);
    MTA_REQUIRE(dw, "conv2d_bwd_weight: null pointer");
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if ((long)N * H * W == 0) {
        MTA_CUDA_OK(cudaMemsetAsync(dw, 0, (size_t)C * R * S * sizeof(float), st));
        return MTA_OK;
    }
    MTA_REQUIRE(x && dy, "conv2d_bwd_weight: null pointer");
    const size_t need = conv2d_bwd_weight_workspace(N, C, H, W, R, S);
    MTA_REQUIRE(workspace && workspace_bytes >= need, "conv2d_bwd_weight: workspace of %zu bytes is smaller than the %zu needed",
                workspace_bytes, need);
    return conv2d_bwd_weight_launch(x, dy, dw, workspace, N, C, H, W, R, S, causal ? 1 : 0, dtype, st);
}

int mta_head_linear_bwd_input(const void* dy, const void* Wm, void* dx, int N, int C, int P, int Q, int causal, int dtype,
                              int w_dtype, void* stream) {
    g_error[0] = 0;
    MTA_REQUIRE(dtype_ok(dtype) && dtype_ok(w_dtype), "head_linear_bwd_input: unknown dtype code (dy %d, w %d)", dtype, w_dtype);
    MTA_REQUIRE(N >= 0 && C >= 1 && P >= 0 && Q >= 0, "head_linear_bwd_input: bad shape N=%d C=%d P=%d Q=%d", N, C, P, Q);
    if ((long)N * P * Q == 0) return MTA_OK;
    MTA_REQUIRE(dy && Wm && dx, "head_linear_bwd_input: null pointer");
    MTA_REQUIRE(dy != dx, "head_linear_bwd_input: in-place operation is not supported");
    if (int rc = check_device()) return rc;
    const PlaneView v = full_view(P, Q);
    return head_linear_launch(dy, v, Wm, w_dtype, dx, v, N, C, P, Q, causal ? 1 : 0, 0.0f, 0, P, true, dtype,
                              static_cast<cudaStream_t>(stream), true);
}

size_t mta_head_linear_bwd_weight_workspace_bytes(int C) {
    if (C < 1 || C > 128) return 0;
    return head_linear_bwd_weight_workspace(C);
}

int mta_head_linear_bwd_weight(const void* x, const void* dy, float* dW, void* workspace, size_t workspace_bytes, int N,
                               int C, int P, int Q, int causal, int dtype, void* stream) {
    g_error[0] = 0;
    MTA_REQUIRE(dtype_ok(dtype), "head_linear_bwd_weight: unknown dtype code %d", dtype);
    MTA_REQUIRE(N >= 0 && C >= 1 && C <= 128 && P >= 0 && Q >= 0, "head_linear_bwd_weight: bad shape N=%d C=%d P=%d Q=%d", N, C, P, Q);
    MTA_REQUIRE(dW, "head_linear_bwd_weight: null pointer");
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if ((long)N * P * Q == 0) {
        MTA_CUDA_OK(cudaMemsetAsync(dW, 0, (size_t)C * C * sizeof(float), st));
        return MTA_OK;
    }
    MTA_REQUIRE(x && dy, "head_linear_bwd_weight: null pointer");
    const size_t need = head_linear_bwd_weight_workspace(C);
    MTA_REQUIRE(workspace && workspace_bytes >= need, "head_linear_bwd_weight: workspace of %zu bytes is smaller than the %zu needed",
                workspace_bytes, need);
    return head_linear_bwd_weight_launch(x, dy, dW, workspace, N, C, P, Q, causal ? 1 : 0, dtype, st);
}

int mta_qk_scores_fwd(const void* q, const void* k, void* s, int B, int H, int S, int D, float scale, int round_scale,
                      int causal, int dtype, void* stream) {
    g_error[0] = 0;
    MTA_REQUIRE(dtype_ok(dtype), "qk_scores: unknown dtype code %d", dtype);
    MTA_REQUIRE(B >= 0 && H >= 1 && S >= 0 && D >= 1, "qk_scores: bad shape B=%d H=%d S=%d D=%d", B, H, S, D);
    if ((long)B * S == 0) return MTA_OK;
    MTA_REQUIRE(q && k && s, "qk_scores: null pointer");
    MTA_REQUIRE((long)B * H <= 65535, "qk_scores: B*H = %ld exceeds 65535", (long)B * H);
    if (int rc = check_device()) return rc;
    return qk_scores_launch(q, k, s, full_view(S, S), B, H, S, D, scale, round_scale, causal ? 1 : 0, 0, S, dtype,
                            static_cast<cudaStream_t>(stream));
}

int mta_pv_fwd(const void* p, const void* v, void* o, int B, int H, int S, int D, int causal, int dtype, void* stream) {
    g_error[0] = 0;
    MTA_REQUIRE(dtype_ok(dtype), "pv: unknown dtype code %d", dtype);
    MTA_REQUIRE(B >= 0 && H >= 1 && S >= 0 && D >= 1, "pv: bad shape B=%d H=%d S=%d D=%d", B, H, S, D);
    if ((long)B * S == 0) return MTA_OK;
    MTA_REQUIRE(p && v && o, "pv: null pointer");
    MTA_REQUIRE((long)B * H <= 65535, "pv: B*H = %ld exceeds 65535", (long)B * H);
    if (int rc = check_device()) return rc;
    return pv_launch(p, full_view(S, S), S, v, o, B, H, S, D, causal ? 1 : 0, 0, S, dtype, static_cast<cudaStream_t>(stream));
}

int mta_device_status(void* stream) {
    g_error[0] = 0;
    int timed_out = 0;
    if (int rc = device_wait_status(static_cast<cudaStream_t>(stream), &timed_out)) return rc;
    if (timed_out) {
        set_error("a device-side bounded wait (mbarrier) gave up: results of the kernels launched since the last check are invalid");
        return MTA_ERR_TIMEOUT;
    }
    return MTA_OK;
}

int mta_inject_wait_timeout(void* stream) {
    g_error[0] = 0;
    return wait_flag_inject(static_cast<cudaStream_t>(stream));
}

}  // extern "C"
