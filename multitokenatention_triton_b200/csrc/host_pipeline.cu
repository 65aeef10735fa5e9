// Full MTA forward for callers whose tensors live in HOST memory.
//
// mta_fused_fwd_host splits the batch into chunks and runs three CUDA streams: chunk c+1 travels host -> device
// while chunk c is computed and chunk c-1 travels device -> host, so a forward costs about what the slower of the
// PCIe transfer and the GPU work costs, not their sum.  Device staging (two slots of q, k, v and o), the scratch
// planes of one chunk, the streams and the events are created on first use and kept per device (grown when a
// larger call arrives) until mta_host_pipeline_release().
//
// What it stands in for: a caller of MTAAttentionTriton.forward (mta_attention_triton.py:61-92) that holds its
// activations on the host and would otherwise pay .cuda() / forward / .cpu() back to back.
#include <mutex>

#include "kernels.cuh"

namespace mta {
namespace {

struct HostPipe {
    bool made = false;
    cudaStream_t s_in = nullptr, s_comp = nullptr, s_out = nullptr;
    cudaEvent_t in_done[2] = {nullptr, nullptr}, comp_done[2] = {nullptr, nullptr}, out_done[2] = {nullptr, nullptr};
    char* stage = nullptr;          // 2 slots x (q, k, v, o) of one chunk
    size_t stage_bytes = 0;
    char* ws = nullptr;             // scratch planes of one chunk
    size_t ws_bytes = 0;
};

constexpr int MAX_DEVICES = 64;
HostPipe g_pipe[MAX_DEVICES];
std::mutex g_pipe_mutex;

int pipe_make(HostPipe& p) {
    if (p.made) return MTA_OK;
    MTA_CUDA_OK(cudaStreamCreateWithFlags(&p.s_in, cudaStreamNonBlocking));
    MTA_CUDA_OK(cudaStreamCreateWithFlags(&p.s_comp, cudaStreamNonBlocking));
    MTA_CUDA_OK(cudaStreamCreateWithFlags(&p.s_out, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
        MTA_CUDA_OK(cudaEventCreateWithFlags(&p.in_done[i], cudaEventDisableTiming));
        MTA_CUDA_OK(cudaEventCreateWithFlags(&p.comp_done[i], cudaEventDisableTiming));
        MTA_CUDA_OK(cudaEventCreateWithFlags(&p.out_done[i], cudaEventDisableTiming));
    }
    p.made = true;
    return MTA_OK;
}

int pipe_grow(char*& buf, size_t& have, size_t need) {
    if (need <= have) return MTA_OK;
    if (buf) MTA_CUDA_OK(cudaFree(buf));
    buf = nullptr;
    have = 0;
    MTA_CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&buf), need));
    have = need;
    return MTA_OK;
}

size_t round256(size_t n) { return (n + 255) & ~size_t(255); }

}  // namespace
}  // namespace mta

using namespace mta;

extern "C" {

int mta_host_pipeline_release(void) {
    std::lock_guard<std::mutex> lock(g_pipe_mutex);
    int dev = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "host pipeline: device index %d is out of range", dev);
    HostPipe& p = g_pipe[dev];
    if (p.stage) MTA_CUDA_OK(cudaFree(p.stage));
    if (p.ws) MTA_CUDA_OK(cudaFree(p.ws));
    if (p.made) {
        cudaStreamDestroy(p.s_in);
        cudaStreamDestroy(p.s_comp);
        cudaStreamDestroy(p.s_out);
        for (int i = 0; i < 2; ++i) {
            cudaEventDestroy(p.in_done[i]);
            cudaEventDestroy(p.comp_done[i]);
            cudaEventDestroy(p.out_done[i]);
        }
    }
    p = HostPipe();
    return MTA_OK;
}

int mta_fused_fwd_host(const void* q, const void* k, const void* v, const void* w1, const void* W1, const void* w2,
                       const void* W2, void* o, int B, int H, int S, int D, int cq, int ck, int cq2, int ck2, int causal,
                       int dtype, int w_dtype, int chunk_batch) {
    set_error("%s", "");
    MTA_REQUIRE(dtype_ok(dtype) && dtype_ok(w_dtype), "fused_fwd_host: unknown dtype code (%d, %d)", dtype, w_dtype);
    MTA_REQUIRE(B >= 0 && H >= 1 && S >= 0 && D >= 1, "fused_fwd_host: bad shape B=%d H=%d S=%d D=%d", B, H, S, D);
    MTA_REQUIRE(chunk_batch >= 0, "fused_fwd_host: chunk_batch = %d must not be negative", chunk_batch);
    if ((long)B * S == 0) return MTA_OK;
    MTA_REQUIRE(q && k && v && w1 && W1 && w2 && W2 && o, "fused_fwd_host: null pointer");
    if (int rc = check_device()) return rc;
    int dev = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "fused_fwd_host: device index %d is out of range", dev);
    std::lock_guard<std::mutex> lock(g_pipe_mutex);
    HostPipe& p = g_pipe[dev];
    if (int rc = pipe_make(p)) return rc;

    // default chunk: one batch element, unless that leaves the GPU short of work (small S): aim at >= 8 chunks
    int cb = chunk_batch > 0 ? chunk_batch : (B >= 8 ? B / 8 : 1);
    if (cb > B) cb = B;
    const size_t per_b = (size_t)H * S * D * dtype_size(dtype);      // bytes of one batch element of q, k, v or o
    const size_t slot = 4 * round256(per_b * cb);
    const size_t ws_need = mta_workspace_bytes(cb, H, S, D, cq, ck, cq2, ck2, 0, S, dtype);
    MTA_REQUIRE(ws_need > 0, "fused_fwd_host: bad kernel sizes %dx%d / %dx%d", cq, ck, cq2, ck2);
    if (int rc = pipe_grow(p.stage, p.stage_bytes, 2 * slot)) return rc;
    if (int rc = pipe_grow(p.ws, p.ws_bytes, ws_need)) return rc;

    const char* hq = static_cast<const char*>(q);
    const char* hk = static_cast<const char*>(k);
    const char* hv = static_cast<const char*>(v);
    char* ho = static_cast<char*>(o);
    int c = 0;
    for (int b0 = 0; b0 < B; b0 += cb, ++c) {
        const int nb = b0 + cb <= B ? cb : B - b0;
        const int s = c & 1;
        const size_t bytes = per_b * nb, off = per_b * b0;
        char* dq = p.stage + s * slot;
        char* dk = dq + round256(per_b * cb);
        char* dv = dk + round256(per_b * cb);
        char* dout = dv + round256(per_b * cb);
        // the slot's inputs are free once the forward of chunk c - 2 has read them
        if (c >= 2) MTA_CUDA_OK(cudaStreamWaitEvent(p.s_in, p.comp_done[s], 0));
        MTA_CUDA_OK(cudaMemcpyAsync(dq, hq + off, bytes, cudaMemcpyHostToDevice, p.s_in));
        MTA_CUDA_OK(cudaMemcpyAsync(dk, hk + off, bytes, cudaMemcpyHostToDevice, p.s_in));
        MTA_CUDA_OK(cudaMemcpyAsync(dv, hv + off, bytes, cudaMemcpyHostToDevice, p.s_in));
        MTA_CUDA_OK(cudaEventRecord(p.in_done[s], p.s_in));
        MTA_CUDA_OK(cudaStreamWaitEvent(p.s_comp, p.in_done[s], 0));
        // the slot's output is free once chunk c - 2 has been copied out
        if (c >= 2) MTA_CUDA_OK(cudaStreamWaitEvent(p.s_comp, p.out_done[s], 0));
        if (int rc = mta_fused_fwd(dq, dk, dv, w1, W1, w2, W2, dout, p.ws, p.ws_bytes, nb, H, S, D, cq, ck, cq2, ck2, 0, S, causal,
                                   dtype, w_dtype, p.s_comp))
            return rc;
        MTA_CUDA_OK(cudaEventRecord(p.comp_done[s], p.s_comp));
        MTA_CUDA_OK(cudaStreamWaitEvent(p.s_out, p.comp_done[s], 0));
        MTA_CUDA_OK(cudaMemcpyAsync(ho + off, dout, bytes, cudaMemcpyDeviceToHost, p.s_out));
        MTA_CUDA_OK(cudaEventRecord(p.out_done[s], p.s_out));
    }
    MTA_CUDA_OK(cudaStreamSynchronize(p.s_out));
    MTA_CUDA_OK(cudaStreamSynchronize(p.s_comp));
    return mta_device_status(p.s_comp);
}

}  // extern "C"
