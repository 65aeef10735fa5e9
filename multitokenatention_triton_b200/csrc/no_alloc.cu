// mta_conv_attn_fwd_static: the conv attention forward for callers that cannot give it scratch memory.
//
// Who needs this: code that runs where device allocation is off limits - a serving loop whose memory pool was
// sized and frozen at start-up, a plugin called from inside another framework's allocator callback, a host
// language binding that has no way to obtain device buffers of its own.  Most problems such a caller has (causal,
// 16-bit, D 64 or 128) run as one kernel that needs no scratch at all; for the others (float32, non-causal, key
// extents beyond 17) the two score-plane scratch buffers of mta_conv_attn_fwd live in a fixed array inside this
// library instead of a caller workspace.
//
// The array is a file-scope __device__ array, so every GPU that loads the library carries its 64 MiB until the
// process exits.  In host code the array's name is only a handle: the device address is obtained once per device
// with cudaGetSymbolAddress (with that device current) and cached.  That lookup is also the moment the CUDA runtime
// loads this module onto the device, which is when the 64 MiB are taken from the device's memory - so it belongs at
// start-up: call mta_static_scratch_prepare() on every device you will use, before the memory pool is frozen and
// before any stream capture.  A first mta_conv_attn_fwd_static call does the same lookup if it has not happened.
// The entry points call no cudaMalloc, cudaFree or other allocating routine.
//
// All calls share the one array and it keeps whatever the previous call left in it.  Nothing in it has to start
// at zero: every element the forward reads was written earlier in the same call, and stale values above the
// causal diagonal are masked before use.  Two calls that overlap on the GPU (different streams, or different host
// threads) would race on the array - serialise them.
#include <atomic>

#include "kernels.cuh"

namespace {

constexpr size_t kStaticScratchBytes = MTA_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of the array, per device ordinal.  Any host thread may fill a slot; two threads that race on the
// same slot store the same address, and the atomic makes each store and load indivisible.
std::atomic<unsigned char*> g_scratch_ptr[64];

int static_scratch_ptr(unsigned char** out) {
    int dev = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
    unsigned char* p = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!p) {
        MTA_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_static_scratch));
        g_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return MTA_OK;
}

}  // namespace

extern "C" {

size_t mta_static_scratch_bytes(void) { return kStaticScratchBytes; }

int mta_static_scratch_prepare(void) {
    mta::set_error("%s", "");
    unsigned char* p = nullptr;
    return static_scratch_ptr(&p);
}

int mta_conv_attn_fwd_static(const void* q, const void* k, const void* v, const void* w, void* o, int B, int H, int S,
                             int D, int cq, int ck, int causal, float scale, int dtype, int w_dtype, void* stream) {
    mta::set_error("%s", "");
    MTA_REQUIRE(mta::dtype_ok(dtype) && B >= 0 && H >= 1 && S >= 0 && D >= 1 && cq >= 1 && ck >= 1,
                "conv_attn_fwd_static: bad shape or dtype (B=%d H=%d S=%d D=%d cq=%d ck=%d dtype=%d)", B, H, S, D, cq, ck, dtype);
    if ((long)B * S == 0) return MTA_OK;
    const size_t need = mta_conv_attn_workspace_bytes(B, H, S, D, cq, ck, causal, dtype, w_dtype);
    MTA_REQUIRE(need <= kStaticScratchBytes,
                "conv_attn_fwd_static: B=%d H=%d S=%d needs %zu bytes of scratch, the built-in array holds %zu; "
                "use mta_conv_attn_fwd with a caller workspace for larger problems",
                B, H, S, need, kStaticScratchBytes);
    // the array belongs to the current device: a stream of another device would run the kernels there with this address
    int dev = 0, stream_dev = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_CUDA_OK(cudaStreamGetDevice(static_cast<cudaStream_t>(stream), &stream_dev));
    MTA_REQUIRE(stream_dev == dev, "conv_attn_fwd_static: the stream belongs to device %d but device %d is current", stream_dev, dev);
    unsigned char* scratch = nullptr;
    if (int rc = static_scratch_ptr(&scratch)) return rc;
    return mta_conv_attn_fwd(q, k, v, w, o, scratch, need, B, H, S, D, cq, ck, causal, scale, dtype, w_dtype, stream);
}

}  // extern "C"
