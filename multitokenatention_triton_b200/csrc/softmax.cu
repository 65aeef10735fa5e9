// Row softmax of score planes over the keys that a query may see.
//
// Stands in for F.softmax(scores.float(), dim=-1).type_as(xq) in the reference's forward
// (mta_attention_triton.py:79): fp32 arithmetic, output in the input dtype, exactly 0 above the
// diagonal.  Only keys q <= p are read when causal, so the -inf fill the reference relies on need
// not exist in memory.  `pre_scale` multiplies the logits first (the conv-attention path scales after
// its conv, conv_attention_pytorch.py:63-64); in a 16-bit dtype the scaled logit is rounded to that
// dtype as the reference's tensor multiply does.
//
// One CTA per row.  The row is read once into shared memory as fp32 (rows of up to ROW_CACHE keys;
// longer rows are re-read from global memory), reduced for the maximum and the sum of exponentials,
// and written once.
#include "kernels.cuh"

namespace mta {
namespace {

constexpr int SM_THREADS = 256;
constexpr int ROW_CACHE = 16384;    // floats of shared memory used as the row cache (64 KB)

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T>
__global__ void __launch_bounds__(SM_THREADS)
softmax_rows_kernel(const T* __restrict__ x, PlaneView xv, T* __restrict__ y, PlaneView yv, int Q, int causal,
                    int row_begin, int write_upper, int cache_elems, float pre_scale, int round_prescaled) {
    extern __shared__ float row[];
    __shared__ float red[SM_THREADS / 32];
    const int p = row_begin + blockIdx.x;
    const long plane = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = causal ? min(p + 1, Q) : Q;
    const T* xr = x + xv.at(plane, p, 0);
    T* yr = y + yv.at(plane, p, 0);
    const bool cached = n <= cache_elems;

    float mx = -INFINITY;
    for (int k = tid; k < n; k += SM_THREADS) {
        float v = to_f32<T>(xr[k]) * pre_scale;
        if (round_prescaled) v = round_to<T>(v);
        if (cached) row[k] = v;
        mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int i = 1; i < SM_THREADS / 32; ++i) mx = fmaxf(mx, red[i]);
    __syncthreads();

    float sum = 0.0f;
    for (int k = tid; k < n; k += SM_THREADS) {
        float v;
        if (cached) v = row[k];
        else { v = to_f32<T>(xr[k]) * pre_scale; if (round_prescaled) v = round_to<T>(v); }
        const float e = (mx == -INFINITY) ? 0.0f : __expf(v - mx);
        if (cached) row[k] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = 0.0f;
#pragma unroll
    for (int i = 0; i < SM_THREADS / 32; ++i) sum += red[i];
    const float inv = 1.0f / sum;

    // x may alias y: every thread re-reads only the elements it writes.
    for (int k = tid; k < n; k += SM_THREADS) {
        float e;
        if (cached) e = row[k];
        else { float v = to_f32<T>(xr[k]) * pre_scale; if (round_prescaled) v = round_to<T>(v); e = __expf(v - mx); }
        yr[k] = from_f32<T>(e * inv);
    }
    if (write_upper)
        for (int k = n + tid; k < Q; k += SM_THREADS) yr[k] = from_f32<T>(0.0f);
}

template <typename T>
int launch(const void* x, PlaneView xv, void* y, PlaneView yv, long planes, int Q, int causal, int row_begin,
           int row_end, bool write_upper, float pre_scale, int round_prescaled, cudaStream_t st) {
    const int cache = Q < ROW_CACHE ? Q : ROW_CACHE;
    const size_t smem = (size_t)cache * sizeof(float);
    if (smem > 48 * 1024)
        MTA_CUDA_OK(cudaFuncSetAttribute(softmax_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)(row_end - row_begin), (unsigned)planes);
    softmax_rows_kernel<T><<<grid, SM_THREADS, smem, st>>>(static_cast<const T*>(x), xv, static_cast<T*>(y), yv, Q, causal,
                                                           row_begin, write_upper ? 1 : 0, cache, pre_scale, round_prescaled);
    MTA_LAUNCH_OK("softmax_rows_kernel");
    return MTA_OK;
}

}  // namespace

int softmax_launch(const void* x, PlaneView xv, void* y, PlaneView yv, long planes, int P, int Q, int causal,
                   int row_begin, int row_end, bool write_upper, float pre_scale, int dtype, cudaStream_t st) {
    (void)P;
    if (planes == 0 || row_end <= row_begin || Q == 0) return MTA_OK;
    MTA_REQUIRE(planes <= 65535, "softmax: N*C = %ld exceeds 65535", planes);
    switch (dtype) {
        case MTA_F32: return launch<float>(x, xv, y, yv, planes, Q, causal, row_begin, row_end, write_upper, pre_scale, (dtype != MTA_F32 && pre_scale != 1.0f) ? 1 : 0, st);
        case MTA_BF16: return launch<__nv_bfloat16>(x, xv, y, yv, planes, Q, causal, row_begin, row_end, write_upper, pre_scale, (dtype != MTA_F32 && pre_scale != 1.0f) ? 1 : 0, st);
        default: return launch<__half>(x, xv, y, yv, planes, Q, causal, row_begin, row_end, write_upper, pre_scale, (dtype != MTA_F32 && pre_scale != 1.0f) ? 1 : 0, st);
    }
}

}  // namespace mta
