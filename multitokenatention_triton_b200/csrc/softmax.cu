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

// Vector version for 16-bit dtypes with 16-byte aligned rows: a CTA of 128 threads owns one row and keeps it
// in registers as NCH chunks of 8 keys per thread (rows of up to NCH*1024 keys), so the row is read once with
// 16-byte loads and written once with 16-byte stores.
constexpr int VT = 128;

template <typename T> __device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]);
template <> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <> __device__ __forceinline__ void unpack8<__half>(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}
template <typename T> __device__ __forceinline__ uint32_t pack2s(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2s<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t pack2s<__half>(float lo, float hi) {
    __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}

template <typename T, int NCH>
__global__ void __launch_bounds__(VT)
softmax_rows_vec_kernel(const T* __restrict__ x, PlaneView xv, T* __restrict__ y, PlaneView yv, int Q, int causal,
                        int row_begin, int write_upper, float pre_scale, int round_prescaled) {
    __shared__ float red[2][VT / 32];
    const int p = row_begin + blockIdx.x;
    const long plane = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = causal ? min(p + 1, Q) : Q;
    const int nch = (n + 7) >> 3;                       // chunks that hold at least one valid key
    const uint4* xr = reinterpret_cast<const uint4*>(x + xv.at(plane, p, 0));
    uint4* yr = reinterpret_cast<uint4*>(y + yv.at(plane, p, 0));
    float v[NCH][8];
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int ch = tid + c * VT;
        if (ch < nch) {
            unpack8<T>(__ldg(xr + ch), v[c]);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float t = v[c][e] * pre_scale;
                if (round_prescaled) t = round_to<T>(t);
                if (ch * 8 + e >= n) t = -INFINITY;     // keys past the diagonal inside the last chunk
                v[c][e] = t;
                mx = fmaxf(mx, t);
            }
        }
    }
    mx = warp_max(mx);
    if (lane == 0) red[0][warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0][0], red[0][1]), fmaxf(red[0][2], red[0][3]));
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        if (tid + c * VT < nch) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float ex = __expf(v[c][e] - mx);   // exp(-inf) = 0 for the masked tail
                v[c][e] = ex;
                sum += ex;
            }
        }
    }
    sum = warp_sum(sum);
    if (lane == 0) red[1][warp] = sum;
    __syncthreads();
    const float inv = 1.0f / (red[1][0] + red[1][1] + red[1][2] + red[1][3]);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int ch = tid + c * VT;
        if (ch < nch) {
            uint4 o;
            o.x = pack2s<T>(v[c][0] * inv, v[c][1] * inv);
            o.y = pack2s<T>(v[c][2] * inv, v[c][3] * inv);
            o.z = pack2s<T>(v[c][4] * inv, v[c][5] * inv);
            o.w = pack2s<T>(v[c][6] * inv, v[c][7] * inv);
            if (!write_upper && ch * 8 + 8 > n) {       // last chunk: keys past the diagonal stay untouched
                T* dst = reinterpret_cast<T*>(yr + ch);
                const T* src = reinterpret_cast<const T*>(&o);
                for (int e = 0; e < 8; ++e)
                    if (ch * 8 + e < n) dst[e] = src[e];
            } else {
                yr[ch] = o;
            }
        }
    }
    if (write_upper)
        for (int ch = nch + tid; ch < (Q >> 3); ch += VT) yr[ch] = make_uint4(0u, 0u, 0u, 0u);
}

template <typename T, int NCH>
int launch_vec(const void* x, PlaneView xv, void* y, PlaneView yv, long planes, int Q, int causal, int row_begin,
               int row_end, bool write_upper, float pre_scale, int round_prescaled, cudaStream_t st) {
    dim3 grid((unsigned)(row_end - row_begin), (unsigned)planes);
    softmax_rows_vec_kernel<T, NCH><<<grid, VT, 0, st>>>(static_cast<const T*>(x), xv, static_cast<T*>(y), yv, Q, causal,
                                                        row_begin, write_upper ? 1 : 0, pre_scale, round_prescaled);
    MTA_LAUNCH_OK("softmax_rows_vec_kernel");
    return MTA_OK;
}

template <typename T>
int launch(const void* x, PlaneView xv, void* y, PlaneView yv, long planes, int Q, int causal, int row_begin,
           int row_end, bool write_upper, float pre_scale, int round_prescaled, cudaStream_t st) {
    if constexpr (sizeof(T) == 2) if (Q % 8 == 0 && Q <= 16 * 8 * VT && xv.plane_stride % 8 == 0 && yv.plane_stride % 8 == 0 &&
        xv.width % 8 == 0 && yv.width % 8 == 0 && aligned16(x) && aligned16(y)) {
        const int longest = causal ? (row_end < Q ? row_end : Q) : Q;
        const int need = (longest + 8 * VT - 1) / (8 * VT);
        if (need <= 1) return launch_vec<T, 1>(x, xv, y, yv, planes, Q, causal, row_begin, row_end, write_upper, pre_scale, round_prescaled, st);
        if (need <= 2) return launch_vec<T, 2>(x, xv, y, yv, planes, Q, causal, row_begin, row_end, write_upper, pre_scale, round_prescaled, st);
        if (need <= 4) return launch_vec<T, 4>(x, xv, y, yv, planes, Q, causal, row_begin, row_end, write_upper, pre_scale, round_prescaled, st);
        if (need <= 8) return launch_vec<T, 8>(x, xv, y, yv, planes, Q, causal, row_begin, row_end, write_upper, pre_scale, round_prescaled, st);
        return launch_vec<T, 16>(x, xv, y, yv, planes, Q, causal, row_begin, row_end, write_upper, pre_scale, round_prescaled, st);
    }
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
