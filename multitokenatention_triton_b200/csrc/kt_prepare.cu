// Key-side filtering for the bilinear form of the score conv.
//
// Away from the causal band every tap of the depthwise conv reads an unmasked score, and the score is bilinear in
// (Q, K), so the key-direction taps can be moved into K once per forward:
//     conv(scale * Q K^T)[q, k] = sum_{i < cq} Q[q - (cq-1) + i] . Kt_i[k],
//     Kt_i[k] = scale * sum_{j < ck} w[h][i][j] * K[k + j - pad_w]        (K rows outside [0,S) are zero)
// This kernel writes Kt as (B*H*cq, S, D) in the activation dtype (fp32 accumulation, one rounding).
#include "kernels.cuh"

namespace mta {
namespace {

template <typename T> __device__ __forceinline__ void unpack8k(const uint4& v, float (&f)[8]);
template <> __device__ __forceinline__ void unpack8k<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <> __device__ __forceinline__ void unpack8k<__half>(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}
template <typename T> __device__ __forceinline__ uint32_t pk2k(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pk2k<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t pk2k<__half>(float lo, float hi) {
    __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}

constexpr int MAX_CQ = 8;

// One thread: one key row, 8 consecutive features, all cq outputs.
template <typename T>
__global__ void __launch_bounds__(256)
kt_prepare_kernel(const T* __restrict__ k, const void* __restrict__ w, int w_dtype, T* __restrict__ kt, int H, int S, int D,
                  int cq, int ck, float scale) {
    extern __shared__ float ws[];          // cq x ck weights of this head, pre-multiplied by scale
    const int bh = blockIdx.y, h = bh % H;
    for (int i = threadIdx.x; i < cq * ck; i += blockDim.x) ws[i] = scale * load_weight(w, (long)h * cq * ck + i, w_dtype);
    __syncthreads();
    const int chunks = D / 8;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int row = idx / chunks, ch = idx % chunks;
    if (row >= S) return;
    const int pad_w = (ck - 1) / 2;
    float acc[MAX_CQ][8];
#pragma unroll
    for (int i = 0; i < MAX_CQ; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[i][e] = 0.0f;
    const T* kb = k + (long)bh * S * D + ch * 8;
    for (int j = 0; j < ck; ++j) {
        const int kr = row + j - pad_w;
        if (kr < 0 || kr >= S) continue;
        float f[8];
        unpack8k<T>(__ldg(reinterpret_cast<const uint4*>(kb + (long)kr * D)), f);
#pragma unroll
        for (int i = 0; i < MAX_CQ; ++i) {
            if (i < cq) {
                const float wv = ws[i * ck + j];
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[i][e] = fmaf(wv, f[e], acc[i][e]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_CQ; ++i) {
        if (i < cq) {
            uint4 o;
            o.x = pk2k<T>(acc[i][0], acc[i][1]);
            o.y = pk2k<T>(acc[i][2], acc[i][3]);
            o.z = pk2k<T>(acc[i][4], acc[i][5]);
            o.w = pk2k<T>(acc[i][6], acc[i][7]);
            *reinterpret_cast<uint4*>(kt + (((long)bh * cq + i) * S + row) * D + ch * 8) = o;
        }
    }
}

}  // namespace

bool kt_supported(int cq, int ck, int D) { return cq >= 1 && cq <= MAX_CQ && D % 8 == 0 && ck >= 1; }

// kt: (B*H*cq, S, D) elements of the activation dtype.
int kt_prepare_launch(const void* k, const void* w, int w_dtype, void* kt, int B, int H, int S, int D, int cq, int ck, float scale,
                      int dtype, cudaStream_t st) {
    const int threads = 256;
    const long items = (long)S * (D / 8);
    dim3 grid((unsigned)((items + threads - 1) / threads), (unsigned)(B * H));
    const size_t smem = (size_t)cq * ck * sizeof(float);
    if (dtype == MTA_BF16)
        kt_prepare_kernel<__nv_bfloat16><<<grid, threads, smem, st>>>(static_cast<const __nv_bfloat16*>(k), w, w_dtype,
                                                                      static_cast<__nv_bfloat16*>(kt), H, S, D, cq, ck, scale);
    else
        kt_prepare_kernel<__half><<<grid, threads, smem, st>>>(static_cast<const __half*>(k), w, w_dtype, static_cast<__half*>(kt), H,
                                                               S, D, cq, ck, scale);
    MTA_LAUNCH_OK("kt_prepare_kernel");
    return MTA_OK;
}

}  // namespace mta
