// Weight gradients of the two stand-alone ops (the input gradients reuse the forward kernels: conv2d.cu with the
// taps reversed and the rows looking forward, head_linear.cu with the weight read transposed).
//
//   conv2d_bwd_weight    dw[c,r,s] = sum_{n,q,k} xh[n,c,q+r-(R-1),k+s-(S-1)/2] * dyh[n,c,q,k]
//                        (reference: conv_bwd_weight_kernel, convolution_2d_trit.py:226-295); xh / dyh are x / dy inside
//                        the plane and, when causal, where key <= query, 0 elsewhere
//   head_linear_bwd_weight  dW[o,h] = sum_{n,p,q<=p} dy[n,o,p,q] * x[n,h,p,q]
//                        (reference: linear_head_kernel_backward_weight, triton_linear_head.py:210-278)
//
// Both reduce over every position of every plane.  The reference accumulates with floating-point atomics; here each
// CTA writes its partial sums to a workspace and a second kernel adds them in a fixed order in double precision, so
// the result does not depend on scheduling.
#include "kernels.cuh"

namespace mta {
namespace {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ------------------------------------------------------------------------------------------------
constexpr int WT_M = 32, WT_N = 128, WT_CPT = 8;
constexpr int WT_THREADS = WT_M * (WT_N / WT_CPT) / 2;     // 256: a thread owns 2 rows x 8 columns of output positions

template <typename T>
__global__ void __launch_bounds__(WT_THREADS)
conv2d_bwd_weight_kernel(const T* __restrict__ x, const T* __restrict__ dy, float* __restrict__ partial, int H, int W,
                         int R, int S, int causal, int tiles_n) {
    extern __shared__ __align__(16) float smem[];
    const int pad_h = R - 1, pad_w = (S - 1) / 2;
    const int tw = WT_N + S - 1, th = WT_M + R - 1;
    float* xs = smem;                               // th x tw, masked input
    float* part = smem + th * tw;                   // (WT_THREADS / 32) x R*S warp partials
    const long plane = blockIdx.y;
    const int tile_m = blockIdx.x / tiles_n, tile_n = blockIdx.x % tiles_n;
    const int m0 = tile_m * WT_M, n0 = tile_n * WT_N;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int taps = R * S;
    float* out = partial + ((long)plane * gridDim.x + blockIdx.x) * taps;
    if (causal && n0 > min(m0 + WT_M, H) - 1) {     // every dy of the tile is masked
        for (int i = tid; i < taps; i += WT_THREADS) out[i] = 0.0f;
        return;
    }
    const T* xp = x + plane * (long)H * W;
    const T* dp = dy + plane * (long)H * W;
    for (int idx = tid; idx < th * tw; idx += WT_THREADS) {
        const int rr = idx / tw, cc = idx - rr * tw;
        const int qq = m0 - pad_h + rr, kk = n0 - pad_w + cc;
        float v = 0.0f;
        if (qq >= 0 && qq < H && kk >= 0 && kk < W && (!causal || kk <= qq)) v = to_f32<T>(xp[(long)qq * W + kk]);
        xs[idx] = v;
    }
    // this thread's output positions: rows (ry, ry + WT_M/2), columns [cx, cx + 8)
    const int ry = tid / (WT_N / WT_CPT), cx = (tid % (WT_N / WT_CPT)) * WT_CPT;
    float g0[WT_CPT], g1[WT_CPT];
#pragma unroll
    for (int e = 0; e < WT_CPT; ++e) {
        const int k = n0 + cx + e, q0 = m0 + ry, q1 = m0 + ry + WT_M / 2;
        g0[e] = (q0 < H && k < W && (!causal || k <= q0)) ? to_f32<T>(dp[(long)q0 * W + k]) : 0.0f;
        g1[e] = (q1 < H && k < W && (!causal || k <= q1)) ? to_f32<T>(dp[(long)q1 * W + k]) : 0.0f;
    }
    __syncthreads();
    for (int i = 0; i < R; ++i) {
        const float* r0 = xs + (ry + i) * tw + cx;
        const float* r1 = xs + (ry + WT_M / 2 + i) * tw + cx;
        for (int j = 0; j < S; ++j) {
            float v = 0.0f;
#pragma unroll
            for (int e = 0; e < WT_CPT; ++e) v = fmaf(r0[j + e], g0[e], fmaf(r1[j + e], g1[e], v));
            v = warp_sum_f(v);
            if (lane == 0) part[warp * taps + i * S + j] = v;
        }
    }
    __syncthreads();
    for (int i = tid; i < taps; i += WT_THREADS) {
        float v = 0.0f;
#pragma unroll
        for (int wv = 0; wv < WT_THREADS / 32; ++wv) v += part[wv * taps + i];
        out[i] = v;
    }
}

// dw[c, tap] = sum over the planes of channel c and their tiles, in a fixed order, in double.
__global__ void conv2d_bwd_weight_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int N, int C,
                                                int tiles, int taps) {
    __shared__ double red[256];
    const int c = blockIdx.x / taps, tap = blockIdx.x % taps;
    double acc = 0.0;
    const long per_channel = (long)N * tiles;
    for (long i = threadIdx.x; i < per_channel; i += blockDim.x) {
        const long n = i / tiles, tile = i - n * tiles;
        acc += (double)partial[((n * C + c) * tiles + tile) * taps + tap];
    }
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) dw[blockIdx.x] = (float)red[0];
}

// ------------------------------------------------------------------------------------------------
constexpr int HW_THREADS = 256;

// PPT = (o,h) pairs per thread; KT = keys per tile.  Persistent CTAs walk the (n, row, key block) tiles.
template <typename T, int PPT, int KT>
__global__ void __launch_bounds__(HW_THREADS)
head_linear_bwd_weight_kernel(const T* __restrict__ x, const T* __restrict__ dy, float* __restrict__ partial, int N, int C,
                              int P, int Q, int causal) {
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;                   // C x KT
    float* gs = smem + (size_t)C * KT;  // C x KT
    const int tid = threadIdx.x;
    const int pairs = C * C;
    float acc[PPT];
#pragma unroll
    for (int i = 0; i < PPT; ++i) acc[i] = 0.0f;
    const int kblocks = (Q + KT - 1) / KT;
    const long tiles = (long)N * P * kblocks;
    for (long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int kb = (int)(tile % kblocks);
        const int p = (int)((tile / kblocks) % P);
        const long n = tile / ((long)kblocks * P);
        const int k0 = kb * KT;
        if (causal && k0 > p) continue;
        __syncthreads();                // the previous tile's reads are done
        for (int idx = tid; idx < C * KT; idx += HW_THREADS) {
            const int h = idx / KT, kk = idx - h * KT, k = k0 + kk;
            const bool ok = k < Q && (!causal || k <= p);
            const long off = ((n * C + h) * P + p) * (long)Q + k;
            xs[idx] = ok ? to_f32<T>(x[off]) : 0.0f;
            gs[idx] = ok ? to_f32<T>(dy[off]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < PPT; ++i) {
            const int pair = tid + i * HW_THREADS;
            if (pair >= pairs) break;
            const int o = pair / C, h = pair - o * C;
            const float4* a = reinterpret_cast<const float4*>(gs + (size_t)o * KT);
            const float4* b = reinterpret_cast<const float4*>(xs + (size_t)h * KT);
            float v = acc[i];
#pragma unroll 4
            for (int k4 = 0; k4 < KT / 4; ++k4) {
                const float4 av = a[k4], bv = b[k4];
                v = fmaf(av.x, bv.x, fmaf(av.y, bv.y, fmaf(av.z, bv.z, fmaf(av.w, bv.w, v))));
            }
            acc[i] = v;
        }
    }
#pragma unroll
    for (int i = 0; i < PPT; ++i) {
        const int pair = tid + i * HW_THREADS;
        if (pair < pairs) partial[(long)blockIdx.x * pairs + pair] = acc[i];
    }
}

__global__ void head_linear_bwd_weight_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dW, int ctas,
                                                     int pairs) {
    const int pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= pairs) return;
    double acc = 0.0;
    for (int i = 0; i < ctas; ++i) acc += (double)partial[(long)i * pairs + pair];
    dW[pair] = (float)acc;
}

int hw_grid(int sms) { return sms * 4; }

template <typename T, int PPT, int KT>
int launch_hw(const void* x, const void* dy, float* partial, int N, int C, int P, int Q, int causal, int grid, cudaStream_t st) {
    const size_t smem = 2 * (size_t)C * KT * sizeof(float);
    if (smem > 48 * 1024)
        MTA_CUDA_OK(cudaFuncSetAttribute(head_linear_bwd_weight_kernel<T, PPT, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    head_linear_bwd_weight_kernel<T, PPT, KT><<<grid, HW_THREADS, smem, st>>>(static_cast<const T*>(x), static_cast<const T*>(dy),
                                                                              partial, N, C, P, Q, causal);
    MTA_LAUNCH_OK("head_linear_bwd_weight_kernel");
    return MTA_OK;
}

template <typename T>
int dispatch_hw(const void* x, const void* dy, float* partial, int N, int C, int P, int Q, int causal, int grid, cudaStream_t st) {
    if (C <= 16) return launch_hw<T, 1, 256>(x, dy, partial, N, C, P, Q, causal, grid, st);
    if (C <= 32) return launch_hw<T, 4, 256>(x, dy, partial, N, C, P, Q, causal, grid, st);
    if (C <= 64) return launch_hw<T, 16, 128>(x, dy, partial, N, C, P, Q, causal, grid, st);
    return launch_hw<T, 64, 64>(x, dy, partial, N, C, P, Q, causal, grid, st);
}

}  // namespace

size_t conv2d_bwd_weight_workspace(int N, int C, int H, int W, int R, int S) {
    const long tiles = (long)((H + WT_M - 1) / WT_M) * ((W + WT_N - 1) / WT_N);
    return (size_t)N * C * tiles * R * S * sizeof(float);
}

int conv2d_bwd_weight_launch(const void* x, const void* dy, float* dw, void* workspace, int N, int C, int H, int W, int R,
                             int S, int causal, int dtype, cudaStream_t st) {
    const int tiles_m = (H + WT_M - 1) / WT_M, tiles_n = (W + WT_N - 1) / WT_N;
    const long planes = (long)N * C;
    MTA_REQUIRE(planes <= 65535, "conv2d_bwd_weight: N*C = %ld exceeds 65535", planes);
    const int taps = R * S;
    const size_t smem = ((size_t)(WT_M + R - 1) * (WT_N + S - 1) + (size_t)(WT_THREADS / 32) * taps) * sizeof(float);
    MTA_REQUIRE(smem <= 200 * 1024, "conv2d_bwd_weight: kernel %dx%d needs %zu bytes of shared memory (max 204800)", R, S, smem);
    float* partial = static_cast<float*>(workspace);
    dim3 grid((unsigned)(tiles_m * tiles_n), (unsigned)planes);
#define MTA_BW_CASE(TT)                                                                                                  \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            MTA_CUDA_OK(cudaFuncSetAttribute(conv2d_bwd_weight_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        conv2d_bwd_weight_kernel<TT><<<grid, WT_THREADS, smem, st>>>(static_cast<const TT*>(x), static_cast<const TT*>(dy), \
                                                                     partial, H, W, R, S, causal, tiles_n);               \
    } while (0)
    if (dtype == MTA_F32) MTA_BW_CASE(float);
    else if (dtype == MTA_BF16) MTA_BW_CASE(__nv_bfloat16);
    else MTA_BW_CASE(__half);
#undef MTA_BW_CASE
    MTA_LAUNCH_OK("conv2d_bwd_weight_kernel");
    conv2d_bwd_weight_reduce_kernel<<<(unsigned)(C * taps), 256, 0, st>>>(partial, dw, N, C, tiles_m * tiles_n, taps);
    MTA_LAUNCH_OK("conv2d_bwd_weight_reduce_kernel");
    return MTA_OK;
}

size_t head_linear_bwd_weight_workspace(int C) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return (size_t)hw_grid(sms) * C * C * sizeof(float);
}

int head_linear_bwd_weight_launch(const void* x, const void* dy, float* dW, void* workspace, int N, int C, int P, int Q,
                                  int causal, int dtype, cudaStream_t st) {
    int dev = 0, sms = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    MTA_REQUIRE(C >= 1 && C <= 128, "head_linear_bwd_weight: C = %d heads is outside the supported range 1..128", C);
    const int grid = hw_grid(sms);
    float* partial = static_cast<float*>(workspace);
    int rc;
    if (dtype == MTA_F32) rc = dispatch_hw<float>(x, dy, partial, N, C, P, Q, causal, grid, st);
    else if (dtype == MTA_BF16) rc = dispatch_hw<__nv_bfloat16>(x, dy, partial, N, C, P, Q, causal, grid, st);
    else rc = dispatch_hw<__half>(x, dy, partial, N, C, P, Q, causal, grid, st);
    if (rc) return rc;
    const int pairs = C * C;
    head_linear_bwd_weight_reduce_kernel<<<(pairs + 255) / 256, 256, 0, st>>>(partial, dW, grid, pairs);
    MTA_LAUNCH_OK("head_linear_bwd_weight_reduce_kernel");
    return MTA_OK;
}

}  // namespace mta
