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

// SC = the key extent when it is one of the common sizes (the window of a row tap then sits in registers and every tap
// indexes it statically), 0 = any size (the window is re-read from shared memory per tap).
template <typename T, int SC>
__global__ void __launch_bounds__(WT_THREADS)
conv2d_bwd_weight_kernel(const T* __restrict__ x, const T* __restrict__ dy, float* __restrict__ partial, int H, int W,
                         int R, int S, int causal, int tiles_n) {
    extern __shared__ __align__(16) float smem[];
    const int pad_h = R - 1, pad_w = (S - 1) / 2;
    const int tw = (WT_N + S - 1 + 3) & ~3, th = WT_M + R - 1;      // row pitch a multiple of 4 floats: 16-byte window loads
    float* xs = smem;                               // th x tw, masked input
    float* part = smem + th * tw + 8;               // (WT_THREADS / 32) x R*S warp partials
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
        if constexpr (SC > 0) {
            constexpr int WIN = (WT_CPT + SC - 1 + 3) & ~3;
            float w0[WIN], w1[WIN];
#pragma unroll
            for (int c4 = 0; c4 < WIN / 4; ++c4) {
                const float4 a = reinterpret_cast<const float4*>(r0)[c4], b = reinterpret_cast<const float4*>(r1)[c4];
                w0[4 * c4] = a.x; w0[4 * c4 + 1] = a.y; w0[4 * c4 + 2] = a.z; w0[4 * c4 + 3] = a.w;
                w1[4 * c4] = b.x; w1[4 * c4 + 1] = b.y; w1[4 * c4 + 2] = b.z; w1[4 * c4 + 3] = b.w;
            }
#pragma unroll
            for (int j = 0; j < SC; ++j) {
                float v = 0.0f;
#pragma unroll
                for (int e = 0; e < WT_CPT; ++e) v = fmaf(w0[j + e], g0[e], fmaf(w1[j + e], g1[e], v));
                v = warp_sum_f(v);
                if (lane == 0) part[warp * taps + i * SC + j] = v;
            }
        } else {
            for (int j = 0; j < S; ++j) {
                float v = 0.0f;
#pragma unroll
                for (int e = 0; e < WT_CPT; ++e) v = fmaf(r0[j + e], g0[e], fmaf(r1[j + e], g1[e], v));
                v = warp_sum_f(v);
                if (lane == 0) part[warp * taps + i * S + j] = v;
            }
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

// Tensor-core version for 16-bit dtypes and C <= 32: dW = dY X^T with the positions as the contraction index of
// mma.sync m16n8k16 (A = dy, rows = output heads; B = x, columns = input heads).  The contraction index may be
// assigned to positions in any order as long as A and B agree, so lane (g,t) reads 16 bytes (8 consecutive keys
// 8t .. 8t+7 of a 32-key group) from planes g and g+8 of dy and of x, and word w of those vectors feeds k-slots
// {2t,2t+1} (w even) or {2t+8,2t+9} (w odd) of MMA w/2.  A warp owns (batch element, row, 128-key block) items and
// accumulates over all of them in registers; MT = 16-head tiles per side.
template <typename T> struct MmaK16;
template <> struct MmaK16<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};
template <> struct MmaK16<__half> {
    static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};

constexpr int HM_WARPS = 4;
constexpr int HM_KEYS = 128;       // keys per item

template <typename T, int MT>
__global__ void __launch_bounds__(HM_WARPS * 32)
head_linear_bwd_weight_mma_kernel(const T* __restrict__ x, const T* __restrict__ dy, float* __restrict__ partial, int N, int C,
                                  int P, int Q, int causal) {
    constexpr int CP = 16 * MT, NV = 2 * MT;            // padded heads; 16-byte vectors per lane, side and 32-key group
    __shared__ float red[HM_WARPS][CP * CP];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    float acc[MT][2 * MT][4];                            // [16-row tile of o][8-column tile of h][fragment]
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
        for (int b = 0; b < 2 * MT; ++b) acc[a][b][0] = acc[a][b][1] = acc[a][b][2] = acc[a][b][3] = 0.0f;
    const int kblocks = (Q + HM_KEYS - 1) / HM_KEYS;
    const long items = (long)N * P * kblocks;
    const long plane = (long)P * Q;
    for (long item = (long)blockIdx.x * HM_WARPS + warp; item < items; item += (long)gridDim.x * HM_WARPS) {
        const int kb = (int)(item % kblocks);
        const int p = (int)((item / kblocks) % P);
        const long n = item / ((long)kblocks * P);
        const int k0 = kb * HM_KEYS;
        if (causal && k0 > p) continue;
        const int n_keys = causal ? min(p + 1, Q) : Q;   // keys of this row that carry a gradient
        const long row_off = n * C * plane + (long)p * Q;
        uint4 gv[4][NV], xv[4][NV];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kq = k0 + 32 * j + 8 * t;
#pragma unroll
            for (int r = 0; r < NV; ++r) {
                const int head = g + 8 * r;
                if (head < C && kq < n_keys) {
                    gv[j][r] = __ldg(reinterpret_cast<const uint4*>(dy + row_off + head * plane + kq));
                    xv[j][r] = __ldg(reinterpret_cast<const uint4*>(x + row_off + head * plane + kq));
                } else {
                    gv[j][r] = make_uint4(0u, 0u, 0u, 0u);
                    xv[j][r] = make_uint4(0u, 0u, 0u, 0u);
                }
                if (kq + 8 > n_keys && kq < n_keys) {     // the vector that holds the last valid key: zero what lies beyond it
                    uint32_t* wd = &gv[j][r].x;
                    uint32_t* wx = &xv[j][r].x;
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        if (kq + e >= n_keys) {
                            wd[e >> 1] &= (e & 1) ? 0x0000ffffu : 0xffff0000u;
                            wx[e >> 1] &= (e & 1) ? 0x0000ffffu : 0xffff0000u;
                        }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int a = 0; a < MT; ++a)
#pragma unroll
                    for (int b = 0; b < 2 * MT; ++b) {
                        const uint32_t* ga = &gv[j][2 * a].x;       // dy of head 16a + g
                        const uint32_t* gb = &gv[j][2 * a + 1].x;   // dy of head 16a + g + 8
                        const uint32_t* xb = &xv[j][b].x;           // x of head 8b + g
                        MmaK16<T>::run(acc[a][b], ga[2 * m], gb[2 * m], ga[2 * m + 1], gb[2 * m + 1], xb[2 * m], xb[2 * m + 1]);
                    }
    }
    // fragment (a, b): c0 c1 = (o = 16a + g, h = 8b + 2t, + 1), c2 c3 = (o + 8, same h)
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
        for (int b = 0; b < 2 * MT; ++b)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int o = 16 * a + g + ((r & 2) ? 8 : 0), h = 8 * b + 2 * t + (r & 1);
                red[warp][o * CP + h] = acc[a][b][r];
            }
    __syncthreads();
    for (int i = threadIdx.x; i < CP * CP; i += HM_WARPS * 32) {
        const int o = i / CP, h = i % CP;
        if (o < C && h < C) partial[(long)blockIdx.x * C * C + o * C + h] = red[0][i] + red[1][i] + red[2][i] + red[3][i];
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
    // rows padded to a multiple of 4 floats, plus slack for the last window's 16-byte over-read
    const size_t smem = ((size_t)(WT_M + R - 1) * ((WT_N + S - 1 + 3) & ~3) + 8 + (size_t)(WT_THREADS / 32) * taps) * sizeof(float);
    MTA_REQUIRE(smem <= 200 * 1024, "conv2d_bwd_weight: kernel %dx%d needs %zu bytes of shared memory (max 204800)", R, S, smem);
    float* partial = static_cast<float*>(workspace);
    dim3 grid((unsigned)(tiles_m * tiles_n), (unsigned)planes);
#define MTA_BW_LAUNCH(TT, SCV)                                                                                           \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            MTA_CUDA_OK(cudaFuncSetAttribute(conv2d_bwd_weight_kernel<TT, SCV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        conv2d_bwd_weight_kernel<TT, SCV><<<grid, WT_THREADS, smem, st>>>(static_cast<const TT*>(x), static_cast<const TT*>(dy), \
                                                                          partial, H, W, R, S, causal, tiles_n);          \
    } while (0)
#define MTA_BW_CASE(TT)                                     \
    do {                                                    \
        switch (S) {                                        \
            case 3: MTA_BW_LAUNCH(TT, 3); break;            \
            case 5: MTA_BW_LAUNCH(TT, 5); break;            \
            case 7: MTA_BW_LAUNCH(TT, 7); break;            \
            case 11: MTA_BW_LAUNCH(TT, 11); break;          \
            case 15: MTA_BW_LAUNCH(TT, 15); break;          \
            default: MTA_BW_LAUNCH(TT, 0); break;           \
        }                                                   \
    } while (0)
    if (dtype == MTA_F32) MTA_BW_CASE(float);
    else if (dtype == MTA_BF16) MTA_BW_CASE(__nv_bfloat16);
    else MTA_BW_CASE(__half);
#undef MTA_BW_CASE
#undef MTA_BW_LAUNCH
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
    const bool vec_ok = dtype != MTA_F32 && C <= 32 && Q % 8 == 0 && aligned16(x) && aligned16(dy);
    if (vec_ok && variant("head_linear") != 1) {         // tensor cores (mta_set_variant("head_linear", 1): CUDA cores)
#define MTA_HM_CASE(TT, MTV)                                                                                              \
    head_linear_bwd_weight_mma_kernel<TT, MTV><<<grid, HM_WARPS * 32, 0, st>>>(static_cast<const TT*>(x), static_cast<const TT*>(dy), \
                                                                               partial, N, C, P, Q, causal)
        if (dtype == MTA_BF16) { if (C <= 16) MTA_HM_CASE(__nv_bfloat16, 1); else MTA_HM_CASE(__nv_bfloat16, 2); }
        else { if (C <= 16) MTA_HM_CASE(__half, 1); else MTA_HM_CASE(__half, 2); }
#undef MTA_HM_CASE
        MTA_LAUNCH_OK("head_linear_bwd_weight_mma_kernel");
        rc = MTA_OK;
    } else if (dtype == MTA_F32) rc = dispatch_hw<float>(x, dy, partial, N, C, P, Q, causal, grid, st);
    else if (dtype == MTA_BF16) rc = dispatch_hw<__nv_bfloat16>(x, dy, partial, N, C, P, Q, causal, grid, st);
    else rc = dispatch_hw<__half>(x, dy, partial, N, C, P, Q, causal, grid, st);
    if (rc) return rc;
    const int pairs = C * C;
    head_linear_bwd_weight_reduce_kernel<<<(pairs + 255) / 256, 256, 0, st>>>(partial, dW, grid, pairs);
    MTA_LAUNCH_OK("head_linear_bwd_weight_reduce_kernel");
    return MTA_OK;
}

}  // namespace mta
