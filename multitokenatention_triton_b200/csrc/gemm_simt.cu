// CUDA-core (fp32 FMA) versions of the two contractions of the forward: scores = Q K^T * scale and
// out = P V, restricted to keys k <= q when causal.  They serve float32 runs (where tensor-core
// TF32 would miss the 1e-3 absolute tolerance) and shapes the tensor-core kernels do not take.
// Stand in for the torch.matmul calls at mta_attention_triton.py:68-71 and :89.
#include "kernels.cuh"

namespace mta {
namespace {

constexpr int BT = 64;      // output tile edge
constexpr int BK = 32;      // contraction chunk
constexpr int GT = 256;     // threads: 16 x 16, each 4 x 4 outputs

// scores tile (BT queries x BT keys) of one (b,h): s[q,k] = sum_d Q[q,d] K[k,d]
template <typename T>
__global__ void __launch_bounds__(GT)
qk_scores_simt_kernel(const T* __restrict__ q, const T* __restrict__ k, T* __restrict__ s, PlaneView sv, int S, int D,
                      float scale, int round_scale, int causal, int row_begin, int row_end, int tiles_k) {
    __shared__ float qs[BK][BT + 1];
    __shared__ float ks[BK][BT + 1];
    const long bh = blockIdx.y;
    const int tq = blockIdx.x / tiles_k, tk = blockIdx.x % tiles_k;
    const int q0 = row_begin + tq * BT, k0 = tk * BT;
    const int q_end = min(q0 + BT, row_end);
    if (causal && k0 > q_end - 1) return;
    const T* qp = q + bh * (long)S * D;
    const T* kp = k + bh * (long)S * D;
    const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
    float acc[4][4] = {};
    for (int d0 = 0; d0 < D; d0 += BK) {
        for (int idx = tid; idx < BT * BK; idx += GT) {
            const int r = idx / BK, d = idx % BK;
            const int qq = q0 + r, kk = k0 + r;
            qs[d][r] = (qq < q_end && d0 + d < D) ? to_f32<T>(qp[(long)qq * D + d0 + d]) : 0.0f;
            ks[d][r] = (kk < S && d0 + d < D) ? to_f32<T>(kp[(long)kk * D + d0 + d]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int d = 0; d < BK; ++d) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = qs[d][ty * 4 + i]; b[i] = ks[d][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    const float sc = round_scale ? round_to<T>(scale) : scale;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qq = q0 + ty * 4 + i;
        if (qq >= q_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kk = k0 + tx * 4 + j;
            if (kk >= S || (causal && kk > qq)) continue;
            const float v = round_scale ? round_to<T>(acc[i][j]) * sc : acc[i][j] * sc;
            s[sv.at(bh, qq, kk)] = from_f32<T>(v);
        }
    }
}

// out tile (BT queries x BT features) of one (b,h): o[q,d] = sum_{k<=q} P[q,k] V[k,d]
template <typename T>
__global__ void __launch_bounds__(GT)
pv_simt_kernel(const T* __restrict__ p, PlaneView pv, const T* __restrict__ v, T* __restrict__ o, int S, int D,
               int causal, int row_begin, int row_end, int tiles_d, DropoutSpec drop) {
    __shared__ float ps[BK][BT + 1];
    __shared__ float vs[BK][BT + 1];
    const long bh = blockIdx.y;
    const int tq = blockIdx.x / tiles_d, td = blockIdx.x % tiles_d;
    const int q0 = row_begin + tq * BT, d0 = td * BT;
    const int q_end = min(q0 + BT, row_end);
    const int k_end = causal ? min(q_end, S) : S;
    const T* vp = v + bh * (long)S * D;
    const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < k_end; k0 += BK) {
        for (int idx = tid; idx < BT * BK; idx += GT) {
            {   // P: BT rows x BK keys, consecutive threads along keys
                const int r = idx / BK, kk = k0 + idx % BK;
                const int qq = q0 + r;
                float val = 0.0f;
                if (qq < q_end && kk < k_end && (!causal || kk <= qq)) val = to_f32<T>(p[pv.at(bh, qq, kk)]);
                if (drop.on() && val != 0.0f) {
                    const uint32_t keep = dropout_keep8(drop.seed, (uint32_t)bh, (uint32_t)qq, (uint32_t)(kk >> 3), drop.keep_threshold());
                    val = (keep >> (kk & 7)) & 1u ? round_to<T>(val * drop.scale()) : 0.0f;
                }
                ps[idx % BK][r] = val;
            }
            {   // V: BK keys x BT features, consecutive threads along features
                const int kr = idx / BT, d = idx % BT;
                const int kk = k0 + kr;
                vs[kr][d] = (kk < k_end && d0 + d < D) ? to_f32<T>(vp[(long)kk * D + d0 + d]) : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = ps[kk][ty * 4 + i]; b[i] = vs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    T* op = o + bh * (long)S * D;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qq = q0 + ty * 4 + i;
        if (qq >= q_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int d = d0 + tx * 4 + j;
            if (d < D) op[(long)qq * D + d] = from_f32<T>(acc[i][j]);
        }
    }
}

}  // namespace

int qk_scores_simt_launch(const void* q, const void* k, void* s, PlaneView sv, int B, int H, int S, int D, float scale,
                          int round_scale, int causal, int row_begin, int row_end, int dtype, cudaStream_t st) {
    const int tiles_q = (row_end - row_begin + BT - 1) / BT, tiles_k = (S + BT - 1) / BT;
    dim3 grid((unsigned)(tiles_q * tiles_k), (unsigned)(B * H));
#define MTA_QK(TT)                                                                                                  \
    qk_scores_simt_kernel<TT><<<grid, GT, 0, st>>>(static_cast<const TT*>(q), static_cast<const TT*>(k),             \
                                                   static_cast<TT*>(s), sv, S, D, scale, round_scale, causal, row_begin, \
                                                   row_end, tiles_k)
    if (dtype == MTA_F32) MTA_QK(float);
    else if (dtype == MTA_BF16) MTA_QK(__nv_bfloat16);
    else MTA_QK(__half);
#undef MTA_QK
    MTA_LAUNCH_OK("qk_scores_simt_kernel");
    return MTA_OK;
}

int pv_simt_launch(const void* p, PlaneView pview, const void* v, void* o, int B, int H, int S, int D, int causal,
                   int row_begin, int row_end, int dtype, cudaStream_t st, DropoutSpec drop) {
    const int tiles_q = (row_end - row_begin + BT - 1) / BT, tiles_d = (D + BT - 1) / BT;
    dim3 grid((unsigned)(tiles_q * tiles_d), (unsigned)(B * H));
#define MTA_PV(TT)                                                                                              \
    pv_simt_kernel<TT><<<grid, GT, 0, st>>>(static_cast<const TT*>(p), pview, static_cast<const TT*>(v),          \
                                            static_cast<TT*>(o), S, D, causal, row_begin, row_end, tiles_d, drop)
    if (dtype == MTA_F32) MTA_PV(float);
    else if (dtype == MTA_BF16) MTA_PV(__nv_bfloat16);
    else MTA_PV(__half);
#undef MTA_PV
    MTA_LAUNCH_OK("pv_simt_kernel");
    return MTA_OK;
}

}  // namespace mta
