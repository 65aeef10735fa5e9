// Depthwise causal 2-D convolution over (query, key) score planes.
//
// Semantics (those of the reference's conv_fwd_kernel, convolution_2d_trit.py:52-135):
//   y[q,k] = sum_{i<R, j<S} w[c,i,j] * xh[q+i-(R-1), k+j-(S-1)/2],  fp32 accumulation,
// where xh is x inside the plane and 0 outside it and, when causal, 0 wherever key > query.  The input
// above the diagonal is therefore never read, and the output above the diagonal is 0.
//
// Kernel in this file (the tensor-core kernels for 16-bit dtypes are in conv2d_tc05.cu and conv2d_mma.cu):
//   conv2d_tile_kernel   any dtype, any R x S, any plane size.  A CTA owns a TM x TN output tile, stages
//                        the (TM+R-1) x (TN+S-1) halo tile in shared memory as fp32 with the causal zero
//                        applied on the way in, and every thread keeps a sliding register window along
//                        the key axis so that each staged value is read from shared memory once per row tap.
#include "kernels.cuh"

namespace mta {
namespace {

constexpr int TM = 32;          // output rows per CTA
constexpr int TN = 128;         // output columns per CTA
constexpr int CPT = 8;          // consecutive output columns per thread
constexpr int NTHREADS = TM * (TN / CPT) / 2;   // 256: each thread owns 2 rows x CPT columns

template <typename T>
__global__ void __launch_bounds__(NTHREADS)
conv2d_tile_kernel(const T* __restrict__ x, PlaneView xv, const void* __restrict__ w, int w_dtype,
                   T* __restrict__ y, PlaneView yv, int C, int H, int W, int R, int S, int causal,
                   int row_begin, int row_end, int write_upper, int tiles_n, int grad_input) {
    extern __shared__ float smem[];
    // grad_input: the same kernel evaluates the gradient with respect to the conv's input (conv_bwd_input_kernel,
    // convolution_2d_trit.py:143-218): dx[q,k] = sum_{i,j} w[R-1-i, S-1-j] * dyh[q + i, k + j - (S-1-pad_w)], i.e. the
    // taps reversed, the rows looking forward instead of back, dyh masked like the forward's input
    const int pad_h = grad_input ? 0 : R - 1, pad_w = grad_input ? S - 1 - (S - 1) / 2 : (S - 1) / 2;
    const int tw = TN + S - 1;                 // staged tile width
    const int th = TM + R - 1;                 // staged tile height
    float* xs = smem;                          // th x tw
    float* ws = smem + th * tw;                // R x S

    const long plane = blockIdx.y;
    const int tile_m = blockIdx.x / tiles_n, tile_n = blockIdx.x % tiles_n;
    const int m0 = row_begin + tile_m * TM, n0 = tile_n * TN;
    const int m_end = min(m0 + TM, row_end);
    const int tid = threadIdx.x;
    T* yp = y + plane * yv.plane_stride;

    if (causal && n0 > m_end - 1) {            // tile entirely above the diagonal: nothing to read
        if (write_upper) {
            for (int idx = tid; idx < TM * TN; idx += NTHREADS) {
                const int q = m0 + idx / TN, k = n0 + idx % TN;
                if (q < m_end && k < W) yp[(long)(q - yv.row0) * yv.width + k] = from_f32<T>(0.0f);
            }
        }
        return;
    }

    const int c = (int)(plane % C);
    for (int idx = tid; idx < R * S; idx += NTHREADS)
        ws[idx] = load_weight(w, (long)c * R * S + (grad_input ? R * S - 1 - idx : idx), w_dtype);
    const T* xp = x + plane * xv.plane_stride;
    // The forward's taps look back, so rows from m_end on feed no stored output and need not be in the input view (a
    // row-range call stores no rows past its range); the input gradient looks forward, up to the plane's last row.
    const int q_hi = grad_input ? H : m_end;
    for (int idx = tid; idx < th * tw; idx += NTHREADS) {
        const int rr = idx / tw, cc = idx - rr * tw;
        const int qq = m0 - pad_h + rr, kk = n0 - pad_w + cc;
        float v = 0.0f;
        if (qq >= 0 && qq < q_hi && kk >= 0 && kk < W && (!causal || kk <= qq))
            v = to_f32<T>(xp[(long)(qq - xv.row0) * xv.width + kk]);
        xs[idx] = v;
    }
    __syncthreads();

    // thread -> rows (ry, ry + TM/2), columns [cx, cx + CPT)
    const int ry = tid / (TN / CPT), cx = (tid % (TN / CPT)) * CPT;
    float acc0[CPT], acc1[CPT];
#pragma unroll
    for (int e = 0; e < CPT; ++e) { acc0[e] = 0.0f; acc1[e] = 0.0f; }
    for (int i = 0; i < R; ++i) {
        const float* r0 = xs + (ry + i) * tw + cx;
        const float* r1 = xs + (ry + TM / 2 + i) * tw + cx;
        float win0[CPT], win1[CPT];
#pragma unroll
        for (int e = 0; e < CPT; ++e) { win0[e] = r0[e]; win1[e] = r1[e]; }
        for (int j = 0; j < S; ++j) {
            const float wv = ws[i * S + j];
#pragma unroll
            for (int e = 0; e < CPT; ++e) { acc0[e] = fmaf(wv, win0[e], acc0[e]); acc1[e] = fmaf(wv, win1[e], acc1[e]); }
#pragma unroll
            for (int e = 0; e < CPT - 1; ++e) { win0[e] = win0[e + 1]; win1[e] = win1[e + 1]; }
            if (j + 1 < S) { win0[CPT - 1] = r0[CPT + j]; win1[CPT - 1] = r1[CPT + j]; }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int q = m0 + ry + half * (TM / 2);
        if (q >= m_end) continue;
        T* yr = yp + (long)(q - yv.row0) * yv.width;
#pragma unroll
        for (int e = 0; e < CPT; ++e) {
            const int k = n0 + cx + e;
            if (k >= W) continue;
            const float v = half ? acc1[e] : acc0[e];
            if (!causal || k <= q) yr[k] = from_f32<T>(v);
            else if (write_upper) yr[k] = from_f32<T>(0.0f);
        }
    }
}

template <typename T>
int launch_tile(const void* x, PlaneView xv, const void* w, int w_dtype, void* y, PlaneView yv, long planes, int C,
                int H, int W, int R, int S, int causal, int row_begin, int row_end, bool write_upper,
                cudaStream_t st, bool grad_input = false) {
    const int tiles_m = (row_end - row_begin + TM - 1) / TM, tiles_n = (W + TN - 1) / TN;
    const size_t smem = ((size_t)(TM + R - 1) * (TN + S - 1) + (size_t)R * S) * sizeof(float);
    MTA_REQUIRE(smem <= 200 * 1024, "conv2d: kernel %dx%d needs %zu bytes of shared memory (max 204800)", R, S, smem);
    MTA_REQUIRE(planes <= 65535, "conv2d: N*C = %ld exceeds 65535", planes);
    if (smem > 48 * 1024)
        MTA_CUDA_OK(cudaFuncSetAttribute(conv2d_tile_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)(tiles_m * tiles_n), (unsigned)planes);
    conv2d_tile_kernel<T><<<grid, NTHREADS, smem, st>>>(static_cast<const T*>(x), xv, w, w_dtype, static_cast<T*>(y), yv,
                                                         C, H, W, R, S, causal, row_begin, row_end, write_upper ? 1 : 0,
                                                         tiles_n, grad_input ? 1 : 0);
    MTA_LAUNCH_OK("conv2d_tile_kernel");
    return MTA_OK;
}

}  // namespace

int conv2d_launch(const void* x, PlaneView xv, long x_rows_stored, const void* w, int w_dtype, void* y, PlaneView yv,
                  long planes, int C, int H, int W, int R, int S, int causal, int row_begin, int row_end,
                  bool write_upper, int dtype, cudaStream_t st) {
    if (planes == 0 || row_end <= row_begin || W == 0) return MTA_OK;
    const int want = variant("conv2d");      // 0 auto, 1 CUDA cores, 2 mma.sync tensor cores, 3 tcgen05 tensor cores
    const bool mma_ok = planes <= 65535 && conv2d_mma_supported(x, xv, y, yv, W, R, S, dtype);
    const bool tc05_ok = planes <= 65535 && conv2d_tc05_supported(x, xv, y, yv, W, R, S, dtype, w_dtype);
    MTA_REQUIRE(want != 2 || mma_ok, "conv2d: the mma.sync variant needs a 16-bit dtype, S <= 17, W %% 8 == 0 and 16-byte aligned planes");
    MTA_REQUIRE(want != 3 || tc05_ok, "conv2d: the tcgen05 variant needs a 16-bit dtype, S <= 17, few row taps, W %% 8 == 0 and 16-byte aligned planes");
    // Measured on the 6 x 11 bf16 case (B4 H16 S2048): tcgen05 kernel 183 us, mma.sync kernel 274 us, CUDA cores 1289 us.
    if (tc05_ok && (want == 0 || want == 3))
        return conv2d_tc05_launch(x, xv, x_rows_stored, w, w_dtype, y, yv, planes, C, H, W, R, S, causal, row_begin,
                                  row_end, write_upper, dtype, st);
    if (mma_ok && want != 1)
        return conv2d_mma_launch(x, xv, x_rows_stored, w, w_dtype, y, yv, planes, C, H, W, R, S, causal, row_begin,
                                 row_end, write_upper, dtype, st);
    switch (dtype) {
        case MTA_F32: return launch_tile<float>(x, xv, w, w_dtype, y, yv, planes, C, H, W, R, S, causal, row_begin, row_end, write_upper, st);
        case MTA_BF16: return launch_tile<__nv_bfloat16>(x, xv, w, w_dtype, y, yv, planes, C, H, W, R, S, causal, row_begin, row_end, write_upper, st);
        default: return launch_tile<__half>(x, xv, w, w_dtype, y, yv, planes, C, H, W, R, S, causal, row_begin, row_end, write_upper, st);
    }
}

// Gradient with respect to the conv's input, full planes: dx has the layout of x, zeros above the diagonal when causal.
int conv2d_bwd_input_launch(const void* dy, const void* w, int w_dtype, void* dx, long planes, int C, int H, int W, int R,
                            int S, int causal, int dtype, cudaStream_t st) {
    if (planes == 0 || H == 0 || W == 0) return MTA_OK;
    const PlaneView v{(long)H * W, 0, W};
    // 16-bit dtypes, small odd key extents: the tcgen05 conv kernel with the taps reversed (mta_set_variant("conv2d", 1)
    // keeps it on the CUDA cores)
    if (variant("conv2d") != 1 && S % 2 == 1 && planes <= 65535 && conv2d_tc05_supported(dy, v, dx, v, W, R, S, dtype, w_dtype))
        return conv2d_tc05_launch(dy, v, H, w, w_dtype, dx, v, planes, C, H, W, R, S, causal, 0, H, true, dtype, st, true);
    switch (dtype) {
        case MTA_F32: return launch_tile<float>(dy, v, w, w_dtype, dx, v, planes, C, H, W, R, S, causal, 0, H, true, st, true);
        case MTA_BF16: return launch_tile<__nv_bfloat16>(dy, v, w, w_dtype, dx, v, planes, C, H, W, R, S, causal, 0, H, true, st, true);
        default: return launch_tile<__half>(dy, v, w, w_dtype, dx, v, planes, C, H, W, R, S, causal, 0, H, true, st, true);
    }
}

}  // namespace mta
