// Head-mixing linear across the head axis of (N,C,P,Q) score planes, without a transpose.
//
// Semantics (reference: linear_head_kernel_forward, triton_linear_head.py:76-139, output pre-fill :294-297):
//   y[n,o,p,q] = sum_h Wm[o,h] * x[n,h,p,q]   for q <= p (everywhere when not causal), fp32 accumulation
//   y[n,o,p,q] = fill                          for q >  p when causal (fill may be -inf)
//
// Kernels:
//   head_linear_simt_kernel  any dtype, any C <= 128, any Q.  One thread per (row, key); the C inputs of
//                            that position sit in registers, the weight in shared memory.
//   head_linear_mma_kernel   16-bit dtypes, C <= 32, Q a multiple of 8 and 16-byte aligned rows.  One warp
//                            owns 64 consecutive keys of a row: every lane reads 16 bytes (8 keys) of
//                            CP/4 head planes, the mix runs as m16n8k8 TF32 tensor-core MMAs (16-bit values
//                            are exact in TF32, accumulation is fp32, so the result equals fp32 FMA up to
//                            summation order), and every lane writes 16-byte vectors.  Key blocks above the
//                            diagonal are never read: they are only filled.
#include "kernels.cuh"

namespace mta {
namespace {

// ------------------------------------------------------------------------------------------------
template <typename T, int CP>
__global__ void __launch_bounds__(256)
head_linear_simt_kernel(const T* __restrict__ x, PlaneView xv, const void* __restrict__ Wm, int w_dtype,
                        T* __restrict__ y, PlaneView yv, int C, int Q, int causal, float fill, int row_begin,
                        int write_upper) {
    extern __shared__ float ws[];   // C x C
    for (int i = threadIdx.x; i < C * C; i += blockDim.x) ws[i] = load_weight(Wm, i, w_dtype);
    __syncthreads();
    const int p = row_begin + blockIdx.y;
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    const long n = blockIdx.z;
    if (q >= Q) return;
    if (causal && q > p) {
        if (write_upper) {
            const T f = from_f32<T>(fill);
            for (int o = 0; o < C; ++o) y[yv.at(n * C + o, p, q)] = f;
        }
        return;
    }
    float xr[CP];
#pragma unroll
    for (int h = 0; h < CP; ++h) xr[h] = h < C ? to_f32<T>(x[xv.at(n * C + h, p, q)]) : 0.0f;
    for (int o = 0; o < C; ++o) {
        float acc = 0.0f;
        const float* wr = ws + o * C;
#pragma unroll
        for (int h = 0; h < CP; ++h)
            if (h < C) acc = fmaf(wr[h], xr[h], acc);
        y[yv.at(n * C + o, p, q)] = from_f32<T>(acc);
    }
}

// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_tf32_m16n8k8(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Element e (0..7) of a 16-byte vector of 16-bit values, as the fp32/TF32 bit pattern.
template <typename T> __device__ __forceinline__ uint32_t elem_bits(const uint4& v, int e);
template <> __device__ __forceinline__ uint32_t elem_bits<__nv_bfloat16>(const uint4& v, int e) {
    const uint32_t w = (&v.x)[e >> 1];
    return (e & 1) ? (w & 0xffff0000u) : (w << 16);
}
template <> __device__ __forceinline__ uint32_t elem_bits<__half>(const uint4& v, int e) {
    const uint32_t w = (&v.x)[e >> 1];
    const __half h = __ushort_as_half((unsigned short)((e & 1) ? (w >> 16) : (w & 0xffffu)));
    return __float_as_uint(__half2float(h));
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}

constexpr int MMA_WARPS = 4;                // warps per CTA
constexpr int MMA_KEYS_PER_WARP = 64;       // keys of one row handled per warp step

// CP = padded head count (8, 16 or 32).  KSTEPS = CP/8 MMA k-steps, MT = number of 16-row output tiles.
// SPLITW: the weight is float32 and is fed as two TF32 terms (high part + remainder), which keeps ~21 of
// its mantissa bits; 16-bit weights are exact in TF32 and need one term.
template <typename T, int CP, bool SPLITW>
__global__ void __launch_bounds__(MMA_WARPS * 32)
head_linear_mma_kernel(const T* __restrict__ x, PlaneView xv, const void* __restrict__ Wm, int w_dtype,
                       T* __restrict__ y, PlaneView yv, int C, int Q, int causal, float fill, int row_begin,
                       int row_end, int rows_per_cta, int write_upper) {
    constexpr int KSTEPS = CP / 8;
    constexpr int MT = (CP + 15) / 16;
    constexpr int NLOAD = CP / 4;            // head planes read per lane: t, t+4, ...
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const long n = blockIdx.z;

    // A fragments of the weight: a0 (g, t) a1 (g+8, t) a2 (g, t+4) a3 (g+8, t+4) of each 16x8 block.
    uint32_t wa[MT][KSTEPS][4];
    uint32_t wl[SPLITW ? MT : 1][SPLITW ? KSTEPS : 1][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int o = 16 * mt + g + ((r & 1) ? 8 : 0);
                const int h = 8 * ks + t + ((r & 2) ? 4 : 0);
                const float v = (o < C && h < C) ? load_weight(Wm, (long)o * C + h, w_dtype) : 0.0f;
                if (SPLITW) {
                    const uint32_t hi = __float_as_uint(v) & 0xffffe000u;
                    wa[mt][ks][r] = hi;
                    wl[SPLITW ? mt : 0][SPLITW ? ks : 0][r] = __float_as_uint(v - __uint_as_float(hi));
                } else {
                    wa[mt][ks][r] = __float_as_uint(v);
                }
            }

    const int key0 = (blockIdx.x * MMA_WARPS + warp) * MMA_KEYS_PER_WARP;
    if (key0 >= Q) return;
    const uint32_t fill2 = pack2<T>(fill, fill);
    const int p_first = row_begin + blockIdx.y * rows_per_cta;
    const int p_last = min(p_first + rows_per_cta, row_end);

    for (int p = p_first; p < p_last; ++p) {
        if (causal && key0 > p) {            // the whole 64-key block is above the diagonal: fill only
            if (write_upper) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int o = 16 * mt + g + 8 * hh;
                        const int kq = key0 + 16 * t;
                        if (o < C && kq < Q) {
                            uint4* dst = reinterpret_cast<uint4*>(y + yv.at(n * C + o, p, kq));
                            const uint4 f = make_uint4(fill2, fill2, fill2, fill2);
                            dst[0] = f;
                            if (kq + 8 < Q) dst[1] = f;
                        }
                    }
            }
            continue;
        }
        // lane (g,t) reads keys [key0+8g, key0+8g+8) of heads t, t+4, ..., t+4(NLOAD-1)
        uint4 xr[NLOAD];
        const int kq_in = key0 + 8 * g;
        const bool in_ok = kq_in < Q && !(causal && kq_in > p);
#pragma unroll
        for (int j = 0; j < NLOAD; ++j) {
            const int h = t + 4 * j;
            if (in_ok && h < C) xr[j] = __ldg(reinterpret_cast<const uint4*>(x + xv.at(n * C + h, p, kq_in)));
            else xr[j] = make_uint4(0u, 0u, 0u, 0u);
        }
        // One MMA column index (n = g) per key offset e: column g of MMA e is key key0 + 8g + e.
        float acc[8][MT][4];
#pragma unroll
        for (int e = 0; e < 8; ++e)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                acc[e][mt][0] = acc[e][mt][1] = acc[e][mt][2] = acc[e][mt][3] = 0.0f;
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ++ks) {
                    const uint32_t b0 = elem_bits<T>(xr[2 * ks], e), b1 = elem_bits<T>(xr[2 * ks + 1], e);
                    if (SPLITW) mma_tf32_m16n8k8(acc[e][mt], wl[SPLITW ? mt : 0][SPLITW ? ks : 0], b0, b1);
                    mma_tf32_m16n8k8(acc[e][mt], wa[mt][ks], b0, b1);
                }
            }
        // D fragment: c0 (row g, col 2t) c1 (g, 2t+1) c2 (g+8, 2t) c3 (g+8, 2t+1); column m of MMA e is key
        // key0 + 8m + e, so c0 of e = 0..7 are the 8 keys from key0 + 16t and c1 the next 8.
        const bool diag = causal && key0 + MMA_KEYS_PER_WARP - 1 > p;   // block straddles the diagonal
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int o = 16 * mt + g + 8 * hh;
                if (o >= C) continue;
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int kq = key0 + 16 * t + 8 * cc;
                    if (kq >= Q) continue;
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = acc[e][mt][2 * hh + cc];
                    T* dst = y + yv.at(n * C + o, p, kq);
                    if (diag && kq + 7 > p) {
                        if (kq > p && !write_upper) continue;
                        if (!write_upper) {           // partial vector, upper part must stay untouched
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                if (kq + e <= p) dst[e] = from_f32<T>(v[e]);
                            continue;
                        }
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (kq + e > p) v[e] = fill;
                    }
                    uint4 out;
                    out.x = pack2<T>(v[0], v[1]);
                    out.y = pack2<T>(v[2], v[3]);
                    out.z = pack2<T>(v[4], v[5]);
                    out.w = pack2<T>(v[6], v[7]);
                    *reinterpret_cast<uint4*>(dst) = out;
                }
            }
    }
}

template <typename T, int CP>
int launch_simt(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C, int Q,
                int causal, float fill, int row_begin, int row_end, bool write_upper, cudaStream_t st) {
    dim3 grid((unsigned)((Q + 255) / 256), (unsigned)(row_end - row_begin), (unsigned)N);
    const size_t smem = (size_t)C * C * sizeof(float);
    if (smem > 48 * 1024)
        MTA_CUDA_OK(cudaFuncSetAttribute(head_linear_simt_kernel<T, CP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    head_linear_simt_kernel<T, CP><<<grid, 256, smem, st>>>(static_cast<const T*>(x), xv, Wm, w_dtype, static_cast<T*>(y),
                                                            yv, C, Q, causal, fill, row_begin, write_upper ? 1 : 0);
    MTA_LAUNCH_OK("head_linear_simt_kernel");
    return MTA_OK;
}

template <typename T>
int dispatch_simt(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C, int Q,
                  int causal, float fill, int row_begin, int row_end, bool write_upper, cudaStream_t st) {
#define MTA_SIMT_CASE(CPV) \
    return launch_simt<T, CPV>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, st)
    if (C <= 8) MTA_SIMT_CASE(8);
    if (C <= 16) MTA_SIMT_CASE(16);
    if (C <= 32) MTA_SIMT_CASE(32);
    if (C <= 64) MTA_SIMT_CASE(64);
    MTA_SIMT_CASE(128);
#undef MTA_SIMT_CASE
}

template <typename T, int CP>
int launch_mma(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C, int Q,
               int causal, float fill, int row_begin, int row_end, bool write_upper, cudaStream_t st) {
    const int rows = row_end - row_begin;
    const int rows_per_cta = rows >= 2048 ? 8 : (rows >= 256 ? 4 : 1);
    dim3 grid((unsigned)((Q + MMA_WARPS * MMA_KEYS_PER_WARP - 1) / (MMA_WARPS * MMA_KEYS_PER_WARP)),
              (unsigned)((rows + rows_per_cta - 1) / rows_per_cta), (unsigned)N);
    if (w_dtype == MTA_F32)
        head_linear_mma_kernel<T, CP, true><<<grid, MMA_WARPS * 32, 0, st>>>(
            static_cast<const T*>(x), xv, Wm, w_dtype, static_cast<T*>(y), yv, C, Q, causal, fill, row_begin, row_end,
            rows_per_cta, write_upper ? 1 : 0);
    else
        head_linear_mma_kernel<T, CP, false><<<grid, MMA_WARPS * 32, 0, st>>>(
            static_cast<const T*>(x), xv, Wm, w_dtype, static_cast<T*>(y), yv, C, Q, causal, fill, row_begin, row_end,
            rows_per_cta, write_upper ? 1 : 0);
    MTA_LAUNCH_OK("head_linear_mma_kernel");
    return MTA_OK;
}

template <typename T>
int dispatch_mma(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C, int Q,
                 int causal, float fill, int row_begin, int row_end, bool write_upper, cudaStream_t st) {
#define MTA_MMA_CASE(CPV) \
    return launch_mma<T, CPV>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, st)
    if (C <= 8) MTA_MMA_CASE(8);
    if (C <= 16) MTA_MMA_CASE(16);
    MTA_MMA_CASE(32);
#undef MTA_MMA_CASE
}

bool vector_ok(const void* p, PlaneView v) {
    return aligned16(p) && v.width % 8 == 0 && v.plane_stride % 8 == 0;
}

}  // namespace

int head_linear_launch(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C,
                       int P, int Q, int causal, float fill, int row_begin, int row_end, bool write_upper, int dtype,
                       cudaStream_t st) {
    (void)P;
    if (N == 0 || row_end <= row_begin || Q == 0) return MTA_OK;
    MTA_REQUIRE(C >= 1 && C <= 128, "head_linear: C = %d heads is outside the supported range 1..128", C);
    MTA_REQUIRE(N <= 65535 && row_end - row_begin <= 65535, "head_linear: N or the row count exceeds 65535");
    const int want = variant("head_linear");
    const bool mma_able = dtype != MTA_F32 && C <= 32 && Q % 8 == 0 && vector_ok(x, xv) && vector_ok(y, yv);
    MTA_REQUIRE(want != 2 || mma_able, "head_linear: the tensor-core variant needs a 16-bit dtype, C <= 32, Q %% 8 == 0 and 16-byte aligned rows");
    const bool use_mma = mma_able && want != 1;
    if (dtype == MTA_F32)
        return dispatch_simt<float>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, st);
    if (dtype == MTA_BF16)
        return use_mma ? dispatch_mma<__nv_bfloat16>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, st)
                       : dispatch_simt<__nv_bfloat16>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, st);
    return use_mma ? dispatch_mma<__half>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, st)
                   : dispatch_simt<__half>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, st);
}

}  // namespace mta
