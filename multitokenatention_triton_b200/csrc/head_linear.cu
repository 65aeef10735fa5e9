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
                        int write_upper, int w_transposed) {
    extern __shared__ float ws[];   // C x C
    for (int i = threadIdx.x; i < C * C; i += blockDim.x)
        ws[i] = load_weight(Wm, w_transposed ? (long)(i % C) * C + i / C : i, w_dtype);
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

// d = a * b (no accumulator input: saves zeroing the accumulators of every key block).
__device__ __forceinline__ void mma_tf32_m16n8k8_first(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
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

// 32-byte global accesses (sm_100): a lane of the tensor-core kernels owns 16 consecutive keys of a head, and two
// separate 16-byte stores would each write half of a 32-byte sector.
__device__ __forceinline__ void st_global_v8(void* p, const uint4& a, const uint4& b) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
                 "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}
// The same store with an L2 eviction policy (createpolicy) attached.
__device__ __forceinline__ void st_global_v8_hint(void* p, const uint4& a, const uint4& b, uint64_t policy) {
    asm volatile("st.global.L2::cache_hint.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8}, %9;" ::"l"(p), "r"(a.x), "r"(a.y),
                 "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void ld_global_v8(const void* p, uint4& a, uint4& b) {
    asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
                 : "l"(p)
                 : "memory");
}
// Rows of a view start on 32-byte boundaries (so 16 keys from a multiple of 16 are one aligned 32-byte piece).
__host__ __device__ inline bool rows_aligned32(const void* p, const PlaneView& v) {
    return (reinterpret_cast<uintptr_t>(p) & 31u) == 0 && v.width % 16 == 0 && v.plane_stride % 16 == 0;
}

constexpr int MMA_WARPS = 4;                // warps per CTA
constexpr int MMA_KEYS_PER_WARP = 64;       // keys of one row handled per warp step

// CP = padded head count (8, 16 or 32).  KSTEPS = CP/8 MMA k-steps, MT = number of 16-row output tiles.
// SPLITW: the weight is float32 and is fed as two TF32 terms (high part + remainder), which keeps ~21 of
// its mantissa bits; 16-bit weights are exact in TF32 and need one term.
constexpr int HL_MIN_CTAS_WIDE = 3;    // resident CTAs per SM asked for when there are more than 16 heads (B1 H32 S8192 bf16:
                                       // 1.015 ms unconstrained at 182 registers, 0.891 with 3, 1.869 with 4, which spills)
// The kernel body; the two __global__ entry points below differ only in their register bound.
template <typename T, int CP, bool SPLITW>
__device__ __forceinline__ void
head_linear_mma_body(const T* __restrict__ x, PlaneView xv, const void* __restrict__ Wm, int w_dtype,
                     T* __restrict__ y, PlaneView yv, int C, int Q, int causal, float fill, int row_begin,
                     int row_end, int rows_per_cta, int write_upper, int w_transposed) {
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
                const float v = (o < C && h < C) ? load_weight(Wm, w_transposed ? (long)h * C + o : (long)o * C + h, w_dtype) : 0.0f;
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
    const bool wide = rows_aligned32(y, yv);
    // rows whose whole 64-key block lies above the diagonal are only filled; they come first
    const int p_mix = causal ? min(max(p_first, key0), p_last) : p_first;
    if (write_upper)
        for (int p = p_first; p < p_mix; ++p) {
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
    if (p_mix >= p_last) return;

    // lane (g,t) reads keys [key0+8g, key0+8g+8) of heads t, t+4, ..., t+4(NLOAD-1); the next row's loads are issued
    // before this row's math
    const int kq_in = key0 + 8 * g;
    const T* xin[NLOAD];
#pragma unroll
    for (int j = 0; j < NLOAD; ++j) xin[j] = x + xv.at(n * C + min(t + 4 * j, C - 1), p_mix, kq_in);
    auto load_row = [&](int p, uint4 (&xr)[NLOAD]) {
        const bool in_ok = kq_in < Q && !(causal && kq_in > p);
#pragma unroll
        for (int j = 0; j < NLOAD; ++j) {
            if (in_ok && t + 4 * j < C) xr[j] = __ldg(reinterpret_cast<const uint4*>(xin[j] + (long)(p - p_mix) * xv.width));
            else xr[j] = make_uint4(0u, 0u, 0u, 0u);
        }
    };
    uint4 xr[NLOAD];
    load_row(p_mix, xr);
#pragma unroll 1
    for (int p = p_mix; p < p_last; ++p) {
        uint4 xn[NLOAD];
        if (p + 1 < p_last) load_row(p + 1, xn);
        // One MMA column index (n = g) per key offset e: column g of MMA e is key key0 + 8g + e.
        float acc[8][MT][4];
#pragma unroll
        for (int e = 0; e < 8; ++e)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ++ks) {
                    const uint32_t b0 = elem_bits<T>(xr[2 * ks], e), b1 = elem_bits<T>(xr[2 * ks + 1], e);
                    if (SPLITW) {
                        if (ks == 0) mma_tf32_m16n8k8_first(acc[e][mt], wl[SPLITW ? mt : 0][SPLITW ? ks : 0], b0, b1);
                        else mma_tf32_m16n8k8(acc[e][mt], wl[SPLITW ? mt : 0][SPLITW ? ks : 0], b0, b1);
                        mma_tf32_m16n8k8(acc[e][mt], wa[mt][ks], b0, b1);
                    } else {
                        if (ks == 0) mma_tf32_m16n8k8_first(acc[e][mt], wa[mt][ks], b0, b1);
                        else mma_tf32_m16n8k8(acc[e][mt], wa[mt][ks], b0, b1);
                    }
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
                const int k16 = key0 + 16 * t;
                if (wide && k16 + 16 <= Q && !(diag && k16 + 15 > p)) {      // 16 valid keys: one 32-byte store
                    uint4 o0, o1;
                    o0.x = pack2<T>(acc[0][mt][2 * hh], acc[1][mt][2 * hh]);
                    o0.y = pack2<T>(acc[2][mt][2 * hh], acc[3][mt][2 * hh]);
                    o0.z = pack2<T>(acc[4][mt][2 * hh], acc[5][mt][2 * hh]);
                    o0.w = pack2<T>(acc[6][mt][2 * hh], acc[7][mt][2 * hh]);
                    o1.x = pack2<T>(acc[0][mt][2 * hh + 1], acc[1][mt][2 * hh + 1]);
                    o1.y = pack2<T>(acc[2][mt][2 * hh + 1], acc[3][mt][2 * hh + 1]);
                    o1.z = pack2<T>(acc[4][mt][2 * hh + 1], acc[5][mt][2 * hh + 1]);
                    o1.w = pack2<T>(acc[6][mt][2 * hh + 1], acc[7][mt][2 * hh + 1]);
                    st_global_v8(y + yv.at(n * C + o, p, k16), o0, o1);
                    continue;
                }
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int kq = k16 + 8 * cc;
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
#pragma unroll
        for (int j = 0; j < NLOAD; ++j) xr[j] = xn[j];
    }
}

// Up to 16 heads: no bound on resident CTAs (the compiler settles at 96 to 120 registers; stating a bound of one CTA
// made it take far more and the kernel slower: 0.84 ms against 0.76 ms at B8 H16 S4096).
template <typename T, int CP, bool SPLITW>
__global__ void __launch_bounds__(MMA_WARPS * 32)
head_linear_mma_kernel(const T* __restrict__ x, PlaneView xv, const void* __restrict__ Wm, int w_dtype,
                       T* __restrict__ y, PlaneView yv, int C, int Q, int causal, float fill, int row_begin,
                       int row_end, int rows_per_cta, int write_upper, int w_transposed) {
    head_linear_mma_body<T, CP, SPLITW>(x, xv, Wm, w_dtype, y, yv, C, Q, causal, fill, row_begin, row_end, rows_per_cta,
                                        write_upper, w_transposed);
}
// More than 16 heads: twice the accumulators and weight fragments; bounded so that HL_MIN_CTAS_WIDE CTAs stay resident.
template <typename T, int CP, bool SPLITW>
__global__ void __launch_bounds__(MMA_WARPS * 32, HL_MIN_CTAS_WIDE)
head_linear_mma_wide_kernel(const T* __restrict__ x, PlaneView xv, const void* __restrict__ Wm, int w_dtype,
                            T* __restrict__ y, PlaneView yv, int C, int Q, int causal, float fill, int row_begin,
                            int row_end, int rows_per_cta, int write_upper, int w_transposed) {
    head_linear_mma_body<T, CP, SPLITW>(x, xv, Wm, w_dtype, y, yv, C, Q, causal, fill, row_begin, row_end, rows_per_cta,
                                        write_upper, w_transposed);
}

// ------------------------------------------------------------------------------------------------
// Head mix followed by the causal row softmax, in one kernel (16-bit dtypes, causal):
//   y[n,o,p,:p+1] = softmax_k( round16( sum_h Wm[o,h] * x[n,h,p,k] ) ),   entries k > p are written as 0 (write_upper)
//   or left untouched.
// Stands in for the reference's head mix with fill -inf followed by F.softmax(scores.float(), -1).type_as(xq)
// (mta_attention_triton.py:76-79) without the extra pass over the score planes that a separate softmax costs.
//
// A CTA owns one (n, p): all heads of one query row.  Phase 1 walks the row in blocks of 64 keys per warp exactly as
// head_linear_mma_kernel does, rounds the mixed logits to the 16-bit dtype (the reference's rounding point), writes
// them to y and keeps a running (max, sum of exponentials) per output head.  The per-head statistics are combined
// across the CTA in a fixed order, and in phase 2 every thread re-reads the vectors it wrote itself (they are still in
// L2), turns them into probabilities and writes them back.  Rows are handed out longest first.
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// (m, s) <- combination of two partial softmax statistics; m = -inf marks an empty part.
__device__ __forceinline__ void stat_merge(float& m, float& s, float m2, float s2) {
    const float mn = fmaxf(m, m2);
    if (mn == -INFINITY) { s = 0.0f; return; }
    s = s * ex2f((m - mn) * LOG2E) + s2 * ex2f((m2 - mn) * LOG2E);
    m = mn;
}

constexpr int MS_DEPTH = 3;        // ring slots per warp: loads run two 64-key blocks ahead (measured: 2 -> 1.371 ms,
                                   // 3 -> 1.359, 4 -> 1.387, 6 -> 1.455 for B8 H16 S4096 bf16)

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid, uint64_t policy) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int n = valid ? 16 : 0;                  // 0 source bytes: the 16 destination bytes are zero filled
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;" ::"r"(d), "l"(gsrc), "r"(n), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Packed maximum of the two 16-bit values of each operand word.
template <typename T> __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b);
template <> __device__ __forceinline__ uint32_t max2<__nv_bfloat16>(uint32_t a, uint32_t b) {
    const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t max2<__half>(uint32_t a, uint32_t b) {
    const __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
// The two 16-bit values of a word as floats.
template <typename T> __device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi);
template <> __device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack2<__half>(uint32_t w, float& lo, float& hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
}

constexpr int MS_WARPS = 4;            // warps of the CTA that owns a row
constexpr int MS_MIN_CTAS = 4;         // resident CTAs per SM the register allocation aims at
constexpr int MS_MIN_CTAS_WIDE = 3;    // the same for more than 16 heads: twice the accumulators and weight fragments spill at
                                       // 128 registers (B1 H32 S8192 bf16: 2.38 ms with 4, 1.67 with 3, 1.73 with 2)
constexpr int ms_min_ctas(int cp) { return cp > 16 ? MS_MIN_CTAS_WIDE : MS_MIN_CTAS; }

template <typename T, int CP, bool SPLITW, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, ms_min_ctas(CP))
head_mix_softmax_kernel(const T* __restrict__ x, PlaneView xv, const void* __restrict__ Wm, int w_dtype, T* y,
                        PlaneView yv, int C, int Q, int row_end, int write_upper) {
    constexpr int KSTEPS = CP / 8;
    constexpr int MT = (CP + 15) / 16;
    constexpr int NLOAD = CP / 4;
    constexpr int KB = MMA_KEYS_PER_WARP;
    __shared__ float red_m[WARPS][MT * 16], red_s[WARPS][MT * 16];
    extern __shared__ uint4 ms_ring[];                     // [warp][MS_DEPTH][NLOAD][lane]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const long n = blockIdx.y;
    const int p = row_end - 1 - (int)blockIdx.x;           // longest rows first
    const int n_keys = min(p + 1, Q);
    const int nblk = (n_keys + KB - 1) / KB;
    const bool wide = rows_aligned32(y, yv);
    // key blocks wholly below the diagonal take the short path when every MMA row and column is a real head
    const bool fast = wide && C == CP && C == 16 * MT;
    // L2 policies: the inputs and the final probabilities stream through (evict first); the logits written in phase 1
    // are read back in phase 2 and should stay (evict last) - a quarter of them did not without the hints (measured)
    const uint64_t pol_stream = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();

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

    // Lane (g,t) reads keys [8g, 8g+8) of every 64-key block of heads t, t+4, ... and owns keys [16t, 16t+16) of
    // output heads g, g+8 (+16 per further 16-row MMA tile): row pointers at those offsets, once per row.
    const T* xin[NLOAD];
#pragma unroll
    for (int j = 0; j < NLOAD; ++j) xin[j] = x + xv.at(n * C + min(t + 4 * j, C - 1), p, 8 * g);
    T* yout[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) yout[mt][hh] = y + yv.at(n * C + min(16 * mt + g + 8 * hh, C - 1), p, 16 * t);

    float rm[MT][2], rs[MT][2];                            // running statistics of output heads 16 mt + g + 8 hh
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) { rm[mt][0] = rm[mt][1] = -INFINITY; rs[mt][0] = rs[mt][1] = 0.0f; }

    // The loads run MS_DEPTH - 1 blocks ahead as asynchronous copies into a ring in shared memory; a lane only ever
    // reads the slots it filled itself, so waiting for its own copy groups is all the synchronisation the ring needs.
    uint4* ring = ms_ring + (size_t)warp * MS_DEPTH * NLOAD * 32 + lane;
    auto issue_block = [&](int blk, int slot) {
        const bool in_ok = blk < nblk && blk * KB + 8 * g < n_keys;
#pragma unroll
        for (int j = 0; j < NLOAD; ++j) {
            const bool ok = in_ok && t + 4 * j < C;
            cp_async16(ring + (slot * NLOAD + j) * 32, ok ? xin[j] + blk * KB : x, ok, pol_stream);   // zero fill when not ok
        }
        cp_async_commit();
    };

    // ---- phase 1: mix, round, write the logits, running statistics ----
#pragma unroll
    for (int d = 0; d < MS_DEPTH - 1; ++d) issue_block(warp + d * WARPS, d);
    int it = 0;
#pragma unroll 1
    for (int blk = warp; blk < nblk; blk += WARPS, ++it) {
        const int key0 = blk * KB;
        issue_block(blk + (MS_DEPTH - 1) * WARPS, (it + MS_DEPTH - 1) % MS_DEPTH);
        cp_async_wait<MS_DEPTH - 1>();                                  // this block's group has landed
        uint4 xr[NLOAD];
#pragma unroll
        for (int j = 0; j < NLOAD; ++j) xr[j] = ring[((it % MS_DEPTH) * NLOAD + j) * 32];
        float acc[8][MT][4];
#pragma unroll
        for (int e = 0; e < 8; ++e)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ++ks) {
                    const uint32_t b0 = elem_bits<T>(xr[2 * ks], e), b1 = elem_bits<T>(xr[2 * ks + 1], e);
                    if (SPLITW) {
                        if (ks == 0) mma_tf32_m16n8k8_first(acc[e][mt], wl[SPLITW ? mt : 0][SPLITW ? ks : 0], b0, b1);
                        else mma_tf32_m16n8k8(acc[e][mt], wl[SPLITW ? mt : 0][SPLITW ? ks : 0], b0, b1);
                        mma_tf32_m16n8k8(acc[e][mt], wa[mt][ks], b0, b1);
                    } else {
                        if (ks == 0) mma_tf32_m16n8k8_first(acc[e][mt], wa[mt][ks], b0, b1);
                        else mma_tf32_m16n8k8(acc[e][mt], wa[mt][ks], b0, b1);
                    }
                }
            }
        // c0 / c1 of MMA e = 0..7 are keys key0 + 16t + e / + 8 + e of head g, c2 / c3 the same keys of head g + 8
        const bool full = fast && key0 + KB <= n_keys;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                // the lane's 16 keys rounded to the 16-bit dtype: word i of pk[cc] holds keys 8 cc + 2 i, + 1
                uint4 pk[2];
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    pk[cc].x = pack2<T>(acc[0][mt][2 * hh + cc], acc[1][mt][2 * hh + cc]);
                    pk[cc].y = pack2<T>(acc[2][mt][2 * hh + cc], acc[3][mt][2 * hh + cc]);
                    pk[cc].z = pack2<T>(acc[4][mt][2 * hh + cc], acc[5][mt][2 * hh + cc]);
                    pk[cc].w = pack2<T>(acc[6][mt][2 * hh + cc], acc[7][mt][2 * hh + cc]);
                }
                float v[16];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    unpack2<T>((&pk[0].x)[i], v[2 * i], v[2 * i + 1]);
                    unpack2<T>((&pk[1].x)[i], v[8 + 2 * i], v[8 + 2 * i + 1]);
                }
                if (full) {
                    uint32_t m2 = max2<T>(max2<T>(max2<T>(pk[0].x, pk[0].y), max2<T>(pk[0].z, pk[0].w)),
                                          max2<T>(max2<T>(pk[1].x, pk[1].y), max2<T>(pk[1].z, pk[1].w)));
                    float mlo, mhi;
                    unpack2<T>(m2, mlo, mhi);
                    const float m_new = fmaxf(rm[mt][hh], fmaxf(mlo, mhi));
                    const float mlog = m_new * LOG2E;
                    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        s0 += ex2f(fmaf(v[i], LOG2E, -mlog));
                        s1 += ex2f(fmaf(v[i + 1], LOG2E, -mlog));
                    }
                    rs[mt][hh] = fmaf(rs[mt][hh], ex2f((rm[mt][hh] - m_new) * LOG2E), s0 + s1);
                    rm[mt][hh] = m_new;
                    st_global_v8_hint(yout[mt][hh] + key0, pk[0], pk[1], pol_keep);
                    continue;
                }
                // block on the diagonal (or a shape the short path does not take): keys past the diagonal are masked
                const int o = 16 * mt + g + 8 * hh;
                if (o >= C) continue;
                const int k16 = key0 + 16 * t;
                float lmax = -INFINITY;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (k16 + i >= n_keys) v[i] = -INFINITY;
                    lmax = fmaxf(lmax, v[i]);
                }
                const float m_new = fmaxf(rm[mt][hh], lmax);
                if (m_new != -INFINITY) {
                    const float mlog = m_new * LOG2E;
                    float ssum = 0.0f;
#pragma unroll
                    for (int i = 0; i < 16; ++i) ssum += ex2f(fmaf(v[i], LOG2E, -mlog));
                    rs[mt][hh] = rs[mt][hh] * ex2f((rm[mt][hh] - m_new) * LOG2E) + ssum;
                    rm[mt][hh] = m_new;
                }
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int kq = k16 + 8 * cc;
                    if (kq >= n_keys) continue;
                    T* dst = yout[mt][hh] + key0 + 8 * cc;
                    if (kq + 8 <= n_keys) {
                        *reinterpret_cast<uint4*>(dst) = pk[cc];
                    } else {                                   // the vector that holds the diagonal: keys past it stay untouched
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (kq + e < n_keys) dst[e] = from_f32<T>(v[8 * cc + e]);
                    }
                }
            }
    }
    cp_async_wait<0>();

    // ---- statistics of the whole row: the four lanes of a head, then the warps, in a fixed order ----
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float m = rm[mt][hh], s = rs[mt][hh];
#pragma unroll
            for (int off = 1; off <= 2; off <<= 1) {
                const float m2 = __shfl_xor_sync(0xffffffffu, m, off), s2 = __shfl_xor_sync(0xffffffffu, s, off);
                stat_merge(m, s, m2, s2);
            }
            if (t == 0) { red_m[warp][16 * mt + g + 8 * hh] = m; red_s[warp][16 * mt + g + 8 * hh] = s; }
        }
    __syncthreads();
    // p = 2^(x log2e - shift), shift = max log2e + log2(sum): the division by the sum is folded into the exponent
    float shift[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int o = 16 * mt + g + 8 * hh;
            float m = red_m[0][o], s = red_s[0][o];
#pragma unroll
            for (int w = 1; w < WARPS; ++w) stat_merge(m, s, red_m[w][o], red_s[w][o]);
            shift[mt][hh] = fmaf(m, LOG2E, log2f(s));
        }

    // ---- phase 2: every thread turns the logits it wrote into probabilities (two blocks per step: the loads of
    // both are in flight together) ----
    auto to_prob = [&](uint4& r, float sh) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float lo, hi;
            unpack2<T>((&r.x)[i], lo, hi);
            (&r.x)[i] = pack2<T>(ex2f(fmaf(lo, LOG2E, -sh)), ex2f(fmaf(hi, LOG2E, -sh)));
        }
    };
    // iterations whose two blocks lie wholly below the diagonal; their loads are issued one iteration ahead
    auto whole = [&](int blk) { return fast && blk < nblk && (blk + WARPS + 1) * KB <= n_keys; };
    auto load_pair = [&](int blk, uint4 (&r)[2][MT][2][2]) {
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
                    ld_global_v8(yout[mt][hh] + (blk + u * WARPS) * KB, r[u][mt][hh][0], r[u][mt][hh][1]);
    };
    uint4 raw[2][MT][2][2];
    bool cur_whole = whole(warp);
    if (cur_whole) load_pair(warp, raw);
#pragma unroll 1
    for (int blk = warp; blk < nblk; blk += 2 * WARPS) {
        const int key0 = blk * KB;
        if (cur_whole) {
            uint4 nxt[2][MT][2][2];
            const bool nxt_whole = whole(blk + 2 * WARPS);
            if (nxt_whole) load_pair(blk + 2 * WARPS, nxt);
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        to_prob(raw[u][mt][hh][0], shift[mt][hh]);
                        to_prob(raw[u][mt][hh][1], shift[mt][hh]);
                        st_global_v8_hint(yout[mt][hh] + key0 + u * WARPS * KB, raw[u][mt][hh][0], raw[u][mt][hh][1], pol_stream);
                    }
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        raw[u][mt][hh][0] = nxt[u][mt][hh][0];
                        raw[u][mt][hh][1] = nxt[u][mt][hh][1];
                    }
            cur_whole = nxt_whole;
            continue;
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int o = 16 * mt + g + 8 * hh;
                    const int k16 = key0 + u * WARPS * KB + 16 * t;
                    if (o >= C) continue;
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int kq = k16 + 8 * cc;
                        if (kq >= n_keys) continue;
                        T* dst = yout[mt][hh] + key0 + u * WARPS * KB + 8 * cc;
                        if (kq + 8 <= n_keys) {
                            uint4 r = *reinterpret_cast<const uint4*>(dst);
                            to_prob(r, shift[mt][hh]);
                            *reinterpret_cast<uint4*>(dst) = r;
                        } else {                               // the vector that holds the diagonal
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                if (kq + e < n_keys)
                                    dst[e] = from_f32<T>(ex2f(fmaf(to_f32<T>(dst[e]), LOG2E, -shift[mt][hh])));
                                else if (write_upper)
                                    dst[e] = from_f32<T>(0.0f);
                            }
                        }
                    }
                }
        cur_whole = whole(blk + 2 * WARPS);
        if (cur_whole) load_pair(blk + 2 * WARPS, raw);
    }
    if (write_upper) {                                     // probabilities above the diagonal are exactly 0
        const int v0 = (n_keys + 7) >> 3, nv = Q >> 3;
        for (int o = 0; o < C; ++o) {
            uint4* row = reinterpret_cast<uint4*>(y + yv.at(n * C + o, p, 0));
            for (int i = v0 + (int)threadIdx.x; i < nv; i += WARPS * 32) row[i] = make_uint4(0u, 0u, 0u, 0u);
        }
    }
}


template <typename T, int CP>
int launch_mix_softmax(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C, int Q,
                       int row_begin, int row_end, bool write_upper, cudaStream_t st) {
    constexpr int WARPS = MS_WARPS;
    dim3 grid((unsigned)(row_end - row_begin), (unsigned)N);
    const size_t smem = (size_t)WARPS * MS_DEPTH * (CP / 4) * 32 * sizeof(uint4);
    constexpr size_t stat_smem = 2 * sizeof(float) * WARPS * 16 * ((CP + 15) / 16);   // the kernel's static arrays count too
    if (smem + stat_smem > 48 * 1024) {
        MTA_CUDA_OK(cudaFuncSetAttribute(head_mix_softmax_kernel<T, CP, true, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        MTA_CUDA_OK(cudaFuncSetAttribute(head_mix_softmax_kernel<T, CP, false, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    if (w_dtype == MTA_F32)
        head_mix_softmax_kernel<T, CP, true, WARPS><<<grid, WARPS * 32, smem, st>>>(static_cast<const T*>(x), xv, Wm, w_dtype,
                                                                               static_cast<T*>(y), yv, C, Q, row_end, write_upper ? 1 : 0);
    else
        head_mix_softmax_kernel<T, CP, false, WARPS><<<grid, WARPS * 32, smem, st>>>(static_cast<const T*>(x), xv, Wm, w_dtype,
                                                                                static_cast<T*>(y), yv, C, Q, row_end, write_upper ? 1 : 0);
    MTA_LAUNCH_OK("head_mix_softmax_kernel");
    return MTA_OK;
}

template <typename T, int CP>
int launch_simt(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C, int Q,
                int causal, float fill, int row_begin, int row_end, bool write_upper, bool wt, cudaStream_t st) {
    dim3 grid((unsigned)((Q + 255) / 256), (unsigned)(row_end - row_begin), (unsigned)N);
    const size_t smem = (size_t)C * C * sizeof(float);
    if (smem > 48 * 1024)
        MTA_CUDA_OK(cudaFuncSetAttribute(head_linear_simt_kernel<T, CP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    head_linear_simt_kernel<T, CP><<<grid, 256, smem, st>>>(static_cast<const T*>(x), xv, Wm, w_dtype, static_cast<T*>(y),
                                                            yv, C, Q, causal, fill, row_begin, write_upper ? 1 : 0, wt ? 1 : 0);
    MTA_LAUNCH_OK("head_linear_simt_kernel");
    return MTA_OK;
}

template <typename T>
int dispatch_simt(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C, int Q,
                  int causal, float fill, int row_begin, int row_end, bool write_upper, bool wt, cudaStream_t st) {
#define MTA_SIMT_CASE(CPV) \
    return launch_simt<T, CPV>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, wt, st)
    if (C <= 8) MTA_SIMT_CASE(8);
    if (C <= 16) MTA_SIMT_CASE(16);
    if (C <= 32) MTA_SIMT_CASE(32);
    if (C <= 64) MTA_SIMT_CASE(64);
    MTA_SIMT_CASE(128);
#undef MTA_SIMT_CASE
}

template <typename T, int CP>
int launch_mma(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C, int Q,
               int causal, float fill, int row_begin, int row_end, bool write_upper, bool wt, cudaStream_t st) {
    const int rows = row_end - row_begin;
    const int rows_per_cta = rows >= 2048 ? 8 : (rows >= 256 ? 4 : 1);
    dim3 grid((unsigned)((Q + MMA_WARPS * MMA_KEYS_PER_WARP - 1) / (MMA_WARPS * MMA_KEYS_PER_WARP)),
              (unsigned)((rows + rows_per_cta - 1) / rows_per_cta), (unsigned)N);
#define MTA_HL_LAUNCH(KERNEL, SPLIT)                                                                                     \
    KERNEL<T, CP, SPLIT><<<grid, MMA_WARPS * 32, 0, st>>>(static_cast<const T*>(x), xv, Wm, w_dtype, static_cast<T*>(y), yv, C, \
                                                         Q, causal, fill, row_begin, row_end, rows_per_cta,            \
                                                         write_upper ? 1 : 0, wt ? 1 : 0)
    if constexpr (CP > 16) {
        if (w_dtype == MTA_F32) MTA_HL_LAUNCH(head_linear_mma_wide_kernel, true);
        else MTA_HL_LAUNCH(head_linear_mma_wide_kernel, false);
    } else {
        if (w_dtype == MTA_F32) MTA_HL_LAUNCH(head_linear_mma_kernel, true);
        else MTA_HL_LAUNCH(head_linear_mma_kernel, false);
    }
#undef MTA_HL_LAUNCH
    MTA_LAUNCH_OK("head_linear_mma_kernel");
    return MTA_OK;
}

template <typename T>
int dispatch_mma(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C, int Q,
                 int causal, float fill, int row_begin, int row_end, bool write_upper, bool wt, cudaStream_t st) {
#define MTA_MMA_CASE(CPV) \
    return launch_mma<T, CPV>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, wt, st)
    if (C <= 8) MTA_MMA_CASE(8);
    if (C <= 16) MTA_MMA_CASE(16);
    MTA_MMA_CASE(32);
#undef MTA_MMA_CASE
}

bool vector_ok(const void* p, PlaneView v) {
    return aligned16(p) && v.width % 8 == 0 && v.plane_stride % 8 == 0;
}

}  // namespace

namespace {
bool mix_softmax_mma_ok(const void* x, PlaneView xv, const void* y, PlaneView yv, int C, int Q, int causal, int dtype) {
    return causal && dtype != MTA_F32 && C <= 32 && Q % 8 == 0 && x != y && vector_ok(x, xv) && vector_ok(y, yv);
}
}  // namespace

bool head_mix_softmax_supported(const void* x, PlaneView xv, const void* y, PlaneView yv, int C, int Q, int causal, int dtype,
                                int w_dtype) {
    return mix_softmax_mma_ok(x, xv, y, yv, C, Q, causal, dtype) ||
           head_mix_softmax_tc05_supported(x, xv, y, yv, C, Q, causal, dtype, w_dtype);
}

int head_mix_softmax_launch(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C,
                            int Q, int row_begin, int row_end, bool write_upper, int dtype, cudaStream_t st) {
    if (N == 0 || row_end <= row_begin || Q == 0) return MTA_OK;
    // variant "mix_softmax": 0 auto (tcgen05 where it applies), 1 the mma.sync kernel, 2 tcgen05 or an error
    const int want = variant("mix_softmax");
    const bool tc05_able = head_mix_softmax_tc05_supported(x, xv, y, yv, C, Q, 1, dtype, w_dtype);
    MTA_REQUIRE(want != 2 || tc05_able,
                "head_mix_softmax: the tcgen05 variant needs 16-bit activations and weights of one dtype and 8, 16, 32, 64 or 128 heads");
    // Measured on B200 (bf16, upper triangle written): the tcgen05 kernel takes 0.40 to 0.73 of the mma.sync kernel's time
    // at every shape tried (B8 H16 S4096: 1.39 against 2.05 ms; B4 H32 S4096: 1.40 against 2.21; B1 H32 S8192: 1.48 against
    // 2.21; B32 H16 S512: 0.16 against 0.39), so it runs wherever it applies.
    if (tc05_able && want != 1)
        return head_mix_softmax_tc05_launch(x, xv, Wm, y, yv, N, C, Q, row_begin, row_end, write_upper, dtype, st);
    MTA_REQUIRE(mix_softmax_mma_ok(x, xv, y, yv, C, Q, 1, dtype),
                "head_mix_softmax: needs a 16-bit dtype, C <= 32, Q %% 8 == 0, 16-byte aligned rows and x != y");
    MTA_REQUIRE(N <= 65535, "head_mix_softmax: N = %d exceeds 65535", N);
#define MTA_MS_CASE(TV, CPV) return launch_mix_softmax<TV, CPV>(x, xv, Wm, w_dtype, y, yv, N, C, Q, row_begin, row_end, write_upper, st)
    if (dtype == MTA_BF16) {
        if (C <= 8) MTA_MS_CASE(__nv_bfloat16, 8);
        if (C <= 16) MTA_MS_CASE(__nv_bfloat16, 16);
        MTA_MS_CASE(__nv_bfloat16, 32);
    }
    if (C <= 8) MTA_MS_CASE(__half, 8);
    if (C <= 16) MTA_MS_CASE(__half, 16);
    MTA_MS_CASE(__half, 32);
#undef MTA_MS_CASE
}

int head_linear_launch(const void* x, PlaneView xv, const void* Wm, int w_dtype, void* y, PlaneView yv, int N, int C,
                       int P, int Q, int causal, float fill, int row_begin, int row_end, bool write_upper, int dtype,
                       cudaStream_t st, bool wt) {
    (void)P;
    if (N == 0 || row_end <= row_begin || Q == 0) return MTA_OK;
    MTA_REQUIRE(C >= 1 && C <= 128, "head_linear: C = %d heads is outside the supported range 1..128", C);
    MTA_REQUIRE(N <= 65535 && row_end - row_begin <= 65535, "head_linear: N or the row count exceeds 65535");
    // variant "head_linear": 0 auto, 1 CUDA cores, 2 mma.sync, 3 tcgen05
    const int want = variant("head_linear");
    const bool mma_able = dtype != MTA_F32 && C <= 32 && Q % 8 == 0 && vector_ok(x, xv) && vector_ok(y, yv);
    const bool tc05_able = head_linear_tc05_supported(x, xv, y, yv, C, Q, dtype, w_dtype);
    MTA_REQUIRE(want != 2 || mma_able, "head_linear: the mma.sync variant needs a 16-bit dtype, C <= 32, Q %% 8 == 0 and 16-byte aligned rows");
    MTA_REQUIRE(want != 3 || tc05_able,
                "head_linear: the tcgen05 variant needs 16-bit activations and weights of one dtype, 8, 16, 32, 64 or 128 heads and x != y");
    // Measured on B200 (bf16, causal, upper triangle written): up to 32 heads the mma.sync kernel already runs at 78 to 87 %
    // of the copy bandwidth and the tcgen05 kernel takes 0.95 to 1.16 of its time (B4 H16 S2048: 0.173 against 0.160 ms),
    // so tcgen05 is the default only for 64 and 128 heads, which the mma.sync kernel does not take.
    if (tc05_able && (want == 3 || (want == 0 && !mma_able)))
        return head_linear_tc05_launch(x, xv, Wm, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, wt, dtype, st);
    const bool use_mma = mma_able && want != 1;
    if (dtype == MTA_F32)
        return dispatch_simt<float>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, wt, st);
    if (dtype == MTA_BF16)
        return use_mma ? dispatch_mma<__nv_bfloat16>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, wt, st)
                       : dispatch_simt<__nv_bfloat16>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, wt, st);
    return use_mma ? dispatch_mma<__half>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, wt, st)
                   : dispatch_simt<__half>(x, xv, Wm, w_dtype, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, wt, st);
}

}  // namespace mta
