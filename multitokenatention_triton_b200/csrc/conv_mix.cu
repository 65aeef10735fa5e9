// Fused "conv + head mix" stage of the MTA forward for 16-bit dtypes: per (batch element, 32 x 128 tile of the
// score plane) it runs the causal depthwise conv of every head and then mixes the heads, so the conv output never
// goes to HBM.  The same kernel serves both halves of the forward:
//
//   first half   logits = W1 . conv_{w1}(scores)            and the per-row softmax statistics of the logits
//                (reference: mta_attention_triton.py:73-75; conv kernel convolution_2d_trit.py:52-135, head mix
//                 triton_linear_head.py:76-139)
//   second half  out = W2 . conv_{w2}(softmax(logits))      with the softmax applied on the fly while the logits
//                tile is staged (reference: mta_attention_triton.py:79-85)
//
// so the row softmax needs no pass of its own.  Every 16-bit rounding point of the reference is kept: the conv
// output, the mixed logits, the probabilities and the final weights are each rounded to the activation dtype.
//
// One CTA owns a block of 32 query rows of one batch element and walks the key tiles left to right (carrying the
// running row maximum / sum for the statistics).  For every key tile it loops over the heads:
//   TMA tiled load of the (32 + R-1) x 152 halo tile of that head's plane + bulk copy of the head's Toeplitz
//   fragments (a ring of up to four stages, issued three (tile, head) steps ahead: a step is far shorter than the
//   latency of a load) -> zero keys above the diagonal / apply the softmax in
//   shared memory -> conv as Toeplitz MMAs (mma.sync m16n8k16, see conv2d_mma.cu) -> 16-bit conv output into a
//   shared-memory tile per head;
// then mixes the heads of the tile with TF32 MMAs (see head_linear.cu) reading those tiles, and writes the mixed
// tile to global memory with 16-byte stores.  Keys above the diagonal are neither read nor written.
#include <cstdlib>

#include "kernels.cuh"
#include "tc05.cuh"

namespace mta {
namespace {
using namespace tc05;

// Per-phase cycle counters of warp 0 of CTA (0,0), compiled in only with -DMTA_CM_PROFILE and printed by the launcher
// when the environment variable MTA_CM_PROFILE is set.
#ifdef MTA_CM_PROFILE
__device__ long long g_cm_prof[16];
#define CM_PROF_START long long prof_t = clock64();
#define CM_PROF(slot)                                                                                   \
    {                                                                                                   \
        const long long prof_n = clock64();                                                             \
        if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 32) g_cm_prof[slot] += prof_n - prof_t;        \
        prof_t = prof_n;                                                                                \
    }
#else
#define CM_PROF_START
#define CM_PROF(slot)
#endif

constexpr int TQ = 32;               // query rows per CTA
constexpr int TK = 128;              // keys per tile
constexpr int SWC = 152;             // staged columns: 8 (left halo, 16-byte aligned) + 128 + 16
constexpr int SPITCH = SWC * 2;      // 304 bytes = 19 x 16: ldmatrix rows fall in distinct banks
constexpr int OPITCH = TK * 2 + 16;  // conv-output row pitch (272 bytes = 17 x 16)
constexpr int HSTRIDE = TQ * OPITCH + 32;   // conv-output head stride: +32 bytes so the 4 heads a lane group reads differ in bank
constexpr int CM_THREADS = 512;      // 16 warps: conv 2 (rows of 16) x 8 (columns of 16); mix 2 rows x 2 halves per warp
constexpr int CM_SMEM_MAX = 227 * 1024;
constexpr int MAXC = 16;             // heads (padded) handled by this kernel

template <typename T> struct MmaBf;
template <> struct MmaBf<__nv_bfloat16> { static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1)); } };
template <> struct MmaBf<__half> { static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1)); } };

__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}

template <typename T> __device__ __forceinline__ uint32_t pk2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pk2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t pk2<__half>(float lo, float hi) {
    __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <typename T> __device__ __forceinline__ float elem_f32(const uint4& v, int e);
template <> __device__ __forceinline__ float elem_f32<__nv_bfloat16>(const uint4& v, int e) {
    const uint32_t w = (&v.x)[e >> 1];
    return __uint_as_float((e & 1) ? (w & 0xffff0000u) : (w << 16));
}
template <> __device__ __forceinline__ float elem_f32<__half>(const uint4& v, int e) {
    const uint32_t w = (&v.x)[e >> 1];
    return __half2float(__ushort_as_half((unsigned short)((e & 1) ? (w >> 16) : (w & 0xffffu))));
}

// Toeplitz B fragments of one head, in MMA register order: [row tap i][variant v (delta = 8v - 8)][lane][2 words];
// fragment element (kk, n) holds w[i][kk - n + delta - a_off].  `lo` (optional) holds the remainder of fp32 weights.
template <typename T>
__global__ void conv_bfrag_prep_kernel(const void* __restrict__ w, int w_dtype, int C, int R, int S, uint32_t* __restrict__ hi_tab,
                                       uint32_t* __restrict__ lo_tab) {
    const int c = blockIdx.x;
    const int pad_w = (S - 1) / 2, a_off = ((pad_w + 7) & ~7) - pad_w;
    for (int idx = threadIdx.x; idx < R * 256; idx += blockDim.x) {
        const int i = idx >> 8, v = (idx >> 6) & 3, ln = (idx >> 1) & 31, reg = idx & 1;
        const int g = ln >> 2, t4 = ln & 3;
        const int delta = 8 * v - 8;
        float hi[2], lo[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int kk = 2 * t4 + e + 8 * reg;
            const int j = kk - g + delta - a_off;
            const float wv = (j >= 0 && j < S) ? load_weight(w, ((long)c * R + i) * S + j, w_dtype) : 0.0f;
            hi[e] = round_to<T>(wv);
            lo[e] = wv - hi[e];
        }
        hi_tab[(long)c * R * 256 + idx] = pk2<T>(hi[0], hi[1]);
        if (lo_tab) lo_tab[(long)c * R * 256 + idx] = pk2<T>(lo[0], lo[1]);
    }
}

struct CmArgs {
    const uint32_t* bf_hi;     // [C][R][256] words
    const uint32_t* bf_lo;     // same, or null
    const void* Wm;            // (C,C) mix weight
    int w_dtype;
    void* y;
    PlaneView yv;
    int x_row0;
    const float2* stats_in;    // per (n, head, row): (row max, row sum) of the logits; read when NORMALISE
    float2* stats_out;         // written when STATS
    int stats_row0, stats_rows;
    int C, W, R, S, row_begin, row_end;
    int nstage;                // stages of the load ring (2..4)
    int* err_flag;
};

template <typename T, bool NORMALISE, bool STATS>
__global__ void __launch_bounds__(CM_THREADS, 1)
conv_mix_kernel(const __grid_constant__ CUtensorMap mx, const CmArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[4];
    __shared__ int abort_flag;
    const int C = a.C, R = a.R, S = a.S, W = a.W;
    const int TH = TQ + R - 1;
    const int raw_bytes = (TH * SPITCH + 127) & ~127;
    const int bf_bytes = R * 1024 * (a.bf_lo ? 2 : 1);
    const int stage_bytes = raw_bytes + bf_bytes;
    const int NST = a.nstage;
    uint8_t* conv_out = smem + NST * stage_bytes;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int pad_w = (S - 1) / 2;
    const int pad8 = (pad_w + 7) & ~7;

    const int n = blockIdx.y;
    const int tiles_q = (a.row_end - a.row_begin + TQ - 1) / TQ;
    const int tq = tiles_q - 1 - (int)blockIdx.x;            // longest rows first
    const int m0 = a.row_begin + tq * TQ;
    const int m_end = min(m0 + TQ, a.row_end);
    const int nk = min((m_end + TK - 1) / TK, (W + TK - 1) / TK);
    const int total = nk * C;

    if (tid == 0) abort_flag = *reinterpret_cast<volatile int*>(a.err_flag);
    __syncthreads();
    if (abort_flag != 0) return;
    if (tid == 0) {
        for (int i = 0; i < 4; ++i) mbar_init(&full_bar[i], 1);
        fence_mbar_init();
        prefetch_tensormap(&mx);
    }
    __syncthreads();

    auto issue = [&](int it) {
        const int st = it % NST, kt = it / C, h = it - kt * C;
        uint8_t* dst = smem + st * stage_bytes;
        fence_proxy_async();        // the stage was last written through the generic proxy (softmax / zeroing pass)
        mbar_expect_tx(&full_bar[st], (uint32_t)(TH * SPITCH + bf_bytes));
        tma_load_3d(dst, &mx, &full_bar[st], kt * TK - pad8, m0 - (R - 1) - a.x_row0, n * C + h);
        bulk_load_1d(dst + raw_bytes, a.bf_hi + (long)h * R * 256, (uint32_t)(R * 1024), &full_bar[st]);
        if (a.bf_lo) bulk_load_1d(dst + raw_bytes + R * 1024, a.bf_lo + (long)h * R * 256, (uint32_t)(R * 1024), &full_bar[st]);
    };
    if (tid == 0)
        for (int it = 0; it < NST - 1 && it < total; ++it) issue(it);

    // mix weight as TF32 A fragments: a0 (g, t4) a1 (g+8, t4) a2 (g, t4+4) a3 (g+8, t4+4) of each 16 x 8 block
    uint32_t wa[2][4], wl[2][4];
    const bool split_mix = a.w_dtype == MTA_F32;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int o = g + ((r & 1) ? 8 : 0), hh = 8 * ks + t4 + ((r & 2) ? 4 : 0);
            const float v = (o < C && hh < C) ? load_weight(a.Wm, (long)o * C + hh, a.w_dtype) : 0.0f;
            const uint32_t hi = split_mix ? (__float_as_uint(v) & 0xffffe000u) : __float_as_uint(v);
            wa[ks][r] = hi;
            wl[ks][r] = __float_as_uint(v - __uint_as_float(hi));
        }

    // running softmax statistics of the rows this warp mixes: row slot ri <-> tile row warp + 16 ri, head g + 8 hh
    float run_m[2][2], run_s[2][2];
#pragma unroll
    for (int ri = 0; ri < 2; ++ri) { run_m[ri][0] = run_m[ri][1] = -INFINITY; run_s[ri][0] = run_s[ri][1] = 0.0f; }

    const int wr = warp & 1, wc = warp >> 1;                 // conv warp tile: rows 16 wr.., columns 16 wc.. (wc 0..7)
    const uint32_t a_lane_off = (uint32_t)((((lane >> 3) & 1) * 8 + (lane & 7)) * SPITCH + (lane >> 4) * 16);
    T* yb = static_cast<T*>(a.y);

    for (int it = 0; it < total; ++it) {
        const int st = it % NST, kt = it / C, h = it - kt * C;
        const int n0 = kt * TK;
        uint8_t* raw = smem + st * stage_bytes;
        const uint32_t* bfs = reinterpret_cast<const uint32_t*>(raw + raw_bytes);
        CM_PROF_START
        mbar_wait(&full_bar[st], (it / NST) & 1, a.err_flag);
        CM_PROF(0)
        // the stage consumed in iteration it-1 was released by the barrier that ended it: refill it NST-1 steps ahead
        if (tid == 0 && it + NST - 1 < total) issue(it + NST - 1);

        CM_PROF(1)
        // ---- staged tile: softmax on the fly (second half) and zero above the causal diagonal ----
        const bool diag = n0 - pad8 + SWC - 1 > m0 - (R - 1);
        if (NORMALISE || diag) {
            for (int idx = tid; idx < TH * (SWC / 8); idx += CM_THREADS) {
                const int sr = idx / (SWC / 8), ch = idx - sr * (SWC / 8);
                const int qq = m0 - (R - 1) + sr;
                const int kfirst = n0 - pad8 + ch * 8;
                uint4* p = reinterpret_cast<uint4*>(raw + sr * SPITCH + ch * 16);
                if (kfirst > qq) {
                    if (diag) *p = make_uint4(0u, 0u, 0u, 0u);
                    continue;
                }
                if (NORMALISE) {
                    if (qq < 0 || qq >= a.row_end || kfirst < 0) continue;     // padding stays zero
                    const float2 ms = __ldg(a.stats_in + ((long)(n * C + h) * a.stats_rows + (qq - a.stats_row0)));
                    const float inv = 1.0f / ms.y;
                    const uint4 v = *p;
                    float f[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) f[e] = (kfirst + e <= qq) ? __expf(elem_f32<T>(v, e) - ms.x) * inv : 0.0f;
                    uint4 o;
                    o.x = pk2<T>(f[0], f[1]);
                    o.y = pk2<T>(f[2], f[3]);
                    o.z = pk2<T>(f[4], f[5]);
                    o.w = pk2<T>(f[6], f[7]);
                    *p = o;
                } else if (kfirst + 7 > qq) {
                    uint16_t* e16 = reinterpret_cast<uint16_t*>(p);
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        if (kfirst + e > qq) e16[e] = 0;
                }
            }
        }
        CM_PROF(2)
        __syncthreads();
        CM_PROF(3)

        // ---- conv of head h: 16 x 16 outputs per warp ----
        {
            float acc[2][4] = {};
            const uint32_t raw_addr = smem_u32(raw);
            for (int i = 0; i < R; ++i) {
                uint32_t bf[4][2], bl[4][2];
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const uint2 t2 = *reinterpret_cast<const uint2*>(bfs + ((i * 4 + v) * 32 + lane) * 2);
                    bf[v][0] = t2.x;
                    bf[v][1] = t2.y;
                    if (a.bf_lo) {
                        const uint2 l2 = *reinterpret_cast<const uint2*>(bfs + R * 256 + ((i * 4 + v) * 32 + lane) * 2);
                        bl[v][0] = l2.x;
                        bl[v][1] = l2.y;
                    } else {
                        bl[v][0] = bl[v][1] = 0u;
                    }
                }
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    uint32_t af[4];
                    ldsm_x4(af, raw_addr + (uint32_t)((16 * wr + i) * SPITCH + (16 * wc + 16 * m) * 2) + a_lane_off);
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        const int v = 2 * m - nt + 1;        // delta = 16 m - 8 nt = 8 v - 8
                        MmaBf<T>::mma(acc[nt], af, bf[v][0], bf[v][1]);
                        if (a.bf_lo) MmaBf<T>::mma(acc[nt], af, bl[v][0], bl[v][1]);
                    }
                }
            }
            uint8_t* co = conv_out + h * HSTRIDE;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                uint8_t* o0 = co + (16 * wr + g) * OPITCH + (16 * wc + nt * 8 + 2 * t4) * 2;
                *reinterpret_cast<uint32_t*>(o0) = pk2<T>(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<uint32_t*>(o0 + 8 * OPITCH) = pk2<T>(acc[nt][2], acc[nt][3]);
            }
        }
        CM_PROF(4)
        __syncthreads();
        CM_PROF(5)
        if (h != C - 1) continue;

        // ---- mix the heads of this tile: warp w takes tile rows w and w+16, two blocks of 64 keys each ----
#pragma unroll
        for (int rb2 = 0; rb2 < 4; ++rb2) {
            const int ri = rb2 >> 1, kb = (rb2 & 1) * 64;        // row slot, key offset of the 64-key block inside the tile
            const int rr = warp + 16 * ri;
            const int q = m0 + rr;
            const int nb = n0 + kb;                              // first key of the block
            if (q >= m_end || nb > q) continue;
            // lane (g,t4) reads keys 8g..8g+7 of heads t4, t4+4, t4+8, t4+12
            uint4 xr[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int hh = t4 + 4 * j;
                xr[j] = hh < C ? *reinterpret_cast<const uint4*>(conv_out + hh * HSTRIDE + rr * OPITCH + kb * 2 + g * 16)
                               : make_uint4(0u, 0u, 0u, 0u);
            }
            float acc[8][4];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                acc[e][0] = acc[e][1] = acc[e][2] = acc[e][3] = 0.0f;
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    const uint32_t b0 = __float_as_uint(elem_f32<T>(xr[2 * ks], e)), b1 = __float_as_uint(elem_f32<T>(xr[2 * ks + 1], e));
                    if (split_mix) mma_tf32(acc[e], wl[ks], b0, b1);
                    mma_tf32(acc[e], wa[ks], b0, b1);
                }
            }
            // D fragment: c0 (head g, col 2 t4) c1 (g, 2 t4 + 1) c2 (g+8, ..) c3; column m of MMA e is key nb + 8 m + e,
            // so c0 over e = 0..7 are keys nb + 16 t4 .. +7 and c1 the next eight
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int o = g + 8 * hh;
                float bm = -INFINITY;
                float vals[2][8];
#pragma unroll
                for (int cc = 0; cc < 2; ++cc)
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float v = round_to<T>(acc[e][2 * hh + cc]);
                        vals[cc][e] = v;
                        if (STATS && nb + 16 * t4 + 8 * cc + e <= q) bm = fmaxf(bm, v);
                    }
                if (STATS && o < C && bm > -INFINITY) {
                    if (bm > run_m[ri][hh]) {
                        run_s[ri][hh] *= __expf(run_m[ri][hh] - bm);      // exp(-inf) = 0 on the first block
                        run_m[ri][hh] = bm;
                    }
                    float s = 0.0f;
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc)
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (nb + 16 * t4 + 8 * cc + e <= q) s += __expf(vals[cc][e] - run_m[ri][hh]);
                    run_s[ri][hh] += s;
                }
                if (o >= C) continue;
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int kq = nb + 16 * t4 + 8 * cc;
                    if (kq >= W || kq > q) continue;
                    T* dst = yb + a.yv.at((long)n * C + o, q, kq);
                    if (kq + 7 <= q) {
                        uint4 ov;
                        ov.x = pk2<T>(vals[cc][0], vals[cc][1]);
                        ov.y = pk2<T>(vals[cc][2], vals[cc][3]);
                        ov.z = pk2<T>(vals[cc][4], vals[cc][5]);
                        ov.w = pk2<T>(vals[cc][6], vals[cc][7]);
                        *reinterpret_cast<uint4*>(dst) = ov;
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (kq + e <= q) dst[e] = from_f32<T>(vals[cc][e]);
                    }
                }
            }
        }
        CM_PROF(6)
        __syncthreads();          // the conv-output tiles are rewritten by the next key tile
        CM_PROF(7)
    }

    if (STATS) {
        // combine the four lanes (t4 = 0..3) that share a (row, head) and write (max, sum)
#pragma unroll
        for (int ri = 0; ri < 2; ++ri)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                float m = run_m[ri][hh], s = run_s[ri][hh];
#pragma unroll
                for (int off = 1; off <= 2; off <<= 1) {
                    const float m2 = __shfl_xor_sync(0xffffffffu, m, off), s2 = __shfl_xor_sync(0xffffffffu, s, off);
                    const float mn = fmaxf(m, m2);
                    const float sa = (m > -INFINITY) ? s * __expf(m - mn) : 0.0f;
                    const float sb = (m2 > -INFINITY) ? s2 * __expf(m2 - mn) : 0.0f;
                    m = mn;
                    s = sa + sb;
                }
                const int q = m0 + warp + 16 * ri, o = g + 8 * hh;
                if (t4 == 0 && q < m_end && o < C)
                    a.stats_out[(long)(n * C + o) * a.stats_rows + (q - a.stats_row0)] = make_float2(m, s);
            }
    }
}

template <typename T>
int launch_cm(const void* x, PlaneView xv, long x_rows_stored, CmArgs a, int N, bool normalise, bool stats, cudaStream_t st) {
    CUtensorMap mx;
    int rc;
    const int TH = TQ + a.R - 1;
    if ((rc = make_tensor_map_3d(&mx, x, (uint64_t)N * a.C, (uint64_t)x_rows_stored, (uint64_t)a.W, (uint64_t)xv.width,
                                 (uint64_t)xv.plane_stride, SWC, (uint32_t)TH, false)))
        return rc;
    if ((rc = wait_flag_ptr(&a.err_flag))) return rc;
    const size_t stage = (size_t)((TH * SPITCH + 127) & ~127) + (size_t)a.R * 1024 * (a.bf_lo ? 2 : 1);
    a.nstage = 4;
    while (a.nstage > 2 && a.nstage * stage + (size_t)a.C * HSTRIDE > CM_SMEM_MAX) --a.nstage;
    const size_t smem = a.nstage * stage + (size_t)a.C * HSTRIDE;
    MTA_REQUIRE(smem <= CM_SMEM_MAX, "conv_mix: %d row taps need %zu bytes of shared memory per CTA", a.R, smem);
    const int tiles_q = (a.row_end - a.row_begin + TQ - 1) / TQ;
    dim3 grid((unsigned)tiles_q, (unsigned)N);
#define MTA_CM_LAUNCH(NORM, STAT)                                                                                        \
    do {                                                                                                                 \
        MTA_CUDA_OK(cudaFuncSetAttribute(conv_mix_kernel<T, NORM, STAT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        conv_mix_kernel<T, NORM, STAT><<<grid, CM_THREADS, smem, st>>>(mx, a);                                           \
    } while (0)
    if (normalise && !stats) MTA_CM_LAUNCH(true, false);
    else if (!normalise && stats) MTA_CM_LAUNCH(false, true);
    else if (!normalise && !stats) MTA_CM_LAUNCH(false, false);
    else MTA_CM_LAUNCH(true, true);
#undef MTA_CM_LAUNCH
    MTA_LAUNCH_OK("conv_mix_kernel");
#ifdef MTA_CM_PROFILE
    if (getenv("MTA_CM_PROFILE")) {
        cudaDeviceSynchronize();
        long long h[16], z[16] = {};
        cudaMemcpyFromSymbol(h, g_cm_prof, sizeof(h));
        cudaMemcpyToSymbol(g_cm_prof, z, sizeof(z));
        const long its = (long)(((a.row_end + TK - 1) / TK)) * a.C;
        fprintf(stderr, "conv_mix clk per (tile, head) step of the longest CTA (%ld steps, warp 1): wait_load %lld issue %lld pass %lld sync %lld "
                "conv %lld sync %lld | per key tile: mix %lld sync %lld\n", its, h[0] / its, h[1] / its, h[2] / its, h[3] / its, h[4] / its,
                h[5] / its, h[6] * a.C / its, h[7] * a.C / its);
    }
#endif
    return MTA_OK;
}

}  // namespace

bool conv_mix_supported(int C, int W, int R, int S, int causal, int dtype, int w_dtype, const void* x, const void* y) {
    if (!(causal && dtype != MTA_F32 && C <= MAXC && S <= 17 && W % 8 == 0 && aligned16(x) && aligned16(y))) return false;
    const size_t stage = (size_t)(((TQ + R - 1) * SPITCH + 127) & ~127) + (size_t)R * 1024 * (w_dtype == MTA_F32 ? 2 : 1);
    return 2 * stage + (size_t)C * HSTRIDE <= CM_SMEM_MAX;
}

size_t conv_mix_table_bytes(int C, int R, int w_dtype) { return (size_t)C * R * 1024 * (w_dtype == MTA_F32 ? 2 : 1); }

// Builds the Toeplitz fragment table of conv weight `w` into `table` (conv_mix_table_bytes bytes, 16-byte aligned).
int conv_mix_prepare(const void* w, int w_dtype, int C, int R, int S, int dtype, void* table, cudaStream_t st) {
    uint32_t* hi = static_cast<uint32_t*>(table);
    uint32_t* lo = w_dtype == MTA_F32 ? hi + (size_t)C * R * 256 : nullptr;
    if (dtype == MTA_BF16) conv_bfrag_prep_kernel<__nv_bfloat16><<<C, 256, 0, st>>>(w, w_dtype, C, R, S, hi, lo);
    else conv_bfrag_prep_kernel<__half><<<C, 256, 0, st>>>(w, w_dtype, C, R, S, hi, lo);
    MTA_LAUNCH_OK("conv_bfrag_prep_kernel");
    return MTA_OK;
}

// y = Wm . conv_w(x') over rows [row_begin,row_end) of every (n, head) plane, x' = x or its row softmax (stats_in);
// optionally writes the row statistics (max, sum of exp) of y to stats_out.  Statistics arrays hold
// [N*C][stats_rows] float2 entries for rows stats_row0 .. stats_row0 + stats_rows - 1.
int conv_mix_launch(const void* x, PlaneView xv, long x_rows_stored, const void* table, const void* Wm, int w_dtype, void* y,
                    PlaneView yv, int N, int C, int W, int R, int S, int row_begin, int row_end, const void* stats_in,
                    void* stats_out, int stats_row0, int stats_rows, int dtype, cudaStream_t st) {
    if (N == 0 || row_end <= row_begin) return MTA_OK;
    MTA_REQUIRE(N <= 65535, "conv_mix: batch %d exceeds 65535", N);
    CmArgs a;
    a.bf_hi = static_cast<const uint32_t*>(table);
    a.bf_lo = w_dtype == MTA_F32 ? a.bf_hi + (size_t)C * R * 256 : nullptr;
    a.Wm = Wm; a.w_dtype = w_dtype; a.y = y; a.yv = yv; a.x_row0 = xv.row0;
    a.stats_in = static_cast<const float2*>(stats_in); a.stats_out = static_cast<float2*>(stats_out);
    a.stats_row0 = stats_row0; a.stats_rows = stats_rows;
    a.C = C; a.W = W; a.R = R; a.S = S; a.row_begin = row_begin; a.row_end = row_end; a.err_flag = nullptr;
    if (dtype == MTA_BF16) return launch_cm<__nv_bfloat16>(x, xv, x_rows_stored, a, N, stats_in != nullptr, stats_out != nullptr, st);
    return launch_cm<__half>(x, xv, x_rows_stored, a, N, stats_in != nullptr, stats_out != nullptr, st);
}

}  // namespace mta
