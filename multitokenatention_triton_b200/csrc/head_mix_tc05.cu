// Head mix followed by the causal row softmax on tcgen05 (16-bit dtypes, 16-bit weights, C a power of two in 8..128):
//   y[n,o,p,:p+1] = softmax_k( round16( sum_h Wm[o,h] * x[n,h,p,k] ) ),   0 above the diagonal up to the end of the key tile
// (reference: the head mix with fill -inf followed by F.softmax(scores.float(), -1).type_as(xq),
// mta_attention_triton.py:76-79, triton_linear_head.py:76-139).
//
// The mix of R = 128 / C consecutive query rows is ONE matrix product per tile of 128 keys:
//   D[(o,r)][key] = sum over (h,r') of A[(o,r)][(h,r')] * B[(h,r')][key],
//   A = the weight spread over diagonal blocks (A[(o,r)][(h,r')] = Wm[o,h] when r = r', else 0), built once per CTA,
//   B = the R rows of all C input planes as they lie in memory (keys contiguous: an MN-major operand), one TMA box of
//       64 keys x R rows x C planes per half tile.
// A block-diagonal A wastes R-1 of R multiplications, which the tensor pipe has to spare, and it puts a whole (row, head)
// on one TMEM lane, keys along the columns: a softmax thread owns one output row of one head and needs no exchange with
// any other thread for the row statistics.
//
// A work unit = (batch element n, group of R rows).  Two passes over the unit's key tiles:
//   pass 1  tiles 0 .. diagonal: MMA -> TMEM -> round to the 16-bit dtype (the reference's rounding point) -> running
//           (maximum, sum of exponentials) per thread; nothing is written;
//   pass 2  the same tiles from the diagonal back to 0 (the input comes from L2: a unit's rows are at most 1 MB):
//           MMA again -> round -> 2^(x log2 e - shift) -> 16-bit -> a staging buffer per softmax group -> one TMA store
//           per 32 keys x 128 rows (a box of 32 keys x R rows x C planes, the mirror image of the input box).
// Recomputing the mix costs tensor time that is free here; in exchange the logits never exist in memory.
//
// Warps: 0 TMA producer (ring of HM_NSTAGE tiles of 32 KB), 1-2 MMA issuers on alternate tiles (an issuer also zeroes
// what lies above the diagonal among the group's R-1 last keys: 0 * NaN must not reach rows for which the key is valid),
// 3..18 softmax: four groups of four warps, group j owns accumulator j (128 TMEM columns) and takes every fourth tile.
// Units are dealt heaviest first in rounds of alternating direction, as in conv_attn_tc05.cu.
#include <algorithm>

#include "kernels.cuh"
#include "tc05.cuh"

namespace mta {
namespace {
using namespace tc05;

constexpr int HM_KEYS = 128;                         // keys per tile = MMA N
constexpr int HM_BOX_BYTES = 128 * 128;              // one TMA box: 128 (head, row) lines of 64 keys
constexpr int HM_STAGE_BYTES = 2 * HM_BOX_BYTES;     // a tile: keys 0..63 and 64..127
constexpr int HM_A_BYTES = 2 * HM_BOX_BYTES;         // the 128 x 128 weight operand: two K blocks of 64
constexpr int HM_NSTAGE = 4;
constexpr int HM_NACC = 4;                           // accumulators = softmax groups
constexpr int HM_SOFTMAX_THREADS = HM_NACC * 128;
constexpr int HM_OUT_BYTES = 128 * 64;                // a group's output staging: 128 rows x 32 keys

constexpr int HM_ISSUERS = 2;                        // MMA-issuing warps 1..HM_ISSUERS
// A barrier's consecutive phases must be awaited by ONE thread: a waiter that looks for the phase after next while the
// next one is still incomplete reads the parity of the phase before as "done" (try_wait tells two phases apart, no more).
// So the tiles that share a stage, or an accumulator, must all belong to the same issuer.
static_assert(HM_NSTAGE % HM_ISSUERS == 0 && HM_NACC % HM_ISSUERS == 0, "a stage or accumulator would alternate between issuers");
constexpr int HM_FIRST_SOFTMAX_WARP = 1 + HM_ISSUERS;  // warp w reads TMEM lanes 32 (w % 4) ..: any four consecutive warps cover all lanes
constexpr int HM_THREADS = HM_FIRST_SOFTMAX_WARP * 32 + HM_SOFTMAX_THREADS;
constexpr float HM_LOG2E = 1.4426950408889634f;

template <typename T> struct AbFmtH;
template <> struct AbFmtH<__nv_bfloat16> { static constexpr int value = 1; };
template <> struct AbFmtH<__half> { static constexpr int value = 0; };

template <typename T> __device__ __forceinline__ uint32_t hm_pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t hm_pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t hm_pack2<__half>(float lo, float hi) {
    __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <typename T> __device__ __forceinline__ void hm_unpack2(uint32_t w, float& lo, float& hi);
template <> __device__ __forceinline__ void hm_unpack2<__nv_bfloat16>(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
}
template <> __device__ __forceinline__ void hm_unpack2<__half>(uint32_t w, float& lo, float& hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
}
template <typename T> __device__ __forceinline__ uint32_t hm_max2(uint32_t a, uint32_t b);
template <> __device__ __forceinline__ uint32_t hm_max2<__nv_bfloat16>(uint32_t a, uint32_t b) {
    const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t hm_max2<__half>(uint32_t a, uint32_t b) {
    const __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ float hm_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 32 fp32 columns of this thread's TMEM lane, rounded to T and packed two per word (word i = columns 2i, 2i+1), as ONE
// asm statement: the 32 loaded values never become C++ variables, only the 16 packed words do.
template <typename T> __device__ __forceinline__ void hm_ld_round32(uint32_t taddr, uint32_t (&pk)[16]);
#define HM_LD_ROUND32(CVT)                                                                                              \
    asm volatile(                                                                                                       \
        "{\n\t.reg .b32 t<32>;\n\t"                                                                                    \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                       \
        "{t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15, "                                       \
        "t16, t17, t18, t19, t20, t21, t22, t23, t24, t25, t26, t27, t28, t29, t30, t31}, [%16];\n\t"                   \
        "tcgen05.wait::ld.sync.aligned;\n\t"                                                                            \
        CVT " %0, t1, t0;\n\t" CVT " %1, t3, t2;\n\t" CVT " %2, t5, t4;\n\t" CVT " %3, t7, t6;\n\t"                      \
        CVT " %4, t9, t8;\n\t" CVT " %5, t11, t10;\n\t" CVT " %6, t13, t12;\n\t" CVT " %7, t15, t14;\n\t"                \
        CVT " %8, t17, t16;\n\t" CVT " %9, t19, t18;\n\t" CVT " %10, t21, t20;\n\t" CVT " %11, t23, t22;\n\t"            \
        CVT " %12, t25, t24;\n\t" CVT " %13, t27, t26;\n\t" CVT " %14, t29, t28;\n\t" CVT " %15, t31, t30;\n\t}\n"       \
        : "=r"(pk[0]), "=r"(pk[1]), "=r"(pk[2]), "=r"(pk[3]), "=r"(pk[4]), "=r"(pk[5]), "=r"(pk[6]), "=r"(pk[7]), "=r"(pk[8]), \
          "=r"(pk[9]), "=r"(pk[10]), "=r"(pk[11]), "=r"(pk[12]), "=r"(pk[13]), "=r"(pk[14]), "=r"(pk[15])                 \
        : "r"(taddr)                                                                                                    \
        : "memory")
template <> __device__ __forceinline__ void hm_ld_round32<__nv_bfloat16>(uint32_t taddr, uint32_t (&pk)[16]) {
    HM_LD_ROUND32("cvt.rn.bf16x2.f32");
}
template <> __device__ __forceinline__ void hm_ld_round32<__half>(uint32_t taddr, uint32_t (&pk)[16]) {
    HM_LD_ROUND32("cvt.rn.f16x2.f32");
}
#undef HM_LD_ROUND32

// Pass 1 on 32 keys of a row: the logits rounded to T, their maximum folded into (m_run, s_run).
template <typename T>
__device__ __forceinline__ void hm_stats32(const uint32_t (&pk)[16], int nvalid, float& m_run, float& s_run) {
    float2 f[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) hm_unpack2<T>(pk[i], f[i].x, f[i].y);
    float cm;
    if (nvalid >= 32) {
        uint32_t mx2 = pk[0];
#pragma unroll
        for (int i = 1; i < 16; ++i) mx2 = hm_max2<T>(mx2, pk[i]);
        float lo, hi;
        hm_unpack2<T>(mx2, lo, hi);
        cm = fmaxf(lo, hi);
    } else {
        cm = -INFINITY;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (2 * i >= nvalid) f[i].x = -INFINITY;
            if (2 * i + 1 >= nvalid) f[i].y = -INFINITY;
            cm = fmaxf(cm, fmaxf(f[i].x, f[i].y));
        }
    }
    if (cm > m_run) {
        s_run *= hm_ex2((m_run - cm) * HM_LOG2E);
        m_run = cm;
    }
    const float2 l2 = make_float2(HM_LOG2E, HM_LOG2E), nm = make_float2(-m_run * HM_LOG2E, -m_run * HM_LOG2E);
    float2 a0 = make_float2(0.0f, 0.0f), a1 = a0;
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        const float2 y0 = __ffma2_rn(f[i], l2, nm), y1 = __ffma2_rn(f[i + 1], l2, nm);
        a0 = __fadd2_rn(a0, make_float2(hm_ex2(y0.x), hm_ex2(y0.y)));
        a1 = __fadd2_rn(a1, make_float2(hm_ex2(y1.x), hm_ex2(y1.y)));
    }
    a0 = __fadd2_rn(a0, a1);
    s_run += a0.x + a0.y;
}

// Pass 2 on 32 keys: the logits rounded to T -> probabilities in T, two per word; keys from nvalid on become 0.
template <typename T>
__device__ __forceinline__ void hm_prob32(const uint32_t (&in)[16], int nvalid, float shift, uint32_t (&pk)[16]) {
    const float2 l2 = make_float2(HM_LOG2E, HM_LOG2E), ns = make_float2(-shift, -shift);
    // two copies of the loop: a compiler that turns the masking into selects would spend two of them on every score
    if (nvalid >= 32) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float2 f;
            hm_unpack2<T>(in[i], f.x, f.y);
            const float2 yv = __ffma2_rn(f, l2, ns);
            pk[i] = hm_pack2<T>(hm_ex2(yv.x), hm_ex2(yv.y));
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float2 f;
            hm_unpack2<T>(in[i], f.x, f.y);
            const float2 yv = __ffma2_rn(f, l2, ns);
            pk[i] = hm_pack2<T>(2 * i < nvalid ? hm_ex2(yv.x) : 0.0f, 2 * i + 1 < nvalid ? hm_ex2(yv.y) : 0.0f);
        }
    }
}

// The plain head mix on 32 keys: the products rounded to T, two per word; keys from nvalid on become `fill`.
template <typename T>
__device__ __forceinline__ void hm_plain32(const uint32_t (&in)[16], int nvalid, float fill, uint32_t (&pk)[16]) {
    if (nvalid >= 32) {
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = in[i];
    } else {
        const uint32_t f2 = hm_pack2<T>(fill, fill);
#pragma unroll
        for (int i = 0; i < 16; ++i)
            pk[i] = (2 * i < nvalid ? in[i] & 0x0000ffffu : f2 & 0x0000ffffu) | (2 * i + 1 < nvalid ? in[i] & 0xffff0000u : f2 & 0xffff0000u);
    }
}

struct HmGeom {
    int N, C, R, Q, row_begin, row_end, groups, write_upper, x_row0, causal, wt;
    float fill;          // value of the entries above the diagonal (plain head mix; the softmax writes 0 there)
    long units;
};

// Key tiles that the rows of the group starting at p0 reach.
__device__ __forceinline__ int hm_tiles(const HmGeom& g, int p0) {
    const int p_last = min(p0 + g.R, g.row_end) - 1;
    return ((g.causal ? min(p_last + 1, g.Q) : g.Q) + HM_KEYS - 1) / HM_KEYS;
}

// SOFTMAX: the two-pass kernel described at the top.  Otherwise the plain head mix (linear_head_kernel_forward,
// triton_linear_head.py:76-139): one pass, the rounded products go out as they are, `fill` above the diagonal.
template <typename T, bool SOFTMAX>
__device__ __forceinline__ void head_mix_tc05_body(const CUtensorMap& mx, const CUtensorMap& my, const T* __restrict__ Wm, int y_row0,
                                                   const HmGeom& g, int* err_flag) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t full_bar[HM_NSTAGE], empty_bar[HM_NSTAGE], acc_full[HM_NACC], acc_empty[HM_NACC];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ float stat_m[2][HM_NACC][128], stat_s[2][HM_NACC][128];   // [unit parity][group][lane]
    uint8_t* a_base = smem;
    uint8_t* stage_base = smem + HM_A_BYTES;
    uint8_t* out_base = stage_base + HM_NSTAGE * HM_STAGE_BYTES;      // HM_NACC staging buffers of HM_OUT_BYTES
    uint8_t* fill_base = out_base + HM_NACC * HM_OUT_BYTES;           // one more, holding `fill` (0 for the softmax) everywhere
    constexpr int PASSES = SOFTMAX ? 2 : 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int C = g.C, R = g.R;

    if (tid == 0) abort_flag = *reinterpret_cast<volatile int*>(err_flag);
    __syncthreads();
    if (abort_flag != 0) return;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < HM_NSTAGE; ++i) {
                mbar_init(&full_bar[i], 1);
                mbar_init(&empty_bar[i], 1);
            }
            for (int i = 0; i < HM_NACC; ++i) {
                mbar_init(&acc_full[i], 1);
                mbar_init(&acc_empty[i], 4);
            }
            fence_mbar_init();
            prefetch_tensormap(&mx);
            prefetch_tensormap(&my);
        }
        __syncwarp();
        tmem_alloc(&tmem_slot, 512);
    }
    // The weight operand, K-major with the 128-byte swizzle: element (m, k) of K block k / 64 at byte
    // m * 128 + (((k % 64) / 8) ^ (m % 8)) * 16 + (k % 8) * 2; m = o * R + r (the order of the output box's lines),
    // k = h * R + r (the order of the input box's lines).
    for (int i = tid; i < HM_A_BYTES / 16; i += HM_THREADS) reinterpret_cast<uint4*>(a_base)[i] = make_uint4(0u, 0u, 0u, 0u);
    {
        const uint32_t f2 = SOFTMAX ? 0u : hm_pack2<T>(g.fill, g.fill);
        for (int i = tid; i < HM_OUT_BYTES / 16; i += HM_THREADS) reinterpret_cast<uint4*>(fill_base)[i] = make_uint4(f2, f2, f2, f2);
    }
    __syncthreads();
    for (int i = tid; i < 128 * C; i += HM_THREADS) {
        const int m = i / C, h = i % C;
        const int r = m % R, o = m / R;
        const int k = h * R + r, kk = k & 63;
        *reinterpret_cast<T*>(a_base + (k >> 6) * HM_BOX_BYTES + m * 128 + (((kk >> 3) ^ (m & 7)) << 4) + (kk & 7) * 2) = g.wt ? Wm[h * C + o] : Wm[o * C + h];
    }
    fence_proxy_async();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;

    // Every role walks the same sequence of units and, within a unit, of 2 * nt tiles: pass 1 upwards, pass 2 downwards.
    // Units, heaviest first, are dealt to the CTAs in rounds of alternating direction (equal tile counts per CTA, as in
    // conv_attn_tc05.cu).  Even CTAs take their rounds first to last, odd CTAs last to first: at any moment half of the
    // CTAs work on long rows and half on short ones, so that the inputs of the units in flight (128 lines x the row
    // length each, up to 1 MB) add up to about half of L2 and pass 2 finds its tiles there.
    const long n_rounds = (g.units + gridDim.x - 1) / gridDim.x;
#define HM_FOR_UNITS                                                                                   \
    for (long ri = 0; ri < n_rounds; ++ri) {                                                           \
        const long rnd = (blockIdx.x & 1) ? n_rounds - 1 - ri : ri;                                    \
        const long u = rnd * gridDim.x + ((rnd & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x);        \
        if (u >= g.units) continue;                                                                    \
        const int n = (int)(u % g.N), p0 = g.row_begin + (g.groups - 1 - (int)(u / g.N)) * R;          \
        const int nt = hm_tiles(g, p0);                                                                \
        (void)n;

    if (warp == 0) {
        if (lane == 0) {
            // Pass 1 asks L2 to keep what it reads (pass 2 reads it again within the unit), pass 2 reads it for the last time.
            const uint64_t pol_keep = l2_policy_evict_last(), pol_drop = l2_policy_evict_first();
            int it = 0;
            bool ok = true;
            HM_FOR_UNITS
                for (int j = 0; j < PASSES * nt && ok; ++j, ++it) {
                    const int kt = j < nt ? j : 2 * nt - 1 - j;
                    const int st = it % HM_NSTAGE;
                    const int use = it / HM_NSTAGE;
                    if (use > 0 && !(ok = mbar_wait(&empty_bar[st], (uint32_t)((use - 1) & 1), err_flag))) break;
                    uint8_t* dst = stage_base + st * HM_STAGE_BYTES;
                    mbar_expect_tx(&full_bar[st], HM_STAGE_BYTES);
                    const uint64_t pol = (SOFTMAX && j < nt) ? pol_keep : pol_drop;
                    tma_load_3d_hint(dst, &mx, &full_bar[st], kt * HM_KEYS, p0 - g.x_row0, n * C, pol);
                    tma_load_3d_hint(dst + HM_BOX_BYTES, &mx, &full_bar[st], kt * HM_KEYS + 64, p0 - g.x_row0, n * C, pol);
                }
                if (!ok) break;
            }
        }
    } else if (warp <= HM_ISSUERS) {
        // Two issuers take alternate tiles (a thread issues an MMA every ~75 cycles, 8 MMAs a tile would be the kernel's pace).
        constexpr uint32_t idesc = instr_desc_f16(AbFmtH<T>::value, 0, 1, 128, HM_KEYS);
        const uint32_t a_addr = smem_u32(a_base);
        const int issuer = warp - 1;
        int it = 0;
        bool ok = true;
        HM_FOR_UNITS
            for (int j = 0; j < PASSES * nt && ok; ++j, ++it) {
                if (it % HM_ISSUERS != issuer) continue;
                const int kt = j < nt ? j : 2 * nt - 1 - j;
                const int st = it % HM_NSTAGE, ab = it % HM_NACC;
                const int use = it / HM_NSTAGE, au = it / HM_NACC;
                uint8_t* sb = stage_base + st * HM_STAGE_BYTES;
                ok = mbar_wait_spin(&full_bar[st], (uint32_t)(use & 1), err_flag);
                // Keys above a row's diagonal may hold anything (NaN included) and would reach the later rows of the group
                // through the zeros of A.  Only keys p0+1 .. p0+R-1 matter (later keys are masked for every row of the
                // group): in line l = h * R + r', which holds row p0 + r', the keys p0+r'+1 .. p0+R-1 become 0.
                const int key0 = kt * HM_KEYS;
                if (g.causal && p0 + R - 1 >= key0 && p0 + 1 < key0 + HM_KEYS) {
                    // the 16-byte pieces (8 keys) that hold keys p0+1 .. p0+R-1 of this tile: one when p0 is a multiple of 8
                    const int c_lo = max(p0 + 1 - key0, 0) >> 3, c_hi = min(p0 + R - 1 - key0, HM_KEYS - 1) >> 3;
                    for (int l = lane; l < 128; l += 32) {
                        const int lim = p0 + l % R - key0;                  // last key of the tile that row p0 + r' may see
                        for (int c = c_lo; c <= c_hi; ++c) {
                            uint4* piece = reinterpret_cast<uint4*>(sb + (c >> 3) * HM_BOX_BYTES + l * 128 + (((c & 7) ^ (l & 7)) << 4));
                            uint4 w = *piece;
                            uint32_t* ww = &w.x;
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int k = c * 8 + 2 * e;
                                ww[e] &= (k > lim ? 0u : 0x0000ffffu) | (k + 1 > lim ? 0u : 0xffff0000u);
                            }
                            *piece = w;
                        }
                    }
                    fence_proxy_async();
                }
                __syncwarp();
                if (ok && au > 0) ok = mbar_wait_spin(&acc_empty[ab], (uint32_t)((au - 1) & 1), err_flag);
                fence_after_sync();
                if (lane == 0 && ok) {
                    const uint32_t b_addr = smem_u32(sb);
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const uint64_t da = smem_desc_sw128(a_addr + (kk >> 2) * HM_BOX_BYTES + (kk & 3) * 32, 16, 1024);
                        const uint64_t db = smem_desc_sw128(b_addr + kk * 16 * 128, HM_BOX_BYTES, 1024);
                        mma_f16_ss(tmem + (uint32_t)(ab * HM_KEYS), da, db, idesc, kk > 0 ? 1u : 0u);
                    }
                    mma_commit(&empty_bar[st]);
                    mma_commit(&acc_full[ab]);
                }
                __syncwarp();
            }
            if (!ok) break;
        }
    } else if (warp >= HM_FIRST_SOFTMAX_WARP) {
        const int sw = warp - HM_FIRST_SOFTMAX_WARP, grp = sw >> 2, quarter = warp & 3;   // a warp reads the TMEM lanes of its index modulo 4
        const int m = quarter * 32 + lane;
        const int r = m % R;
        const uint32_t t_base = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(grp * HM_KEYS);
        uint8_t* out_buf = out_base + grp * HM_OUT_BYTES;
        const int gt = (sw & 3) * 32 + lane;                 // thread index within the group; thread 0 issues the group's stores
        int it = 0;
        int ub = 0;
        bool ok = true;
        HM_FOR_UNITS
            const int p = p0 + r;
            const int n_keys = g.causal ? min(p + 1, g.Q) : g.Q;
            const int unit_keys = g.causal ? min(min(p0 + R, g.row_end), g.Q) : g.Q;   // keys that some row of the unit may see
            float shift = 0.0f;
            if constexpr (SOFTMAX) {
            // ---- pass 1: statistics over this group's tiles ----
            float m_run = -INFINITY, s_run = 0.0f;
            for (int j = 0; j < nt; ++j) {                         // no early exit after a wait gave up (see below)
                const int t = it + j;
                if (t % HM_NACC != grp) continue;
                if (ok) ok = mbar_wait_spin(&acc_full[grp], (uint32_t)((t / HM_NACC) & 1), err_flag);
                fence_after_sync();
                const int key0 = j * HM_KEYS;
                uint32_t cur[16];
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    hm_ld_round32<T>(t_base + (uint32_t)(c * 32), cur);
                    if (c == 3) {
                        fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[grp]);
                    }
                    const int nvalid = n_keys - (key0 + c * 32);
                    if (nvalid > 0) hm_stats32<T>(cur, nvalid, m_run, s_run);
                }
            }
            it += nt;
            // ---- the row's statistics: this thread's and the other three groups' ----
            stat_m[ub][grp][m] = m_run;
            stat_s[ub][grp][m] = s_run;
            named_barrier(1, HM_SOFTMAX_THREADS);
            // Merged in the order of the tile classes j % 4 = 0, 1, 2, 3 (class c went to group (it0 + c) % 4, it0 = the CTA's
            // tile count when the unit began): a row's result does not depend on what the CTA did before, so a row range
            // computed alone is bit-identical to the same rows of a full run.
            const int it0 = it - nt;
            float mm = stat_m[ub][it0 % HM_NACC][m], ss = stat_s[ub][it0 % HM_NACC][m];
#pragma unroll
            for (int q = 1; q < HM_NACC; ++q) {
                const float m2 = stat_m[ub][(it0 + q) % HM_NACC][m], s2 = stat_s[ub][(it0 + q) % HM_NACC][m];
                const float mn = fmaxf(mm, m2);
                if (mn != -INFINITY) {
                    ss = ss * hm_ex2((mm - mn) * HM_LOG2E) + s2 * hm_ex2((m2 - mn) * HM_LOG2E);
                    mm = mn;
                }
            }
            ub ^= 1;
            // p = 2^(x log2 e - shift): the division by the sum is folded into the exponent
            shift = fmaf(mm, HM_LOG2E, log2f(ss));
            }
            // ---- the output pass: for the softmax the tiles again, from the diagonal down ----
            for (int j = 0; j < nt; ++j) {                         // no early exit after a wait gave up (see below)
                const int t = it + j;
                if (t % HM_NACC != grp) continue;
                if (ok) ok = mbar_wait_spin(&acc_full[grp], (uint32_t)((t / HM_NACC) & 1), err_flag);
                fence_after_sync();
                const int key0 = (SOFTMAX ? nt - 1 - j : j) * HM_KEYS;
                uint32_t cur[16];
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    hm_ld_round32<T>(t_base + (uint32_t)(c * 32), cur);
                    if (c == 3) {
                        fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[grp]);
                    }
                    // The 32 keys x 128 rows of the group go out as ONE TMA store (a box of 32 keys x R rows x C planes; rows past
                    // row_end and keys past Q are clipped by the map): every thread puts its 64 bytes into the group's staging
                    // buffer (line m, 16-byte pieces swizzled as the 64-byte TMA swizzle expects, which also spreads a warp's
                    // stores over all banks).  Per-thread stores to global memory, one row each, were the slowest part of pass 2.
                    // The conditions are the same for every thread of the group: they all meet at the two barriers.
                    const int kb = key0 + c * 32;
                    if (kb >= g.Q || (kb >= unit_keys && !g.write_upper)) continue;
                    uint32_t pk[16];
                    if constexpr (SOFTMAX) hm_prob32<T>(cur, n_keys - kb, shift, pk);
                    else hm_plain32<T>(cur, n_keys - kb, g.fill, pk);
                    if (gt == 0) bulk_wait_read();                   // the previous store of this buffer has read it
                    named_barrier(2 + grp, 128);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        *reinterpret_cast<uint4*>(out_buf + m * 64 + ((q4 ^ ((m >> 1) & 3)) << 4)) =
                            make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
                    fence_proxy_async();
                    named_barrier(2 + grp, 128);
                    if (gt == 0) {
                        tma_store_3d(&my, out_buf, kb, p0 - y_row0, n * C);
                        bulk_commit();
                    }
                }
            }
            it += nt;
            if (g.write_upper && gt == 0) {
                // Everything past the unit's last tile is `fill` (0 for the softmax): boxes of the constant buffer, the
                // groups taking turns.  Nobody waits for these stores before the kernel ends.
                for (int kb = nt * HM_KEYS + grp * 32; kb < g.Q; kb += HM_NACC * 32) {
                    tma_store_3d(&my, fill_base, kb, p0 - y_row0, n * C);
                    bulk_commit();
                }
            }
            // no early exit after a wait gave up: every softmax warp must meet the others at every barrier of every unit
        }
    }
#undef HM_FOR_UNITS
    if (warp >= HM_FIRST_SOFTMAX_WARP && ((warp - HM_FIRST_SOFTMAX_WARP) & 3) == 0 && lane == 0) bulk_wait_all();
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

template <typename T>
__global__ void __launch_bounds__(HM_THREADS, 1)
head_mix_softmax_tc05_kernel(const __grid_constant__ CUtensorMap mx, const __grid_constant__ CUtensorMap my, const T* __restrict__ Wm,
                             int y_row0, HmGeom g, int* err_flag) {
    head_mix_tc05_body<T, true>(mx, my, Wm, y_row0, g, err_flag);
}
template <typename T>
__global__ void __launch_bounds__(HM_THREADS, 1)
head_mix_plain_tc05_kernel(const __grid_constant__ CUtensorMap mx, const __grid_constant__ CUtensorMap my, const T* __restrict__ Wm,
                           int y_row0, HmGeom g, int* err_flag) {
    head_mix_tc05_body<T, false>(mx, my, Wm, y_row0, g, err_flag);
}

constexpr size_t HM_SMEM_BYTES = 1024 + HM_A_BYTES + (size_t)HM_NSTAGE * HM_STAGE_BYTES + (size_t)(HM_NACC + 1) * HM_OUT_BYTES;

template <typename T, bool SOFTMAX>
int launch_hm(const void* x, PlaneView xv, const void* Wm, void* y, PlaneView yv, int N, int C, int Q, int causal, float fill,
              int row_begin, int row_end, bool write_upper, bool wt, cudaStream_t st) {
    HmGeom g{};
    g.N = N; g.C = C; g.R = 128 / C; g.Q = Q; g.row_begin = row_begin; g.row_end = row_end;
    g.groups = (row_end - row_begin + g.R - 1) / g.R;
    g.write_upper = (write_upper && causal) ? 1 : 0;
    g.x_row0 = xv.row0;
    g.causal = causal ? 1 : 0;
    g.wt = wt ? 1 : 0;
    g.fill = fill;
    g.units = (long)N * g.groups;
    CUtensorMap mx, my;
    int rc;
    // rows past row_end read as zero (they are lines of the B operand and must not carry anything into the product) and
    // are not written
    if ((rc = make_tensor_map_3d_mode(&mx, x, (uint64_t)N * C, (uint64_t)(row_end - xv.row0), (uint64_t)Q, (uint64_t)xv.width,
                                      (uint64_t)xv.plane_stride, 64, (uint32_t)g.R, 128, (uint32_t)C)))
        return rc;
    if ((rc = make_tensor_map_3d_mode(&my, y, (uint64_t)N * C, (uint64_t)(row_end - yv.row0), (uint64_t)Q, (uint64_t)yv.width,
                                      (uint64_t)yv.plane_stride, 32, (uint32_t)g.R, 64, (uint32_t)C)))
        return rc;
    int* flag = nullptr;
    if ((rc = wait_flag_ptr(&flag))) return rc;
    int dev = 0, sms = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const unsigned grid = (unsigned)std::min<long>(g.units, sms);
    if constexpr (SOFTMAX) {
        MTA_CUDA_OK(cudaFuncSetAttribute(head_mix_softmax_tc05_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)HM_SMEM_BYTES));
        head_mix_softmax_tc05_kernel<T><<<grid, HM_THREADS, HM_SMEM_BYTES, st>>>(mx, my, static_cast<const T*>(Wm), yv.row0, g, flag);
    } else {
        MTA_CUDA_OK(cudaFuncSetAttribute(head_mix_plain_tc05_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)HM_SMEM_BYTES));
        head_mix_plain_tc05_kernel<T><<<grid, HM_THREADS, HM_SMEM_BYTES, st>>>(mx, my, static_cast<const T*>(Wm), yv.row0, g, flag);
    }
    MTA_LAUNCH_OK(SOFTMAX ? "head_mix_softmax_tc05_kernel" : "head_mix_plain_tc05_kernel");
    return MTA_OK;
}

bool hm_tc05_ok(const void* x, PlaneView xv, const void* y, PlaneView yv, int C, int Q, int dtype, int w_dtype) {
    const bool pow2 = C >= 8 && C <= 128 && (C & (C - 1)) == 0;
    return dtype != MTA_F32 && w_dtype == dtype && pow2 && Q % 8 == 0 && x != y && aligned16(x) && aligned16(y) &&
           xv.width % 8 == 0 && xv.plane_stride % 8 == 0 && yv.width % 8 == 0 && yv.plane_stride % 8 == 0;
}

}  // namespace

bool head_mix_softmax_tc05_supported(const void* x, PlaneView xv, const void* y, PlaneView yv, int C, int Q, int causal, int dtype,
                                     int w_dtype) {
    return causal && hm_tc05_ok(x, xv, y, yv, C, Q, dtype, w_dtype);
}

int head_mix_softmax_tc05_launch(const void* x, PlaneView xv, const void* Wm, void* y, PlaneView yv, int N, int C, int Q,
                                 int row_begin, int row_end, bool write_upper, int dtype, cudaStream_t st) {
    if (N == 0 || row_end <= row_begin || Q == 0) return MTA_OK;
    if (dtype == MTA_BF16)
        return launch_hm<__nv_bfloat16, true>(x, xv, Wm, y, yv, N, C, Q, 1, 0.0f, row_begin, row_end, write_upper, false, st);
    return launch_hm<__half, true>(x, xv, Wm, y, yv, N, C, Q, 1, 0.0f, row_begin, row_end, write_upper, false, st);
}

bool head_linear_tc05_supported(const void* x, PlaneView xv, const void* y, PlaneView yv, int C, int Q, int dtype, int w_dtype) {
    return hm_tc05_ok(x, xv, y, yv, C, Q, dtype, w_dtype);
}

int head_linear_tc05_launch(const void* x, PlaneView xv, const void* Wm, void* y, PlaneView yv, int N, int C, int Q, int causal,
                            float fill, int row_begin, int row_end, bool write_upper, bool wt, int dtype, cudaStream_t st) {
    if (N == 0 || row_end <= row_begin || Q == 0) return MTA_OK;
    if (dtype == MTA_BF16)
        return launch_hm<__nv_bfloat16, false>(x, xv, Wm, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, wt, st);
    return launch_hm<__half, false>(x, xv, Wm, y, yv, N, C, Q, causal, fill, row_begin, row_end, write_upper, wt, st);
}

}  // namespace mta
