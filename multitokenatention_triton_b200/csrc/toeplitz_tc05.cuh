// Pieces shared by the kernels that compute a score tile Q K^T into tensor memory, stage it (rounded, scaled, causally
// zeroed) in the swizzled shared-memory layout of conv2d_tc05.cu and run the conv's Toeplitz MMAs over it
// (qk_conv_tc05.cu, conv_attn_tc05.cu): tile constants, packing, descriptors, the conv MMA schedule, the Toeplitz
// slices and the conversion of a staged row.
#pragma once

#include "kernels.cuh"
#include "tc05.cuh"

namespace mta {
namespace qc {
using namespace tc05;

constexpr int TM = 128;            // staged rows = MMA M
constexpr int TN = 128;            // output columns per tile
constexpr int SN = 144;            // staged columns = N of the score MMA: 8 (left halo) + 128 + 8
constexpr int BOX_BYTES = TM * 128;               // one 64-column box of the staged tile: 128 rows x 128 bytes
constexpr int BOX3_BYTES = TM * 32;               // the 16-column box
constexpr int KBOX_BYTES = SN * 128;              // one 64-element box of the K tile: 144 rows x 128 bytes (18 KB)
constexpr int TB_OFF = 2 * BOX_BYTES + ((BOX3_BYTES + 1023) & ~1023);    // Toeplitz slices follow the three boxes

template <typename T> struct AbFmtQ;
template <> struct AbFmtQ<__nv_bfloat16> { static constexpr int value = 1; };
template <> struct AbFmtQ<__half> { static constexpr int value = 0; };

template <typename T> __device__ __forceinline__ uint32_t pack2q(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2q<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t pack2q<__half>(float lo, float hi) {
    __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}

// Matrix descriptor without swizzle: lbo = bytes between the two 8-element k chunks of one MMA, sbo = bytes between
// groups of 8 rows.
__device__ __forceinline__ uint64_t desc_plain(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
__device__ __forceinline__ void sts128q(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Shared-memory bytes of one stage: the staged score tile (three boxes) and the Toeplitz slices of its head.
__host__ __device__ inline int toeplitz_bytes(int R, int split_w) { return (R * 1024 * (split_w ? 2 : 1) + 1023) & ~1023; }
__host__ __device__ inline int stage_bytes(int R, int split_w) { return TB_OFF + toeplitz_bytes(R, split_w); }

// The conv MMAs of one tile for issuer ISSUER (blocks [b0, b1] of the eight 16-column output blocks): the schedule of
// conv2d_tc05.cu over a staged tile at shared-memory address xa_addr with the Toeplitz slices at tb_addr, accumulating
// into TMEM columns d0 .. d0 + 127.
template <typename T, int ISSUER>
__device__ __forceinline__ void issue_conv(uint32_t xa_addr, uint32_t tb_addr, uint32_t d0, int R, int split_w) {
    constexpr uint32_t idesc32 = instr_desc_f16(AbFmtQ<T>::value, 0, 0, TM, 32);
    constexpr uint32_t idesc16 = instr_desc_f16(AbFmtQ<T>::value, 0, 0, TM, 16);
    constexpr int b0 = ISSUER == 0 ? 0 : 4, b1 = ISSUER == 0 ? 3 : 7;
    const uint64_t da0 = smem_desc_sw128(xa_addr, 16, 1024);
    const uint64_t da3 = smem_desc_sw32(xa_addr + (uint32_t)(2 * BOX_BYTES), 256);
    const uint64_t db0 = desc_plain(tb_addr, 512, 128);
    const int parts = split_w ? 2 : 1;
    int batch = 0;
#pragma unroll 1
    for (int i = 0; i < R; ++i)
#pragma unroll 1
        for (int part = 0; part < parts; ++part, ++batch) {
            const uint64_t db = db0 + (uint64_t)((i * 1024 + part * R * 1024) >> 4);
            const uint64_t da = da0 + (uint64_t)((i * 128) >> 4);
            const uint64_t dl = da3 + (uint64_t)((i * 32) >> 4);
#pragma unroll
            for (int pass = 0; pass < 2; ++pass)
#pragma unroll
                for (int s = b0 + 1 - pass; s <= b1 + 1; s += 2) {
                    const bool upper = s == b0, lower = s == b1 + 1;
                    const uint64_t adesc = s < 8 ? da + (uint64_t)(((s / 4) * BOX_BYTES + (s % 4) * 32) >> 4) : dl;
                    const uint64_t bdesc = db + (upper ? 16u : 0u);
                    const uint32_t dcol = upper ? 16u * (uint32_t)s : 16u * (uint32_t)(s - 1);
                    const uint32_t acc = (batch > 0 || pass > 0) ? 1u : 0u;
                    mma_f16_ss(d0 + dcol, adesc, bdesc, (upper || lower) ? idesc16 : idesc32, acc);
                }
        }
}

// Writes the Toeplitz slices of `head` (row tap i, element (n', kk) = w[i][kk + 16 - n' - a_off]; with `split_w` a
// second set holding what the 16-bit rounding of a float32 weight lost) in the no-swizzle K-major layout the conv
// MMAs read: 8 rows x 16 bytes per core matrix, the two k chunks 512 bytes apart, row groups 128 bytes apart.
// Called by `nthreads` threads (whole warps, ft = 0 .. nthreads - 1) that own hardware barrier `bar_id`; the head's
// R x KS weights pass through `wsm` (MAX_TAPS floats of shared memory) so that each is fetched from global memory once.
constexpr int MAX_TAPS = 16 * 17;
constexpr int TAPS_PER_THREAD = (MAX_TAPS + 127) / 128;     // with the 128 drain threads as callers

// The two halves of build_toeplitz for a caller that knows its next head ahead of time: fetch_taps reads the head's
// weights into registers (thread ft of 128 holds taps ft, ft + 128, ...), which hides the global-memory latency behind
// whatever the caller does next; store_taps / build_from_taps turn them into the slices.
__device__ __forceinline__ void fetch_taps(float (&reg)[TAPS_PER_THREAD], const void* w, int w_dtype, int head, int R, int KS, int ft) {
#pragma unroll
    for (int i = 0; i < TAPS_PER_THREAD; ++i) {
        const int idx = ft + 128 * i;
        reg[i] = idx < R * KS ? load_weight(w, (long)head * R * KS + idx, w_dtype) : 0.0f;
    }
}
template <typename T>
__device__ __forceinline__ void build_from_taps(uint8_t* tb, float* wsm, const float (&reg)[TAPS_PER_THREAD], int R, int KS, int a_off,
                                                int split_w, int ft, int bar_id) {
#pragma unroll
    for (int i = 0; i < TAPS_PER_THREAD; ++i)
        if (ft + 128 * i < R * KS) wsm[ft + 128 * i] = reg[i];
    named_barrier(bar_id, 128);
    const int total = R * 512;
    for (int idx = ft; idx < total; idx += 128) {
        const int i = idx >> 9, e = idx & 511;
        const int nn = e >> 4, kk = e & 15;
        const int j = kk + 16 - nn - a_off;
        const float wv = (j >= 0 && j < KS) ? wsm[i * KS + j] : 0.0f;
        const T hi = from_f32<T>(wv);
        const int off = i * 1024 + (kk >> 3) * 512 + (nn >> 3) * 128 + (nn & 7) * 16 + (kk & 7) * 2;
        *reinterpret_cast<T*>(tb + off) = hi;
        if (split_w) *reinterpret_cast<T*>(tb + R * 1024 + off) = from_f32<T>(wv - to_f32<T>(hi));
    }
    named_barrier(bar_id, 128);             // nobody refills wsm while another warp still reads it
}

template <typename T>
__device__ __forceinline__ void build_toeplitz(uint8_t* tb, float* wsm, const void* w, int w_dtype, int head, int R, int KS,
                                               int a_off, int split_w, int ft, int nthreads, int bar_id) {
    for (int idx = ft; idx < R * KS; idx += nthreads) wsm[idx] = load_weight(w, (long)head * R * KS + idx, w_dtype);
    named_barrier(bar_id, nthreads);
    const int total = R * 512;
    for (int idx = ft; idx < total; idx += nthreads) {
        const int i = idx / 512, e = idx % 512;
        const int nn = e / 16, kk = e % 16;
        const int j = kk + 16 - nn - a_off;
        const float wv = (j >= 0 && j < KS) ? wsm[i * KS + j] : 0.0f;
        const T hi = from_f32<T>(wv);
        const int off = i * 1024 + (kk / 8) * 512 + (nn / 8) * 128 + (nn % 8) * 16 + (kk % 8) * 2;
        *reinterpret_cast<T*>(tb + off) = hi;
        if (split_w) *reinterpret_cast<T*>(tb + R * 1024 + off) = from_f32<T>(wv - to_f32<T>(hi));
    }
    named_barrier(bar_id, nthreads);        // nobody refills wsm while another warp still reads it
}

// One thread's share of the drain: staged row sr (query qq) of the score accumulator at TMEM address trow goes into the
// swizzled stage at shared-memory address xa_s (staged column 0 holds key kbase).  SCALED: the staged value is
// round(round(S) * sc), the reference's 16-bit matmul followed by its 16-bit multiply; otherwise round(S).  `diag`
// (warp-uniform): the tile holds keys above some query of the row block, which are staged as 0; tiles wholly below the
// diagonal skip the comparison.  Whole-warp call (the TMEM loads are warp-collective).
template <typename T, bool SCALED>
__device__ __forceinline__ void drain_row(uint32_t trow, uint32_t xa_s, int sr, int qq, int kbase, float sc, bool diag) {
    auto convert8 = [&](const uint32_t* r, int col) -> uint4 {      // staged columns col .. col + 7
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = SCALED ? round_to<T>(__uint_as_float(r[e])) * sc : __uint_as_float(r[e]);
        if (diag) {
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (kbase + col + e > qq) f[e] = 0.0f;
        }
        return make_uint4(pack2q<T>(f[0], f[1]), pack2q<T>(f[2], f[3]), pack2q<T>(f[4], f[5]), pack2q<T>(f[6], f[7]));
    };
    auto store_chunk = [&](int ch, const uint4& v) {     // chunk ch = staged columns 8 ch .. 8 ch + 7
        if (ch < 16) sts128q(xa_s + (uint32_t)((ch >> 3) * BOX_BYTES + sr * 128 + (((ch & 7) ^ (sr & 7)) << 4)), v);
        else sts128q(xa_s + (uint32_t)(2 * BOX_BYTES + sr * 32 + ((((ch - 16) ^ (sr >> 2)) & 1) << 4)), v);
    };
    // 144 columns as loads of 32 + 32 + 8 columns, twice
#pragma unroll 1
    for (int chalf = 0; chalf < 2; ++chalf) {
        const int c0 = chalf * 9;
#pragma unroll 1
        for (int part = 0; part < 2; ++part) {
            uint32_t r[32];
            const int cfirst = chalf == 0 ? c0 + 4 * part : c0 + 1 + 4 * part;    // first chunk of this 32-column load
            tmem_ld_32x32(trow + (uint32_t)(cfirst * 8), r);
            tmem_ld_wait();
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) store_chunk(cfirst + c4, convert8(r + 8 * c4, (cfirst + c4) * 8));
        }
        {
            uint32_t r[8];
            const int cl = chalf == 0 ? c0 + 8 : c0;                                  // the remaining chunk
            tmem_ld_32x8(trow + (uint32_t)(cl * 8), r);
            tmem_ld_wait();
            store_chunk(cl, convert8(r, cl * 8));
        }
    }
}

}  // namespace qc
}  // namespace mta
