// Scaled scores Q K^T and the first causal depthwise conv in one kernel: the score tile a conv tile needs is computed
// into tensor memory, rounded and written straight into the staged shared-memory tile the conv's MMAs read, so the
// score planes are never written to or read from HBM (mta_attention_triton.py:68-73 as one pass).
//
// Per output tile (TMO = 129 - R query rows x 128 keys) of the conv:
//   staged score tile  rows m0-(R-1) .. m0+TMO-1 (exactly 128), keys n0-8 .. n0+135 (144)
//                      S = Q[rows] . K[keys]^T : 8 (D = 128) tcgen05.mma of M128 N144 K16 into TMEM columns 256..399
//   drain (4 warps)    TMEM -> round(round(S) * scale) as the reference's 16-bit matmul and multiply do -> 0 where
//                      key > query -> the swizzled K-major layout of conv2d_tc05.cu (two 64-key boxes with the 128-byte
//                      swizzle, one 16-key box with the 32-byte swizzle).  Rows and keys outside the plane come out 0
//                      because TMA zero-fills Q / K there: that is the conv's zero padding.
//   conv               the MMA schedule of conv2d_tc05.cu (row tap = descriptor address advanced by whole rows; two
//                      issuers owning disjoint output blocks) into TMEM accumulator n % 2.  Row taps i > 0 read up to
//                      R-1 rows past the 128 staged ones; those only reach output rows >= TMO, which are not stored.
//   epilogue (8 warps) TMEM -> 16-bit -> swizzled staging tile -> TMA store of TMO rows.
// Warps: 0 TMA producer (Q tile per row of tiles, K tile per tile, double-buffered), 1 score-MMA issuer, 2-3 conv-MMA
// issuers, 4-7 and 16-19 drain, 8-15 epilogue.  16-bit dtypes, D in {64, 128}, odd key extent <= 17, causal.
#include <cstdlib>

#include "kernels.cuh"
#include "tc05.cuh"

namespace mta {
namespace {
using namespace tc05;

// Per-role cycle counters of CTA 0, compiled in only with -DMTA_QC_PROFILE and printed by the launcher when the
// environment variable MTA_QC_PROFILE is set.
#ifdef MTA_QC_PROFILE
__device__ long long g_qc_prof[32];
#define QP_DECL long long qp_loc[4] = {0, 0, 0, 0}; long long qp_t = clock64();
#define QP_ACC(slot) { const long long qp_n = clock64(); qp_loc[(slot) & 3] += qp_n - qp_t; qp_t = qp_n; }
#define QP_FLUSH(base, cond) if (blockIdx.x == 0 && lane == 0 && (cond)) for (int pi = 0; pi < 4; ++pi) g_qc_prof[(base) + pi] = qp_loc[pi];
#else
#define QP_DECL
#define QP_ACC(slot)
#define QP_FLUSH(base, cond)
#endif

constexpr int TM = 128;            // staged rows = MMA M
constexpr int TN = 128;            // output columns per tile
constexpr int NB = TN / 16;
constexpr int NKS = 9;             // k-steps of 16 staged columns
constexpr int SN = 144;            // staged columns = N of the score MMA
constexpr int BOX_BYTES = TM * 128;               // one 64-column box of the staged tile: 128 rows x 128 bytes
constexpr int BOX3_BYTES = TM * 32;               // the 16-column box
constexpr int OUT_BYTES = 2 * TM * 128;           // output staging: two 64-column boxes
constexpr int KBOX_BYTES = SN * 128;              // one 64-element box of the K tile: 144 rows x 128 bytes (18 KB)
// Drain warps: 4 (warps 4-7, a thread converts its whole staged row) or 8 (warps 16-19 take staged columns 72..143).
// Measured at B8 H16 S4096 D128, 6 x 11: 4 warps with sleeping waits 1.26 ms, 8 warps with spinning waits 1.35 ms - the
// kernel is bound by shared-memory bandwidth (the conv MMAs' operand reads, ~300 KB per tile, plus ~200 KB of tile
// traffic), and extra polling and extra warps only add to it.
constexpr int DRAIN_WARPS = 4;
constexpr int THREADS = DRAIN_WARPS == 4 ? 512 : 640;
constexpr uint32_t S_COL = 256;                   // TMEM column of the score accumulator (conv accumulators: 0..255)

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

struct QcGeom {
    int C, S, R, KS, row_begin, row_end, tiles_n, tiles_m, tmo, split_w, y_row0;
    float scale;
    long tiles_per_plane, total_tiles;
};

__device__ __forceinline__ int qc_key_tiles(const QcGeom& g, int tm) {
    const int q_last = min(g.row_begin + (tm + 1) * g.tmo, g.row_end);
    return min((q_last + TN - 1) / TN, g.tiles_n);
}

struct QcIter {
    int plane, tm, tn, nk;
    __device__ void init(const QcGeom& g, long t) {
        plane = (int)(t / g.tiles_per_plane);
        int r = (int)(t - (long)plane * g.tiles_per_plane);
        for (tm = 0;; ++tm) {
            nk = qc_key_tiles(g, tm);
            if (r < nk) break;
            r -= nk;
        }
        tn = r;
    }
    // returns true when the walk moved on to another row of tiles (another Q tile)
    __device__ bool next(const QcGeom& g) {
        if (++tn == nk) {
            tn = 0;
            if (++tm == g.tiles_m) { tm = 0; ++plane; }
            nk = qc_key_tiles(g, tm);
            return true;
        }
        return false;
    }
    __device__ int m0(const QcGeom& g) const { return g.row_begin + tm * g.tmo; }
    __device__ int n0() const { return tn * TN; }
};

// The conv MMAs of one tile for issuer ISSUER (blocks [b0, b1] of the eight 16-column output blocks): see
// conv2d_tc05.cu for the schedule.
template <typename T, int ISSUER>
__device__ __forceinline__ void issue_conv(uint32_t xa_addr, uint32_t d0, int R, int split_w, int tb_off) {
    constexpr uint32_t idesc32 = instr_desc_f16(AbFmtQ<T>::value, 0, 0, TM, 32);
    constexpr uint32_t idesc16 = instr_desc_f16(AbFmtQ<T>::value, 0, 0, TM, 16);
    constexpr int b0 = ISSUER == 0 ? 0 : 4, b1 = ISSUER == 0 ? 3 : 7;
    const uint64_t da0 = smem_desc_sw128(xa_addr, 16, 1024);
    const uint64_t da3 = smem_desc_sw32(xa_addr + (uint32_t)(2 * BOX_BYTES), 256);
    const uint64_t db0 = desc_plain(xa_addr + (uint32_t)tb_off, 512, 128);
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

template <typename T, int D>
__global__ void __launch_bounds__(THREADS, 1)
qk_conv_tc05_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                    const __grid_constant__ CUtensorMap my, const void* __restrict__ w, int w_dtype, QcGeom g, int* err_flag) {
    constexpr int DBOX = D / 64;                               // 64-element boxes along the head dimension
    constexpr int Q_BYTES = DBOX * BOX_BYTES;                  // Q tile: 128 rows x D
    constexpr int K_BYTES = DBOX * KBOX_BYTES;                 // K tile: 144 keys x D
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t q_full, q_free, k_full[2], k_free[2], s_full, s_free, ready_bar[2], empty_bar[2],
        acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int R = g.R, KS = g.KS;
    const int tb_bytes = (R * 1024 * (g.split_w ? 2 : 1) + 1023) & ~1023;
    const int tb_off = 2 * BOX_BYTES + ((BOX3_BYTES + 1023) & ~1023);
    const int stage_bytes = tb_off + tb_bytes;                 // staged score tile + Toeplitz slices
    uint8_t* out_base = smem;
    uint8_t* q_base = out_base + OUT_BYTES;
    uint8_t* k_base = q_base + Q_BYTES;
    uint8_t* stage_base = k_base + 2 * K_BYTES;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pad_w = (KS - 1) / 2;
    const int a_off = 8 - pad_w;
    const int lead = R - 1;

    const long per = (g.total_tiles + gridDim.x - 1) / gridDim.x;
    const long t_begin = (long)blockIdx.x * per;
    const long t_end = min(t_begin + per, g.total_tiles);
    const int my_tiles = t_end > t_begin ? (int)(t_end - t_begin) : 0;

    if (tid == 0) abort_flag = *reinterpret_cast<volatile int*>(err_flag);
    __syncthreads();
    if (abort_flag != 0 || my_tiles == 0) return;

    if (warp == 0) {
        if (lane == 0) {
            mbar_init(&q_full, 1);
            mbar_init(&q_free, 1);
            mbar_init(&s_full, 1);
            mbar_init(&s_free, DRAIN_WARPS);
            for (int i = 0; i < 2; ++i) {
                mbar_init(&k_full[i], 1);
                mbar_init(&k_free[i], 1);
                mbar_init(&ready_bar[i], DRAIN_WARPS);
                mbar_init(&empty_bar[i], 2);
                mbar_init(&acc_full[i], 2);
                mbar_init(&acc_empty[i], 8);
            }
            fence_mbar_init();
            prefetch_tensormap(&mq);
            prefetch_tensormap(&mk);
            prefetch_tensormap(&my);
        }
        __syncwarp();
        tmem_alloc(&tmem_slot, 512);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        // ---------------- producer: Q tile per row of tiles, K tile per tile ----------------
        if (lane == 0) {
            QcIter it;
            it.init(g, t_begin);
            bool new_q = true;
            int qn = 0;                                        // Q tiles loaded so far
            for (int n = 0; n < my_tiles; ++n) {
                if (new_q) {
                    // the score MMAs of the previous row of tiles have finished reading the Q tile
                    mbar_wait(&q_free, (qn & 1) ^ 1, err_flag);
                    mbar_expect_tx(&q_full, (uint32_t)Q_BYTES);
#pragma unroll
                    for (int j = 0; j < DBOX; ++j) tma_load_3d(q_base + j * BOX_BYTES, &mq, &q_full, 64 * j, it.m0(g) - lead, it.plane);
                    ++qn;
                }
                const int ks = n & 1;
                mbar_wait(&k_free[ks], ((n >> 1) & 1) ^ 1, err_flag);
                mbar_expect_tx(&k_full[ks], (uint32_t)K_BYTES);
#pragma unroll
                for (int j = 0; j < DBOX; ++j)
                    tma_load_3d(k_base + ks * K_BYTES + j * KBOX_BYTES, &mk, &k_full[ks], 64 * j, it.n0() - 8, it.plane);
                new_q = it.next(g);
            }
        }
    } else if (warp == 1) {
        // ---------------- score MMAs: S[128 x 144] = Q K^T into TMEM columns S_COL.. ----------------
        constexpr uint32_t idesc = instr_desc_f16(AbFmtQ<T>::value, 0, 0, TM, SN);
        QcIter it;
        it.init(g, t_begin);
        bool new_q = true;
        int qn = 0;
        QP_DECL
        for (int n = 0; n < my_tiles; ++n) {
            const int ks = n & 1;
            if (new_q) {
                mbar_wait(&q_full, qn & 1, err_flag);
                ++qn;
            }
            mbar_wait(&k_full[ks], (n >> 1) & 1, err_flag);
            QP_ACC(0)
            mbar_wait(&s_free, (n & 1) ^ 1, err_flag);           // the drain warps have read the previous score tile
            QP_ACC(1)
            fence_after_sync();
            new_q = it.next(g);
            if (lane == 0) {
                const uint32_t qa = smem_u32(q_base), ka = smem_u32(k_base + ks * K_BYTES);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t qoff = (kk / 4) * BOX_BYTES + (kk % 4) * 32, koff = (kk / 4) * KBOX_BYTES + (kk % 4) * 32;
                    mma_f16_ss(tmem + S_COL, smem_desc_sw128(qa + qoff, 16, 1024), smem_desc_sw128(ka + koff, 16, 1024), idesc,
                               kk > 0 ? 1u : 0u);
                }
                mma_commit(&k_free[ks]);
                mma_commit(&s_full);
                if (new_q || n == my_tiles - 1) mma_commit(&q_free);     // last tile of this row of tiles
            }
            __syncwarp();
            QP_ACC(2)
        }
        QP_FLUSH(0, true)
    } else if (warp == 2 || warp == 3) {
        // ---------------- conv MMAs ----------------
        QP_DECL
        for (int n = 0; n < my_tiles; ++n) {
            const int st = n & 1, ab = n & 1;
            mbar_wait(&ready_bar[st], (n >> 1) & 1, err_flag);
            QP_ACC(0)
            mbar_wait(&acc_empty[ab], ((n >> 1) & 1) ^ 1, err_flag);
            QP_ACC(1)
            fence_after_sync();
            if (lane == 0) {
                const uint32_t xa_addr = smem_u32(stage_base + st * stage_bytes);
                const uint32_t d0 = tmem + (uint32_t)(ab * TN);
                if (warp == 2) issue_conv<T, 0>(xa_addr, d0, R, g.split_w, tb_off);
                else issue_conv<T, 1>(xa_addr, d0, R, g.split_w, tb_off);
                mma_commit(&empty_bar[st]);
                mma_commit(&acc_full[ab]);
            }
            __syncwarp();
            QP_ACC(2)
        }
        QP_FLUSH(4, warp == 2)
    } else if (warp < 8 || warp >= 16) {
        // ---------------- drain: score tile TMEM -> rounded, scaled, masked -> staged tile; Toeplitz slices ----------------
        const int quarter = warp & 3;
        const int first_half = warp >= 16 ? 1 : 0;           // first half of the staged columns this warp converts
        const int sr = quarter * 32 + lane;                  // staged row = TMEM lane of this thread
        const int ft = warp < 8 ? tid - 128 : tid - 512 + 128;   // 0..255
        const float sc = round_to<T>(g.scale);
        QcIter it;
        it.init(g, t_begin);
        int ph0 = -1, ph1 = -1;                              // head whose Toeplitz slices each stage holds
        QP_DECL
        for (int n = 0; n < my_tiles; ++n, it.next(g)) {
            const int st = n & 1;
            const int m0 = it.m0(g), n0 = it.n0();
            const int head = it.plane % g.C;
            uint8_t* xa = stage_base + st * stage_bytes;
            const uint32_t xa_s = smem_u32(xa);
            // the stage is free once the conv MMAs of tile n - 2 are done
            mbar_wait(&empty_bar[st], ((n >> 1) & 1) ^ 1, err_flag);
            QP_ACC(0)
            int ph;
            if (st == 0) { ph = ph0; ph0 = head; } else { ph = ph1; ph1 = head; }
            if (ph != head) {
                uint8_t* tb = xa + tb_off;
                const int total = R * 512;
                for (int idx = ft; idx < total; idx += DRAIN_WARPS * 32) {
                    const int i = idx / 512, e = idx % 512;
                    const int nn = e / 16, kk = e % 16;
                    const int j = kk + 16 - nn - a_off;
                    const float wv = (j >= 0 && j < KS) ? load_weight(w, ((long)head * R + i) * KS + j, w_dtype) : 0.0f;
                    const T hi = from_f32<T>(wv);
                    const int off = i * 1024 + (kk / 8) * 512 + (nn / 8) * 128 + (nn % 8) * 16 + (kk % 8) * 2;
                    *reinterpret_cast<T*>(tb + off) = hi;
                    if (g.split_w) *reinterpret_cast<T*>(tb + R * 1024 + off) = from_f32<T>(wv - to_f32<T>(hi));
                }
            }
            QP_ACC(1)
            mbar_wait(&s_full, n & 1, err_flag);
            QP_ACC(2)
            __syncwarp();
            fence_after_sync();
            const int qq = m0 - lead + sr;                   // query of this staged row
            const int kbase = n0 - 8;                        // key of staged column 0
            const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16) + S_COL;
            auto convert8 = [&](const uint32_t* r, int col) -> uint4 {      // staged columns col .. col + 7
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    f[e] = round_to<T>(__uint_as_float(r[e])) * sc;
                    if (kbase + col + e > qq) f[e] = 0.0f;
                }
                return make_uint4(pack2q<T>(f[0], f[1]), pack2q<T>(f[2], f[3]), pack2q<T>(f[4], f[5]), pack2q<T>(f[6], f[7]));
            };
            auto store_chunk = [&](int ch, const uint4& v) {     // chunk ch = staged columns 8 ch .. 8 ch + 7
                if (ch < 16) sts128q(xa_s + (uint32_t)((ch >> 3) * BOX_BYTES + sr * 128 + (((ch & 7) ^ (sr & 7)) << 4)), v);
                else sts128q(xa_s + (uint32_t)(2 * BOX_BYTES + sr * 32 + ((((ch - 16) ^ (sr >> 2)) & 1) << 4)), v);
            };
            // nine chunks at a time: 0..8 (columns 0..71) then / or 9..17 (columns 72..143), as loads of 32 + 32 + 8 columns
#pragma unroll 1
            for (int chalf = first_half; chalf < 2; chalf += DRAIN_WARPS / 4) {
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
            fence_before_sync();
            fence_proxy_async();          // generic-proxy writes above must be visible to the MMAs (async proxy)
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&s_free);
                mbar_arrive(&ready_bar[st]);
            }
            QP_ACC(3)
        }
        QP_FLUSH(8, warp == 4)
    } else {
        // ---------------- epilogue: warps 8-11 take columns 0..63, warps 12-15 columns 64..127 ----------------
        const int quarter = warp & 3;
        const int half = warp >= 12 ? 1 : 0;
        const bool issuer = (warp == 8 && lane == 0);
        const int row = quarter * 32 + lane;
        QcIter it;
        it.init(g, t_begin);
        QP_DECL
        for (int n = 0; n < my_tiles; ++n, it.next(g)) {
            const int ab = n & 1;
            const int plane = it.plane, m0 = it.m0(g), n0 = it.n0();
            uint8_t* orow = out_base + half * (TM * 128) + row * 128;
            mbar_wait(&acc_full[ab], (n >> 1) & 1, err_flag);
            QP_ACC(0)
            __syncwarp();
            fence_after_sync();
            if (issuer) bulk_wait_read();                    // the previous tile's store has finished reading the staging tile
            named_barrier(1, 256);
            QP_ACC(1)
            const int q = m0 + row;
#pragma unroll
            for (int cblk = 0; cblk < 2; ++cblk) {
                uint32_t r[32];
                tmem_ld_32x32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ab * TN + half * 64 + cblk * 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int v8 = 0; v8 < 4; ++v8) {
                    const int col = cblk * 32 + v8 * 8;
                    const int k = n0 + half * 64 + col;
                    float f[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v8 * 8 + e]);
                    if (k + 7 > q) {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (k + e > q) f[e] = 0.0f;
                    }
                    uint4 o;
                    o.x = pack2q<T>(f[0], f[1]);
                    o.y = pack2q<T>(f[2], f[3]);
                    o.z = pack2q<T>(f[4], f[5]);
                    o.w = pack2q<T>(f[6], f[7]);
                    *reinterpret_cast<uint4*>(orow + (((col >> 3) ^ (row & 7)) << 4)) = o;
                }
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[ab]);
            QP_ACC(2)
            fence_proxy_async();
            named_barrier(1, 256);
            if (issuer) {
                // the store's box has TMO rows; rows past row_end and columns past S are clipped by the tensor map
                tma_store_3d(&my, out_base, n0, m0 - g.y_row0, plane);
                if (n0 + 64 < g.S) tma_store_3d(&my, out_base + TM * 128, n0 + 64, m0 - g.y_row0, plane);
                bulk_commit();
            }
            QP_ACC(3)
        }
        QP_FLUSH(12, warp == 8)
        if (issuer) bulk_wait_all();
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

size_t qk_conv_smem_bytes(int D, int R, bool split_w) {
    const size_t tb = (size_t)((R * 1024 * (split_w ? 2 : 1) + 1023) & ~1023);
    const size_t stage = 2 * BOX_BYTES + ((BOX3_BYTES + 1023) & ~1023) + tb;
    return 1024 + OUT_BYTES + (size_t)(D / 64) * BOX_BYTES + 2 * (size_t)(D / 64) * KBOX_BYTES + 2 * stage;
}

template <typename T, int D>
int launch_qc(const void* q, const void* k, const void* w, int w_dtype, void* y, PlaneView yv, int B, int H, int S, int R, int KS,
              float scale, int row_begin, int row_end, cudaStream_t st) {
    const long planes = (long)B * H;
    QcGeom g{};
    g.C = H; g.S = S; g.R = R; g.KS = KS; g.row_begin = row_begin; g.row_end = row_end; g.scale = scale;
    g.tmo = TM - (R - 1);
    g.tiles_n = (S + TN - 1) / TN;
    g.tiles_m = (row_end - row_begin + g.tmo - 1) / g.tmo;
    g.split_w = w_dtype == MTA_F32 ? 1 : 0;
    g.y_row0 = yv.row0;
    long per_plane = 0;
    for (int tm = 0; tm < g.tiles_m; ++tm) {
        const int q_last = std::min(row_begin + (tm + 1) * g.tmo, row_end);
        per_plane += std::min((q_last + TN - 1) / TN, g.tiles_n);
    }
    g.tiles_per_plane = per_plane;
    g.total_tiles = per_plane * planes;
    CUtensorMap mq, mk, my;
    int rc;
    if ((rc = make_tensor_map_3d(&mq, q, (uint64_t)planes, S, D, D, (uint64_t)S * D, 64, TM, true))) return rc;
    if ((rc = make_tensor_map_3d(&mk, k, (uint64_t)planes, S, D, D, (uint64_t)S * D, 64, SN, true))) return rc;
    if ((rc = make_tensor_map_3d(&my, y, (uint64_t)planes, (uint64_t)(row_end - yv.row0), S, (uint64_t)yv.width,
                                 (uint64_t)yv.plane_stride, 64, (uint32_t)g.tmo, true)))
        return rc;
    int* flag = nullptr;
    if ((rc = wait_flag_ptr(&flag))) return rc;
    int dev = 0, sms = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const size_t smem = qk_conv_smem_bytes(D, R, g.split_w != 0);
    MTA_CUDA_OK(cudaFuncSetAttribute(qk_conv_tc05_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const unsigned grid = (unsigned)std::min<long>(g.total_tiles, sms);
    qk_conv_tc05_kernel<T, D><<<grid, THREADS, smem, st>>>(mq, mk, my, w, w_dtype, g, flag);
    MTA_LAUNCH_OK("qk_conv_tc05_kernel");
#ifdef MTA_QC_PROFILE
    if (getenv("MTA_QC_PROFILE")) {
        cudaDeviceSynchronize();
        long long h[32], z[32] = {};
        cudaMemcpyFromSymbol(h, g_qc_prof, sizeof(h));
        cudaMemcpyToSymbol(g_qc_prof, z, sizeof(z));
        const long n0 = (g.total_tiles + grid - 1) / grid;
        fprintf(stderr, "qk_conv clk/tile (CTA 0, %ld tiles): score wait_kq %lld wait_s_free %lld issue %lld | conv wait_ready %lld wait_acc %lld "
                "issue %lld | drain wait_stage %lld toeplitz %lld wait_s_full %lld convert %lld | epilogue wait_acc %lld wait_store %lld drain %lld store %lld\n",
                n0, h[0] / n0, h[1] / n0, h[2] / n0, h[4] / n0, h[5] / n0, h[6] / n0, h[8] / n0, h[9] / n0, h[10] / n0, h[11] / n0,
                h[12] / n0, h[13] / n0, h[14] / n0, h[15] / n0);
    }
#endif
    return MTA_OK;
}

}  // namespace

bool qk_conv_supported(const void* q, const void* k, const void* y, PlaneView yv, int S, int D, int R, int KS, int causal, int dtype,
                       int w_dtype) {
    return causal && dtype != MTA_F32 && (D == 64 || D == 128) && S % 8 == 0 && KS % 2 == 1 && KS <= 17 && R >= 1 && R <= 16 &&
           qk_conv_smem_bytes(D, R, w_dtype == MTA_F32) <= 225 * 1024 && yv.width == S && yv.plane_stride % 8 == 0 && aligned16(q) &&
           aligned16(k) && aligned16(y);
}

int qk_conv_launch(const void* q, const void* k, const void* w, int w_dtype, void* y, PlaneView yv, int B, int H, int S, int D,
                   int R, int KS, float scale, int row_begin, int row_end, int dtype, cudaStream_t st) {
    if ((long)B * H == 0 || row_end <= row_begin) return MTA_OK;
#define MTA_QC(TT, DD) return launch_qc<TT, DD>(q, k, w, w_dtype, y, yv, B, H, S, R, KS, scale, row_begin, row_end, st)
    if (dtype == MTA_BF16) { if (D == 64) MTA_QC(__nv_bfloat16, 64); MTA_QC(__nv_bfloat16, 128); }
    if (D == 64) MTA_QC(__half, 64);
    MTA_QC(__half, 128);
#undef MTA_QC
}

}  // namespace mta
