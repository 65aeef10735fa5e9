// Depthwise causal conv over score planes on the tcgen05 tensor cores, 16-bit dtypes, key extent S <= 17.
//
// Toeplitz formulation (as in conv2d_mma.cu): for a fixed row tap i the key-direction taps form a banded matrix,
//   out[q, k] += sum_kk X[q + i - (R-1), kk] * T_i[kk, k],   T_i[kk, k] = w[i, kk - k + pad_w]  (0 outside the band)
// so every row tap and every block of 16 output columns costs two tcgen05 MMAs (M = 128 query rows, N = 16,
// K = 16) of the staged input tile (rows shifted by i) against the two 16x16 slices of T_i.  The legacy mma.sync
// pipe saturates on this op (measured); tcgen05 does not.
//
// Persistent, warp-specialised kernel: one CTA per SM walks a contiguous range of 128 x 128 output tiles
// (only tiles that touch keys <= query when causal):
//   warp 0      TMA producer: two 64-column boxes (128-byte swizzle) and one 16-column box (32-byte swizzle) per tile
//               bring the (128 + R-1) x 144 halo tile straight into the swizzled K-major layouts the MMA reads (3-stage ring; out-of-range rows / columns arrive as
//               zero = the conv's zero padding)
//   warps 2-3, 14-15  zero the keys above the causal diagonal in the staged tile (diagonal tiles only); rebuild the
//               Toeplitz slices when the head changes
//   warps 1, 8  issue the MMAs into TMEM accumulator n % 2; each issuer owns half of the 16-column output blocks,
//               so every output element is accumulated by one thread in program order and the result does not
//               depend on how the issuers interleave (60 MMAs per tile for a 6 x 11 kernel)
//   warp 9      stores the zero tiles above the diagonal when the whole output is wanted
//   warps 4-7, 10-13  epilogue (64 columns each): TMEM -> registers -> 16-bit -> swizzled shared-memory tile (double
//               buffered) -> TMA tiled store (a thread owns one output row, so direct global stores would touch 32
//               different lines per instruction)
//
// MMA schedule.  Staged column sc holds key n0 - 8 + sc; output column x reads staged columns x + a_off + j
// (a_off = 8 - pad_w).  A k-step is 16 staged columns [16 s, 16 s + 16), s = 0..8; it contributes to the two
// 16-column output blocks s-1 and s, so there is one MMA (M = 128 rows, N = 32, K = 16) per (row tap i, k-step s):
//   A = staged rows i .. i+127, columns 16 s .. 16 s + 15.  In the swizzled layout a row is 128 bytes and the swizzle
//       is a function of the shared-memory address alone, so a row tap is just the descriptor's start address
//       advanced by i * 128 bytes (measured: correct for every i with the base-offset field left at 0);
//   B = the 32 x 16 Toeplitz slice of row tap i, element (n', kk) = w[i][kk + 16 - n' - a_off] - the same for every s.
// The first and last k-step touch one block only (N = 16, half of the slice), and so do the k-steps at the edge of
// an issuer's block range (the neighbouring issuer covers the other half).  For i = 0 an issuer first issues, with
// accumulate = 0, k-steps that touch each of its blocks exactly once, then the others.  Measured: at M = 128 a
// tcgen05.mma costs ~44 cycles for any N <= 64, which is why the schedule minimises the MMA count, not the MACs.
#include "kernels.cuh"
#include "tc05.cuh"

namespace mta {

int make_tensor_map_chunked(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols,
                            uint64_t row_pitch_elems, uint64_t plane_pitch_elems, uint32_t box_rows, uint32_t box_chunks);

namespace {
using namespace tc05;

constexpr int TM = 128;            // output rows per tile = MMA M
constexpr int TN = 128;            // output columns per tile
constexpr int NB = TN / 16;        // 16-column blocks
constexpr int NKS = 9;             // k-steps of 16 staged columns: 8 (left halo) + 128 + 8
constexpr int NCH = 2 * NKS;       // staged 8-column chunks
constexpr int NBOX = 2;            // 64-column TMA boxes per staged tile (128-byte swizzle); a third box of 16 columns
                                   // (32-byte swizzle) holds the last k-step
constexpr int NSTAGE = 3;
constexpr int OUT_BYTES = 2 * TM * 128;   // output staging: two 64-column boxes of 128 rows x 128 bytes, 128-byte swizzle
constexpr int NISS = 2;               // MMA-issuing threads (warps 1, 8)
constexpr int ZERO_WARP = 9;          // the warp that stores the zero tiles above the diagonal
// First 16-column output block of issuer k (two issuers: blocks 0-3 and 4-7).
__host__ __device__ constexpr int issuer_block0(int k) { return NISS == 1 ? (k == 0 ? 0 : NB) : (k == 0 ? 0 : k == 1 ? 4 : NB); }
constexpr int THREADS = 512;       // warps: 0 producer, 1 and 8 MMA issuers, 9 zero tiles, 2-3 and 14-15 tile fix-up, 4-7 and 10-13 epilogue

template <typename T> struct AbFmt;
template <> struct AbFmt<__nv_bfloat16> { static constexpr int value = 1; };
template <> struct AbFmt<__half> { static constexpr int value = 0; };

template <typename T> __device__ __forceinline__ uint32_t pack2c(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2c<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t pack2c<__half>(float lo, float hi) {
    __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}

// Matrix descriptor without swizzle: lbo = bytes between the two 8-element k chunks of one MMA, sbo = bytes
// between groups of 8 rows.
__device__ __forceinline__ uint64_t smem_desc_plain(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

struct ConvGeom {
    int C, W, R, S, causal, row_begin, row_end, tiles_n, tiles_m, x_row0, write_upper, split_w;
    int lead;          // staged rows start `lead` rows before the tile: R-1 for the conv (row taps look back), 0 for its
                       // input gradient (taps reversed, looking forward)
    int flip;          // input gradient: tap (i, j) uses w[R-1-i][S-1-j]
    long tiles_per_plane, total_tiles;
    long zero_per_plane, zero_total;     // tiles wholly above the diagonal that must be written as zero (write_upper)
};

// Key tiles that query tile tm reaches.
__device__ __forceinline__ int conv_key_tiles(const ConvGeom& g, int tm) {
    if (!g.causal) return g.tiles_n;
    const int q_last = min(g.row_begin + (tm + 1) * TM, g.row_end);
    return min((q_last + TN - 1) / TN, g.tiles_n);
}

// Walks consecutive tile indices without re-deriving (plane, row tile, column tile) from scratch.
struct TileIter {
    int plane, tm, tn, nk;
    __device__ void init(const ConvGeom& g, long t) {
        plane = (int)(t / g.tiles_per_plane);
        int r = (int)(t - (long)plane * g.tiles_per_plane);
        for (tm = 0;; ++tm) {
            nk = conv_key_tiles(g, tm);
            if (r < nk) break;
            r -= nk;
        }
        tn = r;
    }
    __device__ void next(const ConvGeom& g, int tiles_m) {
        if (++tn == nk) {
            tn = 0;
            if (++tm == tiles_m) { tm = 0; ++plane; }
            nk = conv_key_tiles(g, tm);
        }
    }
    __device__ int m0(const ConvGeom& g) const { return g.row_begin + tm * TM; }
    __device__ int n0() const { return tn * TN; }
};

// The MMAs of one tile that issuer ISSUER is responsible for.  It owns output blocks [b0, b1]; the k-steps that
// reach them are b0 .. b1 + 1.  k-step s is an N = 32 MMA onto blocks s-1 and s, except at the two ends of the range,
// where only one half of the Toeplitz slice is used (N = 16): rows 16..31 (+256 bytes) onto block b0 for s = b0, rows
// 0..15 onto block b1 for s = b1 + 1.  Per (row tap i, term) the k-steps b0+1, b0+3, ... come first: they touch every
// owned block exactly once, so in the first batch they carry accumulate = 0.
template <typename T, int ISSUER>
__device__ __forceinline__ void issue_tile(uint32_t xa_addr, uint32_t d0, int R, int split_w, int box_bytes, int tb_off) {
    constexpr uint32_t idesc32 = instr_desc_f16(AbFmt<T>::value, 0, 0, TM, 32);
    constexpr uint32_t idesc16 = instr_desc_f16(AbFmt<T>::value, 0, 0, TM, 16);
    constexpr int b0 = issuer_block0(ISSUER), b1 = issuer_block0(ISSUER + 1) - 1;
    const uint64_t da0 = smem_desc_sw128(xa_addr, 16, 1024);
    const uint64_t da3 = smem_desc_sw32(xa_addr + (uint32_t)(NBOX * box_bytes), 256);   // the last k-step: 32-byte-row box
    const uint64_t db0 = smem_desc_plain(xa_addr + (uint32_t)tb_off, 512, 128);        // k chunks 512 bytes apart, 8-row groups 128
    const int parts = split_w ? 2 : 1;
    int batch = 0;
#pragma unroll 1
    for (int i = 0; i < R; ++i)
#pragma unroll 1
        for (int part = 0; part < parts; ++part, ++batch) {
            const uint64_t db = db0 + (uint64_t)((i * 1024 + part * R * 1024) >> 4);
            const uint64_t da = da0 + (uint64_t)((i * 128) >> 4);      // a row tap is the start address advanced by i rows
            const uint64_t dl = da3 + (uint64_t)((i * 32) >> 4);
#pragma unroll
            for (int pass = 0; pass < 2; ++pass)
#pragma unroll
                for (int s = b0 + 1 - pass; s <= b1 + 1; s += 2) {
                    const bool upper = s == b0, lower = s == b1 + 1;
                    // k-steps 0..7 live in the two 128-byte-row boxes (four per box), k-step 8 in the 32-byte-row box
                    const uint64_t adesc = s < 8 ? da + (uint64_t)(((s / 4) * box_bytes + (s % 4) * 32) >> 4) : dl;
                    const uint64_t bdesc = db + (upper ? 16u : 0u);
                    const uint32_t dcol = upper ? 16u * (uint32_t)s : 16u * (uint32_t)(s - 1);
                    const uint32_t acc = (batch > 0 || pass > 0) ? 1u : 0u;
                    mma_f16_ss(d0 + dcol, adesc, bdesc, (upper || lower) ? idesc16 : idesc32, acc);
                }
        }
}

template <typename T>
__global__ void __launch_bounds__(THREADS, 1)
conv2d_tc05_kernel(const __grid_constant__ CUtensorMap mx, const __grid_constant__ CUtensorMap mx3,
                   const __grid_constant__ CUtensorMap my,
                   const void* __restrict__ w, int w_dtype, int y_row0, ConvGeom g, int* err_flag) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t full_bar[NSTAGE], ready_bar[NSTAGE], empty_bar[NSTAGE], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ int tiles_loaded;               // compute tiles whose loads the producer has issued (paces the zero tiles)
    const int R = g.R, S = g.S;
    const int TH = TM + R - 1;
    const int box_bytes = (TH * 128 + 1023) & ~1023;          // one 64-column box, 1024-byte aligned (swizzle period)
    const int tb_bytes = (R * 1024 * (g.split_w ? 2 : 1) + 1023) & ~1023;   // Toeplitz slices: 32 x 16 per row tap
    const int box3_bytes = (TH * 32 + 1023) & ~1023;          // the 16-column box: rows of 32 bytes
    const int tb_off = NBOX * box_bytes + box3_bytes;         // Toeplitz slices follow the boxes
    const int stage_bytes = tb_off + tb_bytes;
    uint8_t* out_base = smem;                                  // 1024-byte aligned, as the swizzled TMA store needs
    uint8_t* zero_box = smem + 2 * OUT_BYTES;                 // 16 KB of zeros: source of the zero tiles above the diagonal
    uint8_t* stage_base = zero_box + TM * 128;                // then the stage ring
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pad_w = (S - 1) / 2;
    const int pad8 = (pad_w + 7) & ~7;
    const int a_off = pad8 - pad_w;

    // contiguous range of tiles for this CTA
    const long per = (g.total_tiles + gridDim.x - 1) / gridDim.x;
    const long t_begin = (long)blockIdx.x * per;
    const long t_end = min(t_begin + per, g.total_tiles);
    const int my_tiles = t_end > t_begin ? (int)(t_end - t_begin) : 0;

    if (tid == 0) tiles_loaded = 0;
    if (tid == 0) abort_flag = *reinterpret_cast<volatile int*>(err_flag);
    __syncthreads();
    if (abort_flag != 0 || my_tiles == 0) return;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < NSTAGE; ++i) {
                mbar_init(&full_bar[i], 1);
                mbar_init(&ready_bar[i], 4);
                mbar_init(&empty_bar[i], NISS);
            }
            for (int i = 0; i < 2; ++i) {
                mbar_init(&acc_full[i], NISS);
                mbar_init(&acc_empty[i], 8);
            }
            fence_mbar_init();
            prefetch_tensormap(&mx);
            prefetch_tensormap(&my);
        }
        __syncwarp();
        tmem_alloc(&tmem_slot, 2 * TN);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            TileIter it;
            it.init(g, t_begin);
            for (int n = 0; n < my_tiles; ++n, it.next(g, g.tiles_m)) {
                const int st = n % NSTAGE;
                mbar_wait(&empty_bar[st], ((n / NSTAGE) & 1) ^ 1, err_flag);
                uint8_t* xa = stage_base + st * stage_bytes;
                mbar_expect_tx(&full_bar[st], (uint32_t)(NBOX * TH * 128 + TH * 32));
#pragma unroll
                for (int j = 0; j < NBOX; ++j)
                    tma_load_3d(xa + j * box_bytes, &mx, &full_bar[st], it.n0() - pad8 + 64 * j, it.m0(g) - g.lead - g.x_row0,
                                it.plane);
                tma_load_3d(xa + NBOX * box_bytes, &mx3, &full_bar[st], it.n0() - pad8 + 128, it.m0(g) - g.lead - g.x_row0, it.plane);
                *reinterpret_cast<volatile int*>(&tiles_loaded) = n + 1;
            }
        }
    } else if (warp == ZERO_WARP) {
        // ---------------- zero tiles ----------------
        // The tiles wholly above the diagonal are part of the output the API returns: this warp writes its share of
        // them as TMA stores of a zero box, in step with the producer's progress through the compute tiles, so the two
        // kinds of traffic overlap for the whole run instead of the zero stores flooding the memory system first.
        const long active = (g.total_tiles + per - 1) / per;      // CTAs that own compute tiles (the others have returned)
        const long zper = (g.zero_total + active - 1) / active;
        const long z_begin = min((long)blockIdx.x * zper, g.zero_total), z_end = min(z_begin + zper, g.zero_total);
        const long my_zero = z_end - z_begin;
        if (my_zero > 0) {
            for (int i = lane; i < TM * 128 / 16; i += 32) reinterpret_cast<uint4*>(zero_box)[i] = make_uint4(0u, 0u, 0u, 0u);
            fence_proxy_async();
        }
        __syncwarp();
        if (lane == 0 && my_zero > 0) {
            // walker over (plane, row tile, column tile) with column tiles conv_key_tiles(tm) .. tiles_n - 1
            int zp = (int)(z_begin / g.zero_per_plane), ztm = 0;
            long r = z_begin - (long)zp * g.zero_per_plane;
            for (;; ++ztm) {
                const int nz = g.tiles_n - conv_key_tiles(g, ztm);
                if (r < nz) break;
                r -= nz;
            }
            int ztn = conv_key_tiles(g, ztm) + (int)r;
            for (long zi = 0; zi < my_zero; ++zi) {
                // zero tile zi is due once the producer has loaded compute tile zi * my_tiles / my_zero (bounded wait:
                // the producer always reaches its last tile, and giving up early only changes the pacing)
                const int due = (int)(zi * my_tiles / my_zero);
                for (int spin = 0; *reinterpret_cast<volatile int*>(&tiles_loaded) < due && spin < (1 << 20); ++spin) __nanosleep(256);
                const int zm0 = g.row_begin + ztm * TM, zn0 = ztn * TN;
                tma_store_3d(&my, zero_box, zn0, zm0 - y_row0, zp);
                if (zn0 + 64 < g.W) tma_store_3d(&my, zero_box, zn0 + 64, zm0 - y_row0, zp);
                bulk_commit();
                bulk_wait_read_1();
                if (++ztn == g.tiles_n) {
                    do {
                        if (++ztm == g.tiles_m) { ztm = 0; ++zp; }
                    } while (conv_key_tiles(g, ztm) >= g.tiles_n && zi + 1 < my_zero);
                    ztn = conv_key_tiles(g, ztm);
                }
            }
            bulk_wait_all();
        }
    } else if (warp == 1 || (warp == 8 && NISS >= 2)) {
        // ---------------- MMA issuers ----------------
        // Two threads issue, each onto its own output blocks, so no ordering between them is needed and none affects
        // the result (measured at B8 H16 S4096, 6 x 11: one issuer 1.19 ms, two 0.94 ms, three 1.01 ms; the tensor pipe
        // takes ~49 cycles per MMA, a single thread issues one per ~76).  The schedule of an issuer is compile-time (issue_tile<ISSUER>): every descriptor is the stage's
        // base descriptor plus a constant and a multiple of the row tap, all warp-uniform values.
        for (int n = 0; n < my_tiles; ++n) {
            const int st = n % NSTAGE, ab = n & 1;
            mbar_wait(&ready_bar[st], (n / NSTAGE) & 1, err_flag);
            mbar_wait(&acc_empty[ab], ((n >> 1) & 1) ^ 1, err_flag);
            fence_after_sync();
            if (lane == 0) {
                const uint32_t xa_addr = smem_u32(stage_base + st * stage_bytes);
                const uint32_t d0 = tmem + (uint32_t)(ab * TN);
                if (warp == 1) issue_tile<T, 0>(xa_addr, d0, R, g.split_w, box_bytes, tb_off);
                else issue_tile<T, NISS >= 2 ? 1 : 0>(xa_addr, d0, R, g.split_w, box_bytes, tb_off);
                mma_commit(&empty_bar[st]);
                mma_commit(&acc_full[ab]);
            }
            __syncwarp();
        }
    } else if (warp == 8 || warp == 9) {
        // issuer warp that this build does not use
    } else if (warp < 4 || warp >= 14) {
        // ---------------- (warps 2-3, 14-15) causal zeroing of the staged tile, Toeplitz slices ----------------
        const int ft = warp < 4 ? tid - 64 : tid - 448 + 64;     // 0..127
        TileIter it;
        it.init(g, t_begin);
        int ph0 = -1, ph1 = -1, ph2 = -1;                 // head whose Toeplitz slices each stage holds (NSTAGE == 3)
        for (int n = 0; n < my_tiles; ++n, it.next(g, g.tiles_m)) {
            const int st = n % NSTAGE;
            const int plane = it.plane, m0 = it.m0(g), n0 = it.n0();
            const int head = plane % g.C;
            uint8_t* xa = stage_base + st * stage_bytes;
            uint8_t* tb = xa + tb_off;
            // the stage (and its Toeplitz slices) is free once the MMAs of tile n - NSTAGE are done
            mbar_wait(&empty_bar[st], ((n / NSTAGE) & 1) ^ 1, err_flag);
            int ph;
            if (st == 0) { ph = ph0; ph0 = head; }
            else if (st == 1) { ph = ph1; ph1 = head; }
            else { ph = ph2; ph2 = head; }
            if (ph != head) {
                // slice of row tap i, element (n', kk) = w[i][kk + 16 - n' - a_off]; no-swizzle K-major layout:
                // 8 rows x 16 bytes per core matrix, the two k chunks 512 bytes apart, row groups 128 bytes apart
                const int total = R * 512;
                for (int idx = ft; idx < total; idx += 128) {
                    const int i = idx / 512, e = idx % 512;
                    const int nn = e / 16, kk = e % 16;
                    const int j = kk + 16 - nn - a_off;
                    const float wv = (j >= 0 && j < S) ? load_weight(w, g.flip ? ((long)head * R + (R - 1 - i)) * S + (S - 1 - j)
                                                                             : ((long)head * R + i) * S + j, w_dtype)
                                                       : 0.0f;
                    const T hi = from_f32<T>(wv);
                    const int off = i * 1024 + (kk / 8) * 512 + (nn / 8) * 128 + (nn % 8) * 16 + (kk % 8) * 2;
                    *reinterpret_cast<T*>(tb + off) = hi;
                    if (g.split_w) *reinterpret_cast<T*>(tb + R * 1024 + off) = from_f32<T>(wv - to_f32<T>(hi));
                }
            }
            mbar_wait(&full_bar[st], (n / NSTAGE) & 1, err_flag);
            // staged row sr is query m0-(R-1)+sr; staged column sc is key n0-pad8+sc, in box sc/64 at byte
            // sr*128 + (((sc%64)/8) ^ (sr%8))*16 + (sc%8)*2.  Zero the keys above the query.
            if (g.causal && n0 - pad8 + NCH * 8 - 1 > m0 - g.lead) {
                // one thread per staged row: zero from the first key above the query to the end of the row
                const int c0 = n0 - pad8;
                for (int sr = ft; sr < TH; sr += 128) {
                    const int qq = m0 - g.lead + sr;
                    int first = qq - c0 + 1;                      // first staged column to zero
                    if (first >= NCH * 8) continue;
                    if (first < 0) first = 0;
                    int ch = first >> 3;
                    uint8_t* rowp = xa + sr * 128;
                    // chunk ch of row sr: boxes 0/1 (128-byte rows, chunk index xor row % 8), box 2 (32-byte rows, chunk
                    // index xor bit 2 of the row: the 32-byte swizzle flips address bit 4 with bit 7)
                    auto chunk_ptr = [&](int c) -> uint8_t* {
                        return c < 16 ? rowp + (c >> 3) * box_bytes + (((c & 7) ^ (sr & 7)) << 4)
                                      : xa + NBOX * box_bytes + sr * 32 + ((((c - 16) ^ (sr >> 2)) & 1) << 4);
                    };
                    if (first & 7) {
                        uint16_t* e16 = reinterpret_cast<uint16_t*>(chunk_ptr(ch));
                        for (int e = first & 7; e < 8; ++e) e16[e] = 0;
                        ++ch;
                    }
                    for (; ch < NCH; ++ch) *reinterpret_cast<uint4*>(chunk_ptr(ch)) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            fence_proxy_async();          // generic-proxy writes above must be visible to the MMAs (async proxy)
            __syncwarp();
            if (lane == 0) mbar_arrive(&ready_bar[st]);
        }
    } else {
        // ---------------- epilogue: warps 4-7 drain columns 0..63, warps 10-13 columns 64..127 ----------------
        const int quarter = warp & 3;                        // the TMEM lanes a warp may read depend on its index mod 4
        const int half = warp >= 10 ? 1 : 0;
        const bool issuer = (warp == 4 && lane == 0);
        const int row = quarter * 32 + lane;                 // row of the tile this thread owns
        TileIter it;
        it.init(g, t_begin);
        for (int n = 0; n < my_tiles; ++n, it.next(g, g.tiles_m)) {
            const int ab = n & 1;
            const int plane = it.plane, m0 = it.m0(g), n0 = it.n0();
            uint8_t* obuf = out_base + ab * OUT_BYTES;       // staging tile n % 2: two 64-column boxes
            uint8_t* orow = obuf + half * (TM * 128) + row * 128;
            mbar_wait(&acc_full[ab], (n >> 1) & 1, err_flag);
            __syncwarp();
            fence_after_sync();
            if (issuer) bulk_wait_read_1();                  // the store of tile n-2 has finished reading this staging tile
            named_barrier(1, 256);
            const int q = m0 + row;
#pragma unroll
            for (int cblk = 0; cblk < 2; ++cblk) {
                uint32_t r[32];
                tmem_ld_32x32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ab * TN + half * 64 + cblk * 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int v8 = 0; v8 < 4; ++v8) {
                    const int col = cblk * 32 + v8 * 8;      // column inside this warp's 64-column half
                    const int k = n0 + half * 64 + col;
                    float f[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v8 * 8 + e]);
                    if (g.causal && k + 7 > q) {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (k + e > q) f[e] = 0.0f;          // entries above the diagonal inside the tile are written as 0
                    }
                    uint4 o;
                    o.x = pack2c<T>(f[0], f[1]);
                    o.y = pack2c<T>(f[2], f[3]);
                    o.z = pack2c<T>(f[4], f[5]);
                    o.w = pack2c<T>(f[6], f[7]);
                    *reinterpret_cast<uint4*>(orow + (((col >> 3) ^ (row & 7)) << 4)) = o;
                }
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[ab]);
            fence_proxy_async();                             // staging tile written through the generic proxy, read by TMA
            named_barrier(1, 256);
            if (issuer) {
                // rows past row_end and columns past W are clipped by the tensor map
                tma_store_3d(&my, obuf, n0, m0 - y_row0, plane);
                if (n0 + 64 < g.W) tma_store_3d(&my, obuf + TM * 128, n0 + 64, m0 - y_row0, plane);
                bulk_commit();
            }
        }
        if (issuer) bulk_wait_all();
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 2 * TN);
}

size_t conv2d_tc05_smem_bytes(int R, bool split_w) {
    const int TH = TM + R - 1;
    const size_t box = (size_t)((TH * 128 + 1023) & ~1023);
    const size_t tb = (size_t)((R * 1024 * (split_w ? 2 : 1) + 1023) & ~1023);
    const size_t box3 = (size_t)((TH * 32 + 1023) & ~1023);
    return 1024 + 2 * OUT_BYTES + TM * 128 + NSTAGE * (NBOX * box + box3 + tb);
}

template <typename T>
int launch_tc05(const void* x, PlaneView xv, long x_rows_stored, const void* w, int w_dtype, void* y, PlaneView yv,
                long planes, int C, int W, int R, int S, int causal, int row_begin, int row_end, bool write_upper,
                bool grad_input, cudaStream_t st) {
    CUtensorMap mx;
    int rc;
    const int TH = TM + R - 1;
    if ((rc = make_tensor_map_3d(&mx, x, (uint64_t)planes, (uint64_t)x_rows_stored, (uint64_t)W, (uint64_t)xv.width,
                                 (uint64_t)xv.plane_stride, 64, (uint32_t)TH, true)))
        return rc;
    int* flag = nullptr;
    if ((rc = wait_flag_ptr(&flag))) return rc;
    CUtensorMap mx3;     // the 16-column box of the last k-step
    if ((rc = make_tensor_map_3d_mode(&mx3, x, (uint64_t)planes, (uint64_t)x_rows_stored, (uint64_t)W, (uint64_t)xv.width,
                                      (uint64_t)xv.plane_stride, 16, (uint32_t)TH, 32)))
        return rc;
    CUtensorMap my;      // rows past row_end are outside this map, so a tile's store never touches them
    if ((rc = make_tensor_map_3d(&my, y, (uint64_t)planes, (uint64_t)(row_end - yv.row0), (uint64_t)W, (uint64_t)yv.width,
                                 (uint64_t)yv.plane_stride, 64, TM, true)))
        return rc;
    ConvGeom g;
    g.C = C; g.W = W; g.R = R; g.S = S; g.causal = causal; g.row_begin = row_begin; g.row_end = row_end;
    g.tiles_n = (W + TN - 1) / TN; g.x_row0 = xv.row0; g.write_upper = write_upper ? 1 : 0;
    g.split_w = w_dtype == MTA_F32 ? 1 : 0;
    g.lead = grad_input ? 0 : R - 1;
    g.flip = grad_input ? 1 : 0;
    const int tiles_m = (row_end - row_begin + TM - 1) / TM;
    g.tiles_m = tiles_m;
    long per_plane = 0;
    for (int tm = 0; tm < tiles_m; ++tm) {
        const int q_last = std::min(row_begin + (tm + 1) * TM, row_end);
        per_plane += causal ? std::min((q_last + TN - 1) / TN, g.tiles_n) : g.tiles_n;
    }
    g.tiles_per_plane = per_plane;
    g.total_tiles = per_plane * planes;
    g.zero_per_plane = (causal && write_upper) ? (long)tiles_m * g.tiles_n - per_plane : 0;
    g.zero_total = g.zero_per_plane * planes;
    int dev = 0, sms = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const size_t smem = conv2d_tc05_smem_bytes(R, g.split_w != 0);
    MTA_REQUIRE(smem <= 227 * 1024, "conv2d (tcgen05): kernel with %d row taps needs %zu bytes of shared memory", R, smem);
    MTA_CUDA_OK(cudaFuncSetAttribute(conv2d_tc05_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const unsigned grid = (unsigned)std::min<long>(g.total_tiles, sms);
    conv2d_tc05_kernel<T><<<grid, THREADS, smem, st>>>(mx, mx3, my, w, w_dtype, yv.row0, g, flag);
    MTA_LAUNCH_OK("conv2d_tc05_kernel");
    return MTA_OK;
}

}  // namespace


bool conv2d_tc05_supported(const void* x, PlaneView xv, const void* y, PlaneView yv, int W, int R, int S, int dtype,
                           int w_dtype) {
    return dtype != MTA_F32 && S <= 17 && R <= 16 && conv2d_tc05_smem_bytes(R, w_dtype == MTA_F32) <= 227 * 1024 && W % 8 == 0 && xv.width == W && yv.width == W &&
           xv.plane_stride % 8 == 0 && yv.plane_stride % 8 == 0 && aligned16(x) && aligned16(y);
}

int conv2d_tc05_launch(const void* x, PlaneView xv, long x_rows_stored, const void* w, int w_dtype, void* y, PlaneView yv,
                       long planes, int C, int H, int W, int R, int S, int causal, int row_begin, int row_end,
                       bool write_upper, int dtype, cudaStream_t st, bool grad_input) {
    (void)H;
    MTA_REQUIRE(!grad_input || S % 2 == 1, "conv2d (tcgen05): the input gradient needs an odd key extent");
    if (dtype == MTA_BF16)
        return launch_tc05<__nv_bfloat16>(x, xv, x_rows_stored, w, w_dtype, y, yv, planes, C, W, R, S, causal, row_begin,
                                          row_end, write_upper, grad_input, st);
    return launch_tc05<__half>(x, xv, x_rows_stored, w, w_dtype, y, yv, planes, C, W, R, S, causal, row_begin, row_end,
                               write_upper, grad_input, st);
}

}  // namespace mta
