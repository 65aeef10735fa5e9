// Score tiles on the tcgen05 tensor cores, persistent and warp-specialised:
//
//     C[q, k] = sum_{i < NI}  A[q - (NI-1) + i, :] . B_i[k, :]          (128 x 128 tiles, D = 64 or 128, 16-bit dtypes)
//
//   NI = 1, B_0 = K          plain scaled scores Q K^T * scale (mta_attention_triton.py:68-71)
//   NI = cq, B_i = Kt_i      the causal conv of the scores for tiles that lie wholly below the causal band, through
//                            the bilinear identity conv(Q K^T)[q,k] = sum_i Q[q-(cq-1)+i] . Kt_i[k] with
//                            Kt_i[k] = scale * sum_j w[i][j] K[k + j - pad_w]   (prepared by the caller)
//
// One CTA per SM walks a contiguous range of tiles.  Warp 0 issues the TMA loads (A rows shifted per term, both
// operands in the 128-byte-swizzled K-major layout, out-of-range rows read as zero) into a ring of stages; warp 1
// issues the MMAs (M128 N128 K16, D/16 per term) into one of two TMEM accumulators; eight epilogue warps drain the
// other accumulator: TMEM -> registers -> scale / round -> swizzled shared-memory tile -> TMA tiled store.
#include "kernels.cuh"
#include "tc05.cuh"

namespace mta {
namespace {
using namespace tc05;

constexpr int TILE = 128;
constexpr int BOX_BYTES = TILE * 128;          // one TMA box: 128 rows x 64 elements
constexpr int OUT_BYTES = 2 * BOX_BYTES;       // output staging tile: two 64-column boxes
constexpr int QK_THREADS = 320;                // producer, MMA issuer, 8 epilogue warps

template <typename T> struct AbF;
template <> struct AbF<__nv_bfloat16> { static constexpr int value = 1; };
template <> struct AbF<__half> { static constexpr int value = 0; };

template <typename T> __device__ __forceinline__ uint32_t pk2q(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pk2q<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t pk2q<__half>(float lo, float hi) {
    __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}

struct QkGeom {
    int S, causal, row_begin, row_end, tiles_q, tiles_k;
    int mode;          // 0: every tile that touches keys <= query; 1: only the band (last tiles of a row); 2: only below the band
    int band_cq, band_pw;   // the conv whose band separates modes 1 and 2: cq row taps, pad_w key taps to each side
    int NI;            // terms per tile
    int nstage;
    int s_row0;        // first stored row of the output planes
    float scale;
    int round_scale;
    long tiles_per_bh, total;
};

__host__ __device__ inline int floor_div(int a, int b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }

// Key tiles [lo, hi] of query tile tq (hi < lo: none).
__host__ __device__ inline void tile_range(const QkGeom& g, int tq, int& lo, int& hi) {
    const int q0 = g.row_begin + tq * TILE;
    const int q_last = (q0 + TILE < g.row_end ? q0 + TILE : g.row_end);
    const int d = g.causal ? ((q_last - 1) / TILE < g.tiles_k - 1 ? (q_last - 1) / TILE : g.tiles_k - 1) : g.tiles_k - 1;
    // last key tile whose every conv tap is unmasked for every row of the query tile
    int hb = floor_div(q0 - (g.band_cq - 1) - g.band_pw - (TILE - 1), TILE);
    if (hb > d) hb = d;
    if (g.mode == 0) { lo = 0; hi = d; }
    else if (g.mode == 1) { lo = hb > 0 ? hb : 0; hi = d; }
    else { lo = 0; hi = hb; }
}

struct QkIter {
    int bh, tq, tk, lo, hi;
    __device__ void init(const QkGeom& g, long t) {
        bh = (int)(t / g.tiles_per_bh);
        int r = (int)(t - (long)bh * g.tiles_per_bh);
        for (tq = 0;; ++tq) {
            tile_range(g, tq, lo, hi);
            const int n = hi >= lo ? hi - lo + 1 : 0;
            if (r < n) break;
            r -= n;
        }
        tk = lo + r;
    }
    __device__ void next(const QkGeom& g) {
        if (++tk > hi) {
            do {
                if (++tq == g.tiles_q) { tq = 0; ++bh; }
                tile_range(g, tq, lo, hi);
            } while (hi < lo);
            tk = lo;
        }
    }
};

template <typename T, int D>
__global__ void __launch_bounds__(QK_THREADS, 1)
qk_persistent_kernel(const __grid_constant__ CUtensorMap ma, const __grid_constant__ CUtensorMap mb,
                     const __grid_constant__ CUtensorMap mc, const QkGeom g, int* err_flag) {
    constexpr int NBOX = D / 64;
    constexpr int OPER_BYTES = NBOX * BOX_BYTES;             // one operand tile
    constexpr int STAGE_BYTES = 2 * OPER_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* out_base = smem;
    uint8_t* stage_base = smem + OUT_BYTES;
    __shared__ __align__(8) uint64_t full_bar[4], empty_bar[4], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NST = g.nstage, NI = g.NI;

    const long per = (g.total + gridDim.x - 1) / gridDim.x;
    const long t_begin = (long)blockIdx.x * per;
    const long t_end = min(t_begin + per, g.total);
    const int my_tiles = t_end > t_begin ? (int)(t_end - t_begin) : 0;

    if (tid == 0) abort_flag = *reinterpret_cast<volatile int*>(err_flag);
    __syncthreads();
    if (abort_flag != 0 || my_tiles == 0) return;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < 4; ++i) {
                mbar_init(&full_bar[i], 1);
                mbar_init(&empty_bar[i], 1);
            }
            for (int i = 0; i < 2; ++i) {
                mbar_init(&acc_full[i], 1);
                mbar_init(&acc_empty[i], 8);
            }
            fence_mbar_init();
            prefetch_tensormap(&ma);
            prefetch_tensormap(&mb);
            prefetch_tensormap(&mc);
        }
        __syncwarp();
        tmem_alloc(&tmem_slot, 2 * TILE);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            QkIter it;
            it.init(g, t_begin);
            int f = 0;
            for (int n = 0; n < my_tiles; ++n, it.next(g)) {
                const int q0 = g.row_begin + it.tq * TILE, k0 = it.tk * TILE;
                for (int i = 0; i < NI; ++i, ++f) {
                    const int st = f % NST;
                    mbar_wait(&empty_bar[st], ((f / NST) & 1) ^ 1, err_flag);
                    uint8_t* sa = stage_base + st * STAGE_BYTES;
                    uint8_t* sb = sa + OPER_BYTES;
                    mbar_expect_tx(&full_bar[st], STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < NBOX; ++j) {
                        tma_load_3d(sa + j * BOX_BYTES, &ma, &full_bar[st], j * 64, q0 - (NI - 1) + i, it.bh);
                        tma_load_3d(sb + j * BOX_BYTES, &mb, &full_bar[st], j * 64, k0, it.bh * NI + i);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        constexpr uint32_t idesc = instr_desc_f16(AbF<T>::value, 0, 0, TILE, TILE);
        int f = 0;
        for (int n = 0; n < my_tiles; ++n) {
            const int ab = n & 1;
            mbar_wait(&acc_empty[ab], ((n >> 1) & 1) ^ 1, err_flag);
            for (int i = 0; i < NI; ++i, ++f) {
                const int st = f % NST;
                mbar_wait(&full_bar[st], (f / NST) & 1, err_flag);
                fence_after_sync();
                if (lane == 0) {
                    const uint32_t sa = smem_u32(stage_base + st * STAGE_BYTES), sb = sa + OPER_BYTES;
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t off = (kk / 4) * BOX_BYTES + (kk % 4) * 32;
                        mma_f16_ss(tmem + (uint32_t)(ab * TILE), smem_desc_sw128(sa + off, 16, 1024),
                                   smem_desc_sw128(sb + off, 16, 1024), idesc, (i > 0 || kk > 0) ? 1u : 0u);
                    }
                    mma_commit(&empty_bar[st]);
                    if (i == NI - 1) mma_commit(&acc_full[ab]);
                }
                __syncwarp();
            }
        }
    } else {
        // ---------------- epilogue: warp (2 + e) drains TMEM lanes 32 (e % 4).., columns 64 (e / 4).. ----------------
        const int e = warp - 2;
        const int quarter = warp & 3;                        // the TMEM lanes a warp may read depend on its index mod 4
        const int half = e >> 2;
        const bool issuer = (warp == 2 && lane == 0);
        const int row = quarter * 32 + lane;
        uint8_t* orow = out_base + half * BOX_BYTES + row * 128;
        const float sc = g.round_scale ? round_to<T>(g.scale) : g.scale;
        QkIter it;
        it.init(g, t_begin);
        for (int n = 0; n < my_tiles; ++n, it.next(g)) {
            const int ab = n & 1;
            const int q0 = g.row_begin + it.tq * TILE, k0 = it.tk * TILE;
            mbar_wait(&acc_full[ab], (n >> 1) & 1, err_flag);
            __syncwarp();
            fence_after_sync();
            if (issuer) bulk_wait_read();                    // the previous tile's store has finished reading the staging tile
            named_barrier(1, 256);
            const int q = q0 + row;
#pragma unroll
            for (int cblk = 0; cblk < 2; ++cblk) {
                uint32_t r[32];
                tmem_ld_32x32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ab * TILE + half * 64 + cblk * 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int v8 = 0; v8 < 4; ++v8) {
                    const int col = cblk * 32 + v8 * 8;      // column inside this warp's 64-column half
                    const int k = k0 + half * 64 + col;
                    float f[8];
#pragma unroll
                    for (int x = 0; x < 8; ++x) {
                        const float a = __uint_as_float(r[v8 * 8 + x]);
                        f[x] = g.round_scale ? round_to<T>(a) * sc : a * sc;
                        if (g.causal && k + x > q) f[x] = 0.0f;   // above the diagonal inside a visited tile: written as 0
                    }
                    uint4 o;
                    o.x = pk2q<T>(f[0], f[1]);
                    o.y = pk2q<T>(f[2], f[3]);
                    o.z = pk2q<T>(f[4], f[5]);
                    o.w = pk2q<T>(f[6], f[7]);
                    *reinterpret_cast<uint4*>(orow + (((col >> 3) ^ (row & 7)) << 4)) = o;
                }
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[ab]);
            fence_proxy_async();
            named_barrier(1, 256);
            if (issuer) {
                // rows past row_end and columns past S are outside the tensor map and are clipped
                tma_store_3d(&mc, out_base, k0, q0 - g.s_row0, it.bh);
                if (k0 + 64 < g.S) tma_store_3d(&mc, out_base + BOX_BYTES, k0 + 64, q0 - g.s_row0, it.bh);
                bulk_commit();
            }
        }
        if (issuer) bulk_wait_all();
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 2 * TILE);
}

template <typename T, int D>
int launch(const void* a, const void* b, void* c, PlaneView cv, int BH, QkGeom g, cudaStream_t st) {
    CUtensorMap ma, mb, mc;
    int rc;
    if ((rc = make_tensor_map_3d(&ma, a, (uint64_t)BH, g.S, D, D, (uint64_t)g.S * D, 64, TILE, true))) return rc;
    if ((rc = make_tensor_map_3d(&mb, b, (uint64_t)BH * g.NI, g.S, D, D, (uint64_t)g.S * D, 64, TILE, true))) return rc;
    if ((rc = make_tensor_map_3d(&mc, c, (uint64_t)BH, (uint64_t)(g.row_end - cv.row0), g.S, g.S, (uint64_t)cv.plane_stride, 64, TILE, true)))
        return rc;
    int* flag = nullptr;
    if ((rc = wait_flag_ptr(&flag))) return rc;
    g.tiles_q = (g.row_end - g.row_begin + TILE - 1) / TILE;
    g.tiles_k = (g.S + TILE - 1) / TILE;
    long per_bh = 0;
    for (int tq = 0; tq < g.tiles_q; ++tq) {
        int lo, hi;
        tile_range(g, tq, lo, hi);
        if (hi >= lo) per_bh += hi - lo + 1;
    }
    if (per_bh == 0) return MTA_OK;
    g.tiles_per_bh = per_bh;
    g.total = per_bh * BH;
    g.s_row0 = cv.row0;
    constexpr int STAGE = 2 * (D / 64) * BOX_BYTES;
    g.nstage = D == 128 ? 3 : 4;
    const size_t smem = 1024 + OUT_BYTES + (size_t)g.nstage * STAGE;
    int dev = 0, sms = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    MTA_CUDA_OK(cudaFuncSetAttribute(qk_persistent_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const unsigned grid = (unsigned)std::min<long>(g.total, sms);
    qk_persistent_kernel<T, D><<<grid, QK_THREADS, smem, st>>>(ma, mb, mc, g, flag);
    MTA_LAUNCH_OK("qk_persistent_kernel");
    return MTA_OK;
}

}  // namespace

// mode 0: all tiles with keys <= query; mode 1 / 2: the band of a (band_cq x (2 band_pw + 1)) conv / the tiles below it.
int qk_persistent_launch(const void* a, const void* b, void* c, PlaneView cv, int B, int H, int S, int D, int NI, float scale,
                         int round_scale, int causal, int mode, int band_cq, int band_pw, int row_begin, int row_end, int dtype,
                         cudaStream_t st) {
    QkGeom g{};
    g.S = S; g.causal = causal; g.row_begin = row_begin; g.row_end = row_end; g.mode = mode; g.band_cq = band_cq; g.band_pw = band_pw;
    g.NI = NI; g.scale = scale; g.round_scale = round_scale;
#define MTA_QKP(TT, DD) return launch<TT, DD>(a, b, c, cv, B * H, g, st)
    if (dtype == MTA_BF16) { if (D == 64) MTA_QKP(__nv_bfloat16, 64); MTA_QKP(__nv_bfloat16, 128); }
    if (D == 64) MTA_QKP(__half, 64);
    MTA_QKP(__half, 128);
#undef MTA_QKP
}

}  // namespace mta
