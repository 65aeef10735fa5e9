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
// Warps: 0 TMA producer (Q tile per row of tiles, K tile per tile; a ring of three staged tiles hides the reloads),
// 1 score-MMA issuer, 2-3 conv-MMA
// issuers, 4-7 drain, 8-15 epilogue.  16-bit dtypes, D in {64, 128}, odd key extent <= 17, causal.
#include "toeplitz_tc05.cuh"

namespace mta {
namespace {
using namespace tc05;
using namespace qc;

constexpr int OUT_BYTES = 2 * TM * 128;           // output staging: two 64-column boxes
constexpr int NSTAGE = 3;                         // staged score tiles in flight
// Four drain warps (warps 4-7): a thread converts its whole staged row.  Measured at B8 H16 S4096 D128, 6 x 11: 1.26 ms;
// eight warps with spinning waits 1.35 ms - the kernel is bound by shared-memory bandwidth (the conv MMAs' operand
// reads, ~300 KB per tile, plus ~200 KB of tile traffic), and extra polling and extra warps only add to it.
constexpr int DRAIN_WARPS = 4;
constexpr int THREADS = 512;
constexpr uint32_t S_COL = 256;                   // TMEM column of the score accumulator (conv accumulators: 0..255)

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

template <typename T, int D>
__global__ void __launch_bounds__(THREADS, 1)
qk_conv_tc05_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                    const __grid_constant__ CUtensorMap my, const void* __restrict__ w, int w_dtype, QcGeom g, int* err_flag) {
    constexpr int DBOX = D / 64;                               // 64-element boxes along the head dimension
    constexpr int Q_BYTES = DBOX * BOX_BYTES;                  // Q tile: 128 rows x D
    constexpr int K_BYTES = DBOX * KBOX_BYTES;                 // K tile: 144 keys x D
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t q_full, q_free, k_full, k_free, s_full, s_free, ready_bar[NSTAGE], empty_bar[NSTAGE],
        acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ float wsm[MAX_TAPS];                // the current head's conv weights on their way into the Toeplitz slices
    const int R = g.R, KS = g.KS;
    const int tb_bytes = toeplitz_bytes(R, g.split_w);
    uint8_t* out_base = smem;
    uint8_t* q_base = out_base + OUT_BYTES;
    uint8_t* k_base = q_base + Q_BYTES;                        // one K tile: the ring of staged tiles hides its reload
    uint8_t* stage_base = k_base + K_BYTES;                    // NSTAGE staged tiles of TB_OFF bytes
    uint8_t* tb_base = stage_base + NSTAGE * TB_OFF;           // two sets of Toeplitz slices: successive heads alternate
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
            mbar_init(&k_full, 1);
            mbar_init(&k_free, 1);
            for (int i = 0; i < NSTAGE; ++i) {
                mbar_init(&ready_bar[i], DRAIN_WARPS);
                mbar_init(&empty_bar[i], 2);
            }
            for (int i = 0; i < 2; ++i) {
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
                mbar_wait(&k_free, (n & 1) ^ 1, err_flag);       // the score MMAs of tile n - 1 have read the K tile
                mbar_expect_tx(&k_full, (uint32_t)K_BYTES);
#pragma unroll
                for (int j = 0; j < DBOX; ++j) tma_load_3d(k_base + j * KBOX_BYTES, &mk, &k_full, 64 * j, it.n0() - 8, it.plane);
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
        for (int n = 0; n < my_tiles; ++n) {
            if (new_q) {
                mbar_wait(&q_full, qn & 1, err_flag);
                ++qn;
            }
            mbar_wait(&k_full, n & 1, err_flag);
            mbar_wait(&s_free, (n & 1) ^ 1, err_flag);           // the drain warps have read the previous score tile
            fence_after_sync();
            new_q = it.next(g);
            if (lane == 0) {
                const uint32_t qa = smem_u32(q_base), ka = smem_u32(k_base);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t qoff = (kk / 4) * BOX_BYTES + (kk % 4) * 32, koff = (kk / 4) * KBOX_BYTES + (kk % 4) * 32;
                    mma_f16_ss(tmem + S_COL, smem_desc_sw128(qa + qoff, 16, 1024), smem_desc_sw128(ka + koff, 16, 1024), idesc,
                               kk > 0 ? 1u : 0u);
                }
                mma_commit(&k_free);
                mma_commit(&s_full);
                if (new_q || n == my_tiles - 1) mma_commit(&q_free);     // last tile of this row of tiles
            }
            __syncwarp();
        }
    } else if (warp == 2 || warp == 3) {
        // ---------------- conv MMAs ----------------
        QcIter it;
        it.init(g, t_begin);
        int cur_head = -1, hn = -1;                          // the running head and how many times it has changed
        for (int n = 0; n < my_tiles; ++n, it.next(g)) {
            const int st = n % NSTAGE, ab = n & 1;
            const int head = it.plane % g.C;
            if (head != cur_head) { cur_head = head; ++hn; }
            mbar_wait(&ready_bar[st], (n / NSTAGE) & 1, err_flag);
            mbar_wait(&acc_empty[ab], ((n >> 1) & 1) ^ 1, err_flag);
            fence_after_sync();
            if (lane == 0) {
                const uint32_t xa_addr = smem_u32(stage_base + st * TB_OFF);
                const uint32_t tb_addr = smem_u32(tb_base + (hn & 1) * tb_bytes);
                const uint32_t d0 = tmem + (uint32_t)(ab * TN);
                if (warp == 2) issue_conv<T, 0>(xa_addr, tb_addr, d0, R, g.split_w);
                else issue_conv<T, 1>(xa_addr, tb_addr, d0, R, g.split_w);
                mma_commit(&empty_bar[st]);
                mma_commit(&acc_full[ab]);
            }
            __syncwarp();
        }
    } else if (warp < 8) {
        // ---------------- drain: score tile TMEM -> rounded, scaled, masked -> staged tile; Toeplitz slices ----------------
        const int quarter = warp & 3;
        const int sr = quarter * 32 + lane;                  // staged row = TMEM lane of this thread
        const int ft = tid - 128;                            // 0..127
        const float sc = round_to<T>(g.scale);
        QcIter it;
        it.init(g, t_begin);
        int cur_head = -1, hn = -1;
        for (int n = 0; n < my_tiles; ++n, it.next(g)) {
            const int st = n % NSTAGE;
            const int m0 = it.m0(g), n0 = it.n0();
            const int head = it.plane % g.C;
            uint8_t* xa = stage_base + st * TB_OFF;
            if (head != cur_head) {
                cur_head = head;
                ++hn;
                // this set of slices was read last by the conv MMAs of the head before the previous one: tiles <= n - 2
                if (n >= 2) mbar_wait(&empty_bar[(n - 2) % NSTAGE], ((n - 2) / NSTAGE) & 1, err_flag);
                build_toeplitz<T>(tb_base + (hn & 1) * tb_bytes, wsm, w, w_dtype, head, R, KS, a_off, g.split_w, ft, DRAIN_WARPS * 32, 2);
            }
            // the stage is free once the conv MMAs of tile n - NSTAGE are done
            mbar_wait(&empty_bar[st], ((n / NSTAGE) & 1) ^ 1, err_flag);
            mbar_wait(&s_full, n & 1, err_flag);
            __syncwarp();
            fence_after_sync();
            // The causal comparison runs on every tile, also those wholly below the diagonal (measured: skipping it there
            // made an earlier two-stage version of this kernel slower, because the drain's shared-memory stores then came
            // in denser bursts and held up the operand reads of the conv MMAs).
            drain_row<T, true>(tmem + ((uint32_t)(quarter * 32) << 16) + S_COL, smem_u32(xa), sr, m0 - lead + sr, n0 - 8, sc, true);
            fence_before_sync();
            fence_proxy_async();          // generic-proxy writes above must be visible to the MMAs (async proxy)
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&s_free);
                mbar_arrive(&ready_bar[st]);
            }
        }
    } else {
        // ---------------- epilogue: warps 8-11 take columns 0..63, warps 12-15 columns 64..127 ----------------
        const int quarter = warp & 3;
        const int half = warp >= 12 ? 1 : 0;
        const bool issuer = (warp == 8 && lane == 0);
        const int row = quarter * 32 + lane;
        QcIter it;
        it.init(g, t_begin);
        for (int n = 0; n < my_tiles; ++n, it.next(g)) {
            const int ab = n & 1;
            const int plane = it.plane, m0 = it.m0(g), n0 = it.n0();
            uint8_t* orow = out_base + half * (TM * 128) + row * 128;
            mbar_wait(&acc_full[ab], (n >> 1) & 1, err_flag);
            __syncwarp();
            fence_after_sync();
            if (issuer) bulk_wait_read();                    // the previous tile's store has finished reading the staging tile
            named_barrier(1, 256);
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
            fence_proxy_async();
            named_barrier(1, 256);
            if (issuer) {
                // the store's box has TMO rows; rows past row_end and columns past S are clipped by the tensor map
                tma_store_3d(&my, out_base, n0, m0 - g.y_row0, plane);
                if (n0 + 64 < g.S) tma_store_3d(&my, out_base + TM * 128, n0 + 64, m0 - g.y_row0, plane);
                bulk_commit();
            }
        }
        if (issuer) bulk_wait_all();
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

size_t qk_conv_smem_bytes(int D, int R, bool split_w) {
    return 1024 + OUT_BYTES + (size_t)(D / 64) * (BOX_BYTES + KBOX_BYTES) + (size_t)NSTAGE * TB_OFF +
           2 * (size_t)toeplitz_bytes(R, split_w ? 1 : 0);
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
