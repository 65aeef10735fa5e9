// The two contractions of the forward on the 5th-generation tensor cores (tcgen05), 16-bit dtypes:
//   scores tile  S[128 q x 128 k] = Q[128 x D] K[128 x D]^T   (both operands K-major, D in {64,128})
//   output tile  O[128 q x D]     = sum over key tiles  P[128 q x 128 k] V[128 k x D]   (A K-major, B MN-major)
// Operand tiles arrive by TMA (128-byte swizzle, out-of-range rows and columns read as zero), the
// accumulator lives in tensor memory, and only tiles that touch keys k <= q are visited when causal.
// They stand in for the torch.matmul calls at mta_attention_triton.py:68-71 and :89.
#include <mutex>

#include "kernels.cuh"
#include "tc05.cuh"

namespace mta {

// ---- host helpers ----------------------------------------------------------------------------------
namespace {
__device__ int g_wait_timeout = 0;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

EncodeTiledFn encode_fn() {
    std::call_once(g_encode_once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    });
    return g_encode;
}
}  // namespace

int wait_flag_ptr(int** out) {
    static int* ptrs[64] = {};
    int dev = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
    if (!ptrs[dev]) {
        void* p = nullptr;
        MTA_CUDA_OK(cudaGetSymbolAddress(&p, g_wait_timeout));
        ptrs[dev] = static_cast<int*>(p);
    }
    *out = ptrs[dev];
    return MTA_OK;
}

int make_tensor_map_3d(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols,
                       uint64_t row_pitch_elems, uint64_t plane_pitch_elems, uint32_t box_cols, uint32_t box_rows,
                       bool swizzle128) {
    return make_tensor_map_3d_mode(out, base, planes, rows, cols, row_pitch_elems, plane_pitch_elems, box_cols, box_rows,
                                   swizzle128 ? 128 : 0);
}

int make_tensor_map_3d_mode(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols,
                            uint64_t row_pitch_elems, uint64_t plane_pitch_elems, uint32_t box_cols, uint32_t box_rows,
                            int swizzle_bytes) {
    const bool swizzle128 = swizzle_bytes == 128;
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return MTA_ERR_CUDA;
    }
    MTA_REQUIRE(aligned16(base) && (row_pitch_elems * 2) % 16 == 0 && (plane_pitch_elems * 2) % 16 == 0,
                "tensor map: base and pitches must be multiples of 16 bytes");
    cuuint64_t dims[3] = {cols, rows, planes};
    cuuint64_t strides[2] = {row_pitch_elems * 2, plane_pitch_elems * 2};
    MTA_REQUIRE(box_cols <= 256 && box_rows <= 256 && (box_cols * 2) % 16 == 0 && (!swizzle128 || box_cols == 64) &&
                    (swizzle_bytes != 32 || box_cols == 16) && (swizzle_bytes == 0 || swizzle_bytes == 32 || swizzle_bytes == 128),
                "tensor map: box %u x %u with a %d-byte swizzle is not supported", box_cols, box_rows, swizzle_bytes);
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : (swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE),
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return MTA_ERR_CUDA;
    }
    return MTA_OK;
}

// 4-D map (8 columns, rows, 8-column chunks, planes) of a [planes][rows][cols] tensor of 16-bit elements: a box
// {8, box_rows, box_chunks, 1} lands in shared memory as [chunk][row][8 columns], the layout a tcgen05 matrix
// descriptor without swizzle reads with any row offset.  Out-of-range rows and chunks read as zero.
int make_tensor_map_chunked(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols,
                            uint64_t row_pitch_elems, uint64_t plane_pitch_elems, uint32_t box_rows, uint32_t box_chunks) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return MTA_ERR_CUDA;
    }
    MTA_REQUIRE(aligned16(base) && cols % 8 == 0 && (row_pitch_elems * 2) % 16 == 0 && (plane_pitch_elems * 2) % 16 == 0 &&
                    box_rows <= 256 && box_chunks <= 256,
                "chunked tensor map: unsupported geometry");
    cuuint64_t dims[4] = {8, rows, cols / 8, planes};
    cuuint64_t strides[3] = {row_pitch_elems * 2, 16, plane_pitch_elems * 2};
    cuuint32_t box[4] = {8, box_rows, box_chunks, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (chunked view) failed with CUresult %d", (int)r);
        return MTA_ERR_CUDA;
    }
    return MTA_OK;
}

namespace {
using namespace tc05;

constexpr int TILE = 128;                 // rows of an operand tile / edge of a score tile
constexpr int BOX_BYTES = TILE * 128;     // one TMA box: 128 rows x 64 elements x 2 bytes = 16 KB

template <typename T> struct AbFormat;
template <> struct AbFormat<__nv_bfloat16> { static constexpr int value = 1; };
template <> struct AbFormat<__half> { static constexpr int value = 0; };

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ uint8_t* align_1024(uint8_t* p) {
    return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~uintptr_t(1023));
}

// Number of key tiles that query tile tq reaches: ceil(last query row + 1 / TILE), clamped.
__device__ __forceinline__ int key_tiles_for(int tq, int row_begin, int row_end, int S, int causal) {
    const int all = (S + TILE - 1) / TILE;
    if (!causal) return all;
    const int q_last = min(row_begin + (tq + 1) * TILE, row_end);     // one past the last row of the tile
    return min((q_last + TILE - 1) / TILE, all);
}

// ------------------------------------------------------------------------------------------------
// One CTA (4 warps) per 128 x 128 score tile.  Thread 0 issues the TMA loads and the MMAs; all four warps
// drain the accumulator: warp w owns TMEM lanes 32w..32w+31 = tile rows, each lane one row.  The tile leaves
// through shared memory and a TMA tiled store.
template <typename T, int D>
__global__ void __launch_bounds__(128)
qk_scores_tc05_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                      const __grid_constant__ CUtensorMap ms, int s_row0, int S, float scale, int round_scale, int causal,
                      int row_begin, int row_end, int* err_flag) {
    constexpr int NBOX = D / 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_1024(smem_raw);
    uint8_t* sq = smem;
    uint8_t* sk = smem + NBOX * BOX_BYTES;
    __shared__ __align__(8) uint64_t full_bar, mma_bar;
    __shared__ uint32_t tmem_slot;

    __shared__ int abort_flag;      // an earlier bounded wait on this device gave up: the whole CTA does nothing
    if (threadIdx.x == 0) abort_flag = *reinterpret_cast<volatile int*>(err_flag);
    __syncthreads();
    if (abort_flag != 0) return;
    // linear tile index -> (query tile, key tile)
    int tq = 0, tk = (int)blockIdx.x;
    for (;; ++tq) {
        const int nk = key_tiles_for(tq, row_begin, row_end, S, causal);
        if (tk < nk) break;
        tk -= nk;
    }
    const int bh = (int)blockIdx.y;
    const int q0 = row_begin + tq * TILE, k0 = tk * TILE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (warp == 0) {
        if (lane == 0) {
            mbar_init(&full_bar, 1);
            mbar_init(&mma_bar, 1);
            fence_mbar_init();
            prefetch_tensormap(&mq);
            prefetch_tensormap(&mk);
            prefetch_tensormap(&ms);
        }
        __syncwarp();
        tmem_alloc(&tmem_slot, 128);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;

    if (threadIdx.x == 0) {
        mbar_expect_tx(&full_bar, 2 * NBOX * BOX_BYTES);
#pragma unroll
        for (int j = 0; j < NBOX; ++j) {
            tma_load_3d(sq + j * BOX_BYTES, &mq, &full_bar, j * 64, q0, bh);
            tma_load_3d(sk + j * BOX_BYTES, &mk, &full_bar, j * 64, k0, bh);
        }
        mbar_wait(&full_bar, 0, err_flag);
        fence_after_sync();
        constexpr uint32_t idesc = instr_desc_f16(AbFormat<T>::value, 0, 0, TILE, TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk / 4) * BOX_BYTES + (kk % 4) * 32;
            mma_f16_ss(tmem, smem_desc_sw128(smem_u32(sq) + off, 16, 1024), smem_desc_sw128(smem_u32(sk) + off, 16, 1024),
                       idesc, kk > 0);
        }
        mma_commit(&mma_bar);
    }
    __syncwarp();
    mbar_wait(&mma_bar, 0, err_flag);
    __syncwarp();
    fence_after_sync();

    // Epilogue: a thread owns one row of the tile, so the 16-bit tile is staged in shared memory (over the operand
    // tiles, which are dead now) in the 128-byte-swizzled layout and leaves as two TMA tiled stores.
    const int row = warp * 32 + lane;
    const int q = q0 + row;
    const float sc = round_scale ? round_to<T>(scale) : scale;
    uint8_t* orow = smem + row * 128;
#pragma unroll 1
    for (int c = 0; c < TILE / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c * 32), r);
        tmem_ld_wait();
#pragma unroll
        for (int v8 = 0; v8 < 4; ++v8) {
            const int col = c * 32 + v8 * 8;
            const int k = k0 + col;
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float a = __uint_as_float(r[v8 * 8 + e]);
                f[e] = round_scale ? round_to<T>(a) * sc : a * sc;
                if (causal && k + e > q) f[e] = 0.0f;        // above the diagonal inside a visited tile: written as 0
            }
            uint4 o;
            o.x = pack2<T>(f[0], f[1]);
            o.y = pack2<T>(f[2], f[3]);
            o.z = pack2<T>(f[4], f[5]);
            o.w = pack2<T>(f[6], f[7]);
            const int ch = (col & 63) >> 3;
            *reinterpret_cast<uint4*>(orow + (col >> 6) * BOX_BYTES + ((ch ^ (row & 7)) << 4)) = o;
        }
    }
    fence_proxy_async();
    fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) {
        // rows past row_end and columns past S are outside the tensor map and are clipped
        tma_store_3d(&ms, smem, k0, q0 - s_row0, bh);
        if (k0 + 64 < S) tma_store_3d(&ms, smem + BOX_BYTES, k0 + 64, q0 - s_row0, bh);
        bulk_commit();
        bulk_wait_read();
    }
    if (warp == 0) tmem_dealloc(tmem, 128);
}

// ------------------------------------------------------------------------------------------------
// O tile = sum over key tiles of P tile x V tile.  Warp 0: TMA producer; warp 1: zeroes the part of a
// diagonal P tile that lies above the diagonal, then issues the MMAs; warps 2..5: epilogue.
#ifndef MTA_PV_STAGES
#define MTA_PV_STAGES 3
#endif
constexpr int PV_STAGES = MTA_PV_STAGES;
constexpr int PV_THREADS = 192;
constexpr int PV_KEYS = 64;               // keys per pipeline stage: 32 KB stages, so two CTAs fit on an SM and one CTA's
                                          // start-up and epilogue overlap the other's steady state
constexpr int PV_VBOX_BYTES = PV_KEYS * 128;   // one box of the V tile: 64 keys x 64 elements

template <typename T, int D>
__global__ void __launch_bounds__(PV_THREADS)
pv_tc05_kernel(const __grid_constant__ CUtensorMap mp, const __grid_constant__ CUtensorMap mv, T* __restrict__ o,
               int p_row0, int S, int causal, int row_begin, int row_end, int* err_flag) {
    constexpr int NBOX_V = D / 64;
    constexpr int P_BYTES = BOX_BYTES;                     // 128 q x 64 k
    constexpr int V_BYTES = NBOX_V * PV_VBOX_BYTES;        // 64 k x D
    constexpr int STAGE_BYTES = P_BYTES + V_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_1024(smem_raw);
    __shared__ __align__(8) uint64_t full_bar[PV_STAGES], empty_bar[PV_STAGES], acc_bar;
    __shared__ uint32_t tmem_slot;

    __shared__ int abort_flag;      // an earlier bounded wait on this device gave up: the whole CTA does nothing
    if (threadIdx.x == 0) abort_flag = *reinterpret_cast<volatile int*>(err_flag);
    __syncthreads();
    if (abort_flag != 0) return;
    // heaviest query tiles first: tile index counts down from the last
    const int n_qt = (row_end - row_begin + TILE - 1) / TILE;
    const int tq = n_qt - 1 - (int)blockIdx.x;
    const int bh = (int)blockIdx.y;
    const int q0 = row_begin + tq * TILE;
    const int q_end = min(q0 + TILE, row_end);
    // 64-key steps that hold a key <= the tile's last query
    const int nk = causal ? min((q_end + PV_KEYS - 1) / PV_KEYS, (S + PV_KEYS - 1) / PV_KEYS) : (S + PV_KEYS - 1) / PV_KEYS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < PV_STAGES; ++i) {
                mbar_init(&full_bar[i], 1);
                mbar_init(&empty_bar[i], 1);
            }
            mbar_init(&acc_bar, 1);
            fence_mbar_init();
            prefetch_tensormap(&mp);
            prefetch_tensormap(&mv);
        }
        __syncwarp();
        tmem_alloc(&tmem_slot, D < 32 ? 32 : D);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kt = 0; kt < nk; ++kt) {
                const int st = kt % PV_STAGES, use = kt / PV_STAGES;
                if (use > 0) mbar_wait(&empty_bar[st], (use - 1) & 1, err_flag);
                uint8_t* sp = smem + st * STAGE_BYTES;
                uint8_t* sv = sp + P_BYTES;
                mbar_expect_tx(&full_bar[st], STAGE_BYTES);
                tma_load_3d(sp, &mp, &full_bar[st], kt * PV_KEYS, q0 - p_row0, bh);
#pragma unroll
                for (int j = 0; j < NBOX_V; ++j) tma_load_3d(sv + j * PV_VBOX_BYTES, &mv, &full_bar[st], j * 64, kt * PV_KEYS, bh);
            }
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc = instr_desc_f16(AbFormat<T>::value, 0, 1, TILE, D);
        for (int kt = 0; kt < nk; ++kt) {
            const int st = kt % PV_STAGES, use = kt / PV_STAGES;
            uint8_t* sp = smem + st * STAGE_BYTES;
            uint8_t* sv = sp + P_BYTES;
            mbar_wait(&full_bar[st], use & 1, err_flag);
            const int k0 = kt * PV_KEYS;
            if (causal && k0 + PV_KEYS - 1 > q0) {
                // Keys above the diagonal must contribute nothing, whatever the buffer holds there.
                // Element (row r, key c) of the swizzled tile: byte r*128 + ((c/8) ^ (r%8))*16 + (c%8)*2.
                for (int idx = lane; idx < TILE * 8; idx += 32) {
                    const int r = idx >> 3, ch = idx & 7;              // 16-byte chunk ch covers keys 8ch..8ch+7
                    const int qrow = q0 + r, kfirst = k0 + ch * 8;
                    if (kfirst + 7 <= qrow) continue;
                    uint8_t* chunk = sp + r * 128 + ((ch ^ (r & 7)) << 4);
                    if (kfirst > qrow) {
                        *reinterpret_cast<uint4*>(chunk) = make_uint4(0u, 0u, 0u, 0u);
                    } else {
                        uint16_t* e16 = reinterpret_cast<uint16_t*>(chunk);
                        for (int e = 0; e < 8; ++e)
                            if (kfirst + e > qrow) e16[e] = 0;
                    }
                }
                fence_proxy_async();
            }
            __syncwarp();
            fence_after_sync();
            if (lane == 0) {
#pragma unroll
                for (int kk = 0; kk < PV_KEYS / 16; ++kk) {
                    const uint64_t da = smem_desc_sw128(smem_u32(sp) + kk * 32, 16, 1024);
                    const uint64_t db = smem_desc_sw128(smem_u32(sv) + kk * 16 * 128, PV_VBOX_BYTES, 1024);
                    mma_f16_ss(tmem, da, db, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
                }
                mma_commit(&empty_bar[st]);
                if (kt == nk - 1) mma_commit(&acc_bar);
            }
            __syncwarp();
        }
    } else {
        mbar_wait(&acc_bar, 0, err_flag);
        __syncwarp();
        fence_after_sync();
        const int quarter = warp & 3;                    // TMEM lanes this warp may read
        const int q = q0 + quarter * 32 + lane;
        T* orow = o + ((long)bh * S + (q < q_end ? q : q0)) * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), r);
            tmem_ld_wait();
            if (q >= q_end) continue;
#pragma unroll
            for (int v8 = 0; v8 < 4; ++v8) {
                uint4 w;
                w.x = pack2<T>(__uint_as_float(r[v8 * 8 + 0]), __uint_as_float(r[v8 * 8 + 1]));
                w.y = pack2<T>(__uint_as_float(r[v8 * 8 + 2]), __uint_as_float(r[v8 * 8 + 3]));
                w.z = pack2<T>(__uint_as_float(r[v8 * 8 + 4]), __uint_as_float(r[v8 * 8 + 5]));
                w.w = pack2<T>(__uint_as_float(r[v8 * 8 + 6]), __uint_as_float(r[v8 * 8 + 7]));
                *reinterpret_cast<uint4*>(orow + c * 32 + v8 * 8) = w;
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, D < 32 ? 32 : D);
}

template <typename T, int D>
int launch_qk(const void* q, const void* k, void* s, PlaneView sv, int B, int H, int S, float scale, int round_scale,
              int causal, int row_begin, int row_end, cudaStream_t st) {
    CUtensorMap mq, mk;
    int rc;
    if ((rc = make_tensor_map_3d(&mq, q, (uint64_t)B * H, S, D, D, (uint64_t)S * D, 64, TILE, true))) return rc;
    if ((rc = make_tensor_map_3d(&mk, k, (uint64_t)B * H, S, D, D, (uint64_t)S * D, 64, TILE, true))) return rc;
    CUtensorMap ms;      // rows past row_end are outside this map, so a tile's store never touches them
    if ((rc = make_tensor_map_3d(&ms, s, (uint64_t)B * H, (uint64_t)(row_end - sv.row0), S, S, (uint64_t)sv.plane_stride, 64, TILE, true)))
        return rc;
    int* flag = nullptr;
    if ((rc = wait_flag_ptr(&flag))) return rc;
    const int n_qt = (row_end - row_begin + TILE - 1) / TILE, all_k = (S + TILE - 1) / TILE;
    long tiles = 0;
    for (int tq = 0; tq < n_qt; ++tq) {
        const int q_last = std::min(row_begin + (tq + 1) * TILE, row_end);
        tiles += causal ? std::min((q_last + TILE - 1) / TILE, all_k) : all_k;
    }
    const size_t smem = 2 * (D / 64) * BOX_BYTES + 1024;
    MTA_CUDA_OK(cudaFuncSetAttribute(qk_scores_tc05_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)tiles, (unsigned)(B * H));
    qk_scores_tc05_kernel<T, D><<<grid, 128, smem, st>>>(mq, mk, ms, sv.row0, S, scale, round_scale, causal, row_begin,
                                                         row_end, flag);
    MTA_LAUNCH_OK("qk_scores_tc05_kernel");
    return MTA_OK;
}

template <typename T, int D>
int launch_pv(const void* p, PlaneView pview, const void* v, void* o, int B, int H, int S, int causal, int row_begin,
              int row_end, long p_rows_stored, cudaStream_t st) {
    CUtensorMap mp, mv;
    int rc;
    if ((rc = make_tensor_map_3d(&mp, p, (uint64_t)B * H, (uint64_t)p_rows_stored, S, S, (uint64_t)pview.plane_stride, 64, TILE, true))) return rc;
    if ((rc = make_tensor_map_3d(&mv, v, (uint64_t)B * H, S, D, D, (uint64_t)S * D, 64, PV_KEYS, true))) return rc;
    int* flag = nullptr;
    if ((rc = wait_flag_ptr(&flag))) return rc;
    const int n_qt = (row_end - row_begin + TILE - 1) / TILE;
    const size_t smem = (size_t)PV_STAGES * (BOX_BYTES + (D / 64) * PV_VBOX_BYTES) + 1024;
    MTA_CUDA_OK(cudaFuncSetAttribute(pv_tc05_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)n_qt, (unsigned)(B * H));
    pv_tc05_kernel<T, D><<<grid, PV_THREADS, smem, st>>>(mp, mv, static_cast<T*>(o), pview.row0, S, causal, row_begin,
                                                         row_end, flag);
    MTA_LAUNCH_OK("pv_tc05_kernel");
    return MTA_OK;
}

}  // namespace

bool tc05_contractions_supported(int S, int D, int dtype, const void* a, const void* b, const void* c, PlaneView view) {
    return dtype != MTA_F32 && (D == 64 || D == 128) && S % 8 == 0 && view.width == S && view.plane_stride % 8 == 0 &&
           aligned16(a) && aligned16(b) && aligned16(c);
}

int qk_scores_tc05_launch(const void* q, const void* k, void* s, PlaneView sv, int B, int H, int S, int D, float scale,
                          int round_scale, int causal, int row_begin, int row_end, int dtype, cudaStream_t st) {
#define MTA_QK(TT, DD) return launch_qk<TT, DD>(q, k, s, sv, B, H, S, scale, round_scale, causal, row_begin, row_end, st)
    if (dtype == MTA_BF16) { if (D == 64) MTA_QK(__nv_bfloat16, 64); MTA_QK(__nv_bfloat16, 128); }
    if (D == 64) MTA_QK(__half, 64);
    MTA_QK(__half, 128);
#undef MTA_QK
}

int pv_tc05_launch(const void* p, PlaneView pview, long p_rows_stored, const void* v, void* o, int B, int H, int S, int D,
                   int causal, int row_begin, int row_end, int dtype, cudaStream_t st) {
#define MTA_PV(TT, DD) return launch_pv<TT, DD>(p, pview, v, o, B, H, S, causal, row_begin, row_end, p_rows_stored, st)
    if (dtype == MTA_BF16) { if (D == 64) MTA_PV(__nv_bfloat16, 64); MTA_PV(__nv_bfloat16, 128); }
    if (D == 64) MTA_PV(__half, 64);
    MTA_PV(__half, 128);
#undef MTA_PV
}

// Reads and clears the flag that bounded device-side waits raise.  Synchronises the stream.
int device_wait_status(cudaStream_t st, int* timed_out) {
    int* flag = nullptr;
    if (int rc = wait_flag_ptr(&flag)) return rc;
    int h = 0;
    MTA_CUDA_OK(cudaMemcpyAsync(&h, flag, sizeof(int), cudaMemcpyDeviceToHost, st));
    MTA_CUDA_OK(cudaStreamSynchronize(st));
    if (h) {
        int zero = 0;
        MTA_CUDA_OK(cudaMemcpyAsync(flag, &zero, sizeof(int), cudaMemcpyHostToDevice, st));
        MTA_CUDA_OK(cudaStreamSynchronize(st));
    }
    *timed_out = h;
    return MTA_OK;
}

}  // namespace mta
