// The two contractions of the forward on the 5th-generation tensor cores (tcgen05), 16-bit dtypes:
//   output tile  O[128 q x D]     = sum over key tiles  P[128 q x 128 k] V[128 k x D]   (A K-major, B MN-major)
// Operand tiles arrive by TMA (128-byte swizzle, out-of-range rows and columns read as zero), the
// accumulator lives in tensor memory, and only tiles that touch keys k <= q are visited when causal.
// They stand in for the torch.matmul calls at mta_attention_triton.py:68-71 and :89.
#include <cstddef>
#include <mutex>

#include "kernels.cuh"
#include "tc05.cuh"

namespace mta {

// ---- host helpers ----------------------------------------------------------------------------------
namespace {
// What a bounded wait raises when it gives up: the flag the kernels test on entry, and the address of its mirror in
// page-locked host memory, which lets the entry points see a timeout without synchronising with the device.
struct WaitFlag {
    int flag;
    int pad;
    int* host_mirror;
};
__device__ WaitFlag g_wait_timeout = {0, 0, nullptr};
std::mutex g_flag_mutex;
int* g_flag_dev[64] = {};          // per device: address of g_wait_timeout.flag
int* g_flag_host[64] = {};         // per device: the host mirror (mapped page-locked memory)

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
    int dev = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_flag_mutex);
    if (!g_flag_dev[dev]) {
        // first tcgen05 launch on this device: look up the flag and give it a host-visible mirror (4 bytes of mapped
        // page-locked memory, kept until the process ends)
        void* p = nullptr;
        MTA_CUDA_OK(cudaGetSymbolAddress(&p, g_wait_timeout));
        int* host = nullptr;
        int* host_dev = nullptr;
        MTA_CUDA_OK(cudaHostAlloc(reinterpret_cast<void**>(&host), sizeof(int), cudaHostAllocMapped));
        *host = 0;
        MTA_CUDA_OK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&host_dev), host, 0));
        MTA_CUDA_OK(cudaMemcpy(static_cast<char*>(p) + offsetof(WaitFlag, host_mirror), &host_dev, sizeof(host_dev), cudaMemcpyHostToDevice));
        g_flag_host[dev] = host;
        g_flag_dev[dev] = static_cast<int*>(p);
    }
    *out = g_flag_dev[dev];
    return MTA_OK;
}

// True when a bounded wait has given up on the current device since the last mta_device_status (no synchronisation:
// reads the host mirror the kernel wrote).
bool wait_flag_raised() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    const int* host = g_flag_host[dev];
    return host && *reinterpret_cast<const volatile int*>(host) != 0;
}

// Raises the flag from the host as a kernel's timed-out wait would (fault injection without a fault on the device).
int wait_flag_inject(cudaStream_t st) {
    int* flag = nullptr;
    if (int rc = wait_flag_ptr(&flag)) return rc;
    int dev = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    const int one = 1;
    MTA_CUDA_OK(cudaMemcpyAsync(flag, &one, sizeof(int), cudaMemcpyHostToDevice, st));
    MTA_CUDA_OK(cudaStreamSynchronize(st));
    *reinterpret_cast<volatile int*>(g_flag_host[dev]) = 1;
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
                            int swizzle_bytes, uint32_t box_planes) {
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
    MTA_REQUIRE(box_cols <= 256 && box_rows <= 256 && box_planes >= 1 && box_planes <= 256 && (box_cols * 2) % 16 == 0 && (!swizzle128 || box_cols == 64) &&
                    (swizzle_bytes != 32 || box_cols == 16) && (swizzle_bytes != 64 || box_cols == 32) &&
                    (swizzle_bytes == 0 || swizzle_bytes == 32 || swizzle_bytes == 64 || swizzle_bytes == 128),
                "tensor map: box %u x %u with a %d-byte swizzle is not supported", box_cols, box_rows, swizzle_bytes);
    cuuint32_t box[3] = {box_cols, box_rows, box_planes};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B
                               : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                      : (swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE)),
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

// ------------------------------------------------------------------------------------------------
// O tile = sum over key tiles of P tile x V tile.  Warp 0: TMA producer; warp 1: zeroes the part of a
// diagonal P tile that lies above the diagonal, then issues the MMAs; warps 2..5: epilogue.
constexpr int PV_STAGES = 3;
constexpr int PV_THREADS = 192;
constexpr int PV_KEYS = 64;               // keys per pipeline stage: 32 KB stages, so two CTAs fit on an SM and one CTA's
                                          // start-up and epilogue overlap the other's steady state
constexpr int PV_VBOX_BYTES = PV_KEYS * 128;   // one box of the V tile: 64 keys x 64 elements

// DROP: the four epilogue warps, idle until the accumulator is complete, apply the dropout of dropout.cuh to every P tile
// in shared memory before its MMAs are issued (a thread owns a row of the tile).
template <typename T, int D, bool DROP>
__global__ void __launch_bounds__(PV_THREADS)
pv_tc05_kernel(const __grid_constant__ CUtensorMap mp, const __grid_constant__ CUtensorMap mv, T* __restrict__ o,
               int p_row0, int S, int causal, int row_begin, int row_end, int* err_flag, DropoutSpec drop) {
    constexpr int NBOX_V = D / 64;
    constexpr int P_BYTES = BOX_BYTES;                     // 128 q x 64 k
    constexpr int V_BYTES = NBOX_V * PV_VBOX_BYTES;        // 64 k x D
    constexpr int STAGE_BYTES = P_BYTES + V_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_1024(smem_raw);
    __shared__ __align__(8) uint64_t full_bar[PV_STAGES], empty_bar[PV_STAGES], mask_bar[PV_STAGES], acc_bar;
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
                mbar_init(&mask_bar[i], 4);
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
            if (DROP) mbar_wait(&mask_bar[st], use & 1, err_flag);         // the epilogue warps have applied the dropout
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
        if (DROP) {
            const int r = (int)threadIdx.x - 64;             // row of the P tile this thread owns
            const uint32_t thr = drop.keep_threshold();
            const float scale = drop.scale();
            for (int kt = 0; kt < nk; ++kt) {
                const int st = kt % PV_STAGES, use = kt / PV_STAGES;
                uint8_t* sp = smem + st * STAGE_BYTES;
                mbar_wait(&full_bar[st], use & 1, err_flag);
#pragma unroll 2
                for (int ch = 0; ch < 8; ++ch) {
                    const uint32_t keep = dropout_keep8(drop.seed, (uint32_t)bh, (uint32_t)(q0 + r), (uint32_t)(kt * (PV_KEYS / 8) + ch), thr);
                    T* e8 = reinterpret_cast<T*>(sp + r * 128 + ((ch ^ (r & 7)) << 4));
#pragma unroll
                    for (int e = 0; e < 8; ++e) e8[e] = (keep >> e) & 1u ? from_f32<T>(to_f32<T>(e8[e]) * scale) : from_f32<T>(0.0f);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&mask_bar[st]);
            }
        }
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
int launch_pv(const void* p, PlaneView pview, const void* v, void* o, int B, int H, int S, int causal, int row_begin,
              int row_end, long p_rows_stored, cudaStream_t st, DropoutSpec drop) {
    CUtensorMap mp, mv;
    int rc;
    if ((rc = make_tensor_map_3d(&mp, p, (uint64_t)B * H, (uint64_t)p_rows_stored, S, S, (uint64_t)pview.plane_stride, 64, TILE, true))) return rc;
    if ((rc = make_tensor_map_3d(&mv, v, (uint64_t)B * H, S, D, D, (uint64_t)S * D, 64, PV_KEYS, true))) return rc;
    int* flag = nullptr;
    if ((rc = wait_flag_ptr(&flag))) return rc;
    const int n_qt = (row_end - row_begin + TILE - 1) / TILE;
    const size_t smem = (size_t)PV_STAGES * (BOX_BYTES + (D / 64) * PV_VBOX_BYTES) + 1024;
    dim3 grid((unsigned)n_qt, (unsigned)(B * H));
    if (drop.on()) {
        MTA_CUDA_OK(cudaFuncSetAttribute(pv_tc05_kernel<T, D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        pv_tc05_kernel<T, D, true><<<grid, PV_THREADS, smem, st>>>(mp, mv, static_cast<T*>(o), pview.row0, S, causal, row_begin,
                                                                   row_end, flag, drop);
    } else {
        MTA_CUDA_OK(cudaFuncSetAttribute(pv_tc05_kernel<T, D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        pv_tc05_kernel<T, D, false><<<grid, PV_THREADS, smem, st>>>(mp, mv, static_cast<T*>(o), pview.row0, S, causal, row_begin,
                                                                    row_end, flag, drop);
    }
    MTA_LAUNCH_OK("pv_tc05_kernel");
    return MTA_OK;
}

}  // namespace

bool tc05_contractions_supported(int S, int D, int dtype, const void* a, const void* b, const void* c, PlaneView view) {
    return dtype != MTA_F32 && (D == 64 || D == 128) && S % 8 == 0 && view.width == S && view.plane_stride % 8 == 0 &&
           aligned16(a) && aligned16(b) && aligned16(c);
}

int pv_tc05_launch(const void* p, PlaneView pview, long p_rows_stored, const void* v, void* o, int B, int H, int S, int D,
                   int causal, int row_begin, int row_end, int dtype, cudaStream_t st, DropoutSpec drop) {
#define MTA_PV(TT, DD) return launch_pv<TT, DD>(p, pview, v, o, B, H, S, causal, row_begin, row_end, p_rows_stored, st, drop)
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
    int dev = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    if (h || *reinterpret_cast<volatile int*>(g_flag_host[dev])) {
        int zero = 0;
        MTA_CUDA_OK(cudaMemcpyAsync(flag, &zero, sizeof(int), cudaMemcpyHostToDevice, st));
        MTA_CUDA_OK(cudaStreamSynchronize(st));
        *reinterpret_cast<volatile int*>(g_flag_host[dev]) = 0;
        h = 1;
    }
    *timed_out = h;
    return MTA_OK;
}

}  // namespace mta
