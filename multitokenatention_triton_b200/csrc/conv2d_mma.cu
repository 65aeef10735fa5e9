// Depthwise causal conv over score planes on the tensor cores, 16-bit dtypes, key extent S <= 17.
//
// The key-direction taps of one kernel row are a banded (Toeplitz) matrix: for a fixed row tap i,
//   out[q, k] += sum_kk X[q + i - (R-1), kk] * T_i[kk, k],     T_i[kk, k] = w[i, kk - k + pad_w]  (0 outside the band)
// so a 16-row x 8-column block of outputs is two m16n8k16 MMAs per row tap: A = 16 staged input rows x 16
// input columns (ldmatrix from the staged tile; a row tap is just a different row address), B = a 16 x 8 slice
// of T_i, which only depends on (i, column offset between the slice and the block) - four variants per row
// tap, precomputed once per CTA into shared memory in MMA fragment order.  Products of 16-bit values are exact
// and accumulate in fp32, so the result equals the fp32 CUDA-core kernel up to summation order.
//
// Data movement: one TMA tiled load per CTA brings the (64 + R-1) x 152 halo tile into shared memory
// (out-of-range rows/columns arrive as zero, which is the conv's zero padding); the part of the tile above the
// causal diagonal is then zeroed in shared memory; outputs are staged through shared memory and leave as
// 16-byte coalesced stores.  Tiles entirely above the diagonal read nothing.
#include "kernels.cuh"
#include "tc05.cuh"

namespace mta {
namespace {
using namespace tc05;

constexpr int CM = 64;              // output rows per CTA
constexpr int CN = 128;             // output columns per CTA
constexpr int SW = 152;             // staged columns: CN + 8 (left halo, 16-byte aligned) + 16
constexpr int SPITCH = SW * 2;      // bytes per staged row (19 x 16: ldmatrix rows fall in distinct banks)
constexpr int OPITCH = 272;         // bytes per staged output row (17 x 16)
constexpr int CONV_THREADS = 256;   // 8 warps: 4 along rows x 2 along columns, 16 x 64 outputs each

template <typename T> struct MmaType;
template <> struct MmaType<__nv_bfloat16> { static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1)); } };
template <> struct MmaType<__half> { static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1)); } };

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}

template <typename T> __device__ __forceinline__ uint32_t pack2w(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2w<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t pack2w<__half>(float lo, float hi) {
    __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}

// Shared memory: [staged tile | output staging (aliases the tile)] [B fragments hi] [B fragments lo]
//   B fragments: [row tap i][variant v (column offset delta = 8v - 8)][lane][2 words]
template <typename T>
__global__ void __launch_bounds__(CONV_THREADS)
conv2d_mma_kernel(const __grid_constant__ CUtensorMap mx, const void* __restrict__ w, int w_dtype, T* __restrict__ y,
                  PlaneView yv, int x_row0, int C, int H, int W, int R, int S, int causal, int row_begin, int row_end,
                  int write_upper, int tiles_n, int split_w, int* err_flag) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t bar;
    const int TH = CM + R - 1;
    uint8_t* xs = smem;
    const int xs_bytes = ((TH * SPITCH > CM * OPITCH ? TH * SPITCH : CM * OPITCH) + 127) & ~127;
    uint32_t* bfrag = reinterpret_cast<uint32_t*>(smem + xs_bytes);          // R*4*64 words
    uint32_t* bfrag_lo = bfrag + R * 256;

    const long plane = blockIdx.y;
    const int tile_m = (int)blockIdx.x / tiles_n, tile_n = (int)blockIdx.x % tiles_n;
    const int m0 = row_begin + tile_m * CM, n0 = tile_n * CN;
    const int m_end = min(m0 + CM, row_end);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pad_w = (S - 1) / 2;
    const int pad8 = (pad_w + 7) & ~7;         // left halo rounded up to 8 columns (16 bytes)
    const int a_off = pad8 - pad_w;            // staged column of tap j for output column x: x + a_off + j
    T* yp = y + plane * yv.plane_stride;

    if (causal && n0 > m_end - 1) {            // tile entirely above the diagonal
        if (write_upper) {
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
            for (int idx = tid; idx < CM * (CN / 8); idx += CONV_THREADS) {
                const int q = m0 + idx / (CN / 8), k = n0 + (idx % (CN / 8)) * 8;
                if (q < m_end && k < W) *reinterpret_cast<uint4*>(yp + (long)(q - yv.row0) * yv.width + k) = z;
            }
        }
        return;
    }

    if (tid == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (tid == 0) {
        mbar_expect_tx(&bar, (uint32_t)(TH * SPITCH));
        tma_load_3d(xs, &mx, &bar, n0 - pad8, m0 - (R - 1) - x_row0, (int)plane);
    }

    // B fragments while the tile is in flight.  Fragment element (kk, n) of variant delta holds w[i][kk - n + delta - a_off].
    const int c = (int)(plane % C);
    for (int idx = tid; idx < R * 256; idx += CONV_THREADS) {
        const int i = idx >> 8, v = (idx >> 6) & 3, ln = (idx >> 1) & 31, reg = idx & 1;
        const int g = ln >> 2, t4 = ln & 3;
        const int delta = 8 * v - 8;
        float hi[2], lo[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int kk = 2 * t4 + e + 8 * reg;
            const int j = kk - g + delta - a_off;
            float wv = (j >= 0 && j < S) ? load_weight(w, ((long)c * R + i) * S + j, w_dtype) : 0.0f;
            hi[e] = round_to<T>(wv);
            lo[e] = wv - hi[e];
        }
        bfrag[idx] = pack2w<T>(hi[0], hi[1]);
        if (split_w) bfrag_lo[idx] = pack2w<T>(lo[0], lo[1]);
    }

    mbar_wait(&bar, 0, err_flag);
    // zero what lies above the causal diagonal: staged row sr is query m0-(R-1)+sr, staged column sc is key n0-pad8+sc
    if (causal && n0 - pad8 + SW - 1 > m0 - (R - 1)) {
        const int chunks = SW / 8;
        for (int idx = tid; idx < TH * chunks; idx += CONV_THREADS) {
            const int sr = idx / chunks, ch = idx - sr * chunks;
            const int qq = m0 - (R - 1) + sr;
            const int z0 = qq - (n0 - pad8) + 1;              // first staged column to zero
            const int sc = ch * 8;
            if (sc + 7 < z0) continue;
            uint8_t* p = xs + sr * SPITCH + sc * 2;
            if (sc >= z0) {
                *reinterpret_cast<uint4*>(p) = make_uint4(0u, 0u, 0u, 0u);
            } else {
                uint16_t* e16 = reinterpret_cast<uint16_t*>(p);
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (sc + e >= z0) e16[e] = 0;
            }
        }
    }
    __syncthreads();

    // warp tile: rows r0..r0+15, columns cw..cw+63 of the CTA tile
    const int r0 = (warp & 3) * 16, cw = (warp >> 2) * 64;
    float acc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
    const uint32_t xs_addr = smem_u32(xs);
    // lane's row/column inside a 16 x 16 A fragment for ldmatrix.x4: matrices (r0-7,c0-7) (r8-15,c0-7) (r0-7,c8-15) (r8-15,c8-15)
    const uint32_t a_lane_off = (uint32_t)((((lane >> 3) & 1) * 8 + (lane & 7)) * SPITCH + (lane >> 4) * 16);
    for (int i = 0; i < R; ++i) {
        // B fragments of this row tap: variant v -> 2 words
        uint32_t bf[4][2], bl[4][2];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const uint2 t2 = *reinterpret_cast<const uint2*>(bfrag + ((i * 4 + v) * 32 + lane) * 2);
            bf[v][0] = t2.x;
            bf[v][1] = t2.y;
            if (split_w) {
                const uint2 l2 = *reinterpret_cast<const uint2*>(bfrag_lo + ((i * 4 + v) * 32 + lane) * 2);
                bl[v][0] = l2.x;
                bl[v][1] = l2.y;
            } else {
                bl[v][0] = bl[v][1] = 0u;
            }
        }
        // five 16-column steps cover staged columns cw .. cw+79; step m feeds column blocks 2m-2 .. 2m+1
#pragma unroll
        for (int m = 0; m < 5; ++m) {
            uint32_t a[4];
            ldmatrix_x4(a, xs_addr + (uint32_t)((r0 + i) * SPITCH + (cw + 16 * m) * 2) + a_lane_off);
#pragma unroll
            for (int d = -2; d <= 1; ++d) {
                const int nt = 2 * m + d;
                if (nt < 0 || nt >= 8) continue;
                // delta = (staged start of the step) - (first column of the block) = 16m - 8nt = -8d
                const int v = 1 - d;        // delta = 8v - 8
                MmaType<T>::mma(acc[nt], a, bf[v][0], bf[v][1]);
                if (split_w) MmaType<T>::mma(acc[nt], a, bl[v][0], bl[v][1]);
            }
        }
    }
    __syncthreads();           // every warp is done reading the staged tile: reuse it for the outputs

    {
        const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            uint8_t* o0 = xs + (r0 + g) * OPITCH + (cw + nt * 8 + 2 * t4) * 2;
            *reinterpret_cast<uint32_t*>(o0) = pack2w<T>(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<uint32_t*>(o0 + 8 * OPITCH) = pack2w<T>(acc[nt][2], acc[nt][3]);
        }
    }
    __syncthreads();
    for (int idx = tid; idx < CM * (CN / 8); idx += CONV_THREADS) {
        const int r = idx / (CN / 8), ch = idx % (CN / 8);
        const int q = m0 + r, k = n0 + ch * 8;
        if (q >= m_end || k >= W) continue;
        uint4 val = *reinterpret_cast<const uint4*>(xs + r * OPITCH + ch * 16);
        T* dst = yp + (long)(q - yv.row0) * yv.width + k;
        if (causal && k + 7 > q) {
            if (k > q) {
                if (write_upper) *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
                continue;
            }
            if (!write_upper) {
                const T* v16 = reinterpret_cast<const T*>(&val);
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (k + e <= q) dst[e] = v16[e];
                continue;
            }
            uint16_t* v16 = reinterpret_cast<uint16_t*>(&val);
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (k + e > q) v16[e] = 0;
        }
        *reinterpret_cast<uint4*>(dst) = val;
    }
}

template <typename T>
int launch_mma(const void* x, PlaneView xv, long x_rows_stored, const void* w, int w_dtype, void* y, PlaneView yv,
               long planes, int C, int H, int W, int R, int S, int causal, int row_begin, int row_end, bool write_upper,
               cudaStream_t st) {
    CUtensorMap mx;
    int rc;
    const int TH = CM + R - 1;
    if ((rc = make_tensor_map_3d(&mx, x, (uint64_t)planes, (uint64_t)x_rows_stored, (uint64_t)W, (uint64_t)xv.width,
                                 (uint64_t)xv.plane_stride, SW, (uint32_t)TH, false)))
        return rc;
    int* flag = nullptr;
    if ((rc = wait_flag_ptr(&flag))) return rc;
    const int tiles_m = (row_end - row_begin + CM - 1) / CM, tiles_n = (W + CN - 1) / CN;
    const int xs_bytes = ((TH * SPITCH > CM * OPITCH ? TH * SPITCH : CM * OPITCH) + 127) & ~127;
    const size_t smem = (size_t)xs_bytes + (size_t)R * 256 * 4 * 2;
    if (smem > 48 * 1024)
        MTA_CUDA_OK(cudaFuncSetAttribute(conv2d_mma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)(tiles_m * tiles_n), (unsigned)planes);
    conv2d_mma_kernel<T><<<grid, CONV_THREADS, smem, st>>>(mx, w, w_dtype, static_cast<T*>(y), yv, xv.row0, C, H, W, R, S,
                                                           causal, row_begin, row_end, write_upper ? 1 : 0, tiles_n,
                                                           w_dtype == MTA_F32 ? 1 : 0, flag);
    MTA_LAUNCH_OK("conv2d_mma_kernel");
    return MTA_OK;
}

}  // namespace

bool conv2d_mma_supported(const void* x, PlaneView xv, const void* y, PlaneView yv, int W, int R, int S, int dtype) {
    return dtype != MTA_F32 && S <= 17 && R <= 64 && W % 8 == 0 && xv.width == W && yv.width == W &&
           xv.plane_stride % 8 == 0 && yv.plane_stride % 8 == 0 && aligned16(x) && aligned16(y);
}

int conv2d_mma_launch(const void* x, PlaneView xv, long x_rows_stored, const void* w, int w_dtype, void* y, PlaneView yv,
                      long planes, int C, int H, int W, int R, int S, int causal, int row_begin, int row_end,
                      bool write_upper, int dtype, cudaStream_t st) {
    if (dtype == MTA_BF16)
        return launch_mma<__nv_bfloat16>(x, xv, x_rows_stored, w, w_dtype, y, yv, planes, C, H, W, R, S, causal, row_begin,
                                         row_end, write_upper, st);
    return launch_mma<__half>(x, xv, x_rows_stored, w, w_dtype, y, yv, planes, C, H, W, R, S, causal, row_begin, row_end,
                              write_upper, st);
}

}  // namespace mta
