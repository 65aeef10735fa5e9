// Shared host/device helpers of the mta_b200 library: status codes, error text, dtype plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/mta_b200.h"

namespace mta {

// ---- host side -------------------------------------------------------------------------------
void set_error(const char* fmt, ...);          // thread-local message for mta_last_error()
void count_launch(int n = 1);                  // bumps the per-thread launch counter
int variant(const char* key);                  // value set through mta_set_variant (0 = auto)
int check_device();                            // MTA_OK when the current device is sm_100

#define MTA_REQUIRE(cond, ...)                                  \
    do {                                                        \
        if (!(cond)) {                                          \
            ::mta::set_error(__VA_ARGS__);                      \
            return MTA_ERR_INVALID;                             \
        }                                                       \
    } while (0)

#define MTA_CUDA_OK(expr)                                                                   \
    do {                                                                                    \
        cudaError_t e__ = (expr);                                                           \
        if (e__ != cudaSuccess) {                                                           \
            ::mta::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__),       \
                             __FILE__, __LINE__);                                           \
            return MTA_ERR_CUDA;                                                            \
        }                                                                                   \
    } while (0)

// Launch status after a <<<>>> statement; counts the launch.
#define MTA_LAUNCH_OK(name)                                                                 \
    do {                                                                                    \
        cudaError_t e__ = cudaGetLastError();                                               \
        if (e__ != cudaSuccess) {                                                           \
            ::mta::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__));     \
            return MTA_ERR_CUDA;                                                            \
        }                                                                                   \
        ::mta::count_launch();                                                              \
    } while (0)

inline size_t dtype_size(int dt) { return dt == MTA_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == MTA_F32 || dt == MTA_BF16 || dt == MTA_F16; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- device side -----------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Round a float to T and back: the place where a 16-bit run of the reference rounds an intermediate.
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

// Weight element `i` of an array whose dtype is only known at run time (weights are tiny).
__device__ __forceinline__ float load_weight(const void* w, long i, int w_dtype) {
    if (w_dtype == MTA_F32) return reinterpret_cast<const float*>(w)[i];
    if (w_dtype == MTA_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]);
    return __half2float(reinterpret_cast<const __half*>(w)[i]);
}

template <typename T> struct DTypeOf;
template <> struct DTypeOf<float> { static constexpr int value = MTA_F32; };
template <> struct DTypeOf<__nv_bfloat16> { static constexpr int value = MTA_BF16; };
template <> struct DTypeOf<__half> { static constexpr int value = MTA_F16; };

// A view of score planes stored as [plane][row - row0][col]: the same kernels serve whole (N,C,H,W)
// tensors (row0 = 0, plane_stride = H*W) and row-range scratch buffers of the fused forward.
struct PlaneView {
    long plane_stride;   // elements between consecutive planes
    int row0;            // absolute index of the first stored row
    int width;           // row pitch = number of columns
    __host__ __device__ long at(long plane, int row, int col) const {
        return plane * plane_stride + (long)(row - row0) * width + col;
    }
};

}  // namespace mta
