// Blackwell (sm_100a) building blocks in inline PTX: mbarriers with bounded waits, TMA tiled loads,
// tensor-memory (TMEM) allocation, tcgen05.mma with shared-memory descriptors, tcgen05.ld.
//
// Conventions used by every kernel that includes this file:
//   * operand tiles are written by TMA with the 128-byte swizzle into 1024-byte aligned shared memory:
//     one box = 64 16-bit elements (128 bytes) along the contiguous dimension x R rows, row r at byte r*128;
//   * every wait is bounded: after WAIT_LIMIT polls it gives up, raises the library's device error flag
//     and the kernel carries on to its exit (results are then garbage, but nothing hangs).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace mta {
namespace tc05 {

constexpr uint32_t WAIT_LIMIT = 1u << 20;     // polls of mbarrier.try_wait (each can block ~1 us in hardware)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// A wait gave up: raise the device flag (later kernels return at once) and its mirror in host memory, whose address sits
// two ints after the flag (the host then sees the timeout without synchronising).
__device__ __forceinline__ void raise_wait_flag(int* err_flag) {
    if (atomicExch(err_flag, 1) == 0) {
        int* mirror = *reinterpret_cast<int* volatile*>(err_flag + 2);
        if (mirror) {
            *reinterpret_cast<volatile int*>(mirror) = 1;
            __threadfence_system();
        }
    }
}
// Bounded wait for the phase with the given parity.  Returns false (and raises *err_flag) on timeout.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        // Back off: hundreds of threads polling barriers in shared memory slow down the tensor core's operand reads.
        if (i >= 4) __nanosleep(i < 64 ? 64 : 256);
        // once any wait on the device has given up, every other one gives up quickly
        if ((i & 1023u) == 1023u && *reinterpret_cast<volatile int*>(err_flag) != 0) return false;
    }
    raise_wait_flag(err_flag);
    return false;
}

// The same wait without the back-off, for hand-offs on a kernel's critical path where a few warps poll: a sleeping
// waiter wakes up to 256 ns late, which adds up when several hand-offs follow one another per tile.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, int* err_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT * 8u; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 8191u) == 8191u && *reinterpret_cast<volatile int*>(err_flag) != 0) return false;
    }
    raise_wait_flag(err_flag);
    return false;
}

// ---- TMA -----------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 3-D tiled load (x = contiguous element index, y = row, z = plane) that completes on `bar`.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// The same load with an L2 eviction policy (from createpolicy) attached to the lines it touches.
__device__ __forceinline__ void tma_load_3d_hint(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;\n"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// Plain (untiled) bulk copy global -> shared that completes on `bar`; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// 3-D tiled store of a shared-memory box; completion is tracked by the thread's bulk async-group.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* src, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];\n"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// All earlier bulk groups of this thread have finished READING shared memory (the source may be overwritten).
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
// At most one of this thread's bulk groups is still reading shared memory (for a double-buffered source).
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory"); }
// All earlier bulk groups of this thread are complete.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }
// Barrier among `count` threads (a multiple of 32) on hardware barrier `id` (1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_barrier(int id, int count) {
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(count) : "memory");
}

// ---- tensor memory -------------------------------------------------------------------------------
// Whole-warp calls.  `cols` is a power of two >= 32; the base address lands in *slot (shared memory).
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// ---- descriptors ---------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).  Addresses and offsets in 16-byte units.
//   K-major operand (contraction index contiguous, rows of 128 bytes): sbo = bytes between 8-row groups (1024),
//     lbo unused (1).
//   MN-major operand (row/column index contiguous, 64 of them per 128-byte line, one line per contraction index):
//     sbo = bytes between groups of 8 contraction indices (1024), lbo = bytes between blocks of 64 along M/N.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;      // descriptor version for sm_100
    d |= (uint64_t)2 << 61;      // SWIZZLE_128B
    return d;
}

// The same for the 32-byte swizzle: K-major rows of 32 bytes (16 elements), sbo = bytes between 8-row groups (256).
__device__ __forceinline__ uint64_t smem_desc_sw32(uint32_t saddr, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)6 << 61;      // SWIZZLE_32B
    return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16: fp32 accumulate, A/B both bf16 (1) or both fp16 (0).
__host__ __device__ constexpr uint32_t instr_desc_f16(int ab_format, int a_mn_major, int b_mn_major, int M, int N) {
    return (1u << 4) | ((uint32_t)ab_format << 7) | ((uint32_t)ab_format << 10) | ((uint32_t)a_mn_major << 15) |
           ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.  No "memory" clobber: the instruction is ordered against the
// barriers and fences around it because all of them are volatile asm statements, and a clobber would stop the
// compiler from overlapping the issuing thread's own loads with the MMAs it issues.
__device__ __forceinline__ void mma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate));
}
// The same with the A operand in tensor memory: row r of A in lane r, the 16 contraction elements of one MMA packed two
// per 32-bit column in 8 consecutive columns starting at tmem_a (element 2j in the low half of column j).
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate));
}
// Arrive on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: lane i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// The same for 8 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
// The same for 16 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
// Store of 32 lanes x 32 consecutive fp32 columns: lane i of the warp writes row (lane base + i).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

}  // namespace tc05

// ---- host side: tensor maps ------------------------------------------------------------------------
// 3-D map over [planes][rows][cols] of 16-bit elements (cols contiguous, row pitch `row_pitch_elems`, plane pitch
// `plane_pitch_elems`), box = box_cols x box_rows x 1 plane, with the 128-byte swizzle (box_cols must be 64) or
// without a swizzle; out-of-bounds reads give zero.
// As make_tensor_map_3d with the swizzle given in bytes: 0 (none), 32 (box of 16 columns), 64 (32 columns) or 128 (64 columns),
// and a box that spans box_planes consecutive planes (it lands in shared memory as [plane][row][column]).
int make_tensor_map_3d_mode(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols,
                            uint64_t row_pitch_elems, uint64_t plane_pitch_elems, uint32_t box_cols, uint32_t box_rows,
                            int swizzle_bytes, uint32_t box_planes = 1);

// Device address of the word that bounded waits raise on timeout (one per device, owned by the library; the first call
// on a device also sets up the flag's mirror in page-locked host memory).
int wait_flag_ptr(int** out);

int make_tensor_map_3d(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols,
                       uint64_t row_pitch_elems, uint64_t plane_pitch_elems, uint32_t box_cols, uint32_t box_rows,
                       bool swizzle128);

}  // namespace mta
