// The conv attention forward softmax(scale * conv(Q K^T)) V as ONE kernel (TritonAttention.forward / _attn_fwd /
// _attn_fwd_inner, conv_attention_triton.py:21-147, 352-356, 362-452): no S x S tensor exists anywhere, not even as
// scratch.  Per work unit = (plane, block of TMO = 129 - R query rows) the CTA walks the key tiles 0 .. diagonal:
//   scores     S[128 x 144] = Q[rows m0-(R-1) ..] . K[keys n0-8 ..]^T on tcgen05 into tensor memory (TMEM)
//   drain      TMEM -> round(round(S) * score_scale), 0 above the diagonal -> the swizzled staged tile in shared memory
//   conv       the Toeplitz MMAs of conv2d_tc05.cu over the staged tile -> TMEM accumulator (128 x 128 fp32)
//   softmax    TMEM -> y = conv * scale * log2 e in fp32, -inf above the diagonal -> running (reference max, sum) per
//              query row, P = 2^(y - m) in the 16-bit dtype -> back into TMEM (never through shared memory).  The output
//              accumulator is rescaled (in TMEM) only when the row maximum grew by more than 2^8 since the reference
//              maximum was taken, so almost never after the first key tiles
//   P.V        O[128 x D] += P[128 x 128] V[128 x D] on tcgen05 with P as the TMEM operand, O stays in TMEM for the whole unit
//   epilogue   O / row sum -> 16-bit -> global memory, once per unit (conv_attention_triton.py:352-356)
// Rounding: the scores are rounded to the 16-bit dtype as the reference's matmul does (conv_attention_pytorch.py:48)
// and so are the exponentials that enter P.V; the conv output and the scaled logits, which the reference rounds
// too (:57-64), stay in fp32 here.
//
// Warps: 0 Q / K loads (Q per unit, K per tile) and score MMAs, 1 V loads and P.V MMAs, 2-3 conv MMAs (disjoint output
// columns, so the result is bit-reproducible), 4-7 drain, 8-15 softmax + epilogue (a pair of warps per 32 rows, 64
// columns each).  Every stage of the per-tile pipeline is its own role and the staged tile has a ring of three
// buffers, so the scores and the drain run up to two tiles ahead of the conv MMAs (the tensor pipe, which all three
// kinds of MMA share, is the unit that limits the kernel), and the softmax and P.V follow one tile behind.
// TMEM (512 columns): conv accumulator 0..127, score accumulator 128..271, P (16-bit, two keys per column) 272..335,
// O 384..384+D-1.  The kernel is bound by shared-memory bandwidth (the conv MMAs re-read the staged tile once per row
// tap), which is why P and nothing else that can avoid it goes through shared memory.
// Work units are dealt heaviest first in rounds of alternating direction, which balances the CTAs' tile counts to a
// fraction of a percent (a plain round-robin over (plane, row block) left 10 % between them at B8 H16 S4096).
// 16-bit dtypes, D in {64, 128}, odd key extent <= 17, causal; any S (TMA zero-fills rows past the end).
#include "toeplitz_tc05.cuh"

namespace mta {
namespace {
using namespace tc05;
using namespace qc;

constexpr int CA_THREADS = 16 * 32;
constexpr int NSTAGE = 3;                   // staged score tiles in flight
constexpr uint32_t C_COL = 0, S_COL = 128, P_COL = 272, O_COL = 384;
constexpr int VBOX_BYTES = TN * 128;         // one box of the V tile: 128 keys x 64 elements
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;         // the reference logit moves when the row maximum (base 2) exceeds it by 8

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct CaGeom {
    int C, S, R, KS, row_begin, row_end, tiles_m, tmo, split_w, planes;
    float score_scale, sm_scale;
    long units;
};

// Key tiles that the query rows of row block tm reach.
__device__ __forceinline__ int ca_key_tiles(const CaGeom& g, int tm) {
    const int q_last = min(g.row_begin + (tm + 1) * g.tmo, g.row_end);
    return (q_last + TN - 1) / TN;
}

template <typename T, int D>
__global__ void __launch_bounds__(CA_THREADS, 1)
conv_attn_tc05_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                      const __grid_constant__ CUtensorMap mv, T* __restrict__ o, const void* __restrict__ w, int w_dtype,
                      CaGeom g, int* err_flag) {
    constexpr int DBOX = D / 64;
    constexpr int Q_BYTES = DBOX * BOX_BYTES;      // 128 rows x D
    constexpr int K_BYTES = DBOX * KBOX_BYTES;     // 144 keys x D
    constexpr int V_BYTES = DBOX * VBOX_BYTES;     // 128 keys x D
    constexpr int OH = D / 2;                      // output columns per softmax warp
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t q_full, q_free, k_full, k_free, s_full, s_free, ready_bar[NSTAGE], empty_bar[NSTAGE], acc_full,
        acc_empty, v_full, p_ready, pv_done;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ float xch_max[2][2][TM];           // [tile parity][column half][row]: a warp pair's halves of a row maximum
    __shared__ float xch_sum[2][TM];              // [column half][row]: the halves of a row sum, once per unit
    __shared__ float wsm[MAX_TAPS];               // a head's conv weights on their way into the Toeplitz slices
    const int R = g.R, KS = g.KS;
    const int tb_bytes = toeplitz_bytes(R, g.split_w);
    uint8_t* q_base = smem;
    uint8_t* k_base = q_base + Q_BYTES;
    uint8_t* v_base = k_base + K_BYTES;
    uint8_t* stage_base = v_base + V_BYTES;        // NSTAGE staged tiles of TB_OFF bytes
    uint8_t* tb_base = stage_base + NSTAGE * TB_OFF;     // two sets of Toeplitz slices: units alternate between them
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int a_off = 8 - (KS - 1) / 2;
    const int lead = R - 1;

    if (tid == 0) abort_flag = *reinterpret_cast<volatile int*>(err_flag);
    __syncthreads();
    if (abort_flag != 0) return;

    if (warp == 0) {
        if (lane == 0) {
            mbar_init(&q_full, 1);
            mbar_init(&q_free, 1);
            mbar_init(&k_full, 1);
            mbar_init(&k_free, 1);
            mbar_init(&s_full, 1);
            mbar_init(&s_free, 4);
            for (int i = 0; i < NSTAGE; ++i) {
                mbar_init(&ready_bar[i], 4);
                mbar_init(&empty_bar[i], 2);
            }
            mbar_init(&acc_full, 2);
            mbar_init(&acc_empty, 8);
            mbar_init(&v_full, 1);
            mbar_init(&p_ready, 8);
            mbar_init(&pv_done, 1);
            fence_mbar_init();
            prefetch_tensormap(&mq);
            prefetch_tensormap(&mk);
            prefetch_tensormap(&mv);
        }
        __syncwarp();
        tmem_alloc(&tmem_slot, 512);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;

    // Every role walks the same sequence of units.  All units, heaviest row blocks first (row block tm of every plane
    // before row block tm - 1 of any), are dealt to the CTAs in rounds that alternate direction (0 .. G-1, G-1 .. 0, ...):
    // a round's units cost the same to within one key tile and the alternation cancels the slope, so the CTAs' tile
    // counts agree to a fraction of a percent; n counts the tiles this CTA has started.
#define CA_FOR_UNITS                                                                  \
    for (long rnd = 0;; ++rnd) {                                                      \
        const long u = rnd * gridDim.x + ((rnd & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x); \
        if (u >= g.units) break;                                                      \
        const int plane = (int)(u % g.planes), tm = g.tiles_m - 1 - (int)(u / g.planes); \
        const int m0 = g.row_begin + tm * g.tmo;                                      \
        const int nk = ca_key_tiles(g, tm);                                           \
        (void)plane; (void)m0;

    if (warp == 0) {
        // ---------------- Q / K loads and score MMAs: S[128 x 144] = Q K^T into TMEM columns S_COL.. ----------------
        // One thread does both: the Q and K tiles are single-buffered, so a load can only be issued once the MMAs that
        // read the buffer have completed, which is this thread's own commit.  The ring of staged tiles downstream
        // keeps the conv MMAs fed while a load is in flight.
        constexpr uint32_t idesc = instr_desc_f16(AbFmtQ<T>::value, 0, 0, TM, SN);
        int n = 0, un = 0;
        CA_FOR_UNITS
            mbar_wait(&q_free, (un & 1) ^ 1, err_flag);        // the previous unit's score MMAs have read its Q tile
            if (lane == 0) {
                mbar_expect_tx(&q_full, (uint32_t)Q_BYTES);
#pragma unroll
                for (int j = 0; j < DBOX; ++j) tma_load_3d(q_base + j * BOX_BYTES, &mq, &q_full, 64 * j, m0 - lead, plane);
            }
            for (int tn = 0; tn < nk; ++tn, ++n) {
                mbar_wait(&k_free, (n & 1) ^ 1, err_flag);
                if (lane == 0) {
                    mbar_expect_tx(&k_full, (uint32_t)K_BYTES);
#pragma unroll
                    for (int j = 0; j < DBOX; ++j) tma_load_3d(k_base + j * KBOX_BYTES, &mk, &k_full, 64 * j, tn * TN - 8, plane);
                }
                if (tn == 0) mbar_wait(&q_full, un & 1, err_flag);
                mbar_wait(&k_full, n & 1, err_flag);
                mbar_wait(&s_free, (n & 1) ^ 1, err_flag);       // the drain warps have read the previous score tile
                __syncwarp();
                fence_after_sync();
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
                    if (tn == nk - 1) mma_commit(&q_free);
                }
                __syncwarp();
            }
            ++un;
        }
    } else if (warp == 2 || warp == 3) {
        // ---------------- conv MMAs ----------------
        int n = 0, un = 0;
        CA_FOR_UNITS
            const uint32_t tb_addr = smem_u32(tb_base + (un & 1) * tb_bytes);
            for (int tn = 0; tn < nk; ++tn, ++n) {
                const int st = n % NSTAGE;
                mbar_wait_spin(&ready_bar[st], (n / NSTAGE) & 1, err_flag);
                mbar_wait_spin(&acc_empty, (n & 1) ^ 1, err_flag);    // the softmax warps have read the previous conv tile
                fence_after_sync();
                if (lane == 0) {
                    const uint32_t xa_addr = smem_u32(stage_base + st * TB_OFF);
                    if (warp == 2) issue_conv<T, 0>(xa_addr, tb_addr, tmem + C_COL, R, g.split_w);
                    else issue_conv<T, 1>(xa_addr, tb_addr, tmem + C_COL, R, g.split_w);
                    mma_commit(&empty_bar[st]);
                    mma_commit(&acc_full);
                }
                __syncwarp();
            }
            ++un;
        }
    } else if (warp >= 4 && warp < 8) {
        // ---------------- drain: score tile TMEM -> rounded, scaled, masked -> staged tile; Toeplitz slices ----------------
        const int quarter = warp & 3;
        const int sr = quarter * 32 + lane;                  // staged row = TMEM lane of this thread
        const int ft = tid - 128;                            // 0..127
        const float sc = round_to<T>(g.score_scale);
        const bool scaled = g.score_scale != 1.0f;           // raw scores (the conv attention) are rounded once
        int n = 0, un = 0;
        // The weights of a unit's head are fetched one unit ahead (successive units of a CTA belong to different planes,
        // so every unit rebuilds its slices): the global loads are in flight while the previous unit's tiles are drained.
        float taps[TAPS_PER_THREAD];
        if ((long)blockIdx.x < g.units) fetch_taps(taps, w, w_dtype, (int)(blockIdx.x % g.planes) % g.C, R, KS, ft);
        CA_FOR_UNITS
            {
                // this set of slices was last read by the conv MMAs of unit un - 2, whose tiles all precede tile n - 1
                if (n >= 2) mbar_wait(&empty_bar[(n - 2) % NSTAGE], ((n - 2) / NSTAGE) & 1, err_flag);
                build_from_taps<T>(tb_base + (un & 1) * tb_bytes, wsm, taps, R, KS, a_off, g.split_w, ft, 5);
                const long u_next = (rnd + 1) * gridDim.x + (((rnd + 1) & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x);
                if (u_next < g.units) fetch_taps(taps, w, w_dtype, (int)(u_next % g.planes) % g.C, R, KS, ft);
            }
            for (int tn = 0; tn < nk; ++tn, ++n) {
                const int st = n % NSTAGE;
                uint8_t* xa = stage_base + st * TB_OFF;
                mbar_wait(&empty_bar[st], ((n / NSTAGE) & 1) ^ 1, err_flag);   // conv MMAs of tile n - NSTAGE are done
                mbar_wait(&s_full, n & 1, err_flag);
                __syncwarp();
                fence_after_sync();
                const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16) + S_COL;
                const bool diag = tn * TN + SN - 9 > m0 - lead;              // some staged key lies above some staged query
                if (scaled) drain_row<T, true>(trow, smem_u32(xa), sr, m0 - lead + sr, tn * TN - 8, sc, diag);
                else drain_row<T, false>(trow, smem_u32(xa), sr, m0 - lead + sr, tn * TN - 8, sc, diag);
                fence_before_sync();
                fence_proxy_async();          // generic-proxy writes above must be visible to the MMAs (async proxy)
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&s_free);
                    mbar_arrive(&ready_bar[st]);
                }
            }
            ++un;
        }
    } else if (warp >= 8) {
        // ---------------- softmax + epilogue: warps 8-11 take columns 0..63, warps 12-15 columns 64..127 ----------------
        // The conv output stays in fp32 from the accumulator to the exponential (the reference rounds it to the 16-bit
        // dtype twice on the way, conv_attention_pytorch.py:57-64); logits are handled in the base-2 domain:
        // y = conv * (scale * log2 e), P = 2^(y - m).
        const int quarter = warp & 3;
        const int half = warp >= 12 ? 1 : 0;
        const int row = quarter * 32 + lane;                 // row of the tile = TMEM lane of this thread
        const uint32_t tlane = tmem + ((uint32_t)(quarter * 32) << 16);
        const float c2 = g.sm_scale * LOG2E;
        const bool neg = c2 < 0.0f;                          // a negative scale turns the row maximum into a minimum
        const float masked = neg ? INFINITY : -INFINITY;     // raw value whose logit is -inf
        int n = 0;
        CA_FOR_UNITS
            const int q = m0 + row;
            float m_ref = -INFINITY;       // base-2 logit the exponentials of this row are taken against
            float l_part = 0.0f;           // sum of this thread's exponentials (its 64 columns of every tile)
            for (int tn = 0; tn < nk; ++tn, ++n) {
                const int k0 = tn * TN + half * 64;          // key of this thread's first column
                uint32_t xr[64];
                mbar_wait_spin(&acc_full, n & 1, err_flag);
                __syncwarp();
                fence_after_sync();
                tmem_ld_32x32(tlane + C_COL + (uint32_t)(half * 64), *reinterpret_cast<uint32_t(*)[32]>(&xr[0]));
                tmem_ld_32x32(tlane + C_COL + (uint32_t)(half * 64 + 32), *reinterpret_cast<uint32_t(*)[32]>(&xr[32]));
                tmem_ld_wait();
                fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty);      // the next tile's conv MMAs may overwrite the accumulator
                float* x = reinterpret_cast<float*>(xr);
                if (k0 + 63 > q) {
#pragma unroll
                    for (int e = 0; e < 64; ++e)
                        if (k0 + e > q) x[e] = masked;
                }
                float mx = x[0];
                if (!neg) {
#pragma unroll
                    for (int e = 1; e < 64; ++e) mx = fmaxf(mx, x[e]);
                } else {
#pragma unroll
                    for (int e = 1; e < 64; ++e) mx = fminf(mx, x[e]);
                }
                mx *= c2;                                    // this half's largest logit (-inf when all are masked)
                xch_max[n & 1][half][row] = mx;
                named_barrier(1 + quarter, 64);              // the two warps that share these 32 rows
                const float mt = fmaxf(mx, xch_max[n & 1][half ^ 1][row]);
                float alpha = 1.0f;
                bool moved = false;
                if (mt - m_ref > RESCALE_STEP) {             // also the first tile (m_ref = -inf)
                    alpha = m_ref == -INFINITY ? 0.0f : ex2_approx(m_ref - mt);
                    m_ref = mt;
                    l_part *= alpha;
                    moved = true;
                }
                // P.V of the previous tile has finished: the P tile may be overwritten and O is stable
                if (n > 0) mbar_wait(&pv_done, (n - 1) & 1, err_flag);
                __syncwarp();
                fence_after_sync();
                if (tn > 0 && __any_sync(0xffffffffu, moved)) {
#pragma unroll 1
                    for (int c = 0; c < OH / 32; ++c) {
                        uint32_t r[32];
                        const uint32_t addr = tlane + O_COL + (uint32_t)(half * OH + c * 32);
                        tmem_ld_32x32(addr, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
                        tmem_st_32x32(addr, r);
                    }
                    tmem_st_wait();
                }
                const float mb = m_ref == -INFINITY ? 0.0f : -m_ref;
                uint32_t pk[32];                             // this thread's 64 exponentials, two per column
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const float p0 = ex2_approx(fmaf(x[2 * e], c2, mb)), p1 = ex2_approx(fmaf(x[2 * e + 1], c2, mb));
                    l_part += p0 + p1;
                    pk[e] = pack2q<T>(p0, p1);
                }
                tmem_st_32x32(tlane + P_COL + (uint32_t)(half * 32), pk);
                tmem_st_wait();
                fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_ready);
            }
            // ---- the unit's rows are complete once its last P.V has finished ----
            mbar_wait(&pv_done, (n - 1) & 1, err_flag);
            __syncwarp();
            fence_after_sync();
            xch_sum[half][row] = l_part;
            named_barrier(1 + quarter, 64);
            const float inv = 1.0f / (l_part + xch_sum[half ^ 1][row]);
            const bool store = row < g.tmo && q < g.row_end;
            T* orow = o + ((long)plane * g.S + (store ? q : 0)) * D + half * OH;
#pragma unroll 1
            for (int c = 0; c < OH / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tlane + O_COL + (uint32_t)(half * OH + c * 32), r);
                tmem_ld_wait();
                if (store) {
#pragma unroll
                    for (int v8 = 0; v8 < 4; ++v8) {
                        uint4 v;
                        v.x = pack2q<T>(__uint_as_float(r[v8 * 8 + 0]) * inv, __uint_as_float(r[v8 * 8 + 1]) * inv);
                        v.y = pack2q<T>(__uint_as_float(r[v8 * 8 + 2]) * inv, __uint_as_float(r[v8 * 8 + 3]) * inv);
                        v.z = pack2q<T>(__uint_as_float(r[v8 * 8 + 4]) * inv, __uint_as_float(r[v8 * 8 + 5]) * inv);
                        v.w = pack2q<T>(__uint_as_float(r[v8 * 8 + 6]) * inv, __uint_as_float(r[v8 * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + v8 * 8) = v;
                    }
                }
            }
            fence_before_sync();          // these loads precede the next unit's first P.V, which follows this warp's next arrival
        }
    } else {
        // ---------------- (warp 1) V loads and P.V MMAs: O[128 x D] (+)= P[128 x 128] V[128 x D] ----------------
        constexpr uint32_t idesc = instr_desc_f16(AbFmtQ<T>::value, 0, 1, TM, D);
        int n = 0;
        CA_FOR_UNITS
            for (int tn = 0; tn < nk; ++tn, ++n) {
                if (n > 0) mbar_wait(&pv_done, (n - 1) & 1, err_flag);     // the previous P.V has read the V tile
                if (lane == 0) {
                    mbar_expect_tx(&v_full, (uint32_t)V_BYTES);
#pragma unroll
                    for (int j = 0; j < DBOX; ++j) tma_load_3d(v_base + j * VBOX_BYTES, &mv, &v_full, 64 * j, tn * TN, plane);
                }
                mbar_wait(&p_ready, n & 1, err_flag);
                mbar_wait(&v_full, n & 1, err_flag);
                __syncwarp();
                fence_after_sync();
                if (lane == 0) {
                    const uint32_t va = smem_u32(v_base);
#pragma unroll
                    for (int kk = 0; kk < TN / 16; ++kk) {
                        const uint64_t db = smem_desc_sw128(va + kk * 16 * 128, VBOX_BYTES, 1024);
                        mma_f16_ts(tmem + O_COL, tmem + P_COL + (uint32_t)(kk * 8), db, idesc, (tn > 0 || kk > 0) ? 1u : 0u);
                    }
                    mma_commit(&pv_done);
                }
                __syncwarp();
            }
        }
    }
#undef CA_FOR_UNITS
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

size_t conv_attn_smem_bytes(int D, int R, bool split_w) {
    return 1024 + (size_t)(D / 64) * (BOX_BYTES + KBOX_BYTES + VBOX_BYTES) + (size_t)NSTAGE * TB_OFF + 2 * (size_t)toeplitz_bytes(R, split_w ? 1 : 0);
}

template <typename T, int D>
int launch_ca(const void* q, const void* k, const void* v, const void* w, int w_dtype, void* o, int B, int H, int S, int R, int KS,
              float score_scale, float sm_scale, int row_begin, int row_end, cudaStream_t st) {
    const long planes = (long)B * H;
    CaGeom g{};
    g.C = H; g.S = S; g.R = R; g.KS = KS; g.row_begin = row_begin; g.row_end = row_end;
    g.score_scale = score_scale; g.sm_scale = sm_scale;
    g.tmo = TM - (R - 1);
    g.tiles_m = (row_end - row_begin + g.tmo - 1) / g.tmo;
    g.split_w = w_dtype == MTA_F32 ? 1 : 0;
    g.planes = (int)planes;
    g.units = planes * g.tiles_m;
    CUtensorMap mq, mk, mv;
    int rc;
    if ((rc = make_tensor_map_3d(&mq, q, (uint64_t)planes, S, D, D, (uint64_t)S * D, 64, TM, true))) return rc;
    if ((rc = make_tensor_map_3d(&mk, k, (uint64_t)planes, S, D, D, (uint64_t)S * D, 64, SN, true))) return rc;
    if ((rc = make_tensor_map_3d(&mv, v, (uint64_t)planes, S, D, D, (uint64_t)S * D, 64, TN, true))) return rc;
    int* flag = nullptr;
    if ((rc = wait_flag_ptr(&flag))) return rc;
    int dev = 0, sms = 0;
    MTA_CUDA_OK(cudaGetDevice(&dev));
    MTA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const size_t smem = conv_attn_smem_bytes(D, R, g.split_w != 0);
    MTA_CUDA_OK(cudaFuncSetAttribute(conv_attn_tc05_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const unsigned grid = (unsigned)std::min<long>(g.units, sms);
    conv_attn_tc05_kernel<T, D><<<grid, CA_THREADS, smem, st>>>(mq, mk, mv, static_cast<T*>(o), w, w_dtype, g, flag);
    MTA_LAUNCH_OK("conv_attn_tc05_kernel");
    return MTA_OK;
}

constexpr size_t CA_STATIC_SMEM = 4608;     // barriers, the exchange arrays and the weight buffer, rounded up
constexpr size_t CA_SMEM_LIMIT = 227 * 1024;

}  // namespace

bool conv_attn_fused_shape_ok(int S, int D, int R, int KS, int causal, int dtype, int w_dtype) {
    return causal && dtype != MTA_F32 && (D == 64 || D == 128) && S >= 1 && KS % 2 == 1 && KS <= 17 && R >= 1 && R <= 16 &&
           conv_attn_smem_bytes(D, R, w_dtype == MTA_F32) + CA_STATIC_SMEM <= CA_SMEM_LIMIT;
}

bool conv_attn_fused_supported(const void* q, const void* k, const void* v, const void* o, int S, int D, int R, int KS, int causal,
                               int dtype, int w_dtype) {
    return conv_attn_fused_shape_ok(S, D, R, KS, causal, dtype, w_dtype) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o);
}

int conv_attn_fused_launch(const void* q, const void* k, const void* v, const void* w, int w_dtype, void* o, int B, int H, int S, int D,
                           int R, int KS, float score_scale, float sm_scale, int row_begin, int row_end, int dtype, cudaStream_t st) {
    if ((long)B * H == 0 || row_end <= row_begin) return MTA_OK;
#define MTA_CA(TT, DD) return launch_ca<TT, DD>(q, k, v, w, w_dtype, o, B, H, S, R, KS, score_scale, sm_scale, row_begin, row_end, st)
    if (dtype == MTA_BF16) { if (D == 64) MTA_CA(__nv_bfloat16, 64); MTA_CA(__nv_bfloat16, 128); }
    if (D == 64) MTA_CA(__half, 64);
    MTA_CA(__half, 128);
#undef MTA_CA
}

}  // namespace mta
