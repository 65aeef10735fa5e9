// Dropout on the attention weights inside the P.V kernels (F.dropout(scores, p, training) before the product with V,
// mta_attention_triton.py:87): no mask tensor exists.  The keep decision of weight (plane, query, key) is a pure
// function of (seed, plane, query, key): one Philox4x32-10 block (Salmon et al., "Parallel random numbers: as easy
// as 1, 2, 3", SC11) per 8 consecutive keys, counter = (key / 8, query, plane, 0), key = the 64-bit seed; key 8c + e
// takes the e-th 16-bit field of the 128 output bits and is kept when the field is below round((1 - p) * 65536).
// Kept weights are multiplied by 1 / (1 - p) and rounded to the dtype, as the reference's elementwise op does.
// The result therefore does not depend on tiling, on the kernel that runs or on the row range computed, and
// oracle/mta_oracle.py restates the same function in numpy.
#pragma once

#include <stdint.h>

namespace mta {

struct DropoutSpec {
    float p = 0.0f;                  // probability of dropping a weight; 0 switches the whole thing off
    unsigned long long seed = 0;
    __host__ __device__ bool on() const { return p > 0.0f; }
    __host__ __device__ float scale() const { return 1.0f / (1.0f - p); }
    __host__ __device__ uint32_t keep_threshold() const {
        const float t = (1.0f - p) * 65536.0f + 0.5f;
        return t <= 0.0f ? 0u : (t >= 65536.0f ? 65536u : (uint32_t)t);
    }
};

// Bit e of the result: key 8 * chunk + e of (plane, query) is kept.
__device__ __forceinline__ uint32_t dropout_keep8(unsigned long long seed, uint32_t plane, uint32_t query, uint32_t chunk,
                                                  uint32_t keep_threshold) {
    uint32_t c0 = chunk, c1 = query, c2 = plane, c3 = 0u;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        c0 = hi1 ^ c1 ^ k0;
        c1 = lo1;
        c2 = hi0 ^ c3 ^ k1;
        c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    const uint32_t out[4] = {c0, c1, c2, c3};
    uint32_t keep = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const uint32_t field = (out[e >> 1] >> ((e & 1) * 16)) & 0xffffu;
        keep |= (field < keep_threshold ? 1u : 0u) << e;
    }
    return keep;
}

}  // namespace mta
