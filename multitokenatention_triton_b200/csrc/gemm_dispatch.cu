// Chooses the implementation of the two contractions of the forward: tcgen05 tensor cores for 16-bit
// dtypes with D in {64,128} and 16-byte aligned rows, CUDA cores otherwise.  mta_set_variant("gemm", 1)
// forces the CUDA-core kernels, ("gemm", 2) requires the tensor-core ones.
#include "kernels.cuh"

namespace mta {

int qk_scores_launch(const void* q, const void* k, void* s, PlaneView sv, int B, int H, int S, int D, float scale,
                     int round_scale, int causal, int row_begin, int row_end, int dtype, cudaStream_t st) {
    if (B == 0 || row_end <= row_begin) return MTA_OK;
    const int want = variant("gemm");
    const bool ok = tc05_contractions_supported(S, D, dtype, q, k, s, sv);
    MTA_REQUIRE(want != 2 || ok, "qk_scores: the tensor-core variant needs a 16-bit dtype, D in {64,128}, S %% 8 == 0 and 16-byte aligned tensors");
    if (ok && want != 1)
        return qk_persistent_launch(q, k, s, sv, B, H, S, D, 1, scale, round_scale, causal, 0, 1, 0, row_begin, row_end, dtype, st);
    return qk_scores_simt_launch(q, k, s, sv, B, H, S, D, scale, round_scale, causal, row_begin, row_end, dtype, st);
}

int pv_launch(const void* p, PlaneView pview, long p_rows_stored, const void* v, void* o, int B, int H, int S, int D,
              int causal, int row_begin, int row_end, int dtype, cudaStream_t st, DropoutSpec drop) {
    if (B == 0 || row_end <= row_begin) return MTA_OK;
    const int want = variant("gemm");
    const bool ok = tc05_contractions_supported(S, D, dtype, p, v, o, pview);
    MTA_REQUIRE(want != 2 || ok, "pv: the tensor-core variant needs a 16-bit dtype, D in {64,128}, S %% 8 == 0 and 16-byte aligned tensors");
    if (ok && want != 1)
        return pv_tc05_launch(p, pview, p_rows_stored, v, o, B, H, S, D, causal, row_begin, row_end, dtype, st, drop);
    return pv_simt_launch(p, pview, v, o, B, H, S, D, causal, row_begin, row_end, dtype, st, drop);
}

}  // namespace mta
