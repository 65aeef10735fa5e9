// Chooses the implementation of the two contractions of the forward.
#include "kernels.cuh"

namespace mta {

int qk_scores_launch(const void* q, const void* k, void* s, PlaneView sv, int B, int H, int S, int D, float scale,
                     int round_scale, int causal, int row_begin, int row_end, int dtype, cudaStream_t st) {
    if (B == 0 || row_end <= row_begin) return MTA_OK;
    return qk_scores_simt_launch(q, k, s, sv, B, H, S, D, scale, round_scale, causal, row_begin, row_end, dtype, st);
}

int pv_launch(const void* p, PlaneView pview, const void* v, void* o, int B, int H, int S, int D, int causal,
              int row_begin, int row_end, int dtype, cudaStream_t st) {
    if (B == 0 || row_end <= row_begin) return MTA_OK;
    return pv_simt_launch(p, pview, v, o, B, H, S, D, causal, row_begin, row_end, dtype, st);
}

}  // namespace mta
