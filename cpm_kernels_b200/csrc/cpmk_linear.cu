// One call per column-parallel int8 linear: quantise the activations and this rank's weight rows (one launch), then
// the tensor-core GEMM whose epilogue dequantises and stores the rank's output columns into every rank's full-width
// result (one launch).  What cpm_kernels/torch/gemm.py:86-113 runs as six launches and six allocations per call
// becomes two launches and none: every buffer is the caller's and is reused call after call.
#include "cpmk_common.cuh"

using namespace cpmk;

extern "C" int32_t cpmk_linear_int8_scatter(int32_t tokens, int32_t k, int32_t n_local, const void *x, const void *w, void *scale_x, void *q_x,
                                            void *scale_w, void *q_w, int32_t n_dst, void *const *dst, int64_t dst_row_pitch,
                                            int32_t multicast, cpmk_stream_t stream) {
    CPMK_REQUIRE(tokens > 0 && k > 0 && n_local > 0, "bad size: tokens=%d k=%d n_local=%d", tokens, k, n_local);
    CPMK_REQUIRE(x && w && scale_x && q_x && scale_w && q_w, "null tensor pointer");
    // activations (tokens, k) and weight rows (n_local, k): both are quantised along k, per row
    int32_t rc = cpmk_quantize_rows_pair(1, tokens, x, scale_x, q_x, 1, n_local, w, scale_w, q_w, k, stream);
    if (rc) return rc;
    // kernel-level (m, k, n) = (n_local, k, tokens): A = weight codes (m, k) with aT, B = activation codes (n, k);
    // the output rows are tokens, scale_x multiplies first (cuda/gemm.cu:45-56)
    if (multicast) {
        CPMK_REQUIRE(n_dst == 2 && dst && dst[0] && dst[1], "the multicast form takes two destinations: the local buffer and the multicast address");
        return cpmk_gemm_int8_dequant_multicast(n_local, k, tokens, 1, 1, 1, 0, q_w, q_x, scale_x, scale_w, 1, 1, dst[0], dst[1], dst_row_pitch, stream);
    }
    return cpmk_gemm_int8_dequant_scatter(n_local, k, tokens, 1, 1, 1, 0, q_w, q_x, scale_x, scale_w, 1, 1, n_dst, dst, dst_row_pitch, stream);
}
