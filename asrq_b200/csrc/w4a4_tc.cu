// W4A4 GEMM on tcgen05 kind::i8 (int32 accumulators in TMEM).
#include "tcgen05.cuh"

namespace asrq {

bool w4a4_gemm_tc_supports(int64_t, int64_t, int64_t, int) { return false; }

int w4a4_gemm_tc(const uint8_t*, const float*, const uint8_t*, const void*, const void*, void*, int32_t*, int64_t,
                 int64_t, int64_t, int, int, void*, size_t, int, cudaStream_t) {
  return fail(ASRQ_ERR_SHAPE, "w4a4 tcgen05 gemm: shape not supported");
}

}  // namespace asrq
