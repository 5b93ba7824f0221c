// C entry points of the block-scaled GEMM: argument checks and schedule selection.
#include "common.cuh"

namespace bfp8 {
int launch_gemm_large(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                      const uint8_t* w_codes, int64_t ldw, const float* w_scales, const float* bias, void* out,
                      int out_dtype, int64_t ldo, int64_t m, int64_t n, int64_t k, uint32_t* status_dev,
                      long long wait_limit, int max_ctas, cudaStream_t st);
}

using namespace bfp8;

namespace {
// About one second at B200 clocks: far beyond any legitimate wait, short enough that a broken
// launch returns with BFP8_STATUS_WAIT_TIMEOUT instead of hanging the device.
constexpr long long kDefaultWaitLimit = 2000000000LL;
}

extern "C" size_t bfp8_gemm_block128_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  (void)m; (void)n; (void)k;
  return 0;
}

extern "C" int bfp8_gemm_block128_ex(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                                     const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                                     const float* bias, void* out, int out_dtype, int64_t ldo,
                                     int64_t m, int64_t n, int64_t k,
                                     void* workspace, size_t workspace_bytes, uint32_t* status_dev, void* stream,
                                     int schedule, int max_ctas, int64_t wait_limit_cycles) {
  (void)schedule;
  if (!a_codes || !a_scales || !w_codes || !w_scales || !out || !status_dev) return BFP8_ERR_NULL;
  if (m <= 0 || n <= 0 || k <= 0 || m > (1 << 30) || n > (1 << 30) || k > (1 << 30)) return BFP8_ERR_SHAPE;
  if (lda < k || ldw < k || ldo < n || ldsa < m) return BFP8_ERR_SHAPE;
  if (out_dtype != BFP8_OUT_F32 && out_dtype != BFP8_OUT_BF16) return BFP8_ERR_SHAPE;
  if (!aligned(a_codes, 16) || !aligned(w_codes, 16) || lda % 16 != 0 || ldw % 16 != 0) return BFP8_ERR_ALIGN;
  if (!aligned(a_scales, 4) || !aligned(w_scales, 4) || !aligned(status_dev, 4)) return BFP8_ERR_ALIGN;
  if (bias && !aligned(bias, 4)) return BFP8_ERR_ALIGN;
  if (out_dtype == BFP8_OUT_BF16 && (!aligned(out, 16) || ldo % 8 != 0)) return BFP8_ERR_ALIGN;
  if (out_dtype == BFP8_OUT_F32 && !aligned(out, 4)) return BFP8_ERR_ALIGN;
  const size_t need = bfp8_gemm_block128_workspace_bytes(m, n, k);
  if (need > 0 && (!workspace || workspace_bytes < need)) return BFP8_ERR_WORKSPACE;
  const long long limit = wait_limit_cycles > 0 ? wait_limit_cycles : kDefaultWaitLimit;
  return launch_gemm_large(a_codes, lda, a_scales, ldsa, w_codes, ldw, w_scales, bias, out, out_dtype, ldo, m, n, k,
                           status_dev, limit, max_ctas, static_cast<cudaStream_t>(stream));
}

extern "C" int bfp8_gemm_block128(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                                  const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                                  const float* bias, void* out, int out_dtype, int64_t ldo,
                                  int64_t m, int64_t n, int64_t k,
                                  void* workspace, size_t workspace_bytes, uint32_t* status_dev, void* stream) {
  return bfp8_gemm_block128_ex(a_codes, lda, a_scales, ldsa, w_codes, ldw, w_scales, bias, out, out_dtype, ldo,
                               m, n, k, workspace, workspace_bytes, status_dev, stream, 0, 0, 0);
}
