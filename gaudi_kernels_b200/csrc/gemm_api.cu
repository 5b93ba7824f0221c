// C entry points of the block-scaled GEMM: argument checks and schedule selection.
#include "common.cuh"

namespace bfp8 {
struct PushTarget {
  const void* recv[8];
  int world, rank, rows;
};
struct SmallPush {
  const void* recv[8];
  int world, rank, rows;
};
int launch_gemm_large(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                      const uint8_t* w_codes, int64_t ldw, const float* w_scales, const float* bias, void* out,
                      int out_dtype, int64_t ldo, int64_t m, int64_t n, int64_t k, uint32_t* status_dev,
                      long long wait_limit, int max_ctas, int band, int inter, const PushTarget* push,
                      cudaStream_t st);
int launch_gemm_pair(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                     const uint8_t* w_codes, int64_t ldw, const float* w_scales, const float* bias, void* out,
                     int out_dtype, int64_t ldo, int64_t m, int64_t n, int64_t k, uint32_t* status_dev,
                     long long wait_limit, int max_ctas, cudaStream_t st);
int launch_gemm_smallm(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                       const uint8_t* w_codes, int64_t ldw, const float* w_scales, const float* bias, void* out,
                       int out_dtype, int64_t ldo, int64_t m, int64_t n, int64_t k, void* workspace,
                       uint32_t* status_dev, long long wait_limit, int max_ctas, int inter, const SmallPush* push,
                       cudaStream_t st);
int launch_gemm_channel(const uint8_t* a_codes, int64_t lda, const float* a_scales, const uint8_t* w_codes,
                        int64_t ldw, const float* w_scales, const float* bias, void* out, int out_dtype, int64_t ldo,
                        int64_t m, int64_t n, int64_t k, uint32_t* status_dev, long long wait_limit, int max_ctas,
                        cudaStream_t st);
size_t smallm_workspace_bytes(int64_t m, int64_t n, int max_ctas);
int set_weights_at_rest(int on);
bool smallm_supported(int64_t n);
}

using namespace bfp8;

namespace {
// About one second at B200 clocks: far beyond any legitimate wait, short enough that a broken
// launch returns with BFP8_STATUS_WAIT_TIMEOUT instead of hanging the device.
constexpr long long kDefaultWaitLimit = 2000000000LL;
constexpr int64_t kSmallMRows = 128;     // up to this many activation rows the weight-streaming schedule runs
constexpr int kMaxCtas = 256;            // workspace is sized for this many CTAs, whatever the device has
}

extern "C" size_t bfp8_gemm_block128_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  (void)k;
  if (m <= 0 || n <= 0) return 0;
  // Sized for the small-M schedule whenever it could be selected (automatically or by `schedule`).
  return (m <= kSmallMRows && smallm_supported(n)) ? smallm_workspace_bytes(m, n, kMaxCtas) : 0;
}

extern "C" int bfp8_gemm_block128_ex(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                                     const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                                     const float* bias, void* out, int out_dtype, int64_t ldo,
                                     int64_t m, int64_t n, int64_t k,
                                     void* workspace, size_t workspace_bytes, uint32_t* status_dev, void* stream,
                                     int schedule, int max_ctas, int64_t wait_limit_cycles) {
  if (!a_codes || !a_scales || !w_codes || !w_scales || !out || !status_dev) return BFP8_ERR_NULL;
  if (m <= 0 || n <= 0 || k <= 0 || m > (1 << 30) || n > (1 << 30) || k > (1 << 30)) return BFP8_ERR_SHAPE;
  if (lda < k || ldw < k || ldo < n || ldsa < m) return BFP8_ERR_SHAPE;
  if (out_dtype != BFP8_OUT_F32 && out_dtype != BFP8_OUT_BF16) return BFP8_ERR_SHAPE;
  if (!aligned(a_codes, 16) || !aligned(w_codes, 16) || lda % 16 != 0 || ldw % 16 != 0) return BFP8_ERR_ALIGN;
  if (!aligned(a_scales, 4) || !aligned(w_scales, 4) || !aligned(status_dev, 4)) return BFP8_ERR_ALIGN;
  if (bias && !aligned(bias, 4)) return BFP8_ERR_ALIGN;
  if (out_dtype == BFP8_OUT_BF16 && (!aligned(out, 16) || ldo % 8 != 0)) return BFP8_ERR_ALIGN;
  if (out_dtype == BFP8_OUT_F32 && !aligned(out, 4)) return BFP8_ERR_ALIGN;
  if (schedule < 0 || schedule > 3 || (schedule == 2 && (m > kSmallMRows || !smallm_supported(n)))) return BFP8_ERR_SHAPE;
  const bool small = schedule == 2 || (schedule == 0 && m <= kSmallMRows && smallm_supported(n));
  const long long limit = wait_limit_cycles > 0 ? wait_limit_cycles : kDefaultWaitLimit;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (small) {
    const size_t need = bfp8_gemm_block128_workspace_bytes(m, n, k);
    if (!workspace || workspace_bytes < need) return BFP8_ERR_WORKSPACE;
    if (!aligned(workspace, 256)) return BFP8_ERR_ALIGN;
    if (sm_count() > kMaxCtas) return BFP8_ERR_UNSUPPORTED;
    return launch_gemm_smallm(a_codes, lda, a_scales, ldsa, w_codes, ldw, w_scales, bias, out, out_dtype, ldo,
                              m, n, k, workspace, status_dev, limit, max_ctas, /*inter=*/0, /*push=*/nullptr, st);
  }
  if (schedule == 3)
    return launch_gemm_pair(a_codes, lda, a_scales, ldsa, w_codes, ldw, w_scales, bias, out, out_dtype, ldo, m, n, k,
                            status_dev, limit, max_ctas, st);
  return launch_gemm_large(a_codes, lda, a_scales, ldsa, w_codes, ldw, w_scales, bias, out, out_dtype, ldo, m, n, k,
                           status_dev, limit, max_ctas, /*band=*/0, /*inter=*/0, /*push=*/nullptr, st);
}

extern "C" int bfp8_gemm_block128(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                                  const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                                  const float* bias, void* out, int out_dtype, int64_t ldo,
                                  int64_t m, int64_t n, int64_t k,
                                  void* workspace, size_t workspace_bytes, uint32_t* status_dev, void* stream) {
  return bfp8_gemm_block128_ex(a_codes, lda, a_scales, ldsa, w_codes, ldw, w_scales, bias, out, out_dtype, ldo,
                               m, n, k, workspace, workspace_bytes, status_dev, stream, 0, 0, 0);
}

extern "C" int bfp8_set_weights_at_rest(int on) { return set_weights_at_rest(on); }

extern "C" int bfp8_gemm_token_channel(const uint8_t* a_codes, int64_t lda, const float* a_scales,
                                       const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                                       const float* bias, void* out, int out_dtype, int64_t ldo,
                                       int64_t m, int64_t n, int64_t k, uint32_t* status_dev, void* stream) {
  if (!a_codes || !a_scales || !w_codes || !w_scales || !out || !status_dev) return BFP8_ERR_NULL;
  if (m <= 0 || n <= 0 || k <= 0 || m > (1 << 30) || n > (1 << 30) || k > (1 << 30)) return BFP8_ERR_SHAPE;
  if (lda < k || ldw < k || ldo < n) return BFP8_ERR_SHAPE;
  if (out_dtype != BFP8_OUT_F32 && out_dtype != BFP8_OUT_BF16) return BFP8_ERR_SHAPE;
  if (!aligned(a_codes, 16) || !aligned(w_codes, 16) || lda % 16 != 0 || ldw % 16 != 0) return BFP8_ERR_ALIGN;
  if (!aligned(a_scales, 4) || !aligned(w_scales, 4) || !aligned(status_dev, 4)) return BFP8_ERR_ALIGN;
  if (bias && !aligned(bias, 4)) return BFP8_ERR_ALIGN;
  if (out_dtype == BFP8_OUT_BF16 && (!aligned(out, 16) || ldo % 8 != 0)) return BFP8_ERR_ALIGN;
  if (out_dtype == BFP8_OUT_F32 && !aligned(out, 4)) return BFP8_ERR_ALIGN;
  return launch_gemm_channel(a_codes, lda, a_scales, w_codes, ldw, w_scales, bias, out, out_dtype, ldo, m, n, k,
                             status_dev, kDefaultWaitLimit, 0, static_cast<cudaStream_t>(stream));
}

// ---- gate/up GEMM with the SwiGLU step fused into its epilogue ---------------------------------------

namespace {
constexpr int kSwigluChunk = 64;

// Rows [0, inter) of src are the gate projection, rows [inter, 2 inter) the up projection.  Chunk c of 64
// outputs becomes dst rows [128 c, 128 c + 64) (gate) and [128 c + 64, 128 c + 128) (up).  16 bytes per thread.
__global__ void __launch_bounds__(256)
swiglu_interleave_kernel(const uint8_t* __restrict__ src, int64_t ld_src, uint8_t* __restrict__ dst, int64_t ld_dst,
                         int64_t inter, int64_t vecs_per_row) {
  const int64_t total = 2 * inter * vecs_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vecs_per_row, v = i - r * vecs_per_row;          // destination row, 16-byte column
    const int64_t chunk = r / (2 * kSwigluChunk), in_chunk = r - chunk * 2 * kSwigluChunk;
    const int64_t s_row = in_chunk < kSwigluChunk ? chunk * kSwigluChunk + in_chunk
                                                  : inter + chunk * kSwigluChunk + (in_chunk - kSwigluChunk);
    const uint4 x = __ldcs(reinterpret_cast<const uint4*>(src + s_row * ld_src) + v);
    __stcs(reinterpret_cast<uint4*>(dst + r * ld_dst) + v, x);
  }
}
}  // namespace

extern "C" int bfp8_swiglu_interleave_weight(const uint8_t* w_codes, int64_t ld_src, uint8_t* out, int64_t ld_dst,
                                             int64_t inter, int64_t k, void* stream) {
  if (!w_codes || !out) return BFP8_ERR_NULL;
  if (inter <= 0 || k <= 0 || ld_src < k || ld_dst < k || inter > (1 << 29)) return BFP8_ERR_SHAPE;
  if (inter % 128 != 0) return BFP8_ERR_UNSUPPORTED;
  if (k % 16 != 0 || ld_src % 16 != 0 || ld_dst % 16 != 0 || !aligned(w_codes, 16) || !aligned(out, 16))
    return BFP8_ERR_ALIGN;
  if (w_codes == out) return BFP8_ERR_SHAPE;                       // not an in-place operation
  const int64_t vecs = k / 16, total = 2 * inter * vecs;
  const int64_t want = (total + 255) / 256;
  const int grid = static_cast<int>(want < static_cast<int64_t>(sm_count()) * 16 ? want : static_cast<int64_t>(sm_count()) * 16);
  swiglu_interleave_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(w_codes, ld_src, out, ld_dst, inter, vecs);
  BFP8_CUDA_TRY(cudaGetLastError());
  return BFP8_OK;
}

extern "C" int bfp8_gemm_block128_swiglu(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                                         const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                                         const float* bias, void* out, int64_t ldo,
                                         int64_t m, int64_t inter, int64_t k,
                                         void* workspace, size_t workspace_bytes, uint32_t* status_dev, void* stream) {
  if (!a_codes || !a_scales || !w_codes || !w_scales || !out || !status_dev) return BFP8_ERR_NULL;
  if (m <= 0 || inter <= 0 || k <= 0 || m > (1 << 30) || inter > (1 << 29) || k > (1 << 30)) return BFP8_ERR_SHAPE;
  if (lda < k || ldw < k || ldo < inter || ldsa < m) return BFP8_ERR_SHAPE;
  if (inter % 128 != 0) return BFP8_ERR_UNSUPPORTED;               // gate / up boundary on a scale-block boundary
  if (!aligned(a_codes, 16) || !aligned(w_codes, 16) || lda % 16 != 0 || ldw % 16 != 0) return BFP8_ERR_ALIGN;
  if (!aligned(a_scales, 4) || !aligned(w_scales, 4) || !aligned(status_dev, 4)) return BFP8_ERR_ALIGN;
  if (bias && !aligned(bias, 4)) return BFP8_ERR_ALIGN;
  if (!aligned(out, 16) || ldo % 8 != 0) return BFP8_ERR_ALIGN;
  // decode bucket: the weight-streaming schedule, when the caller brought its scratch
  if (m <= kSmallMRows && smallm_supported(2 * inter) && workspace != nullptr) {
    if (workspace_bytes < bfp8_gemm_block128_workspace_bytes(m, 2 * inter, k)) return BFP8_ERR_WORKSPACE;
    if (!aligned(workspace, 256)) return BFP8_ERR_ALIGN;
    if (sm_count() > kMaxCtas) return BFP8_ERR_UNSUPPORTED;
    return launch_gemm_smallm(a_codes, lda, a_scales, ldsa, w_codes, ldw, w_scales, bias, out, BFP8_OUT_BF16, ldo, m,
                              2 * inter, k, workspace, status_dev, kDefaultWaitLimit, 0, static_cast<int>(inter),
                              /*push=*/nullptr, static_cast<cudaStream_t>(stream));
  }
  return launch_gemm_large(a_codes, lda, a_scales, ldsa, w_codes, ldw, w_scales, bias, out, BFP8_OUT_BF16, ldo,
                           m, 2 * inter, k, status_dev, kDefaultWaitLimit, 0, /*band=*/0, static_cast<int>(inter),
                           /*push=*/nullptr, static_cast<cudaStream_t>(stream));
}

// ---- the SwiGLU step on its own, for results of the schedules that have no fused form (decode bucket) -------

namespace {
// One 16-byte vector (8 outputs) per thread and iteration; gate at column c, up at column c + inter of a row.
__global__ void __launch_bounds__(256)
silu_and_mul_kernel(const uint16_t* __restrict__ gate_up, int64_t ld_in, uint16_t* __restrict__ out, int64_t ld_out,
                    int64_t rows, int64_t inter, int vec_ok) {
  // launched with programmatic stream serialization (see launch_overlapped)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (vec_ok) {
    const int64_t vecs = inter >> 3, total = rows * vecs;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      const int64_t r = i / vecs, v = i - r * vecs;
      const uint4 g = __ldcs(reinterpret_cast<const uint4*>(gate_up + r * ld_in) + v);
      const uint4 u = __ldcs(reinterpret_cast<const uint4*>(gate_up + r * ld_in + inter) + v);
      const uint32_t* gw = reinterpret_cast<const uint32_t*>(&g);
      const uint32_t* uw = reinterpret_cast<const uint32_t*>(&u);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = pack_bf16x2(silu_mul(bf16_lo_to_float(gw[j]), bf16_lo_to_float(uw[j])),
                           silu_mul(bf16_hi_to_float(gw[j]), bf16_hi_to_float(uw[j])));
      __stcs(reinterpret_cast<uint4*>(out + r * ld_out) + v, make_uint4(o[0], o[1], o[2], o[3]));
    }
  } else {
    const int64_t total = rows * inter;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      const int64_t r = i / inter, c = i - r * inter;
      const float g = bf16_bits_to_float(gate_up[r * ld_in + c]), u = bf16_bits_to_float(gate_up[r * ld_in + inter + c]);
      out[r * ld_out + c] = static_cast<uint16_t>(float_to_bf16_bits(silu_mul(g, u)));
    }
  }
}
}  // namespace

extern "C" int bfp8_silu_and_mul_bf16(const uint16_t* gate_up, int64_t ld_in, uint16_t* out, int64_t ld_out,
                                      int64_t rows, int64_t inter, void* stream) {
  if (!gate_up || !out) return BFP8_ERR_NULL;
  if (rows <= 0 || inter <= 0 || ld_in < 2 * inter || ld_out < inter || rows > (1LL << 40) / inter) return BFP8_ERR_SHAPE;
  if (!aligned(gate_up, 2) || !aligned(out, 2)) return BFP8_ERR_ALIGN;
  const int vec = aligned(gate_up, 16) && aligned(out, 16) && inter % 8 == 0 && ld_in % 8 == 0 && ld_out % 8 == 0;
  const int64_t work = vec ? rows * (inter / 8) : rows * inter;
  const int64_t want = (work + 255) / 256, cap = static_cast<int64_t>(sm_count()) * 8;
  return launch_overlapped(silu_and_mul_kernel, dim3(static_cast<unsigned>(want < cap ? want : cap)), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), gate_up, ld_in, out, ld_out, rows, inter, vec);
}

// ---- row-parallel GEMM whose epilogue scatters its tiles to the GPUs that reduce them -------------------

extern "C" int bfp8_gemm_block128_push(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                                       const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                                       void* const* recv, int rank, int world_size,
                                       int64_t m, int64_t n, int64_t k,
                                       void* workspace, size_t workspace_bytes, uint32_t* status_dev, void* stream) {
  if (!a_codes || !a_scales || !w_codes || !w_scales || !recv || !status_dev) return BFP8_ERR_NULL;
  if (m <= 0 || n <= 0 || k <= 0 || m > (1 << 30) || n > (1 << 30) || k > (1 << 30)) return BFP8_ERR_SHAPE;
  if (world_size < 2 || world_size > 8 || rank < 0 || rank >= world_size) return BFP8_ERR_UNSUPPORTED;
  if (lda < k || ldw < k || ldsa < m) return BFP8_ERR_SHAPE;
  // decode bucket: the weight-streaming schedule stores each activation row to the GPU that owns it
  const bool small = m <= kSmallMRows && m % world_size == 0 && n % 64 == 0 && smallm_supported(n) && workspace != nullptr;
  if (!small && (m % (128 * world_size) != 0 || n % 64 != 0)) return BFP8_ERR_UNSUPPORTED;
  if (!aligned(a_codes, 16) || !aligned(w_codes, 16) || lda % 16 != 0 || ldw % 16 != 0) return BFP8_ERR_ALIGN;
  if (!aligned(a_scales, 4) || !aligned(w_scales, 4) || !aligned(status_dev, 4)) return BFP8_ERR_ALIGN;
  PushTarget t = {};
  for (int o = 0; o < world_size; ++o) {
    if (!recv[o]) return BFP8_ERR_NULL;
    if (!aligned(recv[o], 16)) return BFP8_ERR_ALIGN;
    t.recv[o] = recv[o];
  }
  t.world = world_size;
  t.rank = rank;
  t.rows = static_cast<int>(m / world_size);
  if (small) {
    if (workspace_bytes < bfp8_gemm_block128_workspace_bytes(m, n, k)) return BFP8_ERR_WORKSPACE;
    if (!aligned(workspace, 256)) return BFP8_ERR_ALIGN;
    if (sm_count() > kMaxCtas) return BFP8_ERR_UNSUPPORTED;
    SmallPush sp = {};
    for (int o = 0; o < world_size; ++o) sp.recv[o] = t.recv[o];
    sp.world = t.world;
    sp.rank = t.rank;
    sp.rows = t.rows;
    return launch_gemm_smallm(a_codes, lda, a_scales, ldsa, w_codes, ldw, w_scales, nullptr, const_cast<void*>(t.recv[rank]),
                              BFP8_OUT_BF16, n, m, n, k, workspace, status_dev, kDefaultWaitLimit, 0, /*inter=*/0, &sp,
                              static_cast<cudaStream_t>(stream));
  }
  return launch_gemm_large(a_codes, lda, a_scales, ldsa, w_codes, ldw, w_scales, nullptr, const_cast<void*>(t.recv[rank]),
                           BFP8_OUT_BF16, n, m, n, k, status_dev, kDefaultWaitLimit, 0, /*band=*/0, /*inter=*/0, &t,
                           static_cast<cudaStream_t>(stream));
}
