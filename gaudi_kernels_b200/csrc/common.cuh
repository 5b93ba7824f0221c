// Shared helpers for the libbfp8 kernels (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "bfp8.h"

namespace bfp8 {

// Per-thread record of the last failing CUDA call, readable through bfp8_last_cuda_error().
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return BFP8_ERR_CUDA;
}

#define BFP8_CUDA_TRY(expr)                                   \
  do {                                                        \
    cudaError_t e_ = (expr);                                  \
    if (e_ != cudaSuccess) return ::bfp8::cuda_fail(e_);      \
  } while (0)

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Optional in-kernel timeline, for the diagnostic build only (-DBFP8_TIMELINE, written to libbfp8_timeline.so by
// `python -m gaudi_kernels_b200.build --timeline`).  The GEMM kernels then stamp %clock at a few events of every
// unit of work into a shared-memory log, and one CTA copies its log to a device array at teardown, which a
// bfp8_timeline_read_* function of the same file returns.  In the product build the macros expand to nothing.
#ifdef BFP8_TIMELINE
constexpr int kTimelineEvents = 8;      // events per unit of work
constexpr int kTimelineUnits = 40;      // units of work logged (the CTA's first ones; the large-tile kernel has 1.9 KB of shared memory to spare)
constexpr int kTimelineCta = 5;         // the CTA whose log is kept
__device__ __forceinline__ unsigned int timeline_clock() {
  unsigned int t;
  asm volatile("mov.u32 %0, %%clock;" : "=r"(t));
  return t;
}
#define BFP8_TL_DECL                                                                                          \
  __shared__ unsigned int tl_log[::bfp8::kTimelineEvents][::bfp8::kTimelineUnits];                            \
  for (int tl_i_ = threadIdx.x; tl_i_ < ::bfp8::kTimelineEvents * ::bfp8::kTimelineUnits; tl_i_ += blockDim.x) \
    (&tl_log[0][0])[tl_i_] = 0u;   /* made visible by the kernel's first __syncthreads */
#define BFP8_TL(event, unit)                                                                    \
  do {                                                                                          \
    const long long tl_u_ = static_cast<long long>(unit);                                       \
    if (tl_u_ >= 0 && tl_u_ < ::bfp8::kTimelineUnits) tl_log[event][tl_u_] = ::bfp8::timeline_clock(); \
  } while (0)
#define BFP8_TL_DUMP(dst)                                                                                     \
  do {                                                                                                        \
    if (blockIdx.x == ::bfp8::kTimelineCta)                                                                   \
      for (int tl_i_ = threadIdx.x; tl_i_ < ::bfp8::kTimelineEvents * ::bfp8::kTimelineUnits; tl_i_ += blockDim.x) \
        (dst)[tl_i_] = (&tl_log[0][0])[tl_i_];                                                                \
  } while (0)
#else
#define BFP8_TL_DECL
#define BFP8_TL(event, unit) ((void)0)
#define BFP8_TL_DUMP(dst) ((void)0)
#endif

// Number of SMs of the current device (cached per device id).
int sm_count();

// 2-D row-major tensor map (defined in gemm_tcgen05.cu); box_inner * element size must not exceed the swizzle span.
int make_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                       CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);

// One flag per device ordinal, shared by the host threads that call into the library.
typedef std::atomic<bool> DeviceFlags[64];

// Raise a kernel's dynamic shared-memory limit once per device (the attribute is per device context; setting it
// twice from two threads is harmless, so a relaxed flag is enough).  The caches of this library are keyed by
// device ordinal: they do not survive cudaDeviceReset.
template <typename Kernel>
inline int ensure_smem_limit(Kernel kernel, int bytes, DeviceFlags& done) {
  int dev = 0;
  BFP8_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !done[dev].load(std::memory_order_acquire)) {
    BFP8_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    if (dev >= 0 && dev < 64) done[dev].store(true, std::memory_order_release);
  }
  return BFP8_OK;
}

// Launch with the programmatic-stream-serialization attribute: the kernel may be scheduled while the previous
// kernel of the stream is still finishing and must call ptx::griddep_wait() (or the griddepcontrol.wait
// instruction) before it touches global memory.  Used for the short kernels of a decode step, where the launch
// path is a large part of the run time.
template <typename... KArgs, typename... Args>
inline int launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  BFP8_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
  return BFP8_OK;
}

// ---- E4M3 byte arithmetic -----------------------------------------------------------------

// Byte-parallel arithmetic on four packed codes, written with plain 32-bit logic (the __v*4 SIMD
// intrinsics are multi-instruction emulations on this architecture).

// 0xff in every byte whose magnitude (low 7 bits) is >= 16, i.e. has any of bits 4..6 set.
__device__ __forceinline__ uint32_t ge16_mask_x4(uint32_t mag) {
  const uint32_t t = mag & 0x70707070u;
  const uint32_t one = ((t | (t >> 1) | (t >> 2)) >> 4) & 0x01010101u;     // 0 / 1 per byte
  return (one << 8) - one;                                                // 0x00 / 0xff per byte, no cross-byte carry
}

// Half of four packed OCP E4M3FN codes, round-to-nearest-even, in the Gaudi2 encoding
// (the byte map of python/gaudi_kernels/fp8_codec.py:36-40 evaluated on four bytes at once):
// magnitude >= 16 loses one exponent step (magnitude - 8); below that the significand shifts right
// by one and an odd magnitude rounds up only when the shifted value is odd.
__device__ __forceinline__ uint32_t half_e4m3x4(uint32_t w) {
  const uint32_t mag = w & 0x7f7f7f7fu;
  const uint32_t ge16 = ge16_mask_x4(mag);
  // bit 7 is set first so that no byte borrows from its neighbour; bytes below 8 are masked out anyway
  const uint32_t hi = ((mag | 0x80808080u) - 0x08080808u) & 0x7f7f7f7fu;
  const uint32_t sh = (mag >> 1) & 0x3f3f3f3fu;
  const uint32_t lo = sh + (mag & sh & 0x01010101u);
  return (w & 0x80808080u) | (lo ^ ((lo ^ hi) & ge16));
}

// Bit 0 of each byte set where halving that code is inexact (magnitude < 16 and odd).
__device__ __forceinline__ uint32_t half_inexact_x4(uint32_t w) {
  const uint32_t mag = w & 0x7f7f7f7fu;
  return mag & 0x01010101u & ~ge16_mask_x4(mag);
}

// Non-zero where a byte is 0x7f or 0xff: only a magnitude of 0x7f carries into bit 7 when 1 is added.
__device__ __forceinline__ uint32_t nonfinite_x4(uint32_t w) {
  return ((w & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u;
}

// Two fp32 -> two OCP E4M3 codes (RNE, finite saturation), `lo` in bits 0-7.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  return cvt_e4m3x2(a, b) | (cvt_e4m3x2(c, d) << 16);
}

// Two OCP E4M3 codes (bits 0-15) -> two fp32, exact.
__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t v) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(v)));
  float lo, hi;
  asm("{.reg .f16 l, h; mov.b32 {l, h}, %2; cvt.f32.f16 %0, l; cvt.f32.f16 %1, h;}"
      : "=f"(lo), "=f"(hi) : "r"(h2));
  return make_float2(lo, hi);
}

// The activation / weight scale rule of block_fp8_oracle.py:27: max(amax, 1e-10) * fp32(1/448),
// one fp32 multiply rounded to nearest (no contraction).
__device__ __forceinline__ float scale_from_amax(float amax) {
  return __fmul_rn(fmaxf(amax, 1e-10f), static_cast<float>(1.0 / 448.0));
}

// block_fp8_oracle.py:28: IEEE fp32 division, clamp to +-448.
__device__ __forceinline__ float scaled_clamped(float x, float scale) {
  return fminf(fmaxf(__fdiv_rn(x, scale), -448.0f), 448.0f);
}

// Two values -> two OCP E4M3 codes of RNE(clamp(x / scale, +-448)), bit-identical to doing the IEEE
// division, without a division: with rcp = RN(1 / scale), q = RN(x * rcp) is within one ulp of the
// quotient, the residual e = x - q * scale is exact in one FMA, and RN(q + e * rcp) is the correctly
// rounded quotient (Markstein's correction step).  All three steps are packed two-wide fp32 operations.
// Saturating conversion covers the clamp: anything above 448 rounds or saturates to the code of 448.
// Quotients too small to be normal fp32 numbers round to a zero code whatever their last bits are.
__device__ __forceinline__ uint32_t quant_e4m3x2(float x0, float x1, float scale, float rcp) {
  const float2 x = make_float2(x0, x1), r = make_float2(rcp, rcp);
  const float2 q = __fmul2_rn(x, r);
  const float2 e = __ffma2_rn(q, make_float2(-scale, -scale), x);
  const float2 qc = __ffma2_rn(e, r, q);
  return cvt_e4m3x2(qc.x, qc.y);
}

// Half of two packed E4M3 codes with round-to-nearest-even, through the conversion units: the codes
// widen exactly to fp16, halving is exact there, and the narrowing conversion rounds to nearest even
// (subnormals included) - the same two-step rounding as the byte map of half_e4m3x4 for every finite code.
__device__ __forceinline__ uint32_t half_e4m3x2_cvt(uint32_t codes) {
  uint16_t r;
  asm("{\n\t.reg .b32 t, h;\n\t"
      "cvt.rn.f16x2.e4m3x2 t, %1;\n\t"
      "mov.b32 h, 0x38003800;\n\t"                  // 0.5 in both fp16 halves
      "mul.rn.f16x2 t, t, h;\n\t"
      "cvt.rn.satfinite.e4m3x2.f16x2 %0, t;\n\t}"
      : "=h"(r) : "h"(static_cast<uint16_t>(codes)));
  return r;
}

// quant_e4m3x2 followed by the half-range step (block_fp8_oracle.py:31-34), both roundings included.
__device__ __forceinline__ uint32_t quant_half_e4m3x2(float x0, float x1, float scale, float rcp) {
  return half_e4m3x2_cvt(quant_e4m3x2(x0, x1, scale, rcp));
}

__device__ __forceinline__ uint32_t quant_half_e4m3x4(float a, float b, float c, float d, float scale, float rcp) {
  return quant_half_e4m3x2(a, b, scale, rcp) | (quant_half_e4m3x2(c, d, scale, rcp) << 16);
}

// max(a, |b|) that returns NaN if either is NaN, so one test after a reduction catches any NaN or inf input.
__device__ __forceinline__ float max_abs_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(fabsf(b)));
  return r;
}

__device__ __forceinline__ uint32_t quant_e4m3x4(float a, float b, float c, float d, float scale, float rcp) {
  return quant_e4m3x2(a, b, scale, rcp) | (quant_e4m3x2(c, d, scale, rcp) << 16);
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }
// The two halves of a packed bf16 pair.
__device__ __forceinline__ float bf16_lo_to_float(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi_to_float(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }

// fp32 -> bf16 bits, round-to-nearest-even (finite inputs and NaN-preserving).
__device__ __forceinline__ uint32_t float_to_bf16_bits(float f) {
  uint16_t r;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
  return r;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// silu(g) * u as csrc/tpc/generic_dense/silu_and_mul_bf16.c:4-13 defines it: denom = 1 + exp(-g); the quotient
// g / denom is an approximate reciprocal refined by one residual step (q = g * inv; q += fma(-q, denom, g) * inv,
// :6-9), exactly 0 for g <= -88 (:10), and a NaN gate is passed through by bit pattern (:11-12).  The refined
// quotient is the correctly rounded one except in rare last-bit cases; what is left against an exact evaluation
// is the error of ex2.approx in exp(-g).
__device__ __forceinline__ float silu_mul(float g, float u) {
  const float denom = 1.0f + __expf(-g);
  float inv;
  asm("rcp.approx.f32 %0, %1;" : "=f"(inv) : "f"(denom));
  const float q = g * inv;
  const float refined = __fmaf_rn(__fmaf_rn(-q, denom, g), inv, q);
  float val = g <= -88.0f ? 0.0f : refined;
  if ((__float_as_uint(g) & 0x7fffffffu) > 0x7f800000u) val = g;
  return val * u;
}

// 64 output columns of one row as bf16 with plain stores, only the first `valid` of them.  Used for the
// last box of a row when N is not a multiple of 8: a bulk tensor store writes whole 16-byte chunks.
__device__ __forceinline__ void store_row_bf16_guarded(uint16_t* o, const float2* a, int valid) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    if (2 * j < valid) o[2 * j] = static_cast<uint16_t>(float_to_bf16_bits(a[j].x));
    if (2 * j + 1 < valid) o[2 * j + 1] = static_cast<uint16_t>(float_to_bf16_bits(a[j].y));
  }
}

}  // namespace bfp8
