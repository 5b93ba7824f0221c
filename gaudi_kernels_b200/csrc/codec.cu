// E4M3 codec kernels: OCP -> half-range re-encode, 128x128 and 1x128 block-amax quantizers, decode.
// All four are streaming, HBM-bound byte kernels: 128-bit coalesced accesses, everything else in registers.
#include "common.cuh"

namespace bfp8 {

thread_local int g_last_cuda_error = 0;

int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_acquire);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_release);
  }
  return n;
}

// ---------------------------------------------------------------------------------------------
// K1  re-encode: 1 byte in, 1 byte out per code.
// ---------------------------------------------------------------------------------------------
constexpr int kReencodeThreads = 256;
constexpr int kReencodeUnroll = 4;     // 4 x 16 B in flight per thread

__device__ __forceinline__ void reencode_vec(uint4& v, uint32_t& inexact, uint32_t& bad) {
  uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    bad |= nonfinite_x4(w[i]);
    inexact += __popc(half_inexact_x4(w[i]));
    w[i] = half_e4m3x2_cvt(w[i] & 0xffffu) | (half_e4m3x2_cvt(w[i] >> 16) << 16);
  }
}

__global__ void __launch_bounds__(kReencodeThreads)
reencode_half_kernel(const uint8_t* in, uint8_t* out, int64_t n, int vec_ok,          // in == out is allowed
                     const float* scales_in, float* scales_out, int64_t n_scales,
                     unsigned long long* __restrict__ rounded, uint32_t* __restrict__ status) {
  __shared__ uint32_t cta_inexact, cta_bad;
  if (threadIdx.x == 0) { cta_inexact = 0; cta_bad = 0; }
  __syncthreads();
  uint32_t inexact = 0, bad = 0;
  // scales_out = 2 * scales_in with the checks of fp8_codec.py:25-32, spread over the CTAs of this launch
  {
    const int64_t per_cta = (n_scales + gridDim.x - 1) / gridDim.x;
    const int64_t s0 = static_cast<int64_t>(blockIdx.x) * per_cta;
    const int64_t s1 = s0 + per_cta < n_scales ? s0 + per_cta : n_scales;
    bool bad_scale = false;
    for (int64_t i = s0 + threadIdx.x; i < s1; i += kReencodeThreads) {
      const float sc = scales_in[i];
      const float d = __fmul_rn(sc, 2.0f);
      bad_scale |= !(sc >= 0.0f) || isinf(d) || isnan(d);
      scales_out[i] = d;
    }
    if (bad_scale) atomicOr(status, BFP8_STATUS_BAD_SCALE);
  }
  // A CTA owns one contiguous chunk of kReencodeUnroll x 256 vectors (16 KB); a warp access is 512 B.
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * (kReencodeThreads * kReencodeUnroll);
  if (vec_ok) {
    const int64_t nvec = n >> 4;
    const uint4* vin = reinterpret_cast<const uint4*>(in);
    uint4* vout = reinterpret_cast<uint4*>(out);
    uint4 v[kReencodeUnroll];
#pragma unroll
    for (int u = 0; u < kReencodeUnroll; ++u) {
      const int64_t i = chunk + u * kReencodeThreads + threadIdx.x;
      if (i < nvec) v[u] = __ldcs(vin + i);
    }
#pragma unroll
    for (int u = 0; u < kReencodeUnroll; ++u) {
      const int64_t i = chunk + u * kReencodeThreads + threadIdx.x;
      if (i < nvec) {
        reencode_vec(v[u], inexact, bad);
        __stcs(vout + i, v[u]);
      }
    }
    // ragged tail (fewer than 16 bytes): the last CTA's first threads
    if (blockIdx.x == gridDim.x - 1) {
      const int64_t i = (nvec << 4) + threadIdx.x;
      if (i < n) {
        const uint32_t c = in[i];
        bad |= nonfinite_x4(c) & 0xffu;
        inexact += half_inexact_x4(c) & 1u;
        out[i] = static_cast<uint8_t>(half_e4m3x4(c));
      }
    }
  } else {
    // unaligned buffers: the same chunk, byte by byte
    const int64_t first = chunk * 16;
#pragma unroll 4
    for (int j = 0; j < kReencodeUnroll * 16; ++j) {
      const int64_t i = first + static_cast<int64_t>(j) * kReencodeThreads + threadIdx.x;
      if (i < n) {
        const uint32_t c = in[i];
        bad |= nonfinite_x4(c) & 0xffu;
        inexact += half_inexact_x4(c) & 1u;
        out[i] = static_cast<uint8_t>(half_e4m3x4(c));
      }
    }
  }
  // warp reduction, then one shared-memory atomic per warp and one global atomic per CTA at most
  inexact = __reduce_add_sync(0xffffffffu, inexact);
  bad = __reduce_or_sync(0xffffffffu, bad);
  if ((threadIdx.x & 31) == 0) {
    if (inexact) atomicAdd(&cta_inexact, inexact);
    if (bad) atomicOr(&cta_bad, 1u);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (cta_inexact) atomicAdd(rounded, static_cast<unsigned long long>(cta_inexact));
    if (cta_bad) atomicOr(status, BFP8_STATUS_NONFINITE_CODE);
  }
}

// Read-only form of the checks above for checkpoints that are used as they are (OCP codes, no half-range
// step): any 0x7f / 0xff code, any negative or non-finite scale.  Grid-stride, 16 bytes per thread and step.
__global__ void __launch_bounds__(256)
validate_e4m3_kernel(const uint8_t* __restrict__ codes, int64_t n, int vec_ok, const float* __restrict__ scales,
                     int64_t n_scales, uint32_t* __restrict__ status) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  uint32_t bad = 0;
  if (vec_ok) {
    const int64_t nvec = n >> 4;
    const uint4* v = reinterpret_cast<const uint4*>(codes);
    for (int64_t i = tid; i < nvec; i += nthreads) {
      const uint4 x = __ldcs(v + i);
      bad |= nonfinite_x4(x.x) | nonfinite_x4(x.y) | nonfinite_x4(x.z) | nonfinite_x4(x.w);
    }
    for (int64_t i = (nvec << 4) + tid; i < n; i += nthreads) bad |= nonfinite_x4(codes[i]) & 0xffu;
  } else {
    for (int64_t i = tid; i < n; i += nthreads) bad |= nonfinite_x4(codes[i]) & 0xffu;
  }
  bool bad_scale = false;
  for (int64_t i = tid; i < n_scales; i += nthreads) {
    const float sc = scales[i];
    bad_scale |= !(sc >= 0.0f) || isinf(sc);
  }
  bad = __reduce_or_sync(0xffffffffu, bad);
  const uint32_t bs = __reduce_or_sync(0xffffffffu, bad_scale ? 1u : 0u);
  if ((threadIdx.x & 31) == 0) {
    if (bad) atomicOr(status, BFP8_STATUS_NONFINITE_CODE);
    if (bs) atomicOr(status, BFP8_STATUS_BAD_SCALE);
  }
}

// ---------------------------------------------------------------------------------------------
// K2  128x128 block-amax quantizer: one CTA per tile, the 64 KB tile lives in registers
//     (256 threads x 16 float4), so HBM sees exactly one read and one write per element.
// ---------------------------------------------------------------------------------------------
constexpr int kQuantThreads = 256;

template <bool kVec>
__global__ void __launch_bounds__(kQuantThreads, 3)
quant_block128_kernel(const float* __restrict__ w, int64_t rows, int64_t cols, int64_t ld,
                      uint8_t* __restrict__ codes, int64_t ld_codes, float* __restrict__ scales,
                      int col_blocks, int native_half) {
  __shared__ float warp_max[kQuantThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 128, c0 = static_cast<int64_t>(blockIdx.x) * 128;
  const int64_t c = c0 + lane * 4;
  float4 v[16];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t r = r0 + warp + 8 * i;
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < rows) {
      const float* p = w + r * ld + c;
      if (kVec) {
        if (c < cols) v[i] = __ldcs(reinterpret_cast<const float4*>(p));   // cols % 4 == 0 on this path
      } else {
        if (c + 0 < cols) v[i].x = p[0];
        if (c + 1 < cols) v[i].y = p[1];
        if (c + 2 < cols) v[i].z = p[2];
        if (c + 3 < cols) v[i].w = p[3];
      }
    }
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) warp_max[warp] = amax;
  __syncthreads();
  amax = warp_max[0];
#pragma unroll
  for (int i = 1; i < kQuantThreads / 32; ++i) amax = fmaxf(amax, warp_max[i]);
  const float s = scale_from_amax(amax);
  const float rcp = __frcp_rn(s);
  if (threadIdx.x == 0)
    scales[static_cast<int64_t>(blockIdx.y) * col_blocks + blockIdx.x] = native_half ? __fmul_rn(s, 2.0f) : s;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t r = r0 + warp + 8 * i;
    if (r >= rows) continue;
    const uint32_t q = native_half ? quant_half_e4m3x4(v[i].x, v[i].y, v[i].z, v[i].w, s, rcp)
                                   : quant_e4m3x4(v[i].x, v[i].y, v[i].z, v[i].w, s, rcp);
    uint8_t* p = codes + r * ld_codes + c;
    if (kVec) {
      if (c < cols) __stcs(reinterpret_cast<uint32_t*>(p), q);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + j < cols) p[j] = static_cast<uint8_t>(q >> (8 * j));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// K3  1x128 activation quantizer: a quarter-warp (8 lanes x 16 bf16 = 32 B each) owns one group, so the
//     group maximum takes three shuffle steps and the scale arithmetic is shared by 16 elements per lane.
//     A CTA of 32 quarter-warps with two group slots each covers 64 groups per pass: one row when a row has
//     at least 64 groups, otherwise 64 / groups rows at once; no index division sits in the loop.
// ---------------------------------------------------------------------------------------------
constexpr int kActThreads = 256;
constexpr int kActLanes = 8;                                   // lanes per group
constexpr int kActElems = 128 / kActLanes;                     // elements per lane: 16
constexpr int kActPer = 2;                                     // group slots per quarter-warp and pass
constexpr int kActSlots = kActThreads / kActLanes * kActPer;   // group slots per CTA and pass: 64

// silu(g) * u of csrc/tpc/generic_dense/silu_and_mul_bf16.c:4-13, rounded to bf16 as that kernel stores it; the
// same expression as the GEMM's fused epilogue and the stand-alone kernel, so all three agree bit for bit.
__device__ __forceinline__ float silu_mul_bf16_rounded(float g, float u) {
  return bf16_bits_to_float(float_to_bf16_bits(silu_mul(g, u)));
}

// kSilu: x is a gate/up pair [m, 2 k] (gate columns, then up columns, row pitch ldx) and the values quantized are
// bf16(silu(gate) * up) - gk_silu_and_mul_bf16_v1 followed by the 1x128 quantizer, without the round trip of the
// intermediate tensor through HBM.
template <bool kVec, bool kSilu>
__global__ void __launch_bounds__(kActThreads, kSilu ? 4 : 6)
quant_act_1x128_kernel(const uint16_t* __restrict__ x, int64_t m, int64_t k, int64_t ldx,
                       uint8_t* __restrict__ codes, int64_t ld_codes, float* __restrict__ scales,
                       int64_t ssm, int64_t ssg, int groups, int native_half,
                       uint32_t* __restrict__ status, int iters_per_cta) {
  // launched with programmatic stream serialization: let the next kernel be scheduled, then wait for the previous one
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int sub = threadIdx.x & (kActLanes - 1);               // lane inside the quarter-warp
  const int qw = threadIdx.x / kActLanes;                      // quarter-warp inside the CTA, 0..31
  uint32_t nonfinite = 0;
  // slot t = qw + 32 u of a pass is (row offset, group) of this quarter-warp's u-th group
  const bool whole_row = groups >= kActSlots;
  const int rows_per_cta = whole_row ? 1 : kActSlots / groups;
  int row_off[kActPer], g_first[kActPer];
#pragma unroll
  for (int u = 0; u < kActPer; ++u) {
    const int t = qw + (kActThreads / kActLanes) * u;
    row_off[u] = whole_row ? 0 : t / groups;
    g_first[u] = whole_row ? t : t - row_off[u] * groups;
    if (row_off[u] >= rows_per_cta) g_first[u] = groups;       // spare slots stay idle
  }
  // warp-uniform trip counts: shuffles below are warp-wide
  const int g_iters = whole_row ? (groups + kActSlots - 1) / kActSlots : 1;
  // with few rows the passes over a long row are spread over blockIdx.y, so that a decode-sized call is not
  // one CTA walking the whole row
  const int gi_end = min(g_iters, (static_cast<int>(blockIdx.y) + 1) * iters_per_cta);
  for (int gi = blockIdx.y * iters_per_cta; gi < gi_end; ++gi) {
    bool live[kActPer];
    int g[kActPer];
    int64_t row[kActPer], col[kActPer];
    uint4 raw[kActPer][2], raw_up[kSilu ? kActPer : 1][2];
#pragma unroll
    for (int u = 0; u < kActPer; ++u) {
      row[u] = static_cast<int64_t>(blockIdx.x) * rows_per_cta + row_off[u];
      g[u] = g_first[u] + gi * kActSlots;
      // gridDim.z == kActPer (few rows): each CTA serves one of the slots, so twice as many CTAs share a row
      live[u] = row[u] < m && g[u] < groups && (gridDim.z == 1 || static_cast<int>(blockIdx.z) == u);
      col[u] = static_cast<int64_t>(g[u]) * 128 + sub * kActElems;
      const uint16_t* xrow = x + row[u] * ldx;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        raw[u][h] = make_uint4(0u, 0u, 0u, 0u);
        if (kSilu) raw_up[u][h] = make_uint4(0u, 0u, 0u, 0u);
        if (kVec && live[u] && col[u] + 8 * h < k) {                      // k % 8 == 0 on this path
          raw[u][h] = __ldcs(reinterpret_cast<const uint4*>(xrow + col[u] + 8 * h));
          if (kSilu) raw_up[u][h] = __ldcs(reinterpret_cast<const uint4*>(xrow + k + col[u] + 8 * h));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kActPer; ++u) {
      const uint16_t* xrow = x + row[u] * ldx;
      float f[kActElems];
      if (kVec) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t* r = reinterpret_cast<const uint32_t*>(&raw[u][h]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            f[8 * h + 2 * j] = bf16_lo_to_float(r[j]);
            f[8 * h + 2 * j + 1] = bf16_hi_to_float(r[j]);
          }
          if (kSilu) {
            const uint32_t* ru = reinterpret_cast<const uint32_t*>(&raw_up[u][h]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              f[8 * h + 2 * j] = silu_mul_bf16_rounded(f[8 * h + 2 * j], bf16_lo_to_float(ru[j]));
              f[8 * h + 2 * j + 1] = silu_mul_bf16_rounded(f[8 * h + 2 * j + 1], bf16_hi_to_float(ru[j]));
            }
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < kActElems; ++j) {
          f[j] = 0.0f;
          if (live[u] && col[u] + j < k) {
            f[j] = bf16_bits_to_float(xrow[col[u] + j]);
            if (kSilu) f[j] = silu_mul_bf16_rounded(f[j], bf16_bits_to_float(xrow[k + col[u] + j]));
          }
        }
      }
      // NaN-propagating maximum: an inf or NaN anywhere in the group surfaces in amax
      float amax = 0.0f;
#pragma unroll
      for (int j = 0; j < kActElems; ++j) amax = max_abs_nan(amax, f[j]);
#pragma unroll
      for (int o = kActLanes / 2; o > 0; o >>= 1) amax = max_abs_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      nonfinite |= !(amax < __int_as_float(0x7f800000));
      const float s = scale_from_amax(amax);
      const float rcp = __frcp_rn(s);
      uint32_t q[4];
#pragma unroll
      for (int w = 0; w < 4; ++w)
        q[w] = native_half ? quant_half_e4m3x4(f[4 * w], f[4 * w + 1], f[4 * w + 2], f[4 * w + 3], s, rcp)
                           : quant_e4m3x4(f[4 * w], f[4 * w + 1], f[4 * w + 2], f[4 * w + 3], s, rcp);
      if (live[u]) {
        uint8_t* p = codes + row[u] * ld_codes + col[u];
        if (kVec) {
          if (col[u] < k) __stcs(reinterpret_cast<uint2*>(p), make_uint2(q[0], q[1]));
          if (col[u] + 8 < k) __stcs(reinterpret_cast<uint2*>(p + 8), make_uint2(q[2], q[3]));
        } else {
#pragma unroll
          for (int j = 0; j < kActElems; ++j)
            if (col[u] + j < k) p[j] = static_cast<uint8_t>(q[j >> 2] >> (8 * (j & 3)));
        }
        if (sub == 0) scales[row[u] * ssm + g[u] * ssg] = native_half ? __fmul_rn(s, 2.0f) : s;
      }
    }
  }
  if (status != nullptr && __any_sync(0xffffffffu, nonfinite != 0) && (threadIdx.x & 31) == 0)
    atomicOr(status, BFP8_STATUS_NONFINITE_INPUT);
}

// ---------------------------------------------------------------------------------------------
// K5  per-token activation quantizer: one scale per row (the per-token / per-channel FP8 variant,
//     csrc/tpc/block_fp8_framework/activation_token.c:4-26).  One CTA per row; the row is read once into
//     registers (up to 16384 columns; longer rows are read a second time, from L2).
//     scale = amax / 448 as an IEEE division, with 1 substituted for the amax of an all-zero row (:17).
// ---------------------------------------------------------------------------------------------
constexpr int kTokThreads = 256;
constexpr int kTokVecs = 8;            // 16-byte vectors a thread keeps in registers

__global__ void __launch_bounds__(kTokThreads)
quant_act_token_kernel(const uint16_t* __restrict__ x, int64_t k, int64_t ldx, uint8_t* __restrict__ codes,
                       int64_t ld_codes, float* __restrict__ scales, int native_half, int vec_ok,
                       uint32_t* __restrict__ status) {
  __shared__ float warp_max[kTokThreads / 32];
  const int64_t row = blockIdx.x;
  const uint16_t* xrow = x + row * ldx;
  uint8_t* crow = codes + row * ld_codes;
  const int64_t nvec = vec_ok ? (k >> 3) : 0;                    // k % 8 == 0 on the vector path
  uint4 raw[kTokVecs];
  float amax = 0.0f;
#pragma unroll
  for (int u = 0; u < kTokVecs; ++u) {
    const int64_t i = static_cast<int64_t>(u) * kTokThreads + threadIdx.x;
    raw[u] = make_uint4(0u, 0u, 0u, 0u);
    if (i < nvec) raw[u] = __ldcs(reinterpret_cast<const uint4*>(xrow) + i);
    const uint32_t* r = reinterpret_cast<const uint32_t*>(&raw[u]);
#pragma unroll
    for (int j = 0; j < 4; ++j) amax = max_abs_nan(max_abs_nan(amax, bf16_lo_to_float(r[j])), bf16_hi_to_float(r[j]));
  }
  for (int64_t i = static_cast<int64_t>(kTokVecs) * kTokThreads + threadIdx.x; i < nvec; i += kTokThreads) {
    const uint4 v = *(reinterpret_cast<const uint4*>(xrow) + i);
    const uint32_t* r = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) amax = max_abs_nan(max_abs_nan(amax, bf16_lo_to_float(r[j])), bf16_hi_to_float(r[j]));
  }
  for (int64_t i = (nvec << 3) + threadIdx.x; i < k; i += kTokThreads)       // scalar path / ragged tail
    amax = max_abs_nan(amax, bf16_bits_to_float(xrow[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = max_abs_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = warp_max[0];
#pragma unroll
  for (int i = 1; i < kTokThreads / 32; ++i) amax = max_abs_nan(amax, warp_max[i]);
  if (!(amax < __int_as_float(0x7f800000)) && threadIdx.x == 0 && status != nullptr)
    atomicOr(status, BFP8_STATUS_NONFINITE_INPUT);
  const float s = __fdiv_rn(amax == 0.0f ? 1.0f : amax, 448.0f);
  const float rcp = __frcp_rn(s);
  if (threadIdx.x == 0) scales[row] = native_half ? __fmul_rn(s, 2.0f) : s;
  auto quant8 = [&](const uint4& v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(&v);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { f[2 * j] = bf16_lo_to_float(r[j]); f[2 * j + 1] = bf16_hi_to_float(r[j]); }
    uint2 q;
    if (native_half) {
      q.x = quant_half_e4m3x4(f[0], f[1], f[2], f[3], s, rcp);
      q.y = quant_half_e4m3x4(f[4], f[5], f[6], f[7], s, rcp);
    } else {
      q.x = quant_e4m3x4(f[0], f[1], f[2], f[3], s, rcp);
      q.y = quant_e4m3x4(f[4], f[5], f[6], f[7], s, rcp);
    }
    return q;
  };
#pragma unroll
  for (int u = 0; u < kTokVecs; ++u) {
    const int64_t i = static_cast<int64_t>(u) * kTokThreads + threadIdx.x;
    if (i < nvec) __stcs(reinterpret_cast<uint2*>(crow) + i, quant8(raw[u]));
  }
  for (int64_t i = static_cast<int64_t>(kTokVecs) * kTokThreads + threadIdx.x; i < nvec; i += kTokThreads)
    __stcs(reinterpret_cast<uint2*>(crow) + i, quant8(*(reinterpret_cast<const uint4*>(xrow) + i)));
  for (int64_t i = (nvec << 3) + threadIdx.x; i < k; i += kTokThreads) {
    const float f = bf16_bits_to_float(xrow[i]);
    const uint32_t q = native_half ? quant_half_e4m3x2(f, 0.0f, s, rcp) : quant_e4m3x2(f, 0.0f, s, rcp);
    crow[i] = static_cast<uint8_t>(q);
  }
}

// Rows of up to 4096 columns: one warp per row, all 16 of a lane's 16-byte loads in flight before the first use,
// and no CTA-wide barrier between the maximum and the conversion.  Same arithmetic as the CTA-per-row kernel.
constexpr int kTokWarpVecs = 16;
constexpr int kTokWarpMaxK = kTokWarpVecs * 32 * 8;
constexpr int kTokWarpThreads = 128;    // four rows per CTA; three CTAs fit one SM's registers

__global__ void __launch_bounds__(kTokWarpThreads, 3)
quant_act_token_warp_kernel(const uint16_t* __restrict__ x, int64_t m, int64_t k, int64_t ldx,
                            uint8_t* __restrict__ codes, int64_t ld_codes, float* __restrict__ scales,
                            int native_half, uint32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kTokWarpThreads / 32) + (threadIdx.x >> 5);
  if (row >= m) return;
  const uint4* xrow = reinterpret_cast<const uint4*>(x + row * ldx);
  uint2* crow = reinterpret_cast<uint2*>(codes + row * ld_codes);
  const int nvec = static_cast<int>(k >> 3);
  uint4 raw[kTokWarpVecs];
#pragma unroll
  for (int u = 0; u < kTokWarpVecs; ++u) {
    const int i = u * 32 + lane;
    raw[u] = make_uint4(0u, 0u, 0u, 0u);
    if (i < nvec) raw[u] = __ldcs(xrow + i);
  }
  float amax = 0.0f;
#pragma unroll
  for (int u = 0; u < kTokWarpVecs; ++u) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(&raw[u]);
#pragma unroll
    for (int j = 0; j < 4; ++j) amax = max_abs_nan(max_abs_nan(amax, bf16_lo_to_float(r[j])), bf16_hi_to_float(r[j]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = max_abs_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (!(amax < __int_as_float(0x7f800000)) && lane == 0 && status != nullptr)
    atomicOr(status, BFP8_STATUS_NONFINITE_INPUT);
  const float s = __fdiv_rn(amax == 0.0f ? 1.0f : amax, 448.0f);
  const float rcp = __frcp_rn(s);
  if (lane == 0) scales[row] = native_half ? __fmul_rn(s, 2.0f) : s;
#pragma unroll
  for (int u = 0; u < kTokWarpVecs; ++u) {
    const int i = u * 32 + lane;
    const uint32_t* r = reinterpret_cast<const uint32_t*>(&raw[u]);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { f[2 * j] = bf16_lo_to_float(r[j]); f[2 * j + 1] = bf16_hi_to_float(r[j]); }
    uint2 q;
    if (native_half) {
      q.x = quant_half_e4m3x4(f[0], f[1], f[2], f[3], s, rcp);
      q.y = quant_half_e4m3x4(f[4], f[5], f[6], f[7], s, rcp);
    } else {
      q.x = quant_e4m3x4(f[0], f[1], f[2], f[3], s, rcp);
      q.y = quant_e4m3x4(f[4], f[5], f[6], f[7], s, rcp);
    }
    if (i < nvec) __stcs(crow + i, q);
  }
}

// Many rows of up to 8192 columns: kRowThreads threads per row (32, 64, 128 or 256, the smallest that covers the row
// with four 16-byte loads per thread), 256 / kRowThreads rows per CTA, the row maximum combined through shared memory
// and a named barrier of the row's threads.  Fewer registers than the warp-per-row form, so four times as many warps
// are resident and hide the load latency; sizing the thread group to the row keeps every thread loaded.
constexpr int kTokGroupCta = 256;
constexpr int kTokGroupVecs = 4;
constexpr int kTokGroupMaxK = kTokGroupVecs * kTokGroupCta * 8;      // 8192

template <int kRowThreads>
__global__ void __launch_bounds__(kTokGroupCta, 4)
quant_act_token_group_kernel(const uint16_t* __restrict__ x, int64_t m, int64_t k, int64_t ldx,
                             uint8_t* __restrict__ codes, int64_t ld_codes, float* __restrict__ scales,
                             int native_half, uint32_t* __restrict__ status) {
  constexpr int kRows = kTokGroupCta / kRowThreads;                // rows per CTA
  constexpr int kWarps = kRowThreads / 32;                         // warps per row
  __shared__ float warp_max[kRows][kWarps];
  const int grp = threadIdx.x / kRowThreads;                       // which of the CTA's rows
  const int t = threadIdx.x - grp * kRowThreads;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kRows + grp;
  const bool row_ok = row < m;
  const uint4* xrow = reinterpret_cast<const uint4*>(x + (row_ok ? row : 0) * ldx);
  uint2* crow = reinterpret_cast<uint2*>(codes + (row_ok ? row : 0) * ld_codes);
  const int nvec = row_ok ? static_cast<int>(k >> 3) : 0;
  uint4 raw[kTokGroupVecs];
#pragma unroll
  for (int u = 0; u < kTokGroupVecs; ++u) {
    const int i = u * kRowThreads + t;
    raw[u] = make_uint4(0u, 0u, 0u, 0u);
    if (i < nvec) raw[u] = __ldcs(xrow + i);
  }
  float amax = 0.0f;
#pragma unroll
  for (int u = 0; u < kTokGroupVecs; ++u) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(&raw[u]);
#pragma unroll
    for (int j = 0; j < 4; ++j) amax = max_abs_nan(max_abs_nan(amax, bf16_lo_to_float(r[j])), bf16_hi_to_float(r[j]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = max_abs_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (kWarps > 1) {
    if ((t & 31) == 0) warp_max[grp][t >> 5] = amax;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(kRowThreads) : "memory");
    amax = warp_max[grp][0];
#pragma unroll
    for (int i = 1; i < kWarps; ++i) amax = max_abs_nan(amax, warp_max[grp][i]);
  }
  if (row_ok && !(amax < __int_as_float(0x7f800000)) && t == 0 && status != nullptr)
    atomicOr(status, BFP8_STATUS_NONFINITE_INPUT);
  const float s = __fdiv_rn(amax == 0.0f ? 1.0f : amax, 448.0f);
  const float rcp = __frcp_rn(s);
  if (row_ok && t == 0) scales[row] = native_half ? __fmul_rn(s, 2.0f) : s;
#pragma unroll
  for (int u = 0; u < kTokGroupVecs; ++u) {
    const int i = u * kRowThreads + t;
    const uint32_t* r = reinterpret_cast<const uint32_t*>(&raw[u]);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { f[2 * j] = bf16_lo_to_float(r[j]); f[2 * j + 1] = bf16_hi_to_float(r[j]); }
    uint2 q;
    if (native_half) {
      q.x = quant_half_e4m3x4(f[0], f[1], f[2], f[3], s, rcp);
      q.y = quant_half_e4m3x4(f[4], f[5], f[6], f[7], s, rcp);
    } else {
      q.x = quant_e4m3x4(f[0], f[1], f[2], f[3], s, rcp);
      q.y = quant_e4m3x4(f[4], f[5], f[6], f[7], s, rcp);
    }
    if (i < nvec) __stcs(crow + i, q);
  }
}

// ---------------------------------------------------------------------------------------------
// K4  decode: value(code) * block scale.  A thread turns 4 codes (one 32-bit load) into one
//     16-byte (fp32) or 8-byte (bf16) store, so both sides of every warp access are contiguous.
// ---------------------------------------------------------------------------------------------
constexpr int kDecodeThreads = 256;
constexpr int kDecodePer = 4;          // quads per thread

template <bool kVec, bool kBf16, typename Idx>
__global__ void __launch_bounds__(kDecodeThreads)
decode_block128_kernel(const uint8_t* __restrict__ codes, int64_t rows, int64_t cols, int64_t ld,
                       const float* __restrict__ scales, int col_blocks, void* __restrict__ out,
                       int64_t ld_out) {
  // Idx is 32-bit whenever rows * ceil(cols/4) fits, which keeps the row/column split cheap.
  // A thread decodes kDecodePer quads, one grid-stride apart, and issues all of their loads (codes and scale)
  // before the first use: with one quad per thread the kernel sat on the latency of its two 4-byte loads.
  const Idx quads_per_row = static_cast<Idx>((cols + 3) >> 2);
  const Idx total = static_cast<Idx>(rows) * quads_per_row;
  const Idx stride = static_cast<Idx>(gridDim.x) * blockDim.x;
  const Idx first = static_cast<Idx>(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t r[kDecodePer], c[kDecodePer];
  uint32_t q[kDecodePer];
  float s[kDecodePer];
  bool on[kDecodePer];
#pragma unroll
  for (int u = 0; u < kDecodePer; ++u) {
    const Idx i = first + static_cast<Idx>(u) * stride;
    on[u] = i < total;
    r[u] = 0; c[u] = 0; q[u] = 0; s[u] = 0.0f;
    if (on[u]) {
      r[u] = i / quads_per_row;
      c[u] = static_cast<int64_t>(i % quads_per_row) << 2;
      s[u] = __ldg(scales + (r[u] >> 7) * col_blocks + (c[u] >> 7));
      const uint8_t* p = codes + r[u] * ld + c[u];
      if (kVec) {
        q[u] = __ldcs(reinterpret_cast<const uint32_t*>(p));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (c[u] + j < cols) q[u] |= static_cast<uint32_t>(p[j]) << (8 * j);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kDecodePer; ++u) {
    if (!on[u]) continue;
    const float2 lo = e4m3x2_to_float2(q[u] & 0xffffu), hi = e4m3x2_to_float2(q[u] >> 16);
    const float v0 = __fmul_rn(lo.x, s[u]), v1 = __fmul_rn(lo.y, s[u]), v2 = __fmul_rn(hi.x, s[u]), v3 = __fmul_rn(hi.y, s[u]);
    if (kBf16) {
      uint16_t* o = reinterpret_cast<uint16_t*>(out) + r[u] * ld_out + c[u];
      if (kVec) {
        __stcs(reinterpret_cast<uint2*>(o), make_uint2(pack_bf16x2(v0, v1), pack_bf16x2(v2, v3)));
      } else {
        const float v[4] = {v0, v1, v2, v3};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (c[u] + j < cols) o[j] = static_cast<uint16_t>(float_to_bf16_bits(v[j]));
      }
    } else {
      float* o = reinterpret_cast<float*>(out) + r[u] * ld_out + c[u];
      if (kVec) {
        __stcs(reinterpret_cast<float4*>(o), make_float4(v0, v1, v2, v3));
      } else {
        const float v[4] = {v0, v1, v2, v3};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (c[u] + j < cols) o[j] = v[j];
      }
    }
  }
}

}  // namespace bfp8

using namespace bfp8;

extern "C" int bfp8_version(void) { return 1; }

extern "C" int bfp8_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" const char* bfp8_error_string(int code) {
  switch (code) {
    case BFP8_OK: return "ok";
    case BFP8_ERR_NULL: return "null pointer";
    case BFP8_ERR_ALIGN: return "pointer or leading dimension is misaligned";
    case BFP8_ERR_SHAPE: return "size out of range";
    case BFP8_ERR_WORKSPACE: return "workspace too small";
    case BFP8_ERR_CUDA: return "CUDA call failed";
    case BFP8_ERR_UNSUPPORTED: return "not an sm_100 device, or a shape / configuration this entry point does not take";
    case BFP8_ERR_TOO_LARGE: return "problem exceeds the fixed scratch of the no-allocation entry point";
    default: return "unknown error";
  }
}

extern "C" int bfp8_reencode_half(const uint8_t* codes_in, uint8_t* codes_out, int64_t n,
                                  const float* scales_in, float* scales_out, int64_t n_scales,
                                  unsigned long long* rounded_dev, uint32_t* status_dev, void* stream) {
  if (!codes_in || !codes_out || !rounded_dev || !status_dev) return BFP8_ERR_NULL;
  if (n <= 0 || n_scales < 0) return BFP8_ERR_SHAPE;
  if (n_scales > 0 && (!scales_in || !scales_out)) return BFP8_ERR_NULL;
  if (!aligned(rounded_dev, 8) || !aligned(status_dev, 4)) return BFP8_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int vec_ok = aligned(codes_in, 16) && aligned(codes_out, 16);
  const int64_t per_cta = static_cast<int64_t>(kReencodeThreads) * kReencodeUnroll * 16;     // bytes
  const int64_t ctas = (n + per_cta - 1) / per_cta;
  if (ctas > 2147483647LL) return BFP8_ERR_SHAPE;
  const int grid = static_cast<int>(ctas);
  reencode_half_kernel<<<grid, kReencodeThreads, 0, st>>>(codes_in, codes_out, n, vec_ok, scales_in, scales_out, n_scales,
                                                          rounded_dev, status_dev);
  BFP8_CUDA_TRY(cudaGetLastError());
  return BFP8_OK;
}

extern "C" int bfp8_validate_e4m3(const uint8_t* codes, int64_t n, const float* scales, int64_t n_scales,
                                  uint32_t* status_dev, void* stream) {
  if (!codes || !status_dev) return BFP8_ERR_NULL;
  if (n <= 0 || n_scales < 0) return BFP8_ERR_SHAPE;
  if (n_scales > 0 && !scales) return BFP8_ERR_NULL;
  if (!aligned(status_dev, 4) || (scales && !aligned(scales, 4))) return BFP8_ERR_ALIGN;
  const int64_t want = ((n >> 4) + 255) / 256 + 1, cap = static_cast<int64_t>(sm_count()) * 8;
  validate_e4m3_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      codes, n, aligned(codes, 16) ? 1 : 0, scales, n_scales, status_dev);
  BFP8_CUDA_TRY(cudaGetLastError());
  return BFP8_OK;
}

extern "C" int bfp8_quant_block128_f32(const float* w, int64_t rows, int64_t cols, int64_t ld,
                                       uint8_t* codes, int64_t ld_codes, float* scales,
                                       int native_half, void* stream) {
  if (!w || !codes || !scales) return BFP8_ERR_NULL;
  if (rows <= 0 || cols <= 0 || ld < cols || ld_codes < cols) return BFP8_ERR_SHAPE;
  const int64_t rb = (rows + 127) / 128, cb = (cols + 127) / 128;
  if (rb > 65535 || cb > 2147483647LL) return BFP8_ERR_SHAPE;
  if (!aligned(w, 4) || !aligned(scales, 4)) return BFP8_ERR_ALIGN;
  const bool vec = aligned(w, 16) && aligned(codes, 4) && ld % 4 == 0 && ld_codes % 4 == 0 && cols % 4 == 0;
  dim3 grid(static_cast<unsigned>(cb), static_cast<unsigned>(rb));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (vec)
    quant_block128_kernel<true><<<grid, kQuantThreads, 0, st>>>(w, rows, cols, ld, codes, ld_codes, scales,
                                                                static_cast<int>(cb), native_half);
  else
    quant_block128_kernel<false><<<grid, kQuantThreads, 0, st>>>(w, rows, cols, ld, codes, ld_codes, scales,
                                                                 static_cast<int>(cb), native_half);
  BFP8_CUDA_TRY(cudaGetLastError());
  return BFP8_OK;
}

extern "C" int bfp8_quant_act_1x128_bf16(const uint16_t* x, int64_t m, int64_t k, int64_t ldx,
                                         uint8_t* codes, int64_t ld_codes,
                                         float* scales, int64_t scale_stride_m, int64_t scale_stride_g,
                                         int native_half, uint32_t* status_dev, void* stream) {
  if (!x || !codes || !scales) return BFP8_ERR_NULL;
  if (m <= 0 || k <= 0 || ldx < k || ld_codes < k || scale_stride_m <= 0 || scale_stride_g <= 0)
    return BFP8_ERR_SHAPE;
  if (!aligned(x, 2) || !aligned(scales, 4)) return BFP8_ERR_ALIGN;
  const int64_t groups = (k + 127) / 128;
  if (groups > (1 << 24)) return BFP8_ERR_SHAPE;
  const bool vec = aligned(x, 16) && aligned(codes, 8) && ldx % 8 == 0 && ld_codes % 8 == 0 && k % 8 == 0;
  const int rows_per_cta = groups >= kActSlots ? 1 : static_cast<int>(kActSlots / groups);
  const int64_t want = (m + rows_per_cta - 1) / rows_per_cta;           // one CTA per row (or per 64 / groups rows)
  if (want > 2147483647LL) return BFP8_ERR_SHAPE;
  const int grid = static_cast<int>(want);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int passes = static_cast<int>((groups + kActSlots - 1) / kActSlots);
  const int split = (want < 2LL * sm_count() && passes <= 65535) ? passes : 1;      // few rows: one pass per CTA
  return launch_overlapped(vec ? quant_act_1x128_kernel<true, false> : quant_act_1x128_kernel<false, false>,
                           dim3(grid, split, want < 2LL * sm_count() ? kActPer : 1), dim3(kActThreads), 0, st, x, m, k, ldx,
                           codes, ld_codes, scales,
                           scale_stride_m, scale_stride_g, static_cast<int>(groups), native_half, status_dev,
                           split > 1 ? 1 : passes);
}

extern "C" int bfp8_silu_quant_act_1x128_bf16(const uint16_t* gate_up, int64_t m, int64_t inter, int64_t ld_in,
                                              uint8_t* codes, int64_t ld_codes,
                                              float* scales, int64_t scale_stride_m, int64_t scale_stride_g,
                                              int native_half, uint32_t* status_dev, void* stream) {
  if (!gate_up || !codes || !scales) return BFP8_ERR_NULL;
  if (m <= 0 || inter <= 0 || ld_in < 2 * inter || ld_codes < inter || scale_stride_m <= 0 || scale_stride_g <= 0)
    return BFP8_ERR_SHAPE;
  if (!aligned(gate_up, 2) || !aligned(scales, 4)) return BFP8_ERR_ALIGN;
  const int64_t groups = (inter + 127) / 128;
  if (groups > (1 << 24)) return BFP8_ERR_SHAPE;
  const bool vec = aligned(gate_up, 16) && aligned(codes, 8) && ld_in % 8 == 0 && ld_codes % 8 == 0 && inter % 8 == 0;
  const int rows_per_cta = groups >= kActSlots ? 1 : static_cast<int>(kActSlots / groups);
  const int64_t want = (m + rows_per_cta - 1) / rows_per_cta;
  if (want > 2147483647LL) return BFP8_ERR_SHAPE;
  const int passes = static_cast<int>((groups + kActSlots - 1) / kActSlots);
  const int split = (want < 2LL * sm_count() && passes <= 65535) ? passes : 1;
  return launch_overlapped(vec ? quant_act_1x128_kernel<true, true> : quant_act_1x128_kernel<false, true>,
                           dim3(static_cast<unsigned>(want), split, want < 2LL * sm_count() ? kActPer : 1), dim3(kActThreads), 0,
                           static_cast<cudaStream_t>(stream),
                           gate_up, m, inter, ld_in, codes, ld_codes, scales, scale_stride_m, scale_stride_g,
                           static_cast<int>(groups), native_half, status_dev, split > 1 ? 1 : passes);
}

extern "C" int bfp8_decode_block128(const uint8_t* codes, int64_t rows, int64_t cols, int64_t ld,
                                    const float* scales, void* out, int out_dtype, int64_t ld_out,
                                    void* stream) {
  if (!codes || !scales || !out) return BFP8_ERR_NULL;
  if (rows <= 0 || cols <= 0 || ld < cols || ld_out < cols) return BFP8_ERR_SHAPE;
  if (out_dtype != BFP8_OUT_F32 && out_dtype != BFP8_OUT_BF16) return BFP8_ERR_SHAPE;
  const bool bf16 = out_dtype == BFP8_OUT_BF16;
  if (!aligned(out, bf16 ? 2 : 4) || !aligned(scales, 4)) return BFP8_ERR_ALIGN;
  const int cb = static_cast<int>((cols + 127) / 128);
  const bool vec = aligned(codes, 4) && ld % 4 == 0 && cols % 4 == 0 && ld_out % 4 == 0 &&
                   aligned(out, bf16 ? 8 : 16);
  const int64_t quads = rows * ((cols + 3) / 4);
  if ((quads + kDecodeThreads - 1) / kDecodeThreads > 2147483647LL) return BFP8_ERR_SHAPE;
  const int grid = static_cast<int>((quads + kDecodeThreads * kDecodePer - 1) / (kDecodeThreads * kDecodePer));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool small = rows * ((cols + 3) / 4) < (1LL << 30);
#define BFP8_LAUNCH_DECODE(V, B)                                                                            \
  do {                                                                                                      \
    if (small)                                                                                              \
      decode_block128_kernel<V, B, uint32_t><<<grid, kDecodeThreads, 0, st>>>(codes, rows, cols, ld, scales, cb, out, ld_out); \
    else                                                                                                    \
      decode_block128_kernel<V, B, int64_t><<<grid, kDecodeThreads, 0, st>>>(codes, rows, cols, ld, scales, cb, out, ld_out);  \
  } while (0)
  if (vec && bf16) BFP8_LAUNCH_DECODE(true, true);
  else if (vec) BFP8_LAUNCH_DECODE(true, false);
  else if (bf16) BFP8_LAUNCH_DECODE(false, true);
  else BFP8_LAUNCH_DECODE(false, false);
#undef BFP8_LAUNCH_DECODE
  BFP8_CUDA_TRY(cudaGetLastError());
  return BFP8_OK;
}

extern "C" int bfp8_quant_act_token_bf16(const uint16_t* x, int64_t m, int64_t k, int64_t ldx,
                                         uint8_t* codes, int64_t ld_codes, float* scales,
                                         int native_half, uint32_t* status_dev, void* stream) {
  if (!x || !codes || !scales) return BFP8_ERR_NULL;
  if (m <= 0 || k <= 0 || ldx < k || ld_codes < k || m > 2147483647LL) return BFP8_ERR_SHAPE;
  if (!aligned(x, 2) || !aligned(scales, 4)) return BFP8_ERR_ALIGN;
  const int vec = aligned(x, 16) && aligned(codes, 8) && ldx % 8 == 0 && ld_codes % 8 == 0 && k % 8 == 0;
  if (vec && k <= kTokGroupMaxK && m >= 4LL * sm_count()) {
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int vecs = static_cast<int>(k >> 3);
    if (vecs <= 32 * kTokGroupVecs)
      quant_act_token_group_kernel<32><<<static_cast<int>((m + 7) / 8), kTokGroupCta, 0, st>>>(
          x, m, k, ldx, codes, ld_codes, scales, native_half, status_dev);
    else if (vecs <= 64 * kTokGroupVecs)
      quant_act_token_group_kernel<64><<<static_cast<int>((m + 3) / 4), kTokGroupCta, 0, st>>>(
          x, m, k, ldx, codes, ld_codes, scales, native_half, status_dev);
    else if (vecs <= 128 * kTokGroupVecs)
      quant_act_token_group_kernel<128><<<static_cast<int>((m + 1) / 2), kTokGroupCta, 0, st>>>(
          x, m, k, ldx, codes, ld_codes, scales, native_half, status_dev);
    else
      quant_act_token_group_kernel<256><<<static_cast<int>(m), kTokGroupCta, 0, st>>>(
          x, m, k, ldx, codes, ld_codes, scales, native_half, status_dev);
  } else if (vec && k <= kTokWarpMaxK) {
    const int rows_per_cta = kTokWarpThreads / 32;
    quant_act_token_warp_kernel<<<static_cast<int>((m + rows_per_cta - 1) / rows_per_cta), kTokWarpThreads, 0,
                                  static_cast<cudaStream_t>(stream)>>>(x, m, k, ldx, codes, ld_codes, scales,
                                                                       native_half, status_dev);
  } else {
    quant_act_token_kernel<<<static_cast<int>(m), kTokThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        x, k, ldx, codes, ld_codes, scales, native_half, vec, status_dev);
  }
  BFP8_CUDA_TRY(cudaGetLastError());
  return BFP8_OK;
}
