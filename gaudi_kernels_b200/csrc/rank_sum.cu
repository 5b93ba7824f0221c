// Rank-order sum of per-rank partial results, and the peer-memory plumbing of the K-sharded GEMM.
//
// gk_rank_sum_{bf16,f32}_v1 (csrc/tpc/generic_dense/rank_sum.c:4-42) adds `world_size` slices of `elems`
// values in canonical rank order with fp32 accumulation: acc = slice 0, then acc += slice r for r = 1 .. W-1,
// one rounding to bf16 at the end for bf16 data.  On Gaudi2 the slices were gathered into one local buffer
// by the runtime first; here the same kernel takes one pointer per slice, so a slice may just as well live in
// another GPU's memory (plain peer loads over NVLink, no multicast) and the gather disappears: every rank
// reads its share of every rank's partial exactly once and writes the sum.
#include <string.h>

#include "common.cuh"

namespace bfp8 {

namespace {

constexpr int kMaxWorld = 8;               // generic_dense_glue.cpp:576 accepts 2 .. 8 ranks
constexpr int kRankSumThreads = 256;

struct SlicePtrs {
  const void* p[kMaxWorld];
};

template <bool kBf16>
__global__ void __launch_bounds__(kRankSumThreads)
rank_sum_kernel(const SlicePtrs slices, int world, void* __restrict__ dst, int64_t elems,
                const float* __restrict__ bias, int64_t bias_period, int vec_ok) {
  constexpr int kPerVec = kBf16 ? 8 : 4;                         // elements per 16-byte vector
  const int64_t nvec = vec_ok ? elems / kPerVec : 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kRankSumThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kRankSumThreads + threadIdx.x; i < nvec; i += stride) {
    uint4 v[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      if (r < world) v[r] = __ldcs(reinterpret_cast<const uint4*>(slices.p[r]) + i);    // all loads before the first add
    float acc[8];
    if (kBf16) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&v[0]);
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[2 * j] = bf16_lo_to_float(w[j]); acc[2 * j + 1] = bf16_hi_to_float(w[j]); }
#pragma unroll
      for (int r = 1; r < kMaxWorld; ++r) {
        if (r < world) {
          const uint32_t* x = reinterpret_cast<const uint32_t*>(&v[r]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] = __fadd_rn(acc[2 * j], bf16_lo_to_float(x[j]));
            acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], bf16_hi_to_float(x[j]));
          }
        }
      }
    } else {
      const float* w = reinterpret_cast<const float*>(&v[0]);
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] = w[j];
#pragma unroll
      for (int r = 1; r < kMaxWorld; ++r) {
        if (r < world) {
          const float* x = reinterpret_cast<const float*>(&v[r]);
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[j] = __fadd_rn(acc[j], x[j]);
        }
      }
    }
    if (bias != nullptr) {
      const int64_t c0 = (i * kPerVec) % bias_period;            // bias_period is a multiple of kPerVec on this path
#pragma unroll
      for (int j = 0; j < kPerVec; ++j) acc[j] = __fadd_rn(acc[j], __ldg(bias + c0 + j));
    }
    if (kBf16) {
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      __stcs(reinterpret_cast<uint4*>(dst) + i, o);
    } else {
      __stcs(reinterpret_cast<uint4*>(dst) + i, make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]),
                                                           __float_as_uint(acc[2]), __float_as_uint(acc[3])));
    }
  }
  // unaligned buffers and the ragged tail, one element at a time
  for (int64_t i = nvec * kPerVec + static_cast<int64_t>(blockIdx.x) * kRankSumThreads + threadIdx.x; i < elems;
       i += stride) {
    float acc;
    if (kBf16) {
      acc = bf16_bits_to_float(reinterpret_cast<const uint16_t*>(slices.p[0])[i]);
      for (int r = 1; r < world; ++r)
        acc = __fadd_rn(acc, bf16_bits_to_float(reinterpret_cast<const uint16_t*>(slices.p[r])[i]));
    } else {
      acc = reinterpret_cast<const float*>(slices.p[0])[i];
      for (int r = 1; r < world; ++r) acc = __fadd_rn(acc, reinterpret_cast<const float*>(slices.p[r])[i]);
    }
    if (bias != nullptr) acc = __fadd_rn(acc, __ldg(bias + i % bias_period));
    if (kBf16)
      reinterpret_cast<uint16_t*>(dst)[i] = static_cast<uint16_t>(float_to_bf16_bits(acc));
    else
      reinterpret_cast<float*>(dst)[i] = acc;
  }
}

int rank_sum_launch(const SlicePtrs& s, int world, void* dst, int64_t elems, int dtype, const float* bias,
                    int64_t bias_period, cudaStream_t st) {
  const bool bf16 = dtype == BFP8_OUT_BF16;
  const int per_vec = bf16 ? 8 : 4;
  bool vec = aligned(dst, 16) && (bias == nullptr || (bias_period % per_vec == 0 && aligned(bias, 4)));
  for (int r = 0; r < world; ++r) vec = vec && aligned(s.p[r], 16);
  const int64_t work = (elems / per_vec + kRankSumThreads - 1) / kRankSumThreads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int grid = static_cast<int>(work < 1 ? 1 : (work < cap ? work : cap));
  if (bf16)
    rank_sum_kernel<true><<<grid, kRankSumThreads, 0, st>>>(s, world, dst, elems, bias, bias_period, vec ? 1 : 0);
  else
    rank_sum_kernel<false><<<grid, kRankSumThreads, 0, st>>>(s, world, dst, elems, bias, bias_period, vec ? 1 : 0);
  BFP8_CUDA_TRY(cudaGetLastError());
  return BFP8_OK;
}

// One warp: lane r < world tells rank r "this rank has reached epoch e" by writing e into slot [my rank] of
// rank r's flag array, then waits - bounded - until slot [r] of this rank's own array holds at least e.
// Everything this stream did before the barrier (the partial results other ranks are about to read) is
// ordered before the flag by the system-scope fence.
struct FlagPtrs {
  uint32_t* p[kMaxWorld];
};

__global__ void peer_barrier_kernel(const FlagPtrs flags, int rank, int world, uint32_t epoch, long long wait_limit,
                                    uint32_t* __restrict__ status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  volatile uint32_t* theirs = flags.p[r] + rank;
  *theirs = epoch;
  __threadfence_system();
  volatile uint32_t* mine = flags.p[rank] + r;
  const long long t0 = clock64();
  // epochs grow monotonically; the signed difference also survives a wrap of the 32-bit counter
  while (static_cast<int32_t>(*mine - epoch) < 0) {
    if (clock64() - t0 > wait_limit) {
      atomicOr(status, BFP8_STATUS_WAIT_TIMEOUT);
      return;
    }
    __nanosleep(64);
  }
  __threadfence_system();
}

}  // namespace
}  // namespace bfp8

using namespace bfp8;

extern "C" int bfp8_rank_sum(const void* gathered, void* dst, int64_t elems, int world_size, int dtype, void* stream) {
  if (!gathered || !dst) return BFP8_ERR_NULL;
  if (world_size < 2 || world_size > kMaxWorld) return BFP8_ERR_UNSUPPORTED;
  if (elems <= 0 || elems > 2147483647LL / world_size) return BFP8_ERR_SHAPE;
  if (dtype != BFP8_OUT_F32 && dtype != BFP8_OUT_BF16) return BFP8_ERR_SHAPE;
  const size_t esz = dtype == BFP8_OUT_BF16 ? 2 : 4;
  if (!aligned(gathered, esz) || !aligned(dst, esz)) return BFP8_ERR_ALIGN;
  SlicePtrs s = {};
  for (int r = 0; r < world_size; ++r) s.p[r] = static_cast<const uint8_t*>(gathered) + static_cast<size_t>(r) * elems * esz;
  return rank_sum_launch(s, world_size, dst, elems, dtype, nullptr, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int bfp8_rank_sum_slices(const void* const* slices, void* dst, int64_t elems, int world_size, int dtype,
                                    const float* bias, int64_t bias_period, void* stream) {
  if (!slices || !dst) return BFP8_ERR_NULL;
  if (world_size < 2 || world_size > kMaxWorld) return BFP8_ERR_UNSUPPORTED;
  if (elems <= 0) return BFP8_ERR_SHAPE;
  if (dtype != BFP8_OUT_F32 && dtype != BFP8_OUT_BF16) return BFP8_ERR_SHAPE;
  if (bias != nullptr && bias_period <= 0) return BFP8_ERR_SHAPE;
  const size_t esz = dtype == BFP8_OUT_BF16 ? 2 : 4;
  SlicePtrs s = {};
  for (int r = 0; r < world_size; ++r) {
    if (!slices[r]) return BFP8_ERR_NULL;
    if (!aligned(slices[r], esz)) return BFP8_ERR_ALIGN;
    s.p[r] = slices[r];
  }
  if (!aligned(dst, esz)) return BFP8_ERR_ALIGN;
  return rank_sum_launch(s, world_size, dst, elems, dtype, bias, bias ? bias_period : 1, static_cast<cudaStream_t>(stream));
}

extern "C" int bfp8_peer_alloc(size_t bytes, void** ptr) {
  if (!ptr) return BFP8_ERR_NULL;
  if (bytes == 0) return BFP8_ERR_SHAPE;
  void* p = nullptr;
  BFP8_CUDA_TRY(cudaMalloc(&p, bytes));
  const cudaError_t e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e);
  }
  *ptr = p;
  return BFP8_OK;
}

extern "C" int bfp8_peer_free(void* ptr) {
  if (!ptr) return BFP8_ERR_NULL;
  BFP8_CUDA_TRY(cudaFree(ptr));
  return BFP8_OK;
}

extern "C" int bfp8_peer_export(void* ptr, uint8_t handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
  if (!ptr || !handle) return BFP8_ERR_NULL;
  cudaIpcMemHandle_t h;
  BFP8_CUDA_TRY(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle, &h, sizeof(h));
  return BFP8_OK;
}

extern "C" int bfp8_peer_open(const uint8_t handle[64], void** ptr) {
  if (!handle || !ptr) return BFP8_ERR_NULL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  BFP8_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = p;
  return BFP8_OK;
}

extern "C" int bfp8_peer_close(void* ptr) {
  if (!ptr) return BFP8_ERR_NULL;
  BFP8_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return BFP8_OK;
}

extern "C" int bfp8_peer_barrier(uint32_t* const* flags, int rank, int world_size, uint32_t epoch,
                                 int64_t wait_limit_cycles, uint32_t* status_dev, void* stream) {
  if (!flags || !status_dev) return BFP8_ERR_NULL;
  if (world_size < 1 || world_size > kMaxWorld || rank < 0 || rank >= world_size) return BFP8_ERR_SHAPE;
  FlagPtrs f = {};
  for (int r = 0; r < world_size; ++r) {
    if (!flags[r]) return BFP8_ERR_NULL;
    if (!aligned(flags[r], 4)) return BFP8_ERR_ALIGN;
    f.p[r] = flags[r];
  }
  const long long limit = wait_limit_cycles > 0 ? wait_limit_cycles : 4000000000LL;     // about two seconds
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, rank, world_size, epoch, limit, status_dev);
  BFP8_CUDA_TRY(cudaGetLastError());
  return BFP8_OK;
}
