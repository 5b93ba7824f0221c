// Token/channel-scaled E4M3 GEMM for sm_100a: one fp32 scale per activation row and one per output
// channel, so the whole K range accumulates in TMEM and the scales are applied once per tile.
//
//   out[i, j] = (sum_k a(i, k) * w(j, k)) * a_scale[i] * w_scale[j] + bias[j]
//
// This is the per-token / per-channel FP8 variant of the reference (gk_fp8_token_quant_bf16_v1 feeding an
// MME GEMM, finished by gk_fp8_channel_finish_bf16_v1: csrc/tpc/block_fp8_framework/activation_token.c:4-26,
// channel_finish.c:2-18).  Same tile machinery as the block-scaled kernel - TMA (SWIZZLE_128B) -> shared
// memory -> tcgen05.mma kind::f8f6f4 -> TMEM - but without the per-K-block read-back: a 128 x 256 tile's
// MMAs accumulate over all of K into one of two 256-column TMEM buffers, and the epilogue warps drain the
// other buffer (scale, bias, bf16, TMA store) while the next tile's MMAs run.
//
// Warp roles (384 threads): warps 0-7 epilogue (two warpgroups of 128 columns each), warp 8 TMA producer,
// warp 9 TMEM owner + MMA issuer, warps 10-11 idle (setmaxnreg hands their registers to the epilogue).
// Persistent, one CTA per SM; every barrier wait is bounded and raises BFP8_STATUS_WAIT_TIMEOUT.
#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"

namespace bfp8 {


namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;
constexpr int kStages = 4;
constexpr int kEpiWarps = 8;
constexpr int kThreads = (kEpiWarps + 4) * 32;
constexpr int kTmemCols = 512;
constexpr int kABytes = BM * BK;
constexpr int kBBytes = BN * BK;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kOutWarpBytes = 32 * 64 * 2;
constexpr int kOutStageBytes = kEpiWarps * kOutWarpBytes;

struct SmemTail {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kOutStageBytes + sizeof(SmemTail);

struct Params {
  const float* a_scales;   // [M]
  const float* w_scales;   // [N]
  const float* bias;       // [N] or null
  void* out;
  int64_t ldo;
  int m, n, groups;
  int tiles_m, tiles_n;
  long long wait_limit;
  uint32_t* status;
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int kBand = 8;
  const int per_band = kBand * tiles_n;
  const int band = t / per_band;
  const int first = band * kBand;
  const int rows = min(kBand, tiles_m - first);
  const int r = t - band * per_band;
  tm = first + r % rows;
  tn = r / rows;
}

template <bool kOutBf16>
__global__ void __launch_bounds__(kThreads, 1)
gemm_channel_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_out, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  uint8_t* out_stage = smem + kStages * kStageBytes;
  SmemTail* tail = reinterpret_cast<SmemTail*>(out_stage + kOutStageBytes);
  volatile uint32_t* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int G = p.groups;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&tail->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&tail->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(ptx::smem_u32(&tail->tmem_full[b]), 1);
      ptx::mbar_init(ptx::smem_u32(&tail->tmem_empty[b]), kEpiWarps);
    }
    tail->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kEpiWarps + 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tail->tmem_base), kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == kEpiWarps && lane == 0) {
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_w);
    if (kOutBf16) ptx::prefetch_tensormap(&tmap_out);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;

  if (warp >= kEpiWarps) {
    ptx::setmaxnreg_dec<40>();
    if (warp == kEpiWarps) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
          int tm, tn;
          tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
          for (int g = 0; g < G; ++g) {
            ok = ptx::mbar_wait(ptx::smem_u32(&tail->empty[stage]), phase ^ 1u, abort_flag, p.wait_limit);
            if (!ok) break;
            const uint32_t full = ptx::smem_u32(&tail->full[stage]);
            const uint32_t a_dst = smem_base + stage * kStageBytes;
            ptx::mbar_arrive_expect_tx(full, kStageBytes);
            ptx::tma_load_2d(a_dst, &tmap_a, full, g * BK, tm * BM);
            ptx::tma_load_2d(a_dst + kABytes, &tmap_w, full, g * BK, tn * BN);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
      }
    } else if (warp == kEpiWarps + 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc = ptx::umma_idesc_e4m3(BM, BN);
        uint32_t stage = 0, phase = 0, it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
          const uint32_t buf = it & 1u, acc_phase = (it >> 1) & 1u;
          ok = ptx::mbar_wait(ptx::smem_u32(&tail->tmem_empty[buf]), acc_phase ^ 1u, abort_flag, p.wait_limit);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint32_t d = tmem_base + buf * BN;
          for (int g = 0; g < G; ++g) {
            ok = ptx::mbar_wait(ptx::smem_u32(&tail->full[stage]), phase, abort_flag, p.wait_limit);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t a_addr = smem_base + stage * kStageBytes;
            const uint64_t a_desc = ptx::umma_desc_k128(a_addr);
            const uint64_t b_desc = ptx::umma_desc_k128(a_addr + kABytes);
#pragma unroll
            for (int k4 = 0; k4 < BK / 32; ++k4)
              ptx::umma_f8(d, a_desc + 2u * k4, b_desc + 2u * k4, idesc, (g | k4) != 0);
            ptx::umma_commit(ptx::smem_u32(&tail->empty[stage]));
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          ptx::umma_commit(ptx::smem_u32(&tail->tmem_full[buf]));
        }
      }
    }
  } else {
    ptx::setmaxnreg_inc<232>();
    // ------------------------------------------------------------------ epilogue: once per tile
    const int wg = warp >> 2;
    const int quad = warp & 3;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    uint8_t* my_stage = out_stage + warp * kOutWarpBytes;
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int row0 = tm * BM + quad * 32;
      const int row = row0 + lane;
      const int col0 = tn * BN + wg * 128;
      const bool row_ok = row < p.m;
      const float act = row_ok ? __ldg(p.a_scales + row) : 0.0f;
      const uint32_t buf = it & 1u, acc_phase = (it >> 1) & 1u;
      // uniform across the warp: warp-collective TMEM loads follow
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&tail->tmem_full[buf]), acc_phase, abort_flag, p.wait_limit));
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + lane_addr + buf * BN + wg * 128;
      uint32_t ra[32], rb[32];
      ptx::tmem_ld32(taddr, ra);
      ptx::tmem_ld32(taddr + 32, rb);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        // chunk c = columns col0 + 32 c .. + 31, held in ra (even c) or rb (odd c)
        uint32_t (&r)[32] = (c & 1) ? rb : ra;
        if ((c & 1) == 0) {
          ptx::tmem_wait_ld32(ra);
          ptx::tmem_regs_ready32(rb);
        }
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = col0 + c * 32 + j;
          const float ws = col < p.n ? __ldg(p.w_scales + col) : 0.0f;
          const float b = (p.bias != nullptr && col < p.n) ? __ldg(p.bias + col) : 0.0f;
          // (partial * act_scale) * w_scale + bias, the order of channel_finish.c:12-14
          v[j] = fmaf(__uint_as_float(r[j]) * act, ws, b);
        }
        if (c == 1) {
          // second half of the buffer: fetch it into the registers just consumed
          ptx::tmem_ld32(taddr + 64, ra);
          ptx::tmem_ld32(taddr + 96, rb);
        }
        if (c == 3) {
          // every column of the buffer has been read: release it to the MMA warp
          ptx::tc_fence_before_sync();
          __syncwarp();
          ptx::mbar_arrive_lane0(ptx::smem_u32(&tail->tmem_empty[buf]), lane);
        }
        if (kOutBf16) {
          const int box = c >> 1;                        // one TMA box = 64 columns = two chunks
          const bool ragged = (p.n & 7) != 0 && col0 + box * 64 + 64 > p.n;
          if (ragged) {
            if (row_ok) {
              uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0 + c * 32;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + c * 32 + j < p.n) o[j] = static_cast<uint16_t>(float_to_bf16_bits(v[j]));
            }
          } else {
            if ((c & 1) == 0) {
              // the previous TMA store must have finished reading this warp's staging buffer
              if (lane == 0) ptx::tma_store_wait_read_all();
              __syncwarp();
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 q;
              q.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
              q.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
              q.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
              q.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
              const int chunk = (c & 1) * 4 + j;           // 16-byte chunk inside the 128-byte row
              *reinterpret_cast<uint4*>(my_stage + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = q;
            }
            if (c & 1) {
              ptx::fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                if (row0 < p.m && col0 + box * 64 < p.n)
                  ptx::tma_store_2d(&tmap_out, ptx::smem_u32(my_stage), col0 + box * 64, row0);
                ptx::tma_store_commit();
              }
            }
          }
        } else if (row_ok) {
          float* o = reinterpret_cast<float*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0 + c * 32;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + c * 32 + j < p.n) o[j] = v[j];
        }
      }
    }
    if (kOutBf16 && lane == 0) ptx::tma_store_wait_all();
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  ptx::idle_after_abort(abort_flag);
  if (warp == kEpiWarps + 1) ptx::tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && tail->abort_flag != 0) atomicOr(p.status, BFP8_STATUS_WAIT_TIMEOUT);
}

}  // namespace

int launch_gemm_channel(const uint8_t* a_codes, int64_t lda, const float* a_scales, const uint8_t* w_codes,
                        int64_t ldw, const float* w_scales, const float* bias, void* out, int out_dtype, int64_t ldo,
                        int64_t m, int64_t n, int64_t k, uint32_t* status_dev, long long wait_limit, int max_ctas,
                        cudaStream_t st) {
  alignas(64) CUtensorMap tmap_a, tmap_w, tmap_out;
  int rc = make_tensor_map_2d(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a_codes, k, m, lda, BK, BM);
  if (rc != BFP8_OK) return rc;
  rc = make_tensor_map_2d(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, w_codes, k, n, ldw, BK, BN);
  if (rc != BFP8_OK) return rc;
  const bool bf16 = out_dtype == BFP8_OUT_BF16;
  if (bf16) {
    rc = make_tensor_map_2d(&tmap_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, out, n, m, ldo * 2, 64, 32);
    if (rc != BFP8_OK) return rc;
  } else {
    tmap_out = tmap_a;   // unused on the fp32 path
  }
  Params p;
  p.a_scales = a_scales;
  p.w_scales = w_scales;
  p.bias = bias;
  p.out = out;
  p.ldo = ldo;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.groups = static_cast<int>((k + BK - 1) / BK);
  p.tiles_m = static_cast<int>((m + BM - 1) / BM);
  p.tiles_n = static_cast<int>((n + BN - 1) / BN);
  p.wait_limit = wait_limit;
  p.status = status_dev;
  const int tiles = p.tiles_m * p.tiles_n;
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  auto kern = bf16 ? gemm_channel_kernel<true> : gemm_channel_kernel<false>;
  static DeviceFlags done[2];
  rc = ensure_smem_limit(kern, kSmemBytes, done[bf16 ? 1 : 0]);
  if (rc != BFP8_OK) return rc;
  kern<<<grid, kThreads, kSmemBytes, st>>>(tmap_a, tmap_w, tmap_out, p);
  BFP8_CUDA_TRY(cudaGetLastError());
  return BFP8_OK;
}

}  // namespace bfp8
