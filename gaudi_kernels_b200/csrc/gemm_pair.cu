// Block-scaled E4M3 GEMM for sm_100a, CTA-pair schedule: two CTAs of a cluster share every MMA
// (tcgen05 cta_group::2) and work on one 256 x 256 output tile.
//
//   out[i, j] = sum_g sa[g, i] * sw[j/128, g] * ( A_g[i, :] . W_g[j, :] )      A_g, W_g: 128 codes wide
//
// Why pairs: the scale product changes with every 128-wide K block, so each block's partial product is
// accumulated from zero in TMEM, read back by the epilogue warps and folded into register
// accumulators.  An MMA's result becomes visible several hundred cycles after it was issued, so a TMEM
// buffer is busy for much longer than the MMA itself; keeping the tensor pipe fed therefore needs
// more than two buffers in flight.  A pair computes its tile as two column halves of 128: per SM
// that is four 128-column buffers (2 K blocks x 2 halves) in the 512 TMEM columns, each released
// after a single TMEM round trip.  The pair also halves the W traffic per SM: each CTA stages its own
// 128 A rows and only half of the W rows of either column half (32 KB per K block instead of 48 KB).
//
// Per CTA (384 threads): warps 0-7 epilogue (warp w reads TMEM lanes 32 (w%4)..; warpgroup w/4 owns
// columns 64 (w/4).. of each column half), warp 8 TMA producer, warp 9 TMEM owner and - in the pair's
// first CTA only - MMA issuer of the left column half for both CTAs, warp 10 MMA issuer of the right half,
// warp 11 idle (the third warpgroup's registers go to the epilogue).
// Barriers: the first CTA's `full` barriers collect the TMA bytes of both CTAs; tcgen05.commit is
// multicast to both CTAs' `empty` and `tmem_full` barriers; the epilogue warps of both CTAs arrive on
// the first CTA's `tmem_empty` barriers.  Every wait is bounded and raises BFP8_STATUS_WAIT_TIMEOUT.
#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"

namespace bfp8 {

namespace {

constexpr int BM = 256;            // pair tile rows (128 per CTA)
constexpr int BN = 256;            // pair tile columns, as two halves of 128
constexpr int BK = 128;
constexpr int kStages = 6;
constexpr int kEpiWarps = 8;
constexpr int kThreads = (kEpiWarps + 4) * 32;
constexpr int kTmemCols = 512;     // 2 K blocks x 2 column halves x 128 columns
constexpr int kABytes = 128 * BK;              // this CTA's A rows
constexpr int kWHalfBytes = 64 * BK;           // this CTA's share of one column half of W
constexpr int kStageBytes = kABytes + 2 * kWHalfBytes;      // 32 KB
constexpr int kOutWarpBytes = 32 * 64 * 2;
constexpr int kOutStageBytes = kEpiWarps * kOutWarpBytes;

struct SmemTail {
  uint64_t full[kStages];          // used in the pair's first CTA
  uint64_t empty[kStages];
  uint64_t tmem_full[4];           // index = (kblock & 1) * 2 + half
  uint64_t tmem_empty[4];          // used in the pair's first CTA; 16 arrivals (8 warps x 2 CTAs)
  uint32_t tmem_base;
  uint32_t abort_flag;
};

constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kOutStageBytes + sizeof(SmemTail);
static_assert(kSmemBytes <= 232448, "shared memory budget");

struct Params {
  const float* a_scales;   // [G, ldsa]
  const float* w_scales;   // [NB, G]
  const float* bias;
  void* out;
  int64_t ldsa, ldo;
  int m, n, groups;
  int tiles_m, tiles_n;
  long long wait_limit;
  uint32_t* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
  return r;
}
// TMA tile load whose completion bytes are counted on a barrier that may live in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive, once the MMAs issued so far have completed, on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
// The same from lane 0 only, as a predicated instruction (the warp does not branch; see ptx::mbar_arrive_lane0).
__device__ __forceinline__ void mbar_arrive_remote_lane0(uint32_t bar_cluster, int lane) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.s32 p, %1, 0;\n\t"
      "@p mbarrier.arrive.shared::cluster.b64 _, [%0];\n\t}"
      ::"r"(bar_cluster), "r"(lane) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  long long limit_cycles) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t polls = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++polls & 63u) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - t0 > limit_cycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

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

__device__ __forceinline__ void fma32(float2* acc, const uint32_t (&r)[32], float2 sv) {
#pragma unroll
  for (int j = 0; j < 16; ++j)
    acc[j] = __ffma2_rn(make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), sv, acc[j]);
}

template <bool kOutBf16>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                 const __grid_constant__ CUtensorMap tmap_out, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  uint8_t* out_stage = smem + kStages * kStageBytes;
  SmemTail* tail = reinterpret_cast<SmemTail*>(out_stage + kOutStageBytes);
  volatile uint32_t* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: issues the MMAs of the pair
  const int num_pairs = gridDim.x >> 1;
  const int pair = blockIdx.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int G = p.groups;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&tail->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&tail->empty[s]), 2);      // one commit per MMA issuer
    }
    for (int b = 0; b < 4; ++b) {
      ptx::mbar_init(ptx::smem_u32(&tail->tmem_full[b]), 1);
      ptx::mbar_init(ptx::smem_u32(&tail->tmem_empty[b]), 2 * kEpiWarps);
    }
    tail->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kEpiWarps + 1) {
    tmem_alloc_pair(ptx::smem_u32(&tail->tmem_base), kTmemCols);
    tmem_relinquish_pair();
  }
  if (warp == kEpiWarps && lane == 0) {
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_w);
    if (kOutBf16) ptx::prefetch_tensormap(&tmap_out);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                               // both CTAs' barriers exist before any remote arrival
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;

  if (warp >= kEpiWarps) {
    ptx::setmaxnreg_dec<40>();
    if (warp == kEpiWarps) {
      // ------------------------------------------------------------------ TMA producer (both CTAs)
      if (lane == 0) {
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
          int tm, tn;
          tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
          const int a_row = tm * BM + static_cast<int>(rank) * 128;
          const int w_row = tn * BN + static_cast<int>(rank) * 64;
          for (int g = 0; g < G; ++g) {
            ok = ptx::mbar_wait(ptx::smem_u32(&tail->empty[stage]), phase ^ 1u, abort_flag, p.wait_limit);
            if (!ok) break;
            const uint32_t full_local = ptx::smem_u32(&tail->full[stage]);
            const uint32_t full0 = map_to_cta(full_local, 0);
            const uint32_t dst = smem_base + stage * kStageBytes;
            if (rank == 0) ptx::mbar_arrive_expect_tx(full_local, 2 * kStageBytes);
            tma_load_2d_pair(dst, &tmap_a, full0, g * BK, a_row);
            tma_load_2d_pair(dst + kABytes, &tmap_w, full0, g * BK, w_row);
            tma_load_2d_pair(dst + kABytes + kWHalfBytes, &tmap_w, full0, g * BK, w_row + 128);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
      }
    } else if (warp == kEpiWarps + 1 || warp == kEpiWarps + 2) {
      // ------------------------------------------------------------------ MMA issuers (first CTA only)
      // One issuing thread per column half: their barrier polls and commits overlap, and the tensor
      // pipe always has work queued from the other half while one of them waits.
      if (lane == 0 && rank == 0) {
        const int half = warp - (kEpiWarps + 1);
        constexpr uint32_t idesc = ptx::umma_idesc_e4m3(256, 128);
        uint32_t stage = 0, phase = 0, kb = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
          for (int g = 0; g < G; ++g, ++kb) {
            const uint32_t buf = (kb & 1u) * 2 + half, acc_phase = (kb >> 1) & 1u;
            ok = mbar_wait_cluster(ptx::smem_u32(&tail->tmem_empty[buf]), acc_phase ^ 1u, abort_flag, p.wait_limit) &&
                 ptx::mbar_wait(ptx::smem_u32(&tail->full[stage]), phase, abort_flag, p.wait_limit);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t base = smem_base + stage * kStageBytes;
            const uint64_t a_desc = ptx::umma_desc_k128(base);
            const uint64_t b_desc = ptx::umma_desc_k128(base + kABytes + half * kWHalfBytes);
            const uint32_t d = tmem_base + buf * 128;
#pragma unroll
            for (int k4 = 0; k4 < BK / 32; ++k4)
              umma_f8_pair(d, a_desc + 2u * k4, b_desc + 2u * k4, idesc, k4 > 0);
            umma_commit_pair(ptx::smem_u32(&tail->tmem_full[buf]));
            umma_commit_pair(ptx::smem_u32(&tail->empty[stage]));     // second of two arrivals frees the stage
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else {
    ptx::setmaxnreg_inc<232>();
    // ------------------------------------------------------------------ epilogue / promotion
    const int wg = warp >> 2;                      // which 64 columns of each column half
    const int quad = warp & 3;                     // TMEM lane quarter this warp may read
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t col_addr = static_cast<uint32_t>(wg * 64);
    uint8_t* my_stage = out_stage + warp * kOutWarpBytes;
    uint32_t kb = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int row0 = tm * BM + static_cast<int>(rank) * 128 + quad * 32;
      const int row = row0 + lane;
      const int col_l = tn * BN + wg * 64;         // this thread's first column in the left half
      const bool row_ok = row < p.m;
      const bool live_l = row_ok && tn * BN < p.n, live_r = row_ok && tn * BN + 128 < p.n;
      const float* sa_ptr = p.a_scales + row;
      const float* swl_ptr = p.w_scales + static_cast<int64_t>(tn * 2) * G;
      const float* swr_ptr = swl_ptr + G;
      float2 acc[64];                              // [0,32): left half, [32,64): right half
#pragma unroll
      for (int j = 0; j < 64; ++j) acc[j] = make_float2(0.0f, 0.0f);
      // scales are fetched two K blocks ahead; products are formed only when used
      float sa0 = row_ok ? __ldg(sa_ptr) : 0.0f;
      float sl0 = live_l ? __ldg(swl_ptr) : 0.0f, sr0 = live_r ? __ldg(swr_ptr) : 0.0f;
      float sa1 = 0.0f, sl1 = 0.0f, sr1 = 0.0f;
      if (G > 1) {
        sa1 = row_ok ? __ldg(sa_ptr + p.ldsa) : 0.0f;
        sl1 = live_l ? __ldg(swl_ptr + 1) : 0.0f;
        sr1 = live_r ? __ldg(swr_ptr + 1) : 0.0f;
      }
      uint32_t ra[32], rb[32];
      {
        const uint32_t buf = (kb & 1u) * 2, acc_phase = (kb >> 1) & 1u;
        // wait outcomes are made uniform across the warp: warp-collective TMEM loads and __syncwarp follow them
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&tail->tmem_full[buf]), acc_phase, abort_flag, p.wait_limit));
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t taddr = tmem_base + lane_addr + buf * 128 + col_addr;
        ptx::tmem_ld32(taddr, ra);
        ptx::tmem_ld32(taddr + 32, rb);
      }
      for (int g = 0; g < G; ++g, ++kb) {
        float sa2 = 0.0f, sl2 = 0.0f, sr2 = 0.0f;
        if (g + 2 < G) {
          sa2 = row_ok ? __ldg(sa_ptr + static_cast<int64_t>(g + 2) * p.ldsa) : 0.0f;
          sl2 = live_l ? __ldg(swl_ptr + g + 2) : 0.0f;
          sr2 = live_r ? __ldg(swr_ptr + g + 2) : 0.0f;
        }
        const uint32_t acc_phase = (kb >> 1) & 1u;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          // invariant: the 64 columns of (kb, half) are in flight into ra / rb
          const uint32_t buf = (kb & 1u) * 2 + half;
          const float s = sa0 * (half == 0 ? sl0 : sr0);
          const float2 sv = make_float2(s, s);
          ptx::tmem_wait_ld32(ra);
          ptx::tmem_regs_ready32(rb);
          // all of this thread's columns of the buffer are in registers: release it to the MMA issuer
          ptx::tc_fence_before_sync();
          __syncwarp();
          mbar_arrive_remote_lane0(map_to_cta(ptx::smem_u32(&tail->tmem_empty[buf]), 0), lane);
          fma32(acc + half * 32, ra, sv);
          // next buffer in program order: the right half of this K block, or the left half of the next
          const bool has_next = (half == 0) || (g + 1 < G);
          uint32_t naddr = 0;
          if (has_next) {
            const uint32_t nkb = half == 0 ? kb : kb + 1;
            const uint32_t nbuf = (nkb & 1u) * 2 + (half ^ 1);
            const uint32_t nphase = (nkb >> 1) & 1u;
            ok = __all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&tail->tmem_full[nbuf]), nphase, abort_flag, p.wait_limit));
            if (!ok) break;
            ptx::tc_fence_after_sync();
            naddr = tmem_base + lane_addr + nbuf * 128 + col_addr;
            ptx::tmem_ld32(naddr, ra);
          }
          fma32(acc + half * 32 + 16, rb, sv);
          if (has_next) ptx::tmem_ld32(naddr + 32, rb);
        }
        if (!ok) break;
        (void)acc_phase;
        sa0 = sa1; sl0 = sl1; sr0 = sr1;
        sa1 = sa2; sl1 = sl2; sr1 = sr2;
      }
      if (!ok) break;
      // ---- tile done: bias, rounding, store.  acc[half * 32 + j] holds columns col_l + half * 128 + 2j, 2j + 1
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int col0 = col_l + half * 128;
        float2* a = acc + half * 32;
        if (p.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col0 + 2 * j < p.n) a[j].x += __ldg(p.bias + col0 + 2 * j);
            if (col0 + 2 * j + 1 < p.n) a[j].y += __ldg(p.bias + col0 + 2 * j + 1);
          }
        }
        if (kOutBf16 && (p.n & 7) != 0 && col0 + 64 > p.n) {
          // ragged right edge that is not 16-byte granular: guarded element stores
          if (row_ok && col0 < p.n)
            store_row_bf16_guarded(reinterpret_cast<uint16_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0, a,
                                   p.n - col0);
        } else if (kOutBf16) {
          // one box: 32 rows x 64 bf16 (128 B per row), 16-byte chunks XOR-swizzled by row & 7
          if (lane == 0) ptx::tma_store_wait_read_all();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 v;
            v.x = pack_bf16x2(a[4 * j + 0].x, a[4 * j + 0].y);
            v.y = pack_bf16x2(a[4 * j + 1].x, a[4 * j + 1].y);
            v.z = pack_bf16x2(a[4 * j + 2].x, a[4 * j + 2].y);
            v.w = pack_bf16x2(a[4 * j + 3].x, a[4 * j + 3].y);
            *reinterpret_cast<uint4*>(my_stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (row0 < p.m && col0 < p.n) ptx::tma_store_2d(&tmap_out, ptx::smem_u32(my_stage), col0, row0);
            ptx::tma_store_commit();
          }
        } else if (row_ok) {
          float* o = reinterpret_cast<float*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col0 + 2 * j < p.n) o[2 * j] = a[j].x;
            if (col0 + 2 * j + 1 < p.n) o[2 * j + 1] = a[j].y;
          }
        }
      }
    }
    if (kOutBf16 && lane == 0) ptx::tma_store_wait_all();
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                               // the peer may still read this CTA's shared memory or barriers
  ptx::tc_fence_after_sync();
  ptx::idle_after_abort(abort_flag);
  if (warp == kEpiWarps + 1) tmem_dealloc_pair(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && tail->abort_flag != 0) atomicOr(p.status, BFP8_STATUS_WAIT_TIMEOUT);
}

}  // namespace

int launch_gemm_pair(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                     const uint8_t* w_codes, int64_t ldw, const float* w_scales, const float* bias, void* out,
                     int out_dtype, int64_t ldo, int64_t m, int64_t n, int64_t k, uint32_t* status_dev,
                     long long wait_limit, int max_ctas, cudaStream_t st) {
  alignas(64) CUtensorMap tmap_a, tmap_w, tmap_out;
  int rc = make_tensor_map_2d(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a_codes, k, m, lda, BK, 128);
  if (rc != BFP8_OK) return rc;
  rc = make_tensor_map_2d(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, w_codes, k, n, ldw, BK, 64);
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
  p.ldsa = ldsa;
  p.ldo = ldo;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.groups = static_cast<int>((k + BK - 1) / BK);
  p.tiles_m = static_cast<int>((m + BM - 1) / BM);
  p.tiles_n = static_cast<int>((n + BN - 1) / BN);
  p.wait_limit = wait_limit;
  p.status = status_dev;
  const int tiles = p.tiles_m * p.tiles_n;
  int pairs = sm_count() / 2;
  if (max_ctas > 1 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  if (tiles < pairs) pairs = tiles;
  auto kern = bf16 ? gemm_pair_kernel<true> : gemm_pair_kernel<false>;
  static DeviceFlags done[2];
  rc = ensure_smem_limit(kern, kSmemBytes, done[bf16 ? 1 : 0]);
  if (rc != BFP8_OK) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(pairs * 2), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  BFP8_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tmap_a, tmap_w, tmap_out, p));
  return BFP8_OK;
}

}  // namespace bfp8
