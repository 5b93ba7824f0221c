// Block-scaled E4M3 GEMM for sm_100a, CTA-pair schedule: two CTAs of a cluster share every MMA
// (tcgen05 cta_group::2, M = 256) and work on one 256 x 128 output tile, 128 rows in each CTA.
//
//   out[i, j] = sum_g sa[g, i] * sw[j/128, g] * ( A_g[i, :] . W_g[j, :] )      A_g, W_g: 128 codes wide
//
// Why pairs, and why this tile.  The scale product changes with every 128-wide K block, so each block's
// partial product is accumulated from zero in TMEM, read back by the epilogue warps and folded into
// register accumulators.  Between the end of a block's MMAs and the moment its TMEM buffer can be
// written again lie several hundred cycles of latency (completion becoming visible, the TMEM read,
// the hand-back reaching the issuing thread), far more than the 256 cycles the MMAs of one block take,
// so the tensor pipe only stays busy with several buffers in flight.  A tile of 128 columns needs 128
// TMEM columns per K block: four buffers fit in the 512 columns.  A 128-column MMA of a single CTA is
// bound by its shared-memory operand reads (about 74 cycles instead of 64); in a pair each CTA reads
// only half of the W tile and the same MMA runs at the full rate, and W crosses L2 -> shared memory once
// per pair instead of once per CTA.  With 64 accumulator columns per thread there are registers for two
// staging sets, so the TMEM loads of block g + 1 are in flight while block g is folded, and a buffer is
// released right after a single load round.
//
// Per CTA (384 threads): warps 0-7 epilogue (warp w reads TMEM lanes 32 (w % 4).., columns 64 (w / 4)..
// of every buffer), warp 8 TMA producer, warp 9 TMEM owner, and - in the pair's first CTA only - warps 9-11 MMA
// issuers that take the K blocks in turn for both CTAs (the third warpgroup's registers go to the epilogue
// through setmaxnreg).
//
// Barriers, indexed by the running K block number kb of the pair: `full[kb % 8]` (first CTA) completes when
// the stage's TMA bytes of both CTAs have landed AND the sixteen epilogue warps of the pair have drained
// TMEM buffer kb % 4 of K block kb - 4, so the issuer makes one wait per K block; `done[kb % 8]` (both CTAs,
// through one multicast tcgen05.commit) tells the epilogue that buffer kb % 4 is readable and the producer
// that stage kb % 8 is free.  No TMA load is multicast.  Every wait is bounded and raises
// BFP8_STATUS_WAIT_TIMEOUT; the outcome of a wait is made uniform across the warp before any warp-collective
// instruction follows it.
#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"

#ifdef EXP_NOFMA
#define EXP_FMA(x)
#else
#define EXP_FMA(x) x
#endif
#ifdef EXP_NOHANDBACK
#define EXP_HB(x) (void)0
#else
#define EXP_HB(x) x
#endif
#ifdef EXP_FMA_FIRST
#define EXP_FMAFIRST(x) x
#define EXP_NOFMA
#else
#define EXP_FMAFIRST(x)
#endif
#ifdef EXP_HALFFMA
#define EXP_FMA2(x)
#else
#define EXP_FMA2(x) EXP_FMA(x)
#endif
#ifdef EXP_NOSCALE
#define EXP_SCALE_LINES(slot) const float2 sv = make_float2(1.5f, 1.5f);
#else
#define EXP_SCALE_LINES(slot) const float s = sa_q[slot] * sw_q[slot]; const float2 sv = make_float2(s, s); pf_fetch(sa_q[slot], sw_q[slot]);
#endif
#ifdef EXP_NOLD
#define EXP_LD(x)
#else
#define EXP_LD(x) x
#endif
#ifdef EXP_TRACE
__device__ long long g_trace[6 * 512];
#define TRACE(slot, kbv) do { if (blockIdx.x == 0 && (kbv) < 512u) g_trace[(slot) * 512 + (kbv)] = clock64(); } while (0)
extern "C" int bfp8_exp_trace(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_trace, sizeof(g_trace));
}
#else
#define TRACE(slot, kbv) do {} while (0)
#endif
#ifdef EXP_DELTA
__device__ long long g_delta[8 * 16];
extern "C" int bfp8_exp_delta(long long* host_out) { return (int)cudaMemcpyFromSymbol(host_out, g_delta, sizeof(g_delta)); }
#define DSTAMP(i) { const long long now_ = clock64(); dsum[i] += now_ - dlast; dlast = now_; }
#else
#define DSTAMP(i)
#endif
namespace bfp8 {

int make_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

namespace {

constexpr int BM = 256;            // pair tile rows (128 per CTA)
constexpr int BN = 128;            // pair tile columns = one weight scale block
constexpr int BK = 128;
#ifndef EXP_STAGES
#define EXP_STAGES 8
#endif
constexpr int kStages = EXP_STAGES;         // shared-memory stages; also the length of both barrier rings
constexpr int kBufs = 4;           // TMEM accumulator buffers of BN columns
constexpr int kEpiWarps = 8;
constexpr int kScaleAhead = 4;      // K blocks between the request of a scale pair and its use
constexpr int kIssuers = 3;         // MMA-issuing warps (warps 9 .. 11)
constexpr int kThreads = (kEpiWarps + 8) * 32;   // warps 8 and 12 TMA producers, 9-11 MMA issuers, 13-15 idle
constexpr int kTmemCols = kBufs * BN;
constexpr int kABytes = 128 * BK;              // this CTA's A rows
constexpr int kWBytes = (BN / 2) * BK;         // this CTA's half of the W tile
constexpr int kStageBytes = kABytes + kWBytes; // 24 KB
constexpr int kOutWarpBytes = 32 * 64 * 2;     // per warp: one box of 32 rows x 64 bf16
constexpr int kOutStageBytes = kEpiWarps * kOutWarpBytes;

struct SmemTail {
  uint64_t full[kStages];          // used in the pair's first CTA: 1 producer arrival + TMA bytes of both CTAs + 16 warps
  uint64_t done[kStages];          // both CTAs: MMAs of K block kb complete
  uint32_t tmem_base;
  uint32_t abort_flag;
};

constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kOutStageBytes + sizeof(SmemTail);
static_assert(kSmemBytes <= 232448, "shared memory budget");
static_assert((kStages & (kStages - 1)) == 0 && kStages >= kBufs, "ring sizes");

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
  // default semantics (release at CTA scope): a cluster-scope release would first wait for this thread's
  // outstanding global loads; the TMEM reads it orders have completed at the preceding tcgen05.wait::ld
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

// Tiles are walked in bands of 8 tile-rows (2048 rows): the pairs running at any moment share a compact set
// of A and W tiles in L2.
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
  // K blocks this pair walks through, over all of its tiles
  const int my_tiles = pair < num_tiles ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0;
  const uint32_t total_kb = static_cast<uint32_t>(my_tiles) * static_cast<uint32_t>(G);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
#ifdef EXP_NOHANDBACK
      ptx::mbar_init(ptx::smem_u32(&tail->full[s]), 1);
#else
      ptx::mbar_init(ptx::smem_u32(&tail->full[s]), 1 + 2 * kEpiWarps);
#endif
      ptx::mbar_init(ptx::smem_u32(&tail->done[s]), 1);
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
    ptx::setmaxnreg_dec<24>();
    if (warp == kEpiWarps || warp == kEpiWarps + 4) {
      // ------------------------------------------------------------------ TMA producer (both CTAs)
      if (lane == 0) {
        uint32_t stage = 0, phase = 0;
        uint32_t pkb = 0; (void)pkb;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
          int tm, tn;
          tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
          const int a_row = tm * BM + static_cast<int>(rank) * 128;
          const int w_row = tn * BN + static_cast<int>(rank) * (BN / 2);
          for (int g = 0; g < G; ++g) {
            ok = ptx::mbar_wait(ptx::smem_u32(&tail->done[stage]), phase ^ 1u, abort_flag, p.wait_limit);
            if (!ok) break;
            TRACE(0, pkb); ++pkb;   // pkb = 1 for the first K block from here on
            const uint32_t full_local = ptx::smem_u32(&tail->full[stage]);
            const uint32_t full0 = map_to_cta(full_local, 0);
            const uint32_t dst = smem_base + stage * kStageBytes;
            // warp 8 brings the A rows, warp 12 this CTA's half of the W tile: a bulk tensor copy occupies its
            // issuing thread for a couple of hundred cycles, two per K block would pace the whole pipeline
#if defined(EXP_WARMONLY)
            // real loads for the first pass over the stages, afterwards the MMAs re-read the same (real) data
            if (pkb <= kStages) {
              if (warp == kEpiWarps) {
                if (rank == 0) ptx::mbar_arrive_expect_tx(full_local, 2 * kStageBytes);
                tma_load_2d_pair(dst, &tmap_a, full0, g * BK, a_row);
              } else {
                tma_load_2d_pair(dst + kABytes, &tmap_w, full0, g * BK, w_row);
              }
            } else if (warp == kEpiWarps && rank == 0) {
              ptx::mbar_arrive(full_local);
            }
#elif defined(EXP_ONLYA)
            if (warp == kEpiWarps) {
              if (rank == 0) ptx::mbar_arrive_expect_tx(full_local, 2 * kABytes);
              tma_load_2d_pair(dst, &tmap_a, full0, g * BK, a_row);
            }
            (void)w_row;
#elif defined(EXP_SAMETILE)
            if (warp == kEpiWarps) {
              if (rank == 0) ptx::mbar_arrive_expect_tx(full_local, 2 * kStageBytes);
              tma_load_2d_pair(dst, &tmap_a, full0, (g & 3) * BK, (a_row & 128));
            } else {
              tma_load_2d_pair(dst + kABytes, &tmap_w, full0, (g & 3) * BK, (w_row & 64));
            }
#else
            if (warp == kEpiWarps) {
              if (rank == 0) ptx::mbar_arrive_expect_tx(full_local, 2 * kStageBytes);
              tma_load_2d_pair(dst, &tmap_a, full0, g * BK, a_row);
            } else {
              tma_load_2d_pair(dst + kABytes, &tmap_w, full0, g * BK, w_row);
            }
#endif
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
      }
    } else if (warp <= kEpiWarps + kIssuers) {
      // ------------------------------------------------------------------ MMA issuers (first CTA only)
      // Three issuing threads (warps 9-11) take the K blocks in turn.  A tcgen05.commit occupies its thread for
      // several hundred cycles, so one thread needs about 820 cycles per block (four MMAs and a commit), far more
      // than the 262 cycles the tensor pipe needs; the cost is per thread, and threads of different warps overlap.
      if (lane == 0 && rank == 0) {
        constexpr uint32_t idesc = ptx::umma_idesc_e4m3(256, BN);
        for (uint32_t kb = static_cast<uint32_t>(warp - (kEpiWarps + 1)); kb < total_kb; kb += kIssuers) {
          const uint32_t stage = kb & (kStages - 1), phase = (kb / kStages) & 1u;
          if (!ptx::mbar_wait(ptx::smem_u32(&tail->full[stage]), phase, abort_flag, p.wait_limit)) break;
          TRACE(1, kb);
          ptx::tc_fence_after_sync();
          const uint32_t base = smem_base + stage * kStageBytes;
          const uint64_t a_desc = ptx::umma_desc_k128(base);
          const uint64_t b_desc = ptx::umma_desc_k128(base + kABytes);
          const uint32_t d = tmem_base + (kb & (kBufs - 1)) * BN;
#pragma unroll
          for (int k4 = 0; k4 < BK / 32; ++k4)
            umma_f8_pair(d, a_desc + 2u * k4, b_desc + 2u * k4, idesc, k4 > 0);
          umma_commit_pair(ptx::smem_u32(&tail->done[stage]));
          TRACE(2, kb);
        }
      }
    }
  } else {
    ptx::setmaxnreg_inc<232>();
    // ------------------------------------------------------------------ epilogue / promotion
    const int wg = warp >> 2;                      // which 64 columns of the tile
    const int quad = warp & 3;                     // TMEM lane quarter this warp may read
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t col_addr = static_cast<uint32_t>(wg * 64);
    const uint32_t full0_base = map_to_cta(ptx::smem_u32(&tail->full[0]), 0);   // the first CTA's `full` ring
    const int row_in_tile = static_cast<int>(rank) * 128 + quad * 32 + lane;
    uint8_t* my_stage = out_stage + warp * kOutWarpBytes;
    uint32_t kb = 0;
    bool ok = true;
    // the first use of every TMEM buffer has nothing to wait for
    if (lane == 0) {
#pragma unroll
      for (int b = 0; b < kBufs; ++b) EXP_HB(mbar_arrive_remote(full0_base + 8u * b));
    }
    // Scales.  A K block lasts about 260 cycles, far less than a global load takes, so the scale pair of a block is
    // requested kScaleAhead blocks before its use.  The request cursor walks the pair's K blocks on its own (it
    // crosses into the next tile while the current one is still being folded); the values wait in a register
    // ring indexed by kb % kScaleAhead, and their product is formed only at use.
    float sa_q[kScaleAhead], sw_q[kScaleAhead];
    int pf_t = pair, pf_g = 0;
    const float* pf_sa = nullptr;
    const float* pf_sw = nullptr;
    auto pf_locate = [&]() {
      pf_sa = nullptr;
      if (pf_t < num_tiles) {
        int tm, tn;
        tile_coords(pf_t, p.tiles_m, p.tiles_n, tm, tn);
        const int row = tm * BM + row_in_tile;
        if (row < p.m && tn * BN + wg * 64 < p.n) {
          pf_sa = p.a_scales + row;
          pf_sw = p.w_scales + static_cast<int64_t>(tn) * G;
        }
      }
    };
    auto pf_fetch = [&](float& sa, float& sw) {
      sa = 0.0f;
      sw = 0.0f;
      if (pf_sa != nullptr) {
        sa = __ldg(pf_sa + static_cast<int64_t>(pf_g) * p.ldsa);
        sw = __ldg(pf_sw + pf_g);
      }
      if (++pf_g == G) {
        pf_g = 0;
        pf_t += num_pairs;
        pf_locate();
      }
    };
    pf_locate();
#pragma unroll
    for (int i = 0; i < kScaleAhead; ++i) pf_fetch(sa_q[i], sw_q[i]);
    // Two staging sets: while one K block is folded into the accumulators the next one's TMEM loads are in flight;
    // K block kb uses set kb % 2.
    uint32_t s0a[32], s0b[32], s1a[32], s1b[32];
#ifdef EXP_DELTA
    long long dsum[6] = {0, 0, 0, 0, 0, 0}, dlast = clock64();
#endif
    if (total_kb > 0) {
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&tail->done[0]), 0, abort_flag, p.wait_limit));
      if (ok) {
        ptx::tc_fence_after_sync();
        const uint32_t taddr = tmem_base + lane_addr + col_addr;
        EXP_LD(ptx::tmem_ld32(taddr, s0a);)
        EXP_LD(ptx::tmem_ld32(taddr + 32, s0b);)
      }
    }
    for (int t = pair; t < num_tiles && ok; t += num_pairs) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int row0 = tm * BM + static_cast<int>(rank) * 128 + quad * 32;
      const int row = row0 + lane;
      const int col0 = tn * BN + wg * 64;          // this thread's first column
      const bool row_ok = row < p.m;
      float2 acc[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[j] = make_float2(0.0f, 0.0f);

      // One K block: `ca`/`cb` hold (or are receiving) its 64 columns, `na`/`nb` receive the next block's.
#define BFP8_PAIR_STEP(ca, cb, na, nb, slot)                                                                     \
      {                                                                                                          \
        DSTAMP(5)                                                                                                \
        EXP_SCALE_LINES(slot)                                                                                    \
        ptx::tmem_wait_ld32(ca);                                                                                 \
        ptx::tmem_regs_ready32(cb);                                                                              \
        DSTAMP(0)                                                                                                \
        /* all of this thread's columns of the buffer are in registers: release it to the MMA issuer */          \
        ptx::tc_fence_before_sync();                                                                             \
        __syncwarp();                                                                                            \
        if (threadIdx.x == 0) TRACE(4, kb);                                                                      \
        if (lane == 0) EXP_HB(mbar_arrive_remote(full0_base + 8u * ((kb + kBufs) & (kStages - 1))));             \
        const uint32_t nkb = kb + 1;                                                                             \
        DSTAMP(1)                                                                                                \
        EXP_FMAFIRST(fma32(acc, ca, sv); fma32(acc + 16, cb, sv);)                                               \
        if (nkb < total_kb) {                                                                                    \
          ok = __all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&tail->done[nkb & (kStages - 1)]),           \
                                                      (nkb / kStages) & 1u, abort_flag, p.wait_limit));          \
          if (threadIdx.x == 0) TRACE(3, nkb);                                                                   \
          DSTAMP(2)                                                                                              \
          if (ok) {                                                                                              \
            ptx::tc_fence_after_sync();                                                                          \
            const uint32_t naddr = tmem_base + lane_addr + (nkb & (kBufs - 1)) * BN + col_addr;                  \
            EXP_LD(ptx::tmem_ld32(naddr, na);)                                                                   \
            EXP_LD(ptx::tmem_ld32(naddr + 32, nb);)                                                              \
          }                                                                                                      \
        }                                                                                                        \
        DSTAMP(3)                                                                                                \
        EXP_FMA(fma32(acc, ca, sv);)                                                                             \
        EXP_FMA2(fma32(acc + 16, cb, sv);)                                                                       \
        if (threadIdx.x == 0) TRACE(5, kb);                                                                      \
        DSTAMP(4)                                                                                                \
        kb = nkb;                                                                                                \
      }

      static_assert(kScaleAhead == 4, "the switch below lists the ring slots");
      for (int g = 0; g < G && ok; ++g) {
        switch (kb & 3u) {
          case 0: BFP8_PAIR_STEP(s0a, s0b, s1a, s1b, 0) break;
          case 1: BFP8_PAIR_STEP(s1a, s1b, s0a, s0b, 1) break;
          case 2: BFP8_PAIR_STEP(s0a, s0b, s1a, s1b, 2) break;
          default: BFP8_PAIR_STEP(s1a, s1b, s0a, s0b, 3) break;
        }
      }
#undef BFP8_PAIR_STEP
      if (!ok) break;
      // ---- tile done: bias, rounding, store.  acc[j] holds columns col0 + 2j, col0 + 2j + 1
      if (p.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (col0 + 2 * j < p.n) acc[j].x += __ldg(p.bias + col0 + 2 * j);
          if (col0 + 2 * j + 1 < p.n) acc[j].y += __ldg(p.bias + col0 + 2 * j + 1);
        }
      }
      if (kOutBf16 && (p.n & 7) != 0 && col0 + 64 > p.n) {
        // ragged right edge that is not 16-byte granular: guarded element stores
        if (row_ok && col0 < p.n)
          store_row_bf16_guarded(reinterpret_cast<uint16_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0, acc,
                                 p.n - col0);
      } else if (kOutBf16) {
        // one box: 32 rows x 64 bf16 (128 B per row), 16-byte chunks XOR-swizzled by row & 7
        if (lane == 0) ptx::tma_store_wait_read_all();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 v;
          v.x = pack_bf16x2(acc[4 * j + 0].x, acc[4 * j + 0].y);
          v.y = pack_bf16x2(acc[4 * j + 1].x, acc[4 * j + 1].y);
          v.z = pack_bf16x2(acc[4 * j + 2].x, acc[4 * j + 2].y);
          v.w = pack_bf16x2(acc[4 * j + 3].x, acc[4 * j + 3].y);
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
          if (col0 + 2 * j < p.n) o[2 * j] = acc[j].x;
          if (col0 + 2 * j + 1 < p.n) o[2 * j + 1] = acc[j].y;
        }
      }
    }
    if (kOutBf16 && lane == 0) ptx::tma_store_wait_all();
#ifdef EXP_DELTA
    if (blockIdx.x < 2 && lane == 0) {
      for (int i = 0; i < 6; ++i) g_delta[(blockIdx.x * 8 + warp) * 8 + i] = dsum[i];
      g_delta[(blockIdx.x * 8 + warp) * 8 + 6] = total_kb;
    }
#endif
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
  rc = make_tensor_map_2d(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, w_codes, k, n, ldw, BK, BN / 2);
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
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  int pairs = sm_count() / 2;
  if (max_ctas > 1 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  if (tiles < pairs) pairs = static_cast<int>(tiles);
  auto kern = bf16 ? gemm_pair_kernel<true> : gemm_pair_kernel<false>;
  static bool done[2][64] = {};
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
