// Block-scaled E4M3 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma (kind::f8f6f4) -> TMEM,
// with the per-128-K-block fp32 scale promotion done by the epilogue warps.
//
//   out[i, j] = sum_g sa[g, i] * sw[j/128, g] * ( A_g[i, :] . W_g[j, :] )      A_g, W_g: 128 codes wide
//
// One K block (128 E4M3 codes = 128 bytes per row) is exactly one SWIZZLE_128B shared-memory row, so a
// pipeline stage holds one K block of a 128-row A tile and a 256-row W tile, and four K=32 MMAs
// consume it.  Because the scale product changes with every K block, each block is accumulated from
// zero into one of two 256-column TMEM buffers; the epilogue warps read it back (tcgen05.ld), fold
// it into register accumulators with one FMA per element, and hand the buffer back, while the MMA
// warp is already filling the other buffer.
//
// Warp roles (384 threads): warps 0-7 epilogue (two warpgroups; warpgroup w owns output columns
// 128w..128w+127 of the tile, so it sees a single weight scale per K block), warp 8 TMA producer,
// warp 9 TMEM owner and MMA issuer of the even K blocks (TMEM buffer 0), warp 10 MMA issuer of the odd
// K blocks (buffer 1), warp 11 idle; the third warpgroup gives its registers to the epilogue through
// setmaxnreg.  One thread needs about 100 cycles more than the tensor pipe to wait, issue four MMAs and
// commit, so two threads alternate and the pipe stays fed.
//
// Barriers, indexed by K block number kb (a running count over the CTA's tiles), four of each so that no
// waiter can be lapped: `full[kb % 4]` completes when the stage's TMA bytes have landed AND the eight
// epilogue warps have drained the TMEM buffer kb % 2 of K block kb - 2 (one wait for the MMA issuer);
// `done[kb % 4]` completes through the issuer's single tcgen05.commit and tells both the epilogue (TMEM
// buffer ready) and the producer (shared-memory stage free).  The kernel is persistent: one CTA per SM walks a static tile
// list.  Every barrier wait is bounded; on expiry the CTA raises BFP8_STATUS_WAIT_TIMEOUT and leaves.
#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "ptx.cuh"

namespace bfp8 {

namespace {

#ifdef BFP8_TIMELINE
__device__ unsigned int g_timeline_large[kTimelineEvents * kTimelineUnits];
#endif

constexpr int BM = 128;            // tile rows (A rows, TMEM lanes)
constexpr int BN = 256;            // tile columns (W rows, TMEM columns per buffer)
constexpr int BK = 128;            // one scale block of K
constexpr int kStages = 4;          // also the number of barrier pairs; the kb % 4 bookkeeping relies on it
constexpr int kEpiWarps = 8;
constexpr int kThreads = (kEpiWarps + 4) * 32;   // warps 10, 11 only complete the third warpgroup
constexpr int kTmemCols = 512;     // two accumulator buffers of BN columns

constexpr int kABytes = BM * BK;               // 16 KB
constexpr int kBBytes = BN * BK;               // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kOutWarpBytes = 32 * 64 * 2;                  // per warp: one box of 32 rows x 64 bf16
constexpr int kOutStageBytes = kEpiWarps * kOutWarpBytes;

struct SmemTail {
  uint64_t full[kStages];          // TMA bytes of K block kb + release of TMEM buffer kb % 2 by the 8 epilogue warps
  uint64_t done[kStages];          // MMAs of K block kb complete: TMEM buffer readable, stage reusable
  uint32_t tmem_base;
  uint32_t abort_flag;
};

constexpr int kSmemBytes = 1024 /* alignment slack */ + kStages * kStageBytes + kOutStageBytes + sizeof(SmemTail);

// One output tensor map per destination GPU of the push mode.
struct PushMaps {
  CUtensorMap m[8];
};

struct GemmParams {
  const float* a_scales;   // [G, ldsa]
  const float* w_scales;   // [NB, G]
  const float* bias;       // [N] or null
  void* out;               // fp32 or bf16 [M, ldo]
  int64_t ldsa, ldo;
  int m, n, k, groups;
  int tiles_m, tiles_n;
  int band;                // tile-rows per band of the tile walk
  int inter;               // SwiGLU only: width of the gate and of the up projection (N = 2 * inter)
  // Push mode (row-parallel GEMM): the bf16 tile of rows [o R, (o + 1) R) goes to GPU o, into slot `push_rank` of
  // its receive area [push_world][R][N]; push_world == 0 stores to `out` as usual
  int push_world, push_rank, push_rows;
  int band_shift;          // the tile walk starts at this band (all bands full), so that ranks push to different owners
  long long wait_limit;
  uint32_t* status;
};

// Tiles are walked in bands of 16 tile-rows: consecutive tile indices share W tiles inside a band,
// so the CTAs running at any moment touch a compact set of A and W tiles in L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int kBand, int shift, int& tm, int& tn) {
  const int per_band = kBand * tiles_n;
  int band = t / per_band;
  const int r0 = t - band * per_band;
  if (shift != 0) {                       // only used when kBand divides tiles_m
    band += shift;
    const int nbands = tiles_m / kBand;
    band -= (band / nbands) * nbands;
    t = band * per_band + r0;
  }
  const int first = band * kBand;
  const int rows = min(kBand, tiles_m - first);
  const int r = t - band * per_band;
  tm = first + r % rows;
  tn = r / rows;
}

// kSwiGLU: W holds gate and up rows interleaved in chunks of 64 (bfp8_swiglu_interleave_weight), so the 128
// tile columns of a warpgroup are 64 gate columns followed by the 64 up columns of the same outputs, and a
// thread ends a tile holding both factors of its 64 outputs.  The tile's 256 weight rows are outputs
// 128 tn .. 128 tn + 127, which lie in one scale block of the gate grid and one of the up grid.
template <bool kOutBf16, bool kSwiGLU>
__global__ void __launch_bounds__(kThreads, 1)
gemm_block128_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                     const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ PushMaps pmaps,
                     const GemmParams p) {
  BFP8_TL_DECL
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
      ptx::mbar_init(ptx::smem_u32(&tail->full[s]), 1 + kEpiWarps);
      ptx::mbar_init(ptx::smem_u32(&tail->done[s]), 1);
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
   ptx::setmaxnreg_dec<24>();
   if (warp == kEpiWarps) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      long long pkb = 0;                                        // running K block number (timeline build only)
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, p.band, p.band_shift, tm, tn);
        for (int g = 0; g < G; ++g) {
          ok = ptx::mbar_wait(ptx::smem_u32(&tail->done[stage]), phase ^ 1u, abort_flag, p.wait_limit);
          if (!ok) break;
          BFP8_TL(0, pkb);                                      // stage free, copies issued
          ++pkb;
          const uint32_t full = ptx::smem_u32(&tail->full[stage]);
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          ptx::mbar_arrive_expect_tx(full, kStageBytes);
          ptx::tma_load_2d(a_dst, &tmap_a, full, g * BK, tm * BM);
          ptx::tma_load_2d(a_dst + kABytes, &tmap_w, full, g * BK, tn * BN);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == kEpiWarps + 1 || warp == kEpiWarps + 2) {
    // ------------------------------------------------------------------ MMA issuers (even / odd K blocks)
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::umma_idesc_e4m3(BM, BN);
      const uint32_t parity = warp - (kEpiWarps + 1);          // which K blocks, and which TMEM buffer, are mine
      const uint32_t d = tmem_base + parity * BN;
      long long total = 0;                                     // K blocks of this CTA
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) total += G;
      for (long long kb = parity; kb < total; kb += 2) {
        const uint32_t stage = static_cast<uint32_t>(kb) & (kStages - 1), phase = static_cast<uint32_t>(kb >> 2) & 1u;
        if (!ptx::mbar_wait(ptx::smem_u32(&tail->full[stage]), phase, abort_flag, p.wait_limit)) break;
        BFP8_TL(1, kb);                                         // operands landed and TMEM buffer handed back
        ptx::tc_fence_after_sync();
        const uint32_t a_addr = smem_base + stage * kStageBytes;
        const uint64_t a_desc = ptx::umma_desc_k128(a_addr);
        const uint64_t b_desc = ptx::umma_desc_k128(a_addr + kABytes);
#pragma unroll
        for (int k4 = 0; k4 < BK / 32; ++k4)   // +32 bytes along K = +2 in the descriptor's address field
          ptx::umma_f8(d, a_desc + 2u * k4, b_desc + 2u * k4, idesc, k4 > 0);
        ptx::umma_commit(ptx::smem_u32(&tail->done[stage]));
        BFP8_TL(2, kb);                                         // MMAs and commit issued
      }
    }
   }
  } else {
    ptx::setmaxnreg_inc<240>();
    // ------------------------------------------------------------------ epilogue / promotion
    // TMEM loads complete only at a wait that covers all of a thread's outstanding loads, so the
    // latency of one 32-column load is hidden behind the FMAs of the previous one (two register
    // batches), and the first load of the next K block is issued before the last FMAs of this one.
    const int wg = warp >> 2;                      // column half of the tile
    const int quad = warp & 3;                     // TMEM lane quarter this warp may read
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    uint8_t* my_stage = out_stage + warp * kOutWarpBytes;
    uint32_t kb = 0;
    bool ok = true;
    // the first use of either TMEM buffer has nothing to wait for
    if (lane == 0) {
      ptx::mbar_arrive(ptx::smem_u32(&tail->full[0]));
      ptx::mbar_arrive(ptx::smem_u32(&tail->full[1]));
    }
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, p.band, p.band_shift, tm, tn);
      const int row = tm * BM + quad * 32 + lane;
      // first output column of this thread: 128 of the tile's 256, or with SwiGLU 64 of its 128 outputs
      const int col0 = kSwiGLU ? tn * 128 + wg * 64 : tn * BN + wg * 128;
      const bool row_ok = row < p.m;
      const int nb = kSwiGLU ? tn : col0 >> 7;
      const bool live = row_ok && (kSwiGLU || col0 < p.n);
      const float* sa_ptr = p.a_scales + row;
      const float* sw_ptr = p.w_scales + static_cast<int64_t>(nb) * G;
      // SwiGLU: scale row of the up projection's block (the grid lists the gate blocks first)
      const float* su_ptr = p.w_scales + static_cast<int64_t>((p.inter >> 7) + nb) * G;
      float2 acc[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc[j] = make_float2(0.0f, 0.0f);
      // scales are fetched two K blocks ahead of their use; the product is formed only when needed,
      // so no load is waited for at the top of the loop
      float sa0 = live ? __ldg(sa_ptr) : 0.0f, sw0 = live ? __ldg(sw_ptr) : 0.0f;
      float sa1 = (live && G > 1) ? __ldg(sa_ptr + p.ldsa) : 0.0f, sw1 = (live && G > 1) ? __ldg(sw_ptr + 1) : 0.0f;
      float su0 = 0.0f, su1 = 0.0f;
      if (kSwiGLU) {
        su0 = live ? __ldg(su_ptr) : 0.0f;
        su1 = (live && G > 1) ? __ldg(su_ptr + 1) : 0.0f;
      }
      uint32_t ra[32], rb[32];
      {
        const uint32_t buf = kb & 1u;
        // wait outcomes are made uniform across the warp: warp-collective TMEM loads and __syncwarp follow them
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&tail->done[kb & (kStages - 1)]), (kb >> 2) & 1u,
                                                    abort_flag, p.wait_limit));
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t taddr = tmem_base + lane_addr + buf * BN + wg * 128;
        ptx::tmem_ld32(taddr, ra);
        ptx::tmem_ld32(taddr + 32, rb);
      }
      for (int g = 0; g < G; ++g, ++kb) {
        float sa2 = 0.0f, sw2 = 0.0f, su2 = 0.0f;
        if (live && g + 2 < G) {
          sa2 = __ldg(sa_ptr + static_cast<int64_t>(g + 2) * p.ldsa);
          sw2 = __ldg(sw_ptr + g + 2);
          if (kSwiGLU) su2 = __ldg(su_ptr + g + 2);
        }
        const uint32_t buf = kb & 1u;
        const uint32_t taddr = tmem_base + lane_addr + buf * BN + wg * 128;
        const float s = sa0 * sw0;
        const float2 sv = make_float2(s, s);
        const float s_up = kSwiGLU ? sa0 * su0 : s;            // columns 64..127 of the warpgroup
        const float2 sv_up = make_float2(s_up, s_up);
        ptx::tmem_wait_ld32(ra);
        ptx::tmem_regs_ready32(rb);
        if (threadIdx.x == 0) BFP8_TL(3, kb);                   // first 64 columns in registers
        {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            acc[j] = __ffma2_rn(make_float2(__uint_as_float(ra[2 * j]), __uint_as_float(ra[2 * j + 1])), sv, acc[j]);
        }
        ptx::tmem_ld32(taddr + 64, ra);
        {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            acc[16 + j] = __ffma2_rn(make_float2(__uint_as_float(rb[2 * j]), __uint_as_float(rb[2 * j + 1])), sv, acc[16 + j]);
        }
        ptx::tmem_ld32(taddr + 96, rb);
        ptx::tmem_wait_ld32(ra);
        ptx::tmem_regs_ready32(rb);
        // every column of this buffer is in registers: hand it back to the MMA warp
        ptx::tc_fence_before_sync();
        __syncwarp();
        ptx::mbar_arrive_lane0(ptx::smem_u32(&tail->full[(kb + 2) & (kStages - 1)]), lane);
        if (threadIdx.x == 0) BFP8_TL(4, kb);                   // buffer handed back
        {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            acc[32 + j] = __ffma2_rn(make_float2(__uint_as_float(ra[2 * j]), __uint_as_float(ra[2 * j + 1])), sv_up, acc[32 + j]);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            acc[48 + j] = __ffma2_rn(make_float2(__uint_as_float(rb[2 * j]), __uint_as_float(rb[2 * j + 1])), sv_up, acc[48 + j]);
        }
        if (threadIdx.x == 0) BFP8_TL(5, kb);                   // FMAs of the block issued
        if (g + 1 < G) {
          // first half of the next K block's buffer
          const uint32_t nkb = kb + 1, nbuf = nkb & 1u;
          ok = __all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&tail->done[nkb & (kStages - 1)]), (nkb >> 2) & 1u,
                                                      abort_flag, p.wait_limit));
          if (!ok) break;
          if (threadIdx.x == 0) BFP8_TL(6, kb);                 // completion of the next block observed
          ptx::tc_fence_after_sync();
            const uint32_t naddr = tmem_base + lane_addr + nbuf * BN + wg * 128;
          ptx::tmem_ld32(naddr, ra);
          ptx::tmem_ld32(naddr + 32, rb);
        }
        sa0 = sa1; sw0 = sw1;
        sa1 = sa2; sw1 = sw2;
        if (kSwiGLU) { su0 = su1; su1 = su2; }
      }
      if (!ok) break;
      // ---- tile done: bias, rounding, store
      if (kSwiGLU) {
        // gate and up are rounded to bf16 as the unfused GEMM would store them, then silu(gate) * up is
        // formed in fp32 and rounded once (silu_and_mul_bf16.c:16); one box of 32 rows x 64 outputs per warp
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float2 gt = acc[j], up = acc[32 + j];
          if (p.bias != nullptr) {
            gt.x += __ldg(p.bias + col0 + 2 * j);
            gt.y += __ldg(p.bias + col0 + 2 * j + 1);
            up.x += __ldg(p.bias + p.inter + col0 + 2 * j);
            up.y += __ldg(p.bias + p.inter + col0 + 2 * j + 1);
          }
          const uint32_t gp = pack_bf16x2(gt.x, gt.y), upk = pack_bf16x2(up.x, up.y);
          acc[j] = make_float2(silu_mul(bf16_lo_to_float(gp), bf16_lo_to_float(upk)),
                               silu_mul(bf16_hi_to_float(gp), bf16_hi_to_float(upk)));
        }
        if (lane == 0) ptx::tma_store_wait_read_all();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int e = j * 4;
          uint4 v;
          v.x = pack_bf16x2(acc[e + 0].x, acc[e + 0].y);
          v.y = pack_bf16x2(acc[e + 1].x, acc[e + 1].y);
          v.z = pack_bf16x2(acc[e + 2].x, acc[e + 2].y);
          v.w = pack_bf16x2(acc[e + 3].x, acc[e + 3].y);
          *reinterpret_cast<uint4*>(my_stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int y = tm * BM + quad * 32;
          if (y < p.m) ptx::tma_store_2d(&tmap_out, ptx::smem_u32(my_stage), col0, y);
          ptx::tma_store_commit();
        }
        continue;
      }
      if (p.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          if (col0 + 2 * j < p.n) acc[j].x += __ldg(p.bias + col0 + 2 * j);
          if (col0 + 2 * j + 1 < p.n) acc[j].y += __ldg(p.bias + col0 + 2 * j + 1);
        }
      }
      if (kOutBf16) {
        // two passes of one box each: 32 rows x 64 bf16 (128 B per row), 16-byte chunks XOR-swizzled by row & 7
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          if ((p.n & 7) != 0 && col0 + b * 64 + 64 > p.n) {
            // ragged right edge that is not 16-byte granular: guarded element stores
            if (row_ok && col0 + b * 64 < p.n)
              store_row_bf16_guarded(reinterpret_cast<uint16_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0 + b * 64,
                                     acc + b * 32, p.n - (col0 + b * 64));
            continue;
          }
          // the previous TMA store must have finished reading this warp's staging buffer
          if (lane == 0) ptx::tma_store_wait_read_all();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int e = b * 32 + j * 4;                          // float2 index of the chunk's first pair
            uint4 v;
            v.x = pack_bf16x2(acc[e + 0].x, acc[e + 0].y);
            v.y = pack_bf16x2(acc[e + 1].x, acc[e + 1].y);
            v.z = pack_bf16x2(acc[e + 2].x, acc[e + 2].y);
            v.w = pack_bf16x2(acc[e + 3].x, acc[e + 3].y);
            *reinterpret_cast<uint4*>(my_stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int y = tm * BM + quad * 32;
            if (y < p.m && col0 + b * 64 < p.n) {
              if (p.push_world > 0) {
                // a peer's memory is the destination: same bulk store, through that GPU's tensor map
                const int owner = (tm * BM) / p.push_rows;
                ptx::tma_store_2d(&pmaps.m[owner], ptx::smem_u32(my_stage), col0 + b * 64,
                                  p.push_rank * p.push_rows + (y - owner * p.push_rows));
              } else {
                ptx::tma_store_2d(&tmap_out, ptx::smem_u32(my_stage), col0 + b * 64, y);
              }
            }
            ptx::tma_store_commit();
          }
        }
      } else {
        if (row_ok) {
          float* o = reinterpret_cast<float*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0;
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            if (col0 + 2 * j < p.n) o[2 * j] = acc[j].x;
            if (col0 + 2 * j + 1 < p.n) o[2 * j + 1] = acc[j].y;
          }
        }
      }
    }
    if (kOutBf16 && lane == 0) ptx::tma_store_wait_all();
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  BFP8_TL_DUMP(g_timeline_large);
  ptx::idle_after_abort(abort_flag);
  if (warp == kEpiWarps + 1) ptx::tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && tail->abort_flag != 0) atomicOr(p.status, BFP8_STATUS_WAIT_TIMEOUT);
}

}  // namespace

// ---- host side ------------------------------------------------------------------------------------

// Destination of the push mode: recv[o] is GPU o's receive area ([world][rows][n] bf16, mapped in this process).
struct PushTarget {
  const void* recv[8];
  int world, rank, rows;
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so the library has no link-time dependency on libcuda.
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D row-major tensor map; box_inner * element size must not exceed the swizzle span (128 bytes by default).
int make_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return BFP8_ERR_CUDA;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return BFP8_ERR_CUDA;
  }
  return BFP8_OK;
}

int launch_gemm_large(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                      const uint8_t* w_codes, int64_t ldw, const float* w_scales, const float* bias, void* out,
                      int out_dtype, int64_t ldo, int64_t m, int64_t n, int64_t k, uint32_t* status_dev,
                      long long wait_limit, int max_ctas, int band, int inter, const PushTarget* push,
                      cudaStream_t st) {
  // inter > 0 selects the SwiGLU epilogue: W has n = 2 * inter interleaved rows and the output is [m, inter] bf16
  // push != nullptr selects the push mode: bf16 tiles go to the receive areas of the GPUs that own their rows
  alignas(64) CUtensorMap tmap_a, tmap_w, tmap_out;
  alignas(64) PushMaps pmaps;
  memset(&pmaps, 0, sizeof(pmaps));
  int rc = make_tensor_map_2d(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a_codes, k, m, lda, BK, BM);
  if (rc != BFP8_OK) return rc;
  rc = make_tensor_map_2d(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, w_codes, k, n, ldw, BK, BN);
  if (rc != BFP8_OK) return rc;
  const bool bf16 = out_dtype == BFP8_OUT_BF16;
  if (push != nullptr) {
    if (!bf16 || inter > 0 || push->world < 2 || push->world > 8 || push->rows <= 0 || push->rows % BM != 0 ||
        m != static_cast<int64_t>(push->rows) * push->world || n % 64 != 0)
      return BFP8_ERR_UNSUPPORTED;
    for (int o = 0; o < push->world; ++o) {
      // GPU o's receive area: [world][rows][n] bf16, contiguous
      rc = make_tensor_map_2d(&pmaps.m[o], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, push->recv[o], n,
                              static_cast<uint64_t>(push->rows) * push->world, n * 2, 64, 32);
      if (rc != BFP8_OK) return rc;
    }
    tmap_out = pmaps.m[push->rank];   // not used by the kernel in this mode
  } else if (bf16) {
    rc = make_tensor_map_2d(&tmap_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, out, inter > 0 ? inter : n, m, ldo * 2, 64, 32);
    if (rc != BFP8_OK) return rc;
  } else {
    tmap_out = tmap_a;   // unused on the fp32 path
  }
  GemmParams p;
  p.a_scales = a_scales;
  p.w_scales = w_scales;
  p.bias = bias;
  p.out = out;
  p.ldsa = ldsa;
  p.ldo = ldo;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.groups = static_cast<int>((k + BK - 1) / BK);
  p.tiles_m = static_cast<int>((m + BM - 1) / BM);
  p.tiles_n = static_cast<int>((n + BN - 1) / BN);
  p.wait_limit = wait_limit;
  p.status = status_dev;
  p.band = band > 0 ? band : 16;
  p.inter = inter;
  p.push_world = p.push_rank = p.band_shift = 0;
  p.push_rows = 1;
  if (push != nullptr) {
    p.push_world = push->world;
    p.push_rank = push->rank;
    p.push_rows = push->rows;
    // one band per owner, and every rank starts with a different owner (its own rows come last), so that at
    // any moment each GPU receives from one peer instead of from all of them
    p.band = push->rows / BM;
    p.band_shift = (push->rank + 1) % push->world;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  if (inter > 0 && !bf16) return BFP8_ERR_UNSUPPORTED;
  auto kern = inter > 0 ? gemm_block128_kernel<true, true>
                        : (bf16 ? gemm_block128_kernel<true, false> : gemm_block128_kernel<false, false>);
  static DeviceFlags done[3];
  rc = ensure_smem_limit(kern, kSmemBytes, done[inter > 0 ? 2 : (bf16 ? 1 : 0)]);
  if (rc != BFP8_OK) return rc;
  kern<<<grid, kThreads, kSmemBytes, st>>>(tmap_a, tmap_w, tmap_out, pmaps, p);
  BFP8_CUDA_TRY(cudaGetLastError());
  return BFP8_OK;
}

}  // namespace bfp8

#ifdef BFP8_TIMELINE
// Diagnostic build only: the timeline of CTA kTimelineCta of the last large-tile launch on the current device
// ([kTimelineEvents][kTimelineUnits] %clock values per K block; 0 = not reached).  Synchronises the device.
extern "C" int bfp8_timeline_read_large(unsigned int* dst_host) {
  BFP8_CUDA_TRY(cudaDeviceSynchronize());
  BFP8_CUDA_TRY(cudaMemcpyFromSymbol(dst_host, bfp8::g_timeline_large, sizeof(unsigned int) * bfp8::kTimelineEvents * bfp8::kTimelineUnits));
  return BFP8_OK;
}
#endif
