// Small-M ("decode bucket") schedule of the block-scaled E4M3 GEMM for sm_100a.
//
// With at most 128 activation rows the GEMM is a single pass over the weight matrix and is bound
// by HBM, so the schedule is built around streaming W exactly once at full bandwidth:
//   * operands are swapped: 128 weight rows are the MMA's M dimension (TMEM lanes) and the padded
//     activation rows (16 / 32 / 64 / 128) its N dimension, so no tensor-core work is wasted on padding W;
//   * the work is cut into units of (128 weight rows) x (one 128-wide K block) = 16 KB of W, and the
//     unit list - tile-major, K-block-minor - is split evenly over the CTAs (stream-K), so every SM
//     streams the same number of bytes whatever N and K are;
//   * a tile whose K range is spread over several CTAs is finished by the first of them: the others write
//     their fp32 partials to the workspace and count themselves in (per-tile counter); the first CTA, whose
//     part of the tile is the last thing it works on, waits (bounded) for the count, adds the partials to
//     its own sums in CTA order - a fixed order, so results do not depend on timing - applies the bias and
//     stores the tile.  Counters are returned to zero, so a zero-initialised workspace stays reusable.
// When there are at most half as many tiles as SMs, the CTAs that share a tile form a thread-block cluster
// (2, 4 or 8 CTAs, each with an equal slice of the K range) and exchange their partials through distributed
// shared memory instead: every CTA owns MP / cluster-size of the padded activation rows, receives those rows
// from all CTAs of the cluster into the (by then idle) pipeline buffers, adds them in rank order - again a
// fixed order - and stores its rows.  Two cluster barriers replace the store / fence / counter / read-back
// round trip through global memory.
// Each K block is accumulated from zero into one of four small TMEM buffers and folded into register
// accumulators with its scale product sa[g, i] * sw[j/128, g], as in the large-tile schedule.
//
// Warp roles (320 threads; 256 with 64 or 128 activation columns): warps 0-3 epilogue (thread = weight row), warp 4
// TMA producer, warp 5 TMEM owner and first MMA issuer, warps 7-9 (7 alone in the 256-thread form) the other MMA
// issuers - a thread that has issued a unit's four MMAs and its two commits is held until the MMAs have
// completed, several times the unit's HBM time, so the issuers take the units in turn -
// warp 6 scale loader: it fetches the scale products of the units ahead
// (global-memory latency is far longer than a unit's 16 KB of HBM time) and parks them in a small
// shared-memory ring next to the TMEM buffers.  All barrier waits are bounded.
//
// SwiGLU form (Params::inter > 0): W is a fused gate/up weight whose rows were interleaved in chunks of 64
// (bfp8_swiglu_interleave_weight - the layout the large-tile fused kernel reads, so prefill and decode share one
// copy), so a 128-row tile holds the gate rows (TMEM lanes 0-63) and the up rows (lanes 64-127) of the same 64
// outputs.  The two halves take their weight scale from the gate and from the up block of the original scale
// grid (two scale vectors per unit), both factors get their bias and are rounded to bf16 as the unfused GEMM
// would store them, the up half hands its values to the gate half through shared memory, and the gate half
// stores bf16(silu(gate) * up) - csrc/tpc/generic_dense/silu_and_mul_bf16.c:16 - into the [M, inter] output.
#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"

namespace bfp8 {

// Destination of the push form: recv[o] is GPU o's receive area ([world][rows][n] bf16, mapped in this process).
struct SmallPush {
  const void* recv[8];
  int world, rank, rows;
};

namespace {

#ifdef BFP8_TIMELINE
__device__ unsigned int g_timeline_smallm[kTimelineEvents * kTimelineUnits];
#endif

constexpr int BN = 128;            // weight rows per tile = one scale block
constexpr int BK = 128;
constexpr int kEpiWarps = 4;
constexpr int kScaleAhead = 8;     // units whose scales are in flight in the loader's registers
constexpr int kAccBufs = 4;
constexpr int kWBytes = BN * BK;   // 16 KB of W per unit
constexpr int kMaxStages = 10;
constexpr int kSmemBudget = 200 * 1024;
constexpr int kSwigluRows = 64;    // activation rows per exchange round of the SwiGLU form (fewer when MP is smaller)
constexpr int kSwigluExBytes = 2 * kSwigluRows * 64 * 2;   // gate and up values as bf16

template <int MP>
struct Cfg {
  static constexpr int kABytes = MP * BK;
  static constexpr int kStageBytes = kWBytes + kABytes;
  static constexpr int kStages = (kSmemBudget / kStageBytes) < kMaxStages ? (kSmemBudget / kStageBytes) : kMaxStages;
  static constexpr int kTmemCols = (kAccBufs * MP) < 32 ? 32 : (kAccBufs * MP);
  // A thread that issues a unit's MMAs and commits is held until those MMAs have completed, far longer than a unit's
  // HBM time (about 1 300 cycles per unit at 64 activation columns), so several threads take the units in turn:
  // four of them up to 32 activation columns, two beyond: with 64 columns four measured slower than two (16.8 against
  // 15.4 us at K=4096, N=14336 - the extra warps share their schedulers with epilogue warps that now have real
  // work), and with 128 the epilogue needs the registers a larger CTA would take away.
  static constexpr int kIssuers = MP <= 32 ? 4 : 2;
  static constexpr int kThreads = (kEpiWarps + 2 + kIssuers) * 32;
  static_assert(kIssuers <= kAccBufs && kAccBufs % kIssuers == 0 && kIssuers < kStages,
                "issuer i owns TMEM buffers i, i + kIssuers, ... and steps through the stage ring by kIssuers");
};

struct SmemTail {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[kAccBufs];
  uint64_t tmem_empty[kAccBufs];
  float scale[kAccBufs][128];        // sa[g, 0..MP) * sw[tile, g] of the unit in each TMEM buffer
  float scale_up[kAccBufs][128];     // SwiGLU form: the same with the up block's weight scale (lanes 64-127)
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t last_flag;
};

struct Params {
  const float* a_scales;   // [G, ldsa]
  const float* w_scales;   // [NB, G]
  const float* bias;
  void* out;
  uint32_t* counters;      // [tiles], zero on entry, zero on exit
  float* partials;         // [ctas][2][MP][128]
  int64_t ldsa, ldo;
  int m, n, groups, tiles;
  int out_bf16;
  long long total_units;
  long long wait_limit;
  uint32_t* status;
  int cluster;             // CTAs per tile when the kernel runs as clusters (kCluster), else unused
  int inter;               // SwiGLU form: width of the gate and of the up projection (n = 2 * inter), else 0
  // Push form (row-parallel GEMM, bf16): activation row j of this rank's partial goes to GPU j / push_rows, into
  // slot push_rank of its receive area [push_world][push_rows][n]; push_world == 0 stores to `out` as usual
  int push_world, push_rank, push_rows;
  uint16_t* push_recv[8];
  int w_early;             // the weight codes are at rest (bfp8_set_weights_at_rest): request them before griddep_wait
};

// Where activation row j of a bf16 result goes (column 0 of that row).
__device__ __forceinline__ uint16_t* out_row_bf16(const Params& p, int j) {
  if (p.push_world > 0) {
    const int owner = j / p.push_rows;
    return p.push_recv[owner] + (static_cast<int64_t>(p.push_rank) * p.push_rows + (j - owner * p.push_rows)) * p.n;
  }
  return reinterpret_cast<uint16_t*>(p.out) + static_cast<int64_t>(j) * p.ldo;
}

// SwiGLU form: the two halves of a tile (weight rows 0..63: gate, 64..127: up, of the same 64 outputs) publish
// their values - bias added, rounded to bf16 as the unfused GEMM would store them - in shared memory (`ex`:
// [2][kRows][64] bf16), and then every thread finishes the outputs of its column for every second activation
// row (gate threads the even rows, up threads the odd ones), so all four warps share the silu arithmetic.  All
// 128 epilogue threads call this together (two named barriers inside).  `v[j]` is the thread's fp32 sum for
// activation row j0 + j (bias not yet added), `rows` how many of them are valid.
template <int kRows>
__device__ __forceinline__ void swiglu_finish(const Params& p, uint16_t* ex, int tile, int wrow, const float* v,
                                              int j0, int rows, bool write) {
  const bool gate = wrow < 64;
  const int o = gate ? wrow : wrow - 64;                       // output column inside the tile's 64
  const int col = tile * 64 + o;
  float b = 0.0f;
  if (p.bias != nullptr) b = __ldg(p.bias + (gate ? col : p.inter + col));
  uint16_t* mine = ex + (gate ? 0 : kRows * 64);
#pragma unroll
  for (int j = 0; j < kRows; ++j)
    if (j < rows) mine[j * 64 + o] = static_cast<uint16_t>(float_to_bf16_bits(v[j] + b));
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (write) {
    // all products first, without a condition in the loop, so that the exp / reciprocal chains of the rows overlap
    // (with the bounds check inside, the rows were evaluated one after the other: 3.3 us of a 31 us launch at M = 64);
    // rows beyond `rows` read whatever the exchange area holds and are not stored
    uint16_t r[kRows / 2];
#pragma unroll
    for (int jj = 0; jj < kRows / 2; ++jj) {
      const int j = 2 * jj + (gate ? 0 : 1);
      const float g = bf16_bits_to_float(ex[j * 64 + o]), u = bf16_bits_to_float(ex[kRows * 64 + j * 64 + o]);
      r[jj] = static_cast<uint16_t>(float_to_bf16_bits(silu_mul(g, u)));
    }
    uint16_t* out = reinterpret_cast<uint16_t*>(p.out) + col;
#pragma unroll
    for (int jj = 0; jj < kRows / 2; ++jj) {
      const int j = 2 * jj + (gate ? 0 : 1);
      if (j < rows && j0 + j < p.m) out[static_cast<int64_t>(j0 + j) * p.ldo] = r[jj];
    }
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");             // `ex` may be rewritten
}

// First unit of CTA c when `total` units are split over `parts` CTAs.
__host__ __device__ inline long long first_unit(long long c, long long total, long long parts) {
  return c * total / parts;
}
// The CTA whose range contains unit u.
__host__ __device__ inline int cta_of_unit(long long u, long long total, long long parts) {
  return static_cast<int>(((u + 1) * parts - 1) / total);
}

template <int MP, bool kCluster, bool kSwiGLU>
__global__ void __launch_bounds__(Cfg<MP>::kThreads, 1)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                   const Params p) {
  using C = Cfg<MP>;
  BFP8_TL_DECL
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  SmemTail* tail = reinterpret_cast<SmemTail*>(smem + C::kStages * C::kStageBytes);
  uint16_t* swiglu_ex = reinterpret_cast<uint16_t*>(tail + 1);   // [2][rows per round][64] bf16, SwiGLU form only
  volatile uint32_t* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.groups;
  const long long parts = gridDim.x;
  // kCluster: cluster c works on tile c and CTA r of it on K blocks [r G / cs, (r + 1) G / cs)
  const int cs = kCluster ? p.cluster : 1;
  const int crank = kCluster ? static_cast<int>(blockIdx.x % cs) : 0;
  const long long ctile = blockIdx.x / cs;
  const long long u0 = kCluster ? ctile * G + static_cast<long long>(crank) * G / cs
                                : first_unit(blockIdx.x, p.total_units, parts);
  const long long u1 = kCluster ? ctile * G + static_cast<long long>(crank + 1) * G / cs
                                : first_unit(blockIdx.x + 1, p.total_units, parts);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&tail->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&tail->empty[s]), 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      // a buffer is ready for the epilogue when its MMAs have completed (tcgen05.commit) and the scale loader has
      // parked the unit's scale products next to it: two arrivals on one barrier, one poll per unit for the epilogue
      ptx::mbar_init(ptx::smem_u32(&tail->tmem_full[b]), 2);
      ptx::mbar_init(ptx::smem_u32(&tail->tmem_empty[b]), kEpiWarps);
    }
    tail->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kEpiWarps + 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tail->tmem_base), C::kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == kEpiWarps && lane == 0) {
    ptx::prefetch_tensormap(&tmap_w);
    ptx::prefetch_tensormap(&tmap_a);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;
  // Everything above touches only this CTA's shared memory and TMEM, so under a programmatic dependent launch it
  // runs while the previous kernel of the stream is still finishing; from here on global memory is read and
  // written (activations and workspace may come from that kernel), so every thread waits for it first.
  // The one exception is the weight matrix when the caller has declared it at rest (nothing in flight writes
  // it): the producer then asks for the W half of as many units as the pipeline holds before the wait, so the
  // stream from HBM is already running when the previous kernel drains.  Each stage's barrier expects the whole
  // stage; the activation half follows after the wait.
  ptx::griddep_launch_dependents();
  int early = 0;                                               // stages whose W half is already on its way
  if (p.w_early != 0 && warp == kEpiWarps && lane == 0) {
    const uint64_t w_policy = ptx::l2_policy_evict_first();
    int tile = static_cast<int>(u0 / G), g = static_cast<int>(u0 % G);
    for (long long u = u0; u < u1 && early < C::kStages; ++u, ++early) {
      const uint32_t full = ptx::smem_u32(&tail->full[early]);
      ptx::mbar_arrive_expect_tx(full, C::kStageBytes);
      ptx::tma_load_2d_hint(smem_base + early * C::kStageBytes, &tmap_w, full, g * BK, tile * BN, w_policy);
      if (++g == G) { g = 0; ++tile; }
    }
  }
  ptx::griddep_wait();

  if (warp == kEpiWarps) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // Every byte of W is read exactly once per launch, by one CTA: its lines are marked as the first to leave
      // L2.  With the default policy the stream pushed out what the neighbouring kernels of a decode step and the
      // activation tiles (read by every CTA) keep there: a gate/up GEMM followed by a down GEMM at M = 64 took
      // 67 us per pair instead of the 51 us the two take on their own.
      const uint64_t w_policy = ptx::l2_policy_evict_first();
      uint32_t stage = 0, phase = 0;
      int tile = static_cast<int>(u0 / G), g = static_cast<int>(u0 % G);       // kept incrementally: no division per unit
      for (long long u = u0; u < u1; ++u) {
        const uint32_t full = ptx::smem_u32(&tail->full[stage]);
        const uint32_t w_dst = smem_base + stage * C::kStageBytes;
        if (early > 0) {
          // first pass over the ring, W already requested: nothing to wait for, only the activation half is missing
          --early;
          ptx::tma_load_2d(w_dst + kWBytes, &tmap_a, full, g * BK, 0);
        } else {
          if (!ptx::mbar_wait(ptx::smem_u32(&tail->empty[stage]), phase ^ 1u, abort_flag, p.wait_limit)) break;
          BFP8_TL(0, u - u0);                                   // stage free, copies issued
          ptx::mbar_arrive_expect_tx(full, C::kStageBytes);
          ptx::tma_load_2d_hint(w_dst, &tmap_w, full, g * BK, tile * BN, w_policy);
          ptx::tma_load_2d(w_dst + kWBytes, &tmap_a, full, g * BK, 0);
        }
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        if (++g == G) { g = 0; ++tile; }
      }
    }
  } else if (warp == kEpiWarps + 1 || warp >= kEpiWarps + 3) {
    // ------------------------------------------------------------------ MMA issuers (units first, first + kIssuers, ...)
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::umma_idesc_e4m3(BN, MP);
      const uint32_t first = warp == kEpiWarps + 1 ? 0u : static_cast<uint32_t>(warp - (kEpiWarps + 2));   // 0, 1, 2, 3
      uint32_t stage = first, phase = 0, kb = first;
      for (long long u = u0 + first; u < u1; u += C::kIssuers, kb += C::kIssuers) {
        const uint32_t buf = kb % kAccBufs, acc_phase = (kb / kAccBufs) & 1u;
        if (!ptx::mbar_wait(ptx::smem_u32(&tail->tmem_empty[buf]), acc_phase ^ 1u, abort_flag, p.wait_limit)) break;
        BFP8_TL(1, u - u0);                                     // TMEM buffer free
        if (!ptx::mbar_wait(ptx::smem_u32(&tail->full[stage]), phase, abort_flag, p.wait_limit)) break;
        BFP8_TL(2, u - u0);                                     // operands landed
        ptx::tc_fence_after_sync();
        const uint32_t w_addr = smem_base + stage * C::kStageBytes;
        const uint64_t w_desc = ptx::umma_desc_k128(w_addr);
        const uint64_t a_desc = ptx::umma_desc_k128(w_addr + kWBytes);
        const uint32_t d = tmem_base + buf * MP;
#pragma unroll
        for (int k4 = 0; k4 < BK / 32; ++k4)
          ptx::umma_f8(d, w_desc + 2u * k4, a_desc + 2u * k4, idesc, k4 > 0);
        ptx::umma_commit(ptx::smem_u32(&tail->empty[stage]));
        ptx::umma_commit(ptx::smem_u32(&tail->tmem_full[buf]));
        BFP8_TL(3, u - u0);                                     // MMAs and commits issued
        stage += C::kIssuers;
        if (stage >= C::kStages) { stage -= C::kStages; phase ^= 1u; }
      }
    }
  } else if (warp == kEpiWarps + 2) {
    // ------------------------------------------------------------------ scale loader
    constexpr int kPer = (MP + 31) / 32;                         // activation scales per lane and unit
    // Raw scales of the next kScaleAhead units.  They are multiplied only when their unit comes up: using a
    // loaded value right away would stall this warp for a full L2 round trip on every unit.
    float va[kScaleAhead][kPer], vw[kScaleAhead], vu[kSwiGLU ? kScaleAhead : 1];
    constexpr bool swiglu = kSwiGLU;
    int f_tile = static_cast<int>(u0 / G), f_g = static_cast<int>(u0 % G);   // unit the next fetch belongs to
    auto fetch = [&](float (&dst)[kPer], float& sw, float& su) {
      const int tile = f_tile, g = f_g;
      if (++f_g == G) { f_g = 0; ++f_tile; }
      // SwiGLU form: tile t holds outputs 64 t .. 64 t + 63, i.e. scale block t / 2 of the gate rows and of the up rows
      const int nb = swiglu ? (tile >> 1) : tile;
      sw = __ldg(p.w_scales + static_cast<int64_t>(nb) * G + g);
      su = swiglu ? __ldg(p.w_scales + static_cast<int64_t>((p.inter >> 7) + nb) * G + g) : 0.0f;
      const float* sa = p.a_scales + static_cast<int64_t>(g) * p.ldsa;
#pragma unroll
      for (int q = 0; q < kPer; ++q) {
        const int i = lane + 32 * q;
        dst[q] = (i < p.m) ? __ldg(sa + i) : 0.0f;
      }
    };
#pragma unroll
    for (int i = 0; i < kScaleAhead; ++i)
      if (u0 + i < u1) fetch(va[i], vw[i], vu[kSwiGLU ? i : 0]);
    uint32_t kb = 0;
    bool ok = true;
    for (long long base = u0; base < u1 && ok; base += kScaleAhead) {
#pragma unroll
      for (int i = 0; i < kScaleAhead; ++i) {
        const long long u = base + i;
        if (u < u1 && ok) {
          const uint32_t buf = kb % kAccBufs, acc_phase = (kb / kAccBufs) & 1u;
          // the outcome is made uniform across the warp before the warp-wide barrier below
          ok = __all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&tail->tmem_empty[buf]), acc_phase ^ 1u, abort_flag,
                                                      p.wait_limit));
          if (ok) {
#pragma unroll
            for (int q = 0; q < kPer; ++q)
              if (lane + 32 * q < MP) {
                tail->scale[buf][lane + 32 * q] = va[i][q] * vw[i];
                if (swiglu) tail->scale_up[buf][lane + 32 * q] = va[i][q] * vu[kSwiGLU ? i : 0];
              }
            __syncwarp();
            ptx::mbar_arrive_lane0(ptx::smem_u32(&tail->tmem_full[buf]), lane);
            if (lane == 0) BFP8_TL(7, u - u0);                  // scale products parked
            if (u + kScaleAhead < u1) fetch(va[i], vw[i], vu[kSwiGLU ? i : 0]);
            ++kb;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue / promotion
    const int wrow = warp * 32 + lane;                         // weight row inside the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const int epi_tid = threadIdx.x;                           // 0..127
    // SwiGLU form: the up rows (lanes 64-127) use the up block's scale products
    const float* my_scale = (kSwiGLU && wrow >= 64) ? &tail->scale_up[0][0] : &tail->scale[0][0];
    float acc[MP];
#pragma unroll
    for (int j = 0; j < MP; ++j) acc[j] = 0.0f;
    uint32_t kb = 0;
    long long seg_start = u0;
    bool ok = true;
    int tile = static_cast<int>(u0 / G), g = static_cast<int>(u0 % G) - 1;
    // End of this CTA's segment of a tile (plain form).  The four epilogue warps meet at named barriers here, so a
    // thread whose bounded wait expired still calls this for every remaining segment end (alive == false: it takes
    // part in the barriers and the counter protocol, stores nothing), see the loop after the main one.
    long long u = u0;
    int pending_tile = -1;                                     // tile whose partial is stored but not yet counted in
    // makes this CTA's partial of tile t visible and counts the CTA in at that tile (all 128 epilogue threads)
    auto count_in = [&](int t) {
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (epi_tid == 0) atomicAdd(p.counters + t, 1u);
    };
    auto segment_end = [&](bool alive) {
        // ---- end of this CTA's segment of the tile
        if (u == u1 - 1 && pending_tile >= 0) {                  // last segment: settle what the first one left open
          count_in(pending_tile);
          pending_tile = -1;
        }
        const long long tile_first = static_cast<long long>(tile) * G;
        const int c_first = cta_of_unit(tile_first, p.total_units, parts);
        const int c_last = cta_of_unit(tile_first + G - 1, p.total_units, parts);
        const int col = tile * BN + wrow;
        const bool whole = (seg_start == tile_first) && (g == G - 1);
        bool do_store = whole;
        if (!whole) {
          // The tile's first CTA finishes it.  Its segment is the last thing it does, while the CTAs after it met the
          // tile at the start of their ranges, so their partial sums are normally waiting for it: they store them,
          // fence and count themselves in; the first CTA waits (bounded) for the count, adds the partials to its own
          // registers in CTA order - which is K order, a fixed order, and (0 + own) + p1 + ... is what a sum over
          // stored partials starting from zero gives bit for bit - and stores the tile.  One trip through L2 for
          // the finisher instead of the store / fence / count / read-back chain of a last-arriver scheme.
          // A CTA that meets such a tile at the start of its range only stores its partial there and carries on;
          // the fence and the count follow at its last segment end (count_in), where nothing is left to stall.
          const uint32_t others = static_cast<uint32_t>(c_last - c_first);
          if (static_cast<int>(blockIdx.x) != c_first) {
            // partial slot: 0 if this tile is the CTA's first, else 1
            const int slot = (static_cast<long long>(tile) == u0 / G) ? 0 : 1;
            float* dst = p.partials + (static_cast<int64_t>(blockIdx.x) * 2 + slot) * (MP * BN);
#pragma unroll
            for (int j = 0; j < MP; ++j) dst[j * BN + wrow] = acc[j];
            if (u == u1 - 1) count_in(tile);
            else pending_tile = tile;
          } else {
            if (epi_tid == 0) {
              uint32_t arrived = 1u;
              const long long t0 = clock64();
              while (ptx::ld_acquire_gpu_u32(p.counters + tile) != others) {
                if (*abort_flag != 0) { arrived = 0u; break; }
                if (clock64() - t0 > p.wait_limit) { *abort_flag = 1; arrived = 0u; break; }
              }
              if (arrived != 0u) p.counters[tile] = 0;            // leave the workspace reusable
              tail->last_flag = arrived;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            do_store = tail->last_flag != 0;
            if (do_store) {
              __threadfence();
              for (int c = c_first + 1; c <= c_last; ++c) {        // fixed order: results are run-to-run identical
                const int cslot = (static_cast<long long>(tile) == first_unit(c, p.total_units, parts) / G) ? 0 : 1;
                const float* src = p.partials + (static_cast<int64_t>(c) * 2 + cslot) * (MP * BN);
#pragma unroll
                for (int j = 0; j < MP; ++j)
                  if (j < p.m) acc[j] += __ldcg(src + j * BN + wrow);
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");        // last_flag may be rewritten next segment
          }
        }
        if (kSwiGLU) {
          // SwiGLU form: do_store is the same for all 128 threads, so the barriers inside are safe
          if (do_store) {
            constexpr int kRound = MP < kSwigluRows ? MP : kSwigluRows;
#pragma unroll
            for (int j0 = 0; j0 < MP; j0 += kRound)
              swiglu_finish<kRound>(p, swiglu_ex, tile, wrow, acc + j0, j0, kRound, alive);
          }
        } else if (do_store && alive && col < p.n) {
          const float b = p.bias != nullptr ? __ldg(p.bias + col) : 0.0f;
          if (p.out_bf16 && p.push_world > 0) {
#pragma unroll
            for (int j = 0; j < MP; ++j)
              if (j < p.m) out_row_bf16(p, j)[col] = static_cast<uint16_t>(float_to_bf16_bits(acc[j] + b));
          } else if (p.out_bf16) {
            uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + col;
#pragma unroll
            for (int j = 0; j < MP; ++j)
              if (j < p.m) o[static_cast<int64_t>(j) * p.ldo] = static_cast<uint16_t>(float_to_bf16_bits(acc[j] + b));
          } else {
            float* o = reinterpret_cast<float*>(p.out) + col;
#pragma unroll
            for (int j = 0; j < MP; ++j)
              if (j < p.m) o[static_cast<int64_t>(j) * p.ldo] = acc[j] + b;
          }
        }
#pragma unroll
        for (int j = 0; j < MP; ++j) acc[j] = 0.0f;
        seg_start = u + 1;
    };
    for (; u < u1; ++u, ++kb) {
      if (++g == G) { g = 0; ++tile; }
      if (threadIdx.x == 0) BFP8_TL(4, u - u0);                 // epilogue turns to the unit
      const uint32_t buf = kb % kAccBufs, acc_phase = (kb / kAccBufs) & 1u;
      // uniform across the warp before the warp-collective TMEM loads
      ok = __all_sync(0xffffffffu,
                      ptx::mbar_wait(ptx::smem_u32(&tail->tmem_full[buf]), acc_phase, abort_flag, p.wait_limit));
      if (!ok) break;
      if (threadIdx.x == 0) BFP8_TL(5, u - u0);                 // accumulator and scales ready
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + lane_addr + buf * MP;
      constexpr int kChunk = MP < 64 ? MP : 64;                  // columns fetched per TMEM round trip
#pragma unroll
      for (int h = 0; h < MP / kChunk; ++h) {
        uint32_t r[kChunk / 16][16];
#pragma unroll
        for (int c = 0; c < kChunk / 16; ++c) ptx::tmem_ld16(taddr + h * kChunk + c * 16, r[c]);
        float s[kChunk];
#pragma unroll
        for (int j = 0; j < kChunk; j += 4) {
          const float4 t4 = *reinterpret_cast<const float4*>(&my_scale[buf * 128 + h * kChunk + j]);
          s[j] = t4.x; s[j + 1] = t4.y; s[j + 2] = t4.z; s[j + 3] = t4.w;
        }
        ptx::tmem_wait_ld16(r[0]);
#pragma unroll
        for (int c = 1; c < kChunk / 16; ++c) ptx::tmem_regs_ready16(r[c]);
        if (h == MP / kChunk - 1) {
          // every column of the unit and its scales are in registers: the buffer (and the scale slot beside it) goes
          // back before the FMAs are issued, so the barrier operation completes under the arithmetic instead of in
          // front of the next unit's poll
          ptx::tc_fence_before_sync();
          __syncwarp();
          ptx::mbar_arrive_lane0(ptx::smem_u32(&tail->tmem_empty[buf]), lane);
          if (threadIdx.x == 0) BFP8_TL(6, u - u0);             // buffer handed back
        }
#pragma unroll
        for (int c = 0; c < kChunk / 16; ++c)
#pragma unroll
          for (int j = 0; j < 16; ++j)
            acc[h * kChunk + c * 16 + j] = fmaf(__uint_as_float(r[c][j]), s[c * 16 + j], acc[h * kChunk + c * 16 + j]);
      }
      if (!kCluster && (g == G - 1 || u == u1 - 1)) segment_end(true);
    }
    if (!kCluster && !ok) {
      // this thread gave up inside unit u (g and tile already stand at that unit): walk the rest of the list and
      // keep every appointment at the segment ends; the siblings see the abort flag at their next wait and follow
      for (bool first = true; u < u1; ++u, first = false) {
        if (!first && ++g == G) { g = 0; ++tile; }
        if (g == G - 1 || u == u1 - 1) segment_end(false);
      }
    }
    if (kCluster) {
      // ---- reduce-scatter of the cluster's partials through distributed shared memory
      // #1: every CTA of the cluster is done with its pipeline buffers, which now receive the partials
      ptx::cluster_sync_all();
      const int rows_per = MP / cs;                               // padded rows each CTA owns (cs divides MP)
      const int shift = 31 - __clz(rows_per);
      const uint32_t recv = smem_base;                            // [source rank][row of the owner][weight row] fp32
      if (ok) {
#pragma unroll
        for (int j = 0; j < MP; ++j) {
          if (j < p.m) {
            const uint32_t owner = static_cast<uint32_t>(j >> shift), jj = static_cast<uint32_t>(j & (rows_per - 1));
            ptx::st_cluster_f32(ptx::cluster_map(recv, owner) + ((crank * rows_per + jj) * BN + wrow) * 4u, acc[j]);
          }
        }
      }
      // #2: all partials have arrived
      ptx::cluster_sync_all();
      const int col = static_cast<int>(ctile) * BN + wrow;
      if (kSwiGLU) {
        // SwiGLU form: this CTA's rows in rounds of kSwigluRows; every epilogue thread takes part in the barriers
        const float* mine = reinterpret_cast<const float*>(smem);
        constexpr int kRound = 16;
        for (int jj0 = 0; jj0 < rows_per; jj0 += kRound) {
          float v[kRound];
#pragma unroll
          for (int q = 0; q < kRound; ++q) v[q] = 0.0f;
          for (int r = 0; r < cs; ++r) {                           // rank order = K order; the rows' sums side by side
#pragma unroll
            for (int q = 0; q < kRound; ++q)
              if (jj0 + q < rows_per) v[q] += mine[(r * rows_per + jj0 + q) * BN + wrow];
          }
          swiglu_finish<kRound>(p, swiglu_ex, static_cast<int>(ctile), wrow, v, crank * rows_per + jj0,
                                min(kRound, rows_per - jj0), ok);
        }
      } else if (ok && col < p.n) {
        const float b = p.bias != nullptr ? __ldg(p.bias + col) : 0.0f;
        const float* mine = reinterpret_cast<const float*>(smem);
        // four rows at a time, their sums formed side by side (each is a chain of cs dependent shared-memory loads
        // and adds; one row after the other leaves the thread waiting on every link of every chain)
        for (int jj0 = 0; jj0 < rows_per; jj0 += 4) {
          float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
          for (int r = 0; r < cs; ++r) {                           // rank order = K order
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (jj0 + q < rows_per) sum[q] += mine[(r * rows_per + jj0 + q) * BN + wrow];
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int j = crank * rows_per + jj0 + q;
            if (jj0 + q < rows_per && j < p.m) {
              const float v = sum[q] + b;
              if (p.out_bf16)
                out_row_bf16(p, j)[col] = static_cast<uint16_t>(float_to_bf16_bits(v));
              else
                reinterpret_cast<float*>(p.out)[static_cast<int64_t>(j) * p.ldo + col] = v;
            }
          }
        }
      }
    }
  }
  if (kCluster && warp >= kEpiWarps) {
    // the other roles take part in the two cluster barriers of the exchange
    ptx::cluster_sync_all();
    ptx::cluster_sync_all();
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  BFP8_TL_DUMP(g_timeline_smallm);
  ptx::idle_after_abort(abort_flag);
  if (warp == kEpiWarps + 1) ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  if (threadIdx.x == 0 && tail->abort_flag != 0) atomicOr(p.status, BFP8_STATUS_WAIT_TIMEOUT);
}

template <int MP, bool kSwiGLU>
int launch(const CUtensorMap& tmap_w, const CUtensorMap& tmap_a, const Params& p, int grid, cudaStream_t st) {
  using C = Cfg<MP>;
  constexpr int smem = 1024 + C::kStages * C::kStageBytes + sizeof(SmemTail) + (kSwiGLU ? kSwigluExBytes : 0);
  static DeviceFlags done;
  const int rc = ensure_smem_limit(gemm_smallm_kernel<MP, false, kSwiGLU>, smem, done);
  if (rc != BFP8_OK) return rc;
  // launched so that the set-up of this kernel may overlap the tail of the previous kernel in the stream
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(C::kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  BFP8_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_smallm_kernel<MP, false, kSwiGLU>, tmap_w, tmap_a, p));
  return BFP8_OK;
}

// Cluster form: p.tiles clusters of p.cluster CTAs.  Returns BFP8_ERR_UNSUPPORTED without launching when the
// device cannot hold all clusters at once (the caller then uses the plain form).
template <int MP, bool kSwiGLU>
int launch_clustered(const CUtensorMap& tmap_w, const CUtensorMap& tmap_a, const Params& p, cudaStream_t st) {
  using C = Cfg<MP>;
  constexpr int smem = 1024 + C::kStages * C::kStageBytes + sizeof(SmemTail) + (kSwiGLU ? kSwigluExBytes : 0);
  static_assert(MP * BN * 4 <= C::kStages * C::kStageBytes, "the exchange area reuses the pipeline buffers");
  static DeviceFlags done;
  const int rc = ensure_smem_limit(gemm_smallm_kernel<MP, true, kSwiGLU>, smem, done);
  if (rc != BFP8_OK) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.tiles * p.cluster), 1, 1);
  cfg.blockDim = dim3(C::kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(p.cluster);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  // co-residency of all clusters, asked once per device and cluster size (index log2(cluster) - 1)
  static std::atomic<int> max_clusters[64][3];
  int dev = 0;
  BFP8_CUDA_TRY(cudaGetDevice(&dev));
  const int slot = p.cluster == 2 ? 0 : p.cluster == 4 ? 1 : 2;
  int cap = (dev >= 0 && dev < 64) ? max_clusters[dev][slot].load(std::memory_order_acquire) : 0;
  if (cap == 0) {
    BFP8_CUDA_TRY(cudaOccupancyMaxActiveClusters(&cap, gemm_smallm_kernel<MP, true, kSwiGLU>, &cfg));
    if (cap <= 0) cap = -1;
    if (dev >= 0 && dev < 64) max_clusters[dev][slot].store(cap, std::memory_order_release);
  }
  if (cap < p.tiles) return BFP8_ERR_UNSUPPORTED;
  BFP8_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_smallm_kernel<MP, true, kSwiGLU>, tmap_w, tmap_a, p));
  return BFP8_OK;
}

}  // namespace


// Cluster form where it applies (and the device can hold all clusters at once), else the plain form.
template <bool kSwiGLU>
int dispatch(int mp, const CUtensorMap& tmap_w, const CUtensorMap& tmap_a, Params& p, int grid, cudaStream_t st) {
  if (p.cluster >= 2) {
    int crc;
    switch (mp) {
      case 16: crc = launch_clustered<16, kSwiGLU>(tmap_w, tmap_a, p, st); break;
      case 32: crc = launch_clustered<32, kSwiGLU>(tmap_w, tmap_a, p, st); break;
      case 64: crc = launch_clustered<64, kSwiGLU>(tmap_w, tmap_a, p, st); break;
      default: crc = launch_clustered<128, kSwiGLU>(tmap_w, tmap_a, p, st); break;
    }
    if (crc != BFP8_ERR_UNSUPPORTED) return crc;
    p.cluster = 0;
  }
  switch (mp) {
    case 16: return launch<16, kSwiGLU>(tmap_w, tmap_a, p, grid, st);
    case 32: return launch<32, kSwiGLU>(tmap_w, tmap_a, p, grid, st);
    case 64: return launch<64, kSwiGLU>(tmap_w, tmap_a, p, grid, st);
    default: return launch<128, kSwiGLU>(tmap_w, tmap_a, p, grid, st);
  }
}

int smallm_padded_rows(int64_t m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }

// The arrival counters always occupy the first 64 KB of the workspace, whatever the shape, so a
// workspace that is shared by calls of different shapes never sees partial sums where counters live.
constexpr int64_t kMaxTiles = 16384;
constexpr size_t kCounterBytes = kMaxTiles * sizeof(uint32_t);

bool smallm_supported(int64_t n) { return (n + BN - 1) / BN <= kMaxTiles; }

size_t smallm_workspace_bytes(int64_t m, int64_t n, int max_ctas) {
  (void)n;
  return kCounterBytes + static_cast<size_t>(max_ctas) * 2 * smallm_padded_rows(m) * BN * sizeof(float);
}

// Grid size: every CTA should stream the same number of 16 KB units, and as few CTAs as possible should
// end inside a tile (each such end costs a partial-sum round trip through the workspace).  With no more
// tiles than SMs every tile gets the same whole number of CTAs, so a CTA holds exactly one K range of one
// tile.  With more tiles than SMs there are two candidates: the unit list cut evenly over all SMs (every CTA
// then ends inside a tile), or the smallest grid that gives every CTA the same number of whole tiles (224 tiles
// on 148 SMs: 112 CTAs with two tiles each, no partial sums, a quarter of the SMs idle).  Which one is faster
// depends on how much the idle SMs would have contributed, so both are priced with figures measured on B200:
// the rate one CTA streams W at for each padded row count (the epilogue paces it as the row count grows), the
// rate HBM delivers to all of them together, and the cost of the partial-sum round trip.
int smallm_grid(int64_t tiles, int64_t groups, int sms, int mp) {
  const long long units = tiles * groups;
  if (units < sms) return static_cast<int>(units);
  if (tiles <= sms) {
    long long per_tile = sms / tiles;
    if (per_tile > groups) per_tile = groups;
    return static_cast<int>(tiles * per_tile);
  }
  const int64_t waves = (tiles + sms - 1) / sms;
  const int64_t whole_grid = (tiles + waves - 1) / waves;
  if (tiles % whole_grid != 0) return sms;                 // no grid of whole tiles with this many waves
  const double per_cta_gbs = mp <= 16 ? 64.0 : mp <= 32 ? 53.0 : mp <= 64 ? 44.0 : 27.0;
  const double round_trip_us = mp <= 16 ? 3.0 : mp <= 32 ? 5.0 : mp <= 64 ? 6.5 : 11.5;
  const double hbm_gbs = 7200.0;                           // read-only stream, all SMs
  const double unit_kb = kWBytes / 1e3;
  const double whole_rate = per_cta_gbs * whole_grid < hbm_gbs ? per_cta_gbs : hbm_gbs / whole_grid;
  const double even_rate = per_cta_gbs * sms < hbm_gbs ? per_cta_gbs * sms : hbm_gbs;
  const double whole_us = static_cast<double>(waves * groups) * unit_kb / whole_rate;
  const double even_us = static_cast<double>(units) * unit_kb / even_rate + round_trip_us;
  return whole_us <= even_us ? static_cast<int>(whole_grid) : sms;
}

// CTAs per tile for the cluster form, or 0 when it does not apply: at most half as many tiles as SMs, a
// power of two up to the portable cluster size of 8, and no more CTAs than the tile has K blocks.
int smallm_cluster_size(int64_t tiles, int64_t groups, int sms) {
  if (tiles * 2 > sms) return 0;
  const long long per_tile = sms / tiles;
  int cs = per_tile >= 8 ? 8 : per_tile >= 4 ? 4 : 2;
  while (cs > groups) cs >>= 1;
  return cs >= 2 ? cs : 0;
}

// Process-wide promise of the caller that the weight codes given to the decode-bucket GEMMs are not written by
// anything still in flight (bfp8_set_weights_at_rest).
static std::atomic<int> g_weights_at_rest{0};

int set_weights_at_rest(int on) { return g_weights_at_rest.exchange(on != 0 ? 1 : 0, std::memory_order_relaxed); }

int launch_gemm_smallm(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                       const uint8_t* w_codes, int64_t ldw, const float* w_scales, const float* bias, void* out,
                       int out_dtype, int64_t ldo, int64_t m, int64_t n, int64_t k, void* workspace,
                       uint32_t* status_dev, long long wait_limit, int max_ctas, int inter, const SmallPush* push,
                       cudaStream_t st) {
  // inter > 0 selects the SwiGLU form: W has n = 2 * inter interleaved rows, `out` is bf16 [m, inter]
  // push != nullptr selects the push form: bf16 rows go to the receive areas of the GPUs that own them
  // max_ctas > 0 (a caller-imposed CTA limit, used by tests and by the entry point with the built-in scratch)
  // also keeps the launch on the plain, non-cluster form
  const int mp = smallm_padded_rows(m);
  alignas(64) CUtensorMap tmap_w, tmap_a;
  int rc = make_tensor_map_2d(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, w_codes, k, n, ldw, BK, BN);
  if (rc != BFP8_OK) return rc;
  rc = make_tensor_map_2d(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a_codes, k, m, lda, BK, mp);
  if (rc != BFP8_OK) return rc;
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
  p.tiles = static_cast<int>((n + BN - 1) / BN);
  p.out_bf16 = out_dtype == BFP8_OUT_BF16;
  p.total_units = static_cast<long long>(p.tiles) * p.groups;
  p.wait_limit = wait_limit;
  p.status = status_dev;
  const int sms = sm_count();
  int grid = smallm_grid(p.tiles, p.groups, sms, mp);
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  p.counters = reinterpret_cast<uint32_t*>(workspace);
  p.partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + kCounterBytes);
  p.inter = inter;
  p.push_world = p.push_rank = 0;
  p.push_rows = 1;
  for (int o = 0; o < 8; ++o) p.push_recv[o] = nullptr;
  if (push != nullptr) {
    if (out_dtype != BFP8_OUT_BF16 || inter > 0 || push->world < 2 || push->world > 8 || push->rows <= 0 ||
        m != static_cast<int64_t>(push->rows) * push->world)
      return BFP8_ERR_UNSUPPORTED;
    p.push_world = push->world;
    p.push_rank = push->rank;
    p.push_rows = push->rows;
    for (int o = 0; o < push->world; ++o) p.push_recv[o] = reinterpret_cast<uint16_t*>(const_cast<void*>(push->recv[o]));
  }
  p.cluster = max_ctas > 0 ? 0 : smallm_cluster_size(p.tiles, p.groups, sms);
  p.w_early = g_weights_at_rest.load(std::memory_order_relaxed);
  if (inter > 0) return dispatch<true>(mp, tmap_w, tmap_a, p, grid, st);
  return dispatch<false>(mp, tmap_w, tmap_a, p, grid, st);
}

// ---------------------------------------------------------------------------------------------
// Entry point that allocates nothing
// ---------------------------------------------------------------------------------------------
namespace {

// Scratch of bfp8_gemm_block128_noalloc: the 64 KB of per-tile arrival counters followed by room for two
// fp32 partial tiles (32 padded rows x 128 columns) from each of up to 160 CTAs - 5,308,416 bytes in all.
// It is part of the library image: every GPU that loads libbfp8.so holds it until the process exits.
constexpr int kNoAllocMaxRows = 32;
constexpr int kNoAllocMaxCtas = 160;
constexpr size_t kNoAllocScratchBytes =
    kCounterBytes + static_cast<size_t>(kNoAllocMaxCtas) * 2 * kNoAllocMaxRows * BN * sizeof(float);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Device address of the scratch array on the current device.  In host code the array's name is only a
// handle for the runtime, never a pointer a kernel may use, so the address is asked for with that device
// current.  The lookup is a host-side table query and is repeated on every call rather than cached: a cached
// address would be wrong after the device's context has been destroyed and re-created (cudaDeviceReset), and a
// shared cache would need synchronisation between host threads.
int noalloc_scratch_address(void** out) {
  void* p = nullptr;
  BFP8_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
  if (p == nullptr) return BFP8_ERR_CUDA;
  *out = p;
  return BFP8_OK;
}

}  // namespace
}  // namespace bfp8

// The small-M GEMM for callers that cannot hand the library a workspace because they cannot allocate
// one at the point of the call - an inference server that gave all device memory to its own pools at
// start-up and runs its decode steps with the allocator closed, or host code running where CUDA
// allocation calls are not allowed (they synchronise the whole device).  The scratch the weight-streaming
// schedule needs lives in a fixed array inside the library instead; the price is a hard size limit.
//
// Same arguments and results as bfp8_gemm_block128 (minus the workspace), for m <= 32 and
// n <= 2,097,152.  Larger problems return BFP8_ERR_TOO_LARGE and launch nothing.  The call performs no
// cudaMalloc / cudaFree and uses no allocating library routine.  Every call asks the runtime for the scratch
// array's device address; the first call on each device also raises the kernel's shared-memory limit; make it
// before any stream capture.  All calls on a device share the one array: the counters are cleared on the
// stream at the start of every call (the partial sums need no clearing, they are written before they are
// read), and two calls that may overlap on the GPU - different streams, or different host threads - race
// on it.
extern "C" int bfp8_gemm_block128_noalloc(const uint8_t* a_codes, int64_t lda, const float* a_scales, int64_t ldsa,
                                          const uint8_t* w_codes, int64_t ldw, const float* w_scales,
                                          const float* bias, void* out, int out_dtype, int64_t ldo,
                                          int64_t m, int64_t n, int64_t k, uint32_t* status_dev, void* stream) {
  using namespace bfp8;
  if (!a_codes || !a_scales || !w_codes || !w_scales || !out || !status_dev) return BFP8_ERR_NULL;
  if (m <= 0 || n <= 0 || k <= 0 || k > (1 << 30)) return BFP8_ERR_SHAPE;
  if (m > kNoAllocMaxRows || !smallm_supported(n)) return BFP8_ERR_TOO_LARGE;
  if (lda < k || ldw < k || ldo < n || ldsa < m) return BFP8_ERR_SHAPE;
  if (out_dtype != BFP8_OUT_F32 && out_dtype != BFP8_OUT_BF16) return BFP8_ERR_SHAPE;
  if (!aligned(a_codes, 16) || !aligned(w_codes, 16) || lda % 16 != 0 || ldw % 16 != 0) return BFP8_ERR_ALIGN;
  if (!aligned(a_scales, 4) || !aligned(w_scales, 4) || !aligned(status_dev, 4)) return BFP8_ERR_ALIGN;
  if (bias && !aligned(bias, 4)) return BFP8_ERR_ALIGN;
  if (!aligned(out, out_dtype == BFP8_OUT_BF16 ? 2 : 4)) return BFP8_ERR_ALIGN;
  void* scratch = nullptr;
  const int rc = noalloc_scratch_address(&scratch);
  if (rc != BFP8_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t counter_bytes = static_cast<size_t>((n + BN - 1) / BN) * sizeof(uint32_t);
  BFP8_CUDA_TRY(cudaMemsetAsync(scratch, 0, counter_bytes, st));
  return launch_gemm_smallm(a_codes, lda, a_scales, ldsa, w_codes, ldw, w_scales, bias, out, out_dtype, ldo, m, n, k,
                            scratch, status_dev, /*wait_limit=*/2000000000LL, kNoAllocMaxCtas, /*inter=*/0, /*push=*/nullptr, st);
}

#ifdef BFP8_TIMELINE
// Diagnostic build only: the timeline of CTA kTimelineCta of the last small-M launch on the current device
// ([kTimelineEvents][kTimelineUnits] %clock values; 0 = not reached).  Synchronises the device.
extern "C" int bfp8_timeline_read_smallm(unsigned int* dst_host) {
  BFP8_CUDA_TRY(cudaDeviceSynchronize());
  BFP8_CUDA_TRY(cudaMemcpyFromSymbol(dst_host, bfp8::g_timeline_smallm, sizeof(unsigned int) * bfp8::kTimelineEvents * bfp8::kTimelineUnits));
  return BFP8_OK;
}
#endif
