// Gated-MLP kernels for sm_100a: persistent, warp-specialised bf16 GEMM tiles
// on tcgen05 with accumulators in tensor memory, operands staged by TMA.
//
//   mode PLAIN  : C[M,N]  = A[M,K] * B[N,K]^T
//   mode GATEUP : Hd[M,I] = silu(X * Wg^T) (.) (X * Wu^T)
//
// Two variants of one kernel template:
//
//   CTAS == 2 (opt-in, DF_GEMM_CTAS=2): a cluster of two CTAs on neighbouring SMs
//     computes one 256 x 256 accumulator tile with tcgen05.mma.cta_group::2.
//     Each CTA stages its own 128 rows of A and ONE HALF of the B tile
//     (128 of the 256 B rows), so a CTA moves 32 KB per 64-wide k-block through
//     L2 -> shared memory instead of 48 KB, and six stages fit instead of four.
//     Every CTA issues its own (plain, non-broadcast) TMA loads; their bytes are
//     counted on the leader CTA's mbarrier. The leader's single MMA thread drives
//     both SMs' tensor cores; each CTA's epilogue drains its own 128 TMEM lanes.
//   CTAS == 1 (default): one CTA per 128 x 256 tile, four 48 KB stages.
//
// 256 threads per CTA:
//   warp 0      TMA producer (one lane)
//   warp 1      MMA issuer (one lane; leader CTA only when CTAS == 2)
//   warp 2      allocates / frees the 512 tensor-memory columns
//   warps 4..7  epilogue: tcgen05.ld of the finished accumulator, SiLU*mul or
//               plain conversion, 16-byte global stores; runs under the MMAs
//               of the next tile thanks to the second accumulator
//
// In GATEUP mode the two B halves of a stage are rows [i0,i0+128) of W_gate and
// of W_up, so the accumulator holds gate in columns [0,128) and up in
// [128,256) for the same 128 output columns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/dynaflow_b200.h"
#include "gemm_internal.h"
#include "host_util.h"
#include "ptx.cuh"

namespace df {

constexpr int BM = 128;        // rows of A (and of the accumulator) per CTA
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int ACC_COLS = 256;  // fp32 accumulator columns per tile (= MMA N)
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_HALF_BYTES = 128 * BK * 2;
constexpr int GEMM_THREADS = 256;
constexpr int TMEM_COLS = 512;

template <int CTAS>
struct TileCfg {
  static constexpr int kStages = (CTAS == 2) ? 6 : 4;
  static constexpr int kBBytes = (CTAS == 2) ? B_HALF_BYTES : 2 * B_HALF_BYTES;  // per CTA
  static constexpr int kStageBytes = A_BYTES + kBBytes;
  static constexpr int kTileM = BM * CTAS;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 512 /*barriers, tile ring*/;
};

// 1-CTA tiles take their stage geometry at run time: a launch with at most 64 rows of A copies
// only 16, 32 or 64 of them per stage (the MMA still spans 128 accumulator rows; the rows
// beyond the box read whatever follows in the stage, and are never stored), which leaves room
// for more stages -- more weight bytes in flight per SM, the quantity that bounds a launch
// that streams the weights once.
constexpr int kMaxSmemBytes = 227 * 1024;
constexpr int kMaxStages = 12;
static inline int stage_bytes_for(int a_rows) { return a_rows * BK * 2 + 2 * B_HALF_BYTES; }
static inline int stages_for(int a_rows) {
  int n = (kMaxSmemBytes - 1024 - 512) / stage_bytes_for(a_rows);
  return n > kMaxStages ? kMaxStages : n;
}

enum : int { MODE_PLAIN = 0, MODE_GATEUP = 1, MODE_FUSED = 2 };  // FUSED: gate/up tiles then down tiles, one launch
enum : unsigned { WHERE_PRODUCER = 1, WHERE_MMA_FULL = 2, WHERE_MMA_TMEM = 3, WHERE_EPILOGUE = 4 };

#ifdef DF_DEV_KNOBS
constexpr bool kDevKnobs = true;
#else
constexpr bool kDevKnobs = false;
#endif

constexpr int kMaxChunks = 64;

// MODE_FUSED only: the tile index space is a sequence of chunks, each a group of row panels in
// one phase (0 = gate/up, 1 = down), ordered so that the down tiles of a group come one group
// behind its gate/up tiles.
struct FusedChunk {
  int start;    // first tile index of the chunk
  int phase;
  int first_m;  // first row panel of the group
  int gm;       // row panels in the group
};

struct GemmParams {
  int M, N, K;  // N = output columns (I in GATEUP mode)
  int ldc;
  // MODE_FUSED, phase 1 (down projection): C2[M, N2] = h[M, K2] * w_down[N2, K2]^T
  int N2, ldc2, num_kb2, tiles_n2, n_chunks;
  __nv_bfloat16* C2;
  unsigned int* panel_done;  // [tiles_m] gate/up tiles finished per row panel, zero at launch
  int tiles_m, tiles_n, num_tiles, num_kb, group_m;
  // Stream-K (1-CTA tiles only; sk_per == 0 means off): the launch's k-blocks, tile after
  // tile, are cut into equal ranges of sk_per units, one range per CTA, so that every SM
  // streams its share of the weights even when there are fewer tiles than SMs.
  int sk_per;
  // Two slots of 256 x 128 fp32 per CTA (slot 0: a segment that starts inside a tile, slot 1: one
  // that starts a tile). Regular form: [accumulator column][row]; operand-swapped form: [row of A][256].
  float* sk_partials;
  unsigned int* sk_counters;  // [num_tiles] partial segments delivered, zero at launch
  // Dynamic tile order (1-CTA whole-tile launches with a workspace): the first tile of a CTA is
  // its block index, the next ones come from this counter (zero at launch), so a CTA that
  // shares its SM with the reduction kernel of the other micro-batch simply takes fewer tiles.
  unsigned int* tile_counter;
  // Row count known only on the device (tokens routed to an expert): if non-NULL, the kernel
  // processes min(*m_dev, M) rows and M is the capacity the tensor maps were built for.
  const int* m_dev;
  int debug;  // DF_DEV_KNOBS builds only: bit 0 = producer skips the copies, bit 1 = epilogue skips the stores
  // 1-CTA tiles: a_rows = rows of A a stage has room for (a multiple of 16, at most 128), a_tx =
  // bytes one copy of A delivers (its box has exactly the launch's rows when there are fewer than
  // 128, so that no copy runs past the matrix: such rows cost a measured 0.3 us per k-block),
  // stages = pipeline depth.
  int a_rows, a_tx, stages;
  FusedChunk chunks[kMaxChunks];
  unsigned long long timeout_ns;
  __nv_bfloat16* C;
  Status* status;
};

// Tile order: groups of `group_m` row panels; inside a group the row panel
// varies fastest, so the CTAs of one wave share few distinct A and B tiles
// and those stay in L2, and the weights stream from HBM once per group.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tiles_m, int t, int& m_blk, int& n_blk) {
  const int per_group = p.group_m * p.tiles_n;
  const int group = t / per_group;
  const int within = t - group * per_group;
  const int first_m = group * p.group_m;
  const int gm = min(p.group_m, tiles_m - first_m);
  m_blk = first_m + within % gm;
  n_blk = within / gm;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// One stretch of consecutive k-blocks of one tile, processed by one CTA (or CTA pair).
struct Segment {
  int tile, kb0, kb1;
  int phase;         // MODE_FUSED: 0 = gate/up tile, 1 = down tile; otherwise 0
  int m_blk, n_blk;  // tile coordinates
};

// MODE_FUSED: tile index -> (phase, row panel, column tile); `hint` caches the chunk.
__device__ __forceinline__ void fused_coords(const GemmParams& p, int t, int& hint, Segment& s) {
  while (hint + 1 < p.n_chunks && t >= p.chunks[hint + 1].start) ++hint;
  while (hint > 0 && t < p.chunks[hint].start) --hint;
  const FusedChunk& c = p.chunks[hint];
  const int within = t - c.start;
  s.phase = c.phase;
  s.m_blk = c.first_m + within % c.gm;
  s.n_blk = within / c.gm;
}

constexpr int kSchedSlots = 4;
enum : int { ROLE_PRODUCER = 0, ROLE_MMA = 1, ROLE_EPILOGUE = 2 };

// Hand-off of dynamically fetched tile indices from the producer warp to the MMA thread and
// the epilogue warps: a small ring in shared memory guarded by two mbarriers per slot.
struct SchedRing {
  uint64_t* full;      // [kSchedSlots] one arrival: the producer published a tile index
  uint64_t* empty;     // [kSchedSlots] five arrivals: MMA thread + four epilogue warps read it
  volatile int* tile;  // [kSchedSlots] tile index, -1 = no more work
  unsigned int* counter;
};

// The sequence of segments of a CTA. Static: whole tiles unit, unit + num_units, ...
// Dynamic: whole tiles, the first one = unit, then whatever the global counter hands out.
// Stream-K: the units [unit * sk_per, (unit + 1) * sk_per) of the tile-major k-block sequence,
// cut at tile boundaries. All three warp roles walk the same sequence.
struct SegmentIter {
  int cur, end, step, num_kb, num_tiles, tiles_m, iter, first, grid, hint;
  bool streamk, dynamic, fused;
  const GemmParams* gp;
  // rows_tiles_m / rows_num_tiles: the tile grid of the rows actually present (device-side row count)
  __device__ SegmentIter(const GemmParams& p, int rows_tiles_m, int rows_num_tiles, int unit, int num_units,
                         bool is_fused) {
    gp = &p;
    fused = is_fused;
    hint = 0;
    num_kb = p.num_kb;
    tiles_m = rows_tiles_m;
    num_tiles = rows_num_tiles;
    streamk = p.sk_per > 0;
    dynamic = !streamk && p.tile_counter != nullptr;
    iter = 0;
    first = unit;
    grid = num_units;
    if (streamk) {
      const long long total = static_cast<long long>(rows_num_tiles) * p.num_kb;
      const long long b = static_cast<long long>(unit) * p.sk_per;
      const long long e = b + p.sk_per;
      cur = static_cast<int>(b < total ? b : total);
      end = static_cast<int>(e < total ? e : total);
      step = 0;
    } else {
      cur = unit;
      end = rows_num_tiles;
      step = num_units;
    }
  }
  // fills phase, coordinates and (for whole tiles) the k range of segment s from s.tile
  __device__ __forceinline__ void locate(Segment& s, bool whole) {
    if (fused) {
      fused_coords(*gp, s.tile, hint, s);
      if (whole) {
        s.kb0 = 0;
        s.kb1 = s.phase ? gp->num_kb2 : num_kb;
      }
    } else {
      s.phase = 0;
      tile_coords(*gp, tiles_m, s.tile, s.m_blk, s.n_blk);
      if (whole) {
        s.kb0 = 0;
        s.kb1 = num_kb;
      }
    }
  }
  // ROLE_PRODUCER and ROLE_MMA: called by one thread. ROLE_EPILOGUE: by whole warps.
  template <int ROLE>
  __device__ bool next(Segment& s, const SchedRing& ring, const Deadline& dl, int lane) {
    if (dynamic) {
      const int slot = iter % kSchedSlots;
      const uint32_t round = static_cast<uint32_t>(iter / kSchedSlots);
      int t;
      if (ROLE == ROLE_PRODUCER) {
        t = (iter == 0) ? first : grid + static_cast<int>(atomicAdd(ring.counter, 1u));
        if (t >= num_tiles) t = -1;
        if (round > 0 && !mbar_wait(&ring.empty[slot], (round - 1u) & 1u, dl, 6u, static_cast<unsigned>(iter)))
          return false;
        ring.tile[slot] = t;
        mbar_arrive(&ring.full[slot]);  // release: the index is visible to whoever sees the arrival
      } else {
        bool ok = mbar_wait(&ring.full[slot], round & 1u, dl, 6u, static_cast<unsigned>(iter));
        if (ROLE == ROLE_EPILOGUE) ok = __all_sync(0xffffffffu, ok);
        if (!ok) return false;
        t = ring.tile[slot];
        if (ROLE == ROLE_MMA) {
          mbar_arrive(&ring.empty[slot]);
        } else {
          __syncwarp();
          if (lane == 0) mbar_arrive(&ring.empty[slot]);
        }
      }
      ++iter;
      if (t < 0) return false;
      s.tile = t;
      locate(s, true);
      return true;
    }
    if (cur >= end) return false;
    if (streamk) {
      s.tile = cur / num_kb;
      s.kb0 = cur - s.tile * num_kb;
      const int tile_end = (s.tile + 1) * num_kb;
      const int stop = tile_end < end ? tile_end : end;
      s.kb1 = s.kb0 + (stop - cur);
      cur = stop;
      locate(s, false);
    } else {
      s.tile = cur;
      cur += step;
      locate(s, true);
    }
    return true;
  }
};

enum : unsigned { WHERE_SK_PARTIALS = 5 };

// SKINNY (at most 64 rows of A, 1-CTA tiles, stream-K or whole tiles): the operands swap roles
// in the MMA. The 128 weight rows of each half of the B stage span the accumulator's lanes and
// the a_rows rows of A its columns, D0 = B0 * A^T in columns [0, a_rows) and D1 = B1 * A^T in
// [a_rows, 2 a_rows). All 128 epilogue threads then own one output column each and a few values
// per row of A, so folding the stream-K partial sums takes a handful of loads per thread
// instead of a chain of 256-column sweeps by the few threads that own valid rows.
template <int MODE, int CTAS, bool SKINNY = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b0,
               const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_a2,
               const __grid_constant__ CUtensorMap tm_b2, const GemmParams p_in) {
  using Cfg = TileCfg<CTAS>;
  constexpr bool FUSED = MODE == MODE_FUSED;
  const GemmParams& p = p_in;
  // rows actually present: the host's M, or what the device-side count says (at most M)
  int rows_m = p.M, rows_tiles_m = p.tiles_m, rows_num_tiles = p.num_tiles;
  if (!FUSED && p.m_dev != nullptr) {
    const int m = *p.m_dev;
    rows_m = m < 0 ? 0 : (m < p.M ? m : p.M);
    rows_tiles_m = (rows_m + Cfg::kTileM - 1) / Cfg::kTileM;
    rows_num_tiles = rows_tiles_m * p.tiles_n;
  }
  const int STAGES = (CTAS == 2) ? Cfg::kStages : p.stages;
  const int A_STAGE_BYTES = (CTAS == 2) ? A_BYTES : p.a_rows * (BK * 2);
  const int STAGE_BYTES = (CTAS == 2) ? Cfg::kStageBytes : A_STAGE_BYTES + 2 * B_HALF_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);

  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* sched_full = tempty + 2;
  uint64_t* sched_empty = sched_full + kSchedSlots;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sched_empty + kSchedSlots);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile int* sched_tile = reinterpret_cast<volatile int*>(tmem_slot + 2);
  const SchedRing ring{sched_full, sched_empty, sched_tile, p.tile_counter};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;  // 0 = leader
  const int unit = (CTAS == 2) ? (blockIdx.x >> 1) : blockIdx.x;   // CTA or CTA pair
  const int num_units = (CTAS == 2) ? (gridDim.x >> 1) : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], (CTAS == 2) ? 8 : 128);  // CTAS == 2: one arrival per epilogue warp of both CTAs
    }
    for (int i = 0; i < kSchedSlots; ++i) {
      mbar_init(&sched_full[i], 1);
      mbar_init(&sched_empty[i], 5);
    }
    *abort_flag = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b0);
    tma_prefetch_desc(&tm_b1);
    if (FUSED) {
      tma_prefetch_desc(&tm_a2);
      tma_prefetch_desc(&tm_b2);
    }
  }
  if (warp == 2) {
    if (CTAS == 2) {
      tmem_alloc_2cta(tmem_slot, TMEM_COLS);
      tmem_relinquish_2cta();
    } else {
      tmem_alloc(tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if (CTAS == 2) {
    cluster_sync();  // the peer's barriers exist before anything signals them
  } else {
    __syncthreads();
  }
  tc_fence_after();

  const uint32_t tmem_base = *tmem_slot;
  const Deadline dl{globaltimer_ns() + p.timeout_ns, abort_flag, p.status};

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer
    // (Prefetching operand boxes or weight-row chunks into L2 ahead of the copies was measured
    // and made every shape slower, by 20 % to 3x.)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      SegmentIter segs(p, rows_tiles_m, rows_num_tiles, unit, num_units, FUSED);
      Segment sg;
      while (ok && segs.next<ROLE_PRODUCER>(sg, ring, dl, 0)) {
        const int t = sg.tile;
        // per-tile operator: compile-time except in the fused launch
        const int tmode = FUSED ? (sg.phase ? MODE_PLAIN : MODE_GATEUP) : MODE;
        const int bn_out = (tmode == MODE_GATEUP) ? 128 : 256;
        const int m0 = sg.m_blk * Cfg::kTileM + static_cast<int>(cta_rank) * BM;
        const int n0 = sg.n_blk * bn_out;
        const int y1_1cta = (tmode == MODE_GATEUP) ? n0 : n0 + 128;
        const CUtensorMap* map_a = (FUSED && sg.phase) ? &tm_a2 : &tm_a;
        const CUtensorMap* map_b0 = (FUSED && sg.phase) ? &tm_b2 : &tm_b0;
        const CUtensorMap* map_b1 = (tmode == MODE_GATEUP) ? &tm_b1 : map_b0;
        if (FUSED && sg.phase) {
          // the down tile reads the intermediate rows of its panel: wait until every gate/up tile
          // of that panel has published them (they were handed out before this tile)
          const unsigned need = static_cast<unsigned>(p.tiles_n);
          uint32_t spins = 0;
          while (ld_acquire_gpu(p.panel_done + sg.m_blk) < need) {
            if ((++spins & 0xffu) == 0u) {
              if (*dl.abort) {
                ok = false;
                break;
              }
              if (globaltimer_ns() > dl.t_end) {
                *dl.abort = 1u;
                report(dl.status, 1u, 7u, static_cast<unsigned>(t));
                ok = false;
                break;
              }
            }
          }
          if (!ok) break;
          fence_proxy_async_global();  // those rows were written with ordinary stores, TMA reads them
        }
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, dl, WHERE_PRODUCER, t)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          if (kDevKnobs && (p.debug & 1)) {
            if (cta_rank == 0) mbar_arrive(&full[stage]);
          } else if (CTAS == 2) {
            // this CTA's half of B: gate rows on the leader, up rows on its peer (GATEUP);
            // B rows [n0, n0+128) on the leader and [n0+128, n0+256) on its peer (PLAIN)
            const CUtensorMap* map_b = (tmode == MODE_GATEUP && cta_rank == 1) ? &tm_b1 : &tm_b0;
            const int yb = (tmode == MODE_GATEUP) ? n0 : n0 + static_cast<int>(cta_rank) * 128;
            // both CTAs' bytes are counted on the leader's barrier, which the MMA thread waits on
            const uint32_t bar = mapa_shared(smem_u32(&full[stage]), 0u);
            if (cta_rank == 0) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);
            tma_load_2d_2cta(sa, &tm_a, bar, kb * BK, m0);
            tma_load_2d_2cta(sb, map_b, bar, kb * BK, yb);
          } else {
            mbar_expect_tx(&full[stage], p.a_tx + 2 * B_HALF_BYTES);
            tma_load_2d(sa, map_a, &full[stage], kb * BK, m0);
            tma_load_2d(sb, map_b0, &full[stage], kb * BK, n0);
            tma_load_2d(sb + B_HALF_BYTES, map_b1, &full[stage], kb * BK, y1_1cta);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM * CTAS, ACC_COLS);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      SegmentIter segs(p, rows_tiles_m, rows_num_tiles, unit, num_units, FUSED);
      Segment sg;
      for (; ok && segs.next<ROLE_MMA>(sg, ring, dl, 0); ++it) {
        const int t = sg.tile;
        const int acc = it & 1;
        const uint32_t aphase = (it >> 1) & 1u;
        if (!mbar_wait(&tempty[acc], aphase ^ 1u, dl, WHERE_MMA_TMEM, t)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * ACC_COLS);
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, dl, WHERE_MMA_FULL, t)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t da = make_desc_k_sw128(a_addr);
          const uint64_t db = make_desc_k_sw128(a_addr + A_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing 16 elements along K = 32 bytes = 2 descriptor units
            if (SKINNY) {
              // (Spreading the k-steps over several accumulators per half, so that consecutive MMAs
              // do not add to the same columns, was measured and changed nothing: an MMA of 16
              // columns takes about 110 cycles either way.)
              const uint32_t acc_flag = (kb > sg.kb0 || k > 0) ? 1u : 0u;
              const uint32_t idesc_s = make_idesc_bf16(128, p.a_rows);
              umma_bf16(d_tmem, db + 2u * k, da + 2u * k, idesc_s, acc_flag);
              umma_bf16(d_tmem + static_cast<uint32_t>(p.a_rows), db + (B_HALF_BYTES >> 4) + 2u * k, da + 2u * k, idesc_s,
                        acc_flag);
            } else if (CTAS == 2) {
              umma_bf16_2cta(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb > sg.kb0 || k > 0) ? 1u : 0u);
            } else {
              umma_bf16(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb > sg.kb0 || k > 0) ? 1u : 0u);
            }
          }
          if (CTAS == 2) {
            umma_commit_2cta(&empty[stage]);  // frees the stage in both CTAs
          } else {
            umma_commit(&empty[stage]);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          if (CTAS == 2) {
            umma_commit_2cta(&tfull[acc]);
          } else {
            umma_commit(&tfull[acc]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ---------------------------------------------------------- epilogue
    const int q = warp - 4;  // == warp % 4: the TMEM lane quarter this warp may read
    int it = 0;
    int sk_pending = 0, sk_tile[2] = {0, 0}, sk_n0[2] = {0, 0}, sk_mblk[2] = {0, 0};  // stream-K: tiles this CTA delivered partial sums for
    SegmentIter segs(p, rows_tiles_m, rows_num_tiles, unit, num_units, FUSED);
    Segment sg;
    for (; segs.next<ROLE_EPILOGUE>(sg, ring, dl, lane); ++it) {
      const int t = sg.tile;
      const int tmode = FUSED ? (sg.phase ? MODE_PLAIN : MODE_GATEUP) : MODE;
      const int m_blk = sg.m_blk;
      const int n0 = sg.n_blk * ((tmode == MODE_GATEUP) ? 128 : 256);
      const int row_in_tile = q * 32 + lane;
      const int row = m_blk * Cfg::kTileM + static_cast<int>(cta_rank) * BM + row_in_tile;
      __nv_bfloat16* const c_base = (FUSED && sg.phase) ? p.C2 : p.C;
      const int c_ld = (FUSED && sg.phase) ? p.ldc2 : p.ldc;
      const int c_cols = (FUSED && sg.phase) ? p.N2 : p.N;
      const int acc = it & 1;
      const uint32_t aphase = (it >> 1) & 1u;
      bool ok = mbar_wait(&tfull[acc], aphase, dl, WHERE_EPILOGUE, t);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + static_cast<uint32_t>(acc * ACC_COLS) + (static_cast<uint32_t>(q * 32) << 16);
      __nv_bfloat16* crow = c_base + static_cast<size_t>(row) * c_ld;
      const bool row_ok = row < rows_m && !(kDevKnobs && (p.debug & 2));

      if (SKINNY) {
        // this thread owns weight row i of both halves: output column n0 + i (gate/up), or the
        // columns n0 + i and n0 + 128 + i (plain); the accumulator columns are the rows of A
        const int i = row_in_tile;
        const int n_rows = p.a_rows;
        const bool whole = p.sk_per == 0 || (sg.kb0 == 0 && sg.kb1 == p.num_kb);
        // Stream-K: every segment that is not a whole tile delivers its partial sums, [row of A]
        // [256] fp32 (the 128 D0 lanes, then the 128 D1 lanes), to one of this CTA's two slots --
        // slot 0 for a segment that starts inside a tile, slot 1 for one that starts a tile. The
        // tile is finished after the segment loop, by all of its contributors together.
        float* mine = p.sk_partials + static_cast<size_t>(2 * unit + (sg.kb0 > 0 ? 0 : 1)) * (ACC_COLS * BM);
        const int col0 = n0 + i;
        const int col1 = (tmode == MODE_GATEUP) ? col0 : col0 + 128;
#pragma unroll 1
        for (int c = 0; c < n_rows / 16; ++c) {
          uint32_t d0[16], d1[16];
          tmem_ld_32x16(t_acc + c * 16, d0);
          tmem_ld_32x16(t_acc + n_rows + c * 16, d1);
          tmem_ld_wait();
          if (!whole) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (c * 16 + j < rows_m) {
                mine[(c * 16 + j) * ACC_COLS + i] = __uint_as_float(d0[j]);
                mine[(c * 16 + j) * ACC_COLS + 128 + i] = __uint_as_float(d1[j]);
              }
            }
            continue;
          }
          if (kDevKnobs && (p.debug & 2)) continue;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int r = c * 16 + j;
            if (r < rows_m) {
              __nv_bfloat16* dst = c_base + static_cast<size_t>(r) * c_ld;
              if (tmode == MODE_GATEUP) {
                const float g = round_bf16(__uint_as_float(d0[j]));
                const float u = round_bf16(__uint_as_float(d1[j]));
                if (col0 < c_cols) dst[col0] = __float2bfloat16_rn((g / (1.0f + expf(-g))) * u);
              } else {
                if (col0 < c_cols) dst[col0] = __float2bfloat16_rn(__uint_as_float(d0[j]));
                if (col1 < c_cols) dst[col1] = __float2bfloat16_rn(__uint_as_float(d1[j]));
              }
            }
          }
        }
        tc_fence_before();
        mbar_arrive(&tempty[acc]);
        if (!whole) {
          __threadfence();
          epilogue_bar_sync();
          if (threadIdx.x == 4 * 32) atomicAdd(p.sk_counters + t, 1u);
          if (sk_pending < 2) {
            sk_tile[sk_pending] = t;
            sk_n0[sk_pending] = n0;
          }
          ++sk_pending;
        }
        continue;
      }

      // ---- stream-K: a segment that is not a whole tile only delivers its fp32 partial sums,
      // [256 accumulator columns][128 rows] per slot (slot 0 for a segment that starts inside a
      // tile, slot 1 for one that starts a tile); the tile is finished after the segment loop.
      if (CTAS == 1 && p.sk_per > 0 && !(sg.kb0 == 0 && sg.kb1 == p.num_kb)) {
        float* mine = p.sk_partials + static_cast<size_t>(2 * unit + (sg.kb0 > 0 ? 0 : 1)) * (ACC_COLS * BM);
#pragma unroll 1
        for (int c = 0; c < ACC_COLS / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c * 32, r);
          tmem_ld_wait();
          if (row < rows_m) {
#pragma unroll
            for (int j = 0; j < 32; ++j) mine[(c * 32 + j) * BM + row_in_tile] = __uint_as_float(r[j]);
          }
        }
        tc_fence_before();
        mbar_arrive(&tempty[acc]);
        __threadfence();
        epilogue_bar_sync();
        if (threadIdx.x == 4 * 32) atomicAdd(p.sk_counters + t, 1u);
        if (sk_pending < 2) {
          sk_tile[sk_pending] = t;
          sk_n0[sk_pending] = n0;
          sk_mblk[sk_pending] = m_blk;
        }
        ++sk_pending;
        continue;
      }

      if (tmode == MODE_GATEUP) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(t_acc + c * 32, g);
          tmem_ld_32x32(t_acc + 128 + c * 32, u);
          tmem_ld_wait();
          uint32_t o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g0 = round_bf16(__uint_as_float(g[2 * j]));
            const float g1 = round_bf16(__uint_as_float(g[2 * j + 1]));
            const float u0 = round_bf16(__uint_as_float(u[2 * j]));
            const float u1 = round_bf16(__uint_as_float(u[2 * j + 1]));
            const float h0 = (g0 / (1.0f + expf(-g0))) * u0;
            const float h1 = (g1 / (1.0f + expf(-g1))) * u1;
            o[j] = pack_bf16x2(h0, h1);
          }
          if (row_ok) {
            const int col = n0 + c * 32;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col + v * 8 < c_cols) {
                *reinterpret_cast<uint4*>(crow + col + v * 8) =
                    make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
              }
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c * 32, r);
          tmem_ld_wait();
          uint32_t o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
          if (row_ok) {
            const int col = n0 + c * 32;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col + v * 8 < c_cols) {
                *reinterpret_cast<uint4*>(crow + col + v * 8) =
                    make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
              }
            }
          }
        }
      }
      if (FUSED && sg.phase == 0) {
        // publish this tile's rows of the intermediate: all 128 threads' stores, then one count
        __threadfence();
        fence_proxy_async_global();
        epilogue_bar_sync();
        if (threadIdx.x == 4 * 32) atomicAdd(p.panel_done + m_blk, 1u);
      }
      tc_fence_before();
      if (CTAS == 2) {
        // the accumulator is free again once every epilogue warp of BOTH CTAs has drained it;
        // the MMA thread that waits for that lives in the leader CTA
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty[acc]), 0u));
      } else {
        mbar_arrive(&tempty[acc]);
      }
    }
    if (!SKINNY && CTAS == 1 && sk_pending > 0 && !*abort_flag) {
      // Finish the tiles this CTA holds partial sums of (see the operand-swapped form below for
      // the protocol). Here a thread owns one row of the tile; the tile's output columns, in
      // groups of eight, are shared out among the S contributors, and each group is summed over
      // the S partials in k order, four partials in flight at a time.
      const int tid = static_cast<int>(threadIdx.x) - 4 * 32;
      constexpr int GROUPS = (MODE == MODE_GATEUP) ? 16 : 32;  // groups of 8 output columns per tile
      for (int k = 0; k < (sk_pending < 2 ? sk_pending : 2); ++k) {
        const int t = sk_tile[k];
        const int first = static_cast<int>((static_cast<long long>(t) * p.num_kb) / p.sk_per);
        const int last = static_cast<int>((static_cast<long long>(t + 1) * p.num_kb - 1) / p.sk_per);
        const int S = last - first + 1;
        const int s_idx = unit - first;
        if (tid == 0) {
          uint32_t spins = 0;
          while (ld_acquire_gpu(p.sk_counters + t) < static_cast<unsigned>(S)) {
            if ((++spins & 0xffu) == 0u) {
              if (*dl.abort) break;
              if (globaltimer_ns() > dl.t_end) {
                *dl.abort = 1u;
                report(dl.status, 1u, WHERE_SK_PARTIALS, static_cast<unsigned>(t));
                break;
              }
            }
          }
        }
        epilogue_bar_sync();
        if (*dl.abort) break;
        const int row = sk_mblk[k] * Cfg::kTileM + tid;
        if (row >= rows_m || (kDevKnobs && (p.debug & 2))) continue;
        const int g_lo = s_idx * GROUPS / S, g_hi = (s_idx + 1) * GROUPS / S;
        // partial o of the tile: contributor first + o; o = 0 started the tile (slot 1), the others slot 0
        const float* base = p.sk_partials + static_cast<size_t>(2 * first) * (ACC_COLS * BM) + tid;
        __nv_bfloat16* crow = p.C + static_cast<size_t>(row) * p.ldc;
#pragma unroll 1
        for (int g = g_lo; g < g_hi; ++g) {
          const float* src = base + static_cast<size_t>(g * 8) * BM;
          float a[8], b[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            a[j] = __ldcg(src + ACC_COLS * BM + j * BM);
            if (MODE == MODE_GATEUP) b[j] = __ldcg(src + ACC_COLS * BM + (128 + j) * BM);
          }
          constexpr int AT_ONCE = (MODE == MODE_GATEUP) ? 2 : 4;
          int o = 1;
#pragma unroll 1
          for (; o + AT_ONCE <= S; o += AT_ONCE) {
            float va[AT_ONCE][8], vb[AT_ONCE][8];
#pragma unroll
            for (int w = 0; w < AT_ONCE; ++w) {
              const float* so = src + static_cast<size_t>(o + w) * (2 * ACC_COLS * BM);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                va[w][j] = __ldcg(so + j * BM);
                if (MODE == MODE_GATEUP) vb[w][j] = __ldcg(so + (128 + j) * BM);
              }
            }
#pragma unroll
            for (int w = 0; w < AT_ONCE; ++w) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                a[j] += va[w][j];
                if (MODE == MODE_GATEUP) b[j] += vb[w][j];
              }
            }
          }
#pragma unroll 1
          for (; o < S; ++o) {
            const float* so = src + static_cast<size_t>(o) * (2 * ACC_COLS * BM);
            float va[8], vb[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              va[j] = __ldcg(so + j * BM);
              if (MODE == MODE_GATEUP) vb[j] = __ldcg(so + (128 + j) * BM);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              a[j] += va[j];
              if (MODE == MODE_GATEUP) b[j] += vb[j];
            }
          }
          const int col = sk_n0[k] + g * 8;
          if (col < p.N) {
            uint32_t o4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (MODE == MODE_GATEUP) {
                const float g0 = round_bf16(a[2 * j]), g1 = round_bf16(a[2 * j + 1]);
                const float u0 = round_bf16(b[2 * j]), u1 = round_bf16(b[2 * j + 1]);
                o4[j] = pack_bf16x2((g0 / (1.0f + expf(-g0))) * u0, (g1 / (1.0f + expf(-g1))) * u1);
              } else {
                o4[j] = pack_bf16x2(a[2 * j], a[2 * j + 1]);
              }
            }
            *reinterpret_cast<uint4*>(crow + col) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
          }
        }
      }
    }
    if (SKINNY && sk_pending > 0 && !*abort_flag) {
      // Finish the tiles this CTA holds partial sums of. Tile t was cut into S segments, held by
      // the consecutive CTAs first..first+S-1 in k order; once all S have delivered, contributor s
      // sums the s-th share of the tile's (row of A, weight row) pairs over the S partials -- in k
      // order, so the result does not depend on timing -- and stores those outputs. Every CTA has
      // delivered all its partial sums before it waits here, so the waits cannot form a cycle.
      const int tid = static_cast<int>(threadIdx.x) - 4 * 32;
      const int c_ld = p.ldc, c_cols = p.N;
      for (int k = 0; k < (sk_pending < 2 ? sk_pending : 2); ++k) {
        const int t = sk_tile[k];
        const int first = static_cast<int>((static_cast<long long>(t) * p.num_kb) / p.sk_per);
        const int last = static_cast<int>((static_cast<long long>(t + 1) * p.num_kb - 1) / p.sk_per);
        const int S = last - first + 1;
        const int s_idx = unit - first;
        if (tid == 0) {
          uint32_t spins = 0;
          while (ld_acquire_gpu(p.sk_counters + t) < static_cast<unsigned>(S)) {
            if ((++spins & 0xffu) == 0u) {
              if (*dl.abort) break;
              if (globaltimer_ns() > dl.t_end) {
                *dl.abort = 1u;
                report(dl.status, 1u, WHERE_SK_PARTIALS, static_cast<unsigned>(t));
                break;
              }
            }
          }
        }
        epilogue_bar_sync();
        if (*dl.abort) break;
        const int E = rows_m * 128;
        const int lo = static_cast<int>(static_cast<long long>(s_idx) * E / S);
        const int hi = static_cast<int>(static_cast<long long>(s_idx + 1) * E / S);
        const float* base = p.sk_partials + static_cast<size_t>(2 * first) * (ACC_COLS * BM);
        // four pairs per pass and four contributors per batch: 32 loads in flight per thread
        for (int e0 = lo + tid; e0 < hi; e0 += 4 * 128) {
          const float* src[4];
          float a0[4], a1[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = min(e0 + u * 128, hi - 1);  // a clamped pair is summed again and not stored
            src[u] = base + (e >> 7) * ACC_COLS + (e & 127);
            // contributor 0 started the tile (slot 1); the others started inside it (slot 0)
            a0[u] = __ldcg(src[u] + ACC_COLS * BM);
            a1[u] = __ldcg(src[u] + ACC_COLS * BM + 128);
          }
          int o = 1;
          for (; o + 4 <= S; o += 4) {
            float v0[4][4], v1[4][4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                v0[w][u] = __ldcg(src[u] + static_cast<size_t>(o + w) * (2 * ACC_COLS * BM));
                v1[w][u] = __ldcg(src[u] + static_cast<size_t>(o + w) * (2 * ACC_COLS * BM) + 128);
              }
            }
#pragma unroll
            for (int w = 0; w < 4; ++w) {
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                a0[u] += v0[w][u];
                a1[u] += v1[w][u];
              }
            }
          }
          for (; o < S; ++o) {
            float v0[4], v1[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              v0[u] = __ldcg(src[u] + static_cast<size_t>(o) * (2 * ACC_COLS * BM));
              v1[u] = __ldcg(src[u] + static_cast<size_t>(o) * (2 * ACC_COLS * BM) + 128);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              a0[u] += v0[u];
              a1[u] += v1[u];
            }
          }
          if (kDevKnobs && (p.debug & 2)) continue;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * 128;
            if (e >= hi) break;
            __nv_bfloat16* dst = p.C + static_cast<size_t>(e >> 7) * c_ld;
            const int col0 = sk_n0[k] + (e & 127);
            if (MODE == MODE_GATEUP) {
              const float g = round_bf16(a0[u]);
              const float up = round_bf16(a1[u]);
              if (col0 < c_cols) dst[col0] = __float2bfloat16_rn((g / (1.0f + expf(-g))) * up);
            } else {
              if (col0 < c_cols) dst[col0] = __float2bfloat16_rn(a0[u]);
              if (col0 + 128 < c_cols) dst[col0 + 128] = __float2bfloat16_rn(a1[u]);
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before();
  if (CTAS == 2) {
    cluster_sync();  // nothing of the pair touches the other CTA's shared or tensor memory after this
  } else {
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after();
    if (*abort_flag) {
      // error path: give copies and MMAs that are still in flight time to land
      // before the tensor memory and shared memory are handed back
      const uint64_t t_stop = globaltimer_ns() + 2000000ull;
      while (globaltimer_ns() < t_stop) __nanosleep(1000);
    }
    if (CTAS == 2) {
      tmem_dealloc_2cta(tmem_base, TMEM_COLS);
    } else {
      tmem_dealloc(tmem_base, TMEM_COLS);
    }
  }
}

// ------------------------------------------------------------------- host

bool make_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  PFN_encodeTiled fn = get_encode_tiled();
  if (fn == nullptr) return false;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu cols=%llu ld=%llu)", static_cast<int>(r),
              static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols),
              static_cast<unsigned long long>(ld));
    return false;
  }
  return true;
}

// Launch-form options (df_set_launch_option): which of the bit-different but equally valid
// forms of a launch is chosen. Process-wide, read at every launch.
static std::atomic<int> g_launch_option[DF_OPT_COUNT_] = {{1}, {1}, {1}, {1}, {1}, {1}};
static int launch_option(int opt) { return g_launch_option[opt].load(std::memory_order_relaxed); }
int launch_option_value(int option) { return (option >= 0 && option < DF_OPT_COUNT_) ? launch_option(option) : 0; }

// Development knobs exist only in builds with -DDF_DEV_KNOBS (integers taken from the
// environment on every launch, among them switches that skip the copies or the stores and so
// produce invalid results, for timing diagnostics). The shipped library compiles them to
// their defaults.
#ifdef DF_DEV_KNOBS
constexpr bool kDevKnobsHost = true;
static int tuning_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  if (v == nullptr || *v == '\0') return fallback;
  const int x = std::atoi(v);
  return x >= 0 ? x : fallback;
}
#else
constexpr bool kDevKnobsHost = false;
static inline int tuning_int(const char*, int fallback) { return fallback; }
#endif

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// How many CTA pairs of the 2-CTA kernel can be resident at once on the current
// device (cached per device and mode); 0 if the query fails.
template <int MODE>
static int max_active_pairs() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] != 0) return cached[dev] > 0 ? cached[dev] : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 256, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = TileCfg<2>::kSmemBytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<MODE, 2>, &cfg);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  cached[dev] = n > 0 ? n : -1;
  return n;
}

constexpr size_t kSkCounterBytes = 8192;                      // up to 2048 tiles
constexpr size_t kSkPartialBytes = 2 * size_t(ACC_COLS) * BM * 4;  // two 128 x 256 fp32 tiles per CTA

static size_t splitk_workspace_bytes_for(int sms) {
  return kSkCounterBytes + static_cast<size_t>(sms) * kSkPartialBytes;
}

template <int MODE, int CTAS>
static int launch_variant(const CUtensorMap& tm_a, const CUtensorMap& tm_b0, const CUtensorMap& tm_b1, GemmParams p,
                          int max_ctas, int sms, void* sk_ws, size_t sk_ws_bytes, cudaStream_t stream,
                          bool skinny = false) {
  using Cfg = TileCfg<CTAS>;
  constexpr int BN_OUT = (MODE == MODE_GATEUP) ? 128 : 256;
  static_assert(MODE != MODE_FUSED, "the fused launch has its own host path");
  // the attribute is per device; setting it on every call is cheap and covers every device that launches
  const int smem_bytes = (CTAS == 2) ? Cfg::kSmemBytes : p.stages * stage_bytes_for(p.a_rows) + 1024 + 512;
  auto kernel = gemm_tc_kernel<MODE, CTAS, false>;
  if constexpr (CTAS == 1) {
    if (skinny) kernel = gemm_tc_kernel<MODE, 1, true>;
  }
  const cudaError_t attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    (CTAS == 2) ? Cfg::kSmemBytes : kMaxSmemBytes);
  if (attr_err != cudaSuccess) return fail(DF_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(attr_err));

  p.tiles_m = (p.M + Cfg::kTileM - 1) / Cfg::kTileM;
  p.tiles_n = (p.N + BN_OUT - 1) / BN_OUT;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.group_m = tuning_int("DF_GEMM_GROUP_M", 32) / CTAS;  // row panels of kTileM rows: the same rows per group
  if (p.group_m < 1) p.group_m = 1;

  int units = (CTAS == 2) ? max_active_pairs<MODE>() : sms;
  if (units <= 0) units = sms / CTAS;
  if (max_ctas > 0 && max_ctas / CTAS < units) units = max_ctas / CTAS;
  if (units < 1) units = 1;
  // Stream-K when whole tiles would leave more than 40 % of the SMs idle and the caller provided
  // scratch for the partial sums. (At 112 tiles on 148 SMs it measured slower than whole tiles.)
  p.sk_per = 0;
  p.sk_partials = nullptr;
  p.sk_counters = nullptr;
  if (CTAS == 1 && sk_ws != nullptr && p.m_dev == nullptr && launch_option(DF_OPT_STREAM_K) != 0) {
    const int waves = (p.num_tiles + units - 1) / units;
    const double eff = static_cast<double>(p.num_tiles) / (static_cast<double>(waves) * units);
    const long long total = static_cast<long long>(p.num_tiles) * p.num_kb;
    // a launch that streams the weights once (few rows) is bound by the bytes in flight: every SM counts
    const double eff_min = 0.01 * tuning_int(skinny ? "DF_GEMM_SK_EFF_SKINNY" : "DF_GEMM_SK_EFF", 60);
    if (eff < eff_min && (p.num_tiles <= units || tuning_int("DF_GEMM_SK_WAVES", 0) != 0) && p.num_kb >= 8 &&
        static_cast<size_t>(p.num_tiles) * 4 <= kSkCounterBytes - 64) {
      long long g = units;
      if (g > total / 4) g = total / 4;  // at least four k-blocks per CTA
      if (g < 1) g = 1;
      const long long per = (total + g - 1) / g;
      const long long grid = (total + per - 1) / per;
      if (kSkCounterBytes + static_cast<size_t>(grid) * kSkPartialBytes <= sk_ws_bytes) {
        p.sk_per = static_cast<int>(per);
        p.sk_counters = static_cast<unsigned int*>(sk_ws);
        p.sk_partials = reinterpret_cast<float*>(static_cast<uint8_t*>(sk_ws) + kSkCounterBytes);
        units = static_cast<int>(grid);
        cudaError_t me = cudaMemsetAsync(p.sk_counters, 0, static_cast<size_t>(p.num_tiles) * 4, stream);
        if (me != cudaSuccess) return fail(DF_ECUDA, "stream-K counter reset: %s", cudaGetErrorString(me));
      }
    }
  }
  if (p.sk_per == 0 && p.num_tiles < units) units = p.num_tiles;
  // whole tiles, more than one per CTA: hand them out dynamically
  p.tile_counter = nullptr;
  if (CTAS == 1 && p.sk_per == 0 && sk_ws != nullptr && sk_ws_bytes >= kSkCounterBytes && p.num_tiles > units &&
      tuning_int("DF_GEMM_DYNAMIC", 1) != 0) {
    p.tile_counter = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(sk_ws) + kSkCounterBytes - 64);
    cudaError_t me = cudaMemsetAsync(p.tile_counter, 0, 4, stream);
    if (me != cudaSuccess) return fail(DF_ECUDA, "tile counter reset: %s", cudaGetErrorString(me));
  }

  if (tuning_int("DF_DEBUG", 0) > 0)
    std::fprintf(stderr, "[df] gemm mode=%d ctas=%d M=%d N=%d K=%d tiles=%d grid=%d group_m=%d streamk_per=%d a_rows=%d stages=%d skinny=%d\n",
                 MODE, CTAS, p.M, p.N, p.K, p.num_tiles, units * CTAS, p.group_m, p.sk_per, p.a_rows, p.stages, int(skinny));

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(units * CTAS, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  if (CTAS == 2) {
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = CTAS;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  } else if (p.sk_per > 0) {
    // In the stream-K finish every contributor of a tile waits for all the others, which is only
    // free of cycles if all CTAs of the grid are resident at once. A cooperative launch makes the
    // runtime guarantee exactly that, whatever else occupies SMs when the grid starts (a second
    // stream-K launch on another stream, the reduction kernel, a graph replay).
    attr.id = cudaLaunchAttributeCooperative;
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b0, tm_b1, tm_a, tm_b0, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(DF_ECUDA, "gemm launch (%d-CTA tiles): %s", CTAS, cudaGetErrorString(e));
  }
  return DF_OK;
}

// out = (silu(x wg^T) (.) (x wu^T)) wd^T as ONE persistent launch: gate/up tiles and down tiles in
// one dynamically handed-out tile sequence; a down tile waits for its row panel's gate/up tiles
// through a per-panel counter. Needs the workspace (tile counter, panel counters).
static int launch_fused_mlp(const void* x, const void* wg, const void* wu, void* h, const void* wd, void* out, int M,
                            int H, int I, int max_ctas, void* sk_ws, size_t sk_ws_bytes, df_status_t* dev_status,
                            cudaStream_t stream) {
  const int sms = df_sm_count();
  if (sms <= 0) return fail(DF_ECUDA, "no CUDA device");
  using Cfg = TileCfg<1>;
  const cudaError_t attr_err = cudaFuncSetAttribute(gemm_tc_kernel<MODE_FUSED, 1>,
                                                    cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (attr_err != cudaSuccess) return fail(DF_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(attr_err));
  CUtensorMap tm_x, tm_g, tm_u, tm_h, tm_d;
  if (!make_map_bf16(&tm_x, x, M, H, H, M < BM ? M : BM)) return DF_ECUDA;
  if (!make_map_bf16(&tm_g, wg, I, H, H, 128)) return DF_ECUDA;
  if (!make_map_bf16(&tm_u, wu, I, H, H, 128)) return DF_ECUDA;
  if (!make_map_bf16(&tm_h, h, M, I, I, M < BM ? M : BM)) return DF_ECUDA;
  if (!make_map_bf16(&tm_d, wd, H, I, I, 128)) return DF_ECUDA;

  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.M = M;
  p.N = I;
  p.K = H;
  p.ldc = I;
  p.C = static_cast<__nv_bfloat16*>(h);
  p.N2 = H;
  p.ldc2 = H;
  p.C2 = static_cast<__nv_bfloat16*>(out);
  p.num_kb = (H + BK - 1) / BK;
  p.num_kb2 = (I + BK - 1) / BK;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (I + 127) / 128;
  p.tiles_n2 = (H + 255) / 256;
  p.num_tiles = p.tiles_m * (p.tiles_n + p.tiles_n2);
  p.timeout_ns = timeout_ns();
  p.status = reinterpret_cast<Status*>(dev_status);
  p.debug = tuning_int("DF_GEMM_DEBUG", 0);
  p.a_rows = BM;
  p.a_tx = (M < BM ? M : BM) * BK * 2;
  p.stages = Cfg::kStages;
  int g = tuning_int("DF_GEMM_GROUP_M", 32);
  if (g < 1) g = 1;
  // The down projection's tiles of a group are handed out in sub-groups of `gd` row panels: their
  // rows of the intermediate (gd x 3.7 MB at I = 14336) are read once per column tile, and with
  // all 32 panels (117 MB) between two reads of a panel they do not stay in L2 beside the weights.
  int gd = tuning_int("DF_GEMM_GROUP_M_DOWN", 16);
  if (gd < 1 || gd > g) gd = g;
  while (((p.tiles_m + g - 1) / g) * (1 + (g + gd - 1) / gd) > kMaxChunks) {
    g *= 2;
    gd *= 2;
  }
  p.group_m = g;
  // chunk order: up(0), up(1), down(0), up(2), down(1), ..., down(last): a group's down tiles come one
  // group behind its gate/up tiles, so their inputs are long finished when they are handed out
  const int groups = (p.tiles_m + g - 1) / g;
  int start = 0, n = 0;
  auto add = [&](int phase, int grp) {
    const int group_first = grp * g;
    const int group_gm = (p.tiles_m - group_first) < g ? (p.tiles_m - group_first) : g;
    const int step = phase ? gd : g;
    for (int off = 0; off < group_gm; off += step) {
      const int gm = (group_gm - off) < step ? (group_gm - off) : step;
      p.chunks[n].start = start;
      p.chunks[n].phase = phase;
      p.chunks[n].first_m = group_first + off;
      p.chunks[n].gm = gm;
      start += gm * (phase ? p.tiles_n2 : p.tiles_n);
      ++n;
    }
  };
  for (int grp = 0; grp < groups; ++grp) {
    add(0, grp);
    if (grp >= 1) add(1, grp - 1);
  }
  add(1, groups - 1);
  p.n_chunks = n;

  if (sk_ws == nullptr || sk_ws_bytes < kSkCounterBytes || static_cast<size_t>(p.tiles_m) * 4 > kSkCounterBytes - 64)
    return fail(DF_EINVAL, "the fused MLP launch needs the workspace for its tile and panel counters");
  p.panel_done = static_cast<unsigned int*>(sk_ws);
  p.tile_counter = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(sk_ws) + kSkCounterBytes - 64);
  cudaError_t me = cudaMemsetAsync(p.panel_done, 0, static_cast<size_t>(p.tiles_m) * 4, stream);
  if (me == cudaSuccess) me = cudaMemsetAsync(p.tile_counter, 0, 4, stream);
  if (me != cudaSuccess) return fail(DF_ECUDA, "counter reset: %s", cudaGetErrorString(me));

  int units = sms;
  if (max_ctas > 0 && max_ctas < units) units = max_ctas;
  if (p.num_tiles < units) units = p.num_tiles;
  if (tuning_int("DF_DEBUG", 0) > 0)
    std::fprintf(stderr, "[df] fused mlp M=%d H=%d I=%d tiles=%d grid=%d group_m=%d chunks=%d\n", M, H, I, p.num_tiles,
                 units, p.group_m, p.n_chunks);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(units, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<MODE_FUSED, 1>, tm_x, tm_g, tm_u, tm_h, tm_d, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(DF_ECUDA, "fused MLP launch: %s", cudaGetErrorString(e));
  }
  return DF_OK;
}

template <int MODE>
static int launch_gemm(const void* a, const void* b0, const void* b1, void* c, int M, int N, int K, int lda, int ldb,
                       int ldc, int max_ctas, void* sk_ws, size_t sk_ws_bytes, df_status_t* dev_status, void* stream,
                       const int* m_dev = nullptr) {
  if (a == nullptr || b0 == nullptr || b1 == nullptr || c == nullptr || dev_status == nullptr)
    return fail(DF_EINVAL, "NULL pointer argument");
  if (M <= 0 || N <= 0 || K <= 0) return fail(DF_EINVAL, "M, N, K must be positive (got %d, %d, %d)", M, N, K);
  if ((N % 8) != 0 || (K % 8) != 0) return fail(DF_EUNSUPPORTED, "N and K must be multiples of 8 (got %d, %d)", N, K);
  if (lda < K || ldb < K || ldc < N || (lda % 8) != 0 || (ldb % 8) != 0 || (ldc % 8) != 0)
    return fail(DF_EINVAL, "leading dimensions must cover the row and be multiples of 8");
  if (!aligned16(a) || !aligned16(b0) || !aligned16(b1) || !aligned16(c))
    return fail(DF_EINVAL, "matrix base pointers must be 16-byte aligned");
  if (sk_ws != nullptr && (reinterpret_cast<uintptr_t>(sk_ws) & 255u) != 0)
    return fail(DF_EINVAL, "the stream-K workspace must be 256-byte aligned");

  int sms = df_sm_count();
  if (sms <= 0) return fail(DF_ECUDA, "no CUDA device");

  // At most 128 rows: the split-K kernel made for launches that stream the weights once.
  if (M <= BM && m_dev == nullptr && launch_option(DF_OPT_SPLIT_K_SMALL) != 0 && tuning_int("DF_GEMM_CTAS", 1) != 2) {
    int units = sms;
    if (max_ctas > 0 && max_ctas < units) units = max_ctas;
    const int r = launch_small_rows(MODE == MODE_GATEUP, a, b0, b1, c, M, N, K, lda, ldb, ldc, units,
                                    launch_option(DF_OPT_STREAM_K) != 0, tuning_int("DF_SMALL_BH", 0),
                                    tuning_int("DF_SMALL_SPLITS", 0), dev_status, static_cast<cudaStream_t>(stream));
    if (r != DF_SMALL_NOT_APPLICABLE) return r;
  }

  // Otherwise, at most 128 rows: the operand-swapped form with a smaller A stage and a deeper pipeline.
  const bool skinny = M <= tuning_int("DF_GEMM_SKINNY_ROWS", 128) && M <= BM && m_dev == nullptr && launch_option(DF_OPT_OPERAND_SWAP) != 0 &&
                      tuning_int("DF_GEMM_CTAS", 1) != 2;
  const int a_rows = skinny ? ((M + 15) / 16) * 16 : BM;
  const int a_box_rows = M < BM ? M : BM;  // a launch of fewer than 128 rows never copies past its last row
  CUtensorMap tm_a, tm_b0, tm_b1;
  if (!make_map_bf16(&tm_a, a, M, K, lda, a_box_rows)) return DF_ECUDA;
  if (!make_map_bf16(&tm_b0, b0, N, K, ldb, 128)) return DF_ECUDA;
  if (!make_map_bf16(&tm_b1, b1, N, K, ldb, 128)) return DF_ECUDA;

  GemmParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.num_kb = (K + BK - 1) / BK;
  p.timeout_ns = timeout_ns();
  p.C = static_cast<__nv_bfloat16*>(c);
  p.status = reinterpret_cast<Status*>(dev_status);
  p.tiles_m = p.tiles_n = p.num_tiles = p.group_m = 0;
  p.sk_per = 0;
  p.sk_partials = nullptr;
  p.sk_counters = nullptr;
  p.tile_counter = nullptr;
  p.m_dev = m_dev;
  p.debug = tuning_int("DF_GEMM_DEBUG", 0);
  p.a_rows = a_rows;
  p.a_tx = a_box_rows * BK * 2;
  p.stages = skinny ? stages_for(a_rows) : TileCfg<1>::kStages;
  const int stage_cap = tuning_int("DF_GEMM_STAGES", 0);  // development only: a shallower pipeline
  if (stage_cap >= 2 && stage_cap < p.stages) p.stages = stage_cap;

  // One CTA per tile is the default: measured on B200 under the power cap, the CTA-pair
  // variant moves a third less data from L2 but keeps the tensor pipe slightly less busy
  // (67 % vs 75 % active on a 1024-row gate/up launch), and the two end up within +-3 %.
  // DF_GEMM_CTAS=2 selects the pair variant.
  const int want = tuning_int("DF_GEMM_CTAS", 1);
  const bool two = want == 2 && M > BM && (max_ctas <= 0 || max_ctas >= 2) && m_dev == nullptr;
  if (two)
    return launch_variant<MODE, 2>(tm_a, tm_b0, tm_b1, p, max_ctas, sms, nullptr, 0, static_cast<cudaStream_t>(stream));
  return launch_variant<MODE, 1>(tm_a, tm_b0, tm_b1, p, max_ctas, sms, sk_ws, sk_ws_bytes,
                                 static_cast<cudaStream_t>(stream), skinny);
}

}  // namespace df

extern "C" {

int df_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, int lda, int ldb, int ldc, int max_ctas,
                 df_status_t* dev_status, void* stream) {
  return df::launch_gemm<df::MODE_PLAIN>(a, b, b, c, M, N, K, lda, ldb, ldc, max_ctas, nullptr, 0, dev_status, stream);
}

int df_gemm_bf16_ws(const void* a, const void* b, void* c, int M, int N, int K, int lda, int ldb, int ldc, int max_ctas,
                    void* splitk_ws, size_t splitk_ws_bytes, df_status_t* dev_status, void* stream) {
  return df::launch_gemm<df::MODE_PLAIN>(a, b, b, c, M, N, K, lda, ldb, ldc, max_ctas, splitk_ws, splitk_ws_bytes,
                                         dev_status, stream);
}

int df_gateup_silu_bf16(const void* x, const void* w_gate, const void* w_up, void* h, int M, int H, int I, int ldx,
                        int ldw, int ldh, int max_ctas, df_status_t* dev_status, void* stream) {
  return df::launch_gemm<df::MODE_GATEUP>(x, w_gate, w_up, h, M, I, H, ldx, ldw, ldh, max_ctas, nullptr, 0, dev_status,
                                          stream);
}

int df_gateup_silu_bf16_ws(const void* x, const void* w_gate, const void* w_up, void* h, int M, int H, int I, int ldx,
                           int ldw, int ldh, int max_ctas, void* splitk_ws, size_t splitk_ws_bytes,
                           df_status_t* dev_status, void* stream) {
  return df::launch_gemm<df::MODE_GATEUP>(x, w_gate, w_up, h, M, I, H, ldx, ldw, ldh, max_ctas, splitk_ws,
                                          splitk_ws_bytes, dev_status, stream);
}

int df_set_launch_option(int option, int value) {
  if (option < 0 || option >= DF_OPT_COUNT_) return df::fail(DF_EINVAL, "unknown launch option %d", option);
  df::g_launch_option[option].store(value != 0 ? 1 : 0, std::memory_order_relaxed);
  return DF_OK;
}

size_t df_gemm_splitk_workspace_bytes(void) {
  const int sms = df_sm_count();
  return df::splitk_workspace_bytes_for(sms > 0 ? sms : 148);
}

static size_t mlp_h_bytes(int M, int I) {
  const size_t h_bytes = static_cast<size_t>(M) * static_cast<size_t>(I) * 2u;
  return ((h_bytes + 255u) / 256u) * 256u + 256u;
}

size_t df_mlp_workspace_bytes(int M, int H, int I) {
  (void)H;
  if (M <= 0 || I <= 0) return 0;
  return mlp_h_bytes(M, I) + df_gemm_splitk_workspace_bytes();
}

int df_mlp_gated_bf16(const void* x, const void* w_gate, const void* w_up, const void* w_down, void* out,
                      void* workspace, int M, int H, int I, int max_ctas, df_status_t* dev_status, void* stream) {
  if (workspace == nullptr) return df::fail(DF_EINVAL, "workspace is NULL");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return df::fail(DF_EINVAL, "workspace must be 256-byte aligned");
  if (M <= 0 || I <= 0) return df::fail(DF_EINVAL, "M and I must be positive");
  void* h = workspace;
  void* sk = static_cast<uint8_t*>(workspace) + mlp_h_bytes(M, I);
  const size_t sk_bytes = df_gemm_splitk_workspace_bytes();
  // One persistent launch for both GEMMs once there is more than a wave of gate/up tiles and the
  // down projection has enough tiles to fill the SMs (below that the stream-K forms of the two
  // separate launches do better); DF_MLP_FUSED=0 disables it.
  const int sms = df_sm_count();
  const int units = (max_ctas > 0 && max_ctas < sms) ? max_ctas : sms;
  const long long up_tiles = static_cast<long long>((M + 127) / 128) * ((I + 127) / 128);
  const long long down_tiles = static_cast<long long>((M + 127) / 128) * ((H + 127) / 128);
  const bool down_wants_stream_k = down_tiles <= units && down_tiles * 10 < static_cast<long long>(units) * 6;
  if (sms > 0 && up_tiles > units && !down_wants_stream_k && df::launch_option(DF_OPT_MLP_ONE_LAUNCH) != 0 && (H % 8) == 0 && (I % 8) == 0 &&
      x != nullptr && w_gate != nullptr && w_up != nullptr && w_down != nullptr && out != nullptr &&
      dev_status != nullptr && df::aligned16(x) && df::aligned16(w_gate) && df::aligned16(w_up) &&
      df::aligned16(w_down) && df::aligned16(out))
    return df::launch_fused_mlp(x, w_gate, w_up, h, w_down, out, M, H, I, max_ctas, sk, sk_bytes, dev_status,
                                static_cast<cudaStream_t>(stream));
  int r = df_gateup_silu_bf16_ws(x, w_gate, w_up, h, M, H, I, H, H, I, max_ctas, sk, sk_bytes, dev_status, stream);
  if (r != DF_OK) return r;
  return df_gemm_bf16_ws(h, w_down, out, M, H, I, I, I, H, max_ctas, sk, sk_bytes, dev_status, stream);
}

int df_mlp_gated_bf16_rows_on_device(const void* x, const void* w_gate, const void* w_up, const void* w_down, void* out,
                                     void* workspace, int capacity_rows, const int* rows_dev, int H, int I, int max_ctas,
                                     df_status_t* dev_status, void* stream) {
  if (workspace == nullptr || rows_dev == nullptr) return df::fail(DF_EINVAL, "workspace or rows_dev is NULL");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return df::fail(DF_EINVAL, "workspace must be 256-byte aligned");
  if (capacity_rows <= 0 || I <= 0) return df::fail(DF_EINVAL, "capacity_rows and I must be positive");
  void* h = workspace;
  void* sk = static_cast<uint8_t*>(workspace) + mlp_h_bytes(capacity_rows, I);
  const size_t sk_bytes = df_gemm_splitk_workspace_bytes();
  int r = df::launch_gemm<df::MODE_GATEUP>(x, w_gate, w_up, h, capacity_rows, I, H, H, H, I, max_ctas, sk, sk_bytes,
                                           dev_status, stream, rows_dev);
  if (r != DF_OK) return r;
  return df::launch_gemm<df::MODE_PLAIN>(h, w_down, w_down, out, capacity_rows, H, I, I, I, H, max_ctas, sk, sk_bytes,
                                         dev_status, stream, rows_dev);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Variant of df_mlp_gated_bf16 that allocates nothing: the bf16 intermediate
// lives in a static device array owned by the library.
//
// In host code `g_mlp_static_scratch` is only a handle for the runtime's symbol
// table, not a device address: its device address is looked up per device with
// cudaGetSymbolAddress (below) and that pointer is what the kernels receive.
namespace df {

static __device__ __align__(256) unsigned char g_mlp_static_scratch[DF_MLP_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static std::mutex g_static_mutex;
static void* g_static_scratch_ptr[kMaxDevices] = {};

// Device address of the static scratch on the CURRENT device; resolved on the
// first call for that device and cached. Allocates nothing.
static int static_scratch_of_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(DF_ECUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  }
  if (dev < 0 || dev >= kMaxDevices) return fail(DF_EUNSUPPORTED, "device index %d is outside [0, %d)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_mlp_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      return fail(DF_ECUDA, "cudaGetSymbolAddress(static MLP scratch) on device %d: %s", dev, cudaGetErrorString(e));
    }
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return DF_OK;
}

}  // namespace df

extern "C" int df_mlp_gated_bf16_static(const void* x, const void* w_gate, const void* w_up, const void* w_down,
                                        void* out, int M, int H, int I, int max_ctas, df_status_t* dev_status,
                                        void* stream) {
  if (M <= 0 || H <= 0 || I <= 0) return df::fail(DF_EINVAL, "M, H, I must be positive (got %d, %d, %d)", M, H, I);
  const unsigned long long need = 2ull * static_cast<unsigned long long>(M) * static_cast<unsigned long long>(I);
  if (need > DF_MLP_STATIC_SCRATCH_BYTES)
    return df::fail(DF_EUNSUPPORTED,
                    "intermediate of %d x %d bf16 needs %llu bytes, the static scratch holds %u; "
                    "use df_mlp_gated_bf16 with a caller-owned workspace",
                    M, I, need, static_cast<unsigned>(DF_MLP_STATIC_SCRATCH_BYTES));
  void* h = nullptr;
  int r = df::static_scratch_of_current_device(&h);
  if (r != DF_OK) return r;
  r = df_gateup_silu_bf16(x, w_gate, w_up, h, M, H, I, H, H, I, max_ctas, dev_status, stream);
  if (r != DF_OK) return r;
  return df_gemm_bf16(h, w_down, out, M, H, I, I, I, H, max_ctas, dev_status, stream);
}
