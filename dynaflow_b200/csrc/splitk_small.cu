// Split-K GEMM for launches of at most 128 rows (a decode step's projections): the weights are
// streamed exactly once and every other cost is latency, so the launch is shaped to put all
// weight bytes in flight at once and to exchange partial sums without leaving the SMs.
//
//   PLAIN  : C[M,N]  = A[M,K] * B[N,K]^T
//   GATEUP : Hd[M,I] = silu(X * Wg^T) (.) (X * Wu^T)
//
// One CTA per (output tile, k range); the S k ranges of a tile form one thread-block cluster, so
// the hardware schedules them together and nothing has to be arranged for their co-residency. A
// tile has 2 * bh accumulator columns (bh = 32, 64 or 128 weight rows per operand box): two boxes of
// one matrix (PLAIN) or the same rows of W_gate and W_up (GATEUP). Every CTA
//   1. copies its k-blocks through a ring deep enough to hold all of them where possible
//      (the A box has exactly M rows, so a launch of 16 rows stages 2 KB of A per k-block);
//   2. accumulates in tensor memory (tcgen05.mma, 128 x 2bh fp32);
//   3. with S > 1: writes its fp32 partial tile to its own shared memory (the idle copy ring;
//      16-byte chunks XOR-swizzled by row, so that neither this write nor the later reads
//      conflict) and sends to every CTA of the cluster the run of rows that CTA owns (rows are
//      dealt out in S equal runs) with one bulk copy from shared memory to shared memory, which
//      counts its bytes on the receiver's mbarrier; every CTA then sums the S copies of its own
//      rows in k order (the result does not depend on timing) and stores them as bf16 with
//      coalesced 8-byte stores. A cluster barrier at the very end keeps every CTA's shared
//      memory alive until the copies that read it have finished. With S == 1 the rows go from
//      tensor memory to global memory directly.
// No workspace, no counters, no waits on global memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../include/dynaflow_b200.h"
#include "gemm_internal.h"
#include "host_util.h"
#include "ptx.cuh"

namespace df {
namespace {

constexpr int SK_THREADS = 256;
constexpr int SK_BK = 64;
constexpr int SK_MAX_STAGES = 16;
constexpr int SK_SMEM_CAP = 227 * 1024;
constexpr int SK_MISC_BYTES = 512;  // barriers, tensor-memory address, abort flag
constexpr int SK_MAX_CLUSTER = 8;    // the portable limit

enum : int { SMALL_PLAIN = 0, SMALL_GATEUP = 1 };
enum : unsigned { WHERE_SMALL_PRODUCER = 21, WHERE_SMALL_MMA = 22, WHERE_SMALL_EPILOGUE = 23, WHERE_SMALL_RECV = 24 };

struct SmallParams {
  int M, N, K, ldc;
  int bh;        // weight rows per operand box: 32, 64 or 128
  int splits;    // k ranges per tile = CTAs per cluster
  int num_kb;
  int stages, a_bytes, a_tx;
  int ring_bytes;  // the copy ring; the receive area for partial rows follows it
  int rows_per;    // rows of the tile each CTA of the cluster owns: ceil(M / splits)
  __nv_bfloat16* C;
  Status* status;
  unsigned long long timeout_ns;
#ifdef DF_DEV_KNOBS
  unsigned long long* timing;  // development builds: eight time stamps per CTA, or NULL
#endif
};

#ifdef DF_DEV_KNOBS
#define SMALL_STAMP(i) do { if (p.timing != nullptr) p.timing[blockIdx.x * 8 + (i)] = globaltimer_ns(); } while (0)
#else
#define SMALL_STAMP(i) do { } while (0)
#endif

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Bulk copy from this CTA's shared memory into the shared memory of a CTA of the cluster; the
// bytes are counted on an mbarrier of the destination CTA. Both destination addresses are
// shared::cluster addresses (mapa).
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t dst_cluster, const void* src, uint32_t bytes, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_cluster),
               "r"(smem_u32(src)), "r"(bytes), "r"(bar_cluster)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float to_bf16_and_back(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float silu_mul(float g, float u) {
  // gate and up are rounded to bf16 first, as two separate linear layers would deliver them
  g = to_bf16_and_back(g);
  u = to_bf16_and_back(u);
  return (g / (1.0f + expf(-g))) * u;
}

template <int MODE>
__global__ void __launch_bounds__(SK_THREADS, 1)
splitk_small_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b0,
                    const __grid_constant__ CUtensorMap tm_b1, const SmallParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);  // the same offset in every CTA of the cluster

  const int S = p.splits;
  const int b_box_bytes = p.bh * (SK_BK * 2);
  const int stage_bytes = p.a_bytes + 2 * b_box_bytes;
  const int acc_cols = 2 * p.bh;
  const int row_bytes = acc_cols * 4;
  uint8_t* recv = smem + p.ring_bytes;  // [source CTA][rows_per][2 bh] fp32
  const int recv_bytes = S > 1 ? S * p.rows_per * row_bytes : 0;
  uint64_t* full = reinterpret_cast<uint64_t*>(recv + recv_bytes);
  uint64_t* empty = full + SK_MAX_STAGES;
  uint64_t* tfull = empty + SK_MAX_STAGES;
  uint64_t* recv_bar = tfull + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(recv_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile = static_cast<int>(blockIdx.x) / S;
  const int s_idx = static_cast<int>(blockIdx.x) - tile * S;  // = rank in the cluster
  const int kb0 = static_cast<int>((static_cast<long long>(s_idx) * p.num_kb) / S);
  const int kb1 = static_cast<int>((static_cast<long long>(s_idx + 1) * p.num_kb) / S);
  const int n0 = tile * (MODE == SMALL_GATEUP ? p.bh : 2 * p.bh);  // first output column of the tile

  if (threadIdx.x == 0) {
    SMALL_STAMP(0);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tfull, 1);
    mbar_init(recv_bar, 1);
    *abort_flag = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b0);
    tma_prefetch_desc(&tm_b1);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, static_cast<uint32_t>(acc_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // first cluster barrier, split in two: arriving here says "this CTA runs, its shared memory and
  // barriers exist"; the wait comes before the first copy into another CTA
  if (S > 1) cluster_arrive();
  if (threadIdx.x == 0) SMALL_STAMP(1);

  const uint32_t tmem_base = *tmem_slot;
  const Deadline dl{globaltimer_ns() + p.timeout_ns, abort_flag, p.status};

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------ copy producer
      const int y0 = n0;
      const int y1 = (MODE == SMALL_GATEUP) ? n0 : n0 + p.bh;
      int stage = 0;
      uint32_t phase = 0;
      // The weights do not depend on the kernel before this one in the stream: the first ring-full
      // of weight boxes is on its way before the wait for that kernel's results, the rows of A follow it.
      const int ahead = min(kb1 - kb0, p.stages);
      for (int i = 0; i < ahead; ++i) {
        uint8_t* sb = smem + i * stage_bytes + p.a_bytes;
        mbar_expect_tx(&full[i], static_cast<uint32_t>(p.a_tx + 2 * b_box_bytes));
        tma_load_2d(sb, &tm_b0, &full[i], (kb0 + i) * SK_BK, y0);
        tma_load_2d(sb + b_box_bytes, &tm_b1, &full[i], (kb0 + i) * SK_BK, y1);
      }
      grid_dependency_wait();
      grid_launch_dependents();
      for (int i = 0; i < ahead; ++i) tma_load_2d(smem + i * stage_bytes, &tm_a, &full[i], (kb0 + i) * SK_BK, 0);
      if (ahead == p.stages) phase ^= 1u;  // the ring has gone round once
      stage = ahead == p.stages ? 0 : ahead;
      for (int kb = kb0 + ahead; kb < kb1; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1u, dl, WHERE_SMALL_PRODUCER, blockIdx.x)) break;
        uint8_t* sa = smem + stage * stage_bytes;
        uint8_t* sb = sa + p.a_bytes;
        mbar_expect_tx(&full[stage], static_cast<uint32_t>(p.a_tx + 2 * b_box_bytes));
        tma_load_2d(sb, &tm_b0, &full[stage], kb * SK_BK, y0);
        tma_load_2d(sb + b_box_bytes, &tm_b1, &full[stage], kb * SK_BK, y1);
        tma_load_2d(sa, &tm_a, &full[stage], kb * SK_BK, 0);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // -------------------------------------------------------- MMA issuer
      const uint32_t idesc = make_idesc_bf16(128, acc_cols);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full[stage], phase, dl, WHERE_SMALL_MMA, blockIdx.x)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (kb == kb0) SMALL_STAMP(2);
        if (kb == kb1 - 1) SMALL_STAMP(3);
        const uint32_t a_addr = smem_u32(smem + stage * stage_bytes);
        const uint64_t da = make_desc_k_sw128(a_addr);
        const uint64_t db = make_desc_k_sw128(a_addr + static_cast<uint32_t>(p.a_bytes));
#pragma unroll
        for (int k = 0; k < SK_BK / 16; ++k)
          umma_bf16(tmem_base, da + 2u * k, db + 2u * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        umma_commit(&empty[stage]);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) umma_commit(tfull);
    }
    __syncwarp();
  }

  if (warp >= 4) {
    // ---------------------------------------------------------- epilogue
    const int q = warp - 4;
    const int tid = static_cast<int>(threadIdx.x) - 4 * 32;
    const int row = tid;
    bool ok = mbar_wait(tfull, 0u, dl, WHERE_SMALL_EPILOGUE, blockIdx.x);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    grid_dependency_wait();  // long satisfied (the accumulator depends on rows of A fetched after the producer's wait)
    if (tid == 0) SMALL_STAMP(4);
    const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16);

    if (S == 1) {
      if (ok) {
        __nv_bfloat16* crow = p.C + static_cast<size_t>(row) * p.ldc;
        if (MODE == SMALL_GATEUP) {
#pragma unroll 1
          for (int c = 0; c < p.bh / 32; ++c) {
            uint32_t g[32], u[32];
            tmem_ld_32x32(t_acc + c * 32, g);
            tmem_ld_32x32(t_acc + p.bh + c * 32, u);
            tmem_ld_wait();
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)
              o[j] = pack2(silu_mul(__uint_as_float(g[2 * j]), __uint_as_float(u[2 * j])),
                           silu_mul(__uint_as_float(g[2 * j + 1]), __uint_as_float(u[2 * j + 1])));
            if (row < p.M) {
              const int col = n0 + c * 32;
#pragma unroll
              for (int v = 0; v < 4; ++v)
                if (col + v * 8 < p.N)
                  *reinterpret_cast<uint4*>(crow + col + v * 8) = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
            }
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < acc_cols / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_acc + c * 32, r);
            tmem_ld_wait();
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = pack2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            if (row < p.M) {
              const int col = n0 + c * 32;
#pragma unroll
              for (int v = 0; v < 4; ++v)
                if (col + v * 8 < p.N)
                  *reinterpret_cast<uint4*>(crow + col + v * 8) = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
            }
          }
        }
      }
    } else {
      cluster_wait();  // every CTA of the cluster runs: its receive area and barrier may be written
      uint8_t* staging = smem;  // the copy ring is idle: every MMA that read it has finished
      if (ok) {
        uint8_t* my_row = staging + row * row_bytes;
        const int sw = row & 7;
#pragma unroll 1
        for (int c = 0; c < acc_cols / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c * 32, r);
          tmem_ld_wait();
          if (row < p.M) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(my_row + (((c * 8 + j) ^ sw) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          }
        }
      }
      fence_proxy_async_smem();  // the bulk copies below read what the ordinary stores above wrote
      epilogue_bar_sync();
      const int slot_bytes = p.rows_per * row_bytes;
      const int my_r0 = s_idx * p.rows_per;
      const int my_rows = max(0, min(p.M - my_r0, p.rows_per));
      if (tid == 0) SMALL_STAMP(5);
      if (tid == 0 && !*abort_flag) {
        if (my_rows > 0) mbar_expect_tx(recv_bar, static_cast<uint32_t>(S * my_rows * row_bytes));
        const uint32_t slot_local = smem_u32(recv) + static_cast<uint32_t>(s_idx * slot_bytes);
        const uint32_t bar_local = smem_u32(recv_bar);
        for (int i = 0; i < S; ++i) {
          const int o = (s_idx + i) % S;  // start with myself, then round the cluster: no two sources hit one CTA at once
          const int o_r0 = o * p.rows_per;
          const int o_rows = min(p.M - o_r0, p.rows_per);
          if (o_rows > 0)
            bulk_copy_to_cluster(mapa_shared(slot_local, static_cast<uint32_t>(o)), staging + o_r0 * row_bytes,
                                 static_cast<uint32_t>(o_rows * row_bytes), mapa_shared(bar_local, static_cast<uint32_t>(o)));
        }
      }
      bool got = true;
      if (my_rows > 0) got = mbar_wait(recv_bar, 0u, dl, WHERE_SMALL_RECV, blockIdx.x);
      got = __all_sync(0xffffffffu, got);
      if (tid == 0) SMALL_STAMP(6);
      cluster_arrive();  // second cluster barrier, waited for at the very end
      const int r0 = my_r0;
      const int nrows = my_rows;
      if (got && !*abort_flag && nrows > 0) {
        const int groups = (MODE == SMALL_GATEUP ? p.bh : acc_cols) / 4;  // four output columns each
        const int total = nrows * groups;
        for (int idx = tid; idx < total; idx += 128) {
          const int rr = idx / groups;
          const int g = idx - rr * groups;
          const int out_row = r0 + rr;
          const int sw = out_row & 7;
          const uint8_t* base = recv + rr * row_bytes;
          float4 a = *reinterpret_cast<const float4*>(base + ((g ^ sw) << 4));
          float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
          if (MODE == SMALL_GATEUP) b = *reinterpret_cast<const float4*>(base + (((g + p.bh / 4) ^ sw) << 4));
          for (int o = 1; o < S; ++o) {
            const uint8_t* bo = base + o * slot_bytes;
            const float4 va = *reinterpret_cast<const float4*>(bo + ((g ^ sw) << 4));
            a.x += va.x, a.y += va.y, a.z += va.z, a.w += va.w;
            if (MODE == SMALL_GATEUP) {
              const float4 vb = *reinterpret_cast<const float4*>(bo + (((g + p.bh / 4) ^ sw) << 4));
              b.x += vb.x, b.y += vb.y, b.z += vb.z, b.w += vb.w;
            }
          }
          const int col = n0 + 4 * g;
          if (col < p.N) {
            uint2 o2;
            if (MODE == SMALL_GATEUP) {
              o2.x = pack2(silu_mul(a.x, b.x), silu_mul(a.y, b.y));
              o2.y = pack2(silu_mul(a.z, b.z), silu_mul(a.w, b.w));
            } else {
              o2.x = pack2(a.x, a.y);
              o2.y = pack2(a.z, a.w);
            }
            *reinterpret_cast<uint2*>(p.C + static_cast<size_t>(out_row) * p.ldc + col) = o2;
          }
        }
      }
    }
    tc_fence_before();
  } else if (S > 1) {
    // the other warps take part in the cluster barriers only
    cluster_wait();
    cluster_arrive();
  }
  // every CTA of the cluster has received all its rows: no copy reads this CTA's shared memory any more
  if (S > 1) cluster_wait();

  // ------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) SMALL_STAMP(7);
  if (warp == 2) {
    tc_fence_after();
    if (*abort_flag) {
      // error path: give copies and MMAs still in flight time to land before the memories go back
      const uint64_t t_stop = globaltimer_ns() + 2000000ull;
      while (globaltimer_ns() < t_stop) __nanosleep(1000);
    }
    tmem_dealloc(tmem_base, static_cast<uint32_t>(acc_cols));
  }
}

struct Plan {
  int bh, splits, stages, a_bytes, ring_bytes, rows_per, tiles, smem_bytes;
  double cost;
};

// Time model (microseconds, without the launch itself) of one launch form, fitted to per-CTA time
// stamps on a B200: a CTA takes its operand bytes in at about 90 GB/s and all CTAs together at
// about 8.5 TB/s (the rows of A are re-read from L2 by every tile); a cluster exchange costs about
// a microsecond plus the bytes a CTA sends at the 28 GB/s one SM reaches into another's shared memory.
static bool evaluate(int M, int N, int num_kb, bool gateup, int units, int bh, int splits, Plan* out) {
  const int out_per_tile = gateup ? bh : 2 * bh;
  const int tiles = (N + out_per_tile - 1) / out_per_tile;
  if (splits > num_kb) return false;
  const int a_bytes = ((M + 7) / 8) * 1024;
  const int stage_bytes = a_bytes + 2 * bh * 128;
  const int kb_per = (num_kb + splits - 1) / splits;
  const int row_bytes = 2 * bh * 4;
  const int rows_per = (M + splits - 1) / splits;
  const int recv = splits > 1 ? splits * rows_per * row_bytes : 0;
  int stages = (SK_SMEM_CAP - 1024 - SK_MISC_BYTES - recv) / stage_bytes;
  if (stages > SK_MAX_STAGES) stages = SK_MAX_STAGES;
  if (stages > kb_per) stages = kb_per;
  if (stages < 1 || (stages < 2 && kb_per > 1)) return false;
  int ring = stages * stage_bytes;
  // the MMA reads 128 rows (16 KB) of A whatever M is; with few rows and small operand boxes that
  // reaches past the last stage, and it has to stay inside this CTA's shared memory
  if (ring < (stages - 1) * stage_bytes + 128 * 128) ring = (stages - 1) * stage_bytes + 128 * 128;
  if (splits > 1 && ring < M * row_bytes) ring = ((M * row_bytes + 1023) / 1024) * 1024;  // the staged partial tile
  if (ring + recv + 1024 + SK_MISC_BYTES > SK_SMEM_CAP) return false;
  const int ctas = tiles * splits;
  const int waves = (ctas + units - 1) / units;
  if (waves > 1 && splits > 1) return false;  // more than a wave of tiles: nothing to gain from splitting
  const int rounds = (kb_per + stages - 1) / stages;
  const double cta_bytes = static_cast<double>(kb_per) * stage_bytes;
  const double t_one = cta_bytes / 90e3 * waves;
  const double t_all = static_cast<double>(ctas) * cta_bytes / 8.5e6;
  double t = (t_one > t_all ? t_one : t_all) + 1.7 + 0.3 * (rounds - 1);
  const double tile_bytes = static_cast<double>(M) * row_bytes;
  if (splits > 1)
    t += 0.4 + 1.0 + tile_bytes * (splits - 1) / splits / 28e3 + 0.5;
  else
    t += tile_bytes / 2 / 40e3 * waves;
  out->bh = bh;
  out->splits = splits;
  out->stages = stages;
  out->a_bytes = a_bytes;
  out->ring_bytes = ring;
  out->rows_per = rows_per;
  out->tiles = tiles;
  out->smem_bytes = out->ring_bytes + recv + 1024 + SK_MISC_BYTES;
  out->cost = t;
  return true;
}

}  // namespace

// The form a launch would take: the same search launch_small_mode() makes.
static bool plan_small(int M, int N, int K, bool gateup, int units, bool allow_split, int force_bh, int force_splits,
                       Plan* best) {
  const int num_kb = (K + SK_BK - 1) / SK_BK;
  best->cost = -1.0;
  for (int bh = 128; bh >= 32; bh /= 2) {
    if (force_bh > 0 && bh != force_bh) continue;
    // powers of two only: clusters of 5 (28 gate/up tiles x 5 = 140 CTAs) measured 22 us against 13 us for clusters of 4
    for (int s = 1; s <= (allow_split ? SK_MAX_CLUSTER : 1); s *= 2) {
      if (force_splits > 0 && s != force_splits) continue;
      Plan cand;
      if (!evaluate(M, N, num_kb, gateup, units, bh, s, &cand)) continue;
      if (best->cost < 0.0 || cand.cost < best->cost) *best = cand;
    }
  }
  return best->cost >= 0.0;
}

template <int MODE>
static int launch_small_mode(const void* a, const void* b0, const void* b1, void* c, int M, int N, int K, int lda, int ldb,
                             int ldc, int units, bool allow_split, int force_bh, int force_splits,
                             df_status_t* dev_status, cudaStream_t stream) {
  const int num_kb = (K + SK_BK - 1) / SK_BK;
  Plan best;
  if (!plan_small(M, N, K, MODE == SMALL_GATEUP, units, allow_split, force_bh, force_splits, &best)) return DF_SMALL_NOT_APPLICABLE;

  CUtensorMap tm_a, tm_b0, tm_b1;
  if (!make_map_bf16(&tm_a, a, M, K, lda, M)) return DF_ECUDA;
  if (!make_map_bf16(&tm_b0, b0, N, K, ldb, best.bh)) return DF_ECUDA;
  if (!make_map_bf16(&tm_b1, b1, N, K, ldb, best.bh)) return DF_ECUDA;

  SmallParams p;
  std::memset(&p, 0, sizeof(p));
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.bh = best.bh;
  p.splits = best.splits;
  p.num_kb = num_kb;
  p.stages = best.stages;
  p.a_bytes = best.a_bytes;
  p.a_tx = M * SK_BK * 2;
  p.ring_bytes = best.ring_bytes;
  p.rows_per = best.rows_per;
  p.C = static_cast<__nv_bfloat16*>(c);
  p.status = reinterpret_cast<Status*>(dev_status);
  p.timeout_ns = timeout_ns();
#ifdef DF_DEV_KNOBS
  const char* tp = std::getenv("DF_SMALL_TIMING_PTR");
  p.timing = tp != nullptr ? reinterpret_cast<unsigned long long*>(std::strtoull(tp, nullptr, 0)) : nullptr;
#endif

  auto kernel = splitk_small_kernel<MODE>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM_CAP);
  if (e != cudaSuccess) return fail(DF_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(best.tiles * best.splits, 1, 1);
  cfg.blockDim = dim3(SK_THREADS, 1, 1);
  cfg.dynamicSmemBytes = best.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int n_attrs = dependent_launch_attr(&attrs[0]);
  if (best.splits > 1) {
    attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
    attrs[n_attrs].val.clusterDim.x = best.splits;
    attrs[n_attrs].val.clusterDim.y = 1;
    attrs[n_attrs].val.clusterDim.z = 1;
    ++n_attrs;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n_attrs;
  e = cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b0, tm_b1, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(DF_ECUDA, "split-K launch (%d tiles x %d): %s", best.tiles, best.splits, cudaGetErrorString(e));
  }
  return DF_OK;
}

int launch_small_rows(bool gateup, const void* a, const void* b0, const void* b1, void* c, int M, int N, int K, int lda,
                      int ldb, int ldc, int units, bool allow_split, int force_bh, int force_splits,
                      df_status_t* dev_status, cudaStream_t stream) {
  if (M < 1 || M > 128) return DF_SMALL_NOT_APPLICABLE;
  if (gateup)
    return launch_small_mode<SMALL_GATEUP>(a, b0, b1, c, M, N, K, lda, ldb, ldc, units, allow_split, force_bh,
                                           force_splits, dev_status, stream);
  return launch_small_mode<SMALL_PLAIN>(a, b0, b1, c, M, N, K, lda, ldb, ldc, units, allow_split, force_bh, force_splits,
                                        dev_status, stream);
}

}  // namespace df

extern "C" int df_small_gemm_plan(int M, int N, int K, int gate_up, int sms, int* box_rows, int* k_splits, int* stages,
                                  int* tiles, size_t* shared_bytes) {
  if (M < 1 || M > 128 || N <= 0 || K <= 0 || sms <= 0) return df::fail(DF_EINVAL, "need 1 <= M <= 128 and positive N, K, sms");
  df::Plan plan;
  if (!df::plan_small(M, N, K, gate_up != 0, sms, true, 0, 0, &plan)) return df::fail(DF_EUNSUPPORTED, "no launch form fits this shape");
  if (box_rows != nullptr) *box_rows = plan.bh;
  if (k_splits != nullptr) *k_splits = plan.splits;
  if (stages != nullptr) *stages = plan.stages;
  if (tiles != nullptr) *tiles = plan.tiles;
  if (shared_bytes != nullptr) *shared_bytes = static_cast<size_t>(plan.smem_bytes);
  return DF_OK;
}
