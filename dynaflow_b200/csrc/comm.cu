// Tensor-parallel reduction of one micro-batch over NVLink peer memory:
// two-shot all-reduce (reduce-scatter by row slices, then all-gather by peer
// stores) with an optional fused residual-add + RMSNorm epilogue.
//
// Every rank owns a "region" of device memory that all ranks have mapped
// (CUDA IPC): a partial-sum buffer the rank's down projection writes into, a
// sum buffer its peers push reduced rows into, and flag words. One launch:
//
//   barrier 0   block b of every rank tells block b of every peer that the
//               rank's partial buffer is complete
//   phase 1     rank r reduces the rows of slice r: a warp loads one row from
//               all W partial buffers (16-byte peer loads), adds in fp32 in
//               rank order, rounds to bf16 and stores the row into the sum
//               buffer of all W ranks (peer stores)
//   barrier 1   block b of every rank has pushed its rows
//   phase 2     local: the rows that the blocks b delivered are finished on
//               this rank -- nothing (the result is the sum buffer), or
//               r' = y + residual; out = rmsnorm(r') * w
//
// Third form ("sharded residual"): the residual stream is kept sharded by rows, rank r holding
// the rows of slice r. The owner then does r' = y + residual and the RMSNorm BETWEEN the two
// shots, on its own rows only, and the second shot distributes the normalised rows; there is
// no phase 2, no replicated work and no traffic beyond that of the plain all-reduce.
//
// Blocks only ever synchronise with the same-index block of the other ranks,
// and block b consumes in phase 2 exactly the rows that the blocks b produced,
// so there is no grid-wide barrier. Flags carry a per-block sequence number
// kept in device memory, which makes the kernel replayable from a CUDA graph.
// Waits are bounded by the library deadline; a peer that never shows up yields
// DF_ERR_PEER in the status block and the kernel returns.
//
// No multimem / NVLS and no TMA are used here: plain ld/st.global on peer
// pointers through NVSwitch.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#include "../../include/dynaflow_b200.h"
#include "host_util.h"
#include "ptx.cuh"

namespace df {

constexpr int kMaxWorld = DF_COMM_MAX_WORLD;
// 256 threads at <= 104 registers: a CTA of this kernel fits on an SM beside a
// resident GEMM CTA (256 threads x 96 registers, 197 KB shared memory), so the
// reduction does not have to wait for the persistent GEMM to leave.
constexpr int kCommThreads = 256;
constexpr int kWarpsPerBlock = kCommThreads / 32;
constexpr int kMaxCtas = DF_COMM_MAX_CTAS;
constexpr unsigned WHERE_FLAG = 16;
constexpr int kMaxSmemHidden = 8192;  // 16 KB of shared memory for the RMSNorm weight

// Layout of a region (all offsets multiples of 256 bytes):
//   [0, 4096)                         flag words: uint32 flags[2][kMaxCtas][kMaxWorld]
//   [4096, 4096 + 4*kMaxCtas)         block sequence numbers
//   partial buffer  max_rows x hidden bf16
//   sum buffer      max_rows x hidden bf16
constexpr size_t kFlagBytes = 2ull * kMaxCtas * kMaxWorld * 4;  // 4096 with 64 CTAs x 8 ranks
constexpr size_t kSeqOffset = kFlagBytes;
constexpr size_t kHeaderBytes = 8192;

static size_t align256(size_t x) { return (x + 255) / 256 * 256; }

enum : int { EPI_NONE = 0, EPI_ADD_RMSNORM = 1, EPI_ADD_RMSNORM_SHARDED = 2 };

struct RankView {
  int rank;
  const __nv_bfloat16* partial[kMaxWorld];
  __nv_bfloat16* sum[kMaxWorld];
  uint32_t* flags[kMaxWorld];
  uint32_t* seq;               // this rank's per-block sequence numbers
  const __nv_bfloat16* residual_in;
  __nv_bfloat16* residual_out;
  __nv_bfloat16* out;
};

struct CommParams {
  RankView ranks[kMaxWorld];   // [0] only, unless several ranks are emulated on one GPU
  const __nv_bfloat16* weight;
  int world, T, H, mode;
  int coll;  // 0 = all-reduce, 1 = reduce-scatter (keep the reduced slice local), 2 = all-gather of the slices
  float eps;
  unsigned long long timeout_ns;
  Status* status;
};



__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Block-level barrier with the same-index block of every peer. Thread t < world
// signals peer t and then waits for peer t's signal. Returns false (for the
// whole block) if a wait ran out.
__device__ __forceinline__ bool peer_barrier(const RankView& me, int world, int phase, uint32_t seq,
                                             unsigned long long t_end, Status* status, uint32_t* s_abort) {
  __syncthreads();  // all of this block's earlier stores are ordered before the signal
  const int t = threadIdx.x;
  if (t < world) {
    const uint32_t value = seq * 2u + static_cast<uint32_t>(phase) + 1u;
    const size_t slot = (static_cast<size_t>(phase) * kMaxCtas + blockIdx.x) * kMaxWorld;
    __threadfence_system();
    st_release_sys(me.flags[t] + slot + me.rank, value);
    const uint32_t* mine = me.flags[me.rank] + slot + t;
    uint32_t spins = 0;
    // flags only grow; compare as a signed distance so that wrap-around is harmless
    uint32_t seen;
    while (static_cast<int32_t>((seen = ld_acquire_sys(mine)) - value) < 0) {
      if ((++spins & 0xffu) == 0u && globaltimer_ns() > t_end) {
        *s_abort = 1u;
        report(status, 2u /*DF_ERR_PEER*/, WHERE_FLAG + phase, static_cast<unsigned>(t));
        seen = value;
        break;
      }
    }
    // In step, a peer can never be ahead of the value waited for: it reaches its next flag of
    // this phase only through the other phase's barrier, which needs this rank's next signal.
    // A flag that is ahead therefore belongs to a peer that gave up on an earlier barrier and
    // went on alone; its contribution to this launch is missing, so this rank reports it too.
    if (seen != value) {
      *s_abort = 1u;
      report(status, 2u /*DF_ERR_PEER*/, WHERE_FLAG + phase, static_cast<unsigned>(t));
    }
  }
  __syncthreads();
  return *s_abort == 0u;
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// One row of r' = y + residual; out = bf16(r' * rsqrt(mean(r'^2) + eps)) * w, by one warp.
// Each lane keeps kBatch vectors of the sum and of the residual in flight at a time
// (explicit batches: the compiler may not move loads across the stores, the buffers can
// alias). The new residual is read back for the second pass from this thread's own writes.
__device__ __forceinline__ void add_rmsnorm_row(const __nv_bfloat16* y_base, const __nv_bfloat16* rin_base,
                                                __nv_bfloat16* rout_base, __nv_bfloat16* out_base, const uint4* wv,
                                                int row, int H, float eps, int lane) {
  constexpr int kBatch = 8;
  const int nvec = H >> 3;
  const size_t base = static_cast<size_t>(row) * H;
  const uint4* y = reinterpret_cast<const uint4*>(y_base + base);
  const uint4* rin = rin_base != nullptr ? reinterpret_cast<const uint4*>(rin_base + base) : nullptr;
  uint4* res_out = reinterpret_cast<uint4*>(rout_base + base);
  uint4* o = reinterpret_cast<uint4*>(out_base + base);
  float ss = 0.0f;
  for (int v0 = lane; v0 < nvec; v0 += 32 * kBatch) {
    uint4 yv[kBatch], rv[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) {
        yv[u] = __ldcg(y + v);
        rv[u] = rin != nullptr ? rin[v] : make_uint4(0u, 0u, 0u, 0u);
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) {
        float fy[8], fr[8];
        unpack8(yv[u], fy);
        unpack8(rv[u], fr);
#pragma unroll
        for (int i = 0; i < 8; ++i) fy[i] += fr[i];
        const uint4 packed = pack8(fy);
        res_out[v] = packed;
        unpack8(packed, fy);  // the sum of squares is taken over the rounded residual
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += fy[i] * fy[i];
      }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  const float inv = rsqrtf(ss / static_cast<float>(H) + eps);
  for (int v0 = lane; v0 < nvec; v0 += 32 * kBatch) {
    uint4 xv[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) xv[u] = res_out[v];
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) {
        float fx[8], fw[8];
        unpack8(xv[u], fx);
        unpack8(wv[v], fw);
#pragma unroll
        for (int i = 0; i < 8; ++i) fx[i] = __bfloat162float(__float2bfloat16_rn(fx[i] * inv)) * fw[i];
        o[v] = pack8(fx);
      }
    }
  }
}

// Stand-alone residual add + RMSNorm over all SMs (one warp per row): the second half of the
// fused reduction as its own launch, for when the reduction itself runs on few CTAs.
__global__ void __launch_bounds__(kCommThreads) add_rmsnorm_kernel(const __nv_bfloat16* y, const __nv_bfloat16* rin,
                                                                    __nv_bfloat16* rout, __nv_bfloat16* out,
                                                                    const __nv_bfloat16* weight, int T, int H, float eps,
                                                                    bool block_per_row) {
  extern __shared__ uint4 s_weight[];
  const bool staged = H <= kMaxSmemHidden;
  if (staged) {  // the norm weight does not depend on the kernel before this one
    for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) s_weight[v] = reinterpret_cast<const uint4*>(weight)[v];
    __syncthreads();
  }
  grid_dependency_wait();
  grid_launch_dependents();
  const uint4* wv = staged ? s_weight : reinterpret_cast<const uint4*>(weight);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (block_per_row) {
    // few rows (a decode step): a whole CTA per row, every load of the row in flight at once, the row kept in
    // registers between the sum of squares and the scaling (the host chooses this form; H <= 8192)
    constexpr int kRowVecs = 4;
    __shared__ float s_part[kWarpsPerBlock];
    const int nvec = H >> 3;
    for (int row = blockIdx.x; row < T; row += gridDim.x) {
      const size_t base = static_cast<size_t>(row) * H;
      uint4 yv[kRowVecs], rv[kRowVecs];
#pragma unroll
      for (int k = 0; k < kRowVecs; ++k) {
        const int v = threadIdx.x + k * kCommThreads;
        if (v < nvec) {
          yv[k] = __ldcg(reinterpret_cast<const uint4*>(y + base) + v);
          rv[k] = rin != nullptr ? reinterpret_cast<const uint4*>(rin + base)[v] : make_uint4(0u, 0u, 0u, 0u);
        }
      }
      float f[kRowVecs][8];
      float ss = 0.0f;
#pragma unroll
      for (int k = 0; k < kRowVecs; ++k) {
        const int v = threadIdx.x + k * kCommThreads;
        if (v < nvec) {
          float fr[8];
          unpack8(yv[k], f[k]);
          unpack8(rv[k], fr);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[k][i] += fr[i];
          const uint4 packed = pack8(f[k]);
          reinterpret_cast<uint4*>(rout + base)[v] = packed;
          unpack8(packed, f[k]);  // the sum of squares is taken over the rounded residual
#pragma unroll
          for (int i = 0; i < 8; ++i) ss += f[k][i] * f[k][i];
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
      if (lane == 0) s_part[warp] = ss;
      __syncthreads();
      float total = 0.0f;
#pragma unroll
      for (int w = 0; w < kWarpsPerBlock; ++w) total += s_part[w];
      __syncthreads();
      const float inv = rsqrtf(total / static_cast<float>(H) + eps);
#pragma unroll
      for (int k = 0; k < kRowVecs; ++k) {
        const int v = threadIdx.x + k * kCommThreads;
        if (v < nvec) {
          float fw[8];
          unpack8(wv[v], fw);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[k][i] = __bfloat162float(__float2bfloat16_rn(f[k][i] * inv)) * fw[i];
          reinterpret_cast<uint4*>(out + base)[v] = pack8(f[k]);
        }
      }
    }
    return;
  }
  for (int row = blockIdx.x * kWarpsPerBlock + warp; row < T; row += gridDim.x * kWarpsPerBlock)
    add_rmsnorm_row(y, rin, rout, out, wv, row, H, eps, lane);
}

template <int W, bool EMULATE, int EPI>
__global__ void __launch_bounds__(kCommThreads, 2) allreduce_kernel(const CommParams p) {
  __shared__ uint32_t s_abort;
  // RMSNorm weight staged once per CTA (EPI_ADD_RMSNORM, hidden <= kMaxSmemHidden): weight loads
  // from global memory could not be moved across the output stores and cost one exposed L2
  // round trip per vector.
  extern __shared__ uint4 s_weight[];
  const RankView& me = p.ranks[EMULATE ? blockIdx.y : 0];
  if (threadIdx.x == 0) s_abort = 0u;
  if (EPI != EPI_NONE && p.H <= kMaxSmemHidden) {
    for (int v = threadIdx.x; v < (p.H >> 3); v += blockDim.x) s_weight[v] = reinterpret_cast<const uint4*>(p.weight)[v];
  }
  const unsigned long long t_end = globaltimer_ns() + p.timeout_ns;
  const uint32_t seq = me.seq[blockIdx.x];  // same value on every rank: one increment per launch
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = p.H >> 3;
  const int row_stride = gridDim.x * kWarpsPerBlock;
  const int row_first = blockIdx.x * kWarpsPerBlock + warp;

  bool ok = peer_barrier(me, W, 0, seq, t_end, p.status, &s_abort);

  if (ok) {
    // ---- phase 1: reduce this rank's slice and push it to everyone
    const int lo = static_cast<int>(static_cast<long long>(p.T) * me.rank / W);
    const int hi = static_cast<int>(static_cast<long long>(p.T) * (me.rank + 1) / W);
    // U 16-byte vectors per peer in flight per lane: NVLink round trips are a few microseconds,
    // so the bytes in flight (CTAs x 8 warps x 32 lanes x U x 16 B per peer), not the issue
    // rate, set the bandwidth. U x W = 16 loads per lane keeps the register count level.
    constexpr int U = (W <= 2) ? 8 : (W <= 4 ? 4 : 2);
    // reduce-scatter: the reduced rows stay on this rank; all-gather: only this rank's own
    // partial rows are read (they are the data), and they go to everyone
    const bool load_all = p.coll != 2, store_all = p.coll != 1;
    const uint4* wv1 = (p.H <= kMaxSmemHidden) ? s_weight : reinterpret_cast<const uint4*>(p.weight);
    for (int row = lo + row_first; row < hi; row += row_stride) {
      const size_t base = static_cast<size_t>(row) * p.H;
      float ss = 0.0f;
      for (int v0 = lane; v0 < nvec; v0 += 32 * U) {
        uint4 in[U][W];
        uint4 rs[(EPI == EPI_ADD_RMSNORM_SHARDED) ? U : 1];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = v0 + 32 * u;
          if (v < nvec) {
#pragma unroll
            for (int r = 0; r < W; ++r)
              in[u][r] = (load_all || r == me.rank) ? __ldcg(reinterpret_cast<const uint4*>(me.partial[r] + base) + v)
                                                    : make_uint4(0u, 0u, 0u, 0u);
            if (EPI == EPI_ADD_RMSNORM_SHARDED)  // issued together with the peer loads, not behind them
              rs[u] = me.residual_in != nullptr ? reinterpret_cast<const uint4*>(me.residual_in + base)[v]
                                                : make_uint4(0u, 0u, 0u, 0u);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = v0 + 32 * u;
          if (v < nvec) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}, f[8];
#pragma unroll
            for (int r = 0; r < W; ++r) {  // rank order: every element is summed in the same order everywhere
              unpack8(in[u][r], f);
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[i] += f[i];
            }
            const uint4 y = pack8(acc);
            if (EPI == EPI_ADD_RMSNORM_SHARDED) {
              // the owner of the row adds its residual rows here, between the two shots: the
              // new residual stays on this rank only (the residual stream is sharded by rows)
              float fy[8], fr[8];
              unpack8(y, fy);
              unpack8(rs[(EPI == EPI_ADD_RMSNORM_SHARDED) ? u : 0], fr);
#pragma unroll
              for (int i = 0; i < 8; ++i) fy[i] += fr[i];
              const uint4 packed = pack8(fy);
              reinterpret_cast<uint4*>(me.residual_out + base)[v] = packed;
              unpack8(packed, fy);
#pragma unroll
              for (int i = 0; i < 8; ++i) ss += fy[i] * fy[i];
            } else {
#pragma unroll
              for (int r = 0; r < W; ++r)
                if (store_all || r == me.rank) __stcg(reinterpret_cast<uint4*>(me.sum[r] + base) + v, y);
            }
          }
        }
      }
      if (EPI == EPI_ADD_RMSNORM_SHARDED) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        const float inv = rsqrtf(ss / static_cast<float>(p.H) + p.eps);
        const uint4* rnew = reinterpret_cast<const uint4*>(me.residual_out + base);
        constexpr int kBatch = 8;
        for (int v0 = lane; v0 < nvec; v0 += 32 * kBatch) {
          uint4 xv[kBatch];
#pragma unroll
          for (int u = 0; u < kBatch; ++u) {
            const int v = v0 + 32 * u;
            if (v < nvec) xv[u] = rnew[v];  // this thread's own writes
          }
#pragma unroll
          for (int u = 0; u < kBatch; ++u) {
            const int v = v0 + 32 * u;
            if (v < nvec) {
              float fx[8], fw[8];
              unpack8(xv[u], fx);
              unpack8(wv1[v], fw);
#pragma unroll
              for (int i = 0; i < 8; ++i) fx[i] = __bfloat162float(__float2bfloat16_rn(fx[i] * inv)) * fw[i];
              const uint4 outv = pack8(fx);
#pragma unroll
              for (int r = 0; r < W; ++r) __stcg(reinterpret_cast<uint4*>(me.sum[r] + base) + v, outv);
            }
          }
        }
      }
    }
    ok = peer_barrier(me, W, 1, seq, t_end, p.status, &s_abort);
  }

  if (EPI == EPI_ADD_RMSNORM && ok) {
    // ---- phase 2: residual add + RMSNorm of the rows the blocks with this index delivered
    // (local memory traffic only).
    const uint4* wv = (p.H <= kMaxSmemHidden) ? s_weight : reinterpret_cast<const uint4*>(p.weight);
    for (int q = 0; q < W; ++q) {
      const int lo = static_cast<int>(static_cast<long long>(p.T) * q / W);
      const int hi = static_cast<int>(static_cast<long long>(p.T) * (q + 1) / W);
      for (int row = lo + row_first; row < hi; row += row_stride)
        add_rmsnorm_row(me.sum[me.rank], me.residual_in, me.residual_out, me.out, wv, row, p.H, p.eps, lane);
    }
  }

  __syncthreads();
  if (threadIdx.x == 0) me.seq[blockIdx.x] = seq + 1u;  // also after a failed wait: the ranks stay in step
}

// ---------------------------------------------------- in-switch (multicast) form
// The same two shots over an NVLink multicast mapping of the ranks' regions: one
// multimem.ld_reduce returns a 16-byte vector already summed over all ranks by the switch (fp32
// accumulation, rounded to bf16 once), one multimem.st delivers a vector to every rank. Per
// output vector that is one load and one store instead of `world` of each, and for a message
// of S bytes S bytes cross a GPU's links in each direction instead of 2 (W-1)/W * S.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_bf16x8(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

template <int EPI>  // EPI_NONE or EPI_ADD_RMSNORM_SHARDED
__global__ void __launch_bounds__(kCommThreads, 2)
allreduce_multicast_kernel(const CommParams p, const __nv_bfloat16* mc_partial, __nv_bfloat16* mc_sum) {
  __shared__ uint32_t s_abort;
  extern __shared__ uint4 s_weight[];
  const RankView& me = p.ranks[0];
  const int W = p.world;
  if (threadIdx.x == 0) s_abort = 0u;
  if (EPI != EPI_NONE && p.H <= kMaxSmemHidden) {
    for (int v = threadIdx.x; v < (p.H >> 3); v += blockDim.x) s_weight[v] = reinterpret_cast<const uint4*>(p.weight)[v];
  }
  const unsigned long long t_end = globaltimer_ns() + p.timeout_ns;
  const uint32_t seq = me.seq[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = p.H >> 3;
  const int row_stride = gridDim.x * kWarpsPerBlock;
  const int row_first = blockIdx.x * kWarpsPerBlock + warp;

  // every rank's partial rows are complete and visible before the switch reads them
  bool ok = peer_barrier(me, W, 0, seq, t_end, p.status, &s_abort);
  if (ok) {
    const int lo = static_cast<int>(static_cast<long long>(p.T) * me.rank / W);
    const int hi = static_cast<int>(static_cast<long long>(p.T) * (me.rank + 1) / W);
    constexpr int U = (EPI == EPI_NONE) ? 16 : 8;  // vectors in flight per lane
    const uint4* wv1 = (p.H <= kMaxSmemHidden) ? s_weight : reinterpret_cast<const uint4*>(p.weight);
    // (A whole CTA per row for decode-sized inputs -- every switch load of a row in flight at once, the row kept in
    // registers -- was built and measured: the reductions alone got 10 % shorter, the overlapped decode step at 4 ranks
    // 4.6 % longer, 10.55 against 10.08 ms in an A/B/A/B run. The warp per row stays.)
    for (int row = lo + row_first; row < hi; row += row_stride) {
      const size_t base = static_cast<size_t>(row) * p.H;
      float ss = 0.0f;
      for (int v0 = lane; v0 < nvec; v0 += 32 * U) {
        uint4 in[U];
        uint4 rs[(EPI == EPI_ADD_RMSNORM_SHARDED) ? U : 1];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = v0 + 32 * u;
          if (v < nvec) {
            in[u] = multimem_ld_reduce_bf16x8(reinterpret_cast<const uint4*>(mc_partial + base) + v);
            if (EPI == EPI_ADD_RMSNORM_SHARDED)
              rs[u] = me.residual_in != nullptr ? reinterpret_cast<const uint4*>(me.residual_in + base)[v]
                                                : make_uint4(0u, 0u, 0u, 0u);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = v0 + 32 * u;
          if (v < nvec) {
            if (EPI == EPI_ADD_RMSNORM_SHARDED) {
              float fy[8], fr[8];
              unpack8(in[u], fy);
              unpack8(rs[(EPI == EPI_ADD_RMSNORM_SHARDED) ? u : 0], fr);
#pragma unroll
              for (int i = 0; i < 8; ++i) fy[i] += fr[i];
              const uint4 packed = pack8(fy);
              reinterpret_cast<uint4*>(me.residual_out + base)[v] = packed;
              unpack8(packed, fy);
#pragma unroll
              for (int i = 0; i < 8; ++i) ss += fy[i] * fy[i];
            } else {
              multimem_st_bf16x8(reinterpret_cast<uint4*>(mc_sum + base) + v, in[u]);
            }
          }
        }
      }
      if (EPI == EPI_ADD_RMSNORM_SHARDED) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        const float inv = rsqrtf(ss / static_cast<float>(p.H) + p.eps);
        const uint4* rnew = reinterpret_cast<const uint4*>(me.residual_out + base);
        constexpr int kBatch = 8;
        for (int v0 = lane; v0 < nvec; v0 += 32 * kBatch) {
          uint4 xv[kBatch];
#pragma unroll
          for (int u = 0; u < kBatch; ++u) {
            const int v = v0 + 32 * u;
            if (v < nvec) xv[u] = rnew[v];  // this thread's own writes
          }
#pragma unroll
          for (int u = 0; u < kBatch; ++u) {
            const int v = v0 + 32 * u;
            if (v < nvec) {
              float fx[8], fw[8];
              unpack8(xv[u], fx);
              unpack8(wv1[v], fw);
#pragma unroll
              for (int i = 0; i < 8; ++i) fx[i] = __bfloat162float(__float2bfloat16_rn(fx[i] * inv)) * fw[i];
              multimem_st_bf16x8(reinterpret_cast<uint4*>(mc_sum + base) + v, pack8(fx));
            }
          }
        }
      }
    }
    // every rank's slice has landed everywhere before anyone reads the result
    ok = peer_barrier(me, W, 1, seq, t_end, p.status, &s_abort);
  }
  __syncthreads();
  if (threadIdx.x == 0) me.seq[blockIdx.x] = seq + 1u;
}

// ------------------------------------------------------------------- host

struct RegionLayout {
  size_t partial_off, sum_off, total;
};

static RegionLayout region_layout(int max_rows, int hidden) {
  RegionLayout l;
  const size_t buf = align256(static_cast<size_t>(max_rows) * static_cast<size_t>(hidden) * 2u);
  l.partial_off = kHeaderBytes;
  l.sum_off = l.partial_off + buf;
  l.total = l.sum_off + buf;
  return l;
}

// Shared memory a reduction CTA claims beyond what it uses (0 = none). 40 KB keeps such a CTA off
// every SM that holds a GEMM CTA (197 KB of the SM's 227 KB) and a GEMM CTA off every SM that
// holds one: when the GEMMs are launched on fewer CTAs than there are SMs, the reduction then
// runs on the SMs they leave free instead of sharing SMs with them.
static int g_exclusive_smem = 0;

template <bool EMULATE>
static int launch_allreduce(const CommParams& p, int n_ctas, int emulated, void* stream) {
  dim3 grid(n_ctas, EMULATE ? emulated : 1, 1);
  dim3 block(kCommThreads, 1, 1);
  void* args[] = {const_cast<CommParams*>(&p)};
  const void* fn = nullptr;
  switch (p.world) {
#define DF_CASE(W)                                                                               \
  case W:                                                                                        \
    fn = (p.mode == EPI_ADD_RMSNORM)                                                             \
             ? reinterpret_cast<const void*>(&allreduce_kernel<W, EMULATE, EPI_ADD_RMSNORM>)     \
             : (p.mode == EPI_ADD_RMSNORM_SHARDED)                                               \
                   ? reinterpret_cast<const void*>(&allreduce_kernel<W, EMULATE, EPI_ADD_RMSNORM_SHARDED>) \
                   : reinterpret_cast<const void*>(&allreduce_kernel<W, EMULATE, EPI_NONE>);     \
    break;
    DF_CASE(1) DF_CASE(2) DF_CASE(3) DF_CASE(4) DF_CASE(5) DF_CASE(6) DF_CASE(7) DF_CASE(8)
#undef DF_CASE
    default:
      return fail(DF_EUNSUPPORTED, "world size %d is outside [1, %d]", p.world, kMaxWorld);
  }
  cudaError_t e;
  size_t smem = (p.mode != EPI_NONE && p.H <= kMaxSmemHidden) ? static_cast<size_t>(p.H) * 2 : 0;
  if (!EMULATE && g_exclusive_smem > 0) {
    smem += static_cast<size_t>(g_exclusive_smem);
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return fail(DF_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  if (EMULATE) {
    // every emulated rank must be resident at once: its blocks wait on the others'
    e = cudaLaunchCooperativeKernel(fn, grid, block, args, smem, static_cast<cudaStream_t>(stream));
  } else {
    e = cudaLaunchKernel(fn, grid, block, args, smem, static_cast<cudaStream_t>(stream));
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(DF_ECUDA, "all-reduce launch: %s", cudaGetErrorString(e));
  }
  return DF_OK;
}

static int fill_params(CommParams* p, int n_views, const df_comm_rank_t* views, int world, int max_rows, int hidden,
                       int T, int H, int mode, const void* weight, float eps, df_status_t* dev_status, int coll = 0) {
  if (views == nullptr || dev_status == nullptr) return fail(DF_EINVAL, "NULL pointer argument");
  if (world < 1 || world > kMaxWorld) return fail(DF_EUNSUPPORTED, "world size %d is outside [1, %d]", world, kMaxWorld);
  if (T <= 0 || H <= 0 || (H % 8) != 0) return fail(DF_EINVAL, "T must be positive and H a positive multiple of 8");
  if (H != hidden || T > max_rows)
    return fail(DF_EINVAL, "T=%d, H=%d do not fit the region (max_rows=%d, hidden=%d)", T, H, max_rows, hidden);
  if (mode != EPI_NONE && weight == nullptr) return fail(DF_EINVAL, "RMSNorm weight is NULL");
  const RegionLayout l = region_layout(max_rows, hidden);
  std::memset(p, 0, sizeof(*p));
  for (int v = 0; v < n_views; ++v) {
    const df_comm_rank_t& in = views[v];
    RankView& out = p->ranks[v];
    if (in.rank < 0 || in.rank >= world) return fail(DF_EINVAL, "rank %d is outside [0, %d)", in.rank, world);
    out.rank = in.rank;
    for (int r = 0; r < world; ++r) {
      uint8_t* region = static_cast<uint8_t*>(in.regions[r]);
      if (region == nullptr || (reinterpret_cast<uintptr_t>(region) & 255u) != 0)
        return fail(DF_EINVAL, "region pointer of rank %d is NULL or not 256-byte aligned", r);
      out.partial[r] = reinterpret_cast<const __nv_bfloat16*>(region + l.partial_off);
      out.sum[r] = reinterpret_cast<__nv_bfloat16*>(region + l.sum_off);
      out.flags[r] = reinterpret_cast<uint32_t*>(region);
    }
    out.seq = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(in.regions[in.rank]) + kSeqOffset);
    out.residual_in = static_cast<const __nv_bfloat16*>(in.residual_in);
    out.residual_out = static_cast<__nv_bfloat16*>(in.residual_out);
    out.out = static_cast<__nv_bfloat16*>(in.out);
    if (mode == EPI_ADD_RMSNORM_SHARDED) {
      if (in.residual_out == nullptr) return fail(DF_EINVAL, "residual_out is NULL");
      if ((reinterpret_cast<uintptr_t>(in.residual_out) & 15u) || (reinterpret_cast<uintptr_t>(in.residual_in) & 15u) ||
          (reinterpret_cast<uintptr_t>(weight) & 15u))
        return fail(DF_EINVAL, "residual and weight pointers must be 16-byte aligned");
    }
    if (mode == EPI_ADD_RMSNORM) {
      if (in.residual_out == nullptr || in.out == nullptr) return fail(DF_EINVAL, "residual_out / out is NULL");
      if ((reinterpret_cast<uintptr_t>(in.residual_out) & 15u) || (reinterpret_cast<uintptr_t>(in.out) & 15u) ||
          (reinterpret_cast<uintptr_t>(in.residual_in) & 15u) || (reinterpret_cast<uintptr_t>(weight) & 15u))
        return fail(DF_EINVAL, "residual, out and weight pointers must be 16-byte aligned");
    }
  }
  p->weight = static_cast<const __nv_bfloat16*>(weight);
  p->world = world;
  p->T = T;
  p->H = H;
  p->mode = mode;
  p->coll = coll;
  p->eps = eps;
  p->timeout_ns = timeout_ns();
  p->status = reinterpret_cast<Status*>(dev_status);
  return DF_OK;
}

static int clamp_ctas(int n_ctas) {
  if (n_ctas <= 0) n_ctas = 32;
  return n_ctas > kMaxCtas ? kMaxCtas : n_ctas;
}

}  // namespace df

extern "C" {

size_t df_comm_region_bytes(int max_rows, int hidden) {
  if (max_rows <= 0 || hidden <= 0 || (hidden % 8) != 0) return 0;
  return df::region_layout(max_rows, hidden).total;
}

size_t df_comm_partial_offset(int max_rows, int hidden) { return df::region_layout(max_rows, hidden).partial_off; }

size_t df_comm_sum_offset(int max_rows, int hidden) { return df::region_layout(max_rows, hidden).sum_off; }

int df_comm_region_alloc(size_t bytes, void** dev_ptr, unsigned char ipc_handle[64]) {
  if (dev_ptr == nullptr || bytes < df::kHeaderBytes) return df::fail(DF_EINVAL, "bad region size or NULL output pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, df::kHeaderBytes);  // flags and sequence numbers start at zero
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess && ipc_handle != nullptr) {
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) std::memcpy(ipc_handle, &h, 64);
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    if (p != nullptr) cudaFree(p);
    return df::fail(DF_ECUDA, "region alloc: %s", cudaGetErrorString(e));
  }
  *dev_ptr = p;
  return DF_OK;
}

int df_comm_region_open(const unsigned char ipc_handle[64], void** dev_ptr) {
  if (ipc_handle == nullptr || dev_ptr == nullptr) return df::fail(DF_EINVAL, "NULL pointer argument");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, ipc_handle, 64);
  cudaError_t e = cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return df::fail(DF_ECUDA, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  }
  return DF_OK;
}

int df_comm_region_close(void* peer_ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(peer_ptr);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return df::fail(DF_ECUDA, "cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
  }
  return DF_OK;
}

int df_comm_region_free(void* dev_ptr) {
  cudaError_t e = cudaFree(dev_ptr);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return df::fail(DF_ECUDA, "cudaFree: %s", cudaGetErrorString(e));
  }
  return DF_OK;
}

int df_allreduce_bf16(const df_comm_rank_t* view, int world, int max_rows, int hidden, int T, int n_ctas,
                      df_status_t* dev_status, void* stream) {
  df::CommParams p;
  int r = df::fill_params(&p, 1, view, world, max_rows, hidden, T, hidden, df::EPI_NONE, nullptr, 0.0f, dev_status);
  if (r != DF_OK) return r;
  return df::launch_allreduce<false>(p, df::clamp_ctas(n_ctas), 1, stream);
}

int df_reduce_scatter_bf16(const df_comm_rank_t* view, int world, int max_rows, int hidden, int T, int n_ctas,
                           df_status_t* dev_status, void* stream) {
  df::CommParams p;
  int r = df::fill_params(&p, 1, view, world, max_rows, hidden, T, hidden, df::EPI_NONE, nullptr, 0.0f, dev_status, 1);
  if (r != DF_OK) return r;
  return df::launch_allreduce<false>(p, df::clamp_ctas(n_ctas), 1, stream);
}

int df_all_gather_bf16(const df_comm_rank_t* view, int world, int max_rows, int hidden, int T, int n_ctas,
                       df_status_t* dev_status, void* stream) {
  df::CommParams p;
  int r = df::fill_params(&p, 1, view, world, max_rows, hidden, T, hidden, df::EPI_NONE, nullptr, 0.0f, dev_status, 2);
  if (r != DF_OK) return r;
  return df::launch_allreduce<false>(p, df::clamp_ctas(n_ctas), 1, stream);
}

int df_allreduce_add_rmsnorm_bf16(const df_comm_rank_t* view, int world, int max_rows, int hidden, int T,
                                  const void* weight, float eps, int n_ctas, df_status_t* dev_status, void* stream) {
  df::CommParams p;
  int r = df::fill_params(&p, 1, view, world, max_rows, hidden, T, hidden, df::EPI_ADD_RMSNORM, weight, eps, dev_status);
  if (r != DF_OK) return r;
  return df::launch_allreduce<false>(p, df::clamp_ctas(n_ctas), 1, stream);
}

int df_allreduce_add_rmsnorm_sharded_bf16(const df_comm_rank_t* view, int world, int max_rows, int hidden, int T,
                                          const void* weight, float eps, int n_ctas, df_status_t* dev_status,
                                          void* stream) {
  df::CommParams p;
  int r = df::fill_params(&p, 1, view, world, max_rows, hidden, T, hidden, df::EPI_ADD_RMSNORM_SHARDED, weight, eps,
                          dev_status);
  if (r != DF_OK) return r;
  return df::launch_allreduce<false>(p, df::clamp_ctas(n_ctas), 1, stream);
}

int df_comm_set_exclusive_smem(int bytes) {
  if (bytes < 0 || bytes > 96 * 1024) return df::fail(DF_EINVAL, "exclusive shared memory must be within [0, 98304] bytes");
  df::g_exclusive_smem = bytes;
  return DF_OK;
}

int df_allreduce_multicast_bf16(const df_comm_rank_t* view, void* mc_region, int world, int max_rows, int hidden, int T,
                                int fuse, const void* weight, float eps, int n_ctas, df_status_t* dev_status,
                                void* stream) {
  if (mc_region == nullptr || (reinterpret_cast<uintptr_t>(mc_region) & 255u) != 0)
    return df::fail(DF_EINVAL, "the multicast address of the region is NULL or not 256-byte aligned");
  if (fuse != 0 && fuse != 1) return df::fail(DF_EINVAL, "fuse must be 0 (all-reduce) or 1 (sharded add + RMSNorm)");
  df::CommParams p;
  const int mode = fuse ? df::EPI_ADD_RMSNORM_SHARDED : df::EPI_NONE;
  int r = df::fill_params(&p, 1, view, world, max_rows, hidden, T, hidden, mode, weight, eps, dev_status);
  if (r != DF_OK) return r;
  const df::RegionLayout l = df::region_layout(max_rows, hidden);
  const __nv_bfloat16* mc_partial = reinterpret_cast<const __nv_bfloat16*>(static_cast<uint8_t*>(mc_region) + l.partial_off);
  __nv_bfloat16* mc_sum = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(mc_region) + l.sum_off);
  size_t smem = (fuse && hidden <= df::kMaxSmemHidden) ? static_cast<size_t>(hidden) * 2 : 0;
  if (df::g_exclusive_smem > 0) {
    smem += static_cast<size_t>(df::g_exclusive_smem);
    const cudaError_t ae =
        fuse ? cudaFuncSetAttribute(df::allreduce_multicast_kernel<df::EPI_ADD_RMSNORM_SHARDED>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))
             : cudaFuncSetAttribute(df::allreduce_multicast_kernel<df::EPI_NONE>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (ae != cudaSuccess) return df::fail(DF_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(ae));
  }
  const int ctas = df::clamp_ctas(n_ctas);
  if (fuse) {
    df::allreduce_multicast_kernel<df::EPI_ADD_RMSNORM_SHARDED>
        <<<ctas, df::kCommThreads, smem, static_cast<cudaStream_t>(stream)>>>(p, mc_partial, mc_sum);
  } else {
    df::allreduce_multicast_kernel<df::EPI_NONE>
        <<<ctas, df::kCommThreads, smem, static_cast<cudaStream_t>(stream)>>>(p, mc_partial, mc_sum);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return df::fail(DF_ECUDA, "multicast all-reduce launch: %s", cudaGetErrorString(e));
  return DF_OK;
}

int df_add_rmsnorm_bf16(const void* y, const void* residual_in, void* residual_out, void* out, const void* weight,
                        float eps, int T, int H, void* stream) {
  if (y == nullptr || residual_out == nullptr || out == nullptr || weight == nullptr)
    return df::fail(DF_EINVAL, "NULL pointer argument");
  if (T <= 0 || H <= 0 || (H % 8) != 0) return df::fail(DF_EINVAL, "T must be positive and H a positive multiple of 8");
  const uintptr_t bits = reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(residual_in) |
                         reinterpret_cast<uintptr_t>(residual_out) | reinterpret_cast<uintptr_t>(out) |
                         reinterpret_cast<uintptr_t>(weight);
  if (bits & 15u) return df::fail(DF_EINVAL, "pointers must be 16-byte aligned");
  int sms = df_sm_count();
  if (sms <= 0) return df::fail(DF_ECUDA, "no CUDA device");
  int grid = (T + df::kWarpsPerBlock - 1) / df::kWarpsPerBlock;
  if (grid > sms * 8) grid = sms * 8;
  // with a warp per row, fewer CTAs than SMs: a CTA per row instead (hidden <= 8192: four vectors per thread)
  const bool block_per_row = grid < sms && H <= 8192;
  if (block_per_row) grid = T < sms * 2 ? T : sms * 2;
  const size_t smem = H <= df::kMaxSmemHidden ? static_cast<size_t>(H) * 2 : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(df::kCommThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr;
  cfg.numAttrs = df::dependent_launch_attr(&attr);
  cfg.attrs = &attr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, df::add_rmsnorm_kernel, static_cast<const __nv_bfloat16*>(y),
                                     static_cast<const __nv_bfloat16*>(residual_in), static_cast<__nv_bfloat16*>(residual_out),
                                     static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(weight), T, H, eps,
                                     block_per_row);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return df::fail(DF_ECUDA, "add_rmsnorm launch: %s", cudaGetErrorString(e));
  }
  return DF_OK;
}

int df_allreduce_emulated_bf16(const df_comm_rank_t* views, int world, int max_rows, int hidden, int T,
                               const void* weight, float eps, int fuse_rmsnorm, int n_ctas, df_status_t* dev_status,
                               void* stream) {
  df::CommParams p;
  const int mode = fuse_rmsnorm == 2 ? df::EPI_ADD_RMSNORM_SHARDED : (fuse_rmsnorm == 1 ? df::EPI_ADD_RMSNORM : df::EPI_NONE);
  const int coll = fuse_rmsnorm == 3 ? 1 : (fuse_rmsnorm == 4 ? 2 : 0);
  int r = df::fill_params(&p, world, views, world, max_rows, hidden, T, hidden, mode, weight, eps, dev_status, coll);
  if (r != DF_OK) return r;
  for (int v = 0; v < world; ++v)
    if (views[v].rank != v) return df::fail(DF_EINVAL, "emulated views must be listed in rank order");
  return df::launch_allreduce<true>(p, df::clamp_ctas(n_ctas), world, stream);
}

}  // extern "C"
