// Expert-parallel all-to-all over NVLink peer memory: dispatch (every rank PUTS the token rows routed
// to an expert straight into the packed input of the rank that owns the expert, plain peer stores,
// after the per-(source, expert) counts have been exchanged) and combine (every rank PULLS the two
// expert outputs of each of its tokens from the owners' packed outputs and sums them with the
// routing weights in fp32). Only the rows that are actually routed cross the links: 2 x tokens x
// hidden per layer and direction in total, against `world` times that for the all-gather /
// reduce-scatter form.
//
// Every rank owns a "region" that all ranks have mapped:
//   flag words and per-block sequence numbers (the same block-to-block barrier as the reduction
//   kernels: block b of a rank only ever synchronises with block b of its peers)
//   counts[block][source rank][expert]   how many rows source sends to expert, one copy per block
//   rows_total[local expert]             rows that arrived for a local expert (the expert MLP reads
//                                        its row count from here, in device memory)
//   packed_in [local expert][capacity][hidden]   rows, grouped by source rank, in token order
//   packed_out[local expert][capacity][hidden]   the expert MLP's output rows, same positions
//
// Row (token t, choice c) with expert e of source rank s lands at
//   row = sum_{s' < s} counts[s'][e] + pos[t, c]       (pos = rank of the pair among the source's
//                                                       pairs with the same expert, in token order)
// which every rank can compute from the exchanged count matrix; nothing else is communicated.
// Waits are bounded; a peer that never arrives yields DF_ERR_PEER and the kernel returns.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#include "../../include/dynaflow_b200.h"
#include "host_util.h"
#include "ptx.cuh"

namespace df {
namespace a2a {

constexpr int kMaxWorld = DF_COMM_MAX_WORLD;
constexpr int kMaxCtas = DF_COMM_MAX_CTAS;
constexpr int kMaxExperts = DF_A2A_MAX_EXPERTS;
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr unsigned WHERE_A2A_FLAG = 48;

constexpr size_t kFlagBytes = 2ull * kMaxCtas * kMaxWorld * 4;
constexpr size_t kSeqOffset = kFlagBytes;                       // uint32 seq[kMaxCtas]
constexpr size_t kCountsOffset = 8192;                          // int counts[kMaxCtas][kMaxWorld][kMaxExperts]
constexpr size_t kCountsBytes = size_t(kMaxCtas) * kMaxWorld * kMaxExperts * 4;
constexpr size_t kRowsTotalOffset = kCountsOffset + kCountsBytes;  // int rows_total[kMaxExperts]
constexpr size_t kHeaderBytes = kRowsTotalOffset + 1024;

static size_t align256(size_t x) { return (x + 255) / 256 * 256; }

struct Layout {
  size_t in_off, out_off, total;
};
static Layout layout(int local_experts, int capacity, int hidden) {
  Layout l;
  const size_t buf = align256(static_cast<size_t>(local_experts) * capacity * hidden * 2u);
  l.in_off = align256(kHeaderBytes);
  l.out_off = l.in_off + buf;
  l.total = l.out_off + buf;
  return l;
}

struct View {
  int rank;
  uint8_t* region[kMaxWorld];
};

struct Params {
  View ranks[kMaxWorld];  // [0] only, unless several ranks are emulated on one GPU
  int world, experts, local_experts, capacity, H, tokens;
  size_t in_off, out_off;
  // per rank (emulation: one set per emulated rank)
  const __nv_bfloat16* x[kMaxWorld];   // [tokens, H] this rank's token rows (dispatch)
  const int* ids[kMaxWorld];           // [tokens, 2]
  const int* pos[kMaxWorld];           // [tokens, 2]
  const int* counts[kMaxWorld];        // [experts] this rank's pairs per expert
  const float* weights[kMaxWorld];     // [tokens, 2] (combine)
  __nv_bfloat16* out[kMaxWorld];       // [tokens, H] (combine)
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

// Block b of this rank <-> block b of every peer; thread t < world signals peer t and waits for it.
__device__ __forceinline__ bool peer_barrier(const View& me, int world, int phase, uint32_t seq, unsigned long long t_end,
                                             Status* status, uint32_t* s_abort) {
  __syncthreads();
  const int t = threadIdx.x;
  if (t < world) {
    const uint32_t value = seq * 2u + static_cast<uint32_t>(phase) + 1u;
    const size_t slot = (static_cast<size_t>(phase) * kMaxCtas + blockIdx.x) * kMaxWorld;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(me.region[t]) + slot + me.rank, value);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(me.region[me.rank]) + slot + t;
    uint32_t spins = 0, seen;
    while (static_cast<int32_t>((seen = ld_acquire_sys(mine)) - value) < 0) {
      if ((++spins & 0xffu) == 0u && globaltimer_ns() > t_end) {
        seen = value + 1u;  // reported below
        break;
      }
    }
    if (seen != value) {  // timed out, or a peer that is out of step
      *s_abort = 1u;
      report(status, 2u /*DF_ERR_PEER*/, WHERE_A2A_FLAG + phase, static_cast<unsigned>(t));
    }
  }
  __syncthreads();
  return *s_abort == 0u;
}

// Positions of a rank's (token, choice) pairs among its pairs with the same expert, in token
// order, and the per-expert totals. One CTA; the pairs are walked in chunks of 256.
__global__ void __launch_bounds__(kThreads) plan_kernel(const int* __restrict__ ids, int tokens, int experts,
                                                        int* __restrict__ pos, int* __restrict__ counts) {
  __shared__ int base[kMaxExperts];
  __shared__ int warp_cnt[kWarps][kMaxExperts];
  for (int e = threadIdx.x; e < experts; e += kThreads) base[e] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = 2 * tokens;
  for (int i0 = 0; i0 < n; i0 += kThreads) {
    const int i = i0 + threadIdx.x;
    const int e = i < n ? ids[i] : -1;
    // rank of this pair among the earlier lanes of its warp with the same expert
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int in_warp = __popc(same & ((1u << lane) - 1u));
    for (int x = lane; x < experts; x += 32) warp_cnt[warp][x] = 0;
    __syncwarp();
    if (e >= 0 && in_warp == 0) warp_cnt[warp][e] = __popc(same);  // the first lane of each group
    __syncthreads();
    if (e >= 0) {
      int before = base[e];
      for (int w = 0; w < warp; ++w) before += warp_cnt[w][e];
      pos[i] = before + in_warp;
    }
    __syncthreads();
    for (int x = threadIdx.x; x < experts; x += kThreads) {
      int total = 0;
      for (int w = 0; w < kWarps; ++w) total += warp_cnt[w][x];
      base[x] += total;
    }
    __syncthreads();
  }
  for (int e = threadIdx.x; e < experts; e += kThreads) counts[e] = base[e];
}

// rows before (source rank, expert) in the expert's packed buffer, from the block's copy of the counts
__device__ __forceinline__ int segment_start(const int* cnt /*[world][kMaxExperts]*/, int src, int e) {
  int off = 0;
  for (int s = 0; s < src; ++s) off += cnt[s * kMaxExperts + e];
  return off;
}

template <bool EMULATE>
__global__ void __launch_bounds__(kThreads, 2) dispatch_kernel(const Params p) {
  __shared__ uint32_t s_abort;
  __shared__ int s_off[kMaxExperts];
  const int r_idx = EMULATE ? blockIdx.y : 0;
  const View& me = p.ranks[r_idx];
  if (threadIdx.x == 0) s_abort = 0u;
  const unsigned long long t_end = globaltimer_ns() + p.timeout_ns;
  uint32_t* seq_ptr = reinterpret_cast<uint32_t*>(me.region[me.rank] + kSeqOffset);
  const uint32_t seq = seq_ptr[blockIdx.x];
  const int W = p.world, E = p.experts;
  // this block's copy of this rank's counts, to every rank (its own included)
  for (int i = threadIdx.x; i < W * E; i += kThreads) {
    const int dst = i / E, e = i - dst * E;
    int* cnt = reinterpret_cast<int*>(me.region[dst] + kCountsOffset) +
               (static_cast<size_t>(blockIdx.x) * kMaxWorld + me.rank) * kMaxExperts;
    cnt[e] = p.counts[r_idx][e];
  }
  bool ok = peer_barrier(me, W, 0, seq, t_end, p.status, &s_abort);
  if (ok) {
    const int* cnt = reinterpret_cast<const int*>(me.region[me.rank] + kCountsOffset) +
                     static_cast<size_t>(blockIdx.x) * kMaxWorld * kMaxExperts;
    for (int e = threadIdx.x; e < E; e += kThreads) {
      s_off[e] = segment_start(cnt, me.rank, e);
      if (blockIdx.x == 0 && e / p.local_experts == me.rank) {
        // rows that arrive for a local expert, capped at what its buffer holds
        const int total = segment_start(cnt, W, e);
        reinterpret_cast<int*>(me.region[me.rank] + kRowsTotalOffset)[e % p.local_experts] = min(total, p.capacity);
      }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nvec = p.H >> 3;
    const int pairs = 2 * p.tokens;
    for (int i = blockIdx.x * kWarps + warp; i < pairs; i += gridDim.x * kWarps) {
      const int e = p.ids[r_idx][i];
      const int dst = e / p.local_experts, el = e - dst * p.local_experts;
      const int row = s_off[e] + p.pos[r_idx][i];
      if (row >= p.capacity) continue;  // beyond the buffer: dropped (capacity = all tokens never overflows)
      const uint4* src = reinterpret_cast<const uint4*>(p.x[r_idx] + static_cast<size_t>(i >> 1) * p.H);
      uint4* to = reinterpret_cast<uint4*>(me.region[dst] + p.in_off) +
                  (static_cast<size_t>(el) * p.capacity + row) * nvec;
      for (int v0 = lane; v0 < nvec; v0 += 32 * 8) {
        uint4 buf[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v0 + 32 * u < nvec) buf[u] = __ldg(src + v0 + 32 * u);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v0 + 32 * u < nvec) __stcg(to + v0 + 32 * u, buf[u]);
      }
    }
    ok = peer_barrier(me, W, 1, seq, t_end, p.status, &s_abort);  // every rank's rows have landed
  }
  __syncthreads();
  if (threadIdx.x == 0) seq_ptr[blockIdx.x] = seq + 1u;
}

template <bool EMULATE>
__global__ void __launch_bounds__(kThreads, 2) combine_kernel(const Params p) {
  __shared__ uint32_t s_abort;
  __shared__ int s_off[kMaxExperts];
  const int r_idx = EMULATE ? blockIdx.y : 0;
  const View& me = p.ranks[r_idx];
  if (threadIdx.x == 0) s_abort = 0u;
  const unsigned long long t_end = globaltimer_ns() + p.timeout_ns;
  uint32_t* seq_ptr = reinterpret_cast<uint32_t*>(me.region[me.rank] + kSeqOffset);
  const uint32_t seq = seq_ptr[blockIdx.x];
  const int W = p.world, E = p.experts;
  // every rank's expert outputs are complete (its expert launches precede this one on its stream)
  bool ok = peer_barrier(me, W, 0, seq, t_end, p.status, &s_abort);
  if (ok) {
    const int* cnt = reinterpret_cast<const int*>(me.region[me.rank] + kCountsOffset) +
                     static_cast<size_t>(blockIdx.x) * kMaxWorld * kMaxExperts;
    for (int e = threadIdx.x; e < E; e += kThreads) s_off[e] = segment_start(cnt, me.rank, e);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nvec = p.H >> 3;
    for (int t = blockIdx.x * kWarps + warp; t < p.tokens; t += gridDim.x * kWarps) {
      const uint4* src[2];
      float w[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int e = p.ids[r_idx][2 * t + c];
        const int dst = e / p.local_experts, el = e - dst * p.local_experts;
        const int row = s_off[e] + p.pos[r_idx][2 * t + c];
        w[c] = row < p.capacity ? p.weights[r_idx][2 * t + c] : 0.0f;
        src[c] = reinterpret_cast<const uint4*>(me.region[dst] + p.out_off) +
                 (static_cast<size_t>(el) * p.capacity + min(row, p.capacity - 1)) * nvec;
      }
      uint4* to = reinterpret_cast<uint4*>(p.out[r_idx] + static_cast<size_t>(t) * p.H);
      for (int v0 = lane; v0 < nvec; v0 += 32 * 4) {
        uint4 a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (v0 + 32 * u < nvec) {
            a[u] = __ldcg(src[0] + v0 + 32 * u);
            b[u] = __ldcg(src[1] + v0 + 32 * u);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (v0 + 32 * u < nvec) {
            const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a[u]);
            const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b[u]);
            uint4 o;
            __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 fa = __bfloat1622float2(ha[i]), fb = __bfloat1622float2(hb[i]);
              // fp32 products and sum, rounded once
              ho[i] = __floats2bfloat162_rn(fa.x * w[0] + fb.x * w[1], fa.y * w[0] + fb.y * w[1]);
            }
            to[v0 + 32 * u] = o;
          }
        }
      }
    }
    ok = peer_barrier(me, W, 1, seq, t_end, p.status, &s_abort);  // nobody overwrites a buffer a peer still reads
  }
  __syncthreads();
  if (threadIdx.x == 0) seq_ptr[blockIdx.x] = seq + 1u;
}

static int fill_common(Params& p, const df_a2a_rank_t* views, int n_views, int world, int experts, int capacity, int hidden,
                       int tokens, df_status_t* dev_status) {
  if (views == nullptr || dev_status == nullptr) return fail(DF_EINVAL, "NULL pointer argument");
  if (world < 1 || world > kMaxWorld) return fail(DF_EINVAL, "world must be in [1, %d] (got %d)", kMaxWorld, world);
  if (experts < 2 || experts > kMaxExperts || experts % world != 0)
    return fail(DF_EINVAL, "experts must be in [2, %d] and divide evenly across ranks (got %d on %d ranks)", kMaxExperts, experts, world);
  if (capacity <= 0 || tokens <= 0 || hidden <= 0 || (hidden % 8) != 0)
    return fail(DF_EINVAL, "capacity and tokens must be positive, hidden a positive multiple of 8");
  std::memset(&p, 0, sizeof(p));
  p.world = world;
  p.experts = experts;
  p.local_experts = experts / world;
  p.capacity = capacity;
  p.H = hidden;
  p.tokens = tokens;
  const Layout l = layout(p.local_experts, capacity, hidden);
  p.in_off = l.in_off;
  p.out_off = l.out_off;
  p.timeout_ns = timeout_ns();
  p.status = reinterpret_cast<Status*>(dev_status);
  for (int v = 0; v < n_views; ++v) {
    if (views[v].rank < 0 || views[v].rank >= world) return fail(DF_EINVAL, "rank %d is outside [0, %d)", views[v].rank, world);
    p.ranks[v].rank = views[v].rank;
    for (int r = 0; r < world; ++r) {
      if (views[v].regions[r] == nullptr) return fail(DF_EINVAL, "region of rank %d is NULL", r);
      p.ranks[v].region[r] = static_cast<uint8_t*>(views[v].regions[r]);
    }
  }
  return DF_OK;
}

static int grid_for(int n_ctas) {
  if (n_ctas <= 0) n_ctas = 32;
  return n_ctas > kMaxCtas ? kMaxCtas : n_ctas;
}

}  // namespace a2a
}  // namespace df

extern "C" {

size_t df_a2a_region_bytes(int world, int experts, int capacity, int hidden) {
  if (world < 1 || experts < world || experts % world != 0 || capacity <= 0 || hidden <= 0) return 0;
  return df::a2a::layout(experts / world, capacity, hidden).total;
}
size_t df_a2a_packed_in_offset(int world, int experts, int capacity, int hidden) {
  if (world < 1 || experts < world || experts % world != 0 || capacity <= 0 || hidden <= 0) return 0;
  return df::a2a::layout(experts / world, capacity, hidden).in_off;
}
size_t df_a2a_packed_out_offset(int world, int experts, int capacity, int hidden) {
  if (world < 1 || experts < world || experts % world != 0 || capacity <= 0 || hidden <= 0) return 0;
  return df::a2a::layout(experts / world, capacity, hidden).out_off;
}
size_t df_a2a_rows_total_offset(void) { return df::a2a::kRowsTotalOffset; }

int df_a2a_plan(const int* ids, int tokens, int experts, int* pos, int* counts, void* stream) {
  using namespace df;
  if (ids == nullptr || pos == nullptr || counts == nullptr) return fail(DF_EINVAL, "NULL pointer argument");
  if (tokens <= 0 || experts < 2 || experts > a2a::kMaxExperts)
    return fail(DF_EINVAL, "tokens must be positive, experts in [2, %d]", a2a::kMaxExperts);
  a2a::plan_kernel<<<1, a2a::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(ids, tokens, experts, pos, counts);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DF_ECUDA, "a2a plan launch: %s", cudaGetErrorString(e));
  return DF_OK;
}

int df_a2a_dispatch_bf16(const df_a2a_rank_t* view, int world, int experts, int capacity, int hidden, const void* x,
                         const int* ids, const int* pos, const int* counts, int tokens, int n_ctas,
                         df_status_t* dev_status, void* stream) {
  using namespace df;
  if (x == nullptr || ids == nullptr || pos == nullptr || counts == nullptr) return fail(DF_EINVAL, "NULL pointer argument");
  a2a::Params p;
  int rc = a2a::fill_common(p, view, 1, world, experts, capacity, hidden, tokens, dev_status);
  if (rc != DF_OK) return rc;
  p.x[0] = static_cast<const __nv_bfloat16*>(x);
  p.ids[0] = ids;
  p.pos[0] = pos;
  p.counts[0] = counts;
  a2a::dispatch_kernel<false><<<a2a::grid_for(n_ctas), a2a::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DF_ECUDA, "a2a dispatch launch: %s", cudaGetErrorString(e));
  return DF_OK;
}

int df_a2a_combine_bf16(const df_a2a_rank_t* view, int world, int experts, int capacity, int hidden, const int* ids,
                        const int* pos, const float* weights, int tokens, void* out, int n_ctas,
                        df_status_t* dev_status, void* stream) {
  using namespace df;
  if (ids == nullptr || pos == nullptr || weights == nullptr || out == nullptr) return fail(DF_EINVAL, "NULL pointer argument");
  a2a::Params p;
  int rc = a2a::fill_common(p, view, 1, world, experts, capacity, hidden, tokens, dev_status);
  if (rc != DF_OK) return rc;
  p.ids[0] = ids;
  p.pos[0] = pos;
  p.weights[0] = weights;
  p.out[0] = static_cast<__nv_bfloat16*>(out);
  a2a::combine_kernel<false><<<a2a::grid_for(n_ctas), a2a::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DF_ECUDA, "a2a combine launch: %s", cudaGetErrorString(e));
  return DF_OK;
}

int df_a2a_emulated_bf16(const df_a2a_rank_t* views, int world, int experts, int capacity, int hidden, int tokens,
                         const void* const* x, const int* const* ids, const int* const* pos, const int* const* counts,
                         const float* const* weights, void* const* out, int combine, int n_ctas, df_status_t* dev_status,
                         void* stream) {
  using namespace df;
  if (ids == nullptr || pos == nullptr) return fail(DF_EINVAL, "NULL pointer argument");
  a2a::Params p;
  int rc = a2a::fill_common(p, views, world, world, experts, capacity, hidden, tokens, dev_status);
  if (rc != DF_OK) return rc;
  for (int r = 0; r < world; ++r) {
    p.ids[r] = ids[r];
    p.pos[r] = pos[r];
    if (combine) {
      if (weights == nullptr || out == nullptr) return fail(DF_EINVAL, "NULL pointer argument");
      p.weights[r] = weights[r];
      p.out[r] = static_cast<__nv_bfloat16*>(out[r]);
    } else {
      if (x == nullptr || counts == nullptr) return fail(DF_EINVAL, "NULL pointer argument");
      p.x[r] = static_cast<const __nv_bfloat16*>(x[r]);
      p.counts[r] = counts[r];
    }
  }
  // all ranks' blocks wait on one another: they must be co-resident (cooperative launch)
  const dim3 grid(a2a::grid_for(n_ctas), world, 1);
  void* args[] = {&p};
  const void* fn = combine ? reinterpret_cast<const void*>(a2a::combine_kernel<true>)
                           : reinterpret_cast<const void*>(a2a::dispatch_kernel<true>);
  const cudaError_t e = cudaLaunchCooperativeKernel(fn, grid, dim3(a2a::kThreads), args, 0, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(DF_ECUDA, "emulated a2a launch: %s", cudaGetErrorString(e));
  }
  return DF_OK;
}

}  // extern "C"
