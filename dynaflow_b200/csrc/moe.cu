// Routing and token movement of a top-2 mixture-of-experts layer, the parts of the
// dispatch / expert / combine operator triple that are not GEMMs:
//
//   route_top2     softmax over the router logits, two largest, renormalised
//   select_rows    the tokens routed to one expert, in ascending token order, with the
//                  inverse map, and their number left on the device
//   gather_rows    those tokens' hidden rows packed into a dense matrix (the expert MLP's A)
//   scatter_rows   the expert's output rows, scaled by the routing weight, written back to
//                  their token positions of a [T, H] contribution buffer, zeros elsewhere
//
// All of it is integer / byte work bound by HBM; nothing here syncs with the host, so the
// number of routed tokens never leaves the device (the expert GEMMs read it there).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/dynaflow_b200.h"
#include "host_util.h"

namespace df {

constexpr int kMoeThreads = 256;

// One thread per token. Ties resolve to the lower expert index.
__global__ void route_top2_kernel(const __nv_bfloat16* __restrict__ logits, int T, int E, int* __restrict__ ids,
                                  float* __restrict__ weights) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const __nv_bfloat16* row = logits + static_cast<size_t>(t) * E;
  float best = -INFINITY, second = -INFINITY;
  int ibest = 0, isecond = 0;
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) mx = fmaxf(mx, __bfloat162float(row[e]));
  float denom = 0.0f;
  for (int e = 0; e < E; ++e) denom += expf(__bfloat162float(row[e]) - mx);
  for (int e = 0; e < E; ++e) {
    const float p = expf(__bfloat162float(row[e]) - mx) / denom;
    if (p > best) {
      second = best;
      isecond = ibest;
      best = p;
      ibest = e;
    } else if (p > second) {
      second = p;
      isecond = e;
    }
  }
  const float s = best + second;
  ids[2 * t] = ibest;
  ids[2 * t + 1] = isecond;
  weights[2 * t] = best / s;
  weights[2 * t + 1] = second / s;
}

// One CTA walks the tokens in chunks of blockDim.x and compacts, in token order, those whose
// top-2 contains `expert`. rows[k] = token of the k-th selected row, pos[t] = k or -1,
// slot[k] = 0/1 (which of the token's two choices), *count = number selected.
__global__ void select_rows_kernel(const int* __restrict__ ids, int T, int expert, int* __restrict__ rows,
                                   int* __restrict__ slot, int* __restrict__ pos, int* __restrict__ count) {
  __shared__ int warp_sums[kMoeThreads / 32];
  __shared__ int base;
  if (threadIdx.x == 0) base = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int t0 = 0; t0 < T; t0 += blockDim.x) {
    const int t = t0 + threadIdx.x;
    int which = -1;
    if (t < T) {
      if (ids[2 * t] == expert) which = 0;
      else if (ids[2 * t + 1] == expert) which = 1;
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, which >= 0);
    const int in_warp = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) warp_sums[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, total = 0;
    for (int w = 0; w < kMoeThreads / 32; ++w) {
      if (w < warp) before += warp_sums[w];
      total += warp_sums[w];
    }
    const int start = base;
    if (t < T) {
      if (which >= 0) {
        const int k = start + before + in_warp;
        rows[k] = t;
        slot[k] = which;
        pos[t] = k;
      } else {
        pos[t] = -1;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) base = start + total;
    __syncthreads();
  }
  if (threadIdx.x == 0) *count = base;
}

// out[k, :] = x[rows[k], :] for k < min(*count, capacity); one warp per row, 16-byte vectors.
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ rows,
                                   const int* __restrict__ count, int capacity, int H, __nv_bfloat16* __restrict__ out) {
  const int n = min(*count, capacity);
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int k = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; k < n; k += warps) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(rows[k]) * H);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(k) * H);
    for (int v = lane; v < nvec; v += 32) dst[v] = __ldg(src + v);
  }
}

// contrib[t, :] = bf16(weights[t, slot] * y[pos[t], :]) if pos[t] >= 0 else 0; one warp per token.
__global__ void scatter_rows_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos,
                                    const int* __restrict__ slot, const float* __restrict__ weights, int T, int H,
                                    __nv_bfloat16* __restrict__ contrib) {
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    uint4* dst = reinterpret_cast<uint4*>(contrib + static_cast<size_t>(t) * H);
    const int k = pos[t];
    if (k < 0) {
      for (int v = lane; v < nvec; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const float w = weights[2 * t + slot[k]];
    const uint4* src = reinterpret_cast<const uint4*>(y + static_cast<size_t>(k) * H);
    for (int v = lane; v < nvec; v += 32) {
      uint4 in = __ldg(src + v), o;
      const __nv_bfloat162* hi = reinterpret_cast<const __nv_bfloat162*>(&in);
      __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(hi[i]);
        ho[i] = __floats2bfloat162_rn(f.x * w, f.y * w);
      }
      dst[v] = o;
    }
  }
}

static int grid_for_rows(int rows) {
  int sms = df_sm_count();
  if (sms <= 0) sms = 148;
  int g = (rows + (kMoeThreads / 32) - 1) / (kMoeThreads / 32);
  if (g > sms * 8) g = sms * 8;
  return g < 1 ? 1 : g;
}

static int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DF_ECUDA, "%s launch: %s", what, cudaGetErrorString(e));
  return DF_OK;
}

}  // namespace df

extern "C" {

int df_moe_route_top2(const void* logits, int T, int E, int* ids, float* weights, void* stream) {
  if (logits == nullptr || ids == nullptr || weights == nullptr) return df::fail(DF_EINVAL, "NULL pointer argument");
  if (T <= 0 || E < 2) return df::fail(DF_EINVAL, "need T > 0 tokens and E >= 2 experts (got %d, %d)", T, E);
  df::route_top2_kernel<<<(T + df::kMoeThreads - 1) / df::kMoeThreads, df::kMoeThreads, 0,
                          static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(logits), T, E, ids,
                                                               weights);
  return df::check_launch("route_top2");
}

int df_moe_select_rows(const int* ids, int T, int expert, int* rows, int* slot, int* pos, int* count_dev, void* stream) {
  if (ids == nullptr || rows == nullptr || slot == nullptr || pos == nullptr || count_dev == nullptr)
    return df::fail(DF_EINVAL, "NULL pointer argument");
  if (T <= 0 || expert < 0) return df::fail(DF_EINVAL, "need T > 0 and expert >= 0");
  df::select_rows_kernel<<<1, df::kMoeThreads, 0, static_cast<cudaStream_t>(stream)>>>(ids, T, expert, rows, slot, pos,
                                                                                      count_dev);
  return df::check_launch("select_rows");
}

int df_moe_gather_rows(const void* x, const int* rows, const int* count_dev, int capacity, int H, void* out,
                       void* stream) {
  if (x == nullptr || rows == nullptr || count_dev == nullptr || out == nullptr)
    return df::fail(DF_EINVAL, "NULL pointer argument");
  if (capacity <= 0 || H <= 0 || (H % 8) != 0) return df::fail(DF_EINVAL, "capacity must be positive, H a multiple of 8");
  df::gather_rows_kernel<<<df::grid_for_rows(capacity), df::kMoeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), rows, count_dev, capacity, H, static_cast<__nv_bfloat16*>(out));
  return df::check_launch("gather_rows");
}

int df_moe_scatter_rows(const void* y, const int* pos, const int* slot, const float* weights, int T, int H,
                        void* contrib, void* stream) {
  if (y == nullptr || pos == nullptr || slot == nullptr || weights == nullptr || contrib == nullptr)
    return df::fail(DF_EINVAL, "NULL pointer argument");
  if (T <= 0 || H <= 0 || (H % 8) != 0) return df::fail(DF_EINVAL, "T must be positive, H a multiple of 8");
  df::scatter_rows_kernel<<<df::grid_for_rows(T), df::kMoeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), pos, slot, weights, T, H, static_cast<__nv_bfloat16*>(contrib));
  return df::check_launch("scatter_rows");
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Rotary position embedding, rotate-half convention, in place on the q and k
// heads of a fused qkv activation [T, (q_heads + 2 * kv_heads) * head_dim]:
//   (x1, x2) <- (x1 cos - x2 sin, x2 cos + x1 sin) with x1 / x2 the two halves of a head,
//   angle = pos[t] * theta^(-2i / head_dim), computed in fp32.
// One thread per (token, head, 8 consecutive dims of the first half).
namespace df {

__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos, int T, int heads, int head_dim,
                            int row_stride, float theta) {
  const int half = head_dim >> 1;
  const int groups = half >> 3;
  const long long total = static_cast<long long>(T) * heads * groups;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int gidx = static_cast<int>(i % groups);
    const int head = static_cast<int>((i / groups) % heads);
    const int t = static_cast<int>(i / (static_cast<long long>(groups) * heads));
    __nv_bfloat16* base = qkv + static_cast<size_t>(t) * row_stride + head * head_dim + gidx * 8;
    uint4 a = *reinterpret_cast<uint4*>(base), b = *reinterpret_cast<uint4*>(base + half);
    __nv_bfloat16* x1 = reinterpret_cast<__nv_bfloat16*>(&a);
    __nv_bfloat16* x2 = reinterpret_cast<__nv_bfloat16*>(&b);
    const float p = static_cast<float>(pos[t]);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = gidx * 8 + j;
      const float inv_freq = powf(theta, -2.0f * static_cast<float>(d) / static_cast<float>(head_dim));
      float s, c;
      sincosf(p * inv_freq, &s, &c);
      const float u = __bfloat162float(x1[j]), v = __bfloat162float(x2[j]);
      x1[j] = __float2bfloat16_rn(u * c - v * s);
      x2[j] = __float2bfloat16_rn(v * c + u * s);
    }
    *reinterpret_cast<uint4*>(base) = a;
    *reinterpret_cast<uint4*>(base + half) = b;
  }
}

}  // namespace df

extern "C" int df_rope_bf16(void* qkv, const int* positions, int T, int heads, int head_dim, int row_stride, float theta,
                            void* stream) {
  if (qkv == nullptr || positions == nullptr) return df::fail(DF_EINVAL, "NULL pointer argument");
  if (T <= 0 || heads <= 0 || head_dim <= 0 || (head_dim % 16) != 0 || (row_stride % 8) != 0 ||
      row_stride < heads * head_dim)
    return df::fail(DF_EINVAL, "head_dim must be a multiple of 16 and the row stride cover the rotated heads");
  if (reinterpret_cast<uintptr_t>(qkv) & 15u) return df::fail(DF_EINVAL, "qkv must be 16-byte aligned");
  const long long total = static_cast<long long>(T) * heads * (head_dim / 16);
  int grid = static_cast<int>((total + 255) / 256);
  int sms = df_sm_count();
  if (sms <= 0) sms = 148;
  if (grid > sms * 16) grid = sms * 16;
  df::rope_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__nv_bfloat16*>(qkv), positions, T,
                                                                        heads, head_dim, row_stride, theta);
  return df::check_launch("rope");
}
