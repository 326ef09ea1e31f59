// Causal self-attention of a prefill nano-batch for sm_100a: both contractions
// (S = Q K^T and O = P V) on tcgen05 with the accumulators in tensor memory,
// operands staged by plain per-CTA TMA loads, online softmax in the epilogue warps.
//
// A work item is one tile of 128 query rows of one head of one sequence; its keys
// are visited in blocks of 128. Items are ordered by decreasing number of key
// blocks (the last query tile of every sequence first) and dealt round-robin to a
// persistent grid of at most `max_ctas` CTAs, so the launch can leave SMs to the
// reduction kernel of the other micro-batch.
//
// 256 threads per CTA:
//   warp 0      TMA producer: Q once per item, then K_j, V_j through two-stage rings
//   warp 1      MMA issuer (one lane): S_j = Q K_j^T into one of two 128-column
//               accumulators, O += P_j V_j into a third; S_{j+1} is issued before
//               P_j V_j so that it runs under the softmax of block j
//   warp 2      allocates / frees tensor memory
//   warps 4..7  softmax, one thread per query row: tcgen05.ld of the row of S,
//               causal mask on the diagonal block, running maximum, exp2, the
//               bf16 row of P into shared memory (128-byte swizzled, K-major, the
//               layout TMA would have written), rescaling of O in tensor memory
//               only when the maximum grew by more than 2^8 (the exponent then
//               simply stays relative to the older maximum), final 1/l scaling
//               and the stores of the output rows.
//
// V is consumed in the layout it has in memory ([key][dim], i.e. "MN-major" as
// the B operand of P V); the instruction descriptor's B-major bit and a shared
// memory descriptor with the 64-wide column halves 16 KB apart describe it.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../include/dynaflow_b200.h"
#include "host_util.h"
#include "ptx.cuh"

namespace df {
namespace attn {

constexpr int BQ = 128;   // query rows per work item
constexpr int BKV = 128;  // keys per block
constexpr int HD = 128;   // head dimension (the only one built)
constexpr int TILE_BYTES = 128 * 128 * 2;
constexpr int HALF_BYTES = TILE_BYTES / 2;  // one TMA box: 128 rows x 64 columns
constexpr int KV_STAGES = 2;
constexpr int THREADS = 256;
constexpr int TMEM_COLS = 512;  // S0, S1, O: 3 x 128 columns, rounded up to a power of two
constexpr int O_COL = 256;
constexpr int SMEM_BYTES = (2 + 2 * KV_STAGES) * TILE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units

enum : unsigned {
  WHERE_ATTN_PRODUCER = 32,
  WHERE_ATTN_MMA = 33,
  WHERE_ATTN_SOFTMAX = 34,
};

struct Params {
  int batch, seq_len;  // seq_len: the common length, or the longest one when cu_seqlens is given
  int q_heads, group;  // group = query heads per key/value head
  int tiles_q, num_items;
  int ld_out;
  const int* cu_seqlens;  // [batch + 1] row offsets in device memory, or NULL (uniform lengths)
  __nv_bfloat16* out;
  float scale_log2;  // softmax scale times log2(e)
  unsigned long long timeout_ns;
  Status* status;
};

struct Item {
  int head, qi, row0, len;  // row0: first row of the sequence; len: its length
};

// Item t -> coordinates. Heaviest first: the query tile index decreases with t.
__device__ __forceinline__ bool item_coords(const Params& p, int t, Item& it) {
  const int per = p.batch * p.q_heads;
  it.qi = p.tiles_q - 1 - t / per;
  const int rest = t % per;
  const int b = rest / p.q_heads;
  it.head = rest - b * p.q_heads;
  if (p.cu_seqlens != nullptr) {
    it.row0 = p.cu_seqlens[b];
    it.len = p.cu_seqlens[b + 1] - it.row0;
  } else {
    it.row0 = b * p.seq_len;
    it.len = p.seq_len;
  }
  return it.qi * BQ < it.len;
}

// Shared-memory descriptor of a B operand stored [k][n] (n contiguous), as TMA wrote it with
// the 128-byte swizzle in boxes of 64 columns: 8 k-rows are 1024 bytes apart (stride byte
// offset), the next 64 columns start `lbo_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= static_cast<uint64_t>(1u) << 46;
  d |= static_cast<uint64_t>(2u) << 61;
  return d;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;
  uint8_t* sP = sV + KV_STAGES * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;
  uint64_t* k_full = bars + 2;
  uint64_t* k_empty = k_full + KV_STAGES;
  uint64_t* v_full = k_empty + KV_STAGES;
  uint64_t* v_empty = v_full + KV_STAGES;
  uint64_t* s_full = v_empty + KV_STAGES;
  uint64_t* s_empty = s_full + 2;
  uint64_t* p_full = s_empty + 2;
  uint64_t* pv_done = p_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    *abort_flag = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = *tmem_slot;
  const Deadline dl{globaltimer_ns() + p.timeout_ns, abort_flag, p.status};

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int it = 0, n = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < p.num_items; t += gridDim.x) {
        Item w;
        if (!item_coords(p, t, w)) continue;
        const int kv_head = w.head / p.group;
        if (!mbar_wait(q_empty, (it & 1) ^ 1u, dl, WHERE_ATTN_PRODUCER, t)) break;
        mbar_expect_tx(q_full, TILE_BYTES);
        tma_load_2d(sQ, &tm_q, q_full, w.head * HD, w.row0 + w.qi * BQ);
        tma_load_2d(sQ + HALF_BYTES, &tm_q, q_full, w.head * HD + 64, w.row0 + w.qi * BQ);
        const int nb = w.qi + 1;
        for (int j = 0; j < nb; ++j, ++n) {
          const int st = n % KV_STAGES;
          const uint32_t ph = (n / KV_STAGES) & 1u;
          const int krow = w.row0 + j * BKV;
          if (!mbar_wait(&k_empty[st], ph ^ 1u, dl, WHERE_ATTN_PRODUCER, t)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&k_full[st], TILE_BYTES);
          tma_load_2d(sK + st * TILE_BYTES, &tm_k, &k_full[st], kv_head * HD, krow);
          tma_load_2d(sK + st * TILE_BYTES + HALF_BYTES, &tm_k, &k_full[st], kv_head * HD + 64, krow);
          if (!mbar_wait(&v_empty[st], ph ^ 1u, dl, WHERE_ATTN_PRODUCER, t)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&v_full[st], TILE_BYTES);
          tma_load_2d(sV + st * TILE_BYTES, &tm_v, &v_full[st], kv_head * HD, krow);
          tma_load_2d(sV + st * TILE_BYTES + HALF_BYTES, &tm_v, &v_full[st], kv_head * HD + 64, krow);
        }
        ++it;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(BQ, BKV);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BQ, HD) | (1u << 16);  // B operand MN-major
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV), p_addr = smem_u32(sP);
      int it = 0, n = 0;
      bool ok = true;
      // S(g) = Q K^T for the CTA's g-th key block
      auto issue_s = [&](int g, int t) -> bool {
        const int st = g % KV_STAGES;
        const uint32_t ph = (g / KV_STAGES) & 1u;
        const int buf = g & 1;
        const uint32_t bph = (g >> 1) & 1u;
        if (!mbar_wait(&k_full[st], ph, dl, WHERE_ATTN_MMA, t)) return false;
        if (!mbar_wait(&s_empty[buf], bph ^ 1u, dl, WHERE_ATTN_MMA, t)) return false;
        tc_fence_after();
        const uint32_t d = tmem_base + static_cast<uint32_t>(buf * BKV);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t da = make_desc_k_sw128(q_addr + (k >> 2) * HALF_BYTES) + 2u * (k & 3);
          const uint64_t db = make_desc_k_sw128(k_addr + st * TILE_BYTES + (k >> 2) * HALF_BYTES) + 2u * (k & 3);
          umma_bf16(d, da, db, idesc_qk, k > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[buf]);
        return true;
      };
      for (int t = blockIdx.x; ok && t < p.num_items; t += gridDim.x) {
        Item w;
        if (!item_coords(p, t, w)) continue;
        const int nb = w.qi + 1;
        if (!mbar_wait(q_full, it & 1, dl, WHERE_ATTN_MMA, t)) break;
        if (!issue_s(n, t)) break;
        for (int j = 0; j < nb; ++j) {
          if (j + 1 < nb) {
            if (!issue_s(n + j + 1, t)) {
              ok = false;
              break;
            }
          } else {
            umma_commit(q_empty);  // the item's last S has been issued: Q may be replaced once it completes
          }
          const int g = n + j;
          const int st = g % KV_STAGES;
          const uint32_t ph = (g / KV_STAGES) & 1u;
          if (!mbar_wait(&v_full[st], ph, dl, WHERE_ATTN_MMA, t) || !mbar_wait(p_full, g & 1, dl, WHERE_ATTN_MMA, t)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k) {
            const uint64_t da = make_desc_k_sw128(p_addr + (k >> 2) * HALF_BYTES) + 2u * (k & 3);
            // 16 keys further = two groups of eight k-rows
            const uint64_t db = make_desc_mn_sw128(v_addr + st * TILE_BYTES + k * 2 * 1024, HALF_BYTES, 1024);
            umma_bf16(tmem_base + O_COL, da, db, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&v_empty[st]);
          umma_commit(pv_done);
        }
        n += nb;
        ++it;
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------- softmax
    const int q4 = warp - 4;  // the tensor-memory lane quarter this warp may access
    const int r = q4 * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    const float sl2 = p.scale_log2;
    uint8_t* p_row = sP + (r >> 3) * 1024 + (r & 7) * 128;
    int n = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < p.num_items; t += gridDim.x) {
      Item w;
      if (!item_coords(p, t, w)) continue;
      const int nb = w.qi + 1;
      float m_ref = -INFINITY, l = 0.0f;
      for (int j = 0; j < nb; ++j) {
        const int g = n + j;
        const int buf = g & 1;
        ok = mbar_wait(&s_full[buf], (g >> 1) & 1u, dl, WHERE_ATTN_SOFTMAX, t);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t s[4][32];
        const uint32_t t_s = tmem_base + static_cast<uint32_t>(buf * BKV) + lane_base;
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_s + c * 32, s[c]);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&s_empty[buf]);
        if (j == w.qi) {
          // diagonal block: key c of the block is visible to query r of the tile iff c <= r
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (c * 32 + i > r) s[c][i] = 0xff800000u;  // -inf
            }
          }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(s[c][i]));
        }
        bool rescale = false;
        float alpha = 1.0f;
        if (j == 0) {
          m_ref = mx;
        } else {
          const float m_new = fmaxf(m_ref, mx);
          const bool need = (m_new - m_ref) * sl2 > RESCALE_THRESHOLD;
          if (__any_sync(0xffffffffu, need)) {
            rescale = true;
            alpha = ex2((m_ref - m_new) * sl2);
            m_ref = m_new;
            l *= alpha;
          }
        }
        // P's shared memory and the O accumulator are free once the previous P V has completed
        if (g > 0) {
          ok = mbar_wait(pv_done, (g - 1) & 1u, dl, WHERE_ATTN_SOFTMAX, t);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        if (rescale) {
          tc_fence_after();
          const uint32_t t_o = tmem_base + O_COL + lane_base;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(t_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(t_o + c * 32, o);
          }
          tmem_st_wait();
        }
        const float m_sl2 = m_ref * sl2;
        float sum = 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float e[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              e[i] = ex2(fmaf(__uint_as_float(s[c][v * 8 + i]), sl2, -m_sl2));
              sum += e[i];
            }
            const int ch = c * 4 + v;  // 16-byte chunk of the row: keys [8 ch, 8 ch + 8)
            uint8_t* dst = p_row + (ch >> 3) * HALF_BYTES + (((ch & 7) ^ (r & 7)) << 4);
            *reinterpret_cast<uint4*>(dst) =
                make_uint4(pack2(e[0], e[1]), pack2(e[2], e[3]), pack2(e[4], e[5]), pack2(e[6], e[7]));
          }
        }
        l += sum;
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(p_full);
      }
      if (!ok) break;
      // ---- the item's output rows: O / l
      const int g_last = n + nb - 1;
      ok = mbar_wait(pv_done, g_last & 1u, dl, WHERE_ATTN_SOFTMAX, t);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float inv_l = 1.0f / l;
      const int q_in_seq = w.qi * BQ + r;
      const bool row_ok = q_in_seq < w.len;
      __nv_bfloat16* orow = p.out + static_cast<size_t>(w.row0 + q_in_seq) * p.ld_out + w.head * HD;
      const uint32_t t_o = tmem_base + O_COL + lane_base;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(t_o + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              w4[i] = pack2(__uint_as_float(o[v * 8 + 2 * i]) * inv_l, __uint_as_float(o[v * 8 + 2 * i + 1]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
          }
        }
      }
      tc_fence_before();
      n += nb;
    }
  }

  // ------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    if (*abort_flag) {
      const uint64_t t_stop = globaltimer_ns() + 2000000ull;
      while (globaltimer_ns() < t_stop) __nanosleep(1000);
    }
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

static bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld) {
  PFN_encodeTiled fn = get_encode_tiled();
  if (fn == nullptr) return false;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {64, 128};
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

}  // namespace attn
}  // namespace df

extern "C" int df_attention_prefill_bf16(const void* q, const void* k, const void* v, void* out, int total_rows, int batch,
                                         int seq_len, const int* cu_seqlens_dev, int q_heads, int kv_heads, int head_dim,
                                         int ld_q, int ld_k, int ld_v, int ld_out, float scale, int max_ctas,
                                         df_status_t* dev_status, void* stream) {
  using namespace df;
  using namespace df::attn;
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr || dev_status == nullptr)
    return fail(DF_EINVAL, "NULL pointer argument");
  if (head_dim != HD) return fail(DF_EUNSUPPORTED, "head_dim must be %d (got %d)", HD, head_dim);
  if (batch <= 0 || seq_len <= 0 || total_rows <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0)
    return fail(DF_EINVAL, "batch, seq_len, total_rows and the head counts must be positive, q_heads a multiple of kv_heads");
  if (cu_seqlens_dev == nullptr && static_cast<long long>(batch) * seq_len != total_rows)
    return fail(DF_EINVAL, "uniform lengths: total_rows (%d) must equal batch * seq_len (%d x %d)", total_rows, batch, seq_len);
  if (ld_q < q_heads * HD || ld_k < kv_heads * HD || ld_v < kv_heads * HD || ld_out < q_heads * HD || (ld_q % 8) != 0 ||
      (ld_k % 8) != 0 || (ld_v % 8) != 0 || (ld_out % 8) != 0)
    return fail(DF_EINVAL, "row strides must cover the heads and be multiples of 8 elements");
  if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
        reinterpret_cast<uintptr_t>(out)) & 15u) != 0)
    return fail(DF_EINVAL, "q, k, v and out must be 16-byte aligned");
  if (!(scale > 0.0f)) return fail(DF_EINVAL, "scale must be positive");
  const int sms = df_sm_count();
  if (sms <= 0) return fail(DF_ECUDA, "no CUDA device");

  CUtensorMap tm_q, tm_k, tm_v;
  if (!make_map(&tm_q, q, total_rows, static_cast<uint64_t>(q_heads) * HD, ld_q)) return DF_ECUDA;
  if (!make_map(&tm_k, k, total_rows, static_cast<uint64_t>(kv_heads) * HD, ld_k)) return DF_ECUDA;
  if (!make_map(&tm_v, v, total_rows, static_cast<uint64_t>(kv_heads) * HD, ld_v)) return DF_ECUDA;

  Params p;
  std::memset(&p, 0, sizeof(p));
  p.batch = batch;
  p.seq_len = seq_len;
  p.q_heads = q_heads;
  p.group = q_heads / kv_heads;
  p.tiles_q = (seq_len + BQ - 1) / BQ;
  p.num_items = p.tiles_q * batch * q_heads;
  p.ld_out = ld_out;
  p.cu_seqlens = cu_seqlens_dev;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.timeout_ns = timeout_ns();
  p.status = reinterpret_cast<Status*>(dev_status);

  static bool attr_set[64] = {false};
  int dev = 0;
  (void)cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    const cudaError_t ae = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (ae != cudaSuccess) return fail(DF_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(ae));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  int grid = sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (p.num_items < grid) grid = p.num_items;
  attention_prefill_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(tm_q, tm_k, tm_v, p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DF_ECUDA, "attention launch: %s", cudaGetErrorString(e));
  return DF_OK;
}
