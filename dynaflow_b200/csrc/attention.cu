// Attention for sm_100a: causal self-attention of a prefill nano-batch and, from the same kernel
// template, split-KV attention of a decode step. Both contractions (S = Q K^T and O = P V) run on
// tcgen05 with the accumulators in tensor memory, operands staged by plain per-CTA TMA loads,
// online softmax in the epilogue warps, P handed to the second product THROUGH tensor memory.
//
// Prefill. A work item is a PAIR of consecutive 128-row query tiles of one head of one sequence;
// its keys are visited in blocks of 128, and every key and value tile is loaded once for both
// query tiles. Items are ordered by decreasing number of key blocks and dealt round-robin to a
// persistent grid of at most `max_ctas` CTAs, so the launch can leave SMs to the reduction kernel
// of the other micro-batch.
//
// 384 threads per CTA:
//   warp 0      TMA producer: the item's Q tiles, then K_0 V_0 K_1 V_1 ... through a ring of five
//               32 KB tiles
//   warp 1      MMA issuer (one lane). Per key block and query tile: O_t += P_t V_j (A operand P_t
//               read from tensor memory, B operand V_j in its memory layout [key][dim], i.e.
//               MN-major: the instruction descriptor's B-major bit and a shared-memory descriptor
//               with the 64-wide column halves 16 KB apart), then S_t = Q_t K_{j+1}^T over the
//               columns P_t has just been read from. The two query tiles alternate, so one
//               tile's products run while the other tile's softmax computes.
//   warp 2      allocates / frees tensor memory: S of tile 0, S of tile 1, O of tile 0, O of tile 1
//   warps 4..7 / 8..11  softmax of tile 0 / tile 1, one thread per query row: two passes over
//               the row of S with tcgen05.ld (maximum; then exp2 relative to the running maximum),
//               the causal mask on the tile's diagonal block only, the bf16 row of P written back
//               with tcgen05.st over the first 64 columns of S, O rescaled in tensor memory only
//               when the maximum grew by more than 2^8 (the exponent otherwise simply stays
//               relative to the older maximum), final 1/l scaling and the stores of the output rows.
//
// Decode (DECODE = true): one new token per sequence against a key/value cache. A work item is
// (sequence, key/value head, chunk of the cached keys); the query "tile" holds the few query
// heads that share the key/value head in its first rows (the other rows of the 128-row MMA are
// never read back), one softmax warp owns them, S / P alternate between the two accumulators so
// that S of block j + 1 runs under the softmax of block j, and instead of normalised rows an item
// leaves (maximum, sum, unnormalised O) per head, which a small second kernel merges over the
// chunks. That launch is bound by streaming the cache from HBM.
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

constexpr int BQ = 128;   // query rows per tile; a prefill work item is a pair of consecutive tiles
constexpr int BKV = 128;  // keys per block
constexpr int HD = 128;   // head dimension (the only one built)
constexpr int TILE_BYTES = 128 * 128 * 2;
constexpr int HALF_BYTES = TILE_BYTES / 2;  // one TMA box: 128 rows x 64 columns
// Ring of key and value tiles, K_0 V_0 K_1 V_1 ... in this order. Prefill: two 32 KB query tiles and five
// slots. Decode: the few query-head rows take 1 KB per 64-column half (the MMA still addresses 128 rows per
// half; the rows beyond the heads alias the ring and are never read back), which leaves room for seven slots:
// the launch is bound by the bytes in flight from HBM.
constexpr int KV_SLOTS_PREFILL = 5;
constexpr int KV_SLOTS_DECODE = 7;
constexpr int KV_SLOTS_MAX = 7;
constexpr int DECODE_Q_BYTES = 2048;      // two halves of 8 rows x 128 B
constexpr int DECODE_MAX_GROUP = 8;       // query heads per key/value head that fit those rows
constexpr int THREADS = 384;  // warps 0..2 producer / MMA / tensor-memory owner, 3 idle, 4..11 softmax
constexpr int TMEM_COLS = 512;  // S (and P) of tile 0, of tile 1, O of tile 0, O of tile 1: 4 x 128 columns
constexpr int O_COL = 256;
constexpr int kBarrierBytes = 256;
// two Q tiles, the ring, barriers; what is left of the 227 KB is the room the 1024-byte alignment
// of the tiles may cost (checked in the kernel)
constexpr int kSmemUsedPrefill = (2 + KV_SLOTS_PREFILL) * TILE_BYTES + kBarrierBytes;
constexpr int kSmemUsedDecode = DECODE_Q_BYTES + KV_SLOTS_DECODE * TILE_BYTES + kBarrierBytes;
constexpr int SMEM_BYTES = 227 * 1024;
static_assert(kSmemUsedPrefill <= SMEM_BYTES && kSmemUsedDecode <= SMEM_BYTES, "shared-memory budget");
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units

enum : unsigned {
  WHERE_ATTN_PRODUCER = 32,
  WHERE_ATTN_MMA = 33,
  WHERE_ATTN_SOFTMAX = 34,
};

#ifdef DF_ATTN_TIMING
__device__ unsigned long long g_attn_timing[32];
#define TSTART() long long t_mark = clock64()
#define TADD(i) do { long long t_now = clock64(); atomicAdd(&g_attn_timing[i], (unsigned long long)(t_now - t_mark)); t_mark = t_now; } while (0)
#else
#define TSTART() do { } while (0)
#define TADD(i) do { } while (0)
#endif

struct Params {
  int batch, seq_len;  // prefill: seq_len = the common length, or the longest one when cu_seqlens is given
  int q_heads, group;  // group = query heads per key/value head
  int pairs_q, num_items;  // prefill: pairs of query tiles per sequence
  int ld_out;
  const int* cu_seqlens;  // prefill: [batch + 1] row offsets in device memory, or NULL (uniform lengths)
  __nv_bfloat16* out;
  float scale_log2;  // softmax scale times log2(e)
  // decode: the cache of sequence b occupies rows [b * max_len, (b + 1) * max_len) of the K / V matrices,
  // seq_lens[b] of them valid; an item covers chunk_blocks key blocks; partial results per (b, head, split)
  int kv_heads, max_len, chunk_blocks, splits;
  const int* seq_lens;
  float* partial_o;   // [batch, q_heads, splits, 128]
  float* partial_ml;  // [batch, q_heads, splits, 2]: running maximum (log2 units), sum
  unsigned long long timeout_ns;
  Status* status;
};

struct Item {
  int head;       // prefill: the query head; decode: the first query head of the group
  int kv_head;
  int q_row;      // prefill: first row of query tile 0 in the q matrix; decode: the sequence (row of q)
  int q_in_seq;   // prefill: position of tile 0's first query in its sequence
  int len;        // prefill: length of the sequence; decode: valid keys counted from the item's first key
  int kv_row;     // row of the item's first key in the K / V matrices
  int nb[2];      // key blocks tile 0 / tile 1 go through (0: the tile does not exist); nb[1] is nb[0] + 1 or 0
  int seq, split; // decode
};

// Item t -> coordinates; false if there is nothing to do. Prefill: heaviest first (the tile-pair
// index decreases with t); tile 0 of pair i is query tile 2i (key blocks 0..2i, the last one
// diagonal), tile 1 is query tile 2i + 1 (key blocks 0..2i + 1) if the sequence reaches it.
// Decode: t = (sequence * kv_heads + kv_head) * splits + split, one tile.
template <bool DECODE>
__device__ __forceinline__ bool item_coords(const Params& p, int t, Item& it) {
  if (DECODE) {
    it.split = t % p.splits;
    const int rest = t / p.splits;
    it.kv_head = rest % p.kv_heads;
    it.seq = rest / p.kv_heads;
    it.head = it.kv_head * p.group;
    it.q_row = it.seq;
    it.q_in_seq = 0;
    const int len = min(p.seq_lens[it.seq], p.max_len);
    const int first_key = it.split * p.chunk_blocks * BKV;
    if (first_key >= len) return false;
    it.len = len - first_key;
    it.kv_row = it.seq * p.max_len + first_key;
    it.nb[0] = min(p.chunk_blocks, (it.len + BKV - 1) / BKV);
    it.nb[1] = 0;
    return true;
  }
  const int per = p.batch * p.q_heads;
  const int pi = p.pairs_q - 1 - t / per;
  const int rest = t % per;
  const int b = rest / p.q_heads;
  it.head = rest - b * p.q_heads;
  it.kv_head = it.head / p.group;
  int row0;
  if (p.cu_seqlens != nullptr) {
    row0 = p.cu_seqlens[b];
    it.len = p.cu_seqlens[b + 1] - row0;
  } else {
    row0 = b * p.seq_len;
    it.len = p.seq_len;
  }
  it.q_in_seq = 2 * pi * BQ;
  it.q_row = row0 + it.q_in_seq;
  it.kv_row = row0;
  it.nb[0] = 2 * pi + 1;
  it.nb[1] = (it.q_in_seq + BQ < it.len) ? 2 * pi + 2 : 0;
  it.seq = b;
  it.split = 0;
  return it.q_in_seq < it.len;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
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

template <bool DECODE>
__global__ void __launch_bounds__(THREADS, 1)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  constexpr int KV_SLOTS = DECODE ? KV_SLOTS_DECODE : KV_SLOTS_PREFILL;
  constexpr int Q_HALF_STRIDE = DECODE ? DECODE_Q_BYTES / 2 : HALF_BYTES;  // distance of the two 64-column halves of Q
  constexpr int kSmemUsed = DECODE ? kSmemUsedDecode : kSmemUsedPrefill;
  uint8_t* sQ = smem;                                                   // prefill: two tiles; decode: the head rows
  uint8_t* sKV = sQ + (DECODE ? DECODE_Q_BYTES : 2 * TILE_BYTES);       // KV_SLOTS tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + KV_SLOTS * TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;
  uint64_t* kv_full = bars + 2;
  uint64_t* kv_empty = kv_full + KV_SLOTS_MAX;
  uint64_t* s_full = kv_empty + KV_SLOTS_MAX;
  uint64_t* p_full = s_full + 2;
  uint64_t* pv_done = p_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // decode: the group's query heads are rows 0.. of tile 0, owned by the first softmax warp
  constexpr uint32_t kGroupThreads = DECODE ? 32 : 128;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < KV_SLOTS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], kGroupThreads);
      mbar_init(&pv_done[s], 1);
    }
    *abort_flag = 0u;
    if (pad + kSmemUsed > static_cast<uint32_t>(SMEM_BYTES)) {
      // the dynamic shared memory started further from a 1024-byte boundary than the launch budgeted for
      *abort_flag = 1u;
      report(p.status, 1u, WHERE_ATTN_PRODUCER, pad);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  __syncthreads();
  if (*abort_flag) return;  // uniform: nothing has been allocated or issued yet
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
      int it = 0;
      uint32_t u = 0;  // tiles put into the ring so far
      bool ok = true;
      TSTART();
      for (int t = blockIdx.x; ok && t < p.num_items; t += gridDim.x) {
        Item w;
        if (!item_coords<DECODE>(p, t, w)) continue;
        TADD(0);
        if (!mbar_wait(q_empty, (it & 1) ^ 1u, dl, WHERE_ATTN_PRODUCER, t)) break;
        TADD(1);
        if (DECODE) {
          // the group's query heads of this sequence: rows 0..group-1 of tile 0
          mbar_expect_tx(q_full, 2 * p.group * 128);
          tma_load_3d(sQ, &tm_q, q_full, 0, w.head, w.q_row);
          tma_load_3d(sQ + Q_HALF_STRIDE, &tm_q, q_full, 64, w.head, w.q_row);
        } else {
          const int tiles = w.nb[1] > 0 ? 2 : 1;
          mbar_expect_tx(q_full, tiles * TILE_BYTES);
          for (int q = 0; q < tiles; ++q) {
            tma_load_2d(sQ + q * TILE_BYTES, &tm_q, q_full, w.head * HD, w.q_row + q * BQ);
            tma_load_2d(sQ + q * TILE_BYTES + HALF_BYTES, &tm_q, q_full, w.head * HD + 64, w.q_row + q * BQ);
          }
        }
        const int nb = max(w.nb[0], w.nb[1]);
        for (int j = 0; j < nb && ok; ++j) {
          const int krow = w.kv_row + j * BKV;
          for (int kv = 0; kv < 2; ++kv, ++u) {
            const uint32_t slot = u % KV_SLOTS;
            const uint32_t ph = (u / KV_SLOTS) & 1u;
            TADD(0);
            if (!mbar_wait(&kv_empty[slot], ph ^ 1u, dl, WHERE_ATTN_PRODUCER, t)) {
              ok = false;
              break;
            }
            TADD(2 + kv);
            uint8_t* dst = sKV + slot * TILE_BYTES;
            const CUtensorMap* map = kv == 0 ? &tm_k : &tm_v;
            mbar_expect_tx(&kv_full[slot], TILE_BYTES);
            tma_load_2d(dst, map, &kv_full[slot], w.kv_head * HD, krow);
            tma_load_2d(dst + HALF_BYTES, map, &kv_full[slot], w.kv_head * HD + 64, krow);
          }
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
      const uint32_t q_addr = smem_u32(sQ), kv_addr = smem_u32(sKV);
      int it = 0;
      uint32_t u0 = 0;          // ring index of the item's K_0
      uint32_t cnt[2] = {0, 0}; // blocks either tile has gone through so far (phases of its barriers)
      uint32_t cnt_s = 0;       // decode: S products issued so far
      bool ok = true;
      TSTART();
      // S of tile G for the item's key block j
      auto issue_s = [&](int G, int j, const Item& w, int t) -> bool {
        const uint32_t u = u0 + 2u * j;
        const uint32_t slot = u % KV_SLOTS;
        TADD(8);
        if (!mbar_wait(&kv_full[slot], (u / KV_SLOTS) & 1u, dl, WHERE_ATTN_MMA, t)) return false;
        TADD(9);
        // The accumulator of tile G also holds the tile's P: it is free once the P V of the tile's
        // previous block has read it, and that product was issued before this one (the tensor pipe
        // executes one thread's products in order).
        tc_fence_after();
        // decode has one tile: its S / P alternates between the two accumulators, so that S of the
        // next block can run under the softmax of this one
        const uint32_t sb = DECODE ? (cnt_s & 1u) : static_cast<uint32_t>(G);
        const uint32_t d = tmem_base + sb * BKV;
        const uint32_t k_addr = kv_addr + slot * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t da = make_desc_k_sw128(q_addr + G * TILE_BYTES + (k >> 2) * Q_HALF_STRIDE) + 2u * (k & 3);
          const uint64_t db = make_desc_k_sw128(k_addr + (k >> 2) * HALF_BYTES) + 2u * (k & 3);
          umma_bf16(d, da, db, idesc_qk, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[sb]);
        ++cnt_s;
        if (G == 1 || j >= w.nb[1]) umma_commit(&kv_empty[slot]);       // the last tile that reads K_j
        if (j == w.nb[G] - 1 && (G == 1 || w.nb[1] == 0)) umma_commit(q_empty);  // the item's last S
        return true;
      };
      for (int t = blockIdx.x; ok && t < p.num_items; t += gridDim.x) {
        Item w;
        if (!item_coords<DECODE>(p, t, w)) continue;
        const int nb = max(w.nb[0], w.nb[1]);
        TADD(8);
        if (!mbar_wait(q_full, it & 1, dl, WHERE_ATTN_MMA, t)) break;
        TADD(11);
        if (!issue_s(0, 0, w, t)) break;
        if (DECODE) {
          if (w.nb[0] > 1 && !issue_s(0, 1, w, t)) break;
        } else if (w.nb[1] > 0 && !issue_s(1, 0, w, t)) {
          break;
        }
        for (int j = 0; j < nb && ok; ++j) {
          const uint32_t uv = u0 + 2u * j + 1u;
          const uint32_t vslot = uv % KV_SLOTS;
          TADD(8);
          if (!mbar_wait(&kv_full[vslot], (uv / KV_SLOTS) & 1u, dl, WHERE_ATTN_MMA, t)) {
            ok = false;
            break;
          }
          TADD(12);
          for (int G = 0; G < 2; ++G) {
            if (j >= w.nb[G]) continue;
            const uint32_t pb = DECODE ? (cnt[0] & 1u) : static_cast<uint32_t>(G);
            const uint32_t pph = DECODE ? ((cnt[0] >> 1) & 1u) : (cnt[G] & 1u);
            if (!mbar_wait(&p_full[pb], pph, dl, WHERE_ATTN_MMA, t)) {
              ok = false;
              break;
            }
            TADD(13);
            tc_fence_after();
            const uint32_t d_o = tmem_base + O_COL + static_cast<uint32_t>(G * HD);
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k) {
              // P of the tile: bf16 pairs in the first 64 columns of its S accumulator, 16 keys = 8 columns
              const uint32_t a_p = tmem_base + pb * BKV + static_cast<uint32_t>(8 * k);
              // 16 keys further = two groups of eight k-rows
              const uint64_t db = make_desc_mn_sw128(kv_addr + vslot * TILE_BYTES + k * 2 * 1024, HALF_BYTES, 1024);
              umma_bf16_a_tmem(d_o, a_p, db, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(&pv_done[G]);
            ++cnt[G];
            if (G == 1 || j >= w.nb[1]) umma_commit(&kv_empty[vslot]);  // the last tile that reads V_j
            // prefill: S of the tile's next block goes over the P that this product has just read;
            // decode: S of block j + 2 (block j + 1 was issued before this product, into the other accumulator)
            const int next = DECODE ? j + 2 : j + 1;
            if (next < w.nb[G] && !issue_s(G, next, w, t)) {
              ok = false;
              break;
            }
          }
        }
        u0 += 2u * nb;
        ++it;
      }
    }
    __syncwarp();
  } else if (warp >= 4 && (!DECODE || warp == 4)) {
    // ------------------------------------------------------------- softmax
    // Two groups of four warps, one thread per query row; group G owns query tile G of the item:
    // its S accumulator (whose first 64 columns then take the bf16 P), its running maximum and
    // sum, its O accumulator. The two tiles go through the same key and value tiles half a block
    // apart in time: while one group computes its exponentials the tensor pipe works on the other
    // tile. Decode: one tile, and only the first warp takes part (rows 0..group-1 are the heads).
    const int q4 = warp & 3;           // the tensor-memory lane quarter this warp may touch
    const int G = (warp - 4) >> 2;
    const int r = q4 * 32 + lane;
    const bool active = !DECODE || r < p.group;
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    const float sl2 = p.scale_log2;
    const uint32_t t_o = tmem_base + O_COL + static_cast<uint32_t>(G * HD) + lane_base;
    uint32_t cnt = 0;  // blocks this group has gone through (phase of its barriers)
    bool ok = true;
#ifdef DF_ATTN_TIMING
    const bool timed = (threadIdx.x == 128);
    long long t_mark = clock64();
#undef TADD
#define TADD(i) do { long long t_now = clock64(); if (timed) atomicAdd(&g_attn_timing[i], (unsigned long long)(t_now - t_mark)); t_mark = t_now; } while (0)
#endif
    for (int t = blockIdx.x; ok && t < p.num_items; t += gridDim.x) {
      Item w;
      if (!item_coords<DECODE>(p, t, w)) continue;
      const int nb = w.nb[G];
      if (nb == 0) continue;  // the sequence ends before this tile
      float m_ref = -INFINITY, l = 0.0f;
      for (int j = 0; j < nb; ++j, ++cnt) {
        TADD(16);
        const uint32_t sb = DECODE ? (cnt & 1u) : static_cast<uint32_t>(G);   // which S / P accumulator
        const uint32_t sph = DECODE ? ((cnt >> 1) & 1u) : (cnt & 1u);
        const uint32_t t_s = tmem_base + sb * BKV + lane_base;
        ok = mbar_wait(&s_full[sb], sph, dl, WHERE_ATTN_SOFTMAX, t);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        TADD(17);
        tc_fence_after();
        // visible keys of this block: prefill, the tile's diagonal block: key c iff c <= r; decode,
        // the last block of the sequence: key c iff it lies before the end of the cache
        const int limit = DECODE ? (w.len - j * BKV - 1) : (j == nb - 1 ? r : BKV);
        const bool masked = limit < BKV - 1;
        // pass 1: the row's maximum
        float mx = -INFINITY;
#pragma unroll 1
        for (int hcol = 0; hcol < 2; ++hcol) {
          uint32_t s[2][32];
          tmem_ld_32x32(t_s + hcol * 64, s[0]);
          tmem_ld_32x32(t_s + hcol * 64 + 32, s[1]);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            if (masked) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (hcol * 64 + c * 32 + i > limit) s[c][i] = 0xff800000u;  // -inf
              }
            }
            float part[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 32; ++i) part[i & 3] = fmaxf(part[i & 3], __uint_as_float(s[c][i]));
            mx = fmaxf(mx, fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])));
          }
        }
        if (!active) mx = 0.0f;  // rows that are never read back: keep their arithmetic finite
        TADD(18);
        if (j == 0) {
          m_ref = mx;
        } else {
          const float m_new = fmaxf(m_ref, mx);
          const bool need = active && (m_new - m_ref) * sl2 > RESCALE_THRESHOLD;
          if (__any_sync(0xffffffffu, need)) {
            // O still grows by the previous block's P V until that product has completed
            ok = mbar_wait(&pv_done[G], (cnt - 1u) & 1u, dl, WHERE_ATTN_SOFTMAX, t);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const float alpha = ex2((m_ref - m_new) * sl2);
            m_ref = m_new;
            l *= alpha;
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
        }
        TADD(20);
        // pass 2: exponentials; the bf16 row of P goes over the first 64 columns of S, 64 keys at a time
        const float m_sl2 = m_ref * sl2;
        float sum = 0.0f;
#pragma unroll 1
        for (int hcol = 0; hcol < 2; ++hcol) {
          uint32_t s[2][32];
          tmem_ld_32x32(t_s + hcol * 64, s[0]);
          tmem_ld_32x32(t_s + hcol * 64 + 32, s[1]);
          tmem_ld_wait();
          if (masked) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (hcol * 64 + c * 32 + i > limit) s[c][i] = 0xff800000u;  // -inf
              }
            }
          }
          uint32_t pk[32];
          float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
          for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float e0 = ex2(fmaf(__uint_as_float(s[c][2 * i]), sl2, -m_sl2));
              float e1 = ex2(fmaf(__uint_as_float(s[c][2 * i + 1]), sl2, -m_sl2));
              if (DECODE && !active) e0 = e1 = 0.0f;
              part[i & 3] += e0 + e1;
              pk[c * 16 + i] = pack2(e0, e1);
            }
          }
          sum += (part[0] + part[1]) + (part[2] + part[3]);
          // keys [64 hcol, 64 hcol + 64) of this row of P: 32 columns of bf16 pairs, over columns of
          // S that this thread has already read
          tmem_st_32x32(t_s + hcol * 32, pk);
        }
        tmem_st_wait();
        l += sum;
        TADD(21);
        tc_fence_before();
        mbar_arrive(&p_full[sb]);
        TADD(22);
      }
      if (!ok) break;
      // ---- the tile's output rows: O / l (decode: maximum, sum and unnormalised O of this chunk)
      ok = mbar_wait(&pv_done[G], (cnt - 1u) & 1u, dl, WHERE_ATTN_SOFTMAX, t);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float inv_l = DECODE ? 1.0f : 1.0f / l;
      const size_t slot_idx = DECODE ? (static_cast<size_t>(w.seq) * p.q_heads + w.head + (active ? r : 0)) * p.splits + w.split : 0;
      const bool row_ok = DECODE ? active : (w.q_in_seq + G * BQ + r < w.len);
      if (DECODE && active) {
        p.partial_ml[2 * slot_idx] = m_ref * sl2;
        p.partial_ml[2 * slot_idx + 1] = l;
      }
      float* po = DECODE ? p.partial_o + slot_idx * HD : nullptr;
      __nv_bfloat16* orow = DECODE ? nullptr : p.out + static_cast<size_t>(w.q_row + G * BQ + r) * p.ld_out + w.head * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(t_o + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
          if (DECODE) {
#pragma unroll
            for (int v = 0; v < 8; ++v)
              *reinterpret_cast<uint4*>(po + c * 32 + v * 4) = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
          } else {
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
      }
      tc_fence_before();
      TADD(23);
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

// q viewed as [sequence][head][128] with the row stride of the fused activation: a box is the
// `group` heads that share one key/value head, 64 columns wide.
static bool make_map_q_decode(CUtensorMap* map, const void* base, uint64_t batch, uint64_t heads, uint64_t ld,
                              uint32_t group) {
  PFN_encodeTiled fn = get_encode_tiled();
  if (fn == nullptr) return false;
  cuuint64_t gdim[3] = {static_cast<cuuint64_t>(HD), heads, batch};
  cuuint64_t gstride[2] = {static_cast<cuuint64_t>(HD) * 2, ld * 2};
  cuuint32_t box[3] = {64, group, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (decode queries) failed with CUresult %d", static_cast<int>(r));
    return false;
  }
  return true;
}

// Key blocks per work item of the decode launch: enough items to keep `ctas` CTAs evenly busy
// (about six each) without cutting the cache finer than needed.
static int decode_chunk_blocks(int batch, int kv_heads, int max_len, int ctas, bool whole_sequences_allowed) {
  const long long nblk = (max_len + BKV - 1) / BKV;
  // About one (sequence, key/value head) per CTA: no cut at all. Every CTA streams one cache, the result rows
  // leave the attention launch normalised, and the merge launch and the partial results disappear.
  // (Measured, 128 sequences of 4096 keys on 140 CTAs: 45 us against 51 us for 1024 chunks plus the merge.)
  const long long pairs = static_cast<long long>(batch) * kv_heads;
  const long long waves = (pairs + ctas - 1) / (ctas > 0 ? ctas : 1);
  const long long need_pct = waves == 1 ? 85 : 95;  // how full the last wave has to be for whole sequences to win
  if (whole_sequences_allowed && pairs * 100 >= waves * ctas * need_pct) return static_cast<int>(nblk);
  long long chunk = static_cast<long long>(batch) * kv_heads * nblk / (6LL * (ctas > 0 ? ctas : 1));
  if (chunk < 1) chunk = 1;
  if (chunk > nblk) chunk = nblk;
  return static_cast<int>(chunk);
}

// Merges the per-chunk results of the decode launch: out[b, head, :] = sum_s 2^(m_s - M) O_s /
// sum_s 2^(m_s - M) l_s over the chunks that hold keys of sequence b. One warp per (b, head); the
// chunks' maxima and sums are fetched by one lane each and the partial rows eight chunks at a time,
// so that a warp waits for two or three L2 round trips, not for two per chunk.
__global__ void attention_decode_merge_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                              const int* __restrict__ seq_lens, int batch, int q_heads, int splits,
                                              int chunk_keys, int max_len, __nv_bfloat16* __restrict__ out, int ld_out) {
  grid_dependency_wait();
  grid_launch_dependents();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= batch * q_heads) return;
  const int b = warp / q_heads, h = warp - b * q_heads;
  const int len = min(seq_lens[b], max_len);
  int used = (len + chunk_keys - 1) / chunk_keys;
  if (used > splits) used = splits;
  const size_t base = static_cast<size_t>(warp) * splits;
  // pass 1: the largest reference maximum
  float big = -INFINITY;
  for (int s0 = 0; s0 < used; s0 += 32) {
    const float m = s0 + lane < used ? partial_ml[2 * (base + s0 + lane)] : -INFINITY;
    big = fmaxf(big, m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, o));
  // pass 2: weights and weighted rows, eight chunks in flight
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, denom = 0.f;
  for (int s0 = 0; s0 < used; s0 += 32) {
    float wgt_l = 0.f, l_l = 0.f;  // this lane's chunk of the batch of 32
    if (s0 + lane < used) {
      const float2 ml = *reinterpret_cast<const float2*>(partial_ml + 2 * (base + s0 + lane));
      wgt_l = ex2(ml.x - big);
      l_l = ml.y;
    }
    const int n = min(32, used - s0);
    for (int c0 = 0; c0 < n; c0 += 8) {
      float4 o[8];
#pragma unroll
      for (int c = 0; c < 8; ++c)
        o[c] = c0 + c < n ? *reinterpret_cast<const float4*>(partial_o + (base + s0 + c0 + c) * HD + lane * 4)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        // chunks in index order: the same sum whatever the batch size
        const float wgt = __shfl_sync(0xffffffffu, wgt_l, (c0 + c) & 31);
        const float l = __shfl_sync(0xffffffffu, l_l, (c0 + c) & 31);
        if (c0 + c < n) {
          denom += wgt * l;
          acc[0] += wgt * o[c].x;
          acc[1] += wgt * o[c].y;
          acc[2] += wgt * o[c].z;
          acc[3] += wgt * o[c].w;
        }
      }
    }
  }
  const float inv = used > 0 ? 1.0f / denom : 0.0f;
  uint2 packed = make_uint2(pack2(acc[0] * inv, acc[1] * inv), pack2(acc[2] * inv, acc[3] * inv));
  *reinterpret_cast<uint2*>(out + static_cast<size_t>(b) * ld_out + h * HD + lane * 4) = packed;
}

// cache[b, seq_lens[b] - 1, :] = new[b, :] for K and V: the new token's keys and values take the
// last valid position of their sequence. One warp per (sequence, 16-byte vector group).
__global__ void kv_cache_append_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                       int ld_new, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                       int ld_cache, const int* __restrict__ seq_lens, int batch, int max_len, int cols) {
  const int vecs = cols >> 3;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < batch * vecs; i += gridDim.x * blockDim.x) {
    const int b = i / vecs, v = i - b * vecs;
    const int pos = seq_lens[b] - 1;
    if (pos < 0 || pos >= max_len) continue;
    const size_t row = static_cast<size_t>(b) * max_len + pos;
    reinterpret_cast<uint4*>(k_cache + row * ld_cache)[v] = reinterpret_cast<const uint4*>(k_new + static_cast<size_t>(b) * ld_new)[v];
    reinterpret_cast<uint4*>(v_cache + row * ld_cache)[v] = reinterpret_cast<const uint4*>(v_new + static_cast<size_t>(b) * ld_new)[v];
  }
}

// Rotary embedding of the new token's query and key heads at position seq_lens[b] - 1, in place in the
// fused qkv row [q heads | k heads | v heads], and the rotated keys and the values into the last
// valid position of the caches. One thread per (sequence, head, 8 dims of the first half) for the
// rotation, one per (sequence, 16-byte vector) for the values.
__global__ void rope_append_kernel(__nv_bfloat16* __restrict__ qkv, int row_stride, const int* __restrict__ seq_lens, int batch,
                                   int q_heads, int kv_heads, float theta, __nv_bfloat16* __restrict__ k_cache,
                                   __nv_bfloat16* __restrict__ v_cache, int ld_cache, int max_len) {
  grid_dependency_wait();
  grid_launch_dependents();
  constexpr int half = HD / 2, groups = half / 8;
  const int rot_heads = q_heads + kv_heads;
  const int v_vecs = kv_heads * HD / 8;
  const int per_seq = rot_heads * groups + v_vecs;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < batch * per_seq; i += gridDim.x * blockDim.x) {
    const int b = i / per_seq, r = i - b * per_seq;
    const int pos = seq_lens[b] - 1;
    const bool cached = pos >= 0 && pos < max_len;
    const size_t cache_row = (static_cast<size_t>(b) * max_len + (cached ? pos : 0)) * ld_cache;
    __nv_bfloat16* row = qkv + static_cast<size_t>(b) * row_stride;
    if (r >= rot_heads * groups) {
      const int v = r - rot_heads * groups;
      if (cached) reinterpret_cast<uint4*>(v_cache + cache_row)[v] = reinterpret_cast<const uint4*>(row + rot_heads * HD)[v];
      continue;
    }
    const int head = r / groups, gidx = r - head * groups;
    __nv_bfloat16* base = row + head * HD + gidx * 8;
    uint4 a = *reinterpret_cast<uint4*>(base), c4 = *reinterpret_cast<uint4*>(base + half);
    __nv_bfloat16* x1 = reinterpret_cast<__nv_bfloat16*>(&a);
    __nv_bfloat16* x2 = reinterpret_cast<__nv_bfloat16*>(&c4);
    const float pf = static_cast<float>(pos);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = gidx * 8 + j;
      const float inv_freq = powf(theta, -2.0f * static_cast<float>(d) / static_cast<float>(HD));
      float sn, cs;
      sincosf(pf * inv_freq, &sn, &cs);
      const float u = __bfloat162float(x1[j]), v = __bfloat162float(x2[j]);
      x1[j] = __float2bfloat16_rn(u * cs - v * sn);
      x2[j] = __float2bfloat16_rn(v * cs + u * sn);
    }
    *reinterpret_cast<uint4*>(base) = a;
    *reinterpret_cast<uint4*>(base + half) = c4;
    if (head >= q_heads && cached) {
      __nv_bfloat16* dst = k_cache + cache_row + (head - q_heads) * HD + gidx * 8;
      *reinterpret_cast<uint4*>(dst) = a;
      *reinterpret_cast<uint4*>(dst + half) = c4;
    }
  }
}

}  // namespace attn
}  // namespace df

#include "attention_decode.cuh"

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
  p.pairs_q = ((seq_len + BQ - 1) / BQ + 1) / 2;
  p.num_items = p.pairs_q * batch * q_heads;
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
    const cudaError_t ae = cudaFuncSetAttribute(attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (ae != cudaSuccess) return fail(DF_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(ae));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  int grid = sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (p.num_items < grid) grid = p.num_items;
  attention_kernel<false><<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(tm_q, tm_k, tm_v, p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DF_ECUDA, "attention launch: %s", cudaGetErrorString(e));
  return DF_OK;
}


extern "C" size_t df_attention_decode_workspace_bytes(int batch, int q_heads, int kv_heads, int max_len) {
  using namespace df::attn;
  if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || max_len <= 0) return 0;
  // the finest cut any launch on this device can choose: one key block per item
  const size_t splits = static_cast<size_t>((max_len + BKV - 1) / BKV);
  return static_cast<size_t>(batch) * q_heads * splits * (HD + 2) * sizeof(float);
}

extern "C" int df_attention_decode_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        const int* seq_lens_dev, int batch, int max_len, int q_heads, int kv_heads,
                                        int head_dim, int ld_q, int ld_kv, int ld_out, float scale, void* workspace,
                                        size_t workspace_bytes, int max_ctas, df_status_t* dev_status, void* stream) {
  using namespace df;
  using namespace df::attn;
  if (q == nullptr || k_cache == nullptr || v_cache == nullptr || out == nullptr || seq_lens_dev == nullptr ||
      workspace == nullptr || dev_status == nullptr)
    return fail(DF_EINVAL, "NULL pointer argument");
  if (head_dim != HD) return fail(DF_EUNSUPPORTED, "head_dim must be %d (got %d)", HD, head_dim);
  if (batch <= 0 || max_len <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0)
    return fail(DF_EINVAL, "batch, max_len and the head counts must be positive, q_heads a multiple of kv_heads");
  const int group = q_heads / kv_heads;
  if (group > T_MAX_GROUP)
    return fail(DF_EUNSUPPORTED, "at most %d query heads per key/value head (got %d)", T_MAX_GROUP, group);
  if (static_cast<long long>(batch) * max_len > 0x7fffffffLL) return fail(DF_EUNSUPPORTED, "batch * max_len exceeds 2^31 rows");
  if (ld_q < q_heads * HD || ld_kv < kv_heads * HD || ld_out < q_heads * HD || (ld_q % 8) != 0 || (ld_kv % 8) != 0 ||
      (ld_out % 8) != 0)
    return fail(DF_EINVAL, "row strides must cover the heads and be multiples of 8 elements");
  if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
        reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(workspace)) & 15u) != 0)
    return fail(DF_EINVAL, "q, the caches, out and the workspace must be 16-byte aligned");
  if (!(scale > 0.0f)) return fail(DF_EINVAL, "scale must be positive");
  const int sms = df_sm_count();
  if (sms <= 0) return fail(DF_ECUDA, "no CUDA device");
  int grid = sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;

  Params p;
  std::memset(&p, 0, sizeof(p));
  p.batch = batch;
  p.q_heads = q_heads;
  p.kv_heads = kv_heads;
  p.group = group;
  p.max_len = max_len;
  const bool keys_on_lanes = launch_option_value(DF_OPT_DECODE_KEYS_ON_LANES) != 0;
  p.chunk_blocks = decode_chunk_blocks(batch, kv_heads, max_len, grid, keys_on_lanes);
  p.splits = ((max_len + BKV - 1) / BKV + p.chunk_blocks - 1) / p.chunk_blocks;
  p.num_items = batch * kv_heads * p.splits;
  p.seq_lens = seq_lens_dev;
  p.ld_out = ld_out;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.timeout_ns = timeout_ns();
  p.status = reinterpret_cast<Status*>(dev_status);
  const size_t slots = static_cast<size_t>(batch) * q_heads * p.splits;
  if (workspace_bytes < slots * (HD + 2) * sizeof(float))
    return fail(DF_EINVAL, "workspace of %zu bytes is too small (need %zu)", workspace_bytes, slots * (HD + 2) * sizeof(float));
  p.partial_o = static_cast<float*>(workspace);
  p.partial_ml = p.partial_o + slots * HD;

  CUtensorMap tm_q, tm_k, tm_v;
  if (!make_map_q_decode(&tm_q, q, batch, q_heads, ld_q, group)) return DF_ECUDA;
  const uint64_t cache_rows = static_cast<uint64_t>(batch) * max_len;
  if (!make_map(&tm_k, k_cache, cache_rows, static_cast<uint64_t>(kv_heads) * HD, ld_kv)) return DF_ECUDA;
  if (!make_map(&tm_v, v_cache, cache_rows, static_cast<uint64_t>(kv_heads) * HD, ld_kv)) return DF_ECUDA;

  if (p.num_items < grid) grid = p.num_items;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaSuccess;
  if (keys_on_lanes) {
    // keys on the accumulator lanes: every softmax thread owns one key of a block
    auto kernel = group <= 4 ? decode_attention_kernel<4> : (group <= 8 ? decode_attention_kernel<8> : decode_attention_kernel<16>);
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM_BYTES);
    if (e != cudaSuccess) return fail(DF_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(T_THREADS, 1, 1);
    cfg.dynamicSmemBytes = T_SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr;
    cfg.numAttrs = dependent_launch_attr(&attr);
    cfg.attrs = &attr;
    e = cudaLaunchKernelEx(&cfg, kernel, tm_q, tm_k, tm_v, p);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return fail(DF_ECUDA, "decode attention launch: %s", cudaGetErrorString(e));
    }
  } else {
    if (group > DECODE_MAX_GROUP)
      return fail(DF_EUNSUPPORTED, "heads on the accumulator rows: at most %d query heads per key/value head (got %d)",
                  DECODE_MAX_GROUP, group);
    e = cudaFuncSetAttribute(attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return fail(DF_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attention_kernel<true><<<grid, THREADS, SMEM_BYTES, s>>>(tm_q, tm_k, tm_v, p);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DF_ECUDA, "decode attention launch: %s", cudaGetErrorString(e));
  if (keys_on_lanes && p.splits == 1) return DF_OK;  // whole sequences per item: the attention launch wrote the result
  const int warps = batch * q_heads;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((warps * 32 + 255) / 256, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = s;
    cudaLaunchAttribute attr;
    cfg.numAttrs = dependent_launch_attr(&attr);
    cfg.attrs = &attr;
    const float* po = p.partial_o;
    const float* pml = p.partial_ml;
    e = cudaLaunchKernelEx(&cfg, attention_decode_merge_kernel, po, pml, seq_lens_dev, batch, q_heads, p.splits,
                           p.chunk_blocks * BKV, max_len, p.out, ld_out);
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(DF_ECUDA, "decode merge launch: %s", cudaGetErrorString(e));
  }
  return DF_OK;
}

extern "C" int df_kv_cache_append_bf16(const void* k_new, const void* v_new, int ld_new, void* k_cache, void* v_cache,
                                       int ld_cache, const int* seq_lens_dev, int batch, int max_len, int kv_heads,
                                       int head_dim, void* stream) {
  using namespace df;
  if (k_new == nullptr || v_new == nullptr || k_cache == nullptr || v_cache == nullptr || seq_lens_dev == nullptr)
    return fail(DF_EINVAL, "NULL pointer argument");
  const int cols = kv_heads * head_dim;
  if (batch <= 0 || max_len <= 0 || cols <= 0 || (cols % 8) != 0 || ld_new < cols || ld_cache < cols || (ld_new % 8) != 0 ||
      (ld_cache % 8) != 0)
    return fail(DF_EINVAL, "bad shape: rows of kv_heads * head_dim elements, a multiple of 8, strides covering them");
  const int total = batch * (cols >> 3);
  attn::kv_cache_append_kernel<<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(k_new), static_cast<const __nv_bfloat16*>(v_new), ld_new,
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), ld_cache, seq_lens_dev, batch, max_len, cols);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DF_ECUDA, "kv append launch: %s", cudaGetErrorString(e));
  return DF_OK;
}

extern "C" int df_rope_append_bf16(void* qkv, int row_stride, const int* seq_lens_dev, int batch, int q_heads, int kv_heads,
                                   int head_dim, float theta, void* k_cache, void* v_cache, int ld_cache, int max_len,
                                   void* stream) {
  using namespace df;
  if (qkv == nullptr || seq_lens_dev == nullptr || k_cache == nullptr || v_cache == nullptr)
    return fail(DF_EINVAL, "NULL pointer argument");
  if (head_dim != attn::HD) return fail(DF_EUNSUPPORTED, "head_dim must be %d (got %d)", attn::HD, head_dim);
  const int cols = (q_heads + 2 * kv_heads) * head_dim;
  if (batch <= 0 || max_len <= 0 || q_heads <= 0 || kv_heads <= 0 || row_stride < cols || (row_stride % 8) != 0 ||
      ld_cache < kv_heads * head_dim || (ld_cache % 8) != 0)
    return fail(DF_EINVAL, "bad shape: a qkv row of (q_heads + 2 kv_heads) * head_dim elements, strides multiples of 8");
  if (((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15u) != 0)
    return fail(DF_EINVAL, "qkv and the caches must be 16-byte aligned");
  const int total = batch * ((q_heads + kv_heads) * (head_dim / 16) + kv_heads * head_dim / 8);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((total + 127) / 128, 1, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr;
  cfg.numAttrs = dependent_launch_attr(&attr);
  cfg.attrs = &attr;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, attn::rope_append_kernel, static_cast<__nv_bfloat16*>(qkv), row_stride,
                                           seq_lens_dev, batch, q_heads, kv_heads, theta, static_cast<__nv_bfloat16*>(k_cache),
                                           static_cast<__nv_bfloat16*>(v_cache), ld_cache, max_len);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(DF_ECUDA, "rope + append launch: %s", cudaGetErrorString(e));
  }
  return DF_OK;
}

#ifdef DF_ATTN_TIMING
extern "C" int df_debug_attn_timing(unsigned long long* out32, int reset) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out32, df::attn::g_attn_timing, sizeof(unsigned long long) * 32);
  if (reset) {
    unsigned long long z[32] = {0};
    cudaMemcpyToSymbol(df::attn::g_attn_timing, z, sizeof(z));
  }
  return 0;
}
#endif
