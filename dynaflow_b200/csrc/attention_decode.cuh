// Split-KV attention of a decode step with the keys on the accumulator lanes. Included by
// attention.cu (it uses that file's Params, Item, item_coords and helpers).
//
// A decode step has one query row per (sequence, head): with the query heads on the 128 MMA rows
// only `group` of them (the heads that share one key/value head, 4 for Llama-3) would carry data,
// and the softmax of a block would sit in `group` lanes of one warp. Here both products are
// transposed instead:
//
//   S^T[128 keys, 16] = K_j[128 keys, 128] * Q^T        (A = the key tile as TMA wrote it,
//                                                        B = the heads' query rows, N = 16)
//   O^T[128 dims, 16] += V_j^T[128 dims, 128 keys] * P^T (A = the value tile read M-major,
//                                                        B = P[16 heads, 128 keys] in shared memory)
//
// so that a softmax thread owns one KEY of the block (its lane of S^T) and `group` scores: all 128
// threads of four warps work, a block costs `group` exponentials per thread, and the products
// (2 x 8 MMAs of 16 columns) leave the tensor pipe two thirds idle. The per-head maximum over the
// block's keys is a warp shuffle reduction plus one named barrier; the per-head sums stay per
// thread until the item ends. The launch is then bound by the key/value bytes in flight. (Merging
// the chunks of a sequence inside this launch, by the chunk that finishes last, was built and
// measured: the merge's dependent L2 round trips stall that CTA's pipeline, 57 -> 105 us on
// 128 sequences of 4096 keys. The merge stays a second, small launch.)
//
// 256 threads: warp 0 copy producer, warp 1 MMA issuer, warp 2 tensor-memory owner, warps 4..7
// softmax. Tensor memory (128 columns): S^T of even / odd blocks at 0 / 32, O^T of even / odd items
// at 64 / 96. Shared memory: Q of even / odd items (2 x 4 KB: two 64-column halves of 16 rows),
// P of even / odd blocks (2 x 4 KB, same layout), six 32 KB key / value tiles, barriers.
#pragma once

namespace df {
namespace attn {

constexpr int T_THREADS = 256;
constexpr int T_KV_SLOTS = 6;
constexpr int T_HEAD_ROWS = 16;                 // B-operand rows (heads) of both products
constexpr int T_QP_HALF = T_HEAD_ROWS * 128;    // one 64-column half of Q or P: 16 rows x 128 B
constexpr int T_QP_BYTES = 2 * T_QP_HALF;
constexpr int T_TMEM_COLS = 128;
constexpr int T_S_COL = 0, T_O_COL = 64, T_BUF_COLS = 32;
constexpr int T_BAR_BYTES = 1024;
constexpr int kSmemUsedT = 4 * T_QP_BYTES + T_KV_SLOTS * TILE_BYTES + T_BAR_BYTES;
constexpr int T_SMEM_BYTES = kSmemUsedT + 1024;
static_assert(T_SMEM_BYTES <= SMEM_BYTES, "shared-memory budget of the decode kernel");
constexpr int T_MAX_GROUP = 16;

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

template <int GROUP>
__global__ void __launch_bounds__(T_THREADS, 1)
decode_attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* sQ = smem;                          // [2][T_QP_BYTES]
  uint8_t* sP = sQ + 2 * T_QP_BYTES;           // [2][T_QP_BYTES]
  uint8_t* sKV = sP + 2 * T_QP_BYTES;          // T_KV_SLOTS tiles; 16 KB from the start: 1024-aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + T_KV_SLOTS * TILE_BYTES);
  uint64_t* q_full = bars;                     // [2]
  uint64_t* q_empty = q_full + 2;              // [2]
  uint64_t* kv_full = q_empty + 2;             // [T_KV_SLOTS]
  uint64_t* kv_empty = kv_full + T_KV_SLOTS;   // [T_KV_SLOTS]
  uint64_t* s_full = kv_empty + T_KV_SLOTS;    // [2]
  uint64_t* p_full = s_full + 2;               // [2]
  uint64_t* pv_done = p_full + 2;              // [1]
  uint64_t* o_free = pv_done + 1;              // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* red_max = reinterpret_cast<float*>(tmem_slot + 2);  // [2][4][T_HEAD_ROWS]
  float* red_sum = red_max + 2 * 4 * T_HEAD_ROWS;            // [4][T_HEAD_ROWS]
  static_assert(23 * 8 + 8 + (2 * 4 + 4) * T_HEAD_ROWS * 4 <= T_BAR_BYTES, "barrier area");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // The copies fill only the rows of the heads that exist; the other rows of the 16-row operands
  // are zero from here on (their scores, probabilities and outputs are computed and dropped).
  for (int i = threadIdx.x; i < 4 * T_QP_BYTES / 16; i += T_THREADS) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async_smem();
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
      mbar_init(&o_free[s], 128);
    }
    for (int s = 0; s < T_KV_SLOTS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(pv_done, 1);
    *abort_flag = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, T_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = *tmem_slot;
  const Deadline dl{globaltimer_ns() + p.timeout_ns, abort_flag, p.status};
  // Everything above touched this CTA's own memories only. The kernel before this one in the stream
  // wrote the new token's queries and its keys and values (row seq_lens[b] - 1 of the caches):
  // nothing of that is read before grid_dependency_wait(). The copy producer alone runs ahead of
  // the wait, with key / value blocks that END before that row (they are from earlier steps).
  int ahead_tiles = 0;
  if (warp == 0 && lane == 0) {
    for (int t = blockIdx.x; t < p.num_items; t += gridDim.x) {
      Item w;
      if (!item_coords<true>(p, t, w)) continue;
      const int len_b = min(p.seq_lens[w.seq], p.max_len);
      const int first_key = w.split * p.chunk_blocks * BKV;
      const int old_blocks = max(0, min((len_b - 1 - first_key) / BKV, w.nb[0]));  // blocks that hold no key of the new token
      ahead_tiles = min(2 * old_blocks, T_KV_SLOTS);
      for (int u = 0; u < ahead_tiles; ++u) {
        uint8_t* dst = sKV + u * TILE_BYTES;
        const CUtensorMap* map = (u & 1) == 0 ? &tm_k : &tm_v;
        const int krow = w.kv_row + (u >> 1) * BKV;
        mbar_expect_tx(&kv_full[u], TILE_BYTES);
        tma_load_2d(dst, map, &kv_full[u], w.kv_head * HD, krow);
        tma_load_2d(dst + HALF_BYTES, map, &kv_full[u], w.kv_head * HD + 64, krow);
      }
      break;  // the first item only
    }
  }
  grid_dependency_wait();
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t it = 0, u = 0;  // items started, tiles put into the ring
      bool ok = true;
      for (int t = blockIdx.x; ok && t < p.num_items; t += gridDim.x) {
        Item w;
        if (!item_coords<true>(p, t, w)) continue;
        const uint32_t qb = it & 1u;
        if (!mbar_wait(&q_empty[qb], ((it >> 1) & 1u) ^ 1u, dl, WHERE_ATTN_PRODUCER, t)) break;
        // the group's query heads of this sequence: rows 0..group-1 of both halves
        mbar_expect_tx(&q_full[qb], 2 * p.group * 128);
        tma_load_3d(sQ + qb * T_QP_BYTES, &tm_q, &q_full[qb], 0, w.head, w.q_row);
        tma_load_3d(sQ + qb * T_QP_BYTES + T_QP_HALF, &tm_q, &q_full[qb], 64, w.head, w.q_row);
        for (int j = 0; j < w.nb[0] && ok; ++j) {
          const int krow = w.kv_row + j * BKV;
          for (int kv = 0; kv < 2; ++kv, ++u) {
            if (u < static_cast<uint32_t>(ahead_tiles)) continue;  // requested before the wait (the first item's first tiles)
            const uint32_t slot = u % T_KV_SLOTS;
            if (!mbar_wait(&kv_empty[slot], ((u / T_KV_SLOTS) & 1u) ^ 1u, dl, WHERE_ATTN_PRODUCER, t)) {
              ok = false;
              break;
            }
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
      constexpr uint32_t idesc_s = make_idesc_bf16(128, T_HEAD_ROWS);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, T_HEAD_ROWS) | (1u << 15);  // A (the value tile) M-major
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP), kv_addr = smem_u32(sKV);
      uint32_t it = 0, u0 = 0;  // items started, ring index of the item's K_0
      uint32_t blk = 0;         // blocks whose S has been issued / whose P V has been issued
      uint32_t blk_pv = 0;
      bool ok = true;
      auto issue_s = [&](int j, uint32_t qb, bool last, int t) -> bool {
        const uint32_t u = u0 + 2u * j;
        const uint32_t slot = u % T_KV_SLOTS;
        if (!mbar_wait(&kv_full[slot], (u / T_KV_SLOTS) & 1u, dl, WHERE_ATTN_MMA, t)) return false;
        tc_fence_after();
        // accumulator blk & 1: the softmax of block blk - 2 has read it (it signalled p_full for
        // that block, which the P V issued before this product waited for)
        const uint32_t sb = blk & 1u;
        const uint32_t d = tmem_base + T_S_COL + sb * T_BUF_COLS;
        const uint32_t k_addr = kv_addr + slot * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t da = make_desc_k_sw128(k_addr + (k >> 2) * HALF_BYTES) + 2u * (k & 3);
          const uint64_t db = make_desc_k_sw128(q_addr + qb * T_QP_BYTES + (k >> 2) * T_QP_HALF) + 2u * (k & 3);
          umma_bf16(d, da, db, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[sb]);
        umma_commit(&kv_empty[slot]);
        if (last) umma_commit(&q_empty[qb]);
        ++blk;
        return true;
      };
      for (int t = blockIdx.x; ok && t < p.num_items; t += gridDim.x) {
        Item w;
        if (!item_coords<true>(p, t, w)) continue;
        const int nb = w.nb[0];
        const uint32_t qb = it & 1u;
        if (!mbar_wait(&q_full[qb], (it >> 1) & 1u, dl, WHERE_ATTN_MMA, t)) break;
        // this item's O^T accumulator: the softmax threads have read what the item two back left there
        if (!mbar_wait(&o_free[qb], ((it >> 1) & 1u) ^ 1u, dl, WHERE_ATTN_MMA, t)) break;
        if (!issue_s(0, qb, nb == 1, t)) break;
        if (nb > 1 && !issue_s(1, qb, nb == 2, t)) break;
        const uint32_t d_o = tmem_base + T_O_COL + qb * T_BUF_COLS;
        for (int j = 0; j < nb && ok; ++j) {
          const uint32_t uv = u0 + 2u * j + 1u;
          const uint32_t vslot = uv % T_KV_SLOTS;
          if (!mbar_wait(&kv_full[vslot], (uv / T_KV_SLOTS) & 1u, dl, WHERE_ATTN_MMA, t)) {
            ok = false;
            break;
          }
          const uint32_t pb = blk_pv & 1u;
          if (!mbar_wait(&p_full[pb], (blk_pv >> 1) & 1u, dl, WHERE_ATTN_MMA, t)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k) {
            // 16 keys = two groups of eight rows of the value tile; the 64 further dims are HALF_BYTES on
            const uint64_t da = make_desc_mn_sw128(kv_addr + vslot * TILE_BYTES + k * 2 * 1024, HALF_BYTES, 1024);
            const uint64_t db = make_desc_k_sw128(p_addr + pb * T_QP_BYTES + (k >> 2) * T_QP_HALF) + 2u * (k & 3);
            umma_bf16(d_o, da, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(pv_done);
          umma_commit(&kv_empty[vslot]);
          ++blk_pv;
          if (j + 2 < nb && !issue_s(j + 2, qb, j + 2 == nb - 1, t)) {
            ok = false;
            break;
          }
        }
        u0 += 2u * nb;
        ++it;
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------- softmax
    const int wq = warp & 3;
    const int key = wq * 32 + lane;  // this thread's key of every block = its lane of S^T; its dim of O^T
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const float sl2 = p.scale_log2;
    uint32_t blk = 0, it = 0, u0 = 0;  // blocks and items gone through, ring index of the item's K_0
    bool ok = true;
    for (int t = blockIdx.x; ok && t < p.num_items; t += gridDim.x) {
      Item w;
      if (!item_coords<true>(p, t, w)) continue;
      const int nb = w.nb[0];
      const uint32_t qb = it & 1u;
      const uint32_t t_o = tmem_base + T_O_COL + qb * T_BUF_COLS + lane_base;
      float m_ref[GROUP], l[GROUP];
#pragma unroll
      for (int h = 0; h < GROUP; ++h) {
        m_ref[h] = -INFINITY;
        l[h] = 0.0f;
      }
      for (int j = 0; j < nb; ++j, ++blk) {
        const uint32_t sb = blk & 1u;
        ok = mbar_wait(&s_full[sb], (blk >> 1) & 1u, dl, WHERE_ATTN_SOFTMAX, t);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t sv[16];
        tmem_ld_32x16(tmem_base + T_S_COL + sb * T_BUF_COLS + lane_base, sv);
        tmem_ld_wait();
        const bool valid = j * BKV + key < w.len;  // keys past the end of the cache count for nothing
        float s[GROUP], mx[GROUP];
#pragma unroll
        for (int h = 0; h < GROUP; ++h) {
          s[h] = valid ? __uint_as_float(sv[h]) : -INFINITY;
          float v = s[h];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
          mx[h] = v;
        }
        float* rm = red_max + (blk & 1u) * (4 * T_HEAD_ROWS);
#pragma unroll
        for (int h = 0; h < GROUP; ++h)
          if (lane == h) rm[wq * T_HEAD_ROWS + h] = mx[h];
        epilogue_bar_sync();
        bool need = false;
        float m_new[GROUP];
#pragma unroll
        for (int h = 0; h < GROUP; ++h) {
          const float v = fmaxf(fmaxf(rm[h], rm[T_HEAD_ROWS + h]), fmaxf(rm[2 * T_HEAD_ROWS + h], rm[3 * T_HEAD_ROWS + h]));
          m_new[h] = fmaxf(m_ref[h], v);  // the item's first block has at least one key: finite from here on
          need = need || (j > 0 && (m_new[h] - m_ref[h]) * sl2 > RESCALE_THRESHOLD);
        }
        if (j == 0) {
#pragma unroll
          for (int h = 0; h < GROUP; ++h) m_ref[h] = m_new[h];
        } else if (need) {  // the same for all 128 threads
          // O^T still grows by the previous block's P V until that product has completed
          ok = mbar_wait(pv_done, (blk - 1u) & 1u, dl, WHERE_ATTN_SOFTMAX, t);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          uint32_t o[16];
          tmem_ld_32x16(t_o, o);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < GROUP; ++h) {
            const float alpha = ex2((m_ref[h] - m_new[h]) * sl2);
            m_ref[h] = m_new[h];
            l[h] *= alpha;
            o[h] = __float_as_uint(__uint_as_float(o[h]) * alpha);
          }
          tmem_st_32x16(t_o, o);
          tmem_st_wait();
        }
        // P[h][key] as bf16 into the B-operand tile of this block
        uint8_t* prow = sP + sb * T_QP_BYTES + (key >> 6) * T_QP_HALF + (key & 7) * 2;
        const int chunk = (key & 63) >> 3;
#pragma unroll
        for (int h = 0; h < GROUP; ++h) {
          const float e = valid ? ex2(fmaf(s[h], sl2, -m_ref[h] * sl2)) : 0.0f;
          const __nv_bfloat16 eb = __float2bfloat16_rn(e);
          l[h] += __bfloat162float(eb);  // the sum of what the P V product sees
          *reinterpret_cast<__nv_bfloat16*>(prow + (h >> 3) * 1024 + (h & 7) * 128 + ((chunk ^ (h & 7)) << 4)) = eb;
        }
        if ((j + 1) * BKV > w.len) {
          // The cache rows past the end of the sequence hold whatever was there before (possibly NaN
          // patterns), and 0 x NaN would reach O: such rows of the value tile are zeroed in place.
          const uint32_t uv = u0 + 2u * j + 1u;
          const uint32_t vslot = uv % T_KV_SLOTS;
          ok = mbar_wait(&kv_full[vslot], (uv / T_KV_SLOTS) & 1u, dl, WHERE_ATTN_SOFTMAX, t);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (!valid) {
            uint8_t* vrow = sKV + vslot * TILE_BYTES + (key >> 3) * 1024 + (key & 7) * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              reinterpret_cast<uint4*>(vrow)[c] = make_uint4(0u, 0u, 0u, 0u);
              reinterpret_cast<uint4*>(vrow + HALF_BYTES)[c] = make_uint4(0u, 0u, 0u, 0u);
            }
          }
        }
        fence_proxy_async_smem();  // the product reads P (and those rows) through the async proxy
        tc_fence_before();
        mbar_arrive(&p_full[sb]);
      }
      if (!ok) break;
      // ---- the item's results: per head the reference maximum, the sum, and the unnormalised O
      ok = mbar_wait(pv_done, (blk - 1u) & 1u, dl, WHERE_ATTN_SOFTMAX, t);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t o[16];
      tmem_ld_32x16(t_o, o);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&o_free[qb]);
#pragma unroll
      for (int h = 0; h < GROUP; ++h) {
        float v = l[h];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == h) red_sum[wq * T_HEAD_ROWS + h] = v;
      }
      epilogue_bar_sync();
      const size_t slot0 = (static_cast<size_t>(w.seq) * p.q_heads + w.head) * p.splits + w.split;
#pragma unroll
      for (int h = 0; h < GROUP; ++h) {
        if (h >= p.group) break;
        const float l_all = (red_sum[h] + red_sum[T_HEAD_ROWS + h]) + (red_sum[2 * T_HEAD_ROWS + h] + red_sum[3 * T_HEAD_ROWS + h]);
        if (p.splits == 1) {
          // the item is the whole sequence: its normalised rows are the result, nothing to merge
          p.out[static_cast<size_t>(w.seq) * p.ld_out + (w.head + h) * HD + key] = __float2bfloat16_rn(__uint_as_float(o[h]) / l_all);
          continue;
        }
        const size_t slot = slot0 + static_cast<size_t>(h) * p.splits;
        p.partial_o[slot * HD + key] = __uint_as_float(o[h]);
        if (key == h) {
          p.partial_ml[2 * slot] = m_ref[h] * sl2;
          p.partial_ml[2 * slot + 1] = l_all;
        }
      }
      epilogue_bar_sync();  // red_sum is free for the next item
      u0 += 2u * nb;
      ++it;
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
    tmem_dealloc(tmem_base, T_TMEM_COLS);
  }
}

}  // namespace attn
}  // namespace df
