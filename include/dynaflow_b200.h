/*
 * dynaflow_b200 -- C ABI of the B200 (sm_100a) execution backend for DynaFlow's
 * batch-split, overlapped transformer-layer schedule.
 *
 * Conventions
 *   - plain C types only; every pointer named "dev" or documented as device
 *     memory is a CUDA device pointer owned by the caller;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - return value: 0 = launched / done; < 0 = argument or CUDA API error
 *     (df_last_error() has the text); device-side failures (a bounded wait
 *     that ran out) are reported asynchronously in the df_status_t block the
 *     caller passed, never by trapping or spinning forever;
 *   - no entry point allocates or frees device memory and none synchronises the
 *     host with the device, unless its comment says so (df_comm_region_* do);
 *   - bf16 matrices are row-major with an explicit leading dimension counted
 *     in elements; all base pointers 16-byte aligned, leading dimensions a
 *     multiple of 8 elements.
 *
 * The library has no CPU fallback: on a machine without an sm_100 GPU the
 * compute entry points return DF_ECUDA.
 */
#ifndef DYNAFLOW_B200_H_
#define DYNAFLOW_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DF_ABI_VERSION 1

/* host-side return codes */
#define DF_OK 0
#define DF_EINVAL (-1)       /* bad shape, alignment or NULL pointer */
#define DF_ECUDA (-2)        /* a CUDA runtime / driver call failed   */
#define DF_EUNSUPPORTED (-3) /* shape outside what the kernels cover  */

/* device-side codes, written to df_status_t.code */
#define DF_ERR_NONE 0u
#define DF_ERR_TIMEOUT 1u /* a bounded wait ran past the deadline */
#define DF_ERR_PEER 2u    /* a peer rank never raised its flag     */

/* Asynchronous device status block (16 bytes of device memory, zero = ok). */
typedef struct df_status {
  uint32_t code;  /* first DF_ERR_* recorded since the last clear          */
  uint32_t where; /* which wait gave up (producer / mma / epilogue / flag) */
  uint32_t block; /* blockIdx.x of the reporting CTA                       */
  uint32_t aux;   /* tile index or peer rank                               */
} df_status_t;

/* ------------------------------------------------------------------ basics */

/* ABI version of the loaded library (DF_ABI_VERSION). */
int df_version(void);

/* Text of the last host-side error on the calling thread ("" if none). */
const char* df_last_error(void);

/* Deadline, in milliseconds from kernel start, that bounds every device-side
 * wait of kernels launched afterwards (default 2000). The reference has no
 * counterpart: its device waits are unbounded
 * (examples/ae/scheduler/vllm/tokenweave-kernels/include/tokenweave_multimem_utils.cuh:157-169). */
int df_set_timeout_ms(int ms);

/* Number of SMs of the current device (grid sizing of the persistent kernels). */
int df_sm_count(void);

/* Copies the status block to the host; synchronises `stream`. */
int df_status_read(const df_status_t* dev_status, df_status_t* host_out, void* stream);

/* Zeroes the status block on `stream` (asynchronous). */
int df_status_clear(df_status_t* dev_status, void* stream);

/* --------------------------------------------------------------- gated MLP
 *
 * Replaces, for one nano-batch, the three operators a host model runs inside a
 * DynaFlow compute subgraph: gate_up linear -> SiLU*mul -> down linear
 * (operator statement: examples/ae/up-silu-overlap.cu:75-82; subgraph
 * execution: dynaflow/runtime/engine.py:320-381).
 *
 * Weights use the torch.nn.Linear layout [out_features, in_features]:
 *   w_gate, w_up : [I, H]      w_down : [H, I]
 *   x : [M, H]   out : [M, H]  h (intermediate) : [M, I]
 */

/* C[M,N] = A[M,K] * B[N,K]^T, bf16 in, fp32 accumulate, bf16 out.
 * The plain linear layer of a subgraph (down / o / qkv projections).
 * max_ctas <= 0 means "one CTA per SM". */
int df_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, int lda, int ldb, int ldc,
                 int max_ctas, df_status_t* dev_status, void* stream);

/* h[M,I] = silu(x * w_gate^T) (.) (x * w_up^T): gate and up accumulators of the
 * same output columns live side by side in tensor memory and the SiLU*mul runs
 * in the epilogue, so the [M,2I] gate_up activation never exists in HBM.
 * Rounding points follow the reference operator chain: the two GEMM results
 * are rounded to bf16, the product silu(g)*u is computed in fp32 with expf and
 * rounded once to bf16. */
int df_gateup_silu_bf16(const void* x, const void* w_gate, const void* w_up, void* h, int M, int H, int I,
                        int ldx, int ldw, int ldh, int max_ctas, df_status_t* dev_status, void* stream);

/* Small-M forms of the two GEMMs. With fewer output tiles than SMs (decode-sized
 * nano-batches) the launch is bound by streaming the weights from HBM, so the
 * k-blocks of all tiles are divided evenly over the SMs ("stream-K"): every CTA
 * that holds only part of a tile's k-blocks leaves fp32 partial sums in
 * `splitk_ws`; once all contributors of a tile have delivered, each of them adds
 * the partial sums of its share of the tile's outputs in k order (deterministic)
 * and runs the epilogue on them. Launches of at most 128 rows use an
 * operand-swapped form of the same kernel (weight rows on the accumulator lanes)
 * with a deeper copy pipeline. `splitk_ws` is caller-owned device scratch of at least
 * df_gemm_splitk_workspace_bytes() bytes, 256-byte aligned, contents arbitrary;
 * launches that can overlap on the GPU need separate workspaces. With
 * splitk_ws == NULL, or when whole tiles already fill the SMs, these behave
 * exactly like df_gemm_bf16 / df_gateup_silu_bf16. */
size_t df_gemm_splitk_workspace_bytes(void);
int df_gemm_bf16_ws(const void* a, const void* b, void* c, int M, int N, int K, int lda, int ldb, int ldc,
                    int max_ctas, void* splitk_ws, size_t splitk_ws_bytes, df_status_t* dev_status, void* stream);
int df_gateup_silu_bf16_ws(const void* x, const void* w_gate, const void* w_up, void* h, int M, int H, int I,
                           int ldx, int ldw, int ldh, int max_ctas, void* splitk_ws, size_t splitk_ws_bytes,
                           df_status_t* dev_status, void* stream);

/* The form a GEMM launch of at most 128 rows takes on a device of `sms` SMs (no device needed: host arithmetic only):
 * weight rows per operand box (32, 64 or 128), k ranges per output tile (= CTAs per thread-block cluster: 1, 2, 4 or 8),
 * depth of the copy ring, output tiles, and the dynamic shared memory of a CTA. The grid is tiles * k_splits CTAs.
 * Any output pointer may be NULL. */
int df_small_gemm_plan(int M, int N, int K, int gate_up, int sms, int* box_rows, int* k_splits, int* stages, int* tiles,
                       size_t* shared_bytes);

/* Which of several equally valid forms a launch takes (all on by default). The forms differ in
 * the order of the fp32 summation, hence possibly in the last bf16 bit, never in validity; tests
 * switch them off to compare forms with each other. Process-wide; no counterpart in the reference.
 *   DF_OPT_STREAM_K        stream-K partition of launches with fewer tiles than SMs
 *   DF_OPT_MLP_ONE_LAUNCH  df_mlp_gated_bf16 as one persistent launch where it applies
 *   DF_OPT_OPERAND_SWAP    operand-swapped tiles for launches of at most 128 rows
 *   DF_OPT_SPLIT_K_SMALL   launches of at most 128 rows as (tile, k range) CTAs that exchange
 *                          partial sums with bulk copies (with DF_OPT_STREAM_K off: one CTA per tile)
 *   DF_OPT_DECODE_KEYS_ON_LANES  decode attention with both products transposed (a softmax thread per
 *                          key of a block) instead of the query heads on the accumulator rows
 *   DF_OPT_DEPENDENT_LAUNCH  the kernels of a decode step (small-rows GEMM, rotary + append, decode
 *                          attention and its merge, add + RMSNorm) are launched with programmatic
 *                          stream serialization: each starts while its predecessor in the stream
 *                          drains, sets itself up (the GEMM already fetches its weights) and only then
 *                          waits for the predecessor's results. Results are identical either way. */
#define DF_OPT_STREAM_K 0
#define DF_OPT_MLP_ONE_LAUNCH 1
#define DF_OPT_OPERAND_SWAP 2
#define DF_OPT_SPLIT_K_SMALL 3
#define DF_OPT_DECODE_KEYS_ON_LANES 4
#define DF_OPT_DEPENDENT_LAUNCH 5
#define DF_OPT_COUNT_ 6
int df_set_launch_option(int option, int value);

/* Bytes of scratch df_mlp_gated_bf16 needs: the bf16 intermediate h[M,I] plus one
 * stream-K workspace. */
size_t df_mlp_workspace_bytes(int M, int H, int I);

/* out = (silu(x * w_gate^T) (.) (x * w_up^T)) * w_down^T  for one nano-batch.
 * `workspace` is caller-owned device memory of df_mlp_workspace_bytes(M,H,I)
 * bytes, 256-byte aligned; its contents are scratch. */
int df_mlp_gated_bf16(const void* x, const void* w_gate, const void* w_up, const void* w_down, void* out,
                      void* workspace, int M, int H, int I, int max_ctas, df_status_t* dev_status,
                      void* stream);

/* ------------------------------------------- tensor-parallel reduction
 *
 * Replaces the all-reduce (+ residual add + RMSNorm) subgraph that a policy tags
 * `network` and moves to the communication stream: the matched collective
 * (examples/ae/scheduler/vllm/nanoflow.py:59-69), its fused substitute
 * (vllm/nanoflow.py:171-211, flashinfer call) and the in-tree kernel
 * fused_rs_ln_ag_cta (tokenweave-kernels/csrc/tokenweave.cu:38-198), without
 * NVLS/multimem: plain peer loads and stores over NVLink.
 *
 * Each rank owns one "region" per micro-batch slot, mapped by all ranks:
 *   region + df_comm_partial_offset : partial[max_rows, hidden] bf16 -- the rank's
 *        down / o projection writes its partial sums here (pass it as the GEMM's C)
 *   region + df_comm_sum_offset     : sum[max_rows, hidden] bf16 -- after the call,
 *        the reduced rows (identical on every rank)
 *   region + 0                      : flag words, zeroed at allocation
 * Calls that use the same region must be ordered (same stream); every rank must
 * issue the same sequence of calls on a region with the same T and n_ctas.
 */
#define DF_COMM_MAX_WORLD 8
#define DF_COMM_MAX_CTAS 64

typedef struct df_comm_rank {
  int rank;                          /* this rank's index in [0, world)              */
  void* regions[DF_COMM_MAX_WORLD];  /* region base of every rank, as mapped locally */
  const void* residual_in;           /* [T, hidden] bf16 or NULL (= zeros); fused call only */
  void* residual_out;                /* [T, hidden] bf16; may equal residual_in      */
  void* out;                         /* [T, hidden] bf16 normalised output           */
} df_comm_rank_t;

/* Bytes of one region / byte offsets of its two buffers (0 on bad arguments). */
size_t df_comm_region_bytes(int max_rows, int hidden);
size_t df_comm_partial_offset(int max_rows, int hidden);
size_t df_comm_sum_offset(int max_rows, int hidden);

/* Set-up time only (these four are the library's only calls that allocate, map or
 * free device memory, and they synchronise the device): allocate a zero-flagged
 * region and export its 64-byte CUDA IPC handle; map a peer's region from its
 * handle; unmap; free. The reference gets the same from
 * torch.distributed._symmetric_memory (examples/ae/scheduler/vllm/tokenweave.py:97-110). */
int df_comm_region_alloc(size_t bytes, void** dev_ptr, unsigned char ipc_handle[64]);
int df_comm_region_open(const unsigned char ipc_handle[64], void** dev_ptr);
int df_comm_region_close(void* peer_ptr);
int df_comm_region_free(void* dev_ptr);

/* sum = sum over ranks of partial, rows [0, T). n_ctas (<= DF_COMM_MAX_CTAS, <= 0
 * means 32) is the number of 256-thread CTAs, i.e. how many SMs the reduction
 * takes away from the GEMMs of the other micro-batch. */
int df_allreduce_bf16(const df_comm_rank_t* view, int world, int max_rows, int hidden, int T, int n_ctas,
                      df_status_t* dev_status, void* stream);

/* The two halves on their own, for expert parallelism (the all-gather / reduce-scatter pair the
 * reference's MoE dispatch and combine are built from, examples/ae/patch/vllm.patch:145-191).
 * Row slice r = rows [T*r/world, T*(r+1)/world).
 *   df_all_gather_bf16     : every rank has put ITS slice into its own partial buffer (at the
 *                            slice's row position); afterwards every rank's sum buffer holds all rows.
 *   df_reduce_scatter_bf16 : every rank's partial buffer holds T rows of contributions; afterwards
 *                            rank r's sum buffer holds, in slice r, their sum over ranks (fp32 in
 *                            rank order, rounded once). */
int df_all_gather_bf16(const df_comm_rank_t* view, int world, int max_rows, int hidden, int T, int n_ctas,
                       df_status_t* dev_status, void* stream);
int df_reduce_scatter_bf16(const df_comm_rank_t* view, int world, int max_rows, int hidden, int T, int n_ctas,
                           df_status_t* dev_status, void* stream);

/* The fused form: y = sum over ranks of partial; r' = y + residual_in;
 * out = bf16(r' * rsqrt(mean(r'^2) + eps)) * weight; residual_out = r'.
 * Rounding points as in tokenweave.cu:76-103 (bf16 residual, fp32 sum of squares). */
int df_allreduce_add_rmsnorm_bf16(const df_comm_rank_t* view, int world, int max_rows, int hidden, int T,
                                  const void* weight, float eps, int n_ctas, df_status_t* dev_status,
                                  void* stream);

/* The same with the residual stream SHARDED BY ROWS (what a tensor-parallel decoder needs, since
 * the residual is only ever added to the next reduction's output): rank r reads and updates
 * view->residual_in / residual_out for the rows [T*r/world, T*(r+1)/world) only, does the add
 * and the RMSNorm on those rows between the reduce-scatter and the all-gather, and the
 * normalised rows of all ranks land in every rank's `sum` buffer. Same per-row arithmetic as
 * the call above; no work is replicated and no extra bytes move. view->out is unused.
 * (tokenweave.cu:38-113 has this structure with in-switch reduction; here over peer memory.) */
int df_allreduce_add_rmsnorm_sharded_bf16(const df_comm_rank_t* view, int world, int max_rows, int hidden, int T,
                                          const void* weight, float eps, int n_ctas, df_status_t* dev_status,
                                          void* stream);

/* Process-wide: shared memory every reduction CTA of the calls above and below claims beyond what
 * it uses (0, the default, = none). With 40960 a reduction CTA cannot share an SM with a CTA of
 * the GEMM kernels (which hold 197 KB of the SM's 227 KB), nor the other way round: if the GEMMs
 * are launched with max_ctas = SMs - k, the reduction runs on the k SMs they leave free (two of
 * its CTAs per SM) instead of sharing SMs, and their memory traffic, with the GEMM CTAs. If no
 * SM is free the reduction simply starts when GEMM CTAs retire. No counterpart in the reference,
 * whose all-reduce runs on whatever SMs NCCL's kernel is given. */
int df_comm_set_exclusive_smem(int bytes);

/* The all-reduce (fuse = 0) and the sharded-residual fused form (fuse = 1) with the reduction
 * done inside the NVLink switch: `mc_region` is the multicast address of the SAME region that
 * view->regions[r] are the per-rank addresses of (an NVLink multicast object bound to every
 * rank's region, e.g. torch.distributed._symmetric_memory's multicast_ptr; region size and
 * layout as for the calls above). The owner of a row slice reads it with multimem.ld_reduce
 * (summed over all ranks by the switch, fp32 accumulation, rounded to bf16 once) and delivers
 * the result to every rank with multimem.st; the flag barriers still go through the per-rank
 * addresses. The order of the switch's summation is not the rank order of df_allreduce_bf16, so
 * results can differ from it in the last bf16 bit; they are identical on every rank.
 * (tokenweave.cu:38-113, the reference's fused all-reduce + RMSNorm, is built on the same
 * instructions.) weight / eps are unused when fuse = 0. */
int df_allreduce_multicast_bf16(const df_comm_rank_t* view, void* mc_region, int world, int max_rows, int hidden, int T,
                                int fuse, const void* weight, float eps, int n_ctas, df_status_t* dev_status,
                                void* stream);

/* The second half of the fused call as its own launch over all SMs:
 * r' = y + residual_in (NULL = zeros); out = bf16(r' * rsqrt(mean(r'^2) + eps)) * weight;
 * residual_out = r' (may equal residual_in). The RMSNorm(+residual) module a host model
 * runs after an all-reduce (matched together with it by
 * examples/ae/scheduler/vllm/nanoflow.py:59-69). df_allreduce_bf16 followed by this on the
 * result buffer equals df_allreduce_add_rmsnorm_bf16 bit for bit. */
int df_add_rmsnorm_bf16(const void* y, const void* residual_in, void* residual_out, void* out, const void* weight,
                        float eps, int T, int H, void* stream);

/* Test vehicle: runs `world` ranks of the same kernel on ONE GPU as one cooperative
 * launch (grid.y = rank), `views[r]` describing rank r, all regions in this GPU's
 * memory. Exercises the flag protocol and the arithmetic without a second GPU.
 * No counterpart in the reference. */
int df_allreduce_emulated_bf16(const df_comm_rank_t* views, int world, int max_rows, int hidden, int T,
                               const void* weight, float eps, int fuse_rmsnorm /* 0 all-reduce, 1 + replicated norm, 2 + sharded-residual norm,
                                                    3 reduce-scatter, 4 all-gather */,
                               int n_ctas, df_status_t* dev_status, void* stream);

/* -------------------------------------------------------- mixture of experts
 *
 * The parts of the reference's dispatch / expert / combine operator triple
 * (examples/ae/patch/vllm.patch:308-379, 423-527) that are not collectives or GEMMs, for top-2
 * routing with renormalised softmax weights. Nothing here synchronises with the host: the number
 * of tokens routed to an expert stays in device memory, where the expert GEMMs read it.
 */

/* ids[t,0..1] = the two experts with the largest softmax(logits[t,:]) (ties: lower index),
 * weights[t,0..1] = their probabilities divided by their sum. logits bf16 [T,E]. */
int df_moe_route_top2(const void* logits, int T, int E, int* ids, float* weights, void* stream);

/* The tokens routed to `expert`, ascending: rows[k] = token, slot[k] = 0/1 (first or second
 * choice), pos[t] = k or -1, *count_dev = how many. rows/slot need T entries, pos T entries. */
int df_moe_select_rows(const int* ids, int T, int expert, int* rows, int* slot, int* pos, int* count_dev, void* stream);

/* out[k,:] = x[rows[k],:] for k < min(*count_dev, capacity) (bf16, H % 8 == 0; out has `capacity` rows,
 * rows beyond that are not written). */
int df_moe_gather_rows(const void* x, const int* rows, const int* count_dev, int capacity, int H, void* out,
                       void* stream);

/* contrib[t,:] = bf16(weights[t, slot[pos[t]]] * y[pos[t],:]) where pos[t] >= 0, zeros elsewhere:
 * this expert's contribution to every token, ready for the reduce-scatter / sum over experts. */
int df_moe_scatter_rows(const void* y, const int* pos, const int* slot, const float* weights, int T, int H,
                        void* contrib, void* stream);

/* df_mlp_gated_bf16 over the first *rows_dev rows of x (at most capacity_rows, which also sizes
 * the workspace: df_mlp_workspace_bytes(capacity_rows, H, I)); rows beyond are not touched. */
int df_mlp_gated_bf16_rows_on_device(const void* x, const void* w_gate, const void* w_up, const void* w_down, void* out,
                                     void* workspace, int capacity_rows, const int* rows_dev, int H, int I, int max_ctas,
                                     df_status_t* dev_status, void* stream);

/* Expert-parallel all-to-all over peer memory: the dispatch and combine collectives of the reference's
 * all2all managers (examples/ae/patch/vllm.patch:145-191), built as the scope asks: a peer st.global PUT
 * kernel after an exchange of per-(source, expert) counts, and a PULL for the way back. Experts are
 * owned in contiguous blocks (expert e lives on rank e / (experts / world)).
 *
 * Every rank owns one region (df_a2a_region_bytes; allocate and map it with df_comm_region_alloc /
 * _open like the reduction regions) holding flags, the exchanged counts, per local expert the number
 * of rows that arrived (an int at df_a2a_rows_total_offset() + 4 * local_expert: pass its address as
 * rows_dev of df_mlp_gated_bf16_rows_on_device) and two packed buffers [local expert][capacity][hidden]
 * at df_a2a_packed_in_offset / df_a2a_packed_out_offset: the expert MLP of local expert l reads
 * packed_in[l] and writes packed_out[l]. capacity = total tokens of all ranks never overflows; rows
 * beyond it would be dropped (their weight counts as zero in the combine).
 *   df_a2a_plan      local: pos[t,c] = rank of (token t, choice c) among this rank's pairs with the
 *                    same expert, in token order; counts[e] = pairs per expert. ids int32 [tokens, 2].
 *   df_a2a_dispatch  counts to everyone, block-to-block barrier, every routed row of x [tokens, hidden]
 *                    written to its place in the owner's packed_in, barrier.
 *   df_a2a_combine   barrier (all expert outputs complete), out[t] = bf16(w[t,0] y0 + w[t,1] y1) with the
 *                    two rows pulled from the owners' packed_out, barrier.
 * Every rank must issue the same sequence of dispatch / combine calls on a region with the same n_ctas
 * (<= DF_COMM_MAX_CTAS; <= 0 means 32). df_a2a_emulated_bf16 runs all ranks of one call as one
 * cooperative launch on one GPU (test vehicle, arrays indexed by rank; combine = 0 / 1). */
#define DF_A2A_MAX_EXPERTS 64
typedef struct df_a2a_rank {
  int rank;
  void* regions[DF_COMM_MAX_WORLD];
} df_a2a_rank_t;
size_t df_a2a_region_bytes(int world, int experts, int capacity, int hidden);
size_t df_a2a_packed_in_offset(int world, int experts, int capacity, int hidden);
size_t df_a2a_packed_out_offset(int world, int experts, int capacity, int hidden);
size_t df_a2a_rows_total_offset(void);
int df_a2a_plan(const int* ids, int tokens, int experts, int* pos, int* counts, void* stream);
int df_a2a_dispatch_bf16(const df_a2a_rank_t* view, int world, int experts, int capacity, int hidden, const void* x,
                         const int* ids, const int* pos, const int* counts, int tokens, int n_ctas,
                         df_status_t* dev_status, void* stream);
int df_a2a_combine_bf16(const df_a2a_rank_t* view, int world, int experts, int capacity, int hidden, const int* ids,
                        const int* pos, const float* weights, int tokens, void* out, int n_ctas,
                        df_status_t* dev_status, void* stream);
int df_a2a_emulated_bf16(const df_a2a_rank_t* views, int world, int experts, int capacity, int hidden, int tokens,
                         const void* const* x, const int* const* ids, const int* const* pos, const int* const* counts,
                         const float* const* weights, void* const* out, int combine, int n_ctas,
                         df_status_t* dev_status, void* stream);

/* Rotary position embedding (rotate-half), in place on the first `heads` heads of every row of a
 * fused qkv activation (q heads followed by k heads: pass heads = q_heads + kv_heads); row t is
 * rotated by positions[t]. Part of the attention subgraph's prologue in a decoder layer. */
int df_rope_bf16(void* qkv, const int* positions, int T, int heads, int head_dim, int row_stride, float theta,
                 void* stream);

/* ----------------------------------------------------------------- attention
 *
 * The attention core of a decoder layer: the subgraph the reference's policies cut out, tag
 * `attention` and leave to the host model's own kernels, setting the nano-batch's attention
 * metadata before each call (examples/ae/scheduler/vllm/nanoflow.py:91-94, 231).
 *
 * Causal self-attention of a prefill nano-batch, grouped-query: q [total_rows, q_heads * 128],
 * k and v [total_rows, kv_heads * 128], out [total_rows, q_heads * 128], all bf16 with explicit row
 * strides in elements (the three inputs may be column ranges of one fused qkv activation).
 * The rows are `batch` sequences back to back; with cu_seqlens_dev == NULL every sequence has
 * seq_len rows (total_rows == batch * seq_len), otherwise cu_seqlens_dev[b] (device memory,
 * batch + 1 ints) is the first row of sequence b and seq_len the longest length. Query head h
 * reads key/value head h / (q_heads / kv_heads). out = softmax(scale * q k^T + causal mask) v,
 * scores and sums in fp32, probabilities rounded to bf16 before the second product.
 * head_dim must be 128. max_ctas <= 0 means one CTA per SM. */
int df_attention_prefill_bf16(const void* q, const void* k, const void* v, void* out, int total_rows, int batch,
                              int seq_len, const int* cu_seqlens_dev, int q_heads, int kv_heads, int head_dim,
                              int ld_q, int ld_k, int ld_v, int ld_out, float scale, int max_ctas,
                              df_status_t* dev_status, void* stream);

/* Attention of a decode step: one new token per sequence against a key/value cache (the same
 * opaque `attention` subgraph, in the decode phase the reference captures into CUDA graphs per
 * nano-batch: dynaflow/executor/cudagraph.py:84-123).
 *   q        [batch, q_heads * 128] bf16, row stride ld_q (a column range of the fused qkv rows)
 *   k_cache, v_cache  [batch, max_len, kv_heads * 128] bf16, row stride ld_kv elements: sequence b
 *            owns rows [b * max_len, (b + 1) * max_len), of which the first seq_lens_dev[b] are valid
 *            (the new token's key and value included: see df_rope_append_bf16). What lies past the
 *            valid rows is read but never reaches the result, whatever it holds
 *   out      [batch, q_heads * 128] bf16
 * The keys of a sequence are cut into chunks that different CTAs process (split-KV); `workspace`
 * (df_attention_decode_workspace_bytes, 16-byte aligned, contents arbitrary) receives the chunks'
 * partial results, which a second small launch merges (no cut, no second launch, when the (sequence,
 * key/value head) pairs alone fill the SMs). seq_lens_dev stays in device memory, so a captured graph
 * follows growing sequences. head_dim must be 128, q_heads / kv_heads <= 16.
 * With DF_OPT_DEPENDENT_LAUNCH on, the launch starts while its predecessor in the stream drains and, before
 * it waits for that kernel, already reads seq_lens_dev and cache blocks that end BEFORE row seq_lens_dev[b] - 1:
 * a predecessor that itself releases its dependents early (griddepcontrol.launch_dependents: this library's
 * kernels, e.g. df_rope_append_bf16, or a host kernel written that way) may write the new token's row and q,
 * nothing else of these inputs. A predecessor that does not release early is a full dependency. */
size_t df_attention_decode_workspace_bytes(int batch, int q_heads, int kv_heads, int max_len);
int df_attention_decode_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                             const int* seq_lens_dev, int batch, int max_len, int q_heads, int kv_heads,
                             int head_dim, int ld_q, int ld_kv, int ld_out, float scale, void* workspace,
                             size_t workspace_bytes, int max_ctas, df_status_t* dev_status, void* stream);

/* cache[b, seq_lens_dev[b] - 1, :] = new[b, :] for keys and values: the new token of every
 * sequence takes the last valid position of its cache (k_new / v_new: [batch, kv_heads * head_dim]
 * with row stride ld_new, e.g. column ranges of the fused qkv rows after df_rope_bf16). */
int df_kv_cache_append_bf16(const void* k_new, const void* v_new, int ld_new, void* k_cache, void* v_cache,
                            int ld_cache, const int* seq_lens_dev, int batch, int max_len, int kv_heads,
                            int head_dim, void* stream);

/* The two steps before df_attention_decode_bf16 as one launch: rotary embedding (base theta, position
 * seq_lens_dev[b] - 1) of the new token's query and key heads, in place in the fused qkv row
 * [q heads | k heads | v heads] (row stride row_stride elements), and the rotated keys and the values
 * into position seq_lens_dev[b] - 1 of the caches (layout as for df_attention_decode_bf16). Equal,
 * bit for bit, to df_rope_bf16 on the first q_heads + kv_heads heads followed by
 * df_kv_cache_append_bf16. head_dim must be 128. */
int df_rope_append_bf16(void* qkv, int row_stride, const int* seq_lens_dev, int batch, int q_heads, int kv_heads,
                        int head_dim, float theta, void* k_cache, void* v_cache, int ld_cache, int max_len,
                        void* stream);

/* Size of the library-owned scratch behind df_mlp_gated_bf16_static: 64 MiB of
 * static device memory, held by every GPU that loads the library until the
 * process exits. */
#define DF_MLP_STATIC_SCRATCH_BYTES (64u << 20)

/* Same computation as df_mlp_gated_bf16 for callers that have no scratch to give
 * and must not allocate any. (No counterpart in the reference: its operators run
 * inside PyTorch, whose caching allocator provides every temporary.)
 *
 * Who needs it: a policy's `func=` substitute is handed only the subgraph's input
 * tensors, and a serving engine that measured free HBM at start-up and gave the
 * rest to its KV cache has nothing left to allocate from later; a cudaMalloc in
 * the middle of a forward would also synchronise the whole device and serialise
 * the micro-batch streams whose overlap is the point of the schedule. This entry
 * point therefore keeps the bf16 intermediate h[M,I] in a file-scope __device__
 * array of DF_MLP_STATIC_SCRATCH_BYTES inside the library and calls no
 * cudaMalloc, cudaFree or other allocating routine.
 *
 * Limits and rules
 *   - M * I * 2 bytes must fit in DF_MLP_STATIC_SCRATCH_BYTES (e.g. M <= 2340 rows
 *     at I = 14336); larger shapes are refused with DF_EUNSUPPORTED and a message
 *     naming both numbers. Use df_mlp_gated_bf16 with your own workspace then.
 *   - The first call on each device resolves the device address of the array
 *     (once per device, with that device current). Make that first call outside
 *     any stream capture.
 *   - All calls on a device share the one array, and it keeps whatever the last
 *     call left there; nothing in it has to start at zero (every element that is
 *     read has been written earlier in the same call). Two calls whose kernels
 *     can overlap on the GPU (different streams without an ordering between
 *     them) race on it: order them, or give one of them a workspace of its own
 *     through df_mlp_gated_bf16. */
int df_mlp_gated_bf16_static(const void* x, const void* w_gate, const void* w_up, const void* w_down, void* out,
                             int M, int H, int I, int max_ctas, df_status_t* dev_status, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* DYNAFLOW_B200_H_ */
