/*
 * minivllm_b200 — C ABI of the B200 (sm_100a) ragged-batch attention path.
 *
 * Every entry point is `extern "C"`, takes plain device pointers, sizes and a
 * CUDA stream handle (a `cudaStream_t` passed as `void*`), launches on that
 * stream without synchronising the host, and returns an `int` status:
 * 0 = launched, non-zero = rejected before any launch (see mv_status).
 * The library allocates no device memory on these paths and keeps no pointer
 * after a call returns; the caller owns inputs, outputs and scratch.
 *
 * Each declaration cites the function of the reference engine
 * (Wenyueh/MinivLLM, paths relative to that project) whose work it does.
 */
#ifndef MINIVLLM_B200_H
#define MINIVLLM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types of q/k/v and of a non-quantised cache. */
enum mv_dtype { MV_F16 = 0, MV_BF16 = 1 };

enum mv_status {
  MV_OK = 0,
  MV_ERR_NULL = 1,        /* a required pointer is null */
  MV_ERR_ALIGN = 2,       /* a pointer or stride breaks the 16-byte rule */
  MV_ERR_SHAPE = 3,       /* unsupported head_dim / head ratio / negative size */
  MV_ERR_WORKSPACE = 4,   /* scratch buffer too small */
  MV_ERR_DTYPE = 5,
  MV_ERR_CUDA = 6,        /* the launch itself reported an error */
  MV_ERR_LIMIT = 7        /* size beyond a documented fixed maximum */
};

/* Text of the last non-zero status returned on the calling thread. */
const char* mv_last_error_string(void);

/* Library version, bumped when a signature changes. */
int mv_abi_version(void);

/*
 * Scatter new K/V rows into the paged cache.
 * Replaces: src/myvllm/layers/attention.py:67-108 `store_kvcache` and its
 * Triton kernel :7-64.  For every token t with slot_mapping[t] >= 0:
 *   k_cache[slot_mapping[t]] = key[t],  v_cache[slot_mapping[t]] = value[t]
 * with the cache seen as (num_slots, num_kv_heads, head_dim); slot -1 (any
 * negative) is skipped.  key/value are (num_tokens, num_kv_heads, head_dim)
 * with an arbitrary token stride (in elements) so the split view of a fused
 * qkv projection needs no copy; heads and head_dim are contiguous.
 *
 * When k_scale and v_scale are non-null the caches hold int8 codes and the
 * scatter is fused with per-token-per-head symmetric quantisation (no
 * counterpart in the reference, which has no quantisation):
 *   amax = max|x| over head_dim (fp32); s = float(fp16(amax / 127));
 *   code = clamp(rint(x / s), -127, 127), 0 when s == 0;
 * codes go to (num_slots, num_kv_heads, head_dim) int8 and s, as fp16, to
 * (num_slots, num_kv_heads).
 */
int mv_store_kvcache(const void* key, const void* value,
                     int64_t k_stride_tok, int64_t v_stride_tok,
                     void* k_cache, void* v_cache,
                     void* k_scale, void* v_scale,
                     const int64_t* slot_mapping,
                     int64_t num_tokens, int64_t num_slots,
                     int num_kv_heads, int head_dim,
                     int dtype, void* stream);

/*
 * Bytes of scratch mv_paged_decode needs for the given problem (split-K
 * partial results); depends on shapes only, never on context_lens values.
 * Returns -1 for an invalid shape.
 * The first 64 KiB of the scratch hold arrival counters (which piece of a
 * split sequence was written last): they must be ZERO when the buffer is
 * first used, and every call leaves them zero, so fill the buffer with zeros
 * once when it is allocated.  One buffer may serve calls of any shapes, one
 * at a time (calls that overlap on the GPU need buffers of their own).
 */
int64_t mv_paged_decode_workspace_bytes(int batch, int num_heads,
                                        int num_kv_heads, int head_dim,
                                        int max_blocks, int block_size);

/*
 * One-query-per-sequence attention over the paged cache.
 * Replaces: src/myvllm/layers/attention.py:418-473 `paged_attention_decode`
 * and its Triton kernel :283-415.  For sequence b and query head h:
 *   out[b,h] = softmax_j(scale * q[b,h] . K[b,j,h/G]) . V[b,j,h/G],  j < context_lens[b]
 * where token j lives at cache[block_tables[b, j / block_size], j % block_size]
 * and G = num_heads / num_kv_heads.  Tokens whose table entry is negative
 * get zero weight; a row with no live token writes zeros.
 * q/out are (batch, num_heads, head_dim) contiguous; caches are
 * (num_blocks, block_size, num_kv_heads, head_dim) contiguous, of `dtype`,
 * or int8 codes with fp16 scales (num_blocks, block_size, num_kv_heads)
 * when k_scale/v_scale are non-null.  block_tables is (batch, max_blocks)
 * int32 with row stride bt_stride; context_lens is int32 or int64 and is
 * clamped to [0, max_blocks * block_size].
 * The grid depends on shapes only, so the call can be captured in a graph.
 * batch * max_blocks * block_size must stay below 2^31 (status 7 otherwise).
 * The KV tokens of the whole batch are divided evenly among the thread
 * blocks, so where a long sequence is cut depends on the other sequences:
 * a row's result can differ in its last bits between batch compositions.
 */
int mv_paged_decode(void* out, const void* q,
                    const void* k_cache, const void* v_cache,
                    const void* k_scale, const void* v_scale,
                    const int32_t* block_tables, int64_t bt_stride,
                    int max_blocks,
                    const void* context_lens, int ctx_is_i64,
                    int batch, int num_heads, int num_kv_heads, int head_dim,
                    int block_size, int64_t num_blocks, float scale,
                    void* workspace, int64_t workspace_bytes,
                    int dtype, void* stream);

/*
 * mv_paged_decode for callers that cannot allocate device memory.
 * No counterpart in the reference (its Triton decode kernel needs no scratch
 * because it never splits a sequence).  Same arguments and results as
 * mv_paged_decode without `workspace`: the split-K scratch is a fixed array of
 * mv_paged_decode_static_capacity() bytes (8 MiB) inside the library's device
 * image, held by every GPU that loads the library.  Meant for a serving
 * process that gave all free HBM to the KV pool and forbids later
 * allocation, for latency-critical loops where the allocator must not run,
 * and for bindings that only pass inputs and outputs (not for CUDA host
 * callbacks: no launch may be made from one).
 * A problem needing more scratch than the array holds returns MV_ERR_LIMIT
 * and launches nothing.  All calls on a device share the array: calls that
 * overlap on the GPU race, so keep them on one stream or order them.  The
 * first call on each device resolves the array's address (a host-side lookup)
 * and should be made before any stream capture, from one host thread; the
 * address is stale after a cudaDeviceReset.  Neither function calls
 * cudaMalloc, cudaFree or any allocating library routine.
 */
int64_t mv_paged_decode_static_capacity(void);
int mv_paged_decode_static(void* out, const void* q,
                           const void* k_cache, const void* v_cache,
                           const void* k_scale, const void* v_scale,
                           const int32_t* block_tables, int64_t bt_stride,
                           int max_blocks,
                           const void* context_lens, int ctx_is_i64,
                           int batch, int num_heads, int num_kv_heads,
                           int head_dim, int block_size, int64_t num_blocks,
                           float scale, int dtype, void* stream);

/*
 * Varlen causal prefill attention over a packed ragged batch.
 * Replaces: src/myvllm/layers/attention.py:212-280 `flash_attention_prefill`
 * and its Triton kernel :111-209.  Sequence s owns rows
 * [cu_seqlens[s], cu_seqlens[s+1]) of q/k/v; row i attends to rows <= i of
 * its own sequence; query head h reads kv head h / (num_heads/num_kv_heads).
 * q/out are (total_tokens, num_heads, 128), k/v (total_tokens, num_kv_heads,
 * 128); q/k/v take a token stride in elements (heads dense within a token),
 * out is contiguous.  fp32 accumulation on the tcgen05 tensor cores.
 * No host synchronisation: the grid is an upper bound computed from
 * total_tokens and num_seqs, or (up to 320 sequences) one block per SM that
 * takes query tiles from a work counter inside the library; a launch uses
 * the next of 1,024 counters and leaves it zeroed, nothing is allocated.
 * error_word points to one zero-initialised int in device memory that the
 * caller keeps: a kernel wait that runs out of time stores a non-zero code
 * there (and later launches return at once until the caller clears it).
 */
int mv_prefill_varlen(void* out, const void* q, const void* k, const void* v,
                      int64_t q_stride_tok, int64_t k_stride_tok,
                      int64_t v_stride_tok, const int32_t* cu_seqlens,
                      int num_seqs, int64_t total_tokens, int num_heads,
                      int num_kv_heads, int head_dim, float scale,
                      int* error_word, int dtype, void* stream);

/*
 * Prefill attention with a cached prefix (or a chunk of a longer prompt):
 * the queries are the packed UNCACHED tokens (cu_seqlens_q), the keys and
 * values are read from the paged cache through block_tables, which must
 * already hold every token of the step (store_kvcache first).  Sequence s has
 * k_s = cu_seqlens_k[s+1]-cu_seqlens_k[s] keys and q_s queries; query i sits
 * at position k_s - q_s + i and attends to keys at positions <= its own.
 * This is the case the reference prepares (src/myvllm/engine/model_runner.py
 * :198-215 builds cu_seqlens_k != cu_seqlens_q and block_tables on a prefix
 * hit) but never computes: its prefill kernel indexes K/V with the query
 * offsets (src/myvllm/layers/attention.py:135-137,171,194).  block_size must
 * divide 128 (multiple of 8) or be a multiple of 128.  Same error_word
 * contract as mv_prefill_varlen.
 * Precondition: every row of every cache block that a table names must hold
 * FINITE values, also the rows past a sequence's last key (the rest of its
 * last block) and block 0 (read in place of a missing table entry).  Such
 * rows get weight exactly 0, but their V values still pass through the
 * tensor-core product, and 0 x NaN or 0 x Inf is NaN.  Allocate the pool
 * zero-initialised (the engine does); blocks that were used before hold
 * finite stale values and are fine.  mv_paged_decode has no such
 * precondition (it zero-fills rows it does not use).
 */
int mv_prefill_paged(void* out, const void* q, int64_t q_stride_tok,
                     const void* k_cache, const void* v_cache,
                     const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                     const int32_t* block_tables, int64_t bt_stride,
                     int max_blocks, int block_size, int64_t num_blocks,
                     int num_seqs, int64_t total_q_tokens, int num_heads,
                     int num_kv_heads, int head_dim, float scale,
                     int* error_word, int dtype, void* stream);

/*
 * Per-step metadata, built on the GPU from persistent per-sequence state.
 * State (device memory, owned by the caller, one row per sequence "slot"):
 *   tables (num_slots, max_blocks) int32 block table rows, -1 = none;
 *   seq_len_state (num_slots) int32 tokens already in the cache;
 *   last_token_state (num_slots) int64 last sampled token.
 *
 * mv_build_decode_meta replaces src/myvllm/engine/model_runner.py:231-256
 * `prepare_decode` (and the per-layer positions of models/qwen3.py:210-212):
 * for row b < *n_active with slot s and p = seq_len_state[s] it writes
 * input_ids[b] = last_token_state[s], positions[b] = p, context_lens[b] = p+1,
 * slot_mapping[b] = table[s][p/bs]*bs + p%bs, tables_out[b] = table[s], and
 * bumps seq_len_state[s]; rows b >= *n_active (graph padding) get 0/0/0/-1
 * and a table of -1.  n_active is read on the device so a captured graph can
 * be replayed with any batch up to batch_padded.  A slot may appear once.
 *
 * mv_build_prefill_meta replaces model_runner.py:180-227 `prepare_prefill`
 * (and qwen3.py:199-206): sequence i (slot seq_slots[i]) feeds tokens at
 * positions num_cached[i] .. seq_lens[i]-1 (num_cached may be null = 0);
 * writes cu_seqlens_q/k (num_seqs+1, int32), positions and slot_mapping
 * (total_tokens, int64), last_token_index (num_seqs, int64) and sets
 * seq_len_state[slot] = seq_lens[i].  total_tokens = sum of fed tokens.
 *
 * mv_update_block_tables applies `num_updates` (slot, index, block) int32
 * triples to the table state (a sequence gained a block, or was allocated).
 */
int mv_build_decode_meta(const int32_t* seq_slots, const int32_t* n_active,
                         int batch_padded, const int32_t* tables,
                         int64_t tables_stride, int max_blocks, int block_size,
                         int32_t* seq_len_state, const int64_t* last_token_state,
                         int64_t* input_ids, int64_t* positions,
                         int64_t* slot_mapping, int64_t* context_lens,
                         int32_t* tables_out, int64_t out_stride, void* stream);
int mv_build_prefill_meta(const int32_t* seq_slots, const int32_t* seq_lens,
                          const int32_t* num_cached, int num_seqs,
                          int64_t total_tokens, const int32_t* tables,
                          int64_t tables_stride, int max_blocks, int block_size,
                          int32_t* seq_len_state, int32_t* cu_seqlens_q,
                          int32_t* cu_seqlens_k, int64_t* positions,
                          int64_t* slot_mapping, int64_t* last_token_index,
                          void* stream);
int mv_update_block_tables(const int32_t* updates, int num_updates,
                           int32_t* tables, int64_t tables_stride,
                           int max_blocks, int num_slots, void* stream);

/*
 * Fused pre-attention step on the fused qkv projection output
 * qkv (tokens, (num_heads + 2*num_kv_heads) * 128), token stride in elements:
 * RMSNorm of every q and k head row (x * rsqrt(mean(x^2) + eps) * gamma,
 * rounded to the model dtype), rotate-half rotary embedding from fp32
 * cos/sin tables (max_position, 64) at positions[t], then q -> q_out
 * (tokens, num_heads, 128), k -> k_out (tokens, num_kv_heads, 128) and, when
 * slot_mapping is non-null, k and v -> the paged caches at slot_mapping[t]
 * (negative = skip), i.e. store_kvcache fused in.  With k_scale / v_scale
 * non-null the caches are int8 and the rows are quantised on the way in, with
 * the arithmetic and layouts of mv_store_kvcache (codes and fp16 scales equal
 * what mv_store_kvcache writes for k_out and v).
 * Replaces, in one launch: src/myvllm/models/qwen3.py:104-108 (rms_norm of q
 * and k, rotary_emb), layers/layernorm.py:10-17, layers/rotary_embedding.py
 * :4-23,77-83 and the store_kvcache call of layers/attention.py:498-510.
 */
int mv_qk_norm_rope_store(const void* qkv, int64_t qkv_stride_tok,
                          const int64_t* positions, const float* cos_table,
                          const float* sin_table, int max_position,
                          const void* gamma_q, const void* gamma_k, float eps,
                          void* q_out, void* k_out, void* k_cache,
                          void* v_cache, void* k_scale, void* v_scale,
                          const int64_t* slot_mapping,
                          int64_t num_slots, int64_t num_tokens, int num_heads,
                          int num_kv_heads, int head_dim, int dtype,
                          void* stream);

/*
 * Greedy sampling tail.  mv_argmax_rows reduces each row of a logits matrix
 * (rows, cols), row stride in elements, to one signed 64-bit key: high word =
 * the maximum logit in an integer form whose order is the float order (NaN
 * above +inf, as torch.argmax treats it), low word = 2^32-1 minus
 * (index_offset + column).  The larger key is the larger logit and, between
 * equal logits, the lower index, so vocabulary shards merge by an integer MAX
 * (e.g. an all-reduce of 8 bytes per row) -- mv_argmax_decode takes the
 * largest of `shards` keys per row, keys laid out (shards, rows), and writes
 * the token ids.  keys or tokens of mv_argmax_rows may be NULL; with tokens
 * set the decoded ids of this shard alone are written too (single-GPU path,
 * one launch).  Rows that start on 16-byte boundaries (aligned base, stride a
 * multiple of 8 elements) are read with 16-byte loads, others element-wise.
 * Replaces the gather of full-vocabulary logits to rank 0 and the argmax on
 * them: src/myvllm/layers/embedding_head.py:56-77 (ParallelLMHead.forward)
 * and src/myvllm/layers/sampler.py:15-19 in its greedy limit.
 */
int mv_argmax_rows(const void* logits, int64_t row_stride, int64_t rows,
                   int64_t cols, int64_t index_offset, int64_t* keys,
                   int64_t* tokens, int dtype, void* stream);
int mv_argmax_decode(const int64_t* keys, int shards, int64_t rows,
                     int64_t* tokens, void* stream);

/*
 * Temperature sampling tail, vocabulary-sharded.  Replaces the sampler
 * src/myvllm/layers/sampler.py:15-19 (logits / T, softmax, division by an
 * Exp(1) draw per entry, argmax) and the logits gather in front of it
 * (layers/embedding_head.py:56-77):  argmax_i p_i / E_i equals
 * argmax_i (logit_i / T - log E_i), which needs no softmax normaliser, so
 * every rank reduces its shard to the same 64-bit keys as mv_argmax_rows
 * (score in place of the logit) and the shards merge by integer MAX
 * (mv_argmax_decode).  E_i comes from Philox4x32-10 with key = seed and
 * counter = (global column / 4, row, *step): every rank and every
 * tensor-parallel degree draws the same noise for a given global column.
 * temperatures is (rows) fp32; a row with temperature 0 is greedy.  *step is
 * read on the device (a captured graph can advance it between replays).
 * mv_philox4x32_10 evaluates the generator on the host (for checking).
 */
int mv_sample_rows(const void* logits, int64_t row_stride, int64_t rows,
                   int64_t cols, int64_t index_offset,
                   const float* temperatures, uint64_t seed,
                   const int64_t* step, int64_t* keys, int64_t* tokens,
                   int dtype, void* stream);
int mv_philox4x32_10(uint64_t seed, uint64_t step, uint32_t row,
                     uint32_t column_group, uint32_t* out4);

/*
 * Tensor-parallel all-reduce over NVLink peer memory, fused with the residual
 * add and the RMSNorm that follow it.
 * Replaces: the `dist.all_reduce(result)` that ends every row-parallel linear
 * layer (src/myvllm/layers/linear.py:216-221, after o_proj and down_proj) plus
 * the residual add and RMSNorm each rank then repeats on the full activations
 * (src/myvllm/layers/layernorm.py:10-22, called from models/qwen3.py:187,215).
 *
 * A communicator owns, on every rank, one device allocation holding an INPUT
 * buffer (this rank's partial sums, written by the caller's GEMM), a GATHER
 * buffer (the normalised rows of all ranks, read by the caller's next GEMM)
 * and the barrier flags; peers map each other's allocation through CUDA IPC.
 * Set-up (once, allocates): every rank calls mv_comm_create, the caller
 * exchanges the mv_comm_handle_bytes()-byte handles of all ranks in rank order
 * (any host channel), every rank calls mv_comm_connect, and the caller makes
 * sure every rank has connected before the first launch (a host barrier).
 * `data_bytes` bounds rows*hidden*2 of one call; `timeout_ms` bounds every
 * in-kernel wait.
 *
 * mv_allreduce_residual_rmsnorm, with x_p (rows, hidden) in rank p's input
 * buffer and rank r owning rows [r*ceil(rows/N), min(rows, (r+1)*ceil(rows/N))):
 *   o = round(sum_p x_p[row]) (fp32, p ascending);
 *   residual_shard[row - first owned row] = round(residual_shard[...] + o);
 *   h[row] = round(residual * rsqrt(mean(residual^2) + eps) * gamma)
 * and h[row] is stored into the gather buffer of every rank.  The residual
 * stream stays sharded by rows: residual_shard is (owned rows, hidden) and may
 * be null on a rank that owns no row (rows < world).
 * Every rank must make the same sequence of calls with the same rows/hidden,
 * one call at a time per communicator (calls are ordered by the stream).
 * Launch-only (graph-capturable); peers are read and written with plain loads
 * and stores.  A wait that runs out of time stores a non-zero code in
 * *error_word (caller-owned device int, zero-initialised; 0x100|peer = partial
 * sums never arrived, 0x200|peer = result rows never arrived) and the kernel
 * returns; while the word is non-zero later launches return at once.  After
 * such an error the communicator must be reset on every rank (mv_comm_reset,
 * all ranks idle) before it is used again.
 *
 * mv_comm_create_emulated builds all N ranks on the current device; a call
 * then runs every rank in ONE cooperative launch (residual shard of rank p at
 * residual_shard + p*residual_slot_stride elements; mv_comm_input/output take
 * the rank as `slot`).  It exists to test the protocol on a single GPU (the
 * launch uses at most one block per SM in total).  On a real communicator
 * `slot` is 0 and residual_slot_stride is ignored.
 */
int64_t mv_comm_handle_bytes(void);
int mv_comm_create(int rank, int world, int64_t data_bytes, int timeout_ms,
                   void** comm_out, void* handle_out);
int mv_comm_connect(void* comm, const void* all_handles);
int mv_comm_create_emulated(int world, int64_t data_bytes, int timeout_ms,
                            void** comm_out);
int mv_comm_destroy(void* comm);
int mv_comm_reset(void* comm);
/* Caps the grid of the following mv_allreduce_residual_rmsnorm launches of this communicator (0 = no cap).  A
 * block of that kernel occupies a whole SM; a caller that keeps a second stream busy with GEMMs while a
 * bandwidth-bound call runs leaves them the remaining SMs this way.  Results do not depend on the grid. */
int mv_comm_set_max_blocks(void* comm, int max_blocks);
void* mv_comm_input(void* comm, int slot);
void* mv_comm_output(void* comm, int slot);
int mv_allreduce_residual_rmsnorm(void* comm, void* residual_shard,
                                  int64_t residual_slot_stride,
                                  const void* gamma, float eps, int rows,
                                  int hidden, int* error_word, int dtype,
                                  void* stream);
/* The same step (arguments, result, row ownership, error codes, bounded waits) with the two bulk transfers done
 * by the copy engines: barrier, cudaMemcpyAsync of the peers' partial rows of this rank's shard into staging
 * inside the communicator, one local kernel (the same sums and roundings), cudaMemcpyAsync of the normalised
 * rows to every peer, barrier.  For messages that are bound by the link (a prefill wave): the SMs stay free
 * while the bytes move, so another stream's work runs beside it.  Calls of both forms may follow each other on
 * one communicator. */
int mv_allreduce_residual_rmsnorm_staged(void* comm, void* residual_shard,
                                  int64_t residual_slot_stride,
                                  const void* gamma, float eps, int rows,
                                  int hidden, int* error_word, int dtype,
                                  void* stream);

/*
 * Single-rank form of the same step: for every row,
 *   s = x[row] (+ residual_in[row], rounded, when residual_in is non-null);
 *   out[row] = round(s * rsqrt(mean(s^2) + eps) * gamma);
 * and s is stored to residual_out[row - res_lo] for rows in [res_lo, res_hi)
 * (residual_out may be null; it may alias residual_in when res_lo is 0).
 * Replaces src/myvllm/layers/layernorm.py:10-28 (rms_forward and
 * residual_rms_forward).  x/out/residuals are (rows, hidden) contiguous.
 */
int mv_add_rmsnorm(void* out, const void* x, const void* residual_in,
                   void* residual_out, int64_t res_lo, int64_t res_hi,
                   const void* gamma, float eps, int64_t rows, int hidden,
                   int dtype, void* stream);

/*
 * SwiGLU activation on the fused gate_up projection output (rows, 2*inter),
 * row stride in elements: out[t, j] = silu(gu[t, j]) * gu[t, inter + j],
 * computed in fp32 and rounded once; out is (rows, inter) contiguous.
 * Replaces src/myvllm/layers/activation.py:17-20 (SiluAndMul.forward).
 */
int mv_silu_mul(void* out, const void* gate_up, int64_t gate_up_stride,
                int64_t rows, int inter, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MINIVLLM_B200_H */
