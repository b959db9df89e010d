// Per-step attention metadata built on the GPU from persistent device state.
//
// The reference rebuilds everything on the host each step with Python loops and
// ships it through five pinned copies (src/myvllm/engine/model_runner.py:180-256),
// then rebuilds `positions` on the host again in every decoder layer with a
// device->host sync (src/myvllm/models/qwen3.py:196-212).  Here the block
// tables, the per-sequence lengths and the last sampled token live in device
// memory for the lifetime of a sequence ("slot" = row of that state), the host
// sends only the slot ids of the step (and, for prefill, the prompt lengths),
// and one kernel writes every tensor the step needs, once, for all layers.
// Launch-bound index arithmetic: no roofline, microseconds.
#include "common.cuh"

namespace mv {

constexpr int kMetaThreads = 256;

// ------------------------------------------------------------------ decode ---
// For row b < n_active (slot s = seq_slots[b]):
//   position p      = seq_len_state[s]            (tokens already in the cache)
//   input_ids[b]    = last_token_state[s]
//   positions[b]    = p
//   context_lens[b] = p + 1                        (includes the token being fed)
//   slot_mapping[b] = table[s][p / bs] * bs + p % bs
//   block_tables_out[b][:] = table[s][:]
//   seq_len_state[s] = p + 1
// Rows b >= n_active (padding of a captured graph batch) get input 0,
// position 0, context 0, slot -1 and a table of -1.
// Same results as prepare_decode (model_runner.py:231-256) with the reference's
// last_block_num_tokens defect fixed (a full last block counts block_size tokens).
__global__ void __launch_bounds__(kMetaThreads)
build_decode_meta_kernel(const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ n_active_ptr,
                         int batch_padded, const int32_t* __restrict__ tables, int64_t tables_stride, int max_blocks,
                         int block_size, int32_t* __restrict__ seq_len_state,
                         const int64_t* __restrict__ last_token_state, int64_t* __restrict__ input_ids,
                         int64_t* __restrict__ positions, int64_t* __restrict__ slot_mapping,
                         int64_t* __restrict__ context_lens, int32_t* __restrict__ tables_out, int64_t out_stride) {
  const int n_active = min(*n_active_ptr, batch_padded);
  // one warp per row: lane 0 does the scalars, all lanes copy the table row
  const int warps_per_cta = kMetaThreads / 32;
  const int lane = threadIdx.x & 31;
  for (int b = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); b < batch_padded; b += gridDim.x * warps_per_cta) {
    int32_t* trow_out = tables_out + static_cast<int64_t>(b) * out_stride;
    if (b < n_active) {
      const int s = seq_slots[b];
      const int32_t* trow = tables + static_cast<int64_t>(s) * tables_stride;
      const int p = seq_len_state[s];
      for (int j = lane; j < max_blocks; j += 32) trow_out[j] = trow[j];
      __syncwarp();  // every lane has read seq_len_state before lane 0 bumps it
      if (lane == 0) {
        const int blk = p / block_size;
        const int32_t phys = blk < max_blocks ? trow[blk] : -1;
        input_ids[b] = last_token_state[s];
        positions[b] = p;
        context_lens[b] = static_cast<int64_t>(p) + 1;
        slot_mapping[b] = phys >= 0 ? static_cast<int64_t>(phys) * block_size + (p - blk * block_size) : -1;
        seq_len_state[s] = p + 1;
      }
    } else {
      for (int j = lane; j < max_blocks; j += 32) trow_out[j] = -1;
      if (lane == 0) {
        input_ids[b] = 0;
        positions[b] = 0;
        context_lens[b] = 0;
        slot_mapping[b] = -1;
      }
    }
  }
}

// ----------------------------------------------------------------- prefill ---
// Sequence i (slot s = seq_slots[i]) contributes q_i = seq_lens[i] - num_cached[i]
// tokens at positions num_cached[i] .. seq_lens[i]-1.  One CTA:
//   cu_seqlens_q / cu_seqlens_k : prefix sums of q_i / seq_lens[i]      (int32)
//   last_token_index[i]         : cu_seqlens_q[i+1] - 1                 (int64)
//   seq_len_state[s]            : seq_lens[i]
// then all CTAs, token t of sequence i at position p:
//   positions[t] = p;  slot_mapping[t] = table[s][p / bs] * bs + p % bs
// Same results as prepare_prefill (model_runner.py:180-227) plus the positions
// that qwen3.py:199-206 recomputes per layer.
__global__ void __launch_bounds__(kMetaThreads)
build_prefill_cu_kernel(const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_lens,
                        const int32_t* __restrict__ num_cached, int num_seqs, int32_t* __restrict__ cu_q,
                        int32_t* __restrict__ cu_k, int64_t* __restrict__ last_token_index,
                        int32_t* __restrict__ seq_len_state) {
  __shared__ int s_q[kMetaThreads / 32], s_k[kMetaThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int carry_q = 0, carry_k = 0;
  if (threadIdx.x == 0) { cu_q[0] = 0; cu_k[0] = 0; }
  for (int base = 0; base < num_seqs; base += kMetaThreads) {
    const int i = base + threadIdx.x;
    int lq = 0, lk = 0;
    if (i < num_seqs) {
      lk = seq_lens[i];
      lq = lk - (num_cached ? num_cached[i] : 0);
      seq_len_state[seq_slots[i]] = lk;
    }
    int iq = lq, ik = lk;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int vq = __shfl_up_sync(0xffffffffu, iq, off), vk = __shfl_up_sync(0xffffffffu, ik, off);
      if (lane >= off) { iq += vq; ik += vk; }
    }
    if (lane == 31) { s_q[warp] = iq; s_k[warp] = ik; }
    __syncthreads();
    int oq = 0, ok = 0, tq = 0, tk = 0;
#pragma unroll
    for (int w = 0; w < kMetaThreads / 32; ++w) {
      if (w < warp) { oq += s_q[w]; ok += s_k[w]; }
      tq += s_q[w]; tk += s_k[w];
    }
    if (i < num_seqs) {
      cu_q[i + 1] = carry_q + oq + iq;
      cu_k[i + 1] = carry_k + ok + ik;
      last_token_index[i] = static_cast<int64_t>(carry_q + oq + iq) - 1;
    }
    carry_q += tq; carry_k += tk;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kMetaThreads)
build_prefill_tokens_kernel(const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ seq_lens,
                            const int32_t* __restrict__ num_cached, int num_seqs, const int32_t* __restrict__ cu_q,
                            const int32_t* __restrict__ tables, int64_t tables_stride, int max_blocks, int block_size,
                            int64_t* __restrict__ positions, int64_t* __restrict__ slot_mapping, int64_t capacity) {
  // grid.y = sequence, grid.x strides over its tokens
  for (int i = blockIdx.y; i < num_seqs; i += gridDim.y) {
    const int start = cu_q[i], n = cu_q[i + 1] - start;
    const int cached = num_cached ? num_cached[i] : 0;
    const int32_t* trow = tables + static_cast<int64_t>(seq_slots[i]) * tables_stride;
    for (int j = blockIdx.x * kMetaThreads + threadIdx.x; j < n; j += gridDim.x * kMetaThreads) {
      const int64_t t = static_cast<int64_t>(start) + j;
      if (t >= capacity) continue;  // the host sized the outputs from the same lengths; never expected
      const int p = cached + j;
      const int blk = p / block_size;
      const int32_t phys = blk < max_blocks ? trow[blk] : -1;
      positions[t] = p;
      slot_mapping[t] = phys >= 0 ? static_cast<int64_t>(phys) * block_size + (p - blk * block_size) : -1;
    }
  }
}

// Scatter of block-table updates: table[slot[u]][index[u]] = block[u].
__global__ void __launch_bounds__(kMetaThreads)
update_tables_kernel(const int32_t* __restrict__ upd, int num_updates, int32_t* __restrict__ tables,
                     int64_t tables_stride, int max_blocks, int num_slots) {
  for (int u = blockIdx.x * kMetaThreads + threadIdx.x; u < num_updates; u += gridDim.x * kMetaThreads) {
    const int slot = upd[3 * u], idx = upd[3 * u + 1], blk = upd[3 * u + 2];
    if (slot >= 0 && slot < num_slots && idx >= 0 && idx < max_blocks)
      tables[static_cast<int64_t>(slot) * tables_stride + idx] = blk;
  }
}

}  // namespace mv

extern "C" int mv_build_decode_meta(const int32_t* seq_slots, const int32_t* n_active, int batch_padded,
                                    const int32_t* tables, int64_t tables_stride, int max_blocks, int block_size,
                                    int32_t* seq_len_state, const int64_t* last_token_state, int64_t* input_ids,
                                    int64_t* positions, int64_t* slot_mapping, int64_t* context_lens,
                                    int32_t* tables_out, int64_t out_stride, void* stream) {
  using namespace mv;
  if (batch_padded < 0 || max_blocks < 0 || block_size <= 0) return fail(MV_ERR_SHAPE, "build_decode_meta: bad size");
  if (batch_padded == 0) return MV_OK;
  if (!seq_slots || !n_active || !tables || !seq_len_state || !last_token_state || !input_ids || !positions ||
      !slot_mapping || !context_lens || !tables_out)
    return fail(MV_ERR_NULL, "build_decode_meta: null pointer");
  if (tables_stride < max_blocks || out_stride < max_blocks)
    return fail(MV_ERR_SHAPE, "build_decode_meta: table stride smaller than its width");
  const int warps = kMetaThreads / 32;
  int grid = (batch_padded + warps - 1) / warps;
  if (grid > kNumSMs * 4) grid = kNumSMs * 4;
  build_decode_meta_kernel<<<grid, kMetaThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      seq_slots, n_active, batch_padded, tables, tables_stride, max_blocks, block_size, seq_len_state,
      last_token_state, input_ids, positions, slot_mapping, context_lens, tables_out, out_stride);
  return check_launch("build_decode_meta_kernel");
}

extern "C" int mv_build_prefill_meta(const int32_t* seq_slots, const int32_t* seq_lens, const int32_t* num_cached,
                                     int num_seqs, int64_t total_tokens, const int32_t* tables, int64_t tables_stride,
                                     int max_blocks, int block_size, int32_t* seq_len_state, int32_t* cu_seqlens_q,
                                     int32_t* cu_seqlens_k, int64_t* positions, int64_t* slot_mapping,
                                     int64_t* last_token_index, void* stream) {
  using namespace mv;
  if (num_seqs < 0 || total_tokens < 0 || max_blocks < 0 || block_size <= 0)
    return fail(MV_ERR_SHAPE, "build_prefill_meta: bad size");
  if (num_seqs == 0) return MV_OK;
  if (!seq_slots || !seq_lens || !tables || !seq_len_state || !cu_seqlens_q || !cu_seqlens_k || !positions ||
      !slot_mapping || !last_token_index)
    return fail(MV_ERR_NULL, "build_prefill_meta: null pointer");
  if (tables_stride < max_blocks) return fail(MV_ERR_SHAPE, "build_prefill_meta: table stride smaller than its width");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  build_prefill_cu_kernel<<<1, kMetaThreads, 0, st>>>(seq_slots, seq_lens, num_cached, num_seqs, cu_seqlens_q,
                                                      cu_seqlens_k, last_token_index, seq_len_state);
  int rc = check_launch("build_prefill_cu_kernel");
  if (rc) return rc;
  if (total_tokens == 0) return MV_OK;
  int gx = static_cast<int>((total_tokens / num_seqs + kMetaThreads - 1) / kMetaThreads);
  gx = gx < 1 ? 1 : (gx > 64 ? 64 : gx);
  const int gy = num_seqs > 65535 ? 65535 : num_seqs;
  build_prefill_tokens_kernel<<<dim3(gx, gy), kMetaThreads, 0, st>>>(seq_slots, seq_lens, num_cached, num_seqs,
                                                                    cu_seqlens_q, tables, tables_stride, max_blocks,
                                                                    block_size, positions, slot_mapping, total_tokens);
  return check_launch("build_prefill_tokens_kernel");
}

extern "C" int mv_update_block_tables(const int32_t* updates, int num_updates, int32_t* tables, int64_t tables_stride,
                                      int max_blocks, int num_slots, void* stream) {
  using namespace mv;
  if (num_updates < 0 || max_blocks < 0 || num_slots < 0) return fail(MV_ERR_SHAPE, "update_block_tables: bad size");
  if (num_updates == 0) return MV_OK;
  if (!updates || !tables) return fail(MV_ERR_NULL, "update_block_tables: null pointer");
  int grid = (num_updates + kMetaThreads - 1) / kMetaThreads;
  if (grid > kNumSMs) grid = kNumSMs;
  update_tables_kernel<<<grid, kMetaThreads, 0, static_cast<cudaStream_t>(stream)>>>(updates, num_updates, tables,
                                                                                    tables_stride, max_blocks,
                                                                                    num_slots);
  return check_launch("update_tables_kernel");
}
