// store_kvcache: slot_mapping scatter of new K/V rows into the paged cache,
// optionally fused with per-token-per-head symmetric int8 quantisation.
//
// Does the work of src/myvllm/layers/attention.py:7-108 of the reference
// (Triton grid of (tokens, kv_heads) programs, one head row each).  Here the
// unit of work is one 16-byte chunk of a token row: a thread moves the K chunk
// and the V chunk of the same position, so a warp moves 512 contiguous bytes of
// K and of V per step, the slot is read once per chunk through L1 (all lanes of
// a row hit one line) and the grid is sized from the SM count.
// HBM-bound: algorithmic bytes per valid token = num_kv_heads*head_dim *
// (2*in_bytes + 2*out_bytes) + 8 (slot) [+ 4*num_kv_heads for the scales].
#include "common.cuh"
#include "quant.cuh"

namespace mv {

constexpr int kStoreThreads = 256;
constexpr int kStoreUnroll = 4;

// Plain copy.  chunks_per_row = num_kv_heads*head_dim*sizeof(T)/16.
__global__ void __launch_bounds__(kStoreThreads)
store_kv_copy_kernel(const uint4* __restrict__ key, const uint4* __restrict__ value,
                     int64_t k_stride16, int64_t v_stride16,  // token strides in 16-byte units
                     uint4* __restrict__ k_cache, uint4* __restrict__ v_cache,
                     const int64_t* __restrict__ slot_mapping,
                     int64_t total_chunks, uint32_t chunks_per_row, int64_t num_slots) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kStoreThreads * kStoreUnroll;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * kStoreThreads * kStoreUnroll + threadIdx.x;
       base < total_chunks; base += stride) {
    uint4 kv[kStoreUnroll], vv[kStoreUnroll];
    int64_t dst[kStoreUnroll];
#pragma unroll
    for (int u = 0; u < kStoreUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * kStoreThreads;
      dst[u] = -1;
      if (i < total_chunks) {
        const int64_t t = i / chunks_per_row;
        const uint32_t c = static_cast<uint32_t>(i - t * chunks_per_row);
        const int64_t slot = __ldg(slot_mapping + t);
        if (slot >= 0 && slot < num_slots) {
          dst[u] = slot * chunks_per_row + c;
          kv[u] = ld_stream16(key + t * k_stride16 + c);
          vv[u] = ld_stream16(value + t * v_stride16 + c);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kStoreUnroll; ++u) {
      if (dst[u] >= 0) {
        st_global16(k_cache + dst[u], kv[u]);
        st_global16(v_cache + dst[u], vv[u]);
      }
    }
  }
}

// Fused scatter + int8 quantisation.  GROUP = head_dim/8 lanes form one head row.
template <typename T, int GROUP>
__global__ void __launch_bounds__(kStoreThreads)
store_kv_quant_kernel(const uint4* __restrict__ key, const uint4* __restrict__ value,
                      int64_t k_stride16, int64_t v_stride16,
                      uint2* __restrict__ k_codes, uint2* __restrict__ v_codes,
                      __half* __restrict__ k_scale, __half* __restrict__ v_scale,
                      const int64_t* __restrict__ slot_mapping,
                      int64_t total_chunks, uint32_t chunks_per_row, int num_kv_heads, int64_t num_slots) {
  // total_chunks is a multiple of GROUP and warps start on multiples of 32, so
  // a head row is never split between live and idle lanes.
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kStoreThreads;
  const int64_t rounds = (total_chunks + stride - 1) / stride;
  int64_t i = static_cast<int64_t>(blockIdx.x) * kStoreThreads + threadIdx.x;
  // (token, chunk within the row) of chunk i, advanced by the stride each round: one division per thread
  int64_t t = i / chunks_per_row;
  uint32_t c = static_cast<uint32_t>(i - t * chunks_per_row);
  const int64_t t_step = stride / chunks_per_row;
  const uint32_t c_step = static_cast<uint32_t>(stride - t_step * chunks_per_row);
  // Software pipeline, one round deep: the loads of round r+1 are issued before round r is quantised, so the
  // per-row dependency chain (maximum -> shuffle -> scale -> reciprocal -> codes) overlaps a load latency
  // instead of following it.
  auto fetch = [&](int64_t idx, int64_t tok, uint32_t chunk, int64_t& slot, bool& live, uint4& kraw, uint4& vraw) {
    live = false;
    slot = -1;
    kraw = make_uint4(0, 0, 0, 0);
    vraw = make_uint4(0, 0, 0, 0);
    if (idx < total_chunks) {
      slot = __ldg(slot_mapping + tok);
      live = slot >= 0 && slot < num_slots;
      if (live) {
        kraw = ld_stream16(key + tok * k_stride16 + chunk);
        vraw = ld_stream16(value + tok * v_stride16 + chunk);
      }
    }
  };
  auto advance = [&]() {
    i += stride;
    t += t_step;
    c += c_step;
    if (c >= chunks_per_row) {
      c -= chunks_per_row;
      ++t;
    }
  };
  int64_t slot, slot_n;
  bool live, live_n;
  uint4 kraw, vraw, kraw_n, vraw_n;
  fetch(i, t, c, slot, live, kraw, vraw);
  for (int64_t r = 0; r < rounds; ++r) {
    const uint32_t c_now = c;
    advance();
    fetch(r + 1 < rounds ? i : total_chunks, t, c, slot_n, live_n, kraw_n, vraw_n);
    uint2 kc, vc;
    __half ks, vs;
    quant_chunk<T, GROUP>(kraw, kc, ks);
    quant_chunk<T, GROUP>(vraw, vc, vs);
    if (live) {
      const int64_t dst = slot * chunks_per_row + c_now;  // 8-byte units of the int8 row
      st_global8(k_codes + dst, kc);
      st_global8(v_codes + dst, vc);
      if ((c_now & (GROUP - 1)) == 0) {
        const int64_t sidx = slot * num_kv_heads + c_now / GROUP;
        k_scale[sidx] = ks;
        v_scale[sidx] = vs;
      }
    }
    slot = slot_n;
    live = live_n;
    kraw = kraw_n;
    vraw = vraw_n;
  }
}

static int grid_for(int64_t work_items, int per_cta) {
  int64_t want = (work_items + per_cta - 1) / per_cta;
  const int64_t cap = static_cast<int64_t>(kNumSMs) * 8;  // 8 resident 256-thread CTAs per SM
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return static_cast<int>(want);
}

template <typename T>
static int launch_quant(const void* key, const void* value, int64_t ks16, int64_t vs16, void* k_cache, void* v_cache,
                        void* k_scale, void* v_scale, const int64_t* slot_mapping, int64_t total,
                        uint32_t chunks_per_row, int kvh, int head_dim, int64_t num_slots, cudaStream_t st) {
  const int grid = grid_for(total, kStoreThreads);
#define MV_LAUNCH_Q(G)                                                                                      \
  store_kv_quant_kernel<T, G><<<grid, kStoreThreads, 0, st>>>(                                              \
      static_cast<const uint4*>(key), static_cast<const uint4*>(value), ks16, vs16,                         \
      static_cast<uint2*>(k_cache), static_cast<uint2*>(v_cache), static_cast<__half*>(k_scale),            \
      static_cast<__half*>(v_scale), slot_mapping, total, chunks_per_row, kvh, num_slots)
  switch (head_dim) {
    case 64: MV_LAUNCH_Q(8); break;
    case 128: MV_LAUNCH_Q(16); break;
    case 256: MV_LAUNCH_Q(32); break;
    default: return fail(MV_ERR_SHAPE, "store_kvcache int8: head_dim %d not in {64,128,256}", head_dim);
  }
#undef MV_LAUNCH_Q
  return check_launch("store_kv_quant_kernel");
}

}  // namespace mv

extern "C" int mv_store_kvcache(const void* key, const void* value, int64_t k_stride_tok, int64_t v_stride_tok,
                                void* k_cache, void* v_cache, void* k_scale, void* v_scale,
                                const int64_t* slot_mapping, int64_t num_tokens, int64_t num_slots,
                                int num_kv_heads, int head_dim, int dtype, void* stream) {
  using namespace mv;
  if (dtype != MV_F16 && dtype != MV_BF16) return fail(MV_ERR_DTYPE, "store_kvcache: dtype %d", dtype);
  if (num_tokens < 0 || num_slots < 0 || num_kv_heads <= 0 || head_dim <= 0)
    return fail(MV_ERR_SHAPE, "store_kvcache: negative or zero size");
  if (head_dim % 8 != 0) return fail(MV_ERR_SHAPE, "store_kvcache: head_dim %d is not a multiple of 8", head_dim);
  if (num_tokens == 0) return MV_OK;
  if (!key || !value || !k_cache || !v_cache || !slot_mapping) return fail(MV_ERR_NULL, "store_kvcache: null pointer");
  if ((k_scale == nullptr) != (v_scale == nullptr))
    return fail(MV_ERR_NULL, "store_kvcache: k_scale and v_scale must both be set or both be null");
  const int64_t row_elems = static_cast<int64_t>(num_kv_heads) * head_dim;
  if (k_stride_tok < row_elems || v_stride_tok < row_elems)
    return fail(MV_ERR_SHAPE, "store_kvcache: token stride smaller than a row");
  if (k_stride_tok % 8 != 0 || v_stride_tok % 8 != 0 || !aligned16(key) || !aligned16(value) ||
      !aligned16(k_cache) || !aligned16(v_cache))
    return fail(MV_ERR_ALIGN, "store_kvcache: pointers and token strides must be 16-byte aligned");
  const uint32_t chunks_per_row = static_cast<uint32_t>(row_elems / 8);  // 16-byte chunks of 2-byte elements
  const int64_t total = num_tokens * chunks_per_row;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (k_scale) {
    if (dtype == MV_F16)
      return launch_quant<__half>(key, value, k_stride_tok / 8, v_stride_tok / 8, k_cache, v_cache, k_scale, v_scale,
                                  slot_mapping, total, chunks_per_row, num_kv_heads, head_dim, num_slots, st);
    return launch_quant<__nv_bfloat16>(key, value, k_stride_tok / 8, v_stride_tok / 8, k_cache, v_cache, k_scale,
                                       v_scale, slot_mapping, total, chunks_per_row, num_kv_heads, head_dim,
                                       num_slots, st);
  }
  const int grid = grid_for(total, kStoreThreads * kStoreUnroll);
  store_kv_copy_kernel<<<grid, kStoreThreads, 0, st>>>(
      static_cast<const uint4*>(key), static_cast<const uint4*>(value), k_stride_tok / 8, v_stride_tok / 8,
      static_cast<uint4*>(k_cache), static_cast<uint4*>(v_cache), slot_mapping, total, chunks_per_row, num_slots);
  return check_launch("store_kv_copy_kernel");
}
