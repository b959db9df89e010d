// Pieces shared by the fp16/bf16 and the int8 paged-decode kernels: launch
// parameters, the on-device work plan, item lookup and the cross-warp merge.
#pragma once
#include "common.cuh"
#include "mma.cuh"
#include <type_traits>

namespace mv {

constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kDecStages = 3;
constexpr int kTileTok = 16;                    // tokens per warp tile
constexpr int kCtaTok = kTileTok * kDecWarps;   // tokens per CTA step
constexpr int kChunkMax = 2048;                 // longest KV chunk of one work item
constexpr int kDecCtasPerSM = 2;
constexpr int kDecWaves = 2;                    // work items aimed at per resident CTA; 4, 8 and 16 measured slower
                                                // on most shapes (merge, partial results and combine pass per item)
constexpr float kNegBig = -1e30f;               // finite "minus infinity" for running maxima

struct DecodeParams {
  void* out;
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const __half* k_scale;   // int8 caches only: (slots, kv_heads) fp16
  const __half* v_scale;
  const int32_t* block_tables;
  int64_t bt_stride;
  int max_blocks;
  const void* context_lens;
  int ctx_is_i64;
  int batch, num_heads, num_kv_heads, group, mtiles;
  int block_size;
  int64_t num_blocks;
  float scale_log2;
  int target_items;
  int2* binfo;      // per sequence: (first item, number of items)
  float* part_ml;   // (item, head, 2)
  float* part_o;    // (item, head, D)
};

// Work items aimed at per (KV head, row tile): enough to give every resident
// CTA kDecWaves items.  Shapes only, so host and device agree.
__host__ __device__ inline int decode_target_items(int num_kv_heads, int mtiles) {
  const int t = (kNumSMs * kDecCtasPerSM * kDecWaves) / (num_kv_heads * mtiles);
  return t < 1 ? 1 : t;
}
__host__ __device__ inline int64_t decode_items_max(int batch, int num_kv_heads, int mtiles, int max_blocks,
                                                    int block_size) {
  const int64_t lmax = static_cast<int64_t>(max_blocks) * block_size;
  int64_t per_seq = (lmax + kChunkMax - 1) / kChunkMax;
  if (per_seq < 1) per_seq = 1;
  return decode_target_items(num_kv_heads, mtiles) + static_cast<int64_t>(batch) * per_seq;
}

__device__ __forceinline__ int load_ctx(const DecodeParams& p, int b) {
  long long c = p.ctx_is_i64 ? static_cast<const long long*>(p.context_lens)[b]
                             : static_cast<long long>(static_cast<const int*>(p.context_lens)[b]);
  const long long lim = static_cast<long long>(p.max_blocks) * p.block_size;
  c = c < 0 ? 0 : (c > lim ? lim : c);
  return static_cast<int>(c);
}

// Every CTA builds the same plan: chunk length and s_start[b] = first item of
// sequence b (s_start[batch] = number of items).  Returns the chunk length.
__device__ inline int build_plan(const DecodeParams& p, int* s_start, long long* s_red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  long long sum = 0;
  for (int b = tid; b < p.batch; b += kDecThreads) sum += load_ctx(p, b);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if (lane == 0) s_red[warp] = sum;
  __syncthreads();
  long long total = 0;
#pragma unroll
  for (int w = 0; w < kDecWarps; ++w) total += s_red[w];
  long long chunk = (total + p.target_items - 1) / p.target_items;
  chunk = ((chunk + kCtaTok - 1) / kCtaTok) * kCtaTok;
  if (chunk < kCtaTok) chunk = kCtaTok;
  if (chunk > kChunkMax) chunk = kChunkMax;
  const int ch = static_cast<int>(chunk);
  __syncthreads();  // s_red is reused below

  int carry = 0;
  if (tid == 0) s_start[0] = 0;
  for (int base = 0; base < p.batch; base += kDecThreads) {
    const int b = base + tid;
    int n = 0;
    if (b < p.batch) {
      n = (load_ctx(p, b) + ch - 1) / ch;
      if (n < 1) n = 1;  // an empty sequence still owns one item, which writes zeros
    }
    int incl = n;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) s_red[warp] = incl;
    __syncthreads();
    int wofs = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const int v = static_cast<int>(s_red[w]);
      if (w < warp) wofs += v;
      tot += v;
    }
    if (b < p.batch) s_start[b + 1] = carry + wofs + incl;
    carry += tot;
    __syncthreads();
  }
  return ch;
}


// Which (sequence, chunk) a work item is, from the plan in shared memory.
struct DecodeItem {
  int b, nsplit, tok_begin, tok_end;
};
__device__ __forceinline__ DecodeItem find_item(const DecodeParams& p, const int* s_start, int item, int chunk) {
  int lo = 0, hi = p.batch - 1;
  while (lo < hi) {  // last b with s_start[b] <= item
    const int mid = (lo + hi + 1) >> 1;
    if (s_start[mid] <= item) lo = mid; else hi = mid - 1;
  }
  DecodeItem it;
  it.b = lo;
  it.nsplit = s_start[lo + 1] - s_start[lo];
  // The sequence's tokens are spread evenly over its items (in whole CTA steps) instead of full chunks plus a
  // short remainder: CTAs take items in a fixed stride, so items of similar length mean a similar load.
  const int ctx = load_ctx(p, lo);
  int per = (ctx + it.nsplit - 1) / it.nsplit;
  per = ((per + kCtaTok - 1) / kCtaTok) * kCtaTok;   // <= chunk, which is a multiple of kCtaTok
  it.tok_begin = (item - s_start[lo]) * per;
  it.tok_end = min(ctx, it.tok_begin + per);
  return it;
}

// After every warp wrote its unnormalised O rows (sO, row stride `stride`
// floats) and its (m, l) pairs (sML) to shared memory: combine the warps and
// write either the final output (sequence not split) or the partial result.
// A warp's rows sit at (warp * rpw + row): rpw = 16 (the whole MMA tile) or fewer when only the first rows exist.
template <typename T, int D>
__device__ __forceinline__ void merge_and_write(const DecodeParams& p, const float* sO, const float* sML, int stride,
                                                int rows_valid, int h0, int b, int item, int nsplit, int rpw = 16) {
  for (int idx = threadIdx.x; idx < rows_valid * D; idx += kDecThreads) {
    const int row = idx / D, d = idx - row * D;
    float M = kNegBig;
#pragma unroll
    for (int ww = 0; ww < kDecWarps; ++ww) M = fmaxf(M, sML[(ww * rpw + row) * 2]);
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int ww = 0; ww < kDecWarps; ++ww) {
      const float wgt = fast_exp2(sML[(ww * rpw + row) * 2] - M);
      acc += wgt * sO[(ww * rpw + row) * stride + d];
      L += wgt * sML[(ww * rpw + row) * 2 + 1];
    }
    const int h = h0 + row;
    if (nsplit == 1) {
      const float r = L > 0.f ? acc / L : 0.f;
      static_cast<T*>(p.out)[(static_cast<int64_t>(b) * p.num_heads + h) * D + d] = Elem<T>::from_f(r);
    } else {
      const int64_t pi = static_cast<int64_t>(item) * p.num_heads + h;
      p.part_o[pi * D + d] = acc;
      if (d == 0) { p.part_ml[pi * 2] = M; p.part_ml[pi * 2 + 1] = L; }
    }
  }
}

// Launch of the int8-cache kernel (paged_decode_int8.cu); head_dim 128 only.
template <typename T> int launch_decode_int8(const DecodeParams& p, cudaStream_t st);
// Grid of the persistent decode kernels.
inline int decode_grid(const DecodeParams& p) {
  const int64_t items_max = decode_items_max(p.batch, p.num_kv_heads, p.mtiles, p.max_blocks, p.block_size);
  int64_t grid = items_max * p.num_kv_heads * p.mtiles;
  const int64_t resident = static_cast<int64_t>(kNumSMs) * kDecCtasPerSM;
  return static_cast<int>(grid > resident ? resident : grid);
}

}  // namespace mv
