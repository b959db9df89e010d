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
constexpr int kDecCtasPerSM = 2;
constexpr int kDecWaves = 1;                    // work units per resident CTA: units are equal in length, so one each
                                                // is balanced; 2 and 4 measured slower (more pieces to merge)
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
  int2* binfo;      // per sequence: (first item, number of items); read by the separate combine kernel only
  unsigned* arrivals;  // per (sequence, KV head, row tile): pieces of a split sequence that have been written;
                       // zero between launches.  Null when the problem has more such cells than the scratch
                       // reserves: the pieces are then reduced by the separate combine kernel.
  float* part_ml;   // (item, head, 2)
  float* part_o;    // (item, head, D)
};

// Segments of the token stream per (KV head, row tile): every resident CTA gets
// kDecWaves units.  Shapes only, so host and device agree.
__host__ __device__ inline int decode_target_items(int num_kv_heads, int mtiles) {
  const int t = (kNumSMs * kDecCtasPerSM * kDecWaves) / (num_kv_heads * mtiles);
  return t < 1 ? 1 : t;
}
// Upper bound of the item ids: an item id is (sequence index + segment index) and there are at most
// target_items segments, so ids stay below batch + target_items whatever the context lengths are.
__host__ __device__ inline int64_t decode_items_max(int batch, int num_kv_heads, int mtiles) {
  return static_cast<int64_t>(decode_target_items(num_kv_heads, mtiles)) + batch;
}

__device__ __forceinline__ int load_ctx(const DecodeParams& p, int b) {
  long long c = p.ctx_is_i64 ? static_cast<const long long*>(p.context_lens)[b]
                             : static_cast<long long>(static_cast<const int*>(p.context_lens)[b]);
  const long long lim = static_cast<long long>(p.max_blocks) * p.block_size;
  c = c < 0 ? 0 : (c > lim ? lim : c);
  return static_cast<int>(c);
}

// ---- the work plan --------------------------------------------------------------------------------
// The tokens of all sequences form one stream (sequence after sequence).  It is cut into `n_seg`
// segments of equal length `seg_len`; a work UNIT is (segment, KV head, row tile) and a CTA takes whole
// units, so every CTA streams the same number of tokens whatever the mix of context lengths.  Inside a
// unit the work ITEMS are the pieces of sequences that the segment covers: item id = sequence index +
// segment index, which is unique, increases along the stream, and is contiguous per sequence (a sequence
// that spans segments s0..s1 owns ids b+s0 .. b+s1: its partial results, merged by the combine kernel).
// Every CTA builds the same plan: s_tok[b] = tokens before sequence b, s_tok[batch] = all tokens.
struct DecodePlan {
  int seg_len, n_seg;
};
__device__ inline DecodePlan build_plan(const DecodeParams& p, int* s_tok, long long* s_red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int carry = 0;
  if (tid == 0) s_tok[0] = 0;
  for (int base = 0; base < p.batch; base += kDecThreads) {
    const int b = base + tid;
    const int n = b < p.batch ? load_ctx(p, b) : 0;
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
    if (b < p.batch) s_tok[b + 1] = carry + wofs + incl;
    carry += tot;
    __syncthreads();
  }
  const int total = carry;
  DecodePlan plan;
  int seg = (total + p.target_items - 1) / p.target_items;
  seg = ((seg + kCtaTok - 1) / kCtaTok) * kCtaTok;
  if (seg < kCtaTok) seg = kCtaTok;
  plan.seg_len = seg;
  plan.n_seg = (total + seg - 1) / seg;   // <= target_items
  return plan;
}

// (first item id, number of items) of sequence b; an empty sequence has none.
__device__ __forceinline__ int2 seq_items(const int* s_tok, const DecodePlan& plan, int b) {
  const int t0 = s_tok[b], t1 = s_tok[b + 1];
  if (t1 <= t0) return make_int2(0, 0);
  const int s0 = t0 / plan.seg_len, s1 = (t1 - 1) / plan.seg_len;
  return make_int2(b + s0, s1 - s0 + 1);
}

// The sequence whose tokens include stream position `pos` (pos < total): the last b with s_tok[b] <= pos
// (empty sequences share their successor's prefix and are skipped by "last").
__device__ __forceinline__ int seq_at(const DecodeParams& p, const int* s_tok, int pos) {
  int lo = 0, hi = p.batch - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (s_tok[mid] <= pos) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// One piece of a sequence inside a segment.
struct DecodeItem {
  int b, nsplit, tok_begin, tok_end, item;
};
__device__ __forceinline__ DecodeItem piece_of(const int* s_tok, const DecodePlan& plan, int b, int seg) {
  const int t0 = s_tok[b], t1 = s_tok[b + 1];
  const int g0 = seg * plan.seg_len, g1 = g0 + plan.seg_len;
  DecodeItem it;
  it.b = b;
  it.item = b + seg;
  it.tok_begin = max(g0 - t0, 0);
  it.tok_end = min(g1, t1) - t0;
  it.nsplit = (t1 - 1) / plan.seg_len - t0 / plan.seg_len + 1;
  return it;
}

// Walks the items of the units u = first, first + stride, ... in order.
struct ItemWalk {
  long long unit;
  int seg, y, b;      // b < 0: finished
};
__device__ __forceinline__ void walk_enter_unit(const DecodeParams& p, const int* s_tok, const DecodePlan& plan,
                                                int ydim, long long n_units, ItemWalk& w) {
  if (w.unit >= n_units) { w.b = -1; return; }
  w.seg = static_cast<int>(w.unit / ydim);
  w.y = static_cast<int>(w.unit - static_cast<long long>(w.seg) * ydim);
  w.b = seq_at(p, s_tok, w.seg * plan.seg_len);
}
__device__ __forceinline__ void walk_start(const DecodeParams& p, const int* s_tok, const DecodePlan& plan, int ydim,
                                           long long n_units, long long first, ItemWalk& w) {
  w.unit = first;
  walk_enter_unit(p, s_tok, plan, ydim, n_units, w);
}
__device__ __forceinline__ void walk_next(const DecodeParams& p, const int* s_tok, const DecodePlan& plan, int ydim,
                                          long long n_units, long long stride, ItemWalk& w) {
  const int seg_end = (w.seg + 1) * plan.seg_len;
  int b = w.b + 1;
  while (b < p.batch && s_tok[b + 1] == s_tok[b]) ++b;   // empty sequences own no tokens
  if (b < p.batch && s_tok[b] < seg_end) { w.b = b; return; }
  w.unit += stride;
  walk_enter_unit(p, s_tok, plan, ydim, n_units, w);
}

// Rows of sequences without any token: nobody's item covers them, the CTAs share out writing their zeros.
template <typename T, int D>
__device__ __forceinline__ void zero_empty_sequences(const DecodeParams& p, const int* s_tok) {
  for (int b = blockIdx.x; b < p.batch; b += gridDim.x) {
    if (s_tok[b + 1] != s_tok[b]) continue;
    T* row = static_cast<T*>(p.out) + static_cast<int64_t>(b) * p.num_heads * D;
    for (int i = threadIdx.x; i < p.num_heads * D; i += kDecThreads) row[i] = Elem<T>::from_f(0.f);
  }
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

// A sequence that spans segments leaves one partial result per piece.  The CTA that writes the LAST piece of a
// (sequence, KV head, row tile) reduces them all, in item order (so the result does not depend on which CTA
// that was), and writes the output rows: no second launch, and no CTA ever waits for another.  Called by the
// whole CTA after merge_and_write and a __syncthreads().  `s_last` is one int of shared memory.
constexpr int kDecodeArrivalCells = 16384;                       // 64 KiB of counters at the start of the scratch
template <typename T, int D>
__device__ __forceinline__ void combine_if_last(const DecodeParams& p, const int* s_tok, const DecodePlan& plan, int b,
                                                int cell, int h0, int rows_valid, int nsplit, int* s_last) {
  if (p.arrivals == nullptr || nsplit <= 1) return;             // uniform over the CTA
  if (threadIdx.x == 0) {
    __threadfence();                                              // this CTA's partial rows (ordered by the barrier)
    const bool last = atomicAdd(&p.arrivals[cell], 1u) == static_cast<unsigned>(nsplit - 1);
    if (last) {
      __threadfence();                                            // ... and those of the CTAs counted before it
      p.arrivals[cell] = 0;                                       // zero again for the next launch
    }
    *s_last = last;
  }
  __syncthreads();
  if (*s_last) {
    const int2 info = seq_items(s_tok, plan, b);
    for (int idx = threadIdx.x; idx < rows_valid * D; idx += kDecThreads) {
      const int h = h0 + idx / D, d = idx % D;
      float M = kNegBig;
      for (int s = 0; s < info.y; ++s)
        M = fmaxf(M, __ldcg(p.part_ml + (static_cast<int64_t>(info.x + s) * p.num_heads + h) * 2));
      float acc = 0.f, L = 0.f;
      for (int s = 0; s < info.y; ++s) {
        const int64_t pi = static_cast<int64_t>(info.x + s) * p.num_heads + h;
        const float wgt = fast_exp2(__ldcg(p.part_ml + pi * 2) - M);
        acc += wgt * __ldcg(p.part_o + pi * D + d);
        L += wgt * __ldcg(p.part_ml + pi * 2 + 1);
      }
      const float r = L > 0.f ? acc / L : 0.f;
      static_cast<T*>(p.out)[(static_cast<int64_t>(b) * p.num_heads + h) * D + d] = Elem<T>::from_f(r);
    }
  }
  __syncthreads();                                                // s_last is reused by the next item
}

// Launch of the int8-cache kernel (paged_decode_int8.cu); head_dim 128 only.
template <typename T> int launch_decode_int8(const DecodeParams& p, cudaStream_t st);
// Grid of the persistent decode kernels.
inline int decode_grid(const DecodeParams& p) {
  const int64_t items_max = decode_items_max(p.batch, p.num_kv_heads, p.mtiles);
  int64_t grid = items_max * p.num_kv_heads * p.mtiles;
  const int64_t resident = static_cast<int64_t>(kNumSMs) * kDecCtasPerSM;
  return static_cast<int>(grid > resident ? resident : grid);
}

}  // namespace mv
