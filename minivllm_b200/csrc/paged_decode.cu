// Paged decode attention: one query token per sequence against a paged KV
// cache, split over the KV length, sharing each KV read between the query
// heads of a GQA group.
//
// Does the work of src/myvllm/layers/attention.py:283-473 of the reference
// (one Triton program per (sequence, query head), scalar per-token loops, no
// split, KV re-read per query head).  Design here:
//   * the tokens of all sequences form one stream that is cut into segments of
//     equal length; a work unit is (segment, KV head) and every resident CTA
//     takes one, so each CTA streams the same number of bytes whatever the mix
//     of context lengths ("stream-K" over the KV tokens).  The pieces of
//     sequences inside a segment are the work items; a sequence that spans
//     segments leaves partial results.  The segment length is chosen on the
//     device from sum(context_lens); the grid is persistent and depends on
//     shapes only (graph-capturable).  Every CTA recomputes the same plan.
//   * a CTA is 4 independent warps.  Each warp streams its own 16-token tiles
//     of K and V through a private cp.async ring in shared memory (XOR-swizzled
//     16-byte chunks, conflict-free for ldmatrix), so the main loop has no
//     block-wide barrier and ~64 KB per CTA is in flight.
//   * the G query heads of the KV head are the (zero-padded) 16 rows of an
//     m16n8k16 MMA: S = Q K^T and O += P V run on the tensor cores with fp32
//     accumulation, softmax statistics in fp32 registers, exp2 domain.
//   * warps merge through shared memory; a sequence with one piece writes its
//     output directly, otherwise partial (m, l, O) go to the caller's scratch and
//     the CTA that writes the last piece of a (sequence, KV head) reduces them in
//     item order (an arrival counter per cell; nobody waits).  Only when a
//     problem has more cells than the scratch reserves counters for does a
//     separate small combine kernel do that.
// HBM-bound: algorithmic bytes = sum(ctx) * num_kv_heads * head_dim * 2 *
// sizeof(elem) + q and out.
#include "paged_decode.cuh"

namespace mv {

template <typename T, int D>
struct DecodeSmem {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTileBytes = kTileTok * kRowBytes;          // one K or V tile
  static constexpr int kStageBytes = 2 * kTileBytes;               // K then V
  static constexpr int kWarpBytes = kDecStages * kStageBytes;
  static constexpr int kRingBytes = kDecWarps * kWarpBytes;
  static constexpr int kMergeStride = D + 8;                       // floats per merged row
  static constexpr int kMergeBytes = kDecWarps * 16 * kMergeStride * 4 + kDecWarps * 16 * 2 * 4;
  static_assert(kMergeBytes <= kRingBytes, "merge buffer must fit in the ring");
  // streaming variant: a merge buffer of its own, for groups of up to kStreamRows query heads
  static constexpr int kStreamRows = 4;
  static constexpr int kStreamMergeBytes = kDecWarps * kStreamRows * kMergeStride * 4 + kDecWarps * kStreamRows * 2 * 4;
};

// kStream = false: every work item fills its rings from empty and the merge buffer reuses the ring memory.
// kStream = true (groups of up to four query heads, one row tile): the merge buffer has memory of its own and a
// warp's tiles form ONE stream across the work items of its CTA -- the loads run two tiles ahead of the MMAs
// also across an item boundary, so the next item's first tiles arrive during the merge of the current one.
template <typename T, int D, bool kStream>
__global__ void __launch_bounds__(kDecThreads, kDecCtasPerSM)
paged_decode_kernel(const DecodeParams p) {
  using S = DecodeSmem<T, D>;
  constexpr int CPR = D / 8;              // 16-byte chunks per row
  constexpr int RPI = 32 / CPR;           // rows covered by one warp-wide cp.async
  constexpr int LOAD_ITERS = kTileTok / RPI;
  constexpr int KSTEPS = D / 16;
  constexpr int NT = D / 8;               // output n-tiles
  constexpr bool kSplitP = sizeof(typename Elem<T>::T2) == 4 && !std::is_same<T, __half>::value;

  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ long long s_red[kDecWarps];
  __shared__ uint32_t s_mask[kDecWarps][kDecStages];
  __shared__ int s_last;
  int* s_start = reinterpret_cast<int*>(smem + S::kRingBytes + (kStream ? S::kStreamMergeBytes : 0));

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  const DecodePlan plan = build_plan(p, s_start, s_red);
  if (blockIdx.x == 0) {
    for (int b = tid; b < p.batch; b += kDecThreads) p.binfo[b] = seq_items(s_start, plan, b);
  }
  zero_empty_sequences<T, D>(p, s_start);

  const int ydim = p.num_kv_heads * p.mtiles;
  const long long n_units = static_cast<long long>(plan.n_seg) * ydim;
  const uint32_t ring = smem_u32(smem) + warp * S::kWarpBytes;
  const T* kc = static_cast<const T*>(p.k_cache);
  const T* vc = static_cast<const T*>(p.v_cache);
  const int bs = p.block_size;

  // What a warp needs to know of a work item.
  struct Item {
    int b, nsplit, tok_begin, tok_end, kvh, mt, item, my_tiles;
    const int32_t* table;
  };
  auto load_item = [&](const ItemWalk& at, Item& it) -> bool {
    if (at.b < 0) return false;
    it.kvh = at.y / p.mtiles;
    it.mt = at.y - it.kvh * p.mtiles;
    const DecodeItem di = piece_of(s_start, plan, at.b, at.seg);
    it.item = di.item;
    it.b = di.b; it.nsplit = di.nsplit; it.tok_begin = di.tok_begin; it.tok_end = di.tok_end;
    it.table = p.block_tables + static_cast<int64_t>(di.b) * p.bt_stride;
    // tiles of this warp: tokens tok_begin + (i*kDecWarps + warp)*16
    const int span = di.tok_end - di.tok_begin;
    const int cta_tiles = span > 0 ? (span + kTileTok - 1) / kTileTok : 0;
    it.my_tiles = cta_tiles > warp ? (cta_tiles - warp + kDecWarps - 1) / kDecWarps : 0;
    return true;
  };
  // ring stage <- tile i of this warp within item `it` (no commit)
  auto issue_tile = [&](const Item& it, int i, int stage) {
    const int tok0 = it.tok_begin + (i * kDecWarps + warp) * kTileTok;
    const int blk0 = tok0 / bs, off0 = tok0 - blk0 * bs;
    // lane r (r < 16) resolves row r; others mirror it
    const int r_me = lane & 15;
    int off = off0 + r_me, blk = blk0;
    while (off >= bs) { off -= bs; ++blk; }
    int slot = -1;
    if (tok0 + r_me < it.tok_end) {
      const int pb = __ldg(it.table + blk);
      if (pb >= 0 && pb < p.num_blocks) slot = pb * bs + off;
    }
    const uint32_t live = __ballot_sync(0xffffffffu, slot >= 0) & 0xffffu;
    if (lane == 0) s_mask[warp][stage] = live;
    const uint32_t kdst = ring + stage * S::kStageBytes;
    const uint32_t vdst = kdst + S::kTileBytes;
    const int c = lane % CPR, r0 = lane / CPR;
#pragma unroll
    for (int li = 0; li < LOAD_ITERS; ++li) {
      const int r = r0 + li * RPI;
      const int s = __shfl_sync(0xffffffffu, slot, r);
      const int64_t eoff = s >= 0 ? (static_cast<int64_t>(s) * p.num_kv_heads + it.kvh) * D + c * 8 : 0;
      const uint32_t doff = r * S::kRowBytes + ((c ^ (r & 7)) << 4);
      cp_async16(kdst + doff, kc + eoff, s >= 0 ? 16 : 0);
      cp_async16(vdst + doff, vc + eoff, s >= 0 ? 16 : 0);
    }
  };
  // kStream: the load side walks the warp's tile stream on its own, two ring slots ahead of the MMAs.  Every
  // slot is one cp.async group (empty once the stream has ended), so "at most one group pending" always
  // means that the slot about to be consumed has landed.
  ItemWalk load_at;
  Item load_it;
  bool load_valid = false;
  int load_tile = 0, load_slot = 0, use_slot = 0;
  auto issue_next = [&]() {
    while (load_valid && load_tile >= load_it.my_tiles) {
      walk_next(p, s_start, plan, ydim, n_units, gridDim.x, load_at);
      load_valid = load_item(load_at, load_it);
      load_tile = 0;
    }
    if (load_valid) {
      issue_tile(load_it, load_tile, load_slot % kDecStages);
      ++load_tile;
    }
    cp_async_commit();
    ++load_slot;
  };
  if constexpr (kStream) {
    walk_start(p, s_start, plan, ydim, n_units, blockIdx.x, load_at);
    load_valid = load_item(load_at, load_it);
#pragma unroll
    for (int i = 0; i < kDecStages - 1; ++i) issue_next();
  }

  ItemWalk at;
  for (walk_start(p, s_start, plan, ydim, n_units, blockIdx.x, at); at.b >= 0;
       walk_next(p, s_start, plan, ydim, n_units, gridDim.x, at)) {
    Item cur;
    load_item(at, cur);
    const int item = cur.item, kvh = cur.kvh, mt = cur.mt, b = cur.b, nsplit = cur.nsplit, my_tiles = cur.my_tiles;
    const int rows_valid = min(16, p.group - mt * 16);
    const int h0 = kvh * p.group + mt * 16;

    auto issue = [&](int i) {   // not streaming: stage i % kDecStages <- tile i of this item (or nothing past its end)
      if (i < my_tiles) issue_tile(cur, i, i % kDecStages);
      cp_async_commit();
    };

    if constexpr (!kStream) {
#pragma unroll
      for (int i = 0; i < kDecStages - 1; ++i) issue(i);
    }

    // Q fragments: rows g and g+8 of the 16-row tile, zero past the group.
    uint32_t qa[KSTEPS][4];
    {
      const T* qbase = static_cast<const T*>(p.q) + (static_cast<int64_t>(b) * p.num_heads + h0) * D;
      const bool v0 = g < rows_valid, v1 = g + 8 < rows_valid;
      const uint32_t* q0 = reinterpret_cast<const uint32_t*>(qbase + static_cast<int64_t>(g) * D);
      const uint32_t* q1 = reinterpret_cast<const uint32_t*>(qbase + static_cast<int64_t>(g + 8) * D);
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        qa[ks][0] = v0 ? __ldg(q0 + ks * 8 + t) : 0u;
        qa[ks][1] = v1 ? __ldg(q1 + ks * 8 + t) : 0u;
        qa[ks][2] = v0 ? __ldg(q0 + ks * 8 + 4 + t) : 0u;
        qa[ks][3] = v1 ? __ldg(q1 + ks * 8 + 4 + t) : 0u;
      }
    }

    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m0 = kNegBig, m1 = kNegBig, l0 = 0.f, l1 = 0.f;

    for (int i = 0; i < my_tiles; ++i) {
      cp_async_wait<kDecStages - 2>();
      __syncwarp();
      const int stage = (kStream ? use_slot : i) % kDecStages;
      const uint32_t kbase = ring + stage * S::kStageBytes;
      const uint32_t vbase = kbase + S::kTileBytes;
      const uint32_t live = s_mask[warp][stage];

      float s[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
      {
        const int row = (lane & 7) + ((lane >> 4) << 3);
        const int csel = (lane >> 3) & 1;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          uint32_t kb[4];
          ldmatrix_x4(kb, kbase + row * S::kRowBytes + (((2 * ks + csel) ^ (row & 7)) << 4));
          Mma16816<T>::run(s[0], qa[ks], kb[0], kb[1]);
          Mma16816<T>::run(s[1], qa[ks], kb[2], kb[3]);
        }
      }
      // Issue the next tile now: its slot was released at the end of the
      // previous iteration, and the loads overlap the softmax below.
      if constexpr (kStream) issue_next(); else issue(i + kDecStages - 1);

      float mx0 = kNegBig, mx1 = kNegBig;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = n * 8 + 2 * t + (e & 1);
          const bool ok = (live >> col) & 1u;
          s[n][e] = ok ? s[n][e] * p.scale_log2 : -INFINITY;
        }
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float a0 = fast_exp2(m0 - mn0), a1 = fast_exp2(m1 - mn1);
      m0 = mn0; m1 = mn1;
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        s[n][0] = fast_exp2(s[n][0] - mn0); s[n][1] = fast_exp2(s[n][1] - mn0);
        s[n][2] = fast_exp2(s[n][2] - mn1); s[n][3] = fast_exp2(s[n][3] - mn1);
        ps0 += s[n][0] + s[n][1];
        ps1 += s[n][2] + s[n][3];
      }
      l0 = l0 * a0 + ps0;  // per-thread partial sums; the quad is reduced at the end
      l1 = l1 * a1 + ps1;
      uint32_t pa[4];
      pa[0] = pack2<T>(s[0][0], s[0][1]);
      pa[1] = pack2<T>(s[0][2], s[0][3]);
      pa[2] = pack2<T>(s[1][0], s[1][1]);
      pa[3] = pack2<T>(s[1][2], s[1][3]);
      // bf16 keeps 8 significant bits: carry the rounding residue of P in a
      // second operand so that short contexts (few, large weights) stay within
      // tolerance.  The extra MMAs are free in an HBM-bound kernel.
      uint32_t pl[4];
      if constexpr (kSplitP) {
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const float2 hi = Elem<T>::to_f2(*reinterpret_cast<const typename Elem<T>::T2*>(&pa[2 * n + hh]));
            pl[2 * n + hh] = pack2<T>(s[n][2 * hh] - hi.x, s[n][2 * hh + 1] - hi.y);
          }
        }
      }
      // the running maximum rarely moves after the first tiles: rescale only when some row of the warp needs it
      if (__any_sync(0xffffffffu, a0 != 1.f || a1 != 1.f)) {
#pragma unroll
        for (int j = 0; j < NT; ++j) { o[j][0] *= a0; o[j][1] *= a0; o[j][2] *= a1; o[j][3] *= a1; }
      }
      {
        const int row = (lane & 7) + (((lane >> 3) & 1) << 3);
        const int csel = lane >> 4;
#pragma unroll
        for (int jp = 0; jp < KSTEPS; ++jp) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, vbase + row * S::kRowBytes + (((2 * jp + csel) ^ (row & 7)) << 4));
          Mma16816<T>::run(o[2 * jp], pa, vb[0], vb[1]);
          Mma16816<T>::run(o[2 * jp + 1], pa, vb[2], vb[3]);
          if constexpr (kSplitP) {
            Mma16816<T>::run(o[2 * jp], pl, vb[0], vb[1]);
            Mma16816<T>::run(o[2 * jp + 1], pl, vb[2], vb[3]);
          }
        }
      }
      __syncwarp();  // all lanes are done with this stage before it is refilled
      ++use_slot;
    }
    if constexpr (!kStream) cp_async_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // ---- merge the four warps through shared memory ----
    if constexpr (kStream) {
      // buffer of its own (rows of the group only): the rings keep receiving the next item's tiles meanwhile
      constexpr int R = S::kStreamRows;
      float* sO = reinterpret_cast<float*>(smem + S::kRingBytes);
      float* sML = sO + kDecWarps * R * S::kMergeStride;
      if (g < R) {
        float* mine = sO + (warp * R + g) * S::kMergeStride;
#pragma unroll
        for (int j = 0; j < NT; ++j) *reinterpret_cast<float2*>(mine + j * 8 + 2 * t) = make_float2(o[j][0], o[j][1]);
        if (t == 0) {
          sML[(warp * R + g) * 2] = m0;
          sML[(warp * R + g) * 2 + 1] = l0;
        }
      }
      __syncthreads();
      merge_and_write<T, D>(p, sO, sML, S::kMergeStride, rows_valid, h0, b, item, nsplit, R);
      __syncthreads();  // the buffer is free for the next item
      combine_if_last<T, D>(p, s_start, plan, b, b * ydim + kvh * p.mtiles + mt, h0, rows_valid, nsplit, &s_last);
    } else {
      __syncthreads();  // the ring is idle now
      float* sO = reinterpret_cast<float*>(smem);
      float* sML = sO + kDecWarps * 16 * S::kMergeStride;
      {
        float* mine = sO + warp * 16 * S::kMergeStride;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          *reinterpret_cast<float2*>(mine + g * S::kMergeStride + j * 8 + 2 * t) = make_float2(o[j][0], o[j][1]);
          *reinterpret_cast<float2*>(mine + (g + 8) * S::kMergeStride + j * 8 + 2 * t) = make_float2(o[j][2], o[j][3]);
        }
        if (t == 0) {
          sML[(warp * 16 + g) * 2] = m0;
          sML[(warp * 16 + g) * 2 + 1] = l0;
          sML[(warp * 16 + g + 8) * 2] = m1;
          sML[(warp * 16 + g + 8) * 2 + 1] = l1;
        }
      }
      __syncthreads();
      merge_and_write<T, D>(p, sO, sML, S::kMergeStride, rows_valid, h0, b, item, nsplit);
      __syncthreads();  // the ring is handed back to the pipelines
      combine_if_last<T, D>(p, s_start, plan, b, b * ydim + kvh * p.mtiles + mt, h0, rows_valid, nsplit, &s_last);
    }
  }
  if constexpr (kStream) cp_async_wait<0>();   // only empty groups are left
}

// Reduces the partial results of sequences that were split, in item order.
template <typename T, int D>
__global__ void __launch_bounds__(128)
paged_decode_combine_kernel(const DecodeParams p) {
  const int b = blockIdx.x, kvh = blockIdx.y;
  const int2 info = p.binfo[b];
  if (info.y <= 1) return;
  const int h_begin = kvh * p.group;
  for (int idx = threadIdx.x; idx < p.group * D; idx += blockDim.x) {
    const int h = h_begin + idx / D, d = idx % D;
    float M = kNegBig;
    for (int s = 0; s < info.y; ++s)
      M = fmaxf(M, p.part_ml[(static_cast<int64_t>(info.x + s) * p.num_heads + h) * 2]);
    float acc = 0.f, L = 0.f;
    for (int s = 0; s < info.y; ++s) {
      const int64_t pi = static_cast<int64_t>(info.x + s) * p.num_heads + h;
      const float wgt = fast_exp2(p.part_ml[pi * 2] - M);
      acc += wgt * p.part_o[pi * D + d];
      L += wgt * p.part_ml[pi * 2 + 1];
    }
    const float r = L > 0.f ? acc / L : 0.f;
    static_cast<T*>(p.out)[(static_cast<int64_t>(b) * p.num_heads + h) * D + d] = Elem<T>::from_f(r);
  }
}

struct DecodeLayout {
  int64_t arrivals_off, binfo_off, ml_off, o_off, total;
  bool folded;   // arrival counters fit: the last piece's CTA reduces, no combine launch
};
static DecodeLayout decode_layout(int batch, int num_heads, int num_kv_heads, int head_dim, int max_blocks,
                                  int block_size) {
  (void)max_blocks;
  (void)block_size;
  const int mtiles = (num_heads / num_kv_heads + 15) / 16;
  const int64_t items = decode_items_max(batch, num_kv_heads, mtiles);
  DecodeLayout L;
  // The counters sit first and always take the same room, so that calls of different shapes that share one
  // scratch buffer never write anything but counters there.
  L.arrivals_off = 0;
  L.folded = static_cast<int64_t>(batch) * num_kv_heads * mtiles <= kDecodeArrivalCells;
  L.binfo_off = static_cast<int64_t>(kDecodeArrivalCells) * 4;
  L.ml_off = L.binfo_off + ((static_cast<int64_t>(batch) * 8 + 255) / 256) * 256;
  L.o_off = L.ml_off + ((items * num_heads * 2 * 4 + 255) / 256) * 256;
  L.total = L.o_off + items * num_heads * head_dim * 4;
  return L;
}

template <typename T, int D, bool kStream>
static int launch_decode_variant(const DecodeParams& p, size_t smem, cudaStream_t st) {
  static size_t attr_bytes[64] = {};  // per kernel instantiation and per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || attr_bytes[dev] < smem) {
    const cudaError_t e = cudaFuncSetAttribute(paged_decode_kernel<T, D, kStream>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(MV_ERR_CUDA, "paged_decode: cudaFuncSetAttribute(%zu): %s", smem, cudaGetErrorString(e));
    }
    if (dev >= 0 && dev < 64) attr_bytes[dev] = smem;
  }
  const int grid = decode_grid(p);
  paged_decode_kernel<T, D, kStream><<<grid, kDecThreads, smem, st>>>(p);
  return check_launch("paged_decode_kernel");
}

template <typename T, int D>
static int launch_decode(const DecodeParams& p, cudaStream_t st) {
  using S = DecodeSmem<T, D>;
  const size_t plan = static_cast<size_t>(p.batch + 1) * sizeof(int);
  const size_t smem = S::kRingBytes + plan;
  // 227 KB per CTA is the sm_100 limit for static + dynamic shared memory together.
  constexpr size_t kStaticSmem = 256;
  if (smem + kStaticSmem > 227 * 1024)
    return fail(MV_ERR_LIMIT, "paged_decode: batch %d needs %zu bytes of shared memory", p.batch, smem);
  // the streaming variant when the group fits its merge buffer and two CTAs still fit an SM
  const size_t smem_stream = smem + S::kStreamMergeBytes;
  const bool stream = p.mtiles == 1 && p.group <= S::kStreamRows &&
                      kDecCtasPerSM * (smem_stream + kStaticSmem + 1024) <= 227 * 1024;
  int rc = stream ? launch_decode_variant<T, D, true>(p, smem_stream, st)
                  : launch_decode_variant<T, D, false>(p, smem, st);
  if (rc || p.arrivals) return rc;
  paged_decode_combine_kernel<T, D><<<dim3(p.batch, p.num_kv_heads), 128, 0, st>>>(p);
  return check_launch("paged_decode_combine_kernel");
}

}  // namespace mv

extern "C" int64_t mv_paged_decode_workspace_bytes(int batch, int num_heads, int num_kv_heads, int head_dim,
                                                   int max_blocks, int block_size) {
  if (batch <= 0 || num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || max_blocks < 0 || block_size <= 0 ||
      num_heads % num_kv_heads != 0)
    return -1;
  return mv::decode_layout(batch, num_heads, num_kv_heads, head_dim, max_blocks, block_size).total;
}

extern "C" int mv_paged_decode(void* out, const void* q, const void* k_cache, const void* v_cache,
                               const void* k_scale, const void* v_scale, const int32_t* block_tables,
                               int64_t bt_stride, int max_blocks, const void* context_lens, int ctx_is_i64, int batch,
                               int num_heads, int num_kv_heads, int head_dim, int block_size, int64_t num_blocks,
                               float scale, void* workspace, int64_t workspace_bytes, int dtype, void* stream) {
  using namespace mv;
  if (dtype != MV_F16 && dtype != MV_BF16) return fail(MV_ERR_DTYPE, "paged_decode: dtype %d", dtype);
  if (batch < 0 || num_heads <= 0 || num_kv_heads <= 0 || block_size <= 0 || max_blocks < 0 || num_blocks < 0)
    return fail(MV_ERR_SHAPE, "paged_decode: negative or zero size");
  if (num_heads % num_kv_heads != 0)
    return fail(MV_ERR_SHAPE, "paged_decode: num_heads %d is not a multiple of num_kv_heads %d", num_heads, num_kv_heads);
  if (head_dim != 64 && head_dim != 128) return fail(MV_ERR_SHAPE, "paged_decode: head_dim %d not in {64,128}", head_dim);
  if (batch == 0) return MV_OK;
  if (!out || !q || !k_cache || !v_cache || !block_tables || !context_lens || !workspace)
    return fail(MV_ERR_NULL, "paged_decode: null pointer");
  if ((k_scale == nullptr) != (v_scale == nullptr))
    return fail(MV_ERR_NULL, "paged_decode: k_scale and v_scale must both be set or both be null");
  if (k_scale && head_dim != 128) return fail(MV_ERR_SHAPE, "paged_decode: int8 caches need head_dim 128");
  if (k_scale && (!aligned16(k_scale) || !aligned16(v_scale)))
    return fail(MV_ERR_ALIGN, "paged_decode: scale pointers must be 16-byte aligned");
  if (!aligned16(out) || !aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(workspace))
    return fail(MV_ERR_ALIGN, "paged_decode: pointers must be 16-byte aligned");
  if (bt_stride < max_blocks) return fail(MV_ERR_SHAPE, "paged_decode: block table stride smaller than its width");
  if (num_blocks * block_size > 0x7fffffffLL) return fail(MV_ERR_LIMIT, "paged_decode: more than 2^31 cache slots");
  if (static_cast<int64_t>(batch) * max_blocks * block_size > 0x7fffffffLL)
    return fail(MV_ERR_LIMIT, "paged_decode: batch * max_blocks * block_size exceeds 2^31 tokens");
  const DecodeLayout L = decode_layout(batch, num_heads, num_kv_heads, head_dim, max_blocks, block_size);
  if (workspace_bytes < L.total)
    return fail(MV_ERR_WORKSPACE, "paged_decode: workspace %lld < %lld bytes", (long long)workspace_bytes, (long long)L.total);

  DecodeParams p;
  p.out = out; p.q = q; p.k_cache = k_cache; p.v_cache = v_cache;
  p.k_scale = static_cast<const __half*>(k_scale); p.v_scale = static_cast<const __half*>(v_scale);
  p.block_tables = block_tables; p.bt_stride = bt_stride; p.max_blocks = max_blocks;
  p.context_lens = context_lens; p.ctx_is_i64 = ctx_is_i64;
  p.batch = batch; p.num_heads = num_heads; p.num_kv_heads = num_kv_heads;
  p.group = num_heads / num_kv_heads; p.mtiles = (p.group + 15) / 16;
  p.block_size = block_size; p.num_blocks = num_blocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.target_items = decode_target_items(num_kv_heads, p.mtiles);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  p.arrivals = L.folded ? reinterpret_cast<unsigned*>(ws + L.arrivals_off) : nullptr;
  p.binfo = reinterpret_cast<int2*>(ws + L.binfo_off);
  p.part_ml = reinterpret_cast<float*>(ws + L.ml_off);
  p.part_o = reinterpret_cast<float*>(ws + L.o_off);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (k_scale) {
    const int rc = dtype == MV_F16 ? launch_decode_int8<__half>(p, st) : launch_decode_int8<__nv_bfloat16>(p, st);
    if (rc || p.arrivals) return rc;
    if (dtype == MV_F16) paged_decode_combine_kernel<__half, 128><<<dim3(batch, num_kv_heads), 128, 0, st>>>(p);
    else paged_decode_combine_kernel<__nv_bfloat16, 128><<<dim3(batch, num_kv_heads), 128, 0, st>>>(p);
    return check_launch("paged_decode_combine_kernel");
  }
  if (dtype == MV_F16) return head_dim == 128 ? launch_decode<__half, 128>(p, st) : launch_decode<__half, 64>(p, st);
  return head_dim == 128 ? launch_decode<__nv_bfloat16, 128>(p, st) : launch_decode<__nv_bfloat16, 64>(p, st);
}
