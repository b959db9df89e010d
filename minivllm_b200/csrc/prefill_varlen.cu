// Varlen causal prefill flash attention on the Blackwell tensor cores.
//
// Does the work of src/myvllm/layers/attention.py:111-280 of the reference
// (Triton, 32x32 tiles, no causal block skipping, a host sync per call).
//
// One CTA owns a 128-row query tile of one sequence for TWO query heads of the
// same GQA group, so the two 128x128 problems share every K/V tile and the
// tensor pipe always has the other head's MMAs to run while one head's
// softmax is on the CUDA cores.  Roles (384 threads; the last warpgroup gives
// most of its registers to the softmax warpgroups with setmaxnreg):
//   warps 0-3   softmax of head A: thread i owns row i (= TMEM lane i)
//   warps 4-7   softmax of head B
//   warp  8     TMA producer: Q once, then K and V tiles through 2-stage rings
//   warp  9     MMA issuer: one thread issues every tcgen05.mma and commits to mbarriers
// Tensor memory (512 columns): S_A | S_B | O_A | O_B, 128 fp32 columns each.
// S = Q K^T is an SS MMA (both operands in 128B-swizzled shared memory, written
// by TMA); the softmax warps read S with tcgen05.ld, write P (bf16/fp16, packed
// two per column) over the first 64 columns of S with tcgen05.st, and O += P V
// is a TS MMA (P from tensor memory, V from shared memory, MN-major).  The
// running maximum is only moved when it grows by more than 2^8, so O in tensor
// memory is rescaled rarely; l and the final 1/l use the same stale maximum.
// KV tiles above the diagonal are never visited; only tiles that reach past
// the first row's position are masked.  In paged mode (a cached prefix, or a
// chunk of a longer prompt) K and V come from the paged cache through the
// block tables instead of the packed inputs.  No cluster multicast anywhere.
//
// Tensor-bound: FLOPs = 4 * heads * head_dim * sum_s L_s (L_s + 1) / 2.
#include <cuda.h>
#include "tcgen05.cuh"
#include "mma.cuh"
#include <atomic>
#include <type_traits>

namespace mv {

constexpr int kPfThreads = 384;  // 8 softmax warps + TMA warp + MMA warp + 2 idle warps (register donors)
constexpr int kPfTile = 128;         // query rows and KV columns per tile
constexpr int kPfD = 128;
constexpr int kPfHalfBytes = kPfTile * 128;                 // one 64-element half of a 128-row tile
constexpr int kPfTileBytes = 2 * kPfHalfBytes;              // 32 KB
constexpr int kPfStages = 2;
constexpr int kPfSmemBytes = 2 * kPfTileBytes + 2 * kPfStages * kPfTileBytes + 1024;  // Q(2 heads) + K ring + V ring + align
// Which of the 32 score pairs of a half row take the polynomial exp2 (the others use the special-function unit).
#ifndef MV_PF_POLY_PRED
#define MV_PF_POLY_PRED(i) (((i) & 3) == 3)   // a quarter: measured best of 0, 1/4, 1/2, 3/4, all
#endif
constexpr float kRescaleThreshold = 8.f;                    // log2 units

struct PrefillParams {
  void* out;
  int64_t out_stride_tok;  // elements
  int out_align32;         // output rows start on 32-byte boundaries
  int inject;              // test hook, normally 0.  1: head A of tile 0 withholds its first "P ready" arrival,
                           // so that the MMA warp's bounded wait runs out and the abort path is exercised
  const int32_t* cu_seqlens;
  int num_seqs, num_heads, num_kv_heads, group, pairs;  // pairs = ceil(group / 2)
  float scale_log2;
  int fmt;          // 0 fp16, 1 bf16
  int* error_word;
  // Paged mode (prefix hit / chunked prefill): K and V are read from the paged cache through the block
  // tables, and sequence s has cu_seqlens_k-many keys of which the first (keys - queries) are already cached.
  int paged;
  const int32_t* cu_seqlens_k;
  const int32_t* block_tables;
  int64_t bt_stride;
  int max_blocks, block_size, box_rows;   // box_rows = min(block_size, 128): rows of one TMA box of the cache
  int sched_slot;                         // persistent form: which work counter this launch uses
};

enum { BAR_Q = 0, BAR_KFULL = 1, BAR_KEMPTY = 3, BAR_VFULL = 5, BAR_VEMPTY = 7, BAR_SFULL = 9, BAR_PREADY = 11,
       BAR_ODONE = 13, BAR_SPARE = 15, BAR_DRAIN = 16, BAR_COUNT = 17 };

#ifdef MV_PF_TRACE
// Timeline probe (debug builds only, -DMV_PF_TRACE): one thread of each role of ONE CTA writes clock64()
// stamps per KV step, so that the phases of the pipeline can be read off without a profiler.
// Buffer (long long, 2048 entries, set with mv_debug_prefill_trace): entry ((role * 32 + i) * 8 + k) is stamp k
// of role `role` at index i.  One CTA per tile: i = KV step.  Persistent kernel: i = the CTA's unit number,
// roles 0 producer, 1 MMA warp, 2 / 3 first softmax warp of head A / B (entry k = 7 of role 0 holds the unit's
// number of KV steps); PF_STEP adds, from entry 1024 on, per-step stamps of the CTA's fourth unit
// ((role * 8 + step) * 8 + k; roles 0 MMA warp, 1 / 2 softmax A / B).
__device__ long long* g_pf_trace = nullptr;
__device__ int g_pf_trace_cta = -1;
// pf_tr is read once per thread at kernel start: a stamp is then one predicated store, cheap enough not to
// distort the warp it measures.
#define PF_STAMP(role, j, k)                                                      \
  do {                                                                            \
    if (pf_tr && (j) < 32) pf_tr[((role) * 32 + (j)) * 8 + (k)] = clock64();      \
  } while (0)
#define PF_TRACE_INIT() \
  long long* const pf_tr = (static_cast<int>(blockIdx.x) == g_pf_trace_cta && blockIdx.y == 0) ? g_pf_trace : nullptr
#define PF_STEP(unit, role, j, k)                                                              \
  do {                                                                                          \
    if (pf_tr && (unit) == 3 && (j) < 8) pf_tr[1024 + ((role) * 8 + (j)) * 8 + (k)] = clock64(); \
  } while (0)
#else
#define PF_STEP(unit, role, j, k) do {} while (0)
#define PF_STAMP(role, j, k) do {} while (0)
#define PF_TRACE_INIT() do {} while (0)
#endif

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_varlen_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[BAR_COUNT];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_tile[2];       // (sequence, query tile) of this CTA, -1 = none
  __shared__ int s_scan[16];
  __shared__ int s_abort;
  __shared__ int s_sticky;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  PF_TRACE_INIT();
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;                                  // [head 2][half 2][128][128B]
  const uint32_t k_smem = q_smem + 2 * kPfTileBytes;                  // [stage][half][128][128B]
  const uint32_t v_smem = k_smem + kPfStages * kPfTileBytes;
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  volatile int* abort_flag = &s_abort;

  // ---- which (sequence, query tile) is blockIdx.x?  tiles of a sequence in descending order ----
  if (tid == 0) {
    s_tile[0] = -1;
    s_tile[1] = 0;
    s_abort = 0;
    s_sticky = *reinterpret_cast<volatile int*>(p.error_word);  // read once so that the whole CTA agrees
  }
  __syncthreads();
  {
    int carry = 0;
    for (int base = 0; base < p.num_seqs; base += kPfThreads) {
      const int s = base + tid;
      int n = 0;
      if (s < p.num_seqs) {
        const int len = p.cu_seqlens[s + 1] - p.cu_seqlens[s];
        n = len > 0 ? (len + kPfTile - 1) / kPfTile : 0;
      }
      int incl = n;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += v;
      }
      if (lane == 31) s_scan[warp] = incl;
      __syncthreads();
      int wofs = 0, tot = 0;
#pragma unroll
      for (int w2 = 0; w2 < kPfThreads / 32; ++w2) {
        const int v = s_scan[w2];
        if (w2 < warp) wofs += v;
        tot += v;
      }
      const int start = carry + wofs + incl - n;
      const int x = static_cast<int>(blockIdx.x);
      if (n > 0 && x >= start && x < start + n) { s_tile[0] = s; s_tile[1] = n - 1 - (x - start); }
      carry += tot;
      __syncthreads();
    }
  }
  const int seq = s_tile[0], qtile = s_tile[1];
  if (seq < 0) return;  // uniform: the grid is an upper bound on the number of tiles
  // A wait that ran out anywhere (this launch or an earlier one) leaves the
  // error word set: the remaining CTAs return at once instead of waiting too.
  if (s_sticky != 0) return;

  const int kvh = blockIdx.y / p.pairs, pair = blockIdx.y - kvh * p.pairs;
  const int head_a = kvh * p.group + 2 * pair;
  const bool has_b = 2 * pair + 1 < p.group;
  const int seq_start = p.cu_seqlens[seq];
  const int seq_len = p.cu_seqlens[seq + 1] - seq_start;
  const int q0 = qtile * kPfTile;              // first query row of the tile within the sequence
  // keys of this sequence that precede its first query row (0 unless paged: a cached prefix)
  const int n_cached = p.paged ? (p.cu_seqlens_k[seq + 1] - p.cu_seqlens_k[seq]) - seq_len : 0;
  const int first_pos = n_cached + q0;         // position of the tile's first query row within the sequence
  // causal: KV tiles up to the one holding the position of the tile's last real query row
  const int n_kv = (n_cached + min(q0 + kPfTile, seq_len) + kPfTile - 1) / kPfTile;
  // A tile whose first row sits below position 128 has rows with fewer than 128
  // keys, so the rounding of their weights to bf16 (8 significant bits) does not
  // average out: those CTAs (the cheapest ones, one or two KV tiles) also feed
  // the rounding residue of P through a second PV MMA.  fp16 P has 11 bits and
  // needs nothing.
  const bool split_p = std::is_same<T, __nv_bfloat16>::value && first_pos < kPfTile;

  if (tid == 0) {
    tc::mbar_init(bar(BAR_Q), 1);
    for (int s = 0; s < kPfStages; ++s) {
      tc::mbar_init(bar(BAR_KFULL + s), 1);
      tc::mbar_init(bar(BAR_KEMPTY + s), 1);
      tc::mbar_init(bar(BAR_VFULL + s), 1);
      tc::mbar_init(bar(BAR_VEMPTY + s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      tc::mbar_init(bar(BAR_SFULL + t), 1);
      tc::mbar_init(bar(BAR_PREADY + t), 128);
      tc::mbar_init(bar(BAR_ODONE + t), 1);
    }
    tc::mbar_init(bar(BAR_SPARE), 1);   // takes commits that nobody waits for
    tc::mbar_init(bar(BAR_DRAIN), 1);
    tc::mbar_fence_init();
  }
  if (warp == 8) {
    tc::tmem_alloc(smem_u32(&s_tmem_base), 512);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem_base;

  if (warp >= 8) {
    tc::setmaxnreg_dec_40();
    if (warp == 8) {
      // ------------------------------ TMA producer ------------------------------
      if (lane == 0) {
        tc::tma_prefetch_desc(&tmap_q);
        tc::tma_prefetch_desc(&tmap_k);
        tc::tma_prefetch_desc(&tmap_v);
        const int row0 = seq_start + q0;
        tc::mbar_expect_tx(bar(BAR_Q), (has_b ? 2 : 1) * kPfTileBytes);
        for (int t = 0; t < (has_b ? 2 : 1); ++t)
          for (int h = 0; h < 2; ++h)
            tc::tma_load_3d(q_smem + t * kPfTileBytes + h * kPfHalfBytes, &tmap_q, 64 * h, head_a + t, row0, bar(BAR_Q));
        // One 128-token K or V tile: packed rows of this sequence, or (paged) the cache rows that the block
        // table gives for positions 128j.., as 128 / box_rows boxes of box_rows rows each.  A table entry
        // that is missing loads block 0: those keys lie beyond every query row of the tile and are masked.
        auto load_kv_tile = [&](const CUtensorMap* tm, uint32_t dst, int j, uint32_t full_bar) {
          if (!p.paged) {
            for (int h = 0; h < 2; ++h)
              tc::tma_load_3d(dst + h * kPfHalfBytes, tm, 64 * h, kvh, seq_start + j * kPfTile, full_bar);
            return;
          }
          const int32_t* table = p.block_tables + static_cast<int64_t>(seq) * p.bt_stride;
          for (int r = 0; r < kPfTile / p.box_rows; ++r) {
            const int pos = j * kPfTile + r * p.box_rows;
            const int blk = pos / p.block_size, off = pos - blk * p.block_size;
            const int phys = blk < p.max_blocks ? table[blk] : -1;
            const int slot = phys >= 0 ? phys * p.block_size + off : 0;
            for (int h = 0; h < 2; ++h)
              tc::tma_load_3d(dst + h * kPfHalfBytes + r * p.box_rows * 128, tm, 64 * h, kvh, slot, full_bar);
          }
        };
        for (int j = 0; j < n_kv; ++j) {
          const int s = j % kPfStages;
          const uint32_t ph = ((j / kPfStages) & 1) ^ 1;
          tc::mbar_wait(bar(BAR_KEMPTY + s), ph, abort_flag, p.error_word, 1);
          tc::mbar_expect_tx(bar(BAR_KFULL + s), kPfTileBytes);
          load_kv_tile(&tmap_k, k_smem + s * kPfTileBytes, j, bar(BAR_KFULL + s));
          tc::mbar_wait(bar(BAR_VEMPTY + s), ph, abort_flag, p.error_word, 2);
          tc::mbar_expect_tx(bar(BAR_VFULL + s), kPfTileBytes);
          load_kv_tile(&tmap_v, v_smem + s * kPfTileBytes, j, bar(BAR_VFULL + s));
        }
        // After an abort nobody may be left to consume the loads already issued: give them time to land before
        // the CTA (and its shared memory) goes away.  A full barrier completes its phase when its bytes arrive.
        if (*abort_flag) {
          tc::mbar_wait_timed(bar(BAR_Q), 0);
          for (int j = max(n_kv - kPfStages, 0); j < n_kv; ++j) {
            tc::mbar_wait_timed(bar(BAR_KFULL + j % kPfStages), (j / kPfStages) & 1);
            tc::mbar_wait_timed(bar(BAR_VFULL + j % kPfStages), (j / kPfStages) & 1);
          }
        }
      }
    } else if (warp == 9) {
      // ------------------------------- MMA issuer -------------------------------
      // ONE warp, converged, issues every MMA of the CTA through its elected lane.  (Issuing the two heads from two
      // warps was measured: the tensor pipe then serialises, ~1000 cycles per MMA.)
      // A single thread cannot hide the latency of its own instruction stream, so
      // the descriptors are reduced to one add per operand: the fixed part is
      // built once, offsets are compile-time constants in 16-byte units.
      {
        const uint32_t idesc_qk = tc::instr_desc_f16(p.fmt, p.fmt, false, 128, 128);
        // A and B must have the same format: fp16 P against bf16 V is rejected
        // by the hardware as an illegal instruction.
        const uint32_t idesc_pv = tc::instr_desc_f16(p.fmt, p.fmt, true, 128, 128);
        const int nt = has_b ? 2 : 1;
        const uint32_t desc_hi = tc::kDescHiSw128Sbo1024;
        const uint32_t q_lo0 = tc::desc_lo(q_smem, 16);
        const uint32_t k_lo0 = tc::desc_lo(k_smem, 16);
        const uint32_t v_lo0 = tc::desc_lo(v_smem, kPfHalfBytes);
        auto issue_qk = [&](int t, int s) {   // S_t = Q_t K(stage s)^T, then commit to SFULL[t]
          tc::mma_ss_k128_commit(tmem + t * 128, tc::desc64(q_lo0 + t * (kPfTileBytes >> 4), desc_hi),
                                 tc::desc64(k_lo0 + s * (kPfTileBytes >> 4), desc_hi), idesc_qk, bar(BAR_SFULL + t));
        };
        // O_t (+)= P_t V(stage s); commit to `commit_bar` (ODONE[t] after the last PV of the step)
        auto issue_pv = [&](int t, int s, bool accum, int p_col, uint32_t commit_bar) {
          tc::mma_ts_k128_commit(tmem + 256 + t * 128, tmem + t * 128 + p_col,
                                 tc::desc64(v_lo0 + s * (kPfTileBytes >> 4), desc_hi), idesc_pv, accum, commit_bar);
        };
        tc::mbar_wait(bar(BAR_Q), 0, abort_flag, p.error_word, 3);
        tc::mbar_wait(bar(BAR_KFULL + 0), 0, abort_flag, p.error_word, 4);
        tc::fence_after_sync();
        for (int t = 0; t < nt; ++t) issue_qk(t, 0);
        tc::commit_elected(bar(BAR_KEMPTY + 0), 0, false);  // K stage 0 is free once QK(0) of both heads has run
        for (int j = 0; j < n_kv; ++j) {
          const int s = j % kPfStages;
          const uint32_t ph = (j / kPfStages) & 1;
          const bool more = j + 1 < n_kv;
          const int s1 = (j + 1) % kPfStages;
          tc::mbar_wait(bar(BAR_VFULL + s), ph, abort_flag, p.error_word, 5);
          if (more) tc::mbar_wait(bar(BAR_KFULL + s1), ((j + 1) / kPfStages) & 1, abort_flag, p.error_word, 6);
          for (int t = 0; t < nt; ++t) {
            tc::mbar_wait(bar(BAR_PREADY + t), j & 1, abort_flag, p.error_word, 7);
            tc::fence_after_sync();
            if (lane == 0) PF_STAMP(2 + t, j, 0);
            if (split_p) {   // P, then its rounding residue (see the softmax warps); the first commit is a spare arrival-free one
              issue_pv(t, s, j > 0, 0, bar(BAR_SPARE));
              issue_pv(t, s, true, 64, bar(BAR_ODONE + t));
            } else {
              issue_pv(t, s, j > 0, 0, bar(BAR_ODONE + t));
            }
            if (lane == 0) PF_STAMP(2 + t, j, 1);
            if (more) issue_qk(t, s1);
            if (lane == 0) PF_STAMP(2 + t, j, 2);
          }
          // V stage s is free when both PV(j) have run, K stage s1 when both QK(j+1) have
          tc::commit_elected(bar(BAR_VEMPTY + s), bar(BAR_KEMPTY + s1), more);
        }
        // After an abort nobody waits for the last MMAs: they must have run before tensor memory is freed.
        if (*abort_flag) {
          tc::commit_elected(bar(BAR_DRAIN), 0, false);
          tc::mbar_wait_timed(bar(BAR_DRAIN), 0);
        }
      }
    }
  } else {
    // ------------------------------ softmax warps ------------------------------
    tc::setmaxnreg_inc_232();
    const int t = warp >> 2;                       // 0: head A, 1: head B
    if (t == 0 || has_b) {
      const int row = (warp & 3) * 32 + lane;      // row of the tile = TMEM lane
      const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t s_addr = tmem + lane_addr + t * 128;
      const uint32_t o_addr = tmem + lane_addr + 256 + t * 128;
      float m_used = -INFINITY, l = 0.f;
      // Rare: the reference maximum of some row of this warp moved.  PV(j-1) must have landed in O
      // before O is scaled; PV(j) cannot start before this warp arrives at PREADY below.
      auto rescale_o = [&](float alpha, int j, float& l_ref) {
        tc::mbar_wait(bar(BAR_ODONE + t), (j - 1) & 1, abort_flag, p.error_word, 9);
        tc::fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[32];
          tc::tmem_ld32(o_addr + c * 32, ov);
          tc::wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tc::tmem_st32(o_addr + c * 32, ov);
        }
        tc::wait_st();
        l_ref *= alpha;
      };
      for (int j = 0; j < n_kv; ++j) {
        tc::mbar_wait(bar(BAR_SFULL + t), j & 1, abort_flag, p.error_word, 8);
        tc::fence_after_sync();
        if (tid == 0) PF_STAMP(0, j, 0);
        if (tid == 128) PF_STAMP(1, j, 0);
        // Keys of this tile sit at positions 128j + col, query row r at first_pos + r: a key is visible when
        // col <= r + shift.  Tiles that end at or before the first row's position need no mask at all.
        const int shift = first_pos - j * kPfTile;
        const bool diag = shift < kPfTile - 1;
        const int vis = row + shift;            // last visible column of this thread's row
        float sum = 0.f;
        if (!split_p) {
          // ---- fast path: the whole S row in registers, one wait for four loads ----
          uint32_t sv[4][32];
#pragma unroll
          for (int c = 0; c < 4; ++c) tc::tmem_ld32(s_addr + c * 32, sv[c]);
          tc::wait_ld();
          if (tid == 0) PF_STAMP(0, j, 1);
          if (diag) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (c * 32 + i > vis) sv[c][i] = 0xff800000u;  // -inf
          }
          // Row maximum: three-input max, eight independent chains (one chain of 128 dependent ops costs ~500 cycles).
          float mxs[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) mxs[i] = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 16; ++i)
              mxs[i & 7] = tc::max3(mxs[i & 7], __uint_as_float(sv[c][2 * i]), __uint_as_float(sv[c][2 * i + 1]));
          float mx = fmaxf(tc::max3(mxs[0], mxs[1], mxs[2]), tc::max3(mxs[3], mxs[4], mxs[5]));
          mx = tc::max3(mx, mxs[6], mxs[7]);
          mx *= p.scale_log2;  // scale > 0, so max commutes with it
          const bool grow = mx > m_used + kRescaleThreshold;
          if (j > 0 && __any_sync(0xffffffffu, grow)) rescale_o(grow ? ex2(m_used - mx) : 1.f, j, l);
          if (grow) m_used = mx;
          if (tid == 0) PF_STAMP(0, j, 2);
          // exp2(s * scale - m) on packed pairs; a share of the pairs goes to the FMA-pipe polynomial so that
          // the special-function unit (the slowest pipe of the tile) does not see every exponential
          const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m_used, -m_used);
          float2 sums[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int c = 2 * c2 + (i >> 4), k = (i & 15) * 2;
              const float2 x = tc::fma2(make_float2(__uint_as_float(sv[c][k]), __uint_as_float(sv[c][k + 1])), sc2, nm2);
              float2 e;
              if (MV_PF_POLY_PRED(i)) {
                e = tc::ex2_poly2(x);
              } else {
                e.x = tc::ex2_mufu(x.x);
                e.y = tc::ex2_mufu(x.y);
              }
              sums[i & 3] = tc::add2(sums[i & 3], e);
              pk[i] = pack2<T>(e.x, e.y);
            }
            tc::tmem_st32(s_addr + c2 * 32, pk);   // P over the first 64 columns of S (all of S is in registers)
          }
          const float2 s01 = tc::add2(sums[0], sums[1]), s23 = tc::add2(sums[2], sums[3]);
          sum = (s01.x + s01.y) + (s23.x + s23.y);
        } else {
          // ---- rows with few keys, bf16: two passes over S, P plus its rounding residue ----
          float mx = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t sv[32];
            tc::tmem_ld32(s_addr + c * 32, sv);
            tc::wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i)
              mx = fmaxf(mx, (diag && c * 32 + i > vis) ? -INFINITY : __uint_as_float(sv[i]));
          }
          mx *= p.scale_log2;
          const bool grow = mx > m_used + kRescaleThreshold;
          if (j > 0 && __any_sync(0xffffffffu, grow)) rescale_o(grow ? ex2(m_used - mx) : 1.f, j, l);
          if (grow) m_used = mx;
          uint32_t plo[32];
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            uint32_t sa[32], sb[32], pk[32];
            tc::tmem_ld32(s_addr + c2 * 64, sa);
            tc::tmem_ld32(s_addr + c2 * 64 + 32, sb);
            tc::wait_ld();
            // once the second half of S has been read, the residue of the first half can go over columns 64..95
            if (c2 == 1) tc::tmem_st32(s_addr + 64, plo);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int k = (i & 15) * 2, col = c2 * 64 + 2 * i;
              float s0 = __uint_as_float(i < 16 ? sa[k] : sb[k]);
              float s1 = __uint_as_float(i < 16 ? sa[k + 1] : sb[k + 1]);
              if (diag && col > vis) s0 = -INFINITY;
              if (diag && col + 1 > vis) s1 = -INFINITY;
              const float p0 = ex2(fmaf(s0, p.scale_log2, -m_used));
              const float p1 = ex2(fmaf(s1, p.scale_log2, -m_used));
              pk[i] = pack2<T>(p0, p1);
              const float2 hi = Elem<T>::to_f2(*reinterpret_cast<typename Elem<T>::T2*>(&pk[i]));
              plo[i] = pack2<T>(p0 - hi.x, p1 - hi.y);
              sum += p0 + p1;
            }
            tc::tmem_st32(s_addr + c2 * 32, pk);
          }
          tc::tmem_st32(s_addr + 96, plo);
        }
        l += sum;
        if (tid == 0) PF_STAMP(0, j, 3);
        tc::wait_st();
        tc::fence_before_sync();
        if (!(p.inject == 1 && t == 0 && j == 0 && blockIdx.x == 0 && blockIdx.y == 0)) tc::mbar_arrive(bar(BAR_PREADY + t));
        if (tid == 0) PF_STAMP(0, j, 4);
        if (tid == 128) PF_STAMP(1, j, 4);
      }
      // ---- epilogue: O / l -> global ----
      tc::mbar_wait(bar(BAR_ODONE + t), (n_kv - 1) & 1, abort_flag, p.error_word, 10);
      tc::fence_after_sync();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool store = q0 + row < seq_len;
      T* orow = static_cast<T*>(p.out) + static_cast<int64_t>(seq_start + q0 + row) * p.out_stride_tok +
                static_cast<int64_t>(head_a + t) * kPfD;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t ov[32];
        tc::tmem_ld32(o_addr + c * 32, ov);
        tc::wait_ld();
        if (store) {
          auto packed = [&](int i) {   // eight outputs, columns 32c + 8i ..
            uint4 w;
            w.x = pack2<T>(__uint_as_float(ov[8 * i + 0]) * inv_l, __uint_as_float(ov[8 * i + 1]) * inv_l);
            w.y = pack2<T>(__uint_as_float(ov[8 * i + 2]) * inv_l, __uint_as_float(ov[8 * i + 3]) * inv_l);
            w.z = pack2<T>(__uint_as_float(ov[8 * i + 4]) * inv_l, __uint_as_float(ov[8 * i + 5]) * inv_l);
            w.w = pack2<T>(__uint_as_float(ov[8 * i + 6]) * inv_l, __uint_as_float(ov[8 * i + 7]) * inv_l);
            return w;
          };
          // a thread writes its own 256-byte row: whole 32-byte sectors when the output allows it (a warp-wide
          // store touches 32 different lines either way, so fewer, larger requests is what counts)
#pragma unroll
          for (int i = 0; i < 4; i += 2) {
            if (p.out_align32) {
              st_global32(orow + c * 32 + i * 8, packed(i), packed(i + 1));
            } else {
              st_global16(orow + c * 32 + i * 8, packed(i));
              st_global16(orow + c * 32 + i * 8 + 8, packed(i + 1));
            }
          }
        }
      }
    }
  }
  // ---- teardown: everyone is done with tensor memory before it is freed ----
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// Persistent form of the same kernel: one CTA per SM works through units (query tile x head pair).  The first
// unit of a CTA is its block index, further ones come from a counter in device memory (whoever is free takes
// the next; the KV loops of the units differ in length by up to the number of tiles of a sequence).  Tensor
// memory and the mbarriers are set up once; every role treats its units as one continuous stream of KV steps
// (ring stages and barrier phases run on across units), so the producer's loads and the first S = Q K^T of the
// next unit are under way while the softmax warps write the current unit's output, and nothing is torn down
// or set up between units.
//   Units: the producer warp looks a unit up (binary search in the tiles-before-sequence prefix sums, which
//   live in shared memory behind the tile buffers) and publishes what the other roles need of it in a ring of
//   descriptors (UFULL / UEMPTY), one unit ahead of the MMA warp.
//   Q buffer: QEMPTY is committed behind the unit's last QK, the producer waits for it before the next Q.
//   O accumulators: OFREE[t] gets 128 arrivals when head t's softmax warps have read O in the epilogue;
//   the MMA warp waits for it before the first PV of head t's next unit.
//   Output: each softmax warp transposes its 32 rows through a staging buffer so that a store instruction
//   writes whole 128-byte lines (a thread storing its own row makes 32 lines per instruction, and the stores
//   of one unit then hold up every shared-memory access of the SM for about 2,000 cycles).
//   Code size: the MMA warp shares an instruction cache with the large softmax loop.  Its waits are the compact
//   form (rolled spin, the long-wait part a call) and the two warps with few registers keep their loops small;
//   with unrolled waits the same kernel was 25 % slower on the 32-sequence benchmark.
// ---------------------------------------------------------------------------------------------
enum { PB_Q = 0, PB_QEMPTY = 1, PB_KFULL = 2, PB_KEMPTY = 4, PB_VFULL = 6, PB_VEMPTY = 8, PB_SFULL = 10, PB_PREADY = 12,
       PB_ODONE = 14, PB_OFREE = 16, PB_SPARE = 18, PB_DRAIN = 19, PB_UFULL = 20, PB_UEMPTY = 24, PB_COUNT = 28 };
constexpr int kPfOutWarpBytes = 32 * 128;                    // output staging of one softmax warp: 32 rows x 64 outputs
constexpr int kPfOutStageBytes = 8 * kPfOutWarpBytes;
__device__ __forceinline__ void st_shared16(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_shared16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
constexpr int kPfUnitRing = 4;      // units handed from the producer warp to the other roles ahead of time
constexpr int kPfSchedSlots = 1024;  // launches that can be in flight with a work counter of their own
// Work counters of the persistent launches: [slot][0] = units handed out beyond the first one per CTA,
// [slot][1] = CTAs that have finished.  Zero between launches: the last CTA of a launch clears its slot.
static __device__ unsigned int g_pf_sched[kPfSchedSlots][2];

template <typename T>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_persistent_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[PB_COUNT];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_scan[16];
  __shared__ int s_abort;
  __shared__ int s_sticky;
  __shared__ __align__(16) int s_unit[kPfUnitRing][8];   // unit descriptors, see UnitDesc

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  PF_TRACE_INIT();
  if (tid == 0) PF_STAMP(0, 31, 0);
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;                                  // [head 2][half 2][128][128B]
  const uint32_t k_smem = q_smem + 2 * kPfTileBytes;                  // [stage][half][128][128B]
  const uint32_t v_smem = k_smem + kPfStages * kPfTileBytes;
  // output staging of the softmax warps (32 rows x 128 B each), then the tiles before sequence i (num_seqs + 1)
  const uint32_t o_smem = v_smem + kPfStages * kPfTileBytes;
  int* s_pref = reinterpret_cast<int*>(smem_raw + (smem_base - smem_u32(smem_raw)) + 2 * kPfTileBytes +
                                       2 * kPfStages * kPfTileBytes + kPfOutStageBytes);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  volatile int* abort_flag = &s_abort;

  if (tid == 0) {
    s_abort = 0;
    s_sticky = *reinterpret_cast<volatile int*>(p.error_word);  // read once so that the whole CTA agrees
    s_pref[0] = 0;
  }
  __syncthreads();
  {  // block-wide inclusive scan of the tiles per sequence
    int carry = 0;
    for (int base = 0; base < p.num_seqs; base += kPfThreads) {
      const int s = base + tid;
      int n = 0;
      if (s < p.num_seqs) {
        const int len = p.cu_seqlens[s + 1] - p.cu_seqlens[s];
        n = len > 0 ? (len + kPfTile - 1) / kPfTile : 0;
      }
      int incl = n;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += v;
      }
      if (lane == 31) s_scan[warp] = incl;
      __syncthreads();
      int wofs = 0, tot = 0;
#pragma unroll
      for (int w2 = 0; w2 < kPfThreads / 32; ++w2) {
        const int v = s_scan[w2];
        if (w2 < warp) wofs += v;
        tot += v;
      }
      if (s < p.num_seqs) s_pref[s + 1] = carry + wofs + incl;
      carry += tot;
      __syncthreads();
    }
  }
  if (tid == 0) PF_STAMP(0, 31, 1);
  const int n_tiles = s_pref[p.num_seqs];
  const int ydim = p.num_kv_heads * p.pairs;
  const long long total_units = static_cast<long long>(n_tiles) * ydim;
  // A wait that ran out anywhere (this launch or an earlier one) leaves the error word set: return at once.
  unsigned int* sched = g_pf_sched[p.sched_slot];
  auto cta_done = [&]() {   // one thread: count this CTA; the last one leaves the slot zeroed for its next launch
    if (atomicAdd(&sched[1], 1u) == gridDim.x - 1) {
      sched[0] = 0;
      sched[1] = 0;
      __threadfence();
    }
  };
  if (s_sticky != 0 || static_cast<long long>(blockIdx.x) >= total_units) {   // uniform over the CTA
    if (tid == 0) cta_done();
    return;
  }

  // Unit u = (head pair y, query tile x) in the order a grid of one CTA per unit would run them: x fastest, the
  // tiles of a sequence in descending order.  CTAs that run at the same time then work on the query tiles of a
  // few sequences for one KV head and share its K/V tiles in L2.  The first unit of a CTA is its block index;
  // further ones come from a counter (whoever is free takes the next: the KV loops differ in length by up to
  // the number of tiles of a sequence, and any fixed assignment leaves some SMs idle at the end).
  struct Unit {
    int seq, seq_start, seq_len, q0, first_pos, n_kv, kvh, head_a;
    bool has_b, split_p;
  };
  auto get_unit = [&](long long u) {
    Unit w;
    const int y = static_cast<int>(u / n_tiles), x = static_cast<int>(u - static_cast<long long>(y) * n_tiles);
    int lo = 0, hi = p.num_seqs - 1;                   // last sequence with s_pref[seq] <= x
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_pref[mid] <= x) lo = mid; else hi = mid - 1;
    }
    w.seq = lo;
    const int qtile = (s_pref[lo + 1] - s_pref[lo]) - 1 - (x - s_pref[lo]);
    w.kvh = y / p.pairs;
    const int pair = y - w.kvh * p.pairs;
    w.head_a = w.kvh * p.group + 2 * pair;
    w.has_b = 2 * pair + 1 < p.group;
    w.seq_start = p.cu_seqlens[lo];
    w.seq_len = p.cu_seqlens[lo + 1] - w.seq_start;
    w.q0 = qtile * kPfTile;
    const int n_cached = p.paged ? (p.cu_seqlens_k[lo + 1] - p.cu_seqlens_k[lo]) - w.seq_len : 0;
    w.first_pos = n_cached + w.q0;
    w.n_kv = (n_cached + min(w.q0 + kPfTile, w.seq_len) + kPfTile - 1) / kPfTile;
    w.split_p = std::is_same<T, __nv_bfloat16>::value && w.first_pos < kPfTile;
    return w;
  };
  // What the producer warp publishes for unit k of this CTA (slot k % kPfUnitRing): all the other roles need to
  // know about it, so that none of them has the lookup above on its critical path; n_kv = 0 says there is no
  // more work.  Every other warp says when it no longer needs the slot (UEMPTY, one arrival per warp): the MMA
  // warp once it has read the step count, a softmax warp after its epilogue, which reads the output rows' place
  // from the slot only then (four registers fewer across the KV loop).
  // What the MMA warp needs of a unit, in one register (the warp runs on 40): the number of KV steps and two flags.
  constexpr int kUnitHasB = 1 << 30, kUnitSplitP = 1 << 29, kUnitSteps = (1 << 29) - 1;
  auto next_unit_steps = [&](int kk) {
    const int slot = kk % kPfUnitRing;
    tc::mbar_wait_compact<true>(bar(PB_UFULL + slot), (kk / kPfUnitRing) & 1, abort_flag, p.error_word, 13);
    const int d = s_unit[slot][7];
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(bar(PB_UEMPTY + slot));
    return *abort_flag ? 0 : d;
  };

  if (tid == 0) {
    tc::mbar_init(bar(PB_Q), 1);
    tc::mbar_init(bar(PB_QEMPTY), 1);
    for (int s = 0; s < kPfStages; ++s) {
      tc::mbar_init(bar(PB_KFULL + s), 1);
      tc::mbar_init(bar(PB_KEMPTY + s), 1);
      tc::mbar_init(bar(PB_VFULL + s), 1);
      tc::mbar_init(bar(PB_VEMPTY + s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      tc::mbar_init(bar(PB_SFULL + t), 1);
      tc::mbar_init(bar(PB_PREADY + t), 128);
      tc::mbar_init(bar(PB_ODONE + t), 1);
      tc::mbar_init(bar(PB_OFREE + t), 128);
    }
    tc::mbar_init(bar(PB_SPARE), 1);   // takes commits that nobody waits for
    tc::mbar_init(bar(PB_DRAIN), 1);
    for (int i = 0; i < kPfUnitRing; ++i) {
      tc::mbar_init(bar(PB_UFULL + i), 1);
      tc::mbar_init(bar(PB_UEMPTY + i), 9);   // the MMA warp and the eight softmax warps
    }
    tc::mbar_fence_init();
  }
  if (warp == 8) {
    tc::tmem_alloc(smem_u32(&s_tmem_base), 512);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem_base;
  if (tid == 0) PF_STAMP(0, 31, 2);

  if (warp >= 8) {
    tc::setmaxnreg_dec_40();
    if (warp == 8) {
      // ------------------------------ TMA producer ------------------------------
      if (lane == 0) {
        tc::tma_prefetch_desc(&tmap_q);
        tc::tma_prefetch_desc(&tmap_k);
        tc::tma_prefetch_desc(&tmap_v);
        int gk = 0, k = 0;          // KV steps and units so far: ring stages and phases run on across units
        long long u = blockIdx.x;   // first unit; later ones from the counter
        for (;; ++k) {
          // publish unit k (or the end) for the other roles; the index of the one after it is claimed further
          // down, two KV steps before this unit's loads end
          const int slot = k % kPfUnitRing;
          if (k >= kPfUnitRing) tc::mbar_wait_compact<true>(bar(PB_UEMPTY + slot), ((k / kPfUnitRing) - 1) & 1, abort_flag, p.error_word, 14);
          const bool live = u < total_units && !*abort_flag;
          Unit w;
          if (live) {
            w = get_unit(u);
            *reinterpret_cast<int4*>(&s_unit[slot][0]) = make_int4(w.n_kv, w.first_pos, w.seq_start, w.seq_len);
            *reinterpret_cast<int4*>(&s_unit[slot][4]) = make_int4(w.q0, w.head_a, (w.has_b ? 1 : 0) | (w.split_p ? 2 : 0),
                                                                         w.n_kv | (w.has_b ? kUnitHasB : 0) | (w.split_p ? kUnitSplitP : 0));
          } else {
            s_unit[slot][0] = 0;
            s_unit[slot][7] = 0;
          }
          tc::mbar_arrive(bar(PB_UFULL + slot));     // release: the stores above are visible to whoever sees the phase
          if (!live) break;
          PF_STAMP(0, k, 0);
          PF_STAMP(0, k, 1);
          tc::mbar_wait_compact<true>(bar(PB_QEMPTY), (k & 1) ^ 1, abort_flag, p.error_word, 11);   // passes at once for k = 0
          PF_STAMP(0, k, 2);
          const int row0 = w.seq_start + w.q0;
          tc::mbar_expect_tx(bar(PB_Q), (w.has_b ? 2 : 1) * kPfTileBytes);
          for (int t = 0; t < (w.has_b ? 2 : 1); ++t)
            for (int h = 0; h < 2; ++h)
              tc::tma_load_3d(q_smem + t * kPfTileBytes + h * kPfHalfBytes, &tmap_q, 64 * h, w.head_a + t, row0, bar(PB_Q));
          PF_STAMP(0, k, 3);
          auto load_kv_tile = [&](const CUtensorMap* tm, uint32_t dst, int j, uint32_t full_bar) {
            if (!p.paged) {
              for (int h = 0; h < 2; ++h)
                tc::tma_load_3d(dst + h * kPfHalfBytes, tm, 64 * h, w.kvh, w.seq_start + j * kPfTile, full_bar);
              return;
            }
            const int32_t* table = p.block_tables + static_cast<int64_t>(w.seq) * p.bt_stride;
            for (int r = 0; r < kPfTile / p.box_rows; ++r) {
              const int pos = j * kPfTile + r * p.box_rows;
              const int blk = pos / p.block_size, off = pos - blk * p.block_size;
              const int phys = blk < p.max_blocks ? table[blk] : -1;
              const int slot = phys >= 0 ? phys * p.block_size + off : 0;
              for (int h = 0; h < 2; ++h)
                tc::tma_load_3d(dst + h * kPfHalfBytes + r * p.box_rows * 128, tm, 64 * h, w.kvh, slot, full_bar);
            }
          };
          for (int j = 0; j < w.n_kv; ++j, ++gk) {
            // Take the next unit as late as its latency allows (it passes under the waits of this unit's last
            // loads, and the MMA warp wants the unit by this unit's last step): a unit claimed earlier is one
            // that an idle SM cannot take at the end of the launch.
            if (j == max(w.n_kv - 2, 0)) u = static_cast<long long>(gridDim.x) + atomicAdd(&sched[0], 1u);
            const int s = gk % kPfStages;
            const uint32_t ph = ((gk / kPfStages) & 1) ^ 1;
            tc::mbar_wait_compact<true>(bar(PB_KEMPTY + s), ph, abort_flag, p.error_word, 1);
            tc::mbar_expect_tx(bar(PB_KFULL + s), kPfTileBytes);
            load_kv_tile(&tmap_k, k_smem + s * kPfTileBytes, j, bar(PB_KFULL + s));
            tc::mbar_wait_compact<true>(bar(PB_VEMPTY + s), ph, abort_flag, p.error_word, 2);
            tc::mbar_expect_tx(bar(PB_VFULL + s), kPfTileBytes);
            load_kv_tile(&tmap_v, v_smem + s * kPfTileBytes, j, bar(PB_VFULL + s));
            if (j == 0) PF_STAMP(0, k, 4);
          }
          PF_STAMP(0, k, 5);
#ifdef MV_PF_TRACE
          if (pf_tr && k < 32) pf_tr[(0 * 32 + k) * 8 + 7] = w.n_kv;
#endif
        }
        // After an abort nobody may be left to consume the loads already issued: give them time to land before
        // the CTA (and its shared memory) goes away.  A full barrier completes its phase when its bytes arrive.
        if (*abort_flag) {
          if (k > 0) tc::mbar_wait_timed(bar(PB_Q), (k - 1) & 1);
          for (int g2 = max(gk - kPfStages, 0); g2 < gk; ++g2) {
            tc::mbar_wait_timed(bar(PB_KFULL + g2 % kPfStages), (g2 / kPfStages) & 1);
            tc::mbar_wait_timed(bar(PB_VFULL + g2 % kPfStages), (g2 / kPfStages) & 1);
          }
        }
      }
    } else if (warp == 9) {
      // ------------------------------- MMA issuer -------------------------------
      const uint32_t idesc_qk = tc::instr_desc_f16(p.fmt, p.fmt, false, 128, 128);
      const uint32_t idesc_pv = tc::instr_desc_f16(p.fmt, p.fmt, true, 128, 128);
      const uint32_t desc_hi = tc::kDescHiSw128Sbo1024;
      const uint32_t q_lo0 = tc::desc_lo(q_smem, 16);
      const uint32_t k_lo0 = tc::desc_lo(k_smem, 16);
      const uint32_t v_lo0 = tc::desc_lo(v_smem, kPfHalfBytes);
      auto issue_qk = [&](int t, int s) {   // S_t = Q_t K(stage s)^T, then commit to SFULL[t]
        tc::mma_ss_k128_commit(tmem + t * 128, tc::desc64(q_lo0 + t * (kPfTileBytes >> 4), desc_hi),
                               tc::desc64(k_lo0 + s * (kPfTileBytes >> 4), desc_hi), idesc_qk, bar(PB_SFULL + t));
      };
      auto issue_pv = [&](int t, int s, bool accum, int p_col, uint32_t commit_bar) {
        tc::mma_ts_k128_commit(tmem + 256 + t * 128, tmem + t * 128 + p_col,
                               tc::desc64(v_lo0 + s * (kPfTileBytes >> 4), desc_hi), idesc_pv, accum, commit_bar);
      };
      int gk = 0, k = 0;             // KV steps and units so far
      // Barrier phases in one register (this warp runs on 40): bit t = parity of the steps so far of head t
      // (PREADY), bit 2 + t = parity of the units it has finished (OFREE), bit 4 + t = it has finished one.
      uint32_t phases = 0;
      // First QK of a unit whose first KV step has ring index g0.  With a single KV step it is also the last use
      // of the unit's Q tile.
      // PV of head t over V stage s (after the softmax warps' PREADY; at a unit's first step also after the
      // previous unit's O of this head has been read), commit to ODONE[t].
      auto pv_step = [&](int t, int s, bool first, bool split_p) {
        tc::mbar_wait_compact<true>(bar(PB_PREADY + t), (phases >> t) & 1u, abort_flag, p.error_word, 7);
        if (first && ((phases >> (4 + t)) & 1u))
          tc::mbar_wait_compact<true>(bar(PB_OFREE + t), ((phases >> (2 + t)) & 1u) ^ 1u, abort_flag, p.error_word, 12);
        tc::fence_after_sync();
        if (split_p) {
          issue_pv(t, s, !first, 0, bar(PB_SPARE));
          issue_pv(t, s, true, 64, bar(PB_ODONE + t));
        } else {
          issue_pv(t, s, !first, 0, bar(PB_ODONE + t));
        }
        phases ^= 1u << t;
      };
      int cur = next_unit_steps(0);
      if (cur != 0) {
        if (lane == 0) PF_STAMP(1, 0, 0);
        tc::mbar_wait_compact<true>(bar(PB_Q), 0, abort_flag, p.error_word, 3);
        tc::mbar_wait_compact<true>(bar(PB_KFULL + 0), 0, abort_flag, p.error_word, 4);
        tc::fence_after_sync();
        issue_qk(0, 0);
        if (cur & kUnitHasB) issue_qk(1, 0);
        // K stage is free once QK(0) of both heads has run; with a single KV step so is the Q buffer
        tc::commit_elected(bar(PB_KEMPTY + 0), bar(PB_QEMPTY), (cur & kUnitSteps) == 1);
      }
      while (cur != 0) {
        const int n_kv = cur & kUnitSteps;
        const bool has_b = (cur & kUnitHasB) != 0, split_p = (cur & kUnitSplitP) != 0;
        // ---- all steps but the last: PV(j) and QK(j + 1) of each head in turn ----
        for (int j = 0; j + 1 < n_kv; ++j, ++gk) {
          const int s = gk % kPfStages, s1 = s ^ 1;
          tc::mbar_wait_compact<true>(bar(PB_VFULL + s), (gk / kPfStages) & 1, abort_flag, p.error_word, 5);
          tc::mbar_wait_compact<true>(bar(PB_KFULL + s1), ((gk + 1) / kPfStages) & 1, abort_flag, p.error_word, 6);
          if (lane == 0) PF_STEP(k, 0, j, 0);
          pv_step(0, s, j == 0, split_p);
          if (lane == 0) PF_STEP(k, 0, j, 1);
          issue_qk(0, s1);
          if (lane == 0) PF_STEP(k, 0, j, 2);
          if (has_b) {
            pv_step(1, s, j == 0, split_p);
            if (lane == 0) PF_STEP(k, 0, j, 3);
            issue_qk(1, s1);
            if (lane == 0) PF_STEP(k, 0, j, 4);
          }
          // V stage s is free when both PV(j) have run, K stage s1 when both QK(j+1) have
          tc::commit_elected(bar(PB_VEMPTY + s), bar(PB_KEMPTY + s1), true);
          if (j + 2 == n_kv) tc::commit_elected(bar(PB_QEMPTY), 0, false);   // that was the unit's last QK
        }
        // ---- the last step: behind the unit's last PVs goes the first QK of the NEXT unit, so that its scores are
        // there when the softmax warps come back from storing this unit's output.  (Putting each head's QK
        // directly behind that head's PV was measured and is a few per cent slower.) ----
        {
          const int s = gk % kPfStages, s1 = s ^ 1;
          tc::mbar_wait_compact<true>(bar(PB_VFULL + s), (gk / kPfStages) & 1, abort_flag, p.error_word, 5);
          pv_step(0, s, n_kv == 1, split_p);
          if (has_b) pv_step(1, s, n_kv == 1, split_p);
          tc::commit_elected(bar(PB_VEMPTY + s), 0, false);   // V stage s is free when both PV have run
          if (lane == 0) PF_STAMP(1, k, 6);
          const int nxt = next_unit_steps(k + 1);
          if (nxt != 0) {
            if (lane == 0) PF_STAMP(1, k + 1, 0);
            tc::mbar_wait_compact<true>(bar(PB_Q), (k + 1) & 1, abort_flag, p.error_word, 3);
            if (lane == 0) PF_STAMP(1, k + 1, 1);
            tc::mbar_wait_compact<true>(bar(PB_KFULL + s1), ((gk + 1) / kPfStages) & 1, abort_flag, p.error_word, 4);
            if (lane == 0) PF_STAMP(1, k + 1, 2);
            tc::fence_after_sync();
            issue_qk(0, s1);
            if (lane == 0) PF_STAMP(1, k + 1, 5);
          }
          if (lane == 0) PF_STAMP(1, k + 1, 7);
          if (nxt & kUnitHasB) issue_qk(1, s1);
          // with a single KV step the next unit's first QK is also the last use of its Q tile
          if (nxt != 0) tc::commit_elected(bar(PB_KEMPTY + s1), bar(PB_QEMPTY), (nxt & kUnitSteps) == 1);
          if (lane == 0) PF_STAMP(1, k + 1, 3);
          ++gk;
          phases = (phases ^ (has_b ? 0xcu : 0x4u)) | (has_b ? 0x30u : 0x10u);
          cur = nxt;
          ++k;
        }
      }
      // After an abort nobody waits for the last MMAs: they must have run before tensor memory is freed.
      if (*abort_flag) {
        tc::commit_elected(bar(PB_DRAIN), 0, false);
        tc::mbar_wait_timed(bar(PB_DRAIN), 0);
      }
    }
  } else {
    // ------------------------------ softmax warps ------------------------------
    tc::setmaxnreg_inc_232();
    const int t = warp >> 2;                       // 0: head A, 1: head B
    const int row = (warp & 3) * 32 + lane;        // row of the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem + lane_addr + t * 128;
    const uint32_t o_addr = tmem + lane_addr + 256 + t * 128;
    int g = 0;                                     // KV steps of this head so far (barrier phases)
    const uint32_t o_stage = o_smem + warp * kPfOutWarpBytes;   // this warp's 32 rows x 128 B
    for (int ku = 0;; ++ku) {
      const int slot = ku % kPfUnitRing;
      tc::mbar_wait_compact<false>(bar(PB_UFULL + slot), (ku / kPfUnitRing) & 1, abort_flag, p.error_word, 13);
      const int n_kv = *abort_flag ? 0 : s_unit[slot][0];
      if (n_kv == 0) break;
      if ((warp & 3) == 0 && lane == 0) PF_STAMP(2 + t, ku, 0);
      const int first_pos = s_unit[slot][1], flags = s_unit[slot][6];
      const bool split_p = (flags & 2) != 0;
      if (t == 1 && !(flags & 1)) {
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(bar(PB_UEMPTY + slot));
        continue;
      }
      float m_used = -INFINITY, l = 0.f;
      // Rare: the reference maximum of some row of this warp moved.  PV of the previous step must have landed
      // in O before O is scaled; the next PV cannot start before this warp arrives at PREADY below.
      auto rescale_o = [&](float alpha, int gg, float& l_ref) {
        tc::mbar_wait_compact<false>(bar(PB_ODONE + t), (gg - 1) & 1, abort_flag, p.error_word, 9);
        tc::fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[32];
          tc::tmem_ld32(o_addr + c * 32, ov);
          tc::wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tc::tmem_st32(o_addr + c * 32, ov);
        }
        tc::wait_st();
        l_ref *= alpha;
      };
        for (int j = 0; j < n_kv; ++j) {
          tc::mbar_wait_compact<false>(bar(PB_SFULL + t), g & 1, abort_flag, p.error_word, 8);
          if ((warp & 3) == 0 && lane == 0 && j == 0) PF_STAMP(2 + t, ku, 2);
          if ((warp & 3) == 0 && lane == 0) PF_STEP(ku, 1 + t, j, 0);
          tc::fence_after_sync();
          // Keys of this tile sit at positions 128j + col, query row r at first_pos + r: a key is visible when
          // col <= r + shift.  Tiles that end at or before the first row's position need no mask at all.
          const int shift = first_pos - j * kPfTile;
          const bool diag = shift < kPfTile - 1;
          const int vis = row + shift;            // last visible column of this thread's row
          float sum = 0.f;
          if (!split_p) {
            // ---- fast path: the whole S row in registers, one wait for four loads ----
            uint32_t sv[4][32];
  #pragma unroll
            for (int c = 0; c < 4; ++c) tc::tmem_ld32(s_addr + c * 32, sv[c]);
            tc::wait_ld();
            if (diag) {
  #pragma unroll
              for (int c = 0; c < 4; ++c)
  #pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (c * 32 + i > vis) sv[c][i] = 0xff800000u;  // -inf
            }
            // Row maximum: three-input max, eight independent chains (one chain of 128 dependent ops costs ~500 cycles).
            float mxs[8];
  #pragma unroll
            for (int i = 0; i < 8; ++i) mxs[i] = -INFINITY;
  #pragma unroll
            for (int c = 0; c < 4; ++c)
  #pragma unroll
              for (int i = 0; i < 16; ++i)
                mxs[i & 7] = tc::max3(mxs[i & 7], __uint_as_float(sv[c][2 * i]), __uint_as_float(sv[c][2 * i + 1]));
            float mx = fmaxf(tc::max3(mxs[0], mxs[1], mxs[2]), tc::max3(mxs[3], mxs[4], mxs[5]));
            mx = tc::max3(mx, mxs[6], mxs[7]);
            mx *= p.scale_log2;  // scale > 0, so max commutes with it
            const bool grow = mx > m_used + kRescaleThreshold;
            if (j > 0 && __any_sync(0xffffffffu, grow)) rescale_o(grow ? ex2(m_used - mx) : 1.f, g, l);
            if (grow) m_used = mx;
            // exp2(s * scale - m) on packed pairs; a share of the pairs goes to the FMA-pipe polynomial so that
            // the special-function unit (the slowest pipe of the tile) does not see every exponential
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m_used, -m_used);
            float2 sums[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
  #pragma unroll
            for (int c2 = 0; c2 < 2; ++c2) {
              uint32_t pk[32];
  #pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int c = 2 * c2 + (i >> 4), k = (i & 15) * 2;
                const float2 x = tc::fma2(make_float2(__uint_as_float(sv[c][k]), __uint_as_float(sv[c][k + 1])), sc2, nm2);
                float2 e;
                if (MV_PF_POLY_PRED(i)) {
                  e = tc::ex2_poly2(x);
                } else {
                  e.x = tc::ex2_mufu(x.x);
                  e.y = tc::ex2_mufu(x.y);
                }
                sums[i & 3] = tc::add2(sums[i & 3], e);
                pk[i] = pack2<T>(e.x, e.y);
              }
              tc::tmem_st32(s_addr + c2 * 32, pk);   // P over the first 64 columns of S (all of S is in registers)
            }
            const float2 s01 = tc::add2(sums[0], sums[1]), s23 = tc::add2(sums[2], sums[3]);
            sum = (s01.x + s01.y) + (s23.x + s23.y);
          } else {
            // ---- rows with few keys, bf16: two passes over S, P plus its rounding residue ----
            float mx = -INFINITY;
  #pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t sv[32];
              tc::tmem_ld32(s_addr + c * 32, sv);
              tc::wait_ld();
  #pragma unroll
              for (int i = 0; i < 32; ++i)
                mx = fmaxf(mx, (diag && c * 32 + i > vis) ? -INFINITY : __uint_as_float(sv[i]));
            }
            mx *= p.scale_log2;
            const bool grow = mx > m_used + kRescaleThreshold;
            if (j > 0 && __any_sync(0xffffffffu, grow)) rescale_o(grow ? ex2(m_used - mx) : 1.f, g, l);
            if (grow) m_used = mx;
            uint32_t plo[32];
  #pragma unroll
            for (int c2 = 0; c2 < 2; ++c2) {
              uint32_t sa[32], sb[32], pk[32];
              tc::tmem_ld32(s_addr + c2 * 64, sa);
              tc::tmem_ld32(s_addr + c2 * 64 + 32, sb);
              tc::wait_ld();
              // once the second half of S has been read, the residue of the first half can go over columns 64..95
              if (c2 == 1) tc::tmem_st32(s_addr + 64, plo);
  #pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int k = (i & 15) * 2, col = c2 * 64 + 2 * i;
                float s0 = __uint_as_float(i < 16 ? sa[k] : sb[k]);
                float s1 = __uint_as_float(i < 16 ? sa[k + 1] : sb[k + 1]);
                if (diag && col > vis) s0 = -INFINITY;
                if (diag && col + 1 > vis) s1 = -INFINITY;
                const float p0 = ex2(fmaf(s0, p.scale_log2, -m_used));
                const float p1 = ex2(fmaf(s1, p.scale_log2, -m_used));
                pk[i] = pack2<T>(p0, p1);
                const float2 hi = Elem<T>::to_f2(*reinterpret_cast<typename Elem<T>::T2*>(&pk[i]));
                plo[i] = pack2<T>(p0 - hi.x, p1 - hi.y);
                sum += p0 + p1;
              }
              tc::tmem_st32(s_addr + c2 * 32, pk);
            }
            tc::tmem_st32(s_addr + 96, plo);
          }
          l += sum;
          tc::wait_st();
          tc::fence_before_sync();
          if (!(p.inject == 1 && t == 0 && g == 0 && blockIdx.x == 0)) tc::mbar_arrive(bar(PB_PREADY + t));
          if ((warp & 3) == 0 && lane == 0 && j == n_kv - 1) PF_STAMP(2 + t, ku, 3);
          if ((warp & 3) == 0 && lane == 0) PF_STEP(ku, 1 + t, j, 1);
          ++g;
        }

      // ---- epilogue: O / l -> global.  All of O is read into registers so that the accumulator can be handed
      // back (OFREE) at once.  The rows then go through this warp's staging buffer, 64 columns at a time, so that
      // each store instruction writes four whole 128-byte lines instead of 32 bytes of 32 different rows. ----
      tc::mbar_wait_compact<false>(bar(PB_ODONE + t), (g - 1) & 1, abort_flag, p.error_word, 10);
      if ((warp & 3) == 0 && lane == 0) PF_STAMP(2 + t, ku, 4);
      tc::fence_after_sync();
      uint32_t ov[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc::tmem_ld32(o_addr + c * 32, ov[c]);
      tc::wait_ld();
      tc::fence_before_sync();
      tc::mbar_arrive(bar(PB_OFREE + t));
      if ((warp & 3) == 0 && lane == 0) PF_STAMP(2 + t, ku, 5);
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const int2 pl0 = *reinterpret_cast<const int2*>(&s_unit[slot][2]);     // seq_start, seq_len
      const int2 pl1 = *reinterpret_cast<const int2*>(&s_unit[slot][4]);     // q0, head_a
      const int4 place = make_int4(pl0.x, pl0.y, pl1.x, pl1.y);
      const int seq_len = place.y;
      const int row0 = place.z + (warp & 3) * 32;              // first row of this warp within the sequence
      T* obase = static_cast<T*>(p.out) + static_cast<int64_t>(place.x + row0) * p.out_stride_tok +
                 static_cast<int64_t>(place.w + t) * kPfD;
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(bar(PB_UEMPTY + slot));
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {                       // this lane's row: eight chunks of eight outputs
          const int c = half * 2 + (ch >> 2), i0 = (ch & 3) * 8;
          uint4 x;
          x.x = pack2<T>(__uint_as_float(ov[c][i0 + 0]) * inv_l, __uint_as_float(ov[c][i0 + 1]) * inv_l);
          x.y = pack2<T>(__uint_as_float(ov[c][i0 + 2]) * inv_l, __uint_as_float(ov[c][i0 + 3]) * inv_l);
          x.z = pack2<T>(__uint_as_float(ov[c][i0 + 4]) * inv_l, __uint_as_float(ov[c][i0 + 5]) * inv_l);
          x.w = pack2<T>(__uint_as_float(ov[c][i0 + 6]) * inv_l, __uint_as_float(ov[c][i0 + 7]) * inv_l);
          st_shared16(o_stage + lane * 128 + ((ch ^ (lane & 7)) << 4), x);   // chunks swizzled by row: no bank conflicts
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {                          // eight lanes per row, four rows per instruction
          const int r = 4 * i + (lane >> 3), ch = lane & 7;
          const uint4 x = ld_shared16(o_stage + r * 128 + ((ch ^ (r & 7)) << 4));
          if (row0 + r < seq_len)
            st_global16(obase + static_cast<int64_t>(r) * p.out_stride_tok + half * 64 + ch * 8, x);
        }
        __syncwarp();
      }
      if ((warp & 3) == 0 && lane == 0) { PF_STAMP(2 + t, ku, 6); PF_STAMP(2 + t, ku, 7) ; }
    }
  }
  // ---- teardown: everyone is done with tensor memory before it is freed ----
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, 512);
  }
  if (tid == 0) cta_done();
  if (tid == 0) PF_STAMP(0, 31, 3);
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda dependency).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    else
      cudaGetLastError();
  }
  return fn;
}

// (tokens, heads, 128) tensor, token stride given; box = 64 elements x 1 head x 128 tokens, 128B swizzle.
static int make_tmap(CUtensorMap* m, const void* base, int64_t tokens, int heads, int64_t stride_tok, int dtype,
                     int box_rows = kPfTile) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(MV_ERR_CUDA, "prefill: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(kPfD), static_cast<cuuint64_t>(heads),
                              static_cast<cuuint64_t>(tokens)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(kPfD) * 2, static_cast<cuuint64_t>(stride_tok) * 2};
  const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(m, dtype == MV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MV_ERR_CUDA, "prefill: cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
  return MV_OK;
}

}  // namespace mv

#ifdef MV_PF_TRACE
extern "C" int mv_debug_prefill_trace(long long* buffer, int cta) {
  cudaMemcpyToSymbol(mv::g_pf_trace, &buffer, sizeof(buffer));
  cudaMemcpyToSymbol(mv::g_pf_trace_cta, &cta, sizeof(cta));
  return 0;
}
#endif

namespace mv {
static std::atomic<int> g_prefill_inject{0};

static std::atomic<int> g_prefill_form{0};   // measurement hook: 0 = choose, 1 = one CTA per tile, 2 = persistent
constexpr int kPfPersistentMaxSeqs = 320;   // the persistent form keeps num_seqs + 1 prefix sums in what shared
                                            // memory the tile buffers and the output staging leave

template <typename T>
static int launch_prefill_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const PrefillParams& p,
                            int64_t max_tiles, int num_seqs, int ydim, cudaStream_t st) {
  static bool attr_done[64][2] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int form = g_prefill_form.load();
  const bool fits = num_seqs <= kPfPersistentMaxSeqs;
  const bool persistent = form ? form == 2 : fits;
  const int smem = kPfSmemBytes + (persistent ? kPfOutStageBytes + ((num_seqs + 1) * 4 + 15) / 16 * 16 : 0);
  if (dev < 0 || dev >= 64 || !attr_done[dev][persistent]) {
    const cudaError_t e =
        persistent ? cudaFuncSetAttribute(prefill_persistent_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kPfSmemBytes + kPfOutStageBytes + (kPfPersistentMaxSeqs + 1) * 4 + 16)
                   : cudaFuncSetAttribute(prefill_varlen_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmemBytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(MV_ERR_CUDA, "prefill: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    if (dev >= 0 && dev < 64) attr_done[dev][persistent] = true;
  }
  if (persistent) {
    if (!fits) return fail(MV_ERR_LIMIT, "prefill: the persistent form takes at most %d sequences", kPfPersistentMaxSeqs);
    const int64_t units = max_tiles * ydim;
    const unsigned grid = static_cast<unsigned>(units < kNumSMs ? units : kNumSMs);   // one CTA per SM
    static std::atomic<unsigned> next_slot{0};
    PrefillParams pp = p;
    pp.sched_slot = static_cast<int>(next_slot.fetch_add(1) % kPfSchedSlots);
    prefill_persistent_kernel<T><<<grid, kPfThreads, smem, st>>>(tq, tk, tv, pp);
    return check_launch("prefill_persistent_kernel");
  }
  const dim3 grid(static_cast<unsigned>(max_tiles), static_cast<unsigned>(ydim));
  prefill_varlen_kernel<T><<<grid, kPfThreads, smem, st>>>(tq, tk, tv, p);
  return check_launch("prefill_varlen_kernel");
}

static int launch_prefill(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, PrefillParams& p,
                          int64_t total_tokens, int num_seqs, int num_kv_heads, int dtype, void* stream) {
  // Upper bound on the number of query tiles, from shapes only: no host sync.
  const int64_t max_tiles = (total_tokens + kPfTile - 1) / kPfTile + num_seqs;
  if (max_tiles > 0x7fffffffLL || static_cast<int64_t>(num_kv_heads) * p.pairs > 65535)
    return fail(MV_ERR_LIMIT, "prefill: grid too large");
  p.inject = g_prefill_inject.exchange(0);   // one launch only
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int ydim = num_kv_heads * p.pairs;
  return dtype == MV_F16 ? launch_prefill_t<__half>(tq, tk, tv, p, max_tiles, num_seqs, ydim, st)
                         : launch_prefill_t<__nv_bfloat16>(tq, tk, tv, p, max_tiles, num_seqs, ydim, st);
}
}  // namespace mv

// Measurement hook (not in the public header): 0 = choose the form from the problem, 1 = one CTA per query tile,
// 2 = persistent CTAs.
extern "C" int mv_debug_prefill_form(int form) {
  mv::g_prefill_form.store(form);
  return MV_OK;
}

// Test hook: the NEXT prefill launch of this process runs with the given fault injected on the host side of
// the launch (see PrefillParams::inject).  Nothing faults or hangs: a bounded wait runs out, the error word is
// set and the kernel returns.
extern "C" int mv_debug_prefill_inject(int mode) {
  mv::g_prefill_inject.store(mode);
  return MV_OK;
}

extern "C" int mv_prefill_varlen(void* out, const void* q, const void* k, const void* v, int64_t q_stride_tok,
                                 int64_t k_stride_tok, int64_t v_stride_tok, const int32_t* cu_seqlens, int num_seqs,
                                 int64_t total_tokens, int num_heads, int num_kv_heads, int head_dim, float scale,
                                 int* error_word, int dtype, void* stream) {
  using namespace mv;
  if (dtype != MV_F16 && dtype != MV_BF16) return fail(MV_ERR_DTYPE, "prefill: dtype %d", dtype);
  if (num_seqs < 0 || total_tokens < 0 || num_heads <= 0 || num_kv_heads <= 0)
    return fail(MV_ERR_SHAPE, "prefill: negative or zero size");
  if (num_heads % num_kv_heads != 0)
    return fail(MV_ERR_SHAPE, "prefill: num_heads %d is not a multiple of num_kv_heads %d", num_heads, num_kv_heads);
  if (head_dim != kPfD) return fail(MV_ERR_SHAPE, "prefill: head_dim %d is not 128", head_dim);
  if (num_seqs == 0 || total_tokens == 0) return MV_OK;
  if (!out || !q || !k || !v || !cu_seqlens || !error_word) return fail(MV_ERR_NULL, "prefill: null pointer");
  if (!aligned16(out) || !aligned16(q) || !aligned16(k) || !aligned16(v) || q_stride_tok % 8 || k_stride_tok % 8 ||
      v_stride_tok % 8)
    return fail(MV_ERR_ALIGN, "prefill: pointers and token strides must be 16-byte aligned");
  if (q_stride_tok < static_cast<int64_t>(num_heads) * head_dim ||
      k_stride_tok < static_cast<int64_t>(num_kv_heads) * head_dim ||
      v_stride_tok < static_cast<int64_t>(num_kv_heads) * head_dim)
    return fail(MV_ERR_SHAPE, "prefill: token stride smaller than a row");
  if (total_tokens > 0x7fffffffLL) return fail(MV_ERR_LIMIT, "prefill: more than 2^31 tokens");

  CUtensorMap tq, tk, tv;
  int rc = make_tmap(&tq, q, total_tokens, num_heads, q_stride_tok, dtype);
  if (rc) return rc;
  if ((rc = make_tmap(&tk, k, total_tokens, num_kv_heads, k_stride_tok, dtype))) return rc;
  if ((rc = make_tmap(&tv, v, total_tokens, num_kv_heads, v_stride_tok, dtype))) return rc;

  PrefillParams p;
  p.out = out;
  p.out_stride_tok = static_cast<int64_t>(num_heads) * head_dim;
  p.out_align32 = (reinterpret_cast<uintptr_t>(out) & 31u) == 0;   // rows are 256-byte multiples apart
  p.cu_seqlens = cu_seqlens;
  p.num_seqs = num_seqs;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.group = num_heads / num_kv_heads;
  p.pairs = (p.group + 1) / 2;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.fmt = dtype == MV_F16 ? 0 : 1;
  p.error_word = error_word;
  p.paged = 0;
  p.cu_seqlens_k = nullptr;
  p.block_tables = nullptr;
  p.bt_stride = 0;
  p.max_blocks = 0;
  p.block_size = kPfTile;
  p.box_rows = kPfTile;
  return launch_prefill(tq, tk, tv, p, total_tokens, num_seqs, num_kv_heads, dtype, stream);
}

extern "C" int mv_prefill_paged(void* out, const void* q, int64_t q_stride_tok, const void* k_cache,
                                const void* v_cache, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                const int32_t* block_tables, int64_t bt_stride, int max_blocks, int block_size,
                                int64_t num_blocks, int num_seqs, int64_t total_q_tokens, int num_heads,
                                int num_kv_heads, int head_dim, float scale, int* error_word, int dtype,
                                void* stream) {
  using namespace mv;
  if (dtype != MV_F16 && dtype != MV_BF16) return fail(MV_ERR_DTYPE, "prefill_paged: dtype %d", dtype);
  if (num_seqs < 0 || total_q_tokens < 0 || num_heads <= 0 || num_kv_heads <= 0 || max_blocks <= 0 || num_blocks <= 0)
    return fail(MV_ERR_SHAPE, "prefill_paged: negative or zero size");
  if (num_heads % num_kv_heads != 0)
    return fail(MV_ERR_SHAPE, "prefill_paged: num_heads %d is not a multiple of num_kv_heads %d", num_heads, num_kv_heads);
  if (head_dim != kPfD) return fail(MV_ERR_SHAPE, "prefill_paged: head_dim %d is not 128", head_dim);
  // one KV tile is 128 cache rows: whole blocks (block_size divides 128, multiple of 8) or part of one block
  if (block_size < 8 || block_size % 8 != 0 || (block_size % kPfTile != 0 && kPfTile % block_size != 0))
    return fail(MV_ERR_SHAPE, "prefill_paged: block_size %d must divide 128 (and be a multiple of 8) or be a multiple of 128",
                block_size);
  if (num_seqs == 0 || total_q_tokens == 0) return MV_OK;
  if (!out || !q || !k_cache || !v_cache || !cu_seqlens_q || !cu_seqlens_k || !block_tables || !error_word)
    return fail(MV_ERR_NULL, "prefill_paged: null pointer");
  if (!aligned16(out) || !aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || q_stride_tok % 8)
    return fail(MV_ERR_ALIGN, "prefill_paged: pointers and token strides must be 16-byte aligned");
  if (q_stride_tok < static_cast<int64_t>(num_heads) * head_dim)
    return fail(MV_ERR_SHAPE, "prefill_paged: token stride smaller than a row");
  if (bt_stride < max_blocks) return fail(MV_ERR_SHAPE, "prefill_paged: block table stride smaller than its width");
  const int64_t num_slots = num_blocks * block_size;
  if (total_q_tokens > 0x7fffffffLL || num_slots > 0x7fffffffLL) return fail(MV_ERR_LIMIT, "prefill_paged: more than 2^31 rows");
  const int box_rows = block_size < kPfTile ? block_size : kPfTile;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap(&tq, q, total_q_tokens, num_heads, q_stride_tok, dtype);
  if (rc) return rc;
  const int64_t cache_row = static_cast<int64_t>(num_kv_heads) * head_dim;
  if ((rc = make_tmap(&tk, k_cache, num_slots, num_kv_heads, cache_row, dtype, box_rows))) return rc;
  if ((rc = make_tmap(&tv, v_cache, num_slots, num_kv_heads, cache_row, dtype, box_rows))) return rc;
  PrefillParams p;
  p.out = out;
  p.out_stride_tok = static_cast<int64_t>(num_heads) * head_dim;
  p.out_align32 = (reinterpret_cast<uintptr_t>(out) & 31u) == 0;   // rows are 256-byte multiples apart
  p.cu_seqlens = cu_seqlens_q;
  p.num_seqs = num_seqs;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.group = num_heads / num_kv_heads;
  p.pairs = (p.group + 1) / 2;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.fmt = dtype == MV_F16 ? 0 : 1;
  p.error_word = error_word;
  p.paged = 1;
  p.cu_seqlens_k = cu_seqlens_k;
  p.block_tables = block_tables;
  p.bt_stride = bt_stride;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.box_rows = box_rows;
  return launch_prefill(tq, tk, tv, p, total_q_tokens, num_seqs, num_kv_heads, dtype, stream);
}
