// Tensor-parallel all-reduce over NVLink peer memory, fused with the residual
// add and the RMSNorm that follow it in a decoder layer, plus the local
// (single-rank) form of the same add + norm.
//
// What it replaces: the row-parallel linear layers of the reference end in
// `dist.all_reduce(result)` (src/myvllm/layers/linear.py:216-221), and every
// rank then runs the residual add and RMSNorm of layers/layernorm.py:19-22 on
// the full (tokens, hidden) activations.  Here the three are one kernel:
//
//   every rank r holds its partial sums x_r (rows, hidden) in a buffer that
//   its peers can read; rank r owns rows [r*ceil(rows/N), ...) and, for them,
//     o        = round(sum_p x_p[row])              (fp32, ranks in order 0..N-1)
//     residual = round(residual + o)                (kept row-sharded: only the owner stores it)
//     h        = round(residual * rsqrt(mean(residual^2) + eps) * gamma)
//   and writes h[row] into the gather buffer of EVERY rank (peer stores).
//
// "Two-shot": each row crosses NVLink once inbound (N-1 partial rows to the
// owner) and once outbound (the normalised row to N-1 peers), so a rank moves
// (N-1)/N of the message in each direction and the add + norm work shrinks by N.
// Plain peer loads and stores only: no TMA, no multicast, no library kernel
// ever sees a peer pointer.
//
// Synchronisation: two barriers per launch, one flag word per (rank, peer) each.
//   ready: block 0 of a rank (dispatched first) tells every peer "my partial sums are
//          complete" (their producer ran before this kernel in stream order); every
//          block waits for all peers' ready flags before it reads their buffers.
//   done:  a block that has stored its rows fences at system scope and counts itself
//          on a local counter; the LAST block of the rank tells every peer "all my
//          rows have landed" and alone waits for the peers' done flags, so the kernel
//          ends only when this rank's gather buffer is complete.
// A flag is a 32-bit generation number, one higher per launch; the generation lives in
// device memory and is advanced by the kernel itself, so a captured graph replays
// correctly.  No block waits for another block of its own GPU, and what a block waits
// for on a peer is sent by the peer's first block, so the grid size is free.
// Every wait is bounded by a timer (and an iteration cap): on expiry the block records a
// code in the caller's error word and returns; later launches return at once while the
// word is non-zero.  Nothing traps.
//
// A communicator can also be created in EMULATION mode: all N ranks' buffers
// live on one GPU and one cooperative launch runs every rank's blocks side by
// side (grid.y = N).  It exists so the protocol and the arithmetic can be
// tested on a single GPU; kernels that wait on one another are never
// launched separately on one device.
#include <new>
#include "common.cuh"

namespace mv {

constexpr int kMaxRanks = 8;
constexpr int kCommGridCap = 2 * kNumSMs;     // two 512-thread blocks per SM
constexpr size_t kCtrlBytes = 64 << 10;       // flags + counters + rank table, in front of the data buffers

// Barrier state at the start of every rank's region; every word sits in its own 128-byte line.
struct CommCtrl {
  uint32_t ready[kMaxRanks][32];   // ready[src][0]: written by rank src (remote store)
  uint32_t done[kMaxRanks][32];    // done[src][0]:  written by rank src (remote store)
  uint32_t gen[32];                // [0]: generation of the last completed launch (local)
  uint32_t finished[32];           // [0]: blocks of this launch whose rows have landed (local)
};

// One entry per rank slot (one slot in a real communicator, N in emulation).
struct CommSlot {
  const void* in[kMaxRanks];    // every rank's partial-sum buffer, indexed by rank
  void* out[kMaxRanks];         // every rank's gather buffer
  CommCtrl* ctrl[kMaxRanks];    // every rank's barrier state
  int rank, world;
  int skip_signal;              // test hook: this slot withholds its ready signal
};

struct Comm {
  int rank = 0, world = 1, slots = 1;
  bool emulated = false, connected = false;
  int64_t data_bytes = 0;
  size_t region_bytes = 0;
  char* region[kMaxRanks] = {};      // region[rank] is local; others are IPC mappings (or local in emulation)
  bool opened[kMaxRanks] = {};
  CommSlot* table_dev = nullptr;      // inside region[rank] (region[0] in emulation)
  unsigned long long timeout_ns = 0;
  int device = 0;
  int max_blocks = 0;                 // 0 = as many as the rows want; else a cap (mv_comm_set_max_blocks)
  char* stage = nullptr;              // staged form: peers' partial rows land here ((world-1) slots per rank slot)
  size_t stage_slot_bytes = 0;
};

// Control region layout (byte offsets inside a rank's region).
constexpr size_t kOffCtrl = 0;
constexpr size_t kOffTable = 4096;
static_assert(sizeof(CommCtrl) <= kOffTable, "barrier state overlaps the rank table");
static_assert(kOffTable + kMaxRanks * sizeof(CommSlot) <= kCtrlBytes, "control region too small");

static inline size_t round256(size_t x) { return (x + 255) & ~size_t(255); }

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_global16(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Waits until *flag has reached `gen`.  Returns false when the time limit (or the iteration cap behind
// it) ran out.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t gen, unsigned long long timeout_ns) {
  unsigned long long t0 = 0;
  for (uint32_t it = 1; it < (1u << 26); ++it) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - gen) >= 0) return true;
    if ((it & 63u) == 0) {
      const unsigned long long now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > timeout_ns) return false;
    }
  }
  return false;
}

template <typename T> struct Vec8 {
  // eight elements of a 16-byte vector as fp32
  static __device__ __forceinline__ void unpack(const uint4& u, float (&f)[8]) {
    const typename Elem<T>::T2* p = reinterpret_cast<const typename Elem<T>::T2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = Elem<T>::to_f2(p[i]);
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint4 u;
    typename Elem<T>::T2* p = reinterpret_cast<typename Elem<T>::T2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = Elem<T>::from_f2(f[2 * i], f[2 * i + 1]);
    return u;
  }
};

// Sums over the block of R floats per thread; every thread gets the results.  `red` holds 33*R floats.
template <int R>
__device__ __forceinline__ void block_sum_n(float (&v)[R], float* red) {
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[r] += __shfl_xor_sync(0xffffffffu, v[r], o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();                       // `red` may still be read by the previous iteration
  if (lane == 0)
#pragma unroll
    for (int r = 0; r < R; ++r) red[r * 33 + warp] = v[r];
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float s = lane < nwarps ? red[r * 33 + lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) red[r * 33 + 32] = s;
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) v[r] = red[r * 33 + 32];
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  float a[1] = {v};
  block_sum_n<1>(a, red);
  return a[0];
}

// ---------------------------------------------------------------------------------------------
// all-reduce + residual + RMSNorm across ranks
// ---------------------------------------------------------------------------------------------
// W = upper bound of the world size (sizes the register array of peer vectors), R = rows a block works
// on at once (more loads in flight when few peers contribute per row), VPT = 16-byte vectors per thread
// and row.
template <typename T, int W, int R, int VPT>
__global__ void __launch_bounds__(1024, 1)
allreduce_residual_rmsnorm_kernel(CommSlot* __restrict__ table, void* __restrict__ residual_base,
                                  int64_t residual_slot_stride, const void* __restrict__ gamma_, float eps, int rows,
                                  int hidden, unsigned long long timeout_ns, int* __restrict__ error_word) {
  __shared__ float red[33 * R];
  __shared__ int s_flag;
  __shared__ uint32_t s_gen;
  CommSlot& slot = table[blockIdx.y];
  const int rank = slot.rank, world = slot.world, tid = threadIdx.x;
  CommCtrl* mine = slot.ctrl[rank];
  if (tid == 0) {
    s_flag = *reinterpret_cast<volatile int*>(error_word) != 0;
    s_gen = *reinterpret_cast<volatile uint32_t*>(&mine->gen[0]) + 1;
  }
  __syncthreads();
  if (s_flag) return;                                               // an earlier wait ran out: do nothing
  const uint32_t gen = s_gen;

  // ---- ready: block 0 (dispatched first) signals the peers; every block waits for all peers ----
  if (tid < world && tid != rank) {
    if (blockIdx.x == 0 && !slot.skip_signal) st_release_sys(&slot.ctrl[tid]->ready[rank][0], gen);
    if (!wait_flag(&mine->ready[tid][0], gen, timeout_ns)) {
      atomicCAS(error_word, 0, 0x100 | tid);
      s_flag = 1;
    }
  }
  __syncthreads();
  if (s_flag) return;

  const int rows_per = (rows + world - 1) / world;
  const int lo = min(rows, rank * rows_per), hi = min(rows, lo + rows_per);
  const int nvec = hidden >> 3;
  T* residual = reinterpret_cast<T*>(residual_base) + blockIdx.y * residual_slot_stride;
  const uint4* gamma = reinterpret_cast<const uint4*>(gamma_);
  const float inv_hidden = 1.0f / static_cast<float>(hidden);

  for (int row0 = lo + blockIdx.x * R; row0 < hi; row0 += gridDim.x * R) {
    uint4 keep[R][VPT];
    float ss[R];
#pragma unroll
    for (int r = 0; r < R; ++r) ss[r] = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = tid + v * blockDim.x;
      if (c < nvec) {
        uint4 part[R][W];
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (row0 + r < hi) {
            const size_t off = static_cast<size_t>(row0 + r) * nvec + c;
#pragma unroll
            for (int p = 0; p < W; ++p)
              if (p < world) part[r][p] = ld_global16(reinterpret_cast<const uint4*>(slot.in[p]) + off);
          }
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (row0 + r < hi) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, f[8];
#pragma unroll
            for (int p = 0; p < W; ++p)
              if (p < world) {
                Vec8<T>::unpack(part[r][p], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += f[i];
              }
            // round the all-reduced value to the model dtype, then the residual add in that dtype: the
            // same roundings as `all_reduce(o); residual = residual + o`
            const uint4 o = Vec8<T>::pack(acc);
            Vec8<T>::unpack(o, acc);
            Vec8<T>::unpack(reinterpret_cast<const uint4*>(residual)[static_cast<size_t>(row0 + r - lo) * nvec + c], f);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += f[i];
            const uint4 rn = Vec8<T>::pack(acc);
            reinterpret_cast<uint4*>(residual)[static_cast<size_t>(row0 + r - lo) * nvec + c] = rn;
            keep[r][v] = rn;
            Vec8<T>::unpack(rn, f);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss[r] += f[i] * f[i];
          }
      }
    }
    block_sum_n<R>(ss, red);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = tid + v * blockDim.x;
      if (c < nvec) {
        float gf[8];
        Vec8<T>::unpack(gamma[c], gf);
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (row0 + r < hi) {
            const float rstd = rsqrtf(ss[r] * inv_hidden + eps);
            float h[8];
            Vec8<T>::unpack(keep[r][v], h);
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = h[i] * rstd * gf[i];
            const uint4 hv = Vec8<T>::pack(h);
            const size_t off = static_cast<size_t>(row0 + r) * nvec + c;
#pragma unroll
            for (int p = 0; p < W; ++p)
              if (p < world) {
                const int dst = rank + p < world ? rank + p : rank + p - world;   // spread the stores over the links
                st_global16(reinterpret_cast<uint4*>(slot.out[dst]) + off, hv);
              }
          }
      }
    }
  }

  // ---- done: this block's rows have landed everywhere; the last block of the rank tells the peers and
  // waits until every peer's rows have landed here ----
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();                      // this block's stores (ordered by the barrier) are performed
    const bool last = atomicAdd(&mine->finished[0], 1u) == gridDim.x - 1;
    if (last) {
      __threadfence_system();                    // ... and so are those of every block counted before this one
      for (int p = 0; p < world; ++p)
        if (p != rank)
          asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(&slot.ctrl[p]->done[rank][0]), "r"(gen) : "memory");
    }
    s_flag = last;
  }
  __syncthreads();
  if (!s_flag) return;
  if (tid < world && tid != rank)
    if (!wait_flag(&mine->done[tid][0], gen, timeout_ns)) atomicCAS(error_word, 0, 0x200 | tid);
  __syncthreads();
  if (tid == 0) {          // ready for the next launch (ordered before it by the kernel boundary)
    mine->finished[0] = 0;
    mine->gen[0] = gen;
  }
}

// ---------------------------------------------------------------------------------------------
// The same step with the two bulk transfers done by the copy engines ("staged" form)
// ---------------------------------------------------------------------------------------------
// For messages that are bound by the link (a prefill wave: 128 MiB): ready barrier -> cudaMemcpyAsync of the
// peers' partial rows of this rank's shard into local staging -> one local kernel (sum in rank order, residual,
// norm; the same arithmetic and roundings as the fused kernel) -> cudaMemcpyAsync of the normalised rows into
// every peer's gather buffer -> done barrier.  The SMs are free while the bytes move, so another stream's
// GEMMs run beside it (the fused kernel keeps one group of rows in flight per block and needs most SMs to
// fill the link).  The barriers are the fused kernel's, in two one-warp kernels: phase 0 = "my partial sums
// are complete" / wait for the peers'; phase 1 = "my rows have landed at every peer" / wait, then the
// generation advances.  Same flags, same generation counter, same bounded waits and error codes, so calls of
// both forms can follow each other on one communicator.
__global__ void __launch_bounds__(32)
comm_barrier_kernel(CommSlot* __restrict__ table, int phase, unsigned long long timeout_ns, int* __restrict__ error_word) {
  CommSlot& slot = table[0];
  const int rank = slot.rank, world = slot.world, tid = threadIdx.x;
  CommCtrl* mine = slot.ctrl[rank];
  if (*reinterpret_cast<volatile int*>(error_word) != 0) return;     // an earlier wait ran out: do nothing
  const uint32_t gen = *reinterpret_cast<volatile uint32_t*>(&mine->gen[0]) + 1;
  bool ok = true;
  if (phase == 1) __threadfence_system();
  if (tid < world && tid != rank) {
    if (phase == 0) {
      if (!slot.skip_signal) st_release_sys(&slot.ctrl[tid]->ready[rank][0], gen);
      ok = wait_flag(&mine->ready[tid][0], gen, timeout_ns);
      if (!ok) atomicCAS(error_word, 0, 0x100 | tid);
    } else {
      st_release_sys(&slot.ctrl[tid]->done[rank][0], gen);
      ok = wait_flag(&mine->done[tid][0], gen, timeout_ns);
      if (!ok) atomicCAS(error_word, 0, 0x200 | tid);
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (phase == 1 && ok && tid == 0) mine->gen[0] = gen;              // ready for the next launch
}

struct StagedRows {
  const void* src[kMaxRanks];   // src[p] = rank p's partial sums of the owned rows, first owned row first
};

// One block per owned row at a time: sum over the ranks in order, round, add the residual, round, norm.
template <typename T, int VPT>
__global__ void __launch_bounds__(1024, 1)
reduce_staged_kernel(const StagedRows in, int world, void* __restrict__ out_, void* __restrict__ residual_,
                     const void* __restrict__ gamma_, float eps, int n_rows, int hidden,
                     const int* __restrict__ error_word) {
  __shared__ float red[33];
  if (*reinterpret_cast<const volatile int*>(error_word) != 0) return;   // the ready barrier gave up
  const int tid = threadIdx.x, nvec = hidden >> 3;
  const uint4* gamma = reinterpret_cast<const uint4*>(gamma_);
  uint4* residual = reinterpret_cast<uint4*>(residual_);
  uint4* out = reinterpret_cast<uint4*>(out_);
  const float inv_hidden = 1.0f / static_cast<float>(hidden);
  for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {
    uint4 keep[VPT];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = tid + v * blockDim.x;
      if (c < nvec) {
        const size_t off = static_cast<size_t>(row) * nvec + c;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, f[8];
        for (int p = 0; p < world; ++p) {
          Vec8<T>::unpack(ld_global16(reinterpret_cast<const uint4*>(in.src[p]) + off), f);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += f[i];
        }
        const uint4 o = Vec8<T>::pack(acc);
        Vec8<T>::unpack(o, acc);
        Vec8<T>::unpack(residual[off], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
        const uint4 rn = Vec8<T>::pack(acc);
        residual[off] = rn;
        keep[v] = rn;
        Vec8<T>::unpack(rn, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss * inv_hidden + eps);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = tid + v * blockDim.x;
      if (c < nvec) {
        float gf[8], h[8];
        Vec8<T>::unpack(gamma[c], gf);
        Vec8<T>::unpack(keep[v], h);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = h[i] * rstd * gf[i];
        out[static_cast<size_t>(row) * nvec + c] = Vec8<T>::pack(h);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// local form: h = RMSNorm(x (+ residual)) for every row; the sum is stored for rows [res_lo, res_hi)
// ---------------------------------------------------------------------------------------------
template <typename T, int VPT>
__global__ void __launch_bounds__(1024, 1)
add_rmsnorm_kernel(void* __restrict__ out_, const void* __restrict__ x_, const void* residual_in_,
                   void* residual_out_, int res_lo, int res_hi, const void* __restrict__ gamma_, float eps, int rows,
                   int hidden) {
  __shared__ float red[33];
  const int tid = threadIdx.x, nvec = hidden >> 3;
  const uint4* x = reinterpret_cast<const uint4*>(x_);
  const uint4* rin = reinterpret_cast<const uint4*>(residual_in_);
  uint4* rout = reinterpret_cast<uint4*>(residual_out_);
  uint4* out = reinterpret_cast<uint4*>(out_);
  const uint4* gamma = reinterpret_cast<const uint4*>(gamma_);
  const float inv_hidden = 1.0f / static_cast<float>(hidden);
  uint4 g[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int c = tid + v * blockDim.x;
    g[v] = c < nvec ? gamma[c] : make_uint4(0, 0, 0, 0);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * nvec;
    const bool keep_res = rout != nullptr && row >= res_lo && row < res_hi;
    float keep[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = tid + v * blockDim.x;
      if (c < nvec) {
        float acc[8], f[8];
        uint4 rn = ld_stream16(x + off + c);
        if (rin != nullptr) {
          Vec8<T>::unpack(rn, acc);
          Vec8<T>::unpack(rin[off + c], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += f[i];
          rn = Vec8<T>::pack(acc);
        }
        if (keep_res) rout[static_cast<size_t>(row - res_lo) * nvec + c] = rn;
        Vec8<T>::unpack(rn, keep[v]);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += keep[v][i] * keep[v][i];
      }
    }
    const float rstd = rsqrtf(block_sum(ss, red) * inv_hidden + eps);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = tid + v * blockDim.x;
      if (c < nvec) {
        float gf[8], h[8];
        Vec8<T>::unpack(g[v], gf);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = keep[v][i] * rstd * gf[i];
        out[off + c] = Vec8<T>::pack(h);
      }
    }
  }
}

// SwiGLU activation: out[t, j] = silu(gu[t, j]) * gu[t, inter + j], one rounding (fp32 inside).
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_kernel(void* __restrict__ out_, const void* __restrict__ gu_, int64_t gu_stride, int64_t rows, int inter) {
  // blockIdx.y walks the rows, blockIdx.x * 256 + threadIdx.x the 16-byte column chunks: no division per element
  const int nvec = inter >> 3;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= nvec) return;
  const T* gu = reinterpret_cast<const T*>(gu_);
  for (int64_t row = blockIdx.y; row < rows; row += gridDim.y) {
    const T* base = gu + row * gu_stride;
    const uint4 a = ld_stream16(reinterpret_cast<const uint4*>(base) + c);
    const uint4 b = ld_stream16(reinterpret_cast<const uint4*>(base + inter) + c);
    float x[8], y[8], r[8];
    Vec8<T>::unpack(a, x);
    Vec8<T>::unpack(b, y);
#pragma unroll
    for (int k = 0; k < 8; ++k) r[k] = __fdividef(x[k], 1.0f + __expf(-x[k])) * y[k];
    reinterpret_cast<uint4*>(out_)[row * nvec + c] = Vec8<T>::pack(r);
  }
}

static int threads_for(int hidden, int* vpt) {
  const int nvec = hidden / 8;
  int threads = ((nvec + 31) / 32) * 32;
  *vpt = 1;
  if (threads > 1024) {
    *vpt = 2;
    threads = (((nvec + 1) / 2 + 31) / 32) * 32;
  }
  return threads;
}

// Rows a block works on at once: with few peers a row brings few remote bytes, so several rows keep the
// links busy; only worth it when there are rows enough to occupy every resident block that way.
static int comm_rows_at_once(int rows_per, int world, int vpt, int threads) {
  if (vpt != 1) return 1;
  const int cap = threads <= 512 ? kCommGridCap : kNumSMs;
  const int r = world <= 2 ? 4 : (world <= 4 ? 2 : 1);
  return rows_per >= r * cap ? r : 1;
}

static int comm_grid(int rows_per, int at_once, int threads) {
  const int cap = threads <= 512 ? kCommGridCap : kNumSMs;
  const int want = (rows_per + at_once - 1) / at_once;
  return want < 1 ? 1 : (want > cap ? cap : want);
}

static int cuda_fail(const char* what, cudaError_t e) {
  cudaGetLastError();
  return fail(MV_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// Staging of the staged form: per rank slot, one buffer per peer for that peer's partial sums of the slot's rows
// (a shard is ceil(rows/world) rows, so a slot takes data_bytes/world plus one row of slack).
static int alloc_stage(Comm* c) {
  c->stage_slot_bytes = round256(static_cast<size_t>(c->data_bytes) / c->world + 16384 * 2);
  const cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->stage), c->stage_slot_bytes * (c->world - 1) * c->slots);
  return e == cudaSuccess ? MV_OK : cuda_fail("comm: staging buffers", e);
}

static int write_table(Comm* c) {
  CommSlot host[kMaxRanks] = {};
  for (int s = 0; s < c->slots; ++s) {
    const int r = c->emulated ? s : c->rank;
    CommSlot& t = host[s];
    for (int p = 0; p < c->world; ++p) {
      t.in[p] = c->region[p] + kCtrlBytes;
      t.out[p] = c->region[p] + kCtrlBytes + round256(c->data_bytes);
      t.ctrl[p] = reinterpret_cast<CommCtrl*>(c->region[p] + kOffCtrl);
    }
    t.rank = r;
    t.world = c->world;
    t.skip_signal = 0;
  }
  const cudaError_t e = cudaMemcpy(c->table_dev, host, sizeof(CommSlot) * c->slots, cudaMemcpyHostToDevice);
  return e == cudaSuccess ? MV_OK : cuda_fail("comm: table upload", e);
}

}  // namespace mv

using namespace mv;

extern "C" int64_t mv_comm_handle_bytes(void) { return static_cast<int64_t>(sizeof(cudaIpcMemHandle_t)); }

extern "C" int mv_comm_create(int rank, int world, int64_t data_bytes, int timeout_ms, void** comm_out,
                              void* handle_out) {
  if (!comm_out || !handle_out) return fail(MV_ERR_NULL, "comm_create: null output pointer");
  if (world < 2 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(MV_ERR_SHAPE, "comm_create: rank %d of %d (2..%d ranks are supported)", rank, world, kMaxRanks);
  if (data_bytes <= 0 || timeout_ms <= 0) return fail(MV_ERR_SHAPE, "comm_create: data_bytes and timeout_ms must be positive");
  Comm* c = new (std::nothrow) Comm();
  if (!c) return fail(MV_ERR_CUDA, "comm_create: out of host memory");
  c->rank = rank;
  c->world = world;
  c->data_bytes = data_bytes;
  c->timeout_ns = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  c->region_bytes = kCtrlBytes + 2 * round256(static_cast<size_t>(data_bytes));
  cudaError_t e = cudaGetDevice(&c->device);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&c->region[rank]), c->region_bytes);
  if (e == cudaSuccess) e = cudaMemset(c->region[rank], 0, kCtrlBytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, c->region[rank]);
  if (e != cudaSuccess) {
    if (c->region[rank]) cudaFree(c->region[rank]);
    delete c;
    return cuda_fail("comm_create", e);
  }
  memcpy(handle_out, &h, sizeof(h));
  c->table_dev = reinterpret_cast<CommSlot*>(c->region[rank] + kOffTable);
  *comm_out = c;
  return MV_OK;
}

extern "C" int mv_comm_connect(void* comm, const void* all_handles) {
  Comm* c = static_cast<Comm*>(comm);
  if (!c || !all_handles) return fail(MV_ERR_NULL, "comm_connect: null argument");
  if (c->emulated || c->connected) return fail(MV_ERR_SHAPE, "comm_connect: communicator is already connected");
  const cudaIpcMemHandle_t* hs = static_cast<const cudaIpcMemHandle_t*>(all_handles);
  for (int p = 0; p < c->world; ++p) {
    if (p == c->rank) continue;
    void* ptr = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&ptr, hs[p], cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail("comm_connect: cudaIpcOpenMemHandle", e);
    c->region[p] = static_cast<char*>(ptr);
    c->opened[p] = true;
  }
  const int rc = write_table(c);
  if (rc) return rc;
  const int rs = alloc_stage(c);
  if (rs) return rs;
  c->connected = true;
  return MV_OK;
}

extern "C" int mv_comm_create_emulated(int world, int64_t data_bytes, int timeout_ms, void** comm_out) {
  if (!comm_out) return fail(MV_ERR_NULL, "comm_create_emulated: null output pointer");
  if (world < 2 || world > kMaxRanks) return fail(MV_ERR_SHAPE, "comm_create_emulated: 2..%d ranks are supported", kMaxRanks);
  if (data_bytes <= 0 || timeout_ms <= 0) return fail(MV_ERR_SHAPE, "comm_create_emulated: data_bytes and timeout_ms must be positive");
  Comm* c = new (std::nothrow) Comm();
  if (!c) return fail(MV_ERR_CUDA, "comm_create_emulated: out of host memory");
  c->world = world;
  c->slots = world;
  c->emulated = true;
  c->data_bytes = data_bytes;
  c->timeout_ns = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  c->region_bytes = kCtrlBytes + 2 * round256(static_cast<size_t>(data_bytes));
  cudaError_t e = cudaGetDevice(&c->device);
  char* all = nullptr;
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&all), c->region_bytes * world);
  if (e == cudaSuccess) e = cudaMemset(all, 0, c->region_bytes * world);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (all) cudaFree(all);
    delete c;
    return cuda_fail("comm_create_emulated", e);
  }
  for (int p = 0; p < world; ++p) c->region[p] = all + c->region_bytes * p;
  c->table_dev = reinterpret_cast<CommSlot*>(c->region[0] + kOffTable);
  int rc = write_table(c);
  if (!rc) rc = alloc_stage(c);
  if (rc) {
    cudaFree(all);
    delete c;
    return rc;
  }
  c->connected = true;
  *comm_out = c;
  return MV_OK;
}

extern "C" int mv_comm_destroy(void* comm) {
  Comm* c = static_cast<Comm*>(comm);
  if (!c) return MV_OK;
  cudaDeviceSynchronize();
  if (c->stage) cudaFree(c->stage);
  if (c->emulated) {
    cudaFree(c->region[0]);
  } else {
    for (int p = 0; p < c->world; ++p)
      if (c->opened[p]) cudaIpcCloseMemHandle(c->region[p]);
    cudaFree(c->region[c->rank]);
  }
  cudaGetLastError();
  delete c;
  return MV_OK;
}

extern "C" void* mv_comm_input(void* comm, int slot) {
  Comm* c = static_cast<Comm*>(comm);
  if (!c || slot < 0 || slot >= c->slots) return nullptr;
  return c->region[c->emulated ? slot : c->rank] + kCtrlBytes;
}

extern "C" void* mv_comm_output(void* comm, int slot) {
  Comm* c = static_cast<Comm*>(comm);
  if (!c || slot < 0 || slot >= c->slots) return nullptr;
  return c->region[c->emulated ? slot : c->rank] + kCtrlBytes + round256(static_cast<size_t>(c->data_bytes));
}

// Zeroes this rank's flags and generations (every rank of an emulated communicator).  Only valid while no
// rank has a launch in flight; every rank must reset before any rank launches again.
extern "C" int mv_comm_reset(void* comm) {
  Comm* c = static_cast<Comm*>(comm);
  if (!c) return fail(MV_ERR_NULL, "comm_reset: null communicator");
  cudaError_t e = cudaDeviceSynchronize();
  for (int s = 0; s < c->slots && e == cudaSuccess; ++s)
    e = cudaMemset(c->region[c->emulated ? s : c->rank], 0, kOffTable);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail("comm_reset", e);
  return write_table(c);
}

// Caps the grid of the following launches (0 = no cap).  A block of this kernel takes a whole SM; a caller that
// runs another stream's GEMMs beside a bandwidth-bound all-reduce (two prefill waves in flight) leaves them the
// other SMs this way.  Any grid size is valid: rows are strided over blocks and the barriers do not depend on it.
extern "C" int mv_comm_set_max_blocks(void* comm, int max_blocks) {
  Comm* c = static_cast<Comm*>(comm);
  if (!c) return fail(MV_ERR_NULL, "comm_set_max_blocks: null communicator");
  if (max_blocks < 0) return fail(MV_ERR_SHAPE, "comm_set_max_blocks: negative cap");
  c->max_blocks = max_blocks;
  return MV_OK;
}

// Test hook (not in the public header): the next launches of `slot` withhold their first-barrier signal, so
// the other ranks' bounded waits run out and report through the error word.  Cleared by mv_comm_reset.
extern "C" int mv_debug_comm_withhold_signal(void* comm, int slot) {
  Comm* c = static_cast<Comm*>(comm);
  if (!c || slot < 0 || slot >= c->slots) return fail(MV_ERR_SHAPE, "comm: bad slot");
  const int one = 1;
  const cudaError_t e = cudaMemcpy(&c->table_dev[slot].skip_signal, &one, sizeof(int), cudaMemcpyHostToDevice);
  return e == cudaSuccess ? MV_OK : cuda_fail("comm: withhold", e);
}

template <typename T, int W, int R, int VPT>
static int launch_allreduce_as(Comm* c, dim3 grid, int threads, void* residual, int64_t residual_slot_stride,
                               const void* gamma, float eps, int rows, int hidden, int* error_word, cudaStream_t stream) {
  CommSlot* table = c->table_dev;
  unsigned long long timeout = c->timeout_ns;
  if (!c->emulated) {
    allreduce_residual_rmsnorm_kernel<T, W, R, VPT><<<grid, threads, 0, stream>>>(table, residual, residual_slot_stride,
                                                                                  gamma, eps, rows, hidden, timeout, error_word);
    return check_launch("allreduce_residual_rmsnorm");
  }
  // emulation: the blocks of all ranks wait on one another, so they must be co-resident
  void* args[] = {&table, &residual, &residual_slot_stride, &gamma, &eps, &rows, &hidden, &timeout, &error_word};
  const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(&allreduce_residual_rmsnorm_kernel<T, W, R, VPT>),
                                                    grid, dim3(threads), args, 0, stream);
  if (e != cudaSuccess) return cuda_fail("allreduce_residual_rmsnorm (emulated, cooperative launch)", e);
  return MV_OK;
}

template <typename T>
static int launch_allreduce(Comm* c, void* residual, int64_t residual_slot_stride, const void* gamma, float eps, int rows,
                            int hidden, int* error_word, cudaStream_t stream) {
  int vpt = 1;
  const int threads = threads_for(hidden, &vpt);
  const int rows_per = (rows + c->world - 1) / c->world;
  int at_once = comm_rows_at_once(rows_per, c->world, vpt, threads);
  int blocks = comm_grid(rows_per, at_once, threads);
  if (c->emulated) {            // all ranks share one GPU: one row at a time, and few enough blocks to be co-resident
    at_once = 1;
    blocks = comm_grid(rows_per, 1, threads);
    if (blocks * c->slots > kNumSMs) blocks = kNumSMs / c->slots;
  }
  if (c->max_blocks > 0 && blocks > c->max_blocks) blocks = c->max_blocks;
  const dim3 grid(blocks, c->slots);
#define MV_AR(W, R, V) \
  return launch_allreduce_as<T, W, R, V>(c, grid, threads, residual, residual_slot_stride, gamma, eps, rows, hidden, error_word, stream)
  if (vpt == 2) {
    if (c->world <= 2) MV_AR(2, 1, 2);
    if (c->world <= 4) MV_AR(4, 1, 2);
    MV_AR(8, 1, 2);
  }
  if (c->world <= 2) {
    if (at_once == 4) MV_AR(2, 4, 1);
    MV_AR(2, 1, 1);
  }
  if (c->world <= 4) {
    if (at_once == 2) MV_AR(4, 2, 1);
    MV_AR(4, 1, 1);
  }
  MV_AR(8, 1, 1);
#undef MV_AR
}

extern "C" int mv_allreduce_residual_rmsnorm(void* comm, void* residual_shard, int64_t residual_slot_stride,
                                             const void* gamma, float eps, int rows, int hidden, int* error_word,
                                             int dtype, void* stream) {
  Comm* c = static_cast<Comm*>(comm);
  if (!c || !gamma || !error_word) return fail(MV_ERR_NULL, "allreduce_residual_rmsnorm: null argument");
  if (!c->connected) return fail(MV_ERR_SHAPE, "allreduce_residual_rmsnorm: communicator is not connected");
  if (!residual_shard) {      // allowed only for a rank that owns no row of this call
    const int per = rows > 0 ? (rows + c->world - 1) / c->world : 0;
    if (c->emulated || static_cast<int64_t>(c->rank) * per < rows)
      return fail(MV_ERR_NULL, "allreduce_residual_rmsnorm: residual_shard is null but this rank owns rows");
  }
  if (rows < 0 || hidden <= 0 || hidden % 8 != 0)
    return fail(MV_ERR_SHAPE, "allreduce_residual_rmsnorm: hidden (%d) must be a positive multiple of 8, rows >= 0", hidden);
  if (hidden > 16384) return fail(MV_ERR_LIMIT, "allreduce_residual_rmsnorm: hidden %d exceeds 16384", hidden);
  if (static_cast<int64_t>(rows) * hidden * 2 > c->data_bytes)
    return fail(MV_ERR_LIMIT, "allreduce_residual_rmsnorm: %d rows x %d exceed the communicator's %lld-byte buffers", rows,
                hidden, static_cast<long long>(c->data_bytes));
  if (!aligned16(residual_shard) || !aligned16(gamma) || (residual_slot_stride * 2) % 16 != 0)
    return fail(MV_ERR_ALIGN, "allreduce_residual_rmsnorm: residual and gamma must be 16-byte aligned");
  if (c->emulated) {
    const int rows_per = (rows + c->world - 1) / c->world;
    if (c->slots > 1 && residual_slot_stride < static_cast<int64_t>(rows_per) * hidden)
      return fail(MV_ERR_SHAPE, "allreduce_residual_rmsnorm: residual_slot_stride smaller than one rank's shard");
  }
  if (rows == 0) return MV_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == MV_F16) return launch_allreduce<__half>(c, residual_shard, residual_slot_stride, gamma, eps, rows, hidden, error_word, s);
  if (dtype == MV_BF16)
    return launch_allreduce<__nv_bfloat16>(c, residual_shard, residual_slot_stride, gamma, eps, rows, hidden, error_word, s);
  return fail(MV_ERR_DTYPE, "allreduce_residual_rmsnorm: dtype %d", dtype);
}

template <typename T>
static int launch_staged(Comm* c, void* residual_shard, int64_t residual_slot_stride, const void* gamma, float eps,
                         int rows, int hidden, int* error_word, cudaStream_t st) {
  int vpt = 1;
  const int threads = threads_for(hidden, &vpt);
  const int rows_per = (rows + c->world - 1) / c->world;
  const size_t row_bytes = static_cast<size_t>(hidden) * 2;
  if (static_cast<size_t>(rows_per) * row_bytes > c->stage_slot_bytes)
    return fail(MV_ERR_LIMIT, "allreduce_residual_rmsnorm_staged: a shard of %d rows exceeds the staging buffers", rows_per);
  const size_t out_off = kCtrlBytes + round256(static_cast<size_t>(c->data_bytes));
  cudaError_t e = cudaSuccess;
  if (!c->emulated) {
    comm_barrier_kernel<<<1, 32, 0, st>>>(c->table_dev, 0, c->timeout_ns, error_word);
    if (int rc = check_launch("comm_barrier_kernel")) return rc;
  }
  // Every rank slot in turn (one in a real communicator): pull, reduce, push.  In emulation all pulls come
  // first, then all reductions, then all pushes: stream order stands in for the barriers.
  for (int phase = 0; phase < 3; ++phase) {
    for (int sl = 0; sl < c->slots; ++sl) {
      const int r = c->emulated ? sl : c->rank;
      const int lo = rows_per * r < rows ? rows_per * r : rows;
      const int hi = lo + rows_per < rows ? lo + rows_per : rows;
      const int n = hi - lo;
      if (n <= 0) continue;
      char* stage = c->stage + c->stage_slot_bytes * (c->world - 1) * sl;
      char* mine = c->region[r];
      if (phase == 0) {
        for (int k = 1; k < c->world && e == cudaSuccess; ++k) {      // start at the next rank: spreads the load
          const int p = (r + k) % c->world;
          e = cudaMemcpyAsync(stage + c->stage_slot_bytes * (k - 1), c->region[p] + kCtrlBytes + lo * row_bytes,
                              n * row_bytes, cudaMemcpyDefault, st);
        }
      } else if (phase == 1) {
        StagedRows in;
        for (int p = 0; p < kMaxRanks; ++p) in.src[p] = nullptr;
        in.src[r] = mine + kCtrlBytes + lo * row_bytes;
        for (int k = 1; k < c->world; ++k) in.src[(r + k) % c->world] = stage + c->stage_slot_bytes * (k - 1);
        T* residual = static_cast<T*>(residual_shard) + static_cast<int64_t>(sl) * residual_slot_stride;
        const int grid = n < 4 * kNumSMs ? n : 4 * kNumSMs;
        void* out = mine + out_off + lo * row_bytes;
        if (vpt == 1)
          reduce_staged_kernel<T, 1><<<grid, threads, 0, st>>>(in, c->world, out, residual, gamma, eps, n, hidden, error_word);
        else
          reduce_staged_kernel<T, 2><<<grid, threads, 0, st>>>(in, c->world, out, residual, gamma, eps, n, hidden, error_word);
        if (int rc = check_launch("reduce_staged_kernel")) return rc;
      } else {
        for (int k = 1; k < c->world && e == cudaSuccess; ++k) {
          const int p = (r + k) % c->world;
          e = cudaMemcpyAsync(c->region[p] + out_off + lo * row_bytes, mine + out_off + lo * row_bytes, n * row_bytes,
                              cudaMemcpyDefault, st);
        }
      }
    }
    if (e != cudaSuccess) return cuda_fail("allreduce_residual_rmsnorm_staged: cudaMemcpyAsync", e);
  }
  if (!c->emulated) {
    comm_barrier_kernel<<<1, 32, 0, st>>>(c->table_dev, 1, c->timeout_ns, error_word);
    if (int rc = check_launch("comm_barrier_kernel")) return rc;
  }
  return MV_OK;
}

// Same arguments, result and error codes as mv_allreduce_residual_rmsnorm; the bulk transfers run on the copy
// engines (see the staged form above).  Not for CUDA graphs that are replayed while the peers' buffers move:
// the copies are captured with the addresses they were issued with, which is what a replay wants here too.
extern "C" int mv_allreduce_residual_rmsnorm_staged(void* comm, void* residual_shard, int64_t residual_slot_stride,
                                                    const void* gamma, float eps, int rows, int hidden, int* error_word,
                                                    int dtype, void* stream) {
  Comm* c = static_cast<Comm*>(comm);
  if (!c || !gamma || !error_word) return fail(MV_ERR_NULL, "allreduce_residual_rmsnorm_staged: null argument");
  if (!c->connected) return fail(MV_ERR_SHAPE, "allreduce_residual_rmsnorm_staged: communicator is not connected");
  if (!residual_shard) {      // allowed only for a rank that owns no row of this call
    const int per = rows > 0 ? (rows + c->world - 1) / c->world : 0;
    if (c->emulated || static_cast<int64_t>(c->rank) * per < rows)
      return fail(MV_ERR_NULL, "allreduce_residual_rmsnorm_staged: residual_shard is null but this rank owns rows");
  }
  if (rows < 0 || hidden <= 0 || hidden % 8 != 0)
    return fail(MV_ERR_SHAPE, "allreduce_residual_rmsnorm_staged: hidden (%d) must be a positive multiple of 8, rows >= 0", hidden);
  if (hidden > 16384) return fail(MV_ERR_LIMIT, "allreduce_residual_rmsnorm_staged: hidden %d exceeds 16384", hidden);
  if (static_cast<int64_t>(rows) * hidden * 2 > c->data_bytes)
    return fail(MV_ERR_LIMIT, "allreduce_residual_rmsnorm_staged: %d rows x %d exceed the communicator's %lld-byte buffers",
                rows, hidden, static_cast<long long>(c->data_bytes));
  if (!aligned16(residual_shard) || !aligned16(gamma) || (residual_slot_stride * 2) % 16 != 0)
    return fail(MV_ERR_ALIGN, "allreduce_residual_rmsnorm_staged: residual and gamma must be 16-byte aligned");
  if (c->emulated) {
    const int rows_per = (rows + c->world - 1) / c->world;
    if (c->slots > 1 && residual_slot_stride < static_cast<int64_t>(rows_per) * hidden)
      return fail(MV_ERR_SHAPE, "allreduce_residual_rmsnorm_staged: residual_slot_stride smaller than one rank's shard");
  }
  if (rows == 0) return MV_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == MV_F16) return launch_staged<__half>(c, residual_shard, residual_slot_stride, gamma, eps, rows, hidden, error_word, s);
  if (dtype == MV_BF16)
    return launch_staged<__nv_bfloat16>(c, residual_shard, residual_slot_stride, gamma, eps, rows, hidden, error_word, s);
  return fail(MV_ERR_DTYPE, "allreduce_residual_rmsnorm_staged: dtype %d", dtype);
}

extern "C" int mv_add_rmsnorm(void* out, const void* x, const void* residual_in, void* residual_out, int64_t res_lo,
                              int64_t res_hi, const void* gamma, float eps, int64_t rows, int hidden, int dtype,
                              void* stream) {
  if (!out || !x || !gamma) return fail(MV_ERR_NULL, "add_rmsnorm: null argument");
  if (rows < 0 || rows > 0x7fffffff || hidden <= 0 || hidden % 8 != 0)
    return fail(MV_ERR_SHAPE, "add_rmsnorm: hidden (%d) must be a positive multiple of 8, 0 <= rows < 2^31", hidden);
  if (hidden > 16384) return fail(MV_ERR_LIMIT, "add_rmsnorm: hidden %d exceeds 16384", hidden);
  if (!aligned16(out) || !aligned16(x) || !aligned16(gamma) || !aligned16(residual_in) || !aligned16(residual_out))
    return fail(MV_ERR_ALIGN, "add_rmsnorm: pointers must be 16-byte aligned");
  if (residual_out && (res_lo < 0 || res_hi < res_lo || res_hi > rows))
    return fail(MV_ERR_SHAPE, "add_rmsnorm: residual row range [%lld, %lld) outside [0, %lld)", (long long)res_lo,
                (long long)res_hi, (long long)rows);
  if (rows == 0) return MV_OK;
  int vpt = 1;
  const int threads = threads_for(hidden, &vpt);
  const int grid = static_cast<int>(rows < 8 * kNumSMs ? rows : 8 * kNumSMs);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int lo = static_cast<int>(res_lo), hi = static_cast<int>(res_hi), r = static_cast<int>(rows);
#define MV_LAUNCH_ADD_NORM(T, V) \
  add_rmsnorm_kernel<T, V><<<grid, threads, 0, s>>>(out, x, residual_in, residual_out, lo, hi, gamma, eps, r, hidden)
  if (dtype == MV_F16) {
    if (vpt == 1) MV_LAUNCH_ADD_NORM(__half, 1); else MV_LAUNCH_ADD_NORM(__half, 2);
  } else if (dtype == MV_BF16) {
    if (vpt == 1) MV_LAUNCH_ADD_NORM(__nv_bfloat16, 1); else MV_LAUNCH_ADD_NORM(__nv_bfloat16, 2);
  } else {
    return fail(MV_ERR_DTYPE, "add_rmsnorm: dtype %d", dtype);
  }
#undef MV_LAUNCH_ADD_NORM
  return check_launch("add_rmsnorm");
}

extern "C" int mv_silu_mul(void* out, const void* gate_up, int64_t gate_up_stride, int64_t rows, int inter, int dtype,
                           void* stream) {
  if (!out || !gate_up) return fail(MV_ERR_NULL, "silu_mul: null argument");
  if (rows < 0 || inter <= 0 || inter % 8 != 0 || gate_up_stride < 2ll * inter || gate_up_stride % 8 != 0)
    return fail(MV_ERR_SHAPE, "silu_mul: inter (%d) must be a positive multiple of 8 and the row stride a multiple of 8 >= 2*inter", inter);
  if (!aligned16(out) || !aligned16(gate_up)) return fail(MV_ERR_ALIGN, "silu_mul: pointers must be 16-byte aligned");
  if (rows == 0) return MV_OK;
  const int gx = (inter / 8 + 255) / 256;
  int64_t gy = (16ll * kNumSMs + gx - 1) / gx;          // about 16 resident CTAs per SM in total
  if (gy > rows) gy = rows;
  if (gy > 65535) gy = 65535;
  const dim3 grid(gx, static_cast<unsigned>(gy));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == MV_F16) silu_mul_kernel<__half><<<grid, 256, 0, s>>>(out, gate_up, gate_up_stride, rows, inter);
  else if (dtype == MV_BF16) silu_mul_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(out, gate_up, gate_up_stride, rows, inter);
  else return fail(MV_ERR_DTYPE, "silu_mul: dtype %d", dtype);
  return check_launch("silu_mul");
}

// Measurement hook (not in the public header): a plain copy between this rank's buffers and the next rank's,
// with 16-byte loads and stores, `unroll` independent vectors in flight per thread.  mode 0 pulls the peer's
// input buffer into the local gather buffer, mode 1 pushes the local input buffer into the peer's gather buffer.
// It answers "what can plain peer loads / stores reach on this link" next to the fused kernel's figure.
namespace mv {
template <int U>
__global__ void __launch_bounds__(512) peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t nvec) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < nvec) v[u] = ld_global16(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < nvec) st_global16(dst + i + u * stride, v[u]);
  }
}
}  // namespace mv

extern "C" int mv_debug_peer_copy(void* comm, int mode, int64_t bytes, int blocks, int unroll, void* stream) {
  Comm* c = static_cast<Comm*>(comm);
  if (!c || !c->connected || c->emulated) return fail(MV_ERR_SHAPE, "peer_copy: needs a connected multi-GPU communicator");
  if (bytes <= 0 || bytes > c->data_bytes || bytes % 16) return fail(MV_ERR_SHAPE, "peer_copy: bad size");
  const int peer = (c->rank + 1) % c->world;
  const size_t out_off = kCtrlBytes + round256(static_cast<size_t>(c->data_bytes));
  const uint4* src = reinterpret_cast<const uint4*>(c->region[mode == 0 ? peer : c->rank] + kCtrlBytes);
  uint4* dst = reinterpret_cast<uint4*>(c->region[mode == 0 ? c->rank : peer] + out_off);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t nvec = static_cast<size_t>(bytes) / 16;
  if (unroll >= 8) peer_copy_kernel<8><<<blocks, 512, 0, st>>>(src, dst, nvec);
  else if (unroll >= 4) peer_copy_kernel<4><<<blocks, 512, 0, st>>>(src, dst, nvec);
  else if (unroll >= 2) peer_copy_kernel<2><<<blocks, 512, 0, st>>>(src, dst, nvec);
  else peer_copy_kernel<1><<<blocks, 512, 0, st>>>(src, dst, nvec);
  return check_launch("peer_copy_kernel");
}
