// Sampling tail: row-wise argmax of the logits (greedy) or of the exponential-race scores (temperature),
// both mergeable across vocabulary shards.
//
// In the reference every tensor-parallel rank computes its vocabulary shard of
// the logits, rank 0 gathers the full (batch, 151,936) matrix
// (src/myvllm/layers/embedding_head.py:56-77) and the sampler works on that
// (src/myvllm/layers/sampler.py:15-19; greedy decoding is its temperature -> 0
// limit, the plain argmax).  Here a rank reduces its own shard to ONE 64-bit
// key per row -- the maximum logit in an order-preserving integer form in the
// high word, 2^32-1 minus the global column index in the low word -- so that
// the larger key is the larger logit and, between equal logits, the lower
// index.  Shards are merged by an integer MAX (an all-reduce of 8 bytes per
// row instead of a gather of the logits) and decoded to token ids.
// HBM-bound: one read of the logits, rows * cols * 2 bytes.
#include <climits>
#include "common.cuh"

namespace mv {

constexpr int kArgmaxThreads = 256;

// float -> int32 whose signed order is the float order; NaN sorts above +inf (torch.argmax treats NaN as the
// maximum) and -0.0 maps to the key of +0.0 (they compare equal, so the lower index must win between them).
__device__ __forceinline__ int32_t orderable(float v) {
  if (v != v) return 0x7fffffff;
  const int32_t b = __float_as_int(v);
  if (b == static_cast<int32_t>(0x80000000u)) return 0;
  return b < 0 ? (b ^ 0x7fffffff) : b;
}
__device__ __forceinline__ long long make_key(float v, uint32_t index) {
  const unsigned long long hi = static_cast<uint32_t>(orderable(v));
  return static_cast<long long>((hi << 32) | static_cast<unsigned long long>(0xffffffffu - index));
}
__device__ __forceinline__ long long token_of_key(long long key) {
  return static_cast<long long>(0xffffffffu - static_cast<uint32_t>(key & 0xffffffffll));
}

// One CTA per row.  A thread walks its columns in increasing order and keeps the first maximum it meets
// (strict >), so equal logits resolve to the lowest index within a thread; across threads the keys do it.
template <typename T>
__global__ void __launch_bounds__(kArgmaxThreads)
argmax_rows_kernel(const T* __restrict__ logits, int64_t row_stride, int64_t cols, uint32_t index_offset, bool aligned,
                   long long* __restrict__ keys, long long* __restrict__ tokens) {
  using T2 = typename Elem<T>::T2;
  const T* row = logits + static_cast<int64_t>(blockIdx.x) * row_stride;
  float best = -INFINITY;
  bool best_nan = false, have = false;
  uint32_t best_idx = 0;
  auto offer = [&](float v, uint32_t idx) {
    if (best_nan) return;                       // a NaN already won: it is the maximum and came first
    const bool is_nan = v != v;
    if (is_nan || v > best || !have) {
      best = v;
      best_idx = idx;
      best_nan = is_nan;
      have = true;
    }
  };
  const int64_t chunks = aligned ? cols / 8 : 0;  // 16-byte chunks when every row starts on a 16-byte boundary
  // Per chunk of eight logits only its maximum is computed (packed 16-bit maxima, exact, NaN-propagating) and
  // compared with the running one; the chunk that raised it is kept and searched for the position at the end.
  // Chunks are visited in increasing order and only a strictly larger maximum replaces the kept chunk, so the
  // first of equal maxima survives.
  constexpr int kUnroll = 4;
  uint4 best_raw = make_uint4(0, 0, 0, 0);
  int64_t best_chunk = -1;
  float cbest = -INFINITY;
  bool cbest_nan = false;
  for (int64_t c0 = threadIdx.x; c0 < chunks; c0 += static_cast<int64_t>(kArgmaxThreads) * kUnroll) {
    uint4 raw[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t c = c0 + static_cast<int64_t>(u) * kArgmaxThreads;
      if (c < chunks) raw[u] = ld_stream16(row + c * 8);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t c = c0 + static_cast<int64_t>(u) * kArgmaxThreads;
      if (c < chunks && !cbest_nan) {
        const T2* p2 = reinterpret_cast<const T2*>(&raw[u]);
        const float m = Elem<T>::hmax_nan_f(Elem<T>::max2_nan(Elem<T>::max2_nan(p2[0], p2[1]),
                                                              Elem<T>::max2_nan(p2[2], p2[3])));
        const bool is_nan = m != m;
        if (is_nan || m > cbest || best_chunk < 0) {
          cbest = m;
          cbest_nan = is_nan;
          best_chunk = c;
          best_raw = raw[u];
        }
      }
    }
  }
  if (best_chunk >= 0) {   // position of the first maximum (or first NaN) inside the kept chunk
    const T2* p2 = reinterpret_cast<const T2*>(&best_raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = Elem<T>::to_f2(p2[j]);
      offer(f.x, static_cast<uint32_t>(best_chunk * 8 + 2 * j));
      offer(f.y, static_cast<uint32_t>(best_chunk * 8 + 2 * j + 1));
    }
  }
  for (int64_t i = chunks * 8 + threadIdx.x; i < cols; i += kArgmaxThreads)   // ragged tail
    offer(Elem<T>::to_f(row[i]), static_cast<uint32_t>(i));

  long long key = have ? make_key(best, index_offset + best_idx) : LLONG_MIN;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const long long other = __shfl_xor_sync(0xffffffffu, key, off);
    key = other > key ? other : key;
  }
  __shared__ long long s_keys[kArgmaxThreads / 32];
  if ((threadIdx.x & 31) == 0) s_keys[threadIdx.x >> 5] = key;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < kArgmaxThreads / 32; ++w) key = s_keys[w] > key ? s_keys[w] : key;
    if (keys) keys[blockIdx.x] = key;
    if (tokens) tokens[blockIdx.x] = token_of_key(key);
  }
}

// ---------------------------------------------------------------------------------------------
// Temperature sampling: the reference's exponential race (src/myvllm/layers/sampler.py:15-19)
//   token = argmax_i softmax(logits / T)_i / E_i,   E_i ~ Exp(1)
// needs no normaliser: argmax_i p_i / E_i = argmax_i (logit_i / T - log E_i).  The score of a column depends
// only on that column, so the vocabulary shards of a tensor-parallel model reduce independently and merge by
// the same 64-bit MAX as the greedy keys -- provided every rank draws the SAME E_i for global column i.
// Hence a counter-based generator: Philox4x32-10 with key = seed and counter = (global column / 4, row, step),
// whose four 32-bit outputs serve columns 4g .. 4g+3.  u = (top 24 bits + 0.5) / 2^24 lies strictly inside
// (0, 1); E = -log(u) (>= 3e-8, so the reference's clamp at 1e-10 never binds).  A row with T == 0 is greedy.
// ---------------------------------------------------------------------------------------------
struct Philox {
  uint32_t x, y, z, w;
};
__host__ __device__ inline void philox_mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
  const unsigned long long p = static_cast<unsigned long long>(a) * b;
  hi = static_cast<uint32_t>(p >> 32);
  lo = static_cast<uint32_t>(p);
}
__host__ __device__ inline Philox philox4x32_10(Philox c, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    philox_mulhilo(0xD2511F53u, c.x, hi0, lo0);
    philox_mulhilo(0xCD9E8D57u, c.z, hi1, lo1);
    c = Philox{hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0};
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c;
}
// -log E for the 32 random bits of one column: Gumbel noise added to logit / T.
__device__ __forceinline__ float race_noise(uint32_t bits) {
  const float u = (static_cast<float>(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);
  return -__logf(-logf(u));
}

template <typename T>
__global__ void __launch_bounds__(kArgmaxThreads)
sample_rows_kernel(const T* __restrict__ logits, int64_t row_stride, int64_t cols, uint32_t index_offset, bool aligned,
                   const float* __restrict__ temperatures, unsigned long long seed, const long long* __restrict__ step_ptr,
                   long long* __restrict__ keys, long long* __restrict__ tokens) {
  using T2 = typename Elem<T>::T2;
  const uint32_t rowi = blockIdx.x;
  const T* row = logits + static_cast<int64_t>(rowi) * row_stride;
  const float temp = temperatures[rowi];
  const bool greedy = !(temp > 0.f);
  const float inv_t = greedy ? 1.0f : 1.0f / temp;
  const unsigned long long step = static_cast<unsigned long long>(*step_ptr);
  const uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  const uint32_t s0 = static_cast<uint32_t>(step), s1 = static_cast<uint32_t>(step >> 32);
  float best = -INFINITY;
  bool best_nan = false, have = false;
  uint32_t best_idx = 0;
  auto offer = [&](float v, uint32_t idx) {       // first maximum in visiting order; a NaN is the maximum
    if (best_nan) return;
    const bool is_nan = v != v;
    if (is_nan || v > best || !have) {
      best = v;
      best_idx = idx;
      best_nan = is_nan;
      have = true;
    }
  };
  auto noise_of = [&](uint32_t gcol) {           // one column on its own (ragged edges)
    const Philox r = philox4x32_10(Philox{gcol >> 2, rowi, s0, s1}, k0, k1);
    const uint32_t lane = gcol & 3u;
    return race_noise(lane == 0 ? r.x : lane == 1 ? r.y : lane == 2 ? r.z : r.w);
  };
  // 16-byte chunks of eight logits = two Philox groups, when rows and the shard start on such boundaries
  const bool fast = aligned && (index_offset & 7u) == 0;
  const int64_t chunks = fast ? cols / 8 : 0;
  for (int64_t c = threadIdx.x; c < chunks; c += kArgmaxThreads) {
    const uint4 raw = ld_stream16(row + c * 8);
    const T2* p2 = reinterpret_cast<const T2*>(&raw);
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = Elem<T>::to_f2(p2[j]);
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
    const uint32_t g0 = index_offset + static_cast<uint32_t>(c * 8);
    if (!greedy) {
      const Philox a = philox4x32_10(Philox{g0 >> 2, rowi, s0, s1}, k0, k1);
      const Philox b = philox4x32_10(Philox{(g0 >> 2) + 1, rowi, s0, s1}, k0, k1);
      const uint32_t bits[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = v[j] * inv_t + race_noise(bits[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) offer(v[j], static_cast<uint32_t>(c * 8 + j));
  }
  for (int64_t i = chunks * 8 + threadIdx.x; i < cols; i += kArgmaxThreads) {
    float v = Elem<T>::to_f(row[i]);
    if (!greedy) v = v * inv_t + noise_of(index_offset + static_cast<uint32_t>(i));
    offer(v, static_cast<uint32_t>(i));
  }
  long long key = have ? make_key(best, index_offset + best_idx) : LLONG_MIN;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const long long other = __shfl_xor_sync(0xffffffffu, key, off);
    key = other > key ? other : key;
  }
  __shared__ long long s_keys[kArgmaxThreads / 32];
  if ((threadIdx.x & 31) == 0) s_keys[threadIdx.x >> 5] = key;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < kArgmaxThreads / 32; ++w) key = s_keys[w] > key ? s_keys[w] : key;
    if (keys) keys[blockIdx.x] = key;
    if (tokens) tokens[blockIdx.x] = token_of_key(key);
  }
}

// keys (shards, rows) -> tokens (rows): the largest key of each row, decoded.
__global__ void argmax_decode_kernel(const long long* __restrict__ keys, int shards, int64_t rows,
                                     long long* __restrict__ tokens) {
  const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  long long key = keys[r];
  for (int s = 1; s < shards; ++s) {
    const long long other = keys[static_cast<int64_t>(s) * rows + r];
    key = other > key ? other : key;
  }
  tokens[r] = token_of_key(key);
}

}  // namespace mv

extern "C" int mv_argmax_rows(const void* logits, int64_t row_stride, int64_t rows, int64_t cols,
                              int64_t index_offset, int64_t* keys, int64_t* tokens, int dtype, void* stream) {
  using namespace mv;
  if (dtype != MV_F16 && dtype != MV_BF16) return fail(MV_ERR_DTYPE, "argmax_rows: dtype %d", dtype);
  if (rows < 0 || cols <= 0 || index_offset < 0) return fail(MV_ERR_SHAPE, "argmax_rows: negative or zero size");
  if (rows == 0) return MV_OK;
  if (!logits || (!keys && !tokens)) return fail(MV_ERR_NULL, "argmax_rows: null pointer");
  if (row_stride < cols) return fail(MV_ERR_SHAPE, "argmax_rows: row stride smaller than a row");
  const bool aligned = row_stride % 8 == 0 && aligned16(logits);   // otherwise element-wise loads
  if (index_offset + cols > 0xffffffffLL || rows > 0x7fffffffLL)
    return fail(MV_ERR_LIMIT, "argmax_rows: column index beyond 32 bits or too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(rows);
  if (dtype == MV_F16)
    argmax_rows_kernel<__half><<<grid, kArgmaxThreads, 0, st>>>(
        static_cast<const __half*>(logits), row_stride, cols, static_cast<uint32_t>(index_offset), aligned,
        reinterpret_cast<long long*>(keys), reinterpret_cast<long long*>(tokens));
  else
    argmax_rows_kernel<__nv_bfloat16><<<grid, kArgmaxThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(logits), row_stride, cols, static_cast<uint32_t>(index_offset), aligned,
        reinterpret_cast<long long*>(keys), reinterpret_cast<long long*>(tokens));
  return check_launch("argmax_rows_kernel");
}

extern "C" int mv_argmax_decode(const int64_t* keys, int shards, int64_t rows, int64_t* tokens, void* stream) {
  using namespace mv;
  if (shards <= 0 || rows < 0) return fail(MV_ERR_SHAPE, "argmax_decode: negative or zero size");
  if (rows == 0) return MV_OK;
  if (!keys || !tokens) return fail(MV_ERR_NULL, "argmax_decode: null pointer");
  const int threads = 128;
  const int64_t grid = (rows + threads - 1) / threads;
  if (grid > 0x7fffffffLL) return fail(MV_ERR_LIMIT, "argmax_decode: too many rows");
  argmax_decode_kernel<<<static_cast<unsigned>(grid), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(keys), shards, rows, reinterpret_cast<long long*>(tokens));
  return check_launch("argmax_decode_kernel");
}

extern "C" int mv_sample_rows(const void* logits, int64_t row_stride, int64_t rows, int64_t cols, int64_t index_offset,
                              const float* temperatures, uint64_t seed, const int64_t* step, int64_t* keys,
                              int64_t* tokens, int dtype, void* stream) {
  using namespace mv;
  if (dtype != MV_F16 && dtype != MV_BF16) return fail(MV_ERR_DTYPE, "sample_rows: dtype %d", dtype);
  if (rows < 0 || cols <= 0 || index_offset < 0) return fail(MV_ERR_SHAPE, "sample_rows: negative or zero size");
  if (rows == 0) return MV_OK;
  if (!logits || !temperatures || !step || (!keys && !tokens)) return fail(MV_ERR_NULL, "sample_rows: null pointer");
  if (row_stride < cols) return fail(MV_ERR_SHAPE, "sample_rows: row stride smaller than a row");
  if (index_offset + cols > 0xffffffffLL || rows > 0x7fffffffLL)
    return fail(MV_ERR_LIMIT, "sample_rows: column index beyond 32 bits or too many rows");
  const bool aligned = row_stride % 8 == 0 && aligned16(logits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(rows);
  if (dtype == MV_F16)
    sample_rows_kernel<__half><<<grid, kArgmaxThreads, 0, st>>>(
        static_cast<const __half*>(logits), row_stride, cols, static_cast<uint32_t>(index_offset), aligned, temperatures,
        seed, reinterpret_cast<const long long*>(step), reinterpret_cast<long long*>(keys),
        reinterpret_cast<long long*>(tokens));
  else
    sample_rows_kernel<__nv_bfloat16><<<grid, kArgmaxThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(logits), row_stride, cols, static_cast<uint32_t>(index_offset), aligned,
        temperatures, seed, reinterpret_cast<const long long*>(step), reinterpret_cast<long long*>(keys),
        reinterpret_cast<long long*>(tokens));
  return check_launch("sample_rows_kernel");
}

// The generator of mv_sample_rows on the host: the four 32-bit words for (seed, step, row, column group).
extern "C" int mv_philox4x32_10(uint64_t seed, uint64_t step, uint32_t row, uint32_t column_group, uint32_t* out4) {
  if (!out4) return mv::fail(MV_ERR_NULL, "philox: null output");
  const mv::Philox r = mv::philox4x32_10(mv::Philox{column_group, row, static_cast<uint32_t>(step), static_cast<uint32_t>(step >> 32)},
                                         static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
  out4[0] = r.x; out4[1] = r.y; out4[2] = r.z; out4[3] = r.w;
  return MV_OK;
}
