// Greedy sampling tail: row-wise argmax of the logits, mergeable across vocabulary shards.
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

// float -> int32 whose signed order is the float order; NaN sorts above +inf (torch.argmax treats NaN as the maximum).
__device__ __forceinline__ int32_t orderable(float v) {
  if (v != v) return 0x7fffffff;
  const int32_t b = __float_as_int(v);
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
