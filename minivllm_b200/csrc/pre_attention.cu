// Fused pre-attention step: q/k RMSNorm + rotary embedding + store_kvcache in
// one pass over the fused qkv projection output.
//
// In the reference this is three memory-bound passes and a dozen launches per
// layer, right before the attention operators: `self.rms_norm(q)`,
// `self.rms_norm(k)`, `self.rotary_emb(positions, q, k)`
// (src/myvllm/models/qwen3.py:104-108, layers/layernorm.py:10-17,
// layers/rotary_embedding.py:4-23,77-83) and then `store_kvcache` inside
// Attention.forward (layers/attention.py:498-510).  Here eight lanes own one
// (token, head) row of head_dim 128: lane l holds elements 8l..8l+7 and their
// rotate-half partners 64+8l.., so the norm needs a three-step shuffle and
// the rotation needs no data exchange.  q heads are normalised, rotated and
// written to q_out; k heads likewise to k_out and to the paged cache at
// slot_mapping[token]; v heads are copied to the cache.
// Arithmetic: x * rsqrt(mean(x^2) + eps) * gamma in fp32, rounded to the model
// dtype (as the unfused torch path rounds it), then
// (x1*cos - x2*sin, x2*cos + x1*sin) in fp32 from the fp32 cos/sin table,
// rounded once more.  HBM-bound: reads qkv once, writes q, k and the two cache rows.
// With an int8 cache (kInt8) the k row (after norm and rotation, in the model dtype: the values k_out gets) and
// the v row are quantised per token and head on their way into the cache, exactly as the quantising
// store_kvcache does: codes (slots, kv_heads, 128) int8 and fp16 scales (slots, kv_heads).
#include "common.cuh"
#include "quant.cuh"

namespace mv {

constexpr int kPreThreads = 256;

// Eight lanes own one (token, head) row of 128 elements: lane l holds elements
// 8l..8l+7 and their rotate-half partners 64+8l..64+8l+7 (two 16-byte loads),
// so a warp works on four rows at once and keeps 1 KB of loads in flight.
// The eight lanes of a row share its absolute maximum (shuffles among those lanes only: other rows of the warp
// may be on another branch), every lane derives the scale and quantises its two chunks.
template <typename T>
__device__ __forceinline__ void store_row_int8(const uint4& lo, const uint4& hi, int8_t* codes_row, __half* scale_ptr,
                                               int sub) {
  const unsigned mask = 0xffu << (threadIdx.x & 24);
  float amax = fmaxf(chunk_absmax<T>(lo), chunk_absmax<T>(hi));
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 4));
  __half scale16;
  float s, inv;
  quant_scale(amax, scale16, s, inv);
  st_global8(codes_row + 8 * sub, quant_codes<T>(lo, s, inv));
  st_global8(codes_row + 64 + 8 * sub, quant_codes<T>(hi, s, inv));
  if (sub == 0) *scale_ptr = scale16;
}

template <typename T, bool kInt8>
__global__ void __launch_bounds__(kPreThreads)
qk_norm_rope_store_kernel(const T* __restrict__ qkv, int64_t qkv_stride, const int64_t* __restrict__ positions,
                          const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int max_position,
                          const T* __restrict__ gamma_q, const T* __restrict__ gamma_k, float eps,
                          T* __restrict__ q_out, T* __restrict__ k_out, void* __restrict__ k_cache_,
                          void* __restrict__ v_cache_, __half* __restrict__ k_scale, __half* __restrict__ v_scale,
                          const int64_t* __restrict__ slot_mapping, int64_t num_slots, int64_t num_tokens, int num_heads,
                          int num_kv_heads) {
  T* k_cache = static_cast<T*>(k_cache_);
  T* v_cache = static_cast<T*>(v_cache_);
  constexpr int D = 128;
  using T2 = typename Elem<T>::T2;
  const int sub = threadIdx.x & 7;  // lane within the row group
  const int rows_per_token = num_heads + 2 * num_kv_heads;
  const int64_t total_rows = num_tokens * rows_per_token;
  const int64_t group0 = (static_cast<int64_t>(blockIdx.x) * kPreThreads + threadIdx.x) >> 3;
  const int64_t ngroups = (static_cast<int64_t>(gridDim.x) * kPreThreads) >> 3;
  // every lane of a warp runs the same number of rounds: the shuffles below use the full mask
  const int64_t rounds = (total_rows + ngroups - 1) / ngroups;
  for (int64_t it = 0; it < rounds; ++it) {
    const int64_t row = group0 + it * ngroups;
    const bool live = row < total_rows;
    const int64_t t = live ? row / rows_per_token : 0;
    const int h = live ? static_cast<int>(row - t * rows_per_token) : 0;
    const bool is_q = h < num_heads, is_k = !is_q && h < num_heads + num_kv_heads;
    uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
    if (live) {
      const T* src = qkv + t * qkv_stride + static_cast<int64_t>(h) * D;
      lo = ld_stream16(src + 8 * sub);
      hi = ld_stream16(src + 64 + 8 * sub);
    }
    const int64_t slot = (live && slot_mapping != nullptr && !is_q) ? slot_mapping[t] : -1;
    const bool to_cache = slot >= 0 && slot < num_slots;
    float a[8], b[8];
    {
      const T2* l2 = reinterpret_cast<const T2*>(&lo);
      const T2* h2 = reinterpret_cast<const T2*>(&hi);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = Elem<T>::to_f2(l2[j]), fb = Elem<T>::to_f2(h2[j]);
        a[2 * j] = fa.x; a[2 * j + 1] = fa.y; b[2 * j] = fb.x; b[2 * j + 1] = fb.y;
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += a[j] * a[j] + b[j] * b[j];
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    if (!live) continue;
    if (!is_q && !is_k) {  // v: straight copy into the cache
      if (to_cache) {
        const int64_t crow = slot * num_kv_heads + (h - num_heads - num_kv_heads);
        if constexpr (kInt8) {
          store_row_int8<T>(lo, hi, static_cast<int8_t*>(v_cache_) + crow * D, v_scale + crow, sub);
        } else {
          T* dst = v_cache + crow * D;
          st_global16(dst + 8 * sub, lo);
          st_global16(dst + 64 + 8 * sub, hi);
        }
      }
      continue;
    }
    const float rstd = rsqrtf(ss * (1.f / D) + eps);
    const T* gamma = is_q ? gamma_q : gamma_k;
    const uint4 g_lo = *reinterpret_cast<const uint4*>(gamma + 8 * sub);
    const uint4 g_hi = *reinterpret_cast<const uint4*>(gamma + 64 + 8 * sub);
    int64_t pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_position ? max_position - 1 : pos);
    const float4* cp = reinterpret_cast<const float4*>(cos_tab + pos * (D / 2) + 8 * sub);
    const float4* sp = reinterpret_cast<const float4*>(sin_tab + pos * (D / 2) + 8 * sub);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint4 o_lo, o_hi;
    {
      const T2* gl = reinterpret_cast<const T2*>(&g_lo);
      const T2* gh = reinterpret_cast<const T2*>(&g_hi);
      T2* ol = reinterpret_cast<T2*>(&o_lo);
      T2* oh = reinterpret_cast<T2*>(&o_hi);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 ga = Elem<T>::to_f2(gl[j]), gb = Elem<T>::to_f2(gh[j]);
        // round the normalised values to the model dtype, as the separate norm kernel would
        const float2 n1 = Elem<T>::to_f2(Elem<T>::from_f2(a[2 * j] * rstd * ga.x, a[2 * j + 1] * rstd * ga.y));
        const float2 n2 = Elem<T>::to_f2(Elem<T>::from_f2(b[2 * j] * rstd * gb.x, b[2 * j + 1] * rstd * gb.y));
        ol[j] = Elem<T>::from_f2(n1.x * c[2 * j] - n2.x * sn[2 * j], n1.y * c[2 * j + 1] - n2.y * sn[2 * j + 1]);
        oh[j] = Elem<T>::from_f2(n2.x * c[2 * j] + n1.x * sn[2 * j], n2.y * c[2 * j + 1] + n1.y * sn[2 * j + 1]);
      }
    }
    if (is_q) {
      T* dst = q_out + (t * num_heads + h) * D;
      st_global16(dst + 8 * sub, o_lo);
      st_global16(dst + 64 + 8 * sub, o_hi);
    } else {
      const int kh = h - num_heads;
      T* dst = k_out + (t * num_kv_heads + kh) * D;
      st_global16(dst + 8 * sub, o_lo);
      st_global16(dst + 64 + 8 * sub, o_hi);
      if (to_cache) {
        const int64_t crow = slot * num_kv_heads + kh;
        if constexpr (kInt8) {
          store_row_int8<T>(o_lo, o_hi, static_cast<int8_t*>(k_cache_) + crow * D, k_scale + crow, sub);
        } else {
          T* cdst = k_cache + crow * D;
          st_global16(cdst + 8 * sub, o_lo);
          st_global16(cdst + 64 + 8 * sub, o_hi);
        }
      }
    }
  }
}

}  // namespace mv

extern "C" int mv_qk_norm_rope_store(const void* qkv, int64_t qkv_stride_tok, const int64_t* positions,
                                     const float* cos_table, const float* sin_table, int max_position,
                                     const void* gamma_q, const void* gamma_k, float eps, void* q_out, void* k_out,
                                     void* k_cache, void* v_cache, void* k_scale, void* v_scale,
                                     const int64_t* slot_mapping, int64_t num_slots, int64_t num_tokens, int num_heads,
                                     int num_kv_heads, int head_dim, int dtype, void* stream) {
  using namespace mv;
  if (dtype != MV_F16 && dtype != MV_BF16) return fail(MV_ERR_DTYPE, "qk_norm_rope_store: dtype %d", dtype);
  if (num_tokens < 0 || num_heads <= 0 || num_kv_heads <= 0 || max_position <= 0 || num_slots < 0)
    return fail(MV_ERR_SHAPE, "qk_norm_rope_store: negative or zero size");
  if (head_dim != 128) return fail(MV_ERR_SHAPE, "qk_norm_rope_store: head_dim %d is not 128", head_dim);
  if (num_tokens == 0) return MV_OK;
  if (!qkv || !positions || !cos_table || !sin_table || !gamma_q || !gamma_k || !q_out || !k_out)
    return fail(MV_ERR_NULL, "qk_norm_rope_store: null pointer");
  if (slot_mapping && (!k_cache || !v_cache)) return fail(MV_ERR_NULL, "qk_norm_rope_store: slot_mapping without caches");
  if ((k_scale == nullptr) != (v_scale == nullptr))
    return fail(MV_ERR_NULL, "qk_norm_rope_store: k_scale and v_scale must both be set or both be null");
  const bool int8 = k_scale != nullptr;
  if (int8 && !slot_mapping) return fail(MV_ERR_NULL, "qk_norm_rope_store: scales without a slot_mapping");
  const int64_t row = static_cast<int64_t>(num_heads + 2 * num_kv_heads) * head_dim;
  if (qkv_stride_tok < row) return fail(MV_ERR_SHAPE, "qk_norm_rope_store: token stride smaller than a row");
  if (qkv_stride_tok % 8 || !aligned16(qkv) || !aligned16(q_out) || !aligned16(k_out) || !aligned16(cos_table) ||
      !aligned16(sin_table) || !aligned16(gamma_q) || !aligned16(gamma_k) || (k_cache && !aligned16(k_cache)) ||
      (v_cache && !aligned16(v_cache)) || (int8 && (!aligned16(k_scale) || !aligned16(v_scale))))
    return fail(MV_ERR_ALIGN, "qk_norm_rope_store: misaligned pointer or stride");
  const int64_t rows = num_tokens * (num_heads + 2 * num_kv_heads);
  int64_t grid = (rows + kPreThreads / 8 - 1) / (kPreThreads / 8);
  if (grid > static_cast<int64_t>(kNumSMs) * 8) grid = static_cast<int64_t>(kNumSMs) * 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  __half* ks = static_cast<__half*>(k_scale);
  __half* vs = static_cast<__half*>(v_scale);
#define MV_PRE_LAUNCH(T, I8)                                                                                          \
  qk_norm_rope_store_kernel<T, I8><<<static_cast<int>(grid), kPreThreads, 0, st>>>(                                    \
      static_cast<const T*>(qkv), qkv_stride_tok, positions, cos_table, sin_table, max_position,                       \
      static_cast<const T*>(gamma_q), static_cast<const T*>(gamma_k), eps, static_cast<T*>(q_out), static_cast<T*>(k_out), \
      k_cache, v_cache, ks, vs, slot_mapping, num_slots, num_tokens, num_heads, num_kv_heads)
  if (dtype == MV_F16) {
    if (int8) MV_PRE_LAUNCH(__half, true); else MV_PRE_LAUNCH(__half, false);
  } else {
    if (int8) MV_PRE_LAUNCH(__nv_bfloat16, true); else MV_PRE_LAUNCH(__nv_bfloat16, false);
  }
#undef MV_PRE_LAUNCH
  return check_launch("qk_norm_rope_store_kernel");
}
