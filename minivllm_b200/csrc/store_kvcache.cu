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

// Exact code of one element, any scale: the definition evaluated with the
// correctly rounded reciprocal and the exact remainder (see quant_chunk).
__device__ __noinline__ int quant_exact(float x, float s) {
  if (!(s > 0.f) || !(s < INFINITY)) return 0;
  const float inv = __frcp_rn(s);
  float n = rintf(x * inv);
  const float r = fmaf(-n, s, x);
  const float step = copysignf(1.f, r), half_s = 0.5f * s;
  if (fabsf(r) > half_s) n += step;
  else if (fabsf(r) == half_s && (static_cast<int>(n) & 1)) n += step;  // tie: to even
  return static_cast<int>(fminf(fmaxf(n, -127.f), 127.f));
}

// Quantise 8 elements held in one 16-byte chunk; GROUP lanes share a head row.
//
// The codes must equal the CPU definition, rint(fp32(x / s)) clamped to
// +-127, bit for bit.  x has at most 11 significant bits and s is an fp16
// value, so the exact quotient is either a tie (k + 1/2) or at least 2^-19
// (relative) away from one: the product with the correctly rounded reciprocal
// (relative error 2^-23) rounds to the same integer as the quotient unless the
// quotient is a tie.  Fast path, per element: multiply, round by adding
// 1.5*2^23 (the code is then the low byte of the sum), and measure the
// distance of the product from its rounded value; an element that comes
// within 1e-4 of a half-integer is redone on the exact path, and so are all
// eight when the scale is not a normal fp16 number (then |x/s| may exceed
// 127.5 and needs the clamp).  One IEEE division and one IEEE reciprocal per
// head row (lane 0 of the group), none per element.
// The kernel is bound by instruction issue, not by HBM, so the per-element work is packed: the row maximum is
// taken on the 16-bit pairs as they come (|x| and max are exact in any format), products, roundings and the
// near-tie distances run on fp32 pairs.  Lanes of an invalid token hold zeros: amax = 0, inv = 0, codes 0,
// and nothing is stored.
template <typename T, int GROUP>
__device__ __forceinline__ void quant_chunk(const uint4& raw, uint2& codes, __half& scale16) {
  using T2 = typename Elem<T>::T2;
  const T2* p2 = reinterpret_cast<const T2*>(&raw);
  T2 m2 = Elem<T>::absmax2(Elem<T>::absmax2(Elem<T>::from_f2(0.f, 0.f), p2[0]), p2[1]);
  m2 = Elem<T>::absmax2(Elem<T>::absmax2(m2, p2[2]), p2[3]);
  float amax = Elem<T>::hmax_f(m2);
#pragma unroll
  for (int off = GROUP / 2; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  // amax is the same in every lane of the group, so every lane computes the scale itself (no leader branch):
  // fp32(amax / 127) correctly rounded by the multiply-and-correct sequence for division by a constant
  // (q0 = amax * RN(1/127); r = amax - 127*q0 exactly by FMA; q = q0 + r * RN(1/127)), then fp16.
  constexpr float kInv127 = 0x1.020408p-7f;
  const float q0 = amax * kInv127;
  const float quo = fmaf(fmaf(-q0, 127.f, amax), kInv127, q0);
  scale16 = __float2half_rn(quo);
  const float s = __half2float(scale16);
  // An approximate reciprocal is enough for the fast path (its error is covered by the near-tie gate below);
  // 0 marks "take the exact path": scale zero, infinite or not a normal fp16 number.
  float inv = 0.f;
  if (s >= 6.103515625e-05f && s < INFINITY) asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(s));

  constexpr float kMagic = 12582912.f;  // 1.5 * 2^23: adding it rounds to nearest-even integer
  constexpr float kNearTie = 0.4999f;   // product error is < 127 * 2^-21 = 6e-5 (approximate reciprocal + rounding): anything closer to k + 1/2 is re-done
  const float2 inv2 = make_float2(inv, inv), magic2 = make_float2(kMagic, kMagic), nmagic2 = make_float2(-kMagic, -kMagic);
  float2 x2[4];
  uint32_t t[8];
  float worst = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    x2[j] = Elem<T>::to_f2(p2[j]);
    const float2 y = mul_f32x2(x2[j], inv2);
    const float2 tj = add_f32x2(y, magic2);                       // low byte of each word = the code
    const float2 rounded = add_f32x2(tj, nmagic2);
    const float2 d = add_f32x2(y, make_float2(-rounded.x, -rounded.y));   // distance from the rounded value
    t[2 * j] = __float_as_uint(tj.x);
    t[2 * j + 1] = __float_as_uint(tj.y);
    worst = fmaxf(worst, fmaxf(fabsf(d.x), fabsf(d.y)));
  }
  if (inv == 0.f) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      t[2 * j] = static_cast<uint32_t>(quant_exact(x2[j].x, s));
      t[2 * j + 1] = static_cast<uint32_t>(quant_exact(x2[j].y, s));
    }
  } else if (worst > kNearTie) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float x = (j & 1) ? x2[j >> 1].y : x2[j >> 1].x;
      const float y = x * inv;
      if (fabsf(y - ((y + kMagic) - kMagic)) > kNearTie) t[j] = static_cast<uint32_t>(quant_exact(x, s));
    }
  }
  // low bytes of t[0..7] -> two words
  uint32_t a01, a23;
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(a01) : "r"(t[0]), "r"(t[1]));
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(a23) : "r"(t[2]), "r"(t[3]));
  asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(codes.x) : "r"(a01), "r"(a23));
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(a01) : "r"(t[4]), "r"(t[5]));
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(a23) : "r"(t[6]), "r"(t[7]));
  asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(codes.y) : "r"(a01), "r"(a23));
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
