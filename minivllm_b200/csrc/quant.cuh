// Per-token-per-head symmetric int8 quantisation of K/V rows, shared by the quantising store
// (store_kvcache.cu) and the fused pre-attention kernel (pre_attention.cu).
//   amax = max|x| over head_dim (fp32); scale16 = fp16(amax / 127); s = float(scale16);
//   code = clamp(rint(x / s), -127, 127), 0 when s == 0
// evaluated so that codes and scales equal the CPU definition bit for bit.
#pragma once
#include "common.cuh"

namespace mv {

// Exact code of one element, any scale: the definition evaluated with the
// correctly rounded reciprocal and the exact remainder (see quant_chunk).
static __device__ __noinline__ int quant_exact(float x, float s) {
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
// |x| maximum of the eight elements of one 16-byte chunk (exact in any format).
template <typename T>
__device__ __forceinline__ float chunk_absmax(const uint4& raw) {
  using T2 = typename Elem<T>::T2;
  const T2* p2 = reinterpret_cast<const T2*>(&raw);
  T2 m2 = Elem<T>::absmax2(Elem<T>::absmax2(Elem<T>::from_f2(0.f, 0.f), p2[0]), p2[1]);
  m2 = Elem<T>::absmax2(Elem<T>::absmax2(m2, p2[2]), p2[3]);
  return Elem<T>::hmax_f(m2);
}

// Scale of a head row from its absolute maximum.  Every lane of the row computes it itself (no leader
// branch): fp32(amax / 127) correctly rounded by the multiply-and-correct sequence for division by a constant
// (q0 = amax * RN(1/127); r = amax - 127*q0 exactly by FMA; q = q0 + r * RN(1/127)), then fp16.
// `inv` is an approximate reciprocal for the fast path (its error is covered by the near-tie gate of
// quant_codes); 0 marks "take the exact path": scale zero, infinite or not a normal fp16 number.
__device__ __forceinline__ void quant_scale(float amax, __half& scale16, float& s, float& inv) {
  constexpr float kInv127 = 0x1.020408p-7f;
  const float q0 = amax * kInv127;
  const float quo = fmaf(fmaf(-q0, 127.f, amax), kInv127, q0);
  scale16 = __float2half_rn(quo);
  s = __half2float(scale16);
  inv = 0.f;
  if (s >= 6.103515625e-05f && s < INFINITY) asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(s));
}

// int8 codes of the eight elements of one chunk for the row's scale.
template <typename T>
__device__ __forceinline__ uint2 quant_codes(const uint4& raw, float s, float inv) {
  using T2 = typename Elem<T>::T2;
  const T2* p2 = reinterpret_cast<const T2*>(&raw);
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
  uint2 codes;
  uint32_t a01, a23;
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(a01) : "r"(t[0]), "r"(t[1]));
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(a23) : "r"(t[2]), "r"(t[3]));
  asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(codes.x) : "r"(a01), "r"(a23));
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(a01) : "r"(t[4]), "r"(t[5]));
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(a23) : "r"(t[6]), "r"(t[7]));
  asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(codes.y) : "r"(a01), "r"(a23));
  return codes;
}

// One chunk per lane, GROUP lanes form the head row (all 32 lanes of the warp take part in the shuffles).
template <typename T, int GROUP>
__device__ __forceinline__ void quant_chunk(const uint4& raw, uint2& codes, __half& scale16) {
  float amax = chunk_absmax<T>(raw);
#pragma unroll
  for (int off = GROUP / 2; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  float s, inv;
  quant_scale(amax, scale16, s, inv);
  codes = quant_codes<T>(raw, s, inv);
}

}  // namespace mv
