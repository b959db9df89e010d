// Shared helpers for the sm_100a kernels behind include/minivllm_b200.h.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/minivllm_b200.h"

namespace mv {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

// Records the message mv_last_error_string() returns on this thread.
int fail(int status, const char* fmt, ...);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Returns MV_OK or records the CUDA error of the launch just issued.
int check_launch(const char* what);

// ---- device-side conversions -------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ float2 to_f2(__half2 x) { return __half22float2(x); }
  static __device__ __forceinline__ __half2 from_f2(float a, float b) { return __floats2half2_rn(a, b); }
  static __device__ __forceinline__ __half2 absmax2(__half2 m, __half2 x) { return __hmax2(m, __habs2(x)); }
  static __device__ __forceinline__ float hmax_f(__half2 m) { return __half2float(__hmax(__low2half(m), __high2half(m))); }
  // maxima that propagate NaN (a NaN anywhere in the inputs gives NaN)
  static __device__ __forceinline__ __half2 max2_nan(__half2 a, __half2 b) { return __hmax2_nan(a, b); }
  static __device__ __forceinline__ float hmax_nan_f(__half2 m) { return __half2float(__hmax_nan(__low2half(m), __high2half(m))); }
};
template <> struct Elem<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
  static __device__ __forceinline__ float2 to_f2(__nv_bfloat162 x) { return __bfloat1622float2(x); }
  static __device__ __forceinline__ __nv_bfloat162 from_f2(float a, float b) { return __floats2bfloat162_rn(a, b); }
  static __device__ __forceinline__ __nv_bfloat162 absmax2(__nv_bfloat162 m, __nv_bfloat162 x) { return __hmax2(m, __habs2(x)); }
  static __device__ __forceinline__ float hmax_f(__nv_bfloat162 m) {
    return __bfloat162float(__hmax(__low2bfloat16(m), __high2bfloat16(m)));
  }
  static __device__ __forceinline__ __nv_bfloat162 max2_nan(__nv_bfloat162 a, __nv_bfloat162 b) { return __hmax2_nan(a, b); }
  static __device__ __forceinline__ float hmax_nan_f(__nv_bfloat162 m) {
    return __bfloat162float(__hmax_nan(__low2bfloat16(m), __high2bfloat16(m)));
  }
};

// 16-byte streaming load that does not allocate in L1 (data is used once).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_global16(void* p, const uint4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// 32-byte store (a whole sector per thread); the address must be 32-byte aligned.
__device__ __forceinline__ void st_global32(void* p, const uint4& a, const uint4& b) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
               "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
}
__device__ __forceinline__ void st_global8(void* p, const uint2& v) {
  asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// 2^x on the special-function unit (2 ulp, flushes denormals): exp2f() adds range handling that the
// attention kernels do not need (their arguments are <= 0 or -inf).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Blackwell packed fp32 pairs: one issue slot for two lanes of work.
__device__ __forceinline__ float2 mul_f32x2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
  return d;
}
__device__ __forceinline__ float2 add_f32x2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
  return d;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Ampere-style 16-byte async copy global -> shared; src_bytes < 16 zero-fills the rest.
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

}  // namespace mv
