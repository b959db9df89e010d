// Inline-PTX wrappers for the Blackwell (sm_100a) pieces the prefill kernel is
// built from: mbarriers with bounded waits, TMA tensor loads, tensor memory
// (TMEM) allocation and access, and tcgen05.mma with its descriptors.
#pragma once
#include "common.cuh"

namespace mv {
namespace tc {

// ---------------------------------------------------------------- mbarrier ---
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

// Every wait is bounded in time.  When a wait runs out it raises the CTA's
// abort flag (shared memory) and the global error word; after that every wait
// of the CTA returns at once, so all roles run their loops to the end, tensor
// memory is freed and the kernel returns.  The host reads the error word.
constexpr unsigned long long kWaitLimitNs = 200ull * 1000 * 1000;  // a healthy wait is far below a millisecond
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error_word,
                                            int where) {
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > kWaitLimitNs) break;
  }
  *abort_flag = 1;
  atomicCAS(error_word, 0, 0x100 + where);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error_word,
                                          int where) {
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, error_word, where);
}
// The same wait in as little code as possible, for a kernel whose MMA-issuing warp has a dozen waits in its loop:
// that warp shares an instruction cache with the (large) softmax loop, and with the spin loops unrolled its code
// is pushed out of the cache at every unit boundary (measured: 0.61 ms against 0.51 ms on the 32-sequence
// benchmark).  The part that runs when a wait is long is a call.
__device__ __noinline__ bool mbar_wait_long(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error_word,
                                            int where) {
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > kWaitLimitNs) break;
  }
  *abort_flag = 1;
  atomicCAS(error_word, 0, 0x100 + where);
  return false;
}
template <bool kCall>
__device__ __forceinline__ bool mbar_wait_compact(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  int* error_word, int where) {
#pragma unroll 1
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  if (kCall) return mbar_wait_long(bar, parity, abort_flag, error_word, where);
  return mbar_wait_slow(bar, parity, abort_flag, error_word, where);
}
// Wait bounded by time alone (2 ms), for draining copies in flight after an abort.
__device__ __forceinline__ bool mbar_wait_timed(uint32_t bar, uint32_t parity) {
  const unsigned long long t0 = global_ns();
  do {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
  } while (global_ns() - t0 < 2000000ull);
  return false;
}

// --------------------------------------------------------------------- TMA ---
// 3-D tiled load global -> shared, completion counted in bytes on an mbarrier.
// The innermost coordinate times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// -------------------------------------------------------------------- TMEM ---
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane
// (base lane + i), registers r[0..31] = columns col .. col+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// --------------------------------------------------------------------- MMA ---
// Shared-memory operand descriptor, 128-byte swizzle, sm_100 version field.
//   bits  0..13  start address >> 4
//   bits 16..29  leading byte offset >> 4  (K-major: unused, 1; MN-major: stride between 64-element column groups)
//   bits 32..45  stride byte offset >> 4   (distance between 8-row groups)
//   bits 46..47  version = 1
//   bits 61..63  layout = 2 (SWIZZLE_128B)
// The descriptor is kept as its two 32-bit words, so that an issuing thread builds the fixed part once
// and only adds offsets (16-byte units, no carry out of the 14-bit field) to the low word.
constexpr uint32_t kDescHiSw128Sbo1024 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3ffffu) >> 4) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
}
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

// Instruction descriptor of tcgen05.mma.kind::f16: fp32 accumulate, A and B
// formats given separately (0 = fp16, 1 = bf16), A K-major, B K-major or
// MN-major, M x N tile.
__host__ __device__ constexpr uint32_t instr_desc_f16(uint32_t fmt_a, uint32_t fmt_b, bool b_mn_major, uint32_t m,
                                                      uint32_t n) {
  return (1u << 4)                          // accumulator format: f32
         | (fmt_a << 7) | (fmt_b << 10)     // A and B formats
         | (0u << 15)                   // A: K-major
         | ((b_mn_major ? 1u : 0u) << 16)
         | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// The MMA issuer runs its whole loop with all 32 lanes converged and lets ONE elected lane execute the tcgen05
// instructions (elect.sync inside the sequences below): their operands travel through the uniform datapath, and
// a warp that has diverged on `lane == 0` pays ~90-140 cycles per MMA to get them there (measured).
// Eight MMAs over K = 128 and the commit that follows them, issued by one elected lane of a CONVERGED warp in a
// single predicated sequence: the issuing warp shares its scheduler with busy softmax warps, so every
// instruction it does not execute shortens the critical path.  Descriptor offsets (16-byte units) are added
// to the low word; shared-memory addresses stay below 256 KB, so the add never carries out of the address field.
//   D[tmem] (+)= A[smem] * B[smem]; A and B are K-major 128-row tiles stored as two 64-column halves
//   16 KB apart (1024 descriptor units); four K = 16 steps of 32 bytes (2 units) in each half.
__device__ __forceinline__ void mma_ss_k128_commit(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t commit_bar) {
  asm volatile(
      "{\n\t.reg .pred pe, pt, pf;\n\t.reg .b64 da, db;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.eq.u32 pt, %3, %3;\n\t"
      "setp.ne.u32 pf, %3, %3;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
      "add.s64 da, %1, 2;\n\tadd.s64 db, %2, 2;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
      "add.s64 da, %1, 4;\n\tadd.s64 db, %2, 4;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
      "add.s64 da, %1, 6;\n\tadd.s64 db, %2, 6;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
      "add.s64 da, %1, 1024;\n\tadd.s64 db, %2, 1024;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
      "add.s64 da, %1, 1026;\n\tadd.s64 db, %2, 1026;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
      "add.s64 da, %1, 1028;\n\tadd.s64 db, %2, 1028;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
      "add.s64 da, %1, 1030;\n\tadd.s64 db, %2, 1030;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
      "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%4];\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(commit_bar) : "memory");
}
//   D[tmem] (+)= A[tmem] * B[smem]; A holds two 16-bit values per column (8 columns per MMA), B is an MN-major
//   tile whose 16-row slices are 2048 bytes apart.
__device__ __forceinline__ void mma_ts_k128_commit(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                   bool accum, uint32_t commit_bar) {
  const uint32_t acc = accum ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred pe, pt, pf;\n\t.reg .b64 db;\n\t.reg .b32 ta;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.eq.u32 pt, %3, %3;\n\t"
      "setp.ne.u32 pf, %4, 0;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pf;\n\t"
      "add.u32 ta, %1, 8;\n\tadd.s64 db, %2, 128;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, pt;\n\t"
      "add.u32 ta, %1, 16;\n\tadd.s64 db, %2, 256;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, pt;\n\t"
      "add.u32 ta, %1, 24;\n\tadd.s64 db, %2, 384;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, pt;\n\t"
      "add.u32 ta, %1, 32;\n\tadd.s64 db, %2, 512;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, pt;\n\t"
      "add.u32 ta, %1, 40;\n\tadd.s64 db, %2, 640;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, pt;\n\t"
      "add.u32 ta, %1, 48;\n\tadd.s64 db, %2, 768;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, pt;\n\t"
      "add.u32 ta, %1, 56;\n\tadd.s64 db, %2, 896;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, pt;\n\t"
      "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%5];\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc), "r"(commit_bar) : "memory");
}
// One or two commits by the elected lane of a converged warp.
__device__ __forceinline__ void commit_elected(uint32_t bar_a, uint32_t bar_b, bool both) {
  const uint32_t two = both ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred pe, p2;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.ne.u32 p2, %2, 0;\n\t"
      "and.pred p2, p2, pe;\n\t"
      "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "@p2 tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%1];\n\t}"
      ::"r"(bar_a), "r"(bar_b), "r"(two) : "memory");
}
// ------------------------------------------------------- softmax arithmetic ---
// Blackwell packed fp32 pairs (one issue slot for two lanes of work) and the three-input max.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)),
        "l"(reinterpret_cast<unsigned long long&>(c)));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2_mufu(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for a pair on the FMA pipe instead of the 16-per-clock special-function unit:
// round to the nearest integer n by adding 1.5*2^23, a degree-4 polynomial for 2^f on
// f = x - n in [-1/2, 1/2] (relative error 4e-5, well inside the 2^-9 / 2^-11 rounding of P),
// and n added into the exponent field.  x <= -127 gives exactly 0; x must be below 128.
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
  const float kMagic = 12582912.f;
  x.x = fmaxf(x.x, -127.f);
  x.y = fmaxf(x.y, -127.f);
  const float2 t = add2(x, make_float2(kMagic, kMagic));
  const float2 f = add2(x, add2(make_float2(kMagic, kMagic), make_float2(-t.x, -t.y)));   // x - (t - magic)
  float2 p = fma2(f, make_float2(0.0096181291f, 0.0096181291f), make_float2(0.0555041087f, 0.0555041087f));
  p = fma2(p, f, make_float2(0.2402265070f, 0.2402265070f));
  p = fma2(p, f, make_float2(0.6931471806f, 0.6931471806f));
  p = fma2(p, f, make_float2(1.f, 1.f));
  return make_float2(__uint_as_float(__float_as_uint(p.x) + (__float_as_uint(t.x) << 23)),
                     __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(t.y) << 23)));
}

// Register re-partitioning between warpgroups (all four warps of a warpgroup execute it).
__device__ __forceinline__ void setmaxnreg_inc_232() { asm volatile("setmaxnreg.inc.sync.aligned.u32 232;"); }
__device__ __forceinline__ void setmaxnreg_dec_40() { asm volatile("setmaxnreg.dec.sync.aligned.u32 40;"); }

}  // namespace tc
}  // namespace mv
