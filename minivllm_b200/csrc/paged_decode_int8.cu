// Paged decode attention over an int8 KV cache (per-token-per-head symmetric
// codes with fp16 scales, written by the quantising store_kvcache).
//
// Same plan, work items and warp-private cp.async rings as paged_decode.cu;
// what differs is the operand path.  Codes are dequantised in registers: a
// byte c is byte-permuted into the fp16 pattern 0x64xx = 1024 + (c ^ 0x80) =
// c + 1152 (exact), and the constant 1152 is NOT subtracted per element but
// taken out afterwards where it factors: S = Q.(C + 1152) - 1152 * rowsum(Q),
// O = P'.(C + 1152) - 1152 * rowsum(P'), the latter row sum coming from one
// extra MMA against a tile of ones so that it is exactly what the tensor core
// summed.  The MMAs run in fp16 with fp32 accumulation whatever the model
// dtype (q is converted), and the per-token scales are applied where they
// factor out: the K scale on the score column, the V scale on the
// probability column.  The k index of the
// QK^T MMAs and the n index of the PV MMAs are permuted so that every thread
// reads its operands with 16-byte shared-memory loads.
// HBM-bound: algorithmic bytes = sum(ctx) * num_kv_heads * (head_dim + 2) * 2.
#include "paged_decode.cuh"

namespace mv {

// A warp's loop iteration has a fixed latency (wait, dequantise, dependent MMAs, softmax shuffles) that is
// about the same for 16 or 32 tokens, and int8 rows are half as long as fp16 rows: 32-token tiles keep the
// bytes per iteration (8 KB) equal to the fp16 kernel's.
constexpr int kQTok = 32;     // tokens per warp tile
constexpr int kQStages = 3;
constexpr int kQD = 128;

struct Int8Smem {
  static constexpr int kRowBytes = kQD;                              // one row of codes
  static constexpr int kTileBytes = kQTok * kRowBytes;               // K or V codes of a tile
  static constexpr int kScaleBytes = 2 * kQTok * 4;                  // one 4-byte word per token, K then V
  static constexpr int kStageBytes = 2 * kTileBytes + kScaleBytes;
  static constexpr int kWarpBytes = kQStages * kStageBytes;
  static constexpr int kRingBytes = kDecWarps * kWarpBytes;
  static constexpr int kMergeStride = kQD + 8;
  static constexpr int kMergeBytes = kDecWarps * 16 * kMergeStride * 4 + kDecWarps * 16 * 2 * 4;
  static_assert(kMergeBytes <= kRingBytes, "merge buffer must fit in the ring");
};

__device__ __forceinline__ void cp_async4(uint32_t dst_smem, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ float scale_of(uint32_t word, uint32_t odd) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(odd ? (word >> 16) : (word & 0xffffu))));
}

template <typename T>
__global__ void __launch_bounds__(kDecThreads, kDecCtasPerSM)
paged_decode_int8_kernel(const DecodeParams p) {
  using S = Int8Smem;
  constexpr int D = kQD;
  constexpr int KSTEPS = D / 16;
  constexpr int NT = D / 8;
  constexpr uint32_t kMagic = 0x64646464u, kBias = 0x80808080u;

  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ long long s_red[kDecWarps];
  __shared__ uint32_t s_mask[kDecWarps][kQStages][2];  // [0]: live rows of the tile, [1]: rows whose scale index is odd
  __shared__ int s_last;
  int* s_start = reinterpret_cast<int*>(smem + S::kRingBytes);

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
  const int8_t* kc = static_cast<const int8_t*>(p.k_cache);
  const int8_t* vc = static_cast<const int8_t*>(p.v_cache);
  const int bs = p.block_size;

  ItemWalk at;
  for (walk_start(p, s_start, plan, ydim, n_units, blockIdx.x, at); at.b >= 0;
       walk_next(p, s_start, plan, ydim, n_units, gridDim.x, at)) {
    const int kvh = at.y / p.mtiles, mt = at.y - kvh * p.mtiles;
    const DecodeItem di = piece_of(s_start, plan, at.b, at.seg);
    const int item = di.item, b = di.b, nsplit = di.nsplit, tok_begin = di.tok_begin, tok_end = di.tok_end;
    const int32_t* table = p.block_tables + static_cast<int64_t>(b) * p.bt_stride;
    const int rows_valid = min(16, p.group - mt * 16);
    const int h0 = kvh * p.group + mt * 16;

    const int span = tok_end - tok_begin;
    const int cta_tiles = span > 0 ? (span + kQTok - 1) / kQTok : 0;
    const int my_tiles = cta_tiles > warp ? (cta_tiles - warp + kDecWarps - 1) / kDecWarps : 0;

    auto issue = [&](int i) {
      if (i < my_tiles) {
        const int stage = i % kQStages;
        const int tok0 = tok_begin + (i * kDecWarps + warp) * kQTok;
        const int blk0 = tok0 / bs, off0 = tok0 - blk0 * bs;
        int off = off0 + lane, blk = blk0;           // lane r resolves row r of the tile
        while (off >= bs) { off -= bs; ++blk; }
        int slot = -1;
        if (tok0 + lane < tok_end) {
          const int pb = __ldg(table + blk);
          if (pb >= 0 && pb < p.num_blocks) slot = pb * bs + off;
        }
        const int64_t sidx = static_cast<int64_t>(slot) * p.num_kv_heads + kvh;  // scale index of my row
        const bool is_odd = slot >= 0 && (sidx & 1);
        const uint32_t live = __ballot_sync(0xffffffffu, slot >= 0);
        const uint32_t odd = __ballot_sync(0xffffffffu, is_odd);
        if (lane == 0) { s_mask[warp][stage][0] = live; s_mask[warp][stage][1] = odd; }
        const uint32_t kdst = ring + stage * S::kStageBytes;
        const uint32_t vdst = kdst + S::kTileBytes;
        const uint32_t sdst = vdst + S::kTileBytes;
        // scales: one aligned 4-byte word holding the fp16 (low or high half), K words then V words
        {
          const int64_t base = slot >= 0 ? (is_odd ? sidx - 1 : sidx) : 0;
          const int nbytes = slot >= 0 ? (is_odd ? 4 : 2) : 0;
          cp_async4(sdst + lane * 4, p.k_scale + base, nbytes);
          cp_async4(sdst + (kQTok + lane) * 4, p.v_scale + base, nbytes);
        }
        const int c = lane & 7, r0 = lane >> 3;
#pragma unroll
        for (int it = 0; it < kQTok / 4; ++it) {
          const int r = r0 + it * 4;
          const int s = __shfl_sync(0xffffffffu, slot, r);
          const int64_t boff = s >= 0 ? (static_cast<int64_t>(s) * p.num_kv_heads + kvh) * D + c * 16 : 0;
          const uint32_t doff = r * S::kRowBytes + ((c ^ (r & 7)) << 4);
          cp_async16(kdst + doff, kc + boff, s >= 0 ? 16 : 0);
          cp_async16(vdst + doff, vc + boff, s >= 0 ? 16 : 0);
        }
      }
      cp_async_commit();
    };

#pragma unroll
    for (int i = 0; i < kQStages - 1; ++i) issue(i);

    // Q fragments in fp16 with the permuted k index: k-step ks of thread t
    // covers head-dim elements 32t + 4ks .. 32t + 4ks + 3.
    uint32_t qa[KSTEPS][4];
    {
      const T* qbase = static_cast<const T*>(p.q) + (static_cast<int64_t>(b) * p.num_heads + h0) * D;
#pragma unroll
      for (int half_row = 0; half_row < 2; ++half_row) {
        const int row = g + 8 * half_row;
        const bool ok = row < rows_valid;
        const uint2* src = reinterpret_cast<const uint2*>(qbase + static_cast<int64_t>(row) * D + 32 * t);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          uint2 raw = ok ? __ldg(src + ks) : make_uint2(0u, 0u);
          if constexpr (!std::is_same<T, __half>::value) {
            const float2 a = Elem<T>::to_f2(*reinterpret_cast<typename Elem<T>::T2*>(&raw.x));
            const float2 c2 = Elem<T>::to_f2(*reinterpret_cast<typename Elem<T>::T2*>(&raw.y));
            raw.x = pack2<__half>(a.x, a.y);
            raw.y = pack2<__half>(c2.x, c2.y);
          }
          qa[ks][half_row] = raw.x;       // k = 2t, 2t+1
          qa[ks][2 + half_row] = raw.y;   // k = 2t+8, 2t+9
        }
      }
    }

    // -1152 * sum over head_dim of q, per row: the bias of the un-subtracted codes in S
    float nbias0 = 0.f, nbias1 = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&qa[ks][0]));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&qa[ks][2]));
      const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&qa[ks][1]));
      const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&qa[ks][3]));
      nbias0 += (a.x + a.y) + (b.x + b.y);
      nbias1 += (c.x + c.y) + (d.x + d.y);
    }
    nbias0 += __shfl_xor_sync(0xffffffffu, nbias0, 1);
    nbias0 += __shfl_xor_sync(0xffffffffu, nbias0, 2);
    nbias1 += __shfl_xor_sync(0xffffffffu, nbias1, 1);
    nbias1 += __shfl_xor_sync(0xffffffffu, nbias1, 2);
    nbias0 *= -1152.f;
    nbias1 *= -1152.f;

    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float osum[4] = {0.f, 0.f, 0.f, 0.f};   // P' times a tile of ones: row sums of P' as the tensor core adds them
    float m0 = kNegBig, m1 = kNegBig, l0 = 0.f, l1 = 0.f;
    const uint32_t kOnes = 0x3c003c00u;     // fp16 (1, 1)

    for (int i = 0; i < my_tiles; ++i) {
      cp_async_wait<kQStages - 2>();
      __syncwarp();
      const int stage = i % kQStages;
      const uint32_t kbase = ring + stage * S::kStageBytes;
      const uint32_t vbase = kbase + S::kTileBytes;
      const uint32_t sbase = vbase + S::kTileBytes;
      const uint32_t live = s_mask[warp][stage][0], odd = s_mask[warp][stage][1];

      // ---- S = Q K^T on the codes: four n-tiles of 8 tokens ----
      float s[4][4];
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        const int row = 8 * n + g;
        const uint4 w0 = lds128(kbase + row * S::kRowBytes + (((2 * t) ^ (row & 7)) << 4));
        const uint4 w1 = lds128(kbase + row * S::kRowBytes + (((2 * t + 1) ^ (row & 7)) << 4));
        const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          const uint32_t x = words[ks] ^ kBias;
          Mma16816<__half>::run(s[n], qa[ks], prmt(x, kMagic, 0x4140u), prmt(x, kMagic, 0x4342u));
        }
      }
      issue(i + kQStages - 1);

      // ---- K scales, mask, online softmax ----
      float mx0 = kNegBig, mx1 = kNegBig;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
          const int col = n * 8 + 2 * t + e2;
          const bool ok = (live >> col) & 1u;
          const float ks = scale_of(lds32(sbase + col * 4), (odd >> col) & 1u) * p.scale_log2;
          s[n][e2] = ok ? (s[n][e2] + nbias0) * ks : -INFINITY;
          s[n][2 + e2] = ok ? (s[n][2 + e2] + nbias1) * ks : -INFINITY;
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
      uint32_t pa[2][4];   // A fragments of the two 16-token k-steps
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const float p00 = fast_exp2(s[n][0] - mn0), p01 = fast_exp2(s[n][1] - mn0);
        const float p10 = fast_exp2(s[n][2] - mn1), p11 = fast_exp2(s[n][3] - mn1);
        ps0 += p00 + p01;
        ps1 += p10 + p11;
        // V scale of the two tokens of this column pair, folded into P
        const int col = n * 8 + 2 * t;
        const float vs0 = scale_of(lds32(sbase + (kQTok + col) * 4), (odd >> col) & 1u);
        const float vs1 = scale_of(lds32(sbase + (kQTok + col + 1) * 4), (odd >> (col + 1)) & 1u);
        const bool ok0 = (live >> col) & 1u, ok1 = (live >> (col + 1)) & 1u;
        pa[n >> 1][2 * (n & 1)] = pack2<__half>(ok0 ? p00 * vs0 : 0.f, ok1 ? p01 * vs1 : 0.f);
        pa[n >> 1][2 * (n & 1) + 1] = pack2<__half>(ok0 ? p10 * vs0 : 0.f, ok1 ? p11 * vs1 : 0.f);
      }
      l0 = l0 * a0 + ps0;
      l1 = l1 * a1 + ps1;

      // the running maximum rarely moves after the first tiles: rescale only when some row of the warp needs it
      if (__any_sync(0xffffffffu, a0 != 1.f || a1 != 1.f)) {
#pragma unroll
        for (int j = 0; j < NT; ++j) { o[j][0] *= a0; o[j][1] *= a0; o[j][2] *= a1; o[j][3] *= a1; }
        osum[0] *= a0; osum[1] *= a0; osum[2] *= a1; osum[3] *= a1;
      }
      // ---- O += P V on the codes; n-tile j of thread (g, t) is head-dim element 16*col + j ----
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const int ra = 16 * kk + 2 * t, rb = ra + 1, rc = ra + 8, rd = ra + 9;
        const uint4 va = lds128(vbase + ra * S::kRowBytes + ((g ^ (ra & 7)) << 4));
        const uint4 vb = lds128(vbase + rb * S::kRowBytes + ((g ^ (rb & 7)) << 4));
        const uint4 vcx = lds128(vbase + rc * S::kRowBytes + ((g ^ (rc & 7)) << 4));
        const uint4 vd = lds128(vbase + rd * S::kRowBytes + ((g ^ (rd & 7)) << 4));
        const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
        const uint32_t wc[4] = {vcx.x, vcx.y, vcx.z, vcx.w}, wd[4] = {vd.x, vd.y, vd.z, vd.w};
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const uint32_t xa = wa[wi] ^ kBias, xb = wb[wi] ^ kBias, xc = wc[wi] ^ kBias, xd = wd[wi] ^ kBias;
          const uint32_t lo01 = prmt(xa, xb, 0x5140u), lo23 = prmt(xa, xb, 0x7362u);  // tokens ra, ra+1
          const uint32_t hi01 = prmt(xc, xd, 0x5140u), hi23 = prmt(xc, xd, 0x7362u);  // tokens ra+8, ra+9
          const uint32_t lo[4] = {prmt(lo01, kMagic, 0x4140u), prmt(lo01, kMagic, 0x4342u),
                                  prmt(lo23, kMagic, 0x4140u), prmt(lo23, kMagic, 0x4342u)};
          const uint32_t hi[4] = {prmt(hi01, kMagic, 0x4140u), prmt(hi01, kMagic, 0x4342u),
                                  prmt(hi23, kMagic, 0x4140u), prmt(hi23, kMagic, 0x4342u)};
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) Mma16816<__half>::run(o[4 * wi + jj], pa[kk], lo[jj], hi[jj]);
        }
        Mma16816<__half>::run(osum, pa[kk], kOnes, kOnes);
      }
      __syncwarp();
    }
    cp_async_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // every column of the ones tile carries the same row sum: take the bias of the V codes out of O
    {
      const float b0 = 1152.f * osum[0], b1 = 1152.f * osum[2];
#pragma unroll
      for (int j = 0; j < NT; ++j) { o[j][0] -= b0; o[j][1] -= b0; o[j][2] -= b1; o[j][3] -= b1; }
    }

    __syncthreads();
    float* sO = reinterpret_cast<float*>(smem);
    float* sML = sO + kDecWarps * 16 * S::kMergeStride;
    {
      float* mine = sO + warp * 16 * S::kMergeStride;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        // accumulator column 2t+e of n-tile j holds head-dim element 16*(2t+e) + j
        mine[g * S::kMergeStride + 32 * t + j] = o[j][0];
        mine[g * S::kMergeStride + 32 * t + 16 + j] = o[j][1];
        mine[(g + 8) * S::kMergeStride + 32 * t + j] = o[j][2];
        mine[(g + 8) * S::kMergeStride + 32 * t + 16 + j] = o[j][3];
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
    __syncthreads();
    combine_if_last<T, D>(p, s_start, plan, b, b * ydim + kvh * p.mtiles + mt, h0, rows_valid, nsplit, &s_last);
  }
}

template <typename T>
int launch_decode_int8(const DecodeParams& p, cudaStream_t st) {
  const size_t smem = Int8Smem::kRingBytes + static_cast<size_t>(p.batch + 1) * sizeof(int);
  constexpr size_t kStaticSmem = 256;
  if (smem + kStaticSmem > 227 * 1024)
    return fail(MV_ERR_LIMIT, "paged_decode(int8): batch %d needs %zu bytes of shared memory", p.batch, smem);
  static size_t attr_bytes[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || attr_bytes[dev] < smem) {
    const cudaError_t e = cudaFuncSetAttribute(paged_decode_int8_kernel<T>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(MV_ERR_CUDA, "paged_decode(int8): cudaFuncSetAttribute(%zu): %s", smem, cudaGetErrorString(e));
    }
    if (dev >= 0 && dev < 64) attr_bytes[dev] = smem;
  }
  paged_decode_int8_kernel<T><<<decode_grid(p), kDecThreads, smem, st>>>(p);
  return check_launch("paged_decode_int8_kernel");
}

template int launch_decode_int8<__half>(const DecodeParams&, cudaStream_t);
template int launch_decode_int8<__nv_bfloat16>(const DecodeParams&, cudaStream_t);

}  // namespace mv
