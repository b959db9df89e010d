// mv_paged_decode_static: paged decode attention for callers that cannot
// allocate device memory.
//
// mv_paged_decode needs a scratch buffer for the partial results of sequences
// whose KV range was split between CTAs, and its caller has to allocate that
// buffer.  Some callers cannot: a serving process that handed all of its HBM
// to the KV-cache pool at start-up and runs with allocation disabled, a
// latency-critical loop that may not take the allocator's lock, or a host
// binding that was only ever given input and output pointers.  (It is not
// for CUDA host callbacks: like any launch it may not be made from one.)
// For them the scratch lives
// in a fixed array in device memory that is part of this library: every GPU
// that loads the library holds kStaticScratchBytes until the process exits.
//
// Rules that follow from sharing one array:
//   * problems whose scratch need exceeds kStaticScratchBytes are rejected
//     (MV_ERR_LIMIT) before anything is launched;
//   * every call on a device uses the same array and it keeps what the last
//     call left there.  Nothing in it has to start at zero: the kernels write
//     every word they later read, so no clearing is done;
//   * two calls that overlap on the GPU (different streams, or graphs
//     replayed concurrently) race on the array.  Serialise them.
//   * the first call on each device looks up the array's device address; make
//     that first call outside any stream capture, and from one host thread
//     (the per-device table of addresses is filled without locking);
//   * the looked-up address belongs to the device's current context: after a
//     cudaDeviceReset it is stale and the library must be reloaded.
#include "common.cuh"

namespace mv {

constexpr int64_t kStaticScratchBytes = 8ll << 20;  // 8 MiB: e.g. batch 440 at 32 query heads, batch 950 at 16 (any context length)

// In host code this name is only a handle for the runtime, not an address a
// kernel could use: the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

// Device address of the array on the current device, looked up once per device.
static int static_scratch(void** out) {
  static void* cached[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(MV_ERR_CUDA, "paged_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
  }
  if (dev >= 0 && dev < 64 && cached[dev]) {
    *out = cached[dev];
    return MV_OK;
  }
  void* ptr = nullptr;
  e = cudaGetSymbolAddress(&ptr, g_decode_scratch);  // resolves for the device that is current right now
  if (e != cudaSuccess || ptr == nullptr) {
    cudaGetLastError();
    return fail(MV_ERR_CUDA, "paged_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
  }
  if (dev >= 0 && dev < 64) cached[dev] = ptr;
  *out = ptr;
  return MV_OK;
}

}  // namespace mv

extern "C" int64_t mv_paged_decode_static_capacity(void) { return mv::kStaticScratchBytes; }

extern "C" int mv_paged_decode_static(void* out, const void* q, const void* k_cache, const void* v_cache,
                                      const void* k_scale, const void* v_scale, const int32_t* block_tables,
                                      int64_t bt_stride, int max_blocks, const void* context_lens, int ctx_is_i64,
                                      int batch, int num_heads, int num_kv_heads, int head_dim, int block_size,
                                      int64_t num_blocks, float scale, int dtype, void* stream) {
  using namespace mv;
  if (batch == 0) return MV_OK;
  const int64_t need = mv_paged_decode_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, max_blocks, block_size);
  if (need < 0) return fail(MV_ERR_SHAPE, "paged_decode_static: invalid shape");
  if (need > kStaticScratchBytes)
    return fail(MV_ERR_LIMIT,
                "paged_decode_static: this problem needs %lld bytes of scratch, the built-in array holds %lld; "
                "use mv_paged_decode with a caller-owned workspace",
                static_cast<long long>(need), static_cast<long long>(kStaticScratchBytes));
  void* scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc) return rc;
  return mv_paged_decode(out, q, k_cache, v_cache, k_scale, v_scale, block_tables, bt_stride, max_blocks, context_lens,
                         ctx_is_i64, batch, num_heads, num_kv_heads, head_dim, block_size, num_blocks, scale, scratch,
                         kStaticScratchBytes, dtype, stream);
}
