// Status bookkeeping shared by every entry point of include/minivllm_b200.h.
#include <stdarg.h>
#include "common.cuh"

namespace mv {

static thread_local char g_last_error[512] = "";

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaPeekAtLastError();
  if (e == cudaSuccess) return MV_OK;
  // Clear the (non-sticky) launch error so the next call starts clean.
  cudaGetLastError();
  return fail(MV_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

}  // namespace mv

extern "C" const char* mv_last_error_string(void) { return mv::g_last_error; }

extern "C" int mv_abi_version(void) { return 2; }
