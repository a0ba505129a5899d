// Error reporting and version of the mcop_b200 C ABI.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace mcop {
namespace {
thread_local char g_error[512] = "";
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return MCOP_OK;
  return set_error(MCOP_ERR_CUDA, "%s: kernel launch failed: %s", what, cudaGetErrorString(e));
}
}  // namespace mcop

extern "C" int mcop_version(void) { return 100; }
extern "C" const char* mcop_last_error(void) { return mcop::g_error; }
