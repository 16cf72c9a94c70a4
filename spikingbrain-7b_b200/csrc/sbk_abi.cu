// Host-side plumbing shared by the entry points of libsbk: the thread-local
// error string, launch checking and the ABI version.
#include <stdarg.h>
#include <stdio.h>

#include "sbk_common.cuh"

namespace sbk {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return SBK_OK;
  set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
  return SBK_E_LAUNCH;
}

}  // namespace sbk

extern "C" int sbk_abi_version(void) { return SBK_ABI_VERSION; }
extern "C" const char* sbk_last_error(void) { return sbk::g_err; }
