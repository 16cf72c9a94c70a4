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

bool make_gla_fusion(GlaFusion* fu, const char* who, int flags, float gate_normalizer,
                     const void* norm_weight, float norm_eps) {
  if (flags & ~(SBK_GLA_RELU_QK | SBK_GLA_GATE_LOGITS)) {
    set_error("%s: unknown fuse_flags 0x%x", who, flags);
    return false;
  }
  if ((flags & SBK_GLA_GATE_LOGITS) && !(gate_normalizer > 0.f)) {
    set_error("%s: gate_normalizer must be positive with SBK_GLA_GATE_LOGITS", who);
    return false;
  }
  fu->relu_qk = (flags & SBK_GLA_RELU_QK) != 0;
  fu->gate_logits = (flags & SBK_GLA_GATE_LOGITS) != 0;
  fu->gate_normalizer = gate_normalizer;
  fu->norm_weight = norm_weight;
  fu->norm_eps = norm_eps;
  return true;
}

}  // namespace sbk

extern "C" int sbk_abi_version(void) { return SBK_ABI_VERSION; }
extern "C" const char* sbk_last_error(void) { return sbk::g_err; }
