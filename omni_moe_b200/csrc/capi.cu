// Error reporting shared by all entry points of libomni_moe_b200.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace omni {
namespace {
thread_local char g_err[512] = "";
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

bool pdl_enabled() {
  static const bool v = [] {
    const char* e = getenv("OMNI_MOE_B200_PDL");
    return !(e && e[0] == '0');
  }();
  return v;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(-3, "%s: %s", what, cudaGetErrorString(e));
  return 0;
}
}  // namespace omni

extern "C" int omni_version(void) { return 100; }
extern "C" const char* omni_last_error(void) { return omni::g_err; }
