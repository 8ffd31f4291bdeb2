// Library-wide state: the last error message and a version word for the bindings.
#include "common.cuh"

#include <stdlib.h>

namespace ms {
static thread_local char g_error[512] = "";
char* error_buffer() { return g_error; }

static int g_dependent_launch = -1;
bool dependent_launch_enabled() {
  if (g_dependent_launch < 0) {
    const char* value = getenv("MINISERVE_B200_DEPENDENT_LAUNCH");
    g_dependent_launch = (value != nullptr && value[0] == '0') ? 0 : 1;
  }
  return g_dependent_launch == 1;
}
}  // namespace ms

MS_EXPORT const char* ms_last_error() { return ms::error_buffer(); }

// Bumped whenever an exported signature changes; the bindings refuse a library that
// reports another number.
MS_EXPORT int ms_abi_version() { return 5; }

// 1: kernels are launched as programmatic dependents (default); 0: plain stream order.
MS_EXPORT void ms_set_dependent_launch(int enabled) { ms::g_dependent_launch = enabled ? 1 : 0; }
