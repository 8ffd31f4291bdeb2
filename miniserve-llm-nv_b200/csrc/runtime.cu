// Library-wide state: the last error message and a version word for the bindings.
#include "common.cuh"

namespace ms {
static thread_local char g_error[512] = "";
char* error_buffer() { return g_error; }
}  // namespace ms

MS_EXPORT const char* ms_last_error() { return ms::error_buffer(); }

// Bumped whenever an exported signature changes; the bindings refuse a library that
// reports another number.
MS_EXPORT int ms_abi_version() { return 1; }
