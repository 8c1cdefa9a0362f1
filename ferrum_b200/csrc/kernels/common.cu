// Error text of the C entry points.  Every entry point returns 0 on success; on a
// refusal (bad sizes, a failed launch) it returns non-zero and leaves a message that
// ferrum_last_error() returns to the caller on the same thread.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>

static thread_local char g_error[512] = "";

void ferrum_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

FERRUM_API const char* ferrum_last_error() { return g_error; }

// Version of the kernel library's C interface; the Python side refuses a stale build.
FERRUM_API int ferrum_kernels_abi() { return 7; }

// Dependent launch (see common.cuh) can be switched off, e.g. to compare timings.
static bool g_dependent_launch = true;
bool ferrum_dependent_launch_enabled() { return g_dependent_launch; }
FERRUM_API void ferrum_set_dependent_launch(int on) { g_dependent_launch = on != 0; }
