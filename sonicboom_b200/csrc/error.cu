// The last-error string of a kernel library.  Every library built from this folder links its
// own copy, so a message is read from the library whose call failed.
#include <stdarg.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

extern "C" const char* sb_last_error() { return g_error; }

void sb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

