// The last-error string of a kernel library.  Every library built from this folder links its
// own copy, so a message is read from the library whose call failed.
#include <stdarg.h>
#include <stdlib.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

extern "C" const char* sb_last_error() { return g_error; }

void sb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}


// Whether kernels are launched with programmatic dependent launch: SB_PDL=0 never, 1 every
// kernel, 2 only the tcgen05 products (which request weights before their wait).  Off by default: on
// B200 the decode step of the 7B-sized model measured slower with it (the many small blocks of
// the weight-streaming product gain nothing from starting early and delay their neighbours),
// while the tcgen05 products alone gain a few percent.
static int g_pdl = -1;

extern "C" int sb_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("SB_PDL");
    g_pdl = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 0;
  }
  return g_pdl;
}

extern "C" void sb_set_pdl(int level) { g_pdl = level < 0 ? 0 : (level > 2 ? 2 : level); }
