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


// Whether kernels are launched with programmatic dependent launch.  Off unless SB_PDL=1: on
// B200 the decode step of the 7B-sized model measured slower with it (the many small blocks of
// the weight-streaming product gain nothing from starting early and delay their neighbours),
// while the tcgen05 products alone gain a few percent.
static int g_pdl = -1;

extern "C" int sb_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("SB_PDL");
    g_pdl = (e && e[0] == '1') ? 1 : 0;
  }
  return g_pdl;
}

extern "C" void sb_set_pdl(int on) { g_pdl = on ? 1 : 0; }
