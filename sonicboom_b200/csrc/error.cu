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


// Which kernels are launched with programmatic dependent launch: a mask of SbKernelClass bits
// (SB_PDL=<number> in the environment, sb_set_pdl at run time; 0 = none, 63 = all).  The
// default is every class but the weight-streaming products: on B200 the decode step of the
// 7B-sized model gains 4-5 % that way at batch 1 and 8 (1 % at batch 64 and in prefill), and
// loses about 10 % when the weight-streaming products are launched this way as well.
static int g_pdl = -1;

extern "C" int sb_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("SB_PDL");
    g_pdl = e ? atoi(e) & 63 : (63 & ~SB_K_SKINNY);
  }
  return g_pdl;
}

extern "C" void sb_set_pdl(int mask) { g_pdl = mask & 63; }
