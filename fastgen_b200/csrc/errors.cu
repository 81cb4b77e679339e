// Error message plumbing of the C interface.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void fg_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

extern "C" const char* fg_last_error() { return g_error; }

extern "C" int fg_abi_version() { return 1; }

bool fg_pdl_enabled() {
  static int state = -1;
  if (state < 0) {
    const char* v = getenv("FG_NO_PDL");
    state = (v != nullptr && v[0] != 0 && v[0] != '0') ? 0 : 1;
  }
  return state == 1;
}
