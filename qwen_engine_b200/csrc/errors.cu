// Error text of the last refused or failed call of this thread.
#include "common.cuh"
#include <cstdarg>
#include <cstdio>

static thread_local char g_error[512] = "";

void qe_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

extern "C" const char* qe_last_error() { return g_error; }

extern "C" int qe_abi_version() { return 1; }

static int g_pdl_enabled = 1;
extern "C" void qe_set_pdl(int enabled) { g_pdl_enabled = enabled ? 1 : 0; }
int qe_pdl_enabled() { return g_pdl_enabled; }
