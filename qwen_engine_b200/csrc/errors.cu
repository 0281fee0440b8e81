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

// ---- timeline build: the buffer of the probes in pdl_wait / pdl_launch_dependents (common.cuh) -----------
// qe_timeline_begin(capacity) allocates (once) and clears a buffer of that many events and hands it to every
// translation unit; qe_timeline_read copies the events recorded since (four 64-bit words each) to the host and
// returns their number; both synchronise the device.  In a build without QE_TIMELINE they return -1.
#ifdef QE_TIMELINE
static void (*g_tl_setters[64])(unsigned long long*);
static int g_tl_n_setters = 0;
void qe_tl_register(void (*setter)(unsigned long long*)) {
  if (g_tl_n_setters < 64) g_tl_setters[g_tl_n_setters++] = setter;
}
static unsigned long long* g_tl_dev = nullptr;
static unsigned long long g_tl_cap = 0;
extern "C" long qe_timeline_begin(long capacity) {
  cudaDeviceSynchronize();
  if (g_tl_dev == nullptr || (unsigned long long)capacity > g_tl_cap) {
    if (g_tl_dev) cudaFree(g_tl_dev);
    if (cudaMalloc(&g_tl_dev, (4 + 4 * (size_t)capacity) * 8) != cudaSuccess) { g_tl_dev = nullptr; return -2; }
    g_tl_cap = (unsigned long long)capacity;
  }
  const unsigned long long head[2] = {0ull, g_tl_cap};
  cudaMemcpy(g_tl_dev, head, sizeof(head), cudaMemcpyHostToDevice);
  for (int i = 0; i < g_tl_n_setters; ++i) g_tl_setters[i](g_tl_dev);
  cudaDeviceSynchronize();
  return (long)g_tl_cap;
}
extern "C" long qe_timeline_read(unsigned long long* events, long max_events) {
  if (!g_tl_dev) return 0;
  cudaDeviceSynchronize();
  unsigned long long n = 0;
  cudaMemcpy(&n, g_tl_dev, 8, cudaMemcpyDeviceToHost);
  if (n > g_tl_cap) n = g_tl_cap;
  if ((long)n > max_events) n = (unsigned long long)max_events;
  cudaMemcpy(events, g_tl_dev + 4, (size_t)n * 32, cudaMemcpyDeviceToHost);
  return (long)n;
}
#else
extern "C" long qe_timeline_begin(long) { return -1; }
extern "C" long qe_timeline_read(unsigned long long*, long) { return -1; }
#endif
