// Error plumbing shared by every extern "C" entry point.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace fb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
}

int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return FB_OK;
  set_error("%s: %s", what, cudaGetErrorString(e));
  return FB_ERR_LAUNCH;
}

}  // namespace fb

extern "C" int fb_version(void) { return 1; }
extern "C" const char* fb_last_error(void) { return fb::g_error; }

extern "C" int fb_status_word(void) {
  const int a = fb::status_word_tcgen05(), b = fb::status_word_peer(), c = fb::status_word_gemv_stream();  // (all read, so all are cleared)
  return a ? a : b ? b : c;
}
