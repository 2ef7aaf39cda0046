#include <cstdarg>
#include <cstring>

#include "common.cuh"

namespace {
thread_local char g_message[512] = "";
}

void psb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_message, sizeof(g_message), fmt, ap);
  va_end(ap);
}

PSB_API const char* psb_last_error() { return g_message; }
