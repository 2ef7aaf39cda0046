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

int psb_pdl_enabled = 1;

// 1: launch kernels so that each may overlap its start with the end of its predecessor; 0: plain stream order.
PSB_API void psb_set_pdl(int on) { psb_pdl_enabled = on ? 1 : 0; }
PSB_API int psb_get_pdl() { return psb_pdl_enabled; }
