// What every kernel library of the package carries: the error channel and the switches.
// The kernels are built as two libraries, the plain one (everything a float32 model needs)
// and the tensor-core one (bfloat16 products and attention); this file is linked into both, so
// each has an error text and switches of its own.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_last_error[512] = "";
static bool g_pdl = true;

int llmk_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

bool llmk_pdl_enabled() { return g_pdl; }

LLMK_API const char* llmk_last_error() { return g_last_error; }
LLMK_API int llmk_abi_version() { return 2; }
// Programmatic dependent launch between the kernels of a step (on by default).
LLMK_API void llmk_set_pdl(int on) { g_pdl = on != 0; }

