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

// Streaming multiprocessors of the current device, asked once per device.
int llmk_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (cached[dev] <= 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    cached[dev] = n;
  }
  return cached[dev];
}
LLMK_API int llmk_device_sm_count() { return llmk_sm_count(); }

// Error words of the kernels whose waits are bounded: a kernel whose wait gave up stores a code
// in its word and returns.  The words live in a block of four ints that the caller owns
// (llmk_set_error_block: an engine points it at its own status buffer, so that one copy shows
// every word) or, without one, in a block that the library allocates at first use.
static int* g_error_block = nullptr;
static int* g_own_error_block = nullptr;

int* llmk_error_word(int which) {
  if (g_error_block) return g_error_block + which;
  if (!g_own_error_block) {
    if (cudaMalloc(&g_own_error_block, 4 * sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(g_own_error_block, 0, 4 * sizeof(int));
  }
  return g_own_error_block + which;
}

// block: four device ints (word 1: tensor-core product, word 2: tensor-core attention), zero
// when nothing went wrong; nullptr: back to the library's own block.
LLMK_API void llmk_set_error_block(int* block) { g_error_block = block; }

LLMK_API const char* llmk_last_error() { return g_last_error; }
LLMK_API int llmk_abi_version() { return 2; }
// Programmatic dependent launch between the kernels of a step (on by default).
LLMK_API void llmk_set_pdl(int on) { g_pdl = on != 0; }

