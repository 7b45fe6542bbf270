// Next-token choice on the device: greedy argmax (ties to the lowest id, as
// kernel/sampling/Argmax.h:20-43 of the reference) and temperature sampling by
// inverse CDF.  The reference has greedy only; the draw here takes a uniform number
// per row from the host, which derives it from (seed, request, position) so that it
// does not depend on the batch.  Softmax runs in float32 with a fixed summation order.
#include <limits.h>

#include "common.cuh"

namespace {

constexpr int THREADS = 256;

__global__ void __launch_bounds__(THREADS)
sample_rows_kernel(int* __restrict__ out, const float* __restrict__ logits, long long row_stride, int vocab,
                   const float* __restrict__ temperature, const float* __restrict__ uniform) {
  __shared__ float vals[THREADS];
  __shared__ int idxs[THREADS];
  __shared__ float sums[THREADS];
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * row_stride;

  // Each thread owns one contiguous span of the row.
  const int span = (vocab + THREADS - 1) / THREADS;
  const int begin = min(tid * span, vocab), end = min(begin + span, vocab);

  float best = -INFINITY;
  int best_i = INT_MAX;
  for (int i = begin; i < end; ++i) {
    const float v = row[i];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  vals[tid] = best;
  idxs[tid] = best_i;
  __syncthreads();
  for (int s = THREADS / 2; s > 0; s >>= 1) {
    if (tid < s) {
      const float ov = vals[tid + s];
      const int oi = idxs[tid + s];
      if (ov > vals[tid] || (ov == vals[tid] && oi < idxs[tid])) { vals[tid] = ov; idxs[tid] = oi; }
    }
    __syncthreads();
  }
  const float row_max = vals[0];
  const int arg = idxs[0];
  const float temp = temperature ? temperature[r] : 0.f;
  if (!(temp > 0.f)) {
    if (tid == 0) out[r] = arg;
    return;
  }

  const float inv_t = 1.f / temp;
  float local = 0.f;
  for (int i = begin; i < end; ++i) local += expf((row[i] - row_max) * inv_t);
  sums[tid] = local;
  __syncthreads();
  if (tid == 0) {
    float total = 0.f;
    for (int i = 0; i < THREADS; ++i) total += sums[i];
    const float target = uniform[r] * total;
    float run = 0.f;
    int owner = THREADS - 1;
    for (int i = 0; i < THREADS; ++i) {
      if (run + sums[i] > target) { owner = i; break; }
      run += sums[i];
    }
    // Walk the owner's span; fall back to the last id that has any mass.
    const int ob = min(owner * span, vocab), oe = min(ob + span, vocab);
    int pick = -1;
    for (int i = ob; i < oe; ++i) {
      run += expf((row[i] - row_max) * inv_t);
      if (run > target) { pick = i; break; }
    }
    if (pick < 0) pick = (oe > ob) ? oe - 1 : arg;
    out[r] = pick;
  }
}

}  // namespace

// logits [rows, row_stride] float32; temperature[r] <= 0 (or a null pointer) means greedy;
// uniform[r] in [0, 1) is the draw for row r.
LLMK_API int llmk_sample_rows(int* out, const float* logits, long long row_stride, int rows, int vocab,
                              const float* temperature, const float* uniform, cudaStream_t stream) {
  if (rows == 0) return 0;
  LLMK_REQUIRE(vocab > 0 && row_stride >= vocab, "sample_rows: bad vocab %d / stride %lld", vocab, row_stride);
  LLMK_REQUIRE(temperature == nullptr || uniform != nullptr, "sample_rows: temperatures need uniforms");
  launch_kernel(sample_rows_kernel, dim3(rows), dim3(THREADS), 0, stream, out, logits, row_stride, vocab, temperature, uniform);
  LLMK_LAUNCH_CHECK("sample_rows");
}


// token_ids[dst[i]] = sampled[src[i]]: the tokens that the previous step sampled become the
// inputs of this step without a round trip through the host.
__global__ void feed_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ sampled,
                                   const int* __restrict__ dst, const int* __restrict__ src, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) token_ids[dst[i]] = sampled[src[i]];
}

LLMK_API int llmk_feed_tokens(int* token_ids, const int* sampled, const int* dst, const int* src, int n,
                              cudaStream_t stream) {
  if (n == 0) return 0;
  launch_kernel(feed_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, token_ids, sampled, dst, src, n);
  LLMK_LAUNCH_CHECK("feed_tokens");
}
