// Row-wise kernels: embedding gather, residual add fused with RMSNorm, row gather
// for the LM head, SiLU(gate) * up.  The residual stream is float32 in every mode;
// sums, the reciprocal root and the scaling are float32 as well.  An input that comes
// from a split-K product may be given as its float32 partial results, which are summed
// here in a fixed order instead of by a kernel of their own.
#include "common.cuh"

// ---- embedding --------------------------------------------------------------
// resid[t, :] = table[ids[t], :]   (the reference copies rows without scaling,
// kernel/embedding/TokenEmbedding.h:12-17).  An id outside the table sets *status.
template <typename T>
__global__ void embedding_kernel(float* __restrict__ resid, const T* __restrict__ table,
                                 const int* __restrict__ ids, int hidden, int vocab,
                                 int* __restrict__ status) {
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) resid[(size_t)t * hidden + c] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) resid[(size_t)t * hidden + c] = to_f32(row[c]);
}

LLMK_API int llmk_embedding(float* resid, const void* table, const int* ids, int n_tokens, int hidden,
                            int vocab, int dtype, int* status, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(embedding_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, resid, (const T*)table, ids, hidden, vocab, status);
    LLMK_LAUNCH_CHECK("embedding");
  });
}

// ---- residual add + RMSNorm -------------------------------------------------
// resid += delta (if delta); out = resid * rsqrt(mean(resid^2) + eps) * gamma.
// The reference runs the add and the norm as two kernels (kernel/residual/Residual.h:17-19,
// kernel/LayerNorm/RMSNorm.h:13-30,40-42); here they share one pass over the row.
template <typename T, bool VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, MaybePartial<T> delta,
                                   const float* __restrict__ gamma, T* __restrict__ out, int hidden,
                                   float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * hidden;
  const bool has_delta = delta.present();
  float ss = 0.f;
  if (VEC) {
    // eight elements per thread and pass; a row of up to 8 * blockDim stays in registers
    float keep[8];
    const bool single = hidden <= 8 * (int)blockDim.x;
    for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
      float v[8];
      Vec8<float>::load(resid + base + c, v);
      if (has_delta) {
        float d[8];
        delta.at8(base + c, d);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += d[i];
        Vec8<float>::store(resid + base + c, v);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) { ss += v[i] * v[i]; keep[i] = v[i]; }
    }
    const float total = block_sum(ss, scratch);
    const float rstd = rsqrtf(total / (float)hidden + eps);
    if (out) {
      for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
        float v[8], g[8];
        if (single) {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = keep[i];
        } else {
          Vec8<float>::load(resid + base + c, v);
        }
        Vec8<float>::load(gamma + c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = v[i] * rstd * g[i];
        Vec8<T>::store(out + base + c, v);
      }
    }
    return;
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = resid[base + c];
    if (has_delta) {
      v += delta.at(base + c);
      resid[base + c] = v;
    }
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (out) {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
      out[base + c] = from_f32<T>(resid[base + c] * rstd * gamma[c]);
  }
}

// delta: [rows, hidden] of the element kind, or null; partials: [splits][rows][hidden] float32
// (split_stride elements apart), or null.  At most one of the two is given.
LLMK_API int llmk_add_rmsnorm(float* resid, const void* delta, const float* partials, int splits,
                              long long split_stride, const float* gamma, void* out, int rows, int hidden,
                              float eps, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  LLMK_REQUIRE(!(delta && partials), "add_rmsnorm: give delta or partials, not both");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> d{(const T*)delta, partials, splits, split_stride};
    const bool vec = hidden % 8 == 0 && d.vector_ok() && (uintptr_t)resid % 16 == 0 && (uintptr_t)gamma % 16 == 0 &&
                     (uintptr_t)out % 16 == 0;
    if (vec)
      launch_kernel(add_rmsnorm_kernel<T, true>, dim3(rows), dim3(256), 0, stream, resid, d, gamma, (T*)out, hidden, eps);
    else
      launch_kernel(add_rmsnorm_kernel<T, false>, dim3(rows), dim3(256), 0, stream, resid, d, gamma, (T*)out, hidden, eps);
    LLMK_LAUNCH_CHECK("add_rmsnorm");
  });
}

// ---- gather of the rows whose logits are wanted -----------------------------
// out[r, :] = resid[rows[r], :] (+ delta[rows[r], :]).  The reference runs its LM head
// on every row (model/modules/Linear.h:25); gathering first leaves only wanted rows.
template <typename T>
__global__ void gather_rows_kernel(float* __restrict__ out, const float* __restrict__ resid,
                                   MaybePartial<T> delta, const int* __restrict__ rows, int hidden) {
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const size_t src = (size_t)rows[blockIdx.x] * hidden, dst = (size_t)blockIdx.x * hidden;
  const bool has_delta = delta.present();
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = resid[src + c];
    if (has_delta) v += delta.at(src + c);
    out[dst + c] = v;
  }
}

LLMK_API int llmk_gather_rows(float* out, const float* resid, const void* delta, const float* partials,
                              int splits, long long split_stride, const int* rows, int n_rows, int hidden,
                              int dtype, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  LLMK_REQUIRE(!(delta && partials), "gather_rows: give delta or partials, not both");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> d{(const T*)delta, partials, splits, split_stride};
    launch_kernel(gather_rows_kernel<T>, dim3(n_rows), dim3(256), 0, stream, out, resid, d, rows, hidden);
    LLMK_LAUNCH_CHECK("gather_rows");
  });
}

// out[i] = in[i] rounded to the element type: float32 rows handed to a product without a norm
// between (a head that takes the stream as it is).
template <typename T>
__global__ void cast_rows_kernel(T* __restrict__ out, const float* __restrict__ in, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(in[i]);
}

LLMK_API int llmk_cast_rows(void* out, const float* in, long long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  size_t blocks = ((size_t)n + 255) / 256;
  if (blocks > (size_t)llmk_sm_count() * 8) blocks = (size_t)llmk_sm_count() * 8;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(cast_rows_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, in, (size_t)n);
    LLMK_LAUNCH_CHECK("cast_rows");
  });
}

// x[r, c] += bias[c] (float32 sum, rounded once): the bias of a projection whose product is
// already summed.  The reference adds it in its products' epilogues (kernel/Gemm/QKVGemm.h:27-45,
// model/modules/Linear.h:12-34).
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, long long stride, const float* __restrict__ bias, int rows, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)rows * cols;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols;
    const int c = (int)(i - r * cols);
    T* p = x + r * stride + c;
    *p = from_f32<T>(to_f32(*p) + bias[c]);
  }
}

LLMK_API int llmk_add_bias(void* x, long long stride, const float* bias, int rows, int cols, int dtype, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  size_t blocks = ((size_t)rows * cols + 255) / 256;
  if (blocks > (size_t)llmk_sm_count() * 16) blocks = (size_t)llmk_sm_count() * 16;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(add_bias_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)x, stride, bias, rows, cols);
    LLMK_LAUNCH_CHECK("add_bias");
  });
}

// ---- SiLU(gate) * up --------------------------------------------------------
// in [rows, 2*inter]: gate in the first half of a row, up in the second.
// act = g / (1 + exp(-g)) * u in float32 (kernel/activation/SwiGLU.h:31-33).
template <typename T, bool VEC>
__global__ void silu_mul_kernel(T* __restrict__ out, MaybePartial<T> in, int inter, size_t total) {
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  if (VEC) {
    const unsigned per_row = inter / 8;
    const size_t n_vec = total / 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
      const size_t r = i / per_row;
      const unsigned c = (unsigned)(i - r * per_row) * 8;
      float g[8], u[8];
      in.at8(r * 2 * inter + c, g);
      in.at8(r * 2 * inter + inter + c, u);
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = g[k] / (1.0f + expf(-g[k])) * u[k];
      Vec8<T>::store(out + r * inter + c, g);
    }
    return;
  }
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / inter, c = i % inter;
    const float g = in.at(r * 2 * inter + c);
    const float u = in.at(r * 2 * inter + inter + c);
    out[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
  }
}

LLMK_API int llmk_silu_mul(void* out, const void* gate_up, const float* partials, int splits,
                           long long split_stride, int rows, int inter, int dtype, cudaStream_t stream) {
  const size_t total = (size_t)rows * inter;
  if (total == 0) return 0;
  LLMK_REQUIRE((gate_up != nullptr) != (partials != nullptr), "silu_mul: give gate_up or partials");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> in{(const T*)gate_up, partials, splits, split_stride};
    const bool vec = inter % 8 == 0 && in.vector_ok() && (uintptr_t)out % 16 == 0;
    size_t blocks = ((vec ? total / 8 : total) + 255) / 256;
    if (blocks > (size_t)llmk_sm_count() * 32) blocks = (size_t)llmk_sm_count() * 32;
    if (vec)
      launch_kernel(silu_mul_kernel<T, true>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, in, inter, total);
    else
      launch_kernel(silu_mul_kernel<T, false>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, in, inter, total);
    LLMK_LAUNCH_CHECK("silu_mul");
  });
}
