// Rotate-half RoPE on q and k, and the write of k and v into the paged cache.
//
// The reference does this in the epilogue of its QKV product
// (kernel/Gemm/QKVGemm.h:27-63): (a, b) = (x_i, x_{i+HS/2}),
// y_i = a*cos - b*sin, y_{i+HS/2} = a*sin + b*cos with float32 tables
// (kernel/embedding/RoPECache.h:15-20), k and v stored at the physical place that
// the step's metadata names (runtime/Engine.h:62-67).  This stand-alone form serves
// every size; the cache layout is [page][kv_head][token in page][head_dim].
#include "common.cuh"

namespace {

template <typename T, bool VEC>
__global__ void rope_kv_write_kernel(MaybePartial<T> src, long long src_stride, T* __restrict__ q_out,
                                     long long q_out_stride,
                                     const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                     int rot_half, const int* __restrict__ positions,
                                     const int* __restrict__ slot_map, T* __restrict__ k_pages,
                                     T* __restrict__ v_pages, int n_heads, int n_kv, int head_dim,
                                     int page_size) {
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = slot_map[t];
  const int page = slot / page_size, off = slot % page_size;
  const size_t row = (size_t)t * src_stride;
  T* q_row = q_out + (size_t)t * q_out_stride;
  const int half = head_dim / 2;
  const float* cs = cos_table ? cos_table + (size_t)pos * rot_half : nullptr;
  const float* sn = cos_table ? sin_table + (size_t)pos * rot_half : nullptr;
  if (VEC) {
    // eight pairs per thread: half is a multiple of 8 because head_dim is a multiple of 16
    const int per_head = half / 8;
    const int tid = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
    for (int idx = tid; idx < (n_heads + n_kv) * per_head; idx += stride) {
      const int head = idx / per_head, i = (idx % per_head) * 8;
      const size_t h = row + (size_t)head * head_dim;
      float a[8], b[8], c[8], s[8], ya[8], yb[8];
      src.at8(h + i, a);
      src.at8(h + i + half, b);
      if (cs) {
        Vec8<float>::load(cs + i, c);
        Vec8<float>::load(sn + i, s);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) { c[k] = 1.f; s[k] = 0.f; }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) { ya[k] = a[k] * c[k] - b[k] * s[k]; yb[k] = a[k] * s[k] + b[k] * c[k]; }
      T* dst = head < n_heads ? q_row + (size_t)head * head_dim
                              : k_pages + (((size_t)page * n_kv + (head - n_heads)) * page_size + off) * head_dim;
      Vec8<T>::store(dst + i, ya);
      Vec8<T>::store(dst + i + half, yb);
    }
    const size_t v = row + (size_t)(n_heads + n_kv) * head_dim;
    for (int idx = tid * 8; idx < n_kv * head_dim; idx += stride * 8) {
      const int g = idx / head_dim, d = idx % head_dim;
      float x[8];
      src.at8(v + idx, x);
      Vec8<T>::store(v_pages + (((size_t)page * n_kv + g) * page_size + off) * head_dim + d, x);
    }
    return;
  }
  const int rot_items = (n_heads + n_kv) * half;
  for (int idx = threadIdx.x; idx < rot_items; idx += blockDim.x) {
    const int head = idx / half, i = idx % half;
    const size_t h = row + (size_t)head * head_dim;
    const float a = src.at(h + i), b = src.at(h + i + half);
    const float c = cs ? cs[i] : 1.f, s = cs ? sn[i] : 0.f;
    const T ya = from_f32<T>(a * c - b * s), yb = from_f32<T>(a * s + b * c);
    if (head < n_heads) {
      q_row[(size_t)head * head_dim + i] = ya;
      q_row[(size_t)head * head_dim + i + half] = yb;
    } else {
      const int g = head - n_heads;
      T* dst = k_pages + (((size_t)page * n_kv + g) * page_size + off) * head_dim;
      dst[i] = ya;
      dst[i + half] = yb;
    }
  }
  const size_t v = row + (size_t)(n_heads + n_kv) * head_dim;
  for (int idx = threadIdx.x; idx < n_kv * head_dim; idx += blockDim.x) {
    const int g = idx / head_dim, d = idx % head_dim;
    v_pages[(((size_t)page * n_kv + g) * page_size + off) * head_dim + d] = from_f32<T>(src.at(v + idx));
  }
}

}  // namespace

// A row of the source holds q heads, then k heads, then v heads; the source is qkv
// [n_tokens, src_stride] of the element kind, or the float32 partial results
// [splits][n_tokens][src_stride] of a split-K product.  Rotated q goes to q_out (which may be
// the source itself: every pair is read and written by one thread), rotated k and plain v go
// to the pages.  Tables are [max_position, head_dim/2]; without tables (null) nothing is
// rotated and k, v are only stored.
LLMK_API int llmk_rope_kv_write(const void* qkv, const float* partials, int splits, long long split_stride,
                                long long src_stride, void* q_out, long long q_out_stride, const float* cos_table,
                                const float* sin_table, const int* positions, const int* slot_map,
                                void* k_pages, void* v_pages, int n_tokens, int n_heads, int n_kv,
                                int head_dim, int page_size, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE(head_dim % 2 == 0, "rope_kv_write: head_dim %d must be even", head_dim);
  LLMK_REQUIRE((qkv != nullptr) != (partials != nullptr), "rope_kv_write: give qkv or partials");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> src{(const T*)qkv, partials, splits, split_stride};
    const bool vec = head_dim % 16 == 0 && src.vector_ok() && src_stride % 8 == 0 && q_out_stride % 8 == 0 &&
                     (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0 &&
                     (uintptr_t)cos_table % 16 == 0 && (uintptr_t)sin_table % 16 == 0;
    auto kern = vec ? rope_kv_write_kernel<T, true> : rope_kv_write_kernel<T, false>;
    // few tokens: spread a token's heads over several CTAs (the vector path strides over blockIdx.y)
    const int items = (n_heads + n_kv) * (head_dim / 16);
    const int ys = (vec && n_tokens < 64) ? (items + 63) / 64 : 1;
    launch_kernel(kern, dim3(n_tokens, ys), dim3(vec && ys > 1 ? 64 : 128), 0, stream, src, src_stride, (T*)q_out,
                  q_out_stride, cos_table, sin_table, head_dim / 2, positions, slot_map, (T*)k_pages, (T*)v_pages,
                  n_heads, n_kv, head_dim, page_size);
    LLMK_LAUNCH_CHECK("rope_kv_write");
  });
}
