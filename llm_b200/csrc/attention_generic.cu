// Causal grouped-query attention over the paged cache, any sizes, float32 arithmetic.
//
// One warp owns one (token, query head).  Keys are visited in tiles of 32 that start
// at absolute positions 0, 32, 64, ...: lane j scores key tile+j, the warp keeps a
// running maximum and sum (online softmax), then all lanes add p_j * v_j in key order.
// The order of every sum is a function of the token's own position alone, so a
// token's output does not depend on how the prompt was cut or what shares the batch.
// Visible keys: max(0, pos-window+1) <= j <= pos (window 0 = all), as in the reference
// (kernel/attention/attention_NH_32_NKV_4_HS_64.h:169-172,228-232); scores are scaled
// by the given factor instead of the reference's constant for head size 64 (:197).
// This is the attention of the 32-bit path and of bfloat16 shapes that the tensor-core
// kernels refuse.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HEAD_DIM = 256;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int head_dim);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k,
                                                int head_dim) {
  float s = 0.f;
  for (int d = 0; d < head_dim; d += 4) {
    const float4 kv = *reinterpret_cast<const float4*>(k + d);
    s = fmaf(q[d], kv.x, s);
    s = fmaf(q[d + 1], kv.y, s);
    s = fmaf(q[d + 2], kv.z, s);
    s = fmaf(q[d + 3], kv.w, s);
  }
  return s;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q,
                                                        const __nv_bfloat16* __restrict__ k, int head_dim) {
  float s = 0.f;
  for (int d = 0; d < head_dim; d += 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(k + d);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s = fmaf(q[d + 2 * i], __low2float(p[i]), s);
      s = fmaf(q[d + 2 * i + 1], __high2float(p[i]), s);
    }
  }
  return s;
}

// a row that does not start on a 16-byte boundary, or is no whole number of 16-byte pieces
// (head sizes off the 8-grid in bfloat16, off the 4-grid in float32): element by element
template <typename T>
__device__ __forceinline__ float dot_row_scalar(const float* __restrict__ q, const T* __restrict__ k, int head_dim) {
  float s = 0.f;
  for (int d = 0; d < head_dim; ++d) s = fmaf(q[d], to_f32(k[d]), s);
  return s;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_generic_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ q,
                               long long q_stride, const T* __restrict__ k_pages,
                               const T* __restrict__ v_pages, const int* __restrict__ block_table,
                               int table_width, const int* __restrict__ token_entry,
                               const int* __restrict__ positions, int n_tokens, int n_heads, int n_kv,
                               int head_dim, int page_size, int window, float scale, bool vec) {
  __shared__ float q_s[WARPS][MAX_HEAD_DIM];
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)n_tokens * n_heads) return;
  const int t = (int)(item / n_heads), h = (int)(item % n_heads);
  const int g = h / (n_heads / n_kv);
  const int pos = positions[t];
  const int* table = block_table + (size_t)token_entry[t] * table_width;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  const T* q_row = q + (size_t)t * q_stride + (size_t)h * head_dim;
  for (int d = lane; d < head_dim; d += 32) q_s[warp][d] = to_f32(q_row[d]);
  __syncwarp();

  float acc[MAX_HEAD_DIM / 32];
#pragma unroll
  for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int tile = (lo / 32) * 32; tile <= pos; tile += 32) {
    const int kp = tile + lane;
    const bool valid = kp >= lo && kp <= pos;
    long long row = 0;
    float s = -INFINITY;
    if (valid) {
      const int page = table[kp / page_size];
      row = (((long long)page * n_kv + g) * page_size + kp % page_size) * head_dim;
      s = (vec ? dot_row<T>(q_s[warp], k_pages + row, head_dim) : dot_row_scalar<T>(q_s[warp], k_pages + row, head_dim)) * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = expf(m - m_new);  // m = -inf at the first tile gives 0
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) acc[i] *= alpha;
    const int n_valid = min(32, pos - tile + 1);
    for (int j = 0; j < n_valid; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long rj = __shfl_sync(0xffffffffu, row, j);
      if (pj != 0.f) {
        const T* v = v_pages + rj;
#pragma unroll
        for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < head_dim) acc[i] = fmaf(pj, to_f32(v[d]), acc[i]);
        }
      }
    }
  }
  const float inv = 1.f / l;
  T* o = out + (size_t)t * out_stride + (size_t)h * head_dim;
#pragma unroll
  for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < head_dim) o[d] = from_f32<T>(acc[i] * inv);
  }
}

}  // namespace

// q [n_tokens, q_stride] with head h at column h*head_dim; out [n_tokens, out_stride] likewise.
// k_pages / v_pages [pages, n_kv, page_size, head_dim]; block_table [entries, table_width] holds,
// for batch entry e, the page of positions [i*page_size, (i+1)*page_size) at column i.
LLMK_API int llmk_paged_attention_generic(void* out, long long out_stride, const void* q, long long q_stride,
                                          const void* k_pages, const void* v_pages, const int* block_table,
                                          int table_width, const int* token_entry, const int* positions,
                                          int n_tokens, int n_heads, int n_kv, int head_dim, int page_size,
                                          int window, float scale, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE(head_dim > 0 && head_dim <= MAX_HEAD_DIM, "paged_attention: head_dim %d must be 1 to %d", head_dim, MAX_HEAD_DIM);
  LLMK_REQUIRE(n_kv > 0 && n_heads % n_kv == 0, "paged_attention: %d query heads do not divide into %d kv heads",
               n_heads, n_kv);
  LLMK_REQUIRE(page_size > 0 && window >= 0, "paged_attention: bad page_size %d or window %d", page_size, window);
  const long long items = (long long)n_tokens * n_heads;
  const long long blocks = (items + WARPS - 1) / WARPS;
  LLMK_REQUIRE(blocks < (1ll << 31), "paged_attention: too many (token, head) items");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    const bool vec = head_dim % (16 / (int)sizeof(T)) == 0 && (uintptr_t)k_pages % 16 == 0;      // whole 16-byte pieces per key row
    launch_kernel(paged_attention_generic_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream,
        (T*)out, out_stride, (const T*)q, q_stride, (const T*)k_pages, (const T*)v_pages, block_table,
        table_width, token_entry, positions, n_tokens, n_heads, n_kv, head_dim, page_size, window, scale, vec);
    LLMK_LAUNCH_CHECK("paged_attention_generic");
  });
}
