// Attention of single decoded tokens over the paged cache, split along the keys.
//
// A decode step has one query token per request, so the work per (request, kv head) is
// one pass over that head's keys and values: bound by HBM, with too few (request, head)
// pairs to fill the GPU.  The keys of a request are therefore cut into `splits` ranges;
// CTA (split, kv head, request) scores its range for all query heads of the group at
// once (every key and value is read once for the whole group), keeps an unnormalised
// partial result with its maximum and sum, and a second kernel merges the ranges
// (log-sum-exp).  The grid depends on the batch size only, and the ranges are computed
// on the device from the request's length, so the launch can sit in a CUDA graph.
// The reference runs decode through its prefill kernel, one 16-row MMA tile per head with
// one row used and no split (kernel/attention/attention_NH_32_NKV_4_HS_64.h:374-386).
// Softmax and all sums are float32; visible keys are max(0, pos-window+1) .. pos.
#include "common.cuh"

namespace {

constexpr int THREADS = 128;
constexpr int GT = 8;            // query heads handled per pass over the keys
constexpr int SUB = 128;         // keys scored per round (one per thread)
constexpr int MAX_HS = 256;

template <typename T> struct Row;
template <> struct Row<float> {
  static constexpr int VEC = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
  }
  static __device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
};
template <> struct Row<__nv_bfloat16> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __low2float(h[i]); v[2 * i + 1] = __high2float(h[i]); }
  }
  static __device__ __forceinline__ float2 load2(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
};

// partial_o [entries, n_heads, splits, head_dim], partial_ml [entries, n_heads, splits, 2]
template <typename T>
__global__ void __launch_bounds__(THREADS)
decode_split_kernel(float* __restrict__ partial_o, float* __restrict__ partial_ml, const T* __restrict__ q,
                    long long q_stride, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                    const int* __restrict__ block_table, int table_width, const int* __restrict__ kv_lens,
                    int n_heads, int n_kv, int head_dim, int page_size, int window, float scale, int splits) {
  __shared__ __align__(16) float q_s[GT][MAX_HS];
  __shared__ __align__(16) float p_s[SUB][GT];
  __shared__ float red_s[THREADS / 32][GT];
  __shared__ float m_s[GT], l_s[GT], alpha_s[GT];
  __shared__ long long row_s[SUB];

  pdl_wait();
  pdl_launch_dependents();
  const int split = blockIdx.x, g = blockIdx.y, e = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = n_heads / n_kv;
  const int pos = kv_lens[e] - 1;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n_keys = pos - lo + 1;
  int chunk = (n_keys + splits - 1) / splits;
  chunk = (chunk + 31) / 32 * 32;
  const int k_begin = lo + split * chunk;
  const int k_end = min(pos + 1, k_begin + chunk);
  const int* table = block_table + (size_t)e * table_width;
  const int n_dp = head_dim / 2;                 // pairs of output dims
  const int n_kg = THREADS / n_dp;               // key groups in the value phase
  const int dp = tid % n_dp, kg = tid / n_dp;
  const bool pv_active = kg < n_kg;

  for (int h0 = 0; h0 < group; h0 += GT) {
    const int nh = min(GT, group - h0);
    const int head0 = g * group + h0;
    __syncthreads();
    for (int i = tid; i < GT * head_dim; i += THREADS) {
      const int h = i / head_dim, d = i % head_dim;
      q_s[h][d] = h < nh ? to_f32(q[(size_t)e * q_stride + (size_t)(head0 + h) * head_dim + d]) * scale : 0.f;
    }
    if (tid < GT) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
    float acc[GT][2];
#pragma unroll
    for (int h = 0; h < GT; ++h) acc[h][0] = acc[h][1] = 0.f;
    __syncthreads();

    for (int base = k_begin; base < k_end; base += SUB) {
      const int n_sub = min(SUB, k_end - base);
      // ---- scores: one key per thread, all heads of the pass ----
      float s[GT];
#pragma unroll
      for (int h = 0; h < GT; ++h) s[h] = -INFINITY;
      if (tid < n_sub) {
        const int kp = base + tid;
        const long long row = (((long long)table[kp / page_size] * n_kv + g) * page_size + kp % page_size) * head_dim;
        row_s[tid] = row;
#pragma unroll
        for (int h = 0; h < GT; ++h) s[h] = 0.f;
        const T* kr = k_pages + row;
        for (int d = 0; d < head_dim; d += Row<T>::VEC) {
          float kv[Row<T>::VEC];
          Row<T>::load(kr + d, kv);
#pragma unroll
          for (int h = 0; h < GT; ++h) {
#pragma unroll
            for (int i = 0; i < Row<T>::VEC; i += 4) {
              const float4 qv = *reinterpret_cast<const float4*>(&q_s[h][d + i]);
              s[h] = fmaf(kv[i], qv.x, s[h]);
              s[h] = fmaf(kv[i + 1], qv.y, s[h]);
              s[h] = fmaf(kv[i + 2], qv.z, s[h]);
              s[h] = fmaf(kv[i + 3], qv.w, s[h]);
            }
          }
        }
      }
      // ---- running maximum per head over the CTA ----
#pragma unroll
      for (int h = 0; h < GT; ++h) {
        const float wm = warp_max(s[h]);
        if (lane == 0) red_s[warp][h] = wm;
      }
      __syncthreads();
      if (tid < GT) {
        float m_new = m_s[tid];
        for (int w = 0; w < THREADS / 32; ++w) m_new = fmaxf(m_new, red_s[w][tid]);
        alpha_s[tid] = expf(m_s[tid] - m_new);      // 0 at the first round (m = -inf)
        m_s[tid] = m_new;
      }
      __syncthreads();
      float psum[GT];
#pragma unroll
      for (int h = 0; h < GT; ++h) {
        const float p = tid < n_sub ? expf(s[h] - m_s[h]) : 0.f;
        if (tid < n_sub) p_s[tid][h] = p;
        psum[h] = warp_sum(p);
      }
      __syncthreads();                               // p_s, row_s complete; red_s free again
#pragma unroll
      for (int h = 0; h < GT; ++h)
        if (lane == 0) red_s[warp][h] = psum[h];
      // ---- values: thread = (pair of dims, key group) ----
      if (pv_active) {
#pragma unroll
        for (int h = 0; h < GT; ++h) { acc[h][0] *= alpha_s[h]; acc[h][1] *= alpha_s[h]; }
        for (int j = kg; j < n_sub; j += n_kg) {
          const float2 vv = Row<T>::load2(v_pages + row_s[j] + 2 * dp);
          const float4 pa = *reinterpret_cast<const float4*>(&p_s[j][0]);
          const float4 pb = *reinterpret_cast<const float4*>(&p_s[j][4]);
          const float pj[GT] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
          for (int h = 0; h < GT; ++h) {
            acc[h][0] = fmaf(pj[h], vv.x, acc[h][0]);
            acc[h][1] = fmaf(pj[h], vv.y, acc[h][1]);
          }
        }
      }
      __syncthreads();
      if (tid < GT) {
        float t = 0.f;
        for (int w = 0; w < THREADS / 32; ++w) t += red_s[w][tid];
        l_s[tid] = l_s[tid] * alpha_s[tid] + t;
      }
      __syncthreads();
    }

    // ---- sum the key groups and write the partial result ----
    float* out_s = &q_s[0][0];                       // reuse: [GT][head_dim]
    for (int r = 0; r < n_kg; ++r) {
      __syncthreads();
      if (pv_active && kg == r) {
#pragma unroll
        for (int h = 0; h < GT; ++h) {
          float* o = out_s + h * head_dim + 2 * dp;
          if (r == 0) { o[0] = acc[h][0]; o[1] = acc[h][1]; }
          else { o[0] += acc[h][0]; o[1] += acc[h][1]; }
        }
      }
    }
    __syncthreads();
    for (int i = tid; i < nh * head_dim; i += THREADS) {
      const int h = i / head_dim, d = i % head_dim;
      partial_o[(((size_t)e * n_heads + head0 + h) * splits + split) * head_dim + d] = out_s[h * head_dim + d];
    }
    if (tid < nh) {
      float* ml = partial_ml + (((size_t)e * n_heads + head0 + tid) * splits + split) * 2;
      ml[0] = m_s[tid];
      ml[1] = l_s[tid];
    }
  }
}

// out[e, h, :] = sum_s w_s o_s / sum_s w_s l_s with w_s = exp(m_s - max m); splits in order.
template <typename T>
__global__ void decode_combine_kernel(T* __restrict__ out, long long out_stride, const float* __restrict__ partial_o,
                                      const float* __restrict__ partial_ml, int n_heads, int head_dim, int splits) {
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, e = blockIdx.y;
  const size_t base = ((size_t)e * n_heads + h) * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, partial_ml[(base + s) * 2]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = partial_ml[(base + s) * 2];
    if (ms > -INFINITY) l += expf(ms - m) * partial_ml[(base + s) * 2 + 1];
  }
  const float inv = 1.f / l;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = partial_ml[(base + s) * 2];
      if (ms > -INFINITY) acc += expf(ms - m) * partial_o[(base + s) * head_dim + d];
    }
    out[(size_t)e * out_stride + (size_t)h * head_dim + d] = from_f32<T>(acc * inv);
  }
}

}  // namespace

// One query token per batch entry: q [entries, q_stride] (head h at column h*head_dim),
// kv_lens[e] = keys of entry e including the new token.  partial_o needs
// entries*n_heads*splits*head_dim floats, partial_ml entries*n_heads*splits*2.
LLMK_API int llmk_paged_attention_decode(void* out, long long out_stride, const void* q, long long q_stride,
                                         const void* k_pages, const void* v_pages, const int* block_table,
                                         int table_width, const int* kv_lens, int n_entries, int n_heads, int n_kv,
                                         int head_dim, int page_size, int window, float scale, int splits,
                                         float* partial_o, float* partial_ml, int dtype, cudaStream_t stream) {
  if (n_entries == 0) return 0;
  LLMK_REQUIRE(head_dim > 0 && head_dim % 16 == 0 && head_dim <= MAX_HS,
               "attention_decode: head_dim %d must be a multiple of 16 up to %d", head_dim, MAX_HS);
  LLMK_REQUIRE(n_kv > 0 && n_heads % n_kv == 0, "attention_decode: %d query heads do not divide into %d kv heads", n_heads, n_kv);
  LLMK_REQUIRE(splits >= 1 && splits <= 65535 && n_kv <= 65535 && n_entries <= 65535, "attention_decode: grid too large");
  LLMK_REQUIRE(page_size > 0 && window >= 0, "attention_decode: bad page_size %d or window %d", page_size, window);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    dim3 grid(splits, n_kv, n_entries);
    launch_kernel(decode_split_kernel<T>, grid, dim3(THREADS), 0, stream, partial_o, partial_ml, (const T*)q, q_stride, (const T*)k_pages,
                                                        (const T*)v_pages, block_table, table_width, kv_lens, n_heads,
                                                        n_kv, head_dim, page_size, window, scale, splits);
    cudaError_t e1 = cudaPeekAtLastError();
    if (e1 != cudaSuccess) { cudaGetLastError(); return llmk_fail((int)e1, "attention_decode: %s", cudaGetErrorString(e1)); }
    dim3 grid2(n_heads, n_entries);
    launch_kernel(decode_combine_kernel<T>, grid2, dim3(64), 0, stream, (T*)out, out_stride, partial_o, partial_ml, n_heads, head_dim, splits);
    LLMK_LAUNCH_CHECK("attention_decode_combine");
  });
}

// ---- the variant that allocates nothing (declared in no_alloc.h) ----------------
#include "no_alloc.h"

namespace {

// The key ranges' partial results for the static variant.  In host code this name is only
// a stand-in for the symbol: the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_decode_static_scratch[LLMK_DECODE_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_decode_static_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device, looked up once per device.
int decode_static_scratch(float** ptr) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return llmk_fail((int)e, "attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return llmk_fail(-1, "attention_decode_static: device %d out of range", dev);
  if (!g_decode_static_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_decode_static_scratch);
    if (e != cudaSuccess || !p)
      return llmk_fail(e != cudaSuccess ? (int)e : -2, "attention_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_decode_static_ptr[dev] = p;
  }
  *ptr = g_decode_static_ptr[dev];
  return 0;
}

}  // namespace

LLMK_API int llmk_paged_attention_decode_static(void* out, long long out_stride, const void* q, long long q_stride,
                                                const void* k_pages, const void* v_pages, const int* block_table,
                                                int table_width, const int* kv_lens, int n_entries, int n_heads,
                                                int n_kv, int head_dim, int page_size, int window, float scale,
                                                int splits, int dtype, cudaStream_t stream) {
  if (n_entries == 0) return 0;
  LLMK_REQUIRE(n_entries > 0 && n_heads > 0 && splits >= 1 && head_dim > 0, "attention_decode_static: bad sizes");
  const long long n_o = (long long)n_entries * n_heads * splits * head_dim;
  const long long n_ml = (long long)n_entries * n_heads * splits * 2;
  LLMK_REQUIRE(n_o + n_ml <= (long long)LLMK_DECODE_STATIC_SCRATCH_FLOATS,
               "attention_decode_static: %d entries x %d heads x %d splits x (%d + 2) = %lld floats of scratch exceed "
               "the built-in %d", n_entries, n_heads, splits, head_dim, n_o + n_ml, (int)LLMK_DECODE_STATIC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  const int rc = decode_static_scratch(&scratch);
  if (rc) return rc;
  return llmk_paged_attention_decode(out, out_stride, q, q_stride, k_pages, v_pages, block_table, table_width, kv_lens,
                                     n_entries, n_heads, n_kv, head_dim, page_size, window, scale, splits, scratch,
                                     scratch + n_o, dtype, stream);
}
