// Attention of single decoded tokens over the paged cache, split along the keys.
//
// A decode step has one query token per request, so the work per (request, kv head) is
// one pass over that head's keys and values: bound by HBM and by latency, with too few
// (request, head) pairs to fill the GPU.  The keys of a request are therefore cut into
// `splits` ranges; CTA (split, kv head, request) scores its range for all query heads of
// the group at once (every key and value is read once for the whole group) and keeps an
// unnormalised partial result with its maximum and sum.  The CTA that finishes last for a
// (request, kv head) merges the ranges (log-sum-exp, always in the order of the ranges, so
// the result does not depend on which CTA that was) and writes the output.  The grid
// depends on the batch size only and the ranges are computed on the device from the
// request's length, so the launch can sit in a CUDA graph.
// The reference runs decode through its prefill kernel, one 16-row MMA tile per head with
// one row used and no split (kernel/attention/attention_NH_32_NKV_4_HS_64.h:374-386).
// Softmax and all sums are float32; visible keys are max(0, pos-window+1) .. pos.
#include "common.cuh"

namespace {

constexpr int THREADS = 128;
constexpr int GT = 8;            // query heads handled per pass over the keys
constexpr int KT = 4;            // threads that share one key's dot products
constexpr int SUB = THREADS / KT;  // keys scored per round
constexpr int MAX_HS = 256;
constexpr int COUNTER_WORDS = 4096;   // arrival counters at the start of the scratch

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

// Scratch layout (float words): [0, COUNTER_WORDS) arrival counters, one per (entry, kv head),
// zero between launches; then ml [entries, n_heads, splits, 2]; then o [entries, n_heads, splits, head_dim].
//
// HS > 0 fixes the head size at compile time: loops unroll, a key's row is requested in one go
// and the values of a round are staged in shared memory by the threads that own the keys
// (their loads are in flight while the scores are computed).  HS == 0 takes any head size.
// Few keys per round and four threads per key keep the instruction chain of a warp short:
// with so little data per request the kernel is bound by latency, not by bandwidth.
template <typename T, int HS>
__global__ void __launch_bounds__(THREADS)
decode_attention_kernel(T* __restrict__ out, long long out_stride, float* __restrict__ scratch,
                        const T* __restrict__ q, long long q_stride, const T* __restrict__ k_pages,
                        const T* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
                        const int* __restrict__ kv_lens, int n_heads, int n_kv, int head_dim_arg, int page_size,
                        int window, float scale, int splits) {
  constexpr bool STAGE_V = HS > 0;
  constexpr int QW = HS > 0 ? HS : MAX_HS;
  constexpr int V_PITCH = HS + 16 / (int)sizeof(T);                 // elements; rows stay 16-byte aligned
  static_assert(HS == 0 || (HS / KT) % Row<T>::VEC == 0, "a thread's share of a row must be whole vectors");
  constexpr int V_WORDS = STAGE_V ? SUB * V_PITCH * (int)sizeof(T) / 4 : 1;
  constexpr int O_WORDS = GT * QW * (STAGE_V ? THREADS / (HS / 2) : 1);
  constexpr int VO_WORDS = V_WORDS > O_WORDS ? V_WORDS : O_WORDS;
  const int head_dim = HS > 0 ? HS : head_dim_arg;

  __shared__ __align__(16) float q_s[GT][QW];
  __shared__ __align__(16) float p_s[SUB][GT];
  __shared__ __align__(16) float vo_s[VO_WORDS];                     // staged values, later the key groups' sums
  __shared__ float red_s[THREADS / 32][GT];
  __shared__ float m_s[GT], l_s[GT], alpha_s[GT];
  __shared__ long long row_s[SUB];
  __shared__ int last_s;

  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const int split = blockIdx.x, g = blockIdx.y, e = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = n_heads / n_kv;
  // a length beyond the entry's table row is cut to what the row can hold; an entry without keys
  // gets zeros (every range of it sees the same length and leaves here, so nobody waits for anybody)
  const int n_held = min(kv_lens[e], table_width * page_size);
  if (n_held <= 0) {
    if (split == 0)
      for (int i = tid; i < group * (HS > 0 ? HS : head_dim_arg); i += THREADS)
        out[(size_t)e * out_stride + (size_t)g * group * (HS > 0 ? HS : head_dim_arg) + i] = from_f32<T>(0.f);
    return;
  }
  const int pos = n_held - 1;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n_keys = pos - lo + 1;
  int chunk = (n_keys + splits - 1) / splits;
  chunk = (chunk + SUB - 1) / SUB * SUB;        // whole rounds
  const int k_begin = lo + split * chunk;
  const int k_end = min(pos + 1, k_begin + chunk);
  const int* table = block_table + (size_t)e * table_width;
  const int n_dp = head_dim / 2;                 // pairs of output dims
  const int n_kg = THREADS / n_dp;               // key groups in the value phase
  const int dp = tid % n_dp, kg = tid / n_dp;
  const bool pv_active = kg < n_kg;
  T* v_s = reinterpret_cast<T*>(vo_s);

  int* counters = reinterpret_cast<int*>(scratch);
  float* partial_ml = scratch + COUNTER_WORDS;
  float* partial_o = partial_ml + (size_t)gridDim.z * n_heads * splits * 2;

  for (int h0 = 0; h0 < group && k_begin < k_end; h0 += GT) {         // a range without keys only reports in
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
      // ---- scores: KT threads per key, each a quarter of the head's dims, all heads of the pass ----
      float s[GT];
#pragma unroll
      for (int h = 0; h < GT; ++h) s[h] = 0.f;
      constexpr int VEC = Row<T>::VEC;
      const int key = tid / KT, part = tid % KT;
      const bool has_key = key < n_sub;
      if (has_key) {
        const int kp = base + key;
        const long long row = (((long long)table[kp / page_size] * n_kv + g) * page_size + kp % page_size) * head_dim;
        if (part == 0) row_s[key] = row;
        if (STAGE_V) {
          constexpr int PART = (HS > 0 ? HS : KT * VEC) / KT;        // dims of this thread
          constexpr int NV = PART / VEC;
          uint4 v_raw[NV];
          float kv[NV][VEC];
          const T* kr = k_pages + row + part * PART;
#pragma unroll
          for (int c = 0; c < NV; ++c) {
            v_raw[c] = *reinterpret_cast<const uint4*>(v_pages + row + part * PART + c * VEC);
            Row<T>::load(kr + c * VEC, kv[c]);
          }
#pragma unroll
          for (int c = 0; c < NV; ++c) {
#pragma unroll
            for (int h = 0; h < GT; ++h) {
#pragma unroll
              for (int i = 0; i < VEC; i += 4) {
                const float4 qv = *reinterpret_cast<const float4*>(&q_s[h][part * PART + c * VEC + i]);
                s[h] = fmaf(kv[c][i], qv.x, s[h]);
                s[h] = fmaf(kv[c][i + 1], qv.y, s[h]);
                s[h] = fmaf(kv[c][i + 2], qv.z, s[h]);
                s[h] = fmaf(kv[c][i + 3], qv.w, s[h]);
              }
            }
          }
#pragma unroll
          for (int c = 0; c < NV; ++c)
            *reinterpret_cast<uint4*>(v_s + (size_t)key * V_PITCH + part * PART + c * VEC) = v_raw[c];
        } else {
          const int part_dims = head_dim / KT;                      // head_dim is a multiple of 16
          const T* kr = k_pages + row + part * part_dims;
          for (int d = 0; d < part_dims; d += 4) {
            const float k0 = to_f32(kr[d]), k1 = to_f32(kr[d + 1]), k2 = to_f32(kr[d + 2]), k3 = to_f32(kr[d + 3]);
#pragma unroll
            for (int h = 0; h < GT; ++h) {
              const float4 qv = *reinterpret_cast<const float4*>(&q_s[h][part * part_dims + d]);
              s[h] = fmaf(k0, qv.x, s[h]);
              s[h] = fmaf(k1, qv.y, s[h]);
              s[h] = fmaf(k2, qv.z, s[h]);
              s[h] = fmaf(k3, qv.w, s[h]);
            }
          }
        }
      }
#pragma unroll
      for (int h = 0; h < GT; ++h) {                 // the KT threads of a key are neighbouring lanes
        s[h] += __shfl_xor_sync(0xffffffffu, s[h], 1);
        s[h] += __shfl_xor_sync(0xffffffffu, s[h], 2);
        if (!has_key) s[h] = -INFINITY;
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
        const float p = (has_key && part == 0) ? expf(s[h] - m_s[h]) : 0.f;     // one lane per key counts
        if (has_key && part == 0) p_s[key][h] = p;
        psum[h] = warp_sum(p);
      }
      __syncthreads();                               // p_s, row_s, v_s complete; red_s free again
#pragma unroll
      for (int h = 0; h < GT; ++h)
        if (lane == 0) red_s[warp][h] = psum[h];
      // ---- values: thread = (pair of dims, key group) ----
      if (pv_active) {
#pragma unroll
        for (int h = 0; h < GT; ++h) { acc[h][0] *= alpha_s[h]; acc[h][1] *= alpha_s[h]; }
        constexpr int UN = 8;                      // values requested before any is used
        for (int j0 = kg; j0 < n_sub; j0 += UN * n_kg) {
          float2 vv[UN];
#pragma unroll
          for (int u = 0; u < UN; ++u) {
            const int j = j0 + u * n_kg;
            if (j < n_sub)
              vv[u] = STAGE_V ? Row<T>::load2(v_s + (size_t)j * V_PITCH + 2 * dp) : Row<T>::load2(v_pages + row_s[j] + 2 * dp);
            else
              vv[u] = make_float2(0.f, 0.f);
          }
#pragma unroll
          for (int u = 0; u < UN; ++u) {
            const int j = j0 + u * n_kg;
            if (j < n_sub) {
              const float4 pa = *reinterpret_cast<const float4*>(&p_s[j][0]);
              const float4 pb = *reinterpret_cast<const float4*>(&p_s[j][4]);
              const float pj[GT] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
              for (int h = 0; h < GT; ++h) {
                acc[h][0] = fmaf(pj[h], vv[u].x, acc[h][0]);
                acc[h][1] = fmaf(pj[h], vv[u].y, acc[h][1]);
              }
            }
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

    // ---- sum the key groups (in their order) and write this range's result ----
    float* o_sum = &q_s[0][0];                       // [GT][head_dim]; q is not needed any more
    if (STAGE_V) {
      float* grp = vo_s;                             // [n_kg][GT][head_dim]
      if (pv_active) {
#pragma unroll
        for (int h = 0; h < GT; ++h) {
          grp[((size_t)kg * GT + h) * head_dim + 2 * dp] = acc[h][0];
          grp[((size_t)kg * GT + h) * head_dim + 2 * dp + 1] = acc[h][1];
        }
      }
      __syncthreads();
      for (int i = tid; i < GT * head_dim; i += THREADS) {
        float t = 0.f;
        for (int r = 0; r < n_kg; ++r) t += grp[(size_t)r * GT * head_dim + i];
        o_sum[i] = t;
      }
    } else {
      for (int r = 0; r < n_kg; ++r) {
        __syncthreads();
        if (pv_active && kg == r) {
#pragma unroll
          for (int h = 0; h < GT; ++h) {
            float* o = o_sum + h * head_dim + 2 * dp;
            if (r == 0) { o[0] = acc[h][0]; o[1] = acc[h][1]; }
            else { o[0] += acc[h][0]; o[1] += acc[h][1]; }
          }
        }
      }
    }
    __syncthreads();
    if (splits == 1) {
      for (int i = tid; i < nh * head_dim; i += THREADS) {
        const int h = i / head_dim, d = i % head_dim;
        out[(size_t)e * out_stride + (size_t)(head0 + h) * head_dim + d] = from_f32<T>(o_sum[i] / l_s[h]);
      }
    } else {
      for (int i = tid; i < nh * head_dim; i += THREADS) {
        const int h = i / head_dim, d = i % head_dim;
        partial_o[(((size_t)e * n_heads + head0 + h) * splits + split) * head_dim + d] = o_sum[i];
      }
      if (tid < nh) {
        float* ml = partial_ml + (((size_t)e * n_heads + head0 + tid) * splits + split) * 2;
        ml[0] = m_s[tid];
        ml[1] = l_s[tid];
      }
    }
  }
  if (splits == 1) return;

  // ---- the last range to arrive merges all of them ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int arrived = atomicAdd(&counters[e * n_kv + g], 1);
    last_s = arrived == splits - 1;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  const int n_active = min(splits, (n_keys + chunk - 1) / chunk);      // ranges that hold keys
  float* w_s = &q_s[0][0];                                             // [GT][splits] maxima, then merge weights
  float* l_in = reinterpret_cast<float*>(vo_s);                        // [GT][splits] sums of the ranges
  for (int h0 = 0; h0 < group; h0 += GT) {
    const int nh = min(GT, group - h0);
    const size_t base0 = ((size_t)e * n_heads + g * group + h0) * splits;
    __syncthreads();
    for (int i = tid; i < nh * n_active; i += THREADS) {                // maximum and sum of every (head, range): one round trip
      const int h = i / n_active, sp = i % n_active;
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(partial_ml + (base0 + (size_t)h * splits + sp) * 2));
      w_s[h * splits + sp] = ml.x;
      l_in[h * splits + sp] = ml.y;
    }
    __syncthreads();
    if (tid < nh) {                                                     // weights exp(m_s - m) / l, from shared memory only
      float m = -INFINITY;
      for (int sp = 0; sp < n_active; ++sp) m = fmaxf(m, w_s[tid * splits + sp]);
      float l = 0.f;
      for (int sp = 0; sp < n_active; ++sp) {
        const float wgt = expf(w_s[tid * splits + sp] - m);
        l += wgt * l_in[tid * splits + sp];
        w_s[tid * splits + sp] = wgt;
      }
      const float inv = 1.f / l;
      for (int sp = 0; sp < n_active; ++sp) w_s[tid * splits + sp] *= inv;
    }
    __syncthreads();
    for (int i = tid; i < nh * head_dim; i += THREADS) {
      const int h = i / head_dim, d = i % head_dim;
      const float* o = partial_o + (base0 + (size_t)h * splits) * head_dim + d;
      float accum = 0.f;
      int sp = 0;
      for (; sp + 8 <= n_active; sp += 8) {                             // eight loads in flight, fixed order of sums
        float ov[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) ov[u] = __ldcg(o + (size_t)(sp + u) * head_dim);
#pragma unroll
        for (int u = 0; u < 8; ++u) accum = fmaf(w_s[h * splits + sp + u], ov[u], accum);
      }
      for (; sp < n_active; ++sp) accum = fmaf(w_s[h * splits + sp], __ldcg(o + (size_t)sp * head_dim), accum);
      out[(size_t)e * out_stride + (size_t)(g * group + h0 + h) * head_dim + d] = from_f32<T>(accum);
    }
  }
  if (tid == 0) counters[e * n_kv + g] = 0;        // ready for the next launch
}

}  // namespace

// Floats of scratch that a call needs.
LLMK_API long long llmk_paged_attention_decode_scratch(int n_entries, int n_heads, int head_dim, int splits) {
  return COUNTER_WORDS + (long long)n_entries * n_heads * splits * (head_dim + 2);
}


// One query token per batch entry: q [entries, q_stride] (head h at column h*head_dim),
// kv_lens[e] = keys of entry e including the new token.  `scratch` holds
// llmk_paged_attention_decode_scratch(...) floats; its first 4096 words are arrival counters
// that must be zero when the kernel starts and are zero again when it ends.
LLMK_API int llmk_paged_attention_decode(void* out, long long out_stride, const void* q, long long q_stride,
                                         const void* k_pages, const void* v_pages, const int* block_table,
                                         int table_width, const int* kv_lens, int n_entries, int n_heads, int n_kv,
                                         int head_dim, int page_size, int window, float scale, int splits,
                                         float* scratch, int dtype, cudaStream_t stream) {
  if (n_entries == 0) return 0;
  LLMK_REQUIRE(head_dim > 0 && head_dim % 16 == 0 && head_dim <= MAX_HS,
               "attention_decode: head_dim %d must be a multiple of 16 up to %d", head_dim, MAX_HS);
  LLMK_REQUIRE(n_kv > 0 && n_heads % n_kv == 0, "attention_decode: %d query heads do not divide into %d kv heads", n_heads, n_kv);
  LLMK_REQUIRE(splits >= 1 && splits <= 64, "attention_decode: splits %d must be 1 to 64", splits);
  LLMK_REQUIRE(n_kv <= 65535 && n_entries <= 65535, "attention_decode: grid too large");
  LLMK_REQUIRE((long long)n_entries * n_kv <= COUNTER_WORDS, "attention_decode: %d entries x %d kv heads exceed %d counters",
               n_entries, n_kv, COUNTER_WORDS);
  LLMK_REQUIRE(page_size > 0 && window >= 0, "attention_decode: bad page_size %d or window %d", page_size, window);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    dim3 grid(splits, n_kv, n_entries);
    auto kern = decode_attention_kernel<T, 0>;
    if (head_dim == 64) kern = decode_attention_kernel<T, 64>;
    if (head_dim == 128) kern = decode_attention_kernel<T, 128>;
    launch_kernel(kern, grid, dim3(THREADS), 0, stream, (T*)out, out_stride, scratch, (const T*)q, q_stride,
                  (const T*)k_pages, (const T*)v_pages, block_table, table_width, kv_lens, n_heads, n_kv, head_dim,
                  page_size, window, scale, splits);
    LLMK_LAUNCH_CHECK("attention_decode");
  });
}

// ---- the variant that allocates nothing (declared in no_alloc.h) ----------------
#include "no_alloc.h"

namespace {

// The key ranges' partial results (and, in the first 4096 words, their arrival counters) for
// the static variant.  The array starts zeroed and every launch leaves the counters zero.  In
// host code this name is only a stand-in for the symbol: the device address comes from
// cudaGetSymbolAddress below.
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
  const long long need = llmk_paged_attention_decode_scratch(n_entries, n_heads, head_dim, splits);
  LLMK_REQUIRE(need <= (long long)LLMK_DECODE_STATIC_SCRATCH_FLOATS,
               "attention_decode_static: 4096 + %d entries x %d heads x %d splits x (%d + 2) = %lld floats of scratch "
               "exceed the built-in %d", n_entries, n_heads, splits, head_dim, need, (int)LLMK_DECODE_STATIC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  const int rc = decode_static_scratch(&scratch);
  if (rc) return rc;
  return llmk_paged_attention_decode(out, out_stride, q, q_stride, k_pages, v_pages, block_table, table_width, kv_lens,
                                     n_entries, n_heads, n_kv, head_dim, page_size, window, scale, splits, scratch,
                                     dtype, stream);
}
