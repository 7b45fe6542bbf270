// Shared helpers of the hand-written kernels: element conversion, vector access,
// block reductions with a fixed order, and the error channel to the host.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#define LLMK_API extern "C" __attribute__((visibility("default")))

// Element kinds as the host passes them.
enum : int { LLMK_F32 = 0, LLMK_BF16 = 1 };

// Return codes: 0 ok, > 0 a cudaError_t, < 0 an argument that this kernel refuses
// (the text is kept for llmk_last_error()).
int llmk_fail(int code, const char* fmt, ...);

#define LLMK_REQUIRE(cond, ...)                          \
  do {                                                   \
    if (!(cond)) return llmk_fail(-1, __VA_ARGS__);      \
  } while (0)

#define LLMK_LAUNCH_CHECK(name)                                             \
  do {                                                                      \
    cudaError_t e__ = cudaPeekAtLastError();                                \
    if (e__ != cudaSuccess) {                                               \
      cudaGetLastError();                                                   \
      return llmk_fail((int)e__, "%s: %s", name, cudaGetErrorString(e__)); \
    }                                                                       \
    return 0;                                                               \
  } while (0)

template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

template <typename T> __device__ __forceinline__ float to_f32(T v) { return Elem<T>::to_f32(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v) { return Elem<T>::from_f32(v); }

// Sum over a warp, then over the warps of a block, in a fixed order: the result
// for a row never depends on which other rows the launch holds.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// All threads get the sum. `scratch` holds 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nwarps; ++w) t += scratch[w];
  return t;
}

// ---- programmatic dependent launch ---------------------------------------------------
// Kernels of a step are launched back to back on one stream.  With the attribute below the
// next kernel may be scheduled while the previous one still runs; it then does what does
// not depend on earlier kernels (barrier set-up, tensor-memory allocation, weight loads) and
// blocks in pdl_wait() until the previous kernel has completed and its writes are visible.
// Every kernel launched this way calls pdl_wait() before it touches data of other kernels.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool llmk_pdl_enabled();
int llmk_sm_count();                    // SMs of the current device (runtime.cu)
int* llmk_error_word(int which);      // the device word kernels of one kind report a given-up wait in (runtime.cu)

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = llmk_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Eight consecutive elements as float32 (two 16-byte loads of float32, one of bfloat16).
template <typename T> struct Vec8;
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __low2float(h[i]); v[2 * i + 1] = __high2float(h[i]); }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};

// A value that is either an element of a tensor of T or the sum, in the order s = 0, 1, ...,
// of `splits` float32 partial results laid out [split][row][col] (split-K products).
template <typename T>
struct MaybePartial {
  const T* direct;
  const float* parts;
  int splits;
  long long split_stride;
  __device__ __forceinline__ bool present() const { return direct != nullptr || parts != nullptr; }
  __device__ __forceinline__ float at(size_t idx) const {
    if (parts) {
      // loads of four splits are issued together; the additions keep the order of the splits
      float a = 0.f;
      int s = 0;
      for (; s + 4 <= splits; s += 4) {
        const float v0 = parts[(size_t)s * split_stride + idx], v1 = parts[(size_t)(s + 1) * split_stride + idx];
        const float v2 = parts[(size_t)(s + 2) * split_stride + idx], v3 = parts[(size_t)(s + 3) * split_stride + idx];
        a += v0; a += v1; a += v2; a += v3;
      }
      for (; s < splits; ++s) a += parts[(size_t)s * split_stride + idx];
      return a;
    }
    return to_f32(direct[idx]);
  }
  // eight consecutive values starting at idx (idx a multiple of 8, the bases 16-byte aligned)
  __device__ __forceinline__ void at8(size_t idx, float (&v)[8]) const {
    if (parts) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
      int s = 0;
      for (; s + 4 <= splits; s += 4) {              // the loads of four splits in flight, sums in split order
        float t[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) Vec8<float>::load(parts + (size_t)(s + u) * split_stride + idx, t[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] += t[u][i];
      }
      for (; s < splits; ++s) {
        float t[8];
        Vec8<float>::load(parts + (size_t)s * split_stride + idx, t);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += t[i];
      }
      return;
    }
    Vec8<T>::load(direct + idx, v);
  }
  __host__ bool vector_ok() const {
    return ((uintptr_t)direct % 16 == 0) && ((uintptr_t)parts % 16 == 0) && (split_stride % 4 == 0);
  }
};

#define LLMK_ELEM(tag) typename std::remove_pointer<decltype(tag)>::type

template <typename F>
inline int dispatch_dtype(int dtype, F&& f) {
  if (dtype == LLMK_F32) return f((float*)nullptr);
  if (dtype == LLMK_BF16) return f((__nv_bfloat16*)nullptr);
  return llmk_fail(-1, "unknown element kind %d (0 = float32, 1 = bfloat16)", dtype);
}
