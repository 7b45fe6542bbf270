// C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores with float32 accumulation.
//
// This is the matrix product of the true 32-bit path (no tensor-core mode of any
// kind) and the any-size product of the bfloat16 path (sizes the tcgen05 kernel
// refuses).  Every element of C accumulates k = 0..K-1 in the same order for any M,
// so a row's result does not depend on what else is in the batch.  The reference's
// float32 product (kernel/Gemm/Gemm_f32.h:18-141) reads past M and needs K % 16 == 0;
// this one guards every access and takes any M, N, K.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, THREADS = 256;

template <typename T, int VEC>
__device__ __forceinline__ void load_k(const T* __restrict__ row, int k, int K, bool row_ok, float (&v)[4]) {
  if (VEC == 4) {
    if (row_ok && k + 3 < K) {
      if (sizeof(T) == 4) {
        const float4 f = *reinterpret_cast<const float4*>(row + k);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
      } else {
        const uint2 u = *reinterpret_cast<const uint2*>(row + k);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
      }
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = (row_ok && k + i < K) ? to_f32(row[k + i]) : 0.f;
}

template <typename T, typename TC, int VEC>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, TC* __restrict__ C, int M, int N, int K,
                 long long lda, long long ldw, long long ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  const int ty = tid >> 4, tx = tid & 15;
  const bool a_ok = m0 + lrow < M, w_ok = n0 + lrow < N;
  const T* a_row = A + (size_t)(a_ok ? m0 + lrow : 0) * lda;
  const T* w_row = W + (size_t)(w_ok ? n0 + lrow : 0) * ldw;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    float av[4], wv[4];
    load_k<T, VEC>(a_row, k0 + lk, K, a_ok, av);
    load_k<T, VEC>(w_row, k0 + lk, K, w_ok, wv);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[lk + i][lrow] = av[i];
      Ws[lk + i][lrow] = wv[i];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * TM]);
      const float4 w4 = *reinterpret_cast<const float4*>(&Ws[kk][tx * TN]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w};
      const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
    }
  }
}

template <typename T, typename TC>
int launch(const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw,
           long long ldc, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) &&
                   ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
  if (vec)
    launch_kernel(gemm_simt_kernel<T, TC, 4>, grid, dim3(THREADS), 0, stream, (const T*)A, (const T*)W, (TC*)C, M, N, K, lda, ldw, ldc);
  else
    launch_kernel(gemm_simt_kernel<T, TC, 1>, grid, dim3(THREADS), 0, stream, (const T*)A, (const T*)W, (TC*)C, M, N, K, lda, ldw, ldc);
  LLMK_LAUNCH_CHECK("gemm_simt");
}

}  // namespace

// in_dtype: element kind of A and W; out_dtype: element kind of C (float32 or the same as in_dtype).
LLMK_API int llmk_gemm_simt(const void* A, const void* W, void* C, int M, int N, int K, long long lda,
                            long long ldw, long long ldc, int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  LLMK_REQUIRE(K > 0 && lda >= K && ldw >= K && ldc >= N, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
  LLMK_REQUIRE((M + BM - 1) / BM <= 65535, "gemm_simt: M=%d exceeds the grid limit", M);
  if (in_dtype == LLMK_F32 && out_dtype == LLMK_F32) return launch<float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
  if (in_dtype == LLMK_BF16 && out_dtype == LLMK_BF16)
    return launch<__nv_bfloat16, __nv_bfloat16>(A, W, C, M, N, K, lda, ldw, ldc, stream);
  if (in_dtype == LLMK_BF16 && out_dtype == LLMK_F32)
    return launch<__nv_bfloat16, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
  return llmk_fail(-1, "gemm_simt: unsupported element kinds in=%d out=%d", in_dtype, out_dtype);
}
