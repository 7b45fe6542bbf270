// C[M,N] = A[M,K] * W[N,K]^T in bfloat16 on the tcgen05 tensor cores, float32
// accumulation in tensor memory.
//
// Both operands are K-major, as activations and checkpoint weights ([out, in]) already
// are, so nothing is transposed.  One CTA computes one tile (or, in the persistent variants for
// many rows further down, one CTA or a pair of CTAs walks over tiles): a producer thread moves
// [rows x 64] boxes of both operands into a ring of 128-byte-swizzled stages with TMA,
// one thread issues tcgen05.mma (M = 128, N = BNQ, K = 16, four per stage) and frees each
// stage with tcgen05.commit, four warps read the accumulator back with tcgen05.ld and
// store it.  The operand that supplies the 128 rows of the MMA's M side is called P, the
// other Q:
//   normal:  P = activations, Q = weights  (many tokens)
//   swapped: P = weights, Q = activations  (few tokens: decode and short prompt portions;
//            the token count becomes the MMA's N, 16 to 128, so no tensor-core row is
//            spent on padding tokens up to 128)
// Few-token products read every weight once and are bound by HBM; to keep all SMs
// streaming, K is split over blockIdx.z and each split writes a float32 partial result
// [split][M][N] that the consumer (or llmk_reduce_partials) sums in a fixed order.
//
// The reference's products are mma.sync kernels with cp.async double buffering
// (kernel/Gemm/Gemm.h:143-247) and a special-case GEMV (kernel/Gemm/Gemm.h:249-280).
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

namespace tc {

// ---- tensor maps (host) -------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int encode_tensor_map_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                           uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return llmk_fail(-2, "cuTensorMapEncodeTiled is not available from the driver");
  if ((uintptr_t)base % 16 != 0 || (ld * 2) % 16 != 0)
    return llmk_fail(-1, "tensor map: base and row pitch must be multiples of 16 bytes");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return llmk_fail(-2, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

}  // namespace tc

namespace {

using namespace tc;

constexpr int BP = 128;            // rows of P per tile = M of the MMA
constexpr int BK = 64;             // elements of K per stage = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;       // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
constexpr int P_STAGE_BYTES = BP * BK * 2;

__host__ __device__ constexpr int q_stage_bytes(int bnq) { return bnq * BK * 2; }
// Stages of the ring.  In the swapped mode (few rows, bound by the weights' way from memory) two
// CTAs share an SM, so that twice as many CTAs stream weights at a time: their rings are sized to
// about 100 KB each.  In the normal mode one CTA has the SM.
__host__ __device__ constexpr int stages_for(int bnq, bool swap = false) {
  return bnq >= 256 ? 4 : !swap ? 6 : bnq <= 16 ? 6 : bnq <= 32 ? 5 : bnq <= 64 ? 4 : 3;
}
__host__ __device__ constexpr int smem_bytes_for(int bnq, bool swap = false) {
  return stages_for(bnq, swap) * (P_STAGE_BYTES + q_stage_bytes(bnq)) + 1024 /* alignment */ + 256 /* barriers */;
}
__host__ __device__ constexpr uint32_t tmem_cols_for(int bnq) { return bnq < 32 ? 32 : bnq; }

template <typename TOut>
__device__ __forceinline__ void store_one(TOut* p, float v) { *p = from_f32<TOut>(v); }

// Where a tile of 128 rows starts when the tensor has `limit` rows: a tile that would reach past the
// end is moved back to end with the tensor (it then overlaps the tile before it, and both write
// the same values to the shared rows).  A TMA box that lies partly or wholly outside its tensor is
// filled far more slowly than one inside (measured: the gate/up product of 384 rows took 57 us,
// of 512 rows 32 us, before this), so no box of rows is let outside.
__device__ __forceinline__ int tile_row0(int row0, int limit) { return limit >= BP ? min(row0, limit - BP) : row0; }
// The same for a tile of `width` weight rows (output columns) in the normal mode.
__device__ __forceinline__ int tile_col0(int col0, int width, int limit) { return limit >= width ? min(col0, limit - width) : col0; }

// error codes written to *err_flag: which wait gave up
enum : int { ERR_PRODUCER = 1, ERR_MMA = 2, ERR_EPILOGUE = 3 };

// CLUSTER (swapped mode only): the CTAs that split K for one tile form a thread-block cluster
// along blockIdx.z.  Instead of writing float32 partial results to global memory for a later
// kernel to sum, each CTA hands its accumulator to the first CTA of the cluster through
// distributed shared memory; that CTA adds them in the order of the splits and stores the result.
template <int BNQ, bool SWAP, typename TOut, bool CLUSTER>
__global__ void __launch_bounds__(THREADS, SWAP ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
               TOut* __restrict__ C, long long ldc, long long split_stride, int M, int N, int K,
               int kblocks_per_split, int tile_q, int* __restrict__ err_flag) {
  // BNQ sizes the stages and the tensor memory; tile_q <= BNQ (a multiple of 32, or 16 = BNQ) is
  // the width actually computed, chosen on the host so that the grid fills whole waves.
  constexpr int STAGES = stages_for(BNQ, SWAP);
  constexpr int Q_STAGE_BYTES = q_stage_bytes(BNQ);
  constexpr uint32_t TMEM_COLS = tmem_cols_for(BNQ);
  const uint32_t IDESC = idesc_bf16_f32(BP, tile_q);
  // Fewer than 128 rows in the normal mode: the box of rows is only as tall as the tensor (the
  // host encodes the map so), which keeps it inside and brings no bytes for rows that are not
  // there; the MMA still reads 128 rows of the stage, and what it makes of the rest is not stored.
  const int p_box = (!SWAP && M < BP) ? M : BP;
  const uint32_t stage_tx = (uint32_t)(p_box * BK * 2 + tile_q * BK * 2);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_p = smem;
  uint8_t* smem_q = smem + STAGES * P_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * (P_STAGE_BYTES + Q_STAGE_BYTES));
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* accum_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p0 = tile_row0(blockIdx.x * BP, SWAP ? N : M);
  const int q0 = SWAP ? blockIdx.y * tile_q : tile_col0(blockIdx.y * tile_q, tile_q, N);
  const int total_kb = (K + BK - 1) / BK;
  const int kb_begin = blockIdx.z * kblocks_per_split;
  const int kb_end = min(total_kb, kb_begin + kblocks_per_split);
  const int nkb = max(0, kb_end - kb_begin);
  C += (long long)blockIdx.z * split_stride;
  float acc[CLUSTER ? BNQ : 1];          // the accumulator row of an epilogue thread, kept across the cluster barriers
  static_assert(!CLUSTER || (SWAP && BNQ <= 64), "cluster reduction is for the swapped mode with up to 64 rows");

  // The weights do not depend on earlier kernels: their tiles of the first pass over the ring
  // are requested before waiting for the previous kernel (the activations after), and as early
  // as can be: by the thread that has just initialised the barriers, before the CTA's first
  // barrier and while warp 1 still allocates tensor memory.  The earlier they are asked for, the
  // more of their way from memory is hidden behind the kernel before this one.
  uint8_t* smem_w = SWAP ? smem_p : smem_q;
  uint8_t* smem_a = SWAP ? smem_q : smem_p;
  const CUtensorMap* map_w = SWAP ? &map_p : &map_q;
  const CUtensorMap* map_a = SWAP ? &map_q : &map_p;
  constexpr int W_STAGE = SWAP ? P_STAGE_BYTES : Q_STAGE_BYTES;
  constexpr int A_STAGE = SWAP ? Q_STAGE_BYTES : P_STAGE_BYTES;
  const int w0 = SWAP ? p0 : q0, a0 = SWAP ? q0 : p0;
  const int pre = min(nkb, STAGES);
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(accum_bar, 1);
    fence_mbar_init();
    for (int i = 0; i < pre; ++i) {
      mbar_arrive_expect_tx(&full_bar[i], stage_tx);
      tma_load_2d(smem_w + i * W_STAGE, map_w, (kb_begin + i) * BK, w0, &full_bar[i]);
    }
    prefetch_tensormap(map_a);
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: TMA loads into the ring ----
      pdl_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d(smem_a + i * A_STAGE, map_a, (kb_begin + i) * BK, a0, &full_bar[i]);
      int issued = pre;
      bool ok = true;
      for (int i = pre; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (i / STAGES) & 1;
        ok = mbar_wait(&empty_bar[s], phase ^ 1);
        if (!ok) break;
        mbar_arrive_expect_tx(&full_bar[s], stage_tx);
        const int k = (kb_begin + i) * BK;
        tma_load_2d(smem_w + s * W_STAGE, map_w, k, w0, &full_bar[s]);
        tma_load_2d(smem_a + s * A_STAGE, map_a, k, a0, &full_bar[s]);
        issued = i + 1;
      }
      if (!ok) {
        atomicExch(err_flag, ERR_PRODUCER);
        // loads already in flight must land before the CTA may go: wait for them (bounded)
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(&full_bar[i % STAGES], (i / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (i / STAGES) & 1;
        ok = mbar_wait(&full_bar[s], phase);
        if (!ok) break;
        fence_after_sync();
        const uint64_t desc_p = smem_desc_sw128(smem_u32(smem_p + s * P_STAGE_BYTES));
        const uint64_t desc_q = smem_desc_sw128(smem_u32(smem_q + s * Q_STAGE_BYTES));
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // 16 elements of K = 32 bytes further along the swizzled row: +2 in units of 16 bytes
          mma_bf16(tmem_base, desc_p + 2 * k, desc_q + 2 * k, IDESC, (i | k) != 0);
        }
        mma_commit(&empty_bar[s]);
      }
      if (!ok) atomicExch(err_flag, ERR_MMA);
      mma_commit(accum_bar);          // arrives when everything issued above has finished
    }
  } else {
    // ---- epilogue: tensor memory -> registers -> global ----
    const int quad = warp & 3;                       // the lanes this warp may read: 32*quad ..
    const int p = p0 + quad * 32 + lane;             // row of P that this thread holds
    bool ok = mbar_wait(accum_bar, 0);
    if (!ok && lane == 0) atomicExch(err_flag, ERR_EPILOGUE);
    fence_after_sync();
    constexpr int CHUNK = BNQ >= 32 ? 32 : 16;
    const int p_limit = SWAP ? N : M, q_limit = SWAP ? M : N;
    if (CLUSTER) {
#pragma unroll
      for (int c = 0; c < BNQ; c += CHUNK) {
        if (nkb > 0 && ok) {
          const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c;
          if (CHUNK == 32) {
            uint32_t r[32];
            tmem_ld_x32(taddr, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < CHUNK; ++j) acc[(CLUSTER ? c : 0) + (CLUSTER ? j : 0)] = __uint_as_float(r[j]);
          } else {
            uint32_t r[16];
            tmem_ld_x16(taddr, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < CHUNK; ++j) acc[(CLUSTER ? c : 0) + (CLUSTER ? j : 0)] = __uint_as_float(r[j]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < CHUNK; ++j) acc[(CLUSTER ? c : 0) + (CLUSTER ? j : 0)] = 0.f;
        }
      }
    }
#pragma unroll 1
    for (int c = 0; c < (CLUSTER ? 0 : tile_q); c += CHUNK) {
      float v[CHUNK];
      if (nkb > 0 && ok) {
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c;
        if (CHUNK == 32) {
          uint32_t r[32];
          tmem_ld_x32(taddr, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < CHUNK; ++j) v[j] = __uint_as_float(r[j]);
        } else {
          uint32_t r[16];
          tmem_ld_x16(taddr, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < CHUNK; ++j) v[j] = __uint_as_float(r[j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < CHUNK; ++j) v[j] = 0.f;
      }
      if (p >= p_limit) continue;
      const int q = q0 + c;
      if (SWAP) {
        // thread holds C[m = q + j][n = p]: neighbouring lanes are neighbouring n
#pragma unroll
        for (int j = 0; j < CHUNK; ++j)
          if (q + j < q_limit) store_one(C + (long long)(q + j) * ldc + p, v[j]);
      } else {
        // thread holds C[m = p][n = q .. q + CHUNK)
        TOut* row = C + (long long)p * ldc + q;
        const bool vec_ok = (q + CHUNK <= q_limit) && ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
        if (vec_ok) {
          if (sizeof(TOut) == 2) {
#pragma unroll
            for (int j = 0; j < CHUNK; j += 8) {
              uint4 u;
              __nv_bfloat162 b0 = __floats2bfloat162_rn(v[j], v[j + 1]), b1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
              __nv_bfloat162 b2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), b3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
              u.x = *reinterpret_cast<uint32_t*>(&b0); u.y = *reinterpret_cast<uint32_t*>(&b1);
              u.z = *reinterpret_cast<uint32_t*>(&b2); u.w = *reinterpret_cast<uint32_t*>(&b3);
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(row) + j) = u;
            }
          } else {
#pragma unroll
            for (int j = 0; j < CHUNK; j += 4)
              *reinterpret_cast<float4*>(reinterpret_cast<float*>(row) + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < CHUNK; ++j)
            if (q + j < q_limit) store_one(row + j, v[j]);
        }
      }
    }
  }

  if (CLUSTER) {
    // Every MMA of every CTA of the cluster is done once all epilogue threads have passed their
    // accumulator wait, so after the first barrier the stage ring is free to receive the sums.
    const uint32_t rank = cluster_ctarank();
    const int m_valid = min(BNQ, M - q0);
    const int quad = warp & 3;
    const int n_local = quad * 32 + lane;
    cluster_sync();
    if (warp >= 2 && rank != 0) {
      const uint32_t slot = map_to_cta(smem_u32(smem), 0) + (uint32_t)(((rank - 1) * BNQ) * BP + n_local) * 4u;
#pragma unroll
      for (int m = 0; m < BNQ; ++m)
        if (m < m_valid) st_cluster_f32(slot + (uint32_t)(m * BP) * 4u, acc[CLUSTER ? m : 0]);
    }
    cluster_sync();
    if (warp >= 2 && rank == 0) {
      const float* slots = reinterpret_cast<const float*>(smem);
      const int n = p0 + n_local;
#pragma unroll
      for (int m = 0; m < BNQ; ++m) {
        if (m < m_valid && n < N) {
          float v = acc[CLUSTER ? m : 0];
          for (int r = 0; r + 1 < (int)gridDim.z; ++r) v += slots[((size_t)r * BNQ + m) * BP + n_local];
          store_one(C + (long long)(q0 + m) * ldc + n, v);
        }
      }
    }
  }

  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- persistent variant for many rows ---------------------------------------------------
// One CTA per SM walks over the output tiles (blockIdx.x, + gridDim.x, ...).  The accumulator is
// double-buffered in tensor memory (2 x 256 columns), so the epilogue of one tile (tensor memory
// -> registers -> global) runs while the MMA thread already works on the next tile; the stage
// ring keeps running across tiles.  Tiles are numbered with the row tile fastest, so CTAs that
// run at the same time share the same few weight tiles in L2.  Normal mode only (P = rows of A).
//
// SWIGLU: W [2I, K] holds I gate rows followed by I up rows (N = 2I).  A tile then takes 128 gate
// rows and the 128 up rows that belong to them (two TMA boxes per stage) as one 256-wide MMA;
// the epilogue reads a gate column and its up column 128 columns apart and writes
// silu(gate) * up to C [M, I].  The product itself never reaches memory.
enum : int { ERR_P_PRODUCER = 4, ERR_P_MMA = 5, ERR_P_EPILOGUE = 6 };

// silu(gate) * up in float32, as the stand-alone kernel computes it
__device__ __forceinline__ float silu_times(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// 32 values of one row of C, columns q .. q + 32 (those below q_limit), as 16-byte stores where
// the row allows it.
template <typename TOut>
__device__ __forceinline__ void store_row32(TOut* row, const float (&v)[32], int q, int q_limit) {
  const bool vec_ok = (q + 32 <= q_limit) && ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
  if (vec_ok) {
    if (sizeof(TOut) == 2) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 u;
        __nv_bfloat162 b0 = __floats2bfloat162_rn(v[j], v[j + 1]), b1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
        __nv_bfloat162 b2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), b3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
        u.x = *reinterpret_cast<uint32_t*>(&b0); u.y = *reinterpret_cast<uint32_t*>(&b1);
        u.z = *reinterpret_cast<uint32_t*>(&b2); u.w = *reinterpret_cast<uint32_t*>(&b3);
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(row) + j) = u;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(row) + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (q + j < q_limit) store_one(row + j, v[j]);
  }
}

template <typename TOut, bool SWIGLU>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                          TOut* __restrict__ C, long long ldc, int M, int N, int K, int tile_q,
                          int* __restrict__ err_flag) {
  constexpr int BNQ = 256;
  constexpr int STAGES = stages_for(BNQ);
  constexpr int Q_STAGE_BYTES = q_stage_bytes(BNQ);
  constexpr uint32_t TMEM_COLS = 512;
  const uint32_t IDESC = idesc_bf16_f32(BP, tile_q);
  const uint32_t stage_tx = (uint32_t)(P_STAGE_BYTES + tile_q * BK * 2);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_p = smem;
  uint8_t* smem_q = smem + STAGES * P_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * (P_STAGE_BYTES + Q_STAGE_BYTES));
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;       // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;            // [2] epilogue -> MMA (four warps arrive)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int inter = N / 2;                                 // SWIGLU: gate rows, and output columns
  const int m_tiles = (M + BP - 1) / BP, n_tiles = SWIGLU ? (inter + 127) / 128 : (N + tile_q - 1) / tile_q;
  const int total_tiles = m_tiles * n_tiles;
  const int nkb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    fence_mbar_init();
    prefetch_tensormap(&map_p);
    prefetch_tensormap(&map_q);
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // ---- producer ----
      pdl_wait();
      bool ok = true;
      int it = 0;                                             // k-blocks issued so far, over all tiles
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int p0 = tile_row0((tile % m_tiles) * BP, M);
        const int q0 = SWIGLU ? (tile / m_tiles) * 128 : tile_col0((tile / m_tiles) * tile_q, tile_q, N);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1);
          if (!ok) break;
          mbar_arrive_expect_tx(&full_bar[s], stage_tx);
          tma_load_2d(smem_q + s * Q_STAGE_BYTES, &map_q, kb * BK, q0, &full_bar[s]);
          // the up rows of these gate rows: rows 128.. of the stage (a box is 128 rows of 128 bytes)
          if (SWIGLU) tma_load_2d(smem_q + s * Q_STAGE_BYTES + 128 * 128, &map_q, kb * BK, inter + q0, &full_bar[s]);
          tma_load_2d(smem_p + s * P_STAGE_BYTES, &map_p, kb * BK, p0, &full_bar[s]);
        }
      }
      if (!ok) {
        atomicExch(err_flag, ERR_P_PRODUCER);
        for (int i = max(0, it - STAGES); i < it; ++i) mbar_wait(&full_bar[i % STAGES], (i / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      bool ok = true;
      int it = 0, n = 0;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++n) {
        const int buf = n & 1;
        ok = mbar_wait(&acc_empty[buf], ((n >> 1) & 1) ^ 1);   // the epilogue has drained this accumulator
        if (!ok) break;
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BNQ);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&full_bar[s], (it / STAGES) & 1);
          if (!ok) break;
          fence_after_sync();
          const uint64_t desc_p = smem_desc_sw128(smem_u32(smem_p + s * P_STAGE_BYTES));
          const uint64_t desc_q = smem_desc_sw128(smem_u32(smem_q + s * Q_STAGE_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) mma_bf16(d_tmem, desc_p + 2 * k, desc_q + 2 * k, IDESC, (kb | k) != 0);
          mma_commit(&empty_bar[s]);
        }
        mma_commit(&acc_full[buf]);
      }
      if (!ok) {
        atomicExch(err_flag, ERR_P_MMA);
        mma_commit(&acc_full[0]);
        mma_commit(&acc_full[1]);
      }
    }
  } else {
    // ---- epilogue ----
    const int quad = warp & 3;
    bool ok = true;
    int n = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++n) {
      const int buf = n & 1;
      const int p0 = tile_row0((tile % m_tiles) * BP, M);
      const int q0 = SWIGLU ? (tile / m_tiles) * 128 : tile_col0((tile / m_tiles) * tile_q, tile_q, N);
      const int p = p0 + quad * 32 + lane;
      if (ok) ok = mbar_wait(&acc_full[buf], (n >> 1) & 1);
      fence_after_sync();
#pragma unroll 1
      for (int c = 0; c < (SWIGLU ? 128 : tile_q); c += 32) {
        float v[32];
        if (ok) {
          uint32_t r[32];
          tmem_ld_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BNQ + c), r);
          if (SWIGLU) {
            uint32_t u[32];
            tmem_ld_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BNQ + 128 + c), u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = silu_times(__uint_as_float(r[j]), __uint_as_float(u[j]));
          } else {
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        if (p >= M) continue;
        const int q = q0 + c;
        const int q_limit = SWIGLU ? inter : N;
        store_row32(C + (long long)p * ldc + q, v, q, q_limit);
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);             // this warp has read its lanes of the accumulator
    }
    if (!ok && lane == 0) atomicExch(err_flag, ERR_P_EPILOGUE);
  }

  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- persistent variant on pairs of CTAs ---------------------------------------------------
// Two CTAs on neighbouring SMs (a cluster of two) work on one tile of 256 rows x tile_q columns
// with MMAs of cta_group::2: each CTA stages its 128 rows of A and its half of the tile's rows of
// W, the first CTA's MMA thread issues for both, and each CTA's tensor memory holds the
// accumulator of its own 128 rows.  A k-block then costs each SM 32 KB of loads for 128 x 256 x 64
// products where the single-CTA kernel above needs 48 KB, which is what bounds that kernel; the
// ring has six stages instead of four.  Everything else (walk over the tiles, two accumulators,
// the epilogue, SWIGLU) is as above; with SWIGLU the first CTA stages the 128 gate rows and the
// second the 128 up rows.
//
// Barriers: the loads of both CTAs count on the first CTA's full barrier; tcgen05.commit arrives
// on the empty barrier (and on acc_full) of both CTAs; the epilogue warps of both CTAs arrive on
// the first CTA's acc_empty.
enum : int { ERR_2_PRODUCER = 7, ERR_2_MMA = 8, ERR_2_EPILOGUE = 9 };

struct RopeStore;
template <typename TOut>
__device__ __forceinline__ void rope_store_epilogue(uint32_t t_row, bool ok, int p, bool row_valid, int q0, int tile_q,
                                                    int N, TOut* __restrict__ C, long long ldc, const RopeStore& rs);
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_Q_STAGE_BYTES = 128 * BK * 2;      // up to 128 rows of W per CTA
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * (P_STAGE_BYTES + PAIR_Q_STAGE_BYTES) + 1024 + 256;

// What the epilogue EPI_ROPE needs besides the product: W's rows are query heads, then key
// heads, then value heads (n_kv of each; none if n_kv == 0); row t of the product belongs to
// position positions[t] and its key and value go to place slot_map[t] of the pages
// [page][kv head][token in page][head_dim].  Tables [position][head_dim / 2], or null for no rotation.
struct RopeStore {
  const float* cos_table;
  const float* sin_table;
  const int* positions;
  const int* slot_map;
  __nv_bfloat16* k_pages;
  __nv_bfloat16* v_pages;
  int n_heads, n_kv, head_dim, page_size;
};
enum : int { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_ROPE = 2 };

// EPI_ROPE: the product is a QKV projection whose tiles are whole heads (tile_q a multiple of
// head_dim, 64 or 128).  The epilogue rotates the query and key heads of its row by the row's
// position (rotate-half, float32, on the float32 accumulator), writes the queries to C
// [M, n_heads * head_dim] and stores keys and values in the pages, so the product itself never
// reaches memory and no rotate-and-store kernel runs.
template <typename TOut, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                    TOut* __restrict__ C, long long ldc, int M, int N, int K, int tile_q, RopeStore rs,
                    int* __restrict__ err_flag) {
  constexpr bool SWIGLU = EPI == EPI_SWIGLU;
  constexpr int STAGES = PAIR_STAGES;
  constexpr int BNQ = 256;                      // columns of one accumulator
  constexpr uint32_t TMEM_COLS = 512;
  const uint32_t IDESC = idesc_bf16_f32(2 * BP, tile_q);
  const int half_q = tile_q / 2;                // rows of W that each CTA stages
  const uint32_t stage_tx = 2u * (uint32_t)(P_STAGE_BYTES + half_q * BK * 2);      // both CTAs' boxes

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_p = smem;
  uint8_t* smem_q = smem + STAGES * P_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * (P_STAGE_BYTES + PAIR_Q_STAGE_BYTES));
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;       // [2] MMA -> epilogue, in both CTAs
  uint64_t* acc_empty = acc_full + 2;            // [2] epilogue -> MMA: the first CTA's, eight warps arrive
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int inter = N / 2;
  const int m_tiles = (M + 2 * BP - 1) / (2 * BP), n_tiles = SWIGLU ? (inter + 127) / 128 : (N + tile_q - 1) / tile_q;
  const int total_tiles = m_tiles * n_tiles;
  const int nkb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);
    }
    fence_mbar_init();
    prefetch_tensormap(&map_p);
    prefetch_tensormap(&map_q);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
  fence_before_sync();
  cluster_sync();                 // both CTAs' barriers are initialised before either is signalled from the other side
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // ---- producer (both CTAs) ----
      // The weights do not depend on the kernel before: those of the first pass over the ring
      // are requested before waiting for it, the activations after.
      const int early = pair < total_tiles ? min(nkb, STAGES) : 0;
      auto weight_row = [&](int tile) {
        const int q_tile = SWIGLU ? (tile / m_tiles) * 128 : tile_col0((tile / m_tiles) * tile_q, tile_q, N);
        return SWIGLU ? (rank ? inter + q_tile : q_tile) : q_tile + (int)rank * half_q;
      };
      for (int i = 0; i < early; ++i) {
        if (rank == 0) mbar_arrive_expect_tx(&full_bar[i], stage_tx);
        tma_load_2d_pair(smem_q + i * PAIR_Q_STAGE_BYTES, &map_q, i * BK, weight_row(pair), map_to_cta(smem_u32(&full_bar[i]), 0));
      }
      pdl_wait();
      bool ok = true;
      int it = 0;
      for (int tile = pair; tile < total_tiles && ok; tile += pairs) {
        const int p0 = tile_row0((tile % m_tiles) * (2 * BP) + (int)rank * BP, M);
        const int q0 = weight_row(tile);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t full0 = map_to_cta(smem_u32(&full_bar[s]), 0);
          if (it >= early) {
            ok = mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1);
            if (!ok) break;
            if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], stage_tx);
            tma_load_2d_pair(smem_q + s * PAIR_Q_STAGE_BYTES, &map_q, kb * BK, q0, full0);
          }
          tma_load_2d_pair(smem_p + s * P_STAGE_BYTES, &map_p, kb * BK, p0, full0);
        }
      }
      if (!ok) {
        atomicExch(err_flag, ERR_2_PRODUCER);
        // loads in flight must land before the CTA may go: the first CTA can wait for them on its
        // barriers, the second one lets their time pass
        if (rank == 0) {
          for (int i = max(0, it - STAGES); i < it; ++i) mbar_wait(&full_bar[i % STAGES], (i / STAGES) & 1);
        } else {
          const long long t0 = clock64();
          while (clock64() - t0 < 4000000ll) {}
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---- MMA issuer (the first CTA's, for both) ----
      bool ok = true;
      int it = 0, n = 0;
      for (int tile = pair; tile < total_tiles && ok; tile += pairs, ++n) {
        const int buf = n & 1;
        ok = mbar_wait(&acc_empty[buf], ((n >> 1) & 1) ^ 1);   // both epilogues have drained this accumulator
        if (!ok) break;
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BNQ);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&full_bar[s], (it / STAGES) & 1);
          if (!ok) break;
          fence_after_sync();
          const uint64_t desc_p = smem_desc_sw128(smem_u32(smem_p + s * P_STAGE_BYTES));
          const uint64_t desc_q = smem_desc_sw128(smem_u32(smem_q + s * PAIR_Q_STAGE_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) mma_bf16_pair(d_tmem, desc_p + 2 * k, desc_q + 2 * k, IDESC, (kb | k) != 0);
          mma_commit_pair(&empty_bar[s], 3);
        }
        mma_commit_pair(&acc_full[buf], 3);
      }
      if (!ok) {
        atomicExch(err_flag, ERR_2_MMA);
        mma_commit_pair(&acc_full[0], 3);
        mma_commit_pair(&acc_full[1], 3);
      }
    }
  } else {
    // ---- epilogue (both CTAs, each its own 128 rows) ----
    const int quad = warp & 3;
    bool ok = true;
    int n = 0;
    for (int tile = pair; tile < total_tiles; tile += pairs, ++n) {
      const int buf = n & 1;
      const int p0 = tile_row0((tile % m_tiles) * (2 * BP) + (int)rank * BP, M);
      const int q0 = SWIGLU ? (tile / m_tiles) * 128 : tile_col0((tile / m_tiles) * tile_q, tile_q, N);
      const int p = p0 + quad * 32 + lane;
      if (ok) ok = mbar_wait(&acc_full[buf], (n >> 1) & 1);
      fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BNQ);
      if constexpr (EPI == EPI_ROPE) {
        rope_store_epilogue(t_row, ok, p, p < M, q0, tile_q, N, C, ldc, rs);
      } else {
#pragma unroll 1
        for (int c = 0; c < (SWIGLU ? 128 : tile_q); c += 32) {
          float v[32];
          if (ok) {
            uint32_t r[32];
            tmem_ld_x32(t_row + (uint32_t)c, r);
            if (SWIGLU) {
              uint32_t u[32];
              tmem_ld_x32(t_row + (uint32_t)(128 + c), u);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = silu_times(__uint_as_float(r[j]), __uint_as_float(u[j]));
            } else {
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
          if (p >= M) continue;
          const int q = q0 + c;
          store_row32(C + (long long)p * ldc + q, v, q, SWIGLU ? inter : N);
        }
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
    }
    if (!ok && lane == 0) atomicExch(err_flag, ERR_2_EPILOGUE);
  }

  // Neither CTA may go while the other may still read its shared memory or signal its barriers.
  fence_before_sync();
  cluster_sync();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// The epilogue of a QKV projection (see RopeStore): this thread holds row p of the tile, whose
// accumulator row starts at t_row in tensor memory; the tile's columns q0 .. q0 + tile_q are whole
// heads.  Every lane runs the tensor-memory loads (they are warp-wide); only valid rows store.
template <typename TOut>
__device__ __forceinline__ void rope_store_epilogue(uint32_t t_row, bool ok, int p, bool row_valid, int q0, int tile_q,
                                                    int N, TOut* __restrict__ C, long long ldc, const RopeStore& rs) {
  const int hd = rs.head_dim, half = hd / 2;
  int pos = 0, slot = 0;
  if (row_valid) {
    pos = rs.positions[p];
    if (rs.n_kv) slot = rs.slot_map[p];
  }
  const int page = slot / rs.page_size, off = slot % rs.page_size;
  const float* cs = rs.cos_table ? rs.cos_table + (size_t)pos * half : nullptr;
  const float* sn = rs.cos_table ? rs.sin_table + (size_t)pos * half : nullptr;
#pragma unroll 1
  for (int hc = 0; hc < tile_q && q0 + hc < N; hc += hd) {
    const int head = (q0 + hc) / hd;
    const bool is_q = head < rs.n_heads, is_k = !is_q && head < rs.n_heads + rs.n_kv;
    TOut* dst;
    if (is_q) {
      dst = C + (long long)p * ldc + (long long)head * hd;
    } else {
      const int g = head - rs.n_heads - (is_k ? 0 : rs.n_kv);
      __nv_bfloat16* pages = is_k ? rs.k_pages : rs.v_pages;
      dst = reinterpret_cast<TOut*>(pages + (((size_t)page * rs.n_kv + g) * rs.page_size + off) * hd);
    }
    const bool rotate = (is_q || is_k) && cs != nullptr;
#pragma unroll 1
    for (int i = 0; i < half; i += 32) {
      // 32 columns of the first half of the head and their partners in the second half
      float a[32], b[32];
      if (ok) {
        uint32_t ra[32], rb[32];
        tmem_ld_x32(t_row + (uint32_t)(hc + i), ra);
        tmem_ld_x32(t_row + (uint32_t)(hc + half + i), rb);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) { a[j] = __uint_as_float(ra[j]); b[j] = __uint_as_float(rb[j]); }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) { a[j] = 0.f; b[j] = 0.f; }
      }
      if (!row_valid) continue;
      if (rotate) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 c4 = __ldg(reinterpret_cast<const float4*>(cs + i + j));
          const float4 s4 = __ldg(reinterpret_cast<const float4*>(sn + i + j));
          const float c[4] = {c4.x, c4.y, c4.z, c4.w}, s[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float x = a[j + k], y = b[j + k];
            a[j + k] = x * c[k] - y * s[k];
            b[j + k] = x * s[k] + y * c[k];
          }
        }
      }
      store_row32(dst + i, a, 0, 32);
      store_row32(dst + half + i, b, 0, 32);
    }
  }
}

// ---- host side ----------------------------------------------------------------
struct MapKey {
  const void* base; uint64_t rows, cols, ld; uint32_t box;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box == o.box; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.base;
    h = h * 1000003u ^ k.rows; h = h * 1000003u ^ k.cols; h = h * 1000003u ^ k.ld; h = h * 1000003u ^ k.box;
    return h;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
std::mutex g_maps_mutex;

int get_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box) {
  MapKey key{base, rows, cols, ld, box};
  std::lock_guard<std::mutex> lock(g_maps_mutex);
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    CUtensorMap m;
    int rc = encode_tensor_map_bf16(&m, base, rows, cols, ld, box);
    if (rc) return rc;
    if (g_maps.size() > 4096) g_maps.clear();
    it = g_maps.emplace(key, m).first;
  }
  *out = it->second;
  return 0;
}

int* g_err_flag = nullptr;      // the device word of this call: the caller's block or the library's own

int ensure_err_flag() {
  g_err_flag = llmk_error_word(1);
  if (!g_err_flag) return llmk_fail(-1, "gemm_tc: cannot allocate the error word");
  return 0;
}

template <int BNQ, bool SWAP, typename TOut, bool CLUSTER>
int launch_cfg(const CUtensorMap& mp, const CUtensorMap& mq, void* C, long long ldc, long long split_stride, int M,
               int N, int K, int splits, int kb_per_split, int tile_q, cudaStream_t stream) {
  auto kern = gemm_tc_kernel<BNQ, SWAP, TOut, CLUSTER>;
  constexpr int smem = smem_bytes_for(BNQ, SWAP);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return llmk_fail((int)e, "gemm_tc: cannot set %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int p_rows = SWAP ? N : M, q_rows = SWAP ? M : N;
  dim3 grid((p_rows + BP - 1) / BP, (q_rows + tile_q - 1) / tile_q, splits);
  if (CLUSTER) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = llmk_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kern, mp, mq, (TOut*)C, ldc, split_stride, M, N, K, kb_per_split, tile_q, g_err_flag);
  } else {
    launch_kernel(kern, grid, dim3(THREADS), (size_t)smem, stream, mp, mq, (TOut*)C, ldc, split_stride, M, N, K, kb_per_split, tile_q, g_err_flag);
  }
  LLMK_LAUNCH_CHECK("gemm_tc");
}

template <typename TOut, bool SWIGLU>
int launch_persistent(const CUtensorMap& mp, const CUtensorMap& mq, void* C, long long ldc, int M, int N, int K,
                      int tile_q, cudaStream_t stream) {
  auto kern = gemm_tc_persistent_kernel<TOut, SWIGLU>;
  constexpr int smem = smem_bytes_for(256);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return llmk_fail((int)e, "gemm_tc: cannot set %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int tiles = ((M + BP - 1) / BP) * (SWIGLU ? (N / 2 + 127) / 128 : (N + tile_q - 1) / tile_q);
  launch_kernel(kern, dim3(tiles < llmk_sm_count() ? tiles : llmk_sm_count()), dim3(THREADS), (size_t)smem, stream, mp, mq, (TOut*)C, ldc, M, N, K,
                tile_q, g_err_flag);
  LLMK_LAUNCH_CHECK("gemm_tc_persistent");
}

// The pairs that can run at once (one CTA per SM, two neighbouring SMs per pair), asked once.
template <typename Kernel>
int max_pairs(Kernel kern) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * llmk_sm_count());
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
    cudaGetLastError();
    return 0;
  }
  return n < llmk_sm_count() / 2 ? n : llmk_sm_count() / 2;
}

template <typename TOut, int EPI>
int launch_pair(const CUtensorMap& mp, const CUtensorMap& mq, void* C, long long ldc, int M, int N, int K,
                int tile_q, const RopeStore& rs, cudaStream_t stream) {
  constexpr bool SWIGLU = EPI == EPI_SWIGLU;
  auto kern = gemm_tc_pair_kernel<TOut, EPI>;
  static int pairs_max = -1;
  if (pairs_max < 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES);
    if (e != cudaSuccess) return llmk_fail((int)e, "gemm_tc: cannot set %d bytes of shared memory: %s", PAIR_SMEM_BYTES, cudaGetErrorString(e));
    pairs_max = max_pairs(kern);
  }
  if (pairs_max < 1) return llmk_fail(-2, "gemm_tc: no pair of CTAs of the pair kernel fits this device");
  const int tiles = ((M + 2 * BP - 1) / (2 * BP)) * (SWIGLU ? (N / 2 + 127) / 128 : (N + tile_q - 1) / tile_q);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (tiles < pairs_max ? tiles : pairs_max));
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = llmk_pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, kern, mp, mq, (TOut*)C, ldc, M, N, K, tile_q, rs, g_err_flag);
  LLMK_LAUNCH_CHECK("gemm_tc_pair");
}

template <typename TOut>
int launch_out(bool swap, int bnq, bool cluster, const CUtensorMap& mp, const CUtensorMap& mq, void* C, long long ldc,
               long long split_stride, int M, int N, int K, int splits, int kbps, cudaStream_t s) {
  if (swap && cluster) {
    switch (bnq) {
      case 16: return launch_cfg<16, true, TOut, true>(mp, mq, C, ldc, split_stride, M, N, K, splits, kbps, bnq, s);
      case 32: return launch_cfg<32, true, TOut, true>(mp, mq, C, ldc, split_stride, M, N, K, splits, kbps, bnq, s);
      case 64: return launch_cfg<64, true, TOut, true>(mp, mq, C, ldc, split_stride, M, N, K, splits, kbps, bnq, s);
    }
  } else if (swap) {
    switch (bnq) {
      case 16: return launch_cfg<16, true, TOut, false>(mp, mq, C, ldc, split_stride, M, N, K, splits, kbps, bnq, s);
      case 32: return launch_cfg<32, true, TOut, false>(mp, mq, C, ldc, split_stride, M, N, K, splits, kbps, bnq, s);
      case 64: return launch_cfg<64, true, TOut, false>(mp, mq, C, ldc, split_stride, M, N, K, splits, kbps, bnq, s);
      case 128: return launch_cfg<128, true, TOut, false>(mp, mq, C, ldc, split_stride, M, N, K, splits, kbps, bnq, s);
    }
  } else if (bnq % 32 == 0 && bnq >= 32 && bnq <= 256) {
    if (bnq <= 128) return launch_cfg<128, false, TOut, false>(mp, mq, C, ldc, split_stride, M, N, K, splits, kbps, bnq, s);
    return launch_cfg<256, false, TOut, false>(mp, mq, C, ldc, split_stride, M, N, K, splits, kbps, bnq, s);
  }
  return llmk_fail(-1, "gemm_tc: no kernel for swap=%d tile=%d cluster=%d", (int)swap, bnq, (int)cluster);
}

}  // namespace

// Whether the tensor-core product takes this problem: bf16 operands with 16-byte aligned
// rows (K and both pitches multiples of 8 elements).
LLMK_API int llmk_gemm_tc_supported(const void* A, const void* W, int M, int N, int K, long long lda, long long ldw) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 8 || lda % 8 || ldw % 8) return 0;
  if ((uintptr_t)A % 16 || (uintptr_t)W % 16) return 0;
  return 1;
}

// A [M,K] and W [N,K] bf16.  splits == 1: C (bf16 if out_dtype == 1, else float32) [M, ldc].
// splits > 1 without cluster: C must be float32 and is written as [splits][M][ldc] partial sums
// (split_stride = M * ldc elements) over kblocks_per_split blocks of 64 along K each.
// splits > 1 with cluster != 0 (swapped mode, tile up to 64, at most 8 splits): the splits of a
// tile form a thread-block cluster, sum their results on chip and write C as for splits == 1.
// cluster == 2 selects the persistent kernel (normal mode, one split): one CTA per SM walks over
// the tiles with two accumulators in tensor memory.  cluster == 3: the same on pairs of CTAs with
// tiles of 256 rows (cta_group::2).
// swiglu != 0 (persistent kernels only): W [N = 2I, K] is I gate rows followed by I up rows and C
// [M, I] (bfloat16) receives silu(gate) * up instead of the product.
// swap != 0 puts the weights on the 128-row side of the MMA; tile is the other side's width
// (16, 32, 64 or 128 when swapped; a multiple of 32 up to 256 otherwise).
LLMK_API int llmk_gemm_tc(const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw,
                          long long ldc, int out_dtype, int swap, int tile, int splits, int kblocks_per_split,
                          int cluster, int swiglu, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (swiglu) {
    LLMK_REQUIRE((cluster == 2 || cluster == 3) && !swap && splits == 1 && N % 2 == 0 && (N / 2) % 8 == 0,
                 "gemm_tc: silu(gate) * up in the epilogue needs the persistent kernel and an even N with N/2 a multiple of 8, got N=%d", N);
    tile = 256;       // 128 gate rows and their 128 up rows
  }
  LLMK_REQUIRE(llmk_gemm_tc_supported(A, W, M, N, K, lda, ldw), "gemm_tc: K=%d and the row pitches must be multiples of 8 and the bases 16-byte aligned", K);
  LLMK_REQUIRE(splits >= 1 && kblocks_per_split >= 1 && (long long)splits * kblocks_per_split * BK >= K,
               "gemm_tc: %d splits of %d k-blocks do not cover K=%d", splits, kblocks_per_split, K);
  if (splits == 1 && cluster == 1) cluster = 0;
  LLMK_REQUIRE(splits == 1 || cluster || out_dtype == LLMK_F32, "gemm_tc: split-K without a cluster needs a float32 output");
  if (cluster == 1) {
    LLMK_REQUIRE(swap && tile <= 64 && splits <= 8, "gemm_tc: cluster reduction needs the swapped mode, a tile up to 64 and at most 8 splits");
    LLMK_REQUIRE((long long)(splits - 1) * tile * BP * 4 <= (long long)stages_for(tile, true) * (P_STAGE_BYTES + q_stage_bytes(tile)),
                 "gemm_tc: %d splits of a %d-row tile do not fit the stage ring for the on-chip sum", splits, tile);
  }
  LLMK_REQUIRE(splits <= 65535, "gemm_tc: too many splits");
  int rc = ensure_err_flag();
  if (rc) return rc;
  CUtensorMap mp, mq;
  const void* P = swap ? W : A; const void* Q = swap ? A : W;
  const long long ldp = swap ? ldw : lda, ldq = swap ? lda : ldw;
  const int p_rows = swap ? N : M, q_rows = swap ? M : N;
  // the one-tile kernel in the normal mode takes a box of rows no taller than the tensor (see the kernel)
  if ((rc = get_map(&mp, P, p_rows, K, ldp, (!swap && cluster == 0 && M < BP) ? M : BP))) return rc;
  if ((rc = get_map(&mq, Q, q_rows, K, ldq, swiglu ? 128 : cluster == 3 ? tile / 2 : tile))) return rc;
  if (cluster == 3) {       // persistent kernel on pairs of CTAs: normal mode, no split
    LLMK_REQUIRE(!swap && splits == 1 && tile % 32 == 0 && tile >= 32 && tile <= 256,
                 "gemm_tc: the pair kernel takes the normal mode, one split and a tile of 32..256 in steps of 32");
    if (swiglu) {
      if (out_dtype == LLMK_BF16) return launch_pair<__nv_bfloat16, EPI_SWIGLU>(mp, mq, C, ldc, M, N, K, tile, RopeStore{}, stream);
      return llmk_fail(-1, "gemm_tc: silu(gate) * up is written as bfloat16 only");
    }
    if (out_dtype == LLMK_F32) return launch_pair<float, EPI_PLAIN>(mp, mq, C, ldc, M, N, K, tile, RopeStore{}, stream);
    if (out_dtype == LLMK_BF16) return launch_pair<__nv_bfloat16, EPI_PLAIN>(mp, mq, C, ldc, M, N, K, tile, RopeStore{}, stream);
    return llmk_fail(-1, "gemm_tc: unsupported output kind %d", out_dtype);
  }
  if (cluster == 2) {       // persistent kernel: normal mode, no split
    LLMK_REQUIRE(!swap && splits == 1 && tile % 32 == 0 && tile >= 32 && tile <= 256,
                 "gemm_tc: the persistent kernel takes the normal mode, one split and a tile of 32..256 in steps of 32");
    if (swiglu) {
      if (out_dtype == LLMK_BF16) return launch_persistent<__nv_bfloat16, true>(mp, mq, C, ldc, M, N, K, tile, stream);
      return llmk_fail(-1, "gemm_tc: silu(gate) * up is written as bfloat16 only");
    }
    if (out_dtype == LLMK_F32) return launch_persistent<float, false>(mp, mq, C, ldc, M, N, K, tile, stream);
    if (out_dtype == LLMK_BF16) return launch_persistent<__nv_bfloat16, false>(mp, mq, C, ldc, M, N, K, tile, stream);
    return llmk_fail(-1, "gemm_tc: unsupported output kind %d", out_dtype);
  }
  const long long split_stride = (splits > 1 && !cluster) ? (long long)M * ldc : 0;
  if (out_dtype == LLMK_F32) return launch_out<float>(swap != 0, tile, cluster != 0, mp, mq, C, ldc, split_stride, M, N, K, splits, kblocks_per_split, stream);
  if (out_dtype == LLMK_BF16) return launch_out<__nv_bfloat16>(swap != 0, tile, cluster != 0, mp, mq, C, ldc, split_stride, M, N, K, splits, kblocks_per_split, stream);
  return llmk_fail(-1, "gemm_tc: unsupported output kind %d", out_dtype);
}

// Whether llmk_gemm_tc_qkv_rope takes these sizes and pointers.
LLMK_API int llmk_gemm_tc_qkv_rope_supported(const void* A, const void* W, int M, int N, int K, long long lda,
                                             long long ldw, const void* q_out, long long ldq, const float* cos_table,
                                             const float* sin_table, const void* k_pages, const void* v_pages,
                                             int n_heads, int n_kv, int head_dim) {
  if (!llmk_gemm_tc_supported(A, W, M, N, K, lda, ldw)) return 0;
  if (head_dim != 64 && head_dim != 128) return 0;
  if (n_heads < 1 || n_kv < 0 || (long long)(n_heads + 2 * n_kv) * head_dim != N) return 0;
  if ((uintptr_t)q_out % 16 || ldq % 8 || ldq < (long long)n_heads * head_dim) return 0;
  if ((cos_table != nullptr) != (sin_table != nullptr) || (uintptr_t)cos_table % 16 || (uintptr_t)sin_table % 16) return 0;
  if (n_kv && (!k_pages || !v_pages || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16)) return 0;
  return 1;
}

// The QKV projection of a prompt portion with rotation and cache store in its epilogue (the pair
// kernel): A [M, K] and W [(n_heads + 2 n_kv) * head_dim, K] bfloat16; rotated queries go to
// q_out [M, ldq] (bfloat16), rotated keys and plain values to place slot_map[t] of the pages
// [page][n_kv][page_size][head_dim]; positions[t] selects the row of the tables
// [position][head_dim / 2] (null tables: no rotation).  n_kv == 0: W holds query heads only and
// nothing is stored.  tile: columns per tile, a multiple of head_dim up to 256.
LLMK_API int llmk_gemm_tc_qkv_rope(const void* A, const void* W, void* q_out, int M, int N, int K, long long lda,
                                   long long ldw, long long ldq, int tile, const float* cos_table,
                                   const float* sin_table, const int* positions, const int* slot_map, void* k_pages,
                                   void* v_pages, int n_heads, int n_kv, int head_dim, int page_size,
                                   cudaStream_t stream) {
  if (M == 0) return 0;
  LLMK_REQUIRE(llmk_gemm_tc_qkv_rope_supported(A, W, M, N, K, lda, ldw, q_out, ldq, cos_table, sin_table, k_pages, v_pages,
                                               n_heads, n_kv, head_dim),
               "gemm_tc_qkv_rope: needs bfloat16 rows of 16-byte multiples, a head size of 64 or 128 (got %d) and N = (%d + 2 * %d) heads",
               head_dim, n_heads, n_kv);
  LLMK_REQUIRE(tile >= head_dim && tile <= 256 && tile % head_dim == 0, "gemm_tc_qkv_rope: tile %d must be a multiple of the head size %d up to 256", tile, head_dim);
  LLMK_REQUIRE(positions && (n_kv == 0 || (slot_map && page_size > 0)), "gemm_tc_qkv_rope: positions, slot map and page size are needed");
  int rc = ensure_err_flag();
  if (rc) return rc;
  CUtensorMap mp, mq;
  if ((rc = get_map(&mp, A, M, K, lda, BP))) return rc;
  if ((rc = get_map(&mq, W, N, K, ldw, tile / 2))) return rc;
  RopeStore rs{cos_table, sin_table, positions, slot_map, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
               n_heads, n_kv, head_dim, page_size > 0 ? page_size : 1};
  return launch_pair<__nv_bfloat16, EPI_ROPE>(mp, mq, q_out, ldq, M, N, K, tile, rs, stream);
}

// Reads and clears the error word that a kernel sets when one of its waits gave up
// (1 = producer, 2 = MMA issuer, 3 = epilogue of the one-tile kernel; 4 to 6 the same of the
// persistent kernel, 7 to 9 of the pair kernel).  Synchronises the device.
LLMK_API int llmk_gemm_tc_take_error() {
  if (ensure_err_flag()) return 0;
  int v = 0;
  cudaMemcpy(&v, g_err_flag, sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(g_err_flag, 0, sizeof(int));
  return v;
}

// out[m, n] = sum over s of partials[s][m][n], in the order s = 0, 1, ...
template <typename TOut>
__global__ void reduce_partials_kernel(TOut* __restrict__ out, const float* __restrict__ partials, size_t mn, int splits) {
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < mn; i += (size_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partials[(size_t)s * mn + i];
    out[i] = from_f32<TOut>(acc);
  }
}

LLMK_API int llmk_reduce_partials(void* out, const float* partials, long long mn, int splits, int out_dtype,
                                  cudaStream_t stream) {
  if (mn == 0) return 0;
  size_t blocks = ((size_t)mn + 255) / 256;
  if (blocks > (size_t)llmk_sm_count() * 8) blocks = (size_t)llmk_sm_count() * 8;
  return dispatch_dtype(out_dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(reduce_partials_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, partials, (size_t)mn, splits);
    LLMK_LAUNCH_CHECK("reduce_partials");
  });
}
