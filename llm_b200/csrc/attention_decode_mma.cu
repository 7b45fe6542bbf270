// Host side of the warp-level tensor-core decode attention (attention_decode_mma.cuh): the
// launcher, the entry point for queries that are already rotated, and the fused entry point
// that also rotates and stores.  Part of the tensor-core library; the CUDA-core kernel for all
// other sizes and for float32 is in attention_decode.cu.
#include "common.cuh"
#include "attention_decode_mma.cuh"

namespace {

template <bool FUSED>
int launch_decode_mma(void* out, long long out_stride, const void* q, long long q_stride, const void* k_pages,
                      const void* v_pages, const int* block_table, int table_width, const int* kv_lens,
                      int n_entries, int n_heads, int n_kv, int head_dim, int page_size, float scale, int window,
                      int splits, int max_keys, float* scratch, decode_mma::FusedQkv fused, cudaStream_t stream) {
  dim3 grid(splits, n_kv, n_entries);
  const float scale_log2e = scale * 1.4426950408889634f;
  const int group_rows = n_heads / n_kv < decode_mma::ROWS ? n_heads / n_kv : decode_mma::ROWS;
  // 2 to 8 ranges whose shares fit the first CTA's receive buffer, and a grid of at most two
  // waves: merge inside a cluster, no scratch.  (Measured at 64 requests, 512 CTAs: 30 us with
  // clusters against 23 us with the counter-based merge; at 8 requests 9.3 us against 13.5 us.)
  constexpr int RECV_LIMIT = 64 * 1024;
  const int recv_bytes = (splits - 1) * group_rows * head_dim * 4;
  // Only for short ranges (up to 512 keys of the longest request: max_keys, or what the table
  // holds): a cluster's CTA has one stage, which is right when a range is a tile or two per warp
  // and the merge is what counts; a long range wants the deep stages.
  const long long most_keys = max_keys > 0 ? max_keys : (long long)table_width * page_size;
  const long long range_keys = (most_keys + splits - 1) / splits;
  const bool cluster = splits >= 2 && splits <= 8 && (long long)splits * n_kv * n_entries <= 2 * llmk_sm_count() &&
                       recv_bytes <= RECV_LIMIT && range_keys <= 512;
  // Without a cluster: deep stages (three at head size 64, else two) while the whole grid fits on
  // the SMs at once with them (two CTAs per SM at head size 64, one at 128); else the variant
  // with one stage, which at head size 64 is also held to 128 registers so that four CTAs share
  // an SM and the grid still runs as one wave where it can (128 requests x 4 kv heads at 640
  // keys: 22.9 us against 28.0 us).
  const long long ctas = (long long)splits * n_kv * n_entries;
  const bool light = !cluster && ctas > (long long)(head_dim == 64 ? 2 : 1) * llmk_sm_count();
  // per warp its stages of a tile of keys and a tile of values: NST in the kernel
  const int stage_bytes = 4 * ((cluster || light) ? 1 : head_dim == 64 ? 3 : 2) * 2 * decode_mma::TILE * head_dim * 2;
  using Kernel = decltype(&decode_mma::decode_attention_mma_kernel<64, false, FUSED>);
  const Kernel kern = head_dim == 64
      ? (cluster ? decode_mma::decode_attention_mma_kernel<64, true, FUSED>
                 : light ? decode_mma::decode_attention_mma_kernel<64, false, FUSED, true> : decode_mma::decode_attention_mma_kernel<64, false, FUSED>)
      : (cluster ? decode_mma::decode_attention_mma_kernel<128, true, FUSED>
                 : light ? decode_mma::decode_attention_mma_kernel<128, false, FUSED, true> : decode_mma::decode_attention_mma_kernel<128, false, FUSED>);
  static bool configured[2][3] = {{false, false, false}, {false, false, false}};
  const int variant = cluster ? 1 : light ? 2 : 0;
  if (!configured[head_dim == 128][variant]) {
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, stage_bytes + (cluster ? RECV_LIMIT : 0));
    if (err != cudaSuccess) return llmk_fail((int)err, "attention_decode: cannot set the shared memory size: %s", cudaGetErrorString(err));
    configured[head_dim == 128][variant] = true;
  }
  if (cluster) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(decode_mma::THREADS);
    cfg.dynamicSmemBytes = (size_t)(stage_bytes + recv_bytes);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = llmk_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kern, (__nv_bfloat16*)out, out_stride, scratch, (const __nv_bfloat16*)q, q_stride,
                       (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table, table_width, kv_lens, n_heads,
                       n_kv, page_size, window, scale_log2e, splits, fused);
  } else {
    launch_kernel(kern, grid, dim3(decode_mma::THREADS), (size_t)stage_bytes, stream, (__nv_bfloat16*)out, out_stride, scratch,
                  (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table,
                  table_width, kv_lens, n_heads, n_kv, page_size, window, scale_log2e, splits, fused);
  }
  LLMK_LAUNCH_CHECK("attention_decode_mma");
}

}  // namespace

// Whether llmk_paged_attention_decode_mma takes these sizes: bfloat16 with a head size of 64 or
// 128, pages of a power of two, rows of q that start on 4-byte boundaries.
LLMK_API int llmk_paged_attention_decode_mma_supported(const void* q, long long q_stride, int head_dim, int page_size,
                                                       int dtype) {
  return dtype == LLMK_BF16 && (head_dim == 64 || head_dim == 128) && q_stride % 2 == 0 && (uintptr_t)q % 4 == 0 &&
         page_size > 0 && (page_size & (page_size - 1)) == 0;
}

// As llmk_paged_attention_decode (same arguments, same scratch), on the warp-level tensor cores:
// the query heads of a group as rows of the MMAs.  max_keys: an upper bound of kv_lens that the
// host knows (0: what a row of the table holds); it only picks between variants of the kernel.
LLMK_API int llmk_paged_attention_decode_mma(void* out, long long out_stride, const void* q, long long q_stride,
                                             const void* k_pages, const void* v_pages, const int* block_table,
                                             int table_width, const int* kv_lens, int n_entries, int n_heads, int n_kv,
                                             int head_dim, int page_size, int window, float scale, int splits,
                                             float* scratch, int dtype, int max_keys, cudaStream_t stream) {
  if (n_entries == 0) return 0;
  LLMK_REQUIRE(llmk_paged_attention_decode_mma_supported(q, q_stride, head_dim, page_size, dtype),
               "attention_decode_mma: needs bfloat16, a head size of 64 or 128 (got %d) and pages of a power of two (got %d)",
               head_dim, page_size);
  LLMK_REQUIRE(n_kv > 0 && n_heads % n_kv == 0, "attention_decode_mma: %d query heads do not divide into %d kv heads", n_heads, n_kv);
  LLMK_REQUIRE(splits >= 1 && splits <= 64, "attention_decode_mma: splits %d must be 1 to 64", splits);
  LLMK_REQUIRE(n_kv <= 65535 && n_entries <= 65535, "attention_decode_mma: grid too large");
  LLMK_REQUIRE((long long)n_entries * n_kv <= decode_mma::COUNTER_WORDS, "attention_decode_mma: %d entries x %d kv heads exceed %d counters",
               n_entries, n_kv, decode_mma::COUNTER_WORDS);
  LLMK_REQUIRE(window >= 0, "attention_decode_mma: bad window %d", window);
  return launch_decode_mma<false>(out, out_stride, q, q_stride, k_pages, v_pages, block_table, table_width, kv_lens,
                                  n_entries, n_heads, n_kv, head_dim, page_size, scale, window, splits, max_keys, scratch,
                                  decode_mma::FusedQkv{}, stream);
}

// Whether the fused rotate-store-attend kernel takes these sizes and pointers.
LLMK_API int llmk_decode_attention_fused_supported(const void* qkv, const float* partials, long long split_stride,
                                                   long long src_stride, const float* cos_table,
                                                   const float* sin_table, int head_dim, int dtype) {
  if (dtype != LLMK_BF16 || (head_dim != 64 && head_dim != 128)) return 0;
  if ((qkv != nullptr) == (partials != nullptr)) return 0;
  decode_mma::FusedQkv f{{(const __nv_bfloat16*)qkv, partials, 1, split_stride}, src_stride, cos_table, sin_table, 1};
  if (!f.src.vector_ok() || src_stride % 8) return 0;
  if ((uintptr_t)cos_table % 16 || (uintptr_t)sin_table % 16 || ((cos_table != nullptr) != (sin_table != nullptr))) return 0;
  return 1;
}

// A decode step's rotation, cache store and attention in one kernel (bfloat16, head size 64 or
// 128).  Row e of the source holds entry e's q heads, k heads and v heads (the k and v heads
// only when write_kv != 0): a tensor qkv [entries, src_stride] or the float32 partial results
// [qkv_splits][entries][src_stride] of a split-K product.  kv_lens[e] counts the new token, whose
// position is kv_lens[e] - 1; its rotated key and its value are stored at that position's place
// in the entry's block table.  Scratch and splits as for llmk_paged_attention_decode.
LLMK_API int llmk_decode_attention_fused(void* out, long long out_stride, const void* qkv, const float* partials,
                                         int qkv_splits, long long split_stride, long long src_stride,
                                         const float* cos_table, const float* sin_table, void* k_pages,
                                         void* v_pages, const int* block_table, int table_width, const int* kv_lens,
                                         int n_entries, int n_heads, int n_kv, int head_dim, int page_size,
                                         int window, float scale, int splits, int write_kv, float* scratch,
                                         int max_keys, cudaStream_t stream) {
  if (n_entries == 0) return 0;
  LLMK_REQUIRE(llmk_decode_attention_fused_supported(qkv, partials, split_stride, src_stride, cos_table, sin_table, head_dim, LLMK_BF16),
               "decode_attention_fused: needs bfloat16, a head size of 64 or 128 (got %d) and 16-byte aligned rows", head_dim);
  LLMK_REQUIRE(n_kv > 0 && n_heads % n_kv == 0, "decode_attention_fused: %d query heads do not divide into %d kv heads", n_heads, n_kv);
  LLMK_REQUIRE(splits >= 1 && splits <= 64, "decode_attention_fused: splits %d must be 1 to 64", splits);
  LLMK_REQUIRE(n_kv <= 65535 && n_entries <= 65535, "decode_attention_fused: grid too large");
  LLMK_REQUIRE((long long)n_entries * n_kv <= decode_mma::COUNTER_WORDS, "decode_attention_fused: %d entries x %d kv heads exceed %d counters",
               n_entries, n_kv, decode_mma::COUNTER_WORDS);
  LLMK_REQUIRE(page_size > 0 && (page_size & (page_size - 1)) == 0 && window >= 0,
               "decode_attention_fused: the page size %d must be a power of two, the window %d not negative", page_size, window);
  LLMK_REQUIRE(src_stride >= (long long)(n_heads + (write_kv ? 2 * n_kv : 0)) * head_dim,
               "decode_attention_fused: a row of %lld values does not hold the heads", src_stride);
  decode_mma::FusedQkv f{{(const __nv_bfloat16*)qkv, partials, qkv_splits, split_stride}, src_stride, cos_table, sin_table, write_kv};
  return launch_decode_mma<true>(out, out_stride, nullptr, 0, k_pages, v_pages, block_table, table_width, kv_lens,
                                 n_entries, n_heads, n_kv, head_dim, page_size, scale, window, splits, max_keys, scratch, f, stream);
}

