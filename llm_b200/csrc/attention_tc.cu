// Paged grouped-query flash attention on the tcgen05 tensor cores (bfloat16, head size 64
// or 128), for prompt portions and anything else that brings several tokens per request.
//
// A CTA owns one query tile and one kv head.  The tile packs all query heads of the kv
// group: row r = (token r / G, head r % G), up to 128 rows, so every key and value that is
// fetched serves the whole group.  Per block of 128 keys (blocks start at absolute positions
// 0, 128, ...):
//   producer thread   TMA copies the block's pages of K and of V ([page, 64 dims] boxes with the
//                     128-byte swizzle) into two rings of two stages
//   MMA thread        S = Q K^T (tcgen05.mma, M = 128 rows, N = 128 keys) into tensor memory, for
//                     the next block as soon as the softmax warps hold the scores of this one in
//                     registers; after they have written P: O += P V (M = 128, N = head size),
//                     accumulated in tensor memory over all blocks
//   softmax warps     thread r owns row r = lane r of tensor memory: takes its 128 scores with
//                     tcgen05.ld, masks (causal, window), keeps a reference maximum and the sum
//                     in float32 (exp2 of pre-scaled scores) and writes P as bfloat16 into shared
//                     memory in the swizzled K-major layout that the second MMA reads.  The
//                     reference maximum only moves when the true maximum has grown by more than
//                     2^8 (P stays below 256, the sum stays exact in float32 terms); only then
//                     is the row of O in tensor memory rescaled (tcgen05.ld, multiply,
//                     tcgen05.st), which after the first blocks of a row is rare.  At the end
//                     the row of O is divided by the sum.
// Visible keys of a row at position p: max(0, p-window+1) .. p.  The reference's kernel is an
// mma.sync flash attention fixed to 32/4/64 (kernel/attention/attention_NH_32_NKV_4_HS_64.h);
// this one takes any head counts with group size up to 128.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BKV = 128;           // keys per block
constexpr int ROWS = 128;          // rows of a query tile = M of the MMAs
constexpr int THREADS = 192;       // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: softmax
constexpr int KV_STAGES = 2;

enum : int { ERR_Q = 11, ERR_KV = 12, ERR_S = 13, ERR_P = 14, ERR_PV = 15, ERR_ALIGN = 16 };

// MN-major shared-memory operand with the 128-byte swizzle: 64 elements of N are contiguous
// (128 bytes), rows of K are 128 bytes apart, groups of 8 rows 1024 bytes apart (stride byte
// offset), further blocks of 64 along N `lbo_bytes` apart (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Blackwell's three-input maximum and its two-wide float32 arithmetic halve the instruction
// count of the softmax's inner loops.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

template <int HS>
struct Smem {
  static constexpr int KB = HS / 64;                      // 64-dim blocks of a head
  static constexpr int Q_BYTES = ROWS * HS * 2;
  static constexpr int KV_BYTES = BKV * HS * 2;           // one of K or V, one stage
  static constexpr int P_BYTES = ROWS * BKV * 2;
  // No slack for alignment: with head size 64 two CTAs then fit on an SM and fill each other's
  // waits.  Dynamic shared memory starts 1024-byte aligned when a kernel has no static shared
  // memory; the kernel checks this and reports instead of running on a misaligned base.
  static constexpr int TOTAL = Q_BYTES + 2 * KV_STAGES * KV_BYTES + P_BYTES + 256 /* barriers */;
};

template <int HS>
__global__ void __launch_bounds__(THREADS, HS == 64 ? 2 : 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, long long out_stride,
                    const int* __restrict__ block_table, int table_width, const int* __restrict__ cu_tokens,
                    const int* __restrict__ kv_lens, int n_entries, int n_heads, int n_kv, int page_size, int n_pages,
                    int window, float scale_log2e, int* __restrict__ err_flag) {
  using S = Smem<HS>;
  constexpr int KB = S::KB;
  constexpr uint32_t TMEM_COLS = 256;                     // S: 128 columns, O_blk: HS columns
  constexpr uint32_t IDESC_QK = idesc_bf16_f32(ROWS, BKV);
  constexpr uint32_t IDESC_PV = idesc_bf16_f32(ROWS, HS) | (1u << 16);      // B is MN-major

  extern __shared__ __align__(1024) uint8_t smem[];
  const bool aligned = (smem_u32(smem) & 1023u) == 0;
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + S::Q_BYTES;                         // [stage][KB][128 keys][128 bytes]
  uint8_t* v_s = k_s + KV_STAGES * S::KV_BYTES;
  uint8_t* p_s = v_s + KV_STAGES * S::KV_BYTES;            // [2][128 rows][128 bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + S::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                             // [KV_STAGES]
  uint64_t* k_empty = k_full + KV_STAGES;
  uint64_t* v_full = k_empty + KV_STAGES;
  uint64_t* v_empty = v_full + KV_STAGES;
  uint64_t* s_full = v_empty + KV_STAGES;                  // MMA -> softmax: the scores of a block are in tensor memory
  uint64_t* s_free = s_full + 1;                           // softmax -> MMA: they are in registers now
  uint64_t* p_ready = s_free + 1;                          // softmax -> MMA: P is in shared memory (and O rescaled)
  uint64_t* pv_full = p_ready + 1;                         // MMA -> softmax: O holds the blocks so far, P may be overwritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_full + 1);
  int* tile_info = reinterpret_cast<int*>(tmem_slot + 1);  // entry, first row in the batch, tokens, first position

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.x % n_kv;                        // kv heads fastest: the heaviest tiles of every head start first
  const int group = n_heads / n_kv;
  const int tq = ROWS / group;                             // tokens per tile

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 128);
    mbar_init(p_ready, 128);
    mbar_init(pv_full, 1);
    fence_mbar_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  if (threadIdx.x == 0) {
    // which request and which of its tokens this tile covers; the tiles are handed out from the
    // back, so that the late tokens of long prompts (the most key blocks) start first
    int tile = (int)(gridDim.x / n_kv) - 1 - (int)(blockIdx.x / n_kv), entry = -1, t0 = 0, nt = 0, p0 = 0;
    for (int e = 0; e < n_entries; ++e) {
      const int n_e = cu_tokens[e + 1] - cu_tokens[e];
      const int tiles_e = (n_e + tq - 1) / tq;
      if (tile < tiles_e) {
        entry = e;
        t0 = cu_tokens[e] + tile * tq;
        nt = min(tq, n_e - tile * tq);
        p0 = kv_lens[e] - n_e + tile * tq;
        break;
      }
      tile -= tiles_e;
    }
    if (!aligned) { entry = -1; atomicExch(err_flag, ERR_ALIGN); }
    tile_info[0] = entry; tile_info[1] = t0; tile_info[2] = nt; tile_info[3] = p0;
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int entry = tile_info[0], t0 = tile_info[1], nt = tile_info[2], p0 = tile_info[3];

  if (entry >= 0) {
    const int p_last = p0 + nt - 1;
    const int lo_tile = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;   // lowest key any row sees
    const int kb_first = lo_tile / BKV, kb_last = p_last / BKV;
    const int n_blocks = kb_last - kb_first + 1;

    if (warp == 0) {
      // ---- producer: the whole warp.  A block of keys (or values) is pages_per_block * KB boxes;
      // looking up a page and issuing its copy costs a thread a few hundred cycles, so the lanes
      // issue one box each, after lane 0 has told the barrier how many bytes to expect ----
      if (lane == 0) {
        mbar_arrive_expect_tx(q_full, (uint32_t)(KB * group * tq * 128));
        for (int b = 0; b < KB; ++b) tma_load_3d(q_s + b * ROWS * 128, &map_q, b * 64, g * group, t0, q_full);
      }
      const int* table = block_table + (size_t)entry * table_width;
      const int pages_per_block = BKV / page_size;
      const int n_boxes = pages_per_block * KB;
      bool ok = true;
      for (int i = 0; i < n_blocks && ok; ++i) {
        const int s = i % KV_STAGES;
        const uint32_t free_parity = ((i / KV_STAGES) & 1) ^ 1;
        const int key0 = (kb_first + i) * BKV;
        for (int which = 0; which < 2 && ok; ++which) {           // keys first: the next scores need them early
          uint64_t* full = which ? &v_full[s] : &k_full[s];
          if (lane == 0) {
            ok = mbar_wait(which ? &v_empty[s] : &k_empty[s], free_parity);
            if (ok) mbar_arrive_expect_tx(full, S::KV_BYTES);
          }
          ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;         // also orders the lanes' copies after the announcement
          if (!ok) break;
          for (int box = lane; box < n_boxes; box += 32) {
            const int pg = box / KB, b = box % KB;
            int idx = key0 / page_size + pg;
            idx = idx < table_width ? idx : table_width - 1;
            int page = table[idx];
            page = page < 0 ? 0 : (page >= n_pages ? n_pages - 1 : page);     // pages past the request hold masked keys
            const int off = b * BKV * 128 + pg * page_size * 128;
            tma_load_3d((which ? v_s : k_s) + s * S::KV_BYTES + off, which ? &map_v : &map_k, b * 64, 0,
                        page * n_kv + g, full);
          }
        }
      }
      if (!ok && lane == 0) atomicExch(err_flag, ERR_KV);
    } else if (warp == 1) {
      if (lane == 0) {
        // ---- MMA issuer ----
        auto scores = [&](int i) {                                // S = Q K^T of block i
          const int s = i % KV_STAGES;
#pragma unroll
          for (int k = 0; k < HS / 16; ++k) {
            const uint32_t off = (k / 4) * (ROWS * 128) + (k % 4) * 32;
            const uint64_t da = smem_desc_sw128(smem_u32(q_s + off));
            const uint64_t db = smem_desc_sw128(smem_u32(k_s + s * S::KV_BYTES + off));
            mma_bf16(tmem_base, da, db, IDESC_QK, k != 0);
          }
          mma_commit(s_full);
          mma_commit(&k_empty[s]);
        };
        bool ok = mbar_wait(q_full, 0);
        if (!ok) atomicExch(err_flag, ERR_Q);
        if (ok) {
          ok = mbar_wait(&k_full[0], 0);
          if (!ok) atomicExch(err_flag, ERR_KV);
        }
        if (ok) {
          fence_after_sync();
          scores(0);
        }
        for (int i = 0; i < n_blocks && ok; ++i) {
          const int s = i % KV_STAGES;
          if (i + 1 < n_blocks) {
            // the scores of block i are in the softmax warps' registers: block i + 1 may overwrite them
            ok = mbar_wait(s_free, i & 1);
            if (!ok) { atomicExch(err_flag, ERR_S); break; }
            ok = mbar_wait(&k_full[(i + 1) % KV_STAGES], ((i + 1) / KV_STAGES) & 1);
            if (!ok) { atomicExch(err_flag, ERR_KV); break; }
            fence_after_sync();
            scores(i + 1);
          }
          // O += P V once the softmax warps have written P (and rescaled O where they had to)
          ok = mbar_wait(p_ready, i & 1);
          if (!ok) { atomicExch(err_flag, ERR_P); break; }
          ok = mbar_wait(&v_full[s], (i / KV_STAGES) & 1);
          if (!ok) { atomicExch(err_flag, ERR_KV); break; }
          fence_after_sync();
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k) {
            const uint64_t da = smem_desc_sw128(smem_u32(p_s + (k / 4) * (ROWS * 128) + (k % 4) * 32));
            const uint64_t db = smem_desc_sw128_mn(smem_u32(v_s + s * S::KV_BYTES + k * 16 * 128), BKV * 128);
            mma_bf16(tmem_base + BKV, da, db, IDESC_PV, (i | k) != 0);
          }
          mma_commit(pv_full);
          mma_commit(&v_empty[s]);
        }
      }
    } else {
      // ---- softmax and output: thread r owns row r ----
      constexpr float TAU = 8.f;                                  // how far the true maximum may run ahead of the reference
      const int quad = warp & 3;
      const int r = quad * 32 + lane;
      const int tok = r / group, head = r % group;
      const bool row_ok = tok < nt;
      const int pos = p0 + tok;
      const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
      float m_ref = -INFINITY, l = 0.f;
      bool ok = true;

      for (int i = 0; i < n_blocks; ++i) {
        const int key0 = (kb_first + i) * BKV;
        if (ok) ok = mbar_wait(s_full, i & 1);
        fence_after_sync();
        uint32_t raw[2][64];
        tmem_ld_x64(lane_addr, raw[0]);
        tmem_ld_x64(lane_addr + 64, raw[1]);
        tmem_ld_wait();
        fence_before_sync();
        mbar_arrive(s_free);
        // every row sees every key of the block when the block lies inside all windows and below all diagonals
        const bool full = (key0 + BKV - 1 <= p0) && (window <= 0 || key0 >= p_last - window + 1);
        // the row's maximum over the block.  The scale is positive, so it is taken over the raw
        // scores and scaled once.  Four running maxima (and sums below) keep the dependent chains short.
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (full) {
#pragma unroll
            for (int j = 0; j < 64; j += 2)
              mx[(j >> 1) & 3] = max3(mx[(j >> 1) & 3], __uint_as_float(raw[c][j]), __uint_as_float(raw[c][j + 1]));
          } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) {
              const int key = key0 + c * 64 + j;
              if (key <= pos && key >= lo) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(raw[c][j]));
            }
          }
        }
        const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2e;
        // move the reference only when the block's maximum is far above it (or it is the first
        // key this row sees: -inf + TAU is -inf)
        const bool moved = m_blk > m_ref + TAU;
        float alpha = 1.f;
        if (moved) {
          alpha = fast_exp2(m_ref - m_blk);                       // 0 while the reference is -inf
          m_ref = m_blk;
          l *= alpha;
        }
        bool pv_waited = false;
        if (i > 0 && __any_sync(0xffffffffu, moved)) {
          // O holds blocks 0 .. i-1 once their last product is done; rescale this warp's rows
          if (ok) ok = mbar_wait(pv_full, (i - 1) & 1);
          pv_waited = true;
          fence_after_sync();
#pragma unroll
          for (int c = 0; c < HS; c += 32) {
            uint32_t o[32];
            tmem_ld_x32(lane_addr + BKV + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st_x32(lane_addr + BKV + c, o);
          }
          tmem_st_wait();
        }
        const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;   // a row that sees nothing yet
        // P = exp2(score * scale - reference) as bfloat16 pairs, in place of the scores
        const uint64_t scale2 = pack_f32x2(scale_log2e, scale_log2e), neg_m2 = pack_f32x2(neg_m, neg_m);
        uint64_t ls2[4] = {0ull, 0ull, 0ull, 0ull};               // four pairs of running sums (0.f, 0.f)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float xa, xb;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(raw[c][2 * j]), __uint_as_float(raw[c][2 * j + 1])), scale2, neg_m2), xa, xb);
            float pa = fast_exp2(xa), pb = fast_exp2(xb);
            if (!full) {
              const int key = key0 + c * 64 + 2 * j;
              if (key > pos || key < lo) pa = 0.f;
              if (key + 1 > pos || key + 1 < lo) pb = 0.f;
            }
            ls2[j & 3] = add_f32x2(ls2[j & 3], pack_f32x2(pa, pb));
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(pa, pb);
            raw[c][j] = *reinterpret_cast<const uint32_t*>(&h2);
          }
        }
        {
          float a0, a1, b0, b1;
          unpack_f32x2(add_f32x2(ls2[0], ls2[1]), a0, a1);
          unpack_f32x2(add_f32x2(ls2[2], ls2[3]), b0, b1);
          l += (a0 + a1) + (b0 + b1);
        }
        if (i > 0 && !pv_waited && ok) ok = mbar_wait(pv_full, (i - 1) & 1);
#pragma unroll
        for (int cc = 0; cc < 16; ++cc) {
          const int c = cc / 8, q8 = cc % 8;
          uint8_t* dst = p_s + c * (ROWS * 128) + r * 128 + ((q8 ^ (r & 7)) * 16);
          *reinterpret_cast<uint4*>(dst) = make_uint4(raw[c][q8 * 4], raw[c][q8 * 4 + 1], raw[c][q8 * 4 + 2], raw[c][q8 * 4 + 3]);
        }
        fence_proxy_async();                  // the MMA reads P through the async proxy
        fence_before_sync();                  // and O, if it was rescaled, through tensor memory
        mbar_arrive(p_ready);
      }
      if (ok) ok = mbar_wait(pv_full, (n_blocks - 1) & 1);
      fence_after_sync();
      if (!ok && lane == 0) atomicExch(err_flag, ERR_S);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = out + (size_t)(t0 + tok) * out_stride + (size_t)(g * group + head) * HS;
#pragma unroll
      for (int c = 0; c < HS; c += 64) {
        uint32_t o[64];
        tmem_ld_x64(lane_addr + BKV + c, o);                       // the whole warp takes part, whatever its rows
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int d = 0; d < 64; d += 8) {
            uint4 u;
            __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(o[d]) * inv, __uint_as_float(o[d + 1]) * inv);
            __nv_bfloat162 b1 = __floats2bfloat162_rn(__uint_as_float(o[d + 2]) * inv, __uint_as_float(o[d + 3]) * inv);
            __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(o[d + 4]) * inv, __uint_as_float(o[d + 5]) * inv);
            __nv_bfloat162 b3 = __floats2bfloat162_rn(__uint_as_float(o[d + 6]) * inv, __uint_as_float(o[d + 7]) * inv);
            u.x = *reinterpret_cast<uint32_t*>(&b0); u.y = *reinterpret_cast<uint32_t*>(&b1);
            u.z = *reinterpret_cast<uint32_t*>(&b2); u.w = *reinterpret_cast<uint32_t*>(&b3);
            *reinterpret_cast<uint4*>(dst + c + d) = u;
          }
        }
      }
      fence_before_sync();
    }
  }

  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host -----------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn3() {
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

// bf16 tensor [d2][d1][d0] with d0 contiguous; boxes of [1 or b2][b1][64] with the 128-byte swizzle.
int encode_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
              uint64_t stride2_elems, uint32_t b1, uint32_t b2) {
  EncodeTiledFn fn = encode_fn3();
  if (!fn) return llmk_fail(-2, "cuTensorMapEncodeTiled is not available from the driver");
  if ((uintptr_t)base % 16 || (stride1_elems * 2) % 16 || (stride2_elems * 2) % 16)
    return llmk_fail(-1, "attention_tc: tensor bases and pitches must be multiples of 16 bytes");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_elems * 2, stride2_elems * 2};
  cuuint32_t box[3] = {64, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return llmk_fail(-2, "cuTensorMapEncodeTiled (3-D) failed with %d", (int)r);
  return 0;
}

struct Key3 {
  const void* base; uint64_t d0, d1, d2, s1, s2; uint32_t b1, b2;
  bool operator==(const Key3& o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s1 == o.s1 && s2 == o.s2 && b1 == o.b1 && b2 == o.b2;
  }
};
struct Key3Hash {
  size_t operator()(const Key3& k) const {
    size_t h = (size_t)k.base;
    for (uint64_t v : {k.d0, k.d1, k.d2, k.s1, k.s2, (uint64_t)k.b1, (uint64_t)k.b2}) h = h * 1000003u ^ v;
    return h;
  }
};
std::unordered_map<Key3, CUtensorMap, Key3Hash> g_maps3;
std::mutex g_maps3_mutex;

int get_map3(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2,
             uint32_t b1, uint32_t b2) {
  Key3 key{base, d0, d1, d2, s1, s2, b1, b2};
  std::lock_guard<std::mutex> lock(g_maps3_mutex);
  auto it = g_maps3.find(key);
  if (it == g_maps3.end()) {
    CUtensorMap m;
    int rc = encode_3d(&m, base, d0, d1, d2, s1, s2, b1, b2);
    if (rc) return rc;
    if (g_maps3.size() > 4096) g_maps3.clear();
    it = g_maps3.emplace(key, m).first;
  }
  *out = it->second;
  return 0;
}

int* g_attn_err = nullptr;

template <int HS>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, long long out_stride,
           const int* block_table, int table_width, const int* cu_tokens, const int* kv_lens, int n_entries,
           int max_tiles, int n_heads, int n_kv, int page_size, int n_pages, int window, float scale_log2e,
           cudaStream_t stream) {
  auto kern = attention_tc_kernel<HS>;
  constexpr int smem = Smem<HS>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return llmk_fail((int)e, "attention_tc: cannot set %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid(max_tiles * n_kv);
  launch_kernel(kern, grid, dim3(THREADS), (size_t)smem, stream, mq, mk, mv, (__nv_bfloat16*)out, out_stride, block_table,
                table_width, cu_tokens, kv_lens, n_entries, n_heads, n_kv, page_size, n_pages, window, scale_log2e, g_attn_err);
  LLMK_LAUNCH_CHECK("attention_tc");
}

}  // namespace

// Whether the tensor-core attention takes these sizes.
LLMK_API int llmk_attention_tc_supported(int n_heads, int n_kv, int head_dim, int page_size) {
  if (head_dim != 64 && head_dim != 128) return 0;
  if (n_kv <= 0 || n_heads % n_kv || n_heads / n_kv > ROWS) return 0;
  if (page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) return 0;
  return 1;
}

// q [n_tokens, q_stride] bf16 with head h at column h*head_dim; out likewise.  cu_tokens
// [entries + 1] are the entries' row offsets, kv_lens[e] the keys of entry e including its new
// tokens (which are already in the pages).  k_pages / v_pages [n_pages, n_kv, page_size, head_dim].
LLMK_API int llmk_attention_tc(void* out, long long out_stride, const void* q, long long q_stride, const void* k_pages,
                               const void* v_pages, int n_pages, const int* block_table, int table_width,
                               const int* cu_tokens, const int* kv_lens, int n_tokens, int n_entries, int n_heads,
                               int n_kv, int head_dim, int page_size, int window, float scale, cudaStream_t stream) {
  if (n_tokens == 0 || n_entries == 0) return 0;
  LLMK_REQUIRE(llmk_attention_tc_supported(n_heads, n_kv, head_dim, page_size),
               "attention_tc: needs head_dim 64 or 128, page_size 16/32/64/128 and at most %d query heads per kv head "
               "(got heads %d/%d, head_dim %d, page_size %d)", ROWS, n_heads, n_kv, head_dim, page_size);
  LLMK_REQUIRE(out_stride % 8 == 0 && (uintptr_t)out % 16 == 0, "attention_tc: out must have 16-byte aligned rows");
  g_attn_err = llmk_error_word(2);
  LLMK_REQUIRE(g_attn_err != nullptr, "attention_tc: cannot allocate the error word");
  const int group = n_heads / n_kv, tq = ROWS / group;
  const int max_tiles = (n_tokens + tq - 1) / tq + n_entries;
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = get_map3(&mq, q, head_dim, n_heads, n_tokens, head_dim, q_stride, group, tq))) return rc;
  if ((rc = get_map3(&mk, k_pages, head_dim, page_size, (uint64_t)n_pages * n_kv, head_dim, (uint64_t)page_size * head_dim, page_size, 1))) return rc;
  if ((rc = get_map3(&mv, v_pages, head_dim, page_size, (uint64_t)n_pages * n_kv, head_dim, (uint64_t)page_size * head_dim, page_size, 1))) return rc;
  const float scale_log2e = scale * 1.4426950408889634f;
  if (head_dim == 64)
    return launch<64>(mq, mk, mv, out, out_stride, block_table, table_width, cu_tokens, kv_lens, n_entries, max_tiles,
                      n_heads, n_kv, page_size, n_pages, window, scale_log2e, stream);
  return launch<128>(mq, mk, mv, out, out_stride, block_table, table_width, cu_tokens, kv_lens, n_entries, max_tiles,
                     n_heads, n_kv, page_size, n_pages, window, scale_log2e, stream);
}

// The code the attention kernel left when one of its bounded waits gave up (0 = none).
LLMK_API int llmk_attention_tc_take_error() {
  g_attn_err = llmk_error_word(2);
  if (!g_attn_err) return 0;
  int v = 0;
  cudaMemcpy(&v, g_attn_err, sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(g_attn_err, 0, sizeof(int));
  return v;
}
