// Decode attention on the warp-level tensor cores (bfloat16, head size 64 or 128).
//
// The same split of the keys into ranges, one CTA per (range, kv head, request), and the same
// merge by the last CTA as the CUDA-core kernel in attention_decode.cu; what differs is the
// inside of a range.  The query heads of the kv group are the rows of an m16n8k16 MMA (up to 16
// per pass): one instruction scores 8 keys for all of them, so the arithmetic per key no longer
// grows with the group size.  Each of the four warps works alone on tiles of 32 keys, without
// block-wide barriers: keys and values are staged per warp through one to three stages of shared
// memory with cp.async (with several, the next tiles are in flight while one is computed) and read back with ldmatrix
// (values transposed); scores, maxima, sums and the output are float32, P is rounded to
// bfloat16 for the second MMA as in the prompt kernel.  A single decoded token has no use for
// the 128-row tcgen05 MMA; this is the tensor path that fits 8 to 16 rows.
#pragma once

#include "common.cuh"
#include "tcgen05.cuh"

namespace decode_mma {

constexpr int THREADS = 128;
constexpr int ROWS = 16;         // query heads per pass
constexpr int TILE = 32;         // keys per warp tile
constexpr int COUNTER_WORDS = 4096;

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;                      // 0: the 16 bytes are filled with zeros
  // .cg: the keys and values stream through once; they need no place in L1
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Wait until at most n of the most recent groups are still in flight (n = 0..3).
__device__ __forceinline__ void cp_async_wait_pending(int n) {
  if (n <= 0) asm volatile("cp.async.wait_all;" ::: "memory");
  else if (n == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
  else if (n == 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
  else asm volatile("cp.async.wait_group 3;" ::: "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Two adjacent values (idx even): of a tensor, or the sums in split order of split-K partial
// results, with the loads of up to eight splits in flight (a split past the last adds zero).
__device__ __forceinline__ float2 sum2(const MaybePartial<__nv_bfloat16>& s, size_t idx) {
  if (s.parts) {
    float2 acc = make_float2(0.f, 0.f);
    for (int sp = 0; sp < s.splits; sp += 8) {
      float2 t[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        t[u] = sp + u < s.splits ? *reinterpret_cast<const float2*>(s.parts + (size_t)(sp + u) * s.split_stride + idx)
                                 : make_float2(0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 8; ++u) { acc.x += t[u].x; acc.y += t[u].y; }
    }
    return acc;
  }
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(s.direct + idx));
}

// Scratch layout as in attention_decode.cu: counters, then ml [entries, heads, splits, 2] (the
// maximum here in the base-2 domain of the pre-scaled scores), then o [entries, heads, splits, HS].
//
// CLUSTER: the CTAs of the ranges of one (request, kv head) form a thread-block cluster (2 to 8
// along blockIdx.x).  They hand their results to the first CTA through distributed shared memory
// (into its dynamic shared memory, (ranges - 1) x heads of a pass x HS floats) and that CTA
// merges them: no scratch in global memory, no fence, no counter.  Every CTA arrives at a first
// cluster barrier when it starts and waits for it only before it writes to the first CTA, which
// must be running by then; a second barrier publishes the writes.
//
// FUSED: the kernel takes the row of the QKV product itself (a tensor or unsummed split-K
// partial results) instead of rotated queries.  Every CTA sums and rotates its group's queries
// into shared memory; the CTA whose range holds the newest position also sums and rotates that
// token's key, stores key and value in the pages (unless the layer reads another layer's
// pages) and keeps a copy in shared memory for its own use.  This replaces the separate
// rotate-and-store kernel of a decode step.
struct FusedQkv {
  MaybePartial<__nv_bfloat16> src;     // [entries, src_stride]: q heads, then k heads, then v heads
  long long src_stride;
  const float* cos_table;              // [max_position, HS/2], or null: nothing is rotated
  const float* sin_table;
  int write_kv;
};

template <int HS, bool CLUSTER, bool FUSED, bool LIGHT = false>
__global__ void __launch_bounds__(THREADS, (LIGHT && HS == 64) ? 4 : 1)
decode_attention_mma_kernel(__nv_bfloat16* __restrict__ out, long long out_stride, float* __restrict__ scratch,
                            const __nv_bfloat16* __restrict__ q, long long q_stride,
                            __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                            const int* __restrict__ block_table, int table_width, const int* __restrict__ kv_lens,
                            int n_heads, int n_kv, int page_size, int window, float scale_log2e, int splits,
                            FusedQkv fused) {
  constexpr int KS = HS / 16;                  // k-steps of Q K^T
  constexpr int DT = HS / 8;                   // 8-wide tiles of the output row
  constexpr int CH = HS / 8;                   // 16-byte chunks of a row
  constexpr int V_BYTES = TILE * HS * 2;       // one tile of keys, or of values
  // Stages of (keys, values) per warp.  Several let the next tiles fly while one is computed,
  // which pays for long ranges (three where two CTAs then still fit on an SM).  A cluster is only
  // formed for short ranges on a small grid; there one stage keeps the CTA small enough to become
  // resident beside the CTAs of the kernel before it, which is what lets its early requests
  // overlap that kernel.  LIGHT: one stage without a cluster, for grids of more CTAs than fit on
  // the SMs at once with deep stages: more CTAs per SM then keep as many bytes in flight, and
  // the grid runs as one wave instead of two.
  constexpr int NST = (CLUSTER || LIGHT) ? 1 : (HS == 64 ? 3 : 2);
  constexpr int WARP_BYTES = NST * 2 * V_BYTES;
  constexpr int RANGES = CLUSTER ? 8 : 64;     // most ranges that a merge in shared memory takes
  static_assert(4 * WARP_BYTES >= 4 * ROWS * HS * 4, "the warps' results are merged in the stage buffers");
  extern __shared__ __align__(128) uint8_t vbuf[];            // 4 warps x WARP_BYTES, then (CLUSTER) the receive buffer
  __shared__ float wm_s[4][ROWS], wl_s[4][ROWS];
  __shared__ float w_s[ROWS][RANGES], l_in[ROWS][RANGES];    // merge: per (head, range)
  __shared__ int last_s;
  __shared__ __align__(16) __nv_bfloat16 q_s[FUSED ? ROWS * HS : 8];
  __shared__ __align__(16) __nv_bfloat16 kv_new_s[FUSED ? 2 * HS : 8];    // the newest key, then the newest value

  float* recv_s = reinterpret_cast<float*>(vbuf + 4 * WARP_BYTES);   // CLUSTER: what the other ranges send to the first CTA
  pdl_launch_dependents();
  if (CLUSTER) tc::cluster_arrive();
  const int split = blockIdx.x, g = blockIdx.y, e = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = n_heads / n_kv;
  // a length beyond the entry's table row is cut to what the row can hold; an entry without keys
  // gets zeros (every range of it sees the same length and leaves here, so nobody waits for anybody)
  const int n_held = min(kv_lens[e], table_width * page_size);
  if (n_held <= 0) {
    pdl_wait();
    if (split == 0)
      for (int i = tid; i < group * HS; i += THREADS)
        out[(size_t)e * out_stride + (size_t)g * group * HS + i] = __float2bfloat16_rn(0.f);
    return;
  }
  const int pos = n_held - 1;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n_keys = pos - lo + 1;
  int chunk = (n_keys + splits - 1) / splits;
  chunk = (chunk + TILE - 1) / TILE * TILE;
  const int k_begin = lo + split * chunk;
  const int k_end = min(pos + 1, k_begin + chunk);
  const int* table = block_table + (size_t)e * table_width;
  const int qrow = lane >> 2, qcol = (lane & 3) * 2;
  // the row of key k of this request and kv head in the pages.  The page size is a power of two
  // (the host sends other sizes to the CUDA-core kernel): a division per row of every tile would
  // cost more than the tile's arithmetic
  const int page_shift = __ffs(page_size) - 1;
  auto row_of = [&](int k) -> size_t {
    return ((((size_t)table[k >> page_shift] * n_kv + g) << page_shift) + (k & (page_size - 1))) * HS;
  };
  uint8_t* w_buf = vbuf + warp * WARP_BYTES;                 // stage st: keys at st * 2 * V_BYTES, values V_BYTES further
  const uint32_t w_addr = (uint32_t)__cvta_generic_to_shared(w_buf);
  const int t_first = k_begin + warp * TILE;                // this warp's first tile
  const int n_tiles = t_first < k_end ? (k_end - t_first + 4 * TILE - 1) / (4 * TILE) : 0;

  // request a tile's keys and values: 32 rows of CH chunks each, swizzled by the row; rows past
  // the range are filled with zeros
  auto stage_tile = [&](int j) {
    const int t = t_first + j * 4 * TILE;
    const uint32_t dst = w_addr + (j % NST) * 2 * V_BYTES;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int idx = i * 32 + lane;
      const int kl = idx / CH, c = idx % CH;
      const int kp = t + kl;
      const bool valid = kp < k_end;
      const int kq = valid ? kp : k_begin;
      const size_t row = row_of(kq);
      const int cs = (c & ~7) | ((c ^ kl) & 7);
      cp_async_16(dst + kl * (HS * 2) + cs * 16, k_pages + row + c * 8, valid);
      cp_async_16(dst + V_BYTES + kl * (HS * 2) + cs * 16, v_pages + row + c * 8, valid);
    }
    cp_async_commit();
  };

  // Lengths and block tables were copied before the step's first kernel, and every key but the
  // newest was stored by an earlier step.  So each warp requests its first tiles, and the
  // CTA asks the rest of its range into L2, while the kernels before this one still run; only
  // the queries and the newest key and value (stored by a kernel of this step, or by this one)
  // have to wait.  The newest row of a tile is replaced after it has landed, see below.
#pragma unroll
  for (int j = 0; j < NST; ++j)
    if (j < n_tiles) stage_tile(j);
  {
    // at most 32 MB over the whole grid: asking for more than L2 keeps evicts the lines before
    // they are used and fetches them from memory twice (long ranges stream through the stages)
    constexpr int LINES = HS * 2 / 128;                    // 128-byte lines per row
    const int ask_limit = (32 << 20) / (int)(gridDim.x * gridDim.y * gridDim.z) / (HS * 4);
    const int n_rows = min(ask_limit, max(0, k_end - k_begin - NST * 4 * TILE));
    for (int i = tid; i < n_rows * LINES * 2; i += THREADS) {
      const int which = i & 1, line = (i >> 1) % LINES, kp = k_begin + NST * 4 * TILE + (i >> 1) / LINES;
      const size_t row = row_of(kp);
      const __nv_bfloat16* src = (which ? v_pages : k_pages) + row + line * 64;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
    }
  }
  pdl_wait();

  // the newest key and value are read, once they are valid, from the pages, or from this CTA's
  // shared copy when it computes them itself
  const size_t new_row = row_of(pos);
  const bool owner = FUSED && fused.write_kv && k_begin <= pos && pos < k_end;
  // FUSED, owner: the last threads sum the newest token's key (two pairs each) and value (two
  // elements each); their loads are issued here and used after the queries' loads below
  const int kv_item = THREADS - 1 - tid;
  const bool does_k = owner && kv_item < HS / 4, does_v = owner && !does_k && kv_item < HS / 4 + HS / 2;
  float2 nk_a = make_float2(0.f, 0.f), nk_b = nk_a, nv = nk_a;
  if constexpr (FUSED) {
    const size_t src_row = (size_t)e * fused.src_stride;
    if (does_k) {
      const size_t h = src_row + (size_t)(n_heads + g) * HS + kv_item * 2;
      nk_a = sum2(fused.src, h);
      nk_b = sum2(fused.src, h + HS / 2);
    } else if (does_v) {
      nv = sum2(fused.src, src_row + (size_t)(n_heads + n_kv + g) * HS + (kv_item - HS / 4) * 2);
    }
  }

  int* counters = reinterpret_cast<int*>(scratch);
  float* partial_ml = scratch + COUNTER_WORDS;
  float* partial_o = partial_ml + (size_t)gridDim.z * n_heads * splits * 2;

  // a range without keys only reports in; in a cluster it still has to meet the others at the barriers
  for (int h0 = 0; h0 < group && (CLUSTER || k_begin < k_end); h0 += ROWS) {
    const int nh = min(ROWS, group - h0);
    const int head0 = g * group + h0;
    // Q fragments: rows = heads, straight from global memory (4 bytes = 2 bf16 per load)
    uint32_t qf[KS][4];
    const __nv_bfloat16* q0;
    if constexpr (FUSED) {
      // the pass's queries: summed, rotated, rounded to bfloat16 into shared memory; two pairs
      // (i, i+1 and their partners half a head further) per item, all loads issued before any use
      constexpr int ITEMS = ROWS * (HS / 4) / THREADS;
      float2 qa[ITEMS], qb[ITEMS], qc[ITEMS], qs[ITEMS];
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const int idx = tid + it * THREADS;
        if (idx < nh * (HS / 4)) {
          const int h = idx / (HS / 4), i = (idx % (HS / 4)) * 2;
          const size_t src = (size_t)e * fused.src_stride + (size_t)(head0 + h) * HS + i;
          qa[it] = sum2(fused.src, src);
          qb[it] = sum2(fused.src, src + HS / 2);
          qc[it] = fused.cos_table ? *reinterpret_cast<const float2*>(fused.cos_table + (size_t)pos * (HS / 2) + i) : make_float2(1.f, 1.f);
          qs[it] = fused.cos_table ? *reinterpret_cast<const float2*>(fused.sin_table + (size_t)pos * (HS / 2) + i) : make_float2(0.f, 0.f);
        }
      }
      if (h0 == 0 && (does_k || does_v)) {
        if (does_k) {
          const int i = kv_item * 2;
          const float2 c = fused.cos_table ? *reinterpret_cast<const float2*>(fused.cos_table + (size_t)pos * (HS / 2) + i) : make_float2(1.f, 1.f);
          const float2 sn = fused.cos_table ? *reinterpret_cast<const float2*>(fused.sin_table + (size_t)pos * (HS / 2) + i) : make_float2(0.f, 0.f);
          const __nv_bfloat162 ya = __floats2bfloat162_rn(nk_a.x * c.x - nk_b.x * sn.x, nk_a.y * c.y - nk_b.y * sn.y);
          const __nv_bfloat162 yb = __floats2bfloat162_rn(nk_a.x * sn.x + nk_b.x * c.x, nk_a.y * sn.y + nk_b.y * c.y);
          *reinterpret_cast<__nv_bfloat162*>(k_pages + new_row + i) = ya;
          *reinterpret_cast<__nv_bfloat162*>(k_pages + new_row + i + HS / 2) = yb;
          *reinterpret_cast<__nv_bfloat162*>(kv_new_s + i) = ya;
          *reinterpret_cast<__nv_bfloat162*>(kv_new_s + i + HS / 2) = yb;
        } else {
          const int d = (kv_item - HS / 4) * 2;
          const __nv_bfloat162 x = __floats2bfloat162_rn(nv.x, nv.y);
          *reinterpret_cast<__nv_bfloat162*>(v_pages + new_row + d) = x;
          *reinterpret_cast<__nv_bfloat162*>(kv_new_s + HS + d) = x;
        }
      }
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const int idx = tid + it * THREADS;
        if (idx < nh * (HS / 4)) {
          const int h = idx / (HS / 4), i = (idx % (HS / 4)) * 2;
          const float2 a = qa[it], b = qb[it], c = qc[it], sn = qs[it];
          *reinterpret_cast<__nv_bfloat162*>(q_s + h * HS + i) = __floats2bfloat162_rn(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y);
          *reinterpret_cast<__nv_bfloat162*>(q_s + h * HS + i + HS / 2) = __floats2bfloat162_rn(a.x * sn.x + b.x * c.x, a.y * sn.y + b.y * c.y);
        }
      }
      __syncthreads();                  // queries, and the owner's newest key and value, in shared memory
      q0 = q_s + qrow * HS;
    } else {
      q0 = q + (size_t)e * q_stride + (size_t)(head0 + qrow) * HS;
    }
    {
      // Q fragments: rows = heads (4 bytes = 2 bf16 per load)
      const __nv_bfloat16* q1 = q0 + 8 * HS;
      const bool r0 = qrow < nh, r1 = qrow + 8 < nh;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        qf[ks][0] = r0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + qcol) : 0u;
        qf[ks][1] = r1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + qcol) : 0u;
        qf[ks][2] = r0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + qcol) : 0u;
        qf[ks][3] = r1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + qcol) : 0u;
      }
    }
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;        // rows qrow and qrow + 8 (l: this lane's share)

    if (h0 > 0) {                                                 // a later pass requests its tiles again
#pragma unroll
      for (int j = 0; j < NST; ++j)
        if (j < n_tiles) stage_tile(j);
    }
    for (int j = 0; j < n_tiles; ++j) {
      const int t = t_first + j * 4 * TILE;
      const uint32_t k_addr = w_addr + (j % NST) * 2 * V_BYTES, v_addr = k_addr + V_BYTES;
      cp_async_wait_pending(min(n_tiles - 1 - j, NST - 1));          // tile j has landed; later ones may still fly
      __syncwarp();
      if (pos < t + TILE) {                                       // pos >= t: the range ends at pos
        // The newest row: not valid when the tile was requested early (before the wait for the
        // kernels of this step).  It is taken from the CTA's own copy, or from L2.
        if (lane < 2 * CH) {
          const int c = lane % CH, kl = pos - t;
          const bool is_v = lane >= CH;
          const uint4 row = owner ? *reinterpret_cast<const uint4*>(kv_new_s + (is_v ? HS : 0) + c * 8)
                                  : __ldcg(reinterpret_cast<const uint4*>((is_v ? v_pages : k_pages) + new_row + c * 8));
          const int cs = (c & ~7) | ((c ^ kl) & 7);
          *reinterpret_cast<uint4*>(w_buf + (j % NST) * 2 * V_BYTES + (is_v ? V_BYTES : 0) + kl * (HS * 2) + cs * 16) = row;
        }
        __syncwarp();
      }
      // ---- S = Q K^T: K fragments with ldmatrix, two k-steps per instruction ----
      float s[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        const int kl = nt * 8 + (lane & 7);
#pragma unroll
        for (int k2 = 0; k2 < KS / 2; ++k2) {
          const int c = k2 * 4 + (lane >> 3);
          const int cs = (c & ~7) | ((c ^ kl) & 7);
          uint32_t kb[4];
          ldmatrix_x4(kb, k_addr + kl * (HS * 2) + cs * 16);
          mma_16816(s[nt], qf[2 * k2], kb[0], kb[1]);
          mma_16816(s[nt], qf[2 * k2 + 1], kb[2], kb[3]);
        }
      }
      // ---- scale, mask the keys past the range, running maximum and sum ----
      float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int kp = t + nt * 8 + qcol;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const bool valid = kp + j < k_end;
          s[nt][j] = valid ? s[nt][j] * scale_log2e : -INFINITY;
          s[nt][2 + j] = valid ? s[nt][2 + j] * scale_log2e : -INFINITY;
          t0 = fmaxf(t0, s[nt][j]);
          t1 = fmaxf(t1, s[nt][2 + j]);
        }
      }
      t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
      t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
      const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);          // finite: the tile holds at least one key
      const float a0 = ex2(m0 - n0), a1 = ex2(m1 - n1);
      m0 = n0; m1 = n1;
      l0 *= a0; l1 *= a1;
#pragma unroll
      for (int d = 0; d < DT; ++d) { o[d][0] *= a0; o[d][1] *= a0; o[d][2] *= a1; o[d][3] *= a1; }
      uint32_t pf[2][4];                                          // P as the A operand of two k-steps of 16 keys
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float p0 = ex2(s[nt][0] - n0), p1 = ex2(s[nt][1] - n0);
        const float p2 = ex2(s[nt][2] - n1), p3 = ex2(s[nt][3] - n1);
        l0 += p0 + p1;
        l1 += p2 + p3;
        pf[nt >> 1][(nt & 1) * 2] = pack2(p0, p1);
        pf[nt >> 1][(nt & 1) * 2 + 1] = pack2(p2, p3);
      }
      // ---- O += P V ----
      const int mid = lane >> 3, r8 = lane & 7;
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const int kl = kk * 16 + (mid & 1) * 8 + r8;               // the key whose row this lane points at
#pragma unroll
        for (int dp = 0; dp < DT / 2; ++dp) {
          const int c = dp * 2 + (mid >> 1);
          const int cs = (c & ~7) | ((c ^ kl) & 7);
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, v_addr + kl * (HS * 2) + cs * 16);
          mma_16816(o[dp * 2], pf[kk], vb[0], vb[1]);
          mma_16816(o[dp * 2 + 1], pf[kk], vb[2], vb[3]);
        }
      }
      __syncwarp();                                               // the stage is consumed before it is requested again
      if (j + NST < n_tiles) stage_tile(j + NST);
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // ---- the four warps' results, merged in their order ----
    __syncthreads();                                              // every warp is done with its staged values
    float* wo = reinterpret_cast<float*>(vbuf) + (size_t)warp * ROWS * HS;
    if ((lane & 3) == 0) {
      wm_s[warp][qrow] = m0; wm_s[warp][qrow + 8] = m1;
      wl_s[warp][qrow] = l0; wl_s[warp][qrow + 8] = l1;
    }
#pragma unroll
    for (int d = 0; d < DT; ++d) {
      *reinterpret_cast<float2*>(wo + qrow * HS + d * 8 + qcol) = make_float2(o[d][0], o[d][1]);
      *reinterpret_cast<float2*>(wo + (qrow + 8) * HS + d * 8 + qcol) = make_float2(o[d][2], o[d][3]);
    }
    __syncthreads();
    constexpr int PER = ROWS * HS / THREADS;                      // output elements per thread
    float racc[CLUSTER ? PER : 1], rm[CLUSTER ? PER : 1], rl[CLUSTER ? PER : 1];
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int i = tid + k * THREADS;
      if (i >= nh * HS) break;
      const int h = i / HS, d = i % HS;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) m = fmaxf(m, wm_s[w][h]);
      float l = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = wm_s[w][h];
        if (mw > -INFINITY) {
          const float f = ex2(mw - m);
          l += f * wl_s[w][h];
          acc += f * reinterpret_cast<const float*>(vbuf)[((size_t)w * ROWS + h) * HS + d];
        }
      }
      if (CLUSTER) {
        racc[CLUSTER ? k : 0] = acc; rm[CLUSTER ? k : 0] = m; rl[CLUSTER ? k : 0] = l;
      } else if (splits == 1) {
        out[(size_t)e * out_stride + (size_t)(head0 + h) * HS + d] = __float2bfloat16_rn(acc / l);
      } else {
        partial_o[(((size_t)e * n_heads + head0 + h) * splits + split) * HS + d] = acc;
        if (d == 0) {
          float* ml = partial_ml + (((size_t)e * n_heads + head0 + h) * splits + split) * 2;
          ml[0] = m;
          ml[1] = l;
        }
      }
    }
    if (CLUSTER) {
      // every CTA of the cluster has its share in registers; the first CTA runs once the barrier
      // of the kernel's start has completed (a later pass: once it has merged the pass before)
      const uint32_t rank = tc::cluster_ctarank();
      const uint32_t slots = tc::map_to_cta((uint32_t)__cvta_generic_to_shared(recv_s), 0);
      const uint32_t m_remote = tc::map_to_cta((uint32_t)__cvta_generic_to_shared(&w_s[0][0]), 0);
      const uint32_t l_remote = tc::map_to_cta((uint32_t)__cvta_generic_to_shared(&l_in[0][0]), 0);
      if (h0 == 0) tc::cluster_wait(); else tc::cluster_sync();
#pragma unroll
      for (int k = 0; k < PER; ++k) {
        const int i = tid + k * THREADS;
        if (i >= nh * HS) break;
        const int h = i / HS, d = i % HS;
        if (rank != 0 && rm[k] > -INFINITY) tc::st_cluster_f32(slots + (uint32_t)(((rank - 1) * nh + h) * HS + d) * 4u, racc[k]);
        if (d == 0) {
          tc::st_cluster_f32(m_remote + (uint32_t)(h * RANGES + rank) * 4u, rm[k]);
          tc::st_cluster_f32(l_remote + (uint32_t)(h * RANGES + rank) * 4u, rl[k]);
        }
      }
      tc::cluster_sync();
      if (rank == 0) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
          const int i = tid + k * THREADS;
          if (i >= nh * HS) break;
          const int h = i / HS, d = i % HS;
          float m = -INFINITY;
          for (int r = 0; r < splits; ++r) m = fmaxf(m, w_s[h][r]);
          float l = 0.f, acc = 0.f;
          for (int r = 0; r < splits; ++r) {                      // in the order of the ranges
            const float mr = w_s[h][r];
            if (mr > -INFINITY) {
              const float f = ex2(mr - m);
              l += f * l_in[h][r];
              acc += f * (r == 0 ? racc[k] : recv_s[((size_t)(r - 1) * nh + h) * HS + d]);
            }
          }
          out[(size_t)e * out_stride + (size_t)(head0 + h) * HS + d] = __float2bfloat16_rn(acc / l);
        }
      }
    }
    __syncthreads();                                              // vbuf is reused by the next pass
  }
  if (splits == 1 || CLUSTER) return;

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
  const int n_active = min(splits, (n_keys + chunk - 1) / chunk);
  for (int h0 = 0; h0 < group; h0 += ROWS) {
    const int nh = min(ROWS, group - h0);
    const size_t base0 = ((size_t)e * n_heads + g * group + h0) * splits;
    __syncthreads();
    for (int i = tid; i < nh * n_active; i += THREADS) {
      const int h = i / n_active, sp = i % n_active;
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(partial_ml + (base0 + (size_t)h * splits + sp) * 2));
      w_s[h][sp] = ml.x;
      l_in[h][sp] = ml.y;
    }
    __syncthreads();
    if (tid < nh) {
      float m = -INFINITY;
      for (int sp = 0; sp < n_active; ++sp) m = fmaxf(m, w_s[tid][sp]);
      float l = 0.f;
      for (int sp = 0; sp < n_active; ++sp) {
        const float f = ex2(w_s[tid][sp] - m);
        l += f * l_in[tid][sp];
        w_s[tid][sp] = f;
      }
      const float inv = 1.f / l;
      for (int sp = 0; sp < n_active; ++sp) w_s[tid][sp] *= inv;
    }
    __syncthreads();
    for (int i = tid; i < nh * HS; i += THREADS) {
      const int h = i / HS, d = i % HS;
      const float* po = partial_o + (base0 + (size_t)h * splits) * HS + d;
      float acc = 0.f;
      int sp = 0;
      for (; sp + 8 <= n_active; sp += 8) {
        float ov[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) ov[u] = __ldcg(po + (size_t)(sp + u) * HS);
#pragma unroll
        for (int u = 0; u < 8; ++u) acc = fmaf(w_s[h][sp + u], ov[u], acc);
      }
      for (; sp < n_active; ++sp) acc = fmaf(w_s[h][sp], __ldcg(po + (size_t)sp * HS), acc);
      out[(size_t)e * out_stride + (size_t)(g * group + h0 + h) * HS + d] = __float2bfloat16_rn(acc);
    }
  }
  if (tid == 0) counters[e * n_kv + g] = 0;
}

}  // namespace decode_mma
