// Causal grouped-query attention for prefill on the fifth-generation tensor cores
// (bfloat16, head size 64 or 128): scores and the per-tile output products are tcgen05
// MMAs with accumulators in tensor memory (TMEM), operands brought in by TMA with the
// 128-byte swizzle, softmax in float32 by one thread per query row.
//
// A CTA owns up to 128 query rows of one KV head: the G query heads of the group for
// floor(128 / G) consecutive tokens of one sequence (row r = token q0 + r / G, head
// kh*G + r % G; rows past that are idle), so a key tile is fetched once for the whole group.  Keys are visited page by page (a
// page of the cache, 64 keys of one KV head, is one TMA box).  For tile j:
//
//   MMA warp      S_j = Q K_j^T           (M 128, N 64, K = head size)   -> TMEM
//   softmax warps read S_j from TMEM (a row per thread), scale, mask, maximum
//                 and sum, P_j = 2^(s - m) in bfloat16 -> TMEM (a row per lane, two
//                 keys per 32-bit column: the layout of an MMA's first operand there)
//   MMA warp      O += P_j V_j            (M 128, N head size, K 64; P read from TMEM,
//                 V from shared memory)                                  -> TMEM
//
// The output accumulates in TMEM over all tiles and comes to registers once, at
// the end.  m is the reference the exponentials of a row are taken against; it
// follows the row's running maximum lazily: only when the maximum has outgrown it
// by more than 2^8 is m moved and the row of O (and the running sum) rescaled by
// 2^(m_old - m_new), a read-modify-write of TMEM that the softmax threads do
// between two products.  Until then P is at most 2^8, well inside bfloat16 and
// float32.  S and P are double-buffered in TMEM, so the MMAs of
// tile j+1 run while tile j's softmax does; two CTAs share an SM.  Scores are
// (q.k) * scale, key s visible to position p iff lo <= s <= p
// (alpacca/model.py:457-467).
//
// Every mbarrier wait is bounded (see gemm_tc.cu): on a timeout the thread records a
// code in `status` and all roles fall through to the end, where TMEM is given back.
#include "common.cuh"
#include "launch.cuh"
#include <cuda.h>

#define AT_ROWS 128
#define AT_KEYS 64
// Head size HD is 64 or 128.  A row of 64 elements (128 bytes, the width of the swizzle) is one row of a
// "panel"; an operand with 128 elements per row is two panels one after the other (Q: 16 KB each, a K
// or V tile: 8 KB each).  Two CTAs share an SM: 256 TMEM columns each (HD 64: S twice, O, P twice; HD
// 128: S twice with P over the first half of each, O 128 columns) and at most 113 KB of shared memory
// (HD 64: Q and four stages of K and V, 80 KB; HD 128: Q and two stages, 96 KB).
template <int HD> struct AtShape {
  static constexpr int PANELS = HD / 64;
  static constexpr int STAGES = HD == 64 ? 4 : 2;
  static constexpr uint32_t O_COL = 128;
  __host__ __device__ static constexpr uint32_t p_col(int j) { return HD == 64 ? 192u + (j & 1) * 32u : (j & 1) * 64u; }
};
#define AT_THREADS 192
#define AT_SPIN (1u << 20)
#define AT_LOG2E 1.4426950408889634f

__device__ __forceinline__ uint32_t at_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(at_smem(bar)), "r"(count));
}
__device__ __forceinline__ void at_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(at_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = at_smem(bar);
  for (uint32_t i = 0; i < AT_SPIN; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void at_tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void at_tma_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
// operand tiles with 128-byte rows and the 128-byte swizzle; groups of 8 rows are 1024 bytes apart.
// The same descriptor serves a K-major operand (rows = M or N index, the 128 bytes run along k) and
// an MN-major one (rows = k index, the 128 bytes run along n); which it is says the instruction.
__device__ __forceinline__ uint64_t at_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// an MN-major operand wider than one panel: `panel_bytes` from one 64-column panel to the next
__device__ __forceinline__ uint64_t at_desc_mn(uint32_t saddr, uint32_t panel_bytes) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(panel_bytes >> 4) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void at_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the first operand in TMEM (P: a row per lane, two bfloat16 per column)
__device__ __forceinline__ void at_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void at_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ void at_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void at_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void at_st16(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
}
__device__ __forceinline__ void at_st16u(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void at_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
#define AT_LAZY 8.0f     // a row's reference follows its maximum when that is more than 2^8 ahead
__device__ __forceinline__ float at_exp2(float x) {      // 2^x, the hardware approximation (2^-inf = 0)
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HD> struct AtSmem {
  // all tiles are panels of [rows][64] bfloat16 = 128-byte rows, 1024-byte aligned
  static constexpr int Q_PANEL = AT_ROWS * 128;
  static constexpr int KV_PANEL = AT_KEYS * 128;
  static constexpr int Q_BYTES = AtShape<HD>::PANELS * Q_PANEL;
  static constexpr int KV_BYTES = AtShape<HD>::PANELS * KV_PANEL;      // one K or V tile
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = Q_OFF + Q_BYTES;                               // [STAGES][K | V]
  static constexpr int BAR_OFF = KV_OFF + AtShape<HD>::STAGES * 2 * KV_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                            const int* __restrict__ block_table, int table_width, const int* __restrict__ tok_pos,
                            const int* __restrict__ cu_q, const int* __restrict__ tile_seq,
                            const int* __restrict__ tile_q0, int H, int K, float scale_log2, int window,
                            int tokens_per_tile, int* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  using Sm = AtSmem<HD>;
  using Sh = AtShape<HD>;
  constexpr int AT_STAGES = Sh::STAGES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + Sm::BAR_OFF);
  uint64_t* q_full = bars;                       // 1
  uint64_t* kv_full = bars + 1;                  // STAGES
  uint64_t* kv_empty = kv_full + AT_STAGES;      // STAGES
  uint64_t* s_full = kv_empty + AT_STAGES;       // 2
  uint64_t* p_full = s_full + 2;                 // 2
  uint64_t* o_done = p_full + 2;                 // 1: completes once per product O += P_j V_j
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = H / K;
  // CTAs start in the order of their index: tile by tile (the longest key ranges first), the KV heads
  // of a tile side by side, so that no long tile is left for the end (by KV head first, the last heads'
  // longest tiles started when most of the device had run dry: 53 us per layer instead of 44)
  const int tile = blockIdx.x / K, kh = blockIdx.x - tile * K;
  const int b = tile_seq[tile];
  const int q0 = tile_q0[tile];
  const int q_end = cu_q[b + 1];
  const int n_tok = min(tokens_per_tile, q_end - q0);
  const int n_rows = n_tok * G;

  if (threadIdx.x == 0) {
    at_bar_init(q_full, 1);
    for (int s = 0; s < AT_STAGES; ++s) { at_bar_init(kv_full + s, 1); at_bar_init(kv_empty + s, 1); }
    for (int i = 0; i < 2; ++i) { at_bar_init(s_full + i, 1); at_bar_init(p_full + i, 128); }
    at_bar_init(o_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(at_smem(tmem_slot)), "r"(256));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: S tiles at 0 and 64, O from 128; P tiles (32 columns each) at 192 and 224 (HD 64)
  // or over the first half of their S tile (HD 128)
  pdl_wait();
  pdl_trigger();

  const int pos_first = tok_pos[q0], pos_last = tok_pos[q0 + n_tok - 1];
  const int kb_begin = (window > 0 && pos_first - window + 1 > 0) ? (pos_first - window + 1) / AT_KEYS : 0;
  const int kb_end = pos_last / AT_KEYS + 1;
  const int n_tiles = kb_end - kb_begin;
  const int* bt = block_table + (size_t)b * table_width;

  if (warp == 0) {
    if (lane == 0) {
      // the box holds tokens_per_tile x G rows (all of them counted, also where they lie past the
      // sequence's end and are filled with zeros); rows of the tile past the box are never written:
      // whatever they hold stays in their own rows of S, P and O, which nobody stores
      at_expect_tx(q_full, Sh::PANELS * tokens_per_tile * G * 128);
      for (int p = 0; p < Sh::PANELS; ++p)
        at_tma_3d(base + Sm::Q_OFF + p * Sm::Q_PANEL, &map_q, p * 64, kh * G, q0, q_full);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % AT_STAGES;
        if (j >= AT_STAGES && !at_wait(kv_empty + s, ((j / AT_STAGES) - 1) & 1)) { atomicExch(status, 11); break; }
        const int row = (bt[kb_begin + j] * K + kh) * AT_KEYS;
        unsigned char* dst = base + Sm::KV_OFF + s * 2 * Sm::KV_BYTES;
        at_expect_tx(kv_full + s, 2 * Sm::KV_BYTES);
        for (int p = 0; p < Sh::PANELS; ++p) {
          at_tma_2d(dst + p * Sm::KV_PANEL, &map_k, p * 64, row, kv_full + s);
          at_tma_2d(dst + Sm::KV_BYTES + p * Sm::KV_PANEL, &map_v, p * 64, row, kv_full + s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // S = Q K^T: A = Q (K-major), B = K tile (K-major), N = 64
      constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_KEYS >> 3) << 17) |
                                   ((uint32_t)(AT_ROWS >> 4) << 24);
      // T = P V: A = P (K-major over keys), B = V tile [key][d] = MN-major, N = head size
      constexpr uint32_t idesc_t = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                                   ((uint32_t)(AT_ROWS >> 4) << 24);
      const uint32_t q_addr = at_smem(base + Sm::Q_OFF);
      bool ok = at_wait(q_full, 0);
      if (!ok) atomicExch(status, 12);
      auto issue_s = [&](int j) {
        const int s = j % AT_STAGES;
        if (!at_wait(kv_full + s, (j / AT_STAGES) & 1)) { atomicExch(status, 13); ok = false; return; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k_addr = at_smem(base + Sm::KV_OFF + s * 2 * Sm::KV_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)      // 16 elements of the head per MMA: 32 bytes along a panel's rows
          at_mma(tmem + (j & 1) * 64, at_desc(q_addr + (k >> 2) * Sm::Q_PANEL + (k & 3) * 32),
                 at_desc(k_addr + (k >> 2) * Sm::KV_PANEL + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
        at_commit(s_full + (j & 1));
      };
      if (ok && n_tiles > 0) issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) issue_s(j + 1);        // the next tile's scores run while this tile's softmax does
        if (!ok) break;
        if (!at_wait(p_full + (j & 1), (j >> 1) & 1)) { atomicExch(status, 14); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int s = j % AT_STAGES;
        const uint32_t v_addr = at_smem(base + Sm::KV_OFF + s * 2 * Sm::KV_BYTES + Sm::KV_BYTES);
#pragma unroll
        for (int k = 0; k < AT_KEYS / 16; ++k)     // 16 keys per MMA: 8 columns of P, 2 groups of 8 V rows
          at_mma_ts(tmem + Sh::O_COL, tmem + Sh::p_col(j) + k * 8, at_desc_mn(v_addr + k * 2048, Sm::KV_PANEL), idesc_t,
                    (j > 0 || k > 0) ? 1u : 0u);
        at_commit(o_done);
        at_commit(kv_empty + s);                   // K and V of this stage are read when these MMAs are done
      }
    }
  } else {
    // softmax warps 2..5: TMEM lanes 32 * (warp % 4) ..; thread = query row
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const bool row_ok = r < n_rows;
    const int BIG = 0x3fffffff;
    int pos = BIG, lo = 0;
    if (row_ok) {
      pos = tok_pos[q0 + r / G];
      lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    }
    float m_ref = -INFINITY, l_run = 0.f;       // the row's reference and its sum of 2^(s - m_ref)
    bool ok = true;

    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!at_wait(s_full + (j & 1), (j >> 1) & 1)) { atomicExch(status, 16); ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float sc[AT_KEYS];
#pragma unroll
      for (int c0 = 0; c0 < AT_KEYS; c0 += 16) at_ld16(tmem + lane_base + (j & 1) * 64 + c0, sc + c0);
      at_ld_wait();
      const int key0 = (kb_begin + j) * AT_KEYS;
      const bool need_mask = (key0 + AT_KEYS - 1 > pos_first) || (window > 0);
      // the maximum is taken on the raw scores (the scale is positive), and scale and shift ride in
      // the exponent's fused multiply-add: p = 2^(s * scale - m)
      // four running maxima (and below four running sums) keep the dependent chains short
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < AT_KEYS; ++c)
          if (key0 + c > pos || key0 + c < lo) sc[c] = -INFINITY;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < AT_KEYS; c += 4) {
        mx4[0] = fmaxf(mx4[0], sc[c]);
        mx4[1] = fmaxf(mx4[1], sc[c + 1]);
        mx4[2] = fmaxf(mx4[2], sc[c + 2]);
        mx4[3] = fmaxf(mx4[3], sc[c + 3]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      // move the reference only when the maximum has outgrown it by a lot (or there was none yet)
      const bool move = (mx > m_ref + AT_LAZY) || (m_ref == -INFINITY && mx > -INFINITY);
      float corr = 1.f;
      if (move) {
        corr = (m_ref == -INFINITY) ? 0.f : at_exp2(m_ref - mx);
        m_ref = mx;
        l_run *= corr;
      }
      if (j > 0 && __any_sync(0xffffffffu, move)) {
        // rescale this warp's rows of O in TMEM, after the product before this tile has landed there
        if (!at_wait(o_done, (j - 1) & 1)) { atomicExch(status, 15); ok = false; }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          float t[32];
          at_ld16(tmem + lane_base + Sh::O_COL + c0, t);
          at_ld16(tmem + lane_base + Sh::O_COL + c0 + 16, t + 16);
          at_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) t[c] *= corr;
          at_st16(tmem + lane_base + Sh::O_COL + c0, t);
          at_st16(tmem + lane_base + Sh::O_COL + c0 + 16, t + 16);
        }
        at_st_wait();
      }
      const float sub = (m_ref == -INFINITY) ? 0.f : m_ref;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[AT_KEYS / 2];
#pragma unroll
      for (int c = 0; c < AT_KEYS; c += 4) {
        const float p0 = at_exp2(fmaf(sc[c], scale_log2, -sub)), p1 = at_exp2(fmaf(sc[c + 1], scale_log2, -sub));
        const float p2 = at_exp2(fmaf(sc[c + 2], scale_log2, -sub)), p3 = at_exp2(fmaf(sc[c + 3], scale_log2, -sub));
        sum4[0] += p0; sum4[1] += p1; sum4[2] += p2; sum4[3] += p3;
        __nv_bfloat162 pa = __floats2bfloat162_rn(p0, p1), pb = __floats2bfloat162_rn(p2, p3);
        packed[c >> 1] = *reinterpret_cast<uint32_t*>(&pa);
        packed[(c >> 1) + 1] = *reinterpret_cast<uint32_t*>(&pb);
      }
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // P row: 32 columns of this thread's lane (two keys each)
      at_st16u(tmem + lane_base + Sh::p_col(j), packed);
      at_st16u(tmem + lane_base + Sh::p_col(j) + 16, packed + 16);
      at_st_wait();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      at_arrive(p_full + (j & 1));
    }
    if (ok && n_tiles > 0) {
      if (!at_wait(o_done, (n_tiles - 1) & 1)) { atomicExch(status, 17); ok = false; }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* dst = out + ((size_t)(q0 + r / G) * H + kh * G + r % G) * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        float t[32];
        if (n_tiles > 0) {
          at_ld16(tmem + lane_base + Sh::O_COL + c0, t);
          at_ld16(tmem + lane_base + Sh::O_COL + c0 + 16, t + 16);
          at_ld_wait();
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) t[c] = 0.f;
        }
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 pr = __floats2bfloat162_rn(t[c + 2 * e] * inv, t[c + 2 * e + 1] * inv);
              w[e] = *reinterpret_cast<uint32_t*>(&pr);
            }
            *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256));
  }
}

// ---------------------------------------------------------------------------
typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AtEncodeFn at_encode_fn() {
  static AtEncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<AtEncodeFn>(p);
  }
  return fn;
}
static int* at_status_word() {
  static int* p[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!p[dev]) {
    if (cudaMalloc(&p[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p[dev], 0, sizeof(int));
  }
  return p[dev];
}
AB_API int ab_attention_tc_status() {
  int* p = at_status_word();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(p, 0, sizeof(int));
  return v;
}

// 1 if this kernel takes the shape (head size 64 or 128, up to 128 query heads per KV head), else 0
AB_API int ab_attention_prefill_tc_supports(int H, int K, int D) {
  if ((D != 64 && D != 128) || K <= 0 || H % K) return 0;
  return H / K <= AT_ROWS ? 1 : 0;
}

// qkv [n_tokens, (H+2K)*D] (q part read), out [n_tokens, H*D], cache pages [n_pages, K, 64, D].
// tile_seq / tile_q0: the tiles of floor(128 / G) tokens (sequence, first packed token), as for the mma kernel.
AB_API int ab_attention_prefill_tc(const void* qkv, int n_tokens, void* out, const void* k_pages, const void* v_pages,
                                   int n_pages, const int* block_table, int table_width, const int* tok_pos,
                                   const int* cu_q, const int* tile_seq, const int* tile_q0, int n_tiles, int H,
                                   int K, int D, float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return AB_OK;
  if (!ab_attention_prefill_tc_supports(H, K, D) || (long long)n_tiles * K > 0x7fffffffLL) return AB_BAD_ARG;
  AtEncodeFn enc = at_encode_fn();
  int* status = at_status_word();
  if (!enc || !status) return AB_BAD_ARG;
  const int G = H / K, tpt = AT_ROWS / G;
  CUtensorMap mq, mk, mv;
  {
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)(H + 2 * K), (cuuint64_t)n_tokens};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)(H + 2 * K) * D * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)tpt};          // one panel: 64 elements of the head
    cuuint32_t elem[3] = {1, 1, 1};
    if (enc(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(qkv), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return AB_BAD_ARG;
  }
  for (int which = 0; which < 2; ++which) {
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)n_pages * K * AT_KEYS};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, AT_KEYS};
    cuuint32_t elem[2] = {1, 1};
    if (enc(which ? &mv : &mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(which ? v_pages : k_pages),
            dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return AB_BAD_ARG;
  }
  cudaError_t e;
#define AT_GO(HDV)                                                                                                   \
  {                                                                                                                 \
    e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HDV>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                             AtSmem<HDV>::TOTAL);                                                                   \
    if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;                                                              \
    e = ab_launch(attention_prefill_tc_kernel<HDV>, dim3((unsigned)n_tiles * K), dim3(AT_THREADS), (size_t)AtSmem<HDV>::TOTAL, \
                  stream, mq, mk, mv, (bf16*)out, block_table, table_width, tok_pos, cu_q, tile_seq, tile_q0, H, K, \
                  scale * AT_LOG2E, window, tpt, status);                                                           \
  }
  if (D == 64) AT_GO(64) else AT_GO(128)
#undef AT_GO
  if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;
  return ab_launch_status();
}
