// Decode attention that streams the paged cache through a ring of shared-memory stages.
//
// One new token per sequence attends to its sequence's cached keys (causal grouped-query attention,
// alpacca/model.py:447-467: score = (q.k) * scale over the keys lo <= s <= pos, softmax, sum of v).
// The kernel of attention_mma.cu fetches a run of keys per warp, waits, attends, and fetches again:
// simple, and best for a few short sequences, but the memory system idles while the warps compute.
// With many sequences or long contexts the cache is most of what a decode step reads, and this
// kernel is built to keep it streaming:
//
//   - a page of the cache (64 keys of one KV head, K and V) is one stage of a ring in shared memory.
//     One thread (the producer) asks the TMA unit for whole pages, up to STAGES (2 to 12) ahead of the warps that
//     use them: `cp.async.bulk.tensor` with the 128-byte swizzle, completion counted by an mbarrier
//     per stage.  No thread spends instructions on addresses or waits on loads of its own;
//   - four consumer warps take 16 keys of each page.  As in attention_mma.cu the KEYS are the 16 rows
//     of the tensor-core tile and the (up to 8) query heads of the group its 8 columns (S^T = K Q^T,
//     O^T = V^T P^T), so no row of a tile is padding.  A warp rescales its running sums only when a
//     head's maximum has grown, which after the first pages is rare;
//   - work is cut evenly: a CTA takes (sequence, KV head, tile of 8 heads, chunk of `pages_per_cta`
//     pages); chunks past a sequence's end leave at once, so unequal sequences give CTAs of
//     equal size.  The chunks of one (sequence, head) are merged in chunk order, by the CTA that
//     arrives last (through scratch memory) or inside a thread-block cluster (through shared memory);
//   - the position rotation of q and k and the append of this step's k, v to the cache happen here
//     (`fuse`), as in attention_mma.cu.
//
// Head sizes 64 and 128 (rows of 128 bytes per swizzled panel); other sizes take attention_mma.cu.
// Every wait on an mbarrier is bounded: after AS_SPIN tries the kernel records a code in `status`,
// all roles fall through to the end and the output of that CTA is not valid (the host reads the
// status where it synchronises).
#include "attention_common.cuh"
#include "launch.cuh"
#include <cooperative_groups.h>
#include <cuda.h>

#define AS_CONSUMERS 4
#define AS_THREADS ((AS_CONSUMERS + 1) * 32)
#define AS_SPIN (1u << 20)
#define AS_PANEL (PAGE * 128)     // bytes of 64 rows x 64 bfloat16

__device__ __forceinline__ void as_bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void as_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void as_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool as_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < AS_SPIN; ++i) {
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
__device__ __forceinline__ void as_tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void as_consumer_sync() {      // the 128 consumer threads only
  asm volatile("bar.sync 1, %0;" ::"n"(AS_CONSUMERS * 32) : "memory");
}

// byte offset of 16-byte chunk `c` (8 elements) of row `r` inside a tile of HD/64 swizzled panels
__device__ __forceinline__ uint32_t as_off(int r, int c) {
  return (uint32_t)((c >> 3) * AS_PANEL + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

template <int HD>
struct StreamState {
  float o[HD / 16][4];   // O^T[d = 16 dm + g (+8)] of heads 2t, 2t+1
  float m[2];            // running maximum of score * scale * log2(e), per head
  float l[2];            // this thread's part of the running sum
};

// 16 keys (rows r0 .. r0+15 of the stage's K and V tiles) against the group's heads.
template <int HD>
__device__ __forceinline__ void attend_tile16(StreamState<HD>& st, const uint32_t (&qb)[HD / 16][2], uint32_t k_tile,
                                              uint32_t v_tile, int r0, float scale_log2, int key0, int pos, int lo) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int a_row = r0 + (lane & 7) + ((lane >> 3) & 1) * 8, a_chunk = lane >> 4;
  float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int kd = 0; kd < HD / 16; ++kd) {
    uint32_t a0, a1, a2, a3;
    ldmatrix_x4(a0, a1, a2, a3, k_tile + as_off(a_row, kd * 2 + a_chunk));
    mma_bf16(s, a0, a1, a2, a3, qb[kd][0], qb[kd][1]);
  }
  const int ka = key0 + g, kb = ka + 8;
  const bool oka = ka <= pos && ka >= lo, okb = kb <= pos && kb >= lo;
  s[0] = oka ? s[0] * scale_log2 : -INFINITY;
  s[1] = oka ? s[1] * scale_log2 : -INFINITY;
  s[2] = okb ? s[2] * scale_log2 : -INFINITY;
  s[3] = okb ? s[3] * scale_log2 : -INFINITY;
  float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
  // a head's 16 keys are spread over the lanes' g: bits 2..4 of the lane
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
  }
  const float mn0 = fmaxf(st.m[0], mx0), mn1 = fmaxf(st.m[1], mx1);
  if (__any_sync(0xffffffffu, mn0 > st.m[0] || mn1 > st.m[1])) {
    // a maximum grew: bring the sums to the new reference (2^(-inf - x) = 0 clears an empty state)
    const float c0 = (mn0 == -INFINITY) ? 1.f : fast_exp2(st.m[0] - mn0), c1 = (mn1 == -INFINITY) ? 1.f : fast_exp2(st.m[1] - mn1);
    st.l[0] *= c0;
    st.l[1] *= c1;
#pragma unroll
    for (int dm = 0; dm < HD / 16; ++dm) {
      st.o[dm][0] *= c0;
      st.o[dm][1] *= c1;
      st.o[dm][2] *= c0;
      st.o[dm][3] *= c1;
    }
    st.m[0] = mn0;
    st.m[1] = mn1;
  }
  const float sub0 = (mn0 == -INFINITY) ? 0.f : mn0, sub1 = (mn1 == -INFINITY) ? 0.f : mn1;
  s[0] = fast_exp2(s[0] - sub0);
  s[1] = fast_exp2(s[1] - sub1);
  s[2] = fast_exp2(s[2] - sub0);
  s[3] = fast_exp2(s[3] - sub1);
  st.l[0] += s[0] + s[2];
  st.l[1] += s[1] + s[3];
  // O^T += V^T P^T; P^T as the second operand is the transposed accumulator of S^T
  const uint32_t b0 = movmatrix_trans(pack_bf16(s[0], s[1]));
  const uint32_t b1 = movmatrix_trans(pack_bf16(s[2], s[3]));
  const int v_row = r0 + (lane & 7) + (lane >> 4) * 8, v_chunk = (lane >> 3) & 1;
#pragma unroll
  for (int dm = 0; dm < HD / 16; ++dm) {
    uint32_t a0, a1, a2, a3;
    ldmatrix_x4_trans(a0, a1, a2, a3, v_tile + as_off(v_row, dm * 2 + v_chunk));
    mma_bf16(st.o[dm], a0, a1, a2, a3, b0, b1);
  }
}

template <int HD, int STAGES> struct StreamSmem {
  static constexpr int TILE = (HD / 64) * AS_PANEL;            // one K or V tile of a page
  static constexpr int STAGE = 2 * TILE;
  static constexpr int RING = STAGES * STAGE;
  static constexpr int PITCH = HD + 8;                         // q rows and this step's k, v (bfloat16)
  static constexpr int Q_OFF = RING;                           // [8][PITCH] q, [2][PITCH] new k, v
  static constexpr int BAR_OFF = Q_OFF + ((10 * PITCH * 2 + 15) / 16) * 16;
  static constexpr int MERGE = (AS_CONSUMERS * 8 * (HD + 6) + 8 * (HD + 2)) * 4;   // over the ring, when it is done
  static constexpr int TOTAL = 1024 + BAR_OFF + 2 * STAGES * 8 + 16;
  static_assert(MERGE <= RING, "the warps' results are merged in the ring's memory");
};

// merge: 0 = one chunk per (sequence, head): the CTA stores the result; 1 = the chunks are the CTAs
// of a cluster; 2 = through scratch memory, the CTA that arrives last merges.
// fuse: as in attention_mma.cu (0: q rotated and this step's k, v in the cache already; 1: this kernel
// rotates q; 2: it rotates q and k and appends k, v to the cache).
template <int HD, int STAGES>
__global__ void __launch_bounds__(AS_THREADS)
attention_stream_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const bf16* __restrict__ qkv, int q_stride, bf16* __restrict__ out,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ arrivals,
                        bf16* __restrict__ k_out, bf16* __restrict__ v_out, const int* __restrict__ block_table,
                        int table_width, const int* __restrict__ tok_seq, const int* __restrict__ kv_len,
                        const int* __restrict__ row_order, int H, int K, float scale_log2, int window,
                        int pages_per_cta, int n_chunks, int merge, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, int n_rot, int pairing, int fuse,
                        int* __restrict__ status) {
  using Sm = StreamSmem<HD, STAGES>;
  constexpr int D = HD;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  bf16* qs = reinterpret_cast<bf16*>(base + Sm::Q_OFF);
  bf16* new_kv = qs + 8 * Sm::PITCH;
  uint64_t* full = reinterpret_cast<uint64_t*>(base + Sm::BAR_OFF);
  uint64_t* empty = full + STAGES;
  __shared__ int gave_up;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int G = H / K;
  const int row_tiles = (G + 7) / 8;
  // CTAs start in the order of their index: with `row_order` (the rows of the batch, longest sequence
  // first) the long sequences start first and the short ones fill in behind them
  const int tok = row_order ? row_order[blockIdx.x] : (int)blockIdx.x;
  const int kh = blockIdx.y / row_tiles, rt = blockIdx.y - kh * row_tiles;
  const int chunk = blockIdx.z;
  // What is read before the wait was written in earlier steps (lengths, block table, row order, every
  // cached row but the one of this step's token), never by the kernels just before this one.
  const int* bt = block_table + (size_t)tok * table_width;
  const int b = tok_seq[tok];
  const int len = kv_len[tok];
  if (b < 0) { pdl_wait(); pdl_trigger(); return; }          // a row of the batch without a sequence
  const int pos = len - 1;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int first_page = lo / PAGE, last_page = pos / PAGE;
  const int first_chunk = first_page / pages_per_cta, last_chunk = last_page / pages_per_cta;
  const bool active = chunk >= first_chunk && chunk <= last_chunk;
  // a chunk without visible keys has nothing to do; as a member of a cluster it still meets the
  // others at the cluster's barriers
  if (!active && merge != 1) { pdl_wait(); pdl_trigger(); return; }
  const int n_heads = min(8, G - rt * 8);
  const int page_begin = max(chunk * pages_per_cta, first_page);
  const int page_end = active ? min((chunk + 1) * pages_per_cta, last_page + 1) : page_begin;
  const int n_pages = page_end - page_begin;
  const bool holds_new = active && chunk == last_chunk;       // this chunk ends with this step's token

  if (tid == 0) {
    gave_up = 0;
    for (int s = 0; s < STAGES; ++s) { as_bar_init(full + s, 1); as_bar_init(empty + s, AS_CONSUMERS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  StreamState<HD> st;
#pragma unroll
  for (int dm = 0; dm < HD / 16; ++dm) st.o[dm][0] = st.o[dm][1] = st.o[dm][2] = st.o[dm][3] = 0.f;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;

  if (warp == AS_CONSUMERS) {
    // ---- the producer: asks for the chunk's pages, STAGES ahead of the consumers
    if (fuse != 2) pdl_wait();        // this step's row of the cache was written by the kernel before this one
    if (lane == 0) {
      for (int i = 0; i < n_pages; ++i) {
        const int s = i % STAGES;
        if (i >= STAGES && !as_wait(empty + s, ((i / STAGES) - 1) & 1)) { atomicExch(status, 21); gave_up = 1; break; }
        const int row = (bt[page_begin + i] * K + kh) * PAGE;
        unsigned char* dst = base + (size_t)s * Sm::STAGE;
        as_expect_tx(full + s, Sm::STAGE);
#pragma unroll
        for (int p = 0; p < HD / 64; ++p) {
          as_tma_2d(dst + p * AS_PANEL, &map_k, p * 64, row, full + s);
          as_tma_2d(dst + Sm::TILE + p * AS_PANEL, &map_v, p * 64, row, full + s);
        }
      }
    }
    __syncwarp();
    if (fuse == 2) pdl_wait();
    pdl_trigger();
  } else {
    // ---- the consumers
    pdl_wait();
    pdl_trigger();
    if (!fuse) {
      for (int c = tid; c < 8 * (D >> 3); c += AS_CONSUMERS * 32) {
        const int r = c / (D >> 3), cc = c - r * (D >> 3);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < n_heads)
          v = *reinterpret_cast<const uint4*>(qkv + (size_t)tok * q_stride + (size_t)(kh * G + rt * 8 + r) * D + cc * 8);
        *reinterpret_cast<uint4*>(qs + r * Sm::PITCH + cc * 8) = v;
      }
    } else {
      // rows 0..7: the tile's q heads, rotated (rows past the group: zero); rows 8, 9: this step's k
      // (rotated) and v of this KV head, for the chunk that ends with them
      const int upp = D >> 4;
      const float* cos_row = cos_t ? cos_t + (size_t)pos * (n_rot >> 1) : nullptr;
      const float* sin_row = sin_t ? sin_t + (size_t)pos * (n_rot >> 1) : nullptr;
      const bf16* row = qkv + (size_t)tok * q_stride;
      for (int it = tid; it < 10 * upp; it += AS_CONSUMERS * 32) {
        const int r = it / upp, u = it - r * upp;
        if (r < n_heads) {
          rotate_unit(row + (size_t)(kh * G + rt * 8 + r) * D, qs + r * Sm::PITCH, u, cos_row != nullptr, cos_row,
                      sin_row, n_rot, pairing);
        } else if (r < 8) {
          *reinterpret_cast<uint4*>(qs + r * Sm::PITCH + 16 * u) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(qs + r * Sm::PITCH + 16 * u + 8) = make_uint4(0, 0, 0, 0);
        } else if (holds_new && fuse == 2) {
          const bool is_k = r == 8;
          rotate_unit(row + (size_t)(H + (is_k ? 0 : K) + kh) * D, new_kv + (r - 8) * Sm::PITCH, u,
                      is_k && cos_row != nullptr, cos_row, sin_row, n_rot, pairing);
        }
      }
    }
    as_consumer_sync();
    if (fuse == 2 && holds_new && rt == 0) {
      // this step's key and value go to their place in the cache (read by later steps)
      const size_t at = (((size_t)bt[pos / PAGE] * K + kh) * PAGE + (pos % PAGE)) * D;
      for (int c = tid; c < 2 * (D >> 3); c += AS_CONSUMERS * 32) {
        const int which = c / (D >> 3), cc = c - which * (D >> 3);
        *reinterpret_cast<uint4*>((which ? v_out : k_out) + at + cc * 8) =
            *reinterpret_cast<const uint4*>(new_kv + which * Sm::PITCH + cc * 8);
      }
    }
    uint32_t qb[HD / 16][2];
#pragma unroll
    for (int kd = 0; kd < HD / 16; ++kd) {
      qb[kd][0] = *reinterpret_cast<const uint32_t*>(qs + g * Sm::PITCH + kd * 16 + 2 * t4);
      qb[kd][1] = *reinterpret_cast<const uint32_t*>(qs + g * Sm::PITCH + kd * 16 + 8 + 2 * t4);
    }
    for (int i = 0; i < n_pages; ++i) {
      const int s = i % STAGES;
      if (!as_wait(full + s, (i / STAGES) & 1)) { atomicExch(status, 22); gave_up = 1; break; }
      unsigned char* stage = base + (size_t)s * Sm::STAGE;
      const int r0 = warp * 16;
      const int key0 = (page_begin + i) * PAGE + r0;
      if (key0 <= pos && key0 + 15 >= lo) {
        if (fuse == 2 && pos >= key0 && pos < key0 + 16) {
          // this step's token lies in this warp's rows: its key and value come from the staging rows
          // (the cache's copy is being written), into the swizzled tiles
          const int r = pos & (PAGE - 1);
          for (int cc = lane; cc < (D >> 3); cc += 32) {
            *reinterpret_cast<uint4*>(stage + as_off(r, cc)) = *reinterpret_cast<const uint4*>(new_kv + cc * 8);
            *reinterpret_cast<uint4*>(stage + Sm::TILE + as_off(r, cc)) =
                *reinterpret_cast<const uint4*>(new_kv + Sm::PITCH + cc * 8);
          }
          // ordered before the TMA unit's next write to this stage
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
        }
        attend_tile16<HD>(st, qb, smem_u32(stage), smem_u32(stage + Sm::TILE), r0, scale_log2, key0, pos, lo);
      }
      __syncwarp();      // every lane is done with the stage before it is given back
      if (lane == 0) as_arrive(empty + s);
    }
  }

  float l0 = st.l[0], l1 = st.l[1];
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, o);
    l1 += __shfl_xor_sync(0xffffffffu, l1, o);
  }
  __syncthreads();      // every page that was asked for has arrived and been used: the ring is free
  const bool ok = gave_up == 0;
  if (!ok) {
    // a wait gave up: copies into the ring may still be in flight.  Nothing below touches the ring
    // then, and the CTA stays a bounded while (about a millisecond) so that they land in its memory.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }

  // merge the warps: sm_o [4][8][D + 4], sm_m, sm_l [4][8]; cta_o [8][D], cta_ml [8][2] for the cluster
  const int op = D + 4;
  float* sm_o = reinterpret_cast<float*>(base);
  float* sm_m = sm_o + AS_CONSUMERS * 8 * op;
  float* sm_l = sm_m + AS_CONSUMERS * 8;
  float* cta_o = sm_l + AS_CONSUMERS * 8;
  float* cta_ml = cta_o + 8 * D;
  if (ok && warp < AS_CONSUMERS) {
#pragma unroll
    for (int dm = 0; dm < HD / 16; ++dm) {
      const int d = dm * 16 + g;
      sm_o[(warp * 8 + 2 * t4) * op + d] = st.o[dm][0];
      sm_o[(warp * 8 + 2 * t4 + 1) * op + d] = st.o[dm][1];
      sm_o[(warp * 8 + 2 * t4) * op + d + 8] = st.o[dm][2];
      sm_o[(warp * 8 + 2 * t4 + 1) * op + d + 8] = st.o[dm][3];
    }
    if (g == 0) {
      sm_m[warp * 8 + 2 * t4] = st.m[0];
      sm_m[warp * 8 + 2 * t4 + 1] = st.m[1];
      sm_l[warp * 8 + 2 * t4] = l0;
      sm_l[warp * 8 + 2 * t4 + 1] = l1;
    }
  }
  __syncthreads();
  const bool single = (first_chunk == last_chunk);
  if (ok) {
    for (int idx = tid; idx < n_heads * D; idx += AS_THREADS) {
      const int r = idx / D, d = idx - r * D;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < AS_CONSUMERS; ++w) m = fmaxf(m, sm_m[w * 8 + r]);
      float l = 0.f, o = 0.f;
#pragma unroll
      for (int w = 0; w < AS_CONSUMERS; ++w) {
        const float mw = sm_m[w * 8 + r];
        const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
        l += sm_l[w * 8 + r] * f;
        o += sm_o[(w * 8 + r) * op + d] * f;
      }
      const int h = kh * G + rt * 8 + r;
      if (merge == 1) {
        cta_o[r * D + d] = o;
        if (d == 0) { cta_ml[r * 2] = m; cta_ml[r * 2 + 1] = l; }
      } else if (single) {
        out[((size_t)tok * H + h) * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
      } else {
        const size_t p = ((size_t)tok * H + h) * n_chunks + chunk;
        part_o[p * D + d] = o;
        if (d == 0) { part_ml[p * 2] = m; part_ml[p * 2 + 1] = l; }
      }
    }
  }
  if (merge == 1) {
    // The chunks of one (sequence, KV head, head tile) are the CTAs of one cluster: the first of them
    // reads the others' results from their shared memory, in chunk order.
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (chunk == 0 && ok) {
      for (int idx = tid; idx < n_heads * D; idx += AS_THREADS) {
        const int r = idx / D, d = idx - r * D;
        // a cluster has at most 8 chunks: their values are fetched together, then added in chunk order
        float mc[8], lc[8], oc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = first_chunk + j;
          const bool in = c <= last_chunk;
          const float* ml = cluster.map_shared_rank(cta_ml, in ? c : first_chunk);
          mc[j] = in ? ml[r * 2] : -INFINITY;
          lc[j] = in ? ml[r * 2 + 1] : 0.f;
          oc[j] = in ? cluster.map_shared_rank(cta_o, in ? c : first_chunk)[r * D + d] : 0.f;
        }
        float m = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) m = fmaxf(m, mc[j]);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float f = (mc[j] == -INFINITY) ? 0.f : exp2f(mc[j] - m);
          l += lc[j] * f;
          o += oc[j] * f;
        }
        out[((size_t)tok * H + kh * G + rt * 8 + r) * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
      }
    }
    cluster.sync();      // nobody leaves while the first CTA still reads its shared memory
    return;
  }
  if (single) return;

  // The last CTA to arrive for this (sequence, KV head, head tile) merges the chunks.  Each CTA
  // publishes its partials (fence), then counts itself; the one that sees all others has, by the
  // fence on the other side, their partials in view.  It puts the counter back to zero for the
  // next launch.
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int n_active = last_chunk - first_chunk + 1;
    int* counter = arrivals + (size_t)tok * gridDim.y + blockIdx.y;
    const int seen = atomicAdd(counter, 1);
    is_last = (seen == n_active - 1);
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // Eight chunks at a time, their loads issued together (a loop that fetched chunk after chunk took the
  // memory's latency once per chunk: 0.45 us each, 10 us for 22 chunks); always in chunk order.  A
  // thread owns four neighbouring elements of a head's output.
  for (int idx = tid; idx < n_heads * (D / 4); idx += AS_THREADS) {
    const int r = idx / (D / 4), d = (idx - r * (D / 4)) * 4;
    const int h = kh * G + rt * 8 + r;
    const size_t at = ((size_t)tok * H + h) * n_chunks;
    float m = -INFINITY, l = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c0 = first_chunk; c0 <= last_chunk; c0 += 8) {
      float2 ml[8];
      float4 oc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool in = c0 + j <= last_chunk;
        ml[j] = in ? __ldcg(reinterpret_cast<const float2*>(part_ml) + at + c0 + j) : make_float2(-INFINITY, 0.f);
        oc[j] = in ? __ldcg(reinterpret_cast<const float4*>(part_o + (at + c0 + j) * D + d))
                   : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float top = m;
#pragma unroll
      for (int j = 0; j < 8; ++j) top = fmaxf(top, ml[j].x);
      const float keep = (m == -INFINITY) ? 0.f : exp2f(m - top);
      l *= keep;
      o.x *= keep; o.y *= keep; o.z *= keep; o.w *= keep;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = (ml[j].x == -INFINITY) ? 0.f : exp2f(ml[j].x - top);
        l += ml[j].y * f;
        o.x += oc[j].x * f; o.y += oc[j].y * f; o.z += oc[j].z * f; o.w += oc[j].w * f;
      }
      m = top;
    }
    bf16* dst = out + ((size_t)tok * H + h) * D + d;
    *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(l > 0.f ? o.x / l : 0.f, l > 0.f ? o.y / l : 0.f);
    *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(l > 0.f ? o.z / l : 0.f, l > 0.f ? o.w / l : 0.f);
  }
}

// ---------------------------------------------------------------------------
typedef CUresult (*AsEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AsEncodeFn as_encode_fn() {
  static AsEncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<AsEncodeFn>(p);
  }
  return fn;
}
static int* as_status_word() {
  static int* p[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!p[dev]) {
    if (cudaMalloc(&p[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p[dev], 0, sizeof(int));
  }
  return p[dev];
}
// 0, or the code left by a kernel of this library that gave up waiting on a barrier since the last
// call (synchronises the device).
AB_API int ab_attention_stream_status() {
  int* p = as_status_word();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(p, 0, sizeof(int));
  return v;
}

// 1 if this kernel takes the shape: head size 64 or 128 (rows of whole 128-byte panels)
AB_API int ab_attention_stream_supports(int H, int K, int D) {
  return ((D == 64 || D == 128) && K > 0 && H > 0 && H % K == 0) ? 1 : 0;
}

// pages that one CTA holds in its ring for head size D: `ring` 0 = short (four CTAs per processor),
// 1 = the usual one (two), 2 = deep (one)
AB_API int ab_attention_stream_stages(int D, int ring) {
  const int r = ring < 0 ? 0 : (ring > 2 ? 2 : ring);
  return D == 64 ? (r == 0 ? 3 : r == 1 ? 6 : 12) : (r == 0 ? 2 : r == 1 ? 3 : 6);
}

// Decode attention of one new token per row of the batch (see the head of this file).
// qkv [n_tokens, q_stride] (q heads first, then k, v heads when fuse = 2), out [n_tokens, H*D], cache
// pages [n_pages, K, 64, D]; block_table [n_tokens, table_width]; tok_seq[row] < 0: a row without a
// sequence; kv_len[row]: the sequence's length with this step's token; row_order (or null): a
// permutation of the rows, the order in which their CTAs start (longest sequences first pays).
// n_chunks chunks of pages_per_cta pages cover the table; `ring`: see ab_attention_stream_stages.  merge_kind: 1 = cluster (2..8 chunks), 2 =
// scratch: part_o float [n_tokens*H*n_chunks, D], part_ml float [n_tokens*H*n_chunks, 2], arrivals int
// [n_tokens * K * ceil(G/8)], zero before the first launch and left zero by every launch.
AB_API int ab_attention_stream_bf16(const void* qkv, int q_stride, void* out, float* part_o, float* part_ml,
                                    int* arrivals, void* k_pages, void* v_pages, int n_pages,
                                    const int* block_table, int table_width, const int* tok_seq, const int* kv_len,
                                    const int* row_order, int n_tokens, int H, int K, int D, float scale, int window, int pages_per_cta,
                                    int n_chunks, int merge_kind, int ring, const float* cos_t, const float* sin_t,
                                    int n_rot, int pairing, int fuse, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (!ab_attention_stream_supports(H, K, D) || n_chunks < 1 || n_chunks > 65535 || pages_per_cta < 1 || n_pages < 1)
    return AB_BAD_ARG;
  if (fuse < 0 || fuse > 2 || n_rot < 0 || n_rot > D || (n_rot % 16) || pairing < 0 || pairing > 1) return AB_BAD_ARG;
  if (!cos_t || !sin_t || fuse == 0) { cos_t = sin_t = nullptr; }
  if (!cos_t) n_rot = 0;
  if ((long long)pages_per_cta * n_chunks < table_width) return AB_BAD_ARG;   // the chunks must cover the table
  const int G = H / K, row_tiles = (G + 7) / 8;
  if ((long long)K * row_tiles > 65535 || (long long)n_pages * K * PAGE > 0x7fffffffLL) return AB_BAD_ARG;
  int merge = 0;
  if (n_chunks > 1) {
    if (merge_kind == 1 && n_chunks <= 8) merge = 1;
    else if (merge_kind == 2 && part_o && part_ml && arrivals) merge = 2;
    else return AB_BAD_ARG;
  }
  if ((reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages)) & 15) return AB_BAD_ARG;
  AsEncodeFn enc = as_encode_fn();
  int* status = as_status_word();
  if (!enc || !status) return AB_BAD_ARG;
  CUtensorMap mk, mv;
  for (int which = 0; which < 2; ++which) {
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)n_pages * K * PAGE};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, PAGE};
    cuuint32_t elem[2] = {1, 1};
    if (enc(which ? &mv : &mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, which ? v_pages : k_pages, dims, strides, box,
            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return AB_BAD_ARG;
  }
  const float sl = scale * LOG2E;
  dim3 grid(n_tokens, K * row_tiles, n_chunks);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(AS_THREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (ab_pdl_enabled() && !ab_pdl_held) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  if (merge == 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = (unsigned)n_chunks;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  cudaError_t e;
#define AS_GO(HDV, ST)                                                                                              \
  {                                                                                                                 \
    cfg.dynamicSmemBytes = StreamSmem<HDV, ST>::TOTAL;                                                              \
    e = cudaFuncSetAttribute(attention_stream_kernel<HDV, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                             StreamSmem<HDV, ST>::TOTAL);                                                           \
    if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;                                                              \
    e = cudaLaunchKernelEx(&cfg, attention_stream_kernel<HDV, ST>, mk, mv, (const bf16*)qkv, q_stride, (bf16*)out,  \
                           part_o, part_ml, arrivals, (bf16*)k_pages, (bf16*)v_pages, block_table, table_width,     \
                           tok_seq, kv_len, row_order, H, K, sl, window, pages_per_cta, n_chunks, merge, cos_t, sin_t, n_rot,  \
                           pairing, fuse, status);                                                                  \
  }
  if (D == 64) { if (ring <= 0) AS_GO(64, 3) else if (ring == 1) AS_GO(64, 6) else AS_GO(64, 12) }
  else { if (ring <= 0) AS_GO(128, 2) else if (ring == 1) AS_GO(128, 3) else AS_GO(128, 6) }
#undef AS_GO
  if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;
  return ab_launch_status();
}
