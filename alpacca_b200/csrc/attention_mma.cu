// Causal grouped-query attention over the paged cache on the tensor cores,
// bfloat16 operands, float32 scores, softmax and accumulators.
//
// Two kernels share the inner tile code (flash attention: running maximum and
// sum per row, keys visited page by page; a page of the cache, 64 keys of one
// KV head, is exactly one key tile):
//
//   prefill  one CTA per (tile of query rows, KV head).  A row is a pair
//            (token, head of the group): the G query heads that share a KV head
//            sit in the same tile, so a key tile is loaded once for all of
//            them.  Any mix of sequences: tokens on top of cached ones, chunks,
//            single tokens; the host lists the tiles.
//   decode   one new token per sequence: one CTA per (sequence, KV head, chunk
//            of keys); the keys are the rows of the tensor-core tiles and the group's
//            heads the columns; each warp takes a run of 16-key tiles, the warps'
//            results are merged in shared memory.  The chunks' partial results
//            go to scratch memory, and the CTA that finishes last for its
//            (sequence, KV head) merges them, always in chunk order, so the
//            result does not depend on which CTA that is.
//
// Scores: (q.k) * scale; key s is seen by a token at position p iff
// lo <= s <= p, lo = max(0, p - window + 1) (window 0: all)
// (alpacca/model.py:447-467).  Head sizes: multiples of 16 up to 256.
#include "attention_common.cuh"
#include "launch.cuh"
#include <cooperative_groups.h>
#include <cuda_pipeline.h>

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Running state of one warp's 16 rows; thread (g = lane/4, t = lane%4) holds rows g and g+8.
template <int DMAX>
struct RowState {
  float o[DMAX / 8][4];
  float m[2];   // running maximum of score * scale * log2(e)
  float l[2];   // running sum of 2^(score' - m)
};

// One key tile (64 keys) for one warp.
//   qs: this warp's 16 query rows in shared memory, pitch `pitch` elements
//   ks, vs: the key and value tile [64][pitch]
//   pos0/pos1, lo0/lo1: last and first visible key of rows g and g+8; key0: position of the tile's first key
template <int DMAX>
__device__ __forceinline__ void attend_tile(RowState<DMAX>& st, const bf16* qs, const bf16* ks, const bf16* vs,
                                            int pitch, int D, float scale_log2, int key0, int pos0, int pos1,
                                            int lo0, int lo1, bool need_mask) {
  const int lane = threadIdx.x & 31;
  const int t = lane & 3;
  float s[8][4];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;

  // S = Q K^T
  const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
  const int b_key = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
#pragma unroll
  for (int kd = 0; kd < DMAX / 16; ++kd) {
    if (kd * 16 < D) {
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(a0, a1, a2, a3, smem_u32(qs + a_row * pitch + kd * 16 + a_col));
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, smem_u32(ks + (np * 16 + b_key) * pitch + kd * 16 + b_col));
        mma_bf16(s[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }

  // scale, mask, running softmax
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v = s[nt][j] * scale_log2;
      if (need_mask) {
        const int key = key0 + nt * 8 + 2 * t + (j & 1);
        const bool ok = (j < 2) ? (key <= pos0 && key >= lo0) : (key <= pos1 && key >= lo1);
        if (!ok) v = -INFINITY;
      }
      s[nt][j] = v;
      if (j < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
    }
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(st.m[0], mx0), mn1 = fmaxf(st.m[1], mx1);
  // a row that has seen no key yet keeps m = -inf; subtract 0 then, so that exp2(-inf - 0) = 0
  const float sub0 = (mn0 == -INFINITY) ? 0.f : mn0, sub1 = (mn1 == -INFINITY) ? 0.f : mn1;
  const float corr0 = fast_exp2(st.m[0] - sub0), corr1 = fast_exp2(st.m[1] - sub1);
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    s[nt][0] = fast_exp2(s[nt][0] - sub0);
    s[nt][1] = fast_exp2(s[nt][1] - sub0);
    s[nt][2] = fast_exp2(s[nt][2] - sub1);
    s[nt][3] = fast_exp2(s[nt][3] - sub1);
    sum0 += s[nt][0] + s[nt][1];
    sum1 += s[nt][2] + s[nt][3];
  }
  st.m[0] = mn0;
  st.m[1] = mn1;
  st.l[0] = st.l[0] * corr0 + sum0;   // per-thread partial sums; the quad is reduced at the end
  st.l[1] = st.l[1] * corr1 + sum1;
#pragma unroll
  for (int dt = 0; dt < DMAX / 8; ++dt) {
    st.o[dt][0] *= corr0;
    st.o[dt][1] *= corr0;
    st.o[dt][2] *= corr1;
    st.o[dt][3] *= corr1;
  }

  // O += P V
  const int v_key = (lane & 7) + ((lane >> 3) & 1) * 8, v_col = (lane >> 4) * 8;
#pragma unroll
  for (int ks16 = 0; ks16 < 4; ++ks16) {
    const uint32_t a0 = pack_bf16(s[2 * ks16][0], s[2 * ks16][1]);
    const uint32_t a1 = pack_bf16(s[2 * ks16][2], s[2 * ks16][3]);
    const uint32_t a2 = pack_bf16(s[2 * ks16 + 1][0], s[2 * ks16 + 1][1]);
    const uint32_t a3 = pack_bf16(s[2 * ks16 + 1][2], s[2 * ks16 + 1][3]);
#pragma unroll
    for (int dp = 0; dp < DMAX / 16; ++dp) {
      if (dp * 16 < D) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, smem_u32(vs + (ks16 * 16 + v_key) * pitch + dp * 16 + v_col));
        mma_bf16(st.o[2 * dp], a0, a1, a2, a3, b0, b1);
        mma_bf16(st.o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
}

template <int DMAX>
__device__ __forceinline__ void init_state(RowState<DMAX>& st) {
#pragma unroll
  for (int dt = 0; dt < DMAX / 8; ++dt) st.o[dt][0] = st.o[dt][1] = st.o[dt][2] = st.o[dt][3] = 0.f;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;
}

// copies one page tile [64][D] (contiguous in global memory) into shared memory [64][pitch]
__device__ __forceinline__ void load_tile_async(bf16* dst, const bf16* src, int D, int pitch, int tid, int nthreads) {
  const int cpr = D >> 3;                 // 16-byte chunks per row
  if (nthreads % cpr == 0) {              // a thread keeps its column and walks down the rows
    const int cc = tid % cpr, dr = nthreads / cpr;
    for (int r = tid / cpr; r < PAGE; r += dr) cp_async_16(dst + r * pitch + cc * 8, src + (size_t)r * D + cc * 8);
    return;
  }
  for (int c = tid; c < PAGE * cpr; c += nthreads) {
    const int r = c / cpr, cc = c - r * cpr;
    cp_async_16(dst + r * pitch + cc * 8, src + (size_t)r * D + cc * 8);
  }
}

// ---------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------
template <int DMAX>
__global__ void __launch_bounds__(128)
attention_prefill_kernel(const bf16* __restrict__ qkv, int q_stride, bf16* __restrict__ out,
                         const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                         const int* __restrict__ block_table, int table_width, const int* __restrict__ tok_pos,
                         const int* __restrict__ cu_q, const int* __restrict__ tile_seq,
                         const int* __restrict__ tile_q0, int H, int K, int D, float scale_log2, int window,
                         int tokens_per_tile) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int pitch = D + 8;
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);            // [64][pitch]
  bf16* kbuf = qs + 64 * pitch;                            // [2][64][pitch]
  bf16* vbuf = kbuf + 2 * 64 * pitch;                      // [2][64][pitch]

  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int G = H / K;
  // tile by tile (longest key ranges first), the KV heads of a tile side by side: CTAs start in index order
  const int tile = blockIdx.x / K, kh = blockIdx.x - tile * K;
  const int b = tile_seq[tile];
  const int q0 = tile_q0[tile];
  const int q_end = cu_q[b + 1];
  const int n_tok = min(tokens_per_tile, q_end - q0);
  const int n_rows = n_tok * G;

  // stage Q rows: row r = (token q0 + r / G, head kh*G + r % G); rows past the end are zero
  {
    const int cpr = D >> 3;
    for (int c = tid; c < 64 * cpr; c += 128) {
      const int r = c / cpr, cc = c - r * cpr;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < n_rows) {
        const int tok = q0 + r / G, h = kh * G + r % G;
        v = *reinterpret_cast<const uint4*>(qkv + (size_t)tok * q_stride + (size_t)h * D + cc * 8);
      }
      *reinterpret_cast<uint4*>(qs + r * pitch + cc * 8) = v;
    }
  }
  // positions of this thread's two rows
  const int r0 = warp * 16 + g, r1 = r0 + 8;
  const int BIG = 0x3fffffff;
  int pos0 = BIG, pos1 = BIG, lo0 = 0, lo1 = 0;
  if (r0 < n_rows) { pos0 = tok_pos[q0 + r0 / G]; lo0 = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0; }
  if (r1 < n_rows) { pos1 = tok_pos[q0 + r1 / G]; lo1 = (window > 0 && pos1 - window + 1 > 0) ? pos1 - window + 1 : 0; }
  const int pos_first = tok_pos[q0], pos_last = tok_pos[q0 + n_tok - 1];
  const int kb_begin = (window > 0 && pos_first - window + 1 > 0) ? (pos_first - window + 1) / PAGE : 0;
  const int kb_end = pos_last / PAGE + 1;
  const int* bt = block_table + (size_t)b * table_width;

  RowState<DMAX> st;
  init_state(st);

  auto issue = [&](int kb, int stage) {
    const size_t base = ((size_t)bt[kb] * K + kh) * PAGE * D;
    load_tile_async(kbuf + stage * 64 * pitch, k_pages + base, D, pitch, tid, 128);
    load_tile_async(vbuf + stage * 64 * pitch, v_pages + base, D, pitch, tid, 128);
    cp_async_commit();
  };
  issue(kb_begin, 0);
  for (int kb = kb_begin; kb < kb_end; ++kb) {
    const int stage = (kb - kb_begin) & 1;
    if (kb + 1 < kb_end) { issue(kb + 1, stage ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const int key0 = kb * PAGE;
    // rows of this warp that exist at all; a warp without rows still joins the barriers
    if (warp * 16 < n_rows) {
      const bool need_mask = (key0 + PAGE - 1 > pos_first) || (window > 0);
      attend_tile<DMAX>(st, qs + warp * 16 * pitch, kbuf + stage * 64 * pitch, vbuf + stage * 64 * pitch, pitch, D,
                        scale_log2, key0, pos0, pos1, lo0, lo1, need_mask);
    }
    __syncthreads();
  }

  // finish: reduce the row sums over the quad, normalise, store
  float l0 = st.l[0], l1 = st.l[1];
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
  for (int dt = 0; dt < DMAX / 8; ++dt) {
    if (dt * 8 < D) {
      const int d = dt * 8 + 2 * t4;
      if (r0 < n_rows) {
        bf16* o = out + ((size_t)(q0 + r0 / G) * H + kh * G + r0 % G) * D + d;
        *reinterpret_cast<uint32_t*>(o) = pack_bf16(st.o[dt][0] * inv0, st.o[dt][1] * inv0);
      }
      if (r1 < n_rows) {
        bf16* o = out + ((size_t)(q0 + r1 / G) * H + kh * G + r1 % G) * D + d;
        *reinterpret_cast<uint32_t*>(o) = pack_bf16(st.o[dt][2] * inv1, st.o[dt][3] * inv1);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// decode: one token per sequence; grid (sequence, KV head x tile of 8 heads of
// its group, chunk of keys).
//
// With one query token the roles of the operands are swapped: the KEYS are the
// 16 rows of the tensor-core tile and the (up to 8) query heads of the group
// its 8 columns, S^T = K Q^T and O^T = V^T P^T, so that no row of a tile is
// padding.  P^T as the second operand is the transposed accumulator of S^T
// (movmatrix).  A warp takes a run of up to DECODE_RUN consecutive 16-key tiles
// per round; the chunk's tiles are dealt to the warps in equal runs.  Rounds
// follow one another, so the CTA has as many warps as shared memory has room
// for runs: at head size 64, 16 warps x 48 keys = 12 pages in one round.
// ---------------------------------------------------------------------------
#define DECODE_RUN 3
// Running state of one warp: thread (g = lane/4, t = lane%4) holds heads 2t, 2t+1 of
// O^T[d = 16*dm + g (+8)], and the running maximum and (per-thread part of the) sum of those heads.
template <int DMAX>
struct DecodeState {
  float o[DMAX / 16][4];
  float m[2];
  float l[2];
};

// One run of `nt` (1..DECODE_RUN) 16-key tiles; ks, vs: the run's keys and values [nt*16][pitch];
// qb: Q^T as the second operand, per 16 columns of the head; key0: position of the run's first key.
template <int DMAX>
__device__ __forceinline__ void attend_run(DecodeState<DMAX>& st, const uint32_t (&qb)[DMAX / 16][2], const bf16* ks,
                                           const bf16* vs, int pitch, int D, float scale_log2, int nt, int key0,
                                           int pos, int lo) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
  float s[DECODE_RUN][4];
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int i = 0; i < DECODE_RUN; ++i) {
    if (i < nt) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kd = 0; kd < DMAX / 16; ++kd) {
        if (kd * 16 < D) {
          uint32_t a0, a1, a2, a3;
          ldmatrix_x4(a0, a1, a2, a3, smem_u32(ks + (i * 16 + a_row) * pitch + kd * 16 + a_col));
          mma_bf16(s[i], a0, a1, a2, a3, qb[kd][0], qb[kd][1]);
        }
      }
      const int ka = key0 + i * 16 + g, kb = ka + 8;
      const bool oka = ka <= pos && ka >= lo, okb = kb <= pos && kb >= lo;
      s[i][0] = oka ? s[i][0] * scale_log2 : -INFINITY;
      s[i][1] = oka ? s[i][1] * scale_log2 : -INFINITY;
      s[i][2] = okb ? s[i][2] * scale_log2 : -INFINITY;
      s[i][3] = okb ? s[i][3] * scale_log2 : -INFINITY;
    } else {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = -INFINITY;
    }
    mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][2]));
    mx1 = fmaxf(mx1, fmaxf(s[i][1], s[i][3]));
  }
  // a head's keys are spread over the lanes' g: bits 2..4 of the lane
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
  }
  const float mn0 = fmaxf(st.m[0], mx0), mn1 = fmaxf(st.m[1], mx1);
  const float sub0 = (mn0 == -INFINITY) ? 0.f : mn0, sub1 = (mn1 == -INFINITY) ? 0.f : mn1;
  const float corr0 = fast_exp2(st.m[0] - sub0), corr1 = fast_exp2(st.m[1] - sub1);
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int i = 0; i < DECODE_RUN; ++i) {
    s[i][0] = fast_exp2(s[i][0] - sub0);
    s[i][1] = fast_exp2(s[i][1] - sub1);
    s[i][2] = fast_exp2(s[i][2] - sub0);
    s[i][3] = fast_exp2(s[i][3] - sub1);
    sum0 += s[i][0] + s[i][2];
    sum1 += s[i][1] + s[i][3];
  }
  st.m[0] = mn0;
  st.m[1] = mn1;
  st.l[0] = st.l[0] * corr0 + sum0;
  st.l[1] = st.l[1] * corr1 + sum1;
#pragma unroll
  for (int dm = 0; dm < DMAX / 16; ++dm) {
    st.o[dm][0] *= corr0;
    st.o[dm][1] *= corr1;
    st.o[dm][2] *= corr0;
    st.o[dm][3] *= corr1;
  }
  // O^T += V^T P^T
  const int v_key = (lane & 7) + (lane >> 4) * 8, v_col = ((lane >> 3) & 1) * 8;
#pragma unroll
  for (int i = 0; i < DECODE_RUN; ++i) {
    if (i < nt) {
      const uint32_t b0 = movmatrix_trans(pack_bf16(s[i][0], s[i][1]));
      const uint32_t b1 = movmatrix_trans(pack_bf16(s[i][2], s[i][3]));
#pragma unroll
      for (int dm = 0; dm < DMAX / 16; ++dm) {
        if (dm * 16 < D) {
          uint32_t a0, a1, a2, a3;
          ldmatrix_x4_trans(a0, a1, a2, a3, smem_u32(vs + (i * 16 + v_key) * pitch + dm * 16 + v_col));
          mma_bf16(st.o[dm], a0, a1, a2, a3, b0, b1);
        }
      }
    }
  }
}

// Asks for tiles [t0, t1) of KV head kh (16 keys each, inside one page each) into ks, vs [.][pitch].
// `skip_key` (or -1): the row of the token that the step is writing, fetched later.
__device__ __forceinline__ void load_run_async(bf16* ks, bf16* vs, const bf16* __restrict__ k_pages,
                                               const bf16* __restrict__ v_pages, const int* __restrict__ bt, int K,
                                               int kh, int D, int pitch, int t0, int t1, int skip_key, int lane) {
  const int cpr = D >> 3;
  for (int tl = t0; tl < t1; ++tl) {
    const size_t base = ((size_t)bt[tl >> 2] * K + kh) * PAGE * D + (size_t)(tl & 3) * 16 * D;
    for (int c = lane; c < 16 * cpr; c += 32) {
      const int r = c / cpr, cc = c - r * cpr;
      if (tl * 16 + r == skip_key) continue;
      const int dst = ((tl - t0) * 16 + r) * pitch + cc * 8;
      cp_async_16(ks + dst, k_pages + base + (size_t)r * D + cc * 8);
      cp_async_16(vs + dst, v_pages + base + (size_t)r * D + cc * 8);
    }
  }
}

// `fuse`: 0 = q is rotated and this step's key and value are in the cache already (the separate
// rotation kernel ran); 1 = this kernel rotates q; the step's key and value are in the cache (a layer
// that reads the cache of another); 2 = this kernel rotates q and k, takes this step's key and value
// from qkv and writes them to their place in the cache.
template <int DMAX, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
attention_decode_kernel(const bf16* __restrict__ qkv, int q_stride, bf16* __restrict__ out,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ arrivals,
                        const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                        const int* __restrict__ block_table, int table_width, const int* __restrict__ tok_seq,
                        const int* __restrict__ kv_len, int H, int K, int D, float scale_log2, int window,
                        int pages_per_cta, int n_chunks, int cluster_merge, bf16* k_out, bf16* v_out, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                        int n_rot, int pairing, int fuse) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int pitch = D + 8;
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                 // [8][pitch] q, [2][pitch] this step's k, v
  bf16* new_kv = qs + 8 * pitch;
  bf16* kv = qs + 10 * pitch;                                   // [NWARPS][2][16 * DECODE_RUN][pitch]

  // What this kernel reads before the wait was written in earlier steps (lengths, block table,
  // every cached row but the one of this step's token), never by the kernels just before it.
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int G = H / K;
  const int row_tiles = (G + 7) / 8;
  const int tok = blockIdx.x;
  const int kh = blockIdx.y / row_tiles, rt = blockIdx.y - kh * row_tiles;
  const int chunk = blockIdx.z;
  // In a decode step row `tok` of the batch is sequence `tok` (or padding: tok_seq < 0).
  const int* bt = block_table + (size_t)tok * table_width;
  const int b = tok_seq[tok];
  const int len = kv_len[tok];
  if (b < 0) { pdl_wait(); pdl_trigger(); return; }
  const int pos = len - 1;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int first_page = lo / PAGE, last_page = pos / PAGE;
  const int first_chunk = first_page / pages_per_cta, last_chunk = last_page / pages_per_cta;
  // a chunk without visible keys has nothing to do; as a member of a cluster it still has to meet
  // the others at the cluster's barriers
  const bool active = chunk >= first_chunk && chunk <= last_chunk;
  if (!active && !cluster_merge) { pdl_wait(); pdl_trigger(); return; }
  const int n_heads = min(8, G - rt * 8);

  // this chunk's 16-key tiles, dealt to the warps in equal runs of at most DECODE_RUN, round after round
  const int tile_begin = max(chunk * pages_per_cta * (PAGE / 16), lo / 16);
  const int tile_end = active ? min((chunk + 1) * pages_per_cta * (PAGE / 16), pos / 16 + 1) : tile_begin;
  const int n_tiles = max(tile_end - tile_begin, 1);
  const int rounds = (n_tiles + NWARPS * DECODE_RUN - 1) / (NWARPS * DECODE_RUN);
  const int per_run = (n_tiles + NWARPS * rounds - 1) / (NWARPS * rounds);

  DecodeState<DMAX> st;
#pragma unroll
  for (int dm = 0; dm < DMAX / 16; ++dm) st.o[dm][0] = st.o[dm][1] = st.o[dm][2] = st.o[dm][3] = 0.f;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;
  bf16* ks = kv + (size_t)warp * 2 * 16 * DECODE_RUN * pitch;
  bf16* vs = ks + 16 * DECODE_RUN * pitch;
  int t0 = min(tile_end, tile_begin + warp * per_run), t1 = min(tile_end, t0 + per_run);
  load_run_async(ks, vs, k_pages, v_pages, bt, K, kh, D, pitch, t0, t1, pos, lane);
  cp_async_commit();
  pdl_wait();
  pdl_trigger();
  const bool holds_new = active && chunk == last_chunk;        // this chunk ends with this step's token
  if (fuse != 2 && pos >= t0 * 16 && pos < t1 * 16) {
    // the row that this step wrote
    const int tl = pos >> 4, r = pos & 15;
    const size_t base = ((size_t)bt[tl >> 2] * K + kh) * PAGE * D + (size_t)((tl & 3) * 16 + r) * D;
    const int dst = ((tl - t0) * 16 + r) * pitch;
    for (int cc = lane; cc < (D >> 3); cc += 32) {
      cp_async_16(ks + dst + cc * 8, k_pages + base + cc * 8);
      cp_async_16(vs + dst + cc * 8, v_pages + base + cc * 8);
    }
    cp_async_commit();
  }
  if (!fuse) {
    const int cpr = D >> 3;
    for (int c = tid; c < 8 * cpr; c += NWARPS * 32) {
      const int r = c / cpr, cc = c - r * cpr;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < n_heads)
        v = *reinterpret_cast<const uint4*>(qkv + (size_t)tok * q_stride + (size_t)(kh * G + rt * 8 + r) * D + cc * 8);
      *reinterpret_cast<uint4*>(qs + r * pitch + cc * 8) = v;
    }
  } else {
    // rows 0..7: the tile's q heads, rotated (rows past the group: zero); rows 8, 9: this step's k
    // (rotated) and v of this KV head, for the chunk that ends with them
    const int upp = D >> 4;
    const float* cos_row = cos_t ? cos_t + (size_t)pos * (n_rot >> 1) : nullptr;
    const float* sin_row = sin_t ? sin_t + (size_t)pos * (n_rot >> 1) : nullptr;
    const bf16* row = qkv + (size_t)tok * q_stride;
    for (int it = tid; it < 10 * upp; it += NWARPS * 32) {
      const int r = it / upp, u = it - r * upp;
      if (r < n_heads) {
        rotate_unit(row + (size_t)(kh * G + rt * 8 + r) * D, qs + r * pitch, u, cos_row != nullptr, cos_row, sin_row,
                    n_rot, pairing);
      } else if (r < 8) {
        *reinterpret_cast<uint4*>(qs + r * pitch + 16 * u) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(qs + r * pitch + 16 * u + 8) = make_uint4(0, 0, 0, 0);
      } else if (holds_new && fuse == 2) {
        const bool is_k = r == 8;
        rotate_unit(row + (size_t)(H + (is_k ? 0 : K) + kh) * D, new_kv + (r - 8) * pitch, u, is_k && cos_row != nullptr,
                    cos_row, sin_row, n_rot, pairing);
      }
    }
  }
  __syncthreads();
  if (fuse == 2 && holds_new && rt == 0) {
    // this step's key and value go to their place in the cache (read by later steps)
    const size_t base = (((size_t)bt[pos / PAGE] * K + kh) * PAGE + (pos % PAGE)) * D;
    const int cpr = D >> 3;
    for (int c = tid; c < 2 * cpr; c += NWARPS * 32) {
      const int which = c / cpr, cc = c - which * cpr;
      *reinterpret_cast<uint4*>((which ? v_out : k_out) + base + cc * 8) =
          *reinterpret_cast<const uint4*>(new_kv + which * pitch + cc * 8);
    }
  }
  uint32_t qb[DMAX / 16][2];
#pragma unroll
  for (int kd = 0; kd < DMAX / 16; ++kd) {
    if (kd * 16 < D) {
      qb[kd][0] = *reinterpret_cast<const uint32_t*>(qs + g * pitch + kd * 16 + 2 * t4);
      qb[kd][1] = *reinterpret_cast<const uint32_t*>(qs + g * pitch + kd * 16 + 8 + 2 * t4);
    } else {
      qb[kd][0] = qb[kd][1] = 0u;
    }
  }
  for (int round = 0; round < rounds; ++round) {
    if (round > 0) {
      t0 = min(tile_end, tile_begin + (round * NWARPS + warp) * per_run);
      t1 = min(tile_end, t0 + per_run);
      load_run_async(ks, vs, k_pages, v_pages, bt, K, kh, D, pitch, t0, t1, fuse == 2 ? pos : -1, lane);
      cp_async_commit();
    }
    cp_async_wait<0>();
    if (fuse == 2 && pos >= t0 * 16 && pos < t1 * 16) {
      // this step's token lies in this run: its row comes from the staging rows, not from the cache
      const int dst = (pos - t0 * 16) * pitch;
      for (int cc = lane; cc < (D >> 3); cc += 32) {
        *reinterpret_cast<uint4*>(ks + dst + cc * 8) = *reinterpret_cast<const uint4*>(new_kv + cc * 8);
        *reinterpret_cast<uint4*>(vs + dst + cc * 8) = *reinterpret_cast<const uint4*>(new_kv + pitch + cc * 8);
      }
    }
    __syncwarp();
    if (t0 < t1) attend_run<DMAX>(st, qb, ks, vs, pitch, D, scale_log2, t1 - t0, t0 * 16, pos, lo);
    __syncwarp();      // every lane is done reading the run before the next one overwrites it
  }
  float l0 = st.l[0], l1 = st.l[1];
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, o);
    l1 += __shfl_xor_sync(0xffffffffu, l1, o);
  }
  __syncthreads();      // every warp is done with its tiles: shared memory is reused below

  // merge the warps: sm_o [NWARPS][8][D + 4], sm_m, sm_l [NWARPS][8]
  const int op = D + 4;
  float* sm_o = reinterpret_cast<float*>(kv);
  float* sm_m = sm_o + NWARPS * 8 * op;
  float* sm_l = sm_m + NWARPS * 8;
  float* cta_o = sm_l + NWARPS * 8;      // [8][D]: this CTA's result, read by its cluster
  float* cta_ml = cta_o + 8 * D;         // [8][2]
#pragma unroll
  for (int dm = 0; dm < DMAX / 16; ++dm) {
    if (dm * 16 < D) {
      const int d = dm * 16 + g;
      sm_o[(warp * 8 + 2 * t4) * op + d] = st.o[dm][0];
      sm_o[(warp * 8 + 2 * t4 + 1) * op + d] = st.o[dm][1];
      sm_o[(warp * 8 + 2 * t4) * op + d + 8] = st.o[dm][2];
      sm_o[(warp * 8 + 2 * t4 + 1) * op + d + 8] = st.o[dm][3];
    }
  }
  if (g == 0) {
    sm_m[warp * 8 + 2 * t4] = st.m[0];
    sm_m[warp * 8 + 2 * t4 + 1] = st.m[1];
    sm_l[warp * 8 + 2 * t4] = l0;
    sm_l[warp * 8 + 2 * t4 + 1] = l1;
  }
  __syncthreads();
  const bool single = (first_chunk == last_chunk);
  for (int idx = tid; idx < n_heads * D; idx += NWARPS * 32) {
    const int r = idx / D, d = idx - r * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) m = fmaxf(m, sm_m[w * 8 + r]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float mw = sm_m[w * 8 + r];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
      l += sm_l[w * 8 + r] * f;
      o += sm_o[(w * 8 + r) * op + d] * f;
    }
    const int h = kh * G + rt * 8 + r;
    if (cluster_merge) {
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
  if (cluster_merge) {
    // The chunks of one (token, KV head, head tile) are the CTAs of one cluster: the first of them
    // reads the others' results from their shared memory, in chunk order.
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (chunk == 0) {
      for (int idx = tid; idx < n_heads * D; idx += NWARPS * 32) {
        const int r = idx / D, d = idx - r * D;
        float m = -INFINITY;
        for (int c = first_chunk; c <= last_chunk; ++c) m = fmaxf(m, cluster.map_shared_rank(cta_ml, c)[r * 2]);
        float l = 0.f, o = 0.f;
        for (int c = first_chunk; c <= last_chunk; ++c) {
          const float* ml = cluster.map_shared_rank(cta_ml, c);
          const float mc = ml[r * 2];
          const float f = (mc == -INFINITY) ? 0.f : exp2f(mc - m);
          l += ml[r * 2 + 1] * f;
          o += cluster.map_shared_rank(cta_o, c)[r * D + d] * f;
        }
        out[((size_t)tok * H + kh * G + rt * 8 + r) * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
      }
    }
    cluster.sync();      // nobody leaves while the first CTA still reads its shared memory
    return;
  }
  if (single) return;

  // The last CTA to arrive for this (token, KV head, head tile) merges the chunks.  Each CTA
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
  for (int idx = tid; idx < n_heads * D; idx += NWARPS * 32) {
    const int r = idx / D, d = idx - r * D;
    const int h = kh * G + rt * 8 + r;
    const size_t base = ((size_t)tok * H + h) * n_chunks;
    float m = -INFINITY;
    for (int c = first_chunk; c <= last_chunk; ++c) m = fmaxf(m, __ldcg(part_ml + (base + c) * 2));
    float l = 0.f, o = 0.f;
    for (int c = first_chunk; c <= last_chunk; ++c) {
      const float mc = __ldcg(part_ml + (base + c) * 2);
      const float f = (mc == -INFINITY) ? 0.f : exp2f(mc - m);
      l += __ldcg(part_ml + (base + c) * 2 + 1) * f;
      o += __ldcg(part_o + (base + c) * D + d) * f;
    }
    out[((size_t)tok * H + h) * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
  }
}

// ---------------------------------------------------------------------------
// entry points
// ---------------------------------------------------------------------------
static int dmax_of(int D) { return D <= 64 ? 64 : (D <= 128 ? 128 : 256); }

// warps of a decode CTA for head size D; `small` (0, 1, 2) halves the CTA that many times: with
// many (sequence, head) pairs several small CTAs per processor do better than one large one
AB_API int ab_attention_decode_warps(int D, int small) {
  const int dm = dmax_of(D);
  const int full = dm == 64 ? 16 : (dm == 128 ? 8 : 4);
  return full >> (small < 0 ? 0 : (small > 2 ? 2 : small));
}

// keys that a decode CTA covers in one round: its warps' runs of DECODE_RUN tiles of 16 keys
AB_API int ab_attention_decode_round_keys(int D, int small) {
  return ab_attention_decode_warps(D, small) * DECODE_RUN * 16;
}
AB_API int ab_attention_decode_round_pages(int D) { return ab_attention_decode_round_keys(D, 0) / PAGE; }

AB_API int ab_attention_prefill_bf16(const void* qkv, int q_stride, void* out, const void* k_pages,
                                     const void* v_pages, const int* block_table, int table_width,
                                     const int* tok_pos, const int* cu_q, const int* tile_seq, const int* tile_q0,
                                     int n_tiles, int tokens_per_tile, int H, int K, int D, float scale, int window,
                                     cudaStream_t stream) {
  if (n_tiles <= 0) return AB_OK;
  if (D <= 0 || D > 256 || (D % 16) || H % K || K > 65535) return AB_BAD_ARG;
  const int G = H / K;
  if (tokens_per_tile < 1 || tokens_per_tile * G > 64) return AB_BAD_ARG;
  const int pitch = D + 8;
  const size_t smem = (size_t)(64 + 4 * 64) * pitch * sizeof(bf16);
  if ((long long)n_tiles * K > 0x7fffffffLL) return AB_BAD_ARG;
  dim3 grid((unsigned)n_tiles * K);
  const float sl = scale * LOG2E;
#define AB_GO(DM)                                                                                                  \
  {                                                                                                                \
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<DM>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem);                                                               \
    if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;                                                             \
    ab_launch(attention_prefill_kernel<DM>, grid, dim3(128), smem, stream,                                         \
        (const bf16*)qkv, q_stride, (bf16*)out, (const bf16*)k_pages, (const bf16*)v_pages, block_table,           \
        table_width, tok_pos, cu_q, tile_seq, tile_q0, H, K, D, sl, window, tokens_per_tile);                      \
  }
  switch (dmax_of(D)) {
    case 64: AB_GO(64); break;
    case 128: AB_GO(128); break;
    default: AB_GO(256); break;
  }
#undef AB_GO
  return ab_launch_status();
}

// Launch with programmatic dependent launch and, for `cluster_z` > 1, clusters of that many CTAs along z.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_clustered(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, unsigned cluster_z, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (ab_pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = cluster_z;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define AB_DECODE_MAX_CLUSTER 8

AB_API int ab_attention_decode_rope_bf16(const void* qkv, int q_stride, void* out, float* part_o, float* part_ml,
                                         int* arrivals, void* k_pages, void* v_pages, const int* block_table,
                                         int table_width, const int* tok_seq, const int* kv_len, int n_tokens, int H,
                                         int K, int D, float scale, int window, int pages_per_cta, int n_chunks,
                                         int small, const float* cos_t, const float* sin_t, int n_rot, int pairing,
                                         int fuse, cudaStream_t stream);

// The chunks of one (token, KV head) are merged inside a thread-block cluster (through shared
// memory) when there are 2 to 8 of them.  More chunks than that go through scratch memory:
// part_o float [n_tokens * H * n_chunks, D], part_ml float [n_tokens * H * n_chunks, 2], arrivals int
// [n_tokens * K * ceil(G / 8)], which must be zero before the first launch and is left zero by every
// launch.
AB_API int ab_attention_decode_bf16(const void* qkv, int q_stride, void* out, float* part_o, float* part_ml,
                                    int* arrivals, const void* k_pages, const void* v_pages, const int* block_table,
                                    int table_width, const int* tok_seq, const int* kv_len, int n_tokens, int H,
                                    int K, int D, float scale, int window, int pages_per_cta, int n_chunks,
                                    int small, cudaStream_t stream) {
  return ab_attention_decode_rope_bf16(qkv, q_stride, out, part_o, part_ml, arrivals, const_cast<void*>(k_pages),
                                       const_cast<void*>(v_pages), block_table, table_width, tok_seq, kv_len,
                                       n_tokens, H, K, D, scale, window, pages_per_cta, n_chunks, small, nullptr,
                                       nullptr, 0, 0, 0, stream);
}

// The same with the position rotation and the append to the cache inside the kernel (`fuse` 1 or 2,
// see the kernel; 0 is ab_attention_decode_bf16).  cos_t, sin_t: float [positions, n_rot / 2] or null
// (no rotation); n_rot a multiple of 16; pairing 0 = neighbours, 1 = halves.
AB_API int ab_attention_decode_rope_bf16(const void* qkv, int q_stride, void* out, float* part_o, float* part_ml,
                                         int* arrivals, void* k_pages, void* v_pages, const int* block_table,
                                         int table_width, const int* tok_seq, const int* kv_len, int n_tokens, int H,
                                         int K, int D, float scale, int window, int pages_per_cta, int n_chunks,
                                         int small, const float* cos_t, const float* sin_t, int n_rot, int pairing,
                                         int fuse, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (D <= 0 || D > 256 || (D % 16) || H % K || n_chunks < 1 || n_chunks > 65535 || pages_per_cta < 1)
    return AB_BAD_ARG;
  if (small < 0 || small > 2) return AB_BAD_ARG;
  if (fuse < 0 || fuse > 2 || n_rot < 0 || n_rot > D || (n_rot % 16) || pairing < 0 || pairing > 1) return AB_BAD_ARG;
  if (!cos_t || !sin_t || fuse == 0) { cos_t = sin_t = nullptr; }
  if (!cos_t) n_rot = 0;
  if ((long long)pages_per_cta * n_chunks < table_width) return AB_BAD_ARG;   // the chunks must cover the table
  const int G = H / K, row_tiles = (G + 7) / 8;
  if ((long long)K * row_tiles > 65535) return AB_BAD_ARG;
  const int pitch = D + 8;
  const float sl = scale * LOG2E;
  const int cluster_merge = (n_chunks > 1 && n_chunks <= AB_DECODE_MAX_CLUSTER) ? 1 : 0;
  dim3 grid(n_tokens, K * row_tiles, n_chunks);
#define AB_GO(DM, NW)                                                                                               \
  {                                                                                                                 \
    size_t tiles = (size_t)(10 + NW * 2 * 16 * DECODE_RUN) * pitch * sizeof(bf16);                                  \
    size_t merge = (size_t)10 * pitch * sizeof(bf16) + (size_t)(NW * 8 * (D + 6) + 8 * (D + 2)) * sizeof(float);    \
    size_t smem = tiles > merge ? tiles : merge;                                                                    \
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<DM, NW>,                                           \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                   \
    if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;                                                              \
    launch_clustered(attention_decode_kernel<DM, NW>, grid, dim3(NW * 32), smem, stream,                            \
        cluster_merge ? (unsigned)n_chunks : 1u,                                                                    \
        (const bf16*)qkv, q_stride, (bf16*)out, part_o, part_ml, arrivals, (const bf16*)k_pages,                    \
        (const bf16*)v_pages, block_table, table_width, tok_seq, kv_len, H, K, D, sl, window, pages_per_cta,        \
        n_chunks, cluster_merge, (bf16*)k_pages, (bf16*)v_pages, cos_t, sin_t, n_rot, pairing, fuse);               \
  }
  if (n_chunks > AB_DECODE_MAX_CLUSTER && (!part_o || !part_ml || !arrivals)) return AB_BAD_ARG;
  switch (dmax_of(D)) {
    // warps x shared memory of a warp's run of keys and values; `small` halves the CTA once or twice
    case 64:                            // 16 warps x 13.5 KB
      if (small == 0) AB_GO(64, 16) else if (small == 1) AB_GO(64, 8) else AB_GO(64, 4)
      break;
    case 128:                           // 8 warps x 25.5 KB
      if (small == 0) AB_GO(128, 8) else if (small == 1) AB_GO(128, 4) else AB_GO(128, 2)
      break;
    default:                            // 4 warps x 49.5 KB
      if (small == 0) AB_GO(256, 4) else if (small == 1) AB_GO(256, 2) else AB_GO(256, 1)
      break;
  }
#undef AB_GO
  return ab_launch_status();
}

// ---------------------------------------------------------------------------
// The entry point that allocates nothing (declared and described in attention_mma.h).
// ---------------------------------------------------------------------------
#include "attention_mma.h"
#include <stdio.h>

// partial outputs | running (max, sum) pairs | arrival counters
static __device__ __align__(256) unsigned char ab_decode_noalloc_scratch[AB_DECODE_NOALLOC_SCRATCH_BYTES];

#define AB_MAX_DEVICES 64
static unsigned char* ab_noalloc_base[AB_MAX_DEVICES];     // device address of the array, per device
static thread_local char ab_noalloc_message[256];

AB_API const char* ab_attention_decode_bf16_noalloc_error(void) { return ab_noalloc_message; }

AB_API int ab_attention_decode_bf16_noalloc(const void* qkv, int q_stride, void* out, const void* k_pages,
                                            const void* v_pages, const int* block_table, int table_width,
                                            const int* tok_seq, const int* kv_len, int n_tokens, int H, int K,
                                            int D, float scale, int window, int pages_per_cta, int n_chunks,
                                            cudaStream_t stream) {
  ab_noalloc_message[0] = 0;
  if (n_tokens <= 0) return AB_OK;
  if (H <= 0 || K <= 0 || H % K || D <= 0 || n_chunks < 1) {
    snprintf(ab_noalloc_message, sizeof ab_noalloc_message, "bad sizes: H=%d K=%d D=%d n_chunks=%d", H, K, D, n_chunks);
    return AB_BAD_ARG;
  }
  const unsigned long long partial = (unsigned long long)n_tokens * H * n_chunks * D;
  const unsigned long long counters = (unsigned long long)n_tokens * K * ((H / K + 7) / 8);
  if (partial > AB_DECODE_NOALLOC_MAX_PARTIAL || counters > AB_DECODE_NOALLOC_MAX_COUNTERS) {
    snprintf(ab_noalloc_message, sizeof ab_noalloc_message,
             "problem too large for the built-in scratch: n_tokens*H*n_chunks*D = %llu (limit %u), "
             "n_tokens*K*ceil(H/K/8) = %llu (limit %u); use ab_attention_decode_bf16 with scratch of your own",
             partial, AB_DECODE_NOALLOC_MAX_PARTIAL, counters, AB_DECODE_NOALLOC_MAX_COUNTERS);
    return AB_NOALLOC_TOO_LARGE;
  }
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= AB_MAX_DEVICES) {
    snprintf(ab_noalloc_message, sizeof ab_noalloc_message, "no usable current device (%s)", cudaGetErrorString(e));
    return AB_CUDA_ERR + (int)e;
  }
  if (ab_noalloc_base[device] == nullptr) {
    // set-up, once per device, with that device current: the array's name is a host-side handle;
    // the address that a kernel can use has to be asked for
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, ab_decode_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(ab_noalloc_message, sizeof ab_noalloc_message, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return AB_CUDA_ERR + (int)e;
    }
    ab_noalloc_base[device] = p;
  }
  unsigned char* base = ab_noalloc_base[device];
  float* part_o = reinterpret_cast<float*>(base);
  float* part_ml = reinterpret_cast<float*>(base + (size_t)AB_DECODE_NOALLOC_MAX_PARTIAL * 4u);
  int* arrivals = reinterpret_cast<int*>(base + (size_t)AB_DECODE_NOALLOC_MAX_PARTIAL * 4u +
                                         (size_t)(AB_DECODE_NOALLOC_MAX_PARTIAL / 8u) * 4u);
  // the counters must start at zero whatever the last call left (it may have been cut short)
  e = cudaMemsetAsync(arrivals, 0, (size_t)counters * sizeof(int), stream);
  if (e != cudaSuccess) {
    snprintf(ab_noalloc_message, sizeof ab_noalloc_message, "clearing the counters failed: %s", cudaGetErrorString(e));
    return AB_CUDA_ERR + (int)e;
  }
  const int rc = ab_attention_decode_bf16(qkv, q_stride, out, part_o, part_ml, arrivals, k_pages, v_pages, block_table,
                                          table_width, tok_seq, kv_len, n_tokens, H, K, D, scale, window,
                                          pages_per_cta, n_chunks, 0, stream);
  if (rc != AB_OK)
    snprintf(ab_noalloc_message, sizeof ab_noalloc_message, "the launch was refused or failed (code %d)", rc);
  return rc;
}
