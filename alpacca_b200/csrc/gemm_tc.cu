// Matrix product on the fifth-generation tensor cores: D[128 x BN] tiles of
//   A[rowsA, K] . B[rowsB, K]^T      (both bfloat16, K contiguous)
// accumulated in float32 in tensor memory (TMEM) by tcgen05.mma, operands staged in
// shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), a ring of stages
// guarded by mbarriers.
//
// One CTA computes one tile (and, with several K slices, one slice of it).  Six warps:
//   warp 0      one lane issues the TMA loads of the stages,
//   warp 1      allocates TMEM; one lane issues the MMAs (four per stage: K = 16 each)
//               and commits them to the barriers that free the stages,
//   warps 2..5  the epilogue: tcgen05.ld of the accumulator (a warp reads the 32 TMEM
//               lanes it may touch), then the fused tail and the store.
// Two uses share the kernel:
//   rows = tokens   (prefill and large batches)  A = activations, B = weights;
//                   tails: store bfloat16 / float32 (+ bias), or SwiGLU on the
//                   interleaved gate|up matrix (alpacca/model.py:513);
//   rows = features (decode, "swapped")          A = weights, B = the batch (up to 64
//                   rows, one MMA column each): the 128-row MMA shape is filled by
//                   the weights, which stream through once; same tails, transposed.
// The weights never depend on the kernel before, so their first loads are issued
// before the wait of programmatic dependent launch.
//
// K slices (grid z): every CTA parks its float32 tile in scratch memory; the CTA
// that arrives last for a tile adds the slices in slice order and runs the tail.
//
// Large products (rows = tokens, one 128 x 256 tile after another) run a second, persistent form of
// the kernel: one CTA per processor walks its share of the tiles; the accumulator is double-buffered
// in TMEM (2 x 256 columns: all of it), so the tail of one tile (TMEM -> registers -> activation ->
// global memory) runs under the main loop of the next, and the ring of stages never drains between
// tiles.  Tiles that share a 256-row panel of the weights are taken by neighbouring CTAs, so the
// panel is read from memory once and from L2 after that.
//
// Every wait on an mbarrier is bounded: after SPIN_LIMIT failed tries a thread
// records a code in `status`, and every role falls through to the common end, where
// TMEM is given back.  The kernel cannot hang on a barrier that never completes.
#include "common.cuh"
#include "launch.cuh"
#include <cuda.h>

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define SPIN_LIMIT (1u << 22)

#define EPI_STORE_BF16 0
#define EPI_STORE_F32 1
#define EPI_SWIGLU_BF16 2

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// Bounded wait; false when the limit ran out (the caller records it and leaves).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_addr(bar);
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
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
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y) : "memory");
}
// K-major operand tile with 128-byte rows and 128-byte swizzle: 8-row groups are 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// g / (1 + e^-g) with the hardware's approximate exponential and division (relative error about 2^-21,
// far below the bfloat16 rounding of the result): in the tail of a tile, where it runs beside the next
// tile's MMAs, the exact forms cost 9 us of a 100 us product (2048 x 16384 x 2048), these 3.
__device__ __forceinline__ float silu_fast(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

template <int BN> struct TcShape {
  // few columns: the kernel streams weights and is bound by bytes in flight, so a deep ring;
  // many columns: bound by the tensor cores, and two CTAs per SM overlap tails with main loops
  static constexpr int STAGES = BN >= 256 ? 4 : (BN >= 128 ? 3 : 8);
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + ((B_BYTES + 1023) / 1024) * 1024;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
};

// The tail for 16 consecutive accumulator columns c0..c0+15 of row `row` of the tile.
//   !SWAP: row = token (global row m), columns = features n0 + c
//    SWAP: row = feature (global n), columns = batch rows c
template <int EPI, bool SWAP>
__device__ __forceinline__ void tail16(const float* v, int row_g, int col0_g, int rows_total, int cols_total,
                                       const float* __restrict__ bias, void* __restrict__ Y, int ldy, int lane) {
  if (!SWAP) {
    const int m = row_g;
    if (m >= rows_total) return;
    if (EPI == EPI_SWIGLU_BF16) {
      // columns col0..col0+7 gate, +8..+15 up of units (col0/16)*8 + 0..7
      if (col0_g + 16 > cols_total) return;
      bf16* y = reinterpret_cast<bf16*>(Y) + (size_t)m * ldy + (col0_g >> 1);
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int u = 2 * j + e;
          const float g = v[u] + (bias ? bias[col0_g + u] : 0.f), up = v[8 + u] + (bias ? bias[col0_g + 8 + u] : 0.f);
          a[e] = silu_fast(g) * up;
        }
        __nv_bfloat162 r = __floats2bfloat162_rn(a[0], a[1]);
        w[j] = *reinterpret_cast<uint32_t*>(&r);
      }
      *reinterpret_cast<uint4*>(y) = make_uint4(w[0], w[1], w[2], w[3]);
    } else if (EPI == EPI_STORE_F32) {
      float* y = reinterpret_cast<float*>(Y) + (size_t)m * ldy + col0_g;
#pragma unroll
      for (int c = 0; c < 16; ++c)
        if (col0_g + c < cols_total) y[c] = v[c] + (bias ? bias[col0_g + c] : 0.f);
    } else {
      bf16* y = reinterpret_cast<bf16*>(Y) + (size_t)m * ldy + col0_g;
      if (col0_g + 16 <= cols_total && ((ldy & 7) == 0)) {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          __nv_bfloat162 r = __floats2bfloat162_rn(v[2 * j] + (bias ? bias[col0_g + 2 * j] : 0.f),
                                                   v[2 * j + 1] + (bias ? bias[col0_g + 2 * j + 1] : 0.f));
          w[j] = *reinterpret_cast<uint32_t*>(&r);
        }
        *reinterpret_cast<uint4*>(y) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(y + 8) = make_uint4(w[4], w[5], w[6], w[7]);
      } else {
#pragma unroll
        for (int c = 0; c < 16; ++c)
          if (col0_g + c < cols_total) y[c] = __float2bfloat16_rn(v[c] + (bias ? bias[col0_g + c] : 0.f));
      }
    }
  } else {
    // swapped: this thread's row is feature n; column c is batch row m = col0_g + c
    const int n = row_g;
    const float b = (bias && n < rows_total) ? bias[n] : 0.f;
    if (EPI == EPI_SWIGLU_BF16) {
      // rows 16q..16q+7 gate, 16q+8..16q+15 up: lanes with bit 3 clear hold gates, their partner is lane + 8
      const int unit = (n >> 4) * 8 + (n & 7);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float mine = v[c] + b;
        const float partner = __shfl_down_sync(0xffffffffu, mine, 8);
        const int m = col0_g + c;
        if (!(lane & 8) && n < rows_total && m < cols_total)
          reinterpret_cast<bf16*>(Y)[(size_t)m * ldy + unit] = __float2bfloat16_rn(silu_fast(mine) * partner);
      }
    } else {
      if (n >= rows_total) return;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const int m = col0_g + c;
        if (m < cols_total) {
          if (EPI == EPI_STORE_F32) reinterpret_cast<float*>(Y)[(size_t)m * ldy + n] = v[c] + b;
          else reinterpret_cast<bf16*>(Y)[(size_t)m * ldy + n] = __float2bfloat16_rn(v[c] + b);
        }
      }
    }
  }
}

template <int BN, int EPI, bool SWAP>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               void* __restrict__ Y, const float* __restrict__ bias, float* __restrict__ partials,
               int* __restrict__ arrivals, int* __restrict__ status, int rows_a, int rows_b, int K, int ldy,
               int kblocks_per_slice) {
  using S = TcShape<BN>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(base + S::STAGES * S::STAGE_BYTES);
  uint64_t* empty = full + S::STAGES;
  uint64_t* accum = empty + S::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  int* last_flag = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int a_row0 = blockIdx.x * TC_BM, b_row0 = blockIdx.y * BN;
  const int n_kblocks = (K + TC_BK - 1) / TC_BK;
  const int kb0 = blockIdx.z * kblocks_per_slice;
  const int kb1 = min(n_kblocks, kb0 + kblocks_per_slice);
  const int nkb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    mbar_init(accum, 1);
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(S::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  // which operand holds the weights (independent of the kernel before this one)
  const CUtensorMap* map_w = SWAP ? &map_a : &map_b;
  const CUtensorMap* map_x = SWAP ? &map_b : &map_a;

  if (warp == 0) {
    if (lane == 0) {
      auto dst_a = [&](int s) { return base + s * S::STAGE_BYTES; };
      auto dst_b = [&](int s) { return base + s * S::STAGE_BYTES + S::A_BYTES; };
      auto load_w = [&](int s, int kb) {
        if (SWAP) tma_load_2d(dst_a(s), map_w, kb * TC_BK, a_row0, full + s);
        else tma_load_2d(dst_b(s), map_w, kb * TC_BK, b_row0, full + s);
      };
      auto load_x = [&](int s, int kb) {
        if (SWAP) tma_load_2d(dst_b(s), map_x, kb * TC_BK, b_row0, full + s);
        else tma_load_2d(dst_a(s), map_x, kb * TC_BK, a_row0, full + s);
      };
      const int early = min(nkb, S::STAGES);
      for (int i = 0; i < early; ++i) {          // weights of the first stages, before the wait
        mbar_expect_tx(full + i, S::A_BYTES + S::B_BYTES);
        load_w(i, kb0 + i);
      }
      pdl_wait();
      pdl_trigger();
      for (int i = 0; i < early; ++i) load_x(i, kb0 + i);
      for (int i = early; i < nkb; ++i) {
        const int s = i % S::STAGES;
        if (!mbar_wait(empty + s, ((i / S::STAGES) - 1) & 1)) { atomicExch(status, 1); *abort_flag = 1; break; }
        mbar_expect_tx(full + s, S::A_BYTES + S::B_BYTES);
        load_w(s, kb0 + i);
        load_x(s, kb0 + i);
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((BN < 16 ? 16 : BN) >> 3) << 17) |
                                 ((uint32_t)(TC_BM >> 4) << 24);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % S::STAGES;
        if (!mbar_wait(full + s, (i / S::STAGES) & 1)) { atomicExch(status, 2); *abort_flag = 1; ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = smem_addr(base + s * S::STAGE_BYTES), sb = sa + S::A_BYTES;
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k)
          umma_bf16(tmem, umma_desc(sa + k * 32), umma_desc(sb + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(empty + s);           // frees the stage when these MMAs have read it
      }
      umma_commit(accum);                 // the accumulator is complete when everything before is done
    }
  } else {
    pdl_wait();
    // epilogue warps 2..5: TMEM lanes 32 * (warp % 4) .. + 31
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;          // row of the tile
    bool ok = nkb > 0 ? mbar_wait(accum, 0) : true;
    if (!ok) { atomicExch(status, 3); *abort_flag = 1; }
    ok = __all_sync(0xffffffffu, ok);      // tcgen05.ld below is warp-wide
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const bool split = gridDim.z > 1;
    const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
    float* my_part = partials ? partials + ((size_t)tile_id * gridDim.z + blockIdx.z) * (TC_BM * BN) : nullptr;
    const int rows_total = SWAP ? rows_a : rows_a;        // rows of D are rows of A in both uses
    const int cols_total = rows_b;
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16];
        if (nkb > 0) tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + c0, v);
        else {
#pragma unroll
          for (int c = 0; c < 16; ++c) v[c] = 0.f;
        }
        if (!split) {
          tail16<EPI, SWAP>(v, a_row0 + row, b_row0 + c0, rows_total, cols_total, bias, Y, ldy, lane);
        } else {
          // tile stored column-chunk major so that a warp's stores are contiguous: [c0/16][row][16]
          float4* p = reinterpret_cast<float4*>(my_part + ((size_t)(c0 >> 4) * TC_BM + row) * 16);
          p[0] = make_float4(v[0], v[1], v[2], v[3]);
          p[1] = make_float4(v[4], v[5], v[6], v[7]);
          p[2] = make_float4(v[8], v[9], v[10], v[11]);
          p[3] = make_float4(v[12], v[13], v[14], v[15]);
        }
      }
    }
    if (split) {
      // the last CTA to arrive for this tile adds the slices in slice order (see gemv_bf16.cu)
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        const int seen = atomicAdd(arrivals + tile_id, 1);
        const int last = (seen == (int)gridDim.z - 1);
        if (last) arrivals[tile_id] = 0;
        *last_flag = last;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*last_flag && ok) {
        __threadfence();
        const float* tile = partials + (size_t)tile_id * gridDim.z * (TC_BM * BN);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float v[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) v[c] = 0.f;
          for (int s = 0; s < (int)gridDim.z; ++s) {
            const float4* p = reinterpret_cast<const float4*>(tile + (size_t)s * (TC_BM * BN) +
                                                               ((size_t)(c0 >> 4) * TC_BM + row) * 16);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 t = __ldcg(p + q);
              v[4 * q] += t.x; v[4 * q + 1] += t.y; v[4 * q + 2] += t.z; v[4 * q + 3] += t.w;
            }
          }
          tail16<EPI, SWAP>(v, a_row0 + row, b_row0 + c0, rows_total, cols_total, bias, Y, ldy, lane);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(S::TMEM_COLS));
  }
}

// ---------------------------------------------------------------------------
// The persistent form for rows = tokens: tiles of 128 x 256, accumulators double-buffered in TMEM.
// ---------------------------------------------------------------------------
#define TP_BN 256
#define TP_STAGES 4
#define TP_A_BYTES (TC_BM * TC_BK * 2)
#define TP_B_BYTES (TP_BN * TC_BK * 2)
#define TP_STAGE_BYTES (TP_A_BYTES + TP_B_BYTES)
#define TP_SMEM (TP_STAGES * TP_STAGE_BYTES + 1024 + 256)

// The order in which the tiles are walked: bands of TP_BAND tile rows; inside a band one tile column
// after the other, the band's rows of a column side by side.  The CTAs that run at the same time
// (consecutive tiles) then share a band of X (16 x 128 rows: it stays in the L2 for all columns) and a
// few column tiles of W, so W is read once per band and X once: with rows fastest over the whole
// matrix, as before, a prompt of 65,536 tokens re-read X for every tile column (60 GB at the 8B sizes,
// as long as the arithmetic takes).
#define TP_BAND 16
__device__ __forceinline__ void tp_tile_origin(int tile, int tiles_m, int tiles_n, int& m0, int& n0) {
  const int per_band = TP_BAND * tiles_n;
  const int band = tile / per_band, within = tile - band * per_band;
  const int rows = min(TP_BAND, tiles_m - band * TP_BAND);
  const int col = within / rows;
  m0 = (band * TP_BAND + (within - col * rows)) * TC_BM;
  n0 = col * TP_BN;
}

template <int EPI>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                          void* __restrict__ Y, const float* __restrict__ bias, int* __restrict__ status, int M, int N,
                          int K, int ldy, int tiles_m, int n_tiles) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(base + TP_STAGES * TP_STAGE_BYTES);
  uint64_t* empty = full + TP_STAGES;
  uint64_t* acc_full = empty + TP_STAGES;      // [2] the MMAs of a tile are done
  uint64_t* acc_empty = acc_full + 2;          // [2] the tail has read the buffer (one arrival per tail warp)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (K + TC_BK - 1) / TC_BK;
  const int tiles_n = n_tiles / tiles_m;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TP_STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // weights of the first stages before the wait (they do not depend on the kernel before)
      int it = 0;
      bool ok = true;
      const int first = blockIdx.x;
      const int early = first < n_tiles ? min(nkb, TP_STAGES) : 0;
      int n0_first = 0, m0_first = 0;
      if (first < n_tiles) tp_tile_origin(first, tiles_m, tiles_n, m0_first, n0_first);
      for (int i = 0; i < early; ++i) {
        mbar_expect_tx(full + i, TP_STAGE_BYTES);
        tma_load_2d(base + i * TP_STAGE_BYTES + TP_A_BYTES, &map_w, i * TC_BK, n0_first, full + i);
      }
      pdl_wait();
      pdl_trigger();
      for (int i = 0; i < early; ++i) tma_load_2d(base + i * TP_STAGE_BYTES, &map_x, i * TC_BK, m0_first, full + i);
      for (int tile = first; tile < n_tiles && ok; tile += gridDim.x) {
        int m0, n0;
        tp_tile_origin(tile, tiles_m, tiles_n, m0, n0);
        for (int kb = (tile == first ? early : 0); kb < nkb; ++kb) {
          const int i = it + kb;
          const int s = i % TP_STAGES;
          if (i >= TP_STAGES && !mbar_wait(empty + s, ((i / TP_STAGES) - 1) & 1)) { atomicExch(status, 11); ok = false; break; }
          mbar_expect_tx(full + s, TP_STAGE_BYTES);
          tma_load_2d(base + s * TP_STAGE_BYTES + TP_A_BYTES, &map_w, kb * TC_BK, n0, full + s);
          tma_load_2d(base + s * TP_STAGE_BYTES, &map_x, kb * TC_BK, m0, full + s);
        }
        it += nkb;
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TP_BN >> 3) << 17) |
                                 ((uint32_t)(TC_BM >> 4) << 24);
      int it = 0, lt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++lt) {
        const int buf = lt & 1;
        if (lt >= 2 && !mbar_wait(acc_empty + buf, ((lt >> 1) - 1) & 1)) { atomicExch(status, 12); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem + (uint32_t)buf * TP_BN;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % TP_STAGES;
          if (!mbar_wait(full + s, (it / TP_STAGES) & 1)) { atomicExch(status, 13); ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_addr(base + s * TP_STAGE_BYTES), sb = sa + TP_A_BYTES;
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)
            umma_bf16(acc, umma_desc(sa + k * 32), umma_desc(sb + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty + s);
        }
        if (ok) umma_commit(acc_full + buf);
      }
    }
  } else {
    pdl_wait();
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    int lt = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++lt) {
      const int buf = lt & 1;
      int m0, n0;
      tp_tile_origin(tile, tiles_m, tiles_n, m0, n0);
      ok = mbar_wait(acc_full + buf, (lt >> 1) & 1);
      if (!ok) atomicExch(status, 14);
      ok = __all_sync(0xffffffffu, ok);      // tcgen05.ld below is warp-wide
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c0 = 0; c0 < TP_BN; c0 += 16) {
        float v[16];
        tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * TP_BN + c0, v);
        tail16<EPI, false>(v, m0 + row, n0 + c0, M, N, bias, Y, ldy, lane);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + buf);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
  }
}

// ---------------------------------------------------------------------------
// The persistent form on pairs of processors: a cluster of two CTAs computes tiles of 256 x 256 with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of X and HALF of the tile's 256 rows of W
// (32 KB a stage instead of 48: an MMA reads the other half from the partner's shared memory), and
// holds its 128 rows of the accumulator in its own TMEM.  CTA 0 of the pair (the leader) issues all
// MMAs; the copies of both CTAs report to the leader's `full` barriers, the leader's commits arrive at
// the `empty` and `acc_full` barriers of both, and the tails of both report to the leader's `acc_empty`.
// What it buys: the plain persistent form needs 96 bytes a cycle from the L2 per processor to keep
// its MMAs fed, this one 64.
// ---------------------------------------------------------------------------
#define T2_STAGES 6
#define T2_A_BYTES (TC_BM * TC_BK * 2)
#define T2_B_BYTES (128 * TC_BK * 2)
#define T2_STAGE_BYTES (T2_A_BYTES + T2_B_BYTES)
#define T2_SMEM (T2_STAGES * T2_STAGE_BYTES + 1024 + 256)
#define T2_BAND 8            // pair tiles (256 rows) per band, as TP_BAND

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address of `local` (an address in this CTA's shared memory) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_addr(uint32_t local, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local), "r"(rank));
  return a;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// a copy into this CTA's shared memory whose bytes are counted by a barrier of the pair's leader
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_addr(dst)), "l"(map), "r"(leader_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// arrives at the barrier at this offset in both CTAs of the pair when the MMAs before it are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_addr(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ void t2_tile_origin(int tile, int tiles_m, int tiles_n, int& m0, int& n0) {
  const int per_band = T2_BAND * tiles_n;
  const int band = tile / per_band, within = tile - band * per_band;
  const int rows = min(T2_BAND, tiles_m - band * T2_BAND);
  const int col = within / rows;
  m0 = (band * T2_BAND + (within - col * rows)) * (2 * TC_BM);
  n0 = col * TP_BN;
}

template <int EPI>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ Y, const float* __restrict__ bias, int* __restrict__ status, int M, int N,
                    int K, int ldy, int tiles_m, int n_tiles) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(base + T2_STAGES * T2_STAGE_BYTES);
  uint64_t* empty = full + T2_STAGES;
  uint64_t* acc_full = empty + T2_STAGES;      // [2] the MMAs of a tile are done (arrives in both CTAs)
  uint64_t* acc_empty = acc_full + 2;          // [2] leader's: the tails of both CTAs have read the buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (K + TC_BK - 1) / TC_BK;
  const int tiles_n = n_tiles / tiles_m;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T2_STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();          // the partner's barriers are initialised before anything arrives at them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      const int first = pair;
      const int early = first < n_tiles ? min(nkb, T2_STAGES) : 0;
      int n0_first = 0, m0_first = 0;
      if (first < n_tiles) t2_tile_origin(first, tiles_m, tiles_n, m0_first, n0_first);
      // weights of the first stages before the wait (they do not depend on the kernel before)
      for (int i = 0; i < early; ++i) {
        if (leader) mbar_expect_tx(full + i, 2 * T2_STAGE_BYTES);
        tma_load_2d_pair(base + i * T2_STAGE_BYTES + T2_A_BYTES, &map_w, i * TC_BK, n0_first + (int)rank * 128,
                         cluster_addr(smem_addr(full + i), 0));
      }
      pdl_wait();
      pdl_trigger();
      for (int i = 0; i < early; ++i)
        tma_load_2d_pair(base + i * T2_STAGE_BYTES, &map_x, i * TC_BK, m0_first + (int)rank * TC_BM,
                         cluster_addr(smem_addr(full + i), 0));
      for (int tile = first; tile < n_tiles && ok; tile += n_pairs) {
        int m0, n0;
        t2_tile_origin(tile, tiles_m, tiles_n, m0, n0);
        for (int kb = (tile == first ? early : 0); kb < nkb; ++kb) {
          const int i = it + kb;
          const int s = i % T2_STAGES;
          if (i >= T2_STAGES && !mbar_wait(empty + s, ((i / T2_STAGES) - 1) & 1)) { atomicExch(status, 31); ok = false; break; }
          if (leader) mbar_expect_tx(full + s, 2 * T2_STAGE_BYTES);
          const uint32_t bar = cluster_addr(smem_addr(full + s), 0);
          tma_load_2d_pair(base + s * T2_STAGE_BYTES + T2_A_BYTES, &map_w, kb * TC_BK, n0 + (int)rank * 128, bar);
          tma_load_2d_pair(base + s * T2_STAGE_BYTES, &map_x, kb * TC_BK, m0 + (int)rank * TC_BM, bar);
        }
        it += nkb;
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0 && leader) {
      // M = 256 (128 rows in each CTA), N = 256
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TP_BN >> 3) << 17) |
                                 ((uint32_t)((2 * TC_BM) >> 4) << 24);
      int it = 0, lt = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++lt) {
        const int buf = lt & 1;
        if (lt >= 2 && !mbar_wait(acc_empty + buf, ((lt >> 1) - 1) & 1)) { atomicExch(status, 32); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem + (uint32_t)buf * TP_BN;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % T2_STAGES;
          if (!mbar_wait(full + s, (it / T2_STAGES) & 1)) { atomicExch(status, 33); ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_addr(base + s * T2_STAGE_BYTES), sb = sa + T2_A_BYTES;
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)
            umma_bf16_pair(acc, umma_desc(sa + k * 32), umma_desc(sb + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(empty + s);
        }
        if (ok) umma_commit_pair(acc_full + buf);
      }
    }
  } else {
    pdl_wait();
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    int lt = 0;
    bool ok = true;
    for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++lt) {
      const int buf = lt & 1;
      int m0, n0;
      t2_tile_origin(tile, tiles_m, tiles_n, m0, n0);
      ok = mbar_wait(acc_full + buf, (lt >> 1) & 1);
      if (!ok) atomicExch(status, 34);
      ok = __all_sync(0xffffffffu, ok);      // tcgen05.ld below is warp-wide
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c0 = 0; c0 < TP_BN; c0 += 16) {
        float v[16];
        tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * TP_BN + c0, v);
        tail16<EPI, false>(v, m0 + (int)rank * TC_BM + row, n0 + c0, M, N, bias, Y, ldy, lane);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(cluster_addr(smem_addr(acc_empty + buf), 0));
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();          // neither CTA gives its TMEM back, or leaves, while the other still works
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [rows, K] bfloat16, K contiguous, boxes of 64 k x box_rows rows, 128-byte swizzle, zeros outside
static bool make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int* status_word() {
  static int* p[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!p[dev]) {
    if (cudaMalloc(&p[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p[dev], 0, sizeof(int));
  }
  return p[dev];
}

// 0 if no kernel of this library gave up on a barrier since the last call; else the code it left.
// Synchronises the device.
AB_API int ab_gemm_tc_status() {
  int* p = status_word();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(p, 0, sizeof(int));
  return v;
}

template <int BN, int EPI, bool SWAP>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, void* Y, const float* bias, float* partials,
                     int* arrivals, int* status, int rows_a, int rows_b, int K, int ldy, int slices,
                     cudaStream_t stream) {
  using S = TcShape<BN>;
  cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM);
  if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;
  const int n_kblocks = (K + TC_BK - 1) / TC_BK;
  const int per = (n_kblocks + slices - 1) / slices;
  dim3 grid((rows_a + TC_BM - 1) / TC_BM, (rows_b + BN - 1) / BN, (n_kblocks + per - 1) / per);
  e = ab_launch(gemm_tc_kernel<BN, EPI, SWAP>, grid, dim3(TC_THREADS), (size_t)S::SMEM, stream, ma, mb, Y, bias,
                partials, arrivals, status, rows_a, rows_b, K, ldy, per);
  if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;
  return ab_launch_status();
}

template <int EPI, bool SWAP>
static int pick_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, void* Y, const float* bias, float* partials,
                   int* arrivals, int* status, int rows_a, int rows_b, int K, int ldy, int slices, cudaStream_t stream) {
  switch (bn) {
    case 16: return launch_tc<16, EPI, SWAP>(ma, mb, Y, bias, partials, arrivals, status, rows_a, rows_b, K, ldy, slices, stream);
    case 32: return launch_tc<32, EPI, SWAP>(ma, mb, Y, bias, partials, arrivals, status, rows_a, rows_b, K, ldy, slices, stream);
    case 64: return launch_tc<64, EPI, SWAP>(ma, mb, Y, bias, partials, arrivals, status, rows_a, rows_b, K, ldy, slices, stream);
    case 128: return launch_tc<128, EPI, SWAP>(ma, mb, Y, bias, partials, arrivals, status, rows_a, rows_b, K, ldy, slices, stream);
    case 256: return launch_tc<256, EPI, SWAP>(ma, mb, Y, bias, partials, arrivals, status, rows_a, rows_b, K, ldy, slices, stream);
  }
  return AB_BAD_ARG;
}

// Y = X[M,K] . W[N,K]^T with an epilogue (0 bfloat16, 1 float32, 2 SwiGLU: W = interleaved gate|up,
// Y [M, N/2]).  swap = 1: the weights fill the 128-row MMA operand and the batch (M <= 256) the
// columns; bn = MMA columns per tile (16..256, a power of two).  slices > 1 needs scratch: partials
// float [tiles * slices * 128 * bn], arrivals int [tiles] (zero before, left zero).
AB_API int ab_gemm_tc(const void* X, const void* W, const float* bias, void* Y, float* partials, int* arrivals,
                      int M, int N, int K, int ldy, int epilogue_kind, int swap, int bn, int slices,
                      cudaStream_t stream) {
  if (M <= 0 || N <= 0) return AB_OK;
  if (K <= 0 || (K % 8) || slices < 1) return AB_BAD_ARG;
  if (epilogue_kind == EPI_SWIGLU_BF16 && (N % 16)) return AB_BAD_ARG;
  if (slices > 1 && (!partials || !arrivals)) return AB_BAD_ARG;
  int* status = status_word();
  if (!status) return AB_BAD_ARG;
  CUtensorMap ma, mb;
  const int rows_a = swap ? N : M, rows_b = swap ? M : N;
  if (!make_map(&ma, swap ? W : X, rows_a, K, TC_BM)) return AB_BAD_ARG;
  if (!make_map(&mb, swap ? X : W, rows_b, K, bn)) return AB_BAD_ARG;
#define AB_GO(E)                                                                                                   \
  return swap ? pick_bn<E, true>(bn, ma, mb, Y, bias, partials, arrivals, status, rows_a, rows_b, K, ldy, slices, stream) \
              : pick_bn<E, false>(bn, ma, mb, Y, bias, partials, arrivals, status, rows_a, rows_b, K, ldy, slices, stream)
  switch (epilogue_kind) {
    case EPI_STORE_BF16: AB_GO(EPI_STORE_BF16);
    case EPI_STORE_F32: AB_GO(EPI_STORE_F32);
    case EPI_SWIGLU_BF16: AB_GO(EPI_SWIGLU_BF16);
  }
#undef AB_GO
  return AB_BAD_ARG;
}

// The persistent form: Y = X[M,K] . W[N,K]^T for many rows, tiles of 128 x 256, one CTA per processor.
AB_API int ab_gemm_tc_persistent(const void* X, const void* W, const float* bias, void* Y, int M, int N, int K,
                                 int ldy, int epilogue_kind, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return AB_OK;
  if (K <= 0 || (K % 8)) return AB_BAD_ARG;
  if (epilogue_kind == EPI_SWIGLU_BF16 && (N % 16)) return AB_BAD_ARG;
  int* status = status_word();
  if (!status) return AB_BAD_ARG;
  CUtensorMap mx, mw;
  if (!make_map(&mx, X, M, K, TC_BM)) return AB_BAD_ARG;
  if (!make_map(&mw, W, N, K, TP_BN)) return AB_BAD_ARG;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (N + TP_BN - 1) / TP_BN;
  const int n_tiles = tiles_m * tiles_n;
  const int grid = n_tiles < sms ? n_tiles : sms;
#define AB_GO(E)                                                                                                   \
  {                                                                                                                \
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM); \
    if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;                                                             \
    e = ab_launch(gemm_tc_persistent_kernel<E>, dim3(grid), dim3(TC_THREADS), (size_t)TP_SMEM, stream, mx, mw, Y,  \
                  bias, status, M, N, K, ldy, tiles_m, n_tiles);                                                   \
    if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;                                                             \
    return ab_launch_status();                                                                                     \
  }
  switch (epilogue_kind) {
    case EPI_STORE_BF16: AB_GO(EPI_STORE_BF16)
    case EPI_STORE_F32: AB_GO(EPI_STORE_F32)
    case EPI_SWIGLU_BF16: AB_GO(EPI_SWIGLU_BF16)
  }
#undef AB_GO
  return AB_BAD_ARG;
}

// The persistent form on pairs of processors (tiles of 256 x 256, tcgen05.mma.cta_group::2).
AB_API int ab_gemm_tc_pair(const void* X, const void* W, const float* bias, void* Y, int M, int N, int K,
                           int ldy, int epilogue_kind, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return AB_OK;
  if (K <= 0 || (K % 8)) return AB_BAD_ARG;
  if (epilogue_kind == EPI_SWIGLU_BF16 && (N % 16)) return AB_BAD_ARG;
  int* status = status_word();
  if (!status) return AB_BAD_ARG;
  CUtensorMap mx, mw;
  if (!make_map(&mx, X, M, K, TC_BM)) return AB_BAD_ARG;
  if (!make_map(&mw, W, N, K, 128)) return AB_BAD_ARG;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles_m = (M + 2 * TC_BM - 1) / (2 * TC_BM), tiles_n = (N + TP_BN - 1) / TP_BN;
  const int n_tiles = tiles_m * tiles_n;
  const int pairs = n_tiles < sms / 2 ? n_tiles : sms / 2;
#define AB_GO(E)                                                                                                   \
  {                                                                                                                \
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM); \
    if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;                                                             \
    cudaLaunchConfig_t cfg = {};                                                                                   \
    cfg.gridDim = dim3(2 * pairs);                                                                                 \
    cfg.blockDim = dim3(TC_THREADS);                                                                               \
    cfg.dynamicSmemBytes = (size_t)T2_SMEM;                                                                        \
    cfg.stream = stream;                                                                                           \
    cudaLaunchAttribute attr[2];                                                                                   \
    attr[0].id = cudaLaunchAttributeClusterDimension;                                                              \
    attr[0].val.clusterDim.x = 2;                                                                                  \
    attr[0].val.clusterDim.y = 1;                                                                                  \
    attr[0].val.clusterDim.z = 1;                                                                                  \
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                               \
    attr[1].val.programmaticStreamSerializationAllowed = 1;                                                        \
    cfg.attrs = attr;                                                                                              \
    cfg.numAttrs = (ab_pdl_enabled() && !ab_pdl_held) ? 2 : 1;                                                     \
    e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<E>, mx, mw, Y, bias, status, M, N, K, ldy, tiles_m, n_tiles); \
    if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;                                                             \
    return ab_launch_status();                                                                                     \
  }
  switch (epilogue_kind) {
    case EPI_STORE_BF16: AB_GO(EPI_STORE_BF16)
    case EPI_STORE_F32: AB_GO(EPI_STORE_F32)
    case EPI_SWIGLU_BF16: AB_GO(EPI_SWIGLU_BF16)
  }
#undef AB_GO
  return AB_BAD_ARG;
}
