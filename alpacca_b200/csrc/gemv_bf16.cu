// Skinny matrix product for decode steps: Y[M,N] = X[M,K] . W[N,K]^T with few
// rows M (one per sequence of the batch) and bfloat16 operands.
//
// The weights are read exactly once, in 16-byte pieces; the products run on the
// tensor cores (mma.sync m16n8k16, float32 accumulation) with the weights as the
// 16-row operand and the batch as the 8-column operand, so any M up to 8 costs
// one instruction per 16 weight rows x 16 k, and M up to 32 two to four.
//
// The kernel is bound by memory latency, not arithmetic: what matters is how
// many bytes are in flight.  A CTA owns 16 weight rows and one of S slices of K
// (grid N/16 x S); its 8 warps split the slice into runs, and every thread issues the loads
// of up to 8 k-groups (256 bytes) before it consumes any, so a CTA of a
// 2048-wide slice has all its 64 KB in flight at once.  A matrix with no more
// 16-row slabs than the device has processors and a long K (the down projection)
// gets CTAs of 16 warps instead: one CTA per processor either way, and half as
// many rounds of loads one after the other.  S is chosen by the host
// so that even a matrix of few rows gives a few CTAs to every processor.  The
// weights do not depend on earlier kernels, so their loads are issued before the
// wait of programmatic dependent launch and overlap the predecessor's tail.
//
// Sums: the warps' partial sums are added in shared memory in warp order; with
// S > 1 each CTA writes its tile of partial sums to scratch memory and the CTA
// that arrives last for its 16 rows adds the S tiles in slice order and runs the
// epilogue.  Both orders are fixed: a result does not depend on timing.
//
// k is permuted inside each group of 32 so that a thread's two 16-byte loads
// (8 consecutive k of weight rows g and g+8) are its operand registers of two
// MMAs as they are; the batch operand is loaded with the same permutation, so
// the sums are over the same pairs.
//
// Epilogues: plain store (bfloat16 or float32, + bias), or SwiGLU on the fused
// gate|up matrix whose rows are interleaved in groups of 8 (rows 16q..16q+7
// gate, 16q+8..16q+15 up): act[m, 8q+g] = silu(gate) * up
// (alpacca/model.py:513), so the activation costs no pass of its own.
//
// The norm between two products, without a kernel of its own.  An RMS norm is
// x = r * w / rms(r) with r the residual row (alpacca/tensor.py:163-173); the division
// is one factor per row, so it can be applied to the sums of the product that reads
// x instead of to x.  The "residual" epilogue of the product BEFORE the norm adds
// its result to the float32 residual in place, stores bf16(r * w) as the next
// product's input and writes, per 16-column slab, the sum of r^2 of every row
// (float32, from the unrounded residual).  The product AFTER the norm is given
// those partial sums: each CTA adds a row's partials in a fixed order, and its
// epilogue multiplies the sums by 1 / sqrt(sum / width + eps) before the bias.
// bf16(r * w) / rms has the same relative rounding error as bf16(r * w / rms).
// What it is worth (B200, 8 rows, width 2048): a reader whose grid is resident at once (qkv,
// 192 CTAs) is as fast with the owed division as without, the residual epilogue costs the
// product before it up to 0.9 us, and the norm kernel saved took 2.3 us.  A reader of several
// waves (gate|up, the vocabulary head) loses more than that: there every 0.1 us that a CTA spends
// without loads in flight costs memory rate, and the sums of squares need a barrier more
// (measured 12.6 -> 14.7 to 17.3 us for gate|up in four forms of the reduction, among them CTAs
// that stay and walk the slabs with the next slab's loads under the tail: 15.5 us).  The host
// therefore asks for it only when the reader's slabs fit the device at once.
#include "common.cuh"
#include "launch.cuh"

#define GEMV_WARPS 8
#define GEMV_U 8
#define EPI_STORE_BF16 0
#define EPI_STORE_F32 1
#define EPI_SWIGLU_BF16 2
#define EPI_RESIDUAL_BF16 3

// What the norm fusion adds to a launch; all null / 0 without it.
struct GemvNorm {
  const float* ss_in;     // [M, n_part_in] partial sums of squares of this product's input rows, or null
  int n_part_in;
  float inv_width, eps;   // rms^2 = sum * inv_width + eps
  float* residual;        // EPI_RESIDUAL: float32 [M, N], updated in place
  const float* norm_w;    // EPI_RESIDUAL: float32 [N], the weight of the norm that follows
  float* ss_out;          // EPI_RESIDUAL: float32 [M, ceil(N / 16)]
};

__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// activations were written by the kernel before this one: a plain (coherent) load, not the
// read-only path, whose lines might have been fetched before the predecessor finished
__device__ __forceinline__ uint4 ld_act(const bf16* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void cp_async_cg16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

template <int EPI>
__device__ __forceinline__ void epilogue(const float acc[4], int i, int ln, int n0, const float* __restrict__ bias,
                                         void* __restrict__ Y, int M, int N, int ldy, const float* rstd,
                                         const GemvNorm& nf, const float* res_tile, const float* nw_tile) {
  const int gg = ln >> 2, tt = ln & 3;
  const int m0 = i * 8 + 2 * tt;             // batch rows m0, m0 + 1
  const int na = n0 + gg, nb = n0 + gg + 8;  // weight rows of c[0..1] and c[2..3]
  float c[4] = {acc[0], acc[1], acc[2], acc[3]};
  if (rstd) {                                // the division by the rms that the input rows still owe
    const float r0 = rstd[m0], r1 = rstd[m0 + 1];
    c[0] *= r0; c[1] *= r1; c[2] *= r0; c[3] *= r1;
  }
  if (EPI == EPI_SWIGLU_BF16) {
    // na is a gate row, nb the up row of the same unit: output column (n0 / 16) * 8 + gg
    if (na < N) {
      const float bg = bias ? bias[na] : 0.f, bu = bias ? bias[nb] : 0.f;
      const int col = (n0 >> 1) + gg;
      bf16* y = reinterpret_cast<bf16*>(Y);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if (m0 + j < M) {
          const float gate = c[j] + bg, up = c[2 + j] + bu;
          y[(size_t)(m0 + j) * ldy + col] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
        }
      }
    }
  } else if (EPI == EPI_RESIDUAL_BF16) {
    float sq[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = (j < 2) ? na : nb, m = m0 + (j & 1);
      if (n < N && m < M) {
        // the residual tile and the norm weights were staged in shared memory while the weights streamed
        const float before = res_tile ? res_tile[m * 16 + (n - n0)] : __ldcg(nf.residual + (size_t)m * N + n);
        const float w = nw_tile ? nw_tile[n - n0] : nf.norm_w[n];
        const float r = before + (c[j] + (bias ? bias[n] : 0.f));
        nf.residual[(size_t)m * N + n] = r;
        reinterpret_cast<bf16*>(Y)[(size_t)m * ldy + n] = __float2bfloat16_rn(r * w);
        sq[j & 1] += r * r;
      }
    }
    // a row's 16 columns lie in the 8 lanes of equal tt: added in a fixed order
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      sq[0] += __shfl_xor_sync(0xffffffffu, sq[0], o);
      sq[1] += __shfl_xor_sync(0xffffffffu, sq[1], o);
    }
    if (gg == 0) {
      const int n_slabs = (N + 15) >> 4;
      if (m0 < M) nf.ss_out[(size_t)m0 * n_slabs + (n0 >> 4)] = sq[0];
      if (m0 + 1 < M) nf.ss_out[(size_t)(m0 + 1) * n_slabs + (n0 >> 4)] = sq[1];
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = (j < 2) ? na : nb, m = m0 + (j & 1);
      if (n < N && m < M) {
        const float v = c[j] + (bias ? bias[n] : 0.f);
        if (EPI == EPI_STORE_F32) reinterpret_cast<float*>(Y)[(size_t)m * ldy + n] = v;
        else reinterpret_cast<bf16*>(Y)[(size_t)m * ldy + n] = __float2bfloat16_rn(v);
      }
    }
  }
}

// SCALED: the input rows owe the division by their rms (nf.ss_in is given)
template <int NT, int EPI, int WARPS, bool SCALED>
__global__ void __launch_bounds__(WARPS * 32)
gemv_bf16_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, const float* __restrict__ bias,
                 void* __restrict__ Y, float* __restrict__ partials, int* __restrict__ arrivals, int M, int N, int K,
                 int ldy, int groups_per_slice, const GemvNorm nf) {
  __shared__ float red[WARPS][NT][32][4];
  // what the epilogue needs from earlier kernels is copied into shared memory asynchronously right
  // after the wait (no registers, nothing for the main loop to wait on): the input rows' partial sums
  // of squares, and for the residual epilogue this CTA's tile of the residual and the norm's weights
  constexpr int SS_CAP = NT <= 2 ? 256 : 128;
  __shared__ __align__(16) float ss_s[SCALED ? NT * 8 * SS_CAP : 4];
  __shared__ float rstd_s[SCALED ? NT * 8 : 1];
  __shared__ __align__(16) float res_s[EPI == EPI_RESIDUAL_BF16 ? NT * 8 * 16 : 4];
  __shared__ __align__(16) float nw_s[EPI == EPI_RESIDUAL_BF16 ? 16 : 4];
  __shared__ int is_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int S = gridDim.y, slice = blockIdx.y;
  // rows past N read row N-1 again; their sums are never stored
  const bf16* w_lo = W + (size_t)min(n0 + g, N - 1) * K;
  const bf16* w_hi = W + (size_t)min(n0 + g + 8, N - 1) * K;
  const bf16* x_row[NT];
  bool x_ok[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    x_ok[i] = (i * 8 + g) < M;
    x_row[i] = X + (size_t)(x_ok[i] ? i * 8 + g : 0) * K;
  }
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  // this CTA's k-groups (32 k each): [slice_begin, slice_end); each warp takes a contiguous run of
  // them, so that a thread's consecutive loads complete the 128-byte lines they touch
  const int n_groups = (K + 31) / 32;
  const int slice_begin = slice * groups_per_slice;
  const int slice_end = min(n_groups, slice_begin + groups_per_slice);
  const int per_warp = (slice_end - slice_begin + WARPS - 1) / WARPS;
  const int grp_begin = slice_begin + warp * per_warp;
  const int grp_end = min(slice_end, grp_begin + per_warp);
  const bool ss_staged = SCALED && (nf.n_part_in % 4) == 0 && nf.n_part_in <= SS_CAP;
  const bool res_staged = EPI == EPI_RESIDUAL_BF16 && (N % 4) == 0;
  if (res_staged && threadIdx.x < 4 && n0 + (int)threadIdx.x * 4 < N)      // constant: before the wait
    cp_async_cg16(nw_s + threadIdx.x * 4, nf.norm_w + n0 + threadIdx.x * 4);
  auto after_wait = [&]() {
    if (ss_staged) {
      const int per_row = nf.n_part_in >> 2;
      for (int c = threadIdx.x; c < M * per_row; c += WARPS * 32) {
        const int r = c / per_row, q = c - r * per_row;
        cp_async_cg16(ss_s + r * SS_CAP + q * 4, nf.ss_in + (size_t)r * nf.n_part_in + q * 4);
      }
    }
    if (res_staged) {
      for (int c = threadIdx.x; c < M * 4; c += WARPS * 32) {
        const int r = c >> 2, q = c & 3;
        if (n0 + q * 4 < N) cp_async_cg16(res_s + r * 16 + q * 4, nf.residual + (size_t)r * N + n0 + q * 4);
      }
    }
  };
  bool waited = false;
  for (int grp = grp_begin; grp < grp_end; grp += GEMV_U) {
    uint4 wl[GEMV_U], wh[GEMV_U];
#pragma unroll
    for (int u = 0; u < GEMV_U; ++u) {
      const int gi = grp + u;
      const int k = gi * 32 + t * 8;
      if (gi < grp_end && k < K) {   // K is a multiple of 8: a piece of 8 lies inside or outside as a whole
        wl[u] = ldg_stream(w_lo + k);
        wh[u] = ldg_stream(w_hi + k);
      } else {
        wl[u] = wh[u] = make_uint4(0, 0, 0, 0);
      }
    }
    if (!waited) { pdl_wait(); pdl_trigger(); waited = true; after_wait(); }
    // the batch operand, four k-groups at a time: loaded together, then consumed
#pragma unroll
    for (int u0 = 0; u0 < GEMV_U; u0 += 4) {
      uint4 xv[4][NT];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int gi = grp + u0 + u;
        const int k = gi * 32 + t * 8;
        const bool in = gi < grp_end && k < K;
#pragma unroll
        for (int i = 0; i < NT; ++i) xv[u][i] = (in && x_ok[i]) ? ld_act(x_row[i] + k) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          mma_bf16_16816(acc[i], wl[u0 + u].x, wh[u0 + u].x, wl[u0 + u].y, wh[u0 + u].y, xv[u][i].x, xv[u][i].y);
          mma_bf16_16816(acc[i], wl[u0 + u].z, wh[u0 + u].z, wl[u0 + u].w, wh[u0 + u].w, xv[u][i].z, xv[u][i].w);
        }
      }
    }
  }
  if (!waited) { pdl_wait(); pdl_trigger(); after_wait(); }

#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) red[warp][i][lane][j] = acc[i][j];
  if (SCALED || EPI == EPI_RESIDUAL_BF16) cp_async_wait_all();
  __syncthreads();
  if (SCALED) {
    // warp w adds the partial sums of rows w, w + WARPS, ..: lanes stride the row, then the lanes' sums
    // are added in a fixed order
    for (int r = warp; r < M; r += WARPS) {
      float sum = 0.f;
      if (ss_staged) {
        for (int pi = lane; pi < nf.n_part_in; pi += 32) sum += ss_s[r * SS_CAP + pi];
      } else {
        for (int pi = lane; pi < nf.n_part_in; pi += 32) sum += __ldcg(nf.ss_in + (size_t)r * nf.n_part_in + pi);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) rstd_s[r] = rsqrtf(sum * nf.inv_width + nf.eps);
    }
  }
  const float* rstd = SCALED ? rstd_s : nullptr;
  const float* res_tile = res_staged ? res_s : nullptr;
  const float* nw_tile = res_staged ? nw_s : nullptr;
  // threads 0 .. NT*32-1 finish one (n-tile, lane) each
  const bool finisher = threadIdx.x < NT * 32;
  const int i = threadIdx.x >> 5, ln = threadIdx.x & 31;
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  if (finisher) {
#pragma unroll
    for (int w = 0; w < WARPS; ++w)
#pragma unroll
      for (int j = 0; j < 4; ++j) c[j] += red[w][i][ln][j];
  }
  if (SCALED) __syncthreads();      // rstd_s is complete
  if (S == 1) {
    if (finisher) epilogue<EPI>(c, i, ln, n0, bias, Y, M, N, ldy, rstd, nf, res_tile, nw_tile);
    return;
  }
  // several slices: park this CTA's tile; the CTA that arrives last adds the tiles in slice order
  float* tile = partials + ((size_t)blockIdx.x * S) * (NT * 128);
  if (finisher)
    *reinterpret_cast<float4*>(tile + (size_t)slice * (NT * 128) + threadIdx.x * 4) = make_float4(c[0], c[1], c[2], c[3]);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int seen = atomicAdd(arrivals + blockIdx.x, 1);
    is_last = (seen == S - 1);
    if (is_last) arrivals[blockIdx.x] = 0;     // left at zero for the next launch
  }
  __syncthreads();
  if (!is_last || !finisher) return;
  __threadfence();
  c[0] = c[1] = c[2] = c[3] = 0.f;
  for (int s = 0; s < S; ++s) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(tile + (size_t)s * (NT * 128) + threadIdx.x * 4));
    c[0] += v.x; c[1] += v.y; c[2] += v.z; c[3] += v.w;
  }
  epilogue<EPI>(c, i, ln, n0, bias, Y, M, N, ldy, rstd, nf, res_tile, nw_tile);
}

static int gemv_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int EPI>
static int launch(const void* X, const void* W, const float* bias, void* Y, float* partials, int* arrivals, int M,
                  int N, int K, int ldy, int slices, int wide, const GemvNorm& nf, cudaStream_t stream) {
  const int n_groups = (K + 31) / 32;
  const int gps = (n_groups + slices - 1) / slices;
  const dim3 grid((unsigned)((N + 15) / 16), (unsigned)((n_groups + gps - 1) / gps));
#define AB_GO(NT, WARPS)                                                                                           \
  {                                                                                                                \
    if (nf.ss_in)                                                                                                  \
      ab_launch(gemv_bf16_kernel<NT, EPI, WARPS, true>, grid, dim3(WARPS * 32), 0, stream, (const bf16*)X,         \
                (const bf16*)W, bias, Y, partials, arrivals, M, N, K, ldy, gps, nf);                               \
    else                                                                                                           \
      ab_launch(gemv_bf16_kernel<NT, EPI, WARPS, false>, grid, dim3(WARPS * 32), 0, stream, (const bf16*)X,        \
                (const bf16*)W, bias, Y, partials, arrivals, M, N, K, ldy, gps, nf);                               \
  }
  if (M <= 8) { if (wide) AB_GO(1, 16) else AB_GO(1, GEMV_WARPS) }
  else if (M <= 16) { if (wide) AB_GO(2, 16) else AB_GO(2, GEMV_WARPS) }
  else AB_GO(4, GEMV_WARPS)
#undef AB_GO
  return ab_launch_status();
}

// How many slices of K the host should ask for.  Measured on a B200 (2048x2048, 3072x2048,
// 16384x2048, 2048x8192): the merge of the slices (fence, counter, second pass) costs more than the
// added CTAs gain, even for the 128-CTA shapes, so one slice unless K is far longer than any of those.
AB_API int ab_gemv_bf16_slices(int N, int K, int n_sms) {
  const int slabs = (N + 15) / 16;
  if (K < 32768 || slabs >= n_sms) return 1;
  int s = (n_sms + slabs - 1) / slabs;
  return s > 8 ? 8 : s;
}

// epilogue_kind: 0 bfloat16 store, 1 float32 store, 2 SwiGLU (N = 2F interleaved rows, Y is [M, F]),
// 3 residual (see the head of this file): residual float32 [M, N] is updated in place, Y bfloat16 [M, N]
// becomes bf16(residual * norm_w), ss_out float32 [M, ceil(N / 16)] the slabs' sums of squares.
// ss_in (any epilogue, or null): float32 [M, n_part_in], the partial sums of squares of X's rows, whose
// division by sqrt(sum * inv_width + eps) is applied to this product's sums.
// slices > 1 needs scratch: partials float [ceil(N/16) * slices * 128 * (1, 2 or 4 for M <= 8, 16, 32)],
// arrivals int [ceil(N/16)], zero before the first launch and left zero by every launch.
AB_API int ab_gemv_bf16_norm(const void* X, const void* W, const float* bias, void* Y, float* partials,
                             int* arrivals, int M, int N, int K, int ldy, int epilogue_kind, int slices,
                             const float* ss_in, int n_part_in, float inv_width, float eps, float* residual,
                             const float* norm_w, float* ss_out, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return AB_OK;
  if (M > 32 || K <= 0 || (K % 8) || slices < 1 || slices > 65535) return AB_BAD_ARG;
  if (slices > 1 && (!partials || !arrivals)) return AB_BAD_ARG;
  if (epilogue_kind == EPI_SWIGLU_BF16 && (N % 16)) return AB_BAD_ARG;
  if (epilogue_kind == EPI_RESIDUAL_BF16 && (!residual || !norm_w || !ss_out || ldy != N)) return AB_BAD_ARG;
  if (ss_in && (n_part_in < 1 || !(inv_width > 0.f))) return AB_BAD_ARG;
  GemvNorm nf;
  nf.ss_in = ss_in; nf.n_part_in = ss_in ? n_part_in : 0; nf.inv_width = inv_width; nf.eps = eps;
  nf.residual = residual; nf.norm_w = norm_w; nf.ss_out = ss_out;
  // few slabs and more than one round of loads per warp: 16 warps per CTA
  const int wide = (M <= 16 && slices == 1 && (N + 15) / 16 <= gemv_sm_count() && K > 8 * GEMV_U * 32) ? 1 : 0;
  switch (epilogue_kind) {
    case EPI_STORE_BF16: return launch<EPI_STORE_BF16>(X, W, bias, Y, partials, arrivals, M, N, K, ldy, slices, wide, nf, stream);
    case EPI_STORE_F32: return launch<EPI_STORE_F32>(X, W, bias, Y, partials, arrivals, M, N, K, ldy, slices, wide, nf, stream);
    case EPI_SWIGLU_BF16: return launch<EPI_SWIGLU_BF16>(X, W, bias, Y, partials, arrivals, M, N, K, ldy, slices, wide, nf, stream);
    case EPI_RESIDUAL_BF16: return launch<EPI_RESIDUAL_BF16>(X, W, bias, Y, partials, arrivals, M, N, K, ldy, slices, wide, nf, stream);
  }
  return AB_BAD_ARG;
}

AB_API int ab_gemv_bf16(const void* X, const void* W, const float* bias, void* Y, float* partials, int* arrivals,
                        int M, int N, int K, int ldy, int epilogue_kind, int slices, cudaStream_t stream) {
  if (epilogue_kind == EPI_RESIDUAL_BF16) return AB_BAD_ARG;
  return ab_gemv_bf16_norm(X, W, bias, Y, partials, arrivals, M, N, K, ldy, epilogue_kind, slices, nullptr, 0, 0.f,
                           0.f, nullptr, nullptr, nullptr, stream);
}
