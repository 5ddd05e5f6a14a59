// Skinny matrix product for decode steps: Y[M,N] = X[M,K] . W[N,K]^T with few
// rows M (one per sequence of the batch) and bfloat16 operands.
//
// The weights are read exactly once, in 16-byte pieces; the products run on the
// tensor cores (mma.sync m16n8k16, float32 accumulation) with the weights as the
// 16-row operand and the batch as the 8-column operand, so any M up to 8 costs
// one instruction per 16 weight rows x 16 k, and M up to 32 two to four.
// A CTA owns 16 weight rows; its 8 warps split K between them and their partial
// sums are added in shared memory in warp order (a fixed order: the result of
// a row does not depend on timing).
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
#include "common.cuh"
#include "launch.cuh"

#define GEMV_WARPS 8
#define EPI_STORE_BF16 0
#define EPI_STORE_F32 1
#define EPI_SWIGLU_BF16 2

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

template <int NT, int EPI>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_bf16_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, const float* __restrict__ bias,
                 void* __restrict__ Y, int M, int N, int K, int ldy) {
  __shared__ float red[GEMV_WARPS][NT][32][4];
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
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

  // warp w takes the k-groups w, w + 8, w + 16, ... (32 k each); 4 groups are in flight per thread
  constexpr int U = 4;
  const int n_groups = (K + 31) / 32;
  // The weights do not depend on earlier kernels: the first loads of them go out before the
  // wait for the predecessor, whose tail they overlap; the batch operand is read after it.
  bool waited = false;
  for (int grp = warp; grp < n_groups; grp += GEMV_WARPS * U) {
    uint4 wl[U], wh[U], xv[U][NT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (grp + u * GEMV_WARPS) * 32 + t * 8;
      if (k < K) {           // K is a multiple of 8: a group of 8 lies inside or outside as a whole
        wl[u] = ldg_stream(w_lo + k);
        wh[u] = ldg_stream(w_hi + k);
      } else {
        wl[u] = wh[u] = make_uint4(0, 0, 0, 0);
      }
    }
    if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (grp + u * GEMV_WARPS) * 32 + t * 8;
#pragma unroll
      for (int i = 0; i < NT; ++i)
        xv[u][i] = (k < K && x_ok[i]) ? ld_act(x_row[i] + k) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        mma_bf16_16816(acc[i], wl[u].x, wh[u].x, wl[u].y, wh[u].y, xv[u][i].x, xv[u][i].y);
        mma_bf16_16816(acc[i], wl[u].z, wh[u].z, wl[u].w, wh[u].w, xv[u][i].z, xv[u][i].w);
      }
    }
  }

  if (!waited) pdl_wait();
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) red[warp][i][lane][j] = acc[i][j];
  __syncthreads();
  // threads 0 .. NT*32-1 finish one (n-tile, lane) each
  if (threadIdx.x < NT * 32) {
    const int i = threadIdx.x >> 5, ln = threadIdx.x & 31;
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w)
#pragma unroll
      for (int j = 0; j < 4; ++j) c[j] += red[w][i][ln][j];
    const int gg = ln >> 2, tt = ln & 3;
    const int m0 = i * 8 + 2 * tt;          // batch rows m0, m0 + 1
    const int na = n0 + gg, nb = n0 + gg + 8;  // weight rows of c[0..1] and c[2..3]
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
}

template <int EPI>
static int launch(const void* X, const void* W, const float* bias, void* Y, int M, int N, int K, int ldy,
                  cudaStream_t stream) {
  const unsigned blocks = (unsigned)((N + 15) / 16);
  const int threads = GEMV_WARPS * 32;
#define AB_GO(NT) ab_launch(gemv_bf16_kernel<NT, EPI>, blocks, threads, 0, stream, (const bf16*)X, (const bf16*)W, bias, Y, M, N, K, ldy)
  if (M <= 8) AB_GO(1);
  else if (M <= 16) AB_GO(2);
  else AB_GO(4);
#undef AB_GO
  return ab_launch_status();
}

// epilogue: 0 bfloat16 store, 1 float32 store, 2 SwiGLU (N = 2F interleaved rows, Y is [M, F])
AB_API int ab_gemv_bf16(const void* X, const void* W, const float* bias, void* Y, int M, int N, int K, int ldy,
                        int epilogue, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return AB_OK;
  if (M > 32 || K <= 0 || (K % 8)) return AB_BAD_ARG;
  if (epilogue == EPI_SWIGLU_BF16 && (N % 16)) return AB_BAD_ARG;
  switch (epilogue) {
    case EPI_STORE_BF16: return launch<EPI_STORE_BF16>(X, W, bias, Y, M, N, K, ldy, stream);
    case EPI_STORE_F32: return launch<EPI_STORE_F32>(X, W, bias, Y, M, N, K, ldy, stream);
    case EPI_SWIGLU_BF16: return launch<EPI_SWIGLU_BF16>(X, W, bias, Y, M, N, K, ldy, stream);
  }
  return AB_BAD_ARG;
}
