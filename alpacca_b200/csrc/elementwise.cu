// Memory-bound kernels around the matrix products: embedding gather, fused
// residual add + RMSNorm, rotation of q and k with the append of k and v to the
// paged cache, SwiGLU on the fused gate|up product, bias add.
//
// Arithmetic is 32-bit throughout (sums of squares, scaling, rotation, SiLU);
// T is the storage type of activations, weights and cache (float or bfloat16).
// The residual stream itself is always float.
#include "common.cuh"
#include "launch.cuh"

// ---------------------------------------------------------------------------
// x[t,:] = table[token[t],:]   (alpacca/model.py:482; no scaling)
// Tokens outside the table give a row of NaN, never a read outside it.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                  float* __restrict__ out, int n_rows, int width, int vocab) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  if (row >= n_rows) return;
  const int tok = tokens[row];
  float* o = out + (size_t)row * width;
  if (tok < 0 || tok >= vocab) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = __int_as_float(0x7fc00000);
    return;
  }
  const T* src = table + (size_t)tok * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = to_f32(src[i]);
}

AB_API int ab_embed_rows(const void* table, int dtype, const int* tokens, float* out, int n_rows,
                         int width, int vocab, cudaStream_t stream) {
  if (n_rows <= 0) return AB_OK;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == AB_F32)
    ab_launch(embed_rows_kernel<float>, n_rows, threads, 0, stream, (const float*)table, tokens, out, n_rows, width, vocab);
  else if (dtype == AB_BF16)
    ab_launch(embed_rows_kernel<bf16>, n_rows, threads, 0, stream, (const bf16*)table, tokens, out, n_rows, width, vocab);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

// ---------------------------------------------------------------------------
// Fused residual add + RMSNorm (alpacca/tensor.py:163-173):
//   r = residual[src] (+ delta[src]);  residual[src] = r  (when delta is given and
//   rows == nullptr);  inv = 1/sqrt(mean(r^2) + eps);  out[i] = (r * inv) * w.
// `rows` picks source rows (the final norm runs on the wanted rows only); with
// `rows` the residual is left as it is.  One block per output row; the order
// of the sum depends on the width and the block size only.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int n_out, int width, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int i_out = blockIdx.x;
  if (i_out >= n_out) return;
  const int src = rows ? rows[i_out] : i_out;
  float* r = residual + (size_t)src * width;
  const T* d = delta ? delta + (size_t)src * width : nullptr;
  const bool write_back = (d != nullptr) && (rows == nullptr);
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = r[i];
    if (d) {
      v += to_f32(d[i]);
      if (write_back) r[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  if (out == nullptr) return;
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  T* o = out + (size_t)i_out * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = r[i];
    if (d && !write_back) v += to_f32(d[i]);
    o[i] = from_f32<T>((v * inv) * weight[i]);
  }
}

// The same with 4 elements per access, for widths that are multiples of 4.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  float4 v;
  __device__ __forceinline__ void load(const float* p) { v = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = v; }
  __device__ __forceinline__ float get(int i) const { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
  __device__ __forceinline__ void set(float a, float b, float c, float d) { v = make_float4(a, b, c, d); }
};
template <> struct Vec4<bf16> {
  uint2 v;
  __device__ __forceinline__ void load(const bf16* p) { v = *reinterpret_cast<const uint2*>(p); }
  __device__ __forceinline__ void store(bf16* p) const { *reinterpret_cast<uint2*>(p) = v; }
  __device__ __forceinline__ float get(int i) const {
    const uint32_t w = i < 2 ? v.x : v.y;
    return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
  }
  __device__ __forceinline__ void set(float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
  }
};

template <typename T>
__global__ void add_rmsnorm_vec4_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                        const float* __restrict__ weight, T* __restrict__ out,
                                        const int* __restrict__ rows, int n_out, int width, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int i_out = blockIdx.x;
  if (i_out >= n_out) return;
  const int src = rows ? rows[i_out] : i_out;
  float* r = residual + (size_t)src * width;
  const T* d = delta ? delta + (size_t)src * width : nullptr;
  const bool write_back = (d != nullptr) && (rows == nullptr);
  float ss = 0.f;
  // the order of the sum depends on the width and the block size only
  for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(r + i);
    if (d) {
      Vec4<T> dv;
      dv.load(d + i);
      v.x += dv.get(0); v.y += dv.get(1); v.z += dv.get(2); v.w += dv.get(3);
      if (write_back) *reinterpret_cast<float4*>(r + i) = v;
    }
    ss += v.x * v.x;
    ss += v.y * v.y;
    ss += v.z * v.z;
    ss += v.w * v.w;
  }
  ss = block_sum(ss, scratch);
  if (out == nullptr) return;
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  T* o = out + (size_t)i_out * width;
  for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(r + i);
    if (d && !write_back) {
      Vec4<T> dv;
      dv.load(d + i);
      v.x += dv.get(0); v.y += dv.get(1); v.z += dv.get(2); v.w += dv.get(3);
    }
    const float4 w = *reinterpret_cast<const float4*>(weight + i);
    Vec4<T> ov;
    ov.set((v.x * inv) * w.x, (v.y * inv) * w.y, (v.z * inv) * w.z, (v.w * inv) * w.w);
    ov.store(o + i);
  }
}

// The same for rows short enough that a thread keeps its share in registers (up to RV x 4 elements per
// thread): the row, its delta and the norm weights are asked for at once and read once; the sum runs
// over the same elements in the same order as in the kernel above.
template <typename T, int RV>
__global__ void add_rmsnorm_reg_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                       const float* __restrict__ weight, T* __restrict__ out,
                                       const int* __restrict__ rows, int n_out, int width, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int i_out = blockIdx.x;
  if (i_out >= n_out) return;
  const int src = rows ? rows[i_out] : i_out;
  float* r = residual + (size_t)src * width;
  const T* d = delta ? delta + (size_t)src * width : nullptr;
  const bool write_back = (d != nullptr) && (rows == nullptr);
  float4 v[RV], w[RV];
  Vec4<T> dv[RV];
#pragma unroll
  for (int j = 0; j < RV; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < width) {
      v[j] = *reinterpret_cast<const float4*>(r + i);
      if (d) dv[j].load(d + i);
      if (out) w[j] = *reinterpret_cast<const float4*>(weight + i);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < RV; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < width) {
      if (d) {
        v[j].x += dv[j].get(0); v[j].y += dv[j].get(1); v[j].z += dv[j].get(2); v[j].w += dv[j].get(3);
        if (write_back) *reinterpret_cast<float4*>(r + i) = v[j];
      }
      ss += v[j].x * v[j].x;
      ss += v[j].y * v[j].y;
      ss += v[j].z * v[j].z;
      ss += v[j].w * v[j].w;
    }
  }
  ss = block_sum(ss, scratch);
  if (out == nullptr) return;
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  T* o = out + (size_t)i_out * width;
#pragma unroll
  for (int j = 0; j < RV; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < width) {
      Vec4<T> ov;
      ov.set((v[j].x * inv) * w[j].x, (v[j].y * inv) * w[j].y, (v[j].z * inv) * w[j].z, (v[j].w * inv) * w[j].w);
      ov.store(o + i);
    }
  }
}

AB_API int ab_add_rmsnorm(float* residual, const void* delta, const float* weight, void* out, int dtype,
                          const int* rows, int n_out, int width, float eps, cudaStream_t stream) {
  if (n_out <= 0) return AB_OK;
  if (width % 4 == 0) {
    const int vthreads = width >= 4096 ? 512 : (width >= 1024 ? 256 : 128);
    if (width <= vthreads * 4 * 4 && (dtype == AB_F32 || dtype == AB_BF16)) {
      if (dtype == AB_F32)
        ab_launch(add_rmsnorm_reg_kernel<float, 4>, n_out, vthreads, 0, stream, residual, (const float*)delta, weight,
                  (float*)out, rows, n_out, width, eps);
      else
        ab_launch(add_rmsnorm_reg_kernel<bf16, 4>, n_out, vthreads, 0, stream, residual, (const bf16*)delta, weight,
                  (bf16*)out, rows, n_out, width, eps);
      return ab_launch_status();
    }
    if (dtype == AB_F32)
      ab_launch(add_rmsnorm_vec4_kernel<float>, n_out, vthreads, 0, stream, residual, (const float*)delta, weight,
                (float*)out, rows, n_out, width, eps);
    else if (dtype == AB_BF16)
      ab_launch(add_rmsnorm_vec4_kernel<bf16>, n_out, vthreads, 0, stream, residual, (const bf16*)delta, weight,
                (bf16*)out, rows, n_out, width, eps);
    else
      return AB_BAD_ARG;
    return ab_launch_status();
  }
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  if (dtype == AB_F32)
    ab_launch(add_rmsnorm_kernel<float>, n_out, threads, 0, stream, residual, (const float*)delta, weight,
              (float*)out, rows, n_out, width, eps);
  else if (dtype == AB_BF16)
    ab_launch(add_rmsnorm_kernel<bf16>, n_out, threads, 0, stream, residual, (const bf16*)delta, weight,
              (bf16*)out, rows, n_out, width, eps);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

// ---------------------------------------------------------------------------
// y[t, j] += bias[j]
// ---------------------------------------------------------------------------
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ y, const float* __restrict__ bias, size_t total, int width) {
  pdl_wait();
  pdl_trigger();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  y[i] = from_f32<T>(to_f32(y[i]) + bias[i % width]);
}

AB_API int ab_add_bias(void* y, int dtype, const float* bias, int n_rows, int width, cudaStream_t stream) {
  size_t total = (size_t)n_rows * width;
  if (total == 0) return AB_OK;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == AB_F32)
    ab_launch(add_bias_kernel<float>, blocks, 256, 0, stream, (float*)y, bias, total, width);
  else if (dtype == AB_BF16)
    ab_launch(add_bias_kernel<bf16>, blocks, 256, 0, stream, (bf16*)y, bias, total, width);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

// ---------------------------------------------------------------------------
// Rotation of q and k by position, and append of k and v to the paged cache.
//
// qkv: [n_tokens, (H + 2K) * D], q heads first, then k heads, then v heads.
// Rotation (alpacca/model.py:381-435): pair (a, b) of a head, angle from the
// table row of the token's position: out_a = x_a*c - x_b*s, out_b = x_a*s + x_b*c.
// pairing 0 ("llama"): (2i, 2i+1); pairing 1 ("neox"): (i, n_rot/2 + i);
// dims >= n_rot pass through.  cos/sin == nullptr: no rotation at all.
// q is rotated in place; rotated k and plain v go to the cache (written before
// attention so that a token sees itself, alpacca/model.py:501-503).
// Cache pages: [n_pages][K][page_size][D]; the page of position p of sequence b
// is block_table[b * table_width + p / page_size].  Tokens whose tok_seq is
// negative are padding and are skipped.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, const int* __restrict__ tok_pos,
                                   const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                   int table_width, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                   int n_tokens, int H, int K, int D, int n_rot, int pairing, int page_size,
                                   int write_cache) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const int b = tok_seq[t];
  if (b < 0) return;
  const int pos = tok_pos[t];
  const int half_d = D >> 1, half_r = n_rot >> 1;
  const int n_heads = H + 2 * K;
  T* row = qkv + (size_t)t * n_heads * D;
  const float* c_row = cos_t ? cos_t + (size_t)pos * half_r : nullptr;
  const float* s_row = sin_t ? sin_t + (size_t)pos * half_r : nullptr;
  const int page = block_table[(size_t)b * table_width + pos / page_size];
  const int off = pos % page_size;
  const int units = n_heads * half_d;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    const int head = u / half_d, i = u - head * half_d;
    T* x = row + (size_t)head * D;
    int a, bb;
    float xa, xb;
    if (head < H + K && c_row && i < half_r) {
      if (pairing == 0) { a = 2 * i; bb = a + 1; } else { a = i; bb = half_r + i; }
      const float c = c_row[i], s = s_row[i];
      const float x0 = to_f32(x[a]), x1 = to_f32(x[bb]);
      xa = x0 * c - x1 * s;
      xb = x0 * s + x1 * c;
    } else {
      // pass-through dims (and every dim of v): unit i covers two dims of its own
      if (head < H + K && c_row) { a = n_rot + 2 * (i - half_r); } else { a = 2 * i; }
      bb = a + 1;
      xa = to_f32(x[a]);
      xb = to_f32(x[bb]);
    }
    if (head < H) {
      x[a] = from_f32<T>(xa);
      x[bb] = from_f32<T>(xb);
    } else if (write_cache) {
      const bool is_k = head < H + K;
      const int kh = is_k ? head - H : head - H - K;
      T* dst = (is_k ? k_pages : v_pages) + (((size_t)page * K + kh) * page_size + off) * D;
      dst[a] = from_f32<T>(xa);
      dst[bb] = from_f32<T>(xb);
      if (is_k) {  // keep the rotated k in the step's buffer too (parts that read it there)
        x[a] = from_f32<T>(xa);
        x[bb] = from_f32<T>(xb);
      }
    }
  }
}

// 8 consecutive elements to and from float registers
__device__ __forceinline__ void load8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float* v) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void store8(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float* v) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 r = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&r);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// The same for head sizes and rotated sizes that are multiples of 16: one thread per unit of 16
// elements of a head (two pieces of 8), 16-byte accesses throughout.  A rotated unit u covers the
// pairs 8u .. 8u+7 of its head: with pairing 0 the 16 consecutive elements from 16u (even places a,
// odd places b), with pairing 1 the pieces at 8u and n_rot/2 + 8u.
template <typename T>
__global__ void rope_append_vec_kernel(T* __restrict__ qkv, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, const int* __restrict__ tok_pos,
                                       const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                       int table_width, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                       int n_tokens, int H, int K, int D, int n_rot, int pairing, int page_size,
                                       int write_cache) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const int b = tok_seq[t];
  if (b < 0) return;
  const int pos = tok_pos[t];
  const int upp = D >> 4, rot_units = n_rot >> 4, half_r = n_rot >> 1;
  const int n_heads = H + 2 * K;
  T* row = qkv + (size_t)t * n_heads * D;
  const int page = block_table[(size_t)b * table_width + pos / page_size];
  const int off = pos % page_size;
  for (int unit = blockIdx.y * blockDim.x + threadIdx.x; unit < n_heads * upp; unit += gridDim.y * blockDim.x) {
    const int head = unit / upp, u = unit - head * upp;
    T* x = row + (size_t)head * D;
    const bool rotate = head < H + K && cos_t != nullptr && u < rot_units;
    int ia, ib;                       // first elements of the unit's two pieces
    if (rotate && pairing == 1) { ia = 8 * u; ib = half_r + 8 * u; }
    else if (rotate) { ia = 16 * u; ib = ia + 8; }
    else { ia = (head < H + K && cos_t != nullptr) ? n_rot + 16 * (u - rot_units) : 16 * u; ib = ia + 8; }
    float va[8], vb[8];
    load8(x + ia, va);
    load8(x + ib, vb);
    if (rotate) {
      float c[8], sn[8];
      load8(cos_t + (size_t)pos * half_r + 8 * u, c);
      load8(sin_t + (size_t)pos * half_r + 8 * u, sn);
      if (pairing == 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float x0 = va[j], x1 = vb[j];
          va[j] = x0 * c[j] - x1 * sn[j];
          vb[j] = x0 * sn[j] + x1 * c[j];
        }
      } else {
        // pairs (2j, 2j+1) of the 16 consecutive elements: pair j lies in va for j < 4, in vb for j >= 4
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float* v = j < 4 ? va : vb;
          const int e = 2 * (j & 3);
          const float x0 = v[e], x1 = v[e + 1];
          v[e] = x0 * c[j] - x1 * sn[j];
          v[e + 1] = x0 * sn[j] + x1 * c[j];
        }
      }
    }
    if (head < H) {
      store8(x + ia, va);
      store8(x + ib, vb);
    } else if (write_cache) {
      const bool is_k = head < H + K;
      const int kh = is_k ? head - H : head - H - K;
      T* dst = (is_k ? k_pages : v_pages) + (((size_t)page * K + kh) * page_size + off) * D;
      store8(dst + ia, va);
      store8(dst + ib, vb);
      if (is_k) {
        store8(x + ia, va);
        store8(x + ib, vb);
      }
    }
  }
}

AB_API int ab_rope_append(void* qkv, int dtype, const float* cos_t, const float* sin_t, const int* tok_pos,
                          const int* tok_seq, const int* block_table, int table_width, void* k_pages,
                          void* v_pages, int n_tokens, int H, int K, int D, int n_rot, int pairing,
                          int page_size, int write_cache, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if ((D & 1) || (n_rot & 1) || n_rot > D || n_rot < 0) return AB_BAD_ARG;
  if (D % 16 == 0 && n_rot % 16 == 0 && (dtype == AB_F32 || dtype == AB_BF16)) {
    const int vunits = (H + 2 * K) * (D / 16);
    const int vthreads = vunits >= 256 ? 256 : (vunits >= 128 ? 128 : 64);
    const dim3 grid(n_tokens, n_tokens < 64 ? (vunits + vthreads - 1) / vthreads : 1);
    if (dtype == AB_F32)
      ab_launch(rope_append_vec_kernel<float>, grid, dim3(vthreads), 0, stream, (float*)qkv, cos_t, sin_t, tok_pos,
                tok_seq, block_table, table_width, (float*)k_pages, (float*)v_pages, n_tokens, H, K, D, n_rot,
                pairing, page_size, write_cache);
    else
      ab_launch(rope_append_vec_kernel<bf16>, grid, dim3(vthreads), 0, stream, (bf16*)qkv, cos_t, sin_t, tok_pos,
                tok_seq, block_table, table_width, (bf16*)k_pages, (bf16*)v_pages, n_tokens, H, K, D, n_rot,
                pairing, page_size, write_cache);
    return ab_launch_status();
  }
  const int units = (H + 2 * K) * (D / 2);
  const int threads = units >= 1024 ? 256 : 128;
  if (dtype == AB_F32)
    ab_launch(rope_append_kernel<float>, n_tokens, threads, 0, stream,
        (float*)qkv, cos_t, sin_t, tok_pos, tok_seq, block_table, table_width, (float*)k_pages, (float*)v_pages,
        n_tokens, H, K, D, n_rot, pairing, page_size, write_cache);
  else if (dtype == AB_BF16)
    ab_launch(rope_append_kernel<bf16>, n_tokens, threads, 0, stream,
        (bf16*)qkv, cos_t, sin_t, tok_pos, tok_seq, block_table, table_width, (bf16*)k_pages, (bf16*)v_pages,
        n_tokens, H, K, D, n_rot, pairing, page_size, write_cache);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

// ---------------------------------------------------------------------------
// SwiGLU on the fused product gu = h @ [gate|up]^T (alpacca/model.py:513):
//   act[t, j] = g / (1 + exp(-g)) * u
// The fused matrix interleaves gate and up in groups of 8 rows: columns
// 16*q + r hold gate 8*q + r, columns 16*q + 8 + r hold up 8*q + r (r < 8), which
// is the order in which the skinny-matrix kernel's accumulators meet them.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, size_t total, int F) {
  pdl_wait();
  pdl_trigger();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / F;
  const int j = (int)(idx - t * F);
  const T* row = gu + t * (size_t)(2 * F);
  const int q = j >> 3, r = j & 7;
  const float g = to_f32(row[16 * q + r]);
  const float u = to_f32(row[16 * q + 8 + r]);
  act[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// bfloat16, 8 outputs per thread: one 16-byte piece of gate, one of up, one of output
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ act, size_t n_units, int units_per_row) {
  pdl_wait();
  pdl_trigger();
  const size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // unit = 8 outputs
  if (u >= n_units) return;
  const size_t t = u / units_per_row;
  const int q = (int)(u - t * units_per_row);
  const bf16* src = gu + (t * units_per_row + q) * 16;
  const uint4 g4 = *reinterpret_cast<const uint4*>(src);
  const uint4 u4 = *reinterpret_cast<const uint4*>(src + 8);
  const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
  uint32_t ow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float g0 = __uint_as_float(gw[i] << 16), g1 = __uint_as_float(gw[i] & 0xffff0000u);
    const float u0 = __uint_as_float(uw[i] << 16), u1 = __uint_as_float(uw[i] & 0xffff0000u);
    __nv_bfloat162 r = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
    ow[i] = *reinterpret_cast<uint32_t*>(&r);
  }
  *reinterpret_cast<uint4*>(act + u * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

AB_API int ab_swiglu(const void* gu, void* act, int dtype, int n_rows, int F, cudaStream_t stream) {
  size_t total = (size_t)n_rows * F;
  if (total == 0) return AB_OK;
  if (F % 8) return AB_BAD_ARG;
  if (dtype == AB_BF16) {
    const size_t n_units = total / 8;
    ab_launch(swiglu_bf16x8_kernel, (unsigned)((n_units + 255) / 256), 256, 0, stream, (const bf16*)gu, (bf16*)act,
              n_units, F / 8);
    return ab_launch_status();
  }
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == AB_F32)
    ab_launch(swiglu_kernel<float>, blocks, 256, 0, stream, (const float*)gu, (float*)act, total, F);
  else if (dtype == AB_BF16)
    ab_launch(swiglu_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)gu, (bf16*)act, total, F);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

// ---------------------------------------------------------------------------
// After a decode step whose tokens were sampled on the device: feed them back.
// For every live row b (tok_seq[b] >= 0): tokens[b] = sampled[b]; position,
// length and the sampler's step counter go up by one; the token enters the
// row's window of recent tokens (a ring of `window` places, next place in
// recent_pos[b]).  The sampled tokens of all rows are also kept in
// history[(*counter % history_len)][:] for the host to read later.
// ---------------------------------------------------------------------------
__global__ void decode_advance_kernel(int* __restrict__ tokens, int* __restrict__ tok_pos, int* __restrict__ kv_len,
                                      int* __restrict__ rng_step, const int* __restrict__ tok_seq,
                                      const int* __restrict__ sampled, int* __restrict__ recent,
                                      int* __restrict__ recent_pos, int window, int* __restrict__ history,
                                      int* __restrict__ counter, int history_len, int* __restrict__ host_ring,
                                      int ring_len, int n_rows) {
  pdl_wait();
  pdl_trigger();
  const int slot = history ? (*counter % history_len) : 0;
  const int ring_slot = host_ring ? (*counter % ring_len) : 0;
  for (int b = threadIdx.x; b < n_rows; b += blockDim.x) {
    const int tok = sampled[b];
    if (history) history[(size_t)slot * n_rows + b] = tok;
    // pinned host memory that the device can write: the host reads the step's tokens there once the step's
    // event has passed (a copy after the graph costs a change of engines between every two replays)
    if (host_ring) host_ring[(size_t)ring_slot * n_rows + b] = tok;
    if (tok_seq[b] < 0) continue;
    tokens[b] = tok;
    tok_pos[b] += 1;
    kv_len[b] += 1;
    rng_step[b] += 1;
    if (recent && window > 0) {
      const int p = recent_pos[b];
      recent[(size_t)b * window + p] = tok;
      recent_pos[b] = (p + 1) % window;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && counter) *counter += 1;
}

AB_API int ab_decode_advance(int* tokens, int* tok_pos, int* kv_len, int* rng_step, const int* tok_seq,
                             const int* sampled, int* recent, int* recent_pos, int window, int* history,
                             int* counter, int history_len, int* host_ring, int ring_len, int n_rows,
                             cudaStream_t stream) {
  if (n_rows <= 0) return AB_OK;
  if (host_ring && (!counter || ring_len <= 0)) return AB_BAD_ARG;
  ab_launch(decode_advance_kernel, 1, 256, 0, stream, tokens, tok_pos, kv_len, rng_step, tok_seq, sampled, recent,
                                               recent_pos, window, history, counter, history_len, host_ring, ring_len,
                                               n_rows);
  return ab_launch_status();
}
