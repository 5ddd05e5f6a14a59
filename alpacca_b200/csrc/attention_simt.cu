// Attention over the paged cache, one warp per (token, query head), plain
// 32-bit arithmetic.  It is the attention of the 32-bit path (T = float), for
// prefill and decode alike, and takes every head size up to 256; the bfloat16
// path uses it for head sizes that the tensor-core kernel refuses.
//
// For token t at position p of sequence b, head h reads KV head h / (H/K):
//   score_s = (q . k_s) * scale  for lo <= s <= p   (alpacca/model.py:447-467)
//   out = sum_s softmax(score)_s * v_s
// with lo = 0, or p - window + 1 when a window is given.  The softmax is the
// running (online) form, in key order; nothing is shared between warps, so a
// token's result does not depend on the rest of the batch.
#include "common.cuh"

template <typename T, int DPL>
__global__ void attention_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                                      const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                      const int* __restrict__ block_table, int table_width,
                                      const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                      int n_tokens, int H, int K, int D, int page_size, float scale, int window) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)n_tokens * H) return;
  const int t = (int)(w / H), h = (int)(w - (long long)t * H);
  const int b = tok_seq[t];
  T* o = out + ((size_t)t * H + h) * D;
  if (b < 0) return;
  const int pos = tok_pos[t];
  const int kh = h / (H / K);
  const T* qv = q + (size_t)t * q_stride + (size_t)h * D;
  float qr[DPL], acc[DPL];
#pragma unroll
  for (int j = 0; j < DPL; ++j) {
    const int d = lane + 32 * j;
    qr[j] = d < D ? to_f32(qv[d]) : 0.f;
    acc[j] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* bt = block_table + (size_t)b * table_width;
  for (int s = lo; s <= pos; ++s) {
    const int page = bt[s / page_size];
    const size_t base = (((size_t)page * K + kh) * page_size + (s % page_size)) * D;
    const T* kv = k_pages + base;
    const T* vv = v_pages + base;
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const int d = lane + 32 * j;
      if (d < D) part += qr[j] * to_f32(kv[d]);
    }
    const float score = warp_sum(part) * scale;
    const float m_new = fmaxf(m, score);
    const float corr = expf(m - m_new);   // exp(-inf) = 0 on the first key
    const float p = expf(score - m_new);
    l = l * corr + p;
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const int d = lane + 32 * j;
      if (d < D) acc[j] = acc[j] * corr + p * to_f32(vv[d]);
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int j = 0; j < DPL; ++j) {
    const int d = lane + 32 * j;
    if (d < D) o[d] = from_f32<T>(acc[j] * inv);
  }
}

template <typename T>
static int launch(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                  const int* block_table, int table_width, const int* tok_pos, const int* tok_seq, int n_tokens,
                  int H, int K, int D, int page_size, float scale, int window, cudaStream_t stream) {
  const long long warps = (long long)n_tokens * H;
  const int wpb = 4;
  const unsigned blocks = (unsigned)((warps + wpb - 1) / wpb);
#define AB_GO(DPL)                                                                                       \
  attention_simt_kernel<T, DPL><<<blocks, wpb * 32, 0, stream>>>(                                        \
      (const T*)q, q_stride, (T*)out, (const T*)k_pages, (const T*)v_pages, block_table, table_width,   \
      tok_pos, tok_seq, n_tokens, H, K, D, page_size, scale, window)
  if (D <= 32) AB_GO(1);
  else if (D <= 64) AB_GO(2);
  else if (D <= 128) AB_GO(4);
  else AB_GO(8);
#undef AB_GO
  return ab_launch_status();
}

AB_API int ab_attention_simt(const void* q, int q_stride, void* out, int dtype, const void* k_pages,
                             const void* v_pages, const int* block_table, int table_width, const int* tok_pos,
                             const int* tok_seq, int n_tokens, int H, int K, int D, int page_size, float scale,
                             int window, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (D <= 0 || D > 256 || H <= 0 || K <= 0 || H % K) return AB_BAD_ARG;
  if (dtype == AB_F32)
    return launch<float>(q, q_stride, out, k_pages, v_pages, block_table, table_width, tok_pos, tok_seq,
                         n_tokens, H, K, D, page_size, scale, window, stream);
  if (dtype == AB_BF16)
    return launch<bf16>(q, q_stride, out, k_pages, v_pages, block_table, table_width, tok_pos, tok_seq,
                        n_tokens, H, K, D, page_size, scale, window, stream);
  return AB_BAD_ARG;
}
