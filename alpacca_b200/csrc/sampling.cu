// Sampling from rows of float32 logits, one thread block per row.
//
// What the reference's sampler does (alpacca/sample.py:36-76), in its order:
// repeat penalty on the recent tokens, then greedy (temperature <= 0: first
// index of the maximum) or: keep the top_k largest logits (ties to the lower
// index), weights exp((l - max)/T), cut at the shortest prefix in descending
// order whose probability reaches top_p, draw from what is left.
//
// The reference draws with Python's generator from the sorted list.  Here the
// kept set is walked in index order and the draw is u * (kept weight) with u
// from Philox-4x32-10 keyed by the seed and counted by (stream, step), so a
// row's token depends on its own logits, seed, stream and step only, never on
// the rest of the batch.  The kept set always has the form
//   { l > t }  plus the first c indices with  l == t,
// and t, c are found by radix selection on the bit pattern of the floats
// (four passes of 8 bits), by count for top_k and by weight for top_p.
// Weights are summed as 64-bit fixed point (w * 2^40), so every sum is exact
// integer arithmetic and does not depend on the order of the additions.
#include "common.cuh"
#include "launch.cuh"

#define SAMPLE_THREADS 1024
#define W_SHIFT 40

// ---------------------------------------------------------------------------
// Repeat penalty: for each distinct token of the row's recent window,
// l > 0 -> l / p, else l * p   (alpacca/sample.py:40-43).
// recent: int32 [n_rows, window], unused places hold -1.
// ---------------------------------------------------------------------------
__global__ void repeat_penalty_kernel(float* __restrict__ logits, const int* __restrict__ recent, int window,
                                      int vocab, float penalty) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int* r = recent + (size_t)row * window;
  float* l = logits + (size_t)row * vocab;
  for (int i = threadIdx.x; i < window; i += blockDim.x) {
    const int tok = r[i];
    if (tok < 0 || tok >= vocab) continue;
    bool first = true;
    for (int j = 0; j < i; ++j)
      if (r[j] == tok) { first = false; break; }
    if (!first) continue;
    const float v = l[tok];
    l[tok] = v > 0.f ? v / penalty : v * penalty;
  }
}

AB_API int ab_repeat_penalty(float* logits, const int* recent, int n_rows, int window, int vocab, float penalty,
                             cudaStream_t stream) {
  if (n_rows <= 0 || window <= 0) return AB_OK;
  ab_launch(repeat_penalty_kernel, n_rows, 128, 0, stream, logits, recent, window, vocab, penalty);
  return ab_launch_status();
}

// ---------------------------------------------------------------------------

__device__ __forceinline__ unsigned int float_key(float x) {
  // ascending unsigned order == ascending float order
  const unsigned int b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long weight_fx(float l, float m, float inv_t) {
  const float w = expf((l - m) * inv_t);               // in (0, 1]
  // w * 2^40 is exact in float (a shift of the exponent), so this is the truncation of the same real
  // number that the double-precision product would give, without the slow double-precision units
  return __float2ull_rz(w * 1099511627776.0f);
}

__device__ void philox4x32_10(unsigned int c0, unsigned int c1, unsigned int c2, unsigned int c3,
                              unsigned int k0, unsigned int k1, unsigned int* out0) {
#pragma unroll 1
  for (int r = 0; r < 10; ++r) {
    const unsigned long long p0 = 0xD2511F53ull * c0;
    const unsigned long long p1 = 0xCD9E8D57ull * c2;
    const unsigned int n0 = (unsigned int)(p1 >> 32) ^ c1 ^ k0;
    const unsigned int n1 = (unsigned int)p1;
    const unsigned int n2 = (unsigned int)(p0 >> 32) ^ c3 ^ k1;
    const unsigned int n3 = (unsigned int)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  *out0 = c0;
}

struct SampleShared {
  unsigned long long hist_w[256];
  unsigned int hist_c[256];
  unsigned long long scan_w[32];
  unsigned int scan_c[32];
  float red_v[32];
  int red_i[32];
  // broadcast values
  unsigned int prefix, digit;
  unsigned long long acc_w;
  unsigned int acc_c;
  float max_v;
  int arg;
  int result;
  // the segment (a warp's share of the vocabulary) that holds the drawn weight, with what lies before it
  int seg0, seg1;
  unsigned long long seg_w;
  unsigned int seg_ties;
};

// block-wide exclusive scan of one 64-bit and one 32-bit value per thread; also the totals
__device__ void block_scan(unsigned long long w, unsigned int c, unsigned long long* w_excl, unsigned int* c_excl,
                           unsigned long long* w_total, unsigned int* c_total, SampleShared* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long wi = w;
  unsigned int ci = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long wn = __shfl_up_sync(0xffffffffu, wi, o);
    const unsigned int cn = __shfl_up_sync(0xffffffffu, ci, o);
    if (lane >= o) { wi += wn; ci += cn; }
  }
  __syncthreads();
  if (lane == 31) { sh->scan_w[warp] = wi; sh->scan_c[warp] = ci; }
  __syncthreads();
  if (warp == 0) {
    unsigned long long ws = sh->scan_w[lane];
    unsigned int cs = sh->scan_c[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long wn = __shfl_up_sync(0xffffffffu, ws, o);
      const unsigned int cn = __shfl_up_sync(0xffffffffu, cs, o);
      if (lane >= o) { ws += wn; cs += cn; }
    }
    sh->scan_w[lane] = ws;   // inclusive over warps
    sh->scan_c[lane] = cs;
  }
  __syncthreads();
  const unsigned long long wbase = warp ? sh->scan_w[warp - 1] : 0ull;
  const unsigned int cbase = warp ? sh->scan_c[warp - 1] : 0u;
  *w_excl = wbase + wi - w;
  *c_excl = cbase + ci - c;
  *w_total = sh->scan_w[31];
  *c_total = sh->scan_c[31];
  __syncthreads();
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out, float temperature, int top_k,
              float top_p, unsigned int seed_lo, unsigned int seed_hi, const unsigned int* __restrict__ seed_dev,
              const int* __restrict__ streams, const int* __restrict__ steps) {
  __shared__ SampleShared sh;
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const float* l = logits + (size_t)row * vocab;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // ---- maximum and its first index -------------------------------------
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
    // rows start on 16-byte boundaries: four logits per load, several loads in flight
    const float4* l4 = reinterpret_cast<const float4*>(l);
    const int n4 = vocab >> 2;
#pragma unroll 4
    for (int i = tid; i < n4; i += SAMPLE_THREADS) {
      const float4 q = l4[i];
      const float e[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (e[j] > bv || (e[j] == bv && 4 * i + j < bi)) { bv = e[j]; bi = 4 * i + j; }
    }
  } else {
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
      const float v = l[i];
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) { sh.red_v[warp] = bv; sh.red_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = sh.red_v[lane];
    bi = sh.red_i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sh.max_v = bv; sh.arg = bi == 0x7fffffff ? 0 : bi; }
  }
  __syncthreads();
  if (temperature <= 0.f) {
    if (tid == 0) out[row] = sh.arg;
    return;
  }
  const float m = sh.max_v;
  const float inv_t = 1.0f / temperature;

  // ---- top_k: the k-th largest key t_k, n_gt = #{l > t_k}, c_k ties kept ----
  const bool use_k = top_k > 0 && top_k < vocab;
  unsigned int tk_key = 0;     // keys >= this are candidates; with !use_k everything is
  unsigned int ck = 0;         // ties at t_k that are kept (use_k only)
  if (use_k) {
    unsigned int prefix = 0, mask = 0, above = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int i = tid; i < 256; i += SAMPLE_THREADS) sh.hist_c[i] = 0;
      __syncthreads();
      for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const unsigned int key = float_key(l[i]);
        if ((key & mask) == prefix) atomicAdd(&sh.hist_c[(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned int acc = above;
        int d = 255;
        for (; d > 0; --d) {
          if (acc + sh.hist_c[d] >= (unsigned int)top_k) break;
          acc += sh.hist_c[d];
        }
        sh.digit = (unsigned int)d;
        sh.acc_c = acc;
      }
      __syncthreads();
      prefix |= sh.digit << shift;
      mask |= 255u << shift;
      above = sh.acc_c;
      __syncthreads();
    }
    tk_key = prefix;
    ck = (unsigned int)top_k - above;   // >= 1
  }

  // ---- weight above t_k (or of everything) ---------------------------------
  // (only the cuts need it: plain temperature sampling goes straight to the walk)
  const bool use_p = top_p > 0.f && top_p < 1.f;
  unsigned long long w_gt = 0;
  unsigned long long w_tk = 0;   // weight of one element equal to t_k
  if (use_k || use_p) for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
    const float v = l[i];
    const unsigned int key = float_key(v);
    if (!use_k || key > tk_key) w_gt += weight_fx(v, m, inv_t);
    else if (key == tk_key) w_tk = weight_fx(v, m, inv_t);
  }
  {
    unsigned long long e;
    unsigned int ce, ct;
    unsigned long long tot;
    block_scan(w_gt, 0u, &e, &ce, &tot, &ct, &sh);
    w_gt = tot;
    // any thread that saw a tie has the same w_tk; share it
    if (tid == 0) sh.acc_w = 0;
    __syncthreads();
    if (w_tk) sh.acc_w = w_tk;   // benign: every writer writes the same value
    __syncthreads();
    w_tk = sh.acc_w;
    __syncthreads();
  }
  const unsigned long long w_k = w_gt + (use_k ? (unsigned long long)ck * w_tk : 0ull);

  // ---- top_p: threshold t and ties c of the final kept set ----------------------
  unsigned int t_key = use_k ? tk_key : 0u;
  unsigned int c_ties = use_k ? ck : 0u;        // ties at t_key that are kept
  bool ties_limited = use_k;                    // false: every element with key >= t_key is kept
  if (use_p) {
    const unsigned long long P = (unsigned long long)((double)w_k * (double)top_p);
    if (use_k && P > w_gt) {
      // the cut falls among the ties at t_k
      unsigned long long need = w_tk ? (P - w_gt + w_tk - 1) / w_tk : 1ull;
      if (need < 1) need = 1;
      if (need < c_ties) c_ties = (unsigned int)need;
    } else {
      // weighted selection among keys > tk_key (or all): smallest descending prefix with weight >= P
      unsigned int prefix = 0, mask = 0;
      unsigned long long above = 0;
      for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < 256; i += SAMPLE_THREADS) { sh.hist_w[i] = 0; sh.hist_c[i] = 0; }
        __syncthreads();
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
          const float v = l[i];
          const unsigned int key = float_key(v);
          if (use_k && key <= tk_key) continue;
          if ((key & mask) == prefix) {
            const unsigned int d = (key >> shift) & 255u;
            atomicAdd(&sh.hist_w[d], weight_fx(v, m, inv_t));
            atomicAdd(&sh.hist_c[d], 1u);
          }
        }
        __syncthreads();
        if (tid == 0) {
          unsigned long long acc = above;
          int d = 255, last_nonempty = -1;
          for (; d >= 0; --d) {
            if (sh.hist_c[d]) {
              last_nonempty = d;
              if (acc + sh.hist_w[d] >= P) break;
              acc += sh.hist_w[d];
            }
          }
          if (d < 0) {          // weights rounded to zero never reach P: stop at the lowest occupied bin
            d = last_nonempty < 0 ? 0 : last_nonempty;
            acc -= sh.hist_w[d];
          }
          sh.digit = (unsigned int)d;
          sh.acc_w = acc;
        }
        __syncthreads();
        prefix |= sh.digit << shift;
        mask |= 255u << shift;
        above = sh.acc_w;
        __syncthreads();
      }
      t_key = prefix;
      // ties at t: each has the same weight; keep the first c of them
      const unsigned int n_ties = sh.hist_c[sh.digit];
      const unsigned long long w_tie = n_ties ? sh.hist_w[sh.digit] / n_ties : 0ull;
      unsigned long long need = (w_tie && P > above) ? (P - above + w_tie - 1) / w_tie : 1ull;
      if (need < 1) need = 1;
      if (need > n_ties) need = n_ties;
      c_ties = (unsigned int)need;
      ties_limited = true;
      __syncthreads();
    }
  }

  // ---- walk the kept set in index order ---------------------------------------
  // Warp w owns the indices [w * seg, (w + 1) * seg); its lanes read them 32 at a time, side by side
  // (whole lines of memory per load), so "index order" inside a warp is (round, lane).  A tie's rank
  // in index order is the number of ties before it: the warps before (a scan of 32 counts), the
  // rounds before and the lanes before (a ballot).  The kept weight of the warps is scanned the same
  // way; the segment whose share holds the target is then searched by the whole block.
  const int seg = (vocab + 31) / 32;
  const int s0 = min(vocab, warp * seg), s1 = min(vocab, s0 + seg);
  const unsigned int lanes_before = (1u << lane) - 1u;
  unsigned int ties_before = 0;             // ties in the warps before this one
  if (ties_limited) {
    unsigned int n = 0;
    for (int i = s0 + lane; i < s1; i += 32) n += float_key(l[i]) == t_key;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
    unsigned long long we, wt;
    unsigned int ct;
    block_scan(0ull, lane == 0 ? n : 0u, &we, &ties_before, &wt, &ct, &sh);
    ties_before = __shfl_sync(0xffffffffu, ties_before, 0);
  }
  // kept weight of lane's elements of one round; `rank` = ties seen so far in index order
  auto kept_weight = [&](int i, unsigned int& rank) -> unsigned long long {
    const bool in = i < s1;
    const float v = in ? l[i] : 0.f;
    const unsigned int key = float_key(v);
    bool keep = in;
    if (ties_limited) {
      const unsigned int tie = __ballot_sync(0xffffffffu, in && key == t_key);
      if (key > t_key) keep = in;
      else if (key == t_key) keep = in && (rank + __popc(tie & lanes_before)) < c_ties;
      else keep = false;
      rank += __popc(tie);
    }
    return keep ? weight_fx(v, m, inv_t) : 0ull;
  };
  unsigned long long my_w = 0;
  {
    unsigned int rank = ties_before;
    for (int i0 = s0; i0 < s1; i0 += 32) my_w += kept_weight(i0 + lane, rank);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) my_w += __shfl_xor_sync(0xffffffffu, my_w, o);     // the warp's kept weight
  unsigned long long w_before, w_total;
  {
    unsigned int ce, ct;
    block_scan(lane == 0 ? my_w : 0ull, 0u, &w_before, &ce, &w_total, &ct, &sh);
    w_before = __shfl_sync(0xffffffffu, w_before, 0);
  }

  if (seed_dev) {            // the seed lives on the device when the launch is replayed from a graph
    seed_lo = seed_dev[0];
    seed_hi = seed_dev[1];
  }
  unsigned int x0;
  philox4x32_10((unsigned int)steps[row], 0u, (unsigned int)streams[row], 0u, seed_lo, seed_hi, &x0);
  const double u = (double)(x0 >> 8) * (1.0 / 16777216.0);
  const unsigned long long target = (unsigned long long)((double)w_total * u);
  if (tid == 0) { sh.result = sh.arg; sh.seg0 = -1; }     // fallback: the maximum (always kept)
  __syncthreads();
  if (lane == 0 && my_w > 0 && w_before <= target && target < w_before + my_w) {
    // this warp's segment holds the target; the whole block looks for the index in it
    sh.seg0 = s0;
    sh.seg1 = s1;
    sh.seg_w = w_before;
    sh.seg_ties = ties_before;
  }
  __syncthreads();
  if (sh.seg0 >= 0) {
    // every thread takes a few consecutive indices of the segment (a warp walking it alone, round
    // after round, waits for one load per round: 126 round trips for a vocabulary of 128,256)
    const int S0 = sh.seg0, S1 = sh.seg1;
    const int chunk = (S1 - S0 + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int i0 = min(S1, S0 + tid * chunk), i1 = min(S1, i0 + chunk);
    unsigned int rank0 = 0;
    if (ties_limited) {
      unsigned int mine = 0;
      for (int i = i0; i < i1; ++i) mine += float_key(l[i]) == t_key;
      unsigned long long we, wt;
      unsigned int ct;
      block_scan(0ull, mine, &we, &rank0, &wt, &ct, &sh);
    }
    rank0 += sh.seg_ties;
    auto kept = [&](int i, unsigned int& rank) -> unsigned long long {
      const float v = l[i];
      const unsigned int key = float_key(v);
      bool keep = true;
      if (ties_limited) {
        if (key > t_key) keep = true;
        else if (key == t_key) keep = rank++ < c_ties;
        else keep = false;
      }
      return keep ? weight_fx(v, m, inv_t) : 0ull;
    };
    unsigned long long mine_w = 0;
    {
      unsigned int rank = rank0;
      for (int i = i0; i < i1; ++i) mine_w += kept(i, rank);
    }
    unsigned long long before, total;
    unsigned int ce, ct;
    block_scan(mine_w, 0u, &before, &ce, &total, &ct, &sh);
    before += sh.seg_w;
    if (mine_w > 0 && before <= target && target < before + mine_w) {
      unsigned long long acc = before;
      unsigned int rank = rank0;
      for (int i = i0; i < i1; ++i) {
        acc += kept(i, rank);
        if (acc > target) { sh.result = i; break; }
      }
    }
  }
  __syncthreads();
  if (tid == 0) out[row] = sh.result;
}

AB_API int ab_sample(const float* logits, int n_rows, int vocab, int* out, float temperature, int top_k,
                     float top_p, unsigned long long seed, const unsigned int* seed_dev, const int* streams,
                     const int* steps, cudaStream_t stream) {
  if (n_rows <= 0) return AB_OK;
  if (vocab <= 0) return AB_BAD_ARG;
  ab_launch(sample_kernel, n_rows, SAMPLE_THREADS, 0, stream, logits, vocab, out, temperature, top_k, top_p,
            (unsigned int)(seed & 0xffffffffull), (unsigned int)(seed >> 32), seed_dev, streams, steps);
  return ab_launch_status();
}
