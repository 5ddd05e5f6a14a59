// Device helpers shared by the tensor-core attention kernels (attention_mma.cu, attention_stream.cu):
// shared-memory matrix loads, the bfloat16 MMA, and the position rotation of a head.
#pragma once
#include "common.cuh"

#define PAGE 64
#define LOG2E 1.4426950408889634f

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 2^x by the hardware's approximation (relative error 2^-22; 2^-inf = 0): exp2f wraps it in a few more
// instructions for results below the normal range, which a softmax weight does not need
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}


// Position rotation of one unit of 16 elements of a head (the same arithmetic, in the same order, as
// the separate rotation kernel): unit u of a rotated head covers the pairs 8u .. 8u+7, i.e. with
// pairing 0 (neighbours) the 16 consecutive elements from 16u, with pairing 1 (halves) the pieces at 8u
// and n_rot/2 + 8u; units past n_rot / 16 and heads that are not rotated pass through.
// (x0, x1) -> (x0 c - x1 s, x0 s + x1 c), alpacca/model.py:405-438.  Writes bfloat16 to dst.
__device__ __forceinline__ void rotate_unit(const bf16* __restrict__ x, bf16* dst, int u, bool rotated,
                                            const float* __restrict__ cos_row, const float* __restrict__ sin_row,
                                            int n_rot, int pairing) {
  const int rot_units = n_rot >> 4, half_r = n_rot >> 1;
  const bool rotate = rotated && u < rot_units;
  int ia, ib;
  if (rotate && pairing == 1) { ia = 8 * u; ib = half_r + 8 * u; }
  else if (rotate) { ia = 16 * u; ib = ia + 8; }
  else { ia = rotated ? n_rot + 16 * (u - rot_units) : 16 * u; ib = ia + 8; }
  uint4 ra = *reinterpret_cast<const uint4*>(x + ia), rb = *reinterpret_cast<const uint4*>(x + ib);
  if (rotate) {
    float c[8], sn[8], va[8], vb[8];
    const float4 c0 = *reinterpret_cast<const float4*>(cos_row + 8 * u), c1 = *reinterpret_cast<const float4*>(cos_row + 8 * u + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sin_row + 8 * u), s1 = *reinterpret_cast<const float4*>(sin_row + 8 * u + 4);
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    const uint32_t wa[4] = {ra.x, ra.y, ra.z, ra.w}, wb[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      va[2 * i] = __uint_as_float(wa[i] << 16);
      va[2 * i + 1] = __uint_as_float(wa[i] & 0xffff0000u);
      vb[2 * i] = __uint_as_float(wb[i] << 16);
      vb[2 * i + 1] = __uint_as_float(wb[i] & 0xffff0000u);
    }
    if (pairing == 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x0 = va[j], x1 = vb[j];
        va[j] = x0 * c[j] - x1 * sn[j];
        vb[j] = x0 * sn[j] + x1 * c[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float* v = j < 4 ? va : vb;
        const int e = 2 * (j & 3);
        const float x0 = v[e], x1 = v[e + 1];
        v[e] = x0 * c[j] - x1 * sn[j];
        v[e + 1] = x0 * sn[j] + x1 * c[j];
      }
    }
    ra = make_uint4(pack_bf16(va[0], va[1]), pack_bf16(va[2], va[3]), pack_bf16(va[4], va[5]), pack_bf16(va[6], va[7]));
    rb = make_uint4(pack_bf16(vb[0], vb[1]), pack_bf16(vb[2], vb[3]), pack_bf16(vb[4], vb[5]), pack_bf16(vb[6], vb[7]));
  }
  *reinterpret_cast<uint4*>(dst + ia) = ra;
  *reinterpret_cast<uint4*>(dst + ib) = rb;
}

