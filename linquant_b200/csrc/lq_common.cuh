// Device helpers shared by the sm_100a kernels: the INT8 code rule, bf16/fp16 row I/O, the in-register
// Walsh-Hadamard butterfly and the warp-level MMA wrappers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/linquant_b200.h"

namespace lq {

// ---- host-side error plumbing (defined in lq_api.cu)
int fail(int status, const char* fmt, ...);
int check_launch(const char* what);

// ---- the code rule (zoo/simple_gla.py:16-20; invariances.py:91-100)
// y = x * inv (fp32, its own rounding), half away from zero, clamp to +-qmax. Clamping first and truncating
// y + copysign(0.5, y) afterwards gives the same integer for every finite y.
__device__ __forceinline__ int q8(float x, float inv, float qmax) {
  float y = __fmul_rn(x, inv);
  y = fminf(fmaxf(y, -qmax), qmax);
  return __float2int_rz(__fadd_rn(y, copysignf(0.5f, y)));
}

// Four codes on the +-127 grid, packed: the lower clamp by hand, the upper one by the saturating pack (a value above
// 127.5 truncates to >= 127 and saturates to 127). Same codes as q8(x, inv, 127) four times and pack4.
__device__ __forceinline__ uint32_t q8x4_127(float x0, float x1, float x2, float x3, float inv);

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
  uint32_t lo = __byte_perm((uint32_t)a, (uint32_t)b, 0x0040);
  uint32_t hi = __byte_perm((uint32_t)c, (uint32_t)d, 0x0040);
  return __byte_perm(lo, hi, 0x5410);
}

// two int32 codes -> two saturated INT8 in the low half of the result, `upper` shifted into the high half
// (cvt.pack.sat.s8.s32.b32 d, a, b, c:  d = sat8(a) << 8 | sat8(b) | c << 16)
__device__ __forceinline__ uint32_t pack_sat_s8x2(int hi, int lo, uint32_t upper) {
  uint32_t d;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(hi), "r"(lo), "r"(upper));
  return d;
}
__device__ __forceinline__ int q8_lower127(float x, float inv) {
  const float y = fmaxf(__fmul_rn(x, inv), -127.f);
  return __float2int_rz(__fadd_rn(y, copysignf(0.5f, y)));
}
__device__ __forceinline__ uint32_t q8x4_127(float x0, float x1, float x2, float x3, float inv) {
  return pack_sat_s8x2(q8_lower127(x1, inv), q8_lower127(x0, inv), pack_sat_s8x2(q8_lower127(x3, inv), q8_lower127(x2, inv), 0u));
}
// Byte I of w, where w holds four INT8 codes XOR 0x80 (code + 128 as an unsigned byte), as an exact float: the byte
// becomes the low mantissa bits of 2^23 and the offset is subtracted -- no trip through the conversion unit.
template <int I>
__device__ __forceinline__ float s8_to_float(uint32_t w_xor80) {
  return __fsub_rn(__uint_as_float(__byte_perm(w_xor80, 0x4B000000u, 0x7540 | I)), 8388736.0f);
}

// ---- row orders of the two tiles that are B operands of the output contractions
// The k_local tile and the stored-state tile are laid out so that MMA column n of the output kernel is simply row n
// of the tile, while a thread's accumulator fragment still covers four consecutive tokens (k_local) or eight
// consecutive value channels (state). Within each group the row index is a fixed bit permutation of the token /
// channel index.
__device__ __host__ __forceinline__ int kl_row_of_token(int t) {  // low 4 bits [j1 j0 h e] -> [h j1 j0 e]
  return (t & ~15) | (((t >> 1) & 1) << 3) | (((t >> 2) & 3) << 1) | (t & 1);
}
__device__ __host__ __forceinline__ int state_row_of_channel(int v) {  // low 5 bits [j1 j0 n1 n0 e] -> [n1 n0 j1 j0 e]
  return (v & ~31) | (((v >> 1) & 3) << 3) | (((v >> 3) & 3) << 1) | (v & 1);
}

// ---- activation dtype traits
template <typename T>
struct Act;
template <>
struct Act<__half> {
  static __device__ __forceinline__ void unpack8(const uint4& r, float (&x)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      x[2 * i] = f.x;
      x[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ uint32_t pack2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <>
struct Act<__nv_bfloat16> {
  static __device__ __forceinline__ void unpack8(const uint4& r, float (&x)[8]) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  static __device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <>
struct Act<float> {
  static __device__ __forceinline__ float round(float x) { return x; }
};

// ---- Walsh-Hadamard butterfly over a row of D = 8 * LPR values held 8 per lane by LPR consecutive lanes
// (lane-in-row r holds elements 8r .. 8r+7). Sylvester ordering, unnormalised.
template <int LPR>
__device__ __forceinline__ void fwht8(float (&x)[8], int r) {
#pragma unroll
  for (int s = 1; s < 8; s <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if ((i & s) == 0) {
        float a = x[i], b = x[i | s];
        x[i] = a + b;
        x[i | s] = a - b;
      }
    }
  }
#pragma unroll
  for (int m = 1; m < LPR; m <<= 1) {
    const float s = (r & m) ? -1.0f : 1.0f;  // upper half of the butterfly: other - x, lower: x + other (one fma, exact)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float other = __shfl_xor_sync(0xffffffffu, x[i], m);
      x[i] = fmaf(x[i], s, other);
    }
  }
}

// ---- warp MMA wrappers (row.col, A and B both with the reduction index contiguous)
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// first product of an INT8 accumulator chain: C = 0 without zeroing registers
__device__ __forceinline__ void mma_s8_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// four INT8 codes in one word -> two half2 words (codes 0,1 and 2,3), exact: (c ^ 0x80) + 1024 - 1152
__device__ __forceinline__ void s8x4_to_h2x2(uint32_t w, uint32_t& h01, uint32_t& h23) {
  const uint32_t u = w ^ 0x80808080u;
  uint32_t a = __byte_perm(u, 0x64646464u, 0x4140);
  uint32_t b = __byte_perm(u, 0x64646464u, 0x4342);
  const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480));  // 1152.0
  __half2 ha = __hsub2(*reinterpret_cast<__half2*>(&a), bias);
  __half2 hb = __hsub2(*reinterpret_cast<__half2*>(&b), bias);
  h01 = *reinterpret_cast<uint32_t*>(&ha);
  h23 = *reinterpret_cast<uint32_t*>(&hb);
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

}  // namespace lq
