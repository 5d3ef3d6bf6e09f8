// WY-representation helpers shared by the delta-rule prologues: TF32 MMA wrappers, the unit-lower-triangular
// inverse by forward substitution and the T . diag(cw) . B product with the left factor split into three TF32 pieces.
#pragma once
#include "lq_common.cuh"

namespace lq {

__device__ __forceinline__ uint32_t tf32_rna(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float pow_exact01(float x, float e) { return e == 0.f ? 1.f : (e == 1.f ? x : powf(x, e)); }

// acc[NT][4] += (T .* cw[None,:])[16 rows of m-tile mt, tokens 0..16mt+15] . B[tokens, NT*8 columns from n0]
template <int NT>
__device__ __forceinline__ void wy_product(float (&acc)[NT][4], const float* s_T, const float* s_cw, const float* s_B,
                                           int LDB, int mt, int n0, int g, int j) {
  const int ia = 16 * mt + g, ib = ia + 8;
  for (int kk = 0; kk < 2 * mt + 2; ++kk) {
    const int c0 = 8 * kk + j, c1 = c0 + 4;
    const float x[4] = {s_T[ia * 68 + c0] * s_cw[c0], s_T[ib * 68 + c0] * s_cw[c0], s_T[ia * 68 + c1] * s_cw[c1],
                        s_T[ib * 68 + c1] * s_cw[c1]};
    uint32_t hi[4], mi[4], lo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      hi[i] = tf32_rna(x[i]);
      const float r1 = x[i] - __uint_as_float(hi[i]);
      mi[i] = tf32_rna(r1);
      lo[i] = __float_as_uint(r1 - __uint_as_float(mi[i]));
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const uint32_t b0 = __float_as_uint(s_B[c0 * LDB + n0 + 8 * nt + g]);
      const uint32_t b1 = __float_as_uint(s_B[c1 * LDB + n0 + 8 * nt + g]);
      mma_tf32(acc[nt], lo[0], lo[1], lo[2], lo[3], b0, b1);
      mma_tf32(acc[nt], mi[0], mi[1], mi[2], mi[3], b0, b1);
      mma_tf32(acc[nt], hi[0], hi[1], hi[2], hi[3], b0, b1);
    }
  }
}

// Same product with a general fp32 right factor: both factors split into a TF32 "big" part and a TF32 remainder,
// three MMAs per tile (small*big, big*small, big*big), products good to about 2^-21 relative.
template <int NT>
__device__ __forceinline__ void wy_product_split(float (&acc)[NT][4], const float* s_T, const float* s_cw, const float* s_B,
                                                 int LDB, int mt, int n0, int g, int j) {
  const int ia = 16 * mt + g, ib = ia + 8;
  for (int kk = 0; kk < 2 * mt + 2; ++kk) {
    const int c0 = 8 * kk + j, c1 = c0 + 4;
    const float x[4] = {s_T[ia * 68 + c0] * s_cw[c0], s_T[ib * 68 + c0] * s_cw[c0], s_T[ia * 68 + c1] * s_cw[c1],
                        s_T[ib * 68 + c1] * s_cw[c1]};
    uint32_t big[4], sml[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      big[i] = tf32_rna(x[i]);
      sml[i] = tf32_rna(x[i] - __uint_as_float(big[i]));
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float y0 = s_B[c0 * LDB + n0 + 8 * nt + g], y1 = s_B[c1 * LDB + n0 + 8 * nt + g];
      const uint32_t b0 = tf32_rna(y0), b1 = tf32_rna(y1);
      const uint32_t s0 = tf32_rna(y0 - __uint_as_float(b0)), s1 = tf32_rna(y1 - __uint_as_float(b1));
      mma_tf32(acc[nt], sml[0], sml[1], sml[2], sml[3], b0, b1);
      mma_tf32(acc[nt], big[0], big[1], big[2], big[3], s0, s1);
      mma_tf32(acc[nt], big[0], big[1], big[2], big[3], b0, b1);
    }
  }
}

// T = (I + G)^-1 for a strictly lower-triangular 64x64 G (both [64][68] fp32 in shared memory), 256 threads.
// Forward substitution, one column of T per group of four lanes, in its right-looking form: as soon as T[i][col]
// is known, every later row's running sum  sum_j G[row][j] T[j][col]  takes its term j = i. Lane r of the group
// keeps the sums of rows 4m + r in registers, so a step is one shuffle (the owner of row i publishes the value)
// followed by independent multiply-adds; nothing is reduced across lanes. Columns 8w .. 8w+7 belong to warp w and
// are zero above row 8w, so the warp skips those steps (reference: torch.linalg.solve_triangular,
// zoo/gated_delta_rule.py:40-41).
__device__ __forceinline__ void wy_solve(const float* s_G, float* s_T) {
  const int tid = threadIdx.x, lane = tid & 31;
  const int col = tid >> 2, r = tid & 3;
  const int first = 8 * (tid >> 5);
  float part[16];
#pragma unroll
  for (int m = 0; m < 16; ++m) part[m] = 0.f;
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    if (i < first) {  // warp-uniform
      if (r == 0) s_T[i * 68 + col] = 0.f;
      continue;
    }
    float val = (i == col ? 1.f : 0.f) - part[i >> 2];
    val = __shfl_sync(0xffffffffu, val, (lane & ~3) | (i & 3));
    if (r == 0) s_T[i * 68 + col] = val;
#pragma unroll
    for (int m = i >> 2; m < 16; ++m) {
      if (m > (i >> 2) || r > (i & 3)) part[m] = fmaf(s_G[(4 * m + r) * 68 + i], val, part[m]);
    }
  }
}

}  // namespace lq
