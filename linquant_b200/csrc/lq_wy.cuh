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

// One warp: acc (16 x 16, as two m16n8 fragments) += A . B for 16 x 16 fp32 blocks in shared memory (row stride 68),
// both factors split into a TF32 part and a TF32 remainder (three MMAs per k-step; products good to about 2^-21).
__device__ __forceinline__ void blk16_mma(float (&acc)[2][4], const float* A, const float* B, int g, int j) {
#pragma unroll
  for (int kk = 0; kk < 2; ++kk) {
    const int c0 = 8 * kk + j, c1 = c0 + 4;
    const float xa[4] = {A[g * 68 + c0], A[(g + 8) * 68 + c0], A[g * 68 + c1], A[(g + 8) * 68 + c1]};
    uint32_t ab[4], as_[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      ab[e] = tf32_rna(xa[e]);
      as_[e] = tf32_rna(xa[e] - __uint_as_float(ab[e]));
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float y0 = B[c0 * 68 + 8 * nt + g], y1 = B[c1 * 68 + 8 * nt + g];
      const uint32_t b0 = tf32_rna(y0), b1 = tf32_rna(y1);
      const uint32_t s0 = tf32_rna(y0 - __uint_as_float(b0)), s1 = tf32_rna(y1 - __uint_as_float(b1));
      mma_tf32(acc[nt], as_[0], as_[1], as_[2], as_[3], b0, b1);
      mma_tf32(acc[nt], ab[0], ab[1], ab[2], ab[3], s0, s1);
      mma_tf32(acc[nt], ab[0], ab[1], ab[2], ab[3], b0, b1);
    }
  }
}
__device__ __forceinline__ void blk16_store(float* D, const float (&acc)[2][4], float sign, int g, int j) {
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    D[g * 68 + 8 * nt + 2 * j] = sign * acc[nt][0];
    D[g * 68 + 8 * nt + 2 * j + 1] = sign * acc[nt][1];
    D[(g + 8) * 68 + 8 * nt + 2 * j] = sign * acc[nt][2];
    D[(g + 8) * 68 + 8 * nt + 2 * j + 1] = sign * acc[nt][3];
  }
}

// T = (I + G)^-1 for a strictly lower-triangular 64x64 G (both [64][68] fp32 in shared memory), 256 threads, as a
// blocked inverse over 16 x 16 blocks (reference: torch.linalg.solve_triangular, zoo/gated_delta_rule.py:40-41):
//   * the four diagonal blocks D_I = (I + G_II)^-1 by forward substitution, all at once: one column per group of four
//     lanes, sixteen steps, right-looking (lane r keeps the running sums of rows 4m + r; one shuffle per step);
//   * the blocks below the diagonal level by level,  T_IJ = -D_I (sum_{J <= K < I} G_IK T_KJ),  as 16 x 16 x 16 products
//     on the tensor cores (3xTF32), one warp per block; the inner sums are parked in the unused upper blocks of T.
// Six dependent product stages replace forty-eight more substitution steps. Ends with every thread past a barrier.
__device__ __forceinline__ void wy_solve(const float* s_G, float* s_T) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, j = lane & 3;
  auto blkG = [&](int I, int J) { return s_G + (16 * I) * 68 + 16 * J; };
  auto blkT = [&](int I, int J) { return s_T + (16 * I) * 68 + 16 * J; };
  {  // diagonal blocks
    const int col = tid >> 2, r = tid & 3;  // global column; block I = col / 16
    const int I = col >> 4, cl = col & 15;
    const float* G = blkG(I, I);
    float* T = blkT(I, I);
    float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float val = (i == cl ? 1.f : 0.f) - part[i >> 2];
      val = __shfl_sync(0xffffffffu, val, (lane & ~3) | (i & 3));
      if (r == 0) T[i * 68 + cl] = val;
#pragma unroll
      for (int m = i >> 2; m < 4; ++m) {
        if (m > (i >> 2) || r > (i & 3)) part[m] = fmaf(G[(4 * m + r) * 68 + i], val, part[m]);
      }
    }
  }
  __syncthreads();
  // level 1: T_{I,I-1} = -D_I (G_{I,I-1} D_{I-1}), inner product parked in T_{I-1,I}
  if (warp < 3) {
    const int I = warp + 1;
    float acc[2][4] = {};
    blk16_mma(acc, blkG(I, I - 1), blkT(I - 1, I - 1), g, j);
    blk16_store(blkT(I - 1, I), acc, 1.f, g, j);
  }
  __syncthreads();
  if (warp < 3) {
    const int I = warp + 1;
    float acc[2][4] = {};
    blk16_mma(acc, blkT(I, I), blkT(I - 1, I), g, j);
    blk16_store(blkT(I, I - 1), acc, -1.f, g, j);
  }
  __syncthreads();
  // level 2: T_{I,I-2} = -D_I (G_{I,I-2} D_{I-2} + G_{I,I-1} T_{I-1,I-2}), parked in T_{I-2,I}
  if (warp < 2) {
    const int I = warp + 2;
    float acc[2][4] = {};
    blk16_mma(acc, blkG(I, I - 2), blkT(I - 2, I - 2), g, j);
    blk16_mma(acc, blkG(I, I - 1), blkT(I - 1, I - 2), g, j);
    blk16_store(blkT(I - 2, I), acc, 1.f, g, j);
  }
  __syncthreads();
  if (warp < 2) {
    const int I = warp + 2;
    float acc[2][4] = {};
    blk16_mma(acc, blkT(I, I), blkT(I - 2, I), g, j);
    blk16_store(blkT(I, I - 2), acc, -1.f, g, j);
  }
  __syncthreads();
  // level 3: T_30 = -D_3 (G_30 D_0 + G_31 T_10 + G_32 T_20), parked in T_03
  if (warp == 0) {
    float acc[2][4] = {};
    blk16_mma(acc, blkG(3, 0), blkT(0, 0), g, j);
    blk16_mma(acc, blkG(3, 1), blkT(1, 0), g, j);
    blk16_mma(acc, blkG(3, 2), blkT(2, 0), g, j);
    blk16_store(blkT(0, 3), acc, 1.f, g, j);
  }
  __syncthreads();
  if (warp == 0) {
    float acc[2][4] = {};
    blk16_mma(acc, blkT(3, 3), blkT(0, 3), g, j);
    blk16_store(blkT(3, 0), acc, -1.f, g, j);
  }
  __syncthreads();
}

}  // namespace lq
