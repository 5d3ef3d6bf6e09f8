// Row-wise operand preparation shared by the zoo prologue kernels: chunk-local decay scan and the q / k rows
// (rescale, Walsh-Hadamard rotation, activation-dtype rounding, INT8 codes, transposed k_write tile).
#pragma once
#include "lq_common.cuh"

namespace lq {

struct PrologueArgs {
  const void *q, *k, *v;
  const float *g, *signs, *dqk;
  const float *sq, *sk, *skw, *svl, *svw;
  int8_t *qq, *kl, *kwT, *vlT, *vwT;
  float* gc;
  int T, H, NT;
  float scale, eta, qmax;
  int skip_v;  // delta family: the value operand is produced by the WY kernel instead
};

constexpr int kChunk = 64;

__device__ __forceinline__ void chunk_decay_scan(const float* g, int b, int c, int h, int T, int H, float* s_gc) {
  // warp 0 only: inclusive prefix sum of 64 log-decays, accumulated in double
  const int lane = threadIdx.x & 31;
  double run = 0.0;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int t = half * 32 + lane;
    double x = (double)g[((size_t)b * T + (size_t)c * kChunk + t) * H + h];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      double y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    x += run;
    s_gc[t] = (float)x;
    run = __shfl_sync(0xffffffffu, x, 31);
  }
}


// q and k rows of one chunk. Lane-in-row r of LPR = K/8 lanes holds channels 8r..8r+7; a group of LPR lanes walks
// four consecutive tokens so the transposed k_write tile can be packed four tokens to a word.
//   s_fk   [C]    key-side write gate Omega^(1-eta)
//   s_hw   [C]    optional per-token factor of the readout/write key (delta rule: beta^((1-sigma)tau)); the
//                 product is rounded to the activation dtype (reference.py:211)
//   s_kf   [C,LDK] optional fp32 copy of the rotated, rounded key (before s_hw) for the WY products
template <typename T, int K>
__device__ __forceinline__ void prologue_qk_rows(const PrologueArgs& a, int b, int c, int h, size_t tile,
                                                 const float* s_fk, const float* s_hw, float* s_kf, int LDK,
                                                 uint32_t (*s_kw)[17]) {
  constexpr int C = kChunk;
  constexpr int LPR = K / 8, G = 32 / LPR;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int r = lane % LPR, grp = lane / LPR;
  const float inv_sq = 1.0f / a.sq[h], inv_sk = 1.0f / a.sk[h];
  float sgn[8], dmul[8], dinv[8], inv_kw[8];
  const bool rot = a.signs != nullptr;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    sgn[j] = rot ? a.signs[8 * r + j] * (K == 64 ? 0.125f : 0.08838834764831845f) : 1.0f;
    dmul[j] = a.dqk ? a.dqk[h * K + 8 * r + j] : 1.0f;
    dinv[j] = 1.0f / dmul[j];
    inv_kw[j] = 1.0f / a.skw[h * K + 8 * r + j];
  }
  const T* qp = reinterpret_cast<const T*>(a.q);
  const T* kp = reinterpret_cast<const T*>(a.k);
  for (int tg = warp * G + grp; tg < C / 4; tg += nwarps * G) {
    uint32_t kwp[8];
    // all eight row loads of the group are in flight before the first is used (the code stores below would
    // otherwise order them one DRAM round trip after another)
    uint4 rq[4], rk[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const size_t row = (((size_t)b * a.T + (size_t)c * C + 4 * tg + i) * a.H + h) * K + 8 * r;
      rq[i] = __ldg(reinterpret_cast<const uint4*>(qp + row));
      rk[i] = __ldg(reinterpret_cast<const uint4*>(kp + row));
    }
    // tokens in the order 2, 3, 0, 1: the saturating pack takes two codes and an upper half, so the pair (2,3) is
    // packed first and rides along as the upper half when the pair (0,1) is packed
    int kprev[8];
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int i = (ii + 2) & 3;
      const int t = 4 * tg + i;
      const size_t orow = (tile * C + t) * K + 8 * r;
      float x[8];
      int cd[8];
      Act<T>::unpack8(rq[i], x);
      if (a.dqk) {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = __fmul_rn(x[j], dmul[j]);
      }
      if (rot) {
        fwht8<LPR>(x, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = Act<T>::round(__fmul_rn(x[j], sgn[j]));
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) cd[j] = q8(__fmul_rn(x[j], a.scale), inv_sq, a.qmax);
      *reinterpret_cast<uint2*>(a.qq + orow) =
          make_uint2(pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]));
      Act<T>::unpack8(rk[i], x);
      if (a.dqk) {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = __fmul_rn(x[j], dinv[j]);
      }
      if (rot) {
        fwht8<LPR>(x, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = Act<T>::round(__fmul_rn(x[j], sgn[j]));
      }
      if (s_kf != nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j) s_kf[t * LDK + 8 * r + j] = x[j];
      }
      if (s_hw != nullptr) {
        const float hw = s_hw[t];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = Act<T>::round(__fmul_rn(x[j], hw));
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) cd[j] = q8(x[j], inv_sk, a.qmax);
      *reinterpret_cast<uint2*>(a.kl + (tile * C + kl_row_of_token(t)) * K + 8 * r) =
          make_uint2(pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]));
      const float fk = s_fk[t];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int cw = q8(__fmul_rn(x[j], fk), inv_kw[j], a.qmax);
        if (i & 1) kwp[j] = pack_sat_s8x2(cw, kprev[j], i == 3 ? 0u : kwp[j]);
        else kprev[j] = cw;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s_kw[8 * r + j][tg] = kwp[j];
  }
}

}  // namespace lq
