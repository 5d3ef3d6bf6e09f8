// Diagonal (per-channel) decay cells: GLA (linear family) and KDA (delta family).
//
// Three chunk-parallel kernels, one CTA per (batch*head, chunk):
//   rows   chunk-local cumulative log-decay per channel (double accumulate), log envelope, pre-decayed q_read codes,
//          gated k_write codes (Omega * s^-eta), and for the linear family the v_local / v_write codes
//   amat   the intra-chunk matrix A in 16-token secondary chunks: off-diagonal blocks as INT8 MMAs on operands
//          re-scaled around the block's anchor row (optionally rotated by a signed Hadamard on fp16-rounded values),
//          diagonal blocks as an fp32 reduction with the exact per-channel weights on the dequantised codes
//   kda_wy KDA only: unquantised Gram matrix with per-channel weights, (I+G)^-1, W codes, U
// The state pass and the output kernel are the scalar-decay kernels instantiated with per-channel carry decay
// and a precomputed A.
//
// Reference arithmetic: zoo/gla.py:27-63 (_gla_A_inter), :66-99 (_gla_A_intra), :103-148 (state), :171-213 (output),
// :249-250 (cumsum, envelope); zoo/kda.py:22-53 (_prep); reference.py:125-152, :155-163.
#include "lq_wy.cuh"
#include "lq_zoo_rows.cuh"

namespace lq {

struct DiagArgs {
  const void *q, *k, *v;
  const float *g, *beta, *signs;
  const float *sq, *sk, *skw, *svl, *svw, *sw;
  int8_t *qq, *kwT, *vlT, *vwT, *wq;
  float *gc, *genv, *gcl, *fw;
  void* u;
  __half* amat;
  int T, H, NT;
  float scale, eta, sigma, tau, qmax;
};

template <int K, int BATCH = 64 * K / 4 / 256>
__device__ __forceinline__ void load_gc_tile(const float* gc_tile, float* s_gc) {  // 256 threads
  // BATCH 16-byte loads of the thread are requested before the first of them is stored (one or two trips to memory
  // instead of one per load)
  constexpr int NIT = 64 * K / 4 / 256;
#pragma unroll
  for (int b0 = 0; b0 < NIT; b0 += BATCH) {
    float4 v[BATCH];
#pragma unroll
    for (int it = 0; it < BATCH; ++it) v[it] = __ldg(reinterpret_cast<const float4*>(gc_tile) + threadIdx.x + 256 * (b0 + it));
#pragma unroll
    for (int it = 0; it < BATCH; ++it) {
      const int i = threadIdx.x + 256 * (b0 + it), t = i / (K / 4), c4 = i % (K / 4);
      *reinterpret_cast<float4*>(s_gc + t * (K + 4) + 4 * c4) = v[it];
    }
  }
}

// ------------------------------------------------------------------------------------------------ rows
template <typename T, int K, int V, bool DELTA>
__global__ void __launch_bounds__(256) zoo_diag_rows_kernel(DiagArgs a) {
  constexpr int C = 64, LD = K + 4;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  float* s_gc = reinterpret_cast<float*>(smem_raw);
  float* s_le = s_gc + C * LD;
  float* s_hw = s_le + C;
  uint32_t(*s_kw)[17] = reinterpret_cast<uint32_t(*)[17]>(s_hw + C);
  uint32_t(*s_vl)[17] = s_kw + K;
  uint32_t(*s_vw)[17] = s_vl + V;

  const int c = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const size_t tile = (size_t)bh * a.NT + c;
  const float e_hw = (1.f - a.sigma) * a.tau;

  // stage the raw log-decays of the chunk (coalesced), then one thread per channel scans them in double
  {
    constexpr int NIT = C * (K / 4) / 256;
    float4 v[NIT];
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int i = tid + 256 * it, t = i / (K / 4), c4 = i % (K / 4);
      v[it] = __ldg(reinterpret_cast<const float4*>(a.g + (((size_t)b * a.T + (size_t)c * C + t) * a.H + h) * K) + c4);
    }
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int i = tid + 256 * it, t = i / (K / 4), c4 = i % (K / 4);
      *reinterpret_cast<float4*>(s_gc + t * LD + 4 * c4) = v[it];
    }
  }
  if (DELTA && tid >= 128 && tid < 128 + C) {
    const int t = tid - 128;
    const float bt = a.beta[((size_t)b * a.T + (size_t)c * C + t) * a.H + h];
    s_hw[t] = pow_exact01(bt, e_hw);
  }
  __syncthreads();
  if (tid < K) {
    double acc = 0.0;
    float f = 0.f;
#pragma unroll 8
    for (int t = 0; t < C; ++t) {
      acc += (double)s_gc[t * LD + tid];
      f = (float)acc;
      s_gc[t * LD + tid] = f;
    }
    a.gcl[tile * K + tid] = f;
  }
  __syncthreads();
  for (int i = tid; i < C * (K / 4); i += 256) {
    const int t = i / (K / 4), c4 = i % (K / 4);
    reinterpret_cast<float4*>(a.gc + (tile * C + t) * K)[c4] = *reinterpret_cast<const float4*>(s_gc + t * LD + 4 * c4);
  }
  __syncthreads();
  for (int tt = 0; tt < 8; ++tt) {
    const int t = 8 * warp + tt;
    float m = -INFINITY;
    for (int n = lane; n < K; n += 32) m = fmaxf(m, s_gc[(C - 1) * LD + n] - s_gc[t * LD + n]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    if (lane == 0) {
      s_le[t] = m;
      a.genv[tile * C + t] = m;
    }
  }
  __syncthreads();

  {
    constexpr int LPR = K / 8, G = 32 / LPR;
    const int r = lane % LPR, grp = lane / LPR;
    const float inv_sq = 1.0f / a.sq[h];
    float inv_kw[8], gl[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      inv_kw[j] = 1.0f / a.skw[h * K + 8 * r + j];
      gl[j] = s_gc[(C - 1) * LD + 8 * r + j];
    }
    const T* qp = reinterpret_cast<const T*>(a.q);
    const T* kp = reinterpret_cast<const T*>(a.k);
    for (int tg = warp * G + grp; tg < C / 4; tg += 8 * G) {
      uint32_t kwp[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) kwp[j] = 0u;
      // the eight row loads of the group are in flight before the first is used
      uint4 rq[4], rk[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const size_t row = (((size_t)b * a.T + (size_t)c * C + 4 * tg + i) * a.H + h) * K + 8 * r;
        rq[i] = __ldg(reinterpret_cast<const uint4*>(qp + row));
        rk[i] = __ldg(reinterpret_cast<const uint4*>(kp + row));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = 4 * tg + i;
        float x[8], gv[8];
        int cd[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) gv[j] = s_gc[t * LD + 8 * r + j];
        Act<T>::unpack8(rq[i], x);
#pragma unroll
        for (int j = 0; j < 8; ++j) cd[j] = q8(__fmul_rn(__fmul_rn(x[j], __expf(gv[j])), a.scale), inv_sq, a.qmax);
        *reinterpret_cast<uint2*>(a.qq + (tile * C + t) * K + 8 * r) =
            make_uint2(pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]));
        Act<T>::unpack8(rk[i], x);
        if (DELTA && e_hw != 0.f) {
          const float hw = s_hw[t];
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] = Act<T>::round(__fmul_rn(x[j], hw));
        }
        const float ele = a.eta * s_le[t];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float w = __expf(__fsub_rn(__fsub_rn(gl[j], gv[j]), ele));
          kwp[j] |= ((uint32_t)q8(__fmul_rn(x[j], w), inv_kw[j], a.qmax) & 0xffu) << (8 * i);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s_kw[8 * r + j][tg] = kwp[j];
    }
  }
  if (!DELTA) {
    constexpr int LPR = V / 8, G = 32 / LPR;
    const int r = lane % LPR, grp = lane / LPR;
    float inv_vl[8], inv_vw[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      inv_vl[j] = 1.0f / a.svl[h * V + 8 * r + j];
      inv_vw[j] = 1.0f / a.svw[h * V + 8 * r + j];
    }
    const T* vp = reinterpret_cast<const T*>(a.v);
    for (int tg = warp * G + grp; tg < C / 4; tg += 8 * G) {
      uint32_t vlp[8], vwp[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) vlp[j] = vwp[j] = 0u;
      uint4 rv[4];  // the four row loads of the group are in flight before the first is used
#pragma unroll
      for (int i = 0; i < 4; ++i)
        rv[i] = __ldg(reinterpret_cast<const uint4*>(vp + (((size_t)b * a.T + (size_t)c * C + 4 * tg + i) * a.H + h) * V + 8 * r));
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = 4 * tg + i;
        float x[8];
        Act<T>::unpack8(rv[i], x);
        const float fv = expf(a.eta * s_le[t]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          vlp[j] |= ((uint32_t)q8(x[j], inv_vl[j], a.qmax) & 0xffu) << (8 * i);
          vwp[j] |= ((uint32_t)q8(__fmul_rn(x[j], fv), inv_vw[j], a.qmax) & 0xffu) << (8 * i);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s_vl[8 * r + j][tg] = vlp[j];
        s_vw[8 * r + j][tg] = vwp[j];
      }
    }
  }
  __syncthreads();
  uint32_t* kw_out = reinterpret_cast<uint32_t*>(a.kwT + tile * (size_t)(K * C));
  for (int i = tid; i < K * 16; i += 256) kw_out[i] = s_kw[i >> 4][i & 15];
  if (!DELTA) {
    uint32_t* vl_out = reinterpret_cast<uint32_t*>(a.vlT + tile * (size_t)(V * C));
    uint32_t* vw_out = reinterpret_cast<uint32_t*>(a.vwT + tile * (size_t)(V * C));
    for (int i = tid; i < V * 16; i += 256) {
      vl_out[i] = s_vl[i >> 4][i & 15];
      vw_out[i] = s_vw[i >> 4][i & 15];
    }
  }
}

// ------------------------------------------------------------------------------------------------ A matrix
template <typename T, int K>
__global__ void __launch_bounds__(256) zoo_diag_amat_kernel(DiagArgs a) {
  constexpr int C = 64, LD = K + 4, SUB = 16;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  float* s_gc = reinterpret_cast<float*>(smem_raw);
  float* s_A = s_gc + C * LD;
  float* s_hw = s_A + C * 65;
  int8_t* s_qc = reinterpret_cast<int8_t*>(s_hw + C);
  int8_t* s_kc = s_qc + C * K;
  int8_t* s_qa = s_kc + C * K;
  int8_t* s_ka = s_qa + SUB * K;

  const int c = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j4 = lane & 3;
  const size_t tile = (size_t)bh * a.NT + c;
  const float e_hw = (1.f - a.sigma) * a.tau;
  const bool use_hw = a.beta != nullptr && e_hw != 0.f;
  const bool rot = a.signs != nullptr;

  constexpr int LPR = K / 8, G = 32 / LPR;
  const int r = lane % LPR, grp = lane / LPR;
  const T* qp = reinterpret_cast<const T*>(a.q);
  const T* kp = reinterpret_cast<const T*>(a.k);
  auto grow = [&](int t) { return (((size_t)b * a.T + (size_t)c * C + t) * a.H + h) * K + 8 * r; };

  // The rows of the bare operands (diagonal blocks) are requested first of all, so that their trip to memory runs
  // beside that of the log-decay tile; every row load of the thread is issued before the first is used.
  constexpr int NIT = C / (8 * G);
  uint4 rq0[NIT], rk0[NIT];
#pragma unroll
  for (int u = 0; u < NIT; ++u) {
    const int t = warp * G + grp + 8 * G * u;
    rq0[u] = __ldg(reinterpret_cast<const uint4*>(qp + grow(t)));
    rk0[u] = __ldg(reinterpret_cast<const uint4*>(kp + grow(t)));
  }
  load_gc_tile<K, K / 32>(a.gc + tile * (size_t)(C * K), s_gc);
  for (int i = tid; i < C * 65; i += 256) s_A[i] = 0.f;
  if (tid < C) {
    s_hw[tid] = use_hw ? pow_exact01(a.beta[((size_t)b * a.T + (size_t)c * C + tid) * a.H + h], e_hw) : 1.f;
  }
  __syncthreads();

  const float inv_sq = 1.0f / a.sq[h], inv_sk = 1.0f / a.sk[h];
  const float sqk = __fmul_rn(a.sq[h], a.sk[h]);
#pragma unroll
  for (int u = 0; u < NIT; ++u) {
    const int t = warp * G + grp + 8 * G * u;
    float x[8];
    int cd[8];
    Act<T>::unpack8(rq0[u], x);
#pragma unroll
    for (int j = 0; j < 8; ++j) cd[j] = q8(__fmul_rn(x[j], a.scale), inv_sq, a.qmax);
    *reinterpret_cast<uint2*>(s_qc + t * K + 8 * r) = make_uint2(pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]));
    Act<T>::unpack8(rk0[u], x);
    if (use_hw) {
      const float hw = s_hw[t];
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = Act<T>::round(__fmul_rn(x[j], hw));
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) cd[j] = q8(x[j], inv_sk, a.qmax);
    *reinterpret_cast<uint2*>(s_kc + t * K + 8 * r) = make_uint2(pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]));
  }

  // off-diagonal blocks: rows [16I, 16I+16) against columns [0, 16I), operands re-scaled around the anchor row 16I
  float sgn[8];
  {
    const float n16 = __half2float(__float2half_rn(K == 64 ? 0.125f : 0.08838834764831845f));
#pragma unroll
    for (int j = 0; j < 8; ++j) sgn[j] = rot ? a.signs[8 * r + j] * n16 : 1.f;
  }
  for (int I = 1; I < C / SUB; ++I) {
    float anc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) anc[j] = s_gc[(SUB * I) * LD + 8 * r + j];
    const int R = SUB + SUB * I;
    uint4 rrow[NIT];  // this thread's rows of the block row, requested together
#pragma unroll
    for (int u = 0; u < NIT; ++u) {
      const int rr = warp * G + grp + 8 * G * u;
      if (rr < R) rrow[u] = __ldg(reinterpret_cast<const uint4*>((rr < SUB ? qp : kp) + grow(rr < SUB ? SUB * I + rr : rr - SUB)));
    }
#pragma unroll
    for (int u = 0; u < NIT; ++u) {
      const int rr = warp * G + grp + 8 * G * u;
      if (rr >= R) break;
      const bool isq = rr < SUB;
      const int t = isq ? SUB * I + rr : rr - SUB;
      float x[8];
      int cd[8];
      Act<T>::unpack8(rrow[u], x);
      if (isq) {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = __fmul_rn(__fmul_rn(x[j], __expf(__fsub_rn(s_gc[t * LD + 8 * r + j], anc[j]))), a.scale);
      } else {
        if (use_hw) {
          const float hw = s_hw[t];
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] = Act<T>::round(__fmul_rn(x[j], hw));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = __fmul_rn(x[j], __expf(__fsub_rn(anc[j], s_gc[t * LD + 8 * r + j])));
      }
      if (rot) {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = __half2float(__float2half_rn(x[j]));
        fwht8<LPR>(x, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = __fmul_rn(x[j], sgn[j]);
      }
      const float inv = isq ? inv_sq : inv_sk;
#pragma unroll
      for (int j = 0; j < 8; ++j) cd[j] = q8(x[j], inv, a.qmax);
      int8_t* dst = isq ? (s_qa + rr * K) : (s_ka + (rr - SUB) * K);
      *reinterpret_cast<uint2*>(dst + 8 * r) = make_uint2(pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]));
    }
    __syncthreads();
    if (warp < 2 * I) {
      int acc[4] = {0, 0, 0, 0};
#pragma unroll
      for (int kk = 0; kk < K / 64; ++kk) {
        const uint4 qa = *reinterpret_cast<const uint4*>(s_qa + g * K + 64 * kk + 16 * j4);
        const uint4 qb = *reinterpret_cast<const uint4*>(s_qa + (g + 8) * K + 64 * kk + 16 * j4);
        const uint4 kb = *reinterpret_cast<const uint4*>(s_ka + (8 * warp + g) * K + 64 * kk + 16 * j4);
        mma_s8(acc, qa.x, qb.x, qa.y, qb.y, kb.x, kb.y);
        mma_s8(acc, qa.z, qb.z, qa.w, qb.w, kb.z, kb.w);
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        s_A[(SUB * I + g) * 65 + 8 * warp + 2 * j4 + e] = __fmul_rn((float)acc[e], sqk);
        s_A[(SUB * I + g + 8) * 65 + 8 * warp + 2 * j4 + e] = __fmul_rn((float)acc[2 + e], sqk);
      }
    }
    __syncthreads();
  }

  // diagonal blocks: A_ij = s_q s_k sum_n q^_in k^_jn exp(g_in - g_jn), i >= j inside a 16 x 16 block. The weight factors
  // around the block's first row a: exp(g_in - a_n) exp(a_n - g_jn). The first factor is <= 1; the second is >= 1 and grows
  // with the decay across at most 15 tokens, so per block the spread max_n (a_n - g_last,n) decides: up to 60 (a factor
  // below 1.2e26, far inside fp32) the block is two sets of 16 scaled rows (one exp per row element, 16 x fewer) and a
  // 16 x 16 x K fp32 product; beyond it (decays as strong as the g x 40 cases) the block takes one exp per (i, j, n).
  float* s_qd = reinterpret_cast<float*>(s_ka + 48 * K);  // [16][LD] q^ exp(g_i - a), then [16][LD] k^ exp(a - g_j)
  float* s_kd = s_qd + SUB * LD;
  __shared__ int s_exact[C / SUB];
  if (tid < C / SUB) s_exact[tid] = 0;
  __syncthreads();
  for (int i = tid; i < (C / SUB) * K; i += 256) {
    const int I = i / K, n = i - I * K;
    if (__fsub_rn(s_gc[(SUB * I) * LD + n], s_gc[(SUB * I + SUB - 1) * LD + n]) > 60.f) s_exact[I] = 1;
  }
  __syncthreads();
  for (int I = 0; I < C / SUB; ++I) {
    if (s_exact[I]) {  // 136 (i >= j) pairs, eight lanes per pair, four channels per lane and step (128-bit loads)
      for (int pass = 0; pass < 5; ++pass) {
        const int rem_raw = pass * 32 + (tid >> 3);
        const bool valid = rem_raw < 136;  // the last pass has idle pairs: they compute a clamped pair and store nothing
        const int rem = valid ? rem_raw : 135;
        {
          int i = (int)((sqrtf(8.f * rem + 1.f) - 1.f) * 0.5f);
          while ((i + 1) * (i + 2) / 2 <= rem) ++i;
          while (i * (i + 1) / 2 > rem) --i;
          const int jj = rem - i * (i + 1) / 2;
          const int ti = SUB * I + i, tj = SUB * I + jj;
          const int l8 = tid & 7;
          float sum = 0.f;
#pragma unroll
          for (int n4 = 0; n4 < K / 32; ++n4) {
            const int n = 4 * l8 + 32 * n4;  // the eight lanes of a pair read 128 consecutive bytes of a gc row
            const float4 gi = *reinterpret_cast<const float4*>(s_gc + ti * LD + n);
            const float4 gj = *reinterpret_cast<const float4*>(s_gc + tj * LD + n);
            const uint32_t qw = *reinterpret_cast<const uint32_t*>(s_qc + ti * K + n) ^ 0x80808080u;
            const uint32_t kw = *reinterpret_cast<const uint32_t*>(s_kc + tj * K + n) ^ 0x80808080u;
            sum = fmaf(__fmul_rn(s8_to_float<0>(qw), s8_to_float<0>(kw)), __expf(gi.x - gj.x), sum);
            sum = fmaf(__fmul_rn(s8_to_float<1>(qw), s8_to_float<1>(kw)), __expf(gi.y - gj.y), sum);
            sum = fmaf(__fmul_rn(s8_to_float<2>(qw), s8_to_float<2>(kw)), __expf(gi.z - gj.z), sum);
            sum = fmaf(__fmul_rn(s8_to_float<3>(qw), s8_to_float<3>(kw)), __expf(gi.w - gj.w), sum);
          }
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          sum += __shfl_xor_sync(0xffffffffu, sum, 4);
          if (l8 == 0 && valid) s_A[ti * 65 + tj] = __fmul_rn(sum, sqk);
        }
      }
      __syncthreads();
      continue;
    }
    // scaled rows: thread = (row of the block, 4-channel piece); 2 x 16 x K elements over 256 threads
    for (int i = tid; i < SUB * (K / 4); i += 256) {
      const int rr = i / (K / 4), n = 4 * (i - rr * (K / 4));
      const int t = SUB * I + rr;
      const float4 an = *reinterpret_cast<const float4*>(s_gc + (SUB * I) * LD + n);
      const float4 gt = *reinterpret_cast<const float4*>(s_gc + t * LD + n);
      const uint32_t qw = *reinterpret_cast<const uint32_t*>(s_qc + t * K + n) ^ 0x80808080u;
      const uint32_t kw = *reinterpret_cast<const uint32_t*>(s_kc + t * K + n) ^ 0x80808080u;
      *reinterpret_cast<float4*>(s_qd + rr * LD + n) =
          make_float4(__fmul_rn(s8_to_float<0>(qw), __expf(gt.x - an.x)), __fmul_rn(s8_to_float<1>(qw), __expf(gt.y - an.y)),
                      __fmul_rn(s8_to_float<2>(qw), __expf(gt.z - an.z)), __fmul_rn(s8_to_float<3>(qw), __expf(gt.w - an.w)));
      *reinterpret_cast<float4*>(s_kd + rr * LD + n) =
          make_float4(__fmul_rn(s8_to_float<0>(kw), __expf(an.x - gt.x)), __fmul_rn(s8_to_float<1>(kw), __expf(an.y - gt.y)),
                      __fmul_rn(s8_to_float<2>(kw), __expf(an.z - gt.z)), __fmul_rn(s8_to_float<3>(kw), __expf(an.w - gt.w)));
    }
    __syncthreads();
    {  // 16 x 16 x K product on the tensor cores, 3xTF32 (both factors split into a TF32 part and a TF32 remainder: the
       // products are good to about 2^-21). Warp w contracts the channels [K/8 w, K/8 (w + 1)); the eight partial blocks
       // are parked behind the scaled rows and summed in a fixed order.
      float* s_part = s_kd + SUB * LD;  // [8 warps][16][16]
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < K / 64; ++kk) {
        const int c0 = (K / 8) * warp + 8 * kk + j4, c1 = c0 + 4;
        const float xa[4] = {s_qd[g * LD + c0], s_qd[(g + 8) * LD + c0], s_qd[g * LD + c1], s_qd[(g + 8) * LD + c1]};
        uint32_t ab[4], as_[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          ab[e] = tf32_rna(xa[e]);
          as_[e] = tf32_rna(xa[e] - __uint_as_float(ab[e]));
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const float y0 = s_kd[(8 * nt + g) * LD + c0], y1 = s_kd[(8 * nt + g) * LD + c1];
          const uint32_t b0 = tf32_rna(y0), b1 = tf32_rna(y1);
          const uint32_t s0 = tf32_rna(y0 - __uint_as_float(b0)), s1 = tf32_rna(y1 - __uint_as_float(b1));
          mma_tf32(acc[nt], as_[0], as_[1], as_[2], as_[3], b0, b1);
          mma_tf32(acc[nt], ab[0], ab[1], ab[2], ab[3], s0, s1);
          mma_tf32(acc[nt], ab[0], ab[1], ab[2], ab[3], b0, b1);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        float* pw = s_part + warp * 256;
        pw[g * 16 + 8 * nt + 2 * j4] = acc[nt][0];
        pw[g * 16 + 8 * nt + 2 * j4 + 1] = acc[nt][1];
        pw[(g + 8) * 16 + 8 * nt + 2 * j4] = acc[nt][2];
        pw[(g + 8) * 16 + 8 * nt + 2 * j4 + 1] = acc[nt][3];
      }
      __syncthreads();
      {
        const int i = tid >> 4, jj = tid & 15;
        if (jj <= i) {
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < 8; ++w) sum += s_part[w * 256 + tid];
          s_A[(SUB * I + i) * 65 + SUB * I + jj] = __fmul_rn(sum, sqk);
        }
      }
    }
    __syncthreads();
  }
  __syncthreads();
  uint32_t* out = reinterpret_cast<uint32_t*>(a.amat + tile * (size_t)(C * C));
  for (int i = tid; i < C * 32; i += 256) {
    const int row = i >> 5, cp = i & 31;
    out[i] = Act<__half>::pack2(s_A[row * 65 + 2 * cp], s_A[row * 65 + 2 * cp + 1]);
  }
}

// ------------------------------------------------------------------------------------------------ KDA WY prep
// Gram matrix G[i][j] = beta_i^sigma beta_j^(1-sigma) sum_n k[i,n] k[j,n] exp(gc[i,n] - gc[j,n]), i > j, in 16-token
// secondary chunks like the A matrix: inside a diagonal block every (i, j, n) takes its own exp (exponent <= 0);
// for block row I against the earlier tokens the operands are re-scaled around the anchor row 16 I,
//   kd[i,n] = k[i,n] exp(gc[i,n] - gc[16I,n]),  ke[j,n] = k[j,n] exp(gc[16I,n] - gc[j,n])   (both factors <= 1),
// and contracted on the tensor cores as 3xTF32 (big*big + big*small + small*big), which keeps fp32-grade products.
// W and U are T diag(beta^sigma) times k exp(gc) (3xTF32, both operands split) and times v (exact in TF32).
template <typename T, int K>
__device__ __forceinline__ void kda_scaled_rows(const DiagArgs& a, int b, int c, int h, const float* s_gc, float* s_x,
                                                int anchor_row, int first_row, int nrows, int dst_row, bool toward_anchor) {
  // rows [first_row, first_row + nrows) of k, times exp(gc[row] - gc[anchor]) (toward_anchor) or exp(gc[anchor] - gc[row]),
  // or times exp(gc[row]) when anchor_row < 0; written as fp32 to s_x rows dst_row ...
  constexpr int C = 64, LD = K + 4, LPR = K / 8, MAXIT = C * LPR / 256;
  const T* kp = reinterpret_cast<const T*>(a.k);
  // every row piece of the thread is requested before the first is used (at most MAXIT of them: nrows <= 64)
  uint4 raw[MAXIT];
#pragma unroll
  for (int it = 0; it < MAXIT; ++it) {
    const int i = threadIdx.x + 256 * it;
    if (i < nrows * LPR) {
      const int rr = i / LPR, seg = i % LPR;
      raw[it] = __ldg(reinterpret_cast<const uint4*>(kp + (((size_t)b * a.T + (size_t)c * C + first_row + rr) * a.H + h) * K + 8 * seg));
    }
  }
#pragma unroll
  for (int it = 0; it < MAXIT; ++it) {
    const int i = threadIdx.x + 256 * it;
    if (i >= nrows * LPR) break;
    const int rr = i / LPR, seg = i % LPR;
    const int t = first_row + rr;
    float x[8];
    Act<T>::unpack8(raw[it], x);
    const float4 g0 = *reinterpret_cast<const float4*>(s_gc + t * LD + 8 * seg);
    const float4 g1 = *reinterpret_cast<const float4*>(s_gc + t * LD + 8 * seg + 4);
    float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    if (anchor_row >= 0) {
      const float4 a0 = *reinterpret_cast<const float4*>(s_gc + anchor_row * LD + 8 * seg);
      const float4 a1 = *reinterpret_cast<const float4*>(s_gc + anchor_row * LD + 8 * seg + 4);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) gv[e] = toward_anchor ? __fsub_rn(gv[e], av[e]) : __fsub_rn(av[e], gv[e]);
    }
    float y[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = __fmul_rn(x[e], __expf(gv[e]));
    *reinterpret_cast<float4*>(s_x + (dst_row + rr) * LD + 8 * seg) = make_float4(y[0], y[1], y[2], y[3]);
    *reinterpret_cast<float4*>(s_x + (dst_row + rr) * LD + 8 * seg + 4) = make_float4(y[4], y[5], y[6], y[7]);
  }
}

template <typename T, int K, int V>
__global__ void __launch_bounds__(256) zoo_kda_wy_kernel(DiagArgs a) {
  constexpr int C = 64, LD = K + 4, LDV = V + 8, SUB = 16;
  constexpr int REG0 = C * (LD > LDV ? LD : LDV);
  extern __shared__ __align__(16) uint8_t smem_raw[];
  float* s_gc = reinterpret_cast<float*>(smem_raw);  // gc tile; v (fp32) once the decayed keys are formed
  float* s_x = s_gc + REG0;                          // k (fp32), then anchored operands, then k exp(gc)
  float* s_G = s_x + C * LD;
  float* s_T = s_G + C * 68;
  float* s_bs = s_T + C * 68;
  float* s_b1 = s_bs + C;
  float* s_part = s_b1 + C;  // [8 warps][16][16] partial diagonal blocks
  float* s_vf = s_gc;

  const int c = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j4 = lane & 3;
  const size_t tile = (size_t)bh * a.NT + c;

  load_gc_tile<K>(a.gc + tile * (size_t)(C * K), s_gc);
  {
    const T* kp = reinterpret_cast<const T*>(a.k);
    constexpr int NIT = C * (K / 8) / 256;
    uint4 raw[NIT];
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int i = tid + 256 * it, t = i / (K / 8), seg = i % (K / 8);
      raw[it] = __ldg(reinterpret_cast<const uint4*>(kp + (((size_t)b * a.T + (size_t)c * C + t) * a.H + h) * K + 8 * seg));
    }
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int i = tid + 256 * it, t = i / (K / 8), seg = i % (K / 8);
      float x[8];
      Act<T>::unpack8(raw[it], x);
      *reinterpret_cast<float4*>(s_x + t * LD + 8 * seg) = make_float4(x[0], x[1], x[2], x[3]);
      *reinterpret_cast<float4*>(s_x + t * LD + 8 * seg + 4) = make_float4(x[4], x[5], x[6], x[7]);
    }
  }
  if (tid < C) {
    const float bt = a.beta[((size_t)b * a.T + (size_t)c * C + tid) * a.H + h];
    s_bs[tid] = pow_exact01(bt, a.sigma);
    s_b1[tid] = pow_exact01(bt, 1.f - a.sigma);
    a.fw[tile * C + tid] = pow_exact01(bt, (1.f - a.sigma) * (1.f - a.tau));
  }
  for (int i = tid; i < C * 68; i += 256) s_G[i] = 0.f;
  __syncthreads();

  // ---- diagonal blocks (strictly lower pairs of each 16 x 16 block). As in the A matrix the per-channel weight
  // exp(gc_in - gc_jn) factors around the block's first row a into exp(gc_in - a_n) (<= 1) and exp(a_n - gc_jn) (>= 1): two
  // sets of 16 scaled rows (in the space of T, which is not needed yet) and a 16 x 16 x K fp32 product. A block whose
  // decay spread max_n (a_n - gc_last,n) exceeds 60 keeps one exp per (i, j, n).
  {
    float* s_kq = s_T;             // [16][LD] k exp(gc_i - a)
    float* s_kk = s_T + SUB * LD;  // [16][LD] k exp(a - gc_j)
    __shared__ int s_exact[C / SUB];
    if (tid < C / SUB) s_exact[tid] = 0;
    __syncthreads();
    for (int i = tid; i < (C / SUB) * K; i += 256) {
      const int I = i / K, n = i - I * K;
      if (__fsub_rn(s_gc[(SUB * I) * LD + n], s_gc[(SUB * I + SUB - 1) * LD + n]) > 60.f) s_exact[I] = 1;
    }
    __syncthreads();
    for (int I = 0; I < C / SUB; ++I) {
      if (s_exact[I]) {  // 120 strictly-lower pairs, eight lanes per pair
        for (int pass = 0; pass < 4; ++pass) {
          const int rem_raw = pass * 32 + (tid >> 3);
          const bool valid = rem_raw < 120;  // idle pairs of the last pass compute a clamped pair and store nothing
          const int rem = valid ? rem_raw : 119;
          int i = (int)((sqrtf(8.f * rem + 1.f) + 1.f) * 0.5f);
          while (i * (i + 1) / 2 <= rem) ++i;
          while (i * (i - 1) / 2 > rem) --i;
          const int jj = rem - i * (i - 1) / 2;
          const int ti = SUB * I + i, tj = SUB * I + jj;
          const int l8 = tid & 7;
          float sum = 0.f;
#pragma unroll
          for (int n4 = 0; n4 < K / 32; ++n4) {
            const int n = 4 * l8 + 32 * n4;  // the eight lanes of a pair read 128 consecutive bytes of each row
            const float4 gi = *reinterpret_cast<const float4*>(s_gc + ti * LD + n), gj = *reinterpret_cast<const float4*>(s_gc + tj * LD + n);
            const float4 xi = *reinterpret_cast<const float4*>(s_x + ti * LD + n), xj = *reinterpret_cast<const float4*>(s_x + tj * LD + n);
            sum = fmaf(xi.x * xj.x, __expf(gi.x - gj.x), sum);
            sum = fmaf(xi.y * xj.y, __expf(gi.y - gj.y), sum);
            sum = fmaf(xi.z * xj.z, __expf(gi.z - gj.z), sum);
            sum = fmaf(xi.w * xj.w, __expf(gi.w - gj.w), sum);
          }
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          sum += __shfl_xor_sync(0xffffffffu, sum, 4);
          if (l8 == 0 && valid) s_G[ti * 68 + tj] = s_bs[ti] * s_b1[tj] * sum;
        }
        __syncthreads();
        continue;
      }
      for (int i = tid; i < SUB * (K / 4); i += 256) {
        const int rr = i / (K / 4), n = 4 * (i - rr * (K / 4));
        const int t = SUB * I + rr;
        const float4 an = *reinterpret_cast<const float4*>(s_gc + (SUB * I) * LD + n);
        const float4 gt = *reinterpret_cast<const float4*>(s_gc + t * LD + n);
        const float4 xv = *reinterpret_cast<const float4*>(s_x + t * LD + n);
        *reinterpret_cast<float4*>(s_kq + rr * LD + n) = make_float4(__fmul_rn(xv.x, __expf(gt.x - an.x)), __fmul_rn(xv.y, __expf(gt.y - an.y)),
                                                                     __fmul_rn(xv.z, __expf(gt.z - an.z)), __fmul_rn(xv.w, __expf(gt.w - an.w)));
        *reinterpret_cast<float4*>(s_kk + rr * LD + n) = make_float4(__fmul_rn(xv.x, __expf(an.x - gt.x)), __fmul_rn(xv.y, __expf(an.y - gt.y)),
                                                                     __fmul_rn(xv.z, __expf(an.z - gt.z)), __fmul_rn(xv.w, __expf(an.w - gt.w)));
      }
      __syncthreads();
      {  // 16 x 16 x K product on the tensor cores, 3xTF32, as in the A matrix: warp w contracts the channels
         // [K/8 w, K/8 (w + 1)), the eight partial blocks are summed in a fixed order
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int kk = 0; kk < K / 64; ++kk) {
          const int c0 = (K / 8) * warp + 8 * kk + j4, c1 = c0 + 4;
          const float xa[4] = {s_kq[g * LD + c0], s_kq[(g + 8) * LD + c0], s_kq[g * LD + c1], s_kq[(g + 8) * LD + c1]};
          uint32_t ab[4], as_[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            ab[e] = tf32_rna(xa[e]);
            as_[e] = tf32_rna(xa[e] - __uint_as_float(ab[e]));
          }
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            const float y0 = s_kk[(8 * nt + g) * LD + c0], y1 = s_kk[(8 * nt + g) * LD + c1];
            const uint32_t b0 = tf32_rna(y0), b1 = tf32_rna(y1);
            const uint32_t s0 = tf32_rna(y0 - __uint_as_float(b0)), s1 = tf32_rna(y1 - __uint_as_float(b1));
            mma_tf32(acc[nt], as_[0], as_[1], as_[2], as_[3], b0, b1);
            mma_tf32(acc[nt], ab[0], ab[1], ab[2], ab[3], s0, s1);
            mma_tf32(acc[nt], ab[0], ab[1], ab[2], ab[3], b0, b1);
          }
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          float* pw = s_part + warp * 256;
          pw[g * 16 + 8 * nt + 2 * j4] = acc[nt][0];
          pw[g * 16 + 8 * nt + 2 * j4 + 1] = acc[nt][1];
          pw[(g + 8) * 16 + 8 * nt + 2 * j4] = acc[nt][2];
          pw[(g + 8) * 16 + 8 * nt + 2 * j4 + 1] = acc[nt][3];
        }
        __syncthreads();
        const int i = tid >> 4, jj = tid & 15;
        if (jj < i) {
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < 8; ++w) sum += s_part[w * 256 + tid];
          const int ti = SUB * I + i;
          s_G[ti * 68 + SUB * I + jj] = s_bs[ti] * s_b1[SUB * I + jj] * sum;
        }
      }
      __syncthreads();
    }
  }

  // ---- off-diagonal blocks: block row I against tokens [0, 16 I), anchored at row 16 I
  for (int I = 1; I < C / SUB; ++I) {
    kda_scaled_rows<T, K>(a, b, c, h, s_gc, s_x, SUB * I, 0, SUB * I, 0, false);        // ke -> rows 0 .. 16I-1
    kda_scaled_rows<T, K>(a, b, c, h, s_gc, s_x, SUB * I, SUB * I, SUB, 48, true);      // kd -> rows 48 .. 63
    __syncthreads();
    // 2 I column tiles of eight tokens x four quarters of the channels = 8 I units of work, dealt to the eight warps
    // (one column tile per warp would leave 8 - 2 I warps idle); the quarter sums are parked in the space of T, which is
    // not needed before the solve, and added in a fixed order.
    for (int u = warp; u < 8 * I; u += 8) {
      const int nt = u >> 2, kq = u & 3;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const float* ra = s_x + (48 + g) * LD;
      const float* rb = s_x + (56 + g) * LD;
      const float* rn = s_x + (8 * nt + g) * LD;
#pragma unroll
      for (int ks = 0; ks < K / 32; ++ks) {
        const int c0 = 8 * (kq * (K / 32) + ks) + j4, c1 = c0 + 4;
        const float xa[4] = {ra[c0], rb[c0], ra[c1], rb[c1]};
        const float xb[2] = {rn[c0], rn[c1]};
        uint32_t ab[4], as_[4], bb[2], bs_[2];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          ab[e] = tf32_rna(xa[e]);
          as_[e] = tf32_rna(xa[e] - __uint_as_float(ab[e]));
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          bb[e] = tf32_rna(xb[e]);
          bs_[e] = tf32_rna(xb[e] - __uint_as_float(bb[e]));
        }
        mma_tf32(acc, as_[0], as_[1], as_[2], as_[3], bb[0], bb[1]);
        mma_tf32(acc, ab[0], ab[1], ab[2], ab[3], bs_[0], bs_[1]);
        mma_tf32(acc, ab[0], ab[1], ab[2], ab[3], bb[0], bb[1]);
      }
      float* pp = s_T + u * 128;  // [16 rows][8 columns]
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        pp[g * 8 + 2 * j4 + e] = acc[e];
        pp[(g + 8) * 8 + 2 * j4 + e] = acc[2 + e];
      }
    }
    __syncthreads();
    for (int el = tid; el < 256 * I; el += 256) {
      const int i = el / (16 * I), jj = el - i * (16 * I);
      const float* pp = s_T + (4 * (jj >> 3)) * 128 + i * 8 + (jj & 7);
      const float sum = ((pp[0] + pp[128]) + pp[256]) + pp[384];
      const int ia = SUB * I + i;
      s_G[ia * 68 + jj] = s_bs[ia] * s_b1[jj] * sum;
    }
    __syncthreads();
  }
  wy_solve(s_G, s_T);
  // decayed keys k * exp(gc) (the Gram passes are done); then the gc region is free for v
  kda_scaled_rows<T, K>(a, b, c, h, s_gc, s_x, -1, 0, C, 0, false);
  __syncthreads();
  {
    const T* vp = reinterpret_cast<const T*>(a.v);
    constexpr int NIT = C * (V / 8) / 256;
    uint4 raw[NIT];
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int i = tid + 256 * it, t = i / (V / 8), seg = i % (V / 8);
      raw[it] = __ldg(reinterpret_cast<const uint4*>(vp + (((size_t)b * a.T + (size_t)c * C + t) * a.H + h) * V + 8 * seg));
    }
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int i = tid + 256 * it, t = i / (V / 8), seg = i % (V / 8);
      float x[8];
      Act<T>::unpack8(raw[it], x);
      *reinterpret_cast<float4*>(s_vf + t * LDV + 8 * seg) = make_float4(x[0], x[1], x[2], x[3]);
      *reinterpret_cast<float4*>(s_vf + t * LDV + 8 * seg + 4) = make_float4(x[4], x[5], x[6], x[7]);
    }
  }
  // Row tile mt of W and U contracts over 2 mt + 2 steps of eight tokens: every warp takes the row tiles pr and 3 - pr
  // (five steps on average instead of up to eight) and one quarter of the columns.
  const int pr = warp & 1, qd = warp >> 1;
  const float inv_sw = 1.0f / a.sw[h];
  // ---- W = T diag(beta^sigma) (k exp(gc))  -> w_read codes
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int mt = half == 0 ? pr : 3 - pr;
    constexpr int NTW = K / 32;
    float acc[NTW][4];
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    const int n0 = qd * (K / 4);
    wy_product_split<NTW>(acc, s_T, s_bs, s_x, LD, mt, n0, g, j4);
    const int ia = 16 * mt + g, ib = ia + 8;
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt) {
      const int col = n0 + 8 * nt + 2 * j4;
      const int a0 = q8(Act<T>::round(acc[nt][0]), inv_sw, a.qmax), a1 = q8(Act<T>::round(acc[nt][1]), inv_sw, a.qmax);
      const int b0 = q8(Act<T>::round(acc[nt][2]), inv_sw, a.qmax), b1 = q8(Act<T>::round(acc[nt][3]), inv_sw, a.qmax);
      *reinterpret_cast<uint16_t*>(a.wq + (tile * C + ia) * K + col) = (uint16_t)((a0 & 0xff) | ((a1 & 0xff) << 8));
      *reinterpret_cast<uint16_t*>(a.wq + (tile * C + ib) * K + col) = (uint16_t)((b0 & 0xff) | ((b1 & 0xff) << 8));
    }
  }
  __syncthreads();  // v staged by all threads
  // ---- U = T diag(beta^sigma) v (v is exact in TF32)
  T* up = reinterpret_cast<T*>(a.u);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int mt = half == 0 ? pr : 3 - pr;
    constexpr int NTU = V / 32;
    float acc[NTU][4];
#pragma unroll
    for (int nt = 0; nt < NTU; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    const int n0 = qd * (V / 4);
    wy_product<NTU>(acc, s_T, s_bs, s_vf, LDV, mt, n0, g, j4);
    const int ia = 16 * mt + g, ib = ia + 8;
#pragma unroll
    for (int nt = 0; nt < NTU; ++nt) {
      const int col = n0 + 8 * nt + 2 * j4;
      *reinterpret_cast<uint32_t*>(up + (tile * C + ia) * V + col) = Act<T>::pack2(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<uint32_t*>(up + (tile * C + ib) * V + col) = Act<T>::pack2(acc[nt][2], acc[nt][3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ launchers
int validate_zoo_problem(const lq_zoo_problem* p, bool delta, bool diagonal);

static void fill_diag_args(const lq_zoo_problem* p, const lq_zoo_workspace* ws, DiagArgs& a) {
  a.q = p->q; a.k = p->k; a.v = p->v; a.g = p->g; a.beta = p->beta; a.signs = p->rot_signs;
  a.sq = p->sq; a.sk = p->sk; a.skw = p->skw; a.svl = p->svl; a.svw = p->svw; a.sw = p->sw;
  a.qq = ws->qq; a.kwT = ws->kwT; a.vlT = ws->vlT; a.vwT = ws->vwT; a.wq = ws->wq;
  a.gc = ws->gc; a.genv = ws->genv; a.gcl = ws->gcl; a.fw = ws->fw; a.u = ws->u;
  a.amat = reinterpret_cast<__half*>(ws->amat);
  a.T = p->T; a.H = p->H; a.NT = p->T / p->chunk;
  a.scale = p->scale; a.eta = p->eta; a.sigma = p->sigma; a.tau = p->tau; a.qmax = p->qmax;
}

template <typename KernelT>
static int launch_big_smem(KernelT kern, const char* name, dim3 grid, size_t smem, const DiagArgs& a, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "%s: cannot opt in to %zu bytes of shared memory: %s", name, smem, cudaGetErrorString(e));
  kern<<<grid, 256, smem, st>>>(a);
  return check_launch(name);
}

template <typename T, int K, int V>
static int run_diag_T(const lq_zoo_problem* p, const DiagArgs& a, bool delta, int stage, cudaStream_t st) {
  dim3 grid(a.NT, p->B * p->H);
  if (stage == 0) {
    const size_t smem = sizeof(float) * (64 * (K + 4) + 128) + sizeof(uint32_t) * 17 * (K + 2 * V);
    if (delta) return launch_big_smem(zoo_diag_rows_kernel<T, K, V, true>, "zoo_diag_rows_kernel", grid, smem, a, st);
    return launch_big_smem(zoo_diag_rows_kernel<T, K, V, false>, "zoo_diag_rows_kernel", grid, smem, a, st);
  }
  if (stage == 1) {
    const size_t smem = sizeof(float) * (64 * (K + 4) + 64 * 65 + 64 + 2 * 16 * (K + 4) + 8 * 256) + (size_t)(64 * K * 2 + 16 * K + 48 * K);
    return launch_big_smem(zoo_diag_amat_kernel<T, K>, "zoo_diag_amat_kernel", grid, smem, a, st);
  }
  const size_t smem = sizeof(float) * (64 * ((K + 4) > (V + 8) ? (K + 4) : (V + 8)) + 64 * (K + 4) + 2 * 64 * 68 + 128 + 8 * 256);
  return launch_big_smem(zoo_kda_wy_kernel<T, K, V>, "zoo_kda_wy_kernel", grid, smem, a, st);
}

template <typename T>
static int run_diag_KV(const lq_zoo_problem* p, const DiagArgs& a, bool delta, int stage, cudaStream_t st) {
  if (p->K == 64 && p->V == 64) return run_diag_T<T, 64, 64>(p, a, delta, stage, st);
  if (p->K == 64 && p->V == 128) return run_diag_T<T, 64, 128>(p, a, delta, stage, st);
  if (p->K == 128 && p->V == 64) return run_diag_T<T, 128, 64>(p, a, delta, stage, st);
  if (p->K == 128 && p->V == 128) return run_diag_T<T, 128, 128>(p, a, delta, stage, st);
  return fail(LQ_ERR_UNSUPPORTED, "diagonal decay: K and V must be 64 or 128");
}

// stage 0 = rows, 1 = A matrix, 2 = KDA WY prep
int run_diag_stage(const lq_zoo_problem* p, const lq_zoo_workspace* ws, bool delta, int stage, cudaStream_t st) {
  DiagArgs a;
  fill_diag_args(p, ws, a);
  if (p->act_dtype == LQ_F16) return run_diag_KV<__half>(p, a, delta, stage, st);
  if (p->act_dtype == LQ_BF16) return run_diag_KV<__nv_bfloat16>(p, a, delta, stage, st);
  return fail(LQ_ERR_UNSUPPORTED, "diagonal decay: activation dtype must be f16 or bf16");
}

}  // namespace lq

extern "C" int lq_zoo_diag_rows(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream) {
  const bool delta = p && p->beta != nullptr;
  if (int e = lq::validate_zoo_problem(p, delta, true)) return e;
  if (!ws) return lq::fail(LQ_ERR_NULL, "diag rows: workspace descriptor is null");
  return lq::run_diag_stage(p, ws, delta, 0, (cudaStream_t)stream);
}
extern "C" int lq_zoo_diag_amat(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream) {
  const bool delta = p && p->beta != nullptr;
  if (int e = lq::validate_zoo_problem(p, delta, true)) return e;
  if (!ws) return lq::fail(LQ_ERR_NULL, "diag amat: workspace descriptor is null");
  return lq::run_diag_stage(p, ws, delta, 1, (cudaStream_t)stream);
}
extern "C" int lq_zoo_kda_wy(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream) {
  if (int e = lq::validate_zoo_problem(p, true, true)) return e;
  if (!ws) return lq::fail(LQ_ERR_NULL, "kda wy: workspace descriptor is null");
  return lq::run_diag_stage(p, ws, true, 2, (cudaStream_t)stream);
}
