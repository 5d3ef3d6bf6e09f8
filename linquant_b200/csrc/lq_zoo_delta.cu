// Delta-rule family (DeltaNet / Gated DeltaNet, none or scalar decay): WY prologue and the chunk-serial state pass.
//
// Prologue (one CTA per (batch*head, chunk), parallel over chunks):
//   q, k rows as in the linear prologue (rescale, Walsh-Hadamard rotation, rounding, codes); the readout/write
//   key is Hw = round(beta^((1-sigma)tau) * k). Then the WY representation of the chunk in fp32-grade arithmetic:
//     G = tril( (beta^sigma k)(beta^(1-sigma) k)^T * exp(gc_i - gc_j), -1 )      TF32 MMA on exact operands
//     T = (I + G)^-1                                                             forward substitution in smem
//     W = T diag(beta^sigma exp(gc)) k ,  U = T diag(beta^sigma) v              3xTF32 split MMA (A split in three)
//   W is rounded to the activation dtype and quantised per head (w_read codes); U is stored in the activation dtype.
//   Operands k, v are fp16/bf16 values, exactly representable in TF32, and the fp32 left factor is split into three
//   TF32 pieces, so every product is exact and only the fp32 accumulation rounds.
//
// State pass (one CTA per (batch*head, 32 value channels), serial over chunks, fp32 carry [v,k] in registers):
//   hq = q8(carry)  -> stored state (global + shared);  ws = wq . hq (INT8 MMA);  E = (U - deq(ws)) * fw
//   e_local codes from the activation-rounded E, e_write codes from E * Omega^eta;  carry <- gamma carry + deq(ew^T kw)
//
// Reference arithmetic: zoo/gated_delta_rule.py:20-47 (_prep), :51-115 (_delta_state_body);
// reference.py:202-229 (_chunk_delta).
#include <type_traits>

#include "lq_wy.cuh"
#include "lq_zoo_rows.cuh"

namespace lq {

struct DeltaPrepArgs {
  PrologueArgs pro;
  const float *beta, *sw;
  int8_t* wq;
  void* u;
  float* fw;
  float sigma, tau;
};

template <typename T, int K, int V>
__global__ void __launch_bounds__(256) zoo_prologue_delta_kernel(DeltaPrepArgs d) {
  constexpr int C = kChunk, LDK = K + 8, LDV = V + 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  float* s_gc = reinterpret_cast<float*>(smem_raw);
  float* s_fk = s_gc + C;
  float* s_bs = s_fk + C;
  float* s_b1 = s_bs + C;
  float* s_hw = s_b1 + C;
  float* s_cwW = s_hw + C;  // beta^sigma * exp(gc)
  float* s_kf = s_cwW + C;
  float* s_vf = s_kf + C * LDK;
  float* s_G = s_vf + C * LDV;
  float* s_T = s_G + C * 68;
  uint32_t(*s_kw)[17] = reinterpret_cast<uint32_t(*)[17]>(s_T + C * 68);

  const PrologueArgs& a = d.pro;
  const int c = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;
  const size_t tile = (size_t)bh * a.NT + c;
  const float e_hw = (1.f - d.sigma) * d.tau;

  if (warp == 0) {
    if (a.g != nullptr) {
      chunk_decay_scan(a.g, b, c, h, a.T, a.H, s_gc);
    } else {
      s_gc[lane] = 0.f;
      s_gc[lane + 32] = 0.f;
    }
  }
  __syncthreads();
  if (tid < C) {
    const float dd = s_gc[C - 1] - s_gc[tid];
    s_fk[tid] = a.g ? expf((1.0f - a.eta) * dd) : 1.0f;
    a.gc[tile * C + tid] = s_gc[tid];
    const float bt = d.beta[((size_t)b * a.T + (size_t)c * C + tid) * a.H + h];
    const float bs = pow_exact01(bt, d.sigma);
    s_bs[tid] = bs;
    s_b1[tid] = pow_exact01(bt, 1.f - d.sigma);
    s_hw[tid] = pow_exact01(bt, e_hw);
    s_cwW[tid] = a.g ? bs * expf(s_gc[tid]) : bs;
    d.fw[tile * C + tid] = pow_exact01(bt, (1.f - d.sigma) * (1.f - d.tau));
  }
  __syncthreads();

  // the v rows are requested before the q / k rows are processed, and staged afterwards
  const T* vp = reinterpret_cast<const T*>(a.v);
  constexpr int NV = C * (V / 8) / 256;
  uint4 rv[NV];
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    const int i = tid + 256 * u, t = i / (V / 8), seg = i % (V / 8);
    rv[u] = __ldg(reinterpret_cast<const uint4*>(vp + (((size_t)b * a.T + (size_t)c * C + t) * a.H + h) * V + 8 * seg));
  }
  prologue_qk_rows<T, K>(a, b, c, h, tile, s_fk, e_hw != 0.f ? s_hw : nullptr, s_kf, LDK, s_kw);
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    const int i = tid + 256 * u, t = i / (V / 8), seg = i % (V / 8);
    float x[8];
    Act<T>::unpack8(rv[u], x);
    *reinterpret_cast<float4*>(s_vf + t * LDV + 8 * seg) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(s_vf + t * LDV + 8 * seg + 4) = make_float4(x[4], x[5], x[6], x[7]);
  }
  __syncthreads();

  // Work split of the three triangular products. Row tile mt (16 tokens) of G, W and U contracts over 2 mt + 2 steps
  // of eight tokens, so the cost grows 1 : 2 : 3 : 4 with mt: every warp takes the row tiles pr and 3 - pr (five steps on
  // average instead of up to eight) and one quarter of the columns.
  const int pr = warp & 1, qd = warp >> 1;
  // ---- Gram matrix (strictly lower triangle): 8-column tiles nt <= 2 mt + 1 of row tile mt, ten per pair of row tiles,
  // dealt round-robin to the pair's four warps. Tiles above the diagonal blocks are never read and stay unwritten.
  for (int u = qd; u < 10; u += 4) {
    const int lo = 2 * pr + 2;  // tiles of the lighter row tile of the pair
    const int mt = u < lo ? pr : 3 - pr, nt = u < lo ? u : u - lo;
    const int ia = 16 * mt + g, ib = ia + 8;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int kk = 0; kk < K / 8; ++kk) {
      const int c0 = 8 * kk + j;
      mma_tf32(acc, __float_as_uint(s_kf[ia * LDK + c0]), __float_as_uint(s_kf[ib * LDK + c0]),
               __float_as_uint(s_kf[ia * LDK + c0 + 4]), __float_as_uint(s_kf[ib * LDK + c0 + 4]),
               __float_as_uint(s_kf[(8 * nt + g) * LDK + c0]), __float_as_uint(s_kf[(8 * nt + g) * LDK + c0 + 4]));
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int jj = 8 * nt + 2 * j + e;
      s_G[ia * 68 + jj] = (ia > jj) ? s_bs[ia] * s_b1[jj] * acc[e] * expf(s_gc[ia] - s_gc[jj]) : 0.f;
      s_G[ib * 68 + jj] = (ib > jj) ? s_bs[ib] * s_b1[jj] * acc[2 + e] * expf(s_gc[ib] - s_gc[jj]) : 0.f;
    }
  }
  __syncthreads();
  wy_solve(s_G, s_T);
  __syncthreads();
  const float inv_sw = 1.0f / d.sw[h];
  T* up = reinterpret_cast<T*>(d.u);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int mt = half == 0 ? pr : 3 - pr;
    const int ia = 16 * mt + g, ib = ia + 8;
    // ---- W = T diag(beta^sigma exp(gc)) k  -> w_read codes
    {
      constexpr int NTW = K / 32;
      float acc[NTW][4];
#pragma unroll
      for (int nt = 0; nt < NTW; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
      const int n0 = qd * (K / 4);
      wy_product<NTW>(acc, s_T, s_cwW, s_kf, LDK, mt, n0, g, j);
#pragma unroll
      for (int nt = 0; nt < NTW; ++nt) {
        const int col = n0 + 8 * nt + 2 * j;
        const int a0 = q8(Act<T>::round(acc[nt][0]), inv_sw, a.qmax), a1 = q8(Act<T>::round(acc[nt][1]), inv_sw, a.qmax);
        const int b0 = q8(Act<T>::round(acc[nt][2]), inv_sw, a.qmax), b1 = q8(Act<T>::round(acc[nt][3]), inv_sw, a.qmax);
        *reinterpret_cast<uint16_t*>(d.wq + (tile * C + ia) * K + col) = (uint16_t)((a0 & 0xff) | ((a1 & 0xff) << 8));
        *reinterpret_cast<uint16_t*>(d.wq + (tile * C + ib) * K + col) = (uint16_t)((b0 & 0xff) | ((b1 & 0xff) << 8));
      }
    }
    // ---- U = T diag(beta^sigma) v  -> activation dtype
    {
      constexpr int NTU = V / 32;
      float acc[NTU][4];
#pragma unroll
      for (int nt = 0; nt < NTU; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
      const int n0 = qd * (V / 4);
      wy_product<NTU>(acc, s_T, s_bs, s_vf, LDV, mt, n0, g, j);
#pragma unroll
      for (int nt = 0; nt < NTU; ++nt) {
        const int col = n0 + 8 * nt + 2 * j;
        *reinterpret_cast<uint32_t*>(up + (tile * C + ia) * V + col) = Act<T>::pack2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<uint32_t*>(up + (tile * C + ib) * V + col) = Act<T>::pack2(acc[nt][2], acc[nt][3]);
      }
    }
  }
  uint32_t* kw_out = reinterpret_cast<uint32_t*>(a.kwT + tile * (size_t)(K * C));
  for (int i = tid; i < K * 16; i += 256) kw_out[i] = s_kw[i >> 4][i & 15];
}

// ------------------------------------------------------------------------------------------------ state pass
struct DeltaStateArgs {
  const int8_t *wq, *kwT;
  const void* u;
  const float *fw, *gc, *skw, *sw, *sel, *sew, *ss;
  const float *gcl, *genv;  // diagonal decay: [BH,NT,K] end-of-chunk log-decay, [BH,NT,C] log envelope
  int8_t *hT, *elT;
  float* final_state;
  const float* initial_state;  // [B,H,K,V] fp32 carry entering the first chunk, or null
  int H, NT, use_g;
  float eta, qmax;
};

template <int ROWB>
__device__ __forceinline__ int swz_row(int row, int chunk) {
  if (ROWB == 128) return row * 128 + ((chunk ^ ((row & 1) << 2)) << 4);
  return row * 64 + (chunk << 4);
}

template <typename T, int K, int V, bool DIAG>
__global__ void __launch_bounds__(128) zoo_state_delta_kernel(DeltaStateArgs a) {
  constexpr int C = 64, BV = 32;
  constexpr int NTK = K / 32;  // key n-tiles per warp in the carry layout
  constexpr int KK = K / 64;
  __shared__ __align__(128) uint8_t s_h[BV * K];
  __shared__ __align__(128) uint8_t s_ew[BV * C];
  __shared__ __align__(128) uint8_t s_el[BV * C];

  const int v0 = blockIdx.x * BV;
  const int bh = blockIdx.y, h = bh % a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;
  const int kw0 = warp * (K / 4);
  const int kown = kw0 + 2 * NTK * j;  // first of the 2*NTK consecutive key channels this thread owns

  // carry rows (value channels, local index) and their scales
  float sew_r[4], iss_r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int vl = 16 * (i >> 1) + g + 8 * (i & 1);
    sew_r[i] = a.sew[h * V + v0 + vl];
    iss_r[i] = 1.0f / a.ss[h * V + v0 + vl];
  }
  float skw[2 * NTK];
#pragma unroll
  for (int i = 0; i < 2 * NTK; ++i) skw[i] = a.skw[h * K + kown + i];
  // E columns: eight consecutive value channels v0 + 8j .. + 7
  float ss_c[8], isel_c[8], isew_c[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ss_c[i] = a.ss[h * V + v0 + 8 * j + i];
    isel_c[i] = 1.0f / a.sel[h * V + v0 + 8 * j + i];
    isew_c[i] = 1.0f / a.sew[h * V + v0 + 8 * j + i];
  }
  const float sw = a.sw[h];

  int krow[NTK];
#pragma unroll
  for (int nt = 0; nt < NTK; ++nt) krow[nt] = kw0 + 2 * NTK * (g >> 1) + 2 * nt + (g & 1);

  const size_t base_tile = (size_t)bh * a.NT;
  const int ta = 16 * warp + g, tb = ta + 8;
  const T* up = reinterpret_cast<const T*>(a.u);

  float carry[2][NTK][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < NTK; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const size_t kk_ = (size_t)bh * K + kown + 2 * nt + e;
        carry[mt][nt][e] = a.initial_state ? a.initial_state[kk_ * V + v0 + 16 * mt + g] : 0.f;
        carry[mt][nt][2 + e] = a.initial_state ? a.initial_state[kk_ * V + v0 + 16 * mt + g + 8] : 0.f;
      }
    }

  uint4 wa[KK], wb[KK], ua, ub, kb[NTK];
  float fwa, fwb, gca, gcb, glast;
  auto fetch = [&](int c, uint4 (&wa_)[KK], uint4 (&wb_)[KK], uint4& ua_, uint4& ub_, uint4 (&kb_)[NTK], float& fwa_,
                   float& fwb_, float& gca_, float& gcb_, float& gl_) {
    const size_t tile = base_tile + c;
    const int8_t* wqc = a.wq + tile * (size_t)(C * K);
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
      wa_[kk] = __ldg(reinterpret_cast<const uint4*>(wqc + ta * K + 64 * kk + 16 * j));
      wb_[kk] = __ldg(reinterpret_cast<const uint4*>(wqc + tb * K + 64 * kk + 16 * j));
    }
    ua_ = __ldg(reinterpret_cast<const uint4*>(up + (tile * C + ta) * V + v0 + 8 * j));
    ub_ = __ldg(reinterpret_cast<const uint4*>(up + (tile * C + tb) * V + v0 + 8 * j));
    const int8_t* kwc = a.kwT + tile * (size_t)(K * C);
#pragma unroll
    for (int nt = 0; nt < NTK; ++nt) kb_[nt] = __ldg(reinterpret_cast<const uint4*>(kwc + krow[nt] * C + 16 * j));
    fwa_ = __ldg(a.fw + tile * C + ta);
    fwb_ = __ldg(a.fw + tile * C + tb);
    if (DIAG) {  // gca/gcb carry the log envelope of the two token rows; the carry decay is per key channel
      gca_ = __ldg(a.genv + tile * C + ta);
      gcb_ = __ldg(a.genv + tile * C + tb);
      gl_ = 0.f;
    } else {
      gca_ = a.use_g ? __ldg(a.gc + tile * C + ta) : 0.f;
      gcb_ = a.use_g ? __ldg(a.gc + tile * C + tb) : 0.f;
      gl_ = a.use_g ? __ldg(a.gc + tile * C + C - 1) : 0.f;
    }
  };
  fetch(0, wa, wb, ua, ub, kb, fwa, fwb, gca, gcb, glast);

  for (int c = 0; c < a.NT; ++c) {
    const size_t tile = base_tile + c;
    uint4 nwa[KK], nwb[KK], nua = ua, nub = ub, nkb[NTK];
    float nfwa = 0.f, nfwb = 0.f, ngca = 0.f, ngcb = 0.f, ngl = 0.f;
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) { nwa[kk] = wa[kk]; nwb[kk] = wb[kk]; }
#pragma unroll
    for (int nt = 0; nt < NTK; ++nt) nkb[nt] = kb[nt];
    if (c + 1 < a.NT) fetch(c + 1, nwa, nwb, nua, nub, nkb, nfwa, nfwb, ngca, ngcb, ngl);

    // ---- 1. INT8 copy of the carry entering the chunk: global stored state + shared B operand
    {
      int8_t* hc = a.hT + tile * (size_t)(V * K);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int mt = i >> 1, hi = i & 1;
        const int vl = 16 * mt + g + 8 * hi;
        int cd[2 * NTK];
#pragma unroll
        for (int nt = 0; nt < NTK; ++nt) {
          cd[2 * nt] = q8_lower127(carry[mt][nt][2 * hi], iss_r[i]);  // upper clamp: the saturating pack below
          cd[2 * nt + 1] = q8_lower127(carry[mt][nt][2 * hi + 1], iss_r[i]);
        }
        uint8_t* sdst = s_h + swz_row<K>(vl, kown >> 4) + (kown & 15);
        int8_t* gdst = hc + (size_t)state_row_of_channel(v0 + vl) * K + kown;
        if (NTK == 4) {
          const uint2 w = make_uint2(pack_sat_s8x2(cd[1], cd[0], pack_sat_s8x2(cd[3], cd[2], 0u)),
                                     pack_sat_s8x2(cd[5 % (2 * NTK)], cd[4 % (2 * NTK)],
                                                   pack_sat_s8x2(cd[7 % (2 * NTK)], cd[6 % (2 * NTK)], 0u)));
          *reinterpret_cast<uint2*>(sdst) = w;
          *reinterpret_cast<uint2*>(gdst) = w;
        } else {
          const uint32_t w = pack_sat_s8x2(cd[1], cd[0], pack_sat_s8x2(cd[3], cd[2], 0u));
          *reinterpret_cast<uint32_t*>(sdst) = w;
          *reinterpret_cast<uint32_t*>(gdst) = w;
        }
      }
    }
    __syncthreads();

    // ---- 2. ws = wq . hq ; E ; e_local / e_write codes
    {
      int acc[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0;
        const int vr = 8 * (g >> 1) + 2 * nt + (g & 1);
#pragma unroll
        for (int kk = 0; kk < KK; ++kk) {
          const uint4 bs = *reinterpret_cast<const uint4*>(s_h + swz_row<K>(vr, 4 * kk + j));
          mma_s8(acc[nt], wa[kk].x, wb[kk].x, wa[kk].y, wb[kk].y, bs.x, bs.y);
          mma_s8(acc[nt], wa[kk].z, wb[kk].z, wa[kk].w, wb[kk].w, bs.z, bs.w);
        }
      }
      float Ua[8], Ub[8];
      Act<T>::unpack8(ua, Ua);
      Act<T>::unpack8(ub, Ub);
      const float fva = DIAG ? expf(a.eta * gca) : (a.use_g ? expf(a.eta * (glast - gca)) : 1.f);
      const float fvb = DIAG ? expf(a.eta * gcb) : (a.use_g ? expf(a.eta * (glast - gcb)) : 1.f);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int i = 2 * nt + e;
          const int vl = 8 * j + i;
          const float wsa = __fmul_rn(__fmul_rn((float)acc[nt][e], sw), ss_c[i]);
          const float wsb = __fmul_rn(__fmul_rn((float)acc[nt][2 + e], sw), ss_c[i]);
          const float Ea = __fmul_rn(__fsub_rn(Ua[i], wsa), fwa);
          const float Eb = __fmul_rn(__fsub_rn(Ub[i], wsb), fwb);
          s_el[vl * C + ta] = (uint8_t)q8(Act<T>::round(Ea), isel_c[i], a.qmax);
          s_el[vl * C + tb] = (uint8_t)q8(Act<T>::round(Eb), isel_c[i], a.qmax);
          s_ew[vl * C + ta] = (uint8_t)q8(__fmul_rn(Ea, fva), isew_c[i], a.qmax);
          s_ew[vl * C + tb] = (uint8_t)q8(__fmul_rn(Eb, fvb), isew_c[i], a.qmax);
        }
      }
    }
    __syncthreads();

    // ---- 3. write product and carry update; e_local tile out
    {
      reinterpret_cast<uint4*>(a.elT + tile * (size_t)(V * C) + (size_t)v0 * C)[tid] = reinterpret_cast<const uint4*>(s_el)[tid];
      float gamv[2 * NTK];
      if (DIAG) {
#pragma unroll
        for (int i = 0; i < 2 * NTK; ++i) gamv[i] = expf(__ldg(a.gcl + tile * K + kown + i));
      } else {
        const float gs = a.use_g ? expf(glast) : 1.0f;
#pragma unroll
        for (int i = 0; i < 2 * NTK; ++i) gamv[i] = gs;
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const uint4 ea = *reinterpret_cast<const uint4*>(s_ew + (16 * mt + g) * C + 16 * j);
        const uint4 eb = *reinterpret_cast<const uint4*>(s_ew + (16 * mt + g + 8) * C + 16 * j);
#pragma unroll
        for (int nt = 0; nt < NTK; ++nt) {
          int acc[4] = {0, 0, 0, 0};
          mma_s8(acc, ea.x, eb.x, ea.y, eb.y, kb[nt].x, kb[nt].y);
          mma_s8(acc, ea.z, eb.z, ea.w, eb.w, kb[nt].z, kb[nt].w);
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float ta_ = __fmul_rn(__fmul_rn((float)acc[e], skw[2 * nt + e]), sew_r[2 * mt]);
            const float tb_ = __fmul_rn(__fmul_rn((float)acc[2 + e], skw[2 * nt + e]), sew_r[2 * mt + 1]);
            carry[mt][nt][e] = fmaf(carry[mt][nt][e], gamv[2 * nt + e], ta_);
            carry[mt][nt][2 + e] = fmaf(carry[mt][nt][2 + e], gamv[2 * nt + e], tb_);
          }
        }
      }
    }
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) { wa[kk] = nwa[kk]; wb[kk] = nwb[kk]; }
#pragma unroll
    for (int nt = 0; nt < NTK; ++nt) kb[nt] = nkb[nt];
    ua = nua; ub = nub; fwa = nfwa; fwb = nfwb; gca = ngca; gcb = ngcb; glast = ngl;
  }

  if (a.final_state != nullptr) {
    float* fs = a.final_state + (size_t)bh * K * V;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < NTK; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kk_ = kown + 2 * nt + e;
          fs[(size_t)kk_ * V + v0 + 16 * mt + g] = carry[mt][nt][e];
          fs[(size_t)kk_ * V + v0 + 16 * mt + g + 8] = carry[mt][nt][2 + e];
        }
  }
}

// ------------------------------------------------------------------------------------------------ state pass, canonical storage
// Delta-rule state pass when v arrives rotated by R_V and the state is stored canonical (zoo/gated_delta_rule.py,
// zoo/kda.py with unrot=; reference.py:218-227). Per chunk:
//   ws   = fp16(dequant(W_q . S_q)) . R_V            the canonical state read, taken into the rotated value basis
//   E    = (U - ws) * fw,   e_local / e_write codes   (E stays rotated)
//   carry <- gamma carry + fp16(dequant(kw_q^T . ew_q)) . R_V^T     the write product, un-rotated
// Both basis changes mix all value channels and the read contracts over all key channels, so one CTA owns the whole
// K x V state of a (batch, head): eight warps, warp w keeping key rows 16w .. 16w+15 x all value channels of the fp32
// carry in the accumulator layout of the un-rotation MMA. The fp16 products go through shared memory; R_V and R_V^T
// both sit in shared memory with the contraction index contiguous. This path trades parallelism (B*H CTAs) for
// exactness of the reference's rounding points.
template <typename T, int K, int V, bool DIAG>
__global__ void __launch_bounds__(256) zoo_state_delta_unrot_kernel(DeltaStateArgs a, const __half* unrot_t) {
  constexpr int C = 64, LDH = V + 8, KK = K / 64, KW = K / 16;
  constexpr int NT2 = V / 16;                 // value n-tiles per warp in the read phase (two value halves)
  constexpr int MTV = V / 16, NHALF = 8 / MTV, NTW = (K / 8) / NHALF;  // write product: value m-tile, key n-tiles per warp
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t* s_h = smem_raw;                                   // [V][K]   INT8 state, B operand of the read
  uint8_t* s_ew = s_h + V * K;                               // [V][C]   e_write codes (token index contiguous)
  uint8_t* s_el = s_ew + V * C;                              // [V][C]   e_local codes
  uint8_t* s_kw = s_el + V * C;                              // [K][C]   k_write codes of the chunk
  __half* s_r = reinterpret_cast<__half*>(s_kw + K * C);     // [V][LDH] unrot   : B operand of the read rotation (rows v', v contiguous)
  __half* s_rt = s_r + V * LDH;                              // [V][LDH] unrot^T : B operand of the write un-rotation
  __half* s_x = s_rt + V * LDH;                              // [K][LDH] fp16 products: ws [64][LDH], then the write product [K][LDH]
  float* s_ss = reinterpret_cast<float*>(s_x + K * LDH);     // [V] state scale, then 1/state, 1/sel, 1/sew, sew
  float* s_iss = s_ss + V;
  float* s_isel = s_iss + V;
  float* s_isew = s_isel + V;
  float* s_sew = s_isew + V;
  float* s_skw = s_sew + V;                                  // [K]

  const int bh = blockIdx.x, h = bh % a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;
  const int tw = warp & 3, vh = warp >> 2;
  const int ta = 16 * tw + g, tb = ta + 8;
  const int ka = 16 * warp + g, kb_ = ka + 8;   // carry rows (warps below KW)
  const bool owner = warp < KW;

  for (int i = tid; i < V * (V / 8); i += 256) {
    const int row = i / (V / 8), ch = i % (V / 8);
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(unrot_t + (size_t)row * V) + ch);
    *reinterpret_cast<uint4*>(s_rt + row * LDH + 8 * ch) = w;
    const __half* hv = reinterpret_cast<const __half*>(&w);
#pragma unroll
    for (int e = 0; e < 8; ++e) s_r[(8 * ch + e) * LDH + row] = hv[e];  // transposed copy
  }
  for (int i = tid; i < V; i += 256) {
    s_ss[i] = a.ss[h * V + i];
    s_iss[i] = 1.0f / a.ss[h * V + i];
    s_isel[i] = 1.0f / a.sel[h * V + i];
    s_isew[i] = 1.0f / a.sew[h * V + i];
    s_sew[i] = a.sew[h * V + i];
  }
  for (int i = tid; i < K; i += 256) s_skw[i] = a.skw[h * K + i];
  const float sw = a.sw[h];
  const size_t base_tile = (size_t)bh * a.NT;
  const T* up = reinterpret_cast<const T*>(a.u);

  float carry[V / 8][4];
#pragma unroll
  for (int nt = 0; nt < V / 8; ++nt) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int kr = (i >> 1) ? kb_ : ka;
      carry[nt][i] = (a.initial_state && owner) ? a.initial_state[((size_t)bh * K + kr) * V + 8 * nt + 2 * j + (i & 1)] : 0.f;
    }
  }

  auto stage_kw = [&](int c) {
    const int8_t* kwc = a.kwT + (base_tile + c) * (size_t)(K * C);
    for (int i = tid; i < K * C / 16; i += 256) cp_async16(s_kw + 16 * i, kwc + 16 * i);
    cp_async_commit();
  };
  stage_kw(0);
  __syncthreads();

  for (int c = 0; c < a.NT; ++c) {
    const size_t tile = base_tile + c;
    // operands of the read phase (token rows ta, tb)
    uint4 wa[KK], wb[KK];
    {
      const int8_t* wqc = a.wq + tile * (size_t)(C * K);
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
        wa[kk] = __ldg(reinterpret_cast<const uint4*>(wqc + ta * K + 64 * kk + 16 * j));
        wb[kk] = __ldg(reinterpret_cast<const uint4*>(wqc + tb * K + 64 * kk + 16 * j));
      }
    }
    const float fwa = __ldg(a.fw + tile * C + ta), fwb = __ldg(a.fw + tile * C + tb);
    float gca, gcb, glast = 0.f;
    if (DIAG) {
      gca = __ldg(a.genv + tile * C + ta);
      gcb = __ldg(a.genv + tile * C + tb);
    } else {
      gca = a.use_g ? __ldg(a.gc + tile * C + ta) : 0.f;
      gcb = a.use_g ? __ldg(a.gc + tile * C + tb) : 0.f;
      glast = a.use_g ? __ldg(a.gc + tile * C + C - 1) : 0.f;
    }

    // ---- 1. INT8 copy of the canonical carry entering the chunk
    if (owner) {
#pragma unroll
      for (int nt = 0; nt < V / 8; ++nt) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int vc = 8 * nt + 2 * j + (i & 1), kr = (i >> 1) ? kb_ : ka;
          s_h[swz_row<K>(vc, kr >> 4) + (kr & 15)] = (uint8_t)q8(carry[nt][i], s_iss[vc], 127.f);
        }
      }
    }
    __syncthreads();
    {
      int8_t* hc = a.hT + tile * (size_t)(V * K);
      for (int i = tid; i < V * (K / 16); i += 256) {
        const int vr = i / (K / 16), ch = i % (K / 16);
        *reinterpret_cast<uint4*>(hc + (size_t)state_row_of_channel(vr) * K + 16 * ch) =
            *reinterpret_cast<const uint4*>(s_h + swz_row<K>(vr, ch));
      }
    }

    // ---- 2. ws = wq . hq, dequantised, fp16, token-major
    {
#pragma unroll
      for (int n2 = 0; n2 < NT2; ++n2) {
        const int nt = NT2 * vh + n2;
        int acc[4] = {0, 0, 0, 0};
        const int vr = 8 * nt + g;
#pragma unroll
        for (int kk = 0; kk < KK; ++kk) {
          const uint4 bs = *reinterpret_cast<const uint4*>(s_h + swz_row<K>(vr, 4 * kk + j));
          mma_s8(acc, wa[kk].x, wb[kk].x, wa[kk].y, wb[kk].y, bs.x, bs.y);
          mma_s8(acc, wa[kk].z, wb[kk].z, wa[kk].w, wb[kk].w, bs.z, bs.w);
        }
        const int vc = 8 * nt + 2 * j;
        const float s0 = s_ss[vc], s1 = s_ss[vc + 1];
        *reinterpret_cast<uint32_t*>(s_x + ta * LDH + vc) =
            Act<__half>::pack2(__fmul_rn(__fmul_rn((float)acc[0], sw), s0), __fmul_rn(__fmul_rn((float)acc[1], sw), s1));
        *reinterpret_cast<uint32_t*>(s_x + tb * LDH + vc) =
            Act<__half>::pack2(__fmul_rn(__fmul_rn((float)acc[2], sw), s0), __fmul_rn(__fmul_rn((float)acc[3], sw), s1));
      }
    }
    __syncthreads();

    // ---- 3. read rotation, E, codes
    {
      const float fva = DIAG ? expf(a.eta * gca) : (a.use_g ? expf(a.eta * (glast - gca)) : 1.f);
      const float fvb = DIAG ? expf(a.eta * gcb) : (a.use_g ? expf(a.eta * (glast - gcb)) : 1.f);
#pragma unroll
      for (int n2 = 0; n2 < NT2; ++n2) {
        const int nt = NT2 * vh + n2;
        float u[4] = {0.f, 0.f, 0.f, 0.f};
        const __half* brow = s_r + (8 * nt + g) * LDH;
#pragma unroll
        for (int kk = 0; kk < V / 16; ++kk) {
          const uint32_t a0 = *reinterpret_cast<const uint32_t*>(s_x + ta * LDH + 16 * kk + 2 * j);
          const uint32_t a1 = *reinterpret_cast<const uint32_t*>(s_x + tb * LDH + 16 * kk + 2 * j);
          const uint32_t a2 = *reinterpret_cast<const uint32_t*>(s_x + ta * LDH + 16 * kk + 8 + 2 * j);
          const uint32_t a3 = *reinterpret_cast<const uint32_t*>(s_x + tb * LDH + 16 * kk + 8 + 2 * j);
          mma_f16(u, a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(brow + 16 * kk + 2 * j),
                  *reinterpret_cast<const uint32_t*>(brow + 16 * kk + 8 + 2 * j));
        }
        const int vc = 8 * nt + 2 * j;
        const uint32_t ura = __ldg(reinterpret_cast<const uint32_t*>(up + (tile * C + ta) * V + vc));
        const uint32_t urb = __ldg(reinterpret_cast<const uint32_t*>(up + (tile * C + tb) * V + vc));
        float Ua[2], Ub[2];
        if (std::is_same<T, __half>::value) {
          const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&ura)), fb = __half22float2(*reinterpret_cast<const __half2*>(&urb));
          Ua[0] = fa.x; Ua[1] = fa.y; Ub[0] = fb.x; Ub[1] = fb.y;
        } else {
          Ua[0] = __uint_as_float(ura << 16); Ua[1] = __uint_as_float(ura & 0xffff0000u);
          Ub[0] = __uint_as_float(urb << 16); Ub[1] = __uint_as_float(urb & 0xffff0000u);
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int vl = vc + e;
          const float Ea = __fmul_rn(__fsub_rn(Ua[e], u[e]), fwa);
          const float Eb = __fmul_rn(__fsub_rn(Ub[e], u[2 + e]), fwb);
          s_el[vl * C + ta] = (uint8_t)q8(Act<T>::round(Ea), s_isel[vl], a.qmax);
          s_el[vl * C + tb] = (uint8_t)q8(Act<T>::round(Eb), s_isel[vl], a.qmax);
          s_ew[vl * C + ta] = (uint8_t)q8(__fmul_rn(Ea, fva), s_isew[vl], a.qmax);
          s_ew[vl * C + tb] = (uint8_t)q8(__fmul_rn(Eb, fvb), s_isew[vl], a.qmax);
        }
      }
    }
    cp_async_wait<0>();  // this chunk's k_write tile
    __syncthreads();

    // ---- 4. e_local tile out; write product in the rotated basis, dequantised, fp16, key-major
    {
      uint4* eout = reinterpret_cast<uint4*>(a.elT + tile * (size_t)(V * C));
      for (int i = tid; i < V * C / 16; i += 256) eout[i] = reinterpret_cast<const uint4*>(s_el)[i];
      const int mtv = warp % MTV, nhf = warp / MTV;
      const int va = 16 * mtv + g, vb = va + 8;
      const uint4 ea = *reinterpret_cast<const uint4*>(s_ew + va * C + 16 * j);
      const uint4 eb = *reinterpret_cast<const uint4*>(s_ew + vb * C + 16 * j);
      const float sewa = s_sew[va], sewb = s_sew[vb];
#pragma unroll
      for (int n2 = 0; n2 < NTW; ++n2) {
        const int nt = NTW * nhf + n2;
        const uint4 kq = *reinterpret_cast<const uint4*>(s_kw + (8 * nt + g) * C + 16 * j);
        int acc[4] = {0, 0, 0, 0};
        mma_s8(acc, ea.x, eb.x, ea.y, eb.y, kq.x, kq.y);
        mma_s8(acc, ea.z, eb.z, ea.w, eb.w, kq.z, kq.w);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kc = 8 * nt + 2 * j + e;
          const float sk = s_skw[kc];
          s_x[kc * LDH + va] = __float2half_rn(__fmul_rn(__fmul_rn((float)acc[e], sk), sewa));
          s_x[kc * LDH + vb] = __float2half_rn(__fmul_rn(__fmul_rn((float)acc[2 + e], sk), sewb));
        }
      }
    }
    __syncthreads();
    if (c + 1 < a.NT) stage_kw(c + 1);  // the k_write tile of the next chunk travels during the un-rotation

    // ---- 5. un-rotation of the write product, folded into the canonical carry
    if (owner) {
      float gam[2] = {1.f, 1.f};
      if (DIAG) {
        gam[0] = expf(__ldg(a.gcl + tile * K + ka));
        gam[1] = expf(__ldg(a.gcl + tile * K + kb_));
      } else if (a.use_g) {
        gam[0] = gam[1] = expf(glast);
      }
#pragma unroll
      for (int nt = 0; nt < V / 8; ++nt) {
        float u[4] = {0.f, 0.f, 0.f, 0.f};
        const __half* brow = s_rt + (8 * nt + g) * LDH;
#pragma unroll
        for (int kk = 0; kk < V / 16; ++kk) {
          const uint32_t a0 = *reinterpret_cast<const uint32_t*>(s_x + ka * LDH + 16 * kk + 2 * j);
          const uint32_t a1 = *reinterpret_cast<const uint32_t*>(s_x + kb_ * LDH + 16 * kk + 2 * j);
          const uint32_t a2 = *reinterpret_cast<const uint32_t*>(s_x + ka * LDH + 16 * kk + 8 + 2 * j);
          const uint32_t a3 = *reinterpret_cast<const uint32_t*>(s_x + kb_ * LDH + 16 * kk + 8 + 2 * j);
          mma_f16(u, a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(brow + 16 * kk + 2 * j),
                  *reinterpret_cast<const uint32_t*>(brow + 16 * kk + 8 + 2 * j));
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) carry[nt][i] = fmaf(carry[nt][i], gam[i >> 1], u[i]);
      }
    }
    __syncthreads();
  }

  if (a.final_state != nullptr && owner) {
    float* fs = a.final_state + (size_t)bh * K * V;
#pragma unroll
    for (int nt = 0; nt < V / 8; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) fs[(size_t)((i >> 1) ? kb_ : ka) * V + 8 * nt + 2 * j + (i & 1)] = carry[nt][i];
    }
  }
}

int validate_zoo_problem(const lq_zoo_problem* p, bool delta, bool diagonal);
void fill_prologue_args(const lq_zoo_problem* p, const lq_zoo_workspace* ws, PrologueArgs& a);

template <typename T, int K, int V>
static int launch_delta_prep(const DeltaPrepArgs& d, int BH, cudaStream_t st) {
  constexpr size_t smem = sizeof(float) * (6 * 64 + 64 * (K + 8) + 64 * (V + 8) + 2 * 64 * 68) + sizeof(uint32_t) * K * 17;
  cudaError_t e = cudaFuncSetAttribute(zoo_prologue_delta_kernel<T, K, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "delta prologue: cannot opt in to %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  zoo_prologue_delta_kernel<T, K, V><<<dim3(d.pro.NT, BH), 256, smem, st>>>(d);
  return check_launch("zoo_prologue_delta_kernel");
}

template <typename T>
static int dispatch_delta_prep(const lq_zoo_problem* p, const DeltaPrepArgs& d, cudaStream_t st) {
  const int BH = p->B * p->H;
  if (p->K == 64 && p->V == 64) return launch_delta_prep<T, 64, 64>(d, BH, st);
  if (p->K == 64 && p->V == 128) return launch_delta_prep<T, 64, 128>(d, BH, st);
  if (p->K == 128 && p->V == 64) return launch_delta_prep<T, 128, 64>(d, BH, st);
  if (p->K == 128 && p->V == 128) return launch_delta_prep<T, 128, 128>(d, BH, st);
  return fail(LQ_ERR_UNSUPPORTED, "delta prologue: K and V must be 64 or 128");
}

int run_prologue_delta(const lq_zoo_problem* p, const lq_zoo_workspace* ws, cudaStream_t st) {
  DeltaPrepArgs d;
  fill_prologue_args(p, ws, d.pro);
  d.beta = p->beta; d.sw = p->sw; d.wq = ws->wq; d.u = ws->u; d.fw = ws->fw; d.sigma = p->sigma; d.tau = p->tau;
  if (p->act_dtype == LQ_F16) return dispatch_delta_prep<__half>(p, d, st);
  if (p->act_dtype == LQ_BF16) return dispatch_delta_prep<__nv_bfloat16>(p, d, st);
  return fail(LQ_ERR_UNSUPPORTED, "delta prologue: activation dtype must be f16 or bf16");
}

template <typename T, int K, int V>
static int launch_delta_state_unrot(const lq_zoo_problem* p, const DeltaStateArgs& a, cudaStream_t st) {
  const size_t smem = (size_t)V * K + 2 * (size_t)V * 64 + (size_t)K * 64 + sizeof(__half) * (size_t)(2 * V + K) * (V + 8) +
                      sizeof(float) * (5 * V + K);
  const __half* rt = reinterpret_cast<const __half*>(p->unrot_t);
  cudaError_t e;
  if (p->decay == LQ_DECAY_DIAGONAL) {
    e = cudaFuncSetAttribute(zoo_state_delta_unrot_kernel<T, K, V, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) zoo_state_delta_unrot_kernel<T, K, V, true><<<p->B * p->H, 256, smem, st>>>(a, rt);
  } else {
    e = cudaFuncSetAttribute(zoo_state_delta_unrot_kernel<T, K, V, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) zoo_state_delta_unrot_kernel<T, K, V, false><<<p->B * p->H, 256, smem, st>>>(a, rt);
  }
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "delta state (canonical storage): shared memory opt-in failed: %s", cudaGetErrorString(e));
  return check_launch("zoo_state_delta_unrot_kernel");
}

template <typename T>
static int dispatch_delta_state(const lq_zoo_problem* p, const DeltaStateArgs& a, cudaStream_t st) {
  if (p->unrot_t != nullptr) {  // canonical storage: one CTA per (batch, head) owns the whole state
    if (p->K == 64 && p->V == 64) return launch_delta_state_unrot<T, 64, 64>(p, a, st);
    if (p->K == 64 && p->V == 128) return launch_delta_state_unrot<T, 64, 128>(p, a, st);
    if (p->K == 128 && p->V == 64) return launch_delta_state_unrot<T, 128, 64>(p, a, st);
    if (p->K == 128 && p->V == 128) return launch_delta_state_unrot<T, 128, 128>(p, a, st);
    return fail(LQ_ERR_UNSUPPORTED, "delta state: K and V must be 64 or 128");
  }
  dim3 grid(p->V / 32, p->B * p->H), block(128);
  const bool diag = p->decay == LQ_DECAY_DIAGONAL;
#define LQ_LAUNCH_DSTATE(KK_, VV_)                                                         \
  if (diag) zoo_state_delta_kernel<T, KK_, VV_, true><<<grid, block, 0, st>>>(a);          \
  else zoo_state_delta_kernel<T, KK_, VV_, false><<<grid, block, 0, st>>>(a)
  if (p->K == 64 && p->V == 64) { LQ_LAUNCH_DSTATE(64, 64); }
  else if (p->K == 64 && p->V == 128) { LQ_LAUNCH_DSTATE(64, 128); }
  else if (p->K == 128 && p->V == 64) { LQ_LAUNCH_DSTATE(128, 64); }
  else if (p->K == 128 && p->V == 128) { LQ_LAUNCH_DSTATE(128, 128); }
  else return fail(LQ_ERR_UNSUPPORTED, "delta state: K and V must be 64 or 128");
#undef LQ_LAUNCH_DSTATE
  return check_launch("zoo_state_delta_kernel");
}

int run_state_delta(const lq_zoo_problem* p, const lq_zoo_workspace* ws, cudaStream_t st) {
  DeltaStateArgs a;
  a.wq = ws->wq; a.kwT = ws->kwT; a.u = ws->u; a.fw = ws->fw; a.gc = ws->gc;
  a.skw = p->skw; a.sw = p->sw; a.sel = p->sel; a.sew = p->sew; a.ss = p->sstate;
  a.hT = ws->hT; a.elT = ws->vlT; a.final_state = p->final_state; a.initial_state = p->initial_state; a.gcl = ws->gcl; a.genv = ws->genv;
  a.H = p->H; a.NT = p->T / p->chunk; a.use_g = p->g != nullptr; a.eta = p->eta; a.qmax = p->qmax;
  if (p->act_dtype == LQ_F16) return dispatch_delta_state<__half>(p, a, st);
  if (p->act_dtype == LQ_BF16) return dispatch_delta_state<__nv_bfloat16>(p, a, st);
  return fail(LQ_ERR_UNSUPPORTED, "delta state: activation dtype must be f16 or bf16");
}

}  // namespace lq

extern "C" int lq_zoo_prologue_delta(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream) {
  if (int e = lq::validate_zoo_problem(p, true, false)) return e;
  if (!ws) return lq::fail(LQ_ERR_NULL, "delta prologue: workspace descriptor is null");
  return lq::run_prologue_delta(p, ws, (cudaStream_t)stream);
}

extern "C" int lq_zoo_state_delta(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream) {
  if (int e = lq::validate_zoo_problem(p, true, p && p->decay == LQ_DECAY_DIAGONAL)) return e;
  if (!ws) return lq::fail(LQ_ERR_NULL, "delta state: workspace descriptor is null");
  return lq::run_state_delta(p, ws, (cudaStream_t)stream);
}
