// Inter-chunk state pass of the linear family (none / scalar decay) on INT8 tiles.
//
// Every (k, v) element of the state is an independent scalar recurrence over the chunks,
//     carry <- carry * exp(gc_last) + dequant( sum_t kw[t,k] * vw[t,v] ),
// so the grid tiles the state: one CTA owns a 32(v) x 64(k) tile of one (batch, head) and walks the chunks,
// four warps each holding a 16 x 32 sub-tile of the fp32 carry in registers. Per chunk it stores the INT8 copy
// of the carry *entering* the chunk (what the output kernel and the next chunk read), runs the INT8 write
// product on the tensor cores straight from the prologue's transposed code tiles (both operands have the token
// index contiguous, fragments are fetched with one 128-bit load per row), and folds it into the carry.
// The operand tiles of the next chunk are fetched while the current one is being multiplied.
//
// Reference arithmetic: zoo/simple_gla.py:46-72 (_state_body), reference.py:77-103 (fp32 carry, INT8 stored
// copy, no error feedback).  Stored-state layout: hT [BH, NT, V, K] (k contiguous) = B operand of q.S.
#include "lq_common.cuh"

namespace lq {

struct StateArgs {
  const int8_t *kwT, *vwT;
  const float *gc, *skw, *svw, *ss;
  const float* gcl;  // diagonal decay: [BH,NT,K] cumulative log-decay at the chunk end, per key channel
  int8_t* hT;
  float* final_state;  // [B,H,K,V] or null
  const float* initial_state;  // [B,H,K,V] or null
  int H, NT, use_g;
};

template <int K, int V, bool DIAG>
__global__ void __launch_bounds__(128) zoo_state_linear_kernel(StateArgs a) {
  constexpr int C = 64;
  constexpr int TK = K / 64;
  const int vt = blockIdx.x / TK, kt = blockIdx.x % TK;
  const int bh = blockIdx.y, h = bh % a.H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, j = lane & 3;
  const int v0 = vt * 32 + (warp & 1) * 16;
  const int k0 = kt * 64 + (warp >> 1) * 32;
  const int va = v0 + g, vb = v0 + g + 8;

  // MMA column (nt, cn) carries the physical key channel k0 + 8*(cn/2) + 2*nt + (cn%2): a thread then owns
  // eight consecutive channels k0 + 8j .. k0 + 8j + 7 of its two value rows.
  int krow[4];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) krow[nt] = k0 + 8 * (g >> 1) + 2 * nt + (g & 1);

  const float svw_a = a.svw[h * V + va], svw_b = a.svw[h * V + vb];
  const float iss_a = 1.0f / a.ss[h * V + va], iss_b = 1.0f / a.ss[h * V + vb];
  float skw[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) skw[i] = a.skw[h * K + k0 + 8 * j + i];

  const int8_t* vw = a.vwT + (size_t)bh * a.NT * V * C;
  const int8_t* kw = a.kwT + (size_t)bh * a.NT * K * C;
  int8_t* hT = a.hT + (size_t)bh * a.NT * V * K;
  const float* gc = a.gc + (size_t)bh * a.NT * C;

  float carry_a[8], carry_b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) carry_a[i] = carry_b[i] = 0.f;
  if (a.initial_state != nullptr) {
    const float* is = a.initial_state + (size_t)bh * K * V;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      carry_a[i] = is[(size_t)(k0 + 8 * j + i) * V + va];
      carry_b[i] = is[(size_t)(k0 + 8 * j + i) * V + vb];
    }
  }

  uint4 A_lo, A_hi, Bq[4];
  float glast = 0.f;
  float4 gk0 = make_float4(0.f, 0.f, 0.f, 0.f), gk1 = gk0;
  const float* gcl = DIAG ? a.gcl + (size_t)bh * a.NT * K + k0 + 8 * j : nullptr;
  auto fetch = [&](int c, uint4& alo, uint4& ahi, uint4 (&bq)[4], float& gl, float4& g0, float4& g1) {
    const int8_t* vwc = vw + (size_t)c * V * C;
    const int8_t* kwc = kw + (size_t)c * K * C;
    alo = __ldg(reinterpret_cast<const uint4*>(vwc + va * C + 16 * j));
    ahi = __ldg(reinterpret_cast<const uint4*>(vwc + vb * C + 16 * j));
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) bq[nt] = __ldg(reinterpret_cast<const uint4*>(kwc + krow[nt] * C + 16 * j));
    gl = (a.use_g && !DIAG) ? __ldg(gc + (size_t)c * C + (C - 1)) : 0.f;
    if (DIAG) {
      g0 = __ldg(reinterpret_cast<const float4*>(gcl + (size_t)c * K));
      g1 = __ldg(reinterpret_cast<const float4*>(gcl + (size_t)c * K) + 1);
    }
  };
  fetch(0, A_lo, A_hi, Bq, glast, gk0, gk1);

  for (int c = 0; c < a.NT; ++c) {
    uint4 nA_lo = A_lo, nA_hi = A_hi, nB[4] = {Bq[0], Bq[1], Bq[2], Bq[3]};
    float ngl = 0.f;
    float4 ng0 = gk0, ng1 = gk1;
    if (c + 1 < a.NT) fetch(c + 1, nA_lo, nA_hi, nB, ngl, ng0, ng1);

    // INT8 copy of the carry entering chunk c
    {
      int8_t* hc = hT + (size_t)c * V * K;
      *reinterpret_cast<uint2*>(hc + state_row_of_channel(va) * K + k0 + 8 * j) =
          make_uint2(q8x4_127(carry_a[0], carry_a[1], carry_a[2], carry_a[3], iss_a), q8x4_127(carry_a[4], carry_a[5], carry_a[6], carry_a[7], iss_a));
      *reinterpret_cast<uint2*>(hc + state_row_of_channel(vb) * K + k0 + 8 * j) =
          make_uint2(q8x4_127(carry_b[0], carry_b[1], carry_b[2], carry_b[3], iss_b), q8x4_127(carry_b[4], carry_b[5], carry_b[6], carry_b[7], iss_b));
    }

    int acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      mma_s8_first(acc[nt], A_lo.x, A_hi.x, A_lo.y, A_hi.y, Bq[nt].x, Bq[nt].y);
      mma_s8(acc[nt], A_lo.z, A_hi.z, A_lo.w, A_hi.w, Bq[nt].z, Bq[nt].w);
    }
    float gamv[8];
    if (DIAG) {
      const float gl8[8] = {gk0.x, gk0.y, gk0.z, gk0.w, gk1.x, gk1.y, gk1.z, gk1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) gamv[i] = expf(gl8[i]);
    } else {
      const float gs = a.use_g ? expf(glast) : 1.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) gamv[i] = gs;
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int i = 2 * nt + e;
        const float gam = gamv[i];
        const float ta = __fmul_rn(__fmul_rn((float)acc[nt][e], skw[i]), svw_a);
        const float tb = __fmul_rn(__fmul_rn((float)acc[nt][2 + e], skw[i]), svw_b);
        carry_a[i] = fmaf(carry_a[i], gam, ta);
        carry_b[i] = fmaf(carry_b[i], gam, tb);
      }
    }
    A_lo = nA_lo; A_hi = nA_hi; glast = ngl; gk0 = ng0; gk1 = ng1;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) Bq[nt] = nB[nt];
  }

  if (a.final_state != nullptr) {
    float* fs = a.final_state + (size_t)bh * K * V;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      fs[(size_t)(k0 + 8 * j + i) * V + va] = carry_a[i];
      fs[(size_t)(k0 + 8 * j + i) * V + vb] = carry_b[i];
    }
  }
}

int validate_zoo_problem(const lq_zoo_problem* p, bool delta, bool diagonal);

int run_state_linear_unrot(const lq_zoo_problem* p, const lq_zoo_workspace* ws, cudaStream_t st);

int run_state_linear(const lq_zoo_problem* p, const lq_zoo_workspace* ws, cudaStream_t st) {
  if (p->unrot_t != nullptr) return run_state_linear_unrot(p, ws, st);  // canonical storage: CTA spans all value channels
  StateArgs a;
  a.kwT = ws->kwT; a.vwT = ws->vwT; a.gc = ws->gc; a.skw = p->skw; a.svw = p->svw; a.ss = p->sstate;
  a.hT = ws->hT; a.final_state = p->final_state; a.initial_state = p->initial_state; a.H = p->H; a.NT = p->T / p->chunk;
  a.use_g = p->g != nullptr;
  a.gcl = ws->gcl;
  const bool diag = p->decay == LQ_DECAY_DIAGONAL;
  dim3 grid((p->V / 32) * (p->K / 64), p->B * p->H), block(128);
#define LQ_LAUNCH_STATE(KK_, VV_)                                                          \
  if (diag) zoo_state_linear_kernel<KK_, VV_, true><<<grid, block, 0, st>>>(a);            \
  else zoo_state_linear_kernel<KK_, VV_, false><<<grid, block, 0, st>>>(a)
  if (p->K == 64 && p->V == 64) { LQ_LAUNCH_STATE(64, 64); }
  else if (p->K == 64 && p->V == 128) { LQ_LAUNCH_STATE(64, 128); }
  else if (p->K == 128 && p->V == 64) { LQ_LAUNCH_STATE(128, 64); }
  else if (p->K == 128 && p->V == 128) { LQ_LAUNCH_STATE(128, 128); }
  else return fail(LQ_ERR_UNSUPPORTED, "state: K and V must be 64 or 128");
#undef LQ_LAUNCH_STATE
  return check_launch("zoo_state_linear_kernel");
}

}  // namespace lq

extern "C" int lq_zoo_state_linear(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream) {
  if (int e = lq::validate_zoo_problem(p, false, p && p->decay == LQ_DECAY_DIAGONAL)) return e;
  if (!ws) return lq::fail(LQ_ERR_NULL, "state: workspace descriptor is null");
  return lq::run_state_linear(p, ws, (cudaStream_t)stream);
}
