// Fused operand prologue of the zoo-lineage INT8 chunk prefill (none / scalar decay).
//
// One CTA per (batch*head, chunk of 64 tokens). In one pass over q, k, v (128-bit loads) it applies the optional
// diagonal rescale D_QK, the optional signed Walsh-Hadamard rotation R_QK (registers + warp shuffles), the
// rounding to the activation dtype, the q scale, and the per-role static INT8 code rule, and it emits
//   qq  [C,K]  q codes (read and local product share one tile)      kl  [C,K]  k_local codes
//   kwT [K,C]  k_write codes, gated by Omega^(1-eta), transposed   vlT [V,C]  v_local codes, transposed
//   vwT [V,C]  v_write codes, gated by Omega^eta, transposed        gc  [C]    chunk-local cumulative log-decay
// The transposed tiles put the token (reduction) index contiguous, which is what both MMA operands of the
// state pass and the B operand of the A.v product want.
//
// Reference arithmetic: zoo/simple_gla.py:16-20 (_q8), :57-67 (write gating and codes), :129-130,:149 (read /
// local codes), :191 (chunk-local cumsum of the fp32 log-decay; the scan here accumulates in double and rounds each
// prefix to fp32), reference.py:41-47 (rotate -> round to activation dtype -> scale).
#include "lq_zoo_rows.cuh"

namespace lq {

template <typename T, int K, int V>
__global__ void __launch_bounds__(256) zoo_prologue_linear_kernel(PrologueArgs a) {
  constexpr int C = kChunk;
  __shared__ float s_gc[C], s_fk[C], s_fv[C];
  __shared__ uint32_t s_kw[K][17];
  __shared__ uint32_t s_vl[V][17];
  __shared__ uint32_t s_vw[V][17];

  const int c = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const size_t tile = (size_t)bh * a.NT + c;

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
    const float d = s_gc[C - 1] - s_gc[tid];
    s_fk[tid] = a.g ? expf((1.0f - a.eta) * d) : 1.0f;
    s_fv[tid] = a.g ? expf(a.eta * d) : 1.0f;
    a.gc[tile * C + tid] = s_gc[tid];
  }
  __syncthreads();

  prologue_qk_rows<T, K>(a, b, c, h, tile, s_fk, nullptr, nullptr, 0, s_kw);
  // ------------------------------------------------------------------ v rows (V channels)
  if (!a.skip_v) {
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
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = 4 * tg + i;
        const size_t row = (((size_t)b * a.T + (size_t)c * C + t) * a.H + h) * V + 8 * r;
        float x[8];
        Act<T>::unpack8(*reinterpret_cast<const uint4*>(vp + row), x);
        const float fv = s_fv[t];
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
  // ------------------------------------------------------------------ transposed tiles out, coalesced
  uint32_t* kw_out = reinterpret_cast<uint32_t*>(a.kwT + tile * (size_t)(K * C));
  for (int i = tid; i < K * 16; i += 256) kw_out[i] = s_kw[i >> 4][i & 15];
  if (!a.skip_v) {
    uint32_t* vl_out = reinterpret_cast<uint32_t*>(a.vlT + tile * (size_t)(V * C));
    uint32_t* vw_out = reinterpret_cast<uint32_t*>(a.vwT + tile * (size_t)(V * C));
    for (int i = tid; i < V * 16; i += 256) {
      vl_out[i] = s_vl[i >> 4][i & 15];
      vw_out[i] = s_vw[i >> 4][i & 15];
    }
  }
}

template <typename T>
static int launch_prologue(const lq_zoo_problem* p, const PrologueArgs& a, cudaStream_t st) {
  dim3 grid(a.NT, p->B * p->H), block(256);
  if (p->K == 64 && p->V == 64) zoo_prologue_linear_kernel<T, 64, 64><<<grid, block, 0, st>>>(a);
  else if (p->K == 64 && p->V == 128) zoo_prologue_linear_kernel<T, 64, 128><<<grid, block, 0, st>>>(a);
  else if (p->K == 128 && p->V == 64) zoo_prologue_linear_kernel<T, 128, 64><<<grid, block, 0, st>>>(a);
  else if (p->K == 128 && p->V == 128) zoo_prologue_linear_kernel<T, 128, 128><<<grid, block, 0, st>>>(a);
  else return fail(LQ_ERR_UNSUPPORTED, "prologue: K and V must be 64 or 128 (got K=%d V=%d)", p->K, p->V);
  return check_launch("zoo_prologue_linear_kernel");
}

int validate_zoo_problem(const lq_zoo_problem* p, bool delta, bool diagonal);

void fill_prologue_args(const lq_zoo_problem* p, const lq_zoo_workspace* ws, PrologueArgs& a) {
  a.q = p->q; a.k = p->k; a.v = p->v; a.g = p->g; a.signs = p->rot_signs; a.dqk = p->dqk;
  a.sq = p->sq; a.sk = p->sk; a.skw = p->skw; a.svl = p->svl; a.svw = p->svw;
  a.qq = ws->qq; a.kl = ws->kl; a.kwT = ws->kwT; a.vlT = ws->vlT; a.vwT = ws->vwT; a.gc = ws->gc;
  a.T = p->T; a.H = p->H; a.NT = p->T / p->chunk;
  a.scale = p->scale; a.eta = p->eta; a.qmax = p->qmax; a.skip_v = 0;
}

int run_prologue_linear_mma(const lq_zoo_problem* p, const PrologueArgs& a, cudaStream_t st);

int run_prologue_linear(const lq_zoo_problem* p, const lq_zoo_workspace* ws, int skip_v, cudaStream_t st) {
  PrologueArgs a;
  fill_prologue_args(p, ws, a);
  a.skip_v = skip_v;
  // the tensor-core rotation needs operands that are exact in the activation dtype: with a D_QK rescale ahead of the
  // rotation the fp32 butterfly kernel below is used instead
  if (p->dqk == nullptr) return run_prologue_linear_mma(p, a, st);
  if (p->act_dtype == LQ_F16) return launch_prologue<__half>(p, a, st);
  if (p->act_dtype == LQ_BF16) return launch_prologue<__nv_bfloat16>(p, a, st);
  return fail(LQ_ERR_UNSUPPORTED, "prologue: activation dtype must be f16 or bf16");
}

}  // namespace lq

extern "C" int lq_zoo_prologue_linear(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream) {
  if (int e = lq::validate_zoo_problem(p, false, false)) return e;
  if (!ws) return lq::fail(LQ_ERR_NULL, "prologue: workspace descriptor is null");
  if (p->decay == LQ_DECAY_DIAGONAL) return lq::fail(LQ_ERR_UNSUPPORTED, "prologue_linear: diagonal decay uses lq_zoo_prologue_diag");
  return lq::run_prologue_linear(p, ws, 0, (cudaStream_t)stream);
}
