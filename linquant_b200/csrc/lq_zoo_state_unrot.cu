// Inter-chunk state pass of the linear family with canonical storage under a value rotation R_V
// (zoo/simple_gla.py:31-33, :69-72; zoo/gla.py:139-146).
//
// v arrives rotated, so the INT8 write product  P[v,k] = sum_t vw[t,v] kw[t,k]  is in the rotated value basis. It
// is dequantised, rounded to fp16 and multiplied by the un-rotation M (fp16, out = x . M over the value index)
// before it joins the fp32 carry, so the carry and its stored INT8 copy are canonical:
//     carry[k,:] <- gamma_k carry[k,:] + fp16(P[:,k] svw skw_k) . M
// The un-rotation mixes all value channels, so a CTA owns sixteen key channels x ALL value channels of one
// (batch, head) and walks the chunks; the un-rotation runs as an fp16 MMA with the product tile transposed through
// shared memory, and the canonical carry lives in that MMA's accumulator layout (rows = key channels).
#include "lq_common.cuh"

namespace lq {

struct StateUnrotArgs {
  const int8_t *kwT, *vwT;
  const float *gc, *skw, *svw, *ss, *gcl;
  const __half* unrot_t;  // [V,V] fp16, element [v'][v] = M[v][v']
  int8_t* hT;
  float* final_state;
  const float* initial_state;
  int H, NT, use_g;
};

template <int K, int V, bool DIAG>
__global__ void __launch_bounds__(128) zoo_state_linear_unrot_kernel(StateUnrotArgs a) {
  constexpr int C = 64, KB = 16, LDR = V + 8;
  constexpr int MTW = V / 64;   // 16-row value tiles of the write product per warp
  constexpr int NTW = V / 32;   // 8-column canonical value tiles of the carry per warp
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __half* s_rt = reinterpret_cast<__half*>(smem_raw);  // [V][LDR]   M^T
  __half* s_pt = s_rt + V * LDR;                       // [KB][LDR]  dequantised product, key-major
  int8_t* s_hq = reinterpret_cast<int8_t*>(s_pt + KB * LDR);  // [V][KB] codes of the carry, for the 16-byte row stores

  const int k0 = blockIdx.x * KB;
  const int bh = blockIdx.y, h = bh % a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;

  for (int i = tid; i < V * (V / 8); i += 128) {
    const int row = i / (V / 8), ch = i % (V / 8);
    *reinterpret_cast<uint4*>(s_rt + row * LDR + 8 * ch) = __ldg(reinterpret_cast<const uint4*>(a.unrot_t + (size_t)row * V) + ch);
  }

  const int8_t* vw = a.vwT + (size_t)bh * a.NT * V * C;
  const int8_t* kw = a.kwT + (size_t)bh * a.NT * K * C;
  int8_t* hT = a.hT + (size_t)bh * a.NT * V * K;
  const float* gc = a.gc + (size_t)bh * a.NT * C;

  float svw_r[MTW][2];
#pragma unroll
  for (int m = 0; m < MTW; ++m) {
    svw_r[m][0] = a.svw[h * V + 16 * (MTW * warp + m) + g];
    svw_r[m][1] = a.svw[h * V + 16 * (MTW * warp + m) + g + 8];
  }
  float skw_c[2][2];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) skw_c[nt][e] = a.skw[h * K + k0 + 8 * nt + 2 * j + e];
  float iss[NTW][2];
#pragma unroll
  for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) iss[nt][e] = 1.0f / a.ss[h * V + 8 * (NTW * warp + nt) + 2 * j + e];

  // canonical carry: rows k0 + g, k0 + g + 8; columns 8 (NTW warp + nt) + 2j + e
  float carry[NTW][4];
#pragma unroll
  for (int nt = 0; nt < NTW; ++nt) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int kr = k0 + g + 8 * (i >> 1), vc = 8 * (NTW * warp + nt) + 2 * j + (i & 1);
      carry[nt][i] = a.initial_state ? a.initial_state[((size_t)bh * K + kr) * V + vc] : 0.f;
    }
  }
  __syncthreads();

  for (int c = 0; c < a.NT; ++c) {
    const int8_t* vwc = vw + (size_t)c * V * C;
    const int8_t* kwc = kw + (size_t)c * K * C;
    uint4 A_lo[MTW], A_hi[MTW], Bq[2];
#pragma unroll
    for (int m = 0; m < MTW; ++m) {
      const int vr = 16 * (MTW * warp + m) + g;
      A_lo[m] = __ldg(reinterpret_cast<const uint4*>(vwc + vr * C + 16 * j));
      A_hi[m] = __ldg(reinterpret_cast<const uint4*>(vwc + (vr + 8) * C + 16 * j));
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) Bq[nt] = __ldg(reinterpret_cast<const uint4*>(kwc + (k0 + 8 * nt + g) * C + 16 * j));

    // INT8 copy of the carry entering chunk c -> hT[c][row(v)][k0 .. k0+15]
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int kr = g + 8 * (i >> 1), vc = 8 * (NTW * warp + nt) + 2 * j + (i & 1);
        s_hq[vc * KB + kr] = (int8_t)q8(carry[nt][i], iss[nt][i & 1], 127.f);
      }
    }
    __syncthreads();
    for (int vc = tid; vc < V; vc += 128) {
      *reinterpret_cast<uint4*>(hT + ((size_t)c * V + state_row_of_channel(vc)) * K + k0) =
          *reinterpret_cast<const uint4*>(s_hq + vc * KB);
    }

    // write product in the rotated basis, dequantised, fp16, key-major
#pragma unroll
    for (int m = 0; m < MTW; ++m) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        int acc[4] = {0, 0, 0, 0};
        mma_s8(acc, A_lo[m].x, A_hi[m].x, A_lo[m].y, A_hi[m].y, Bq[nt].x, Bq[nt].y);
        mma_s8(acc, A_lo[m].z, A_hi[m].z, A_lo[m].w, A_hi[m].w, Bq[nt].z, Bq[nt].w);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int vr = 16 * (MTW * warp + m) + g + 8 * (i >> 1), kc = 8 * nt + 2 * j + (i & 1);
          const float val = __fmul_rn(__fmul_rn((float)acc[i], skw_c[nt][i & 1]), svw_r[m][i >> 1]);
          s_pt[kc * LDR + vr] = __float2half_rn(val);
        }
      }
    }
    __syncthreads();

    // un-rotation on the tensor cores, folded into the carry
    float gam[2] = {1.f, 1.f};
    if (DIAG) {
      gam[0] = expf(a.gcl[((size_t)bh * a.NT + c) * K + k0 + g]);
      gam[1] = expf(a.gcl[((size_t)bh * a.NT + c) * K + k0 + g + 8]);
    } else if (a.use_g) {
      gam[0] = gam[1] = expf(gc[(size_t)c * C + (C - 1)]);
    }
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt) {
      float u[4] = {0.f, 0.f, 0.f, 0.f};
      const __half* rrow = s_rt + (8 * (NTW * warp + nt) + g) * LDR;
#pragma unroll
      for (int kk = 0; kk < V / 16; ++kk) {
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(s_pt + g * LDR + 16 * kk + 2 * j);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(s_pt + (g + 8) * LDR + 16 * kk + 2 * j);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(s_pt + g * LDR + 16 * kk + 8 + 2 * j);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(s_pt + (g + 8) * LDR + 16 * kk + 8 + 2 * j);
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(rrow + 16 * kk + 2 * j);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(rrow + 16 * kk + 8 + 2 * j);
        mma_f16(u, a0, a1, a2, a3, b0, b1);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) carry[nt][i] = fmaf(carry[nt][i], gam[i >> 1], u[i]);
    }
    __syncthreads();  // s_pt and s_hq are rewritten by the next chunk
  }

  if (a.final_state != nullptr) {
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int kr = k0 + g + 8 * (i >> 1), vc = 8 * (NTW * warp + nt) + 2 * j + (i & 1);
        a.final_state[((size_t)bh * K + kr) * V + vc] = carry[nt][i];
      }
    }
  }
}

template <int K, int V>
static int launch_state_unrot(const lq_zoo_problem* p, const StateUnrotArgs& a, cudaStream_t st) {
  const size_t smem = sizeof(__half) * (size_t)(V + 16) * (V + 8) + (size_t)V * 16;
  dim3 grid(K / 16, p->B * p->H);
  cudaError_t e;
  if (p->decay == LQ_DECAY_DIAGONAL) {
    e = cudaFuncSetAttribute(zoo_state_linear_unrot_kernel<K, V, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) zoo_state_linear_unrot_kernel<K, V, true><<<grid, 128, smem, st>>>(a);
  } else {
    e = cudaFuncSetAttribute(zoo_state_linear_unrot_kernel<K, V, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) zoo_state_linear_unrot_kernel<K, V, false><<<grid, 128, smem, st>>>(a);
  }
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "state (canonical storage): shared memory opt-in failed: %s", cudaGetErrorString(e));
  return check_launch("zoo_state_linear_unrot_kernel");
}

int run_state_linear_unrot(const lq_zoo_problem* p, const lq_zoo_workspace* ws, cudaStream_t st) {
  StateUnrotArgs a;
  a.kwT = ws->kwT; a.vwT = ws->vwT; a.gc = ws->gc; a.skw = p->skw; a.svw = p->svw; a.ss = p->sstate; a.gcl = ws->gcl;
  a.unrot_t = reinterpret_cast<const __half*>(p->unrot_t);
  a.hT = ws->hT; a.final_state = p->final_state; a.initial_state = p->initial_state; a.H = p->H; a.NT = p->T / p->chunk;
  a.use_g = p->g != nullptr;
  if (p->K == 64 && p->V == 64) return launch_state_unrot<64, 64>(p, a, st);
  if (p->K == 64 && p->V == 128) return launch_state_unrot<64, 128>(p, a, st);
  if (p->K == 128 && p->V == 64) return launch_state_unrot<128, 64>(p, a, st);
  if (p->K == 128 && p->V == 128) return launch_state_unrot<128, 128>(p, a, st);
  return fail(LQ_ERR_UNSUPPORTED, "state (canonical storage): K and V must be 64 or 128");
}

}  // namespace lq
