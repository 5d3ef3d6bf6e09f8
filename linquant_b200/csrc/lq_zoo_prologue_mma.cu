// Linear-family prologue, tensor-core version (used when no D_QK rescale is requested).
//
// Same outputs as zoo_prologue_linear_kernel, different machine mapping:
//  * the signed Walsh-Hadamard rotation is an MMA of the activation rows (bf16/fp16, exact operands) with the +-1
//    Sylvester matrix (exact in either dtype), fp32 accumulate. A warp owns 16 tokens; its A fragments are eight
//    128-bit loads issued up front, the B fragments come from a per-CTA table in shared memory (one 64-bit load each);
//  * MMA rows are mapped to tokens (2g, 2g+1) and MMA columns are permuted so that a thread ends up with eight
//    consecutive channels of two consecutive tokens: row-major code tiles leave as 64-bit stores, transposed tiles
//    as 16-bit stores into the shared-memory transposer;
//  * the code rule keeps its arithmetic (fp32 x*inv, clamp, +-0.5, truncate) but saturates the upper side in the
//    pack instruction, and a CTA walks several chunks so the table and the scale staging are amortised.
// Arithmetic and references as in lq_zoo_prologue.cu.
#include <type_traits>

#include "lq_zoo_rows.cuh"

namespace lq {

__device__ __forceinline__ uint32_t pack_sat2(int hi, int lo, uint32_t upper) {
  uint32_t d;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(hi), "r"(lo), "r"(upper));
  return d;
}
// code before the final saturation: with Q127 the upper clamp is left to the saturating pack
template <bool Q127>
__device__ __forceinline__ int code32(float x, float inv, float qmax) {
  float y = __fmul_rn(x, inv);
  y = fmaxf(y, -qmax);
  if (!Q127) y = fminf(y, qmax);
  return __float2int_rz(__fadd_rn(y, copysignf(0.5f, y)));
}
__device__ __forceinline__ uint32_t pack4s(const int (&c)[8], int o) {
  return pack_sat2(c[o + 1], c[o], pack_sat2(c[o + 3], c[o + 2], 0u));
}

template <typename T>
__device__ __forceinline__ void mma_act(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_act<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  mma_f16(c, a0, a1, a2, a3, b0, b1);
}
template <>
__device__ __forceinline__ void mma_act<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  mma_bf16(c, a0, a1, a2, a3, b0, b1);
}

template <typename T, int K, int V, bool Q127>
__global__ void __launch_bounds__(256, 2) zoo_prologue_linear_mma_kernel(PrologueArgs a, int chunks_per_cta) {
  constexpr int C = kChunk;
  constexpr int KS = K / 16, NTK = K / 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint2* s_tab = reinterpret_cast<uint2*>(smem_raw);                    // [KS][NTK][32] B fragments of the Hadamard matrix
  uint32_t(*s_kw)[17] = reinterpret_cast<uint32_t(*)[17]>(s_tab + KS * NTK * 32);
  uint32_t(*s_vl)[17] = s_kw + K;
  uint32_t(*s_vw)[17] = s_vl + V;
  float* s_sgn = reinterpret_cast<float*>(s_vw + V);                    // [K] sign * 1/sqrt(K)
  float* s_ikw = s_sgn + K;                                             // [K] 1 / skw
  float* s_ivl = s_ikw + K;                                             // [V]
  float* s_ivw = s_ivl + V;                                             // [V]
  float* s_gc = s_ivw + V;                                              // [C]
  float* s_fk = s_gc + C;
  float* s_fv = s_fk + C;

  const int bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;
  const bool rot = a.signs != nullptr;

  // ---- per-CTA staging: Hadamard B-fragment table, channel scales
  if (rot) {
    const uint32_t one = std::is_same<T, __half>::value ? 0x3C00u : 0x3F80u;
    for (int i = tid; i < KS * NTK * 32; i += 256) {
      const int ln = i & 31, nt = (i >> 5) % NTK, s = (i >> 5) / NTK;
      const int gg = ln >> 2, jj = ln & 3;
      const int n = 32 * (nt >> 2) + 8 * (gg >> 1) + 2 * (nt & 3) + (gg & 1);
      const int ch = 32 * (s >> 1) + 8 * jj + 4 * (s & 1);
      uint32_t w[2];
#pragma unroll
      for (int hi = 0; hi < 2; ++hi) {
        const uint32_t lo16 = one | ((__popc((ch + 2 * hi) & n) & 1) << 15);
        const uint32_t hi16 = one | ((__popc((ch + 2 * hi + 1) & n) & 1) << 15);
        w[hi] = lo16 | (hi16 << 16);
      }
      s_tab[i] = make_uint2(w[0], w[1]);
    }
  }
  const float norm = K == 64 ? 0.125f : 0.08838834764831845f;
  for (int i = tid; i < K; i += 256) {
    s_sgn[i] = rot ? a.signs[i] * norm : 1.0f;
    s_ikw[i] = 1.0f / a.skw[h * K + i];
  }
  for (int i = tid; i < V; i += 256) {
    s_ivl[i] = 1.0f / a.svl[h * V + i];
    s_ivw[i] = 1.0f / a.svw[h * V + i];
  }
  const float inv_sq = 1.0f / a.sq[h], inv_sk = 1.0f / a.sk[h];
  const T* qp = reinterpret_cast<const T*>(a.q);
  const T* kp = reinterpret_cast<const T*>(a.k);
  const T* vp = reinterpret_cast<const T*>(a.v);

  const int c_end = min(a.NT, (int)(blockIdx.x + 1) * chunks_per_cta);
  for (int c = blockIdx.x * chunks_per_cta; c < c_end; ++c) {
    const size_t tile = (size_t)bh * a.NT + c;
    __syncthreads();  // previous chunk's transposer reads are done; staging is visible
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

    const int mt = warp & 3;
    const int ta = 16 * mt + 2 * g, tb = ta + 1;  // this thread's two tokens of the m-tile
    const size_t rowa = (((size_t)b * a.T + (size_t)c * C + ta) * a.H + h);
    // ---------------------------------------------------------------- q (warps 0-3) or k (warps 4-7)
    {
      const bool is_q = warp < 4;
      const T* src = is_q ? qp : kp;
      uint4 ra[K / 32], rb[K / 32];
#pragma unroll
      for (int u = 0; u < K / 32; ++u) {
        ra[u] = __ldg(reinterpret_cast<const uint4*>(src + rowa * K + 32 * u + 8 * j));
        rb[u] = __ldg(reinterpret_cast<const uint4*>(src + (rowa + a.H) * K + 32 * u + 8 * j));
      }
      const float fka = s_fk[ta], fkb = s_fk[tb];
      int8_t* rowmajor = (is_q ? a.qq : a.kl) + (tile * C) * K;
#pragma unroll
      for (int ng = 0; ng < K / 32; ++ng) {
        float va[8], vb[8];
        if (rot) {
          float acc[4][4];
#pragma unroll
          for (int n4 = 0; n4 < 4; ++n4) acc[n4][0] = acc[n4][1] = acc[n4][2] = acc[n4][3] = 0.f;
#pragma unroll
          for (int s = 0; s < KS; ++s) {
            const uint32_t* wa = reinterpret_cast<const uint32_t*>(&ra[s >> 1]);
            const uint32_t* wb = reinterpret_cast<const uint32_t*>(&rb[s >> 1]);
            const uint32_t a0 = wa[2 * (s & 1)], a2 = wa[2 * (s & 1) + 1], a1 = wb[2 * (s & 1)], a3 = wb[2 * (s & 1) + 1];
#pragma unroll
            for (int n4 = 0; n4 < 4; ++n4) {
              const uint2 bf = s_tab[(s * NTK + 4 * ng + n4) * 32 + lane];
              mma_act<T>(acc[n4], a0, a1, a2, a3, bf.x, bf.y);
            }
          }
          const float4 s0 = *reinterpret_cast<const float4*>(s_sgn + 32 * ng + 8 * j);
          const float4 s1 = *reinterpret_cast<const float4*>(s_sgn + 32 * ng + 8 * j + 4);
          const float sg[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
          for (int n4 = 0; n4 < 4; ++n4)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              va[2 * n4 + e] = Act<T>::round(__fmul_rn(acc[n4][e], sg[2 * n4 + e]));
              vb[2 * n4 + e] = Act<T>::round(__fmul_rn(acc[n4][2 + e], sg[2 * n4 + e]));
            }
        } else {
          Act<T>::unpack8(ra[ng], va);
          Act<T>::unpack8(rb[ng], vb);
        }
        const int cb = 32 * ng + 8 * j;
        int ca[8], cc[8];
        if (is_q) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            ca[i] = code32<Q127>(__fmul_rn(va[i], a.scale), inv_sq, a.qmax);
            cc[i] = code32<Q127>(__fmul_rn(vb[i], a.scale), inv_sq, a.qmax);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            ca[i] = code32<Q127>(va[i], inv_sk, a.qmax);
            cc[i] = code32<Q127>(vb[i], inv_sk, a.qmax);
          }
        }
        *reinterpret_cast<uint2*>(rowmajor + (size_t)ta * K + cb) = make_uint2(pack4s(ca, 0), pack4s(ca, 4));
        *reinterpret_cast<uint2*>(rowmajor + (size_t)tb * K + cb) = make_uint2(pack4s(cc, 0), pack4s(cc, 4));
        if (!is_q) {
          const float4 i0 = *reinterpret_cast<const float4*>(s_ikw + cb);
          const float4 i1 = *reinterpret_cast<const float4*>(s_ikw + cb + 4);
          const float ik[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int wa_ = code32<Q127>(__fmul_rn(va[i], fka), ik[i], a.qmax);
            const int wb_ = code32<Q127>(__fmul_rn(vb[i], fkb), ik[i], a.qmax);
            reinterpret_cast<uint16_t*>(&s_kw[cb + i][0])[ta >> 1] = (uint16_t)pack_sat2(wb_, wa_, 0u);
          }
        }
      }
    }
    // ---------------------------------------------------------------- v: eight warps, m-tile x channel half
    if (!a.skip_v) {
      const int half = warp >> 2;
      const float fva = s_fv[ta], fvb = s_fv[tb];
#pragma unroll
      for (int uu = 0; uu < V / 64; ++uu) {
        const int cb = 32 * (half * (V / 64) + uu) + 8 * j;
        float va[8], vb[8];
        Act<T>::unpack8(__ldg(reinterpret_cast<const uint4*>(vp + rowa * V + cb)), va);
        Act<T>::unpack8(__ldg(reinterpret_cast<const uint4*>(vp + (rowa + a.H) * V + cb)), vb);
        const float4 l0 = *reinterpret_cast<const float4*>(s_ivl + cb), l1 = *reinterpret_cast<const float4*>(s_ivl + cb + 4);
        const float4 w0 = *reinterpret_cast<const float4*>(s_ivw + cb), w1 = *reinterpret_cast<const float4*>(s_ivw + cb + 4);
        const float il[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
        const float iw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int la = code32<Q127>(va[i], il[i], a.qmax), lb = code32<Q127>(vb[i], il[i], a.qmax);
          const int wa_ = code32<Q127>(__fmul_rn(va[i], fva), iw[i], a.qmax);
          const int wb_ = code32<Q127>(__fmul_rn(vb[i], fvb), iw[i], a.qmax);
          reinterpret_cast<uint16_t*>(&s_vl[cb + i][0])[ta >> 1] = (uint16_t)pack_sat2(lb, la, 0u);
          reinterpret_cast<uint16_t*>(&s_vw[cb + i][0])[ta >> 1] = (uint16_t)pack_sat2(wb_, wa_, 0u);
        }
      }
    }
    __syncthreads();
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
}

template <typename T, int K, int V>
static int launch_mma(const lq_zoo_problem* p, const PrologueArgs& a, cudaStream_t st) {
  const int cpb = (a.NT % 4 == 0 && (long long)a.NT * p->B * p->H >= 4096) ? 4 : 1;
  dim3 grid((a.NT + cpb - 1) / cpb, p->B * p->H), block(256);
  const size_t smem = sizeof(uint2) * (K / 16) * (K / 8) * 32 + sizeof(uint32_t) * 17 * (K + 2 * V) +
                      sizeof(float) * (2 * K + 2 * V + 3 * 64);
  cudaError_t e;
  if (p->qmax == 127.f) {
    e = cudaFuncSetAttribute(zoo_prologue_linear_mma_kernel<T, K, V, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) zoo_prologue_linear_mma_kernel<T, K, V, true><<<grid, block, smem, st>>>(a, cpb);
  } else {
    e = cudaFuncSetAttribute(zoo_prologue_linear_mma_kernel<T, K, V, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) zoo_prologue_linear_mma_kernel<T, K, V, false><<<grid, block, smem, st>>>(a, cpb);
  }
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "prologue: cannot opt in to %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  return check_launch("zoo_prologue_linear_mma_kernel");
}

template <typename T>
static int dispatch_mma(const lq_zoo_problem* p, const PrologueArgs& a, cudaStream_t st) {
  if (p->K == 64 && p->V == 64) return launch_mma<T, 64, 64>(p, a, st);
  if (p->K == 64 && p->V == 128) return launch_mma<T, 64, 128>(p, a, st);
  if (p->K == 128 && p->V == 64) return launch_mma<T, 128, 64>(p, a, st);
  if (p->K == 128 && p->V == 128) return launch_mma<T, 128, 128>(p, a, st);
  return fail(LQ_ERR_UNSUPPORTED, "prologue: K and V must be 64 or 128 (got K=%d V=%d)", p->K, p->V);
}

int run_prologue_linear_mma(const lq_zoo_problem* p, const PrologueArgs& a, cudaStream_t st) {
  if (p->act_dtype == LQ_F16) return dispatch_mma<__half>(p, a, st);
  if (p->act_dtype == LQ_BF16) return dispatch_mma<__nv_bfloat16>(p, a, st);
  return fail(LQ_ERR_UNSUPPORTED, "prologue: activation dtype must be f16 or bf16");
}

}  // namespace lq
