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

__device__ __forceinline__ uint32_t pack_sat2(int hi, int lo, uint32_t upper) { return pack_sat_s8x2(hi, lo, upper); }
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

// Hadamard product step: the B fragment arrives as one 64-bit register pair (the MMA wants its two B registers adjacent;
// separate 32-bit operands chosen per step made the compiler copy them into place before every instruction), and the
// first step of a chain takes C = 0 instead of zeroed accumulators.
template <typename T, bool FIRST>
__device__ __forceinline__ void mma_had(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint64_t bp) {
  if (std::is_same<T, __half>::value) {
    if (FIRST)
      asm volatile("{\n.reg .b32 b0, b1;\nmov.b64 {b0, b1}, %8;\n"
                   "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {b0,b1}, {%9,%9,%9,%9};\n}\n"
                   : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "l"(bp), "f"(0.f));
    else
      asm volatile("{\n.reg .b32 b0, b1;\nmov.b64 {b0, b1}, %8;\n"
                   "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {b0,b1}, {%0,%1,%2,%3};\n}\n"
                   : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "l"(bp));
  } else {
    if (FIRST)
      asm volatile("{\n.reg .b32 b0, b1;\nmov.b64 {b0, b1}, %8;\n"
                   "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {b0,b1}, {%9,%9,%9,%9};\n}\n"
                   : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "l"(bp), "f"(0.f));
    else
      asm volatile("{\n.reg .b32 b0, b1;\nmov.b64 {b0, b1}, %8;\n"
                   "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {b0,b1}, {%0,%1,%2,%3};\n}\n"
                   : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "l"(bp));
  }
}

template <typename T, int K, int V, bool Q127>
__global__ void __launch_bounds__(256, 2) zoo_prologue_linear_mma_kernel(PrologueArgs a, int n_tiles) {
  constexpr int C = kChunk;
  constexpr int KS = K / 16;
  constexpr int RAW_Q = C * K * 2, RAW_V = C * V * 2;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint32_t(*s_kw)[17] = reinterpret_cast<uint32_t(*)[17]>(smem_raw);
  uint32_t(*s_vl)[17] = s_kw + K;
  uint32_t(*s_vw)[17] = s_vl + V;
  float* s_sgn = reinterpret_cast<float*>(s_vw + V);  // [K] sign * 1/sqrt(K)
  float* s_ikw = s_sgn + K;                           // [K] 1 / skw
  float* s_ivl = s_ikw + K;                           // [V]
  float* s_ivw = s_ivl + V;                           // [V]
  // raw activation tiles (cp.async): q,k of two chunks in flight, v of one; 16-byte pieces XOR-swizzled with bit 1
  // of the token index so that the 128-bit fragment reads are conflict free
  uint8_t* s_qk = reinterpret_cast<uint8_t*>(s_ivw + V);  // [2 buf][q|k][C][K*2]
  uint8_t* s_v = s_qk + 4 * RAW_Q;                        // [C][V*2]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;
  const bool rot = a.signs != nullptr;
  const float norm = K == 64 ? 0.125f : 0.08838834764831845f;
  const T* qp = reinterpret_cast<const T*>(a.q);
  const T* kp = reinterpret_cast<const T*>(a.k);
  const T* vp = reinterpret_cast<const T*>(a.v);

  // B fragments of the Sylvester matrix without a table. With input channel c = 32u + 8j + 4h + 2hi + e (k-step
  // s = 2u + h, register hi, half e) and output channel n = 32(nt>>2) + 8(g>>1) + 2(nt&3) + (g&1), the sign
  // (-1)^popc(c & n) splits into a per-lane part (e*g0 ^ j0*g1 ^ j1*g2), a part hi*(nt&1), and a part that depends
  // on (s, nt) only. The last two are compile-time choices between the base register and its negation.
  uint32_t hb0, hb0n;
  {
    const uint32_t one = std::is_same<T, __half>::value ? 0x3C00u : 0x3F80u;
    const uint32_t L = ((j & 1) & ((g >> 1) & 1)) ^ (((j >> 1) & 1) & ((g >> 2) & 1));
    hb0 = (one | (L << 15)) | ((one | ((L ^ (g & 1)) << 15)) << 16);
    hb0n = hb0 ^ 0x80008000u;
  }
  // the four (b0, b1) sign combinations as register pairs, index 2*neg(b0) + neg(b1)
  const uint64_t hbp[4] = {(uint64_t)hb0 | ((uint64_t)hb0 << 32), (uint64_t)hb0 | ((uint64_t)hb0n << 32),
                           (uint64_t)hb0n | ((uint64_t)hb0 << 32), (uint64_t)hb0n | ((uint64_t)hb0n << 32)};

  // persistent CTAs: tile t = (batch, chunk, head) with the head fastest, strided by the grid: every CTA gets the same
  // number of tiles to within one, and the CTAs in flight read all heads of the same tokens (adjacent in memory)
  // staging copies: thread -> (token row r0 + RPI it, 16-byte piece ch0); the swizzle bit of the row does not change
  // with it, so source and destination advance by constants. Tile indices are decoded once per tile (integer
  // divisions by run-time extents are the expensive part of this bookkeeping).
  constexpr int PPRK = K / 8, RPIK = 256 / PPRK, PPRV = V / 8, RPIV = 256 / PPRV;
  const int rk0 = tid / PPRK, chk0 = tid % PPRK, rv0 = tid / PPRV, chv0 = tid % PPRV;
  const uint32_t dstk0 = rk0 * (K * 2) + ((chk0 ^ (((rk0 >> 1) & 1) << 2)) << 4);
  const uint32_t dstv0 = rv0 * (V * 2) + ((chv0 ^ (((rv0 >> 1) & 1) << 2)) << 4);
  auto stage_qk = [&](int h, int c, int b, int buf) {
    uint8_t* dst = s_qk + buf * 2 * RAW_Q + dstk0;
    const size_t off = (((size_t)b * a.T + (size_t)c * C + rk0) * a.H + h) * K + 8 * chk0;
    const T* sq = qp + off;
    const T* sk = kp + off;
    const size_t step = (size_t)RPIK * a.H * K;
#pragma unroll
    for (int it = 0; it < C / RPIK; ++it) {
      cp_async16(dst + it * RPIK * (K * 2), sq);
      cp_async16(dst + RAW_Q + it * RPIK * (K * 2), sk);
      sq += step;
      sk += step;
    }
  };
  auto stage_v = [&](int h, int c, int b) {
    if (a.skip_v) return;
    const T* sv = vp + (((size_t)b * a.T + (size_t)c * C + rv0) * a.H + h) * V + 8 * chv0;
    const size_t step = (size_t)RPIV * a.H * V;
#pragma unroll
    for (int it = 0; it < C / RPIV; ++it) {
      cp_async16(s_v + dstv0 + it * RPIV * (V * 2), sv);
      sv += step;
    }
  };
  auto load_g = [&](int h, int c, int b, float& g0, float& g1) {
    if (a.g == nullptr) { g0 = g1 = 0.f; return; }
    const size_t base = ((size_t)b * a.T + (size_t)c * C) * a.H + h;
    g0 = __ldg(a.g + base + (size_t)lane * a.H);
    g1 = __ldg(a.g + base + (size_t)(lane + 32) * a.H);
  };
  auto decode = [&](int t, int& h, int& c, int& b) {
    h = t % a.H;
    const int r = t / a.H;
    c = r % a.NT;
    b = r / a.NT;
  };
  const int t_begin = blockIdx.x, t_step = gridDim.x;
  if (t_begin >= n_tiles) return;
  int h, c, b, hn = 0, cn = 0, bn = 0;
  decode(t_begin, h, c, b);
  stage_qk(h, c, b, 0);
  stage_v(h, c, b);
  cp_async_commit();
  float gn0, gn1;
  load_g(h, c, b, gn0, gn1);

  const int mt = warp & 3;
  const int ta = 16 * mt + 2 * g, tb = ta + 1;  // this thread's two tokens of the m-tile
  const int swz = ((ta >> 1) & 1) << 2;         // tb shares bit 1 of the token index

  int h_staged = -1;
  float inv_sq = 1.f, inv_sk = 1.f;
  for (int t = t_begin, it = 0; t < n_tiles; t += t_step, ++it, h = hn, c = cn, b = bn) {
    const size_t tile = ((size_t)b * a.H + h) * a.NT + c;
    const int buf = it & 1;
    const bool more = t + t_step < n_tiles;
    cp_async_wait<0>();
    __syncthreads();  // raw tiles of this chunk have landed; the previous chunk's compute and copy-out are done
    if (more) {
      decode(t + t_step, hn, cn, bn);
      stage_qk(hn, cn, bn, buf ^ 1);
      cp_async_commit();
    }
    if (h != h_staged) {  // per-head channel scales (uniform branch)
      for (int i = tid; i < K; i += 256) {
        s_sgn[i] = rot ? a.signs[i] * norm : 1.0f;
        s_ikw[i] = 1.0f / a.skw[h * K + i];
      }
      for (int i = tid; i < V; i += 256) {
        s_ivl[i] = 1.0f / a.svl[h * V + i];
        s_ivw[i] = 1.0f / a.svw[h * V + i];
      }
      h_staged = h;
      inv_sq = 1.0f / a.sq[h];
      inv_sk = 1.0f / a.sk[h];
      __syncthreads();
    }
    // ---- chunk-local cumulative log-decay, per warp (double accumulate), no shared memory
    float gca, gcb, glast;
    {
      double x0 = (double)gn0, x1 = (double)gn1;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const double y0 = __shfl_up_sync(0xffffffffu, x0, d), y1 = __shfl_up_sync(0xffffffffu, x1, d);
        if (lane >= d) { x0 += y0; x1 += y1; }
      }
      x1 += __shfl_sync(0xffffffffu, x0, 31);
      const float f0 = (float)x0, f1 = (float)x1;
      if (warp == 0) {
        a.gc[tile * C + lane] = f0;
        a.gc[tile * C + 32 + lane] = f1;
      }
      glast = __shfl_sync(0xffffffffu, f1, 31);
      const float sel = (mt >> 1) ? f1 : f0;
      gca = __shfl_sync(0xffffffffu, sel, ta & 31);
      gcb = __shfl_sync(0xffffffffu, sel, tb & 31);
      if (more) load_g(hn, cn, bn, gn0, gn1);
    }
    const bool use_g = a.g != nullptr;
    const float da = glast - gca, db = glast - gcb;
    // ---------------------------------------------------------------- q then k: a warp owns an m-tile and one half
    // of the output channels of both operands (equal work in every warp)
#pragma unroll
    for (int op = 0; op < 2; ++op) {
      const bool is_q = op == 0;
      const int half = warp >> 2;
      // the channel half of the warp flips the sign of the steps whose input channels carry that bit: applied to the
      // A fragments of those steps (an XOR on their way into the MMA's register quad)
      const uint32_t sflip = half ? 0x80008000u : 0u;
      const uint8_t* src = s_qk + buf * 2 * RAW_Q + (is_q ? 0 : RAW_Q);
      uint4 ra[K / 32], rb[K / 32];
#pragma unroll
      for (int u = 0; u < K / 32; ++u) {
        ra[u] = *reinterpret_cast<const uint4*>(src + ta * (K * 2) + (((4 * u + j) ^ swz) << 4));
        rb[u] = *reinterpret_cast<const uint4*>(src + tb * (K * 2) + (((4 * u + j) ^ swz) << 4));
      }
      const float fka = use_g ? expf((1.0f - a.eta) * da) : 1.0f, fkb = use_g ? expf((1.0f - a.eta) * db) : 1.0f;
      int8_t* rowmajor = (is_q ? a.qq : a.kl) + (tile * C) * K;
#pragma unroll
      for (int ngl = 0; ngl < K / 64; ++ngl) {
        const int ng = half * (K / 64) + ngl;
        float va[8], vb[8];
        if (rot) {
          float acc[4][4];
#pragma unroll
          for (int s = 0; s < KS; ++s) {
            const uint32_t* wa = reinterpret_cast<const uint32_t*>(&ra[s >> 1]);
            const uint32_t* wb = reinterpret_cast<const uint32_t*>(&rb[s >> 1]);
            const bool dep = K == 128 ? ((s >> 2) & 1) : ((s >> 1) & 1);
            const uint32_t fl = dep ? sflip : 0u;
            const uint32_t a0 = wa[2 * (s & 1)] ^ fl, a2 = wa[2 * (s & 1) + 1] ^ fl, a1 = wb[2 * (s & 1)] ^ fl, a3 = wb[2 * (s & 1) + 1] ^ fl;
#pragma unroll
            for (int n4 = 0; n4 < 4; ++n4) {
              // output n-tile nt = 4*ng + n4; its bits above n4 are ngl (compile time) and the warp's channel half
              const int Uc = ((s & 1) & ((n4 >> 1) & 1)) ^ (K == 128 ? (((s >> 1) & 1) & (ngl & 1)) : 0);
              if (s == 0) mma_had<T, true>(acc[n4], a0, a1, a2, a3, hbp[2 * Uc + (Uc ^ (n4 & 1))]);
              else mma_had<T, false>(acc[n4], a0, a1, a2, a3, hbp[2 * Uc + (Uc ^ (n4 & 1))]);
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
          Act<T>::unpack8(half ? ra[K / 64 + ngl] : ra[ngl], va);
          Act<T>::unpack8(half ? rb[K / 64 + ngl] : rb[ngl], vb);
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
        const int pa_ = is_q ? ta : kl_row_of_token(ta), pb_ = is_q ? tb : kl_row_of_token(tb);
        *reinterpret_cast<uint2*>(rowmajor + (size_t)pa_ * K + cb) = make_uint2(pack4s(ca, 0), pack4s(ca, 4));
        *reinterpret_cast<uint2*>(rowmajor + (size_t)pb_ * K + cb) = make_uint2(pack4s(cc, 0), pack4s(cc, 4));
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
      const float fva = use_g ? expf(a.eta * da) : 1.0f, fvb = use_g ? expf(a.eta * db) : 1.0f;
#pragma unroll
      for (int uu = 0; uu < V / 64; ++uu) {
        const int cb = 32 * (half * (V / 64) + uu) + 8 * j;
        float va[8], vb[8];
        Act<T>::unpack8(*reinterpret_cast<const uint4*>(s_v + ta * (V * 2) + (((cb >> 3) ^ swz) << 4)), va);
        Act<T>::unpack8(*reinterpret_cast<const uint4*>(s_v + tb * (V * 2) + (((cb >> 3) ^ swz) << 4)), vb);
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
    if (more) {  // the single v buffer is free again
      stage_v(hn, cn, bn);
      cp_async_commit();
    }
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
  const int tiles = a.NT * p->B * p->H;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // a grid that is a multiple of the head count keeps every CTA on one head (its scales are staged once)
  int ctas = 2 * sms;
  if (p->H <= ctas) ctas = (ctas / p->H) * p->H;
  dim3 grid(tiles < ctas ? tiles : ctas), block(256);
  const size_t smem = sizeof(uint32_t) * 17 * (K + 2 * V) + sizeof(float) * (2 * K + 2 * V) + (size_t)(4 * 64 * K * 2 + 64 * V * 2);
  cudaError_t e;
  if (p->qmax == 127.f) {
    e = cudaFuncSetAttribute(zoo_prologue_linear_mma_kernel<T, K, V, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(zoo_prologue_linear_mma_kernel<T, K, V, true>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e == cudaSuccess) zoo_prologue_linear_mma_kernel<T, K, V, true><<<grid, block, smem, st>>>(a, tiles);
  } else {
    e = cudaFuncSetAttribute(zoo_prologue_linear_mma_kernel<T, K, V, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(zoo_prologue_linear_mma_kernel<T, K, V, false>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e == cudaSuccess) zoo_prologue_linear_mma_kernel<T, K, V, false><<<grid, block, smem, st>>>(a, tiles);
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
