// Intra-chunk output of the none / scalar decay cells on INT8 tiles (linear and delta families share it).
//
// One CTA per (chunk, batch*head); four warps, each owning 16 tokens x all V value channels:
//   S2 = qq . kl^T            INT8 MMA, int32   (only the 16-token column blocks at or below the warp's rows)
//   P  = fp16( S2 * sq*sk * exp(gc_i - gc_j) ), zero above the diagonal, kept in registers as the A operand of
//   O2 = P . vl               fp16 MMA on the value codes (codes widened to fp16 with a byte permute, exact)
//   S1 = qq . hT^T            INT8 MMA against the stored state entering the chunk
//   o  = S1 * sq*ss[v] * exp(gc_i) + O2 * svl[v]
// The tiles arrive by 16-byte cp.async into XOR-swizzled shared memory so that every 128-bit fragment load is
// bank-conflict free; column indices of the MMA tiles are permuted (the B operand rows are gathered) so that a
// thread ends up with eight consecutive value channels of a row and stores them with one 16-byte write.
//
// Reference arithmetic: zoo/simple_gla.py:99-153 (_output_body); reference.py:167-171 (read with the decay
// applied after the product), :130-132 (masked local product), :182-187 (fp16 value product).
#include "lq_common.cuh"

namespace lq {

struct OutputArgs {
  const int8_t *qq, *kl, *vlT, *hT;
  const float *gc, *sq, *sk, *svl, *ss;
  const __half* amat;  // diagonal decay: [BH,NT,C,C] intra-chunk matrix A, already masked and in fp16
  const __half* unrot_t;  // canonical storage: [V,V] fp16, element [v'][v] = M[v][v'] of the un-rotation o_local . M
  void* o;
  int T, H, NT;
};

template <int ROWB>
__device__ __forceinline__ int swz_k(int row, int chunk) {
  if (ROWB == 128) return row * 128 + ((chunk ^ ((row & 1) << 2)) << 4);
  return row * 64 + (chunk << 4);
}
__device__ __forceinline__ int swz_v(int row, int chunk) { return row * 64 + ((chunk ^ ((row >> 3) & 3)) << 4); }

template <typename OT>
__device__ __forceinline__ void store8(OT* dst, const float (&x)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* dst, const float (&x)[8]) {
  reinterpret_cast<float4*>(dst)[0] = make_float4(x[0], x[1], x[2], x[3]);
  reinterpret_cast<float4*>(dst)[1] = make_float4(x[4], x[5], x[6], x[7]);
}
template <>
__device__ __forceinline__ void store8<__half>(__half* dst, const float (&x)[8]) {
  *reinterpret_cast<uint4*>(dst) = make_uint4(Act<__half>::pack2(x[0], x[1]), Act<__half>::pack2(x[2], x[3]),
                                              Act<__half>::pack2(x[4], x[5]), Act<__half>::pack2(x[6], x[7]));
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* dst, const float (&x)[8]) {
  *reinterpret_cast<uint4*>(dst) =
      make_uint4(Act<__nv_bfloat16>::pack2(x[0], x[1]), Act<__nv_bfloat16>::pack2(x[2], x[3]),
                 Act<__nv_bfloat16>::pack2(x[4], x[5]), Act<__nv_bfloat16>::pack2(x[6], x[7]));
}

template <int K, int V, typename OT, bool DIAG, bool UNROT>
__global__ void __launch_bounds__(128) zoo_output_scalar_kernel(OutputArgs a) {
  constexpr int C = 64, LDR = V + 8;
  constexpr int KK = K / 64;  // 64-byte reduction blocks per row
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* s_q = smem;
  uint8_t* s_k = s_q + C * K;
  uint8_t* s_h = s_k + C * K;
  uint8_t* s_v = s_h + V * K;
  float* s_gc = reinterpret_cast<float*>(s_v + V * C);
  float* s_ss = s_gc + C;
  float* s_svl = s_ss + V;
  __half* s_rt = reinterpret_cast<__half*>(s_svl + V);  // [V][LDR] un-rotation, input index contiguous (UNROT only)

  const int c = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;
  const size_t tile = (size_t)bh * a.NT + c;

  // ---- stage the tiles
  {
    const int8_t* gq = a.qq + tile * (size_t)(C * K);
    const int8_t* gk = a.kl + tile * (size_t)(C * K);
    const int8_t* gh = a.hT + tile * (size_t)(V * K);
    const int8_t* gv = a.vlT + tile * (size_t)(V * C);
    constexpr int CPR = K / 16;  // 16-byte chunks per K-row
    for (int i = tid; i < C * CPR; i += 128) {
      const int row = i / CPR, ch = i % CPR;
      cp_async16(s_q + swz_k<K>(row, ch), gq + (size_t)i * 16);
      if (!DIAG) cp_async16(s_k + swz_k<K>(row, ch), gk + (size_t)i * 16);
    }
    for (int i = tid; i < V * CPR; i += 128) {
      const int row = i / CPR, ch = i % CPR;
      cp_async16(s_h + swz_k<K>(row, ch), gh + (size_t)i * 16);
    }
    for (int i = tid; i < V * 4; i += 128) {
      const int row = i >> 2, ch = i & 3;
      cp_async16(s_v + swz_v(row, ch), gv + (size_t)i * 16);
    }
    if (UNROT) {
      for (int i = tid; i < V * (V / 8); i += 128) {
        const int row = i / (V / 8), ch = i % (V / 8);
        cp_async16(s_rt + row * LDR + 8 * ch, a.unrot_t + (size_t)row * V + 8 * ch);
      }
    }
    cp_async_commit();
    if (tid < C) s_gc[tid] = DIAG ? 0.f : a.gc[tile * C + tid];
    for (int i = tid; i < V; i += 128) {
      s_ss[i] = a.ss[h * V + i];
      s_svl[i] = a.svl[h * V + i];
    }
    cp_async_wait<0>();
    __syncthreads();
  }

  const float sq = a.sq[h], sk = a.sk[h];
  const float sqk = __fmul_rn(sq, sk);
  const int ia = warp * 16 + g, ib = ia + 8;
  const float gia = s_gc[ia], gib = s_gc[ib];

  uint4 qa[KK], qb[KK];
#pragma unroll
  for (int kk = 0; kk < KK; ++kk) {
    qa[kk] = *reinterpret_cast<const uint4*>(s_q + swz_k<K>(ia, 4 * kk + j));
    qb[kk] = *reinterpret_cast<const uint4*>(s_q + swz_k<K>(ib, 4 * kk + j));
  }

  // ---- S2 and P. MMA column (nt, cn) of S2 is token 16*(nt/2) + 4*(cn/2) + 2*(nt%2) + (cn%2).
  uint32_t P[4][4];
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    if (DIAG) {
      // A operand straight from the precomputed matrix: slots (2j,2j+1 | 8+2j,8+2j+1) of k-step ks are the
      // tokens 16ks + 4j + {0,1 | 2,3}
      if (ks <= warp) {
        const uint2 ra = *reinterpret_cast<const uint2*>(a.amat + (tile * C + ia) * C + 16 * ks + 4 * j);
        const uint2 rb = *reinterpret_cast<const uint2*>(a.amat + (tile * C + ib) * C + 16 * ks + 4 * j);
        P[ks][0] = ra.x; P[ks][1] = rb.x; P[ks][2] = ra.y; P[ks][3] = rb.y;
      } else {
        P[ks][0] = P[ks][1] = P[ks][2] = P[ks][3] = 0u;
      }
    } else if (ks <= warp) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        int acc[4] = {0, 0, 0, 0};
        const int tok_row = 16 * ks + 8 * half + g;  // row n of the k_local tile is MMA column n
#pragma unroll
        for (int kk = 0; kk < KK; ++kk) {
          const uint4 bk = *reinterpret_cast<const uint4*>(s_k + swz_k<K>(tok_row, 4 * kk + j));
          mma_s8(acc, qa[kk].x, qb[kk].x, qa[kk].y, qb[kk].y, bk.x, bk.y);
          mma_s8(acc, qa[kk].z, qb[kk].z, qa[kk].w, qb[kk].w, bk.z, bk.w);
        }
        float pa[2], pb[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tj = 16 * ks + 4 * j + 2 * half + e;
          const float gj = s_gc[tj];
          pa[e] = (ia >= tj) ? __fmul_rn((float)acc[e], sqk) * __expf(gia - gj) : 0.f;
          pb[e] = (ib >= tj) ? __fmul_rn((float)acc[2 + e], sqk) * __expf(gib - gj) : 0.f;
        }
        P[ks][2 * half + 0] = Act<__half>::pack2(pa[0], pa[1]);
        P[ks][2 * half + 1] = Act<__half>::pack2(pb[0], pb[1]);
      }
    } else {
      P[ks][0] = P[ks][1] = P[ks][2] = P[ks][3] = 0u;
    }
  }

  // ---- O2 = P . vl.  MMA column (nt, cn) is value channel 32*(nt/4) + 8*(cn/2) + 2*(nt%4) + (cn%2).
  float acco[V / 8][4];
#pragma unroll
  for (int nt = 0; nt < V / 8; ++nt) acco[nt][0] = acco[nt][1] = acco[nt][2] = acco[nt][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    if (ks <= warp) {
#pragma unroll
      for (int nt = 0; nt < V / 8; ++nt) {
        const int vr = 32 * (nt >> 2) + 8 * (g >> 1) + 2 * (nt & 3) + (g & 1);
        const uint32_t w = *reinterpret_cast<const uint32_t*>(s_v + swz_v(vr, ks) + 4 * j);
        uint32_t h01, h23;
        s8x4_to_h2x2(w, h01, h23);
        mma_f16(acco[nt], P[ks][0], P[ks][1], P[ks][2], P[ks][3], h01, h23);
      }
    }
  }

  // ---- canonical storage: the local product (rotated value basis) is scaled, rounded to fp16 and multiplied by the
  // un-rotation on the tensor cores (zoo/simple_gla.py:150-153). The accumulator pairs of two n-tiles are the A
  // fragment of one k16 step; gathering the rows of M^T with the same channel permutation as the value codes makes
  // the result come out in the column order the combine below expects.
  if (UNROT) {
    uint32_t A[V / 16][4];
#pragma unroll
    for (int kk = 0; kk < V / 16; ++kk) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int nt = 2 * kk + hh;
        const int cb = 32 * (nt >> 2) + 8 * j + 2 * (nt & 3);
        const float s0 = s_svl[cb], s1 = s_svl[cb + 1];
        A[kk][2 * hh] = Act<__half>::pack2(__fmul_rn(acco[nt][0], s0), __fmul_rn(acco[nt][1], s1));
        A[kk][2 * hh + 1] = Act<__half>::pack2(__fmul_rn(acco[nt][2], s0), __fmul_rn(acco[nt][3], s1));
      }
    }
#pragma unroll
    for (int nt2 = 0; nt2 < V / 8; ++nt2) {
      const int vr = 32 * (nt2 >> 2) + 8 * (g >> 1) + 2 * (nt2 & 3) + (g & 1);
      const __half* row = s_rt + vr * LDR;
      float u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < V / 16; ++kk) {
        const int c0 = 32 * ((2 * kk) >> 2) + 8 * j + 2 * ((2 * kk) & 3);
        const int c1 = 32 * ((2 * kk + 1) >> 2) + 8 * j + 2 * ((2 * kk + 1) & 3);
        mma_f16(u, A[kk][0], A[kk][1], A[kk][2], A[kk][3], *reinterpret_cast<const uint32_t*>(row + c0),
                *reinterpret_cast<const uint32_t*>(row + c1));
      }
      acco[nt2][0] = u[0]; acco[nt2][1] = u[1]; acco[nt2][2] = u[2]; acco[nt2][3] = u[3];
    }
  }

  // ---- S1 against the stored state, combine, store
  const float ega = DIAG ? 1.f : __expf(gia), egb = DIAG ? 1.f : __expf(gib);
  OT* op = reinterpret_cast<OT*>(a.o);
  const size_t rowa = (((size_t)b * a.T + (size_t)c * C + ia) * a.H + h) * V;
  const size_t rowb = (((size_t)b * a.T + (size_t)c * C + ib) * a.H + h) * V;
#pragma unroll
  for (int ng = 0; ng < V / 32; ++ng) {
    float outa[8], outb[8];
#pragma unroll
    for (int n4 = 0; n4 < 4; ++n4) {
      const int nt = 4 * ng + n4;
      const int vr = 8 * nt + g;  // row n of the stored-state tile is MMA column n
      int acc[4] = {0, 0, 0, 0};
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
        const uint4 bs = *reinterpret_cast<const uint4*>(s_h + swz_k<K>(vr, 4 * kk + j));
        mma_s8(acc, qa[kk].x, qb[kk].x, qa[kk].y, qb[kk].y, bs.x, bs.y);
        mma_s8(acc, qa[kk].z, qb[kk].z, qa[kk].w, qb[kk].w, bs.z, bs.w);
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int vc = 32 * ng + 8 * j + 2 * n4 + e;
        const float ss = s_ss[vc], svl = s_svl[vc];
        const float ra = __fmul_rn(__fmul_rn(__fmul_rn((float)acc[e], sq), ss), ega);
        const float rb = __fmul_rn(__fmul_rn(__fmul_rn((float)acc[2 + e], sq), ss), egb);
        outa[2 * n4 + e] = UNROT ? __fadd_rn(acco[nt][e], ra) : fmaf(acco[nt][e], svl, ra);
        outb[2 * n4 + e] = UNROT ? __fadd_rn(acco[nt][2 + e], rb) : fmaf(acco[nt][2 + e], svl, rb);
      }
    }
    store8<OT>(op + rowa + 32 * ng + 8 * j, outa);
    store8<OT>(op + rowb + 32 * ng + 8 * j, outb);
  }
}

template <int K, int V>
static int launch_output(const lq_zoo_problem* p, const OutputArgs& a, cudaStream_t st) {
  dim3 grid(a.NT, p->B * p->H), block(128);
  const bool diag = p->decay == LQ_DECAY_DIAGONAL, unrot = a.unrot_t != nullptr;
  const size_t smem = (size_t)64 * K * 2 + (size_t)V * K + (size_t)V * 64 + sizeof(float) * (64 + 2 * V) +
                      (unrot ? sizeof(__half) * (size_t)V * (V + 8) : 0);
#define LQ_LAUNCH_ONE(OT_, DIAG_, UNROT_)                                                                              \
  do {                                                                                                                 \
    auto kern = zoo_output_scalar_kernel<K, V, OT_, DIAG_, UNROT_>;                                                    \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
    kern<<<grid, block, smem, st>>>(a);                                                                                \
  } while (0)
#define LQ_LAUNCH_OUT(OT_)                                 \
  if (diag && unrot) LQ_LAUNCH_ONE(OT_, true, true);       \
  else if (diag) LQ_LAUNCH_ONE(OT_, true, false);          \
  else if (unrot) LQ_LAUNCH_ONE(OT_, false, true);         \
  else LQ_LAUNCH_ONE(OT_, false, false)
  if (p->out_dtype == LQ_F16) { LQ_LAUNCH_OUT(__half); }
  else if (p->out_dtype == LQ_BF16) { LQ_LAUNCH_OUT(__nv_bfloat16); }
  else if (p->out_dtype == LQ_F32) { LQ_LAUNCH_OUT(float); }
  else return fail(LQ_ERR_UNSUPPORTED, "output: out dtype must be f16, bf16 or f32");
#undef LQ_LAUNCH_OUT
#undef LQ_LAUNCH_ONE
  return check_launch("zoo_output_scalar_kernel");
}

int validate_zoo_problem(const lq_zoo_problem* p, bool delta, bool diagonal);

// k_local codes and local value codes/scales are parameters so the delta family can pass (Hw, E) tiles.
int run_output_tc(const lq_zoo_problem* p, const lq_zoo_workspace* ws, const float* s_local_value, cudaStream_t st);

int run_output_scalar(const lq_zoo_problem* p, const lq_zoo_workspace* ws, const float* s_local_value,
                      cudaStream_t st) {
  // K = 128 with none / scalar decay runs on the tcgen05 + TMA kernel; other shapes and the diagonal-decay variant
  // (A precomputed, no q.k^T product) on the warp-level MMA kernel below
  if (p->K == 128 && p->decay != LQ_DECAY_DIAGONAL && ws->status != nullptr && p->unrot_t == nullptr)
    return run_output_tc(p, ws, s_local_value, st);
  OutputArgs a;
  a.qq = ws->qq; a.kl = ws->kl; a.vlT = ws->vlT; a.hT = ws->hT; a.gc = ws->gc;
  a.sq = p->sq; a.sk = p->sk; a.svl = s_local_value; a.ss = p->sstate; a.o = p->o;
  a.amat = reinterpret_cast<const __half*>(ws->amat);
  a.unrot_t = reinterpret_cast<const __half*>(p->unrot_t);
  a.T = p->T; a.H = p->H; a.NT = p->T / p->chunk;
  if (p->K == 64 && p->V == 64) return launch_output<64, 64>(p, a, st);
  if (p->K == 64 && p->V == 128) return launch_output<64, 128>(p, a, st);
  if (p->K == 128 && p->V == 64) return launch_output<128, 64>(p, a, st);
  if (p->K == 128 && p->V == 128) return launch_output<128, 128>(p, a, st);
  return fail(LQ_ERR_UNSUPPORTED, "output: K and V must be 64 or 128");
}

}  // namespace lq

extern "C" int lq_zoo_output_scalar(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream) {
  if (int e = lq::validate_zoo_problem(p, p && p->beta != nullptr, p && p->decay == LQ_DECAY_DIAGONAL)) return e;
  if (!ws) return lq::fail(LQ_ERR_NULL, "output: workspace descriptor is null");
  return lq::run_output_scalar(p, ws, p->beta != nullptr ? p->sel : p->svl, (cudaStream_t)stream);  // delta family: E scales
}
