// Intra-chunk output kernel, Blackwell tensor-core version (K = 128, none / scalar decay; linear and delta families).
//
// One CTA per (chunk, batch*head), 128 threads:
//   * one elected thread loads the three INT8 operand tiles with TMA (cp.async.bulk.tensor, 128-byte swizzle) straight
//     into the K-major shared-memory layout tcgen05 reads: q codes [64,128], k_local codes [64,128], stored state [V,128];
//   * the same thread issues the two INT8 contractions as tcgen05.mma.kind::i8 (M = 64, 4 k-steps of 32 each):
//        S2 = qq . kl^T  -> TMEM columns [0, 64)        S1 = qq . hT^T  -> TMEM columns [64, 64 + V)
//     and commits each to its own mbarrier, so the epilogue of S2 overlaps the S1 product;
//   * with M = 64 the accumulator rows 16w .. 16w+15 sit in the first 16 lanes of warp w's TMEM quadrant; every warp
//     reads them with tcgen05.ld.16x256b, which hands each thread the (row g / g+8, column 2j / 2j+1) fragment of a
//     warp-level MMA. The decay-masked P therefore feeds the fp16 A.v product (mma.sync on the value codes, staged by
//     cp.async) directly from registers, exactly as in the mma.sync version of this kernel.
// Every wait on an mbarrier is bounded; on expiry the CTA raises the status word, skips its stores and still frees TMEM.
// Arithmetic and references: see lq_zoo_output.cu.
#include "lq_tc.cuh"

namespace lq {

struct OutputTcArgs {
  const int8_t* vlT;
  const float *gc, *sq, *sk, *svl, *ss;
  void* o;
  int* status;
  int T, H, NT;
};

template <typename OT>
__device__ __forceinline__ void store8_tc(OT* dst, const float (&x)[8]);
template <>
__device__ __forceinline__ void store8_tc<float>(float* dst, const float (&x)[8]) {
  reinterpret_cast<float4*>(dst)[0] = make_float4(x[0], x[1], x[2], x[3]);
  reinterpret_cast<float4*>(dst)[1] = make_float4(x[4], x[5], x[6], x[7]);
}
template <>
__device__ __forceinline__ void store8_tc<__half>(__half* dst, const float (&x)[8]) {
  *reinterpret_cast<uint4*>(dst) = make_uint4(Act<__half>::pack2(x[0], x[1]), Act<__half>::pack2(x[2], x[3]),
                                              Act<__half>::pack2(x[4], x[5]), Act<__half>::pack2(x[6], x[7]));
}
template <>
__device__ __forceinline__ void store8_tc<__nv_bfloat16>(__nv_bfloat16* dst, const float (&x)[8]) {
  *reinterpret_cast<uint4*>(dst) =
      make_uint4(Act<__nv_bfloat16>::pack2(x[0], x[1]), Act<__nv_bfloat16>::pack2(x[2], x[3]),
                 Act<__nv_bfloat16>::pack2(x[4], x[5]), Act<__nv_bfloat16>::pack2(x[6], x[7]));
}

__device__ __forceinline__ int swz_v_tc(int row, int chunk) { return row * 64 + ((chunk ^ ((row >> 3) & 3)) << 4); }

template <int V, typename OT>
__global__ void __launch_bounds__(128) zoo_output_tc_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                            const __grid_constant__ CUtensorMap tm_k,
                                                            const __grid_constant__ CUtensorMap tm_h, OutputTcArgs a) {
  constexpr int C = 64, K = 128;
  constexpr uint32_t TMEM_COLS = 128;  // S2 in [0,64), first 64 state columns in [64,128); the second 64 reuse [0,64)
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;                 // [64][128]  TMA, 128B swizzle
  uint8_t* s_k = s_q + C * K;          // [64][128]
  uint8_t* s_h = s_k + C * K;          // [V][128]
  uint8_t* s_v = s_h + V * K;          // [V][64]    cp.async, 16-byte pieces XOR-swizzled for the 32-bit fragment loads
  float* s_gc = reinterpret_cast<float*>(s_v + V * C);
  float* s_ss = s_gc + C;
  float* s_svl = s_ss + V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_svl + V);  // [0] operands landed, [1] S2, [2] S1 first half, [3] second half
  uint32_t* s_tbase = reinterpret_cast<uint32_t*>(bars + 4);

  const int c = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;
  const size_t tile = (size_t)bh * a.NT + c;
  const uint32_t bar_ld = smem_u32(&bars[0]), bar_s2 = smem_u32(&bars[1]), bar_s1 = smem_u32(&bars[2]), bar_s1b = smem_u32(&bars[3]);

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_ld));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_s2));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_s1));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_s1b));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar_ld), "r"((uint32_t)(2 * C * K + V * K)) : "memory");
    tma_load_2d(smem_u32(s_q), &tm_q, 0, (int)(tile * C), bar_ld);
    tma_load_2d(smem_u32(s_k), &tm_k, 0, (int)(tile * C), bar_ld);
    tma_load_2d(smem_u32(s_h), &tm_h, 0, (int)(tile * V), bar_ld);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(s_tbase)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  {
    const int8_t* gv = a.vlT + tile * (size_t)(V * C);
    for (int i = tid; i < V * 4; i += 128) cp_async16(s_v + swz_v_tc(i >> 2, i & 3), gv + (size_t)i * 16);
    cp_async_commit();
    if (tid < C) s_gc[tid] = a.gc[tile * C + tid];
    for (int i = tid; i < V; i += 128) {
      s_ss[i] = a.ss[h * V + i];
      s_svl[i] = a.svl[h * V + i];
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tbase = *s_tbase;

  bool ok = true;
  if (tid == 0) {
    ok = mbar_wait_bounded(bar_ld, 0);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t idesc_s2 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(C >> 3) << 17) | ((uint32_t)(64 >> 4) << 24);
      const uint32_t idesc_s1 = idesc_s2;  // the state product runs in halves of 64 value channels
      const uint64_t dq = desc_kmajor_sw128(smem_u32(s_q)), dk = desc_kmajor_sw128(smem_u32(s_k)), dh = desc_kmajor_sw128(smem_u32(s_h));
#pragma unroll
      for (int ks = 0; ks < K / 32; ++ks) umma_i8(tbase, dq + 2 * ks, dk + 2 * ks, idesc_s2, ks > 0);
      umma_commit(bar_s2);
#pragma unroll
      for (int ks = 0; ks < K / 32; ++ks) umma_i8(tbase + 64, dq + 2 * ks, dh + 2 * ks, idesc_s1, ks > 0);
      umma_commit(bar_s1);
    } else {
      atomicExch(a.status, 1);
      // release the waiters: nothing was issued, so arrive on both accumulator barriers by hand
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar_s2) : "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar_s1) : "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar_s1b) : "memory");
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  ok = __syncthreads_and(ok ? 1 : 0) != 0;

  const float sq = a.sq[h], sk = a.sk[h];
  const float sqk = __fmul_rn(sq, sk);
  const int ia = warp * 16 + g, ib = ia + 8;
  const float gia = s_gc[ia], gib = s_gc[ib];
  const uint32_t tq = tbase + ((uint32_t)(32 * warp) << 16);  // this warp's TMEM quadrant

  // ---- S2 -> P (fp16 A fragments). S2 column n is row n of the k_local tile = token 16*(n/16) + 4j + 2*half + e
  // for n = 16ks + 8*half + 2j + e.
  uint32_t P[4][4];
  if (tid == 0 && ok) ok = mbar_wait_bounded(bar_s2, 0);  // one poller per barrier; the block barrier releases the rest
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    P[ks][0] = P[ks][1] = P[ks][2] = P[ks][3] = 0u;
    if (ok && ks <= warp) {
      uint32_t r[8];
      tmem_ld_16x256b_x2(tq + 16 * ks, r);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float pa[2], pb[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tj = 16 * ks + 4 * j + 2 * half + e;
          const float gj = s_gc[tj];
          pa[e] = (ia >= tj) ? __fmul_rn((float)(int)r[4 * half + e], sqk) * __expf(gia - gj) : 0.f;
          pb[e] = (ib >= tj) ? __fmul_rn((float)(int)r[4 * half + 2 + e], sqk) * __expf(gib - gj) : 0.f;
        }
        P[ks][2 * half + 0] = Act<__half>::pack2(pa[0], pa[1]);
        P[ks][2 * half + 1] = Act<__half>::pack2(pb[0], pb[1]);
      }
    }
  }

  if (V == 128) {  // S2 has been read by every warp: its columns now take the second half of the state product
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      if (ok) {
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(64 >> 4) << 24);
        const uint64_t dq = desc_kmajor_sw128(smem_u32(s_q)), dh = desc_kmajor_sw128(smem_u32(s_h + 64 * K));
#pragma unroll
        for (int ks = 0; ks < K / 32; ++ks) umma_i8(tbase, dq + 2 * ks, dh + 2 * ks, idesc, ks > 0);
        umma_commit(bar_s1b);
      } else {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar_s1b) : "memory");
      }
    }
  }

  // ---- O2 = P . vl on the warp-level fp16 MMA. Column (nt, cn) is value channel 32*(nt/4) + 8*(cn/2) + 2*(nt%4) + (cn%2).
  float acco[V / 8][4];
#pragma unroll
  for (int nt = 0; nt < V / 8; ++nt) acco[nt][0] = acco[nt][1] = acco[nt][2] = acco[nt][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    if (ks <= warp) {
#pragma unroll
      for (int nt = 0; nt < V / 8; ++nt) {
        const int vr = 32 * (nt >> 2) + 8 * (g >> 1) + 2 * (nt & 3) + (g & 1);
        const uint32_t w = *reinterpret_cast<const uint32_t*>(s_v + swz_v_tc(vr, ks) + 4 * j);
        uint32_t h01, h23;
        s8x4_to_h2x2(w, h01, h23);
        mma_f16(acco[nt], P[ks][0], P[ks][1], P[ks][2], P[ks][3], h01, h23);
      }
    }
  }

  // ---- S1 from TMEM, combine, store. S1 column n is row n of the state tile = channel 32*(n/32) + 8j + 2*n4 + e.
  if (tid == 0 && ok) ok = mbar_wait_bounded(bar_s1, 0);
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  if (ok) {
    const float ega = __expf(gia), egb = __expf(gib);
    OT* op = reinterpret_cast<OT*>(a.o);
    const size_t rowa = (((size_t)b * a.T + (size_t)c * C + ia) * a.H + h) * V;
    const size_t rowb = (((size_t)b * a.T + (size_t)c * C + ib) * a.H + h) * V;
#pragma unroll
    for (int ng = 0; ng < V / 32; ++ng) {
      if (ng == 2) {  // second half of the value channels (V = 128 only)
        if (!mbar_wait_bounded(bar_s1b, 0)) {
          atomicExch(a.status, 1);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      }
      uint32_t r[16];
      tmem_ld_16x256b_x4(ng < 2 ? tq + 64 + 32 * ng : tq + 32 * (ng - 2), r);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      float outa[8], outb[8];
#pragma unroll
      for (int n4 = 0; n4 < 4; ++n4) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int vc = 32 * ng + 8 * j + 2 * n4 + e;
          const float ss = s_ss[vc], svl = s_svl[vc];
          const float ra = __fmul_rn(__fmul_rn(__fmul_rn((float)(int)r[4 * n4 + e], sq), ss), ega);
          const float rb = __fmul_rn(__fmul_rn(__fmul_rn((float)(int)r[4 * n4 + 2 + e], sq), ss), egb);
          outa[2 * n4 + e] = fmaf(acco[4 * ng + n4][e], svl, ra);
          outb[2 * n4 + e] = fmaf(acco[4 * ng + n4][2 + e], svl, rb);
        }
      }
      store8_tc<OT>(op + rowa + 32 * ng + 8 * j, outa);
      store8_tc<OT>(op + rowb + 32 * ng + 8 * j, outb);
    }
  } else if (tid == 0) {
    atomicExch(a.status, 1);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tbase), "r"(TMEM_COLS) : "memory");
}


// ------------------------------------------------------------------------------------------------ host side
// 2-D map over an INT8 matrix [rows][128] (row = 128 bytes), box = [box_rows][128], 128-byte swizzle
static int make_map(CUtensorMap* m, const void* base, size_t rows, int box_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(LQ_ERR_LAUNCH, "output: the driver does not export cuTensorMapEncodeTiled");
  const cuuint64_t gdim[2] = {128, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {128};
  const cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LQ_ERR_LAUNCH, "output: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return LQ_OK;
}

template <int V>
static int launch_output_tc(const lq_zoo_problem* p, const lq_zoo_workspace* ws, const OutputTcArgs& a, cudaStream_t st) {
  const size_t tiles = (size_t)p->B * p->H * a.NT;
  CUtensorMap tq, tk, th;
  if (int e = make_map(&tq, ws->qq, tiles * 64, 64)) return e;
  if (int e = make_map(&tk, ws->kl, tiles * 64, 64)) return e;
  if (int e = make_map(&th, ws->hT, tiles * V, V)) return e;
  const size_t smem = (size_t)2 * 64 * 128 + (size_t)V * 128 + (size_t)V * 64 + sizeof(float) * (64 + 2 * V) + 64 + 1024;  // + barriers, TMEM base, 1 KiB alignment slack
  dim3 grid(a.NT, p->B * p->H), block(128);
  if (p->out_dtype == LQ_F16) zoo_output_tc_kernel<V, __half><<<grid, block, smem, st>>>(tq, tk, th, a);
  else if (p->out_dtype == LQ_BF16) zoo_output_tc_kernel<V, __nv_bfloat16><<<grid, block, smem, st>>>(tq, tk, th, a);
  else if (p->out_dtype == LQ_F32) zoo_output_tc_kernel<V, float><<<grid, block, smem, st>>>(tq, tk, th, a);
  else return fail(LQ_ERR_UNSUPPORTED, "output: out dtype must be f16, bf16 or f32");
  return check_launch("zoo_output_tc_kernel");
}

// K = 128, none / scalar decay. s_local_value: v_local (linear family) or e_local (delta family) scales.
int run_output_tc(const lq_zoo_problem* p, const lq_zoo_workspace* ws, const float* s_local_value, cudaStream_t st) {
  OutputTcArgs a;
  a.vlT = ws->vlT; a.gc = ws->gc; a.sq = p->sq; a.sk = p->sk; a.svl = s_local_value; a.ss = p->sstate; a.o = p->o;
  a.status = p->status != nullptr ? p->status : ws->status; a.T = p->T; a.H = p->H; a.NT = p->T / p->chunk;
  if (p->V == 128) return launch_output_tc<128>(p, ws, a, st);
  if (p->V == 64) return launch_output_tc<64>(p, ws, a, st);
  return fail(LQ_ERR_UNSUPPORTED, "output: V must be 64 or 128");
}

}  // namespace lq
