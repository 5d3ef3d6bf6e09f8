// Mamba-2 C.B^T per chunk on the Blackwell tensor cores (d_state 128, chunk 128 or 256).
//
//   cb[m, n] = clamp( rint( int32(C_q[m, :] . B_q[n, :]) * (s_C s_B / S_cb) ), +-127 )          (mamba2/bmm_chunk.py:103-139)
//
// One CTA per (chunk, group, batch), 256 threads. Both INT8 tiles [chunk tokens x 128 states] come by TMA exactly as
// q_C and q_B lie in memory (state index contiguous: K-major for both operands, 128-byte rows, 128-byte swizzle);
// tcgen05.mma.kind::i8 with M = 128 rows of C per instruction, N = the chunk's tokens of B, four steps of 32 states,
// accumulates the whole chunk x chunk tile in tensor memory (512 columns at chunk 256); every thread then requantises
// half a row at a time and writes its codes as 16-byte pieces of the row-major cb tile. On the key side B arrives
// unquantised (fp16 / bf16): the threads quantise its rows, rint(b / s_B) clamped to +-127, straight into the same
// swizzled tile the TMA load would have filled.
// Every wait is bounded; on expiry the CTA raises the status word, stores nothing and still frees its tensor memory.
#include "lq_tc.cuh"

namespace lq {

namespace bmmtc {
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ int code_rint127(float y) { return __float2int_rn(fminf(fmaxf(y, -127.f), 127.f)); }
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.u32 [%0], {%1,%2};\n" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
}  // namespace bmmtc

template <typename T, int C, bool B_IS_FP>
__global__ void __launch_bounds__(256, 1) ssd_bmm_tc_kernel(const __grid_constant__ CUtensorMap tm_c,
                                                           const __grid_constant__ CUtensorMap tm_b, lq_ssd_problem p, int* status) {
  using namespace bmmtc;
  constexpr int N = 128, MB = C / 128, COLS = C * MB;  // accumulator columns: one [128 x C] block per 128 rows of C_q
  const int NC = p.L / C;
  extern __shared__ uint8_t smem_dyn[];
  const uint32_t s_A = (smem_u32(smem_dyn) + 1023u) & ~1023u;  // q_C tile [C][128] INT8, SW128
  const uint32_t s_B = s_A + C * 128;                          // q_B tile [C][128] INT8, SW128
  const uint32_t s_bars = s_B + C * 128;                       // [0] tiles landed, [1] accumulator complete
  const uint32_t s_tbase = s_bars + 16;
  const int c = blockIdx.x / p.G, grp = blockIdx.x % p.G, b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_in = s_bars, bar_mma = s_bars + 8;

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_in));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_mma));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar_in), "r"((uint32_t)((B_IS_FP ? 1 : 2) * C * 128))
                 : "memory");
    tma_load_2d(s_A, &tm_c, grp * N, b * p.L + c * C, bar_in);
    if (!B_IS_FP) tma_load_2d(s_B, &tm_b, grp * N, b * p.L + c * C, bar_in);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s_tbase), "r"((uint32_t)COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  const float inv_scb = __fmul_rn(p.C_scale[grp], p.B_scale[grp]) / p.cb_scale[grp];
  if (B_IS_FP) {  // row = token, 16-byte piece j of the 128-byte row at (j ^ (token & 7)); a thread's eight codes are half a piece
    const float b_inv = 1.0f / p.B_scale[grp];
    const int oct = lane & 15, trow = lane >> 4;
    const T* bp = reinterpret_cast<const T*>(p.b_fp) + (((size_t)b * p.L + (size_t)c * C + 2 * warp + trow) * p.G + grp) * N + 8 * oct;
    const size_t bstep = (size_t)16 * p.G * N;
    constexpr int ITERS = C / 16, UNROLL = 8;
#pragma unroll
    for (int i0 = 0; i0 < ITERS; i0 += UNROLL) {
      uint4 raw[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) raw[u] = __ldg(reinterpret_cast<const uint4*>(bp + (size_t)(i0 + u) * bstep));
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int t = 16 * (i0 + u) + 2 * warp + trow;
        float v[8];
        int cd[8];
        Act<T>::unpack8(raw[u], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) cd[i] = code_rint127(__fmul_rn(v[i], b_inv));
        sts64(s_B + t * 128 + ((((oct >> 1)) ^ (t & 7)) << 4) + 8 * (oct & 1), pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]));
      }
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic-proxy writes -> visible to the tensor core
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tbase = lds_u32(s_tbase);

  bool ok = true;
  if (tid == 0) {
    ok = mbar_wait_bounded(bar_in, 0);
    if (ok) {
      const uint32_t idesc = idesc_i8(128, C);
      const uint64_t db = desc_kmajor_sw128(s_B);
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        const uint64_t da = desc_kmajor_sw128(s_A + mb * 16384);
#pragma unroll
        for (int ks = 0; ks < N / 32; ++ks) umma_i8(tbase + mb * C, da + 2 * ks, db + 2 * ks, idesc, ks > 0);
      }
      umma_commit(bar_mma);
      ok = mbar_wait_bounded(bar_mma, 0);
    }
  }
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");

  if (ok) {
    // warp w reads the tensor-memory lanes 32 (w & 3) ..; the two warps of a lane quadrant take half of the columns each
    const int q4 = warp & 3, half = warp >> 2;
    int8_t* out = p.cb + (((size_t)b * NC + c) * p.G + grp) * (size_t)C * C;
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      const int row = 128 * mb + 32 * q4 + lane;
      const uint32_t taddr = tbase + ((uint32_t)(32 * q4) << 16) + mb * C + half * (C / 2);
      uint4* orow = reinterpret_cast<uint4*>(out + (size_t)row * C + half * (C / 2));
#pragma unroll 2
      for (int ch = 0; ch < C / 32; ++ch) {
        uint32_t r[16];
        tmem_ld16(taddr + 16 * ch, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        int cd[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) cd[e] = code_rint127(__fmul_rn((float)(int)r[e], inv_scb));
        orow[ch] = make_uint4(pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]), pack4(cd[8], cd[9], cd[10], cd[11]),
                              pack4(cd[12], cd[13], cd[14], cd[15]));
      }
    }
  } else if (tid == 0 && status != nullptr) {
    atomicExch(status, 1);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tbase), "r"((uint32_t)COLS) : "memory");
}

// ------------------------------------------------------------------------------------------------ host side
static int encode_codes(CUtensorMap* m, const void* base, size_t row_bytes, size_t rows, int box_rows, const char* what) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(LQ_ERR_LAUNCH, "%s: the driver does not export cuTensorMapEncodeTiled", what);
  const cuuint64_t gdim[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LQ_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, (int)r);
  return LQ_OK;
}

template <typename T, int C, bool B_IS_FP>
static int launch_bmm_tc(const lq_ssd_problem* p, const CUtensorMap& tc, const CUtensorMap& tb, int* status, cudaStream_t st) {
  const size_t smem = (size_t)2 * C * 128 + 16 + 16 + 1024;
  cudaError_t e = cudaFuncSetAttribute(ssd_bmm_tc_kernel<T, C, B_IS_FP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "bmm_chunk: shared memory opt-in failed: %s", cudaGetErrorString(e));
  dim3 grid((p->L / C) * p->G, p->B);
  ssd_bmm_tc_kernel<T, C, B_IS_FP><<<grid, 256, smem, st>>>(tc, tb, *p, status);
  return check_launch("ssd_bmm_tc_kernel");
}

// d_state 128, chunk 128 or 256, 16-byte aligned operands; B as INT8 codes or (b_is_fp) as fp16 / bf16 values
bool bmm_tc_applies(const lq_ssd_problem* p, bool b_is_fp) {
  const void* bsrc = b_is_fp ? p->b_fp : static_cast<const void*>(p->q_B);
  return p->N == 128 && (p->chunk == 128 || p->chunk == 256) && bsrc != nullptr && !(reinterpret_cast<uintptr_t>(bsrc) & 15u) &&
         !(reinterpret_cast<uintptr_t>(p->q_C) & 15u) && !(reinterpret_cast<uintptr_t>(p->cb) & 15u);
}
int run_bmm_tc(const lq_ssd_problem* p, bool b_is_fp, int* status, cudaStream_t st) {
  CUtensorMap tc, tb;
  if (int e = encode_codes(&tc, p->q_C, (size_t)p->G * 128, (size_t)p->B * p->L, p->chunk, "bmm_chunk (q_C)")) return e;
  if (!b_is_fp) {
    if (int e = encode_codes(&tb, p->q_B, (size_t)p->G * 128, (size_t)p->B * p->L, p->chunk, "bmm_chunk (q_B)")) return e;
    return p->chunk == 256 ? launch_bmm_tc<__half, 256, false>(p, tc, tb, status, st) : launch_bmm_tc<__half, 128, false>(p, tc, tb, status, st);
  }
  tb = tc;  // not read
  if (p->x_dtype == LQ_F16)
    return p->chunk == 256 ? launch_bmm_tc<__half, 256, true>(p, tc, tb, status, st) : launch_bmm_tc<__half, 128, true>(p, tc, tb, status, st);
  return p->chunk == 256 ? launch_bmm_tc<__nv_bfloat16, 256, true>(p, tc, tb, status, st)
                         : launch_bmm_tc<__nv_bfloat16, 128, true>(p, tc, tb, status, st);
}

}  // namespace lq
