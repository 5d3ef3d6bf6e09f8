// Value-side Mamba-2 chunk state on the Blackwell tensor cores, both operands in their natural layouts (headdim 64,
// d_state 128, chunk 128 or 256, an even number of heads per group).
//
//   states[p, n] = half_away( (sum_t xq[t, p] * qB[t, n]) * (alpha_p / S_p) * s_B ),   xq = half_away((x / alpha_p) * gate_t)
//   (mamba2/chunk_state.py:186-246)
//
// One CTA per (chunk, pair of heads, batch), 256 threads, three CTAs per SM:
//   * the INT8 B tile [C tokens x 128 states] comes by TMA exactly as q_B lies in memory (state index contiguous);
//   * the x rows of the two heads (256 contiguous bytes per token) are read with 16-byte loads, quantised in fp32 (per-
//     channel reciprocal scale, per-token gate, half away from zero, clamp) and stored as the INT8 A tile [C tokens x 128
//     channels] with the channel index contiguous: both operands are "MN-major" for tcgen05, so neither is transposed and
//     no transposed copy of q_B is needed;
//   * tcgen05.mma.kind::i8 (M = 128 channels of the two heads, N = 128 states, 32 tokens per instruction) accumulates into
//     tensor memory; every thread then requantises half a row of the accumulator and the two INT8 state tiles leave by
//     TMA stores.
// Every wait is bounded; on expiry the CTA raises the status word, skips its stores and still frees its tensor memory.
#include <type_traits>

#include "lq_tc.cuh"

namespace lq {

namespace statetc2 {
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.u32 [%0], {%1,%2};\n" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ float lds_f(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src),
               "r"(c0), "r"(c1)
               : "memory");
}
// half away from zero on the +-127 grid: the lower clamp here, the upper one in the saturating pack of the caller
__device__ __forceinline__ int code_lower127(float y) {
  y = fmaxf(y, -127.f);
  return __float2int_rz(__fadd_rn(y, copysignf(0.5f, y)));
}
}  // namespace statetc2

template <typename T, int C>
__global__ void __launch_bounds__(256, 3) ssd_chunk_state_tc2_kernel(const __grid_constant__ CUtensorMap tm_b,
                                                                    const __grid_constant__ CUtensorMap tm_out, lq_ssd_problem p,
                                                                    int* status) {
  using namespace statetc2;
  constexpr int P = 64, N = 128;
  const int NC = p.L / C;
  extern __shared__ uint8_t smem_dyn[];
  const uint32_t s_A = (smem_u32(smem_dyn) + 1023u) & ~1023u;  // [C tokens][128 channels] INT8, SW128; later the output tiles
  const uint32_t s_B = s_A + C * 128;                          // [C tokens][128 states] INT8 by TMA, SW128
  const uint32_t s_gate = s_B + C * 128;                       // f32 [2][C]
  const uint32_t s_bars = s_gate + 2 * C * 4;                  // [0] B landed, [1] accumulator complete
  const uint32_t s_tbase = s_bars + 16;

  const int c = blockIdx.x, h0 = 2 * blockIdx.y, b = blockIdx.z;
  const int grp = h0 / (p.H / p.G);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_b = s_bars, bar_mma = s_bars + 8;

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_b));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_mma));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar_b), "r"((uint32_t)(C * 128)) : "memory");
    tma_load_2d(s_B, &tm_b, grp * N, b * p.L + c * C, bar_b);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s_tbase), "r"(128u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  // ---- gates of the two heads: exp(dA_last - dA_t) * dt_t
  for (int i = tid; i < 2 * C; i += 256) {
    const int hh = i / C, t = i - hh * C;
    const size_t cbase = (((size_t)b * p.H + h0 + hh) * NC + c) * C;
    const float last = p.dA[cbase + C - 1];
    sts_u32(s_gate + 4 * i, __float_as_uint(__fmul_rn(expf(__fsub_rn(last, p.dA[cbase + t])), p.dt[cbase + t])));
  }
  // lane = (token parity, octet of the 128-channel row): per-thread reciprocal scales of its eight channels
  const int oct = lane & 15, trow = lane >> 4;
  const int hh = oct >> 3;
  float xinv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) xinv[i] = 1.0f / p.alpha_hp[(h0 + hh) * P + 8 * (oct & 7) + i];
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tbase = lds_u32(s_tbase);

  // ---- quantise x into the A tile: row = token, 16-byte piece j of the row at (j ^ (token & 7)); this thread's eight
  // codes are bytes 8 (oct & 1) .. of piece oct >> 1
  {
    const T* xp = reinterpret_cast<const T*>(p.x) + (size_t)b * p.x_stride_b + (size_t)(h0 + hh) * p.x_stride_h + 8 * (oct & 7) +
                  (size_t)(c * C + 2 * warp + trow) * p.x_stride_t;
    const uint32_t gate0 = s_gate + 4 * (hh * C + 2 * warp + trow);
    constexpr int ITERS = C / 16, UNROLL = 8;
#pragma unroll
    for (int i0 = 0; i0 < ITERS; i0 += UNROLL) {
      uint4 raw[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) raw[u] = __ldg(reinterpret_cast<const uint4*>(xp + (size_t)(16 * (i0 + u)) * p.x_stride_t));
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int t = 16 * (i0 + u) + 2 * warp + trow;
        const float gk = lds_f(gate0 + 64 * (i0 + u));
        float x[8];
        Act<T>::unpack8(raw[u], x);
        int cd[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) cd[i] = code_lower127(__fmul_rn(__fmul_rn(x[i], xinv[i]), gk));
        const uint32_t w0 = pack_sat_s8x2(cd[1], cd[0], pack_sat_s8x2(cd[3], cd[2], 0u));
        const uint32_t w1 = pack_sat_s8x2(cd[5], cd[4], pack_sat_s8x2(cd[7], cd[6], 0u));
        sts64(s_A + t * 128 + ((((oct >> 1)) ^ (t & 7)) << 4) + 8 * (oct & 1), w0, w1);
      }
    }
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic-proxy writes -> visible to the tensor core
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();

  bool ok = true;
  if (tid == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    ok = mbar_wait_bounded(bar_b, 0);
    if (ok) {
      // s8 x s8 -> s32, M = 128, N = 128, both operands MN-major (bits 15 and 16): rows of 128 bytes are tokens, eight
      // tokens per 1 KB swizzle group, 32 tokens (4 KB) per instruction
      const uint32_t idesc = idesc_i8(128, N) | (1u << 15) | (1u << 16);
      const uint64_t da = desc_kmajor_sw128(s_A), db = desc_kmajor_sw128(s_B);
#pragma unroll
      for (int ks = 0; ks < C / 32; ++ks) umma_i8(tbase, da + (uint64_t)(ks * (4096 >> 4)), db + (uint64_t)(ks * (4096 >> 4)), idesc, ks > 0);
      umma_commit(bar_mma);
      ok = mbar_wait_bounded(bar_mma, 0);
    }
  }
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");

  // ---- requantise: thread = (accumulator row = channel of one of the two heads, half of the 128 states)
  if (ok) {
    const int row = 32 * (warp & 3) + lane, half = warp >> 2;
    const int eh = row >> 6, pp = row & 63;
    const float bs = p.bscale_g[grp];
    const float ra = __fmul_rn(p.alpha_hp[(h0 + eh) * P + pp] / p.state_scale[(h0 + eh) * P + pp], bs);
    const uint32_t taddr = tbase + ((uint32_t)(32 * (warp & 3)) << 16) + 64 * half;
    // output tiles [head][64 channels][128 states] INT8 in the A region, SW128 rows of 128 bytes
    const uint32_t orow = s_A + eh * 8192 + pp * 128;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      uint32_t r[16];
      tmem_ld16(taddr + 16 * ch, r);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      int cd[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) cd[e] = code_lower127(__fmul_rn((float)(int)r[e], ra));
      uint4 o;
      o.x = pack_sat_s8x2(cd[1], cd[0], pack_sat_s8x2(cd[3], cd[2], 0u));
      o.y = pack_sat_s8x2(cd[5], cd[4], pack_sat_s8x2(cd[7], cd[6], 0u));
      o.z = pack_sat_s8x2(cd[9], cd[8], pack_sat_s8x2(cd[11], cd[10], 0u));
      o.w = pack_sat_s8x2(cd[13], cd[12], pack_sat_s8x2(cd[15], cd[14], 0u));
      sts128(orow + (((4 * half + ch) ^ (pp & 7)) << 4), o);
    }
  } else if (tid == 0 && status != nullptr) {
    atomicExch(status, 1);
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (tid == 0 && ok) {
    const int row0 = (int)((((size_t)b * NC + c) * p.H + h0) * P);
    tma_store_2d(&tm_out, s_A, 0, row0);
    tma_store_2d(&tm_out, s_A + 8192, 0, row0 + P);
    asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
  }
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tbase), "r"(128u) : "memory");
}

// ------------------------------------------------------------------------------------------------ host side
static int encode_u8_rows(CUtensorMap* m, const void* base, size_t row_bytes, size_t rows, int box_rows, const char* what) {
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

template <typename T, int C>
static int launch_state_tc2(const lq_ssd_problem* p, const CUtensorMap& tb, const CUtensorMap& to, int* status, cudaStream_t st) {
  const size_t smem = (size_t)2 * C * 128 + 2 * C * 4 + 16 + 16 + 1024;
  cudaError_t e = cudaFuncSetAttribute(ssd_chunk_state_tc2_kernel<T, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "chunk_state: shared memory opt-in failed: %s", cudaGetErrorString(e));
  dim3 grid(p->L / C, p->H / 2, p->B);
  ssd_chunk_state_tc2_kernel<T, C><<<grid, 256, smem, st>>>(tb, to, *p, status);
  return check_launch("ssd_chunk_state_tc2_kernel");
}

// value side, d_state 128, chunk 128 or 256, heads per group even: no transposed copy of q_B is read or written
bool chunk_state_value_tc2_applies(const lq_ssd_problem* p) {
  return p->N == 128 && (p->chunk == 128 || p->chunk == 256) && p->P == 64 && ((p->H / p->G) % 2 == 0) &&
         !(reinterpret_cast<uintptr_t>(p->q_B) & 15u) && !(reinterpret_cast<uintptr_t>(p->states) & 15u);
}
int run_chunk_state_value_tc2(const lq_ssd_problem* p, int* status, cudaStream_t st) {
  const int C = p->chunk, NC = p->L / C;
  CUtensorMap tb, to;
  if (int e = encode_u8_rows(&tb, p->q_B, (size_t)p->G * 128, (size_t)p->B * p->L, C, "chunk_state (q_B)")) return e;
  if (int e = encode_u8_rows(&to, p->states, 128, (size_t)p->B * NC * p->H * 64, 64, "chunk_state (states)")) return e;
  if (p->x_dtype == LQ_F16) return C == 256 ? launch_state_tc2<__half, 256>(p, tb, to, status, st) : launch_state_tc2<__half, 128>(p, tb, to, status, st);
  return C == 256 ? launch_state_tc2<__nv_bfloat16, 256>(p, tb, to, status, st) : launch_state_tc2<__nv_bfloat16, 128>(p, tb, to, status, st);
}

}  // namespace lq
