// Key-side Mamba-2 chunk state on the Blackwell tensor cores (headdim 64, d_state 128, chunk 128 or 256, an even number
// of heads per group).
//
//   states[p, n] = clamp( rint( (sum_t xq[t, p] * Bq[t, n]) * (bg_n / 127) * (xs_p / S_p) ), +-127 )
//   xq = clamp(rint(x / xs_p)),  Bq = clamp(rint(B[t, n] * gate_t * 127 / bg_n)),  gate_t = exp(dA_last - dA_t) dt_t
//   (mamba2/chunk_state_keyside.py:267-321)
//
// One CTA per (chunk, pair of heads, batch), 256 threads, two CTAs per SM. The gate-weighted B is quantised per head, so
// the two heads of the pair have their own INT8 B tiles; its floating-point rows are read once and quantised for both
// heads. The x rows of the two heads are quantised into one A tile [C tokens x 128 channels], as on the value side.
// All three tiles are written with the token index as the row: both operands are "MN-major" for tcgen05, nothing is
// transposed. Two tcgen05.mma.kind::i8 chains (M = 128 channels of both heads, N = 128 states, 32 tokens per
// instruction) accumulate A . B_h into two blocks of tensor memory; of block h only the rows of head h are used (the
// other half of the rows is the cross product of one head's x with the other head's B and is ignored: the tensor pipe
// is far from busy, a second operand layout would cost more). Every thread then requantises half a row and the two INT8
// state tiles leave by TMA stores.
// Every wait is bounded; on expiry the CTA raises the status word, skips its stores and still frees its tensor memory.
#include <type_traits>

#include "lq_tc.cuh"

namespace lq {

namespace statekey {
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
// round to nearest even on the +-127 grid
__device__ __forceinline__ int code_rint127(float y) { return __float2int_rn(fminf(fmaxf(y, -127.f), 127.f)); }
}  // namespace statekey

template <typename T, int C>
__global__ void __launch_bounds__(256, 2) ssd_chunk_state_key_tc_kernel(const __grid_constant__ CUtensorMap tm_out, lq_ssd_problem p,
                                                                       int* status) {
  using namespace statekey;
  constexpr int P = 64, N = 128;
  const int NC = p.L / C;
  extern __shared__ uint8_t smem_dyn[];
  const uint32_t s_A = (smem_u32(smem_dyn) + 1023u) & ~1023u;  // [C tokens][128 channels] INT8, SW128; later the output tiles
  const uint32_t s_B = s_A + C * 128;                          // [2 heads][C tokens][128 states] INT8, SW128
  const uint32_t s_gate = s_B + 2 * C * 128;                   // f32 [2][C]
  const uint32_t s_sn = s_gate + 2 * C * 4;                    // f32 [2][128] bg_n / 127 of the two heads
  const uint32_t s_bars = s_sn + 2 * N * 4;                    // [0] accumulators complete
  const uint32_t s_tbase = s_bars + 16;

  const int c = blockIdx.x, h0 = 2 * blockIdx.y, b = blockIdx.z;
  const int grp = h0 / (p.H / p.G);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_mma = s_bars;

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_mma));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s_tbase), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  // ---- gates of the two heads, exp(dA_last - dA_t) * dt_t, and the per-state scales of the gate-weighted B
  for (int i = tid; i < 2 * C; i += 256) {
    const int gh = i / C, t = i - gh * C;
    const size_t cbase = (((size_t)b * p.H + h0 + gh) * NC + c) * C;
    const float last = p.dA[cbase + C - 1];
    sts_u32(s_gate + 4 * i, __float_as_uint(__fmul_rn(expf(__fsub_rn(last, p.dA[cbase + t])), p.dt[cbase + t])));
  }
  {
    const int gh = tid >> 7, n = tid & 127;  // 256 threads: one (head, state) each
    const float bg = p.b_gate_scale[b * p.bgs_stride[0] + c * p.bgs_stride[1] + (h0 + gh) * p.bgs_stride[2] + n * p.bgs_stride[3]];
    sts_u32(s_sn + 4 * tid, __float_as_uint(bg / 127.0f));
  }
  // lane = (token parity, 16-byte piece of the 128-byte row): for x the piece is eight channels of head oct >> 3, for B
  // eight states
  const int oct = lane & 15, trow = lane >> 4;
  const int hh = oct >> 3;
  float xinv[8], binv[2][8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    xinv[i] = 1.0f / fmaxf(p.x_scale_hp[(h0 + hh) * P + 8 * (oct & 7) + i], 1e-10f);
#pragma unroll
    for (int gh = 0; gh < 2; ++gh)
      binv[gh][i] = 127.0f / p.b_gate_scale[b * p.bgs_stride[0] + c * p.bgs_stride[1] + (h0 + gh) * p.bgs_stride[2] +
                                            (8 * oct + i) * p.bgs_stride[3]];
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tbase = lds_u32(s_tbase);

  // ---- quantise x into the A tile and the gate-weighted B into the two B tiles: row = token, 16-byte piece j of the row
  // at (j ^ (token & 7)); this thread's eight codes are bytes 8 (oct & 1) .. of piece oct >> 1
  {
    const T* xp = reinterpret_cast<const T*>(p.x) + (size_t)b * p.x_stride_b + (size_t)(h0 + hh) * p.x_stride_h + 8 * (oct & 7) +
                  (size_t)(c * C + 2 * warp + trow) * p.x_stride_t;
    const T* bp = reinterpret_cast<const T*>(p.b_fp) + (((size_t)b * p.L + (size_t)c * C + 2 * warp + trow) * p.G + grp) * N + 8 * oct;
    const size_t bstep = (size_t)16 * p.G * N;
    constexpr int ITERS = C / 16, UNROLL = 4;
#pragma unroll
    for (int i0 = 0; i0 < ITERS; i0 += UNROLL) {
      uint4 rawx[UNROLL], rawb[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        rawx[u] = __ldg(reinterpret_cast<const uint4*>(xp + (size_t)(16 * (i0 + u)) * p.x_stride_t));
        rawb[u] = __ldg(reinterpret_cast<const uint4*>(bp + (size_t)(i0 + u) * bstep));
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int t = 16 * (i0 + u) + 2 * warp + trow;
        const uint32_t off = t * 128 + ((((oct >> 1)) ^ (t & 7)) << 4) + 8 * (oct & 1);
        float v[8];
        int cd[8];
        Act<T>::unpack8(rawx[u], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) cd[i] = code_rint127(__fmul_rn(v[i], xinv[i]));
        sts64(s_A + off, pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]));
        Act<T>::unpack8(rawb[u], v);
#pragma unroll
        for (int gh = 0; gh < 2; ++gh) {
          const float gk = lds_f(s_gate + 4 * (gh * C + t));
#pragma unroll
          for (int i = 0; i < 8; ++i) cd[i] = code_rint127(__fmul_rn(__fmul_rn(v[i], gk), binv[gh][i]));
          sts64(s_B + gh * (C * 128) + off, pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]));
        }
      }
    }
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic-proxy writes -> visible to the tensor core
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();

  bool ok = true;
  if (tid == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    // s8 x s8 -> s32, M = 128, N = 128, both operands MN-major (bits 15 and 16): rows of 128 bytes are tokens, eight
    // tokens per 1 KB swizzle group, 32 tokens (4 KB) per instruction
    const uint32_t idesc = idesc_i8(128, N) | (1u << 15) | (1u << 16);
    const uint64_t da = desc_kmajor_sw128(s_A);
#pragma unroll
    for (int gh = 0; gh < 2; ++gh) {
      const uint64_t db = desc_kmajor_sw128(s_B + gh * (C * 128));
#pragma unroll
      for (int ks = 0; ks < C / 32; ++ks)
        umma_i8(tbase + 128 * gh, da + (uint64_t)(ks * (4096 >> 4)), db + (uint64_t)(ks * (4096 >> 4)), idesc, ks > 0);
    }
    umma_commit(bar_mma);
    ok = mbar_wait_bounded(bar_mma, 0);
  }
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");

  // ---- requantise: thread = (accumulator row = channel of one of the two heads, half of the 128 states); the rows of
  // head eh are taken from accumulator block eh
  if (ok) {
    const int row = 32 * (warp & 3) + lane, half = warp >> 2;
    const int eh = row >> 6, pp = row & 63;
    const float ra = p.x_scale_hp[(h0 + eh) * P + pp] / p.state_scale[(h0 + eh) * P + pp];
    const uint32_t taddr = tbase + ((uint32_t)(32 * (warp & 3)) << 16) + 128 * eh + 64 * half;
    const uint32_t snp = s_sn + 4 * (128 * eh + 64 * half);
    // output tiles [head][64 channels][128 states] INT8 in the A region, SW128 rows of 128 bytes
    const uint32_t orow = s_A + eh * 8192 + pp * 128;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      uint32_t r[16];
      tmem_ld16(taddr + 16 * ch, r);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      int cd[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) cd[e] = code_rint127(__fmul_rn(__fmul_rn((float)(int)r[e], lds_f(snp + 4 * (16 * ch + e))), ra));
      sts128(orow + (((4 * half + ch) ^ (pp & 7)) << 4),
             make_uint4(pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]), pack4(cd[8], cd[9], cd[10], cd[11]),
                        pack4(cd[12], cd[13], cd[14], cd[15])));
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
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tbase), "r"(256u) : "memory");
}

// ------------------------------------------------------------------------------------------------ host side
static int encode_state_rows(CUtensorMap* m, const void* base, size_t rows, const char* what) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(LQ_ERR_LAUNCH, "%s: the driver does not export cuTensorMapEncodeTiled", what);
  const cuuint64_t gdim[2] = {128, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {128};
  const cuuint32_t box[2] = {128, 64};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LQ_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, (int)r);
  return LQ_OK;
}

template <typename T, int C>
static int launch_state_key_tc(const lq_ssd_problem* p, const CUtensorMap& to, int* status, cudaStream_t st) {
  const size_t smem = (size_t)3 * C * 128 + 2 * C * 4 + 2 * 128 * 4 + 16 + 16 + 1024;
  cudaError_t e = cudaFuncSetAttribute(ssd_chunk_state_key_tc_kernel<T, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "chunk_state_key: shared memory opt-in failed: %s", cudaGetErrorString(e));
  dim3 grid(p->L / C, p->H / 2, p->B);
  ssd_chunk_state_key_tc_kernel<T, C><<<grid, 256, smem, st>>>(to, *p, status);
  return check_launch("ssd_chunk_state_key_tc_kernel");
}

// key side, d_state 128, chunk 128 or 256, heads per group even, 16-byte aligned rows
bool chunk_state_key_tc_applies(const lq_ssd_problem* p) {
  return p->N == 128 && (p->chunk == 128 || p->chunk == 256) && p->P == 64 && ((p->H / p->G) % 2 == 0) &&
         !(reinterpret_cast<uintptr_t>(p->b_fp) & 15u) && !(reinterpret_cast<uintptr_t>(p->states) & 15u) &&
         !(reinterpret_cast<uintptr_t>(p->x) & 15u) && p->x_stride_t % 8 == 0 && p->x_stride_h % 8 == 0 && p->x_stride_b % 8 == 0;
}
int run_chunk_state_key_tc(const lq_ssd_problem* p, int* status, cudaStream_t st) {
  const int C = p->chunk, NC = p->L / C;
  CUtensorMap to;
  if (int e = encode_state_rows(&to, p->states, (size_t)p->B * NC * p->H * 64, "chunk_state_key (states)")) return e;
  if (p->x_dtype == LQ_F16) return C == 256 ? launch_state_key_tc<__half, 256>(p, to, status, st) : launch_state_key_tc<__half, 128>(p, to, status, st);
  return C == 256 ? launch_state_key_tc<__nv_bfloat16, 256>(p, to, status, st) : launch_state_key_tc<__nv_bfloat16, 128>(p, to, status, st);
}

}  // namespace lq
