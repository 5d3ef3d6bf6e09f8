// Value-side Mamba-2 chunk state on the Blackwell tensor cores (headdim 64, chunk 128 or 256, d_state 64 or 128).
//
//   states[p, n] = half_away( (sum_t xq[t, p] * qB[t, n]) * (alpha_p / S_p) * s_B ),   xq = half_away((x / alpha_p) * gate_t)
//   (mamba2/chunk_state.py:186-246)
//
// One CTA per (chunk, head, batch), 128 threads:
//   * all threads fetch the x tile with cp.async, quantise it (gate table, per-channel reciprocal scale, half away
//     from zero) and write the codes transposed -- channel rows, token index contiguous -- directly in the K-major
//     128-byte-swizzled layout tcgen05 reads, four tokens to a word; the lane mapping (4 channel pairs x 8 token
//     quads) makes both the reads of the staged tile and these writes bank-conflict free;
//   * an elected thread then loads the pre-transposed INT8 B tile (q_BT: d_state rows, token index contiguous) with TMA
//     (cp.async.bulk.tensor.2d, 128-byte swizzle, blocks of 128 tokens) into the space the staged x rows occupied, and
//     issues tcgen05.mma.kind::i8 (M = 64, N = d_state, 32 tokens per instruction) into tensor
//     memory and commits to an mbarrier;
//   * every warp reads its 16 accumulator rows with tcgen05.ld.16x256b, requantises, and the INT8 tile leaves through
//     shared memory as 16-byte stores.
// Every wait is bounded; on expiry the CTA raises the status word (when the caller supplied one), skips its stores
// and still frees its tensor memory.
#include <type_traits>

#include "lq_tc.cuh"

namespace lq {

__device__ __forceinline__ int ssd_half_away(float y, float lim) {
  y = fminf(fmaxf(y, -lim), lim);
  return __float2int_rz(__fadd_rn(y, copysignf(0.5f, y)));
}

template <typename T, int N>
__global__ void __launch_bounds__(128) ssd_chunk_state_tc_kernel(const __grid_constant__ CUtensorMap tm_b, lq_ssd_problem p,
                                                                 int* status) {
  constexpr int P = 64;
  const int C = p.chunk, KB = C >> 7, NC = p.L / C;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint8_t* s_A = smem;                                       // [KB][64 channels][128 tokens]   SW128, K-major
  uint8_t* s_raw = s_A + KB * 8192;                          // [C tokens][128 B]: x as stored, until it is quantised; then
  uint8_t* s_B = s_raw;                                      // [KB][N states][128 tokens] SW128 by TMA; then the output tile
  float* s_gate = reinterpret_cast<float*>(s_raw + C * 128); // [C]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_gate + C);  // [0] B landed, [1] accumulator complete
  uint32_t* s_tbase = reinterpret_cast<uint32_t*>(bars + 2);

  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int grp = h / (p.H / p.G);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;
  const uint32_t bar_ld = smem_u32(&bars[0]), bar_mma = smem_u32(&bars[1]);

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_ld));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_mma));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(s_tbase)), "r"((uint32_t)N) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  {  // x rows of the chunk; 16-byte piece ch of token t lands at piece ch ^ ((t >> 2) & 7)
    const T* xrow = reinterpret_cast<const T*>(p.x) + (size_t)b * p.x_stride_b + (size_t)h * p.x_stride_h;
    for (int i = tid; i < C * 8; i += 128) {
      const int t = i >> 3, ch = i & 7;
      cp_async16(s_raw + t * 128 + ((ch ^ ((t >> 2) & 7)) << 4), xrow + (size_t)(c * C + t) * p.x_stride_t + 8 * ch);
    }
    cp_async_commit();
  }
  const size_t cbase = (((size_t)b * p.H + h) * NC + c) * C;
  {
    const float last = p.dA[cbase + C - 1];
    for (int t = tid; t < C; t += 128) s_gate[t] = __fmul_rn(expf(__fsub_rn(last, p.dA[cbase + t])), p.dt[cbase + t]);
  }
  // lane = (channel pair cp, token quad tq): channels 8 pg + 2 cp + {0,1} for pg = 0..7
  const int cp = lane & 3, tq = lane >> 2;
  float xinv[8][2];
#pragma unroll
  for (int pg = 0; pg < 8; ++pg) {
    xinv[pg][0] = 1.0f / p.alpha_hp[h * P + 8 * pg + 2 * cp];
    xinv[pg][1] = 1.0f / p.alpha_hp[h * P + 8 * pg + 2 * cp + 1];
  }
  cp_async_wait<0>();
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tbase = *s_tbase;

  // ---- quantise and transpose x into the A tiles. Shared-memory accesses go through 32-bit shared addresses with the
  // swizzles reduced to one XOR (loads) or an immediate offset (stores): generic 64-bit addressing cost more integer
  // instructions here than the quantiser itself.
  const uint32_t raw_u32 = smem_u32(s_raw), sA_u32 = smem_u32(s_A);
  for (int blk = warp; blk < C / 32; blk += 4) {
    const int t0 = 32 * blk + 4 * tq;           // first of this lane's four tokens
    const int kb = t0 >> 7, tl = t0 & 127;
    const int ch16 = tl >> 4, off = tl & 15;
    const float4 gk4 = *reinterpret_cast<const float4*>(s_gate + t0);
    const float gk[4] = {gk4.x, gk4.y, gk4.z, gk4.w};
    // row t0+i, piece (pg ^ tq), bytes 4cp..: the row base carries tq in the piece bits, pg is XORed in
    const uint32_t ld0 = raw_u32 + t0 * 128 + (tq << 4) + 4 * cp;
    const int r0 = 2 * cp, r1 = 2 * cp + 1;  // rows within the 8-row group pg
    const uint32_t st0 = sA_u32 + kb * 8192 + r0 * 128 + ((ch16 ^ r0) << 4) + off;
    const uint32_t st1 = sA_u32 + kb * 8192 + r1 * 128 + ((ch16 ^ r1) << 4) + off;
#pragma unroll
    for (int pg = 0; pg < 8; ++pg) {
      int c0v[4], c1v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t raw = lds_u32((ld0 + i * 128) ^ (pg << 4));
        float x0, x1;
        if (std::is_same<T, __half>::value) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&raw));
          x0 = f.x; x1 = f.y;
        } else {
          x0 = __uint_as_float(raw << 16); x1 = __uint_as_float(raw & 0xffff0000u);
        }
        // half away from zero; the lower clamp here, the upper one in the saturating pack below
        const float y0 = fmaxf(__fmul_rn(__fmul_rn(x0, xinv[pg][0]), gk[i]), -127.f);
        const float y1 = fmaxf(__fmul_rn(__fmul_rn(x1, xinv[pg][1]), gk[i]), -127.f);
        c0v[i] = __float2int_rz(__fadd_rn(y0, copysignf(0.5f, y0)));
        c1v[i] = __float2int_rz(__fadd_rn(y1, copysignf(0.5f, y1)));
      }
      sts_u32(st0 + pg * 1024, pack_sat_s8x2(c0v[1], c0v[0], pack_sat_s8x2(c0v[3], c0v[2], 0u)));
      sts_u32(st1 + pg * 1024, pack_sat_s8x2(c1v[1], c1v[0], pack_sat_s8x2(c1v[3], c1v[2], 0u)));
    }
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic-proxy writes -> visible to the tensor core
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();

  bool ok = true;
  if (tid == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    // the staged x rows are consumed: their space takes the B tiles (the proxy fence above orders the reuse)
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar_ld), "r"((uint32_t)(KB * N * 128)) : "memory");
    const int row0 = (int)((((size_t)b * NC + c) * p.G + grp) * N);
    for (int kb = 0; kb < KB; ++kb) tma_load_2d(smem_u32(s_B + kb * N * 128), &tm_b, 128 * kb, row0, bar_ld);
    ok = mbar_wait_bounded(bar_ld, 0);
    if (ok) {
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(64 >> 4) << 24);
      const uint64_t da = desc_kmajor_sw128(smem_u32(s_A)), db = desc_kmajor_sw128(smem_u32(s_B));
      for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_i8(tbase, da + (uint64_t)(kb * (8192 >> 4) + 2 * ks), db + (uint64_t)(kb * ((N * 128) >> 4) + 2 * ks), idesc,
                  (kb | ks) != 0);
      }
      umma_commit(bar_mma);
    } else {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar_mma) : "memory");
    }
  }
  if (tid == 0 && ok) ok = mbar_wait_bounded(bar_mma, 0);  // one poller; the block barrier releases the rest
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");

  // ---- requantise: warp w owns accumulator rows (channels) 16w .. 16w+15 in the first 16 lanes of its quadrant
  int8_t* s_out = reinterpret_cast<int8_t*>(s_raw);  // [64][N]
  if (ok) {
    const int pa = 16 * warp + g, pb = pa + 8;
    const float bs = p.bscale_g[grp];
    const float ra = __fmul_rn(p.alpha_hp[h * P + pa] / p.state_scale[h * P + pa], bs);
    const float rb = __fmul_rn(p.alpha_hp[h * P + pb] / p.state_scale[h * P + pb], bs);
    const uint32_t tq_addr = tbase + ((uint32_t)(32 * warp) << 16);
    const uint32_t out_a = smem_u32(s_out) + pa * N + 2 * j, out_b = smem_u32(s_out) + pb * N + 2 * j;
#pragma unroll
    for (int ng = 0; ng < N / 32; ++ng) {
      uint32_t r[16];
      tmem_ld_16x256b_x4(tq_addr + 32 * ng, r);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
      for (int n4 = 0; n4 < 4; ++n4) {
        const int col = 32 * ng + 8 * n4;
        const int a0 = ssd_half_away(__fmul_rn((float)(int)r[4 * n4 + 0], ra), 127.f);
        const int a1 = ssd_half_away(__fmul_rn((float)(int)r[4 * n4 + 1], ra), 127.f);
        const int b0 = ssd_half_away(__fmul_rn((float)(int)r[4 * n4 + 2], rb), 127.f);
        const int b1 = ssd_half_away(__fmul_rn((float)(int)r[4 * n4 + 3], rb), 127.f);
        sts_u16(out_a + col, (uint16_t)((a0 & 0xff) | ((a1 & 0xff) << 8)));
        sts_u16(out_b + col, (uint16_t)((b0 & 0xff) | ((b1 & 0xff) << 8)));
      }
    }
  } else if (tid == 0 && status != nullptr) {
    atomicExch(status, 1);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (ok) {
    uint4* dst = reinterpret_cast<uint4*>(p.states + ((((size_t)b * NC + c) * p.H + h) * P) * N);
    const uint4* src = reinterpret_cast<const uint4*>(s_out);
    for (int i = tid; i < P * N / 16; i += 128) dst[i] = src[i];
  }
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tbase), "r"((uint32_t)N) : "memory");
}

// ------------------------------------------------------------------------------------------------ host side
template <typename T, int N>
static int launch_state_tc(const lq_ssd_problem* p, int* status, cudaStream_t st) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(LQ_ERR_LAUNCH, "chunk_state: the driver does not export cuTensorMapEncodeTiled");
  const int C = p->chunk, NC = p->L / C;
  CUtensorMap tm;
  const cuuint64_t gdim[2] = {(cuuint64_t)C, (cuuint64_t)p->B * NC * p->G * N};
  const cuuint64_t gstride[1] = {(cuuint64_t)C};
  const cuuint32_t box[2] = {128, (cuuint32_t)N};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, p->q_BT, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LQ_ERR_LAUNCH, "chunk_state: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  const int KB = C / 128;
  const size_t smem = (size_t)KB * 8192 + (size_t)C * 128 + sizeof(float) * C + 64 + 1024;  // N <= 128: the B tiles fit the x region
  cudaError_t e = cudaFuncSetAttribute(ssd_chunk_state_tc_kernel<T, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "chunk_state: shared memory opt-in failed: %s", cudaGetErrorString(e));
  dim3 grid(NC, p->H, p->B);
  ssd_chunk_state_tc_kernel<T, N><<<grid, 128, smem, st>>>(tm, *p, status);
  return check_launch("ssd_chunk_state_tc_kernel");
}

// value side, chunk a multiple of 128 tokens; q_BT already holds the transposed B codes
int run_chunk_state_value_tc(const lq_ssd_problem* p, int* status, cudaStream_t st) {
  if (p->x_dtype == LQ_F16) return p->N == 128 ? launch_state_tc<__half, 128>(p, status, st) : launch_state_tc<__half, 64>(p, status, st);
  return p->N == 128 ? launch_state_tc<__nv_bfloat16, 128>(p, status, st) : launch_state_tc<__nv_bfloat16, 64>(p, status, st);
}

}  // namespace lq
