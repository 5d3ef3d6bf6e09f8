// Mamba-2 chunk scan on the Blackwell tensor cores (headdim 64, d_state 128, chunk 128 or 256).
//
//   out[t,p] = (C_q[t,:] . S_q[p,:]) s_C S_p exp(dA_t)  +  sum_{k<=t} M[t,k] x[k,p]  +  D x[t,p]
//   M[t,k]   = fp16( cb_q[t,k] S_cb exp(dA_t - dA_k) dt_k )                       (mamba2/chunk_scan_v2.py:120-250)
//
// One CTA per (chunk, head, batch), 256 threads, two accumulators per 128-token row block in tensor memory:
//   * state read: TMA brings the q_C tile [128 tokens x 128 states] per row block and the INT8 state [64 x 128]
//     (128-byte swizzle); an elected thread issues tcgen05.mma.kind::i8 (M = 128, N = 64) into the int32 accumulator;
//   * causal product: all warps build the decay-masked matrix M tile by tile (128 tokens x 64 source tokens, fp16)
//     directly in the K-major swizzled layout of a two-slot ring in shared memory; the elected thread multiplies each
//     tile with the transposed x tile (staged once, channel rows, token index contiguous) by tcgen05.mma.kind::f16
//     into the fp32 accumulator and commits to the slot's mbarrier, so building tile i+1 overlaps the product of
//     tile i. The ring reuses the q_C space once the state products have completed;
//   * decay weights: tiles strictly below a row's 16-token group take  S_cb exp(dA[16 g] - dA_k) dt_k  from a table
//     and the row factor exp(dA_t - dA[16 g]) (both exponents <= 0); the 16 x 16 diagonal blocks take
//     S_cb exp(dA_t - dA_k) dt_k under the causal mask from a second table that every row fills for itself;
//   * epilogue: one thread per token row reads both accumulators (tcgen05.ld.32x32b), combines them with the D x
//     residual and stores the fp16 row.
// Every wait is bounded; on expiry the CTA raises the status word, skips its stores and still frees tensor memory.
#include <type_traits>

#include "lq_tc.cuh"

namespace lq {

template <typename T>
__global__ void __launch_bounds__(256) ssd_chunk_scan_tc_kernel(const __grid_constant__ CUtensorMap tm_qc,
                                                                const __grid_constant__ CUtensorMap tm_s, lq_ssd_problem p,
                                                                int* status) {
  constexpr int P = 64, N = 128;
  const int C = p.chunk, MB = C >> 7, KBT = C >> 6, NC = p.L / C;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint8_t* s_xT = smem;                    // [KBT][64 channels][64 tokens fp16]  SW128, K-major: B operand of the causal product
  uint8_t* s_qc = s_xT + C * 128;          // [MB][128 tokens][128 states] by TMA; afterwards the two M-tile slots of 16 KB
  uint8_t* s_S = s_qc + 32768;             // [64 channels][128 states] by TMA
  float* s_tab = reinterpret_cast<float*>(s_S + 8192);  // [C/16][C]
  float* s_dA = s_tab + (C >> 4) * C;
  float* s_dt = s_dA + C;
  float* s_ea = s_dt + C;
  float* s_ss = s_ea + C;
  float* s_D = s_ss + P;
  float* s_dg = s_D + P;                   // [C][16] decay weights of the 16 x 16 diagonal blocks (masked), fp32
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_dg + 16 * C);  // [0] TMA landed, [1] state products done, [2],[3] ring slots
  uint32_t* s_tbase = reinterpret_cast<uint32_t*>(bars + 4);

  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int grp = h / (p.H / p.G);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_tma = smem_u32(&bars[0]), bar_state = smem_u32(&bars[1]);
  const uint32_t bar_ring[2] = {smem_u32(&bars[2]), smem_u32(&bars[3])};
  const uint32_t tmem_cols = (uint32_t)(128 * MB);

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&bars[i])));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar_tma), "r"((uint32_t)(MB * 16384 + 8192)) : "memory");
    for (int mb = 0; mb < MB; ++mb)
      tma_load_2d(smem_u32(s_qc + mb * 16384), &tm_qc, grp * N, b * p.L + c * C + 128 * mb, bar_tma);
    tma_load_2d(smem_u32(s_S), &tm_s, 0, (int)((((size_t)b * NC + c) * p.H + h) * P), bar_tma);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(s_tbase)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }

  const size_t cbase = (((size_t)b * p.H + h) * NC + c) * C;
  for (int t = tid; t < C; t += 256) {
    s_dA[t] = p.dA[cbase + t];
    s_dt[t] = p.dt[cbase + t];
  }
  if (tid < P) {
    s_ss[tid] = p.state_scale[h * P + tid];
    s_D[tid] = p.D == nullptr ? 0.f : (p.D_has_hdim ? p.D[h * P + tid] : p.D[h]);
  }
  const T* xp = reinterpret_cast<const T*>(p.x) + (size_t)b * p.x_stride_b + (size_t)h * p.x_stride_h;
  // ---- x, transposed: lane = token pair of a 64-token block, one channel octet per step, two tokens to a word.
  // All global loads of the warp's steps are issued before the first is used.
  {
    constexpr int MAXIT = 4;  // KBT * 8 steps over 8 warps: 4 for a 256-token chunk, 2 for 128
    uint4 r0[MAXIT], r1[MAXIT];
    const int tl = 2 * lane;
#pragma unroll
    for (int u = 0; u < MAXIT; ++u) {
      const int it = warp + 8 * u;
      if (it < KBT * 8) {
        const int kbt = it >> 3, oct = it & 7;
        const size_t row = (size_t)(c * C + 64 * kbt + tl);
        r0[u] = __ldg(reinterpret_cast<const uint4*>(xp + row * p.x_stride_t + 8 * oct));
        r1[u] = __ldg(reinterpret_cast<const uint4*>(xp + (row + 1) * p.x_stride_t + 8 * oct));
      }
    }
#pragma unroll
    for (int u = 0; u < MAXIT; ++u) {
      const int it = warp + 8 * u;
      if (it < KBT * 8) {
        const int kbt = it >> 3, oct = it & 7;
        uint4 a0 = r0[u], a1 = r1[u];
        if (!std::is_same<T, __half>::value) {
          float f[8];
          Act<T>::unpack8(a0, f);
          a0 = make_uint4(Act<__half>::pack2(f[0], f[1]), Act<__half>::pack2(f[2], f[3]), Act<__half>::pack2(f[4], f[5]), Act<__half>::pack2(f[6], f[7]));
          Act<T>::unpack8(a1, f);
          a1 = make_uint4(Act<__half>::pack2(f[0], f[1]), Act<__half>::pack2(f[2], f[3]), Act<__half>::pack2(f[4], f[5]), Act<__half>::pack2(f[6], f[7]));
        }
        const uint32_t w0[4] = {a0.x, a0.y, a0.z, a0.w}, w1[4] = {a1.x, a1.y, a1.z, a1.w};
        uint8_t* grp8 = s_xT + kbt * 8192 + oct * 1024;
        const int chunk = tl >> 3, off = (tl & 7) * 2;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const uint32_t word = __byte_perm(w0[jj >> 1], w1[jj >> 1], (jj & 1) ? 0x7632 : 0x5410);
          *reinterpret_cast<uint32_t*>(grp8 + jj * 128 + ((chunk ^ jj) << 4) + off) = word;
        }
      }
    }
  }
  __syncthreads();  // s_dA, s_dt
  const float Scb = p.cb_scale[grp];
  for (int t = tid; t < C; t += 256) s_ea[t] = __expf(__fsub_rn(s_dA[t], s_dA[t & ~15]));
  for (int g16 = 1; g16 < (C >> 4); ++g16) {
    const float dref = s_dA[16 * g16];
    for (int k = tid; k < 16 * g16; k += 256)
      s_tab[g16 * C + k] = __fmul_rn(__fmul_rn(Scb, __expf(__fsub_rn(dref, s_dA[k]))), s_dt[k]);
  }
  for (int t = tid; t < C; t += 256) {  // diagonal blocks: every row evaluates its own sixteen weights, masked
    const float dAt = s_dA[t];
    const int kq = t & ~15;
#pragma unroll
    for (int e4 = 0; e4 < 4; ++e4) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int k = kq + 4 * e4 + e;
        v[e] = (k <= t) ? __fmul_rn(__fmul_rn(Scb, __expf(__fsub_rn(dAt, s_dA[k]))), s_dt[k]) : 0.f;
      }
      *reinterpret_cast<float4*>(s_dg + t * 16 + 4 * e4) = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the x tile was written by ordinary stores
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tbase = *s_tbase;
  const uint32_t tacc_i = tbase, tacc_f = tbase + 64 * MB;

  bool ok = true;
  if (tid == 0) {
    ok = mbar_wait_bounded(bar_tma, 0);
    if (ok) {
      const uint32_t idesc = idesc_i8(128, P);
      const uint64_t ds = desc_kmajor_sw128(smem_u32(s_S));
      for (int mb = 0; mb < MB; ++mb) {
        const uint64_t dq = desc_kmajor_sw128(smem_u32(s_qc + mb * 16384));
#pragma unroll
        for (int ks = 0; ks < N / 32; ++ks) umma_i8(tacc_i + 64 * mb, dq + 2 * ks, ds + 2 * ks, idesc, ks > 0);
      }
      umma_commit(bar_state);
    }
  }
  // the M-tile ring takes over the q_C space: wait until the state products have read it. One thread polls each
  // mbarrier and the block barrier releases the others (polling from every thread would take issue slots from the
  // warps of the co-resident CTA)
  if (tid == 0 && ok) ok = mbar_wait_bounded(bar_state, 0);
  ok = __syncthreads_and(ok ? 1 : 0) != 0;

  // ---- causal product, tile by tile. Tile i of the sequence is (row block mb, source block kb): block 0 takes source
  // blocks 0..1, block 1 takes 0..3. The CB codes of tile i+1 are fetched while tile i is built.
  const int8_t* cbp = p.cb + (((size_t)b * NC + c) * p.G + grp) * (size_t)C * C;
  const int r = tid & 127, hf = tid >> 7;
  const int ntiles = MB == 2 ? 6 : 2;
  auto tile_mb = [](int i) { return i < 2 ? 0 : 1; };
  auto tile_kb = [](int i) { return i < 2 ? i : i - 2; };
  auto fetch = [&](int i, uint4& c0, uint4& c1) {
    const int t = 128 * tile_mb(i) + r, k0 = 64 * tile_kb(i) + 32 * hf;
    if (k0 <= t) {
      c0 = __ldg(reinterpret_cast<const uint4*>(cbp + (size_t)t * C + k0));
      c1 = __ldg(reinterpret_cast<const uint4*>(cbp + (size_t)t * C + k0 + 16));
    }
  };
  uint4 n0 = make_uint4(0u, 0u, 0u, 0u), n1 = n0;
  fetch(0, n0, n1);
  int tile_i = 0;
  for (; tile_i < ntiles; ++tile_i) {
    const int mb = tile_mb(tile_i), kb = tile_kb(tile_i);
    const int t = 128 * mb + r, g16 = t >> 4;
    const float ea = s_ea[t], dAt = s_dA[t];
    {
      const int slot = tile_i & 1;
      const uint4 c0 = n0, c1 = n1;
      if (tile_i + 1 < ntiles) fetch(tile_i + 1, n0, n1);
      if (tile_i >= 2) {  // the slot is free once the product that read it has completed
        if (tid == 0 && ok) ok = mbar_wait_bounded(bar_ring[slot], (uint32_t)(((tile_i >> 1) - 1) & 1));
        ok = __syncthreads_and(ok ? 1 : 0) != 0;
      }
      uint8_t* srow = s_qc + slot * 16384 + (r >> 3) * 1024 + (r & 7) * 128;
      const int k0 = 64 * kb + 32 * hf;
      if (ok) {
        if (k0 > t) {
#pragma unroll
          for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(srow + (((4 * hf + q) ^ (r & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
        } else {
          const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
          for (int q = 0; q < 2; ++q) {  // 16 source tokens each
            const int kq = k0 + 16 * q;
            uint32_t hw[8];
            if (kq > t) {
#pragma unroll
              for (int e = 0; e < 8; ++e) hw[e] = 0u;
            } else {
              // below the row's 16-token group: table entry times the row factor; on the diagonal block: the row's own
              // masked weights (row factor 1)
              const bool diag = kq + 16 > 16 * g16;
              const float* tb = diag ? s_dg + t * 16 : s_tab + g16 * C + kq;
              const float rf = diag ? 1.0f : ea;
#pragma unroll
              for (int e4 = 0; e4 < 4; ++e4) {
                const float4 tv = *reinterpret_cast<const float4*>(tb + 4 * e4);
                const uint32_t w = cw[4 * q + e4] ^ 0x80808080u;
                const float v0 = __fmul_rn(__fmul_rn(s8_to_float<0>(w), rf), tv.x);
                const float v1 = __fmul_rn(__fmul_rn(s8_to_float<1>(w), rf), tv.y);
                const float v2 = __fmul_rn(__fmul_rn(s8_to_float<2>(w), rf), tv.z);
                const float v3 = __fmul_rn(__fmul_rn(s8_to_float<3>(w), rf), tv.w);
                hw[2 * e4] = Act<__half>::pack2(v0, v1);
                hw[2 * e4 + 1] = Act<__half>::pack2(v2, v3);
              }
            }
            *reinterpret_cast<uint4*>(srow + (((4 * hf + 2 * q) ^ (r & 7)) << 4)) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            *reinterpret_cast<uint4*>(srow + (((4 * hf + 2 * q + 1) ^ (r & 7)) << 4)) = make_uint4(hw[4], hw[5], hw[6], hw[7]);
          }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      ok = __syncthreads_and(ok ? 1 : 0) != 0;
      if (tid == 0 && ok) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t idesc = idesc_f16(128, P);
        const uint64_t da = desc_kmajor_sw128(smem_u32(s_qc + slot * 16384));
        const uint64_t db = desc_kmajor_sw128(smem_u32(s_xT + kb * 8192));
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) umma_f16(tacc_f + 64 * mb, da + 2 * ks, db + 2 * ks, idesc, (kb | ks) != 0);
        umma_commit(bar_ring[slot]);
      }
    }
  }
  // the commit of the last tile covers every product issued before it
  {
    const int last = tile_i - 1;
    if (tid == 0 && ok) ok = mbar_wait_bounded(bar_ring[last & 1], (uint32_t)((last >> 1) & 1));
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  }

  // ---- epilogue: one thread per token row
  if (ok) {
    const int q4 = warp & 3;
    const int mb = MB == 2 ? (warp >> 2) : 0;
    const int t = 128 * mb + 32 * q4 + lane;
    const float gscale = p.C_scale[grp];
    const float ga = expf(s_dA[t]);
    __half* op = reinterpret_cast<__half*>(p.out) + (((size_t)b * p.L + (size_t)c * C + t) * p.H + h) * P;
    const T* xr = xp + (size_t)(c * C + t) * p.x_stride_t;
    for (int ch = (MB == 2 ? 0 : (warp >> 2)); ch < (MB == 2 ? 2 : (warp >> 2) + 1); ++ch) {
      const int col0 = 32 * ch;
      uint4 xraw[4];  // the row's x values for the residual, all four loads in flight together
#pragma unroll
      for (int o8 = 0; o8 < 4; ++o8) xraw[o8] = __ldg(reinterpret_cast<const uint4*>(xr + col0 + 8 * o8));
      uint32_t ri[32], rf[32];
      const uint32_t lane_addr = (uint32_t)(32 * q4) << 16;
      tmem_ld_32x32b_x32(tacc_i + lane_addr + 64 * mb + col0, ri);
      tmem_ld_32x32b_x32(tacc_f + lane_addr + 64 * mb + col0, rf);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      uint4 ov[4];
#pragma unroll
      for (int o8 = 0; o8 < 4; ++o8) {
        float xv[8];
        if (std::is_same<T, __half>::value) {
          Act<__half>::unpack8(xraw[o8], xv);
        } else {  // the products saw x rounded to fp16; the residual uses the same values
          float f[8];
          Act<T>::unpack8(xraw[o8], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) xv[e] = __half2float(__float2half_rn(f[e]));
        }
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int pc = col0 + 8 * o8 + e;
          const float sread = __fmul_rn(__fmul_rn(__fmul_rn((float)(int)ri[8 * o8 + e], gscale), s_ss[pc]), ga);
          float v = __fadd_rn(sread, __uint_as_float(rf[8 * o8 + e]));
          if (p.D != nullptr) v = __fadd_rn(v, __fmul_rn(xv[e], s_D[pc]));
          o[e] = v;
        }
        ov[o8] = make_uint4(Act<__half>::pack2(o[0], o[1]), Act<__half>::pack2(o[2], o[3]), Act<__half>::pack2(o[4], o[5]),
                            Act<__half>::pack2(o[6], o[7]));
      }
#pragma unroll
      for (int o8 = 0; o8 < 4; ++o8) *reinterpret_cast<uint4*>(op + col0 + 8 * o8) = ov[o8];
    }
  } else if (tid == 0 && status != nullptr) {
    atomicExch(status, 1);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tbase), "r"(tmem_cols) : "memory");
}

// ------------------------------------------------------------------------------------------------ host side
static int encode_u8_2d(CUtensorMap* m, const void* base, size_t inner, size_t rows, int box_rows, const char* what) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(LQ_ERR_LAUNCH, "%s: the driver does not export cuTensorMapEncodeTiled", what);
  const cuuint64_t gdim[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)inner};
  const cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LQ_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, (int)r);
  return LQ_OK;
}

// d_state 128, chunk a multiple of 128 tokens
int run_chunk_scan_tc(const lq_ssd_problem* p, int* status, cudaStream_t st) {
  const int C = p->chunk, NC = p->L / C;
  CUtensorMap tq, ts;
  if (int e = encode_u8_2d(&tq, p->q_C, (size_t)p->G * 128, (size_t)p->B * p->L, 128, "chunk_scan")) return e;
  if (int e = encode_u8_2d(&ts, p->passed, 128, (size_t)p->B * NC * p->H * 64, 64, "chunk_scan")) return e;
  const size_t smem = (size_t)C * 128 + 32768 + 8192 + sizeof(float) * ((size_t)(C >> 4) * C + 3 * C + 128 + 16 * (size_t)C) + 64 + 1024;
  dim3 grid(NC, p->H, p->B);
  cudaError_t e;
  if (p->x_dtype == LQ_F16) {
    e = cudaFuncSetAttribute(ssd_chunk_scan_tc_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) ssd_chunk_scan_tc_kernel<__half><<<grid, 256, smem, st>>>(tq, ts, *p, status);
  } else {
    e = cudaFuncSetAttribute(ssd_chunk_scan_tc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) ssd_chunk_scan_tc_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(tq, ts, *p, status);
  }
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "chunk_scan: shared memory opt-in failed: %s", cudaGetErrorString(e));
  return check_launch("ssd_chunk_scan_tc_kernel");
}

}  // namespace lq
