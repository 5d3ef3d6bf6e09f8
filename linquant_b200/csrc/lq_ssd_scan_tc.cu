// Mamba-2 chunk scan as a persistent, software-pipelined tcgen05 kernel (headdim 64, d_state 128, chunk 128 or 256).
//
//   out[t,p] = (C_q[t,:] . S_q[p,:]) s_C S_p exp(dA_t)  +  sum_{k<=t} M[t,k] x[k,p]  +  D x[t,p]
//   M[t,k]   = fp16( cb_q[t,k] S_cb exp(dA_t - dA_k) dt_k )                       (mamba2/chunk_scan_v2.py:120-250)
//
// One CTA per SM walks the (batch, chunk, head) items i, i + grid, i + 2 grid, ... (neighbouring CTAs work on heads of
// the same chunk at the same time, so the q_C tile and the CB codes they share stay in L2). Two stages of input tiles
// and two sets of accumulators in tensor memory let the phases of consecutive items overlap:
//
//   producer warp     TMA loads of item i+1 (x tile as it lies in memory, q_C tile(s), INT8 state, dA and dt rows) into the
//                     stage that item i-1 has left, after storing that stage's output tile (TMA store) first
//   MMA warp          state read of item i as soon as its tiles land (tcgen05.mma.kind::i8, M = 128, N = 64), then the causal
//                     product tile by tile (kind::f16, A = decay-masked matrix tile from the ring, B = the x tile in its
//                     natural channel-contiguous layout); commits free the ring slots and publish the accumulators
//   512 worker threads  per item: the epilogue of the PREVIOUS item (both accumulators from tensor memory, fp16 row written
//                     over the x row, one arrival per warp on the stage's out_ready barrier; placing it after this item's
//                     tables instead measured 8 % slower), then the fp16 rounding of a bf16 x tile in place, this
//                     item's weight tables, and the six (two) tiles of the decay-masked matrix M into a ring of three
//                     slots, one 16-token group of one row per thread and tile
//
// so the tensor core works on item i while the workers finish item i-1 and build item i, and the loads of item i+1 are
// in flight. Decay weights as fp16 tables: for source tokens before the row's 16-token group  S_cb dt_k exp(dA[16 g] -
// dA_k)  (built by a running product over g) times the row factor exp(dA_t - dA[16 g]) (both exponents <= 0), for the
// group itself the row's own sixteen masked weights S_cb dt_k exp(dA_t - dA_k).
// Every wait is bounded. A role whose wait runs out raises the status word and leaves its loop; the roles that depend on
// it run into their own limits and leave too; nothing is stored for the items concerned, tensor memory is freed.
#include <type_traits>

#include "lq_tc.cuh"

namespace lq {

namespace scantc {

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float lds_f(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_f(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void sts_h(uint32_t addr, __half v) {
  asm volatile("st.shared.u16 [%0], %1;\n" ::"r"(addr), "h"(__half_as_ushort(v)) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint32_t hfma2u(uint32_t a, uint32_t b, uint32_t c) {
  const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b), *reinterpret_cast<const __half2*>(&c));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hmul2u(uint32_t a, uint32_t b) {
  const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];\n" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
// plain (untiled) bulk copy global -> shared: both addresses 16-byte aligned, size a multiple of 16 bytes
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src), "r"(bytes),
               "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ float exp_decay(float x) {  // ex2.approx.ftz(x log2 e): decay factors, a denormal may be zero
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(__fmul_rn(x, 1.4426950408889634f)));
  return y;
}
constexpr int kWorkers = 512;
constexpr int kRing = 3;  // slots of the M-tile ring: the round trip through the tensor core takes longer than building one tile
// Barrier of the worker threads that also ANDs a predicate: every decision to leave the pipeline is taken here, so
// all workers take it together (a bounded wait may run out in some warps and not in others).
__device__ __forceinline__ bool worker_and(bool ok) {
  uint32_t r;
  asm volatile("{\n.reg .pred p, q;\nsetp.ne.b32 q, %1, 0;\nbar.red.and.pred p, 1, 512, q;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(r) : "r"((uint32_t)ok) : "memory");
  return r != 0;
}
// Bounded wait on an mbarrier phase. Each probe may suspend the thread for up to the hinted time (so a waiting role does not
// spin through the issue slots of the working ones); 2^13 probes of at most 50 us bound the wait to well under a second.
__device__ __forceinline__ bool mbar_wait_suspending(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < (1 << 13); ++it) {
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(bar), "r"(parity), "r"(50000u) : "memory");
    if (done) return true;
  }
  return false;
}
// by every lane (each needs its own acquire of the barrier's phase), warp-uniform result. Most waits of the workers find
// their phase complete already: one non-suspending probe first.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  if (__all_sync(0xffffffffu, done != 0u)) return true;
  return __all_sync(0xffffffffu, mbar_wait_suspending(bar, parity) ? 1 : 0) != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}

constexpr int kStageBytes = 77824;  // x 32 KB | q_C 32 KB | state 8 KB | dA 1 KB | dt 1 KB | pad (a multiple of 1 KB)
constexpr int kOffQc = 32768, kOffS = 65536, kOffDa = 73728, kOffDt = 74752;

// the walk over the items blockIdx.x + j * gridDim.x without divisions in the loop
struct ItemWalk {
  int b, c, h, dh, dc, H, NC;
  __device__ __forceinline__ void init(int first, int stride, int H_, int NC_) {
    H = H_; NC = NC_;
    h = first % H;
    const int q = first / H;
    c = q % NC;
    b = q / NC;
    dh = stride % H;
    dc = stride / H;
  }
  __device__ __forceinline__ void next() {
    h += dh;
    int cc = c + dc;
    if (h >= H) { h -= H; ++cc; }
    while (cc >= NC) { cc -= NC; ++b; }
    c = cc;
  }
};

}  // namespace scantc

template <typename T, int MB>
__global__ void __launch_bounds__(576, 1) ssd_chunk_scan_tc_kernel(const __grid_constant__ CUtensorMap tm_qc,
                                                                  const __grid_constant__ CUtensorMap tm_s,
                                                                  const __grid_constant__ CUtensorMap tm_x,
                                                                  const __grid_constant__ CUtensorMap tm_out, lq_ssd_problem p,
                                                                  int* status, int n_items) {
  using namespace scantc;
  constexpr int P = 64, N = 128, C = 128 * MB, NT = MB == 2 ? 6 : 2;
  constexpr bool XBF16 = !std::is_same<T, __half>::value;
  const int NC = p.L / C, hpg = p.H / p.G;
  extern __shared__ uint8_t smem_dyn[];
  const uint32_t s_stage0 = (smem_u32(smem_dyn) + 1023u) & ~1023u;  // two input stages
  const uint32_t s_ring = s_stage0 + 2 * kStageBytes;             // kRing M-tile slots of 16 KB
  const uint32_t s_tab = s_ring + kRing * 16384;                       // fp16 [C/16][C] below-group weights (8 KB at C = 256)
  const uint32_t s_dg = s_tab + 8192;                             // fp16 [C][16] weights of the row's own group, masked (8 KB)
  const uint32_t s_dts = s_dg + 8192;                             // f32 [C] S_cb * dt
  const uint32_t s_ratio = s_dts + 1024;                          // f32 [16] exp(dA[16 g] - dA[16 (g-1)])
  const uint32_t s_zero = s_ratio + 64;                           // 32 bytes of zeros: the weights of a group above the diagonal
  const uint32_t s_dvec = s_zero + 64;                            // fp16 [16][16]: D on the diagonal (a per-head D joins M there)
  const uint32_t s_cs = s_dvec + 512;                             // f32 [2][64] s_C * state scale, per stage
  const uint32_t s_D = s_cs + 512;                                // f32 [2][64]
  const uint32_t s_bars = s_D + 512;                              // full_in[2] out_ready[2] acc_full[2] ring_full[3] ring_empty[3]
  const uint32_t s_tbase = s_bars + 96;
  enum { FULL_IN = 0, OUT_READY = 2, ACC_FULL = 4, RING_FULL = 6, RING_EMPTY = 6 + kRing, kBars = 6 + 2 * kRing };
  auto bar = [&](int which, int idx) { return s_bars + 8u * (which + idx); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kProducerWarp = kWorkers / 32, kMmaWarp = kProducerWarp + 1;
  const int n_mine = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;  // items blockIdx.x + j * gridDim.x
  // The D x residual: a per-head D is added to the diagonal of M (M[t,t] + D, then one product with x on the tensor core);
  // a per-channel D cannot be, and is applied in the epilogue from the x row.
  const int dmode = p.D == nullptr ? 0 : (p.D_has_hdim ? 2 : 1);

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < kBars; ++i) {  // out_ready and ring_full take one arrival per worker warp, the others a single one
      const bool per_warp = (i >= OUT_READY && i < OUT_READY + 2) || (i >= RING_FULL && i < RING_FULL + kRing);
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(s_bars + 8u * i), "r"(per_warp ? (uint32_t)(kWorkers / 32) : 1u));
    }
    sts128(s_zero, make_uint4(0u, 0u, 0u, 0u));
    sts128(s_zero + 16, make_uint4(0u, 0u, 0u, 0u));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == kProducerWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s_tbase), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tbase = lds_u32(s_tbase);
  bool failed = false;

  // The whole warp stays inside its role loop (a block barrier must not be reached by part of a warp): every lane waits,
  // lane 0 issues.
  if (warp == kProducerWarp) {
    // ============================================================ producer: TMA loads, TMA stores
    ItemWalk ld, stw;
    ld.init(blockIdx.x, gridDim.x, p.H, NC);
    stw = ld;
    int issued = 0;
    for (int j = 0; j < n_mine + 2 && !failed; ++j) {
      const int s = j & 1;
      if (j >= 2) {  // the stage still holds item j-2: its output tile is written over the x tile by the workers
        if (!warp_wait(bar(OUT_READY, s), (uint32_t)(((j - 2) >> 1) & 1))) { failed = true; break; }
        if (lane == 0) {
          tma_store_4d(&tm_out, s_stage0 + s * kStageBytes, 0, stw.h, stw.c * C, stw.b);
          asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");  // the tile has been read: the stage is free
        }
        stw.next();
        __syncwarp();
      }
      if (j < n_mine) {
        if (lane == 0) {
          const int b = ld.b, c = ld.c, h = ld.h;
          const int grp = p.G == 1 ? 0 : h / hpg;
          const uint32_t st = s_stage0 + s * kStageBytes, fb = bar(FULL_IN, s);
          mbar_expect(fb, (uint32_t)(C * 128 + MB * 16384 + 8192 + 2 * C * 4));
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) tma_load_2d(st + kOffQc + mb * 16384, &tm_qc, grp * N, b * p.L + c * C + 128 * mb, fb);
          tma_load_2d(st + kOffS, &tm_s, 0, (int)((((size_t)b * NC + c) * p.H + h) * P), fb);
          const size_t cbase = (((size_t)b * p.H + h) * NC + c) * C;
          bulk_load(st + kOffDa, p.dA + cbase, (uint32_t)(C * 4), fb);
          bulk_load(st + kOffDt, p.dt + cbase, (uint32_t)(C * 4), fb);
          tma_load_4d(st, &tm_x, 0, h, c * C, b, fb);
        }
        ld.next();
        ++issued;
        __syncwarp();
      }
    }
    if (failed) {
      if (lane == 0 && status != nullptr) atomicExch(status, 1);
      // copies still in flight must land before the CTA may exit: wait (bounded) on the stages that were filled last
      for (int j = max(0, issued - 2); j < issued; ++j) warp_wait(bar(FULL_IN, j & 1), (uint32_t)((j >> 1) & 1));
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");  // every store complete
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ============================================================ MMA issuer
    const uint32_t idesc_s = idesc_i8(128, P);
    // B operand MN-major (the x tile as it lies in memory). Both operands are fp16: kind::f16 does not take an fp16 A with
    // a bf16 B (the instruction is rejected), so a bf16 x tile is rounded to fp16 in shared memory by the workers first.
    const uint32_t idesc_c = idesc_f16(128, P) | (1u << 16);
    int slot = 0;       // ring slot of the next tile
    uint32_t rph = 0u;  // parity of that slot's use count
    for (int j = 0; j < n_mine && !failed; ++j) {
      const int s = j & 1;
      const uint32_t st = s_stage0 + s * kStageBytes;
      const uint32_t tacc_i = tbase + 256 * s, tacc_f = tacc_i + 64 * MB;
      if (!warp_wait(bar(FULL_IN, s), (uint32_t)((j >> 1) & 1))) { failed = true; break; }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      if (lane == 0) {
        const uint64_t ds = desc_kmajor_sw128(st + kOffS);
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const uint64_t dq = desc_kmajor_sw128(st + kOffQc + mb * 16384);
#pragma unroll
          for (int ks = 0; ks < N / 32; ++ks) umma_i8(tacc_i + 64 * mb, dq + 2 * ks, ds + 2 * ks, idesc_s, ks > 0);
        }
      }
      __syncwarp();
#pragma unroll
      for (int ti = 0; ti < NT; ++ti) {
        const int mb = ti < 2 ? 0 : 1, kb = ti < 2 ? ti : ti - 2;
        if (NT % kRing == 0) { slot = ti % kRing; rph = (uint32_t)((ti / kRing) & 1); }  // whole laps per item: known at compile time
        if (!warp_wait(bar(RING_FULL, slot), rph)) { failed = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (lane == 0) {
          const uint64_t da = desc_kmajor_sw128(s_ring + slot * 16384);
          const uint64_t db = desc_kmajor_sw128(st + kb * 8192);  // 64 tokens x 128 B; 16 tokens (two 8-row groups) per step
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) umma_f16(tacc_f + 64 * mb, da + 2 * ks, db + (uint64_t)(ks * (2048 >> 4)), idesc_c, (kb | ks) != 0);
          umma_commit(bar(RING_EMPTY, slot));
          if (ti == NT - 1) umma_commit(bar(ACC_FULL, s));
        }
        __syncwarp();
        if (++slot == kRing) { slot = 0; rph ^= 1u; }
      }
    }
    if (failed && lane == 0 && status != nullptr) atomicExch(status, 1);
  } else {
    // ============================================================ workers (512 threads)
    // M tiles: thread = (row r of the 128-row block, quarter qt of the tile's 64 source tokens). The causal mask leaves a
    // warp (32 rows, one quarter) between two and six of the six tiles to build; evening that out (mirrored shares in the
    // last two tiles, or one warp of every row quarter per scheduler) measured no faster.
    const int r = tid & 127, qt = tid >> 7;
    // epilogue: warp w reads TMEM lanes 32 (w & 3) ..; the four warps of a lane quadrant split (row block, column half)
    const int q4 = warp & 3, sel = warp >> 2;
    const int e_mb = MB == 2 ? (sel & 1) : 0, e_ch0 = MB == 2 ? 2 * (sel >> 1) : sel;  // first 16-channel chunk (of 2, or of 1)
    constexpr int E_NCH = MB == 2 ? 2 : 1;
    constexpr int E_STEP = 1;  // chunks loaded per tcgen05.wait::ld; both at once costs registers the tile loop needs
    int slot = 0, g = 0;  // ring slot of the next tile and the running tile counter, as in the MMA issuer
    uint32_t rph = 0u;
    ItemWalk w;
    w.init(blockIdx.x, gridDim.x, p.H, NC);

    // The epilogue of item j: every warp reads its 32 rows of both accumulators and posts its own arrival on the stage's
    // out_ready barrier (no block barrier). Returns the warp's verdict on its waits; a warp whose wait ran out stores and
    // posts nothing, and the decision to leave is taken by all workers together at the next block barrier.
    auto epilogue = [&](int j, bool ok_so_far) -> bool {
      const int s = j & 1;
      const bool ok = warp_wait(bar(ACC_FULL, s), (uint32_t)((j >> 1) & 1)) && ok_so_far;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t st = s_stage0 + s * kStageBytes;
      const uint32_t tacc_i = tbase + 256 * s, tacc_f = tacc_i + 64 * MB;
      const int t = 128 * e_mb + 32 * q4 + lane;
      const uint32_t xrow = st + t * 128;
      const uint32_t lane_addr = (uint32_t)(32 * q4) << 16;
      if (ok) {
        const float ga = exp_decay(lds_f(st + kOffDa + 4 * t));
#pragma unroll
        for (int c0 = 0; c0 < E_NCH; c0 += E_STEP) {
        uint32_t ri[E_NCH][16], rf[E_NCH][16];  // E_STEP chunks of 16 channels are loaded per wait
#pragma unroll
        for (int cc = c0; cc < c0 + E_STEP; ++cc) {
          tmem_ld16(tacc_i + lane_addr + 64 * e_mb + 16 * (e_ch0 + cc), ri[cc]);
          tmem_ld16(tacc_f + lane_addr + 64 * e_mb + 16 * (e_ch0 + cc), rf[cc]);
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
        for (int cc = c0; cc < c0 + E_STEP; ++cc) {
          const int ch = e_ch0 + cc, col0 = 16 * ch;
          const uint32_t pa = xrow + (((2 * ch) ^ (t & 7)) << 4), pb = xrow + (((2 * ch + 1) ^ (t & 7)) << 4);
          uint32_t o[8];
          if (dmode == 2) {
            const uint4 xa = lds128(pa), xb = lds128(pb);
            float xv[16];
            Act<__half>::unpack8(xa, *reinterpret_cast<float (*)[8]>(&xv[0]));
            Act<__half>::unpack8(xb, *reinterpret_cast<float (*)[8]>(&xv[8]));
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
              const float4 cs = lds_f4(s_cs + 256 * s + 4 * (col0 + 4 * v4)), d = lds_f4(s_D + 256 * s + 4 * (col0 + 4 * v4));
              const float csv[4] = {cs.x, cs.y, cs.z, cs.w}, Dv[4] = {d.x, d.y, d.z, d.w};
              float v[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int e = 4 * v4 + u;
                const float sread = __fmul_rn(__fmul_rn((float)(int)ri[cc][e], csv[u]), ga);
                v[u] = fmaf(xv[e], Dv[u], __fadd_rn(sread, __uint_as_float(rf[cc][e])));
              }
              o[2 * v4] = Act<__half>::pack2(v[0], v[1]);
              o[2 * v4 + 1] = Act<__half>::pack2(v[2], v[3]);
            }
          } else {
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
              const float4 cs = lds_f4(s_cs + 256 * s + 4 * (col0 + 4 * v4));
              const float csv[4] = {cs.x, cs.y, cs.z, cs.w};
              float v[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int e = 4 * v4 + u;
                v[u] = fmaf(__fmul_rn((float)(int)ri[cc][e], csv[u]), ga, __uint_as_float(rf[cc][e]));
              }
              o[2 * v4] = Act<__half>::pack2(v[0], v[1]);
              o[2 * v4 + 1] = Act<__half>::pack2(v[2], v[3]);
            }
          }
          sts128(pa, make_uint4(o[0], o[1], o[2], o[3]));
          sts128(pb, make_uint4(o[4], o[5], o[6], o[7]));
        }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the output rows -> visible to the TMA store
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");  // accumulator reads done before the stage is reused
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(bar(OUT_READY, s));
      return ok;
    };

    uint4 nxt[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
    bool ok = true;  // of this warp's waits since the last worker-wide decision
    for (int j = 0; j < n_mine && !failed; ++j, w.next()) {
      const int s = j & 1;
      const int b = w.b, c = w.c, h = w.h;
      const int grp = p.G == 1 ? 0 : h / hpg;  // (no division on the common single-group path: its latency opens every item)
      // per-head constants of this item (global loads issued before the epilogue below, used after it)
      float cs_v = 0.f, D_v = 0.f;
      if (tid < P) cs_v = __fmul_rn(p.C_scale[grp], p.state_scale[h * P + tid]);
      if (dmode == 2 && tid < P) D_v = p.D[h * P + tid];
      if (dmode == 1) D_v = p.D[h];
      const float Scb = p.cb_scale[grp];
      // CB rows of this thread: row block 0 and (C = 256) row block 1, at its quarter of a 64-token source block
      const int8_t* cb0 = p.cb + (((size_t)b * NC + c) * p.G + grp) * (size_t)C * C + (size_t)r * C + 16 * qt;
      auto fetch = [&](int ti) {  // ti is a compile-time constant at every call; two tiles are kept in flight
        const int mb = ti < 2 ? 0 : 1, kb = ti < 2 ? ti : ti - 2;
        if (64 * kb + 16 * qt <= 128 * mb + r) nxt[ti & 1] = __ldg(reinterpret_cast<const uint4*>(cb0 + mb * 128 * C + 64 * kb));
      };
      fetch(0);
      fetch(1);
      if (j >= 1) ok = epilogue(j - 1, ok);
      if (tid < P) {
        sts_f(s_cs + 256 * s + 4 * tid, cs_v);
        sts_f(s_D + 256 * s + 4 * tid, D_v);
      }
      ok = warp_wait(bar(FULL_IN, s), (uint32_t)((j >> 1) & 1)) && ok;  // (the epilogue above returned the warp's verdict so far)
      const uint32_t st = s_stage0 + s * kStageBytes;
      const uint32_t dAs = st + kOffDa;
      if (tid < C) sts_f(s_dts + 4 * tid, __fmul_rn(Scb, lds_f(st + kOffDt + 4 * tid)));
      else if (tid < C + (C >> 4) && tid > C) {  // ratio[g] = exp(dA[16 g] - dA[16 (g-1)]), g = 1 .. C/16 - 1
        const int gq = tid - C;
        sts_f(s_ratio + 4 * gq, exp_decay(__fsub_rn(lds_f(dAs + 64 * gq), lds_f(dAs + 64 * (gq - 1)))));
      }
      if (XBF16) {  // a bf16 x tile becomes fp16 in place (elementwise, so the swizzle does not matter)
#pragma unroll
        for (int i = 0; i < C * 8 / kWorkers; ++i) {
          const uint32_t a = st + (tid + i * kWorkers) * 16;
          const uint4 raw = lds128(a);
          float f[8];
          Act<T>::unpack8(raw, f);
          sts128(a, make_uint4(Act<__half>::pack2(f[0], f[1]), Act<__half>::pack2(f[2], f[3]), Act<__half>::pack2(f[4], f[5]),
                               Act<__half>::pack2(f[6], f[7])));
        }
      }
      if (!worker_and(ok)) { failed = true; break; }  // s_dts, ratio complete (and the tables of the previous item no longer read)
      if (dmode == 1 && tid >= kWorkers - 256) {  // D on the diagonal of a 16 x 16 block, fp16
        const int i = tid - (kWorkers - 256);
        sts_h(s_dvec + 2 * i, __float2half_rn((i >> 4) == (i & 15) ? D_v : 0.f));
      }
      // Two threads per token (C = 256) share its two table rows evenly. The row's own 16-token group, masked to k <= t:
      // eight weights each. The below-group weights of the token as a source, for every later group, as a running product
      // over g: the first thread takes the first half of the groups, the second starts from its own exponential.
      for (int i = tid; i < 2 * C; i += kWorkers) {
        const int t = i >> 1, hf = i & 1, kq = t & ~15;
        const float dAt = lds_f(dAs + 4 * t);
        {
          uint32_t hw[4];
#pragma unroll
          for (int v4 = 0; v4 < 2; ++v4) {
            const int k = kq + 8 * hf + 4 * v4;
            const float4 d = lds_f4(dAs + 4 * k), ws = lds_f4(s_dts + 4 * k);
            const float v0 = (k <= t) ? __fmul_rn(exp_decay(__fsub_rn(dAt, d.x)), ws.x) : 0.f;
            const float v1 = (k + 1 <= t) ? __fmul_rn(exp_decay(__fsub_rn(dAt, d.y)), ws.y) : 0.f;
            const float v2 = (k + 2 <= t) ? __fmul_rn(exp_decay(__fsub_rn(dAt, d.z)), ws.z) : 0.f;
            const float v3 = (k + 3 <= t) ? __fmul_rn(exp_decay(__fsub_rn(dAt, d.w)), ws.w) : 0.f;
            hw[2 * v4] = Act<__half>::pack2(v0, v1);
            hw[2 * v4 + 1] = Act<__half>::pack2(v2, v3);
          }
          sts128(s_dg + 32 * t + 16 * hf, make_uint4(hw[0], hw[1], hw[2], hw[3]));
        }
        const int g0 = (t >> 4) + 1, n = (C >> 4) - g0, n0 = (n + 1) >> 1;  // groups g0 .. C/16 - 1 read this token from below
        const int gs = hf ? g0 + n0 : g0, ge = hf ? (C >> 4) : g0 + n0;
        if (gs < ge) {
          float v = __fmul_rn(exp_decay(__fsub_rn(lds_f(dAs + 64 * gs), dAt)), lds_f(s_dts + 4 * t));
          uint32_t a = s_tab + 2 * (gs * C + t);
          sts_h(a, __float2half_rn(v));
          for (int gq = gs + 1; gq < ge; ++gq) {
            v = __fmul_rn(v, lds_f(s_ratio + 4 * gq));
            a += 2 * C;
            sts_h(a, __float2half_rn(v));
          }
        }
      }
      // row factors of this thread's rows (one per row block)
      uint32_t rfu[MB];
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        const int t = 128 * mb + r;
        const __half2 rf2 = __half2half2(__float2half_rn(exp_decay(__fsub_rn(lds_f(dAs + 4 * t), lds_f(dAs + 4 * (t & ~15))))));
        rfu[mb] = *reinterpret_cast<const uint32_t*>(&rf2);
      }
      worker_and(true);  // tables complete
      // ---- the tiles of M: (row block mb, source block kb); block 0 takes source blocks 0..1, block 1 takes 0..3.
      // No block barrier here: each warp posts its share of a tile on the slot's mbarrier (one arrival per warp), and a
      // slot is rewritten only after the product that read it has completed, so a warp runs at most kRing tiles ahead. A
      // wait that runs out is remembered in `ok` and acted on by all workers together at the next item's barrier.
#pragma unroll
      for (int ti = 0; ti < NT; ++ti, ++g) {
        const int mb = ti < 2 ? 0 : 1, kb = ti < 2 ? ti : ti - 2;
        if (NT % kRing == 0) { slot = ti % kRing; rph = (uint32_t)((ti / kRing) & 1); }
        const int t = 128 * mb + r, g0 = t & ~15;
        const uint4 cq = nxt[ti & 1];
        if (ti + 2 < NT) fetch(ti + 2);
        // A slot is rewritten only after the product that read it has completed. When an item is a whole number of laps of
        // the ring, its first lap needs no wait: this warp has seen the previous item's accumulators complete (epilogue
        // above), and with them every product that read the ring.
        if (NT % kRing == 0 ? ti >= kRing : g >= kRing) ok = warp_wait(bar(RING_EMPTY, slot), rph ^ 1u) && ok;
        const uint32_t srow = s_ring + slot * 16384 + (r >> 3) * 1024 + (r & 7) * 128;
        const int kq = 64 * kb + 16 * qt;
        // weights of this 16-token group for this row: zeros above the diagonal, the row's own masked weights on it, the
        // group table times the row factor below it (selected, not branched); a warp whose 32 rows all lie above the
        // diagonal of this group (about a quarter of all groups) only stores zeros
        uint32_t hw[8];
        if (__all_sync(0xffffffffu, kq > t)) {
#pragma unroll
          for (int e = 0; e < 8; ++e) hw[e] = 0u;
        } else {
          const uint32_t wp = kq > t ? s_zero : (kq == g0 ? s_dg + 32 * t : s_tab + 2 * ((g0 >> 4) * C + kq));
          const uint32_t mult = kq < g0 ? rfu[mb] : 0x3C003C00u;  // half2(1, 1)
          const uint32_t ap = (dmode == 1 && kq == g0) ? s_dvec + 32 * (t & 15) : s_zero;  // + D on the diagonal element
          const uint4 wa = lds128(wp), wb = lds128(wp + 16);
          const uint4 aa = lds128(ap), ab = lds128(ap + 16);
          const uint32_t av[8] = {aa.x, aa.y, aa.z, aa.w, ab.x, ab.y, ab.z, ab.w};
          const uint32_t wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
          const uint32_t cw[4] = {cq.x, cq.y, cq.z, cq.w};
#pragma unroll
          for (int e4 = 0; e4 < 4; ++e4) {
            uint32_t h01, h23;
            s8x4_to_h2x2(cw[e4], h01, h23);
            hw[2 * e4] = hfma2u(hmul2u(h01, wv[2 * e4]), mult, av[2 * e4]);
            hw[2 * e4 + 1] = hfma2u(hmul2u(h23, wv[2 * e4 + 1]), mult, av[2 * e4 + 1]);
          }
        }
        sts128(srow + (((2 * qt) ^ (r & 7)) << 4), make_uint4(hw[0], hw[1], hw[2], hw[3]));
        sts128(srow + (((2 * qt + 1) ^ (r & 7)) << 4), make_uint4(hw[4], hw[5], hw[6], hw[7]));
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(RING_FULL, slot));
        if (++slot == kRing) { slot = 0; rph ^= 1u; }
      }
    }
    if (!failed && n_mine > 0 && !epilogue(n_mine - 1, ok)) failed = true;
    if (failed && lane == 0 && status != nullptr) atomicExch(status, 1);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == kProducerWarp) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tbase), "r"(512u) : "memory");
}

// ------------------------------------------------------------------------------------------------ host side
static int encode_map4(CUtensorMap* m, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* gdim,
                       const cuuint64_t* gstride_bytes, const cuuint32_t* box, const char* what) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(LQ_ERR_LAUNCH, "%s: the driver does not export cuTensorMapEncodeTiled", what);
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(m, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride_bytes, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LQ_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, (int)r);
  return LQ_OK;
}

template <typename T, int MB>
static cudaError_t launch_scan_tc(int grid, size_t smem, cudaStream_t st, const CUtensorMap& tq, const CUtensorMap& ts, const CUtensorMap& tx,
                             const CUtensorMap& to, const lq_ssd_problem* p, int* status, int items) {
  cudaError_t e = cudaFuncSetAttribute(ssd_chunk_scan_tc_kernel<T, MB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) ssd_chunk_scan_tc_kernel<T, MB><<<grid, scantc::kWorkers + 64, smem, st>>>(tq, ts, tx, to, *p, status, items);
  return e;
}

// d_state 128, chunk 128 or 256, headdim 64; every tensor map covers memory of the launching GPU only
int run_chunk_scan_tc(const lq_ssd_problem* p, int* status, cudaStream_t st) {
  const int C = p->chunk, NC = p->L / C;
  if ((reinterpret_cast<uintptr_t>(p->out) & 15u) || (reinterpret_cast<uintptr_t>(p->q_C) & 15u) || (reinterpret_cast<uintptr_t>(p->passed) & 15u) ||
      (reinterpret_cast<uintptr_t>(p->dA) & 15u) || (reinterpret_cast<uintptr_t>(p->dt) & 15u) || (reinterpret_cast<uintptr_t>(p->cb) & 15u))
    return fail(LQ_ERR_ALIGN, "chunk_scan: out, q_C, cb, the passed states, dA and dt must be 16-byte aligned");
  const long long items = (long long)p->B * NC * p->H;
  if (items > 0x7fffffffLL) return fail(LQ_ERR_SHAPE, "chunk_scan: too many (batch, chunk, head) items");
  CUtensorMap tq, ts, tx, to;
  {
    const cuuint64_t gdim[2] = {(cuuint64_t)p->G * 128, (cuuint64_t)p->B * p->L};
    const cuuint64_t gstr[1] = {(cuuint64_t)p->G * 128};
    const cuuint32_t box[2] = {128, 128};
    if (int e = encode_map4(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, p->q_C, gdim, gstr, box, "chunk_scan (q_C)")) return e;
  }
  {
    const cuuint64_t gdim[2] = {128, (cuuint64_t)p->B * NC * p->H * 64};
    const cuuint64_t gstr[1] = {128};
    const cuuint32_t box[2] = {128, 64};
    if (int e = encode_map4(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, p->passed, gdim, gstr, box, "chunk_scan (states)")) return e;
  }
  {
    // x [B, L, H, 64] with element strides (a view into xBC is fine: strides are multiples of 16 bytes); a batch of one
    // gets a dummy batch stride
    const cuuint64_t gdim[4] = {64, (cuuint64_t)p->H, (cuuint64_t)p->L, (cuuint64_t)p->B};
    const cuuint64_t sb = p->B > 1 ? (cuuint64_t)p->x_stride_b * 2 : (cuuint64_t)p->x_stride_t * 2 * p->L;
    const cuuint64_t gstr[3] = {(cuuint64_t)p->x_stride_h * 2, (cuuint64_t)p->x_stride_t * 2, sb};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)C, 1};
    const CUtensorMapDataType dt = p->x_dtype == LQ_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    if (int e = encode_map4(&tx, dt, 4, p->x, gdim, gstr, box, "chunk_scan (x)")) return e;
  }
  {
    const cuuint64_t gdim[4] = {64, (cuuint64_t)p->H, (cuuint64_t)p->L, (cuuint64_t)p->B};
    const cuuint64_t gstr[3] = {128, (cuuint64_t)p->H * 128, (cuuint64_t)p->L * p->H * 128};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)C, 1};
    if (int e = encode_map4(&to, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, p->out, gdim, gstr, box, "chunk_scan (out)")) return e;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t smem = 2 * (size_t)scantc::kStageBytes + scantc::kRing * 16384 + 2 * 8192 + 1024 + 64 + 64 + 512 + 512 + 512 + 96 + 16 + 1024;
  const int grid = (int)(items < sms ? items : sms);
  cudaError_t e;
  if (p->x_dtype == LQ_F16) e = C == 256 ? launch_scan_tc<__half, 2>(grid, smem, st, tq, ts, tx, to, p, status, (int)items)
                                         : launch_scan_tc<__half, 1>(grid, smem, st, tq, ts, tx, to, p, status, (int)items);
  else e = C == 256 ? launch_scan_tc<__nv_bfloat16, 2>(grid, smem, st, tq, ts, tx, to, p, status, (int)items)
                    : launch_scan_tc<__nv_bfloat16, 1>(grid, smem, st, tq, ts, tx, to, p, status, (int)items);
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "chunk_scan: shared memory opt-in failed: %s", cudaGetErrorString(e));
  return check_launch("ssd_chunk_scan_tc_kernel");
}

}  // namespace lq
