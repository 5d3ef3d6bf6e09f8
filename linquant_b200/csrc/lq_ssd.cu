// Mamba-2 SSD op surface, SSDi8 arithmetic lineage: chunk cumsum, INT8 chunk states (value- and key-side
// absorption), INT32 fixed-point state passing, INT8 C.B^T, and the chunk scan.
//
// Reference arithmetic: linquant/kernels/mamba2/{chunk_cumsum,chunk_state,chunk_state_keyside,state_passing,
// bmm_chunk,chunk_scan_v2}.py (line ranges at each kernel).
#include <mutex>
#include <type_traits>

#include "lq_common.cuh"

namespace lq {

__device__ __forceinline__ int round_half_away(float y, float lim) {
  y = fminf(fmaxf(y, -lim), lim);
  return __float2int_rz(__fadd_rn(y, copysignf(0.5f, y)));
}
__device__ __forceinline__ int round_rint(float y, float lo, float hi) {
  return __float2int_rn(fminf(fmaxf(y, lo), hi));
}

// ------------------------------------------------------------------------------------------------ cumsum
// mamba2/chunk_cumsum.py:52-74. One CTA per (chunk, batch) takes the chunk's dt rows for ALL heads, which are one
// contiguous block of C * H floats in memory (16-byte loads, fully coalesced), transforms them and parks them in shared
// memory; each warp then scans heads with the token index across its lanes, so both outputs are written with the token
// index contiguous. The running sum is kept in double and rounded to fp32 per prefix: a warp scan per 32 tokens plus a
// carry.
__global__ void __launch_bounds__(1024) ssd_cumsum_kernel(lq_ssd_problem p) {
  extern __shared__ float s_dtv[];  // [C][H + 1]
  const int c = blockIdx.x, b = blockIdx.y;
  const int C = p.chunk, NC = p.L / C, H = p.H, LD = H + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float a_scale = p.A_log_scale_dev ? *p.A_log_scale_dev : p.A_log_scale;
  const float d_scale = p.dt_scale_dev ? *p.dt_scale_dev : p.dt_scale;
  {
    const float* src = p.dt_in + ((size_t)b * p.L + (size_t)c * C) * H;
    const int total = C * H;
    auto put = [&](int i, float x) {
      const int t = i / H, h = i - t * H;
      x = __fmul_rn(d_scale, x);
      if (p.dt_bias) x = __fadd_rn(x, p.dt_bias[h]);
      if (p.dt_softplus) x = x > 20.f ? x : logf(__fadd_rn(1.0f, expf(x)));
      s_dtv[t * LD + h] = fminf(fmaxf(x, p.dt_min), p.dt_max);
    };
    if ((total & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
      for (int i = 4 * threadIdx.x; i < total; i += 4 * blockDim.x) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(src + i));
        put(i, v.x); put(i + 1, v.y); put(i + 2, v.z); put(i + 3, v.w);
      }
    } else {
      for (int i = threadIdx.x; i < total; i += blockDim.x) put(i, __ldg(src + i));
    }
  }
  __syncthreads();
  for (int h = warp; h < H; h += (int)(blockDim.x >> 5)) {
    const float A = -expf(__fmul_rn(a_scale, p.A_log[h]));
    const size_t obase = (((size_t)b * H + h) * NC + c) * C;
    double carry = 0.0;
    for (int t0 = 0; t0 < C; t0 += 32) {
      const float x = s_dtv[(t0 + lane) * LD + h];
      p.dt[obase + t0 + lane] = x;
      double v = (double)__fmul_rn(x, A);
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const double o = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += o;
      }
      v += carry;
      p.dA[obase + t0 + lane] = (float)v;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
  }
}

// ------------------------------------------------------------------------------------------------ B transpose
// q_B [B,L,G,N] -> q_BT [B,NC,G,N,C] (token index contiguous) so both operands of the value-side chunk-state
// product have the reduction index contiguous. One CTA per (64-token block, group, batch).
__global__ void __launch_bounds__(256) ssd_transpose_b_kernel(const int8_t* qB, int8_t* qBT, int L, int G, int N, int C) {
  __shared__ uint32_t s[128][17];
  const int blk = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int t0 = blk * 64;
  const int c = t0 / C, tc = t0 % C;
  const int tid = threadIdx.x;
  // thread: token group tg (4 tokens) x 4 consecutive channels
  for (int i = tid; i < 16 * (N / 4); i += 256) {
    const int tg = i / (N / 4), n4 = i % (N / 4);
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      w[k] = *reinterpret_cast<const uint32_t*>(qB + (((size_t)b * L + t0 + 4 * tg + k) * G + g) * N + 4 * n4);
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      const uint32_t lo = __byte_perm(w[0], w[1], 0x0040 + 0x11 * ch), hi = __byte_perm(w[2], w[3], 0x0040 + 0x11 * ch);
      s[4 * n4 + ch][tg] = __byte_perm(lo, hi, 0x5410);
    }
  }
  __syncthreads();
  const int NC = L / C;
  int8_t* dst = qBT + ((((size_t)b * NC + c) * G + g) * N) * C + tc;
  for (int i = tid; i < N * 16; i += 256) {
    const int n = i >> 4, w = i & 15;
    *reinterpret_cast<uint32_t*>(dst + (size_t)n * C + 4 * w) = s[n][w];
  }
}

// ------------------------------------------------------------------------------------------------ state passing
// mamba2/state_passing.py:55-93: s32 <- ((s32 * gate_q + 64) >> 7) + new, gate_q = clamp(half_away(exp(dA_last)*128)),
// out[:, c] = clamp(s32 entering chunk c), final = clamp(s32 after the last chunk). Eight state bytes per thread.
//
// The unclamped INT32 carry can enter and leave the call (carry_in / carry_out), which is what makes a sequence cut
// into segments -- several calls, or one segment per GPU -- reproduce the one-shot result bit for bit. In the
// sequence-parallel mode carry_out and post_flags point into the NEXT GPU's memory: each CTA stores its slice of the
// carry with plain stores, makes them visible system-wide and then posts its own flag; the next GPU's CTA of the same
// index polls its local flag for a bounded time before it reads carry_in.
struct PassingLink {
  const int* carry_in;
  int* carry_out;
  const unsigned* wait_flags;
  unsigned* post_flags;
  unsigned epoch;
  unsigned long long wait_ns;
  int* status;
};
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(256) ssd_state_passing_kernel(const int8_t* states, const float* dA, int8_t* out,
                                                                int8_t* final_state, int H, int NC, int C, int D,
                                                                PassingLink link) {
  extern __shared__ int s_gq[];  // [NC] Q0.7 gate of every chunk: the serial loop must not wait on its loads
  __shared__ int s_ok;
  const int h = blockIdx.y, b = blockIdx.z;
  const size_t cta = ((size_t)b * H + h) * gridDim.x + blockIdx.x;
  {
    const float* dAl = dA + (((size_t)b * H + h) * NC) * C + (C - 1);
    for (int c = threadIdx.x; c < NC; c += 256) s_gq[c] = round_half_away(__fmul_rn(expf(dAl[(size_t)c * C]), 128.f), 127.f);
  }
  if (link.wait_flags != nullptr && threadIdx.x == 0) {
    // bounded poll of this CTA's flag: a time limit on the global timer, and an iteration limit as a second guard
    const unsigned long long limit = link.wait_ns ? link.wait_ns : 2000000000ull;
    const unsigned long long t0 = globaltimer_ns();
    int ok = 0;
    const long long max_it = (long long)(limit >> 6) + 1024;  // each round costs at least the 200 ns sleep
    for (long long it = 0; it < max_it; ++it) {
      if (ld_acquire_sys(link.wait_flags + cta) >= link.epoch) { ok = 1; break; }
      if (globaltimer_ns() - t0 > limit) break;
      __nanosleep(200);
    }
    s_ok = ok;
    if (!ok && link.status != nullptr) atomicExch(link.status, 2);
  }
  __syncthreads();
  if (link.wait_flags != nullptr && !s_ok) return;  // nothing stored, nothing posted: the host reads the status word
  // eight state bytes per thread: the walk over the chunks is serial, so the threads have to be many
  const int d0 = (blockIdx.x * 256 + threadIdx.x) * 8;
  const bool live = d0 < D;
  int s32[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) s32[i] = 0;
  if (live && link.carry_in != nullptr) {
    const int4* ci = reinterpret_cast<const int4*>(link.carry_in + ((size_t)b * H + h) * D + d0);
    const int4 lo = ci[0], hi = ci[1];
    s32[0] = lo.x; s32[1] = lo.y; s32[2] = lo.z; s32[3] = lo.w;
    s32[4] = hi.x; s32[5] = hi.y; s32[6] = hi.z; s32[7] = hi.w;
  }
  if (live) {
    // stored copy: clamp to +-127 (the lower bound by hand, the saturating pack gives the upper one)
    auto codes = [&]() {
      int m[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) m[i] = max(s32[i], -127);
      return make_uint2(pack_sat_s8x2(m[1], m[0], pack_sat_s8x2(m[3], m[2], 0u)), pack_sat_s8x2(m[5], m[4], pack_sat_s8x2(m[7], m[6], 0u)));
    };
    const size_t cstride = (size_t)H * D;
    const int8_t* src = states + ((size_t)b * NC * H + h) * D + d0;
    int8_t* dst = out + ((size_t)b * NC * H + h) * D + d0;
    constexpr int DEPTH = 4;  // chunk tiles in flight per thread
    uint2 ring[DEPTH];
#pragma unroll
    for (int u = 0; u < DEPTH; ++u)
      if (u < NC) ring[u] = __ldg(reinterpret_cast<const uint2*>(src + (size_t)u * cstride));
    for (int c0 = 0; c0 < NC; c0 += DEPTH) {
#pragma unroll
      for (int u = 0; u < DEPTH; ++u) {
        const int c = c0 + u;
        if (c >= NC) break;
        const uint2 cur = ring[u];
        if (c + DEPTH < NC) ring[u] = __ldg(reinterpret_cast<const uint2*>(src + (size_t)(c + DEPTH) * cstride));
        *reinterpret_cast<uint2*>(dst + (size_t)c * cstride) = codes();
        const int gq = s_gq[c];
        const uint32_t cw[2] = {cur.x, cur.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int nw = (int)(int8_t)((cw[i >> 2] >> (8 * (i & 3))) & 0xff);
          s32[i] = ((s32[i] * gq + 64) >> 7) + nw;
        }
      }
    }
    *reinterpret_cast<uint2*>(final_state + ((size_t)b * H + h) * D + d0) = codes();
    if (link.carry_out != nullptr) {
      int4* co = reinterpret_cast<int4*>(link.carry_out + ((size_t)b * H + h) * D + d0);
      co[0] = make_int4(s32[0], s32[1], s32[2], s32[3]);
      co[1] = make_int4(s32[4], s32[5], s32[6], s32[7]);
    }
  }
  if (link.post_flags != nullptr) {
    __threadfence_system();  // every thread's carry stores before the flag
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(link.post_flags + cta, link.epoch);
  }
}

// ------------------------------------------------------------------------------------------------ chunk state
// One CTA per (chunk, head, batch), headdim 64: states[p, n] = sum_k xq[k, p] * Bq[k, n] over the chunk's tokens.
// Both operands need the token index contiguous: x is quantised on the fly and transposed through shared memory
// (four tokens packed per word); value side reads the pre-transposed INT8 B straight from global memory, key side
// quantises the gate-weighted B per head into shared memory the same way.
//   value side  mamba2/chunk_state.py:186-246        xq = half_away((x / alpha_p) * gate_k), requant (alpha/S_out)*bscale_g
//   key side    mamba2/chunk_state_keyside.py:267-321  xq = rint(x / x_scale_p), Bq = rint(B*gate_k*127/bg_n), rint requant
template <typename T, int N, bool KEYSIDE>
__global__ void __launch_bounds__(128) ssd_chunk_state_kernel(lq_ssd_problem p) {
  constexpr int P = 64, LDW = 20;
  __shared__ __align__(16) uint32_t s_x[2][P][LDW];
  __shared__ __align__(16) uint32_t s_b[KEYSIDE ? 2 : 1][KEYSIDE ? N : 1][LDW];
  __shared__ float s_gate[256];
  extern __shared__ __align__(16) uint8_t s_raw[];  // [C][128 B]: the chunk's x rows as stored, fetched up front

  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int C = p.chunk, NC = p.L / C, grp = h / (p.H / p.G);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;

  {
    const T* xrow = reinterpret_cast<const T*>(p.x) + (size_t)b * p.x_stride_b + (size_t)h * p.x_stride_h;
    for (int i = tid; i < C * 8; i += 128) {
      const int row = i >> 3, ch = i & 7;
      cp_async16(s_raw + row * 128 + ch * 16, xrow + (size_t)(c * C + row) * p.x_stride_t + 8 * ch);
    }
    cp_async_commit();
  }
  const size_t cbase = (((size_t)b * p.H + h) * NC + c) * C;
  {
    const float last = p.dA[cbase + C - 1];
    for (int t = tid; t < C; t += 128) s_gate[t] = __fmul_rn(expf(__fsub_rn(last, p.dA[cbase + t])), p.dt[cbase + t]);
  }
  float xinv[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int pp = 2 * lane + e;
    xinv[e] = KEYSIDE ? 1.0f / fmaxf(p.x_scale_hp[h * P + pp], 1e-10f) : 1.0f / p.alpha_hp[h * P + pp];
  }
  float binv[KEYSIDE ? N / 32 : 1];
  const float* bgs = nullptr;
  if (KEYSIDE) {
    bgs = p.b_gate_scale + b * p.bgs_stride[0] + c * p.bgs_stride[1] + h * p.bgs_stride[2];
#pragma unroll
    for (int q = 0; q < N / 32; ++q) binv[q] = 127.0f / bgs[(64 * (q >> 1) + 2 * lane + (q & 1)) * p.bgs_stride[3]];
  }
  cp_async_wait<0>();
  __syncthreads();

  const T* bp = reinterpret_cast<const T*>(p.b_fp);
  const int8_t* qbt = KEYSIDE ? nullptr : p.q_BT + ((((size_t)b * NC + c) * p.G + grp) * N) * C;

  int acc[N / 8][4];
#pragma unroll
  for (int nt = 0; nt < N / 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0;

  for (int s = 0; s < C / 64; ++s) {
    const int buf = s & 1;
    for (int tg = warp; tg < 16; tg += 4) {
      uint32_t w0 = 0u, w1 = 0u;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = 64 * s + 4 * tg + i;
        const uint32_t raw = *reinterpret_cast<const uint32_t*>(s_raw + t * 128 + 4 * lane);
        float x0, x1;
        if (sizeof(T) == 2 && std::is_same<T, __half>::value) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&raw));
          x0 = f.x; x1 = f.y;
        } else {
          x0 = __uint_as_float(raw << 16); x1 = __uint_as_float(raw & 0xffff0000u);
        }
        int c0, c1;
        if (KEYSIDE) {
          c0 = round_rint(__fmul_rn(x0, xinv[0]), -127.f, 127.f);
          c1 = round_rint(__fmul_rn(x1, xinv[1]), -127.f, 127.f);
        } else {
          const float gk = s_gate[t];
          c0 = round_half_away(__fmul_rn(__fmul_rn(x0, xinv[0]), gk), 127.f);
          c1 = round_half_away(__fmul_rn(__fmul_rn(x1, xinv[1]), gk), 127.f);
        }
        w0 |= ((uint32_t)c0 & 0xffu) << (8 * i);
        w1 |= ((uint32_t)c1 & 0xffu) << (8 * i);
      }
      s_x[buf][2 * lane][tg] = w0;
      s_x[buf][2 * lane + 1][tg] = w1;
    }
    if (KEYSIDE) {
      for (int tg = warp; tg < 16; tg += 4) {
#pragma unroll
        for (int half = 0; half < N / 64; ++half) {
          uint32_t w0 = 0u, w1 = 0u;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int t = 64 * s + 4 * tg + i;
            const uint32_t raw = *reinterpret_cast<const uint32_t*>(
                bp + (((size_t)b * p.L + (size_t)c * C + t) * p.G + grp) * N + 64 * half + 2 * lane);
            float x0, x1;
            if (std::is_same<T, __half>::value) {
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&raw));
              x0 = f.x; x1 = f.y;
            } else {
              x0 = __uint_as_float(raw << 16); x1 = __uint_as_float(raw & 0xffff0000u);
            }
            const float gk = s_gate[t];
            const int c0 = round_rint(__fmul_rn(__fmul_rn(x0, gk), binv[2 * half]), -127.f, 127.f);
            const int c1 = round_rint(__fmul_rn(__fmul_rn(x1, gk), binv[2 * half + 1]), -127.f, 127.f);
            w0 |= ((uint32_t)c0 & 0xffu) << (8 * i);
            w1 |= ((uint32_t)c1 & 0xffu) << (8 * i);
          }
          s_b[KEYSIDE ? buf : 0][KEYSIDE ? 64 * half + 2 * lane : 0][tg] = w0;
          s_b[KEYSIDE ? buf : 0][KEYSIDE ? 64 * half + 2 * lane + 1 : 0][tg] = w1;
        }
      }
    }
    __syncthreads();
    const uint4 xa = *reinterpret_cast<const uint4*>(&s_x[buf][16 * warp + g][4 * j]);
    const uint4 xb = *reinterpret_cast<const uint4*>(&s_x[buf][16 * warp + g + 8][4 * j]);
#pragma unroll
    for (int nt = 0; nt < N / 8; ++nt) {
      const int nr = 32 * (nt >> 2) + 8 * (g >> 1) + 2 * (nt & 3) + (g & 1);
      uint4 bq;
      if (KEYSIDE) bq = *reinterpret_cast<const uint4*>(&s_b[KEYSIDE ? buf : 0][KEYSIDE ? nr : 0][4 * j]);
      else bq = __ldg(reinterpret_cast<const uint4*>(qbt + (size_t)nr * C + 64 * s + 16 * j));
      mma_s8(acc[nt], xa.x, xb.x, xa.y, xb.y, bq.x, bq.y);
      mma_s8(acc[nt], xa.z, xb.z, xa.w, xb.w, bq.z, bq.w);
    }
  }

  // epilogue: requantise to INT8, eight consecutive state channels per thread and row
  const int pa = 16 * warp + g, pb = pa + 8;
  int8_t* st = p.states + ((((size_t)b * NC + c) * p.H + h) * P) * N;
  float ra, rb;
  if (KEYSIDE) {
    ra = p.x_scale_hp[h * P + pa] / p.state_scale[h * P + pa];
    rb = p.x_scale_hp[h * P + pb] / p.state_scale[h * P + pb];
  } else {
    const float bs = p.bscale_g[grp];
    ra = __fmul_rn(p.alpha_hp[h * P + pa] / p.state_scale[h * P + pa], bs);
    rb = __fmul_rn(p.alpha_hp[h * P + pb] / p.state_scale[h * P + pb], bs);
  }
#pragma unroll
  for (int ng = 0; ng < N / 32; ++ng) {
    int ca[8], cb[8];
#pragma unroll
    for (int n4 = 0; n4 < 4; ++n4) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int i = 2 * n4 + e;
        const float fa = (float)acc[4 * ng + n4][e], fb = (float)acc[4 * ng + n4][2 + e];
        if (KEYSIDE) {
          const float sn = bgs[(32 * ng + 8 * j + i) * p.bgs_stride[3]] / 127.0f;
          ca[i] = round_rint(__fmul_rn(__fmul_rn(fa, sn), ra), -127.f, 127.f);
          cb[i] = round_rint(__fmul_rn(__fmul_rn(fb, sn), rb), -127.f, 127.f);
        } else {
          ca[i] = round_half_away(__fmul_rn(fa, ra), 127.f);
          cb[i] = round_half_away(__fmul_rn(fb, rb), 127.f);
        }
      }
    }
    *reinterpret_cast<uint2*>(st + (size_t)pa * N + 32 * ng + 8 * j) =
        make_uint2(pack4(ca[0], ca[1], ca[2], ca[3]), pack4(ca[4], ca[5], ca[6], ca[7]));
    *reinterpret_cast<uint2*>(st + (size_t)pb * N + 32 * ng + 8 * j) =
        make_uint2(pack4(cb[0], cb[1], cb[2], cb[3]), pack4(cb[4], cb[5], cb[6], cb[7]));
  }
}

// ------------------------------------------------------------------------------------------------ C.B^T
// mamba2/bmm_chunk.py:103-139: cb[m, n] = rint( int32(C_i8[m,:] . B_i8[n,:]) * (s_C*s_B/S_cb) ) clamped to +-127.
// One CTA per 64x64 output tile; fragments come straight from global memory (the state index is contiguous in both
// operands). B_IS_FP quantises B in the fragment load: rint(b / s_B), clamp +-127.
template <typename T, int N, bool B_IS_FP>
__global__ void __launch_bounds__(128) ssd_bmm_kernel(lq_ssd_problem p) {
  const int C = p.chunk, NC = p.L / C;
  const int tiles = C / 64;
  const int m0 = (blockIdx.x / tiles) * 64, n0 = (blockIdx.x % tiles) * 64;
  const int c = blockIdx.y / p.G, grp = blockIdx.y % p.G, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, j = lane & 3;
  const int ma = m0 + 16 * warp + g, mb = ma + 8;
  const size_t rowC = ((size_t)b * p.L + (size_t)c * C) * p.G + grp;  // + token * G
  const float a_sc = p.C_scale[grp], b_sc = p.B_scale[grp];
  const float b_inv = 1.0f / b_sc;
  uint4 qa[N / 64], qb[N / 64];
#pragma unroll
  for (int kk = 0; kk < N / 64; ++kk) {
    qa[kk] = __ldg(reinterpret_cast<const uint4*>(p.q_C + (rowC + (size_t)ma * p.G) * N + 64 * kk + 16 * j));
    qb[kk] = __ldg(reinterpret_cast<const uint4*>(p.q_C + (rowC + (size_t)mb * p.G) * N + 64 * kk + 16 * j));
  }
  const float inv_scb = __fmul_rn(a_sc, b_sc) / p.cb_scale[grp];
  int8_t* out = p.cb + (((size_t)b * NC + c) * p.G + grp) * C * C;
#pragma unroll
  for (int ng = 0; ng < 2; ++ng) {
    int ca[8], cb[8];
#pragma unroll
    for (int n4 = 0; n4 < 4; ++n4) {
      const int tok = n0 + 32 * ng + 8 * (g >> 1) + 2 * n4 + (g & 1);
      int acc[4] = {0, 0, 0, 0};
#pragma unroll
      for (int kk = 0; kk < N / 64; ++kk) {
        uint4 bq;
        if (B_IS_FP) {
          const T* bp = reinterpret_cast<const T*>(p.b_fp) + (rowC + (size_t)tok * p.G) * N + 64 * kk + 16 * j;
          float x[16];
          float (&x0)[8] = *reinterpret_cast<float (*)[8]>(&x[0]);
          float (&x1)[8] = *reinterpret_cast<float (*)[8]>(&x[8]);
          Act<T>::unpack8(__ldg(reinterpret_cast<const uint4*>(bp)), x0);
          Act<T>::unpack8(__ldg(reinterpret_cast<const uint4*>(bp + 8)), x1);
          int cd[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) cd[i] = round_rint(__fmul_rn(x[i], b_inv), -127.f, 127.f);
          bq = make_uint4(pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]),
                          pack4(cd[8], cd[9], cd[10], cd[11]), pack4(cd[12], cd[13], cd[14], cd[15]));
        } else {
          bq = __ldg(reinterpret_cast<const uint4*>(p.q_B + (rowC + (size_t)tok * p.G) * N + 64 * kk + 16 * j));
        }
        mma_s8(acc, qa[kk].x, qb[kk].x, qa[kk].y, qb[kk].y, bq.x, bq.y);
        mma_s8(acc, qa[kk].z, qb[kk].z, qa[kk].w, qb[kk].w, bq.z, bq.w);
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        ca[2 * n4 + e] = round_rint(__fmul_rn((float)acc[e], inv_scb), -127.f, 127.f);
        cb[2 * n4 + e] = round_rint(__fmul_rn((float)acc[2 + e], inv_scb), -127.f, 127.f);
      }
    }
    *reinterpret_cast<uint2*>(out + (size_t)ma * C + n0 + 32 * ng + 8 * j) =
        make_uint2(pack4(ca[0], ca[1], ca[2], ca[3]), pack4(ca[4], ca[5], ca[6], ca[7]));
    *reinterpret_cast<uint2*>(out + (size_t)mb * C + n0 + 32 * ng + 8 * j) =
        make_uint2(pack4(cb[0], cb[1], cb[2], cb[3]), pack4(cb[4], cb[5], cb[6], cb[7]));
  }
}

// ------------------------------------------------------------------------------------------------ chunk scan
// mamba2/chunk_scan_v2.py:160-256. One CTA per (chunk, head, batch), headdim 64; a warp owns one 16-row tile of the
// chunk at a time (light and heavy causal rows paired). All INT8 tiles and the x tile (fp16) are staged in shared
// memory once.
//   out[m,:] = int32(C_i8[m,:] . S_i8) s_C s_state[p] exp(dA_m)
//            + sum_{k<=m} fp16(cb[m,k] S_cb exp(dA_m - dA_k) dt_k) fp16(x[k,:]) + D x[m,:]
// With r = the first row of the warp's tile the decay splits as exp(dA_m - dA_r) exp(dA_r - dA_k) for k < r (both
// exponents <= 0), so one fp32 accumulator serves everything:
//   acc  = int32(C.S) s_C s_state[p] exp(dA_r)                      state read, entered at the tile's first row
//   acc += fp16(cb) * fp16(S_cb exp(dA_r - dA_k) dt_k) . x          tiles strictly below the diagonal: the codes go to
//                                                                   fp16 exactly, one half2 multiply per two elements
//   acc *= exp(dA_m - dA_r)                                         row factor, once
//   acc += fp16(cb S_cb exp(dA_m - dA_k) dt_k, k <= m) . x          the diagonal tile, evaluated per element
template <int IMM>
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4+%5];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr), "n"(IMM));
}
// exp(x) as ex2.approx.ftz(x log2 e): decay factors only, where a denormal result may as well be zero
__device__ __forceinline__ float exp_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(__fmul_rn(x, 1.4426950408889634f)));
  return y;
}
// Two INT8 codes (bytes LO and LO+1 of w, each XOR 0x80) times a half2 factor: the bytes become the low mantissa
// bits of 1024 in fp16 (exact), 1152 is subtracted (exact) and the product is rounded once.
template <int LO>
__device__ __forceinline__ uint32_t codes_times_half2(uint32_t w_xor80, uint32_t factor) {
  const uint32_t bits = __byte_perm(w_xor80, 0x64646464u, LO == 0 ? 0x5140 : 0x7362);
  const __half2 c = __hsub2(*reinterpret_cast<const __half2*>(&bits), __half2half2(__ushort_as_half((unsigned short)0x6480)));
  const __half2 r = __hmul2(c, *reinterpret_cast<const __half2*>(&factor));
  return *reinterpret_cast<const uint32_t*>(&r);
}
// One k16 step of the causal product: A fragment af against 64 value channels whose x rows ldmatrix reads at
// base[n2] ^ xorv (+ IMM bytes).
template <int IMM>
__device__ __forceinline__ void scan_kstep(float (&conv)[8][4], const uint32_t (&af)[4], uint32_t base, uint32_t xorv) {
  // the four fragment loads go out together: the assembly statements issue in program order, and a load placed
  // between two tiles' products would expose its latency four times per step. Value-tile pair n2 sits 32 n2 bytes
  // further along the swizzled row, which is an XOR on the same address bits as the step's.
  uint32_t r[4][4];
#pragma unroll
  for (int n2 = 0; n2 < 4; ++n2) ldsm_x4_trans<IMM>(r[n2], base ^ (xorv ^ (uint32_t)(n2 << 5)));
#pragma unroll
  for (int n2 = 0; n2 < 4; ++n2) {
    mma_f16(conv[2 * n2], af[0], af[1], af[2], af[3], r[n2][0], r[n2][1]);
    mma_f16(conv[2 * n2 + 1], af[0], af[1], af[2], af[3], r[n2][2], r[n2][3]);
  }
}

template <typename T, int N>
__global__ void __launch_bounds__(256, 2) ssd_chunk_scan_kernel(lq_ssd_problem p) {
  constexpr int P = 64;
  extern __shared__ __align__(128) uint8_t smem[];
  const int C = p.chunk, NC = p.L / C;
  // x tile [C][128 B] fp16; the 16-byte piece ch of row r sits at piece ch ^ f(r), f(r) = (((r>>4)^(r>>2))&3)<<1 | (r&1):
  // both row orders ldmatrix uses below (16a+b and 4a+b, a = 0..3, b = 0..1) then touch eight different pieces
  uint8_t* s_x = smem;
  float* s_dA = reinterpret_cast<float*>(smem + (size_t)C * 128);
  float* s_dts = s_dA + C;                                   // S_cb * dt
  __half* s_tab = reinterpret_cast<__half*>(s_dts + C);      // [8 warps][C] fp16 below-diagonal factors of the warp's tile
  int8_t* s_S = reinterpret_cast<int8_t*>(s_tab + 8 * C);    // [64][N] INT8 state entering the chunk
  float* s_cs = reinterpret_cast<float*>(s_S + 64 * N);      // [64] s_C * state scale, [64] D
  float* s_D = s_cs + 64;
  // byte offset of 16-byte piece `ch` of row `row` in the two INT8 tiles: an MMA fragment load touches two rows x
  // four pieces per quarter-warp, so odd rows swap their 64-byte halves (rows of 64 bytes interleave by themselves)
  auto frag_off = [](int row, int ch) { return N == 128 ? row * 128 + ((ch ^ ((row & 1) << 2)) << 4) : row * 64 + (ch << 4); };
  auto x_piece = [](int row, int ch) { return ch ^ (((((row >> 4) ^ (row >> 2)) & 3) << 1) | (row & 1)); };

  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int grp = h / (p.H / p.G);
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // tells the compiler the tile index is warp-uniform
  const int g = lane >> 2, j = lane & 3;
  const size_t cbase = (((size_t)b * p.H + h) * NC + c) * C;

  const int8_t* qc = p.q_C + (((size_t)b * p.L + (size_t)c * C) * p.G + grp) * N;
  const int8_t* sp = p.passed + ((((size_t)b * NC + c) * p.H + h) * P) * N;
  for (int i = tid; i < 64 * (N / 16); i += 256) {
    const int row = i / (N / 16), ch = i % (N / 16);
    cp_async16(s_S + frag_off(row, ch), sp + (size_t)row * N + 16 * ch);
  }
  const float Scb = p.cb_scale[grp];
  for (int t = tid; t < C; t += 256) {
    s_dA[t] = p.dA[cbase + t];
    s_dts[t] = __fmul_rn(Scb, p.dt[cbase + t]);
  }
  if (tid < 64) {
    s_cs[tid] = __fmul_rn(p.C_scale[grp], p.state_scale[h * P + tid]);
    s_D[tid] = p.D == nullptr ? 0.f : (p.D_has_hdim ? p.D[h * P + tid] : p.D[h]);
  }
  {
    const T* xp = reinterpret_cast<const T*>(p.x) + (size_t)b * p.x_stride_b + (size_t)h * p.x_stride_h;
    for (int i = tid; i < C * 8; i += 256) {
      const int row = i >> 3, ch = i & 7;
      if (std::is_same<T, __half>::value) {
        cp_async16(s_x + row * 128 + (x_piece(row, ch) << 4), xp + (size_t)(c * C + row) * p.x_stride_t + 8 * ch);
        continue;
      }
      uint4 raw = __ldg(reinterpret_cast<const uint4*>(xp + (size_t)(c * C + row) * p.x_stride_t + 8 * ch));
      if (!std::is_same<T, __half>::value) {
        float x[8];
        Act<T>::unpack8(raw, x);
        raw = make_uint4(Act<__half>::pack2(x[0], x[1]), Act<__half>::pack2(x[2], x[3]), Act<__half>::pack2(x[4], x[5]),
                         Act<__half>::pack2(x[6], x[7]));
      }
      *reinterpret_cast<uint4*>(s_x + row * 128 + (x_piece(row, ch) << 4)) = raw;
    }
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  const int MT = C / 16;
  const int8_t* cbp = p.cb + (((size_t)b * NC + c) * p.G + grp) * C * C;
  __half* op = reinterpret_cast<__half*>(p.out) + (((size_t)b * p.L + (size_t)c * C) * p.H + h) * P + 2 * j;
  const size_t orow = (size_t)p.H * P;

  // ldmatrix lanes: matrix mi = lane>>3 (k half mi&1, value tile mi>>1), stored row rr = lane&7 <-> MMA k slot
  // 8 (mi&1) + rr, which is token offset a-th group of the lane pair (a = rr>>1) + 2 (mi&1) + (rr&1). Two token
  // orders are used: "grouped" steps cover 64 tokens in four k16 steps, lane j owning tokens 16j + 4u + e of step u
  // (one 16-byte load of CB codes per row and group); "single" steps cover 16 tokens, lane j owning 4j + e.
  const int mi = lane >> 3, rr = lane & 7;
  const uint32_t sx_u32 = (uint32_t)__cvta_generic_to_shared(s_x);
  const uint32_t piece0 = (uint32_t)((mi >> 1) ^ rr) << 4;  // f() of the lane's row without the step bits, value tiles 0/1
  const uint32_t baseG = sx_u32 + (16 * (rr >> 1) + 2 * (mi & 1) + (rr & 1)) * 128 + piece0;
  const uint32_t baseS = sx_u32 + (4 * (rr >> 1) + 2 * (mi & 1) + (rr & 1)) * 128 + piece0;

  for (int it = 0; it * 8 < MT; ++it) {
    const int mt = (it & 1) ? it * 8 + 7 - warp : it * 8 + warp;  // pair light and heavy causal rows
    if (mt >= MT) continue;
    const int ma = 16 * mt + g, mb = ma + 8;
    const int qfull = mt >> 2, rem = mt & 3;
    const float dref = s_dA[16 * mt];
    const float dAa = s_dA[ma], dAb = s_dA[mb];
    const int8_t* cba = cbp + (size_t)ma * C;
    const int8_t* cbb = cbp + (size_t)mb * C;

    // CB codes of the last, partial group (single steps; the diagonal tile is step `rem` of it) and of the first full group
    uint32_t ta[4], tb[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      ta[u] = __ldg(reinterpret_cast<const uint32_t*>(cba + 64 * qfull + 16 * u + 4 * j));
      tb[u] = __ldg(reinterpret_cast<const uint32_t*>(cbb + 64 * qfull + 16 * u + 4 * j));
    }
    // q_C rows of the tile: every code is used once per CTA, so the fragments come straight from global memory
    uint4 qa[N / 64], qb[N / 64];
#pragma unroll
    for (int kk = 0; kk < N / 64; ++kk) {
      qa[kk] = __ldg(reinterpret_cast<const uint4*>(qc + (size_t)ma * p.G * N + 64 * kk + 16 * j));
      qb[kk] = __ldg(reinterpret_cast<const uint4*>(qc + (size_t)mb * p.G * N + 64 * kk + 16 * j));
    }
    uint4 ga = make_uint4(0, 0, 0, 0), gb = ga;
    if (qfull > 0) {
      ga = __ldg(reinterpret_cast<const uint4*>(cba + 16 * j));
      gb = __ldg(reinterpret_cast<const uint4*>(cbb + 16 * j));
    }

    // ---- below-diagonal factors of this tile: tab[k] = fp16(S_cb exp(dA_r - dA_k) dt_k), k < 16 mt
    __half* tab = s_tab + warp * C;
    __syncwarp();
    for (int k = 2 * lane; k < 16 * mt; k += 64) {
      const float2 d = *reinterpret_cast<const float2*>(s_dA + k), t = *reinterpret_cast<const float2*>(s_dts + k);
      *reinterpret_cast<__half2*>(tab + k) =
          __floats2half2_rn(__fmul_rn(exp_ftz(__fsub_rn(dref, d.x)), t.x), __fmul_rn(exp_ftz(__fsub_rn(dref, d.y)), t.y));
    }
    __syncwarp();

    // ---- state read (INT8), entered at the tile's first row
    float conv[8][4];
    {
      const float er = exp_ftz(dref);
      // eight independent accumulator chains: the products of one value tile would otherwise wait on each other
      int acc[8][4];
#pragma unroll
      for (int kk = 0; kk < N / 64; ++kk) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const uint4 bs = *reinterpret_cast<const uint4*>(s_S + frag_off(8 * nt + g, 4 * kk + j));
          if (kk == 0) mma_s8_first(acc[nt], qa[kk].x, qb[kk].x, qa[kk].y, qb[kk].y, bs.x, bs.y);
          else mma_s8(acc[nt], qa[kk].x, qb[kk].x, qa[kk].y, qb[kk].y, bs.x, bs.y);
          mma_s8(acc[nt], qa[kk].z, qb[kk].z, qa[kk].w, qb[kk].w, bs.z, bs.w);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float2 cs = *reinterpret_cast<const float2*>(s_cs + 8 * nt + 2 * j);
        const float c0 = __fmul_rn(cs.x, er), c1 = __fmul_rn(cs.y, er);
        conv[nt][0] = __fmul_rn((float)acc[nt][0], c0);
        conv[nt][1] = __fmul_rn((float)acc[nt][1], c1);
        conv[nt][2] = __fmul_rn((float)acc[nt][2], c0);
        conv[nt][3] = __fmul_rn((float)acc[nt][3], c1);
      }
    }

    // ---- full groups of 64 tokens below the diagonal
    for (int q = 0; q < qfull; ++q) {
      uint4 na = ga, nb = gb;
      if (q + 1 < qfull) {
        na = __ldg(reinterpret_cast<const uint4*>(cba + 64 * (q + 1) + 16 * j));
        nb = __ldg(reinterpret_cast<const uint4*>(cbb + 64 * (q + 1) + 16 * j));
      }
      const uint32_t wa[4] = {ga.x ^ 0x80808080u, ga.y ^ 0x80808080u, ga.z ^ 0x80808080u, ga.w ^ 0x80808080u};
      const uint32_t wb[4] = {gb.x ^ 0x80808080u, gb.y ^ 0x80808080u, gb.z ^ 0x80808080u, gb.w ^ 0x80808080u};
      const uint4 tv0 = *reinterpret_cast<const uint4*>(tab + 64 * q + 16 * j);       // steps 0, 1
      const uint4 tv1 = *reinterpret_cast<const uint4*>(tab + 64 * q + 16 * j + 8);   // steps 2, 3
      const uint32_t tv[8] = {tv0.x, tv0.y, tv0.z, tv0.w, tv1.x, tv1.y, tv1.z, tv1.w};
      const uint32_t bq = baseG + q * 8192;
      {
        const uint32_t af[4] = {codes_times_half2<0>(wa[0], tv[0]), codes_times_half2<0>(wb[0], tv[0]),
                                codes_times_half2<2>(wa[0], tv[1]), codes_times_half2<2>(wb[0], tv[1])};
        scan_kstep<0>(conv, af, bq, 0u);
      }
      {
        const uint32_t af[4] = {codes_times_half2<0>(wa[1], tv[2]), codes_times_half2<0>(wb[1], tv[2]),
                                codes_times_half2<2>(wa[1], tv[3]), codes_times_half2<2>(wb[1], tv[3])};
        scan_kstep<512>(conv, af, bq, 1u << 5);
      }
      {
        const uint32_t af[4] = {codes_times_half2<0>(wa[2], tv[4]), codes_times_half2<0>(wb[2], tv[4]),
                                codes_times_half2<2>(wa[2], tv[5]), codes_times_half2<2>(wb[2], tv[5])};
        scan_kstep<1024>(conv, af, bq, 2u << 5);
      }
      {
        const uint32_t af[4] = {codes_times_half2<0>(wa[3], tv[6]), codes_times_half2<0>(wb[3], tv[6]),
                                codes_times_half2<2>(wa[3], tv[7]), codes_times_half2<2>(wb[3], tv[7])};
        scan_kstep<1536>(conv, af, bq, 3u << 5);
      }
      ga = na;
      gb = nb;
    }
    // ---- single steps of the partial group, below the diagonal (at most three)
    const uint32_t bs_ = baseS + qfull * 8192;
#pragma unroll
    for (int u = 0; u < 3; ++u) {
      if (u < rem) {
        const uint2 tvv = *reinterpret_cast<const uint2*>(tab + 64 * qfull + 16 * u + 4 * j);
        const uint32_t wa = ta[u] ^ 0x80808080u, wb = tb[u] ^ 0x80808080u;
        const uint32_t af[4] = {codes_times_half2<0>(wa, tvv.x), codes_times_half2<0>(wb, tvv.x),
                                codes_times_half2<2>(wa, tvv.y), codes_times_half2<2>(wb, tvv.y)};
        if (u == 0) scan_kstep<0>(conv, af, bs_, 0u);
        if (u == 1) scan_kstep<2048>(conv, af, bs_, 1u << 5);
        if (u == 2) scan_kstep<4096>(conv, af, bs_, 2u << 5);
      }
    }
    // ---- row factor, then the diagonal tile per element
    {
      const float ea = exp_ftz(__fsub_rn(dAa, dref)), eb = exp_ftz(__fsub_rn(dAb, dref));
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        conv[nt][0] *= ea; conv[nt][1] *= ea; conv[nt][2] *= eb; conv[nt][3] *= eb;
      }
      const uint32_t wda = (rem == 0 ? ta[0] : rem == 1 ? ta[1] : rem == 2 ? ta[2] : ta[3]) ^ 0x80808080u;
      const uint32_t wdb = (rem == 0 ? tb[0] : rem == 1 ? tb[1] : rem == 2 ? tb[2] : tb[3]) ^ 0x80808080u;
      const float4 dk4 = *reinterpret_cast<const float4*>(s_dA + 16 * mt + 4 * j);
      const float4 sk4 = *reinterpret_cast<const float4*>(s_dts + 16 * mt + 4 * j);
      const float dk[4] = {dk4.x, dk4.y, dk4.z, dk4.w}, sk[4] = {sk4.x, sk4.y, sk4.z, sk4.w};
      const float fa[4] = {s8_to_float<0>(wda), s8_to_float<1>(wda), s8_to_float<2>(wda), s8_to_float<3>(wda)};
      const float fb[4] = {s8_to_float<0>(wdb), s8_to_float<1>(wdb), s8_to_float<2>(wdb), s8_to_float<3>(wdb)};
      float va[4], vb[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kl = 4 * j + e;  // token within the tile; rows g and g + 8
        va[e] = (g >= kl) ? __fmul_rn(__fmul_rn(fa[e], exp_ftz(__fsub_rn(dAa, dk[e]))), sk[e]) : 0.f;
        vb[e] = (g + 8 >= kl) ? __fmul_rn(__fmul_rn(fb[e], exp_ftz(__fsub_rn(dAb, dk[e]))), sk[e]) : 0.f;
      }
      const uint32_t af[4] = {Act<__half>::pack2(va[0], va[1]), Act<__half>::pack2(vb[0], vb[1]),
                              Act<__half>::pack2(va[2], va[3]), Act<__half>::pack2(vb[2], vb[3])};
      scan_kstep<0>(conv, af, bs_ + rem * 2048, (uint32_t)rem << 5);
    }
    // ---- D*x residual, store fp16
    {
      const uint32_t xa_row = ma * 128 + 4 * j + (x_piece(ma, 0) << 4), xb_row = mb * 128 + 4 * j + (x_piece(mb, 0) << 4);
      __half* oa_p = op + (size_t)ma * orow;
      __half* ob_p = op + (size_t)mb * orow;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float2 xa = __half22float2(*reinterpret_cast<const __half2*>(s_x + (xa_row ^ (nt << 4))));
        const float2 xb = __half22float2(*reinterpret_cast<const __half2*>(s_x + (xb_row ^ (nt << 4))));
        const float2 Dv = *reinterpret_cast<const float2*>(s_D + 8 * nt + 2 * j);
        *reinterpret_cast<uint32_t*>(oa_p + 8 * nt) = Act<__half>::pack2(fmaf(xa.x, Dv.x, conv[nt][0]), fmaf(xa.y, Dv.y, conv[nt][1]));
        *reinterpret_cast<uint32_t*>(ob_p + 8 * nt) = Act<__half>::pack2(fmaf(xb.x, Dv.x, conv[nt][2]), fmaf(xb.y, Dv.y, conv[nt][3]));
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ B/C prologue
// mamba2/fused_split_rotate_xBC.py:90-138 and kernels/hadamard.py:70-103. A row of N state channels is held by
// N/8 lanes; the H_2 (x) H_{N/2} product on bf16-rounded inputs is the full Walsh-Hadamard butterfly scaled by the
// bf16 value of 1/sqrt(N/2) and then by 1/sqrt(2) in fp32.
__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float fp16r(float x) { return __half2float(__float2half_rn(x)); }

template <typename T, int N, bool QUANT>
__global__ void __launch_bounds__(256) ssd_rotate_rows_kernel(const T* x, long long stride_b, long long stride_t,
                                                              long long off_b, long long off_c, int T_len, int G,
                                                              const float* signs, const float* inv_b, const float* inv_c,
                                                              const float* dqk_b, const float* dqk_c, int8_t* q_b,
                                                              int8_t* q_c, T* y, int rows_per_cta) {
  // QUANT: blockIdx.y in [0, 2G) selects (B|C, group); otherwise blockIdx.y is the head and y is the dense output.
  // A CTA walks rows_per_cta consecutive tokens: a row is short (N values), so the per-row constants (signs, D_QK,
  // reciprocal scale) are loaded once per thread and four rows per thread are in flight at a time.
  constexpr int LPR = N / 8, RPW = 32 / LPR, STEP = 8 * RPW, UNROLL = 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane % LPR, sub = lane / LPR;
  const int b = blockIdx.z;
  const int which = QUANT ? blockIdx.y / G : 0, grp = QUANT ? blockIdx.y % G : blockIdx.y;
  const T* src0 = x + (size_t)b * stride_b + (which ? off_c : off_b) + (size_t)grp * N + 8 * r;
  const float* dq = QUANT ? (which ? dqk_c : dqk_b) : nullptr;
  float sg[8], dqv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    sg[i] = signs != nullptr ? signs[grp * N + 8 * r + i] : 1.f;
    dqv[i] = dq != nullptr ? fp16r(dq[grp * N + 8 * r + i]) : 1.f;
  }
  const float inv = QUANT ? (which ? inv_c[grp] : inv_b[grp]) : 1.f;
  const float hs = bf16r(N == 128 ? 0.125f : 0.17677669529663687f);
  const int row_end = min(T_len, (int)(blockIdx.x + 1) * rows_per_cta);
  // the loop bound is warp-uniform (the butterfly shuffles across all lanes of the warp)
  for (int tw = blockIdx.x * rows_per_cta + warp * RPW; tw < row_end; tw += STEP * UNROLL) {
    const int t0 = tw + sub;
    uint4 raw[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int t = t0 + u * STEP;
      // rows past the end are clamped for the load (the shuffles below need every lane) and never stored
      raw[u] = __ldg(reinterpret_cast<const uint4*>(src0 + (size_t)min(t, T_len - 1) * stride_t));
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int t = t0 + u * STEP;
      const bool live = t < row_end;
      float v[8];
      Act<T>::unpack8(raw[u], v);
      if (dq != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = fp16r(__fmul_rn(v[i], dqv[i]));
      }
      if (signs != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = bf16r(__fmul_rn(v[i], sg[i]));
        fwht8<LPR>(v, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(v[i], hs), 0.70710678118654752f);
      }
      if (QUANT) {
        int cd[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) cd[i] = round_rint(__fmul_rn(fp16r(v[i]), inv), -128.f, 127.f);
        if (live) {
          int8_t* dst = (which ? q_c : q_b) + (((size_t)b * T_len + t) * G + grp) * N + 8 * r;
          *reinterpret_cast<uint2*>(dst) = make_uint2(pack4(cd[0], cd[1], cd[2], cd[3]), pack4(cd[4], cd[5], cd[6], cd[7]));
        }
      } else if (live) {
        T* dst = y + (((size_t)b * T_len + t) * G + grp) * N + 8 * r;
        *reinterpret_cast<uint4*>(dst) = make_uint4(Act<T>::pack2(v[0], v[1]), Act<T>::pack2(v[2], v[3]),
                                                    Act<T>::pack2(v[4], v[5]), Act<T>::pack2(v[6], v[7]));
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ launchers
static int ssd_check(const lq_ssd_problem* p, const char* what) {
  if (!p) return fail(LQ_ERR_NULL, "%s: problem descriptor is null", what);
  if (p->B <= 0 || p->L <= 0 || p->H <= 0 || p->G <= 0) return fail(LQ_ERR_SHAPE, "%s: non-positive extent", what);
  if (p->chunk <= 0 || p->chunk % 64 != 0 || p->chunk > 256) return fail(LQ_ERR_UNSUPPORTED, "%s: chunk size %d (64, 128, 192 or 256 supported)", what, p->chunk);
  if (p->L % p->chunk != 0) return fail(LQ_ERR_SHAPE, "%s: L=%d must be a multiple of the chunk size %d", what, p->L, p->chunk);
  if (p->H % p->G != 0) return fail(LQ_ERR_SHAPE, "%s: nheads %d not divisible by ngroups %d", what, p->H, p->G);
  return LQ_OK;
}
static int ssd_check_pn(const lq_ssd_problem* p, const char* what) {
  if (p->P != 64) return fail(LQ_ERR_UNSUPPORTED, "%s: headdim %d (this build implements headdim 64)", what, p->P);
  if (p->N != 64 && p->N != 128) return fail(LQ_ERR_UNSUPPORTED, "%s: d_state %d (64 or 128 supported)", what, p->N);
  if (p->x_dtype != LQ_F16 && p->x_dtype != LQ_BF16) return fail(LQ_ERR_UNSUPPORTED, "%s: x must be f16 or bf16", what);
  if (!p->x || (reinterpret_cast<uintptr_t>(p->x) & 15u) || (p->x_stride_t % 8) || (p->x_stride_b % 8) || (p->x_stride_h % 8))
    return fail(LQ_ERR_ALIGN, "%s: x must be 16-byte aligned with strides that are multiples of 8 elements", what);
  return LQ_OK;
}

template <typename T, int N, bool KEYSIDE>
static void launch_chunk_state_T(const lq_ssd_problem* p, dim3 grid, cudaStream_t st) {
  const int smem = p->chunk * 128;  // static + dynamic shared memory exceeds 48 KB on the key side: opt in
  cudaFuncSetAttribute(ssd_chunk_state_kernel<T, N, KEYSIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  ssd_chunk_state_kernel<T, N, KEYSIDE><<<grid, 128, smem, st>>>(*p);
}
template <bool KEYSIDE>
static void launch_chunk_state(const lq_ssd_problem* p, dim3 grid, cudaStream_t st) {
  if (p->x_dtype == LQ_F16) {
    if (p->N == 128) launch_chunk_state_T<__half, 128, KEYSIDE>(p, grid, st);
    else launch_chunk_state_T<__half, 64, KEYSIDE>(p, grid, st);
  } else {
    if (p->N == 128) launch_chunk_state_T<__nv_bfloat16, 128, KEYSIDE>(p, grid, st);
    else launch_chunk_state_T<__nv_bfloat16, 64, KEYSIDE>(p, grid, st);
  }
}
template <bool B_IS_FP>
static void launch_bmm(const lq_ssd_problem* p, dim3 grid, cudaStream_t st) {
  if (p->x_dtype == LQ_BF16) {
    if (p->N == 128) ssd_bmm_kernel<__nv_bfloat16, 128, B_IS_FP><<<grid, 128, 0, st>>>(*p);
    else ssd_bmm_kernel<__nv_bfloat16, 64, B_IS_FP><<<grid, 128, 0, st>>>(*p);
  } else {
    if (p->N == 128) ssd_bmm_kernel<__half, 128, B_IS_FP><<<grid, 128, 0, st>>>(*p);
    else ssd_bmm_kernel<__half, 64, B_IS_FP><<<grid, 128, 0, st>>>(*p);
  }
}

}  // namespace lq

using namespace lq;

extern "C" int lq_ssd_chunk_cumsum(const lq_ssd_problem* p, lq_stream stream) {
  if (int e = ssd_check(p, "chunk_cumsum")) return e;
  if (!p->dt_in || !p->A_log || !p->dt || !p->dA) return fail(LQ_ERR_NULL, "chunk_cumsum: dt_in, A_log, dt, dA required");
  const size_t smem = (size_t)p->chunk * (p->H + 1) * sizeof(float);
  if (smem > 200 * 1024) return fail(LQ_ERR_UNSUPPORTED, "chunk_cumsum: chunk * nheads = %d * %d exceeds the shared-memory tile", p->chunk, p->H);
  cudaFuncSetAttribute(ssd_cumsum_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ssd_cumsum_kernel<<<dim3(p->L / p->chunk, p->B), 1024, smem, (cudaStream_t)stream>>>(*p);
  return check_launch("ssd_cumsum_kernel");
}

extern "C" int lq_ssd_state_passing(const lq_ssd_problem* p, lq_stream stream) {
  if (int e = ssd_check(p, "state_passing")) return e;
  if (!p->states || !p->passed || !p->final_state || !p->dA) return fail(LQ_ERR_NULL, "state_passing: states, passed, final_state, dA required");
  const int D = p->P * p->N;
  if (D % 8 != 0) return fail(LQ_ERR_SHAPE, "state_passing: P*N must be a multiple of 8");
  if ((p->carry_in && (reinterpret_cast<uintptr_t>(p->carry_in) & 15u)) || (p->carry_out && (reinterpret_cast<uintptr_t>(p->carry_out) & 15u)))
    return fail(LQ_ERR_ALIGN, "state_passing: carry_in / carry_out must be 16-byte aligned");
  if ((p->wait_flags || p->post_flags) && p->epoch == 0) return fail(LQ_ERR_SHAPE, "state_passing: the flag hand-off needs epoch >= 1");
  if (p->wait_flags && !p->carry_in) return fail(LQ_ERR_NULL, "state_passing: wait_flags without carry_in");
  dim3 grid((D / 8 + 255) / 256, p->H, p->B);
  if ((size_t)(p->L / p->chunk) * sizeof(int) > 48 * 1024) return fail(LQ_ERR_UNSUPPORTED, "state_passing: more than 12288 chunks");
  PassingLink link{p->carry_in, p->carry_out, p->wait_flags, p->post_flags, p->epoch, p->wait_ns, p->status};
  ssd_state_passing_kernel<<<grid, 256, (size_t)(p->L / p->chunk) * sizeof(int), (cudaStream_t)stream>>>(p->states, p->dA, p->passed, p->final_state, p->H,
                                                                    p->L / p->chunk, p->chunk, D, link);
  return check_launch("ssd_state_passing_kernel");
}

namespace lq {
int run_chunk_state_value_tc(const lq_ssd_problem* p, int* status, cudaStream_t st);
bool chunk_state_value_tc2_applies(const lq_ssd_problem* p);
int run_chunk_state_value_tc2(const lq_ssd_problem* p, int* status, cudaStream_t st);
int run_chunk_scan_tc(const lq_ssd_problem* p, int* status, cudaStream_t st);
bool chunk_state_key_tc_applies(const lq_ssd_problem* p);
int run_chunk_state_key_tc(const lq_ssd_problem* p, int* status, cudaStream_t st);
bool bmm_tc_applies(const lq_ssd_problem* p, bool b_is_fp);
int run_bmm_tc(const lq_ssd_problem* p, bool b_is_fp, int* status, cudaStream_t st);
}
// with_qbt: take the path that goes through the transposed copy of q_B even where the transposition-free kernel applies
static int ssd_chunk_state(const lq_ssd_problem* p, bool keyside, lq_stream stream, bool with_qbt = false) {
  const char* what = keyside ? "chunk_state_key" : "chunk_state_value";
  if (int e = ssd_check(p, what)) return e;
  if (int e = ssd_check_pn(p, what)) return e;
  if (!p->dt || !p->dA || !p->states || !p->state_scale) return fail(LQ_ERR_NULL, "%s: dt, dA, states, state_scale required", what);
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(p->L / p->chunk, p->H, p->B);
  if (keyside) {
    if (!p->b_fp || !p->x_scale_hp || !p->b_gate_scale) return fail(LQ_ERR_NULL, "%s: b_fp, x_scale_hp, b_gate_scale required", what);
    // d_state 128 with chunks of 128 / 256 tokens: tcgen05, two heads per CTA; else the warp-level MMA kernel
    if (chunk_state_key_tc_applies(p)) return run_chunk_state_key_tc(p, p->status, st);
    launch_chunk_state<true>(p, grid, st);
  } else {
    if (!p->q_B || !p->alpha_hp || !p->bscale_g) return fail(LQ_ERR_NULL, "%s: q_B, alpha_hp, bscale_g required", what);
    // d_state 128 with chunks of 128 / 256 tokens: both tcgen05 operands in their natural layouts, no scratch at all
    if (!with_qbt && chunk_state_value_tc2_applies(p)) return run_chunk_state_value_tc2(p, p->status, st);
    if (!p->q_BT) return fail(LQ_ERR_NULL, "%s: q_BT (scratch for the transposed q_B) required for this shape", what);
    ssd_transpose_b_kernel<<<dim3(p->L / 64, p->G, p->B), 256, 0, st>>>(p->q_B, p->q_BT, p->L, p->G, p->N, p->chunk);
    if (int e = check_launch("ssd_transpose_b_kernel")) return e;
    // chunks of 128 or 256 tokens run on tcgen05 + TMA; 64- and 192-token chunks on the warp-level MMA kernel
    if (p->chunk % 128 == 0) return run_chunk_state_value_tc(p, p->status, st);
    launch_chunk_state<false>(p, grid, st);
  }
  return check_launch("ssd_chunk_state_kernel");
}
extern "C" int lq_ssd_chunk_state_value(const lq_ssd_problem* p, lq_stream stream) { return ssd_chunk_state(p, false, stream); }

// ---- value-side chunk state without any caller-provided or freshly allocated scratch
// The transposed copy of q_B normally lives in a buffer the caller allocates (p->q_BT). Some hosts cannot do that at
// call time: a serving process that handed all device memory to its own pools at start-up, or a plugin that runs
// under a runtime which forbids allocation once the model is loaded. For them the scratch is this fixed array inside
// the library image. Every GPU that loads the library holds these bytes until the process exits.
namespace lq {
constexpr size_t kStaticScratchBytes = size_t(8) << 20;  // 8 MiB: B * L * ngroups * d_state may not exceed this
static __device__ __align__(256) int8_t g_static_qbt[kStaticScratchBytes];
static int8_t* g_static_qbt_addr[64];  // device address of the array, per device ordinal (the host-side name of a
static std::mutex g_static_mu;         // __device__ array is only a handle: a kernel must be given this address)

static int static_scratch(int8_t** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "static scratch: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(LQ_ERR_UNSUPPORTED, "static scratch: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_qbt_addr[dev] == nullptr) {
    int8_t* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_static_qbt);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(LQ_ERR_LAUNCH, "static scratch: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_static_qbt_addr[dev] = ptr;
  }
  *out = g_static_qbt_addr[dev];
  return LQ_OK;
}
}  // namespace lq

extern "C" size_t lq_ssd_static_scratch_bytes(void) { return lq::kStaticScratchBytes; }

extern "C" int lq_ssd_chunk_state_value_static(const lq_ssd_problem* p, lq_stream stream) {
  // the ordinary shape checks first (non-positive or unsupported extents are shape errors, not capacity errors)
  if (int e = ssd_check(p, "chunk_state_value_static")) return e;
  if (int e = ssd_check_pn(p, "chunk_state_value_static")) return e;
  // B, L, G are positive ints and N is 64 or 128 here, so the 64-bit product cannot wrap
  const unsigned long long need = (unsigned long long)p->B * (unsigned long long)p->L * (unsigned long long)p->G * (unsigned long long)p->N;
  if (need > lq::kStaticScratchBytes)
    return fail(LQ_ERR_WORKSPACE, "chunk_state_value_static: B*L*G*N = %llu bytes of scratch needed, the built-in array holds %zu; "
                "use lq_ssd_chunk_state_value with a caller-owned q_BT for larger problems", need, lq::kStaticScratchBytes);
  lq_ssd_problem q = *p;
  if (int e = lq::static_scratch(&q.q_BT)) return e;
  return ssd_chunk_state(&q, false, stream, true);
}
extern "C" int lq_ssd_chunk_state_key(const lq_ssd_problem* p, lq_stream stream) { return ssd_chunk_state(p, true, stream); }

extern "C" int lq_ssd_bmm_chunk(const lq_ssd_problem* p, int b_is_fp, lq_stream stream) {
  if (int e = ssd_check(p, "bmm_chunk")) return e;
  if (p->N != 64 && p->N != 128) return fail(LQ_ERR_UNSUPPORTED, "bmm_chunk: d_state %d (64 or 128 supported)", p->N);
  if (!p->q_C || !p->C_scale || !p->B_scale || !p->cb_scale || !p->cb) return fail(LQ_ERR_NULL, "bmm_chunk: q_C, scales, cb required");
  if (b_is_fp ? !p->b_fp : !p->q_B) return fail(LQ_ERR_NULL, "bmm_chunk: B operand missing");
  const int tiles = p->chunk / 64;
  dim3 grid(tiles * tiles, (p->L / p->chunk) * p->G, p->B);
  cudaStream_t st = (cudaStream_t)stream;
  // d_state 128 and chunks of 128 / 256 tokens: tcgen05 + TMA, one CTA per chunk; else the warp-level MMA kernel
  if (bmm_tc_applies(p, b_is_fp != 0)) return run_bmm_tc(p, b_is_fp != 0, p->status, st);
  if (b_is_fp) launch_bmm<true>(p, grid, st);
  else launch_bmm<false>(p, grid, st);
  return check_launch("ssd_bmm_kernel");
}

template <typename T, int N>
static int launch_scan(const lq_ssd_problem* p, cudaStream_t st) {
  const size_t smem = (size_t)p->chunk * 128 + 6 * sizeof(float) * p->chunk + (size_t)64 * N + 128 * sizeof(float);
  dim3 grid(p->L / p->chunk, p->H, p->B);
  cudaFuncSetAttribute(ssd_chunk_scan_kernel<T, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  ssd_chunk_scan_kernel<T, N><<<grid, 256, smem, st>>>(*p);
  return check_launch("ssd_chunk_scan_kernel");
}
extern "C" int lq_ssd_chunk_scan(const lq_ssd_problem* p, lq_stream stream) {
  if (int e = ssd_check(p, "chunk_scan")) return e;
  if (int e = ssd_check_pn(p, "chunk_scan")) return e;
  if (!p->cb || !p->dt || !p->dA || !p->q_C || !p->C_scale || !p->passed || !p->state_scale || !p->cb_scale || !p->out)
    return fail(LQ_ERR_NULL, "chunk_scan: cb, dt, dA, q_C, C_scale, passed, state_scale, cb_scale, out required");
  cudaStream_t st = (cudaStream_t)stream;
  // Two kernels: a persistent, software-pipelined tcgen05 + TMA kernel (d_state 128, chunks of 128 or 256 tokens: the
  // Mamba-2 shapes), which is the library's choice where it applies, and the warp-level MMA kernel (every supported shape).
  const bool tc_ok = p->N == 128 && p->chunk % 128 == 0;
  if (p->scan_kernel == 2 && !tc_ok) return fail(LQ_ERR_UNSUPPORTED, "chunk_scan: the tcgen05 kernel needs d_state 128 and chunk 128 or 256");
  if (p->scan_kernel < 0 || p->scan_kernel > 2) return fail(LQ_ERR_SHAPE, "chunk_scan: scan_kernel must be 0, 1 or 2");
  if (p->scan_kernel == 2 || (p->scan_kernel == 0 && tc_ok)) return run_chunk_scan_tc(p, p->status, st);
  if (p->x_dtype == LQ_F16) return p->N == 128 ? launch_scan<__half, 128>(p, st) : launch_scan<__half, 64>(p, st);
  return p->N == 128 ? launch_scan<__nv_bfloat16, 128>(p, st) : launch_scan<__nv_bfloat16, 64>(p, st);
}

template <typename T, bool QUANT>
static int launch_rotate(const T* x, long long sb, long long stt, long long ob, long long oc, int B, int T_len, int G, int N,
                         int gy, const float* signs, const float* ib, const float* ic, const float* db, const float* dc,
                         int8_t* qb, int8_t* qc, T* y, cudaStream_t st) {
  // 256 rows per CTA amortise the per-thread constants; a problem too small to fill the GPU that way takes 128 or 64
  int rows_per_cta = 256;
  while (rows_per_cta > 64 && (long long)((T_len + rows_per_cta - 1) / rows_per_cta) * gy * B < 592) rows_per_cta >>= 1;
  dim3 grid((T_len + rows_per_cta - 1) / rows_per_cta, gy, B);
  if (N == 128) ssd_rotate_rows_kernel<T, 128, QUANT><<<grid, 256, 0, st>>>(x, sb, stt, ob, oc, T_len, G, signs, ib, ic, db, dc, qb, qc, y, rows_per_cta);
  else if (N == 64) ssd_rotate_rows_kernel<T, 64, QUANT><<<grid, 256, 0, st>>>(x, sb, stt, ob, oc, T_len, G, signs, ib, ic, db, dc, qb, qc, y, rows_per_cta);
  else return fail(LQ_ERR_UNSUPPORTED, "Hadamard rows: width %d (64 or 128 supported)", N);
  return check_launch("ssd_rotate_rows_kernel");
}

extern "C" int lq_ssd_split_rotate_quant(const void* xBC, int dtype, int B, int T, int d_ssm, int G, int N, const float* signs,
                                         const float* B_inv_scale, const float* C_inv_scale, const float* dqk_b,
                                         const float* dqk_c, int8_t* q_B, int8_t* q_C, lq_stream stream) {
  if (!xBC || !B_inv_scale || !C_inv_scale || !q_B || !q_C) return fail(LQ_ERR_NULL, "split_rotate_quant: null argument");
  if (B <= 0 || T <= 0 || G <= 0) return fail(LQ_ERR_SHAPE, "split_rotate_quant: non-positive extent");
  if ((d_ssm % 8) || (reinterpret_cast<uintptr_t>(xBC) & 15u)) return fail(LQ_ERR_ALIGN, "split_rotate_quant: xBC must be 16-byte aligned, d_ssm a multiple of 8");
  if ((dqk_b == nullptr) != (dqk_c == nullptr)) return fail(LQ_ERR_NULL, "split_rotate_quant: dqk_b and dqk_c go together");
  const long long xdim = (long long)d_ssm + 2LL * G * N;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == LQ_F16)
    return launch_rotate<__half, true>(reinterpret_cast<const __half*>(xBC), (long long)T * xdim, xdim, d_ssm, d_ssm + (long long)G * N,
                                       B, T, G, N, 2 * G, signs, B_inv_scale, C_inv_scale, dqk_b, dqk_c, q_B, q_C, nullptr, st);
  if (dtype == LQ_BF16)
    return launch_rotate<__nv_bfloat16, true>(reinterpret_cast<const __nv_bfloat16*>(xBC), (long long)T * xdim, xdim, d_ssm,
                                              d_ssm + (long long)G * N, B, T, G, N, 2 * G, signs, B_inv_scale, C_inv_scale, dqk_b,
                                              dqk_c, q_B, q_C, nullptr, st);
  return fail(LQ_ERR_UNSUPPORTED, "split_rotate_quant: xBC must be f16 or bf16");
}

extern "C" int lq_kronecker_hadamard(const void* x, void* y, int dtype, int B, int T, int H, int D, long long in_stride_t,
                                     const float* signs, lq_stream stream) {
  if (!x || !y || !signs) return fail(LQ_ERR_NULL, "kronecker_hadamard: null argument");
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (in_stride_t % 8)) return fail(LQ_ERR_ALIGN, "kronecker_hadamard: x must be 16-byte aligned, token stride a multiple of 8");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == LQ_F16)
    return launch_rotate<__half, false>(reinterpret_cast<const __half*>(x), (long long)T * in_stride_t, in_stride_t, 0, 0, B, T, H, D, H,
                                        signs, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, reinterpret_cast<__half*>(y), st);
  if (dtype == LQ_BF16)
    return launch_rotate<__nv_bfloat16, false>(reinterpret_cast<const __nv_bfloat16*>(x), (long long)T * in_stride_t, in_stride_t, 0, 0,
                                               B, T, H, D, H, signs, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                               reinterpret_cast<__nv_bfloat16*>(y), st);
  return fail(LQ_ERR_UNSUPPORTED, "kronecker_hadamard: x must be f16 or bf16");
}
