/*
 * linquant_b200 — C ABI of the sm_100a INT8 chunk-prefill kernels.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless it says "host". Nothing here allocates
 * device memory (the lq_peer_buffer_* set-up calls of the multi-GPU hand-off excepted): callers own inputs, outputs
 * and the workspace. All launches go to the given stream and return
 * without synchronising. Every entry returns an lq_status (0 = ok); lq_last_error_string() gives the detail of
 * the most recent failure on the calling thread.
 *
 * The reference project has no C boundary on this path: its hot path is Python calling Triton JIT kernels.
 * Each entry below therefore names the reference *Python* function (file:line in the reference tree) whose
 * device work it replaces; the Python wrappers in linquant_b200/kernels keep those functions' signatures.
 */
#ifndef LINQUANT_B200_H
#define LINQUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  LQ_OK = 0,
  LQ_ERR_NULL = 1,        /* a required pointer is null */
  LQ_ERR_SHAPE = 2,       /* T % chunk != 0, unsupported K/V/chunk, non-positive extent */
  LQ_ERR_ALIGN = 3,       /* a pointer or stride breaks the 16-byte rule of the vector loads */
  LQ_ERR_UNSUPPORTED = 4, /* valid request this build has no kernel for */
  LQ_ERR_LAUNCH = 5,      /* cudaGetLastError() after the launch was not cudaSuccess */
  LQ_ERR_TIMEOUT = 6,     /* a bounded device-side wait ran out (status word written by the kernel) */
  LQ_ERR_WORKSPACE = 7    /* workspace too small */
} lq_status;

typedef enum { LQ_F16 = 0, LQ_BF16 = 1, LQ_F32 = 2 } lq_dtype;

/* decay kinds of the recurrence (reference.py:107-122) */
typedef enum { LQ_DECAY_NONE = 0, LQ_DECAY_SCALAR = 1, LQ_DECAY_DIAGONAL = 2 } lq_decay;

typedef void* lq_stream; /* a cudaStream_t */

int lq_version(void);
/* sizeof the two descriptor structs as the library was compiled: a binding checks its own layout against these (0 = zoo, 1 = ssd, 2 = workspace) */
unsigned long long lq_struct_bytes(int which);
const char* lq_last_error_string(void);

/* Drains `stream`, reads the device status word and clears it. Returns LQ_ERR_TIMEOUT when a kernel raised it since the
 * last poll (the outputs of the calls in between are then not valid), LQ_OK otherwise. The launches themselves are
 * asynchronous, so this is how a bounded device-side wait that ran out (TMA / MMA barrier, peer hand-off flag) reaches the
 * host. No counterpart in the reference (its Triton kernels have no device-side waits). */
int lq_status_poll(int* status, lq_stream stream);

/* Self-test of the bounded-wait machinery, for test suites: one CTA initialises an mbarrier that nothing ever arrives
 * on (no copy or MMA is issued, so nothing is in flight), optionally holds 32 tensor-memory columns meanwhile, lets the
 * bounded wait of the tcgen05 kernels run out, raises *status, writes its own progress marks to trace[0..3]
 * (1 = reached the wait, 2 = the wait gave up, 3 = tensor memory freed, 4 = returned normally) and returns. The GPU
 * is not faulted or hung: the kernel ends by itself after the poll limit (about a millisecond). */
int lq_selftest_wait_timeout(int* status, int* trace, int hold_tmem, lq_stream stream);

/* ------------------------------------------------------------------------------------------------------------
 * Problem descriptor shared by the zoo-lineage entries (linear attention / Simple GLA / GLA / DeltaNet /
 * Gated DeltaNet / KDA). Layouts follow the reference: q,k [B,T,H,K], v,o [B,T,H,V] dense, act dtype f16/bf16;
 * g [B,T,H] (scalar) or [B,T,H,K] (diagonal) fp32 log-decay or null; beta [B,T,H] fp32 or null.
 * Scales are fp32: sq,sk,sw [H]; skw [H,K]; svl,svw,sel,sew,sstate [H,V]  (invariances.py:102-112).
 * ------------------------------------------------------------------------------------------------------------ */
typedef struct {
  int B, T, H, K, V, chunk;
  int act_dtype; /* lq_dtype of q,k,v */
  int out_dtype; /* lq_dtype of o */
  int decay;     /* lq_decay */
  float scale;   /* multiplies q before quantisation (reference.py:47) */
  float eta;     /* write-decay split: key gets Omega^(1-eta), value Omega^eta */
  float sigma;   /* delta rule: Gram exponent (reference "rho") */
  float tau;     /* delta rule: placement of the outer beta factor */
  float qmax;    /* 127 (INT8) or 31 (INT6 codes in INT8 containers) */
  const void* q;
  const void* k;
  const void* v;
  const float* g;
  const float* beta;
  const float* rot_signs; /* [K] +-1: fused signed-Hadamard R_QK (persistent for none/scalar decay, local for
                             diagonal decay); null = operands are used as given */
  const float* dqk;       /* [H,K] diagonal rescale D_QK (q*D, k/D) applied before the rotation; null = off */
  const float *sq, *sk, *skw, *svl, *svw, *sstate; /* linear-family scales */
  const float *sw, *sel, *sew;                     /* delta-family extras (null for the linear family) */
  void* o;                /* [B,T,H,V] */
  float* final_state;     /* [B,H,K,V] fp32 carry after the last chunk, or null */
  const float* initial_state; /* [B,H,K,V] fp32 carry entering the first chunk, or null = zero */
  const void* unrot_t;        /* canonical storage under a value rotation (the reference's unrot=, zoo/simple_gla.py:31-33,
                                 :150-153): [V,V] fp16, TRANSPOSED, element [v'][v] = unrot[v][v']; v arrives rotated and
                                 every value-side product is multiplied by unrot before it joins the carry / the output
                                 (the delta family also takes the state read into the rotated basis); null = off */
  int* status;                /* optional device int32 owned by the caller: when given, a kernel whose bounded wait ran out
                                 raises THIS word instead of the workspace's, and the entries do not clear it (a host keeps
                                 one word per device and polls it with lq_status_poll when convenient); null = the
                                 workspace's own word, cleared by the whole-call entries */
} lq_zoo_problem;

/* Bytes of workspace the zoo entries need for this problem (a host-side computation). */
size_t lq_zoo_workspace_bytes(const lq_zoo_problem* p, int delta_family);

/* Workspace carve-up, exposed so tests can read the recorded INT8 codes back. All tiles are per (b*H+h, chunk):
 *   qq  [BH,NT,C,K]  q codes (read == local, invariances.py:54)      kl  [BH,NT,C,K]  k_local codes
 *   kwT [BH,NT,K,C]  k_write codes, token index contiguous            vlT [BH,NT,V,C]  v_local / e_local codes
 *   vwT [BH,NT,V,C]  v_write codes                                     hT  [BH,NT,V,K]  stored state entering the chunk
 *   gc  [BH,NT,C]    chunk-local cumulative log-decay (fp32)           wq  [BH,NT,C,K]  w_read codes (delta)
 *   u   [BH,NT,C,V]  WY right-hand side U in the activation dtype (delta)
 *   fw  [BH,NT,C]    value-side share of the outer beta factor (delta)
 * Diagonal decay adds gc [BH,NT,C,K], amat, genv, gcl (see the fields below).
 */
typedef struct {
  int8_t *qq, *kl, *kwT, *vlT, *vwT, *hT, *wq;
  float* gc;
  void* u;
  float* fw;
  void* amat;  /* [BH,NT,C,C] fp16 intra-chunk matrix (diagonal decay) */
  float* genv; /* [BH,NT,C]   log of the scalar write envelope (diagonal decay) */
  float* gcl;  /* [BH,NT,K]   cumulative log-decay at the chunk end (diagonal decay) */
  int* status; /* one word, zeroed by the whole-call entries; a kernel whose bounded device-side wait expired sets it */
} lq_zoo_workspace;
int lq_zoo_carve_workspace(const lq_zoo_problem* p, int delta_family, void* workspace, size_t workspace_bytes,
                           lq_zoo_workspace* out);

/* Fused prologue: [D_QK] -> [signed Hadamard R_QK] -> act-dtype rounding -> x scale -> per-role static INT8, plus
 * the chunk-local cumulative log-decay. Replaces the torch-side cumsum (zoo/simple_gla.py:191), the bench-side
 * rotation GEMMs (bench/zoo_kernels.py:135-140) and the per-tile _q8 calls inside the reference kernels
 * (zoo/simple_gla.py:16-20,66-67,129-130,149). */
int lq_zoo_prologue_linear(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream);

/* Inter-chunk state pass of the linear family: INT8 stored copy of the fp32 carry entering every chunk, INT8
 * write product, fp32 carry update. Replaces _state_kernel (zoo/simple_gla.py:24-87). */
int lq_zoo_state_linear(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream);

/* Intra-chunk output: INT8 q.S read, INT8 q.k^T with the decay mask, fp16 A.v on the value codes.
 * Replaces _output_kernel (zoo/simple_gla.py:99-165). */
int lq_zoo_output_scalar(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream);

/* Whole call of chunk_simple_gla_int8 (zoo/simple_gla.py:175-212): prologue + state pass + output. */
int lq_simple_gla_fwd(const lq_zoo_problem* p, void* workspace, size_t workspace_bytes, lq_stream stream);

/* Delta-rule WY prologue: q/k rows as above plus Gram matrix, (I+G)^-1 by forward substitution and the W / U
 * products, in fp32-grade arithmetic (TF32 tensor-core MMA on exactly representable operands, left factor split
 * in three). Replaces the torch-side _prep (zoo/gated_delta_rule.py:20-47) and the FLA prep kernels it may call
 * (zoo/gated_delta_rule.py:139-156). */
int lq_zoo_prologue_delta(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream);

/* Delta-rule state pass: stored INT8 state, INT8 W.S read, pseudo-values E, INT8 write product, fp32 carry.
 * Replaces _delta_state_kernel (zoo/gated_delta_rule.py:51-136). */
int lq_zoo_state_delta(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream);

/* Whole call of chunk_delta_int8 (zoo/gated_delta_rule.py:159-203): WY prologue + state pass + output. */
int lq_delta_fwd(const lq_zoo_problem* p, void* workspace, size_t workspace_bytes, lq_stream stream);

/* Diagonal (per-channel) decay, row pass: chunk-local cumulative log-decay per channel, log envelope, pre-decayed
 * q_read codes, gated k_write codes, and for the linear family the value codes. Replaces the torch-side cumsum /
 * amax (zoo/gla.py:249-250, zoo/kda.py:168-170) and the operand quantisation inside _gla_state_body /
 * _gla_output_body (zoo/gla.py:137-140,201). */
int lq_zoo_diag_rows(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream);

/* Diagonal decay, intra-chunk matrix A in 16-token secondary chunks. Replaces _gla_A_inter and _gla_A_intra
 * (zoo/gla.py:27-99). */
int lq_zoo_diag_amat(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream);

/* KDA WY prep with per-channel Gram weights. Replaces _prep / _prep_fla (zoo/kda.py:22-65). */
int lq_zoo_kda_wy(const lq_zoo_problem* p, const lq_zoo_workspace* ws, lq_stream stream);

/* Whole call of chunk_gla_int8 (zoo/gla.py:235-279). */
int lq_gla_fwd(const lq_zoo_problem* p, void* workspace, size_t workspace_bytes, lq_stream stream);

/* Whole call of chunk_kda_int8 (zoo/kda.py:154-203). */
int lq_kda_fwd(const lq_zoo_problem* p, void* workspace, size_t workspace_bytes, lq_stream stream);

/* ------------------------------------------------------------------------------------------------------------
 * Mamba-2 SSD op surface (SSDi8 arithmetic lineage): INT32 fixed-point carry, INT8 requantised CB, mixed roundings.
 * x [B,L,H,P] f16/bf16 with element strides (it may be a view into xBC; P contiguous); q_B,q_C [B,L,G,N] int8;
 * dt, dA [B,H,NC,C] fp32; states / passed [B,NC,H,P,N] int8; cb [B,NC,G,C,C] int8; out [B,L,H,P] fp16.
 * (H,P) scale tensors are dense fp32 (callers materialise stride-0 views). L must be a multiple of chunk.
 * ------------------------------------------------------------------------------------------------------------ */
typedef struct {
  int B, L, H, P, G, N, chunk;
  int x_dtype;
  long long x_stride_b, x_stride_t, x_stride_h; /* in elements */
  const void* x;
  const float* dt_in;   /* [B,L,H] raw dt (fp32) */
  const float* A_log;   /* [H] */
  const float* dt_bias; /* [H] or null */
  float dt_scale, A_log_scale, dt_min, dt_max;
  const float *dt_scale_dev, *A_log_scale_dev; /* optional one-element device tensors; they override the two floats */
  int dt_softplus;
  float *dt, *dA;
  const int8_t *q_B, *q_C;
  int8_t* q_BT;         /* scratch [B,NC,G,N,C]: q_B with the token index contiguous (value-side chunk state) */
  const void* b_fp;     /* key side: unquantised B, same dtype as x, [B,L,G,N] */
  const float *B_scale, *C_scale, *bscale_g, *cb_scale;     /* [G] */
  const float *alpha_hp, *x_scale_hp, *state_scale;         /* [H,P] */
  const float* b_gate_scale;                                /* key side, 4-D broadcastable (B,NC,H,N) */
  long long bgs_stride[4];                                  /* its element strides (0 on broadcast dims) */
  int8_t *states, *passed, *final_state, *cb;
  const float* D;       /* [H] or [H,P] (already multiplied by its scale) or null */
  int D_has_hdim;
  void* out;
  int scan_kernel;      /* lq_ssd_chunk_scan: 0 = the library's choice (the faster one as measured on B200: the tcgen05 kernel
                           where it applies), 1 = warp-level MMA kernel, 2 = persistent tcgen05 + TMA kernel (d_state 128
                           and chunk 128 or 256 only) */
  int* status;          /* optional device int32: set to 1 by a kernel whose bounded wait on a TMA / MMA barrier ran out
                           (its output is then not valid); the caller zeroes it and reads it after synchronising */
  /* ---- lq_ssd_state_passing only: the integer carry across calls / GPUs (all optional, null = a zero carry, nothing
     handed on). The recurrence's carry is the unclamped INT32 state (state_passing.py:62-93), so a sequence cut into
     segments reproduces the one-shot result bit for bit when this carry, not its INT8 copy, crosses the cut. */
  const int* carry_in;  /* [B,H,P*N] int32 carry entering the first chunk of this call */
  int* carry_out;       /* [B,H,P*N] int32 carry after the last chunk; may point into ANOTHER GPU's memory (a peer
                           mapping): the kernel writes it with plain stores */
  const unsigned* wait_flags; /* [B,H,ceil(P*N/2048)] in THIS GPU's memory: CTA i reads carry_in only after flag i >= epoch,
                                 polling at most wait_ns nanoseconds; on expiry it raises *status and stores nothing */
  unsigned* post_flags;       /* same shape, next to carry_out (peer memory allowed): CTA i sets flag i = epoch after its
                                 carry_out stores are visible system-wide */
  unsigned epoch;             /* value posted / awaited; the caller increases it on every call so flags need no reset */
  unsigned long long wait_ns; /* bound of the flag wait (0 = 2 s) */
} lq_ssd_problem;

/* dt = clamp(softplus(dt_scale*dt + bias)), dA = dt * -exp(A_log_scale*A_log), chunk-local cumsum.
 * Replaces _quant_chunk_cumsum_fwd (mamba2/chunk_cumsum.py:15-100). */
int lq_ssd_chunk_cumsum(const lq_ssd_problem* p, lq_stream stream);
/* Value-side chunk state (x gate-weighted and quantised with alpha_hp against INT8 B).
 * Replaces _quant_chunk_state_fwd_xfp_static_int8 (mamba2/chunk_state.py:24-349). */
int lq_ssd_chunk_state_value(const lq_ssd_problem* p, lq_stream stream);
/* The same op for hosts that cannot allocate device memory when they call it (a server that gave all of HBM to its own
 * pools at start-up, a plugin under a runtime that forbids allocation after load). It has no counterpart in the
 * reference. p->q_BT is ignored: the transposed copy of q_B goes to an 8 MiB array that is part of the library image
 * (lq_ssd_static_scratch_bytes()), so B*L*G*N must not exceed that, else LQ_ERR_WORKSPACE. Inputs and the states
 * output are still the caller's. The entry calls no allocating routine. The first call on each device looks up the
 * array's device address (cudaGetSymbolAddress) with that device current: make that first call before any stream
 * capture. All calls on a device share the one array and it keeps the previous call's contents (every byte that is
 * read is rewritten first, nothing relies on zeros); two calls whose kernels overlap on the GPU race on it. */
size_t lq_ssd_static_scratch_bytes(void);
int lq_ssd_chunk_state_value_static(const lq_ssd_problem* p, lq_stream stream);
/* Key-side chunk state (INT8 x against gate-weighted B quantised in-kernel).
 * Replaces _chunk_state_keyside_fwd (mamba2/chunk_state_keyside.py:17-424). */
int lq_ssd_chunk_state_key(const lq_ssd_problem* p, lq_stream stream);
/* INT32 fixed-point inter-chunk recurrence with a Q0.7 gate.
 * Replaces _fixedpoint_state_passing_fwd (mamba2/state_passing.py:14-121). With carry_in / carry_out / the flag
 * fields it is also the hand-off step of the sequence-parallel mode: the producer GPU's kernel stores its final carry
 * and a flag into the consumer GPU's memory, the consumer's kernel waits (bounded) on its local flag. */
int lq_ssd_state_passing(const lq_ssd_problem* p, lq_stream stream);
/* Receive buffers of the sequence-parallel hand-off (set-up calls; the only entries of this library that allocate).
 * create: cudaMalloc + zero-fill on the current device and the 64-byte CUDA IPC handle of the allocation. open: maps
 * another process's buffer (owner_device = the CUDA ordinal it lives on) into this process, with peer access enabled
 * from the current device; the mapping is only ever written with plain stores by lq_ssd_state_passing
 * (carry_out / post_flags). close / destroy undo open / create. No counterpart in the reference (single GPU). */
int lq_peer_buffer_create(size_t bytes, void** dev_ptr, unsigned char* handle64);
int lq_peer_buffer_open(const unsigned char* handle64, int owner_device, void** dev_ptr);
int lq_peer_buffer_close(void* dev_ptr);
int lq_peer_buffer_destroy(void* dev_ptr);

/* Per-chunk INT8 C.B^T requantised to INT8 (b_is_fp: B quantised in-kernel from b_fp).
 * Replaces _quant_bmm_chunk_fwd (mamba2/bmm_chunk.py:11-217). */
int lq_ssd_bmm_chunk(const lq_ssd_problem* p, int b_is_fp, lq_stream stream);
/* Output: INT8 C.S_prev with row gate + fp16 causal (CB*decay*dt).x + D*x.
 * Replaces _quant_chunk_scan_fwd (mamba2/chunk_scan_v2.py:14-366). */
int lq_ssd_chunk_scan(const lq_ssd_problem* p, lq_stream stream);

/* Mamba-2 prologue on the B and C lanes of xBC [B,T,d_ssm+2*G*N] f16: [x D_QK, fp16 round] -> signs ->
 * H_2 (x) H_{N/2} on bf16-rounded values -> fp16 round -> rint(. * inv_scale) clamp [-128,127].
 * Replaces fused_split_rotate_quant_xBC (mamba2/fused_split_rotate_xBC.py:31-329). */
int lq_ssd_split_rotate_quant(const void* xBC, int dtype, int B, int T, int d_ssm, int G, int N, const float* signs,
                              const float* B_inv_scale, const float* C_inv_scale, const float* dqk_b,
                              const float* dqk_c, int8_t* q_B, int8_t* q_C, lq_stream stream);
/* Standalone Kronecker Hadamard rotation y = (x*signs) @ (H_2 (x) H_{D/2}); x [B,T,H,D] with token stride
 * in_stride_t, y dense. Replaces kronecker_hadamard_fwd (kernels/hadamard.py:141-179). */
int lq_kronecker_hadamard(const void* x, void* y, int dtype, int B, int T, int H, int D, long long in_stride_t,
                          const float* signs, lq_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* LINQUANT_B200_H */
