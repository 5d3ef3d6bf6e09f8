// C-ABI glue: status / error strings, argument validation, workspace carve-up and the whole-call entry points.
#include <stdarg.h>
#include <stdio.h>

#include "lq_common.cuh"

namespace lq {

static thread_local char g_err[512] = "";

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(LQ_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return LQ_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Mirrors the reference's asserts (zoo/gla.py:246, zoo/gated_delta_rule.py:170, zoo/kda.py:165): T % chunk == 0,
// K <= 128; plus what the vector loads of this implementation need.
int validate_zoo_problem(const lq_zoo_problem* p, bool delta, bool diagonal) {
  if (!p) return fail(LQ_ERR_NULL, "problem descriptor is null");
  if (p->B <= 0 || p->T <= 0 || p->H <= 0) return fail(LQ_ERR_SHAPE, "B, T, H must be positive (B=%d T=%d H=%d)", p->B, p->T, p->H);
  if (p->chunk != 64) return fail(LQ_ERR_UNSUPPORTED, "chunk size %d: this build implements chunk_size=64", p->chunk);
  if (p->T % p->chunk != 0) return fail(LQ_ERR_SHAPE, "T=%d must be a multiple of the chunk size %d", p->T, p->chunk);
  if (!((p->K == 64 || p->K == 128) && (p->V == 64 || p->V == 128)))
    return fail(LQ_ERR_UNSUPPORTED, "K=%d V=%d: K and V must each be 64 or 128", p->K, p->V);
  if (!p->q || !p->k || !p->v || !p->o) return fail(LQ_ERR_NULL, "q, k, v, o must be non-null");
  if (!p->sq || !p->sk || !p->skw || !p->sstate) return fail(LQ_ERR_NULL, "scales sq, sk, skw, sstate must be non-null");
  if (!delta && (!p->svl || !p->svw)) return fail(LQ_ERR_NULL, "linear family needs svl and svw");
  if (delta && (!p->sw || !p->sel || !p->sew || !p->beta)) return fail(LQ_ERR_NULL, "delta family needs beta, sw, sel, sew");
  if (diagonal != (p->decay == LQ_DECAY_DIAGONAL)) return fail(LQ_ERR_SHAPE, "decay kind does not match the entry point");
  if ((p->decay != LQ_DECAY_NONE) != (p->g != nullptr)) return fail(LQ_ERR_SHAPE, "g must be given exactly when decay != none");
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->o))
    return fail(LQ_ERR_ALIGN, "q, k, v, o must be 16-byte aligned");
  if (p->act_dtype != LQ_F16 && p->act_dtype != LQ_BF16) return fail(LQ_ERR_UNSUPPORTED, "activation dtype must be f16 or bf16");
  if (p->unrot_t != nullptr && !aligned16(p->unrot_t)) return fail(LQ_ERR_ALIGN, "unrot_t must be 16-byte aligned");
  if (!(p->qmax >= 1.f && p->qmax <= 127.f)) return fail(LQ_ERR_SHAPE, "qmax=%f out of range", (double)p->qmax);
  return LQ_OK;
}

struct Carver {
  uint8_t* base;
  size_t off;
  template <typename T>
  T* take(size_t n) {
    off = (off + 255) & ~size_t(255);
    T* r = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += n * sizeof(T);
    return r;
  }
};

static size_t carve(const lq_zoo_problem* p, int delta, void* ws, lq_zoo_workspace* out) {
  const size_t BH = (size_t)p->B * p->H, NT = p->T / p->chunk, C = p->chunk, K = p->K, V = p->V;
  Carver cv{reinterpret_cast<uint8_t*>(ws), 0};
  lq_zoo_workspace w;
  w.qq = cv.take<int8_t>(BH * NT * C * K);
  w.kl = cv.take<int8_t>(BH * NT * C * K);
  w.kwT = cv.take<int8_t>(BH * NT * K * C);
  w.vlT = cv.take<int8_t>(BH * NT * V * C);
  w.vwT = cv.take<int8_t>(BH * NT * V * C);
  w.hT = cv.take<int8_t>(BH * NT * V * K);
  w.gc = cv.take<float>(BH * NT * C * (p->decay == LQ_DECAY_DIAGONAL ? K : 1));
  w.wq = delta ? cv.take<int8_t>(BH * NT * C * K) : nullptr;
  w.u = delta ? cv.take<uint16_t>(BH * NT * C * V) : nullptr;
  w.fw = delta ? cv.take<float>(BH * NT * C) : nullptr;
  w.amat = p->decay == LQ_DECAY_DIAGONAL ? cv.take<uint16_t>(BH * NT * C * C) : nullptr;
  w.genv = p->decay == LQ_DECAY_DIAGONAL ? cv.take<float>(BH * NT * C) : nullptr;
  w.gcl = p->decay == LQ_DECAY_DIAGONAL ? cv.take<float>(BH * NT * K) : nullptr;
  w.status = cv.take<int>(64);
  if (out) *out = w;
  return (cv.off + 255) & ~size_t(255);
}

int run_prologue_linear(const lq_zoo_problem* p, const lq_zoo_workspace* ws, int skip_v, cudaStream_t st);
int run_state_linear(const lq_zoo_problem* p, const lq_zoo_workspace* ws, cudaStream_t st);
int run_output_scalar(const lq_zoo_problem* p, const lq_zoo_workspace* ws, const float* s_local_value, cudaStream_t st);
int run_prologue_delta(const lq_zoo_problem* p, const lq_zoo_workspace* ws, cudaStream_t st);
int run_state_delta(const lq_zoo_problem* p, const lq_zoo_workspace* ws, cudaStream_t st);
int run_diag_stage(const lq_zoo_problem* p, const lq_zoo_workspace* ws, bool delta, int stage, cudaStream_t st);

}  // namespace lq

extern "C" int lq_version(void) { return 100; }
extern "C" unsigned long long lq_struct_bytes(int which) {
  return which == 0 ? sizeof(lq_zoo_problem) : which == 1 ? sizeof(lq_ssd_problem) : which == 2 ? sizeof(lq_zoo_workspace) : 0;
}
extern "C" const char* lq_last_error_string(void) { return lq::g_err; }

extern "C" int lq_status_poll(int* status, lq_stream stream) {
  if (!status) return lq::fail(LQ_ERR_NULL, "status_poll: status word is null");
  cudaStream_t st = (cudaStream_t)stream;
  int host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return lq::fail(LQ_ERR_LAUNCH, "status_poll: %s", cudaGetErrorString(e));
  if (host == 0) return LQ_OK;
  cudaMemsetAsync(status, 0, sizeof(int), st);
  return lq::fail(LQ_ERR_TIMEOUT, "a bounded device-side wait ran out (status word %d): the outputs written since the last poll are not valid", host);
}

extern "C" size_t lq_zoo_workspace_bytes(const lq_zoo_problem* p, int delta_family) {
  if (!p || p->chunk <= 0) return 0;
  return lq::carve(p, delta_family, nullptr, nullptr);
}

extern "C" int lq_zoo_carve_workspace(const lq_zoo_problem* p, int delta_family, void* workspace,
                                      size_t workspace_bytes, lq_zoo_workspace* out) {
  if (!p || !workspace || !out) return lq::fail(LQ_ERR_NULL, "carve: null argument");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return lq::fail(LQ_ERR_ALIGN, "workspace must be 256-byte aligned");
  const size_t need = lq::carve(p, delta_family, nullptr, nullptr);
  if (workspace_bytes < need) return lq::fail(LQ_ERR_WORKSPACE, "workspace holds %zu bytes, %zu needed", workspace_bytes, need);
  lq::carve(p, delta_family, workspace, out);
  return LQ_OK;
}

extern "C" int lq_simple_gla_fwd(const lq_zoo_problem* p, void* workspace, size_t workspace_bytes, lq_stream stream) {
  if (int e = lq::validate_zoo_problem(p, false, false)) return e;
  lq_zoo_workspace ws;
  if (int e = lq_zoo_carve_workspace(p, 0, workspace, workspace_bytes, &ws)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  if (p->status == nullptr) cudaMemsetAsync(ws.status, 0, sizeof(int), st);
  if (int e = lq::run_prologue_linear(p, &ws, 0, st)) return e;
  if (int e = lq::run_state_linear(p, &ws, st)) return e;
  return lq::run_output_scalar(p, &ws, p->svl, st);
}

extern "C" int lq_delta_fwd(const lq_zoo_problem* p, void* workspace, size_t workspace_bytes, lq_stream stream) {
  if (int e = lq::validate_zoo_problem(p, true, false)) return e;
  lq_zoo_workspace ws;
  if (int e = lq_zoo_carve_workspace(p, 1, workspace, workspace_bytes, &ws)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  if (p->status == nullptr) cudaMemsetAsync(ws.status, 0, sizeof(int), st);
  if (int e = lq::run_prologue_delta(p, &ws, st)) return e;
  if (int e = lq::run_state_delta(p, &ws, st)) return e;
  return lq::run_output_scalar(p, &ws, p->sel, st);
}

extern "C" int lq_gla_fwd(const lq_zoo_problem* p, void* workspace, size_t workspace_bytes, lq_stream stream) {
  if (int e = lq::validate_zoo_problem(p, false, true)) return e;
  lq_zoo_workspace ws;
  if (int e = lq_zoo_carve_workspace(p, 0, workspace, workspace_bytes, &ws)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  if (p->status == nullptr) cudaMemsetAsync(ws.status, 0, sizeof(int), st);
  if (int e = lq::run_diag_stage(p, &ws, false, 0, st)) return e;
  if (int e = lq::run_diag_stage(p, &ws, false, 1, st)) return e;
  if (int e = lq::run_state_linear(p, &ws, st)) return e;
  return lq::run_output_scalar(p, &ws, p->svl, st);
}

extern "C" int lq_kda_fwd(const lq_zoo_problem* p, void* workspace, size_t workspace_bytes, lq_stream stream) {
  if (int e = lq::validate_zoo_problem(p, true, true)) return e;
  lq_zoo_workspace ws;
  if (int e = lq_zoo_carve_workspace(p, 1, workspace, workspace_bytes, &ws)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  if (p->status == nullptr) cudaMemsetAsync(ws.status, 0, sizeof(int), st);
  if (int e = lq::run_diag_stage(p, &ws, true, 0, st)) return e;
  if (int e = lq::run_diag_stage(p, &ws, true, 1, st)) return e;
  if (int e = lq::run_diag_stage(p, &ws, true, 2, st)) return e;
  if (int e = lq::run_state_delta(p, &ws, st)) return e;
  return lq::run_output_scalar(p, &ws, p->sel, st);
}
