// The C ABI of libnnlib_b200.so (include/nnlib_b200.h): argument checking,
// defaults, kernel selection.  No exceptions leave this file, no device memory
// is allocated, nothing synchronises except nnlib_b200_device_health.
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "launchers.h"

namespace nb200 {

static std::atomic<unsigned long long> g_launches{0};
static thread_local int t_last_cuda_error = 0;

void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }
void set_last_cuda_error(cudaError_t e) { t_last_cuda_error = (int)e; }

namespace {

bool force_simt() {
  static const bool v = [] {
    const char* e = std::getenv("NNLIB_B200_FORCE_SIMT");
    return e && e[0] && e[0] != '0';
  }();
  return v;
}

// NNLIB_B200_LOG=1: one line per call on stderr (entry point, sizes, options, kernel family and, when the
// tensor-core kernels were not taken, why) so that a call that silently runs on the CUDA-core kernels —
// an unaligned pointer, a stride that is not a multiple of 8 elements — can be found.
bool log_calls() {
  static const bool v = [] {
    const char* e = std::getenv("NNLIB_B200_LOG");
    return e && e[0] && e[0] != '0';
  }();
  return v;
}

// NNLIB_B200_CHECK_POINTERS=1 (implied by NNLIB_B200_LOG=1): every pointer of the struct is looked up,
// not only q and x.
bool check_all_pointers() {
  static const bool v = [] {
    const char* e = std::getenv("NNLIB_B200_CHECK_POINTERS");
    return (e && e[0] && e[0] != '0') || log_calls();
  }();
  return v;
}

// Is `ptr` device (or managed) memory of the device that is current on this thread?  NULL passes.
bool on_current_device(const void* ptr, int dev) {
  if (!ptr) return true;
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, ptr) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  if (at.type == cudaMemoryTypeManaged) return true;
  return at.type == cudaMemoryTypeDevice && at.device == dev;
}

// The caller's arrays must live on the current device: the kernels are launched there and the library
// never switches devices.  q and x are always looked up (a result written to another GPU's memory, or a
// host pointer, must not go unnoticed); the remaining pointers under NNLIB_B200_CHECK_POINTERS.
int check_devices(const nnlib_b200_attn_params* p) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return NNLIB_B200_CUDA_ERROR;
  }
  if (!on_current_device(p->q, dev) || !on_current_device(p->x, dev)) return NNLIB_B200_INVALID_ARG;
  if (check_all_pointers()) {
    const void* rest[] = {p->k, p->v, p->bias, p->mask, p->lse, p->alpha, p->status};
    for (const void* r : rest)
      if (!on_current_device(r, dev)) return NNLIB_B200_INVALID_ARG;
  }
  return NNLIB_B200_OK;
}

void log_call(const char* entry, const nnlib_b200_attn_params* p, const AttnArgs& a, const char* path,
              const char* why) {
  if (!log_calls()) return;
  static const char* const names[] = {"f16", "bf16", "f32"};
  std::fprintf(stderr,
               "[nnlib_b200] %s %s d=%d dv=%d H=%d Lq=%d Lkv=%d B=%d causal=%d mask=%d bias=%d dropout=%g -> %s%s%s\n",
               entry, names[p->dtype], a.d, a.dv, a.H, a.Lq, a.Lkv, a.B, a.causal, a.mask ? 1 : 0, a.bias ? 1 : 0,
               (double)a.dropout_p, path, why ? ": " : "", why ? why : "");
}

enum Need : unsigned {
  NEED_V = 1u,      // v and x
  NEED_LSE_IN = 2u, // lse must be given
  NEED_ALPHA = 4u,  // alpha must be given
  NEED_QK = 8u      // q and k
};

int dtype_ok(int dt) { return dt == NNLIB_B200_F16 || dt == NNLIB_B200_BF16 || dt == NNLIB_B200_F32; }

// Validate the caller's struct and turn it into the kernels' argument block.
// `launching`: the call is about to enqueue kernels, so the arrays' device is checked too (the path queries
// are pure host logic and skip that).
int resolve(const nnlib_b200_attn_params* p, unsigned need, AttnArgs* out, bool launching = true) {
  if (!p || p->struct_size != sizeof(nnlib_b200_attn_params)) return NNLIB_B200_INVALID_ARG;
  if (!dtype_ok(p->dtype)) return NNLIB_B200_INVALID_ARG;
  if (p->d < 1 || p->H < 1 || p->Lq < 0 || p->Lkv < 0 || p->B < 0) return NNLIB_B200_INVALID_ARG;
  if ((need & NEED_V) && p->dv < 1) return NNLIB_B200_INVALID_ARG;
  if (p->Lq > 0x7fffffffLL || p->Lkv > 0x7fffffffLL || p->H > 0x7fffffffLL || p->B > 0x7fffffffLL ||
      p->d > 0x7fffffffLL || p->dv > 0x7fffffffLL)
    return NNLIB_B200_INVALID_ARG;
  const bool empty = (p->Lq == 0 || p->B == 0);
  AttnArgs a;
  std::memset(&a, 0, sizeof(a));
  a.d = (int)p->d; a.dv = (int)p->dv; a.H = (int)p->H; a.Lq = (int)p->Lq; a.Lkv = (int)p->Lkv; a.B = (int)p->B;
  const long long E = p->H * p->d, Ev = p->H * p->dv;
  a.q = p->q; a.k = p->k; a.v = p->v; a.x = p->x;
  a.q_sl = p->q_stride_l ? p->q_stride_l : E;   a.q_sb = p->q_stride_b ? p->q_stride_b : a.q_sl * p->Lq;
  a.k_sl = p->k_stride_l ? p->k_stride_l : E;   a.k_sb = p->k_stride_b ? p->k_stride_b : a.k_sl * p->Lkv;
  a.v_sl = p->v_stride_l ? p->v_stride_l : Ev;  a.v_sb = p->v_stride_b ? p->v_stride_b : a.v_sl * p->Lkv;
  a.x_sl = p->x_stride_l ? p->x_stride_l : Ev;  a.x_sb = p->x_stride_b ? p->x_stride_b : a.x_sl * p->Lq;
  if (a.q_sl < E || a.k_sl < E || a.q_sb < 0 || a.k_sb < 0) return NNLIB_B200_INVALID_ARG;
  if ((need & NEED_V) && (a.v_sl < Ev || a.x_sl < Ev || a.v_sb < 0 || a.x_sb < 0)) return NNLIB_B200_INVALID_ARG;
  if (!empty) {
    if ((need & NEED_QK) && (!p->q || (p->Lkv > 0 && !p->k))) return NNLIB_B200_INVALID_ARG;
    if ((need & NEED_V) && (!p->x || (p->Lkv > 0 && !p->v))) return NNLIB_B200_INVALID_ARG;
    if ((need & NEED_LSE_IN) && !p->lse) return NNLIB_B200_INVALID_ARG;
    if ((need & NEED_ALPHA) && p->Lkv > 0 && !p->alpha) return NNLIB_B200_INVALID_ARG;
  }
  a.bias = p->bias;
  a.bias_dtype = p->bias_dtype;
  if (p->bias && !dtype_ok(p->bias_dtype)) return NNLIB_B200_INVALID_ARG;
  a.mask = p->mask;
  for (int i = 0; i < 4; ++i) {
    if (p->bias_stride[i] < 0 || p->mask_stride[i] < 0) return NNLIB_B200_INVALID_ARG;
    a.bias_s[i] = p->bias_stride[i];
    a.mask_s[i] = p->mask_stride[i];
  }
  a.causal = p->causal ? 1 : 0;
  if (p->causal_offset > 0x3fffffffLL || p->causal_offset < -0x3fffffffLL) return NNLIB_B200_INVALID_ARG;
  a.coff = a.causal ? (int)p->causal_offset : 0;
  a.nan_fm = p->nan_on_fully_masked ? 1 : 0;
  a.allow_tf32 = p->allow_tf32 ? 1 : 0;
  if (!(p->scale >= 0.f) || std::isinf(p->scale)) return NNLIB_B200_INVALID_ARG;
  a.scale = (p->scale == 0.f) ? (float)(1.0 / std::sqrt((double)p->d)) : p->scale;
  if (!(p->dropout_p >= 0.f && p->dropout_p < 1.f)) return NNLIB_B200_INVALID_ARG;
  a.dropout_p = p->dropout_p;
  a.inv_keep = (float)(1.0 / (1.0 - (double)p->dropout_p));
  {
    const double th = std::floor((double)p->dropout_p * 65536.0);
    a.drop_thresh = (unsigned int)(th > 65535.0 ? 65535.0 : th);
  }
  a.key0 = (unsigned int)(p->philox_seed & 0xffffffffull);
  a.key1 = (unsigned int)(p->philox_seed >> 32);
  for (int r = 0; r < 10; ++r) {
    a.rkey[2 * r] = a.key0 + (unsigned int)r * kPhiloxW0;
    a.rkey[2 * r + 1] = a.key1 + (unsigned int)r * kPhiloxW1;
  }
  a.off_lo = (unsigned int)(p->philox_offset & 0xffffffffull);
  a.off_hi = (unsigned int)(p->philox_offset >> 32);
  if (p->rng_h0 < 0 || p->rng_b0 < 0 || p->rng_H < 0) return NNLIB_B200_INVALID_ARG;
  a.rng_h0 = p->rng_h0; a.rng_b0 = p->rng_b0; a.rng_H = p->rng_H ? p->rng_H : p->H;
  a.lse = p->lse;
  a.lse_sb = p->lse_stride_b ? p->lse_stride_b : p->Lq * p->H;
  a.alpha = p->alpha;
  a.alpha_sb = p->alpha_stride_b ? p->alpha_stride_b : p->Lkv * p->Lq * p->H;
  if (a.lse_sb < p->Lq * p->H || a.alpha_sb < p->Lkv * p->Lq * p->H) return NNLIB_B200_INVALID_ARG;
  a.status = p->status;
  if (!empty && launching) {
    const int rc = check_devices(p);
    if (rc) return rc;
  }
  *out = a;
  return NNLIB_B200_OK;
}

int finish(cudaError_t e) {
  if (e == cudaSuccess) return NNLIB_B200_OK;
  set_last_cuda_error(e);
  return NNLIB_B200_CUDA_ERROR;
}

// the two-tile tensor-core kernels: 16-bit arrays with d = dv <= 128 a multiple of 8
bool use_umma_fwd(const AttnArgs& a, int dtype, bool need_v) {
  return !force_simt() && umma_fwd_reject_reason(a, dtype, need_v) == nullptr;
}

// the one-tile tensor-core kernels: other head sizes, dv != d, Float32 on the TF32 path
bool use_tile(const AttnArgs& a, int dtype, bool need_v) {
  return !force_simt() && tile_reject_reason(a, dtype, need_v, a.allow_tf32 != 0) == nullptr;
}

// why a call does not run on the tensor-core kernels (for the log)
const char* simt_reason(const AttnArgs& a, int dtype, bool need_v) {
  return force_simt() ? "NNLIB_B200_FORCE_SIMT is set" : tile_reject_reason(a, dtype, need_v, a.allow_tf32 != 0);
}

}  // namespace

// Arguments of the x + alpha composite (attn_fwd followed by attn_scores), checked as a whole so that a
// bad alpha cannot surface after x and lse were already written.  Not exported.
int attention_validate(const nnlib_b200_attn_params* p, bool launching) {
  AttnArgs a;
  const int rc = resolve(p, NEED_QK | NEED_V | NEED_LSE_IN | NEED_ALPHA, &a, launching);
  if (rc) return rc;
  if (a.Lq == 0 || a.B == 0) return NNLIB_B200_OK;
  const bool fwd_ok = use_umma_fwd(a, p->dtype, true) || use_tile(a, p->dtype, true) || simt_supports(a.d, a.dv);
  const bool sc_ok = use_umma_fwd(a, p->dtype, false) || use_tile(a, p->dtype, false) || simt_supports(a.d, 1);
  return (fwd_ok && sc_ok) ? NNLIB_B200_OK : NNLIB_B200_UNSUPPORTED_SHAPE;
}

// x and alpha for validated arguments (lse given): one kernel when a query's whole score row fits in tensor
// memory, else the fused forward followed by the score-rebuild kernel
int attention_both(const nnlib_b200_attn_params* p, void* stream) {
  AttnArgs a;
  int rc = resolve(p, NEED_QK | NEED_V | NEED_LSE_IN | NEED_ALPHA, &a, false);
  if (rc) return rc;
  if (a.Lq > 0 && a.B > 0 && a.Lkv > 0 && !force_simt() && short_supports(a, p->dtype)) {
    log_call("attention", p, a, "tcgen05 (x and alpha in one pass)", nullptr);
    return finish(short_attention(a, p->dtype, (cudaStream_t)stream));
  }
  rc = nnlib_b200_attn_fwd(p, stream);
  if (rc) return rc;
  return nnlib_b200_attn_scores(p, stream);
}

}  // namespace nb200

using namespace nb200;

extern "C" {

int nnlib_b200_attn_fwd(const nnlib_b200_attn_params* p, void* stream) {
  AttnArgs a;
  const int rc = resolve(p, NEED_QK | NEED_V, &a);
  if (rc) return rc;
  if (a.Lq == 0 || a.B == 0) return NNLIB_B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (use_umma_fwd(a, p->dtype, true)) {
    log_call("attn_fwd", p, a, "tcgen05", nullptr);
    return finish(umma_fwd(a, p->dtype, false, st));
  }
  if (use_tile(a, p->dtype, true)) {
    log_call("attn_fwd", p, a, "tcgen05 (one query tile per CTA)", umma_fwd_reject_reason(a, p->dtype, true));
    return finish(tile_fwd(a, p->dtype, st));
  }
  if (!simt_supports(a.d, a.dv)) return NNLIB_B200_UNSUPPORTED_SHAPE;
  log_call("attn_fwd", p, a, "cuda-core", simt_reason(a, p->dtype, true));
  return finish(simt_fwd(a, p->dtype, st));
}

// does the split-key forward apply to this call, and is it worth it (a long key sequence, too few units to
// fill the GPU otherwise)?
static bool use_split(const AttnArgs& a, int dtype) {
  if (a.Lq > 128 || force_simt()) return false;
  if (tile_reject_reason(a, dtype, true, a.allow_tf32 != 0) != nullptr) return false;
  return tile_split_count(a) > 1;
}

size_t nnlib_b200_attn_decode_workspace_bytes(const nnlib_b200_attn_params* p) {
  AttnArgs a;
  if (resolve(p, NEED_QK | NEED_V, &a, false) != NNLIB_B200_OK) return 0;
  if (a.Lq == 0 || a.B == 0 || !use_split(a, p->dtype)) return 0;
  return tile_split_workspace_bytes(a);
}

int nnlib_b200_attn_decode(const nnlib_b200_attn_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  AttnArgs a;
  const int rc = resolve(p, NEED_QK | NEED_V, &a);
  if (rc) return rc;
  if (a.Lq == 0 || a.B == 0) return NNLIB_B200_OK;
  if (!use_split(a, p->dtype)) return nnlib_b200_attn_fwd(p, stream);
  const size_t need = tile_split_workspace_bytes(a);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0)
    return NNLIB_B200_WORKSPACE_TOO_SMALL;
  a.ws = static_cast<float*>(workspace);
  if (log_calls()) {
    char what[96];
    std::snprintf(what, sizeof(what), "tcgen05 (keys split over %d CTAs per unit)", tile_split_count(a));
    log_call("attn_decode", p, a, what, nullptr);
  }
  return finish(tile_split(a, p->dtype, (cudaStream_t)stream));
}

int nnlib_b200_attn_stats(const nnlib_b200_attn_params* p, void* stream) {
  AttnArgs a;
  const int rc = resolve(p, NEED_QK | NEED_LSE_IN, &a);   // lse is this entry point's output: required
  if (rc) return rc;
  if (a.Lq == 0 || a.B == 0) return NNLIB_B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (use_umma_fwd(a, p->dtype, false)) {
    log_call("attn_stats", p, a, "tcgen05", nullptr);
    return finish(umma_fwd(a, p->dtype, true, st));
  }
  if (use_tile(a, p->dtype, false)) {
    log_call("attn_stats", p, a, "tcgen05 (one query tile per CTA)", umma_fwd_reject_reason(a, p->dtype, false));
    return finish(tile_stats(a, p->dtype, st));
  }
  if (!simt_supports(a.d, 1)) return NNLIB_B200_UNSUPPORTED_SHAPE;
  log_call("attn_stats", p, a, "cuda-core", simt_reason(a, p->dtype, false));
  return finish(simt_stats(a, p->dtype, st));
}

int nnlib_b200_attn_scores(const nnlib_b200_attn_params* p, void* stream) {
  AttnArgs a;
  const int rc = resolve(p, NEED_QK | NEED_LSE_IN | NEED_ALPHA, &a);
  if (rc) return rc;
  if (a.Lq == 0 || a.B == 0 || a.Lkv == 0) return NNLIB_B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (use_umma_fwd(a, p->dtype, false)) {
    log_call("attn_scores", p, a, "tcgen05", nullptr);
    return finish(umma_scores(a, p->dtype, st));
  }
  if (use_tile(a, p->dtype, false)) {
    log_call("attn_scores", p, a, "tcgen05 (one query tile per CTA)", umma_fwd_reject_reason(a, p->dtype, false));
    return finish(tile_scores(a, p->dtype, st));
  }
  if (!simt_supports(a.d, 1)) return NNLIB_B200_UNSUPPORTED_SHAPE;
  log_call("attn_scores", p, a, "cuda-core", simt_reason(a, p->dtype, false));
  return finish(simt_scores(a, p->dtype, st));
}

int nnlib_b200_attn_apply(const nnlib_b200_attn_params* p, void* stream) {
  AttnArgs a;
  const int rc = resolve(p, NEED_V | NEED_ALPHA, &a);
  if (rc) return rc;
  if (a.Lq == 0 || a.B == 0) return NNLIB_B200_OK;
  if (a.Lkv > 0 && !force_simt() && umma_apply_supports(a, p->dtype)) {
    log_call("attn_apply", p, a, "tcgen05", nullptr);
    return finish(umma_apply(a, p->dtype, (cudaStream_t)stream));
  }
  if (!simt_supports(1, a.dv)) return NNLIB_B200_UNSUPPORTED_SHAPE;
  log_call("attn_apply", p, a, "cuda-core", force_simt() ? "NNLIB_B200_FORCE_SIMT is set"
                                                         : "16-bit arrays with dv a multiple of 8 up to 128, Lkv % 8 == 0 and "
                                                           "16-byte aligned rows only");
  return finish(simt_apply(a, p->dtype, (cudaStream_t)stream));
}

// shared front half of attn_bwd / attn_bwd_path: validates and resolves both argument blocks
static int resolve_bwd(const nnlib_b200_attn_params* p, const nnlib_b200_attn_grads* g, AttnArgs* a, BwdArgs* b,
                       bool launching = true) {
  const int rc = resolve(p, NEED_QK | NEED_V | NEED_LSE_IN, a, false);   // the device check comes last
  if (rc) return rc;
  if (!g || g->struct_size != sizeof(nnlib_b200_attn_grads)) return NNLIB_B200_INVALID_ARG;
  const bool empty = (a->Lq == 0 || a->B == 0);
  if (!empty && (!g->dx || !g->dq || !g->delta)) return NNLIB_B200_INVALID_ARG;
  // dk and dv are written (zeros) even when there are no queries, as long as there are keys
  if (a->B > 0 && a->Lkv > 0 && (!g->dk || !g->dv)) return NNLIB_B200_INVALID_ARG;
  std::memset(b, 0, sizeof(*b));
  const long long Ev = (long long)a->H * a->dv;
  b->dx = g->dx;
  b->dx_sl = g->dx_stride_l ? g->dx_stride_l : Ev;
  b->dx_sb = g->dx_stride_b ? g->dx_stride_b : b->dx_sl * a->Lq;
  if (b->dx_sl < Ev || b->dx_sb < 0) return NNLIB_B200_INVALID_ARG;
  b->dq = g->dq; b->dk = g->dk; b->dv = g->dv;
  b->dbias = g->dbias;
  for (int i = 0; i < 4; ++i) {
    if (g->dbias_stride[i] < 0) return NNLIB_B200_INVALID_ARG;
    b->dbias_s[i] = g->dbias_stride[i];
  }
  b->delta = g->delta;
  if (launching && !empty) return check_devices(p);
  return NNLIB_B200_OK;
}

int nnlib_b200_attn_bwd(const nnlib_b200_attn_params* p, const nnlib_b200_attn_grads* g, void* stream) {
  AttnArgs a;
  BwdArgs b;
  const int rc = resolve_bwd(p, g, &a, &b);
  if (rc) return rc;
  if (a.B == 0 || (a.Lq == 0 && a.Lkv == 0)) return NNLIB_B200_OK;
  if (!force_simt() && umma_bwd_supports(a, b, p->dtype)) {
    log_call("attn_bwd", p, a, "tcgen05", nullptr);
    return finish(umma_bwd(a, b, p->dtype, (cudaStream_t)stream));
  }
  if (!simt_bwd_supports(a.d, a.dv)) return NNLIB_B200_UNSUPPORTED_SHAPE;
  log_call("attn_bwd", p, a, "cuda-core", force_simt() ? "NNLIB_B200_FORCE_SIMT is set"
                                                       : "16-bit arrays with d = dv a multiple of 8 up to 128 and 16-byte aligned rows only");
  return finish(simt_bwd(a, b, p->dtype, (cudaStream_t)stream));
}

int nnlib_b200_attn_bwd_path(const nnlib_b200_attn_params* p, const nnlib_b200_attn_grads* g) {
  AttnArgs a;
  BwdArgs b;
  const int rc = resolve_bwd(p, g, &a, &b, false);
  if (rc) return rc;
  if (!force_simt() && umma_bwd_supports(a, b, p->dtype)) return NNLIB_B200_PATH_UMMA;
  if (!simt_bwd_supports(a.d, a.dv)) return NNLIB_B200_UNSUPPORTED_SHAPE;
  return NNLIB_B200_PATH_SIMT;
}

size_t nnlib_b200_workspace_bytes(const nnlib_b200_attn_params* p) {
  if (!p || p->struct_size != sizeof(nnlib_b200_attn_params)) return 0;
  if (p->lse) return 0;
  if (p->Lq < 0 || p->H < 0 || p->B < 0) return 0;
  return (size_t)p->Lq * (size_t)p->H * (size_t)p->B * sizeof(float);
}

int nnlib_b200_attention(const nnlib_b200_attn_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  if (!p || p->struct_size != sizeof(nnlib_b200_attn_params)) return NNLIB_B200_INVALID_ARG;
  nnlib_b200_attn_params q = *p;
  if (!q.lse) {
    const size_t need = nnlib_b200_workspace_bytes(p);
    if (need > 0 && (!workspace || workspace_bytes < need)) return NNLIB_B200_WORKSPACE_TOO_SMALL;
    q.lse = static_cast<float*>(workspace);
    q.lse_stride_b = 0;
  }
  // every argument of both halves is checked before the first kernel is enqueued
  int rc = attention_validate(&q);
  if (rc) return rc;
  return attention_both(&q, stream);
}

static int check_softmax(const nnlib_b200_softmax_params* p, bool backward) {
  if (!p || p->struct_size != sizeof(nnlib_b200_softmax_params)) return NNLIB_B200_INVALID_ARG;
  if (p->dtype != NNLIB_B200_F16 && p->dtype != NNLIB_B200_BF16 && p->dtype != NNLIB_B200_F32) return NNLIB_B200_INVALID_ARG;
  if (p->inner < 0 || p->n < 0 || p->outer < 0) return NNLIB_B200_INVALID_ARG;
  const bool empty = (p->inner == 0 || p->n == 0 || p->outer == 0);
  if (!empty && (!p->x || !p->out || (backward && !p->dy))) return NNLIB_B200_INVALID_ARG;
  if (!empty && p->inner > (1ll << 62) / p->n / p->outer) return NNLIB_B200_INVALID_ARG;
  return empty ? 1 : NNLIB_B200_OK;   // 1: nothing to do
}

int nnlib_b200_softmax_fwd(const nnlib_b200_softmax_params* p, void* stream) {
  const int rc = check_softmax(p, false);
  if (rc) return rc < 0 ? rc : NNLIB_B200_OK;
  return finish(softmax_forward(p->dtype, p->log != 0, p->x, p->out, p->inner, p->n, p->outer, (cudaStream_t)stream));
}

int nnlib_b200_softmax_bwd(const nnlib_b200_softmax_params* p, void* stream) {
  const int rc = check_softmax(p, true);
  if (rc) return rc < 0 ? rc : NNLIB_B200_OK;
  return finish(softmax_backward(p->dtype, p->log != 0, p->dy, p->x, p->out, p->inner, p->n, p->outer, (cudaStream_t)stream));
}

// validates the caller's struct and fills the kernels' argument block
static int resolve_gemm(const nnlib_b200_gemm_params* p, GemmArgs* out) {
  if (!p || p->struct_size != sizeof(nnlib_b200_gemm_params)) return NNLIB_B200_INVALID_ARG;
  if (!dtype_ok(p->dtype)) return NNLIB_B200_INVALID_ARG;
  if ((p->transA != 0 && p->transA != 1) || (p->transB != 0 && p->transB != 1)) return NNLIB_B200_INVALID_ARG;
  if (p->M < 0 || p->N < 0 || p->K < 0 || p->batch < 0) return NNLIB_B200_INVALID_ARG;
  if (p->M > 0x7fffffffLL || p->N > 0x7fffffffLL || p->K > 0x7fffffffLL || p->batch > 0x7fffffffLL)
    return NNLIB_B200_INVALID_ARG;
  if (!std::isfinite(p->alpha) || !std::isfinite(p->beta)) return NNLIB_B200_INVALID_ARG;
  const bool empty = (p->M == 0 || p->N == 0 || p->batch == 0);
  // stored shapes: A is (M, K) or, transposed, (K, M); B is (K, N) or (N, K); the leading dimension covers a column
  const int64_t a_rows = p->transA ? p->K : p->M, b_rows = p->transB ? p->N : p->K;
  if (p->lda < (a_rows > 1 ? a_rows : 1) || p->ldb < (b_rows > 1 ? b_rows : 1) || p->ldc < (p->M > 1 ? p->M : 1))
    return NNLIB_B200_INVALID_ARG;
  if (p->strideA < 0 || p->strideB < 0 || p->strideC < 0) return NNLIB_B200_INVALID_ARG;
  if (!empty) {
    if (!p->C || (p->K > 0 && (!p->A || !p->B))) return NNLIB_B200_INVALID_ARG;
    if (p->batch > 1 && p->strideC < p->ldc * (p->N - 1) + p->M) return NNLIB_B200_INVALID_ARG;   // batches of C overlap
  }
  GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.A = p->A; g.B = p->B; g.C = p->C;
  g.lda = p->lda; g.ldb = p->ldb; g.ldc = p->ldc;
  g.strideA = p->strideA; g.strideB = p->strideB; g.strideC = p->strideC;
  g.M = (int)p->M; g.N = (int)p->N; g.K = (int)p->K; g.batch = (int)p->batch;
  g.transA = p->transA; g.transB = p->transB;
  g.a_bcast = (p->strideA == 0) ? 1 : 0;
  g.b_bcast = (p->strideB == 0) ? 1 : 0;
  g.alpha = p->alpha; g.beta = p->beta;
  g.status = p->status;
  *out = g;
  return NNLIB_B200_OK;
}

int nnlib_b200_batched_gemm(const nnlib_b200_gemm_params* p, void* stream) {
  GemmArgs g;
  const int rc = resolve_gemm(p, &g);
  if (rc) return rc;
  if (g.M == 0 || g.N == 0 || g.batch == 0) return NNLIB_B200_OK;
  {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return NNLIB_B200_CUDA_ERROR; }
    if (!on_current_device(g.C, dev) || !on_current_device(g.A, dev)) return NNLIB_B200_INVALID_ARG;
    if (check_all_pointers() && !on_current_device(g.B, dev)) return NNLIB_B200_INVALID_ARG;
  }
  const char* why = force_simt() ? "NNLIB_B200_FORCE_SIMT is set" : gemm_umma_reject_reason(g, p->dtype);
  if (log_calls()) {
    static const char* const names[] = {"f16", "bf16", "f32"};
    std::fprintf(stderr, "[nnlib_b200] batched_gemm %s %c%c M=%d N=%d K=%d batch=%d alpha=%g beta=%g -> %s%s%s\n",
                 names[p->dtype], g.transA ? 'T' : 'N', g.transB ? 'T' : 'N', g.M, g.N, g.K, g.batch, (double)g.alpha,
                 (double)g.beta, why ? "cuda-core" : "tcgen05", why ? ": " : "", why ? why : "");
  }
  if (!why) return finish(gemm_umma(g, p->dtype, (cudaStream_t)stream));
  return finish(gemm_simt(g, p->dtype, (cudaStream_t)stream));
}

int nnlib_b200_batched_gemm_path(const nnlib_b200_gemm_params* p) {
  GemmArgs g;
  const int rc = resolve_gemm(p, &g);
  if (rc) return rc;
  return (!force_simt() && gemm_umma_reject_reason(g, p->dtype) == nullptr) ? NNLIB_B200_PATH_UMMA : NNLIB_B200_PATH_SIMT;
}

int nnlib_b200_causal_fill(uint8_t* mask, int64_t L, void* stream) {
  if (L < 0 || (L > 0 && !mask)) return NNLIB_B200_INVALID_ARG;
  return finish(causal_fill(mask, L, (cudaStream_t)stream));
}

int nnlib_b200_causal_check(const uint8_t* mask, int64_t L, int32_t* flag, void* stream) {
  if (L < 0 || (L > 0 && !mask) || !flag) return NNLIB_B200_INVALID_ARG;
  return finish(causal_check(mask, L, flag, (cudaStream_t)stream));
}

int nnlib_b200_attn_path(const nnlib_b200_attn_params* p) {
  AttnArgs a;
  const int rc = resolve(p, NEED_QK | NEED_V, &a, false);
  if (rc) return rc;
  if (use_umma_fwd(a, p->dtype, true)) return NNLIB_B200_PATH_UMMA;
  if (use_tile(a, p->dtype, true)) return NNLIB_B200_PATH_TILE;
  if (!simt_supports(a.d, a.dv)) return NNLIB_B200_UNSUPPORTED_SHAPE;
  return NNLIB_B200_PATH_SIMT;
}

int nnlib_b200_device_health(void* stream) {
  int v = 0, w = 0, u = 0, t = 0, s = 0;
  cudaError_t e = short_take_abort(&s, (cudaStream_t)stream);
  v = 0;
  if (e == cudaSuccess) e = umma_take_abort(&v, (cudaStream_t)stream);
  if (e == cudaSuccess) e = umma_bwd_take_abort(&w, (cudaStream_t)stream);
  if (e == cudaSuccess) e = gemm_take_abort(&u, (cudaStream_t)stream);
  if (e == cudaSuccess) e = tile_take_abort(&t, (cudaStream_t)stream);
  if (e != cudaSuccess) return finish(e);
  return (v || w || u || t || s) ? NNLIB_B200_TIMEOUT : NNLIB_B200_OK;
}

int nnlib_b200_selftest_wait_runout(uint64_t limit_ns, int32_t* status, void* stream) {
  if (limit_ns == 0 || limit_ns > 1000000000ull) return NNLIB_B200_INVALID_ARG;   // at most the kernels' own 1 s
  return finish(umma_wait_runout(limit_ns, status, (cudaStream_t)stream));
}

const char* nnlib_b200_strerror(int code) {
  switch (code) {
    case NNLIB_B200_OK: return "ok";
    case NNLIB_B200_INVALID_ARG: return "invalid argument (null pointer, size, stride, dtype or dropout probability)";
    case NNLIB_B200_UNSUPPORTED_SHAPE: return "head dimension not supported by any kernel of this library";
    case NNLIB_B200_CUDA_ERROR: return "a CUDA call failed (see nnlib_b200_last_cuda_error)";
    case NNLIB_B200_TIMEOUT: return "a kernel gave up on a bounded wait; results of that launch are invalid";
    case NNLIB_B200_WORKSPACE_TOO_SMALL: return "workspace smaller than nnlib_b200_workspace_bytes";
    default: return "unknown nnlib_b200 status";
  }
}

int nnlib_b200_version(void) { return NNLIB_B200_VERSION; }
int nnlib_b200_last_cuda_error(void) { return t_last_cuda_error; }
uint64_t nnlib_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
