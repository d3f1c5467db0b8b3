// Backward of the attention path on CUDA cores (fp32 arithmetic, any shape).
//
// Given the forward inputs, the forward output x, the saved log-sum-exp and the
// cotangent dx, computes what Zygote composes from NNlib.jl's own rules for
// this path: rrule(batched_mul) (src/batched/batchedmul.jl:96-110), ∇softmax
// (src/softmax.jl:84-110), the dropout pullback (src/dropout.jl:106-122) and
// the 1/sqrt(d) scaling of q (src/attention.jl:118).  With
//   alpha  = exp(logit - lse)            (recomputed, never stored)
//   alpha' = alpha * keep / (1-p)        (same Philox positions as the forward)
//   D_i    = dx_i · x_i                  (= sum_j alpha'_ij dalpha'_ij)
//   ds_ij  = alpha_ij * (keep/(1-p) * dx_i·v_j - D_i)
// the results are dq_i = scale * sum_j ds_ij k_j, dk_j = scale * sum_i ds_ij q_i,
// dv_j = sum_i alpha'_ij dx_i and dbias = ds reduced over the broadcast dims.
// Two kernels, one warp per query row (dq, D, dbias) and one warp per key row
// (dk, dv); both recompute the logits.
#include "common.cuh"
#include "launchers.h"

namespace nb200 {
namespace {

constexpr int kWarps = 4;
constexpr int kMaxRegs = 16;  // d, dv <= 512

__device__ __forceinline__ float ninf() { return __int_as_float(0xff800000); }

template <typename T>
__device__ __forceinline__ float logit_qk(const AttnArgs& a, const T* qrow, const T* krow, int j, int i, int h, int b) {
  float s = 0.f;
  for (int e = 0; e < a.d; ++e) s = fmaf(Elem<T>::to_f(qrow[e]), Elem<T>::to_f(krow[e]), s);
  s *= a.scale;
  if (a.bias) s += load_bias(a.bias, j * a.bias_s[0] + i * a.bias_s[1] + h * a.bias_s[2] + b * a.bias_s[3], a.bias_dtype);
  bool keep = true;
  if (a.causal) keep = (j <= i + a.coff);
  if (a.mask) keep = keep && (a.mask[j * a.mask_s[0] + i * a.mask_s[1] + h * a.mask_s[2] + b * a.mask_s[3]] != 0);
  return keep ? s : ninf();
}

// keep/(1-p) factor of score (j, row)
__device__ __forceinline__ float drop_factor(const AttnArgs& a, unsigned long long srow, int j) {
  if (!(a.dropout_p > 0.f)) return 1.f;
  return dropout_keep1(a, srow, (unsigned int)j) ? a.inv_keep : 0.f;
}

// ---- one warp per query row: D_i, dq_i, dbias --------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) attn_bwd_dq_kernel(const AttnArgs a, const BwdArgs g) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long total = (long long)a.Lq * a.H * a.B;
  const long long row = (long long)blockIdx.x * kWarps + warp;
  if (row >= total) return;
  const int i = (int)(row % a.Lq), h = (int)((row / a.Lq) % a.H), b = (int)(row / ((long long)a.Lq * a.H));
  const T* qrow = reinterpret_cast<const T*>(a.q) + (long long)i * a.q_sl + (long long)b * a.q_sb + (long long)h * a.d;
  const T* xrow = reinterpret_cast<const T*>(a.x) + (long long)i * a.x_sl + (long long)b * a.x_sb + (long long)h * a.dv;
  const T* dxrow = reinterpret_cast<const T*>(g.dx) + (long long)i * g.dx_sl + (long long)b * g.dx_sb + (long long)h * a.dv;
  const float lse = a.lse[i + (long long)a.Lq * h + a.lse_sb * b];
  const unsigned long long srow = score_row(a, i, h, b);

  float dl = 0.f;
  for (int e = lane; e < a.dv; e += 32) dl = fmaf(Elem<T>::to_f(dxrow[e]), Elem<T>::to_f(xrow[e]), dl);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) dl += __shfl_xor_sync(0xffffffffu, dl, off);
  if (lane == 0) g.delta[i + (long long)a.Lq * h + (long long)a.Lq * a.H * b] = dl;

  float acc[kMaxRegs];
#pragma unroll
  for (int r = 0; r < kMaxRegs; ++r) acc[r] = 0.f;
  const bool dead = (lse == ninf());   // nothing attended: the forward produced NaN (or 0); no gradient flows
  for (int j0 = 0; j0 < a.Lkv; j0 += 32) {
    const int j = j0 + lane;
    float ds = 0.f;
    if (j < a.Lkv && !dead) {
      const T* krow = reinterpret_cast<const T*>(a.k) + (long long)j * a.k_sl + (long long)b * a.k_sb + (long long)h * a.d;
      const float s = logit_qk<T>(a, qrow, krow, j, i, h, b);
      if (s != ninf()) {
        const float p = expf(s - lse);
        const T* vrow = reinterpret_cast<const T*>(a.v) + (long long)j * a.v_sl + (long long)b * a.v_sb + (long long)h * a.dv;
        float dp = 0.f;
        for (int e = 0; e < a.dv; ++e) dp = fmaf(Elem<T>::to_f(dxrow[e]), Elem<T>::to_f(vrow[e]), dp);
        ds = p * (dp * drop_factor(a, srow, j) - dl);
        if (g.dbias)
          atomicAdd(g.dbias + j * g.dbias_s[0] + i * g.dbias_s[1] + h * g.dbias_s[2] + b * g.dbias_s[3], ds);
      }
    }
    const int nj = min(32, a.Lkv - j0);
    for (int jj = 0; jj < nj; ++jj) {
      const float dsj = __shfl_sync(0xffffffffu, ds, jj);
      if (dsj != 0.f) {
        const T* krow = reinterpret_cast<const T*>(a.k) + (long long)(j0 + jj) * a.k_sl + (long long)b * a.k_sb + (long long)h * a.d;
#pragma unroll
        for (int r = 0; r < kMaxRegs; ++r) {
          const int e = lane + 32 * r;
          if (e < a.d) acc[r] = fmaf(dsj, Elem<T>::to_f(krow[e]), acc[r]);
        }
      }
    }
  }
  T* dqrow = reinterpret_cast<T*>(g.dq) + ((long long)i + (long long)a.Lq * b) * ((long long)a.H * a.d) + (long long)h * a.d;
#pragma unroll
  for (int r = 0; r < kMaxRegs; ++r) {
    const int e = lane + 32 * r;
    if (e < a.d) dqrow[e] = Elem<T>::from_f(acc[r] * a.scale);
  }
}

// ---- one warp per key row: dk_j, dv_j ------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) attn_bwd_dkv_kernel(const AttnArgs a, const BwdArgs g) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long total = (long long)a.Lkv * a.H * a.B;
  const long long row = (long long)blockIdx.x * kWarps + warp;
  if (row >= total) return;
  const int j = (int)(row % a.Lkv), h = (int)((row / a.Lkv) % a.H), b = (int)(row / ((long long)a.Lkv * a.H));
  const T* krow = reinterpret_cast<const T*>(a.k) + (long long)j * a.k_sl + (long long)b * a.k_sb + (long long)h * a.d;
  const T* vrow = reinterpret_cast<const T*>(a.v) + (long long)j * a.v_sl + (long long)b * a.v_sb + (long long)h * a.dv;

  float dk[kMaxRegs], dv[kMaxRegs];
#pragma unroll
  for (int r = 0; r < kMaxRegs; ++r) { dk[r] = 0.f; dv[r] = 0.f; }
  for (int i0 = 0; i0 < a.Lq; i0 += 32) {
    const int i = i0 + lane;
    float ds = 0.f, ad = 0.f;   // ds_ij and alpha'_ij of this lane's query
    if (i < a.Lq) {
      const float lse = a.lse[i + (long long)a.Lq * h + a.lse_sb * b];
      if (lse != ninf()) {
        const T* qrow = reinterpret_cast<const T*>(a.q) + (long long)i * a.q_sl + (long long)b * a.q_sb + (long long)h * a.d;
        const float s = logit_qk<T>(a, qrow, krow, j, i, h, b);
        if (s != ninf()) {
          const float p = expf(s - lse);
          const T* dxrow = reinterpret_cast<const T*>(g.dx) + (long long)i * g.dx_sl + (long long)b * g.dx_sb + (long long)h * a.dv;
          float dp = 0.f;
          for (int e = 0; e < a.dv; ++e) dp = fmaf(Elem<T>::to_f(dxrow[e]), Elem<T>::to_f(vrow[e]), dp);
          const float f = drop_factor(a, score_row(a, i, h, b), j);
          const float dl = g.delta[i + (long long)a.Lq * h + (long long)a.Lq * a.H * b];
          ad = p * f;
          ds = p * (dp * f - dl);
        }
      }
    }
    const int ni = min(32, a.Lq - i0);
    for (int ii = 0; ii < ni; ++ii) {
      const float dsi = __shfl_sync(0xffffffffu, ds, ii);
      const float adi = __shfl_sync(0xffffffffu, ad, ii);
      if (dsi != 0.f || adi != 0.f) {
        const T* qrow = reinterpret_cast<const T*>(a.q) + (long long)(i0 + ii) * a.q_sl + (long long)b * a.q_sb + (long long)h * a.d;
        const T* dxrow = reinterpret_cast<const T*>(g.dx) + (long long)(i0 + ii) * g.dx_sl + (long long)b * g.dx_sb + (long long)h * a.dv;
#pragma unroll
        for (int r = 0; r < kMaxRegs; ++r) {
          const int e = lane + 32 * r;
          if (e < a.d) dk[r] = fmaf(dsi, Elem<T>::to_f(qrow[e]), dk[r]);
          if (e < a.dv) dv[r] = fmaf(adi, Elem<T>::to_f(dxrow[e]), dv[r]);
        }
      }
    }
  }
  T* dkrow = reinterpret_cast<T*>(g.dk) + ((long long)j + (long long)a.Lkv * b) * ((long long)a.H * a.d) + (long long)h * a.d;
  T* dvrow = reinterpret_cast<T*>(g.dv) + ((long long)j + (long long)a.Lkv * b) * ((long long)a.H * a.dv) + (long long)h * a.dv;
#pragma unroll
  for (int r = 0; r < kMaxRegs; ++r) {
    const int e = lane + 32 * r;
    if (e < a.d) dkrow[e] = Elem<T>::from_f(dk[r] * a.scale);
    if (e < a.dv) dvrow[e] = Elem<T>::from_f(dv[r]);
  }
}

template <typename T>
cudaError_t launch_bwd(const AttnArgs& a, const BwdArgs& g, cudaStream_t st) {
  const long long rows_q = (long long)a.Lq * a.H * a.B, rows_k = (long long)a.Lkv * a.H * a.B;
  const long long bq = (rows_q + kWarps - 1) / kWarps, bk = (rows_k + kWarps - 1) / kWarps;
  if (bq > 0x7fffffffLL || bk > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  if (bq > 0) {
    attn_bwd_dq_kernel<T><<<(unsigned)bq, kWarps * 32, 0, st>>>(a, g);
    count_launch();
  }
  if (bk > 0) {
    attn_bwd_dkv_kernel<T><<<(unsigned)bk, kWarps * 32, 0, st>>>(a, g);
    count_launch();
  }
  return cudaGetLastError();
}

}  // namespace

bool simt_bwd_supports(int d, int dv) { return d >= 1 && d <= 32 * kMaxRegs && dv >= 1 && dv <= 32 * kMaxRegs; }

cudaError_t simt_bwd(const AttnArgs& a, const BwdArgs& g, int dtype, cudaStream_t st) {
  switch (dtype) {
    case NNLIB_B200_F16:  return launch_bwd<__half>(a, g, st);
    case NNLIB_B200_BF16: return launch_bwd<__nv_bfloat16>(a, g, st);
    default:              return launch_bwd<float>(a, g, st);
  }
}

}  // namespace nb200
