// CUDA-core attention kernels: one warp per query row, fp32 arithmetic.
//
// They implement every entry point of the C ABI for ANY shape, stride and
// element type (f16 / bf16 / f32), with the exact two-pass softmax of the
// reference (NNlib.jl src/softmax.jl:69-79): pass A finds the row's
// log-sum-exp, pass B forms alpha = exp(logit - lse), applies dropout and
// accumulates x = sum_j alpha'_j v_j (src/attention.jl:96-98,117-126).
// Shapes the tensor-core kernels do not take (f32 inputs, head sizes other
// than 64/128, unaligned rows) run here.
#include "common.cuh"
#include "launchers.h"

namespace nb200 {

namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxDvRegs = 16;  // dv <= 32 * kMaxDvRegs

enum : int { MODE_FWD = 0, MODE_STATS = 1, MODE_SCORES = 2, MODE_APPLY = 3 };

__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }

// logit of (kv j, query i, head h, batch b): scaled q·k + bias, then masks.
template <typename T>
__device__ __forceinline__ float logit_at(const AttnArgs& a, const float* qs, int j, int i, int h, int b) {
  const T* kp = reinterpret_cast<const T*>(a.k) + (long long)j * a.k_sl + (long long)b * a.k_sb + (long long)h * a.d;
  float s = 0.f;
  for (int e = 0; e < a.d; ++e) s = fmaf(qs[e], Elem<T>::to_f(kp[e]), s);
  if (a.bias) {
    s += load_bias(a.bias, j * a.bias_s[0] + i * a.bias_s[1] + h * a.bias_s[2] + b * a.bias_s[3], a.bias_dtype);
  }
  bool keep = true;
  if (a.causal) keep = (j <= i + a.coff);
  if (a.mask) keep = keep && (a.mask[j * a.mask_s[0] + i * a.mask_s[1] + h * a.mask_s[2] + b * a.mask_s[3]] != 0);
  return keep ? s : neg_inf();
}

template <typename T, int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) attn_simt_kernel(const AttnArgs a) {
  extern __shared__ float smem_q[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long total = (long long)a.Lq * a.H * a.B;
  const long long row = (long long)blockIdx.x * kWarpsPerBlock + warp;
  if (row >= total) return;  // whole warps leave; no block-wide barrier follows
  const int i = (int)(row % a.Lq);
  const int h = (int)((row / a.Lq) % a.H);
  const int b = (int)(row / ((long long)a.Lq * a.H));

  float* qs = smem_q + warp * a.d;
  if (MODE != MODE_APPLY) {
    const T* qp = reinterpret_cast<const T*>(a.q) + (long long)i * a.q_sl + (long long)b * a.q_sb + (long long)h * a.d;
    for (int e = lane; e < a.d; e += 32) qs[e] = Elem<T>::to_f(qp[e]) * a.scale;
    __syncwarp();
  }

  float lse = 0.f;
  if (MODE == MODE_FWD || MODE == MODE_STATS) {
    // pass A: per-lane online max/sum over the lane's kv positions, then a butterfly merge
    // +Inf logits are counted apart and a NaN poisons the row (the slow branch of the reference's softmax,
    // src/softmax.jl:71-76)
    float m = neg_inf(), l = 0.f;
    int n_inf = 0;
    bool has_nan = false;
    for (int j = lane; j < a.Lkv; j += 32) {
      const float t = logit_at<T>(a, qs, j, i, h, b);
      if (t != t) {
        has_nan = true;
      } else if (t == __int_as_float(0x7f800000)) {
        ++n_inf;
      } else if (t > neg_inf()) {
        if (t > m) { l = l * expf(m - t) + 1.f; m = t; }
        else       { l += expf(t - m); }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, off);
      const float l2 = __shfl_xor_sync(0xffffffffu, l, off);
      const float mn = fmaxf(m, m2);
      const float la = (m == neg_inf()) ? 0.f : l * expf(m - mn);
      const float lb = (m2 == neg_inf()) ? 0.f : l2 * expf(m2 - mn);
      l = la + lb;
      m = mn;
      n_inf += __shfl_xor_sync(0xffffffffu, n_inf, off);
    }
    has_nan = __any_sync(0xffffffffu, has_nan);
    lse = (l > 0.f) ? m + logf(l) : neg_inf();
    if (n_inf > 0) lse = lse_inf_rows((float)n_inf);
    if (has_nan) lse = __int_as_float(0x7fc00000);
    if (a.lse && lane == 0) a.lse[i + (long long)a.Lq * h + a.lse_sb * b] = lse;
  } else if (MODE == MODE_SCORES) {
    lse = a.lse[i + (long long)a.Lq * h + a.lse_sb * b];
  }
  if (MODE == MODE_STATS) return;

  // pass B
  float acc[kMaxDvRegs];
#pragma unroll
  for (int r = 0; r < kMaxDvRegs; ++r) acc[r] = 0.f;
  const bool dead_row = (lse == neg_inf());
  const bool inf_row = lse_is_inf_rows(lse);
  const bool nan_row = (lse != lse) && !inf_row;
  const float inf_share = inf_row ? 1.f / lse_inf_count(lse) : 0.f;
  const unsigned long long srow = score_row(a, i, h, b);
  T* alpha_row = reinterpret_cast<T*>(a.alpha) +
                 ((long long)i + (long long)a.Lq * h) * a.Lkv + a.alpha_sb * b;
  const T* vbase = reinterpret_cast<const T*>(a.v) + (long long)b * a.v_sb + (long long)h * a.dv;

  for (int j0 = 0; j0 < a.Lkv; j0 += 32) {
    const int j = j0 + lane;
    float al = 0.f;
    if (j < a.Lkv) {
      if (MODE == MODE_APPLY) {
        al = Elem<T>::to_f(alpha_row[j]);
      } else {
        const float t = logit_at<T>(a, qs, j, i, h, b);
        if (dead_row)      al = a.nan_fm ? __int_as_float(0x7fc00000) : 0.f;
        else if (nan_row)  al = __int_as_float(0x7fc00000);
        else if (inf_row)  al = (t == __int_as_float(0x7f800000)) ? inf_share : 0.f;
        else               al = (t == neg_inf()) ? 0.f : expf(t - lse);
        if (a.dropout_p > 0.f) {
          al = dropout_keep1(a, srow, (unsigned int)j) ? al * a.inv_keep : 0.f;
        }
        if (MODE == MODE_SCORES) alpha_row[j] = Elem<T>::from_f(al);
      }
    }
    if (MODE == MODE_SCORES) continue;
    const int nj = min(32, a.Lkv - j0);
    for (int jj = 0; jj < nj; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, al, jj);
      if (pj != 0.f) {  // NaN compares unequal to 0 and propagates
        const T* vp = vbase + (long long)(j0 + jj) * a.v_sl;
#pragma unroll
        for (int r = 0; r < kMaxDvRegs; ++r) {
          const int e = lane + 32 * r;
          if (e < a.dv) acc[r] = fmaf(pj, Elem<T>::to_f(vp[e]), acc[r]);
        }
      }
    }
  }
  if (MODE == MODE_SCORES) return;
  T* xp = reinterpret_cast<T*>(a.x) + (long long)i * a.x_sl + (long long)b * a.x_sb + (long long)h * a.dv;
#pragma unroll
  for (int r = 0; r < kMaxDvRegs; ++r) {
    const int e = lane + 32 * r;
    if (e < a.dv) xp[e] = Elem<T>::from_f(acc[r]);
  }
}

template <typename T>
cudaError_t launch_mode(const AttnArgs& a, int mode, cudaStream_t st) {
  const long long total = (long long)a.Lq * a.H * a.B;
  if (total == 0) return cudaSuccess;
  const long long blocks = (total + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  const size_t smem = (size_t)kWarpsPerBlock * a.d * sizeof(float);
  const dim3 grid((unsigned)blocks), block(kWarpsPerBlock * 32);
  switch (mode) {
    case MODE_FWD:    attn_simt_kernel<T, MODE_FWD><<<grid, block, smem, st>>>(a); break;
    case MODE_STATS:  attn_simt_kernel<T, MODE_STATS><<<grid, block, smem, st>>>(a); break;
    case MODE_SCORES: attn_simt_kernel<T, MODE_SCORES><<<grid, block, smem, st>>>(a); break;
    default:          attn_simt_kernel<T, MODE_APPLY><<<grid, block, smem, st>>>(a); break;
  }
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_any(const AttnArgs& a, int dtype, int mode, cudaStream_t st) {
  switch (dtype) {
    case NNLIB_B200_F16:  return launch_mode<__half>(a, mode, st);
    case NNLIB_B200_BF16: return launch_mode<__nv_bfloat16>(a, mode, st);
    default:              return launch_mode<float>(a, mode, st);
  }
}

}  // namespace

bool simt_supports(int d, int dv) { return d >= 1 && d <= 1024 && dv >= 1 && dv <= 32 * kMaxDvRegs; }

cudaError_t simt_fwd(const AttnArgs& a, int dtype, cudaStream_t st) { return launch_any(a, dtype, MODE_FWD, st); }
cudaError_t simt_stats(const AttnArgs& a, int dtype, cudaStream_t st) { return launch_any(a, dtype, MODE_STATS, st); }
cudaError_t simt_scores(const AttnArgs& a, int dtype, cudaStream_t st) { return launch_any(a, dtype, MODE_SCORES, st); }
cudaError_t simt_apply(const AttnArgs& a, int dtype, cudaStream_t st) { return launch_any(a, dtype, MODE_APPLY, st); }

// ---- make_causal_mask fill / check ----------------------------------------
namespace {
__global__ void causal_fill_kernel(unsigned char* m, long long L) {
  const long long n = L * L;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long i = idx % L, j = idx / L;  // i = kv (contiguous), j = query
    m[idx] = (i <= j) ? 1 : 0;
  }
}
__global__ void causal_check_kernel(const unsigned char* m, long long L, int* flag) {
  const long long n = L * L;
  int bad = 0;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long i = idx % L, j = idx / L;
    bad |= ((m[idx] != 0) != (i <= j));
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicExch(flag, 0);
}
__global__ void set_flag_kernel(int* flag, int v) { *flag = v; }
}  // namespace

cudaError_t causal_fill(unsigned char* m, long long L, cudaStream_t st) {
  if (L == 0) return cudaSuccess;
  const long long n = L * L;
  const int blocks = (int)(((n + 255) / 256 < 148LL * 16) ? (n + 255) / 256 : 148LL * 16);
  causal_fill_kernel<<<blocks, 256, 0, st>>>(m, L);
  count_launch();
  return cudaGetLastError();
}

cudaError_t causal_check(const unsigned char* m, long long L, int* flag, cudaStream_t st) {
  set_flag_kernel<<<1, 1, 0, st>>>(flag, 1);
  count_launch();
  if (L == 0) return cudaGetLastError();
  const long long n = L * L;
  const int blocks = (int)(((n + 255) / 256 < 148LL * 16) ? (n + 255) / 256 : 148LL * 16);
  causal_check_kernel<<<blocks, 256, 0, st>>>(m, L, flag);
  count_launch();
  return cudaGetLastError();
}

}  // namespace nb200
