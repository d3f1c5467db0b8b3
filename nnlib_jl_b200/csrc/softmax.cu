// softmax / logsoftmax over one dimension of a column-major array and their
// pullbacks (NNlib.jl src/softmax.jl:69-79 `_softmax!`, :147-157
// `_logsoftmax!`, :98-101 `_∇softmax!`, :170-190 `∇logsoftmax`), the op in the
// middle of the attention path as a stand-alone entry point.
//
// The array is seen as (inner, n, outer) with the reduction over the middle
// extent: element (i, j, o) lives at i + inner*(j + n*o).  Bound by HBM: one
// read and one write per element (the second pass over a column re-reads it
// from L2).  Arithmetic in fp32 whatever the element type.
//
// Non-finite inputs follow the reference (src/softmax.jl:71-76): a column
// whose maximum is +Inf puts its weight on the +Inf entries in equal shares, a
// column whose maximum is -Inf or that contains a NaN becomes NaN.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "launchers.h"

namespace nb200 {
namespace {

enum : int { SM_FWD = 0, LSM_FWD = 1, SM_BWD = 2, LSM_BWD = 3 };

__device__ __forceinline__ float f_inf() { return __int_as_float(0x7f800000); }
__device__ __forceinline__ float f_ninf() { return __int_as_float(0xff800000); }
__device__ __forceinline__ float f_nan() { return __int_as_float(0x7fc00000); }

// running statistics of a column (forward): maximum, sum of exp(x - max), number of +Inf entries, NaN seen
struct ColStat {
  float m, s;
  int n_inf;
  int nan;
};
__device__ __forceinline__ ColStat stat_init() { return ColStat{f_ninf(), 0.f, 0, 0}; }
__device__ __forceinline__ void stat_add(ColStat& c, float x) {
  if (x != x) { c.nan = 1; return; }
  if (x == f_inf()) { c.n_inf += 1; c.m = f_inf(); return; }
  if (x > c.m) {
    c.s = c.s * ((c.m == f_ninf()) ? 0.f : __expf(c.m - x)) + 1.f;
    c.m = x;
  } else if (x != f_ninf()) {
    c.s += __expf(x - c.m);
  }
}
__device__ __forceinline__ ColStat stat_merge(const ColStat& a, const ColStat& b) {
  ColStat c;
  c.nan = a.nan | b.nan;
  c.n_inf = a.n_inf + b.n_inf;
  c.m = fmaxf(a.m, b.m);
  if (c.m == f_ninf() || c.m == f_inf()) {
    c.s = 0.f;
  } else {
    c.s = ((a.m == f_ninf()) ? 0.f : a.s * __expf(a.m - c.m)) + ((b.m == f_ninf()) ? 0.f : b.s * __expf(b.m - c.m));
  }
  return c;
}
__device__ __forceinline__ ColStat stat_shfl_xor(const ColStat& a, int off) {
  ColStat b;
  b.m = __shfl_xor_sync(0xffffffffu, a.m, off);
  b.s = __shfl_xor_sync(0xffffffffu, a.s, off);
  b.n_inf = __shfl_xor_sync(0xffffffffu, a.n_inf, off);
  b.nan = __shfl_xor_sync(0xffffffffu, a.nan, off);
  return b;
}
// value of one output element given the finished statistics of its column
template <int MODE>
__device__ __forceinline__ float fwd_value(const ColStat& c, float x, float log_s) {
  if (c.nan || c.m == f_ninf()) return f_nan();
  if (c.m == f_inf()) {
    if (MODE == SM_FWD) return (x == f_inf()) ? 1.f / (float)c.n_inf : 0.f;
    return (x == f_inf()) ? -log_s : f_ninf();       // log_s = log(number of +Inf entries)
  }
  if (MODE == SM_FWD) return __expf(x - c.m) / c.s;
  return x - c.m - log_s;
}

// 16-byte packets: V = 16 / sizeof(T) consecutive elements of a column
template <typename T> struct Pack { static constexpr int V = 16 / sizeof(T); };
template <typename T>
__device__ __forceinline__ void load_pack(const T* p, float (&f)[Pack<T>::V]) {
  const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
  const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
  for (int u = 0; u < Pack<T>::V; ++u) f[u] = Elem<T>::to_f(e[u]);
}
template <typename T>
__device__ __forceinline__ void store_pack(T* p, const float (&f)[Pack<T>::V]) {
  uint4 q;
  T* e = reinterpret_cast<T*>(&q);
#pragma unroll
  for (int u = 0; u < Pack<T>::V; ++u) e[u] = Elem<T>::from_f(f[u]);
  *reinterpret_cast<uint4*>(p) = q;
}

// ---- reduction dimension contiguous (inner == 1): G threads per column ----------------------------
// VECT: columns are whole 16-byte packets (n a multiple of the packet, arrays 16-byte aligned)
template <typename T, int MODE, int G, bool VECT>
__global__ void __launch_bounds__(256) softmax_cols_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                           T* __restrict__ out, long long n, long long cols) {
  constexpr int kPerBlock = 256 / G;
  constexpr int V = Pack<T>::V;
  const long long np = n / V;   // packets per column (VECT)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  __shared__ ColStat sh_stat[8];
  __shared__ float sh_sum[8];
  for (long long col = (long long)blockIdx.x * kPerBlock + g; col < cols || G == 256; col += (long long)gridDim.x * kPerBlock) {
    if (G == 256 && col >= cols) break;
    const T* xc = x + col * n;
    T* oc = out + col * n;
    if (MODE == SM_FWD || MODE == LSM_FWD) {
      ColStat c = stat_init();
      if (VECT) {
        for (long long jp = t; jp < np; jp += G) {
          float f[V];
          load_pack<T>(xc + jp * V, f);
#pragma unroll
          for (int u = 0; u < V; ++u) stat_add(c, f[u]);
        }
      } else {
        for (long long j = t; j < n; j += G) stat_add(c, Elem<T>::to_f(xc[j]));
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) c = stat_merge(c, stat_shfl_xor(c, off));
      if (G == 256) {
        if (lane == 0) sh_stat[warp] = c;
        __syncthreads();
        c = sh_stat[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) c = stat_merge(c, sh_stat[w]);
        __syncthreads();
      }
      const float log_s = (MODE == LSM_FWD) ? __logf(c.m == f_inf() ? (float)c.n_inf : c.s) : 0.f;
      if (VECT) {
        for (long long jp = t; jp < np; jp += G) {
          float f[V];
          load_pack<T>(xc + jp * V, f);
#pragma unroll
          for (int u = 0; u < V; ++u) f[u] = fwd_value<MODE>(c, f[u], log_s);
          store_pack<T>(oc + jp * V, f);
        }
      } else {
        for (long long j = t; j < n; j += G) oc[j] = Elem<T>::from_f(fwd_value<MODE>(c, Elem<T>::to_f(xc[j]), log_s));
      }
    } else {
      // pullbacks: x holds y = softmax(x) or logsoftmax(x)
      const T* dc = dy + col * n;
      float acc = 0.f;
      if (VECT) {
        for (long long jp = t; jp < np; jp += G) {
          float d[V], y[V];
          load_pack<T>(dc + jp * V, d);
          if (MODE == SM_BWD) load_pack<T>(xc + jp * V, y);
#pragma unroll
          for (int u = 0; u < V; ++u) acc += (MODE == SM_BWD) ? d[u] * y[u] : d[u];
        }
      } else {
        for (long long j = t; j < n; j += G) {
          const float d = Elem<T>::to_f(dc[j]);
          acc += (MODE == SM_BWD) ? d * Elem<T>::to_f(xc[j]) : d;
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (G == 256) {
        if (lane == 0) sh_sum[warp] = acc;
        __syncthreads();
        acc = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) acc += sh_sum[w];
        __syncthreads();
      }
      if (VECT) {
        for (long long jp = t; jp < np; jp += G) {
          float d[V], y[V];
          load_pack<T>(dc + jp * V, d);
          load_pack<T>(xc + jp * V, y);
#pragma unroll
          for (int u = 0; u < V; ++u) d[u] = (MODE == SM_BWD) ? y[u] * (d[u] - acc) : d[u] - __expf(y[u]) * acc;
          store_pack<T>(oc + jp * V, d);
        }
      } else {
        for (long long j = t; j < n; j += G) {
          const float d = Elem<T>::to_f(dc[j]), y = Elem<T>::to_f(xc[j]);
          oc[j] = Elem<T>::from_f((MODE == SM_BWD) ? y * (d - acc) : d - __expf(y) * acc);
        }
      }
    }
  }
}

// ---- reduction dimension strided (inner > 1): one thread per (i, o), neighbours along i coalesce ----
template <typename T, int MODE>
__global__ void __launch_bounds__(256) softmax_strided_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                              T* __restrict__ out, long long inner, long long n,
                                                              long long outer) {
  const long long total = inner * outer;
  for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < total; p += (long long)gridDim.x * blockDim.x) {
    const long long i = p % inner, o = p / inner;
    const long long base = i + inner * n * o;
    if (MODE == SM_FWD || MODE == LSM_FWD) {
      ColStat c = stat_init();
      for (long long j = 0; j < n; ++j) stat_add(c, Elem<T>::to_f(x[base + j * inner]));
      const float log_s = (MODE == LSM_FWD) ? __logf(c.m == f_inf() ? (float)c.n_inf : c.s) : 0.f;
      for (long long j = 0; j < n; ++j)
        out[base + j * inner] = Elem<T>::from_f(fwd_value<MODE>(c, Elem<T>::to_f(x[base + j * inner]), log_s));
    } else {
      float acc = 0.f;
      for (long long j = 0; j < n; ++j) {
        const float d = Elem<T>::to_f(dy[base + j * inner]);
        acc += (MODE == SM_BWD) ? d * Elem<T>::to_f(x[base + j * inner]) : d;
      }
      for (long long j = 0; j < n; ++j) {
        const float d = Elem<T>::to_f(dy[base + j * inner]), y = Elem<T>::to_f(x[base + j * inner]);
        out[base + j * inner] = Elem<T>::from_f((MODE == SM_BWD) ? y * (d - acc) : d - __expf(y) * acc);
      }
    }
  }
}

template <typename T, int MODE>
cudaError_t launch_softmax(const void* x, const void* dy, void* out, long long inner, long long n, long long outer,
                           cudaStream_t st) {
  const T* xp = static_cast<const T*>(x);
  const T* dp = static_cast<const T*>(dy);
  T* op = static_cast<T*>(out);
  if (inner == 1) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vect = (n % Pack<T>::V) == 0 && al16(x) && al16(out) && (dy == nullptr || al16(dy));
    // a whole block per long column, a warp per short one
    if (n > 2048) {
      const long long blocks = outer < 148ll * 16 ? outer : 148ll * 16;
      if (vect) softmax_cols_kernel<T, MODE, 256, true><<<(unsigned)blocks, 256, 0, st>>>(xp, dp, op, n, outer);
      else      softmax_cols_kernel<T, MODE, 256, false><<<(unsigned)blocks, 256, 0, st>>>(xp, dp, op, n, outer);
    } else {
      const long long need = (outer + 7) / 8;
      const long long blocks = need < 148ll * 16 ? need : 148ll * 16;
      if (vect) softmax_cols_kernel<T, MODE, 32, true><<<(unsigned)blocks, 256, 0, st>>>(xp, dp, op, n, outer);
      else      softmax_cols_kernel<T, MODE, 32, false><<<(unsigned)blocks, 256, 0, st>>>(xp, dp, op, n, outer);
    }
  } else {
    const long long need = (inner * outer + 255) / 256;
    const long long blocks = need < 148ll * 32 ? need : 148ll * 32;
    softmax_strided_kernel<T, MODE><<<(unsigned)blocks, 256, 0, st>>>(xp, dp, op, inner, n, outer);
  }
  count_launch();
  return cudaGetLastError();
}

template <int MODE>
cudaError_t dispatch_softmax(int dtype, const void* x, const void* dy, void* out, long long inner, long long n,
                             long long outer, cudaStream_t st) {
  switch (dtype) {
    case NNLIB_B200_F16:  return launch_softmax<__half, MODE>(x, dy, out, inner, n, outer, st);
    case NNLIB_B200_BF16: return launch_softmax<__nv_bfloat16, MODE>(x, dy, out, inner, n, outer, st);
    default:              return launch_softmax<float, MODE>(x, dy, out, inner, n, outer, st);
  }
}

}  // namespace

cudaError_t softmax_forward(int dtype, bool log, const void* x, void* y, long long inner, long long n, long long outer,
                            cudaStream_t st) {
  return log ? dispatch_softmax<LSM_FWD>(dtype, x, nullptr, y, inner, n, outer, st)
             : dispatch_softmax<SM_FWD>(dtype, x, nullptr, y, inner, n, outer, st);
}

cudaError_t softmax_backward(int dtype, bool log, const void* dy, const void* y, void* dx, long long inner, long long n,
                             long long outer, cudaStream_t st) {
  return log ? dispatch_softmax<LSM_BWD>(dtype, y, dy, dx, inner, n, outer, st)
             : dispatch_softmax<SM_BWD>(dtype, y, dy, dx, inner, n, outer, st);
}

}  // namespace nb200
