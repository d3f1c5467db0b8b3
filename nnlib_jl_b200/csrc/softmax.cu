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
__device__ __forceinline__ void unpack(const uint4& q, float (&f)[Pack<T>::V]) {
  const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
  for (int u = 0; u < Pack<T>::V; ++u) f[u] = Elem<T>::to_f(e[u]);
}
template <typename T>
__device__ __forceinline__ uint4 repack(const float (&f)[Pack<T>::V]) {
  uint4 q;
  T* e = reinterpret_cast<T*>(&q);
#pragma unroll
  for (int u = 0; u < Pack<T>::V; ++u) e[u] = Elem<T>::from_f(f[u]);
  return q;
}
// 16-bit types: two values per conversion instruction
template <>
__device__ __forceinline__ uint4 repack<__nv_bfloat16>(const float (&f)[8]) {
  uint4 q;
  __nv_bfloat162* e = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int u = 0; u < 4; ++u) e[u] = __floats2bfloat162_rn(f[2 * u], f[2 * u + 1]);
  return q;
}
template <>
__device__ __forceinline__ uint4 repack<__half>(const float (&f)[8]) {
  uint4 q;
  __half2* e = reinterpret_cast<__half2*>(&q);
#pragma unroll
  for (int u = 0; u < 4; ++u) e[u] = __floats2half2_rn(f[2 * u], f[2 * u + 1]);
  return q;
}
// Every kernel exists twice.  NA (no alias: the host saw that the output overlaps neither input) takes
// `__restrict__` pointers and loads through the non-coherent path, which lets the compiler start the next
// column's loads before this column's stores.  The other variant serves the in-place forms (softmax!(x, x) of the
// reference, a pullback written over dy): plain coherent loads, no promise about aliasing — a column longer than a
// thread's register share is read a second time after other threads may have written theirs.
template <typename T, bool NA> struct Ptrs { using In = const T*; using Out = T*; };
template <typename T> struct Ptrs<T, true> { using In = const T* __restrict__; using Out = T* __restrict__; };
template <typename T, bool NA>
__device__ __forceinline__ uint4 load_raw(const T* p) {
  if constexpr (NA) return __ldg(reinterpret_cast<const uint4*>(p));
  else return *reinterpret_cast<const uint4*>(p);
}
template <typename T, bool NA>
__device__ __forceinline__ T load_elem(const T* p) {
  if constexpr (NA) return __ldg(p);
  else return *p;
}
template <typename T, bool NA>
__device__ __forceinline__ void load_pack(const T* p, float (&f)[Pack<T>::V]) { unpack<T>(load_raw<T, NA>(p), f); }
template <typename T>
__device__ __forceinline__ void store_pack(T* p, const float (&f)[Pack<T>::V]) {
  *reinterpret_cast<uint4*>(p) = repack<T>(f);
}

// branch-free update of the running statistics with one packet of V values: one rescaling exponential
// per packet instead of a data-dependent branch per value
template <int V>
__device__ __forceinline__ void stat_add_pack(ColStat& c, const float (&f)[V]) {
  float pm = f_ninf();
  float xv[V];
#pragma unroll
  for (int u = 0; u < V; ++u) {
    const float x = f[u];
    c.nan |= (x != x) ? 1 : 0;
    const bool is_inf = (x == f_inf());
    c.n_inf += is_inf ? 1 : 0;
    xv[u] = (is_inf || x != x) ? f_ninf() : x;      // +Inf and NaN are accounted for by the flags
    pm = fmaxf(pm, xv[u]);
  }
  const float m_new = fmaxf(c.m, pm);
  const float m_safe = (m_new == f_ninf()) ? 0.f : m_new;
  float s = c.s * __expf(c.m - m_safe);              // c.m = -Inf: exp(-Inf) = 0
#pragma unroll
  for (int u = 0; u < V; ++u) s += __expf(xv[u] - m_safe);
  c.s = s;
  c.m = m_new;
}
// first sweep over a register-cached column: a NaN-propagating maximum is all the common case needs
// (one instruction per value); +Inf entries are counted only when the maximum turns out to be +Inf
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
// (the maximum above ignores +Inf entries; a column that has some is marked here)
__device__ __forceinline__ void stat_finish(ColStat& c) {
  if (c.n_inf > 0) c.m = f_inf();
}
// output values of a packet given the finished statistics
template <int MODE, int V>
__device__ __forceinline__ void fwd_pack(const ColStat& c, float inv_s, float log_s, float (&f)[V]) {
  const bool special = c.nan || c.m == f_ninf() || c.m == f_inf();
#pragma unroll
  for (int u = 0; u < V; ++u) {
    if (special) f[u] = fwd_value<MODE>(c, f[u], log_s);
    else f[u] = (MODE == SM_FWD) ? __expf(f[u] - c.m) * inv_s : f[u] - c.m - log_s;
  }
}

// ---- reduction dimension contiguous (inner == 1): G threads per column ----------------------------
// VECT: columns are whole 16-byte packets (n a multiple of the packet, arrays 16-byte aligned).
// KP > 0 (with VECT): a thread's packets (at most KP, as raw 16-byte words) stay in registers between
// the two passes, so the column is read from memory once.
template <typename T, int MODE, int G, bool VECT, int KP, bool NA>
__global__ void __launch_bounds__((G > 256 ? G : 256)) softmax_cols_kernel(typename Ptrs<T, NA>::In x, typename Ptrs<T, NA>::In dy,
                                                                            typename Ptrs<T, NA>::Out out, long long n, long long cols) {
  constexpr int kBlock = G > 256 ? G : 256;
  constexpr int kPerBlock = kBlock / G;
  constexpr int kWarps = kBlock / 32;
  constexpr int V = Pack<T>::V;
  constexpr bool FWD = (MODE == SM_FWD || MODE == LSM_FWD);
  const long long np = n / V;   // packets per column (VECT)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  __shared__ ColStat sh_stat[32];
  __shared__ float sh_sum[32];
  for (long long col = (long long)blockIdx.x * kPerBlock + g; col < cols || G >= 256; col += (long long)gridDim.x * kPerBlock) {
    if (G >= 256 && col >= cols) break;
    const T* xc = x + col * n;
    const T* dc = FWD ? xc : dy + col * n;
    T* oc = out + col * n;
    constexpr bool CACHE = KP > 0;
    uint4 cx[CACHE ? KP : 1];                 // forward: x; pullbacks: y
    uint4 cd[(CACHE && !FWD) ? KP : 1];       // pullbacks: dy
    ColStat c = stat_init();
    float acc = 0.f;
    // ---- pass 1: column statistics (forward) or the column sum (pullbacks)
    if (VECT && CACHE) {
#pragma unroll
      for (int k = 0; k < (CACHE ? KP : 1); ++k) {
        const long long jp = t + (long long)k * G;
        if (jp < np) {
          cx[k] = load_raw<T, NA>(xc + jp * V);
          if (!FWD) cd[k] = load_raw<T, NA>(dc + jp * V);
        }
      }
#pragma unroll
      for (int k = 0; k < (CACHE ? KP : 1); ++k) {
        const long long jp = t + (long long)k * G;
        if (jp < np) {
          float f[V];
          unpack<T>(cx[k], f);
          if (FWD) {
#pragma unroll
            for (int u = 0; u < V; ++u) c.m = max_nan(c.m, f[u]);   // the exponentials follow once the maximum is known
          } else {
            float d[V];
            unpack<T>(cd[k], d);
#pragma unroll
            for (int u = 0; u < V; ++u) acc += (MODE == SM_BWD) ? d[u] * f[u] : d[u];
          }
        }
      }
    } else if (VECT) {
      for (long long jp = t; jp < np; jp += G) {
        float f[V], d[V];
        load_pack<T, NA>(xc + jp * V, f);
        if (FWD) {
          stat_add_pack<V>(c, f);
        } else {
          load_pack<T, NA>(dc + jp * V, d);
#pragma unroll
          for (int u = 0; u < V; ++u) acc += (MODE == SM_BWD) ? d[u] * f[u] : d[u];
        }
      }
    } else {
      for (long long j = t; j < n; j += G) {
        if (FWD) {
          stat_add(c, Elem<T>::to_f(xc[j]));
        } else {
          const float d = Elem<T>::to_f(dc[j]);
          acc += (MODE == SM_BWD) ? d * Elem<T>::to_f(xc[j]) : d;
        }
      }
    }
    // ---- reduce over the G threads of the column
    auto group_sum = [&](float v) -> float {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (G >= 256) {
        if (lane == 0) sh_sum[warp] = v;
        __syncthreads();
        v = 0.f;
        for (int w = 0; w < kWarps; ++w) v += sh_sum[w];
        __syncthreads();
      }
      return v;
    };
    if (FWD && VECT && CACHE) {
      // register-cached column: only the (NaN-propagating) maximum exists so far
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) c.m = max_nan(c.m, __shfl_xor_sync(0xffffffffu, c.m, off));
      if (G >= 256) {
        if (lane == 0) sh_sum[warp] = c.m;
        __syncthreads();
        c.m = sh_sum[0];
        for (int w = 1; w < kWarps; ++w) c.m = max_nan(c.m, sh_sum[w]);
        __syncthreads();
      }
      if (c.m != c.m) {            // a NaN somewhere in the column
        c.nan = 1;
        c.m = 0.f;
      } else if (c.m == f_inf()) { // rare: count the +Inf entries (src/softmax.jl:71-76 shares the weight among them)
        float cnt = 0.f;
#pragma unroll
        for (int k = 0; k < (CACHE ? KP : 1); ++k) {
          const long long jp = t + (long long)k * G;
          if (jp < np) {
            float f[V];
            unpack<T>(cx[k], f);
#pragma unroll
            for (int u = 0; u < V; ++u) cnt += (f[u] == f_inf()) ? 1.f : 0.f;
          }
        }
        c.n_inf = (int)group_sum(cnt);
      }
    } else if (FWD) {
      stat_finish(c);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) c = stat_merge(c, stat_shfl_xor(c, off));
      if (G >= 256) {
        if (lane == 0) sh_stat[warp] = c;
        __syncthreads();
        c = sh_stat[0];
        for (int w = 1; w < kWarps; ++w) c = stat_merge(c, sh_stat[w]);
        __syncthreads();
      }
    }
    if (FWD) {
      if (VECT && CACHE) {
        // second sweep over the registers: one exponential per element, summed in fp32; softmax keeps the
        // exponentials (in the element type) in place of x for the write sweep
        const bool special = c.nan || c.m == f_ninf() || c.m == f_inf();
        float part = 0.f;
        if (!special) {
#pragma unroll
          for (int k = 0; k < (CACHE ? KP : 1); ++k) {
            const long long jp = t + (long long)k * G;
            if (jp < np) {
              float f[V];
              unpack<T>(cx[k], f);
#pragma unroll
              for (int u = 0; u < V; ++u) {
                f[u] = __expf(f[u] - c.m);
                part += f[u];
              }
              if (MODE == SM_FWD) cx[k] = repack<T>(f);
            }
          }
        }
        c.s = group_sum(part);
      }
    } else {
      acc = group_sum(acc);
    }
    const float sum_or_cnt = (c.m == f_inf()) ? (float)c.n_inf : c.s;
    const float log_s = (MODE == LSM_FWD) ? __logf(sum_or_cnt) : 0.f;
    const float inv_s = (MODE == SM_FWD) ? 1.f / c.s : 0.f;
    // ---- pass 2: write
    if (VECT && CACHE) {
#pragma unroll
      for (int k = 0; k < (CACHE ? KP : 1); ++k) {
        const long long jp = t + (long long)k * G;
        if (jp < np) {
          float f[V];
          unpack<T>(cx[k], f);
          if (FWD) {
            const bool special = c.nan || c.m == f_ninf() || c.m == f_inf();
            if (MODE == SM_FWD && !special) {
#pragma unroll
              for (int u = 0; u < V; ++u) f[u] *= inv_s;      // f holds exp(x - max) from the second sweep
            } else {
              fwd_pack<MODE, V>(c, inv_s, log_s, f);
            }
            store_pack<T>(oc + jp * V, f);
          } else {
            float d[V];
            unpack<T>(cd[k], d);
#pragma unroll
            for (int u = 0; u < V; ++u) d[u] = (MODE == SM_BWD) ? f[u] * (d[u] - acc) : d[u] - __expf(f[u]) * acc;
            store_pack<T>(oc + jp * V, d);
          }
        }
      }
    } else if (VECT) {
      for (long long jp = t; jp < np; jp += G) {
        float f[V], d[V];
        load_pack<T, NA>(xc + jp * V, f);
        if (FWD) {
          fwd_pack<MODE, V>(c, inv_s, log_s, f);
          store_pack<T>(oc + jp * V, f);
        } else {
          load_pack<T, NA>(dc + jp * V, d);
#pragma unroll
          for (int u = 0; u < V; ++u) d[u] = (MODE == SM_BWD) ? f[u] * (d[u] - acc) : d[u] - __expf(f[u]) * acc;
          store_pack<T>(oc + jp * V, d);
        }
      }
    } else {
      for (long long j = t; j < n; j += G) {
        if (FWD) {
          oc[j] = Elem<T>::from_f(fwd_value<MODE>(c, Elem<T>::to_f(xc[j]), log_s));
        } else {
          const float d = Elem<T>::to_f(dc[j]), y = Elem<T>::to_f(xc[j]);
          oc[j] = Elem<T>::from_f((MODE == SM_BWD) ? y * (d - acc) : d - __expf(y) * acc);
        }
      }
    }
  }
}

// ---- reduction dimension strided (inner > 1): one thread per (i, o), neighbours along i coalesce ----
template <typename T, int MODE, bool NA>
__global__ void __launch_bounds__(256) softmax_strided_kernel(typename Ptrs<T, NA>::In x, typename Ptrs<T, NA>::In dy,
                                                              typename Ptrs<T, NA>::Out out, long long inner, long long n,
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
  // does the output overlap an input?  (the in-place forms of the reference: the same array, same extent)
  const uintptr_t bytes = (uintptr_t)(inner * n * outer) * sizeof(T);
  auto overlaps = [bytes](const void* a, const void* b) {
    const uintptr_t pa = reinterpret_cast<uintptr_t>(a), pb = reinterpret_cast<uintptr_t>(b);
    return a != nullptr && b != nullptr && pa < pb + bytes && pb < pa + bytes;
  };
  const bool no_alias = !overlaps(x, out) && !overlaps(dy, out);
  if (inner == 1) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vect = (n % Pack<T>::V) == 0 && al16(x) && al16(out) && (dy == nullptr || al16(dy));
    const long long np = n / Pack<T>::V;
    const long long cap = 148ll * 16;
    // a warp per short column, a 256- or 1024-thread block per long one; the column stays in registers
    // between the passes whenever a thread's share is small enough (1024-thread blocks have 64 registers
    // per thread: 8 raw packets for Float32 forward, 4 otherwise, 4 + 4 in the pullbacks)
    constexpr bool FWD = (MODE == SM_FWD || MODE == LSM_FWD);
    constexpr int kBig = (FWD && sizeof(T) == 4) ? 8 : 4;
#define NB_SM_LAUNCH(GG, VV, KK)                                                                       \
  do {                                                                                                 \
    constexpr int kBlock = (GG) > 256 ? (GG) : 256;                                                    \
    const long long need = (outer + (kBlock / (GG)) - 1) / (kBlock / (GG));                            \
    const long long blocks = need < cap ? need : cap;                                                  \
    if (no_alias)                                                                                      \
      softmax_cols_kernel<T, MODE, GG, VV, KK, true><<<(unsigned)blocks, kBlock, 0, st>>>(xp, dp, op, n, outer);  \
    else                                                                                               \
      softmax_cols_kernel<T, MODE, GG, VV, KK, false><<<(unsigned)blocks, kBlock, 0, st>>>(xp, dp, op, n, outer); \
  } while (0)
    if (!vect) {
      if (n > 2048) NB_SM_LAUNCH(256, false, 0); else NB_SM_LAUNCH(32, false, 0);
    } else if (np <= 32ll * 2) {
      // short columns (attention-sized rows of scores): two packets per lane, few registers, so that enough
      // warps are resident to keep the memory system busy with so little in flight per warp
      NB_SM_LAUNCH(32, true, 2);
    } else if (np <= 32ll * 4) {
      NB_SM_LAUNCH(32, true, 4);
    } else if (np <= 32ll * 8) {
      NB_SM_LAUNCH(32, true, 8);
    } else if (sizeof(T) == 2 && FWD && np <= 32ll * 16) {
      // 16-bit columns of up to 4096 elements still fit a warp's registers (16 packets per lane): no block-wide
      // barrier between the passes, sixteen independent loads in flight per lane
      NB_SM_LAUNCH(32, true, 16);
    } else if (np <= 256ll * 8) {
      NB_SM_LAUNCH(256, true, 8);
    } else if (np <= 1024ll * kBig) {
      NB_SM_LAUNCH(1024, true, kBig);
    } else {
      NB_SM_LAUNCH(1024, true, 0);
    }
#undef NB_SM_LAUNCH
  } else {
    const long long need = (inner * outer + 255) / 256;
    const long long blocks = need < 148ll * 32 ? need : 148ll * 32;
    if (no_alias)
      softmax_strided_kernel<T, MODE, true><<<(unsigned)blocks, 256, 0, st>>>(xp, dp, op, inner, n, outer);
    else
      softmax_strided_kernel<T, MODE, false><<<(unsigned)blocks, 256, 0, st>>>(xp, dp, op, inner, n, outer);
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
