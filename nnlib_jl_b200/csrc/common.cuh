// Shared definitions of the attention kernels: the resolved argument block the
// host hands to every kernel, element-type helpers and the Philox4x32-10
// counter-based generator that decides which attention scores dropout keeps.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nnlib_b200.h"

namespace nb200 {

// Kernel-side view of nnlib_b200_attn_params with every default filled in
// (dense strides, scale = 1/sqrt(d), rng_H = H) and dropout pre-digested.
struct AttnArgs {
  const void* q;
  const void* k;
  const void* v;
  void* x;
  long long q_sl, q_sb, k_sl, k_sb, v_sl, v_sb, x_sl, x_sb;
  const void* bias;
  long long bias_s[4];
  const unsigned char* mask;
  long long mask_s[4];
  float* lse;
  long long lse_sb;
  void* alpha;
  long long alpha_sb;
  int* status;
  float* ws;                 // split-key forward: per-split partial results (see attn_tile.cu)
  long long rng_h0, rng_b0, rng_H;
  unsigned int key0, key1, off_lo, off_hi;
  unsigned int rkey[20];   // the ten round keys of Philox4x32-10 (key0 + r*W0, key1 + r*W1), bumped once on the host
  unsigned int drop_thresh;  // floor(p * 2^16): a score is dropped iff its 16-bit lane is below it
  float inv_keep;            // 1/(1-p)
  float dropout_p;
  float scale;               // multiplies q·k (natural units)
  int bias_dtype;
  int causal, nan_fm;
  int coff;                  // causal: key j is kept iff j <= i + coff (0: the square make_causal_mask pattern)
  int allow_tf32;            // Float32 arrays may run their products on the TF32 tensor-core path
  int d, dv, H, Lq, Lkv, B;
};

// Kernel-side view of nnlib_b200_attn_grads (defaults filled in).
struct BwdArgs {
  const void* dx;
  long long dx_sl, dx_sb;
  void* dq;
  void* dk;
  void* dv;
  float* dbias;
  long long dbias_s[4];
  float* delta;
};

// Kernel-side view of nnlib_b200_gemm_params: C = alpha * op(A) * op(B) + beta * C per batch, column-major.
struct GemmArgs {
  const void* A;
  const void* B;
  void* C;
  long long lda, ldb, ldc;               // elements between successive columns of the stored matrices
  long long strideA, strideB, strideC;   // elements between successive batches
  int M, N, K, batch;
  int transA, transB;                    // 1: the stored matrix is the transpose of the factor
  int a_bcast, b_bcast;                  // 1: one matrix for every batch
  float alpha, beta;
  int c_vec;                             // 16-byte stores into C are possible
  int tiles_m, tiles_n;
  long long tiles;
  int* status;
};

// ---- element types --------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};

// bias may have any of the three element types, chosen at run time
__device__ __forceinline__ float load_bias(const void* p, long long idx, int dtype) {
  if (dtype == NNLIB_B200_F16) return __half2float(reinterpret_cast<const __half*>(p)[idx]);
  if (dtype == NNLIB_B200_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
  return reinterpret_cast<const float*>(p)[idx];
}

// ---- Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11) ----
constexpr unsigned int kPhiloxW0 = 0x9E3779B9u, kPhiloxW1 = 0xBB67AE85u;
__host__ __device__ __forceinline__ void philox4x32_10(unsigned int& c0, unsigned int& c1, unsigned int& c2,
                                                       unsigned int& c3, unsigned int k0, unsigned int k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned long long p0 = 0xD2511F53ull * c0;
    const unsigned long long p1 = 0xCD9E8D57ull * c2;
    const unsigned int n0 = (unsigned int)(p1 >> 32) ^ c1 ^ k0;
    const unsigned int n1 = (unsigned int)p1;
    const unsigned int n2 = (unsigned int)(p0 >> 32) ^ c3 ^ k1;
    const unsigned int n3 = (unsigned int)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += kPhiloxW0;
    k1 += kPhiloxW1;
  }
}
// The same ten rounds with the round keys read from a table (kernel arguments: they are operands from the
// constant bank, so a round is two wide multiplies and two three-input XORs, no key arithmetic).
__device__ __forceinline__ void philox4x32_10_keyed(unsigned int& c0, unsigned int& c1, unsigned int& c2,
                                                    unsigned int& c3, const unsigned int (&rk)[20]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned long long p0 = 0xD2511F53ull * c0;
    const unsigned long long p1 = 0xCD9E8D57ull * c2;
    const unsigned int n0 = (unsigned int)(p1 >> 32) ^ c1 ^ rk[2 * r];
    const unsigned int n1 = (unsigned int)p1;
    const unsigned int n2 = (unsigned int)(p0 >> 32) ^ c3 ^ rk[2 * r + 1];
    const unsigned int n3 = (unsigned int)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
  }
}

// The four random words (eight 16-bit lanes) that cover kv positions 8*j8 .. 8*j8+7 of score row r.
__device__ __forceinline__ void dropout_words(const AttnArgs& a, unsigned long long r, unsigned int j8,
                                              unsigned int w[4]) {
  unsigned int c0 = j8, c1 = (unsigned int)r, c2 = (unsigned int)(r >> 32) + a.off_hi, c3 = a.off_lo;
  philox4x32_10_keyed(c0, c1, c2, c3, a.rkey);
  w[0] = c0; w[1] = c1; w[2] = c2; w[3] = c3;
}

// Does score (row r, key j) survive?  Lane j%8: the low (even j) or high (odd j) half of word (j%8)/2.
__device__ __forceinline__ bool dropout_keep1(const AttnArgs& a, unsigned long long r, unsigned int j) {
  unsigned int w[4];
  dropout_words(a, r, j >> 3, w);
  const unsigned int e = j & 7u;
  const unsigned int word = (e < 4u) ? ((e < 2u) ? w[0] : w[1]) : ((e < 6u) ? w[2] : w[3]);
  return ((word >> (16u * (e & 1u))) & 0xffffu) >= a.drop_thresh;
}

// Keep-bits of 32 consecutive keys (bit e: key 32*c32 + e of score row r survives).  Two calls at a time:
// their ten rounds interleave (each round waits on the previous one's multiplies), more would cost registers.
__device__ __forceinline__ unsigned int dropout_keep32(const AttnArgs& a, unsigned long long r, unsigned int c32) {
  unsigned int bits = 0;
#pragma unroll 2
  for (int g = 0; g < 4; ++g) {
    unsigned int w[4];
    dropout_words(a, r, c32 * 4 + g, w);
    unsigned int byte = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      byte |= ((w[e] & 0xffffu) >= a.drop_thresh ? 1u : 0u) << (2 * e);
      byte |= ((w[e] >> 16) >= a.drop_thresh ? 1u : 0u) << (2 * e + 1);
    }
    bits |= byte << (8 * g);
  }
  return bits;
}

// global score-row number of query i, head h, batch b (see nnlib_b200.h, dropout)
__device__ __forceinline__ unsigned long long score_row(const AttnArgs& a, int i, int h, int b) {
  return (unsigned long long)i +
         (unsigned long long)a.Lq * ((unsigned long long)(h + a.rng_h0) +
                                     (unsigned long long)a.rng_H * (unsigned long long)(b + a.rng_b0));
}

// ---- log-sum-exp of a query whose largest logit is +Inf ---------------------------------------------
// The reference's softmax gives such a query equal shares on its +Inf logits (NNlib.jl src/softmax.jl:73-75),
// so what the scores kernel needs later is their number, not a logarithm.  It travels in the lse array as a
// NaN whose quiet bit is clear and whose low 22 bits hold the count (at least 1, saturating); an ordinary
// NaN (a NaN among the logits: the reference's whole column is NaN) has the quiet bit set.
__device__ __forceinline__ float lse_inf_rows(float count) {
  unsigned int n = (count >= 4194303.f) ? 0x3fffffu : (unsigned int)count;
  if (n == 0u) n = 1u;
  return __uint_as_float(0x7f800000u | n);
}
__device__ __forceinline__ bool lse_is_inf_rows(float lse) {
  const unsigned int b = __float_as_uint(lse);
  return (b & 0xffc00000u) == 0x7f800000u && (b & 0x003fffffu) != 0u;
}
__device__ __forceinline__ float lse_inf_count(float lse) { return (float)(__float_as_uint(lse) & 0x003fffffu); }

// launch bookkeeping shared by all translation units
void count_launch(int n = 1);
void set_last_cuda_error(cudaError_t e);

}  // namespace nb200
