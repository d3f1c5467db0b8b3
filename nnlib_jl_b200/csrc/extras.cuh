// Bias and Bool-mask access for one query row of the tensor-core kernels.
//
// A softmax / epilogue thread owns one query row and walks over its keys in
// chunks of 32.  bias (NNlib.jl src/attention.jl:129-131) and mask (:133-138)
// may have any strides; when the key stride is 1 and the row starts on a
// 16-byte boundary, a chunk is fetched with 16-byte loads that are issued one
// chunk ahead of their use, otherwise element by element.
#pragma once

#include "common.cuh"

namespace nb200 {

struct RowSide {
  const unsigned char* bias_row;  // address of bias(kv = 0) of this row (nullptr: no bias or row out of range)
  const unsigned char* mask_row;  // address of mask(kv = 0) of this row
  long long bias_s0, mask_s0;     // key strides in elements
  int bias_dtype;
  bool bias_vec;                  // 2-byte elements, key stride 1, 16-byte aligned row
  bool mask_vec;                  // key stride 1, 16-byte aligned row
};

__device__ __forceinline__ RowSide make_row_side(const AttnArgs& a, int i, int h, int b, bool row_ok) {
  RowSide rs;
  rs.bias_row = nullptr;
  rs.mask_row = nullptr;
  rs.bias_s0 = a.bias_s[0];
  rs.mask_s0 = a.mask_s[0];
  rs.bias_dtype = a.bias_dtype;
  rs.bias_vec = false;
  rs.mask_vec = false;
  if (row_ok && a.bias) {
    const long long off = (long long)i * a.bias_s[1] + (long long)h * a.bias_s[2] + (long long)b * a.bias_s[3];
    const int esz = (a.bias_dtype == NNLIB_B200_F32) ? 4 : 2;
    rs.bias_row = reinterpret_cast<const unsigned char*>(a.bias) + off * esz;
    rs.bias_vec = (esz == 2) && (a.bias_s[0] == 1) && ((reinterpret_cast<unsigned long long>(rs.bias_row) & 15ull) == 0);
  }
  if (row_ok && a.mask) {
    const long long off = (long long)i * a.mask_s[1] + (long long)h * a.mask_s[2] + (long long)b * a.mask_s[3];
    rs.mask_row = a.mask + off;
    rs.mask_vec = (a.mask_s[0] == 1) && ((reinterpret_cast<unsigned long long>(rs.mask_row) & 15ull) == 0);
  }
  return rs;
}

// Start the 16-byte loads of keys jj0 .. jj0+31 (only when the whole chunk lies inside the array).
template <bool WITH_BIAS>
__device__ __forceinline__ void side_issue(const RowSide& rs, int jj0, int Lkv, uint4 (&bq)[4], uint4 (&mq)[2]) {
  const bool inside = jj0 + 32 <= Lkv;
  if (WITH_BIAS && rs.bias_vec && inside) {
    const uint4* p = reinterpret_cast<const uint4*>(rs.bias_row + (long long)jj0 * 2);
#pragma unroll
    for (int v = 0; v < 4; ++v) bq[v] = __ldg(p + v);
  }
  if (rs.mask_vec && inside) {
    const uint4* p = reinterpret_cast<const uint4*>(rs.mask_row + jj0);
#pragma unroll
    for (int v = 0; v < 2; ++v) mq[v] = __ldg(p + v);
  }
}

// bit 7 of every byte of the result is set iff that byte of w is non-zero
__device__ __forceinline__ unsigned int nonzero_bytes(unsigned int w) {
  return (w | ((w & 0x7f7f7f7fu) + 0x7f7f7f7fu)) & 0x80808080u;
}

__device__ __forceinline__ unsigned int u4_word(const uint4& q, int w) {
  return w == 0 ? q.x : (w == 1 ? q.y : (w == 2 ? q.z : q.w));
}

// the four "non-zero" flags of a word of mask bytes as bits 0..3
__device__ __forceinline__ unsigned int nonzero_nibble(unsigned int w) {
  return (((nonzero_bytes(w) >> 7) * 0x00204081u) >> 21) & 0xfu;
}

// bit e: mask byte e of the 32 bytes (lo, hi) is non-zero
__device__ __forceinline__ unsigned int mask_word_bits(const uint4& lo, const uint4& hi) {
  return nonzero_nibble(lo.x) | (nonzero_nibble(lo.y) << 4) | (nonzero_nibble(lo.z) << 8) |
         (nonzero_nibble(lo.w) << 12) | (nonzero_nibble(hi.x) << 16) | (nonzero_nibble(hi.y) << 20) |
         (nonzero_nibble(hi.z) << 24) | (nonzero_nibble(hi.w) << 28);
}

// bit e: key jj0+e lies inside the row's range (keys 0 .. lim; none when the row itself is out of range)
__device__ __forceinline__ unsigned int range_keep_bits(int jj0, int lim, bool row_ok) {
  const int lim_e = row_ok ? lim - jj0 : -1;
  return lim_e >= 31 ? 0xffffffffu : (lim_e < 0 ? 0u : (0xffffffffu >> (31 - lim_e)));
}

// Keep bits of keys jj0 .. jj0+31 of a row whose mask cannot be fetched with 16-byte loads: one byte at a time.
__device__ __forceinline__ unsigned int mask_keep_bits_bytes(const RowSide& rs, int jj0, unsigned int range) {
  if (range == 0u || !rs.mask_row) return range;
  unsigned int m = 0u;
  for (int e = 0; e < 32; ++e)
    if (((range >> e) & 1u) && rs.mask_row[(jj0 + e) * rs.mask_s0] != 0) m |= 1u << e;
  return m;
}

// s[e] (raw q·k of keys jj0+e) -> scaled base-2 logit with bias added, or -inf where the key is
// masked, beyond `lim` (causal / end of the keys) or the row is out of range.  Works in place.
// BIAS_STAGED: bq was filled from a shared-memory copy of the bias tile (zero beyond the array), so the
// vector form applies to every chunk.
template <bool WITH_BIAS, bool BIAS_STAGED = false>
__device__ __forceinline__ void side_apply(const RowSide& rs, unsigned int (&s)[32], const uint4 (&bq)[4],
                                           const uint4 (&mq)[2], int jj0, int Lkv, int lim, bool row_ok, float c2) {
  constexpr float kLog2eF = 1.4426950408889634f;
  const bool inside = jj0 + 32 <= Lkv;
  const int lim_e = row_ok ? lim - jj0 : -1;   // element e of the chunk is in range iff e <= lim_e
  // ---- scale (+ bias)
  if (WITH_BIAS && rs.bias_row && (BIAS_STAGED || (rs.bias_vec && inside))) {
    if (rs.bias_dtype == NNLIB_B200_BF16) {
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        const unsigned int w = u4_word(bq[e >> 3], (e >> 1) & 3);
        s[e] = __float_as_uint(fmaf(__uint_as_float(s[e]), c2, __uint_as_float(w << 16) * kLog2eF));
        s[e + 1] = __float_as_uint(fmaf(__uint_as_float(s[e + 1]), c2, __uint_as_float(w & 0xffff0000u) * kLog2eF));
      }
    } else {
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        const unsigned int w = u4_word(bq[e >> 3], (e >> 1) & 3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
        s[e] = __float_as_uint(fmaf(__uint_as_float(s[e]), c2, f.x * kLog2eF));
        s[e + 1] = __float_as_uint(fmaf(__uint_as_float(s[e + 1]), c2, f.y * kLog2eF));
      }
    }
  } else if (WITH_BIAS && rs.bias_row) {   // any stride / element type: one load per key
    // (the same expression as the vector form above, so that a row gives the same bits whichever form its
    // alignment selects: a shard of an array and the array itself must agree exactly)
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      float bv = 0.f;
      if (e <= lim_e) bv = load_bias(rs.bias_row, (jj0 + e) * rs.bias_s0, rs.bias_dtype) * kLog2eF;
      s[e] = __float_as_uint(fmaf(__uint_as_float(s[e]), c2, bv));
      asm volatile("" ::: "memory");   // one load at a time: this path must not cost registers
    }
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e) s[e] = __float_as_uint(__uint_as_float(s[e]) * c2);
  }
  // ---- range and mask
  if (rs.mask_row && rs.mask_vec && inside) {
    // most chunks of a padding-style mask are all true: one test instead of 32 byte extractions
    const unsigned int nz = nonzero_bytes(mq[0].x) & nonzero_bytes(mq[0].y) & nonzero_bytes(mq[0].z) &
                            nonzero_bytes(mq[0].w) & nonzero_bytes(mq[1].x) & nonzero_bytes(mq[1].y) &
                            nonzero_bytes(mq[1].z) & nonzero_bytes(mq[1].w);
    if (nz != 0x80808080u || lim_e < 31) {
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const unsigned int byte = (u4_word(mq[e >> 4], (e >> 2) & 3) >> ((e & 3) * 8)) & 0xffu;
        if (e > lim_e || byte == 0u) s[e] = 0xff800000u;
      }
    }
  } else if (rs.mask_row) {
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      bool keep = e <= lim_e;
      if (keep) keep = rs.mask_row[(jj0 + e) * rs.mask_s0] != 0;
      if (!keep) s[e] = 0xff800000u;
      asm volatile("" ::: "memory");     // one load at a time: this path must not cost registers
    }
  } else if (lim_e < 31) {
#pragma unroll
    for (int e = 0; e < 32; ++e)
      if (e > lim_e) s[e] = 0xff800000u;
  }
}

}  // namespace nb200
