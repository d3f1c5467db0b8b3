// Definitions shared by the translation units that hold tcgen05 kernels: tile constants, small
// device helpers and the host-side construction of TMA tensor maps.  Everything sits in an unnamed
// namespace, so each translation unit gets its own copy.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "common.cuh"
#include "umma.cuh"

namespace nb200 {
namespace {

using namespace ptx;

constexpr int kBM = 128;               // queries per tile
constexpr int kBN = 128;               // keys per tile
constexpr int kChunkBytes = 128 * 128; // 128 rows x 64 halves: one TMA box
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr unsigned long long kDrainNs = 20ull * 1000 * 1000;  // 20 ms for in-flight copies on abort

__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }
__device__ __forceinline__ float pos_inf() { return __int_as_float(0x7f800000); }

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// (features, positions, batch) array with 128-byte-swizzled boxes of 64 features x 128 positions
bool make_map(CUtensorMap* m, const void* base, int dtype, long long feat, long long len, long long batch,
              long long stride_l, long long stride_b) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)feat, (cuuint64_t)len, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)stride_l * 2, (cuuint64_t)stride_b * 2};
  const cuuint32_t box[3] = {64, 128, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(m, dtype == NNLIB_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// (features of one head, heads, positions, batch) view of q, k or v with 128-byte-swizzled boxes of 64 features x
// 128 positions of one head; features beyond the head's own are filled with zeros by the copy
bool make_head_map(CUtensorMap* m, const void* base, int dtype, long long dhead, long long H, long long len,
                          long long batch, long long stride_l, long long stride_b) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)dhead, (cuuint64_t)H, (cuuint64_t)len, (cuuint64_t)batch};
  const cuuint64_t strides[3] = {(cuuint64_t)dhead * 2, (cuuint64_t)stride_l * 2, (cuuint64_t)stride_b * 2};
  const cuuint32_t box[4] = {64, 1, 128, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(m, dtype == NNLIB_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// (Lkv, Lq, H, B) score array with 128-byte-swizzled boxes of 64 keys x 128 queries
bool make_alpha_map(CUtensorMap* m, const AttnArgs& a, int dtype) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)a.Lkv, (cuuint64_t)a.Lq, (cuuint64_t)a.H, (cuuint64_t)a.B};
  const cuuint64_t strides[3] = {(cuuint64_t)a.Lkv * 2, (cuuint64_t)a.Lkv * a.Lq * 2, (cuuint64_t)a.alpha_sb * 2};
  const cuuint32_t box[4] = {64, 128, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(m, dtype == NNLIB_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        4, a.alpha, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool stride_ok(long long s) { return s > 0 && (s % 8) == 0 && s * 2 < (1ll << 40); }

}  // namespace
}  // namespace nb200
