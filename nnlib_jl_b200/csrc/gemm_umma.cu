// Strided-batched matrix product on the sm_100a tensor cores:
//
//     C[:, :, b] = alpha * op(A[:, :, b]) * op(B[:, :, b]) + beta * C[:, :, b]
//
// for column-major Float16 / BFloat16 arrays — what NNlib.jl's batched_mul
// reaches through NNlib._batched_gemm! (src/batched/batchedmul.jl:256-303,
// src/gemm.jl:89-188).  The reference's CUDA method hands BlasFloat arrays to
// cuBLAS (ext/NNlibCUDAExt/batchedmul.jl:3-4); 16-bit element types miss that
// route and fall to the per-slice generic loop (src/batched/batchedmul.jl:306-325).
//
// The tensor core computes D[r, c] = sum_k P[r, k] Q[c, k] with the rows r of P
// in the 128 lanes of tensor memory and c along its columns.  C is column-major
// (m contiguous), so the roles are swapped: P = op(B)^T (rows = n), Q = op(A)
// (rows = m); a thread of the epilogue then owns one column n of C and writes
// runs of consecutive m with 16-byte stores.
//
// One CTA owns an (NH*128 n) x (MT m) tile of C and walks over K in blocks of
// 64; the grid is persistent (one CTA per SM, tiles dealt round-robin).
//   warp 0      TMA producer: a ring of stages, each holding the n-side rows
//               and the m-side rows of one K block (128-byte swizzle)
//   warp 1      allocates tensor memory, issues every tcgen05.mma
//   warps 2-9   epilogue: TMEM -> registers -> alpha / beta -> C
// Whether an operand is K-major or MN-major in shared memory follows from the
// transpose flags: op(A) = A ('N') has m contiguous (MN-major), A^T ('T') has k
// contiguous (K-major); B ('N') has k contiguous (K-major), B^T has n contiguous.
// With NH*MT <= 256 two accumulators alternate, so the epilogue of one tile
// overlaps the products of the next.
#include <cuda.h>

#include "common.cuh"
#include "launchers.h"
#include "umma.cuh"
#include "umma_shared.cuh"

namespace nb200 {

__device__ int g_gemm_abort = 0;  // sticky: a bounded wait of a product kernel ran out

namespace {

constexpr int kGemmThreads = 320;
constexpr int kBK = 64;                  // K elements per stage: one 128-byte swizzle row
constexpr int kHalfBytes = 128 * 128;    // 128 rows x 64 K elements, either layout

template <int NH, int MT>
struct GCfg {
  static constexpr int kNBytes = NH * kHalfBytes;
  static constexpr int kMBytes = (MT / 128) * kHalfBytes;
  static constexpr int kStage = kNBytes + kMBytes;
  static constexpr int kStages = (200 * 1024) / kStage;          // 3 (64 KB), 4 (48 KB), 6 (32 KB)
  static constexpr int kAccCols = NH * MT;                       // fp32 columns of one tile
  static constexpr int kAccBufs = (kAccCols <= 256) ? 2 : 1;
  static constexpr int kTmemCols = (kAccCols * kAccBufs <= 256) ? 256 : 512;
  static constexpr int kBarOff = kStages * kStage;
  static constexpr int kSmemBytes = kBarOff + 256 + 1024;
};
static_assert(GCfg<2, 256>::kStages == 3 && GCfg<1, 256>::kStages == 4 && GCfg<1, 128>::kStages == 6, "ring depth");
static_assert(GCfg<2, 256>::kSmemBytes <= 232448, "shared memory budget");

struct GBarriers {
  uint64_t full[8], empty[8];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(GBarriers) <= 256, "barrier block");

template <bool BF16, int NH, int MT, bool N_KMAJ, bool M_KMAJ>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap tm_n, const __grid_constant__ CUtensorMap tm_m, const GemmArgs g) {
  using C = GCfg<NH, MT>;
  using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  GBarriers* bars = reinterpret_cast<GBarriers*>(smem + C::kBarOff);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (g.K + kBK - 1) / kBK;
  const long long per_batch = (long long)g.tiles_m * g.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 8; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->acc_full[s], 1);
      mbar_init(&bars->acc_empty[s], 8);
    }
    bars->abort_flag = *reinterpret_cast<volatile int*>(&g_gemm_abort);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  const bool start_ok = (*abort_flag == 0);

  if (start_ok && warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&tm_n);
      prefetch_tensormap(&tm_m);
      bool ok = true;
      long long it = 0;
      for (long long t = blockIdx.x; t < g.tiles && ok; t += gridDim.x) {
        const int b = (int)(t / per_batch);
        const int r = (int)(t % per_batch);
        const int n0 = (r / g.tiles_m) * (NH * 128), m0 = (r % g.tiles_m) * MT;
        const int bn = g.b_bcast ? 0 : b, bm = g.a_bcast ? 0 : b;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = (int)(it % C::kStages);
          if (it >= C::kStages) ok = mbar_wait(&bars->empty[s], (uint32_t)((it / C::kStages) - 1) & 1u, abort_flag);
          if (!ok) break;
          uint8_t* dn = smem + s * C::kStage;
          uint8_t* dm = dn + C::kNBytes;
          mbar_arrive_expect_tx(&bars->full[s], C::kStage);
          if (N_KMAJ) {
#pragma unroll
            for (int i = 0; i < NH; ++i) tma_load_3d(dn + i * kHalfBytes, &tm_n, &bars->full[s], kb * kBK, n0 + i * 128, bn);
          } else {
#pragma unroll
            for (int i = 0; i < 2 * NH; ++i)
              tma_load_3d(dn + i * (kHalfBytes / 2), &tm_n, &bars->full[s], n0 + i * 64, kb * kBK, bn);
          }
          if (M_KMAJ) {
#pragma unroll
            for (int i = 0; i < MT / 128; ++i)
              tma_load_3d(dm + i * kHalfBytes, &tm_m, &bars->full[s], kb * kBK, m0 + i * 128, bm);
          } else {
#pragma unroll
            for (int i = 0; i < MT / 64; ++i)
              tma_load_3d(dm + i * (kHalfBytes / 2), &tm_m, &bars->full[s], m0 + i * 64, kb * kBK, bm);
          }
        }
      }
      if (*abort_flag) {
        // give copies still in flight a bounded chance to land before the CTA leaves
        for (long long jj = (it > C::kStages ? it - C::kStages : 0); jj < it; ++jj)
          mbar_wait_drain(&bars->full[jj % C::kStages], (uint32_t)(jj / C::kStages) & 1u, kDrainNs);
      }
    }
  } else if (start_ok && warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(BF16, 128, MT, !N_KMAJ, !M_KMAJ);
      bool ok = true;
      long long it = 0;
      int ti = 0;
      for (long long t = blockIdx.x; t < g.tiles && ok; t += gridDim.x, ++ti) {
        const int ab = ti % C::kAccBufs;
        if (ti >= C::kAccBufs) {
          ok = mbar_wait(&bars->acc_empty[ab], (uint32_t)((ti / C::kAccBufs) - 1) & 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t acc = tmem + ab * C::kAccCols;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = (int)(it % C::kStages);
          ok = mbar_wait(&bars->full[s], (uint32_t)(it / C::kStages) & 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t na = smem_u32(smem + s * C::kStage);
          const uint32_t ma = na + C::kNBytes;
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            // K-major rows: 16 K elements further along the 128-byte row; MN-major: 16 K rows of 128 bytes further
            const uint64_t mdesc = M_KMAJ ? make_smem_desc_sw128(ma + kk * 32, 16, 1024)
                                          : make_smem_desc_sw128(ma + kk * 2048, kHalfBytes / 2, 1024);
#pragma unroll
            for (int i = 0; i < NH; ++i) {
              const uint32_t nb = na + i * kHalfBytes;
              const uint64_t ndesc = N_KMAJ ? make_smem_desc_sw128(nb + kk * 32, 16, 1024)
                                            : make_smem_desc_sw128(nb + kk * 2048, kHalfBytes / 2, 1024);
              umma_ss(acc + i * MT, ndesc, mdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
          }
          umma_commit(&bars->empty[s]);
        }
        if (ok) umma_commit(&bars->acc_full[ab]);
      }
    }
  } else if (start_ok && warp >= 2) {
    // ----------------------------------------------------------------- epilogue
    const int wq = warp & 3;                 // TMEM lane quarter this warp may touch
    const int part = (warp - 2) >> 2;        // NH = 2: which 128 rows of n; NH = 1: which half of the m columns
    const int half = (NH == 2) ? part : 0;
    constexpr int kCols = (NH == 2) ? MT : MT / 2;
    const int col0 = (NH == 2) ? 0 : part * kCols;
    const float alpha = g.alpha, beta = g.beta;
    bool ok = true;
    int ti = 0;
    for (long long t = blockIdx.x; t < g.tiles && ok; t += gridDim.x, ++ti) {
      const int ab = ti % C::kAccBufs;
      const int b = (int)(t / per_batch);
      const int r = (int)(t % per_batch);
      const int n0 = (r / g.tiles_m) * (NH * 128), m0 = (r % g.tiles_m) * MT;
      ok = mbar_wait_warp(&bars->acc_full[ab], (uint32_t)(ti / C::kAccBufs) & 1u, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int n = n0 + half * 128 + wq * 32 + lane;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(wq * 32) << 16) + ab * C::kAccCols + half * MT + col0;
      T* ccol = reinterpret_cast<T*>(g.C) + (long long)b * g.strideC + (long long)n * g.ldc;
#pragma unroll 1
      for (int c = 0; c < kCols / 32; ++c) {
        uint32_t acc[32];
        tmem_ld32(taddr + c * 32, acc);
        tmem_wait_ld();
        if (c == kCols / 32 - 1) {
          // this warp has read its share of the accumulator: the issuer may start the tile after next
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->acc_empty[ab]);
        }
        const int m = m0 + col0 + c * 32;
        if (n < g.N && m < g.M) {
          T* dst = ccol + m;
          if (g.c_vec && m + 32 <= g.M) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              float f[8];
#pragma unroll
              for (int u = 0; u < 8; ++u) f[u] = alpha * __uint_as_float(acc[e + u]);
              if (beta != 0.f) {
                const uint4 old = *reinterpret_cast<const uint4*>(dst + e);
                const T* o = reinterpret_cast<const T*>(&old);
#pragma unroll
                for (int u = 0; u < 8; ++u) f[u] = fmaf(beta, Elem<T>::to_f(o[u]), f[u]);
              }
              uint4 v;
              v.x = pack2<BF16>(f[0], f[1]);
              v.y = pack2<BF16>(f[2], f[3]);
              v.z = pack2<BF16>(f[4], f[5]);
              v.w = pack2<BF16>(f[6], f[7]);
              *reinterpret_cast<uint4*>(dst + e) = v;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              if (m + e < g.M) {
                float f = alpha * __uint_as_float(acc[e]);
                if (beta != 0.f) f = fmaf(beta, Elem<T>::to_f(dst[e]), f);
                dst[e] = Elem<T>::from_f(f);
              }
            }
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) {
    atomicExch(&g_gemm_abort, 1);
    if (g.status) atomicExch(g.status, NNLIB_B200_TIMEOUT);
  }
}

// ---- any shape, stride and element type on the CUDA cores: one thread per element of C ---------------
template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const GemmArgs g) {
  const int m = blockIdx.x * 32 + (threadIdx.x & 31);
  const int n = blockIdx.y * 8 + (threadIdx.x >> 5);
  const int b = blockIdx.z;
  if (m >= g.M || n >= g.N) return;
  const T* A = reinterpret_cast<const T*>(g.A) + (g.a_bcast ? 0 : (long long)b * g.strideA);
  const T* B = reinterpret_cast<const T*>(g.B) + (g.b_bcast ? 0 : (long long)b * g.strideB);
  const long long a_m = g.transA ? g.lda : 1, a_k = g.transA ? 1 : g.lda;
  const long long b_k = g.transB ? g.ldb : 1, b_n = g.transB ? 1 : g.ldb;
  float acc = 0.f;
  for (int k = 0; k < g.K; ++k)
    acc = fmaf(Elem<T>::to_f(A[m * a_m + k * a_k]), Elem<T>::to_f(B[k * b_k + n * b_n]), acc);
  T* c = reinterpret_cast<T*>(g.C) + (long long)b * g.strideC + (long long)n * g.ldc + m;
  float out = g.alpha * acc;
  if (g.beta != 0.f) out = fmaf(g.beta, Elem<T>::to_f(*c), out);
  *c = Elem<T>::from_f(out);
}

// (contiguous extent, rows, batch) view of one operand with the box its layout needs:
// K-major: contiguous = K, box 64 x 128; MN-major: contiguous = M or N, box 64 x 64
bool make_operand_map(CUtensorMap* m, const void* base, int dtype, long long contiguous, long long rows, long long batch,
                      long long ld, long long stride, bool kmajor) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)contiguous, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch > 1 ? stride : ld * rows) * 2};
  const cuuint32_t box[3] = {64, kmajor ? 128u : 64u, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(m, dtype == NNLIB_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      n < 1)
    n = 148;
  return n;
}

template <bool BF16, int NH, int MT, bool N_KMAJ, bool M_KMAJ>
cudaError_t launch_gemm(const CUtensorMap& mn, const CUtensorMap& mm, GemmArgs g, cudaStream_t st) {
  using C = GCfg<NH, MT>;
  auto kern = gemm_umma_kernel<BF16, NH, MT, N_KMAJ, M_KMAJ>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  g.tiles_m = (g.M + MT - 1) / MT;
  g.tiles_n = (g.N + NH * 128 - 1) / (NH * 128);
  g.tiles = (long long)g.tiles_m * g.tiles_n * g.batch;
  const long long grid = g.tiles < sm_count() ? g.tiles : sm_count();
  kern<<<(unsigned)grid, kGemmThreads, C::kSmemBytes, st>>>(mn, mm, g);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

const char* gemm_umma_reject_reason(const GemmArgs& g, int dtype) {
  if (dtype != NNLIB_B200_F16 && dtype != NNLIB_B200_BF16) return "element type is not Float16 / BFloat16";
  if (g.M < 1 || g.N < 1 || g.K < 1 || g.batch < 1) return "empty product";
  if (!aligned16(g.A) || !aligned16(g.B)) return "A or B is not 16-byte aligned";
  if (!stride_ok(g.lda) || !stride_ok(g.ldb)) return "a leading dimension of A or B is not a positive multiple of 8 elements";
  if (!g.a_bcast && g.batch > 1 && !stride_ok(g.strideA)) return "the batch stride of A is not a positive multiple of 8 elements";
  if (!g.b_bcast && g.batch > 1 && !stride_ok(g.strideB)) return "the batch stride of B is not a positive multiple of 8 elements";
  if ((long long)((g.M + 127) / 128) * ((g.N + 127) / 128) * g.batch > 0x7fffffffLL) return "too many tiles";
  if (encode_tiled_fn() == nullptr) return "the driver does not export cuTensorMapEncodeTiled";
  return nullptr;
}

cudaError_t gemm_umma(const GemmArgs& g0, int dtype, cudaStream_t st) {
  GemmArgs g = g0;
  const bool n_kmaj = !g.transB;    // B stored (K, N): k contiguous
  const bool m_kmaj = g.transA;     // A stored (K, M): k contiguous
  CUtensorMap mn, mm;
  const long long bn = g.b_bcast ? 1 : g.batch, bm = g.a_bcast ? 1 : g.batch;
  if (!(n_kmaj ? make_operand_map(&mn, g.B, dtype, g.K, g.N, bn, g.ldb, g.strideB, true)
               : make_operand_map(&mn, g.B, dtype, g.N, g.K, bn, g.ldb, g.strideB, false)))
    return cudaErrorInvalidValue;
  if (!(m_kmaj ? make_operand_map(&mm, g.A, dtype, g.K, g.M, bm, g.lda, g.strideA, true)
               : make_operand_map(&mm, g.A, dtype, g.M, g.K, bm, g.lda, g.strideA, false)))
    return cudaErrorInvalidValue;
  g.c_vec = (aligned16(g.C) && g.ldc % 8 == 0 && (g.batch == 1 || g.strideC % 8 == 0)) ? 1 : 0;
  const bool bf16 = dtype == NNLIB_B200_BF16;
  // tile: 256 x 256 for large products, 128 n-rows for narrow ones, 128 m-columns for short ones
  // (a short K leaves the 256 x 256 tile, whose accumulator fills all of tensor memory, with nothing to overlap
  // its epilogue with: 128 rows of n then, two accumulators in turn)
  const int nh = (g.N > 128 && g.M > 128 && g.K > 512) ? 2 : 1;
  const int mt = (g.M > 128) ? 256 : 128;
#define NB_G4(BF, NHH, MTT)                                                               \
  do {                                                                                    \
    if (n_kmaj) {                                                                         \
      if (m_kmaj) return launch_gemm<BF, NHH, MTT, true, true>(mn, mm, g, st);            \
      return launch_gemm<BF, NHH, MTT, true, false>(mn, mm, g, st);                       \
    }                                                                                     \
    if (m_kmaj) return launch_gemm<BF, NHH, MTT, false, true>(mn, mm, g, st);             \
    return launch_gemm<BF, NHH, MTT, false, false>(mn, mm, g, st);                        \
  } while (0)
#define NB_G3(BF)                                            \
  do {                                                       \
    if (nh == 2) NB_G4(BF, 2, 256);                          \
    if (mt == 256) NB_G4(BF, 1, 256);                        \
    NB_G4(BF, 1, 128);                                       \
  } while (0)
  if (bf16) NB_G3(true);
  NB_G3(false);
#undef NB_G3
#undef NB_G4
  return cudaErrorInvalidValue;
}

cudaError_t gemm_simt(const GemmArgs& g, int dtype, cudaStream_t st) {
  if (g.M < 1 || g.N < 1 || g.batch < 1) return cudaSuccess;
  const long long gx = (g.M + 31) / 32, gy = (g.N + 7) / 8;
  if (gx > 0x7fffffffLL || gy > 65535 || g.batch > 65535) return cudaErrorInvalidConfiguration;
  const dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)g.batch);
  switch (dtype) {
    case NNLIB_B200_F16:  gemm_simt_kernel<__half><<<grid, 256, 0, st>>>(g); break;
    case NNLIB_B200_BF16: gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(g); break;
    default:              gemm_simt_kernel<float><<<grid, 256, 0, st>>>(g); break;
  }
  count_launch();
  return cudaGetLastError();
}

// Reads and clears the sticky "a bounded wait ran out" flag of the product kernels on the current device.
cudaError_t gemm_take_abort(int* out, cudaStream_t st) {
  int v = 0;
  cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyFromSymbol(&v, g_gemm_abort, sizeof(int));
  if (e != cudaSuccess) return e;
  if (v) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_gemm_abort, &zero, sizeof(int));
  }
  *out = v;
  return e;
}

}  // namespace nb200
