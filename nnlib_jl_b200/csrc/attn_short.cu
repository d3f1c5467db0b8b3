// x AND alpha in one pass for short key sequences (encoder-style self-attention: every query's whole score
// row fits in tensor memory).
//
// dot_product_attention returns the scores eagerly (NNlib.jl src/attention.jl:83,112-127).  The general route
// here (fused forward, then the score-rebuild kernel) computes Q K^T twice and reads q and k twice; when
// Lkv <= 512 (d = 64) or <= 256 (d = 128) one CTA can hold the 128 x Lkv score block of its 128 queries in the
// 512 TMEM columns, so the exact two-pass softmax of the reference (src/softmax.jl:69-79) needs no online
// rescaling and no log-sum-exp round trip, and every exponential is taken once:
//   warp 4     allocates tensor memory; TMA: Q, all K tiles, all V tiles (no ring: everything is resident)
//   warp 5     tcgen05.mma: S_t = Q K_t^T for every key tile, later O = sum_t P_t V_t
//   warps 0-3  thread r owns query row r:
//                pass 1  logits -> scale, bias (src/attention.jl:129-131), masks (:133-138) -> row maximum;
//                        the prepared logits go back to their TMEM columns
//                pass 2  p = exp2(s - m), row sum, dropout (src/dropout.jl:77-87); the 16-bit probabilities
//                        are packed into the low half of the score columns (chunk g of 32 scores moves from
//                        columns [32g, 32g+32) to [16g, 16g+16): always behind the reader)
//                pass 3  alpha' = P / l / (1-p) into 128-byte swizzled staging boxes (64 keys x 128 queries)
//                epilogue x = O / l / (1-p)
//   warp 6     ships every filled staging box with one cp.async.bulk.tensor store into the (Lkv, Lq, H, B) array
// O lives in the columns the packing freed.  Bound by the HBM write of alpha.
#include <cuda.h>

#include "common.cuh"
#include "extras.cuh"
#include "launchers.h"
#include "umma.cuh"
#include "umma_shared.cuh"

namespace nb200 {

__device__ int g_short_abort = 0;  // sticky: a bounded wait of this kernel ran out

namespace {

constexpr int kShThreads = 224;
constexpr int kShStageBytes = 128 * 128;   // staging box of the TMA store: 128 queries x 64 scores

template <int D>
struct ShCfg {
  static constexpr int kMaxTiles = (D == 64) ? 4 : 2;          // key tiles of 128 the CTA can hold
  static constexpr int kChunks = D / 64;
  static constexpr int kTileBytes = kChunks * kChunkBytes;     // 128 rows x D features
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kTileBytes;
  static constexpr int kVOff = kKOff + kMaxTiles * kTileBytes;
  static constexpr int kStOff = kVOff + kMaxTiles * kTileBytes;
  static constexpr int kBarOff = kStOff + 2 * kShStageBytes;
  static constexpr int kSmemBytes = kBarOff + 256 + 1024;
  static constexpr int kTmemCols = kMaxTiles * 128;            // 512 / 256
  static constexpr int kOCol = kMaxTiles * 64;                 // first column behind the packed probabilities
};
static_assert(ShCfg<64>::kSmemBytes <= 232448 && ShCfg<128>::kSmemBytes <= 232448, "shared memory budget");
static_assert(ShCfg<64>::kOCol + 64 <= ShCfg<64>::kTmemCols && ShCfg<128>::kOCol + 128 <= ShCfg<128>::kTmemCols, "O fits");

struct ShBarriers {
  uint64_t qk_full, v_full, s_full, p_ready, o_full;
  uint64_t stage_full[2], stage_free[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int D, bool BF16>
__global__ void __launch_bounds__(kShThreads, 1)
attn_short_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_a, const AttnArgs a,
                  const int n_qtiles) {
  using C = ShCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  ShBarriers* bars = reinterpret_cast<ShBarriers*>(smem + C::kBarOff);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int unit = blockIdx.x / n_qtiles;
  const int qt = n_qtiles - 1 - (blockIdx.x % n_qtiles);
  const int h = unit % a.H, b = unit / a.H;
  const int q0 = qt * kBM;
  const int n_total = (a.Lkv + kBN - 1) / kBN;                 // <= kMaxTiles (the host checked)
  const int n_live = a.causal ? min(n_total, (min(a.Lkv, max(q0 + kBM + a.coff, 1)) + kBN - 1) / kBN) : n_total;

  if (threadIdx.x == 0) {
    mbar_init(&bars->qk_full, 1);
    mbar_init(&bars->v_full, 1);
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->p_ready, 4);
    mbar_init(&bars->o_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->stage_full[s], 4);
      mbar_init(&bars->stage_free[s], 1);
    }
    bars->abort_flag = *reinterpret_cast<volatile int*>(&g_short_abort);
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(&bars->tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  const bool start_ok = (*abort_flag == 0);

  if (start_ok && warp == 4) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      mbar_arrive_expect_tx(&bars->qk_full, (1 + n_live) * C::kTileBytes);
      for (int c = 0; c < C::kChunks; ++c)
        tma_load_3d(smem + C::kQOff + c * kChunkBytes, &tm_q, &bars->qk_full, h * D + c * 64, q0, b);
      for (int t = 0; t < n_live; ++t)
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_3d(smem + C::kKOff + t * C::kTileBytes + c * kChunkBytes, &tm_k, &bars->qk_full, h * D + c * 64,
                      t * kBN, b);
      mbar_arrive_expect_tx(&bars->v_full, n_live * C::kTileBytes);
      for (int t = 0; t < n_live; ++t)
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_3d(smem + C::kVOff + t * C::kTileBytes + c * kChunkBytes, &tm_v, &bars->v_full, h * D + c * 64,
                      t * kBN, b);
      // the copies land whatever happens to the rest of the CTA: wait for them on the way out of an abort
      if (!mbar_wait(&bars->qk_full, 0, abort_flag)) mbar_wait_drain(&bars->qk_full, 0, kDrainNs);
      if (!mbar_wait(&bars->v_full, 0, abort_flag)) mbar_wait_drain(&bars->v_full, 0, kDrainNs);
    }
  } else if (start_ok && warp == 5) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(BF16, kBM, kBN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(BF16, kBM, D, false, true);
      const uint32_t qa = smem_u32(smem + C::kQOff);
      bool ok = mbar_wait(&bars->qk_full, 0, abort_flag);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < n_live; ++t) {
          const uint32_t ka = smem_u32(smem + C::kKOff + t * C::kTileBytes);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
            umma_ss(tmem + t * kBN, make_smem_desc_sw128(qa + off, 16, 1024), make_smem_desc_sw128(ka + off, 16, 1024),
                    idesc_qk, kk > 0 ? 1u : 0u);
          }
        }
        umma_commit(&bars->s_full);
        // every row's probabilities are packed (and every score column has been read): O may be written
        ok = mbar_wait(&bars->p_ready, 0, abort_flag);
        if (ok) ok = mbar_wait(&bars->v_full, 0, abort_flag);
        if (ok) {
          tc_fence_after();
          for (int t = 0; t < n_live; ++t) {
            const uint32_t va = smem_u32(smem + C::kVOff + t * C::kTileBytes);
#pragma unroll
            for (int kk = 0; kk < kBN / 16; ++kk)
              umma_ts(tmem + C::kOCol, tmem + t * 64 + kk * 8, make_smem_desc_sw128(va + kk * 2048, kChunkBytes, 1024),
                      idesc_pv, (t > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&bars->o_full);
        }
      }
    }
  } else if (start_ok && warp == 6) {
    // ---- store thread: each filled staging box (128 queries x 64 scores) goes out as one TMA store
    if (lane == 0) {
      prefetch_tensormap(&tm_a);
      bool ok = true;
      const int n_half = 2 * n_total;
      for (int n = 0; n < n_half && ok; ++n) {
        ok = mbar_wait(&bars->stage_full[n & 1], (n >> 1) & 1, abort_flag);
        if (!ok) break;
        tma_store_4d(&tm_a, smem + C::kStOff + (n & 1) * kShStageBytes, n * 64, q0, h, b);
        tma_store_commit();
        if (n >= 1) {
          tma_store_wait_read<1>();                 // the previous box has been read out of shared memory
          mbar_arrive(&bars->stage_free[(n - 1) & 1]);
        }
      }
      tma_store_wait_read<0>();                     // shared memory must stay valid until the last read
    }
  } else if (start_ok && warp < 4) {
    // ----------------------------------------------------------- softmax warps
    const int r = warp * 32 + lane;
    const int i = q0 + r;
    const bool row_ok = i < a.Lq;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    const float c2 = a.scale * kLog2e;
    const int lim = a.causal ? min(i + a.coff, a.Lkv - 1) : a.Lkv - 1;   // last key this row attends to (< 0: none)
    const unsigned long long srow = score_row(a, row_ok ? i : 0, h, b);
    const bool drop = a.dropout_p > 0.f;
    RowSide rs = make_row_side(a, i, h, b, row_ok);
    const int n_chunks = n_live * 4;     // chunks of 32 keys

    bool ok = mbar_wait_warp(&bars->s_full, 0, abort_flag);
    float m = neg_inf();
    float l = 0.f;
    if (ok) {
      tc_fence_after();
      // ---- pass 1: prepared logits (scaled base 2, bias added, masked keys -inf) and the row maximum
      // (two chunks per turn, so that the bias / mask words of the next chunk are in flight while one is worked on)
      uint4 bq0[4], bq1[4], mq0[2], mq1[2];
      auto prepare = [&](int g, const uint4 (&bq)[4], const uint4 (&mq)[2]) {
        uint32_t s[32];
        tmem_ld32(lane_base + g * 32, s);
        tmem_wait_ld();
        side_apply<true>(rs, s, bq, mq, g * 32, a.Lkv, lim, row_ok, c2);
#pragma unroll
        for (int e = 0; e < 32; e += 2) m = max3(m, __uint_as_float(s[e]), __uint_as_float(s[e + 1]));
        __syncwarp();                     // the bias / mask code above branches per row
        tmem_st32(lane_base + g * 32, s);
      };
      side_issue<true>(rs, 0, a.Lkv, bq0, mq0);
#pragma unroll 1
      for (int g = 0; g < n_chunks; g += 2) {
        side_issue<true>(rs, (g + 1) * 32, a.Lkv, bq1, mq1);
        prepare(g, bq0, mq0);
        if (g + 2 < n_chunks) side_issue<true>(rs, (g + 2) * 32, a.Lkv, bq0, mq0);
        prepare(g + 1, bq1, mq1);
      }
      tmem_wait_st();
      // ---- pass 2: exponentials, row sum, dropout, packed probabilities
      const bool row_inf = (m == pos_inf());          // a +Inf bias: equal shares on the +Inf keys (src/softmax.jl:73-75)
      const float m_sub = (m == neg_inf()) ? 0.f : m;
#pragma unroll 1
      for (int g = 0; g < n_chunks; ++g) {
        unsigned int kb = 0xffffffffu;
        if (drop) kb = dropout_keep32(a, srow, (unsigned int)g);
        uint32_t s[32];
        tmem_ld32(lane_base + g * 32, s);
        tmem_wait_ld();
        uint32_t pk[16];
        float sum = 0.f;
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0 = ex2_approx(__uint_as_float(s[e]) - m_sub);
          float p1 = ex2_approx(__uint_as_float(s[e + 1]) - m_sub);
          if (row_inf) {
            p0 = (s[e] == 0x7f800000u) ? 1.f : 0.f;
            p1 = (s[e + 1] == 0x7f800000u) ? 1.f : 0.f;
          }
          sum += p0 + p1;                 // dropout follows the softmax: the row sum keeps the dropped scores
          if (!((kb >> e) & 1u)) p0 = 0.f;
          if (!((kb >> (e + 1)) & 1u)) p1 = 0.f;
          pk[e >> 1] = pack2<BF16>(p0, p1);
        }
        l += sum;
        tmem_st16(lane_base + g * 16, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready);
    }

    // ---- pass 3: alpha' = P / l / (1-p), box by box
    bool okst = ok;
    if (ok) {
      const bool dead = !(l > 0.f);
      const float nanv = __int_as_float(0x7fc00000);
      const float scale = dead ? 0.f : a.inv_keep / l;
      const float dead_val = (a.nan_fm || l != l) ? nanv : 0.f;
      if (a.lse && row_ok) {
        float lse_v = (l != l) ? nanv : dead ? neg_inf() : (m + log2f(l)) * kLn2;
        if (m == pos_inf() && !dead) lse_v = lse_inf_rows(l);
        a.lse[i + (long long)a.Lq * h + a.lse_sb * b] = lse_v;
      }
      const int n_half = 2 * n_total;
#pragma unroll 1
      for (int n = 0; n < n_half; ++n) {
        uint32_t pk[32];
        if (n < 2 * n_live) {
          tmem_ld32(lane_base + n * 32, pk);          // 64 packed probabilities of this row
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float lo, hi;
            if (BF16) {
              lo = __uint_as_float(pk[e] << 16);
              hi = __uint_as_float(pk[e] & 0xffff0000u);
            } else {
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pk[e]));
              lo = f.x; hi = f.y;
            }
            lo *= scale; hi *= scale;
            if (dead) { lo = dead_val; hi = dead_val; }
            pk[e] = pack2<BF16>(lo, hi);
          }
        } else {
          // key tiles entirely above the causal diagonal
          const uint32_t z = dead ? pack2<BF16>(dead_val, dead_val) : 0u;
#pragma unroll
          for (int e = 0; e < 32; ++e) pk[e] = z;
        }
        if (n >= 2) {
          okst = mbar_wait_warp(&bars->stage_free[n & 1], ((n >> 1) - 1) & 1, abort_flag);
          if (!okst) break;
        }
        uint8_t* row = smem + C::kStOff + (n & 1) * kShStageBytes + r * 128;
#pragma unroll
        for (int v = 0; v < 8; ++v)
          *reinterpret_cast<uint4*>(row + ((v ^ (r & 7)) << 4)) =
              make_uint4(pk[v * 4], pk[v * 4 + 1], pk[v * 4 + 2], pk[v * 4 + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->stage_full[n & 1]);
      }

      // ---- epilogue: x = O / l / (1-p)
      if (okst) {
        ok = mbar_wait_warp(&bars->o_full, 0, abort_flag);
        if (ok) {
          tc_fence_after();
          uint8_t* xrow = reinterpret_cast<uint8_t*>(a.x) +
                          2ll * ((long long)i * a.x_sl + (long long)b * a.x_sb + (long long)h * D);
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(lane_base + C::kOCol + c * 32, o);
            tmem_wait_ld();
            if (row_ok) {
#pragma unroll
              for (int e = 0; e < 32; e += 8) {
                float f[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) f[u] = dead ? dead_val : __uint_as_float(o[e + u]) * scale;
                uint4 v;
                v.x = pack2<BF16>(f[0], f[1]);
                v.y = pack2<BF16>(f[2], f[3]);
                v.z = pack2<BF16>(f[4], f[5]);
                v.w = pack2<BF16>(f[6], f[7]);
                *reinterpret_cast<uint4*>(xrow + (c * 32 + e) * 2) = v;
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
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) {
    atomicExch(&g_short_abort, 1);
    if (a.status) atomicExch(a.status, NNLIB_B200_TIMEOUT);
  }
}

template <int D, bool BF16>
cudaError_t launch_short(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& ma,
                         const AttnArgs& a, cudaStream_t st) {
  auto kern = attn_short_kernel<D, BF16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ShCfg<D>::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int n_qtiles = (a.Lq + kBM - 1) / kBM;
  const long long blocks = (long long)n_qtiles * a.H * a.B;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  kern<<<(unsigned)blocks, kShThreads, ShCfg<D>::kSmemBytes, st>>>(mq, mk, mv, ma, a, n_qtiles);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

// x and alpha together for a short key sequence: the fused forward's shapes (16-bit, d = dv in {64, 128},
// 16-byte aligned rows), every key of a query within one CTA's tensor memory, and score rows the TMA store
// can address.
bool short_supports(const AttnArgs& a, int dtype) {
  if (!umma_supports(a, dtype, true)) return false;
  const int max_keys = (a.d == 64) ? 512 : 256;
  if (a.Lkv > max_keys) return false;
  if (!a.alpha || a.Lkv % 8 != 0 || !aligned16(a.alpha) || a.alpha_sb % 8 != 0) return false;
  return true;
}

cudaError_t short_attention(const AttnArgs& a, int dtype, cudaStream_t st) {
  CUtensorMap mq, mk, mv, ma;
  const long long E = (long long)a.H * a.d;
  if (!make_map(&mq, a.q, dtype, E, a.Lq, a.B, a.q_sl, a.q_sb)) return cudaErrorInvalidValue;
  if (!make_map(&mk, a.k, dtype, E, a.Lkv, a.B, a.k_sl, a.k_sb)) return cudaErrorInvalidValue;
  if (!make_map(&mv, a.v, dtype, E, a.Lkv, a.B, a.v_sl, a.v_sb)) return cudaErrorInvalidValue;
  if (!make_alpha_map(&ma, a, dtype)) return cudaErrorInvalidValue;
  const bool bf16 = dtype == NNLIB_B200_BF16;
  if (a.d == 128) return bf16 ? launch_short<128, true>(mq, mk, mv, ma, a, st) : launch_short<128, false>(mq, mk, mv, ma, a, st);
  return bf16 ? launch_short<64, true>(mq, mk, mv, ma, a, st) : launch_short<64, false>(mq, mk, mv, ma, a, st);
}

// Reads and clears the sticky "a bounded wait ran out" flag of this kernel on the current device.
cudaError_t short_take_abort(int* out, cudaStream_t st) {
  int v = 0;
  cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyFromSymbol(&v, g_short_abort, sizeof(int));
  if (e != cudaSuccess) return e;
  if (v) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_short_abort, &zero, sizeof(int));
  }
  *out = v;
  return e;
}

}  // namespace nb200
