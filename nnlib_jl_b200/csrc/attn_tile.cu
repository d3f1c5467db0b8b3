// Tensor-core attention for the shapes the two-tile fused kernel (attn_umma.cu) does not take:
// head sizes other than 64 / 128 (any multiple of 8 up to 128), value heads of another size than the
// query / key heads (NNlib.jl allows Ev != E: docstring example src/attention.jl:36, bias test
// test/attention.jl:61-68), and Float32 arrays on the TF32 tensor-core path (behind
// nnlib_b200_attn_params.allow_tf32; Float32 otherwise stays on the exact CUDA-core kernels).
//
// One CTA owns 128 queries of one (head, batch) unit and walks over the keys in tiles of 64:
//   warps 0-3   softmax / epilogue: thread r owns query row r (a TMEM lane), no cross-lane reductions
//   warp 4      allocates tensor memory, TMA producer of Q (once) and of the K and V rings
//   warp 5      issues every tcgen05.mma:  S = Q K_j^T  (smem x smem)  and  O += P_j V_j  (TMEM x smem)
// TMEM columns: S_0 [0,64)  S_1 [64,128)  O [128, 128+DV).  The scores alternate between two buffers, so
// Q K_{j+2}^T follows P_j V_j into the buffer P_j leaves; the probabilities overwrite their scores in place
// (16-bit types packed two per column, Float32 as they are: the tensor core reads them as TF32).  V is the
// MN-major operand of P V; for 32-bit elements that layout exists only as the 128-byte swizzle with a
// 32-byte unit, so the Float32 V tiles are copied with that swizzle.
// Operand tiles are 128-byte swizzled; a head's features are addressed through a 4-d tensor map
// (d, H, L, B), so a head narrower than the 64- or 32-element box is padded with zeros by the copy engine
// and a padded product costs nothing but idle multiplier lanes.
// MODE selects what the CTA produces, like the modes of the CUDA-core kernel:
//   TM_FWD     x and the per-query log-sum-exp (online softmax of src/softmax.jl:69-79 in base 2, bias
//              src/attention.jl:129-131, masks :133-138, dropout src/dropout.jl:77-87 on P after the row sum)
//   TM_STATS   the log-sum-exp only
//   TM_SCORES  alpha (after dropout) from a given log-sum-exp, written straight to the (Lkv, Lq, H, B) array
//   TM_SPLIT   few queries (Lq <= 128: one query tile) against many keys: the key tiles of a unit are dealt to
//              `n_splits` CTAs, each leaving its running maximum, its sum and its unnormalised O in a
//              workspace; attn_split_reduce_kernel merges them into x and the log-sum-exp.  This is what
//              keeps every SM busy when H*B is small (one new token against a long key / value history).
#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "extras.cuh"
#include "launchers.h"
#include "umma.cuh"
#include "umma_shared.cuh"

namespace nb200 {

__device__ int g_tile_abort = 0;  // sticky: a bounded wait of these kernels ran out

namespace {

enum : int { TM_FWD = 0, TM_STATS = 1, TM_SCORES = 2, TM_SPLIT = 3 };
constexpr int kTThreads = 192;
constexpr int kTBM = 128;          // queries per CTA
constexpr int kTBN = 64;           // keys per tile
constexpr int kTMaxStages = 4;
constexpr float kTRescaleGap = 8.0f;

template <typename T, int DQ, int DV>
struct TCfg {
  static constexpr int kEsz = sizeof(T);
  static constexpr int kEpc = 128 / kEsz;                    // elements in a 128-byte swizzle row
  static constexpr int kQChunks = DQ / kEpc;
  static constexpr int kVChunks = DV / kEpc;
  static constexpr int kQChunkBytes = kTBM * 128;            // 128 queries x 128 bytes
  static constexpr int kKChunkBytes = kTBN * 128;            // 64 keys x 128 bytes
  static constexpr int kQBytes = kQChunks * kQChunkBytes;
  static constexpr int kKBytes = kQChunks * kKChunkBytes;
  static constexpr int kVBytes = kVChunks * kKChunkBytes;
  // ring depth: a 64-key tile is little work, so the copies of several tiles must be in flight to cover the
  // latency of a load that misses L2 (two stages left the tensor core waiting: 6.6 k cycles per tile measured)
  static constexpr int kStagesFit = (200 * 1024 - kQBytes) / (kKBytes + kVBytes);
  static constexpr int kStages = kStagesFit >= kTMaxStages ? kTMaxStages : (kStagesFit < 2 ? 2 : kStagesFit);
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQBytes;
  static constexpr int kVOff = kKOff + kStages * kKBytes;
  static constexpr int kBarOff = kVOff + kStages * kVBytes;
  static constexpr int kSmemBytes = kBarOff + 256 + 1024;
  static constexpr int kKStep = 32 / kEsz;                   // K elements of one tcgen05.mma (32 bytes)
  // tensor memory: two 64-column score buffers and DV columns of O, rounded up to a power of two
  static constexpr int kTmemCols = (2 * kTBN + DV <= 256) ? 256 : 512;
  static constexpr int kCtasPerSm = (kSmemBytes <= 110 * 1024 && kTmemCols <= 256) ? 2 : 1;
};
static_assert(TCfg<float, 128, 128>::kSmemBytes <= 232448, "shared memory budget");
static_assert(TCfg<__half, 256, 256>::kSmemBytes <= 232448 && TCfg<__half, 256, 256>::kStages >= 2, "shared memory budget (d = 256)");

struct TBarriers {
  uint64_t q_full;
  uint64_t k_full[kTMaxStages], k_empty[kTMaxStages], v_full[kTMaxStages], v_empty[kTMaxStages];
  uint64_t s_full[2], p_ready[2], o_ready, o_final;
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(TBarriers) <= 256, "barrier block");

// Workspace of the split-key forward, in floats: (maximum, sum) per (unit, split, query), rounded up so that
// the O rows behind them start on a 16-byte boundary, then dv floats of unnormalised O per (unit, split, query).
__host__ __device__ inline long long split_ml_floats(const AttnArgs& a, int n_splits) {
  return (((long long)a.H * a.B * n_splits * a.Lq * 2) + 3) & ~3LL;
}
__host__ __device__ inline long long split_ws_floats(const AttnArgs& a, int n_splits) {
  return split_ml_floats(a, n_splits) + (long long)a.H * a.B * n_splits * a.Lq * a.dv;
}

// Second stage of the split-key forward: one block per (unit, query) merges the partial results of the
// splits, x = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s, and writes the query's log-sum-exp.
template <typename T>
__global__ void __launch_bounds__(128) attn_split_reduce_kernel(const AttnArgs a, const int n_splits) {
  const long long row = blockIdx.x;              // unit * Lq + i
  const int i = (int)(row % a.Lq);
  const int unit = (int)(row / a.Lq);
  const int h = unit % a.H, b = unit / a.H;
  const float* ml = a.ws + ((long long)unit * n_splits * a.Lq + i) * 2;
  const float* o = a.ws + split_ml_floats(a, n_splits) + ((long long)unit * n_splits * a.Lq + i) * a.dv;
  const long long sstride = a.Lq;                // splits of one unit are Lq slots apart
  float M = __int_as_float(0xff800000);
  bool any_nan = false;
  for (int s = 0; s < n_splits; ++s) {
    const float m = ml[s * sstride * 2], l = ml[s * sstride * 2 + 1];
    if (l != l) any_nan = true;
    if (l > 0.f) M = fmaxf(M, m);
  }
  const bool inf_row = (M == __int_as_float(0x7f800000));
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float m = ml[s * sstride * 2], l = ml[s * sstride * 2 + 1];
    if (!(l > 0.f)) continue;
    const float w = inf_row ? (m == M ? 1.f : 0.f) : exp2f(m - M);
    L += w * l;
  }
  const bool dead = !(L > 0.f) && !any_nan;
  const float nanv = __int_as_float(0x7fc00000);
  if (threadIdx.x == 0 && a.lse) {
    float lse = dead ? __int_as_float(0xff800000) : (M + log2f(L)) * 0.6931471805599453f;
    if (inf_row && !dead) lse = lse_inf_rows(L);
    if (any_nan) lse = nanv;
    a.lse[i + (long long)a.Lq * h + a.lse_sb * b] = lse;
  }
  T* xrow = reinterpret_cast<T*>(a.x) + (long long)i * a.x_sl + (long long)b * a.x_sb + (long long)h * a.dv;
  for (int e = threadIdx.x; e < a.dv; e += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float m = ml[s * sstride * 2], l = ml[s * sstride * 2 + 1];
      if (!(l > 0.f)) continue;
      const float w = inf_row ? (m == M ? 1.f : 0.f) : exp2f(m - M);
      acc = fmaf(w, o[(long long)s * sstride * a.dv + e], acc);
    }
    float out = acc * (a.inv_keep / L);
    if (dead) out = a.nan_fm ? nanv : 0.f;
    if (any_nan) out = nanv;
    xrow[e] = Elem<T>::from_f(out);
  }
}

template <typename T> struct Fmt;
template <> struct Fmt<__half> { static constexpr uint32_t v = 0; };
template <> struct Fmt<__nv_bfloat16> { static constexpr uint32_t v = 1; };
template <> struct Fmt<float> { static constexpr uint32_t v = 2; };

// SIDE: bias / Bool mask arrays are handled (through the per-row helpers of extras.cuh, chosen at run time);
// without it the loop holds no trace of them — the generic helpers cost 1.6 k of a tile's 3.7 k cycles even
// when a call has neither.
template <typename T, int DQ, int DV, int MODE, bool SIDE>
__global__ void __launch_bounds__(kTThreads, TCfg<T, DQ, DV>::kCtasPerSm)
attn_tile_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const AttnArgs a, const int n_qtiles, const int n_splits,
                 const int tail_units) {
  using C = TCfg<T, DQ, DV>;
  constexpr bool TF32 = (sizeof(T) == 4);
  constexpr bool BF16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr bool PV = (MODE == TM_FWD || MODE == TM_SPLIT);     // the modes that form O = P V
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  TBarriers* bars = reinterpret_cast<TBarriers*>(smem + C::kBarOff);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // block -> (unit, query tile); within a unit the longest causal rows come first, and the last `tail_units` units
  // are dealt out together, all their longest tiles first (the launch then does not end on the long tiles of the
  // last unit).  (TM_SPLIT: block -> (unit, split); there is one query tile)
  int unit, split = 0, qt = 0;
  if (MODE == TM_SPLIT) {
    unit = blockIdx.x / n_splits;
    split = blockIdx.x % n_splits;
  } else {
    const int n_units = gridDim.x / n_qtiles;
    const int head = (n_units - tail_units) * n_qtiles;
    if ((int)blockIdx.x < head) {
      unit = blockIdx.x / n_qtiles;
      qt = n_qtiles - 1 - (blockIdx.x % n_qtiles);
    } else {
      const int j = blockIdx.x - head;
      unit = (n_units - tail_units) + j % tail_units;
      qt = n_qtiles - 1 - j / tail_units;
    }
  }
  const int h = unit % a.H, b = unit / a.H;
  const int q0 = qt * kTBM;
  const int n_total = (a.Lkv + kTBN - 1) / kTBN;
  // tiles with live keys; causal: query i sees keys j <= i + coff, and a tile whose rows see none still walks
  // one (fully masked) key tile so that its rows come out as queries with nothing to attend to
  const int nt_all = a.causal ? min(n_total, (min(a.Lkv, max(q0 + kTBM + a.coff, 1)) + kTBN - 1) / kTBN) : n_total;
  // this CTA's share of them: tiles t0 .. t0 + nt - 1 (all of them unless the keys are split)
  const int per_split = (nt_all + n_splits - 1) / n_splits;
  const int t0 = (MODE == TM_SPLIT) ? split * per_split : 0;
  const int nt = (MODE == TM_SPLIT) ? max(0, min(nt_all, t0 + per_split) - t0) : nt_all;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kTMaxStages; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->p_ready[s], 4);
    }
    mbar_init(&bars->o_ready, 1);
    mbar_init(&bars->o_final, 1);
    bars->abort_flag = *reinterpret_cast<volatile int*>(&g_tile_abort);
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
    if (lane == 0 && nt > 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      if (PV) prefetch_tensormap(&tm_v);
      mbar_arrive_expect_tx(&bars->q_full, C::kQBytes);
#pragma unroll
      for (int c = 0; c < C::kQChunks; ++c)
        tma_load_4d(smem + C::kQOff + c * C::kQChunkBytes, &tm_q, &bars->q_full, c * C::kEpc, h, q0, b);
      bool ok = true;
      int j = 0;
      for (; j < nt; ++j) {
        const int s = j % C::kStages;
        if (j >= C::kStages) ok = mbar_wait(&bars->k_empty[s], ((j / C::kStages) - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars->k_full[s], C::kKBytes);
#pragma unroll
        for (int c = 0; c < C::kQChunks; ++c)
          tma_load_4d(smem + C::kKOff + s * C::kKBytes + c * C::kKChunkBytes, &tm_k, &bars->k_full[s], c * C::kEpc, h,
                      (t0 + j) * kTBN, b);
        if (PV) {
          if (j >= C::kStages) ok = mbar_wait(&bars->v_empty[s], ((j / C::kStages) - 1) & 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars->v_full[s], C::kVBytes);
#pragma unroll
          for (int c = 0; c < C::kVChunks; ++c)
            tma_load_4d(smem + C::kVOff + s * C::kVBytes + c * C::kKChunkBytes, &tm_v, &bars->v_full[s], c * C::kEpc, h,
                        (t0 + j) * kTBN, b);
        }
      }
      if (*abort_flag) {
        // give copies still in flight a bounded chance to land before the CTA leaves
        mbar_wait_drain(&bars->q_full, 0, kDrainNs);
        for (int jj = max(0, j - C::kStages); jj < j; ++jj) {
          mbar_wait_drain(&bars->k_full[jj % C::kStages], (jj / C::kStages) & 1, kDrainNs);
          if (PV) mbar_wait_drain(&bars->v_full[jj % C::kStages], (jj / C::kStages) & 1, kDrainNs);
        }
      }
    }
  } else if (start_ok && warp == 5) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && nt > 0) {
      constexpr uint32_t idesc_qk = make_idesc_fmt(Fmt<T>::v, kTBM, kTBN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_fmt(Fmt<T>::v, kTBM, DV, false, true);
      const uint32_t qa = smem_u32(smem + C::kQOff);
      const uint32_t tO = tmem + 2 * kTBN;
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag);
      // S(j) = Q K_j^T into score buffer j & 1
      auto issue_qk = [&](int j) {
        const int s = j % C::kStages;
        ok = mbar_wait(&bars->k_full[s], (j / C::kStages) & 1, abort_flag);
        if (!ok) return;
        tc_fence_after();
        const uint32_t ka = smem_u32(smem + C::kKOff + s * C::kKBytes);
#pragma unroll
        for (int c = 0; c < C::kQChunks; ++c)
#pragma unroll
          for (int st = 0; st < 4; ++st)
            umma_ss_kind<TF32>(tmem + (j & 1) * kTBN,
                               make_smem_desc_sw128(qa + c * C::kQChunkBytes + st * 32, 16, 1024),
                               make_smem_desc_sw128(ka + c * C::kKChunkBytes + st * 32, 16, 1024), idesc_qk,
                               (c > 0 || st > 0) ? 1u : 0u);
        umma_commit(&bars->s_full[j & 1]);
        umma_commit(&bars->k_empty[s]);
      };
      if (ok) issue_qk(0);
      if (ok && nt > 1) issue_qk(1);
      for (int j = 0; j < nt && ok; ++j) {
        // P(j) is in tensor memory (the modes that form P V) / S(j) has been read (the other modes)
        ok = mbar_wait(&bars->p_ready[j & 1], (j >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (PV) {
          const int s = j % C::kStages;
          ok = mbar_wait(&bars->v_full[s], (j / C::kStages) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t va = smem_u32(smem + C::kVOff + s * C::kVBytes);
#pragma unroll
          for (int ks = 0; ks < kTBN / C::kKStep; ++ks)
            umma_ts_kind<TF32>(tO, tmem + (j & 1) * kTBN + ks * 8,
                               TF32 ? make_smem_desc_sw128_32b(va + ks * C::kKStep * 128, C::kKChunkBytes, 512)
                                    : make_smem_desc_sw128(va + ks * C::kKStep * 128, C::kKChunkBytes, 1024),
                               idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&bars->v_empty[s]);
          umma_commit(&bars->o_ready);
          // The epilogue has a barrier of its own: a warp that is done early knows only that P(nt-3) V(nt-3) has
          // completed, and a parity wait on o_ready cannot tell phase nt - 1 from phase nt - 3.
          if (j == nt - 1) umma_commit(&bars->o_final);
        }
        if (j + 2 < nt) issue_qk(j + 2);
      }
    }
  } else if (start_ok && warp < 4 && nt > 0) {
    // ----------------------------------------------------------- softmax warps
    const int r = warp * 32 + lane;
    const int i = q0 + r;
    const bool row_ok = i < a.Lq;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    const uint32_t tO = lane_base + 2 * kTBN;
    const float c2 = a.scale * kLog2e;
    const int lim = a.causal ? min(i + a.coff, a.Lkv - 1) : a.Lkv - 1;   // last key this row attends to (< 0: none)
    const unsigned long long srow = score_row(a, row_ok ? i : 0, h, b);
    const bool drop = a.dropout_p > 0.f;
    RowSide rs;
    if (SIDE) rs = make_row_side(a, i, h, b, row_ok);
    // SIDE: the prepared logits are already scaled; plain logits get scale*log2(e) inside the exponential's FMA
    const float cs = SIDE ? 1.f : c2;

    float m_used = neg_inf();   // running maximum (scaled, base 2) the stored exponentials refer to
    float l = 0.f;
    // TM_SCORES: what the saved log-sum-exp says about this row
    float lse2 = 0.f, inf_share = 0.f, const_val = 0.f;
    bool row_const = false, rinf = false;
    T* arow = nullptr;
    if (MODE == TM_SCORES) {
      const float lse_nat = row_ok ? a.lse[i + (long long)a.Lq * h + a.lse_sb * b] : 0.f;
      rinf = lse_is_inf_rows(lse_nat);
      row_const = (lse_nat == neg_inf()) || (lse_nat != lse_nat && !rinf);   // nothing to attend to / a NaN logit
      const_val = (a.nan_fm || lse_nat != lse_nat) ? __int_as_float(0x7fc00000) : 0.f;
      inf_share = rinf ? 1.f / lse_inf_count(lse_nat) : 0.f;
      lse2 = lse_nat * kLog2e;
      arow = reinterpret_cast<T*>(a.alpha) + ((long long)i + (long long)a.Lq * h) * a.Lkv + a.alpha_sb * b;
    }
    bool ok = true;

    for (int j = 0; j < nt; ++j) {
      const int sb = j & 1;
      const int j0 = (t0 + j) * kTBN;
      // (one set of bias / mask words: the second chunk's are fetched once the first chunk's have been used, so
      // that the forward modes fit two CTAs on an SM)
      uint4 bq[4], mq[2];
      if (SIDE) side_issue<true>(rs, j0, a.Lkv, bq, mq);
      unsigned int kb[2] = {0xffffffffu, 0xffffffffu};
      if (MODE != TM_STATS && drop) {
#pragma unroll
        for (int c = 0; c < 2; ++c) kb[c] = dropout_keep32(a, srow, (unsigned int)(j0 >> 5) + c);
      }
      ok = mbar_wait_warp(&bars->s_full[sb], (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld32(lane_base + sb * kTBN, sr[0]);
      tmem_ld32(lane_base + sb * kTBN + 32, sr[1]);
      tmem_wait_ld();
      if (!PV) {
        // the scores are in registers: the issuer may refill this buffer
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_ready[sb]);
      }
      // scaled base-2 logits with bias, masks, causal limit and the end of the keys applied
      if (SIDE) {
        side_apply<true>(rs, sr[0], bq, mq, j0, a.Lkv, lim, row_ok, c2);
        side_issue<true>(rs, j0 + 32, a.Lkv, bq, mq);
        side_apply<true>(rs, sr[1], bq, mq, j0 + 32, a.Lkv, lim, row_ok, c2);
      } else if (__any_sync(0xffffffffu, j0 + kTBN - 1 > lim || !row_ok)) {
        // the causal diagonal, the end of the keys or the end of the queries runs through this tile
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (j0 + c * 32 + e > lim || !row_ok) sr[c][e] = 0xff800000u;
      }

      if (MODE == TM_SCORES) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float al = ex2_approx(fmaf(__uint_as_float(sr[c][e]), cs, -lse2));   // -inf (masked) gives 0
            if (rinf) al = (sr[c][e] == 0x7f800000u) ? inf_share : 0.f;
            if (row_const) al = const_val;
            if (drop) al = ((kb[c] >> e) & 1u) ? al * a.inv_keep : 0.f;
            sr[c][e] = __float_as_uint(al);
          }
        if (row_ok) {
          T* dst = arow + j0;
          const int n = min(kTBN, a.Lkv - j0);
          if (n == kTBN && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
            if (TF32) {
#pragma unroll
              for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int e = 0; e < 32; e += 4)
                  *reinterpret_cast<uint4*>(reinterpret_cast<float*>(dst) + c * 32 + e) =
                      make_uint4(sr[c][e], sr[c][e + 1], sr[c][e + 2], sr[c][e + 3]);
            } else {
#pragma unroll
              for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int e = 0; e < 32; e += 8) {
                  uint4 v;
                  v.x = pack2<BF16>(__uint_as_float(sr[c][e]), __uint_as_float(sr[c][e + 1]));
                  v.y = pack2<BF16>(__uint_as_float(sr[c][e + 2]), __uint_as_float(sr[c][e + 3]));
                  v.z = pack2<BF16>(__uint_as_float(sr[c][e + 4]), __uint_as_float(sr[c][e + 5]));
                  v.w = pack2<BF16>(__uint_as_float(sr[c][e + 6]), __uint_as_float(sr[c][e + 7]));
                  *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(dst) + (c * 32 + e) * 2) = v;
                }
            }
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int e = 0; e < 32; ++e)
                if (c * 32 + e < n) dst[c * 32 + e] = Elem<T>::from_f(__uint_as_float(sr[c][e]));
          }
        }
        continue;
      }

      // ---- running maximum (raised only when it grew by more than 2^8), rescale of what was gathered
      float mx = neg_inf();
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int e = 0; e < 32; e += 2) mx = max3(mx, __uint_as_float(sr[c][e]), __uint_as_float(sr[c][e + 1]));
      const float m_new = fmaxf(m_used, mx * cs);
      const bool raise = m_new > m_used + kTRescaleGap;        // also true for m_used = -inf < m_new
      if (__any_sync(0xffffffffu, raise)) {
        const float f = (raise && j > 0) ? ex2_approx(m_used - m_new) : 1.f;   // exp2(-inf) = 0: nothing gathered yet
        l *= f;
        if (PV && j > 0) {
          // O still receives P(j-1) V(j-1): wait for that product before touching the accumulator
          ok = mbar_wait_warp(&bars->o_ready, (j - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < DV / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tO + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
            tmem_st32(tO + c * 32, o);
          }
          tmem_wait_st();
        }
        if (raise) m_used = m_new;
      }
      // a row whose reference is +Inf (a +Inf bias) counts its +Inf logits instead (src/softmax.jl:73-75)
      const bool row_inf = (m_used == pos_inf());
      const float m_sub = (m_used == neg_inf()) ? 0.f : m_used;
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float p = ex2_approx(fmaf(__uint_as_float(sr[c][e]), cs, -m_sub));
          if (SIDE && row_inf) p = (sr[c][e] == 0x7f800000u) ? 1.f : 0.f;
          sum += p;
          // dropout follows the softmax: the row sum keeps the dropped scores
          sr[c][e] = ((kb[c] >> e) & 1u) ? (TF32 ? to_tf32(p) : __float_as_uint(p)) : 0u;
        }
      l += sum;
      if (PV) {
        if (TF32) {
          tmem_st32(lane_base + sb * kTBN, sr[0]);
          tmem_st32(lane_base + sb * kTBN + 32, sr[1]);
        } else {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 32; e += 2) pk[e >> 1] = pack2<BF16>(__uint_as_float(sr[c][e]), __uint_as_float(sr[c][e + 1]));
            tmem_st16(lane_base + sb * kTBN + c * 16, pk);
          }
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_ready[sb]);
      }
    }

    // ------------------------------------------------------------------ epilogue
    if (ok && MODE == TM_SCORES && row_ok) {
      // key tiles entirely above the causal diagonal
      const T z = Elem<T>::from_f(row_const ? const_val : 0.f);
      for (int jj = nt * kTBN; jj < a.Lkv; ++jj) arow[jj] = z;
    }
    if (ok && MODE == TM_SPLIT) {
      // partial result of this split: running maximum, sum, unnormalised O (first dv columns), fp32
      const long long slot = ((long long)unit * n_splits + split) * a.Lq + i;
      float* ml = a.ws + slot * 2;
      float* orow = a.ws + split_ml_floats(a, n_splits) + slot * a.dv;
      if (row_ok) { ml[0] = m_used; ml[1] = l; }
      ok = mbar_wait_warp(&bars->o_final, 0, abort_flag);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < DV / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              if (c * 32 + e < a.dv)
                *reinterpret_cast<uint4*>(orow + c * 32 + e) = make_uint4(o[e], o[e + 1], o[e + 2], o[e + 3]);
          }
        }
      }
    }
    if (ok && MODE != TM_SCORES && MODE != TM_SPLIT) {
      const bool dead = !(l > 0.f);
      if (a.lse && row_ok) {
        float lse_v = (l != l) ? __int_as_float(0x7fc00000) : dead ? neg_inf() : (m_used + log2f(l)) * kLn2;
        if (m_used == pos_inf() && !dead) lse_v = lse_inf_rows(l);
        a.lse[i + (long long)a.Lq * h + a.lse_sb * b] = lse_v;
      }
      if (MODE == TM_FWD) {
        ok = mbar_wait_warp(&bars->o_final, 0, abort_flag);
        if (ok) {
          tc_fence_after();
          const float inv = dead ? (a.nan_fm ? __int_as_float(0x7fc00000) : 0.f) : a.inv_keep / l;
          T* xrow = reinterpret_cast<T*>(a.x) + (long long)i * a.x_sl + (long long)b * a.x_sb + (long long)h * a.dv;
#pragma unroll
          for (int c = 0; c < DV / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tO + c * 32, o);
            tmem_wait_ld();
            if (row_ok) {
              constexpr int kVec = 16 / sizeof(T);       // elements per 16-byte store; dv is a multiple of it
#pragma unroll
              for (int e = 0; e < 32; e += kVec) {
                if (c * 32 + e < a.dv) {
                  float f[kVec];
#pragma unroll
                  for (int u = 0; u < kVec; ++u) f[u] = dead ? inv : __uint_as_float(o[e + u]) * inv;
                  uint4 v;
                  if (TF32) {
                    v = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2 % kVec]),
                                   __float_as_uint(f[3 % kVec]));
                  } else {
                    v.x = pack2<BF16>(f[0], f[1]);
                    v.y = pack2<BF16>(f[2], f[3]);
                    v.z = pack2<BF16>(f[4 % kVec], f[5 % kVec]);
                    v.w = pack2<BF16>(f[6 % kVec], f[7 % kVec]);
                  }
                  *reinterpret_cast<uint4*>(xrow + c * 32 + e) = v;
                }
              }
            }
          }
        }
      }
    }
  } else if (start_ok && warp < 4 && nt == 0) {
    // no key at all (Lkv = 0): every query is one with nothing to attend to
    const int i = q0 + warp * 32 + lane;
    if (i < a.Lq && MODE != TM_SCORES) {
      if (a.lse) a.lse[i + (long long)a.Lq * h + a.lse_sb * b] = neg_inf();
      if (MODE == TM_FWD) {
        T* xrow = reinterpret_cast<T*>(a.x) + (long long)i * a.x_sl + (long long)b * a.x_sb + (long long)h * a.dv;
        const T z = Elem<T>::from_f(a.nan_fm ? __int_as_float(0x7fc00000) : 0.f);
        for (int e = 0; e < a.dv; ++e) xrow[e] = z;
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
    atomicExch(&g_tile_abort, 1);
    if (a.status) atomicExch(a.status, NNLIB_B200_TIMEOUT);
  }
}

// (features of one head, heads, positions, batch) view of q, k or v: a box of one 128-byte row of features
// x `rows` positions of one head; features beyond the head's own are filled with zeros by the copy
// `mn_major`: the tile is read as an MN-major operand (V); for 32-bit elements that asks for the 128-byte
// swizzle with a 32-byte unit
bool make_head_map(CUtensorMap* m, const void* base, int dtype, long long dhead, long long H, long long len,
                   long long batch, long long stride_l, long long stride_b, int rows, bool mn_major = false) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t esz = (dtype == NNLIB_B200_F32) ? 4 : 2;
  const cuuint64_t dims[4] = {(cuuint64_t)dhead, (cuuint64_t)H, (cuuint64_t)len, (cuuint64_t)batch};
  const cuuint64_t strides[3] = {(cuuint64_t)dhead * esz, (cuuint64_t)stride_l * esz, (cuuint64_t)stride_b * esz};
  const cuuint32_t box[4] = {(cuuint32_t)(128 / esz), 1, (cuuint32_t)rows, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  // Float32 arrays are rounded to TF32 (to nearest) by the copy engine on their way into shared memory; the
  // tensor core itself would cut the mantissa off
  const CUtensorMapDataType dt = dtype == NNLIB_B200_F32    ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32
                                 : dtype == NNLIB_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                            : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUtensorMapSwizzle sw = (mn_major && esz == 4) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  const CUresult r = fn(m, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool tile_stride_ok(long long s, int esz) { return s > 0 && (s * esz) % 16 == 0 && s * esz < (1ll << 40); }

template <typename T, int DQ, int DV, int MODE, bool SIDE>
cudaError_t launch_tile_side(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnArgs& a,
                             cudaStream_t st, int n_splits) {
  using C = TCfg<T, DQ, DV>;
  auto kern = attn_tile_kernel<T, DQ, DV, MODE, SIDE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int n_qtiles = (a.Lq + kTBM - 1) / kTBM;
  const long long blocks = (long long)((MODE == TM_SPLIT) ? n_splits : n_qtiles) * a.H * a.B;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  // causal tiles differ in length: the units of the last two waves are dealt out longest tiles first
  long long tail_units = 0;
  if (MODE != TM_SPLIT && a.causal) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
      sms = 148;
    const long long resident = (long long)sms * C::kCtasPerSm;
    tail_units = 2 * ((resident + n_qtiles - 1) / n_qtiles);
    if (tail_units > (long long)a.H * a.B) tail_units = (long long)a.H * a.B;
  }
  kern<<<(unsigned)blocks, kTThreads, C::kSmemBytes, st>>>(mq, mk, mv, a, n_qtiles, n_splits, (int)tail_units);
  count_launch();
  if (MODE == TM_SPLIT) {
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const long long rows = (long long)a.Lq * a.H * a.B;
    attn_split_reduce_kernel<T><<<(unsigned)rows, 128, 0, st>>>(a, n_splits);
    count_launch();
  }
  return cudaGetLastError();
}

template <typename T, int DQ, int DV, int MODE>
cudaError_t launch_tile(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnArgs& a,
                        cudaStream_t st, int n_splits = 1) {
  if (a.bias != nullptr || a.mask != nullptr) return launch_tile_side<T, DQ, DV, MODE, true>(mq, mk, mv, a, st, n_splits);
  return launch_tile_side<T, DQ, DV, MODE, false>(mq, mk, mv, a, st, n_splits);
}

template <typename T, int MODE>
cudaError_t launch_tile_dims(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnArgs& a,
                             cudaStream_t st, int n_splits) {
  // head sizes are padded (with zeros, by the copy engine) to 64, 128 or — 16-bit element types only — 256
  if constexpr (sizeof(T) == 2 && (MODE == TM_FWD || MODE == TM_SPLIT)) {
    if (a.dv > 128) return launch_tile<T, 256, 256, MODE>(mq, mk, mv, a, st, n_splits);
    if (a.d > 128) return launch_tile<T, 256, 128, MODE>(mq, mk, mv, a, st, n_splits);
  } else if constexpr (sizeof(T) == 2) {
    if (a.d > 128) return launch_tile<T, 256, 64, MODE>(mq, mk, mv, a, st, n_splits);
  }
  const bool q128 = a.d > 64;
  if (MODE != TM_FWD && MODE != TM_SPLIT) {   // the value heads play no part: one instantiation per query-head size
    if (q128) return launch_tile<T, 128, 64, MODE>(mq, mk, mv, a, st, n_splits);
    return launch_tile<T, 64, 64, MODE>(mq, mk, mv, a, st, n_splits);
  }
  const bool v128 = a.dv > 64;
  if (q128 && v128) return launch_tile<T, 128, 128, MODE>(mq, mk, mv, a, st, n_splits);
  if (q128) return launch_tile<T, 128, 64, MODE>(mq, mk, mv, a, st, n_splits);
  if (v128) return launch_tile<T, 64, 128, MODE>(mq, mk, mv, a, st, n_splits);
  return launch_tile<T, 64, 64, MODE>(mq, mk, mv, a, st, n_splits);
}

template <int MODE>
cudaError_t tile_run(const AttnArgs& a, int dtype, cudaStream_t st, int n_splits = 1) {
  CUtensorMap mq, mk, mv;
  if (!make_head_map(&mq, a.q, dtype, a.d, a.H, a.Lq, a.B, a.q_sl, a.q_sb, kTBM)) return cudaErrorInvalidValue;
  if (!make_head_map(&mk, a.k, dtype, a.d, a.H, a.Lkv, a.B, a.k_sl, a.k_sb, kTBN)) return cudaErrorInvalidValue;
  if (MODE == TM_FWD || MODE == TM_SPLIT) {
    if (!make_head_map(&mv, a.v, dtype, a.dv, a.H, a.Lkv, a.B, a.v_sl, a.v_sb, kTBN, true)) return cudaErrorInvalidValue;
  } else {
    mv = mk;
  }
  switch (dtype) {
    case NNLIB_B200_F16:  return launch_tile_dims<__half, MODE>(mq, mk, mv, a, st, n_splits);
    case NNLIB_B200_BF16: return launch_tile_dims<__nv_bfloat16, MODE>(mq, mk, mv, a, st, n_splits);
    default:              return launch_tile_dims<float, MODE>(mq, mk, mv, a, st, n_splits);
  }
}

}  // namespace

// nullptr when these kernels take the call, else the reason they do not.  Float32 arrays only with
// `allow_tf32` (the products then run with a 10-bit mantissa).
const char* tile_reject_reason(const AttnArgs& a, int dtype, bool need_v, bool allow_tf32) {
  if (dtype == NNLIB_B200_F32 && !allow_tf32) return "Float32 arrays without allow_tf32 (exact CUDA-core arithmetic)";
  const int esz = (dtype == NNLIB_B200_F32) ? 4 : 2;
  const int vec = 16 / esz;
  const int dmax = (esz == 2) ? 256 : 128;   // a 128-query tile of Float32 heads of 256 would not leave room for the key ring
  if (a.d < 1 || a.d > dmax || a.d % vec != 0)
    return "head size d is not a multiple of 16 bytes of elements up to 256 (16-bit types) / 128 (Float32)";
  if (need_v && (a.dv < 1 || a.dv > dmax || a.dv % vec != 0))
    return "head size dv is not a multiple of 16 bytes of elements up to 256 (16-bit types) / 128 (Float32)";
  if (!(a.scale > 0.f)) return "scale is not positive";
  if (a.Lq < 1 || a.Lkv < 1 || a.H < 1 || a.B < 1) return "empty problem";
  if (!aligned16(a.q) || !aligned16(a.k)) return "q or k is not 16-byte aligned";
  if (!tile_stride_ok(a.q_sl, esz) || !tile_stride_ok(a.k_sl, esz) || !tile_stride_ok(a.q_sb, esz) ||
      !tile_stride_ok(a.k_sb, esz))
    return "a stride of q or k is not a positive multiple of 16 bytes";
  if (need_v) {
    if (!aligned16(a.v) || !aligned16(a.x)) return "v or x is not 16-byte aligned";
    if (!tile_stride_ok(a.v_sl, esz) || !tile_stride_ok(a.v_sb, esz) || !tile_stride_ok(a.x_sl, esz) ||
        !tile_stride_ok(a.x_sb, esz))
      return "a stride of v or x is not a positive multiple of 16 bytes";
  }
  if (encode_tiled_fn() == nullptr) return "the driver does not export cuTensorMapEncodeTiled";
  return nullptr;
}

cudaError_t tile_fwd(const AttnArgs& a, int dtype, cudaStream_t st) { return tile_run<TM_FWD>(a, dtype, st); }
cudaError_t tile_stats(const AttnArgs& a, int dtype, cudaStream_t st) { return tile_run<TM_STATS>(a, dtype, st); }
cudaError_t tile_scores(const AttnArgs& a, int dtype, cudaStream_t st) { return tile_run<TM_SCORES>(a, dtype, st); }

// Split-key forward for few queries (Lq <= 128).  How many CTAs share the key tiles of one unit: enough to
// give every SM about two CTAs, at least four 64-key tiles each, never an empty share.
int tile_split_count(const AttnArgs& a) {
  if (a.Lq < 1 || a.Lq > kTBM || a.Lkv < 1) return 0;
  const int n_total = (a.Lkv + kTBN - 1) / kTBN;
  const int nt = a.causal ? std::min(n_total, (std::min(a.Lkv, std::max(kTBM + a.coff, 1)) + kTBN - 1) / kTBN) : n_total;
  const long long units = (long long)a.H * a.B;
  // with a CTA for at least half of the SMs already, the two-tile kernel (one CTA per unit walking all the
  // keys) moves the keys faster than these kernels would with the keys split
  if (units * 2 > 148) return 1;
  long long want = (2LL * 148 + units - 1) / units;
  want = std::min<long long>(want, std::max(1, nt / 4));
  want = std::max<long long>(want, 1);
  const int per = (int)((nt + want - 1) / want);
  return (nt + per - 1) / per;
}
size_t tile_split_workspace_bytes(const AttnArgs& a) {
  const int n = tile_split_count(a);
  return n > 0 ? (size_t)split_ws_floats(a, n) * sizeof(float) : 0;
}
cudaError_t tile_split(const AttnArgs& a, int dtype, cudaStream_t st) {
  return tile_run<TM_SPLIT>(a, dtype, st, tile_split_count(a));
}

// Reads and clears the sticky "a bounded wait ran out" flag of these kernels on the current device.
cudaError_t tile_take_abort(int* out, cudaStream_t st) {
  int v = 0;
  cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyFromSymbol(&v, g_tile_abort, sizeof(int));
  if (e != cudaSuccess) return e;
  if (v) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_tile_abort, &zero, sizeof(int));
  }
  *out = v;
  return e;
}

}  // namespace nb200
