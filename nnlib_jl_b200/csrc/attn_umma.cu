// Fused attention forward on the sm_100a tensor cores.
//
// One CTA owns 256 consecutive queries (two 128-row tiles) of one (head,
// batch) unit and walks over the keys/values in 128-row tiles.  Heads are
// addressed through 4-d tensor maps (features of a head, heads, positions,
// batch), so a head narrower than the padded size D (64 or 128) arrives with
// zeros behind its own features and any d = dv <= 128 that is a multiple of 8
// runs here:
//
//   warp 0      TMA producer of Q (once) and of the ring of K tiles
//   warp 3      TMA producer of the ring of V tiles
//   warp 1      issues every tcgen05.mma:  S_t = Q_t K_j^T   (smem x smem -> TMEM)
//                                          O_t += P_t V_j    (TMEM x smem -> TMEM)
//   warp 2      allocates / frees the 512 TMEM columns
//   warps 4-7   softmax of query tile 0 (thread r owns query row r: no shuffles)
//   warps 8-11  softmax of query tile 1
//
// TMEM columns: S_0 [0,128) S_1 [128,256) O_0 [256,384) O_1 [384,512); the
// half-precision probabilities P_t overwrite the first 64 columns of S_t.
// The two query tiles ping-pong: while the softmax warps of one tile run
// exponentials, the tensor core works on the other tile's products.
//
// Softmax is the online form of the reference's max-subtracted softmax
// (NNlib.jl src/softmax.jl:69-79) in base 2: logits are scaled by
// scale*log2(e), bias (src/attention.jl:129-131) and masks (:133-138) are
// applied in registers, the running maximum is only raised when it grows by
// more than 8 (so the O accumulator is rarely rescaled), dropout
// (src/dropout.jl:77-87) multiplies P after the row sum was taken, and
// x = O / l / (1-p) is written straight into the (Ev, Lq, B) array.
// Per-query log-sum-exp is stored so that the scores can be rebuilt later.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "extras.cuh"
#include "launchers.h"
#include "umma.cuh"
#include "umma_shared.cuh"

namespace nb200 {

__device__ int g_umma_abort = 0;  // sticky: a bounded wait ran out somewhere


namespace {

constexpr int kQT = 2;                 // query tiles per CTA
constexpr int kThreads = 384;
constexpr float kRescaleGap = 8.0f;    // raise the running max only when it grew by > 2^8

template <int D>
struct Cfg {
  static constexpr int kChunks = D / 64;
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  // A K tile is released early in the round after its last use, a V tile only at the end of its
  // round, so V needs the deeper ring to keep a full round of copy latency hidden.
  static constexpr int kStagesK = (D == 128) ? 2 : 4;
  static constexpr int kStagesV = (D == 128) ? 3 : 4;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kQT * kTileBytes;
  static constexpr int kVOff = kKOff + kStagesK * kTileBytes;
  static constexpr int kBarOff = kVOff + kStagesV * kTileBytes;
  static constexpr int kSmemBytes = kBarOff + 512 + 1024;  // barrier block + alignment slack
  // staged-bias variant (d = 64): per query tile two half tiles (64 keys x 128 queries) of the bias
  static constexpr int kBiasOff = kBarOff;
  static constexpr int kBiasBytes = kQT * 2 * kChunkBytes;
  static constexpr int kBarOffStaged = kBiasOff + kBiasBytes;
  static constexpr int kSmemBytesStaged = kBarOffStaged + 512 + 1024;
};
static_assert(Cfg<128>::kSmemBytes <= 232448 && Cfg<64>::kSmemBytes <= 232448, "shared memory budget");
static_assert(Cfg<64>::kSmemBytesStaged <= 232448, "shared memory budget (staged bias)");

struct Barriers {
  uint64_t q_full[kQT];
  uint64_t k_full[4], k_empty[4], v_full[4], v_empty[4];
  uint64_t s_full[kQT], p_half[kQT][2], o_full[kQT];
  uint64_t bias_full[kQT][2], bias_empty[kQT][2];   // staged bias half tiles
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(Barriers) <= 512, "barrier block");

// XM = side + 3*drop.  side: 0 = no side input (optionally causal), 1 = Bool mask array only,
// 2 = bias (and mask); drop: dropout code compiled in.  Each combination is its own kernel so that
// the registers of one feature (bias prefetch buffers, Philox state) are not paid for by the others.
// BSM: the bias tiles arrive in shared memory by TMA (a whole round ahead, issued by the otherwise
// idle warp 2) instead of through per-thread loads; needs a 16-bit bias with key stride 1 whose rows
// the tensor map can address (the host decides).
template <int D, bool BF16, int XM, bool STATS, bool BSM>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_umma_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_b,
                     const AttnArgs a, const int n_qblocks, const int tail_units) {
  using C = Cfg<D>;
  constexpr bool EXTRAS = (XM % 3) != 0;
  constexpr bool XBIAS = (XM % 3) == 2;   // bias code compiled in
  constexpr bool DROP = XM >= 3;          // dropout code compiled in
  static_assert(!BSM || (XBIAS && D == 64 && !STATS), "staged bias: d = 64 forward with bias only");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + (BSM ? C::kBarOffStaged : C::kBarOff));
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // block -> (unit, query block).  Unit by unit, so that the CTAs running at one time share K and V in L2; within
  // a unit the longest causal rows first.  The last `tail_units` units are dealt out together, all their longest
  // blocks first: taken unit by unit, the long blocks of the last unit would start when the others are nearly
  // done (3 - 4 % of a launch of 256 units, more of a shorter one).
  int unit, qb;
  {
    const int n_units = gridDim.x / n_qblocks;
    const int head = (n_units - tail_units) * n_qblocks;
    if ((int)blockIdx.x < head) {
      unit = blockIdx.x / n_qblocks;
      qb = n_qblocks - 1 - (blockIdx.x % n_qblocks);
    } else {
      const int j = blockIdx.x - head;
      unit = (n_units - tail_units) + j % tail_units;
      qb = n_qblocks - 1 - j / tail_units;
    }
  }
  const int h = unit % a.H, b = unit / a.H;
  const int q0 = qb * (kQT * kBM);

  // number of kv tiles each query tile walks over
  int n_t0, n_t1;
  {
    int kv_end0 = a.Lkv, kv_end1 = a.Lkv;
    // causal: query i sees keys j <= i + coff; a tile whose rows see no key at all still walks one key tile
    // (everything masked), so that its rows come out as queries with nothing to attend to
    if (a.causal) {
      kv_end0 = min(kv_end0, max(q0 + kBM + a.coff, 1));
      kv_end1 = min(kv_end1, max(q0 + 2 * kBM + a.coff, 1));
    }
    n_t0 = (q0 < a.Lq) ? (kv_end0 + kBN - 1) / kBN : 0;
    n_t1 = (q0 + kBM < a.Lq) ? (kv_end1 + kBN - 1) / kBN : 0;
  }
  const int n_kv = max(n_t0, n_t1);

  if (threadIdx.x == 0) {
    for (int t = 0; t < kQT; ++t) {
      mbar_init(&bars->q_full[t], 1);
      mbar_init(&bars->s_full[t], 1);
      mbar_init(&bars->p_half[t][0], 4);
      mbar_init(&bars->p_half[t][1], 4);
      mbar_init(&bars->o_full[t], 1);
      for (int hf = 0; hf < 2; ++hf) {
        mbar_init(&bars->bias_full[t][hf], 1);
        mbar_init(&bars->bias_empty[t][hf], 4);
      }
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    bars->abort_flag = *reinterpret_cast<volatile int*>(&g_umma_abort);
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  const bool start_ok = (*abort_flag == 0);

  // The softmax threads hold a whole 128-wide score row in registers: move the
  // register budget from the copy / issue warps to them.
  if (warp < 4) {
    setmaxnreg_dec<72>();
    if (start_ok && warp == 0 && lane == 0) {
      // ------------------------------------------------- producer of Q and K
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
#pragma unroll
      for (int t = 0; t < kQT; ++t) {
        if ((t == 0 ? n_t0 : n_t1) == 0) continue;
        mbar_arrive_expect_tx(&bars->q_full[t], C::kTileBytes);
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_4d(smem + C::kQOff + t * C::kTileBytes + c * kChunkBytes, &tm_q, &bars->q_full[t],
                      c * 64, h, q0 + t * kBM, b);
      }
      bool ok = true;
      int j = 0;
      for (; j < n_kv; ++j) {
        const int s = j % C::kStagesK;
        if (j >= C::kStagesK) ok = mbar_wait(&bars->k_empty[s], ((j / C::kStagesK) - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars->k_full[s], C::kTileBytes);
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_4d(smem + C::kKOff + s * C::kTileBytes + c * kChunkBytes, &tm_k, &bars->k_full[s],
                      c * 64, h, j * kBN, b);
      }
      if (*abort_flag) {
        // give copies still in flight a bounded chance to land before the CTA leaves
        for (int jj = max(0, j - C::kStagesK); jj < j; ++jj)
          mbar_wait_drain(&bars->k_full[jj % C::kStagesK], (jj / C::kStagesK) & 1, kDrainNs);
      }
    } else if (!STATS && start_ok && warp == 3 && lane == 0) {
      // ------------------------------------------------------ producer of V
      // (its own thread: a K tile must never queue behind a V slot that is still in use)
      prefetch_tensormap(&tm_v);
      bool ok = true;
      int j = 0;
      for (; j < n_kv; ++j) {
        const int s = j % C::kStagesV;
        if (j >= C::kStagesV) ok = mbar_wait(&bars->v_empty[s], ((j / C::kStagesV) - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars->v_full[s], C::kTileBytes);
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_4d(smem + C::kVOff + s * C::kTileBytes + c * kChunkBytes, &tm_v, &bars->v_full[s],
                      c * 64, h, j * kBN, b);
      }
      if (*abort_flag) {
        for (int jj = max(0, j - C::kStagesV); jj < j; ++jj)
          mbar_wait_drain(&bars->v_full[jj % C::kStagesV], (jj / C::kStagesV) & 1, kDrainNs);
      }
    } else if (BSM && start_ok && warp == 2 && lane == 0) {
      // --------------------------------------------------- producer of bias
      // half tile (64 keys x 128 queries) = one 128-byte-swizzled box; a slot is refilled for the
      // next round as soon as the four softmax warps of the tile have read it
      prefetch_tensormap(&tm_b);
      const int hb = a.bias_s[2] ? h : 0, bb = a.bias_s[3] ? b : 0;   // broadcast dimensions have extent 1
      bool ok = true;
      int j = 0;
      for (; j < n_kv && ok; ++j) {
#pragma unroll
        for (int t = 0; t < kQT; ++t) {
          if (j >= ((t == 0) ? n_t0 : n_t1)) continue;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            if (j > 0 && ok) ok = mbar_wait(&bars->bias_empty[t][hf], (j - 1) & 1, abort_flag);
            if (!ok) break;
            mbar_arrive_expect_tx(&bars->bias_full[t][hf], kChunkBytes);
            tma_load_4d(smem + C::kBiasOff + (t * 2 + hf) * kChunkBytes, &tm_b, &bars->bias_full[t][hf],
                        j * kBN + hf * 64, q0 + t * kBM, hb, bb);
          }
        }
      }
      if (*abort_flag) {
        for (int t = 0; t < kQT; ++t)
          for (int hf = 0; hf < 2; ++hf) {
            const int nt = (t == 0) ? n_t0 : n_t1;
            const int last = min(j, nt) - 1;
            if (last >= 0) mbar_wait_drain(&bars->bias_full[t][hf], last & 1, kDrainNs);
          }
      }
    } else if (start_ok && warp == 1 && lane == 0 && n_kv > 0) {
      // -------------------------------------------------------- MMA issuer
      // One thread issues for both query tiles, tile 0 then tile 1 in every round; serving them in
      // turn is also what keeps the two softmax warpgroups half a period apart.  Descriptors: the
      // high word is constant, the low word is the tile address (>>4) plus the leading-byte-offset
      // field; stepping along K only adds to the address field.
      constexpr uint32_t idesc_qk = make_idesc_f16(BF16, kBM, kBN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(BF16, kBM, D, false, true);
      constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1 KB, sm_100 version, 128B swizzle
      constexpr uint32_t lbo_k = (16u >> 4) << 16;                          // K-major operands: unused, 16
      constexpr uint32_t lbo_v = (static_cast<uint32_t>(kChunkBytes) >> 4) << 16;  // V: next 64-wide dv block
      constexpr uint32_t tile16 = C::kTileBytes >> 4;
      const uint32_t q_lo = (smem_u32(smem + C::kQOff) >> 4) | lbo_k;
      const uint32_t k_lo = (smem_u32(smem + C::kKOff) >> 4) | lbo_k;
      const uint32_t v_lo = (smem_u32(smem + C::kVOff) >> 4) | lbo_v;
      bool ok = true;

#define NB_ISSUE_QK(T_, STAGE_)                                                                  \
  do {                                                                                           \
    _Pragma("unroll") for (int kk = 0; kk < D / 16; ++kk) {                                      \
      const uint32_t off = (kk >> 2) * (kChunkBytes >> 4) + (kk & 3) * 2;                        \
      umma_ss_lohi(tmem + (T_) * kBN, q_lo + (T_) * tile16 + off, k_lo + (STAGE_) * tile16 + off, desc_hi, \
                   idesc_qk, kk > 0 ? 1u : 0u);                                                  \
    }                                                                                            \
  } while (0)
#define NB_ISSUE_PV(T_, STAGE_, KK0_, KK1_, FIRST_)                                              \
  do {                                                                                           \
    _Pragma("unroll") for (int kk = (KK0_); kk < (KK1_); ++kk) {                                 \
      umma_ts_lohi(tmem + kQT * kBN + (T_) * D, tmem + (T_) * kBN + kk * 8,                      \
                   v_lo + (STAGE_) * tile16 + kk * (2048 >> 4), desc_hi, idesc_pv,               \
                   ((FIRST_) && kk == 0) ? 0u : 1u);                                             \
    }                                                                                            \
  } while (0)

      if (n_t0 > 0) ok = mbar_wait(&bars->q_full[0], 0, abort_flag);
      if (ok && n_t1 > 0) ok = mbar_wait(&bars->q_full[1], 0, abort_flag);
      if (ok) ok = mbar_wait(&bars->k_full[0], 0, abort_flag);
      if (ok) {
        if (n_t0 > 0) { NB_ISSUE_QK(0, 0); umma_commit(&bars->s_full[0]); }
        if (n_t1 > 0) { NB_ISSUE_QK(1, 0); umma_commit(&bars->s_full[1]); }
        umma_commit(&bars->k_empty[0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int sv = j % C::kStagesV;
        const int sk = (j + 1) % C::kStagesK;
        const uint32_t par = j & 1;
        // operand tiles first: they land long before the probabilities are ready, so these two
        // waits cost nothing on the softmax -> MMA -> softmax chain
        if (!STATS) ok = mbar_wait(&bars->v_full[sv], (j / C::kStagesV) & 1, abort_flag);
        if (ok && j + 1 < n_kv) ok = mbar_wait(&bars->k_full[sk], ((j + 1) / C::kStagesK) & 1, abort_flag);
#pragma unroll
        for (int t = 0; t < kQT; ++t) {
          const int nt = (t == 0) ? n_t0 : n_t1;
          if (!ok || j >= nt) continue;
          // first half of P_t(j) is in TMEM (STATS: S_t(j) has been read)
          ok = mbar_wait(&bars->p_half[t][0], par, abort_flag);
          if (!ok) continue;
          tc_fence_after();
          if (!STATS) {
            NB_ISSUE_PV(t, sv, 0, kBN / 32, j == 0);
            ok = mbar_wait(&bars->p_half[t][1], par, abort_flag);
            if (!ok) continue;
            tc_fence_after();
            NB_ISSUE_PV(t, sv, kBN / 32, kBN / 16, false);
          }
          if (j + 1 < nt) {
            NB_ISSUE_QK(t, sk);
            umma_commit(&bars->s_full[t]);
          } else if (!STATS) {
            umma_commit(&bars->o_full[t]);
          }
        }
        if (!ok) break;
        if (!STATS) umma_commit(&bars->v_empty[sv]);
        if (j + 1 < n_kv) umma_commit(&bars->k_empty[sk]);
      }
#undef NB_ISSUE_QK
#undef NB_ISSUE_PV
    }
  } else {
    setmaxnreg_inc<216>();
    const int t = (warp - 4) >> 2;        // query tile of this warpgroup
    const int nt = (t == 0) ? n_t0 : n_t1;
    if (start_ok && nt > 0) {
      // ----------------------------------------------------- softmax warps
      const int wq = warp & 3;              // TMEM lane quarter this warp may touch
      const int r = wq * 32 + lane;         // row inside the tile
      const int i = q0 + t * kBM + r;       // query index
      const bool row_ok = i < a.Lq;
      const uint32_t lane_base = tmem + (static_cast<uint32_t>(wq * 32) << 16);
      const uint32_t tS = lane_base + t * kBN;
      const uint32_t tO = lane_base + kQT * kBN + t * D;
      const float c2 = a.scale * kLog2e;
      const int lim = a.causal ? min(i + a.coff, a.Lkv - 1) : a.Lkv - 1;  // last kv index this row attends to (< 0: none)
      const unsigned long long srow = score_row(a, row_ok ? i : 0, h, b);

      float m_used = neg_inf();  // running maximum (scaled, base 2) the stored exponentials refer to
      float l = 0.f;             // running sum of exponentials
      bool ok = true;
      RowSide rs;
      if (EXTRAS) rs = make_row_side(a, i, h, b, row_ok);

      for (int j = 0; j < nt; ++j) {
        // bias / mask of the first 64 keys of this tile: in flight while the scores are awaited
        uint4 bq[2][4], mq[2][2];
        if (EXTRAS) {
          side_issue<XBIAS && !BSM>(rs, j * kBN, a.Lkv, bq[0], mq[0]);
          side_issue<XBIAS && !BSM>(rs, j * kBN + 32, a.Lkv, bq[1], mq[1]);
        }
        // which of this tile's 128 scores survive dropout depends on their position only: drawn while
        // the tensor core still works on the scores
        unsigned int kb[4] = {0u, 0u, 0u, 0u};
        if (DROP) {
#pragma unroll
          for (int c = 0; c < 4; ++c) kb[c] = dropout_keep32(a, srow, (unsigned int)(j * kBN >> 5) + c);
        }
        ok = mbar_wait(&bars->s_full[t], j & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t sr[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, sr[c]);
        tmem_wait_ld();

        const int j0 = j * kBN;
        if (STATS) {
          // S is in registers: the MMA warp may overwrite it with the next tile's scores
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->p_half[t][0]);
        }

        // ---- logits -> (masked, biased) values the exponentials are taken of
        if (EXTRAS) {
          // scaled base-2 units, bias added, masks applied; the loads of chunk c+2 start as chunk c is consumed
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (BSM) {
              // this thread's 32 bias values of chunk c from the staged half tile (row r, swizzled pieces)
              const int hf = c >> 1;
              if ((c & 1) == 0) {
                ok = mbar_wait(&bars->bias_full[t][hf], j & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
              }
              const uint8_t* brow = smem + C::kBiasOff + (t * 2 + hf) * kChunkBytes + r * 128;
#pragma unroll
              for (int v = 0; v < 4; ++v)
                bq[c & 1][v] = *reinterpret_cast<const uint4*>(brow + ((((c & 1) * 4 + v) ^ (r & 7)) << 4));
              if ((c & 1) == 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->bias_empty[t][hf]);
              }
            }
            side_apply<XBIAS, BSM>(rs, sr[c], bq[c & 1], mq[c & 1], j0 + c * 32, a.Lkv, lim, row_ok, c2);
            if (c + 2 < 4) side_issue<XBIAS && !BSM>(rs, j0 + (c + 2) * 32, a.Lkv, bq[c & 1], mq[c & 1]);
          }
          if (!ok) break;
        } else if (j0 + kBN - 1 > lim) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (j0 + c * 32 + e > lim) sr[c][e] = 0xff800000u;
        }
        // EXTRAS values are already scaled; plain logits get scale*log2(e) inside the exponential's FMA
        const float cs = EXTRAS ? 1.f : c2;

        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        unsigned long long sum2[2] = {0ull, 0ull};   // the plain variants: two pairs of partial row sums (packed fp32 adds)
        const unsigned long long cs2 = pair_of(cs);
        uint32_t pk[32];
        // exponentials of 64 keys (chunks 2*HF, 2*HF+1) relative to REF, packed into pk, summed into sum2
        // SEL (a literal): rows whose reference is +Inf put weight 1 on their +Inf logits and 0 elsewhere
        // (the slow branch of the reference's softmax, src/softmax.jl:73-75) instead of exp2(Inf - Inf)
#define NB_EXP_HALF(HF, REF, SEL)                                                                  \
  do {                                                                                             \
    const float ref_ = (REF);                                                                      \
    const float nref_ = -ref_;                                                                     \
    const unsigned long long nref2_ = pair_of(nref_);                                              \
    _Pragma("unroll") for (int cc = 0; cc < 2; ++cc) {                                             \
      _Pragma("unroll") for (int e = 0; e < 32; e += 2) {                                          \
        float p0, p1;                                                                              \
        if (EXTRAS) {                                                                              \
          /* the variants with side inputs measured slower with the packed forms */               \
          p0 = ex2_approx(fmaf(__uint_as_float(sr[(HF) * 2 + cc][e]), cs, nref_));                 \
          p1 = ex2_approx(fmaf(__uint_as_float(sr[(HF) * 2 + cc][e + 1]), cs, nref_));             \
          if ((SEL) && ref_ == pos_inf()) {                                                        \
            p0 = (sr[(HF) * 2 + cc][e] == 0x7f800000u) ? 1.f : 0.f;                                \
            p1 = (sr[(HF) * 2 + cc][e + 1] == 0x7f800000u) ? 1.f : 0.f;                            \
          }                                                                                        \
          sum4[(e >> 1) & 3] += p0 + p1;                                                           \
        } else {                                                                                   \
          /* two logits per instruction: scale and subtract the reference, add to the row sum */  \
          float x0, x1;                                                                            \
          fma2(x0, x1, __uint_as_float(sr[(HF) * 2 + cc][e]), __uint_as_float(sr[(HF) * 2 + cc][e + 1]), cs2, nref2_); \
          p0 = ex2_approx(x0);                                                                     \
          p1 = ex2_approx(x1);                                                                     \
          add2(sum2[(e >> 1) & 1], p0, p1);                                                        \
        }                                                                                          \
        pk[cc * 16 + (e >> 1)] = pack2<BF16>(p0, p1);                                              \
      }                                                                                            \
    }                                                                                              \
  } while (0)
        // one of the two expansions, chosen per warp: the +Inf form only when a row of this warp needs it
#define NB_EXP_HALF_W(HF, REF)                                                                     \
  do {                                                                                             \
    if (XBIAS && infw) NB_EXP_HALF(HF, REF, 1); else NB_EXP_HALF(HF, REF, 0);                      \
  } while (0)

        // full-tile maximum (3-input max: 64 instructions); independent of the first exponentials below
        float mx;
        {
          float m0 = neg_inf(), m1 = neg_inf(), m2 = neg_inf(), m3 = neg_inf();
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              m0 = max3(m0, __uint_as_float(sr[c][e]), __uint_as_float(sr[c][e + 1]));
              m1 = max3(m1, __uint_as_float(sr[c][e + 2]), __uint_as_float(sr[c][e + 3]));
              m2 = max3(m2, __uint_as_float(sr[c][e + 4]), __uint_as_float(sr[c][e + 5]));
              m3 = max3(m3, __uint_as_float(sr[c][e + 6]), __uint_as_float(sr[c][e + 7]));
            }
          mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * cs;
        }
        const float m_new = fmaxf(m_used, mx);
        const bool raise = m_new > m_used + kRescaleGap;   // also true for m_used = -inf < m_new
        // A +Inf logit can only come from the bias.  A row that meets one moves its reference to +Inf
        // (the rescale factor exp2(old - Inf) = 0 clears what it had gathered) and from then on counts
        // its +Inf logits; the warp takes the selecting form of the exponentials while it has such a row.
        const bool infw = XBIAS && __any_sync(0xffffffffu, m_new == pos_inf());

        if (!STATS) {
          // First 64 exponentials against the running reference while the maximum above is still being
          // reduced (different pipes).  Later tiles almost never move the reference; when one does, the
          // half is simply redone below.  The very first tile has no reference yet and skips the guess.
          const bool guess = (j > 0) && !infw;
          if (guess) NB_EXP_HALF(0, (m_used == neg_inf()) ? 0.f : m_used, 0);
          if (!guess || __any_sync(0xffffffffu, raise)) {
            if (j > 0) {
              const float f = raise ? ex2_approx(m_used - m_new) : 1.f;  // m_used = -inf gives 0: O is still 0 there
              l *= f;
#pragma unroll
              for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(tO + c * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
                tmem_st32(tO + c * 32, o);
              }
            }
            if (raise) m_used = m_new;
            sum4[0] = sum4[1] = sum4[2] = sum4[3] = 0.f;
            sum2[0] = sum2[1] = 0ull;
            NB_EXP_HALF_W(0, (m_used == neg_inf()) ? 0.f : m_used);
          }
          const float m_sub = (m_used == neg_inf()) ? 0.f : m_used;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            if (hf == 1) NB_EXP_HALF_W(1, m_sub);
            if (DROP) {
              // the row sum keeps the dropped scores (dropout follows the softmax)
#pragma unroll
              for (int cc = 0; cc < 2; ++cc) {
                const unsigned int kbc = kb[hf * 2 + cc];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                  // pk[cc*16 + e] holds keys 2e (low half) and 2e+1 (high half) of this 32-key chunk
                  const unsigned int m = (((kbc >> (2 * e)) & 1u) ? 0x0000ffffu : 0u) |
                                         (((kbc >> (2 * e + 1)) & 1u) ? 0xffff0000u : 0u);
                  pk[cc * 16 + e] &= m;
                }
              }
            }
            tmem_st32(tS + hf * 32, pk);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->p_half[t][hf]);
          }
        } else {
          // statistics only: running maximum and sum
          if (raise) {
            l *= (m_used == neg_inf()) ? 0.f : ex2_approx(m_used - m_new);
            m_used = m_new;
          }
          const float m_sub = (m_used == neg_inf()) ? 0.f : m_used;
          NB_EXP_HALF_W(0, m_sub);
          NB_EXP_HALF_W(1, m_sub);
        }
#undef NB_EXP_HALF_W
#undef NB_EXP_HALF
        l += EXTRAS ? (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]) : pair_sum(sum2[0]) + pair_sum(sum2[1]);
      }

      // ---------------------------------------------------------- epilogue
      if (ok) {
        const bool dead = !(l > 0.f);
        if (a.lse && row_ok) {
          float lse_v = (l != l) ? __int_as_float(0x7fc00000) : dead ? neg_inf() : (m_used + log2f(l)) * kLn2;
          if (XBIAS && m_used == pos_inf() && !dead) lse_v = lse_inf_rows(l);   // l = number of +Inf logits
          a.lse[i + (long long)a.Lq * h + a.lse_sb * b] = lse_v;
        }
        if (!STATS) {
          ok = mbar_wait(&bars->o_full[t], 0, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (ok) {
            tc_fence_after();
            const float inv = dead ? (a.nan_fm ? __int_as_float(0x7fc00000) : 0.f) : a.inv_keep / l;
            uint8_t* xrow = reinterpret_cast<uint8_t*>(a.x) +
                            2ll * ((long long)i * a.x_sl + (long long)b * a.x_sb + (long long)h * a.dv);
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t o[32];
              tmem_ld32(tO + c * 32, o);
              tmem_wait_ld();
              if (row_ok) {
#pragma unroll
                for (int e = 0; e < 32; e += 8) {
                  if (c * 32 + e >= a.dv) continue;   // a head narrower than the padded size: the rest is padding
                  float f[8];
#pragma unroll
                  for (int u = 0; u < 8; ++u) f[u] = dead ? inv : __uint_as_float(o[e + u]) * inv;
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
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) {
    atomicExch(&g_umma_abort, 1);
    if (a.status) atomicExch(a.status, NNLIB_B200_TIMEOUT);
  }
}

// ===========================================================================
// Scores kernel: alpha (after dropout) rebuilt from Q, K, bias, masks and the
// saved log-sum-exp.  One CTA owns 128 queries of one unit and walks over all
// key tiles; S = Q K^T is double-buffered in TMEM so the tensor core runs one
// tile ahead of the four warps that turn logits into probabilities and write
// them to the (Lkv, Lq, H, B) array (kv contiguous: each thread writes the
// 128 consecutive scores of its own query).  Bound by the HBM writes.
//   warps 0-3  epilogue (thread r owns query row r)
//   warp 4     TMA producer, TMEM allocation
//   warp 5     MMA issuer
// ===========================================================================
constexpr int kScThreads = 224;
constexpr int kStageBytes = 128 * 128;   // staging box of the TMA store: 128 queries x 64 scores (128 bytes)

template <int D, bool TST>
struct ScCfg {
  static constexpr int kChunks = D / 64;
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kStages = (D == 128) ? 2 : (TST ? 3 : 4);
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kTileBytes;
  static constexpr int kStOff = kKOff + kStages * kTileBytes;          // two staging boxes (TST only)
  static constexpr int kBarOff = kStOff + (TST ? 2 * kStageBytes : 0);
  static constexpr int kSmemBytes = kBarOff + 256 + 1024;
};

struct ScBarriers {
  uint64_t q_full;
  uint64_t k_full[4], k_empty[4];
  uint64_t s_full[2], s_empty[2];
  uint64_t stage_full[2], stage_free[2];
  uint32_t tmem_base;
  int abort_flag;
};

// write min(n, 32) scores of one query, given as 16 packed pairs (n <= 0: nothing)
template <typename T>
__device__ __forceinline__ void store_score_chunk(T* dst, const uint32_t (&pk)[16], int n) {
  if (n >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
    for (int e = 0; e < 16; e += 4)
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(dst) + e * 4) = make_uint4(pk[e], pk[e + 1], pk[e + 2], pk[e + 3]);
  } else {
    unsigned short* d16 = reinterpret_cast<unsigned short*>(dst);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      if (2 * e < n) d16[2 * e] = static_cast<unsigned short>(pk[e] & 0xffffu);
      if (2 * e + 1 < n) d16[2 * e + 1] = static_cast<unsigned short>(pk[e] >> 16);
    }
  }
}

template <int D, bool BF16, int XM, bool TST>
__global__ void __launch_bounds__(kScThreads, 2)
attn_scores_umma_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_a, const AttnArgs a, const int n_qtiles) {
  using C = ScCfg<D, TST>;
  constexpr bool EXTRAS = XM != 0;
  constexpr bool XBIAS = XM == 2;     // bias / dropout code compiled in
  using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  ScBarriers* bars = reinterpret_cast<ScBarriers*>(smem + C::kBarOff);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int unit = blockIdx.x / n_qtiles;
  const int qt = n_qtiles - 1 - (blockIdx.x % n_qtiles);
  const int h = unit % a.H, b = unit / a.H;
  const int q0 = qt * kBM;
  const int n_total = (a.Lkv + kBN - 1) / kBN;
  const int n_live = a.causal ? min(n_total, (min(a.Lkv, max(q0 + kBM + a.coff, 1)) + kBN - 1) / kBN) : n_total;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->s_empty[s], 4);
      mbar_init(&bars->stage_full[s], 4);
      mbar_init(&bars->stage_free[s], 1);
    }
    bars->abort_flag = *reinterpret_cast<volatile int*>(&g_umma_abort);
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(&bars->tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  const bool start_ok = (*abort_flag == 0);

  if (start_ok && warp == 4) {
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      mbar_arrive_expect_tx(&bars->q_full, C::kTileBytes);
      for (int c = 0; c < C::kChunks; ++c)
        tma_load_4d(smem + C::kQOff + c * kChunkBytes, &tm_q, &bars->q_full, c * 64, h, q0, b);
      bool ok = true;
      int j = 0;
      for (; j < n_live; ++j) {
        const int s = j % C::kStages;
        if (j >= C::kStages) ok = mbar_wait(&bars->k_empty[s], ((j / C::kStages) - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars->k_full[s], C::kTileBytes);
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_4d(smem + C::kKOff + s * C::kTileBytes + c * kChunkBytes, &tm_k, &bars->k_full[s],
                      c * 64, h, j * kBN, b);
      }
      if (*abort_flag) {
        mbar_wait_drain(&bars->q_full, 0, kDrainNs);
        for (int jj = max(0, j - C::kStages); jj < j; ++jj)
          mbar_wait_drain(&bars->k_full[jj % C::kStages], (jj / C::kStages) & 1, kDrainNs);
      }
    }
  } else if (start_ok && warp == 5) {
    if (lane == 0 && n_live > 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(BF16, kBM, kBN, false, false);
      const uint32_t qa = smem_u32(smem + C::kQOff);
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag);
      for (int j = 0; j < n_live && ok; ++j) {
        const int s = j % C::kStages, sb = j & 1;
        ok = mbar_wait(&bars->k_full[s], (j / C::kStages) & 1, abort_flag);
        if (ok && j >= 2) ok = mbar_wait(&bars->s_empty[sb], ((j >> 1) - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t ka = smem_u32(smem + C::kKOff + s * C::kTileBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
          umma_ss(tmem + sb * kBN, make_smem_desc_sw128(qa + off, 16, 1024), make_smem_desc_sw128(ka + off, 16, 1024),
                  idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->s_full[sb]);
        umma_commit(&bars->k_empty[s]);
      }
    }
  } else if (TST && start_ok && warp == 6) {
    // ---- store thread: each filled staging box (128 queries x 64 scores) goes out as one TMA store
    if (lane == 0) {
      prefetch_tensormap(&tm_a);
      bool ok = true;
      const int n_half = 2 * n_total;
      for (int n = 0; n < n_half && ok; ++n) {
        ok = mbar_wait(&bars->stage_full[n & 1], (n >> 1) & 1, abort_flag);
        if (!ok) break;
        tma_store_4d(&tm_a, smem + C::kStOff + (n & 1) * kStageBytes, n * 64, q0, h, b);
        tma_store_commit();
        if (n >= 1) {
          tma_store_wait_read<1>();                 // the previous box has been read out of shared memory
          mbar_arrive(&bars->stage_free[(n - 1) & 1]);
        }
      }
      tma_store_wait_read<0>();                     // shared memory must stay valid until the last read
    }
  } else if (start_ok && warp < 4) {
    const int r = warp * 32 + lane;
    const int i = q0 + r;
    const bool row_ok = i < a.Lq;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    const float c2 = a.scale * kLog2e;
    const int lim = a.causal ? min(i + a.coff, a.Lkv - 1) : a.Lkv - 1;
    const unsigned long long srow = score_row(a, row_ok ? i : 0, h, b);
    const float lse_nat = row_ok ? a.lse[i + (long long)a.Lq * h + a.lse_sb * b] : 0.f;
    // rows that need a constant instead of an exponential: nothing to attend to (NaN like the reference,
    // or 0), or a NaN among the logits (the reference's column is NaN throughout)
    const bool dead = (lse_nat == neg_inf()) || (lse_nat != lse_nat && !lse_is_inf_rows(lse_nat));
    const float lse2 = dead ? 0.f : lse_nat * kLog2e;
    const float dead_val = (a.nan_fm || lse_nat != lse_nat) ? __int_as_float(0x7fc00000) : 0.f;
    // a row whose largest logit is +Inf: equal shares on its +Inf logits (src/softmax.jl:73-75)
    const bool rinf = XBIAS && lse_is_inf_rows(lse_nat);
    const float inf_share = rinf ? 1.f / lse_inf_count(lse_nat) : 0.f;
    T* arow = reinterpret_cast<T*>(a.alpha) + ((long long)i + (long long)a.Lq * h) * a.Lkv + a.alpha_sb * b;
    RowSide rs;
    if (EXTRAS) rs = make_row_side(a, i, h, b, row_ok);
    bool okst = true;
    // 32 scores (16 packed pairs) of chunk number CH_ (4 per tile) leave the thread: either straight to
    // global memory, or into the 128B-swizzled staging box of their 64-key half (two chunks per box),
    // which the store thread ships once all four warps have filled it.
#define NB_STORE_CHUNK(CH_, PK_)                                                                   \
  do {                                                                                             \
    if (!TST) {                                                                                    \
      if (row_ok) store_score_chunk<T>(arow + (CH_) * 32, PK_, a.Lkv - (CH_) * 32);                \
    } else {                                                                                       \
      const int n_ = (CH_) >> 1;                                                                   \
      if (((CH_) & 1) == 0 && n_ >= 2) {                                                           \
        okst = mbar_wait(&bars->stage_free[n_ & 1], ((n_ >> 1) - 1) & 1, abort_flag);              \
        okst = __all_sync(0xffffffffu, okst);                                                      \
      }                                                                                            \
      if (okst) {                                                                                  \
        uint8_t* row_ = smem + C::kStOff + (n_ & 1) * kStageBytes + r * 128;                        \
        _Pragma("unroll") for (int v_ = 0; v_ < 4; ++v_) {                                         \
          const int pc_ = ((CH_) & 1) * 4 + v_;                                                    \
          *reinterpret_cast<uint4*>(row_ + ((pc_ ^ (r & 7)) << 4)) =                               \
              make_uint4(PK_[v_ * 4], PK_[v_ * 4 + 1], PK_[v_ * 4 + 2], PK_[v_ * 4 + 3]);          \
        }                                                                                          \
        if (((CH_) & 1) == 1) {                                                                    \
          fence_proxy_async_smem();                                                                \
          __syncwarp();                                                                            \
          if (lane == 0) mbar_arrive(&bars->stage_full[n_ & 1]);                                   \
        }                                                                                          \
      }                                                                                            \
    }                                                                                              \
  } while (0)

    for (int j = 0; j < n_total; ++j) {
      const int j0 = j * kBN;
      if (j < n_live) {
        const int sb = j & 1;
        uint4 bq[2][4], mq[2][2];
        if (EXTRAS) {   // bias / mask of the first 64 keys: in flight while the scores are awaited
          side_issue<XBIAS>(rs, j0, a.Lkv, bq[0], mq[0]);
          side_issue<XBIAS>(rs, j0 + 32, a.Lkv, bq[1], mq[1]);
        }
        bool ok = mbar_wait(&bars->s_full[sb], (j >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // 32 keys at a time (the next 32 scores are fetched from TMEM meanwhile):
        // logits -> probabilities -> dropout -> 64 bytes of the score row
        uint32_t sr[2][32];
        tmem_ld32(lane_base + sb * kBN, sr[0]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int jc = j0 + c * 32;
          __syncwarp();   // the previous chunk's bias / mask / store code branches per row
          tmem_wait_ld();
          if (c + 1 < 4) {
            tmem_ld32(lane_base + sb * kBN + (c + 1) * 32, sr[(c + 1) & 1]);
          } else {
            // the whole tile is in registers: the issuer may refill this buffer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->s_empty[sb]);
          }
          if (EXTRAS) {
            side_apply<XBIAS>(rs, sr[c & 1], bq[c & 1], mq[c & 1], jc, a.Lkv, lim, row_ok, c2);
            if (c + 2 < 4) side_issue<XBIAS>(rs, j0 + (c + 2) * 32, a.Lkv, bq[c & 1], mq[c & 1]);
          }
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float a0, a1;
            if (EXTRAS) {
              a0 = ex2_approx(__uint_as_float(sr[c & 1][e]) - lse2);        // -inf (masked) gives 0
              a1 = ex2_approx(__uint_as_float(sr[c & 1][e + 1]) - lse2);
              if (XBIAS && rinf) {
                a0 = (sr[c & 1][e] == 0x7f800000u) ? inf_share : 0.f;
                a1 = (sr[c & 1][e + 1] == 0x7f800000u) ? inf_share : 0.f;
              }
            } else {
              a0 = (jc + e <= lim) ? ex2_approx(fmaf(__uint_as_float(sr[c & 1][e]), c2, -lse2)) : 0.f;
              a1 = (jc + e + 1 <= lim) ? ex2_approx(fmaf(__uint_as_float(sr[c & 1][e + 1]), c2, -lse2)) : 0.f;
            }
            if (dead) { a0 = dead_val; a1 = dead_val; }
            sr[c & 1][e] = __float_as_uint(a0);
            sr[c & 1][e + 1] = __float_as_uint(a1);
          }
          if (XBIAS && a.dropout_p > 0.f) {
            const unsigned int kb = dropout_keep32(a, srow, (unsigned int)(jc >> 5));
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float al = __uint_as_float(sr[c & 1][e]);
              sr[c & 1][e] = __float_as_uint(((kb >> e) & 1u) ? al * a.inv_keep : 0.f);
            }
          }
#pragma unroll
          for (int e = 0; e < 32; e += 2)
            pk[e >> 1] = pack2<BF16>(__uint_as_float(sr[c & 1][e]), __uint_as_float(sr[c & 1][e + 1]));
          NB_STORE_CHUNK(j * 4 + c, pk);
        }
      } else if (TST || row_ok) {
        // tiles entirely above the causal diagonal
        const uint32_t z = dead ? pack2<BF16>(dead_val, dead_val) : 0u;
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) pk[e] = z;
#pragma unroll
        for (int c = 0; c < 4; ++c) NB_STORE_CHUNK(j * 4 + c, pk);
      }
      if (!okst) break;
    }
#undef NB_STORE_CHUNK
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
  if (threadIdx.x == 0 && *abort_flag) {
    atomicExch(&g_umma_abort, 1);
    if (a.status) atomicExch(a.status, NNLIB_B200_TIMEOUT);
  }
}

// ===========================================================================
// Apply kernel: x = V · alpha' for scores the caller already holds (the second
// batched_mul of NNlib.jl src/attention.jl:96-98, used when fdrop is an opaque
// callable that was applied to the materialised scores).  A plain batched GEMM
// on the tensor cores, bound by the HBM read of alpha: per (128 queries, unit)
// CTA, alpha tiles (128 queries x 128 keys, K-major: the keys are contiguous in
// the (Lkv, Lq, H, B) array) and V tiles (MN-major) stream through a ring,
// O accumulates in TMEM and is written once.
//   warps 0-3  epilogue (thread r owns query row r)
//   warp 4     TMA producer, TMEM allocation
//   warp 5     MMA issuer
// ===========================================================================
constexpr int kApThreads = 192;

template <int D>
struct ApCfg {
  static constexpr int kATile = 2 * kChunkBytes;              // 128 queries x 128 keys
  static constexpr int kVTile = (D / 64) * kChunkBytes;       // 128 keys x D features
  static constexpr int kStage = kATile + kVTile;
  static constexpr int kStages = 2;                           // two CTAs per SM keep four tiles in flight
  static constexpr int kBarOff = kStages * kStage;
  static constexpr int kSmemBytes = kBarOff + 128 + 1024;
};

struct ApBarriers {
  uint64_t full[4], empty[4], o_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <int D, bool BF16>
__global__ void __launch_bounds__(kApThreads, 2)
attn_apply_umma_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_v,
                       const AttnArgs a, const int n_qtiles) {
  using C = ApCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  ApBarriers* bars = reinterpret_cast<ApBarriers*>(smem + C::kBarOff);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit = blockIdx.x / n_qtiles, qt = blockIdx.x % n_qtiles;
  const int h = unit % a.H, b = unit / a.H;
  const int q0 = qt * kBM;
  const int n_kv = (a.Lkv + kBN - 1) / kBN;
  constexpr uint32_t kTmemCols = (D <= 64) ? 64 : 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 4; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->o_full, 1);
    bars->abort_flag = *reinterpret_cast<volatile int*>(&g_umma_abort);
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  const bool start_ok = (*abort_flag == 0);

  if (start_ok && warp == 4) {
    if (lane == 0) {
      prefetch_tensormap(&tm_a);
      prefetch_tensormap(&tm_v);
      bool ok = true;
      int j = 0;
      for (; j < n_kv; ++j) {
        const int s = j % C::kStages;
        if (j >= C::kStages) ok = mbar_wait(&bars->empty[s], ((j / C::kStages) - 1) & 1, abort_flag);
        if (!ok) break;
        uint8_t* st = smem + s * C::kStage;
        mbar_arrive_expect_tx(&bars->full[s], C::kStage);
        for (int c = 0; c < 2; ++c)
          tma_load_4d(st + c * kChunkBytes, &tm_a, &bars->full[s], j * kBN + c * 64, q0, h, b);
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(st + C::kATile + c * kChunkBytes, &tm_v, &bars->full[s], c * 64, h, j * kBN, b);
      }
      if (*abort_flag)
        for (int jj = max(0, j - C::kStages); jj < j; ++jj)
          mbar_wait_drain(&bars->full[jj % C::kStages], (jj / C::kStages) & 1, kDrainNs);
    }
  } else if (start_ok && warp == 5) {
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idesc = make_idesc_f16(BF16, kBM, D, false, true);   // A K-major, B (= V) MN-major
      constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t lbo_k = (16u >> 4) << 16;
      constexpr uint32_t lbo_v = (static_cast<uint32_t>(kChunkBytes) >> 4) << 16;
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % C::kStages;
        ok = mbar_wait(&bars->full[s], (j / C::kStages) & 1, abort_flag);
        if (!ok) break;
        const uint32_t a_lo = (smem_u32(smem + s * C::kStage) >> 4) | lbo_k;
        const uint32_t v_lo = (smem_u32(smem + s * C::kStage + C::kATile) >> 4) | lbo_v;
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
          const uint32_t aoff = (kk >> 2) * (kChunkBytes >> 4) + (kk & 3) * 2;
          umma_ss_lohi(tmem, a_lo + aoff, v_lo + kk * (2048 >> 4), desc_hi, idesc, (j == 0 && kk == 0) ? 0u : 1u);
        }
        umma_commit(&bars->empty[s]);
      }
      if (ok) umma_commit(&bars->o_full);
    }
  } else if (start_ok && warp < 4) {
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const int i = q0 + warp * 32 + lane;
    const bool row_ok = i < a.Lq;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    uint8_t* xrow = reinterpret_cast<uint8_t*>(a.x) + 2ll * ((long long)i * a.x_sl + (long long)b * a.x_sb + (long long)h * a.dv);
    bool ok = true;
    if (n_kv > 0) {
      ok = mbar_wait(&bars->o_full, 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) tc_fence_after();
    }
    if (ok) {
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (n_kv > 0) {
          tmem_ld32(lane_base + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            if (c * 32 + e >= a.dv) continue;   // a head narrower than the padded size: the rest is padding
            uint4 v;
            v.x = pack2<BF16>(__uint_as_float(o[e]), __uint_as_float(o[e + 1]));
            v.y = pack2<BF16>(__uint_as_float(o[e + 2]), __uint_as_float(o[e + 3]));
            v.z = pack2<BF16>(__uint_as_float(o[e + 4]), __uint_as_float(o[e + 5]));
            v.w = pack2<BF16>(__uint_as_float(o[e + 6]), __uint_as_float(o[e + 7]));
            *reinterpret_cast<uint4*>(xrow + (c * 32 + e) * 2) = v;
          }
        }
      }
    }
    (void)sizeof(T);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) {
    atomicExch(&g_umma_abort, 1);
    if (a.status) atomicExch(a.status, NNLIB_B200_TIMEOUT);
  }
}

// ------------------------------------------------------------------ host side
int fwd_sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      n < 1)
    n = 148;
  return n;
}

template <int D, bool BF16, int XM, bool STATS, bool BSM>
cudaError_t launch_fwd_impl(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mb,
                            const AttnArgs& a, cudaStream_t st) {
  auto kern = attn_fwd_umma_kernel<D, BF16, XM, STATS, BSM>;
  constexpr int smem = BSM ? Cfg<D>::kSmemBytesStaged : Cfg<D>::kSmemBytes;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  const int n_qblocks = (a.Lq + kQT * kBM - 1) / (kQT * kBM);
  const long long blocks = (long long)n_qblocks * a.H * a.B;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  // causal blocks differ in length: the units of the last two waves are dealt out longest blocks first
  const long long n_units = (long long)a.H * a.B;
  long long tail_units = a.causal ? 2 * ((fwd_sm_count() + n_qblocks - 1) / n_qblocks) : 0;
  if (tail_units > n_units) tail_units = n_units;
  kern<<<(unsigned)blocks, kThreads, smem, st>>>(mq, mk, mv, mb, a, n_qblocks, (int)tail_units);
  count_launch();
  return cudaGetLastError();
}

// `mb` != nullptr: the bias can be staged through shared memory by TMA (d = 64 forward with bias)
template <int D, bool BF16, int XM, bool STATS>
cudaError_t launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap* mb,
                       const AttnArgs& a, cudaStream_t st) {
  if constexpr (D == 64 && (XM % 3) == 2 && !STATS) {
    if (mb) return launch_fwd_impl<D, BF16, XM, STATS, true>(mq, mk, mv, *mb, a, st);
  }
  return launch_fwd_impl<D, BF16, XM, STATS, false>(mq, mk, mv, mq, a, st);
}

template <int D, bool BF16, int XM, bool TST>
cudaError_t launch_scores(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& ma, const AttnArgs& a,
                          cudaStream_t st) {
  auto kern = attn_scores_umma_kernel<D, BF16, XM, TST>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ScCfg<D, TST>::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int n_qtiles = (a.Lq + kBM - 1) / kBM;
  const long long blocks = (long long)n_qtiles * a.H * a.B;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  kern<<<(unsigned)blocks, kScThreads, ScCfg<D, TST>::kSmemBytes, st>>>(mq, mk, ma, a, n_qtiles);
  count_launch();
  return cudaGetLastError();
}

// Tensor map over the bias array as (Lkv, Lq, H or 1, B or 1) with 64-key x 128-query boxes, for the
// staged-bias forward.  Possible when the bias has 16-bit elements, key stride 1, query / head / batch
// strides that are multiples of 8 elements (0 = broadcast for head and batch) and a 16-byte aligned base.
bool make_bias_map(CUtensorMap* m, const AttnArgs& a) {
  static const bool disabled = [] {
    const char* e = std::getenv("NNLIB_B200_NO_STAGED_BIAS");
    return e && e[0] && e[0] != '0';
  }();
  if (disabled) return false;
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || !a.bias) return false;
  if (a.bias_dtype != NNLIB_B200_F16 && a.bias_dtype != NNLIB_B200_BF16) return false;
  if (a.bias_s[0] != 1 || !aligned16(a.bias)) return false;
  if (a.bias_s[1] <= 0 || a.bias_s[1] % 8 != 0 || a.bias_s[2] % 8 != 0 || a.bias_s[3] % 8 != 0) return false;
  const long long lim = 1ll << 39;
  if (a.bias_s[1] >= lim || a.bias_s[2] >= lim || a.bias_s[3] >= lim) return false;
  const cuuint64_t row = (cuuint64_t)a.bias_s[1] * 2;
  const cuuint64_t dims[4] = {(cuuint64_t)a.Lkv, (cuuint64_t)a.Lq, (cuuint64_t)(a.bias_s[2] ? a.H : 1),
                              (cuuint64_t)(a.bias_s[3] ? a.B : 1)};
  const cuuint64_t strides[3] = {row, a.bias_s[2] ? (cuuint64_t)a.bias_s[2] * 2 : row,
                                 a.bias_s[3] ? (cuuint64_t)a.bias_s[3] * 2 : row};
  const cuuint32_t box[4] = {64, 128, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(m, a.bias_dtype == NNLIB_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        4, const_cast<void*>(a.bias), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

// the rules of the two compiled head sizes: nullptr when the tensor-core kernels take the call, else the reason
static const char* umma_reject_reason(const AttnArgs& a, int dtype, bool need_v) {
  if (dtype != NNLIB_B200_F16 && dtype != NNLIB_B200_BF16) return "element type is not Float16 / BFloat16";
  if (!(a.d == 64 || a.d == 128)) return "head size d is not 64 or 128";
  if (need_v && a.dv != a.d) return "dv differs from d";
  if (!(a.scale > 0.f)) return "scale is not positive";
  if (a.Lq < 1 || a.Lkv < 1 || a.H < 1 || a.B < 1) return "empty problem";
  if (!aligned16(a.q) || !aligned16(a.k)) return "q or k is not 16-byte aligned";
  if (!stride_ok(a.q_sl) || !stride_ok(a.k_sl) || !stride_ok(a.q_sb) || !stride_ok(a.k_sb))
    return "a stride of q or k is not a positive multiple of 8 elements";
  if (need_v) {
    if (!aligned16(a.v) || !aligned16(a.x)) return "v or x is not 16-byte aligned";
    if (!stride_ok(a.v_sl) || !stride_ok(a.v_sb) || !stride_ok(a.x_sl) || !stride_ok(a.x_sb))
      return "a stride of v or x is not a positive multiple of 8 elements";
  }
  if (encode_tiled_fn() == nullptr) return "the driver does not export cuTensorMapEncodeTiled";
  return nullptr;
}

// The fused forward, its statistics-only form, the score-rebuild kernel and the short-sequence kernel take any
// d = dv <= 128 that is a multiple of 8, padded to 64 or 128 by the copy engine.
const char* umma_fwd_reject_reason(const AttnArgs& a, int dtype, bool need_v) {
  if (a.d == 64 || a.d == 128) return umma_reject_reason(a, dtype, need_v);
  if (a.d < 8 || a.d > 128 || a.d % 8 != 0) return "head size d is not a multiple of 8 up to 128";
  AttnArgs b = a;
  b.d = 128;                      // every other condition is that of the 64 / 128 sizes
  if (need_v) {
    if (a.dv != a.d) return "dv differs from d";
    b.dv = 128;
  }
  return umma_reject_reason(b, dtype, need_v);
}

cudaError_t umma_fwd(const AttnArgs& a, int dtype, bool stats_only, cudaStream_t st) {
  CUtensorMap mq, mk, mv;
  if (!make_head_map(&mq, a.q, dtype, a.d, a.H, a.Lq, a.B, a.q_sl, a.q_sb)) return cudaErrorInvalidValue;
  if (!make_head_map(&mk, a.k, dtype, a.d, a.H, a.Lkv, a.B, a.k_sl, a.k_sb)) return cudaErrorInvalidValue;
  if (stats_only) {
    mv = mk;
  } else if (!make_head_map(&mv, a.v, dtype, a.dv, a.H, a.Lkv, a.B, a.v_sl, a.v_sb)) {
    return cudaErrorInvalidValue;
  }
  const bool bf16 = dtype == NNLIB_B200_BF16;
  const int side = a.bias != nullptr ? 2 : (a.mask != nullptr ? 1 : 0);
  const int xm = side + ((!stats_only && a.dropout_p > 0.f) ? 3 : 0);   // the statistics ignore dropout
  CUtensorMap mbias;
  const CUtensorMap* mb = nullptr;
  if (side == 2 && !stats_only && a.d == 64 && make_bias_map(&mbias, a)) mb = &mbias;
#define NB_FWD(DD, BF, EX, ST) return launch_fwd<DD, BF, EX, ST>(mq, mk, mv, mb, a, st)
#define NB_FWD_EX(DD, BF)                                \
  do {                                                   \
    if (stats_only) {                                    \
      switch (xm) {                                      \
        case 0: NB_FWD(DD, BF, 0, true);                 \
        case 1: NB_FWD(DD, BF, 1, true);                 \
        default: NB_FWD(DD, BF, 2, true);                \
      }                                                  \
    } else {                                             \
      switch (xm) {                                      \
        case 0: NB_FWD(DD, BF, 0, false);                \
        case 1: NB_FWD(DD, BF, 1, false);                \
        case 2: NB_FWD(DD, BF, 2, false);                \
        case 3: NB_FWD(DD, BF, 3, false);                \
        case 4: NB_FWD(DD, BF, 4, false);                \
        default: NB_FWD(DD, BF, 5, false);               \
      }                                                  \
    }                                                    \
  } while (0)
#define NB_FWD_BF(DD) \
  do { if (bf16) NB_FWD_EX(DD, true); else NB_FWD_EX(DD, false); } while (0)
  if (a.d > 64) NB_FWD_BF(128); else NB_FWD_BF(64);
#undef NB_FWD_BF
#undef NB_FWD_EX
#undef NB_FWD
  return cudaErrorInvalidValue;
}

bool umma_apply_supports(const AttnArgs& a, int dtype) {
  if (dtype != NNLIB_B200_F16 && dtype != NNLIB_B200_BF16) return false;
  if (a.dv < 8 || a.dv > 128 || a.dv % 8 != 0) return false;   // padded to 64 / 128 by the copy engine
  if (a.Lq < 1 || a.Lkv < 1 || a.H < 1 || a.B < 1) return false;
  if (a.Lkv % 8 != 0 || !aligned16(a.alpha) || a.alpha_sb % 8 != 0) return false;
  if ((long long)a.Lkv * a.Lq * 2 >= (1ll << 40)) return false;
  if (!aligned16(a.v) || !aligned16(a.x) || !stride_ok(a.v_sl) || !stride_ok(a.v_sb) || !stride_ok(a.x_sl) ||
      !stride_ok(a.x_sb))
    return false;
  return encode_tiled_fn() != nullptr;
}

cudaError_t umma_apply(const AttnArgs& a, int dtype, cudaStream_t st) {
  CUtensorMap ma, mv;
  if (!make_alpha_map(&ma, a, dtype)) return cudaErrorInvalidValue;
  if (!make_head_map(&mv, a.v, dtype, a.dv, a.H, a.Lkv, a.B, a.v_sl, a.v_sb)) return cudaErrorInvalidValue;
  const int n_qtiles = (a.Lq + kBM - 1) / kBM;
  const long long blocks = (long long)n_qtiles * a.H * a.B;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  const bool bf16 = dtype == NNLIB_B200_BF16;
#define NB_AP(DD, BF)                                                                                        \
  do {                                                                                                       \
    auto kern = attn_apply_umma_kernel<DD, BF>;                                                              \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ApCfg<DD>::kSmemBytes); \
    if (e != cudaSuccess) return e;                                                                          \
    kern<<<(unsigned)blocks, kApThreads, ApCfg<DD>::kSmemBytes, st>>>(ma, mv, a, n_qtiles);                  \
  } while (0)
  if (a.dv > 64) { if (bf16) NB_AP(128, true); else NB_AP(128, false); }
  else             { if (bf16) NB_AP(64, true);  else NB_AP(64, false); }
#undef NB_AP
  count_launch();
  return cudaGetLastError();
}

cudaError_t umma_scores(const AttnArgs& a, int dtype, cudaStream_t st) {
  CUtensorMap mq, mk;
  if (!make_head_map(&mq, a.q, dtype, a.d, a.H, a.Lq, a.B, a.q_sl, a.q_sb)) return cudaErrorInvalidValue;
  if (!make_head_map(&mk, a.k, dtype, a.d, a.H, a.Lkv, a.B, a.k_sl, a.k_sb)) return cudaErrorInvalidValue;
  const bool bf16 = dtype == NNLIB_B200_BF16;
  const int xm = (a.bias != nullptr || a.dropout_p > 0.f) ? 2 : (a.mask != nullptr ? 1 : 0);
  // the staged TMA store needs 16-byte aligned score rows
  CUtensorMap ma = mq;
  const bool tst = (a.Lkv % 8 == 0) && aligned16(a.alpha) && (a.alpha_sb % 8 == 0) &&
                   ((long long)a.Lkv * a.Lq * 2 < (1ll << 40)) && make_alpha_map(&ma, a, dtype);
#define NB_SC(DD, BF, EX) \
  do { if (tst) return launch_scores<DD, BF, EX, true>(mq, mk, ma, a, st); \
       else return launch_scores<DD, BF, EX, false>(mq, mk, ma, a, st); } while (0)
#define NB_SC_EX(DD, BF) \
  do { if (xm == 2) NB_SC(DD, BF, 2); else if (xm == 1) NB_SC(DD, BF, 1); else NB_SC(DD, BF, 0); } while (0)
#define NB_SC_BF(DD) \
  do { if (bf16) NB_SC_EX(DD, true); else NB_SC_EX(DD, false); } while (0)
  if (a.d > 64) NB_SC_BF(128); else NB_SC_BF(64);
#undef NB_SC_BF
#undef NB_SC_EX
#undef NB_SC
  return cudaErrorInvalidValue;
}


// Self-test of the bounded wait: one CTA waits, with the same mbar_wait every kernel here uses, on a
// barrier that nobody ever arrives at.  The wait gives up after `limit_ns`, the CTA leaves through the
// same exit the attention kernels take (sticky device flag, optional status word) and the kernel returns
// by itself.  Nothing faults or hangs; the device stays usable.
namespace {
__global__ void wait_runout_kernel(unsigned long long limit_ns, int* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, &abort_flag, limit_ns);
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag) {
    atomicExch(&g_umma_abort, 1);
    if (status) atomicExch(status, NNLIB_B200_TIMEOUT);
  }
}
}  // namespace

cudaError_t umma_wait_runout(unsigned long long limit_ns, int* status, cudaStream_t st) {
  wait_runout_kernel<<<1, 32, 0, st>>>(limit_ns, status);
  count_launch();
  return cudaGetLastError();
}

// Reads and clears the sticky "a bounded wait ran out" flag of the current
// device.  Synchronises the stream.
cudaError_t umma_take_abort(int* out, cudaStream_t st) {
  int v = 0;
  cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyFromSymbol(&v, g_umma_abort, sizeof(int));
  if (e != cudaSuccess) return e;
  if (v) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_umma_abort, &zero, sizeof(int));
  }
  *out = v;
  return e;
}

}  // namespace nb200
