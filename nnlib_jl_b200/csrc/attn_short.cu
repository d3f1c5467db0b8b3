// x AND alpha in one pass for short key sequences (encoder-style self-attention: every query's whole score
// row fits in tensor memory).
//
// dot_product_attention returns the scores eagerly (NNlib.jl src/attention.jl:83,112-127).  The general route
// here (fused forward, then the score-rebuild kernel) computes Q K^T twice and reads q and k twice; when
// Lkv <= 512 (d = 64) or <= 256 (d = 128) one CTA can hold the 128 x Lkv score block of its 128 queries in the
// 512 TMEM columns, so the exact two-pass softmax of the reference (src/softmax.jl:69-79) needs no online
// rescaling and no log-sum-exp round trip, and every exponential is taken once:
//   warp 8     allocates tensor memory; TMA: Q, all K tiles, all V tiles (no ring: everything is resident)
//   warp 9     tcgen05.mma: S_t = Q K_t^T for every key tile, later O = sum_t P_t V_t
//   warps 0-7  two threads per query row r (TMEM lane r): warps 0-3 own the first half of the key tiles,
//              warps 4-7 the second half; the halves of a row meet through shared memory at two barriers
//                pass 1  logits -> scale, bias (src/attention.jl:129-131), masks (:133-138) -> row maximum;
//                        the prepared logits go back to their TMEM columns
//                pass 2  p = exp2(s - m), row sum, dropout (src/dropout.jl:77-87); the 16-bit probabilities
//                        are packed into the low half of their own tile's columns (chunk c of tile t moves
//                        from [128t + 32c, +32) to [128t + 16c, +16): always behind the reader)
//                pass 3  alpha' = P / l / (1-p) into 128-byte swizzled staging boxes (64 keys x 128 queries)
//                epilogue x = O / l / (1-p), each half writing half of the features
//   warp 10    ships every filled staging box with one cp.async.bulk.tensor store into the (Lkv, Lq, H, B) array
//   warp 11    a mask array that does not depend on the query: its bytes -> keep bits, one item ahead
// Without bias and dropout one CTA per SM walks over the work items, and the loads of the next item run under the
// passes of the current one (the bias / dropout variants have no registers to spare for the walk).
// O lives in columns the packing freed (d = 64: the upper half of tile 0) or behind the scores (d = 128).
// Bound by the HBM write of alpha.
#include <cuda.h>

#include "common.cuh"
#include "extras.cuh"
#include "launchers.h"
#include "umma.cuh"
#include "umma_shared.cuh"

namespace nb200 {

__device__ int g_short_abort = 0;  // sticky: a bounded wait of this kernel ran out

namespace {

constexpr int kShThreads = 384;
constexpr int kShStageBytes = 128 * 128;   // staging box of the TMA store: 128 queries x 64 scores

template <int D>
struct ShCfg {
  static constexpr int kMaxTiles = (D == 64) ? 4 : 2;          // key tiles of 128 the CTA can hold
  static constexpr int kTilesPerPart = kMaxTiles / 2;          // key tiles of one half of the softmax warps
  static constexpr int kChunks = D / 64;
  static constexpr int kTileBytes = kChunks * kChunkBytes;     // 128 rows x D features
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kTileBytes;
  static constexpr int kVOff = kKOff + kMaxTiles * kTileBytes;
  static constexpr int kStOff = kVOff + kMaxTiles * kTileBytes;   // 2 halves x 2 staging boxes
  static constexpr int kBarOff = kStOff + 4 * kShStageBytes;
  // A CTA may walk over several work items and load the next item's Q, K, V while the current one is in its
  // passes; nothing of one item may then share memory with the operands of the next.
  // Row maxima and sums of the two halves, [2 halves][128 rows] each.  d = 128 fills shared memory but for 1.5 KB:
  // there the sums take the place of the maxima (a barrier of the softmax threads lies between the last read of
  // one and the first write of the other).
  static constexpr int kXOff = kBarOff + 512;
  static constexpr int kXSum = (D == 64) ? 256 : 0;              // where the sums start, in floats
  static constexpr int kXBytes = (D == 64) ? 2048 : 1024;
  // Keep bits of a mask array that depends on the query, [chunk of 32 keys][query row].  d = 64: an area of their
  // own.  d = 128: in the staging boxes, which pass 3 is the first to fill (every thread is through pass 1, the
  // last reader of the bits, by then) — such a call is launched with one work item per CTA, since the boxes of
  // one item are still being read when the bits of the next would be written.
  static constexpr bool kKeepOwn = (D == 64);
  static constexpr int kKeepOff = kKeepOwn ? kXOff + kXBytes : kStOff;
  static constexpr int kSmemBytes = kXOff + kXBytes + (kKeepOwn ? kMaxTiles * 4 * 128 * 4 : 0) + 1024;
  static constexpr int kTmemCols = 512;
  static constexpr int kOCol = (D == 64) ? 64 : 256;
};
static_assert(ShCfg<64>::kSmemBytes <= 232448 && ShCfg<128>::kSmemBytes <= 232448, "shared memory budget");

struct ShBarriers {
  uint64_t qk_full, v_full, s_full[2], p_ready, o_full, p_free, tmem_free;
  uint64_t stage_full[2][2], stage_free[2][2];
  uint64_t bits_full[2], bits_free[2];   // keep bits of a row-invariant mask: two slots, used by alternate items
  uint32_t maskbits[2][16];              // [slot][chunk of 32 keys]
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(ShBarriers) <= 512, "barrier block");

// d = a * b + c and d = a * b on pairs of 16-bit values, in the arrays' own type
template <bool BF16>
__device__ __forceinline__ uint32_t fma16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  if (BF16) asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  else asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
template <bool BF16>
__device__ __forceinline__ uint32_t mul16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  if (BF16) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  else asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// all 256 softmax threads (and nobody else)
__device__ __forceinline__ void softmax_threads_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// the same barrier, which also tells every thread whether any of them brought `flag`
__device__ __forceinline__ bool softmax_threads_sync_any(bool flag) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.or.pred q, 1, 256, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t"
      "}"
      : "=r"(r)
      : "r"(flag ? 1u : 0u)
      : "memory");
  return r != 0;
}

// XM = side + 3*drop as in the fused forward (attn_umma.cu): side 0 = no side input (optionally causal),
// 1 = Bool mask array, 2 = bias (and mask); drop: dropout code compiled in.  The passes are bound by
// instruction issue, so what a call does not use must not be in its loop.
template <int D, bool BF16, int XM>
__global__ void __launch_bounds__(kShThreads, 1)
attn_short_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_a, const AttnArgs a,
                  const int n_qtiles, const int n_work) {
  using C = ShCfg<D>;
  constexpr int TPP = C::kTilesPerPart;
  constexpr bool EXTRAS = (XM % 3) != 0;
  constexpr bool XBIAS = (XM % 3) == 2;
  constexpr bool DROP = XM >= 3;
  constexpr bool MASK_ONLY = EXTRAS && !XBIAS;
  // The walk over several items costs registers; the bias and dropout variants have none to spare and take one
  // item per CTA.
  constexpr bool LOOP = XM < 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  ShBarriers* bars = reinterpret_cast<ShBarriers*>(smem + C::kBarOff);
  // [2 (max, sum)][2 halves][128 rows]; written only after ALL scores are complete, i.e. after the last read of K
  float* xstat = reinterpret_cast<float*>(smem + C::kXOff);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Work item w = (128 queries, head, batch element).  This CTA takes items blockIdx.x, blockIdx.x + gridDim.x, ...;
  // every role walks over them in the same order, `it` counting them, and every barrier completes one phase per
  // item (the staging-box barriers: one per box), so a waiter is never more than one phase behind.
  const int n_total = (a.Lkv + kBN - 1) / kBN;                 // <= kMaxTiles (the host checked)
  // A mask that does not depend on the query (key padding): one warp turns the mask bytes of the next item into
  // bits while the current item is in its passes, instead of every thread fetching the same bytes for its own row.
  // (A call without a mask array that runs this variant counts as one with an all-true mask.)
  const bool rowinv = MASK_ONLY && (a.mask == nullptr || a.mask_s[1] == 0);
  struct Work { int h, b, q0, n_live; };
  auto work_of = [&](int w) {
    Work k;
    const int unit = w / n_qtiles;
    k.h = unit % a.H;
    k.b = unit / a.H;
    k.q0 = (n_qtiles - 1 - (w % n_qtiles)) * kBM;
    k.n_live = a.causal ? min(n_total, (min(a.Lkv, max(k.q0 + kBM + a.coff, 1)) + kBN - 1) / kBN) : n_total;
    return k;
  };

  if (threadIdx.x == 0) {
    mbar_init(&bars->qk_full, 1);
    mbar_init(&bars->v_full, 1);
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->p_ready, 8);
    mbar_init(&bars->o_full, 1);
    mbar_init(&bars->p_free, 8);
    mbar_init(&bars->tmem_free, 8);
    for (int p = 0; p < 2; ++p) {
      mbar_init(&bars->bits_full[p], 1);
      mbar_init(&bars->bits_free[p], 8);
    }
    for (int p = 0; p < 2; ++p)
      for (int s = 0; s < 2; ++s) {
        mbar_init(&bars->stage_full[p][s], 4);
        mbar_init(&bars->stage_free[p][s], 1);
      }
    bars->abort_flag = *reinterpret_cast<volatile int*>(&g_short_abort);
    fence_mbar_init();
  }
  if (warp == 8) {
    tmem_alloc(&bars->tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  const bool start_ok = (*abort_flag == 0);

  if (start_ok && warp == 8) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      int n_qk = 0, n_v = 0;                         // loads issued so far
      bool ok = true;
      for (int it = 0, w = blockIdx.x; (LOOP ? w < n_work : it < 1) && ok; w += gridDim.x, ++it) {
        const Work wk = work_of(w);
        // Q and K of the previous item have been read by its last score product (tile 0's: see the issuer)
        if (it > 0) ok = mbar_wait(&bars->s_full[0], (it - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars->qk_full, (1 + wk.n_live) * C::kTileBytes);
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_4d(smem + C::kQOff + c * kChunkBytes, &tm_q, &bars->qk_full, c * 64, wk.h, wk.q0, wk.b);
        for (int t = 0; t < wk.n_live; ++t)
          for (int c = 0; c < C::kChunks; ++c)
            tma_load_4d(smem + C::kKOff + t * C::kTileBytes + c * kChunkBytes, &tm_k, &bars->qk_full, c * 64, wk.h,
                        t * kBN, wk.b);
        ++n_qk;
        // V's memory of the previous item: read by its last P V product, then used by the epilogue to stage x
        if (it > 0) ok = mbar_wait(&bars->tmem_free, (it - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars->v_full, wk.n_live * C::kTileBytes);
        for (int t = 0; t < wk.n_live; ++t)
          for (int c = 0; c < C::kChunks; ++c)
            tma_load_4d(smem + C::kVOff + t * C::kTileBytes + c * kChunkBytes, &tm_v, &bars->v_full, c * 64, wk.h,
                        t * kBN, wk.b);
        ++n_v;
      }
      // the copies land whatever happens to the rest of the CTA: wait for the last ones on the way out of an abort
      // (the earlier ones were waited for by the products that freed their buffers)
      if (n_qk > 0 && !mbar_wait(&bars->qk_full, (n_qk - 1) & 1, abort_flag))
        mbar_wait_drain(&bars->qk_full, (n_qk - 1) & 1, kDrainNs);
      if (n_v > 0 && !mbar_wait(&bars->v_full, (n_v - 1) & 1, abort_flag))
        mbar_wait_drain(&bars->v_full, (n_v - 1) & 1, kDrainNs);
    }
  } else if (start_ok && warp == 9) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(BF16, kBM, kBN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(BF16, kBM, D, false, true);
      const uint32_t qa = smem_u32(smem + C::kQOff);
      bool ok = true;
      for (int it = 0, w = blockIdx.x; (LOOP ? w < n_work : it < 1) && ok; w += gridDim.x, ++it) {
        const int n_live = work_of(w).n_live;
        const uint32_t ph = it & 1;
        ok = mbar_wait(&bars->qk_full, ph, abort_flag);
        // Order of the score tiles: every tile but the first as soon as each softmax warp has fetched the previous
        // item's probabilities (pass 3), the first — O shares or neighbours its columns — once the warps have read
        // O as well.  The second half's scores are complete first.
        if (ok && it > 0) ok = mbar_wait(&bars->p_free, (it - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        auto scores = [&](int t) {
          if (t < n_live) {
            const uint32_t ka = smem_u32(smem + C::kKOff + t * C::kTileBytes);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t off = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
              umma_ss(tmem + t * kBN, make_smem_desc_sw128(qa + off, 16, 1024), make_smem_desc_sw128(ka + off, 16, 1024),
                      idesc_qk, kk > 0 ? 1u : 0u);
            }
          }
        };
        for (int t = TPP; t < C::kMaxTiles; ++t) scores(t);
        umma_commit(&bars->s_full[1]);                  // the scores of the second half of the warps
        for (int t = 1; t < TPP; ++t) scores(t);
        if (it > 0) ok = mbar_wait(&bars->tmem_free, (it - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        scores(0);
        umma_commit(&bars->s_full[0]);                  // the scores of the first half: the last product of Q and K
        // every row's probabilities are packed (and every score column has been read): O may be written
        ok = mbar_wait(&bars->p_ready, ph, abort_flag);
        if (ok) ok = mbar_wait(&bars->v_full, ph, abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int t = 0; t < n_live; ++t) {
          const uint32_t va = smem_u32(smem + C::kVOff + t * C::kTileBytes);
#pragma unroll
          for (int kk = 0; kk < kBN / 16; ++kk)
            umma_ts(tmem + C::kOCol, tmem + t * kBN + kk * 8, make_smem_desc_sw128(va + kk * 2048, kChunkBytes, 1024),
                    idesc_pv, (t > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bars->o_full);
      }
    }
  } else if (start_ok && warp == 10) {
    // ---- store thread: each filled staging box (128 queries x 64 scores) goes out as one TMA store.  The two
    // halves of the softmax warps fill their k-th boxes at about the same time: both are sent, then handed back
    // the moment the copy engine has read them (the softmax warps fill the other two boxes meanwhile).
    if (lane == 0) {
      prefetch_tensormap(&tm_a);
      bool ok = true;
      const int n_box = 2 * n_total;                  // boxes of 64 keys per item; half p owns [2 TPP p, 2 TPP (p + 1))
      const int n0 = min(n_box, 2 * TPP), n1 = n_box - n0;
      int cb0 = 0, cb1 = 0;                           // boxes of each half so far, over all items
      for (int it = 0, w = blockIdx.x; (LOOP ? w < n_work : it < 1) && ok; w += gridDim.x, ++it) {
        const Work wk = work_of(w);
        for (int k = 0; k < n0 && ok; ++k) {
          ok = mbar_wait(&bars->stage_full[0][cb0 & 1], (cb0 >> 1) & 1, abort_flag);
          if (!ok) break;
          tma_store_4d(&tm_a, smem + C::kStOff + (cb0 & 1) * kShStageBytes, k * 64, wk.q0, wk.h, wk.b);
          tma_store_commit();
          const bool second = k < n1;
          if (second) {
            ok = mbar_wait(&bars->stage_full[1][cb1 & 1], (cb1 >> 1) & 1, abort_flag);
            if (ok) {
              tma_store_4d(&tm_a, smem + C::kStOff + (2 + (cb1 & 1)) * kShStageBytes, (2 * TPP + k) * 64, wk.q0, wk.h,
                           wk.b);
              tma_store_commit();
            }
          }
          tma_store_wait_read<0>();                   // also keeps shared memory valid until the last read
          mbar_arrive(&bars->stage_free[0][cb0 & 1]);
          ++cb0;
          if (second && ok) {
            mbar_arrive(&bars->stage_free[1][cb1 & 1]);
            ++cb1;
          }
        }
      }
    }
  } else if (start_ok && warp == 11) {
    // ---- mask warp: lane c gathers the keep bits of keys [32 c, 32 c + 32) of the item's (head, batch element)
    if (rowinv) {
      bool ok = true;
      for (int it = 0, w = blockIdx.x; (LOOP ? w < n_work : it < 1) && ok; w += gridDim.x, ++it) {
        const Work wk = work_of(w);
        const int slot = it & 1;
        // the slot's previous user (two items back) is through its pass 1
        if (it >= 2) ok = mbar_wait_warp(&bars->bits_free[slot], ((it >> 1) - 1) & 1, abort_flag);
        if (!ok) break;
        if (lane < n_total * 4) {
          const unsigned char* mrow = a.mask + (long long)wk.h * a.mask_s[2] + (long long)wk.b * a.mask_s[3];
          const int jj0 = lane * 32;
          unsigned int bits = 0u;
          if (a.mask == nullptr) {
            bits = 0xffffffffu;
          } else if (a.mask_s[0] == 1 && (reinterpret_cast<unsigned long long>(mrow) & 15ull) == 0 && jj0 + 32 <= a.Lkv) {
            const uint4* p = reinterpret_cast<const uint4*>(mrow + jj0);
            bits = mask_word_bits(__ldg(p), __ldg(p + 1));
          } else {
            for (int e = 0; e < 32; ++e)
              if (jj0 + e < a.Lkv && mrow[(long long)(jj0 + e) * a.mask_s[0]] != 0) bits |= 1u << e;
          }
          bars->maskbits[slot][lane] = bits;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->bits_full[slot]);
      }
    }
  } else if (start_ok && warp < 8) {
    // ----------------------------------------------------------- softmax warps
    const int part = warp >> 2;                       // which half of the key tiles
    const int r = (warp & 3) * 32 + lane;             // row inside the tile = TMEM lane
    const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const float c2 = a.scale * kLog2e;
    // with a bias the prepared logits are already scaled; otherwise (plain, or a mask array only) the scores stay
    // raw and get scale*log2(e) inside the exponential's FMA
    const float cs = XBIAS ? 1.f : c2;
    const int t_first = part * TPP;
    int cb = 0;                                       // staging boxes of this half so far, over all items
#pragma unroll 1
    for (int it = 0, w = blockIdx.x; LOOP ? w < n_work : it < 1; w += gridDim.x, ++it) {
      const Work wk = work_of(w);
      const int h = wk.h, b = wk.b, q0 = wk.q0, n_live = wk.n_live;
      const uint32_t ph = it & 1;                       // phase of the once-per-item barriers
      const int i = q0 + r;
      const bool row_ok = i < a.Lq;
      const int lim = a.causal ? min(i + a.coff, a.Lkv - 1) : a.Lkv - 1;   // last key this row attends to (< 0: none)
      const unsigned long long srow = score_row(a, row_ok ? i : 0, h, b);
      RowSide rs;
      if (EXTRAS) rs = make_row_side(a, i, h, b, row_ok);
      const int t_end = min(n_live, t_first + TPP);     // this thread's live tiles: [t_first, t_end)

      // Every softmax thread goes through both exchange barriers of an item whatever happens, and all of them leave
      // the walk together (the second barrier tells each whether any wait ran out), so that a wait that ran out in
      // one warp cannot leave the others at a barrier; the results of an aborted CTA are discarded anyway.
      // A mask array without a bias: the keep bits of this thread's chunks are gathered while the loads and the
      // score products are under way (the softmax threads have nothing to do until then), so that pass 1 has no
      // global load in it.  Each thread reads back only what it wrote itself.
      uint32_t* keepbits = reinterpret_cast<uint32_t*>(smem + C::kKeepOff);
      if (MASK_ONLY && !rowinv) {
        // all the 16-byte loads first, so that their latencies overlap
        uint4 mw[TPP * 4][2];
        const bool vec = rs.mask_row != nullptr && rs.mask_vec;
#pragma unroll
        for (int c = 0; c < TPP * 4; ++c) {
          const int g = t_first * 4 + c;
          const bool in = vec && g < t_end * 4 && g * 32 + 32 <= a.Lkv;
          const uint4* p = reinterpret_cast<const uint4*>(rs.mask_row + (in ? g * 32 : 0));
          mw[c][0] = in ? __ldg(p) : make_uint4(0u, 0u, 0u, 0u);
          mw[c][1] = in ? __ldg(p + 1) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int c = 0; c < TPP * 4; ++c) {
          const int g = t_first * 4 + c;
          if (g >= t_end * 4) continue;
          const unsigned int range = range_keep_bits(g * 32, lim, row_ok);
          const bool in = vec && g * 32 + 32 <= a.Lkv;
          keepbits[g * 128 + r] = in ? (range & mask_word_bits(mw[c][0], mw[c][1])) : mask_keep_bits_bytes(rs, g * 32, range);
        }
      }
      bool okb = true;
      if (rowinv) okb = mbar_wait_warp(&bars->bits_full[it & 1], (it >> 1) & 1, abort_flag);
      bool ok = mbar_wait_warp(&bars->s_full[part], ph, abort_flag);
      ok = ok && okb;
      float m = neg_inf();
      if (ok && t_end > t_first) {
        tc_fence_after();
        // ---- pass 1: prepared logits (scaled base 2, bias added, masked keys -inf) and the row maximum
        // Two chunks per turn: the bias words of the next chunk and its scores (the other register buffer) are in
        // flight while one chunk is worked on.
        uint4 bq0[4], bq1[4], mq0[2], mq1[2];
        uint32_t s0[32], s1[32];
        auto prepare = [&](int g, uint32_t (&s)[32], const uint4 (&bq)[4], const uint4 (&mq)[2]) {
          if (XBIAS) {
            side_apply<true>(rs, s, bq, mq, g * 32, a.Lkv, lim, row_ok, c2);
          } else {
            // keep bits of the chunk: the row's range (the causal diagonal, the end of the keys), and the mask array
            unsigned int kb;
            if (!EXTRAS) kb = range_keep_bits(g * 32, lim, true);
            else if (rowinv) kb = range_keep_bits(g * 32, lim, row_ok) & bars->maskbits[it & 1][g];
            else kb = keepbits[g * 128 + r];
            if (!__any_sync(0xffffffffu, kb != 0xffffffffu)) {
              // every key of the chunk is kept for every row of the warp: the raw scores stay where they are
#pragma unroll
              for (int e = 0; e < 32; e += 2) m = max3(m, __uint_as_float(s[e]), __uint_as_float(s[e + 1]));
              return;
            }
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (!((kb >> e) & 1u)) s[e] = 0xff800000u;
          }
#pragma unroll
          for (int e = 0; e < 32; e += 2) m = max3(m, __uint_as_float(s[e]), __uint_as_float(s[e + 1]));
          __syncwarp();                     // the code above branches per row
          tmem_st32(lane_base + g * 32, s);
        };
        const int g_end = t_end * 4;
        if (XBIAS) side_issue<true>(rs, t_first * kBN, a.Lkv, bq0, mq0);
        tmem_ld32(lane_base + t_first * kBN, s0);
#pragma unroll 1
        for (int g = t_first * 4; g < g_end; g += 2) {
          if (XBIAS) side_issue<true>(rs, (g + 1) * 32, a.Lkv, bq1, mq1);
          tmem_wait_ld();
          tmem_ld32(lane_base + (g + 1) * 32, s1);
          prepare(g, s0, bq0, mq0);
          if (XBIAS && g + 2 < g_end) side_issue<true>(rs, (g + 2) * 32, a.Lkv, bq0, mq0);
          tmem_wait_ld();
          if (g + 2 < g_end) tmem_ld32(lane_base + (g + 2) * 32, s0);
          prepare(g + 1, s1, bq1, mq1);
        }
        tmem_wait_st();
      }
      if (rowinv) {                                     // this warp is done with the slot of mask bits
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->bits_free[it & 1]);
      }
      xstat[part * 128 + r] = m * cs;                   // in scaled base-2 units from here on (scale > 0)
      softmax_threads_sync();
      m = fmaxf(xstat[r], xstat[128 + r]);              // fmaxf drops a NaN: a NaN logit shows up in the sum instead

      float l = 0.f;
      if (ok && t_end > t_first) {
        // ---- pass 2: exponentials, row sum, dropout, packed probabilities
        const bool row_inf = XBIAS && (m == pos_inf());  // a +Inf bias: equal shares on the +Inf keys (src/softmax.jl:73-75)
        const float m_neg = (m == neg_inf()) ? 0.f : -m;
        const unsigned long long cs2 = pair_of(cs), mneg2 = pair_of(m_neg);
        uint32_t s0[32], s1[32];
        auto exps = [&](int g, const uint32_t (&s)[32]) {
          unsigned int kb = 0xffffffffu;
          if (DROP) kb = dropout_keep32(a, srow, (unsigned int)g);
          uint32_t pk[16];
          float sum0 = 0.f, sum1 = 0.f;
          unsigned long long sum2[2] = {0ull, 0ull};
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float p0, p1;
            if (XBIAS) {
              p0 = ex2_approx(fmaf(__uint_as_float(s[e]), cs, m_neg));
              p1 = ex2_approx(fmaf(__uint_as_float(s[e + 1]), cs, m_neg));
              if (row_inf) {
                p0 = (s[e] == 0x7f800000u) ? 1.f : 0.f;
                p1 = (s[e + 1] == 0x7f800000u) ? 1.f : 0.f;
              }
              sum0 += p0;                   // dropout follows the softmax: the row sum keeps the dropped scores
              sum1 += p1;
            } else {
              // two logits per instruction (packed fp32): scale and subtract the maximum, add to the row sum
              float x0, x1;
              fma2(x0, x1, __uint_as_float(s[e]), __uint_as_float(s[e + 1]), cs2, mneg2);
              p0 = ex2_approx(x0);
              p1 = ex2_approx(x1);
              add2(sum2[(e >> 1) & 1], p0, p1);
            }
            pk[e >> 1] = pack2<BF16>(p0, p1);
            if (DROP) pk[e >> 1] &= (((kb >> e) & 1u) ? 0x0000ffffu : 0u) | (((kb >> (e + 1)) & 1u) ? 0xffff0000u : 0u);
          }
          l += XBIAS ? sum0 + sum1 : pair_sum(sum2[0]) + pair_sum(sum2[1]);
          tmem_st16(lane_base + (g >> 2) * kBN + (g & 3) * 16, pk);   // chunk c of tile t -> [128 t + 16 c, +16)
        };
        // the next chunk's scores are fetched while one chunk is turned into probabilities; the packed
        // probabilities of chunk g land in columns chunk g / 2 of the same tile has already left
        const int g_end = t_end * 4;
        tmem_ld32(lane_base + t_first * kBN, s0);
#pragma unroll 1
        for (int g = t_first * 4; g < g_end; g += 2) {
          tmem_wait_ld();
          tmem_ld32(lane_base + (g + 1) * 32, s1);
          exps(g, s0);
          tmem_wait_ld();
          if (g + 2 < g_end) tmem_ld32(lane_base + (g + 2) * 32, s0);
          exps(g + 1, s1);
        }
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&bars->p_ready);
      if (C::kXSum == 0) softmax_threads_sync();        // every thread has read the maxima the sums overwrite
      xstat[C::kXSum + part * 128 + r] = l;
      if (softmax_threads_sync_any(!ok || *abort_flag != 0)) break;
      l = xstat[C::kXSum + r] + xstat[C::kXSum + 128 + r];

      // ---- pass 3: alpha' = P / l / (1-p), box by box
      if (ok) {
        const bool dead = !(l > 0.f);
        const float nanv = __int_as_float(0x7fc00000);
        const float scale = dead ? 0.f : a.inv_keep / l;
        const float dead_val = (a.nan_fm || l != l) ? nanv : 0.f;
        // alpha' = P * scale in the arrays' own 16-bit arithmetic: the scale as a leading 16-bit value plus a 16-bit
        // remainder, so that the result is P * scale to within its final rounding (the remainder's rounding error
        // is 2^-8 of a term that is itself 2^-8 of the result)
        const uint32_t scale_hi2 = pack2<BF16>(scale, scale);
        float scale_hi;
        if (BF16) {
          scale_hi = __uint_as_float(scale_hi2 << 16);
        } else {
          scale_hi = __half2float(__ushort_as_half(static_cast<unsigned short>(scale_hi2 & 0xffffu)));
        }
        const uint32_t scale_lo2 = pack2<BF16>(scale - scale_hi, scale - scale_hi);
        if (part == 0 && a.lse && row_ok) {
          float lse_v = (l != l) ? nanv : dead ? neg_inf() : (m + log2f(l)) * kLn2;
          if (m == pos_inf() && !dead) lse_v = lse_inf_rows(l);
          a.lse[i + (long long)a.Lq * h + a.lse_sb * b] = lse_v;
        }
        const int n_first = 2 * TPP * part;
        const int n_mine = max(0, min(2 * n_total, 2 * TPP * (part + 1)) - n_first);
        const bool any_dead = __any_sync(0xffffffffu, dead);
        bool okst = true;
        // packed probabilities of box n (keys [64 n, 64 n + 64)) of this row: fetched one box ahead
        auto fetch = [&](int n, uint32_t (&pk)[32]) {
          if (n < 2 * n_live) tmem_ld32(lane_base + (n >> 1) * kBN + (n & 1) * 32, pk);
        };
        auto emit = [&](int k, uint32_t (&pk)[32]) {
          const int n = n_first + k;
          if (n < 2 * n_live) {
            // two scores per instruction: P * scale_hi + (P * scale_lo), rounded once by the fused multiply-add
#pragma unroll
            for (int e = 0; e < 32; ++e) pk[e] = fma16x2<BF16>(pk[e], scale_hi2, mul16x2<BF16>(pk[e], scale_lo2));
            if (any_dead) {                 // rows with nothing to attend to (or a NaN logit): a constant
              const uint32_t z = pack2<BF16>(dead_val, dead_val);
#pragma unroll
              for (int e = 0; e < 32; ++e)
                if (dead) pk[e] = z;
            }
          } else {
            // key tiles entirely above the causal diagonal
            const uint32_t z = dead ? pack2<BF16>(dead_val, dead_val) : 0u;
#pragma unroll
            for (int e = 0; e < 32; ++e) pk[e] = z;
          }
          const int ck = cb + k;            // box number over all items: slot ck & 1, its use number ck >> 1
          if (ck >= 2) {
            okst = mbar_wait_warp(&bars->stage_free[part][ck & 1], ((ck >> 1) - 1) & 1, abort_flag);
            if (!okst) return;
          }
          uint8_t* row = smem + C::kStOff + (part * 2 + (ck & 1)) * kShStageBytes + r * 128;
#pragma unroll
          for (int v = 0; v < 8; ++v)
            *reinterpret_cast<uint4*>(row + ((v ^ (r & 7)) << 4)) =
                make_uint4(pk[v * 4], pk[v * 4 + 1], pk[v * 4 + 2], pk[v * 4 + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->stage_full[part][ck & 1]);
        };
        uint32_t pk0[32], pk1[32];
        if (n_mine > 0) fetch(n_first, pk0);
#pragma unroll 1
        for (int k = 0; k < n_mine && okst; k += 2) {
          tmem_wait_ld();
          if (k + 1 < n_mine) fetch(n_first + k + 1, pk1);
          emit(k, pk0);
          if (!okst || k + 1 >= n_mine) break;
          tmem_wait_ld();
          if (k + 2 < n_mine) fetch(n_first + k + 2, pk0);
          emit(k + 1, pk1);
        }

        // this warp has fetched all its probabilities: the issuer may overwrite their columns with the next scores
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_free);

        // ---- epilogue: x = O / l / (1-p); each half of the warps handles half of the features.  A thread owns a
        // row, and rows lie far apart in x: the rows go through shared memory (V's, which the last P V product has
        // finished with; swizzled against bank conflicts) so that a warp writes whole runs of a row's features
        // instead of 32 scattered 16-byte pieces per instruction.  A warp reads back only what it wrote itself.
        if (okst) {
          ok = mbar_wait_warp(&bars->o_full, ph, abort_flag);
          if (ok) {
            tc_fence_after();
            constexpr int PPR = D / 16;               // 16-byte pieces of a row per half of the warps
            uint8_t* xst = smem + C::kVOff;           // [128 rows][D features], 16-byte pieces XOR-swizzled by row
#pragma unroll
            for (int cc = 0; cc < D / 64; ++cc) {
              const int c = part * (D / 64) + cc;     // 32-column chunk of O
              uint32_t o[32];
              tmem_ld32(lane_base + C::kOCol + c * 32, o);
              tmem_wait_ld();
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
                const int piece = c * 4 + (e >> 3);
                *reinterpret_cast<uint4*>(xst + r * (D * 2) + ((piece ^ (r & 7)) << 4)) = v;
              }
            }
            __syncwarp();
            const int pc = part * PPR + (lane % PPR);   // this lane's piece of a row
#pragma unroll
            for (int g = 0; g < PPR; ++g) {
              const int rr = (warp & 3) * 32 + g * (32 / PPR) + lane / PPR;
              const uint4 v = *reinterpret_cast<const uint4*>(xst + rr * (D * 2) + ((pc ^ (rr & 7)) << 4));
              if (q0 + rr < a.Lq && pc * 8 < a.dv)      // rows beyond Lq; a head narrower than the padded size
                *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.x) +
                                          2ll * ((long long)(q0 + rr) * a.x_sl + (long long)b * a.x_sb +
                                                 (long long)h * a.dv + pc * 8)) = v;
            }
            fence_proxy_async_smem();                   // the next item's V is written by the copy engine
          }
        }
      }
      cb += max(0, min(2 * n_total, 2 * TPP * (part + 1)) - 2 * TPP * part);   // the boxes of this half per item
      // this warp has read everything it needs out of tensor memory: the next item's scores may overwrite it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_free);
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) {
    atomicExch(&g_short_abort, 1);
    if (a.status) atomicExch(a.status, NNLIB_B200_TIMEOUT);
  }
}

int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      n < 1)
    n = 148;
  return n;
}

template <int D, bool BF16, int XM>
cudaError_t launch_short(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& ma,
                         const AttnArgs& a, cudaStream_t st) {
  auto kern = attn_short_kernel<D, BF16, XM>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ShCfg<D>::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int n_qtiles = (a.Lq + kBM - 1) / kBM;
  const long long n_work = (long long)n_qtiles * a.H * a.B;
  if (n_work > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  // without bias and dropout one CTA per SM walks over the work items (XM < 2, as LOOP in the kernel), unless the
  // keep bits of a query-dependent mask have no area of their own; otherwise one item per CTA
  const bool loop = XM < 2 && (ShCfg<D>::kKeepOwn || a.mask == nullptr || a.mask_s[1] == 0);
  long long blocks = loop ? (n_work < sm_count() ? n_work : sm_count()) : n_work;
  // Causal tiles of a unit differ in length, and a CTA takes items blockIdx.x, + gridDim.x, ...: with a grid that
  // shares a factor with the tiles per unit it would meet the same tiles (always the long ones, or always the
  // short ones) in every unit.  A grid coprime to the tiles per unit walks through all of them in turn.
  if (loop && a.causal && blocks < n_work && n_qtiles > 1) {
    auto gcd = [](long long x, long long y) { while (y) { const long long t = x % y; x = y; y = t; } return x; };
    while (blocks > 1 && gcd(blocks, n_qtiles) != 1) --blocks;
  }
  kern<<<(unsigned)blocks, kShThreads, ShCfg<D>::kSmemBytes, st>>>(mq, mk, mv, ma, a, n_qtiles, (int)n_work);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

// x and alpha together for a short key sequence: the fused forward's shapes (16-bit, d = dv <= 128 a multiple of 8,
// 16-byte aligned rows), every key of a query within one CTA's tensor memory, and score rows the TMA store
// can address.
bool short_supports(const AttnArgs& a, int dtype) {
  if (umma_fwd_reject_reason(a, dtype, true) != nullptr) return false;   // any d = dv <= 128 that is a multiple of 8
  const int max_keys = (a.d <= 64) ? 512 : 256;
  if (a.Lkv > max_keys) return false;
  if (!a.alpha || a.Lkv % 8 != 0 || !aligned16(a.alpha) || a.alpha_sb % 8 != 0) return false;
  return true;
}

cudaError_t short_attention(const AttnArgs& a, int dtype, cudaStream_t st) {
  CUtensorMap mq, mk, mv, ma;
  if (!make_head_map(&mq, a.q, dtype, a.d, a.H, a.Lq, a.B, a.q_sl, a.q_sb)) return cudaErrorInvalidValue;
  if (!make_head_map(&mk, a.k, dtype, a.d, a.H, a.Lkv, a.B, a.k_sl, a.k_sb)) return cudaErrorInvalidValue;
  if (!make_head_map(&mv, a.v, dtype, a.d, a.H, a.Lkv, a.B, a.v_sl, a.v_sb)) return cudaErrorInvalidValue;
  if (!make_alpha_map(&ma, a, dtype)) return cudaErrorInvalidValue;
  const bool bf16 = dtype == NNLIB_B200_BF16;
  const int side = a.bias != nullptr ? 2 : (a.mask != nullptr ? 1 : 0);
  const int xm = side + (a.dropout_p > 0.f ? 3 : 0);
#define NB_SH(DD, BF)                                                           \
  do {                                                                          \
    switch (xm) {                                                               \
      /* no mask array: the mask variant with an all-true mask (its passes are the lighter code) */ \
      case 0: return launch_short<DD, BF, 1>(mq, mk, mv, ma, a, st);            \
      case 1: return launch_short<DD, BF, 1>(mq, mk, mv, ma, a, st);            \
      case 2: return launch_short<DD, BF, 2>(mq, mk, mv, ma, a, st);            \
      case 3: return launch_short<DD, BF, 3>(mq, mk, mv, ma, a, st);            \
      case 4: return launch_short<DD, BF, 4>(mq, mk, mv, ma, a, st);            \
      default: return launch_short<DD, BF, 5>(mq, mk, mv, ma, a, st);           \
    }                                                                           \
  } while (0)
  if (a.d > 64) { if (bf16) NB_SH(128, true); NB_SH(128, false); }
  if (bf16) NB_SH(64, true);
  NB_SH(64, false);
#undef NB_SH
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
