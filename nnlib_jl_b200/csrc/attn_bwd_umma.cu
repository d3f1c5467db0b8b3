// Backward of attention (plain, causal, Bool mask, dropout, bias) on the sm_100a tensor cores.
//
// The gradients Zygote composes from NNlib.jl's rules for this path
// (rrule(batched_mul) src/batched/batchedmul.jl:96-110, ∇softmax
// src/softmax.jl:84-110, the 1/sqrt(d) scaling src/attention.jl:118) are, with
//   P_ij  = exp(scale q_i·k_j - lse_i)          (recomputed from the saved lse)
//   D_i   = dx_i · x_i
//   dS_ij = P_ij (dx_i·v_j - D_i)
//   dq_i = scale Σ_j dS_ij k_j,   dk_j = scale Σ_i dS_ij q_i,   dv_j = Σ_i P_ij dx_i.
// One kernel template covers both halves.  A CTA keeps one 128-row tile pair
// (A, B) resident and streams two rings of 128-row tiles (A', B'):
//   DKV = false  (dq):      A = Q_i,  B = dX_i,  rings A' = K_j, B' = V_j
//   DKV = true   (dk, dv):  A = K_j,  B = V_j,   rings A' = Q_i, B' = dX_i
// and per ring step issues   S = A A'^T,  dP = B B'^T   (both 128x128 in TMEM),
// lets the compute warps turn them into P and dS, and accumulates
//   DKV = false:  dQ += dS · K_j                       (dS from TMEM, K_j MN-major)
//   DKV = true:   dV += P^T · dX_i  (P^T from shared memory),  dK += dS^T · Q_i.
//   warps 0-3   compute, columns 0-63 of the step (thread r owns row r of the resident tile)
//   warps 4-7   compute, columns 64-127
//   warp 8      TMA producer of the resident pair and of ring A'; TMEM allocation
//   warp 9      MMA issuer
//   warp 10     TMA producer of ring B'
//   warp 11     idle (completes the warpgroup of warps 8-10)
// TMEM columns: S [0,128)  dP [128,256)  accumulator 0 [256,256+D)  accumulator 1 [384,384+D).
// dS (half precision): the dq half double-buffers it in columns [384,512) (its second accumulator is
// unused), the dk/dv half writes it over dP: columns [128,160) for ring rows 0-63, [192,224) for rows 64-127.
#include <cuda.h>

#include "common.cuh"
#include "launchers.h"
#include "umma.cuh"
#include "umma_shared.cuh"

namespace nb200 {

__device__ int g_bwd_abort = 0;  // sticky: a bounded wait of a backward kernel ran out


namespace {

// 12 warps = three whole warpgroups: setmaxnreg is a warpgroup-wide instruction, so the copy / issue
// warps 8-10 need their (idle) fourth warp 11
constexpr int kBwThreads = 384;

template <int D, bool DKV>
struct BwCfg {
  static constexpr int kTile = (D / 64) * kChunkBytes;  // 128 rows x D halves
  // Ring A' feeds S early and the accumulation late; ring B' of the dq half (V) is free as soon as dP
  // is done, so the dq half can afford a third A' stage.  The dk/dv half keeps P^T in shared memory.
  static constexpr int kStagesA = DKV ? 2 : 3;
  static constexpr int kStagesB = 2;
  static constexpr int kFixOff = 0;                               // resident pair
  static constexpr int kAOff = 2 * kTile;
  static constexpr int kBOff = kAOff + kStagesA * kTile;
  static constexpr int kPOff = kBOff + kStagesB * kTile;          // P^T tile (DKV): 128 x 128 halves
  static constexpr int kColOff = kPOff + (DKV ? 2 * kChunkBytes : 0);  // per-query lse, D of two ring tiles (DKV)
  static constexpr int kBarOff = kColOff + (DKV ? 2048 : 0);
  static constexpr int kSmemBytes = kBarOff + 256;                // no slack: the kernel checks its 1 KB alignment
};
static_assert(BwCfg<128, true>::kSmemBytes <= 232448 && BwCfg<128, false>::kSmemBytes <= 232448, "shared memory budget");

struct BwBarriers {
  uint64_t fix_full, a_full[3], a_empty[3], b_full[2], b_empty[2];
  uint64_t s_full, dp_full, s_read, ds_ready, acc_full, col_ready;
  uint64_t dp_read;    // dq half: dP is in registers
  uint64_t pt_ready;   // dk/dv half: P^T is in shared memory
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(BwBarriers) <= 256, "barrier block");

// eight consecutive halves (one 16-byte load) times eight more, accumulated in fp32
template <bool BF16>
__device__ __forceinline__ float dot8(const uint4& x, const uint4& y, float acc) {
  const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float2 fx, fy;
    if (BF16) {
      fx = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xs[e]));
      fy = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ys[e]));
    } else {
      fx = __half22float2(*reinterpret_cast<const __half2*>(&xs[e]));
      fy = __half22float2(*reinterpret_cast<const __half2*>(&ys[e]));
    }
    acc = fmaf(fx.x, fy.x, acc);
    acc = fmaf(fx.y, fy.y, acc);
  }
  return acc;
}

// 64 Bool-mask bytes p[e * stride], e = 0..63, packed four to a word; entries e >= n_valid read as 0.
// vec16: stride 1 and p 16-byte aligned, so a full group takes four 16-byte loads.
__device__ __forceinline__ void load_mask64(const unsigned char* p, long long stride, int n_valid, bool vec16,
                                            unsigned int (&mw)[16]) {
  if (vec16 && n_valid >= 64) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(p) + v);
      mw[4 * v + 0] = q.x; mw[4 * v + 1] = q.y; mw[4 * v + 2] = q.z; mw[4 * v + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int w = 0; w < 16; ++w) {
      unsigned int word = 0;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = 4 * w + u;
        if (e < n_valid && __ldg(p + (long long)e * stride) != 0) word |= 1u << (8 * u);
      }
      mw[w] = word;
    }
  }
}

// 64 bias values of 16 bits, p[e * stride] (stride in elements), packed two to a word; entries
// e >= n_valid read as 0.  vec16: stride 1 and p 16-byte aligned.
__device__ __forceinline__ void load_bias16x64(const unsigned char* p, long long stride, int n_valid, bool vec16,
                                               unsigned int (&bw)[32]) {
  if (vec16 && n_valid >= 64) {
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(p) + v);
      bw[4 * v + 0] = q.x; bw[4 * v + 1] = q.y; bw[4 * v + 2] = q.z; bw[4 * v + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int w = 0; w < 32; ++w) {
      unsigned int lo = 0, hi = 0;
      if (2 * w < n_valid) lo = __ldg(reinterpret_cast<const unsigned short*>(p + 2ll * (2 * w) * stride));
      if (2 * w + 1 < n_valid) hi = __ldg(reinterpret_cast<const unsigned short*>(p + 2ll * (2 * w + 1) * stride));
      bw[w] = lo | (hi << 16);
    }
  }
}
__device__ __forceinline__ float bias16_value(unsigned int word, int odd, int dtype) {
  const unsigned int h = odd ? (word >> 16) : (word & 0xffffu);
  if (dtype == NNLIB_B200_BF16) return __uint_as_float(h << 16);
  return __half2float(__ushort_as_half((unsigned short)h));
}


// score row held as raw TMEM words: element e lives in su[e / 32][e % 32]
#define NB_SR(e) __uint_as_float(su[(e) >> 5][(e) & 31])
#define NB_SR_SET(e, val) su[(e) >> 5][(e) & 31] = __float_as_uint(val)

// MASKED: a Bool mask array (NNlib.jl src/attention.jl:133-138, any broadcast strides) takes part.
// DROP: the forward dropped scores (src/dropout.jl:77-87); the same Philox positions are drawn again:
// alpha' = P keep/(1-p) feeds dV, and dS = P (keep/(1-p) dP - D).
// BIAS: the logits carried an additive bias (src/attention.jl:129-131); it is added again and the dq
// half writes its gradient dbias = dS (reduced over the bias' broadcast dimensions by atomic adds).
// FEAT = MASKED | DROP << 1 | BIAS << 2.
template <int D, bool BF16, bool DKV, int FEAT>
__global__ void __launch_bounds__(kBwThreads, 1)
attn_bwd_umma_kernel(const __grid_constant__ CUtensorMap tm_fa, const __grid_constant__ CUtensorMap tm_fb,
                     const __grid_constant__ CUtensorMap tm_ra, const __grid_constant__ CUtensorMap tm_rb,
                     const AttnArgs a, const BwdArgs g, const int n_tiles, const int tail_units) {
  using C = BwCfg<D, DKV>;
  constexpr bool MASKED = (FEAT & 1) != 0, DROP = (FEAT & 2) != 0, BIAS = (FEAT & 4) != 0;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    // the swizzled tiles need 1 KB alignment and the budget leaves no room to round up: refuse cleanly
    if (threadIdx.x == 0) {
      atomicExch(&g_bwd_abort, 1);
      if (a.status) atomicExch(a.status, NNLIB_B200_CUDA_ERROR);
    }
    return;
  }
  BwBarriers* bars = reinterpret_cast<BwBarriers*>(smem + C::kBarOff);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // block -> (unit, resident tile).  Unit by unit (the CTAs of one time share the unit's arrays in L2), the tiles
  // with the longest causal walk first; the last `tail_units` units are dealt out together, all their longest
  // walks first, so that the launch does not end on the long walks of the last unit.
  int unit, rank;                       // rank: 0 = the longest walk of its unit
  {
    const int n_units = gridDim.x / n_tiles;
    const int head = (n_units - tail_units) * n_tiles;
    if ((int)blockIdx.x < head) {
      unit = blockIdx.x / n_tiles;
      rank = blockIdx.x % n_tiles;
    } else {
      const int j = blockIdx.x - head;
      unit = (n_units - tail_units) + j % tail_units;
      rank = j / tail_units;
    }
  }
  const int tix = DKV ? rank : (n_tiles - 1 - rank);
  const int h = unit % a.H, b = unit / a.H;
  const int t0 = tix * 128;             // first row of the resident tile (query for dq, key for dk/dv)

  // ring range: tiles r_first .. r_first + n - 1 of the other sequence
  int r_first = 0, n;
  if (!DKV) {
    const int kv_end = a.causal ? min(a.Lkv, t0 + 128) : a.Lkv;
    n = (kv_end + 127) / 128;
  } else {
    const int n_q = (a.Lq + 127) / 128;
    r_first = a.causal ? tix : 0;       // query tiles before the key tile never see it
    n = max(0, n_q - r_first);
  }

  if (threadIdx.x == 0) {
    mbar_init(&bars->fix_full, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&bars->a_full[s], 1);
      mbar_init(&bars->a_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->b_full[s], 1);
      mbar_init(&bars->b_empty[s], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->s_read, 8);
    mbar_init(&bars->ds_ready, 8);
    mbar_init(&bars->acc_full, 1);
    mbar_init(&bars->col_ready, 8);
    mbar_init(&bars->dp_read, 8);
    mbar_init(&bars->pt_ready, 8);
    bars->abort_flag = *reinterpret_cast<volatile int*>(&g_bwd_abort);
    fence_mbar_init();
  }
  if (warp == 8) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  const bool start_ok = (*abort_flag == 0);
  constexpr uint32_t kColS = 0, kColDP = 128, kColAcc0 = 256, kColAcc1 = 384;
  constexpr uint32_t kColDS = 384;   // dq half: two 64-column dS buffers where the dk/dv half keeps its second accumulator

  // the compute threads hold 64 scores plus side inputs in registers: move the register budget of the
  // copy / issue warps to them
  // (each setmaxnreg sits inside its role's branch: the register allocator budgets per region)
  if (warp >= 8) {
  setmaxnreg_dec<72>();
  if (start_ok && warp == 8) {
    // ------------------------------------- TMA producer: resident pair and ring A'
    if (lane == 0 && n > 0) {
      prefetch_tensormap(&tm_fa);
      prefetch_tensormap(&tm_fb);
      prefetch_tensormap(&tm_ra);
      mbar_arrive_expect_tx(&bars->fix_full, 2 * C::kTile);
      for (int c = 0; c < D / 64; ++c) {
        tma_load_4d(smem + C::kFixOff + c * kChunkBytes, &tm_fa, &bars->fix_full, c * 64, h, t0, b);
        tma_load_4d(smem + C::kFixOff + C::kTile + c * kChunkBytes, &tm_fb, &bars->fix_full, c * 64, h, t0, b);
      }
      bool ok = true;
      int it = 0;
      for (; it < n; ++it) {
        const int s = it % C::kStagesA;
        if (it >= C::kStagesA) ok = mbar_wait(&bars->a_empty[s], ((it / C::kStagesA) - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars->a_full[s], C::kTile);
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem + C::kAOff + s * C::kTile + c * kChunkBytes, &tm_ra, &bars->a_full[s], c * 64, h,
                      (r_first + it) * 128, b);
      }
      if (*abort_flag) {
        mbar_wait_drain(&bars->fix_full, 0, kDrainNs);
        for (int jj = max(0, it - C::kStagesA); jj < it; ++jj)
          mbar_wait_drain(&bars->a_full[jj % C::kStagesA], (jj / C::kStagesA) & 1, kDrainNs);
      }
    }
  } else if (start_ok && warp == 10) {
    // ------------------------------------------------- TMA producer: ring B'
    if (lane == 0 && n > 0) {
      prefetch_tensormap(&tm_rb);
      bool ok = true;
      int it = 0;
      for (; it < n; ++it) {
        const int s = it % C::kStagesB;
        if (it >= C::kStagesB) ok = mbar_wait(&bars->b_empty[s], ((it / C::kStagesB) - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars->b_full[s], C::kTile);
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem + C::kBOff + s * C::kTile + c * kChunkBytes, &tm_rb, &bars->b_full[s], c * 64, h,
                      (r_first + it) * 128, b);
      }
      if (*abort_flag)
        for (int jj = max(0, it - C::kStagesB); jj < it; ++jj)
          mbar_wait_drain(&bars->b_full[jj % C::kStagesB], (jj / C::kStagesB) & 1, kDrainNs);
    }
  } else if (start_ok && warp == 9) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_nt = make_idesc_f16(BF16, 128, 128, false, false);  // both operands K-major
      constexpr uint32_t idesc_acc = make_idesc_f16(BF16, 128, D, false, true);    // B MN-major
      constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t lbo_k = (16u >> 4) << 16;
      constexpr uint32_t lbo_mn = (static_cast<uint32_t>(kChunkBytes) >> 4) << 16;
      constexpr uint32_t tile16 = C::kTile >> 4;
      const uint32_t fix_a = (smem_u32(smem + C::kFixOff) >> 4) | lbo_k;
      const uint32_t fix_b = fix_a + tile16;
      const uint32_t ra_k = (smem_u32(smem + C::kAOff) >> 4) | lbo_k;     // ring A' read K-major (for S)
      const uint32_t ra_mn = (smem_u32(smem + C::kAOff) >> 4) | lbo_mn;   // ring A' read MN-major (accumulation)
      const uint32_t rb_k = (smem_u32(smem + C::kBOff) >> 4) | lbo_k;     // ring B' read K-major (for dP)
      const uint32_t rb_mn = (smem_u32(smem + C::kBOff) >> 4) | lbo_mn;   // ring B' read MN-major (dV)
      const uint32_t p_lo = (smem_u32(smem + C::kPOff) >> 4) | lbo_k;

      auto issue_s = [&](int it) {           // S = A A'^T
        const uint32_t st = (it % C::kStagesA) * tile16;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (kChunkBytes >> 4) + (kk & 3) * 2;
          umma_ss_lohi(tmem + kColS, fix_a + off, ra_k + st + off, desc_hi, idesc_nt, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->s_full);
      };
      auto issue_dp = [&](int it) {          // dP = B B'^T
        const uint32_t st = (it % C::kStagesB) * tile16;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (kChunkBytes >> 4) + (kk & 3) * 2;
          umma_ss_lohi(tmem + kColDP, fix_b + off, rb_k + st + off, desc_hi, idesc_nt, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->dp_full);
        if (!DKV) umma_commit(&bars->b_empty[it % C::kStagesB]);   // V_j is not needed again
      };
      // dQ += dS K_j  (dq half, dS buffer it&1)   or   dK += dS^T Q_i  (dk/dv half, dS over dP)
      auto issue_ds_acc = [&](int it) {
        const uint32_t sa = (it % C::kStagesA) * tile16;
        const uint32_t ds_col = DKV ? kColDP : (kColDS + (it & 1) * 64);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ts_lohi(tmem + (DKV ? kColAcc1 : kColAcc0), tmem + ds_col + (kk >> 2) * (DKV ? 64 : 32) + (kk & 3) * 8,
                       ra_mn + sa + kk * (2048 >> 4), desc_hi, idesc_acc, (it == 0 && kk == 0) ? 0u : 1u);
        umma_commit(&bars->a_empty[it % C::kStagesA]);   // also tells the dq half that dS buffer it&1 is free
      };
      auto issue_dv = [&](int it) {          // dV += P^T dX_i
        const uint32_t sb = (it % C::kStagesB) * tile16;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t aoff = (kk >> 2) * (kChunkBytes >> 4) + (kk & 3) * 2;
          umma_ss_lohi(tmem + kColAcc0, p_lo + aoff, rb_mn + sb + kk * (2048 >> 4), desc_hi, idesc_acc,
                       (it == 0 && kk == 0) ? 0u : 1u);
        }
        umma_commit(&bars->b_empty[it % C::kStagesB]);   // also tells that P^T has been consumed
      };

      // S and dP of the next step are issued as early as the compute warps allow (they have the
      // previous S / dP in registers), the accumulating products when dS (and P^T) are ready.
      bool ok = mbar_wait(&bars->fix_full, 0, abort_flag);
      if (ok) ok = mbar_wait(&bars->a_full[0], 0, abort_flag);
      if (ok) issue_s(0);
      if (ok) ok = mbar_wait(&bars->b_full[0], 0, abort_flag);
      if (ok) issue_dp(0);
      for (int it = 0; it < n && ok; ++it) {
        const uint32_t par = it & 1;
        const bool more = it + 1 < n;
        if (more) {
          ok = mbar_wait(&bars->a_full[(it + 1) % C::kStagesA], ((it + 1) / C::kStagesA) & 1, abort_flag);
          if (ok) ok = mbar_wait(&bars->s_read, par, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_s(it + 1);
        }
        if (!DKV) {
          if (more) {
            ok = mbar_wait(&bars->b_full[(it + 1) % C::kStagesB], ((it + 1) / C::kStagesB) & 1, abort_flag);
            if (ok) ok = mbar_wait(&bars->dp_read, par, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_dp(it + 1);
          }
          ok = mbar_wait(&bars->ds_ready, par, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_ds_acc(it);
        } else {
          ok = mbar_wait(&bars->ds_ready, par, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_ds_acc(it);
          if (more) {
            ok = mbar_wait(&bars->b_full[(it + 1) % C::kStagesB], ((it + 1) / C::kStagesB) & 1, abort_flag);
            if (!ok) break;
            issue_dp(it + 1);   // overwrites dS: ordered behind the dK products above
          }
          ok = mbar_wait(&bars->pt_ready, par, abort_flag);
          if (!ok) break;
          issue_dv(it);
        }
      }
      if (ok) umma_commit(&bars->acc_full);
    }
  }
  } else {
  setmaxnreg_inc<208>();
  if (start_ok) {
    // ----------------------------------------------------------- compute warps
    const int half = warp >> 2;               // which 64 columns of every step this thread handles
    const int wq = warp & 3;                  // TMEM lane quarter this warp may touch
    const int r = wq * 32 + lane;             // row of the resident tile = TMEM lane
    const int row = t0 + r;                   // query (dq) or key (dk/dv) index
    const bool row_ok = row < (DKV ? a.Lkv : a.Lq);
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(wq * 32) << 16);
    const uint32_t tS = lane_base + kColS + half * 64, tDP = lane_base + kColDP + half * 64;
    const float c2 = a.scale * kLog2e;
    const float pos_inf = __int_as_float(0x7f800000);
    const float* lse_u = a.lse + (long long)a.Lq * h + a.lse_sb * b;
    float* delta_u = g.delta + (long long)a.Lq * h + (long long)a.Lq * a.H * b;
    float* col_lse = reinterpret_cast<float*>(smem + C::kColOff);   // [2][128] lse (base 2) of the ring tile's queries
    float* col_dl = col_lse + 256;                                  // [2][128] D of the ring tile's queries
    bool ok = true;

    // dq half: per-row constants lse_i (base 2) and D_i = dx_i · x_i
    float lse2_row = pos_inf, dl_row = 0.f;
    if (!DKV && row_ok) {
      // a query that attends to nothing (lse = -inf, possible with a mask array) gets and gives no gradient
      const float lse_nat = __ldg(lse_u + row);
      const bool dead = lse_nat == neg_inf();
      lse2_row = dead ? pos_inf : lse_nat * kLog2e;
      const uint4* dxr = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(g.dx) +
                         2ll * ((long long)row * g.dx_sl + (long long)b * g.dx_sb + (long long)h * a.d));
      const uint4* xr = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.x) +
                        2ll * ((long long)row * a.x_sl + (long long)b * a.x_sb + (long long)h * a.d));
#pragma unroll
      for (int e = 0; e < D / 8; ++e)
        if (e * 8 < a.d) dl_row = dot8<BF16>(__ldg(dxr + e), __ldg(xr + e), dl_row);   // the head's own features
      if (dead) dl_row = 0.f;   // its x is NaN (or 0)
      if (half == 0) delta_u[row] = dl_row;
    }
    // dk/dv half: lse and D belong to the COLUMNS (queries of the ring tile).  Thread (half, r) fetches
    // one of the 256 values a step ahead and parks it in shared memory for everyone.
    auto col_fetch = [&](int it) -> float {
      const int qi = (r_first + it) * 128 + r;
      if (qi >= a.Lq) return half == 0 ? pos_inf : 0.f;     // padded query: P = exp2(-inf) = 0
      if (half == 1) return __ldg(delta_u + qi);
      const float l = __ldg(lse_u + qi);
      return (l == neg_inf()) ? pos_inf : l * kLog2e;         // dead query: P = 0
    };
    // Bool mask array: the dq half reads the 64 keys of its row per step; in the dk/dv half a thread owns
    // a key and needs the step's 64 queries -- one byte for the whole kernel when the mask does not depend
    // on the query (key padding), else a strided gather per step
    const unsigned char* mask_p = nullptr;
    bool mask_row_keep = true;
    const bool mask_per_step = MASKED && (!DKV || a.mask_s[1] != 0);
    if (MASKED && row_ok) {
      mask_p = a.mask + (long long)h * a.mask_s[2] + (long long)b * a.mask_s[3] + (long long)row * a.mask_s[DKV ? 0 : 1];
      if (DKV && a.mask_s[1] == 0) mask_row_keep = __ldg(mask_p) != 0;
    }
    const long long mask_step = MASKED ? a.mask_s[DKV ? 1 : 0] : 0;   // stride along the columns of a step
    // bias: like the mask, a row of 64 keys per step in the dq half, a column of 64 queries in the dk/dv
    // half (one value for the whole kernel when the bias does not depend on the query)
    const int bias_esz = (BIAS && a.bias_dtype == NNLIB_B200_F32) ? 4 : 2;
    const unsigned char* bias_p = nullptr;
    float bias_uniform = 0.f;
    const bool bias_per_step = BIAS && (!DKV || a.bias_s[1] != 0);
    const long long bias_step = BIAS ? a.bias_s[DKV ? 1 : 0] : 0;
    if (BIAS) {
      // rows past the end of the sequence read the last row's bias (their P is forced to zero below): every
      // lane of a warp then takes the same path through the loads
      const long long row_c = min((long long)row, (long long)(DKV ? a.Lkv : a.Lq) - 1);
      bias_p = reinterpret_cast<const unsigned char*>(a.bias) +
               ((long long)h * a.bias_s[2] + (long long)b * a.bias_s[3] + row_c * a.bias_s[DKV ? 0 : 1]) * bias_esz;
      if (DKV && a.bias_s[1] == 0) bias_uniform = load_bias(bias_p, 0, a.bias_dtype) * kLog2e;
    }
    // dbias (dq half): plain stores when every score has its own element, atomic adds when a stride of 0
    // folds several scores onto one
    float* dbias_p = nullptr;
    bool dbias_exclusive = false;
    if (BIAS && !DKV && g.dbias && row_ok) {
      dbias_p = g.dbias + (long long)row * g.dbias_s[1] + (long long)h * g.dbias_s[2] + (long long)b * g.dbias_s[3];
      dbias_exclusive = g.dbias_s[0] != 0 && (g.dbias_s[1] != 0 || a.Lq == 1) && (g.dbias_s[2] != 0 || a.H == 1) &&
                        (g.dbias_s[3] != 0 || a.B == 1);
    }
    auto col_store = [&](int it, float v) {
      (half == 0 ? col_lse : col_dl)[(it & 1) * 128 + r] = v;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->col_ready);
    };
    if (DKV && n > 0) col_store(0, col_fetch(0));

    for (int it = 0; it < n && ok; ++it) {
      const uint32_t par = it & 1;
      const int c0 = (r_first + it) * 128 + half * 64;   // first column of this thread: key (dq) or query (dk/dv)
      float col_next = 0.f;
      if (DKV && it + 1 < n) col_next = col_fetch(it + 1);
      unsigned int mw[16];
      if (mask_per_step && mask_p) {
        const unsigned char* mp = mask_p + (long long)c0 * mask_step;
        load_mask64(mp, mask_step, (DKV ? a.Lq : a.Lkv) - c0,
                    mask_step == 1 && (reinterpret_cast<uintptr_t>(mp) & 15u) == 0, mw);
      }
      unsigned int bw[32];
      const bool bias16 = bias_per_step && bias_p && bias_esz == 2;
      if (bias16) {
        const unsigned char* bp = bias_p + (long long)c0 * bias_step * 2;
        // 16-byte loads only when every row of the warp allows them
        const bool vec = __all_sync(0xffffffffu, bias_step == 1 && (reinterpret_cast<uintptr_t>(bp) & 15u) == 0);
        load_bias16x64(bp, bias_step, (DKV ? a.Lq : a.Lkv) - c0, vec, bw);
      }
      // which of this thread's 64 scores survived the forward's dropout (bit e: column c0 + e)
      unsigned int kb[2] = {0xffffffffu, 0xffffffffu};
      if (DROP) {
        if (!DKV) {
          // a row of scores: eight consecutive keys share one Philox call, as in the forward
          const unsigned long long srow = score_row(a, row_ok ? row : 0, h, b);
          kb[0] = dropout_keep32(a, srow, (unsigned int)(c0 >> 5));
          kb[1] = dropout_keep32(a, srow, (unsigned int)(c0 >> 5) + 1u);
        } else {
          // a column of scores (one key, 64 queries): lane L draws the call of (query L%8 of an 8-query
          // block, key group L/8 of this warp's 32 keys) and the lanes trade the 8-bit results
          const unsigned int j8 = (unsigned int)(t0 + wq * 32) / 8u + (unsigned int)(lane >> 3);
          kb[0] = kb[1] = 0u;
#pragma unroll 2
          for (int cb = 0; cb < 8; ++cb) {
            const int qi = c0 + cb * 8 + (lane & 7);
            unsigned int w[4];
            dropout_words(a, score_row(a, qi, h, b), j8, w);
            unsigned int byte = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              byte |= ((w[e] & 0xffffu) >= a.drop_thresh ? 1u : 0u) << (2 * e);
              byte |= ((w[e] >> 16) >= a.drop_thresh ? 1u : 0u) << (2 * e + 1);
            }
            unsigned int bits8 = 0;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const unsigned int other = __shfl_sync(0xffffffffu, byte, q + (lane & 24));
              bits8 |= ((other >> (lane & 7)) & 1u) << q;
            }
            kb[cb >> 2] |= bits8 << ((cb & 3) * 8);
          }
        }
      }
      ok = mbar_wait(&bars->s_full, par, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t su[2][32];
      tmem_ld32(tS, su[0]);
      tmem_ld32(tS + 32, su[1]);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->s_read);

      if (!DKV) {
        const int lim = row_ok ? (a.causal ? min(row, a.Lkv - 1) : a.Lkv - 1) : -1;  // last key of this row
        if (BIAS && bias_p) {
          if (bias16) {
#pragma unroll
            for (int e = 0; e < 64; ++e)
              NB_SR_SET(e, ex2_approx(fmaf(NB_SR(e), c2, fmaf(bias16_value(bw[e >> 1], e & 1, a.bias_dtype), kLog2e, -lse2_row))));
          } else {   // Float32 bias: fetched here, eight at a time
#pragma unroll
            for (int e0 = 0; e0 < 64; e0 += 8) {
              float bv[8];
#pragma unroll
              for (int u = 0; u < 8; ++u)
                bv[u] = (c0 + e0 + u < a.Lkv) ? __ldg(reinterpret_cast<const float*>(bias_p) + (long long)(c0 + e0 + u) * bias_step) : 0.f;
#pragma unroll
              for (int u = 0; u < 8; ++u)
                NB_SR_SET(e0 + u, ex2_approx(fmaf(NB_SR(e0 + u), c2, fmaf(bv[u], kLog2e, -lse2_row))));
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 64; ++e) NB_SR_SET(e, ex2_approx(fmaf(NB_SR(e), c2, -lse2_row)));
        }
        if (c0 + 63 > lim) {
#pragma unroll
          for (int e = 0; e < 64; ++e)
            if (c0 + e > lim) NB_SR_SET(e, 0.f);
        }
        if (MASKED && mask_p) {
#pragma unroll
          for (int e = 0; e < 64; ++e)
            if (((mw[e >> 2] >> ((e & 3) * 8)) & 0xffu) == 0u) NB_SR_SET(e, 0.f);
        }
      } else {
        ok = mbar_wait(&bars->col_ready, par, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float4* L4 = reinterpret_cast<const float4*>(col_lse + par * 128 + half * 64);
#pragma unroll
        for (int e = 0; e < 64; e += 4) {
          const float4 L = L4[e >> 2];
          float b0 = bias_uniform, b1 = bias_uniform, b2 = bias_uniform, b3 = bias_uniform;   // 0 without bias
          if (BIAS && bias_per_step && bias_p) {
            if (bias16) {
              b0 = bias16_value(bw[e >> 1], 0, a.bias_dtype) * kLog2e;
              b1 = bias16_value(bw[e >> 1], 1, a.bias_dtype) * kLog2e;
              b2 = bias16_value(bw[(e >> 1) + 1], 0, a.bias_dtype) * kLog2e;
              b3 = bias16_value(bw[(e >> 1) + 1], 1, a.bias_dtype) * kLog2e;
            } else {
              const float* bf = reinterpret_cast<const float*>(bias_p);
              b0 = (c0 + e + 0 < a.Lq) ? __ldg(bf + (long long)(c0 + e + 0) * bias_step) * kLog2e : 0.f;
              b1 = (c0 + e + 1 < a.Lq) ? __ldg(bf + (long long)(c0 + e + 1) * bias_step) * kLog2e : 0.f;
              b2 = (c0 + e + 2 < a.Lq) ? __ldg(bf + (long long)(c0 + e + 2) * bias_step) * kLog2e : 0.f;
              b3 = (c0 + e + 3 < a.Lq) ? __ldg(bf + (long long)(c0 + e + 3) * bias_step) * kLog2e : 0.f;
            }
          }
          NB_SR_SET(e + 0, ex2_approx(fmaf(NB_SR(e + 0), c2, b0 - L.x)));
          NB_SR_SET(e + 1, ex2_approx(fmaf(NB_SR(e + 1), c2, b1 - L.y)));
          NB_SR_SET(e + 2, ex2_approx(fmaf(NB_SR(e + 2), c2, b2 - L.z)));
          NB_SR_SET(e + 3, ex2_approx(fmaf(NB_SR(e + 3), c2, b3 - L.w)));
        }
        // queries before this key (causal) and padded key rows contribute nothing
        const int cmin = (row_ok && mask_row_keep) ? (a.causal ? row - c0 : 0) : 64;
        if (cmin > 0) {
#pragma unroll
          for (int e = 0; e < 64; ++e)
            if (e < cmin) NB_SR_SET(e, 0.f);
        }
        if (mask_per_step && mask_p) {
#pragma unroll
          for (int e = 0; e < 64; ++e)
            if (((mw[e >> 2] >> ((e & 3) * 8)) & 0xffu) == 0u) NB_SR_SET(e, 0.f);
        }
      }

      ok = mbar_wait(&bars->dp_full, par, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();

      // dS = P (dP - D), rounded to the element type: the A operand of the dQ / dK product
      uint32_t pk[32];
      uint32_t dpq[2][32];   // dq half: this thread's 64 dP values (kept for the dbias pass below)
      // dS of score e of the dq half: P (keep/(1-p) dP - D)
      auto ds_of = [&](int e) -> float {
        float gval = __uint_as_float(dpq[e >> 5][e & 31]);
        if (DROP) gval = ((kb[e >> 5] >> (e & 31)) & 1u) ? gval * a.inv_keep : 0.f;
        return (gval - dl_row) * NB_SR(e);
      };
      if (!DKV) {
        tmem_ld32(tDP, dpq[0]);
        tmem_ld32(tDP + 32, dpq[1]);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->dp_read);   // the next dP may be issued
#pragma unroll
        for (int e = 0; e < 64; e += 2) pk[e >> 1] = pack2<BF16>(ds_of(e), ds_of(e + 1));
        if (it >= 2) {   // the products of step it-2 have finished reading this dS buffer
          ok = mbar_wait(&bars->a_empty[(it - 2) % C::kStagesA], ((it - 2) / C::kStagesA) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
        }
        __syncwarp();
        tmem_st32(lane_base + kColDS + par * 64 + half * 32, pk);
      } else {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t dp[32];
          tmem_ld32(tDP + cc * 32, dp);
          tmem_wait_ld();
          const float4* D4 = reinterpret_cast<const float4*>(col_dl + par * 128 + half * 64 + cc * 32);
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const float4 Dl = D4[e >> 2];
            float g0 = __uint_as_float(dp[e + 0]), g1 = __uint_as_float(dp[e + 1]);
            float g2 = __uint_as_float(dp[e + 2]), g3 = __uint_as_float(dp[e + 3]);
            if (DROP) {
              const unsigned int k4 = kb[cc] >> e;
              g0 = (k4 & 1u) ? g0 * a.inv_keep : 0.f;
              g1 = (k4 & 2u) ? g1 * a.inv_keep : 0.f;
              g2 = (k4 & 4u) ? g2 * a.inv_keep : 0.f;
              g3 = (k4 & 8u) ? g3 * a.inv_keep : 0.f;
            }
            const float d0 = (g0 - Dl.x) * NB_SR(cc * 32 + e + 0);
            const float d1 = (g1 - Dl.y) * NB_SR(cc * 32 + e + 1);
            const float d2 = (g2 - Dl.z) * NB_SR(cc * 32 + e + 2);
            const float d3 = (g3 - Dl.w) * NB_SR(cc * 32 + e + 3);
            pk[cc * 16 + e / 2] = pack2<BF16>(d0, d1);
            pk[cc * 16 + e / 2 + 1] = pack2<BF16>(d2, d3);
          }
        }
        __syncwarp();
        tmem_st32(tDP, pk);     // over the first half of this thread's own dP columns
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ds_ready);

      if (BIAS && !DKV && dbias_p) {
        // gradient of the bias = dS in fp32 (masked and dropped-out positions included: they are zero /
        // scaled).  Written after dS has been handed to the tensor core: the stores are per-row branches
        // and off the products' critical path.
#pragma unroll
        for (int e = 0; e < 64; e += 2) {
          const float d0 = ds_of(e), d1 = ds_of(e + 1);
          float* o0 = dbias_p + (long long)(c0 + e) * g.dbias_s[0];
          if (dbias_exclusive) {
            if (g.dbias_s[0] == 1 && c0 + e + 1 < a.Lkv && (reinterpret_cast<uintptr_t>(o0) & 7u) == 0) {
              *reinterpret_cast<float2*>(o0) = make_float2(d0, d1);
            } else {
              if (c0 + e < a.Lkv) *o0 = d0;
              if (c0 + e + 1 < a.Lkv) *(o0 + g.dbias_s[0]) = d1;
            }
          } else {
            if (c0 + e < a.Lkv) atomicAdd(o0, d0);
            if (c0 + e + 1 < a.Lkv) atomicAdd(o0 + g.dbias_s[0], d1);
          }
        }
      }
      if (BIAS && !DKV) __syncwarp();   // (outside the per-row branch: every lane takes part)

      if (DKV) {
        // P^T as the K-major A operand of dV += P^T dX: row r, 16-byte pieces in 128-byte-swizzled order,
        // once the previous step's product has finished reading the tile
        if (it > 0) {
          ok = mbar_wait(&bars->b_empty[(it - 1) % C::kStagesB], ((it - 1) / C::kStagesB) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        uint8_t* prow = smem + C::kPOff + half * kChunkBytes + r * 128;
        if (DROP) {   // dV takes the scores the forward multiplied V with: alpha' = P keep/(1-p)
#pragma unroll
          for (int e = 0; e < 64; ++e)
            NB_SR_SET(e, ((kb[e >> 5] >> (e & 31)) & 1u) ? NB_SR(e) * a.inv_keep : 0.f);
        }
#pragma unroll
        for (int piece = 0; piece < 8; ++piece) {
          uint4 v;
          v.x = pack2<BF16>(NB_SR(piece * 8 + 0), NB_SR(piece * 8 + 1));
          v.y = pack2<BF16>(NB_SR(piece * 8 + 2), NB_SR(piece * 8 + 3));
          v.z = pack2<BF16>(NB_SR(piece * 8 + 4), NB_SR(piece * 8 + 5));
          v.w = pack2<BF16>(NB_SR(piece * 8 + 6), NB_SR(piece * 8 + 7));
          *reinterpret_cast<uint4*>(prow + ((piece ^ (r & 7)) << 4)) = v;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->pt_ready);
        if (it + 1 < n) col_store(it + 1, col_next);
      }
    }

    // ---------------------------------------------------------------- epilogue
    if (ok && n > 0) {
      ok = mbar_wait(&bars->acc_full, 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) tc_fence_after();
    }
    if (ok) {
      // dq half: the two column groups share dQ's 32-column chunks; dk/dv half: group 0 stores dV, group 1 dK
      const long long Lrow = DKV ? a.Lkv : a.Lq;
      const long long dense = 2ll * (((long long)row + Lrow * b) * ((long long)a.H * a.d) + (long long)h * a.d);
      uint8_t* out = reinterpret_cast<uint8_t*>(DKV ? (half == 0 ? g.dv : g.dk) : g.dq) + dense;
      const float mul = (DKV && half == 0) ? 1.f : a.scale;
      const uint32_t col = (DKV && half == 1) ? kColAcc1 : kColAcc0;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        if (!DKV && (c & 1) != half) continue;
        uint32_t o[32];
        if (n > 0) {
          __syncwarp();   // the stores of the previous chunk are per-row branches
          tmem_ld32(lane_base + col + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            if (c * 32 + e >= a.d) continue;   // a head narrower than the padded size: the rest is padding
            uint4 v;
            v.x = pack2<BF16>(__uint_as_float(o[e]) * mul, __uint_as_float(o[e + 1]) * mul);
            v.y = pack2<BF16>(__uint_as_float(o[e + 2]) * mul, __uint_as_float(o[e + 3]) * mul);
            v.z = pack2<BF16>(__uint_as_float(o[e + 4]) * mul, __uint_as_float(o[e + 5]) * mul);
            v.w = pack2<BF16>(__uint_as_float(o[e + 6]) * mul, __uint_as_float(o[e + 7]) * mul);
            *reinterpret_cast<uint4*>(out + (c * 32 + e) * 2) = v;
          }
        }
      }
    }
  }
  }   // compute warps

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) {
    atomicExch(&g_bwd_abort, 1);
    if (a.status) atomicExch(a.status, NNLIB_B200_TIMEOUT);
  }
}

#undef NB_SR
#undef NB_SR_SET

template <int D, bool BF16, bool DKV, int FEAT>
cudaError_t launch_bwd_umma(const CUtensorMap& fa, const CUtensorMap& fb, const CUtensorMap& ra, const CUtensorMap& rb,
                            const AttnArgs& a, const BwdArgs& g, cudaStream_t st) {
  auto kern = attn_bwd_umma_kernel<D, BF16, DKV, FEAT>;
  constexpr int smem = BwCfg<D, DKV>::kSmemBytes;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  const int n_tiles = ((DKV ? a.Lkv : a.Lq) + 127) / 128;
  const long long blocks = (long long)n_tiles * a.H * a.B;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  // causal walks differ in length: the units of the last two waves are dealt out longest walks first
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      sms < 1)
    sms = 148;
  const long long n_units = (long long)a.H * a.B;
  long long tail_units = a.causal ? 2 * ((sms + n_tiles - 1) / n_tiles) : 0;
  if (tail_units > n_units) tail_units = n_units;
  // ... as long as the arrays of those units (q, dx, k, v of each) stay well inside L2 together: with very long
  // sequences the interleaved units evict each other and the launch gets slower instead (L = 32768: + 0.5 %)
  const long long unit_bytes = 2ll * ((long long)a.Lq + a.Lkv) * a.d * 2;
  if (tail_units * unit_bytes > (48ll << 20)) tail_units = (48ll << 20) / unit_bytes;
  if (tail_units < 2) tail_units = 0;
  kern<<<(unsigned)blocks, kBwThreads, smem, st>>>(fa, fb, ra, rb, a, g, n_tiles, (int)tail_units);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

// The tensor-core backward covers half-precision arrays with d = dv any multiple of 8 up to 128 (heads are
// addressed through 4-d tensor maps and padded with zeros to 64 / 128) and every feature of the
// forward: causal flag, Bool mask arrays, Philox dropout and bias (any element type and strides).
bool umma_bwd_supports(const AttnArgs& a, const BwdArgs& g, int dtype) {
  if (dtype != NNLIB_B200_F16 && dtype != NNLIB_B200_BF16) return false;
  if (a.d < 8 || a.d > 128 || a.d % 8 != 0 || a.dv != a.d) return false;   // padded to 64 / 128 by the copy engine
  if (g.dbias && !a.bias) return false;
  if (a.causal && a.coff != 0) return false;      // the tile skipping here assumes the square causal pattern
  if (a.Lq < 1 || a.Lkv < 1 || a.H < 1 || a.B < 1 || !a.lse || !g.delta) return false;
  const void* ptrs[] = {a.q, a.k, a.v, a.x, g.dx, g.dq, g.dk, g.dv};
  for (const void* p : ptrs)
    if (!p || !aligned16(p)) return false;
  const long long strides[] = {a.q_sl, a.q_sb, a.k_sl, a.k_sb, a.v_sl, a.v_sb, a.x_sl, a.x_sb, g.dx_sl, g.dx_sb};
  for (long long s : strides)
    if (!stride_ok(s)) return false;
  return encode_tiled_fn() != nullptr;
}

cudaError_t umma_bwd(const AttnArgs& a, const BwdArgs& g, int dtype, cudaStream_t st) {
  CUtensorMap mq, mk, mv, mdx;
  if (!make_head_map(&mq, a.q, dtype, a.d, a.H, a.Lq, a.B, a.q_sl, a.q_sb)) return cudaErrorInvalidValue;
  if (!make_head_map(&mk, a.k, dtype, a.d, a.H, a.Lkv, a.B, a.k_sl, a.k_sb)) return cudaErrorInvalidValue;
  if (!make_head_map(&mv, a.v, dtype, a.d, a.H, a.Lkv, a.B, a.v_sl, a.v_sb)) return cudaErrorInvalidValue;
  if (!make_head_map(&mdx, g.dx, dtype, a.d, a.H, a.Lq, a.B, g.dx_sl, g.dx_sb)) return cudaErrorInvalidValue;
  const bool bf16 = dtype == NNLIB_B200_BF16;
  cudaError_t e;
#define NB_BW2(DD, BF, FT)                                                                       \
  do {                                                                                           \
    e = launch_bwd_umma<DD, BF, false, FT>(mq, mdx, mk, mv, a, g, st);                           \
    if (e == cudaSuccess) e = launch_bwd_umma<DD, BF, true, FT>(mk, mv, mq, mdx, a, g, st);      \
  } while (0)
#define NB_BW(DD, BF)                                                                            \
  do {                                                                                           \
    switch (feat) {                                                                              \
      case 0: NB_BW2(DD, BF, 0); break;                                                          \
      case 1: NB_BW2(DD, BF, 1); break;                                                          \
      case 2: NB_BW2(DD, BF, 2); break;                                                          \
      case 3: NB_BW2(DD, BF, 3); break;                                                          \
      case 4: NB_BW2(DD, BF, 4); break;                                                          \
      case 5: NB_BW2(DD, BF, 5); break;                                                          \
      case 6: NB_BW2(DD, BF, 6); break;                                                          \
      default: NB_BW2(DD, BF, 7); break;                                                         \
    }                                                                                            \
  } while (0)
  const int feat = (a.mask ? 1 : 0) | (a.dropout_p > 0.f ? 2 : 0) | (a.bias ? 4 : 0);
  if (a.d > 64) { if (bf16) NB_BW(128, true); else NB_BW(128, false); }
  else            { if (bf16) NB_BW(64, true);  else NB_BW(64, false); }
#undef NB_BW
#undef NB_BW2
  return e;
}


// Reads and clears the backward kernels' sticky "a bounded wait ran out" flag of the current device.
// Synchronises the stream.
cudaError_t umma_bwd_take_abort(int* out, cudaStream_t st) {
  int v = 0;
  cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyFromSymbol(&v, g_bwd_abort, sizeof(int));
  if (e != cudaSuccess) return e;
  if (v) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_bwd_abort, &zero, sizeof(int));
  }
  *out = v;
  return e;
}

}  // namespace nb200
