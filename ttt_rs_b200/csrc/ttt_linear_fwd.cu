// Fused TTT-Linear forward scan for sm_100a: one 4-warp CTA per (batch, head) stream walks all mini-batches.
//
// What it computes is the reference's multi-stage forward kernel
// (rust/fused/src/linear_fused_tile/forward/kernel.rs:92-176, stage body forward/stage.rs:29-208, semantics
// rust/core/src/linear.rs:91-149): per 16-token stage
//     Z1 = K W + b;  G = d/dZ1 of 0.5|LN(Z1) - (V-K)|^2;  M = eta o (1 + tril(Q K^T)),  eta[i,j] = te[i] lr[j] (j<=i)
//     out = Q + LN(Q W + b - M G);   W -= (te[15] lr o K)^T G;   b -= sum_j te[15] lr[j] G[j,:]
// with (W, b) checkpointed before the update of every K-th stage.
//
// How it is laid out here (none of this follows the reference's design):
//   * The state is held transposed, W^T[n][k], as float32 mma accumulators: warp w owns output features
//     n in [16w,16w+16) and all 64 k (32 registers per thread).  In that layout the same registers are,
//     after one cvt to bf16, the B operand of K.W / Q.W, and the rank-16 update W^T += (-te15 lr G)^T K
//     accumulates straight into them, so W never leaves registers between stages.
//   * Q/K/V tiles of the next three stages are in flight as TMA loads (128B swizzle) on mbarriers.
//   * Row statistics for the two LayerNorms are warp-shuffle reduced and exchanged across the 4 warps through
//     512 bytes of shared memory; G reaches the tensor cores as an A/B operand through movmatrix.
//   * Output tiles leave through a double-buffered staging tile and a TMA store.
//
// head_dim 32 (template parameter SEG = 32) runs on the same 64-wide tiling: a CTA takes a PAIR of heads of one batch
// element, their 16 x 32 tiles side by side in the 16 x 64 tile (warps 0,1 = first head, warps 2,3 = second), and the
// state as a block-diagonal 64 x 64 matrix whose off-diagonal blocks stay zero.  K.W and Q.W need no change (the zero
// blocks contribute nothing); what is per head -- the LayerNorm row sums, Q.K^T and the k-range of the state update
// -- is restricted to the head's own 32 columns.
#include <type_traits>

#include "ttt_kernels.h"
#include "ttt_stage.cuh"

namespace ttt {

constexpr int FWD_NST = 3;  // TMA pipeline depth (stages in flight); the stage loop is unrolled by it
static_assert(FWD_NST == 3, "the stage loop below is written out for three slots");

template <typename T, int SEG>
struct FwdSmem {
  using TF = TileFmt<T>;
  static constexpr uint32_t SLOT = 3 * TF::BYTES;                  // q, k, v
  static constexpr uint32_t OFF_OUT = FWD_NST * SLOT;              // staging (raw format): 2 x output, 2 x Gp
  static constexpr uint32_t LR_SLOT = (SEG == 32) ? 128 : 64;      // lr of one stage: 16 elements (x 2 heads when paired)
  static constexpr uint32_t OFF_LR = OFF_OUT + 4 * TF::RAW_BYTES;  // FWD_NST x LR_SLOT
  static constexpr uint32_t OFF_XCH = OFF_LR + FWD_NST * LR_SLOT;  // 2 x Xch4
  static constexpr uint32_t OFF_BAR = OFF_XCH + 2 * sizeof(Xch4);
  static constexpr uint32_t TOTAL = OFF_BAR + FWD_NST * 8;
  static constexpr uint32_t DYN_BYTES = TOTAL + 1024;  // slack for manual 1024-byte alignment
};

template <typename T, int SEG, int MB>
__global__ void __launch_bounds__(NTHREADS, (sizeof(T) == 2 ? 3 : 1))
    ttt_linear_fwd_kernel(const __grid_constant__ typename PairIo<T, SEG>::Ref tm_q,
                          const __grid_constant__ typename PairIo<T, SEG>::Ref tm_k,
                          const __grid_constant__ typename PairIo<T, SEG>::Ref tm_v,
                          const __grid_constant__ typename PairIo<T, SEG>::Ref tm_o,
                          const __grid_constant__ CUtensorMap tm_g, const LinFwdParams p) {
  using TF = TileFmt<T>;
  using SM = FwdSmem<T, SEG>;
  constexpr int NP = TF::NP;
  constexpr bool TWO_PASS = (sizeof(T) == 4);
  constexpr float INV_F = 1.f / SEG;  // features per head (LayerNorm row length)
  constexpr bool GATHER = PairIo<T, SEG>::GATHER;  // q, k, v, out tiles moved by the threads instead of TMA

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw_u32);
  Xch4* xch = reinterpret_cast<Xch4*>(gbase + SM::OFF_XCH);
  const uint32_t bar0 = base + SM::OFF_BAR;

  const Lane L;
  const int tid = L.tid, lane = L.lane, g = L.g, t = L.t, nb = L.nb;
  const int hsel = L.warp >> 1;              // SEG = 32: which head of the pair this warp's columns belong to
  const int khalf = (SEG == 32) ? hsel : -1; // and the k-range of the state that is its own block
  const int stream = blockIdx.x;             // (batch, head) stream, or (batch, pair of heads) when SEG = 32
  const int head = stream % p.H;
  const int NS = p.NS;
  const int row_base = stream * p.T;  // first row of this stream in the [B*H*T, 64] view
  // inference launches pass no saved-state buffers: nothing is kept for a backward (no checkpoints, gradient tiles,
  // row statistics or per-stage biases are written)
  const bool save = (p.w_ckpt != nullptr);

  if (tid == 0) {
    if constexpr (!GATHER) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      prefetch_tmap(&tm_o);
    }
    prefetch_tmap(&tm_g);
    // arrivals per phase: thread 0's expect_tx, plus every thread's cp.async arrival where tiles are gathered
    for (int i = 0; i < FWD_NST; ++i) mbar_init(bar0 + 8 * i, GATHER ? 1 + NTHREADS : 1);
    fence_mbar_init();
  }
  if constexpr (MB < CS) {
    // padding rows of every tile of the ring, and the lr slots: zero once; the copies only ever write the first MB rows
    for (uint32_t e = tid * 16; e < FWD_NST * SM::SLOT; e += NTHREADS * 16) {
      const uint32_t in_tile = e % TF::BYTES;
      // raw tile: 16 rows of 128 bytes (bf16) or two halves of 16 rows of 128 bytes (f32); planes are derived from it
      const bool raw = in_tile < TF::RAW_BYTES;
      if (!raw || (in_tile % 2048) >= MB * 128)
        asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(base + e), "r"(0u) : "memory");
    }
    for (uint32_t e = tid * 4; e < FWD_NST * SM::LR_SLOT; e += NTHREADS * 4)
      asm volatile("st.shared.b32 [%0], %1;" ::"r"(base + SM::OFF_LR + e), "r"(0u) : "memory");
  }
  __syncthreads();

  // thread 0: TMA / bulk copies of one stage into its ring slot
  auto issue_loads = [&](int s) {
    const int slot = s % FWD_NST;
    const uint32_t bar = bar0 + 8 * slot;
    const uint32_t tq = base + slot * SM::SLOT;
    if constexpr (SEG == 64) {
      mbar_expect_tx(bar, (3 * TF::RAW_BYTES + CS * TF::ELT) * MB / CS);
      const int r0 = row_base + s * MB;
      tma_load_tile<T>(tq, &tm_q, r0, bar);
      tma_load_tile<T>(tq + TF::BYTES, &tm_k, r0, bar);
      tma_load_tile<T>(tq + 2 * TF::BYTES, &tm_v, r0, bar);
      bulk_load_1d(base + SM::OFF_LR + slot * 64,
                   static_cast<const uint8_t*>(p.lr) + (size_t)(row_base + s * MB) * TF::ELT, MB * TF::ELT, bar);
    } else {
      mbar_expect_tx(bar, ((GATHER ? 0 : 3 * TF::RAW_BYTES) + 2 * CS * TF::ELT) * MB / CS);
      if constexpr (!GATHER) {
        tma_load_pair<T>(tq, &tm_q, stream, s * MB, p.T, bar);
        tma_load_pair<T>(tq + TF::BYTES, &tm_k, stream, s * MB, p.T, bar);
        tma_load_pair<T>(tq + 2 * TF::BYTES, &tm_v, stream, s * MB, p.T, bar);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)  // ttt_lr_eta is [B, H, T]: the two heads of the pair are T elements apart
        bulk_load_1d(base + SM::OFF_LR + slot * SM::LR_SLOT + j * CS * TF::ELT,
                     static_cast<const uint8_t*>(p.lr) + ((size_t)(2 * stream + j) * p.T + s * MB) * TF::ELT,
                     MB * TF::ELT, bar);
    }
  };
  // every thread, where tiles are gathered: its 16-byte chunk of the q, k, v tiles, then its arrival on the barrier
  auto issue_gather = [&](int s) {
    if constexpr (GATHER) {
      const int slot = s % FWD_NST;
      const uint32_t tq = base + slot * SM::SLOT;
      gather_pair_tile_bf16<MB>(tq, tm_q.ptr, stream, s * MB, p.T, tid);
      gather_pair_tile_bf16<MB>(tq + TF::BYTES, tm_k.ptr, stream, s * MB, p.T, tid);
      gather_pair_tile_bf16<MB>(tq + 2 * TF::BYTES, tm_v.ptr, stream, s * MB, p.T, tid);
      cp_async_mbar_arrive_noinc(bar0 + 8 * slot);
    }
  };
  if (tid == 0) {
    for (int s = 0; s < FWD_NST && s < NS; ++s) issue_loads(s);
  }
  if constexpr (GATHER)
    for (int s = 0; s < FWD_NST && s < NS; ++s) issue_gather(s);

  // ---- per-thread constants: 4 owned columns c(nt,e) = nb + 8nt + 2t + e, rows g and g+8
  F2 gam[2], bet[2];
  float bias[4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    const int c = nb + 8 * nt + 2 * t;
    gam[nt] = f2(ld_as_float<T>(p.ln_g, (size_t)head * HD + c), ld_as_float<T>(p.ln_g, (size_t)head * HD + c + 1));
    bet[nt] = f2(ld_as_float<T>(p.ln_b, (size_t)head * HD + c), ld_as_float<T>(p.ln_b, (size_t)head * HD + c + 1));
    bias[2 * nt] = ld_as_float<T>(p.b0, (size_t)stream * HD + c);
    bias[2 * nt + 1] = ld_as_float<T>(p.b0, (size_t)stream * HD + c + 1);
  }
  // (MB = 8: rows 8..15 of every tile are padding -- zero K, Q, V, lr and token_eta, so they neither move the state
  // nor reach the output, and nothing of them is stored)
  const float te_row[2] = {ld_as_float<T>(p.token_eta, g), MB == CS ? ld_as_float<T>(p.token_eta, g + 8) : 0.f};
  const float te15 = ld_as_float<T>(p.token_eta, MB - 1);
  // The state is carried as What = W / wscale with wscale = -te15, so that the update W -= te15 Gp^T K becomes
  // What += Gp^T K, accumulated by the tensor cores straight into the registers.  (te15 == 0: W never changes.)
  const bool w_moves = (te15 != 0.f);
  const float wscale = w_moves ? -te15 : 1.f;
  const float winv = 1.f / wscale;

  // ---- state W^T[n][k], n in {nb+g, nb+g+8}: wt[kt][2*rn + e] = W[k = 8kt+2t+e][n = nb+g+8rn]
  float wt[8][4];
#pragma unroll
  for (int kt = 0; kt < 8; ++kt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = 8 * kt + 2 * t + (i & 1), n = nb + g + 8 * (i >> 1);
      if constexpr (SEG == 64) {
        wt[kt][i] = ld_as_float<T>(p.w0, (size_t)stream * HD * HD + k * HD + n) * winv;
      } else {
        // block-diagonal: head hsel's 32 x 32 state at rows / columns [32 hsel, 32 hsel + 32); zero elsewhere
        wt[kt][i] = ((kt >> 2) == hsel)
                        ? ld_as_float<T>(p.w0, (size_t)(2 * stream + hsel) * 32 * 32 + (k & 31) * 32 + (n & 31)) * winv
                        : 0.f;
      }
    }

  int xsel = 0;
  bool failed = false;
  // where the next checkpoint and the next per-stage bias record go, and the stages left until the next checkpoint
  float4* ck_ptr = save ? reinterpret_cast<float4*>(p.w_ckpt + (size_t)stream * (p.NCK + 1) * HD * HD) : nullptr;
  float* bs_ptr = save ? p.b_stage + (size_t)stream * (NS + 1) * HD : nullptr;
  int ck_left = 0;

  // One stage with its ring slot known at compile time, so every shared-memory address is a hoisted lane offset plus
  // an immediate.  Returns false after a timed-out wait.
  auto stage = [&](const int s, auto slot_tag) -> bool {
    constexpr int slot = decltype(slot_tag)::value;
    const uint32_t tq = base + slot * SM::SLOT, tk = tq + TF::BYTES, tv = tk + TF::BYTES;
    const uint32_t pq = tq + TF::PLANE_OFF, pk = tk + TF::PLANE_OFF;
    int fail = mbar_wait_bounded(bar0 + 8 * slot, (s / FWD_NST) & 1) ? 0 : 1;
    if constexpr (NP == 3) {
      if (!fail) {
        split_tile_f32(tq, tid);
        split_tile_f32(tk, tid);
      }
      fail = __syncthreads_or(fail);
      if (fail) {
        failed = true;
        if (tid == 0) report_timeout(p.status, 1, s);
        return false;
      }
    }

    // (SEG = 32: the pair's second head has its 16 values right after the first head's)
    const float lr_row[2] = {
        ld_as_float<T>(gbase + SM::OFF_LR + slot * SM::LR_SLOT, (SEG == 32 ? hsel * CS : 0) + g),
        ld_as_float<T>(gbase + SM::OFF_LR + slot * SM::LR_SLOT, (SEG == 32 ? hsel * CS : 0) + g + 8)};

    // ---- Z1 = K W + b, Zq = Q W + b (columns nb..nb+15), Attn = Q K^T (full 16x16, every warp)
    float z1[2][4], zq[2][4], at[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) z1[nt][i] = zq[nt][i] = at[nt][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      Pk<NP> bw[2][2];
      bfrag_from_state<NP>(wt, ks, bw);
      Pk<NP> ak[4], aq[4];
      ldsm_np<NP>(ak, pk + lane_off_A(lane, 16 * ks), TILE_BF16_BYTES, false);
      ldsm_np<NP>(aq, pq + lane_off_A(lane, 16 * ks), TILE_BF16_BYTES, false);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        mma_np<NP>(z1[nt], ak, bw[nt]);
        mma_np<NP>(zq[nt], aq, bw[nt]);
      }
      // the A fragments of K are also the B fragments of Q K^T (the same four 8x8 blocks in another order)
      const Pk<NP> bj0[2] = {ak[0], ak[2]}, bj1[2] = {ak[1], ak[3]};
      if (SEG == 64 || (ks >> 1) == hsel) {  // Q K^T contracts over the head's own features only
        mma_np<NP>(at[0], aq, bj0);
        mma_np<NP>(at[1], aq, bj1);
      }
    }
    // ---- saved state: W before the update of every K-th stage, the bias before every stage.  Issued behind the
    // products so that the stores' address arithmetic runs under the tensor cores' latency; the places are advanced
    // from stage to stage (no division by the runtime interval on the chain).
    if (save) {
      if (ck_left == 0) {
        // kept as the threads hold it (float4 kt of thread tid at [kt][tid]): eight coalesced 16-byte stores per
        // thread, read back the same way by the backward
#pragma unroll
        for (int kt = 0; kt < 8; ++kt)
          ck_ptr[kt * NTHREADS + tid] =
              make_float4(wt[kt][0] * wscale, wt[kt][1] * wscale, wt[kt][2] * wscale, wt[kt][3] * wscale);
        ck_ptr += HD * HD / 4;
        ck_left = p.K;
      }
      --ck_left;
      if (g == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) bs_ptr[nb + 8 * (j >> 1) + 2 * t + (j & 1)] = bias[j];
      }
      bs_ptr += HD;
    }

    // products were taken with What: Z = wscale * acc + b
    F2 z1p[2][2], zqp[2][2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const F2 b2 = f2(bias[2 * nt], bias[2 * nt + 1]);
        z1p[nt][r] = f2fma(pr(z1[nt], r), f2(wscale), b2);
        zqp[nt][r] = f2fma(pr(zq[nt], r), f2(wscale), b2);
      }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      zq[nt][0] = zqp[nt][0].x; zq[nt][1] = zqp[nt][0].y; zq[nt][2] = zqp[nt][1].x; zq[nt][3] = zqp[nt][1].y;
    }

    // ---- LN statistics of Z1, then G = dL/dZ1 and Gp = lr[row] * G
    float mean[2], rstd[2];
    ln_row_stats<TWO_PASS, SEG>(z1p, xch, xsel, L, p.eps, mean, rstd, fail);
    if (fail) {
      failed = true;
      if (tid == 0) report_timeout(p.status, 2, s);
      return false;
    }
    F2 gp[2][2];
    float4 st1[2];  // saved row statistics of Z1: (mean, rstd, mean(gx), mean(gx * x_hat))
    {
      F2 xh[2][2], gy[2][2], gx[2][2];
      float sa[2], sb[2];
      ln_l2_pieces<T>(z1p, mean, rstd, gam, bet, tk, tv, L, xh, gy, gx, sa, sb);
      float2 a0, a1;
      int f2_ = 0;
      xch_rows2<SEG, false>(&xch[xsel], L, sa[0], sb[0], sa[1], sb[1], a0, a1, f2_);
      xsel ^= 1;
      const float A[2] = {a0.x * INV_F, a1.x * INV_F}, Bv[2] = {a0.y * INV_F, a1.y * INV_F};
      const float rs[2] = {rstd[0] * lr_row[0], rstd[1] * lr_row[1]};
      g_from_pieces(gx, xh, A, Bv, rs, gp);
      st1[0] = make_float4(mean[0], rstd[0], A[0], Bv[0]);
      st1[1] = make_float4(mean[1], rstd[1], A[1], Bv[1]);
    }

    // ---- Gp as tensor-core operands, transposed through movmatrix: gt[nt][r] = (Gp block rows 8r.., cols nb+8nt..)^T
    // The same values go to the saved Gp tile the backward reads (bf16: exactly the operand bits used here).
    const uint32_t sg = base + SM::OFF_OUT + (2 + (s & 1)) * TF::RAW_BYTES;
    Pk<NP> gt[2][2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const Pk<NP> pkd = split_pack<NP>(gp[nt][r].x, gp[nt][r].y);
        if (save) {
          if constexpr (NP == 1) {
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(sg + off_bf16(g + 8 * r, nb + 8 * nt + 2 * t)), "r"(pkd.p[0]) : "memory");
          } else {
            st_pair<T>(sg, g + 8 * r, nb + 8 * nt + 2 * t, gp[nt][r].x, gp[nt][r].y);
          }
        }
        gt[nt][r] = movm_t_np<NP>(pkd);
      }

    // ---- Zbar = Zq - M' Gp,  M'[i][j] = te[i] (1 + Attn[i][j]) for j <= i
    {
      Pk<NP> am[4];
#pragma unroll
      for (int jt = 0; jt < 2; ++jt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int i = g + 8 * r, j = 8 * jt + 2 * t;
          const F2 m = f2fma(pr(at[jt], r), f2(-te_row[r]), f2(-te_row[r]));
          am[2 * jt + r] = split_pack<NP>((j <= i) ? m.x : 0.f, (j + 1 <= i) ? m.y : 0.f);
        }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const Pk<NP> bg[2] = {gt[nt][0], gt[nt][1]};
        mma_np<NP>(zq[nt], am, bg);
      }
    }

    // ---- state update: W^T[nb.., :] -= te15 * Gp^T K ; b -= te15 * colsum(Gp)
    {
      const Pk<NP> agt[4] = {gt[0][0], gt[1][0], gt[0][1], gt[1][1]};
      if (w_moves) state_update_direct<NP>(wt, agt, pk, lane, khalf);
      if constexpr (NP == 1) {
        // column sums of the bf16 Gp tile as a product with a tile of ones (every row of the result is the sum)
        constexpr uint32_t ONES = 0x3F803F80u;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          float cs[4] = {0.f, 0.f, 0.f, 0.f};
          mma_bf16(cs, ONES, ONES, ONES, ONES, gt[nt][0].p[0], gt[nt][1].p[0]);
          bias[2 * nt] -= te15 * cs[0];
          bias[2 * nt + 1] -= te15 * cs[1];
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const F2 cs = f2add(gp[nt][0], gp[nt][1]);
          bias[2 * nt] -= te15 * col_sum(cs.x);
          bias[2 * nt + 1] -= te15 * col_sum(cs.y);
        }
      }
    }

    // ---- out = Q + LN(Zbar)
    int fl2 = 0;
    F2 zb[2][2];
    slab_pairs(zq, zb);
    ln_row_stats<TWO_PASS, SEG, false>(zb, xch, xsel, L, p.eps, mean, rstd, fl2);
    if constexpr (SEG == 64) {
      if (save && L.warp == 0 && t == 0) {
        float4* sp = p.stats + ((size_t)row_base + (size_t)s * MB) * 2;
        sp[2 * g] = st1[0];
        sp[2 * g + 1] = make_float4(mean[0], rstd[0], 0.f, 0.f);
        if constexpr (MB == CS) {
          sp[2 * (g + 8)] = st1[1];
          sp[2 * (g + 8) + 1] = make_float4(mean[1], rstd[1], 0.f, 0.f);
        }
      }
    } else if (save && (L.warp & 1) == 0 && t == 0) {
      // two float4 per (token, head): record index 2 * token + head of the pair
      float4* sp = p.stats + ((size_t)row_base + (size_t)s * MB) * 4;
      sp[2 * (2 * g + hsel)] = st1[0];
      sp[2 * (2 * g + hsel) + 1] = make_float4(mean[0], rstd[0], 0.f, 0.f);
      if constexpr (MB == CS) {
        sp[2 * (2 * (g + 8) + hsel)] = st1[1];
        sp[2 * (2 * (g + 8) + hsel) + 1] = make_float4(mean[1], rstd[1], 0.f, 0.f);
      }
    }
    const uint32_t so = base + SM::OFF_OUT + (s & 1) * TF::RAW_BYTES;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r, col = nb + 8 * nt + 2 * t;
        const F2 x = f2mul(f2sub(zb[nt][r], f2(mean[r])), f2(rstd[r]));
        const F2 o = f2add(ld_pair<T>(tq, row, col), f2fma(gam[nt], x, bet[nt]));
        st_pair<T>(so, row, col, o.x, o.y);
      }
    fence_proxy_async_smem();
    __syncthreads();
    if constexpr (GATHER) scatter_pair_tile_bf16<MB>(tm_o.ptr, stream, s * MB, p.T, so, tid);
    if (tid == 0) {
      if constexpr (SEG == 64) tma_store_tile<T>(&tm_o, row_base + s * MB, so);
      else if constexpr (!GATHER) tma_store_pair<T>(&tm_o, stream, s * MB, p.T, so);
      if (save) tma_store_tile<T>(&tm_g, row_base + s * MB, sg);  // saved tiles are kept in the packed 64-wide form
      bulk_commit();
      bulk_wait_read<1>();
    }
    // (the next loads by the first thread of warp 1: thread 0 is busy with the stores, and a warp that does both
    // arrives at the next stage's first barrier that much later than the other three)
    if (tid == 32 && s + FWD_NST < NS) issue_loads(s + FWD_NST);
    if constexpr (GATHER)
      if (s + FWD_NST < NS) issue_gather(s + FWD_NST);
    return true;
  };
  for (int s0 = 0; s0 < NS; s0 += FWD_NST) {
    if (!stage(s0, std::integral_constant<int, 0>{})) break;
    if (s0 + 1 < NS && !stage(s0 + 1, std::integral_constant<int, 1>{})) break;
    if (s0 + 2 < NS && !stage(s0 + 2, std::integral_constant<int, 2>{})) break;
  }

  if (!failed) {
    // ---- final state (returned, and kept as the last checkpoint / last bias record for the backward)
    float4* wc = save ? reinterpret_cast<float4*>(p.w_ckpt + ((size_t)stream * (p.NCK + 1) + p.NCK) * HD * HD) : nullptr;
#pragma unroll
    for (int kt = 0; kt < 8; ++kt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = (8 * kt + 2 * t + (i & 1)) * HD + nb + g + 8 * (i >> 1);
        if constexpr (SEG == 64) {
          st_from_float<T>(p.w_out, (size_t)stream * HD * HD + idx, wt[kt][i] * wscale);
        } else if ((kt >> 2) == hsel) {
          // the head's own 32 x 32 block (rows and columns 32 hsel .. of the tile's state)
          st_from_float<T>(p.w_out, (size_t)(2 * stream + hsel) * 32 * 32 + ((idx >> 6) & 31) * 32 + (idx & 31),
                           wt[kt][i] * wscale);
        }
        if (save && i == 3)
          wc[kt * NTHREADS + tid] =
              make_float4(wt[kt][0] * wscale, wt[kt][1] * wscale, wt[kt][2] * wscale, wt[kt][3] * wscale);
      }
    if (g == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = nb + 8 * (j >> 1) + 2 * t + (j & 1);
        st_from_float<T>(p.b_out, (size_t)stream * HD + c, bias[j]);
        if (save) p.b_stage[((size_t)stream * (NS + 1) + NS) * HD + c] = bias[j];
      }
    }
  }
  if (tid == 0) bulk_wait_all<0>();
  if constexpr (GATHER) cp_async_wait_all();  // (a stage that gave up may leave gathers in flight)
}

template <typename T, int SEG, int MB>
static cudaError_t launch_fwd_t(const CUtensorMap* m, const void* const* io, const LinFwdParams& p, int nstreams,
                                cudaStream_t st) {
  using SM = FwdSmem<T, SEG>;
  auto kfn = ttt_linear_fwd_kernel<T, SEG, MB>;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM::DYN_BYTES);
  if (e != cudaSuccess) return e;
  if constexpr (PairIo<T, SEG>::GATHER) {
    kfn<<<nstreams, NTHREADS, SM::DYN_BYTES, st>>>(RawTensor{const_cast<void*>(io[0])}, RawTensor{const_cast<void*>(io[1])},
                                                   RawTensor{const_cast<void*>(io[2])},
                                                   RawTensor{const_cast<void*>(io[3])}, m[4], p);
  } else {
    kfn<<<nstreams, NTHREADS, SM::DYN_BYTES, st>>>(m[0], m[1], m[2], m[3], m[4], p);
  }
  return cudaGetLastError();
}

template <typename T, int SEG>
static cudaError_t launch_fwd_mb(int mb, const CUtensorMap* m, const void* const* io, const LinFwdParams& p,
                                 int nstreams, cudaStream_t st) {
  return mb == 8 ? launch_fwd_t<T, SEG, 8>(m, io, p, nstreams, st) : launch_fwd_t<T, SEG, 16>(m, io, p, nstreams, st);
}

// mb: tokens per mini-batch, 16 or 8 (the maps' boxes then have 8 rows)
cudaError_t launch_linear_fwd(int dtype, int seg, int mb, const CUtensorMap* maps, const void* const* io,
                              const LinFwdParams& p, int nstreams, cudaStream_t st) {
  if (seg == 32) {
    if (dtype == 1) return launch_fwd_mb<__nv_bfloat16, 32>(mb, maps, io, p, nstreams, st);
    return launch_fwd_mb<float, 32>(mb, maps, io, p, nstreams, st);
  }
  if (dtype == 1) return launch_fwd_mb<__nv_bfloat16, 64>(mb, maps, io, p, nstreams, st);
  return launch_fwd_mb<float, 64>(mb, maps, io, p, nstreams, st);
}

}  // namespace ttt
