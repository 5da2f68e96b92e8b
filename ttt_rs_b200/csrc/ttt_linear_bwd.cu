// Fused TTT-Linear backward scan for sm_100a: one 4-warp CTA per (batch, head) stream walks the mini-batches in
// reverse, recomputing what it needs from the forward's checkpoints.
//
// What it computes is the reference's multi-stage backward kernel
// (rust/fused/src/linear_fused_tile/backward/kernel.rs:254-429 with the stage body backward/stage.rs:42-1006 and the
// LN + L2 second derivative layer_norm.rs:429-709): gradients of sum(grad_output * output) w.r.t. xq, xk, xv,
// the initial state (per batch element), ttt_lr_eta, token_eta, and the LayerNorm weight/bias; gradients flowing
// into the returned final state are zero (launch.rs:188-194).
//
// How it is organised here (none of this follows the reference's design):
//   * Checkpoint groups are walked last to first.  A group (or sub-group of SG stages when the checkpoint interval
//     is larger) is first re-simulated forward ONCE from its checkpoint; each simulated stage leaves in shared
//     memory the lr-scaled LN gradient Gp (as tensor-core operand planes), its four row statistics and the stage's
//     bias.  The reference instead re-simulates from the checkpoint for every stage.
//   * The state W^T and its gradient dW^T stay in registers as float32 accumulators (warp w owns rows n in
//     [16w,16w+16)).  Walking back, W_s is recovered from W_{s+1} by re-applying the stage's rank-16 update with the
//     opposite sign from the stashed Gp, so no per-stage copy of W is kept anywhere.
//   * Products contracting over the feature axis that is split across warps (dZ.W^T, G.dW^T) read bf16 copies of
//     W_s / dW and of the dZ tiles from shared memory; all other operands chain through registers
//     (accumulator -> A fragment, movmatrix for transposes).
//   * The three gradients that the reference accumulates with float atomics (token_eta, LN weight/bias) are written as
//     per-stream partials to a workspace and summed by a second kernel in a fixed order, so results are
//     bitwise reproducible.
#include "ttt_kernels.h"
#include "ttt_stage.cuh"

#ifndef TTT_BWD_SG_BF16
#define TTT_BWD_SG_BF16 16  // stages stashed per re-simulation pass (bf16 I/O)
#endif
#ifndef TTT_BWD_MINB_BF16
#define TTT_BWD_MINB_BF16 2  // resident blocks per SM the bf16 kernel is compiled for
#endif

namespace ttt {

template <typename T>
struct BwdSmem {
  using TF = TileFmt<T>;
  static constexpr int NP = TF::NP;
  static constexpr int SG = (sizeof(T) == 2) ? TTT_BWD_SG_BF16 : 8;  // stages stashed per re-simulation pass
  static constexpr int NSLOT = 2;
  static constexpr uint32_t PLANES = NP * TILE_BF16_BYTES;             // one operand tile
  static constexpr uint32_t OFF_Q = 0, OFF_K = TF::BYTES, OFF_V = 2 * TF::BYTES, OFF_DO = 2 * TF::BYTES + TF::RAW_BYTES;
  static constexpr uint32_t SLOT = 2 * TF::BYTES + 2 * TF::RAW_BYTES;  // q, k (raw+planes), v, d_out (raw)
  static constexpr uint32_t OFF_STASH = NSLOT * SLOT;                  // SG operand tiles of Gp
  static constexpr uint32_t OFF_W = OFF_STASH + SG * PLANES;           // W_s^T, 4 sub-tiles [16 n][64 k]
  static constexpr uint32_t OFF_DW = OFF_W + 4 * PLANES;               // dW^T, same layout
  static constexpr uint32_t OFF_DZ = OFF_DW + 4 * PLANES;              // dZbar operand tile
  static constexpr uint32_t OFF_DZ1 = OFF_DZ + PLANES;                 // dZ1 operand tile
  static constexpr uint32_t OFF_OUT = OFF_DZ1 + PLANES;                // staging: dq, dk, dv (raw format)
  static constexpr uint32_t OFF_STAT = OFF_OUT + 3 * TF::RAW_BYTES;    // SG x 16 rows x float4 (mean, rstd, A, Bv)
  static constexpr uint32_t OFF_BIAS = OFF_STAT + SG * 256;            // SG x 64 floats
  static constexpr uint32_t OFF_LR = OFF_BIAS + SG * 256;              // NSLOT x 64 bytes
  static constexpr uint32_t OFF_XCH = OFF_LR + NSLOT * 64;             // 2 x Xch4
  static constexpr uint32_t OFF_BAR = OFF_XCH + 2 * sizeof(Xch4);
  static constexpr uint32_t TOTAL = OFF_BAR + NSLOT * 8;
  static constexpr uint32_t DYN_BYTES = TOTAL + 1024;
};

// Order in which stages are visited: for each checkpoint group (last first), for each sub-group of SG stages
// (last first): simulate stages g0..e-1 forward (stashing those >= a), then run the backward of stages e-1..a.
struct OpIter {
  int K, NS, SG;
  int gi, si, g0, g1, a, e, s;
  bool sim, done, first;
  __device__ __forceinline__ void start_sub() {
    a = g0 + si * SG;
    e = min(a + SG, g1);
    sim = true;
    s = g0;
    first = true;
  }
  __device__ __forceinline__ void start_group() {
    g0 = gi * K;
    g1 = min(g0 + K, NS);
    si = (g1 - g0 + SG - 1) / SG - 1;
    start_sub();
  }
  __device__ __forceinline__ void init(int K_, int NS_, int NCK, int SG_) {
    K = K_;
    NS = NS_;
    SG = SG_;
    gi = NCK - 1;
    done = false;
    start_group();
  }
  __device__ __forceinline__ void next() {
    if (done) return;
    first = false;
    if (sim) {
      if (s + 1 < e) {
        ++s;
      } else {
        sim = false;
        s = e - 1;
      }
    } else if (s > a) {
      --s;
    } else if (si > 0) {
      --si;
      start_sub();
    } else if (gi > 0) {
      --gi;
      start_group();
    } else {
      done = true;
    }
  }
};

template <typename T>
__global__ void __launch_bounds__(NTHREADS, (sizeof(T) == 2 ? TTT_BWD_MINB_BF16 : 1))
    ttt_linear_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                          const __grid_constant__ CUtensorMap tm_dq, const __grid_constant__ CUtensorMap tm_dk,
                          const __grid_constant__ CUtensorMap tm_dv, const LinBwdParams p) {
  using TF = TileFmt<T>;
  using SM = BwdSmem<T>;
  constexpr int NP = TF::NP;
  constexpr bool TWO_PASS = (sizeof(T) == 4);
  constexpr uint32_t PL = TILE_BF16_BYTES;  // plane stride

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw_u32);
  Xch4* xch = reinterpret_cast<Xch4*>(gbase + SM::OFF_XCH);
  float4* stat = reinterpret_cast<float4*>(gbase + SM::OFF_STAT);  // [SG][16]
  float* bstash = reinterpret_cast<float*>(gbase + SM::OFF_BIAS);  // [SG][64]
  const uint32_t bar0 = base + SM::OFF_BAR;
  const uint32_t tW = base + SM::OFF_W, tDW = base + SM::OFF_DW, tDZ = base + SM::OFF_DZ, tDZ1 = base + SM::OFF_DZ1;

  const Lane L;
  const int tid = L.tid, lane = L.lane, g = L.g, t = L.t, nb = L.nb, warp = L.warp;
  const int stream = blockIdx.x;
  const int head = stream % p.H;
  const int row_base = stream * p.T;

  if (tid == 0) {
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
    prefetch_tmap(&tm_do);
    prefetch_tmap(&tm_dq);
    prefetch_tmap(&tm_dk);
    prefetch_tmap(&tm_dv);
    for (int i = 0; i < SM::NSLOT; ++i) mbar_init(bar0 + 8 * i, 1);
    fence_mbar_init();
  }
  __syncthreads();

  // loads of one visit: K, V, lr always; Q and d_out only for a backward visit
  auto issue_loads = [&](int n, int s, bool sim) {
    const int slot = n % SM::NSLOT;
    const uint32_t bar = bar0 + 8 * slot;
    const uint32_t sl = base + slot * SM::SLOT;
    const int r0 = row_base + s * CS;
    mbar_expect_tx(bar, (sim ? 2u : 4u) * TF::RAW_BYTES + CS * TF::ELT);
    tma_load_tile<T>(sl + SM::OFF_K, &tm_k, r0, bar);
    tma_load_tile<T>(sl + SM::OFF_V, &tm_v, r0, bar);
    if (!sim) {
      tma_load_tile<T>(sl + SM::OFF_Q, &tm_q, r0, bar);
      tma_load_tile<T>(sl + SM::OFF_DO, &tm_do, r0, bar);
    }
    bulk_load_1d(base + SM::OFF_LR + slot * 64, static_cast<const uint8_t*>(p.lr) + (size_t)r0 * TF::ELT,
                 CS * TF::ELT, bar);
  };

  OpIter cur, ahead;
  cur.init(p.K, p.NS, p.NCK, SM::SG);
  ahead = cur;
  if (tid == 0) issue_loads(0, ahead.s, ahead.sim);
  ahead.next();

  // ---- per-thread constants and accumulators (4 owned columns, rows g and g+8)
  float gam[4], bet[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = nb + 8 * (j >> 1) + 2 * t + (j & 1);
    gam[j] = ld_as_float<T>(p.ln_g, (size_t)head * HD + c);
    bet[j] = ld_as_float<T>(p.ln_b, (size_t)head * HD + c);
  }
  const float te_row[2] = {ld_as_float<T>(p.token_eta, g), ld_as_float<T>(p.token_eta, g + 8)};
  const float te15 = ld_as_float<T>(p.token_eta, CS - 1);
  float bias[4] = {0.f, 0.f, 0.f, 0.f};
  float dbias[4] = {0.f, 0.f, 0.f, 0.f};                                    // gradient w.r.t. the bias after this stage
  float dgam[4] = {0.f, 0.f, 0.f, 0.f}, dbet[4] = {0.f, 0.f, 0.f, 0.f};     // un-reduced over the 8 row lanes
  float wt[8][4], dwt[8][4];
#pragma unroll
  for (int kt = 0; kt < 8; ++kt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      wt[kt][i] = 0.f;
      dwt[kt][i] = 0.f;
    }

  int xsel = 0;
  bool failed = false;
  int n = 0;  // visit counter (slot = n % NSLOT)

  // `ahead` stays exactly one visit in front of `cur`; its loads are issued during the current visit
  for (; !cur.done; cur.next(), ahead.next(), ++n) {
    const int s = cur.s;
    const int slot = n % SM::NSLOT;
    const uint32_t sl = base + slot * SM::SLOT;
    const uint32_t tq = sl + SM::OFF_Q, tk = sl + SM::OFF_K, tv = sl + SM::OFF_V, tdo = sl + SM::OFF_DO;
    const uint32_t pq = tq + TF::PLANE_OFF, pk = tk + TF::PLANE_OFF;
    const int j = s - cur.a;  // stash index (valid when s >= a)
    const uint32_t tG = base + SM::OFF_STASH + (uint32_t)(j < 0 ? 0 : j) * SM::PLANES;

    if (cur.first) {
      // state at the group's checkpoint (float32)
      const size_t ck = (size_t)stream * p.NCK + cur.gi;
      const float* wc = p.w_ckpt + ck * HD * HD;
#pragma unroll
      for (int kt = 0; kt < 8; ++kt)
#pragma unroll
        for (int i = 0; i < 4; ++i) wt[kt][i] = wc[(8 * kt + 2 * t + (i & 1)) * HD + nb + g + 8 * (i >> 1)];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) bias[jj] = p.b_ckpt[ck * HD + nb + 8 * (jj >> 1) + 2 * t + (jj & 1)];
    }

    int fail = mbar_wait_bounded(bar0 + 8 * slot, (n / SM::NSLOT) & 1) ? 0 : 1;
    bool next_issued = false;
    auto issue_next = [&]() {
      // runs right after the first CTA barrier of this visit: every thread has left the previous visit,
      // so the other slot may be overwritten
      if (!next_issued) {
        next_issued = true;
        if (tid == 0 && !ahead.done) issue_loads(n + 1, ahead.s, ahead.sim);
      }
    };
    if constexpr (NP == 3) {
      if (!fail) {
        split_tile_f32(tk, tid);
        if (!cur.sim) split_tile_f32(tq, tid);
      }
      fail = __syncthreads_or(fail);
      if (fail) {
        failed = true;
        if (tid == 0) report_timeout(p.status, 11, s);
        break;
      }
      issue_next();
    }
    const float lr_row[2] = {ld_as_float<T>(gbase + SM::OFF_LR + slot * 64, g),
                             ld_as_float<T>(gbase + SM::OFF_LR + slot * 64, g + 8)};

    if (cur.sim) {
      // =========================== forward re-simulation of stage s ===========================
      float z1[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) z1[nt][i] = bias[2 * nt + (i & 1)];
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        Pk<NP> bw[2][2], ak[4];
        bfrag_from_state<NP>(wt, ks, bw);
        ldsm_np<NP>(ak, pk + lane_off_A(lane, 16 * ks), PL, false);
        mma_np<NP>(z1[0], ak, bw[0]);
        mma_np<NP>(z1[1], ak, bw[1]);
      }
      float mean[2], rstd[2];
      ln_row_stats<TWO_PASS>(z1, xch, xsel, L, p.eps, mean, rstd, fail);
      if (fail) {
        failed = true;
        if (tid == 0) report_timeout(p.status, 12, s);
        break;
      }
      issue_next();
      float gp[2][4];
      {
        float xh[2][4], gy[2][4], gx[2][4], sa[2], sb[2];
        ln_l2_pieces<T>(z1, mean, rstd, gam, bet, tk, tv, L, xh, gy, gx, sa, sb);
        float2 a0, a1;
        int f2 = 0;
        xch_rows2(&xch[xsel], L, sa[0], sb[0], sa[1], sb[1], a0, a1, f2);
        xsel ^= 1;
        const float A[2] = {a0.x * (1.f / HD), a1.x * (1.f / HD)}, Bv[2] = {a0.y * (1.f / HD), a1.y * (1.f / HD)};
        g_from_pieces(gx, xh, A, Bv, rstd, gp);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) gp[nt][i] *= lr_row[i >> 1];
        if (j >= 0) {
          if (warp == 0 && t == 0) {
            stat[j * CS + g] = make_float4(mean[0], rstd[0], A[0], Bv[0]);
            stat[j * CS + g + 8] = make_float4(mean[1], rstd[1], A[1], Bv[1]);
          }
          if (g == 0) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) bstash[j * HD + nb + 8 * (jj >> 1) + 2 * t + (jj & 1)] = bias[jj];
          }
        }
      }
      Pk<NP> gt[2][2];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const Pk<NP> pkd = split_pack<NP>(gp[nt][2 * r], gp[nt][2 * r + 1]);
          if (j >= 0) {
            const uint32_t a = tG + off_bf16(g + 8 * r, nb + 8 * nt + 2 * t);
#pragma unroll
            for (int pp = 0; pp < NP; ++pp) asm volatile("st.shared.b32 [%0], %1;" ::"r"(a + pp * PL), "r"(pkd.p[pp]) : "memory");
          }
          gt[nt][r] = movm_t_np<NP>(pkd);
        }
      {
        const Pk<NP> agt[4] = {gt[0][0], gt[1][0], gt[0][1], gt[1][1]};
        state_update<NP>(wt, agt, pk, lane, -te15);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) bias[2 * nt + e] -= te15 * col_sum(gp[nt][e] + gp[nt][2 + e]);
      }
      continue;
    }

    // =============================== backward of stage s ===============================
    // ---- 1. W_s from W_{s+1}: undo the stage's update with the stashed Gp; b_s from the stash
    {
      Pk<NP> agt[4];
      ldsm_np<NP>(agt, tG + lane_off_B_nk(lane, nb), PL, true);
      state_update<NP>(wt, agt, pk, lane, te15);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) bias[jj] = bstash[j * HD + nb + 8 * (jj >> 1) + 2 * t + (jj & 1)];
    }
    // ---- 2. operand copies of W_s^T and dW^T (this warp's 16 rows) for the products that contract over n
#pragma unroll
    for (int kt = 0; kt < 8; ++kt)
#pragma unroll
      for (int rn = 0; rn < 2; ++rn) {
        st_pair_planes<NP>(tW + warp * SM::PLANES, g + 8 * rn, 8 * kt + 2 * t, wt[kt][2 * rn], wt[kt][2 * rn + 1]);
        st_pair_planes<NP>(tDW + warp * SM::PLANES, g + 8 * rn, 8 * kt + 2 * t, dwt[kt][2 * rn], dwt[kt][2 * rn + 1]);
      }
    // ---- 3. Z1 = K W + b, Zq = Q W + b, KdW = K dW, Attn = Q K^T
    float z1[2][4], zq[2][4], kdw[2][4], at[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        z1[nt][i] = bias[2 * nt + (i & 1)];
        zq[nt][i] = bias[2 * nt + (i & 1)];
        kdw[nt][i] = 0.f;
        at[nt][i] = 0.f;
      }
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      Pk<NP> bw[2][2], bdw[2][2], ak[4], aq[4], bk[4];
      bfrag_from_state<NP>(wt, ks, bw);
      bfrag_from_state<NP>(dwt, ks, bdw);
      ldsm_np<NP>(ak, pk + lane_off_A(lane, 16 * ks), PL, false);
      ldsm_np<NP>(aq, pq + lane_off_A(lane, 16 * ks), PL, false);
      ldsm_np<NP>(bk, pk + lane_off_B_nk(lane, 16 * ks), PL, false);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        mma_np<NP>(z1[nt], ak, bw[nt]);
        mma_np<NP>(zq[nt], aq, bw[nt]);
        mma_np<NP>(kdw[nt], ak, bdw[nt]);
      }
      const Pk<NP> bj0[2] = {bk[0], bk[1]}, bj1[2] = {bk[2], bk[3]};
      mma_np<NP>(at[0], aq, bj0);
      mma_np<NP>(at[1], aq, bj1);
    }
    // ---- 4. LN + L2 pieces of Z1 from the stashed row statistics
    float mean1[2], rstd1[2], Bv1[2];
    float xh[2][4], gy[2][4], gx[2][4], G[2][4];
    {
      const float4 st0 = stat[j * CS + g], st1 = stat[j * CS + g + 8];
      mean1[0] = st0.x; rstd1[0] = st0.y; mean1[1] = st1.x; rstd1[1] = st1.y;
      const float A[2] = {st0.z, st1.z};
      Bv1[0] = st0.w; Bv1[1] = st1.w;
      float sa[2], sb[2];
      ln_l2_pieces<T>(z1, mean1, rstd1, gam, bet, tk, tv, L, xh, gy, gx, sa, sb);
      g_from_pieces(gx, xh, A, Bv1, rstd1, G);
    }
    // ---- 5. Zbar = Zq - M' Gp   (am holds -M')
    Pk<NP> am[4];
#pragma unroll
    for (int jt = 0; jt < 2; ++jt)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int i = g + 8 * r, jj = 8 * jt + 2 * t;
        const float m0 = (jj <= i) ? -te_row[r] * (1.f + at[jt][2 * r]) : 0.f;
        const float m1 = (jj + 1 <= i) ? -te_row[r] * (1.f + at[jt][2 * r + 1]) : 0.f;
        am[2 * jt + r] = split_pack<NP>(m0, m1);
      }
    {
      Pk<NP> bg[4];
      ldsm_np<NP>(bg, tG + lane_off_B_kn(lane, nb), PL, true);
      const Pk<NP> b0[2] = {bg[0], bg[1]}, b1[2] = {bg[2], bg[3]};
      mma_np<NP>(zq[0], am, b0);
      mma_np<NP>(zq[1], am, b1);
    }
    // ---- 6. LN statistics of Zbar; 7. LN backward of the output -> dZbar
    float dzb[2][4], dzsum[4];
    float dq[2][4];
    {
      float mean2[2], rstd2[2];
      ln_row_stats<TWO_PASS>(zq, xch, xsel, L, p.eps, mean2, rstd2, fail);
      if (fail) {
        failed = true;
        if (tid == 0) report_timeout(p.status, 13, s);
        break;
      }
      issue_next();
      float s1[2] = {0.f, 0.f}, s2[2] = {0.f, 0.f};
      float tt[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float2 dv = ld_pair<T>(tdo, g + 8 * r, nb + 8 * nt + 2 * t);
          const float d[2] = {dv.x, dv.y};
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int i = 2 * r + e, jj = 2 * nt + e;
            const float xz = (zq[nt][i] - mean2[r]) * rstd2[r];
            zq[nt][i] = xz;  // keep x_hat of Zbar
            dq[nt][i] = d[e];
            dgam[jj] += d[e] * xz;
            dbet[jj] += d[e];
            const float tv_ = d[e] * gam[jj];
            tt[nt][i] = tv_;
            s1[r] += tv_;
            s2[r] += tv_ * xz;
          }
        }
      float2 a0, a1;
      int f2 = 0;
      xch_rows2(&xch[xsel], L, s1[0], s2[0], s1[1], s2[1], a0, a1, f2);
      xsel ^= 1;
      const float c1[2] = {a0.x * (1.f / HD), a1.x * (1.f / HD)}, c2[2] = {a0.y * (1.f / HD), a1.y * (1.f / HD)};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = i >> 1;
          dzb[nt][i] = (tt[nt][i] - c1[r] - zq[nt][i] * c2[r]) * rstd2[r];
        }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) dzsum[jj] = dzb[jj >> 1][jj & 1] + dzb[jj >> 1][2 + (jj & 1)];
    }
    // ---- 8. dZbar to shared memory as an operand tile; barrier also publishes tW / tDW
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 2; ++r)
        st_pair_planes<NP>(tDZ, g + 8 * r, nb + 8 * nt + 2 * t, dzb[nt][2 * r], dzb[nt][2 * r + 1]);
    __syncthreads();

    // ---- 9. products that need dZbar
    float pp[2][4], gl[2][4], dk[2][4], dgp[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) pp[nt][i] = gl[nt][i] = dk[nt][i] = dgp[nt][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      Pk<NP> adz[4], bgn[4], bwt[4], ags[4], bdw[4];
      ldsm_np<NP>(adz, tDZ + lane_off_A(lane, 16 * ks), PL, false);
      ldsm_np<NP>(bgn, tG + lane_off_B_nk(lane, 16 * ks), PL, false);
      ldsm_np<NP>(bwt, tW + ks * SM::PLANES + lane_off_B_kn(lane, nb), PL, true);
      ldsm_np<NP>(ags, tG + lane_off_A(lane, 16 * ks), PL, false);
      ldsm_np<NP>(bdw, tDW + ks * SM::PLANES + lane_off_B_kn(lane, nb), PL, true);
      {  // P' = dZbar Gp^T (16x16)
        const Pk<NP> b0[2] = {bgn[0], bgn[1]}, b1[2] = {bgn[2], bgn[3]};
        mma_np<NP>(pp[0], adz, b0);
        mma_np<NP>(pp[1], adz, b1);
      }
      {  // dq += dZbar W^T (columns nb..nb+15)
        const Pk<NP> b0[2] = {bwt[0], bwt[1]}, b1[2] = {bwt[2], bwt[3]};
        mma_np<NP>(dq[0], adz, b0);
        mma_np<NP>(dq[1], adz, b1);
      }
      {  // Gl' = Gp dW^T (columns nb..nb+15)
        const Pk<NP> b0[2] = {bdw[0], bdw[1]}, b1[2] = {bdw[2], bdw[3]};
        mma_np<NP>(gl[0], ags, b0);
        mma_np<NP>(gl[1], ags, b1);
      }
    }
    // dM' = -tril(P');  dA = dM' o te[i];  d te[i] = sum_j dM'[i,j] (1 + Attn[i,j])
    float dte_row[2] = {0.f, 0.f};
    Pk<NP> ada[4];
#pragma unroll
    for (int jt = 0; jt < 2; ++jt)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int i = g + 8 * r, jj = 8 * jt + 2 * t;
        const float d0 = (jj <= i) ? -pp[jt][2 * r] : 0.f;
        const float d1 = (jj + 1 <= i) ? -pp[jt][2 * r + 1] : 0.f;
        dte_row[r] += d0 * (1.f + at[jt][2 * r]) + d1 * (1.f + at[jt][2 * r + 1]);
        ada[2 * jt + r] = split_pack<NP>(d0 * te_row[r], d1 * te_row[r]);
      }
    dte_row[0] = quad_sum(dte_row[0]);
    dte_row[1] = quad_sum(dte_row[1]);
    {
      Pk<NP> bkt[4], bqt[4], bdz[4];
      ldsm_np<NP>(bkt, pk + lane_off_B_kn(lane, nb), PL, true);
      ldsm_np<NP>(bqt, pq + lane_off_B_kn(lane, nb), PL, true);
      ldsm_np<NP>(bdz, tDZ + lane_off_B_kn(lane, nb), PL, true);
      const Pk<NP> adat[4] = {movm_t_np<NP>(ada[0]), movm_t_np<NP>(ada[2]), movm_t_np<NP>(ada[1]), movm_t_np<NP>(ada[3])};
      const Pk<NP> amt[4] = {movm_t_np<NP>(am[0]), movm_t_np<NP>(am[2]), movm_t_np<NP>(am[1]), movm_t_np<NP>(am[3])};
      const Pk<NP> k0[2] = {bkt[0], bkt[1]}, k1[2] = {bkt[2], bkt[3]};
      const Pk<NP> q0[2] = {bqt[0], bqt[1]}, q1[2] = {bqt[2], bqt[3]};
      const Pk<NP> z0[2] = {bdz[0], bdz[1]}, zz1[2] = {bdz[2], bdz[3]};
      mma_np<NP>(dq[0], ada, k0);  // dq += dA K
      mma_np<NP>(dq[1], ada, k1);
      mma_np<NP>(dk[0], adat, q0);  // dk = dA^T Q
      mma_np<NP>(dk[1], adat, q1);
      mma_np<NP>(dgp[0], amt, z0);  // dGp = -M'^T dZbar
      mma_np<NP>(dgp[1], amt, zz1);
    }
    // dW^T += dZbar^T Q
    {
      Pk<NP> adzt[4];
      ldsm_np<NP>(adzt, tDZ + lane_off_B_nk(lane, nb), PL, true);
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {
        Pk<NP> bq[4];
        ldsm_np<NP>(bq, pq + lane_off_B_kn(lane, 16 * kp), PL, true);
        const Pk<NP> b0[2] = {bq[0], bq[1]}, b1[2] = {bq[2], bq[3]};
        mma_np<NP>(dwt[2 * kp], adzt, b0);
        mma_np<NP>(dwt[2 * kp + 1], adzt, b1);
      }
    }
    // ---- 10. gradient reaching Gp, the lr / token_eta terms, and the first pair of second-derivative sums
    float u[2][4], v[2][4];
    float s1t[2], s2t[2];
    {
      float p1[2] = {0.f, 0.f}, p2[2] = {0.f, 0.f}, dl[2] = {0.f, 0.f}, rt[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float2 kv = ld_pair<T>(tk, g + 8 * r, nb + 8 * nt + 2 * t);
          const float kk[2] = {kv.x, kv.y};
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int i = 2 * r + e, jj = 2 * nt + e;
            const float dg = dgp[nt][i] - te15 * (kdw[nt][i] + dbias[jj]);  // dL/dGp
            dk[nt][i] -= te15 * gl[nt][i];
            rt[r] += kk[e] * gl[nt][i] + (lr_row[r] * G[nt][i]) * dbias[jj];
            dl[r] += dg * G[nt][i];
            const float uu = lr_row[r] * dg;  // dL/dG
            const float vv = -uu * rstd1[r];
            u[nt][i] = uu;
            v[nt][i] = vv;
            p1[r] += vv;
            p2[r] += vv * xh[nt][i];
          }
        }
      float4 o0, o1;
      int f2 = 0;
      xch_rows(&xch[xsel], L, make_float4(p1[0], p2[0], dl[0], rt[0]), make_float4(p1[1], p2[1], dl[1], rt[1]), o0, o1, f2);
      xsel ^= 1;
      s1t[0] = o0.x * (1.f / HD); s2t[0] = o0.y * (1.f / HD);
      s1t[1] = o1.x * (1.f / HD); s2t[1] = o1.y * (1.f / HD);
      const float rt_all = col_sum(o0.w + o1.w);  // sum over the 16 rows
      if (warp == 0 && t == 0) {
        const size_t o = (size_t)row_base + (size_t)s * CS;
        st_from_float<T>(p.d_lr, o + g, o0.z);
        st_from_float<T>(p.d_lr, o + g + 8, o1.z);
        p.part_te[o + g] = dte_row[0];
        p.part_te[o + g + 8] = dte_row[1] - (g == 7 ? rt_all : 0.f);
      }
    }
    // ---- 11. second derivative through LN + L2 gradient -> dZ1, dT
    float dz1[2][4], dT[2][4];
    {
      float pd[2] = {0.f, 0.f}, ps[2] = {0.f, 0.f};
      float dxh[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = i >> 1, jj = 2 * nt + (i & 1);
          const float dgxh = -v[nt][i] + s1t[r] + xh[nt][i] * s2t[r];
          const float dy = gam[jj] * dgxh;
          dgam[jj] += gy[nt][i] * dgxh + dy * xh[nt][i];
          dbet[jj] += dy;
          const float dx = dy * gam[jj] + gx[nt][i] * s2t[r] + v[nt][i] * Bv1[r];
          dxh[nt][i] = dx;
          dT[nt][i] = -dy;
          pd[r] += dx;
          ps[r] -= (dx * xh[nt][i] + u[nt][i] * G[nt][i]) * rstd1[r];
        }
      float2 a0, a1;
      int f2 = 0;
      xch_rows2(&xch[xsel], L, pd[0], ps[0], pd[1], ps[1], a0, a1, f2);
      xsel ^= 1;
      const float D[2] = {a0.x * (1.f / HD), a1.x * (1.f / HD)}, S[2] = {a0.y * (1.f / HD), a1.y * (1.f / HD)};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = i >> 1;
          dz1[nt][i] = (dxh[nt][i] - D[r]) * rstd1[r] + xh[nt][i] * S[r];
        }
    }
    // ---- 12. dZ1 to shared memory as an operand tile
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 2; ++r)
        st_pair_planes<NP>(tDZ1, g + 8 * r, nb + 8 * nt + 2 * t, dz1[nt][2 * r], dz1[nt][2 * r + 1]);
    if (tid == 0) bulk_wait_read<0>();  // the previous stage's output tiles have left the staging buffers
    __syncthreads();
    // ---- 13. dk += dZ1 W^T ; dW^T += dZ1^T K ; bias gradient
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      Pk<NP> adz1[4], bwt[4];
      ldsm_np<NP>(adz1, tDZ1 + lane_off_A(lane, 16 * ks), PL, false);
      ldsm_np<NP>(bwt, tW + ks * SM::PLANES + lane_off_B_kn(lane, nb), PL, true);
      const Pk<NP> b0[2] = {bwt[0], bwt[1]}, b1[2] = {bwt[2], bwt[3]};
      mma_np<NP>(dk[0], adz1, b0);
      mma_np<NP>(dk[1], adz1, b1);
    }
    {
      Pk<NP> adzt[4];
      ldsm_np<NP>(adzt, tDZ1 + lane_off_B_nk(lane, nb), PL, true);
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {
        Pk<NP> bk[4];
        ldsm_np<NP>(bk, pk + lane_off_B_kn(lane, 16 * kp), PL, true);
        const Pk<NP> b0[2] = {bk[0], bk[1]}, b1[2] = {bk[2], bk[3]};
        mma_np<NP>(dwt[2 * kp], adzt, b0);
        mma_np<NP>(dwt[2 * kp + 1], adzt, b1);
      }
    }
#pragma unroll
    for (int jj = 0; jj < 4; ++jj)
      dbias[jj] += col_sum(dzsum[jj] + dz1[jj >> 1][jj & 1] + dz1[jj >> 1][2 + (jj & 1)]);
    // ---- 14. outputs: dq = d_out + ..., dk = -dT + ..., dv = dT
    {
      const uint32_t so_q = base + SM::OFF_OUT, so_k = so_q + TF::RAW_BYTES, so_v = so_k + TF::RAW_BYTES;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int row = g + 8 * r, col = nb + 8 * nt + 2 * t;
          st_pair<T>(so_q, row, col, dq[nt][2 * r], dq[nt][2 * r + 1]);
          st_pair<T>(so_k, row, col, dk[nt][2 * r] - dT[nt][2 * r], dk[nt][2 * r + 1] - dT[nt][2 * r + 1]);
          st_pair<T>(so_v, row, col, dT[nt][2 * r], dT[nt][2 * r + 1]);
        }
      fence_proxy_async_smem();
      __syncthreads();
      if (tid == 0) {
        const int r0 = row_base + s * CS;
        tma_store_tile<T>(&tm_dq, r0, so_q);
        tma_store_tile<T>(&tm_dk, r0, so_k);
        tma_store_tile<T>(&tm_dv, r0, so_v);
        bulk_commit();
      }
    }
  }

  if (!failed) {
    // ---- gradients w.r.t. the initial state (per batch element) and per-stream partials for the reduction
    const size_t wo = (size_t)stream * HD * HD;
#pragma unroll
    for (int kt = 0; kt < 8; ++kt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = (8 * kt + 2 * t + (i & 1)) * HD + nb + g + 8 * (i >> 1);
        st_from_float<T>(p.d_w, wo + idx, dwt[kt][i]);
        if (p.part_w != nullptr) p.part_w[(size_t)stream * (HD * HD + HD) + idx] = dwt[kt][i];
      }
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const float dg_ = col_sum(dgam[jj]), db_ = col_sum(dbet[jj]);
      if (g == 0) {
        const int c = nb + 8 * (jj >> 1) + 2 * t + (jj & 1);
        st_from_float<T>(p.d_b, (size_t)stream * HD + c, dbias[jj]);
        if (p.part_w != nullptr) p.part_w[(size_t)stream * (HD * HD + HD) + HD * HD + c] = dbias[jj];
        p.part_ln[(size_t)stream * 2 * HD + c] = dg_;
        p.part_ln[(size_t)stream * 2 * HD + HD + c] = db_;
      }
    }
  }
  if (tid == 0) bulk_wait_all<0>();
}

// ----------------------------------------------------------------------------------------------------
// Second pass: fixed-order sums of the per-stream partials.
//   d_token_eta[t]   = sum over streams of part_te[stream][t]
//   d_ln_w/b[h][f]   = sum over batch of part_ln[b*H+h][0/1][f]
//   packed (optional) = { sum_b dW[b,h], sum_b db[b,h], d_ln_w, d_ln_b, d_token_eta folded to [CS] }
//                       (the fold is a second tiny kernel over the reduced d_token_eta)
// ----------------------------------------------------------------------------------------------------
__global__ void ttt_linear_bwd_reduce_kernel(const ReduceParams p) {
  const int H = p.H, B = p.B, T = p.T;
  const int n_te = T, n_ln = 2 * H * HD, n_w = (p.packed != nullptr) ? H * (HD * HD + HD) : 0;
  const int total = n_te + n_ln + n_w;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    if (i < n_te) {
      float acc = 0.f;
      for (int st = 0; st < B * H; ++st) acc += p.part_te[(size_t)st * T + i];
      p.d_token_eta[i] = acc;
    } else if (i < n_te + n_ln) {
      const int k = i - n_te, which = k / (H * HD), hf = k % (H * HD), h = hf / HD, f = hf % HD;
      float acc = 0.f;
      for (int b = 0; b < B; ++b) acc += p.part_ln[((size_t)(b * H + h) * 2 + which) * HD + f];
      (which == 0 ? p.d_ln_g : p.d_ln_b)[hf] = acc;
      if (p.packed != nullptr) p.packed[(size_t)H * HD * HD + H * HD + k] = acc;
    } else {
      const int k = i - n_te - n_ln;
      const bool is_w = k < H * HD * HD;
      const int h = is_w ? k / (HD * HD) : (k - H * HD * HD) / HD;
      const int e = is_w ? k % (HD * HD) : HD * HD + (k - H * HD * HD) % HD;
      float acc = 0.f;
      for (int b = 0; b < B; ++b) acc += p.part_w[(size_t)(b * H + h) * (HD * HD + HD) + e];
      p.packed[k] = acc;
    }
  }
}

// token_eta gradient folded over stages into [CS] (runs after the kernel above, same stream): one warp per
// mini-batch position, lanes stride over stages, fixed-order shuffle tree.
__global__ void ttt_linear_bwd_fold_kernel(const ReduceParams p) {
  const int c = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float acc = 0.f;
  for (int s = lane; s < p.T / CS; s += 32) acc += p.d_token_eta[s * CS + c];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) p.packed[(size_t)p.H * HD * HD + 3 * p.H * HD + c] = acc;
}

template <typename T>
static cudaError_t launch_bwd_t(const CUtensorMap* m, const LinBwdParams& p, int nstreams, cudaStream_t st) {
  auto kfn = ttt_linear_bwd_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BwdSmem<T>::DYN_BYTES);
  if (e != cudaSuccess) return e;
  kfn<<<nstreams, NTHREADS, BwdSmem<T>::DYN_BYTES, st>>>(m[0], m[1], m[2], m[3], m[4], m[5], m[6], p);
  return cudaGetLastError();
}

cudaError_t launch_linear_bwd(int dtype, const CUtensorMap* maps, const LinBwdParams& p, int nstreams,
                              cudaStream_t st) {
  if (dtype == 1) return launch_bwd_t<__nv_bfloat16>(maps, p, nstreams, st);
  return launch_bwd_t<float>(maps, p, nstreams, st);
}

cudaError_t launch_linear_bwd_reduce(const ReduceParams& p, cudaStream_t st) {
  const int total = p.T + 2 * p.H * HD + (p.packed != nullptr ? p.H * (HD * HD + HD) : 0);
  const int threads = 128;
  int blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ttt_linear_bwd_reduce_kernel<<<blocks, threads, 0, st>>>(p);
  if (p.packed != nullptr) ttt_linear_bwd_fold_kernel<<<1, CS * 32, 0, st>>>(p);
  return cudaGetLastError();
}

}  // namespace ttt
