// Fused TTT-Linear backward scan for sm_100a: one 4-warp CTA per (batch, head) stream walks the mini-batches in
// reverse.
//
// What it computes is the reference's multi-stage backward kernel
// (rust/fused/src/linear_fused_tile/backward/kernel.rs:254-429 with the stage body backward/stage.rs:42-1006 and the
// LN + L2 second derivative layer_norm.rs:429-709): gradients of sum(grad_output * output) w.r.t. xq, xk, xv,
// the initial state (per batch element), ttt_lr_eta, token_eta, and the LayerNorm weight/bias; gradients flowing
// into the returned final state are zero (launch.rs:188-194).
//
// How it is organised here (none of this follows the reference's design):
//   * No forward re-simulation.  The forward saved, per stage, the lr-scaled LN gradient tile Gp (the operand of its
//     state update), four + two row statistics per token and the bias; per checkpoint interval it saved W in float32
//     (and the final W).  Walking back, W_s is recovered in registers from W_{s+1} by re-applying the stage's rank-16
//     update from Gp with the opposite sign; at every checkpoint boundary W is re-read exactly, which bounds the
//     rounding drift of the reversal to one interval.  (The reference re-simulates the forward from the checkpoint
//     for every stage, backward/kernel.rs:339-382.)
//   * The state W^T and its gradient dW^T stay in registers as float32 accumulators (warp w owns rows n in
//     [16w,16w+16)).  Products contracting over the feature axis that is split across warps (dZ.W^T, Gp.dW^T) read bf16
//     copies of W_s / dW and of the dZ tiles from shared memory; all other operands chain through registers
//     (accumulator -> A fragment, movmatrix for transposes).
//   * Element-wise math runs on column pairs with packed float32x2 instructions.
//   * The three gradients that the reference accumulates with float atomics (token_eta, LN weight/bias) are written as
//     per-stream partials to a workspace and summed by a second kernel in a fixed order, so results are
//     bitwise reproducible.
//
// head_dim 32 (SEG = 32): as in the forward, a CTA takes a pair of heads side by side in the 64-wide tiles with
// block-diagonal W^T and dW^T; the row sums, Q.K^T, dZbar.Gp^T and the k-ranges of the rank-16 updates are restricted
// to the head's own 32 columns, and everything written per head (ttt_lr_eta gradient, token_eta terms, state
// gradients) goes to the head's own place in the caller's [B, H, ...] tensors.
#include "ttt_kernels.h"
#include "ttt_stage.cuh"

namespace ttt {

template <typename T, int SEG>
struct BwdSmem {
  using TF = TileFmt<T>;
  static constexpr int NP = TF::NP;
  static constexpr int NSLOT = 2;
  static constexpr uint32_t PLANES = NP * TILE_BF16_BYTES;  // one operand tile
  // one slot = the tiles of one stage: q, k, gp (raw + operand planes), v, d_out (raw), then small records
  static constexpr uint32_t OFF_Q = 0, OFF_K = TF::BYTES, OFF_G = 2 * TF::BYTES, OFF_V = 3 * TF::BYTES;
  static constexpr uint32_t OFF_DO = OFF_V + TF::RAW_BYTES;
  static constexpr uint32_t STAT_BYTES = (SEG == 32) ? 1024 : 512;  // 16 tokens x 2 float4 (x 2 heads when paired)
  static constexpr uint32_t OFF_STAT = OFF_DO + TF::RAW_BYTES;
  static constexpr uint32_t OFF_BS = OFF_STAT + STAT_BYTES;     // 64 floats: bias at the start of the stage
  static constexpr uint32_t OFF_LR = OFF_BS + 256;              // 16 x element (x 2 heads when paired)
  static constexpr uint32_t SLOT = OFF_STAT + 2 * STAT_BYTES;   // (keeps every tile 1024-byte aligned)
  static constexpr uint32_t OFF_W = NSLOT * SLOT;               // W_s^T, 4 sub-tiles [16 n][64 k]
  static constexpr uint32_t OFF_DW = OFF_W + 4 * PLANES;        // dW^T, same layout
  static constexpr uint32_t OFF_DZ = OFF_DW + 4 * PLANES;       // dZbar operand tile
  static constexpr uint32_t OFF_DZ1 = OFF_DZ + PLANES;          // dZ1 operand tile
  static constexpr uint32_t OFF_OUT = OFF_DZ1 + PLANES;         // staging: dq, dk, dv (raw format)
  static constexpr uint32_t OFF_XCH = OFF_OUT + 3 * TF::RAW_BYTES;
  static constexpr uint32_t OFF_BAR = OFF_XCH + 2 * sizeof(Xch4);
  static constexpr uint32_t TOTAL = OFF_BAR + NSLOT * 8;
  static constexpr uint32_t DYN_BYTES = TOTAL + 1024;
};

#ifndef TTT_BWD_MINB_BF16
#define TTT_BWD_MINB_BF16 2  // resident blocks per SM the bf16 kernel is compiled for
#endif

template <typename T, int SEG, int MB>
__global__ void __launch_bounds__(NTHREADS, (sizeof(T) == 2 ? TTT_BWD_MINB_BF16 : 1))
    ttt_linear_bwd_kernel(const __grid_constant__ typename PairIo<T, SEG>::Ref tm_q,
                          const __grid_constant__ typename PairIo<T, SEG>::Ref tm_k,
                          const __grid_constant__ typename PairIo<T, SEG>::Ref tm_v,
                          const __grid_constant__ typename PairIo<T, SEG>::Ref tm_do,
                          const __grid_constant__ typename PairIo<T, SEG>::Ref tm_dq,
                          const __grid_constant__ typename PairIo<T, SEG>::Ref tm_dk,
                          const __grid_constant__ typename PairIo<T, SEG>::Ref tm_dv,
                          const __grid_constant__ CUtensorMap tm_g, const LinBwdParams p) {
  using TF = TileFmt<T>;
  using SM = BwdSmem<T, SEG>;
  constexpr int NP = TF::NP;
  constexpr uint32_t PL = TILE_BF16_BYTES;  // plane stride
  constexpr float INV_F = 1.f / SEG;        // features per head (LayerNorm row length)
  constexpr int NH = (SEG == 32) ? 2 : 1;   // heads per tile
  // The loads of the next stage are issued by the first thread of warp 1, the stores (and their bulk groups) by thread
  // 0: one warp doing both arrives at the stage's barriers that much later than the other three.
  constexpr int LOADER = 32;
  constexpr bool GATHER = PairIo<T, SEG>::GATHER;  // q, k, v, d_out, d_q, d_k, d_v tiles moved by the threads, not TMA

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw_u32);
  Xch4* xch = reinterpret_cast<Xch4*>(gbase + SM::OFF_XCH);
  const uint32_t bar0 = base + SM::OFF_BAR;
  const uint32_t tW = base + SM::OFF_W, tDW = base + SM::OFF_DW, tDZ = base + SM::OFF_DZ, tDZ1 = base + SM::OFF_DZ1;

  const Lane L;
  const int tid = L.tid, lane = L.lane, g = L.g, t = L.t, nb = L.nb, warp = L.warp;
  const int hsel = warp >> 1;                 // SEG = 32: which head of the pair this warp's columns belong to
  const int khalf = (SEG == 32) ? hsel : -1;  // and the k-range of W^T / dW^T that is its own block
  const int NS = p.NS;
  // work item = (stream, chunk of CH stages); set per item below
  int stream = 0, row_base = 0;
  __shared__ int s_item;
  // W^T and dW^T (32 + 32 float32 words per thread) are parked in tensor memory between the places of a stage that use
  // them (see tmem_ld_8x4), so that they do not occupy 64 registers through the middle of the stage.  64 columns per
  // block, freed by the warp that allocated them after the item loop, where every way out of the loop ends.
  __shared__ uint32_t s_tmem;
  if (warp == 0) tmem_alloc(smem_u32(&s_tmem), 64);
  tmem_fence_before_sync();
  __syncthreads();
  tmem_fence_after_sync();
  const uint32_t tm_w = s_tmem + ((32u * (uint32_t)warp) << 16), tm_dw = tm_w + 32u;

  if (tid == 0) {
    if constexpr (!GATHER) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      prefetch_tmap(&tm_do);
    }
    prefetch_tmap(&tm_g);
    if constexpr (!GATHER) {
      prefetch_tmap(&tm_dq);
      prefetch_tmap(&tm_dk);
      prefetch_tmap(&tm_dv);
    }
    // arrivals per phase: thread 0's expect_tx, plus every thread's cp.async arrival where tiles are gathered
    for (int i = 0; i < SM::NSLOT; ++i) mbar_init(bar0 + 8 * i, GATHER ? 1 + NTHREADS : 1);
    fence_mbar_init();
  }
  if constexpr (MB < CS) {
    // padding rows of every tile of both slots, and of the statistics and lr records: zero once; the copies only ever
    // write the first MB rows / records
    for (uint32_t e = tid * 4; e < SM::NSLOT * SM::SLOT; e += NTHREADS * 4) {
      const uint32_t o = e % SM::SLOT;
      bool pad = false;
      if (o < 3 * TF::BYTES) {  // q, k, gp: raw tile, then operand planes derived from it
        const uint32_t in_tile = o % TF::BYTES;
        pad = in_tile >= TF::RAW_BYTES || (in_tile % 2048) >= MB * 128;
      } else if (o < SM::OFF_STAT) {  // v, d_out: raw tiles
        pad = ((o - 3 * TF::BYTES) % 2048) >= MB * 128;
      } else if (o < SM::OFF_BS) {
        pad = (o - SM::OFF_STAT) >= MB * 32 * NH;
      } else if (o >= SM::OFF_LR) {
        pad = ((o - SM::OFF_LR) % (CS * TF::ELT)) >= MB * TF::ELT;
      }
      if (pad) asm volatile("st.shared.b32 [%0], %1;" ::"r"(base + e), "r"(0u) : "memory");
    }
  }
  __syncthreads();

  // everything stage s needs, into slot n % NSLOT (thread 0: TMA / bulk copies)
  auto issue_loads = [&](int n, int s) {
    const int slot = n % SM::NSLOT;
    const uint32_t bar = bar0 + 8 * slot;
    const uint32_t sl = base + slot * SM::SLOT;
    const int r0 = row_base + s * MB;
    if constexpr (SEG == 64) {
      mbar_expect_tx(bar, (5u * TF::RAW_BYTES + 512u + CS * TF::ELT) * MB / CS + 256u);
      tma_load_tile<T>(sl + SM::OFF_K, &tm_k, r0, bar);
      tma_load_tile<T>(sl + SM::OFF_G, &tm_g, r0, bar);
      tma_load_tile<T>(sl + SM::OFF_Q, &tm_q, r0, bar);
      tma_load_tile<T>(sl + SM::OFF_V, &tm_v, r0, bar);
      tma_load_tile<T>(sl + SM::OFF_DO, &tm_do, r0, bar);
      bulk_load_1d(sl + SM::OFF_STAT, p.stats + (size_t)r0 * 2, 512u * MB / CS, bar);
      bulk_load_1d(sl + SM::OFF_BS, p.b_stage + ((size_t)stream * (NS + 1) + s) * HD, 256u, bar);
      bulk_load_1d(sl + SM::OFF_LR, static_cast<const uint8_t*>(p.lr) + (size_t)r0 * TF::ELT, MB * TF::ELT, bar);
    } else {
      mbar_expect_tx(bar, ((GATHER ? 1u : 5u) * TF::RAW_BYTES + 1024u + 2 * CS * TF::ELT) * MB / CS + 256u);
      tma_load_tile<T>(sl + SM::OFF_G, &tm_g, r0, bar);  // saved tiles are kept in the packed 64-wide form
      if constexpr (!GATHER) {
        tma_load_pair<T>(sl + SM::OFF_K, &tm_k, stream, s * MB, p.T, bar);
        tma_load_pair<T>(sl + SM::OFF_Q, &tm_q, stream, s * MB, p.T, bar);
        tma_load_pair<T>(sl + SM::OFF_V, &tm_v, stream, s * MB, p.T, bar);
        tma_load_pair<T>(sl + SM::OFF_DO, &tm_do, stream, s * MB, p.T, bar);
      }
      bulk_load_1d(sl + SM::OFF_STAT, p.stats + (size_t)r0 * 4, 1024u * MB / CS, bar);
      bulk_load_1d(sl + SM::OFF_BS, p.b_stage + ((size_t)stream * (NS + 1) + s) * HD, 256u, bar);
#pragma unroll
      for (int j = 0; j < 2; ++j)  // ttt_lr_eta is [B, H, T]: the two heads of the pair are T elements apart
        bulk_load_1d(sl + SM::OFF_LR + j * CS * TF::ELT,
                     static_cast<const uint8_t*>(p.lr) + ((size_t)(2 * stream + j) * p.T + s * MB) * TF::ELT,
                     MB * TF::ELT, bar);
    }
  };
  // every thread, where tiles are gathered: its 16-byte chunk of the k, q, v, d_out tiles, then its arrival
  auto issue_gather = [&](int n, int s) {
    if constexpr (GATHER) {
      const int slot = n % SM::NSLOT;
      const uint32_t sl = base + slot * SM::SLOT;
      gather_pair_tile_bf16<MB>(sl + SM::OFF_K, tm_k.ptr, stream, s * MB, p.T, tid);
      gather_pair_tile_bf16<MB>(sl + SM::OFF_Q, tm_q.ptr, stream, s * MB, p.T, tid);
      gather_pair_tile_bf16<MB>(sl + SM::OFF_V, tm_v.ptr, stream, s * MB, p.T, tid);
      gather_pair_tile_bf16<MB>(sl + SM::OFF_DO, tm_do.ptr, stream, s * MB, p.T, tid);
      cp_async_mbar_arrive_noinc(bar0 + 8 * slot);
    }
  };

  // ---- per-thread constants and accumulators (column pairs nt = 0,1; rows g and g+8)
  F2 gam[2], bet[2];
  // (MB = 8: rows 8..15 of every tile are padding -- zero operands, statistics, lr and token_eta, so every value
  // derived from them is finite and multiplies a zero; nothing of them is stored)
  const float te_row[2] = {ld_as_float<T>(p.token_eta, g), MB == CS ? ld_as_float<T>(p.token_eta, g + 8) : 0.f};
  const float te15 = ld_as_float<T>(p.token_eta, MB - 1);
  // as in the forward, the state is carried as What = W / wscale (wscale = -te15), which turns the reversal of a
  // stage's update into one tensor-core accumulation What -= Gp^T K
  const bool w_moves = (te15 != 0.f);
  const float wscale = w_moves ? -te15 : 1.f;
  const float winv = 1.f / wscale;
  F2 dbias[2] = {f2(0.f), f2(0.f)};                                 // gradient w.r.t. the bias after this stage
  F2 dgam[2] = {f2(0.f), f2(0.f)}, dbet[2] = {f2(0.f), f2(0.f)};    // un-reduced over the 8 row lanes
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
  int n = 0;  // stages visited by this block so far (TMA slot = n % NSLOT)
  const int nitems = p.nstreams * p.NCH;
  const size_t HOFF = 2 * HD * HD + HD;

  // Persistent block: items are handed out in increasing order, last chunks of all streams first.  An item only
  // waits for an item with a smaller index (the later chunk of the same stream), which was taken by a block that runs
  // or has finished (a block takes an item only once it runs), so the wait graph has no cycle and the launch cannot
  // deadlock, whether or not every block of the grid is resident.
  while (!failed) {
    if (tid == 0) s_item = atomicAdd(&p.sched[0], 1);
    __syncthreads();
    const int item = s_item + p.item_base;
    __syncthreads();
    if (item >= nitems) break;
    const int crank = item / p.nstreams;  // 0 = last chunk of the sequence
    const int chunk = p.NCH - 1 - crank;
    stream = item - crank * p.nstreams;
    row_base = stream * p.T;
    const int head = stream % p.H;
    const int s_lo = chunk * p.CH, s_hi = min(s_lo + p.CH, NS) - 1;
    if (tid == LOADER) issue_loads(n, s_hi);
    issue_gather(n, s_hi);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int c = nb + 8 * nt + 2 * t;
      gam[nt] = f2(ld_as_float<T>(p.ln_g, (size_t)head * HD + c), ld_as_float<T>(p.ln_g, (size_t)head * HD + c + 1));
      bet[nt] = f2(ld_as_float<T>(p.ln_b, (size_t)head * HD + c), ld_as_float<T>(p.ln_b, (size_t)head * HD + c + 1));
      dgam[nt] = dbet[nt] = f2(0.f);
    }
    float* ho = p.handoff + (size_t)stream * HOFF;
    if (crank == 0) {
      // gradient flowing into the final state: zero (the reference's behaviour) unless the caller supplies it
      dbias[0] = dbias[1] = f2(0.f);
#pragma unroll
      for (int kt = 0; kt < 8; ++kt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if constexpr (SEG == 64) {
            dwt[kt][i] = (p.dw_in == nullptr)
                             ? 0.f
                             : ld_as_float<T>(p.dw_in, (size_t)stream * HD * HD + (8 * kt + 2 * t + (i & 1)) * HD + nb +
                                                           g + 8 * (i >> 1));
          } else {
            // the head's own 32 x 32 block of the pair's block-diagonal dW^T; zero elsewhere
            const int k = 8 * kt + 2 * t + (i & 1), nn = nb + g + 8 * (i >> 1);
            dwt[kt][i] = (p.dw_in == nullptr || (kt >> 2) != hsel)
                             ? 0.f
                             : ld_as_float<T>(p.dw_in, (size_t)(2 * stream + hsel) * 32 * 32 + (k & 31) * 32 + (nn & 31));
          }
        }
      if (p.db_in != nullptr) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const size_t o = (size_t)stream * HD + nb + 8 * nt + 2 * t;
          dbias[nt] = f2(ld_as_float<T>(p.db_in, o), ld_as_float<T>(p.db_in, o + 1));
        }
      }
    } else {
      // wait (bounded) until the later chunk of this stream has published its hand-off
      int ok = 1;
      if (tid == 0) {
        ok = 0;
        const volatile int* flag = p.sched + 1 + stream;
        for (uint32_t it = 0; it < p.handoff_polls; ++it) {
          if (*flag >= crank) {
            ok = 1;
            break;
          }
          __nanosleep(100);
        }
        __threadfence();
      }
      if (__syncthreads_or(ok ? 0 : 1)) {
        failed = true;
        if (tid == 0) report_timeout(p.status, 15, s_hi);
        // the loads of stage s_hi are in flight into this block's shared memory: let them land before leaving
        mbar_wait_bounded(bar0 + 8 * (n % SM::NSLOT), (n / SM::NSLOT) & 1);
        break;
      }
#pragma unroll
      for (int kt = 0; kt < 8; ++kt) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(ho) + kt * NTHREADS + tid);
        const float4 b = __ldcg(reinterpret_cast<const float4*>(ho + HD * HD) + kt * NTHREADS + tid);
        wt[kt][0] = a.x; wt[kt][1] = a.y; wt[kt][2] = a.z; wt[kt][3] = a.w;
        dwt[kt][0] = b.x; dwt[kt][1] = b.y; dwt[kt][2] = b.z; dwt[kt][3] = b.w;
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
        dbias[nt] = __ldcg(reinterpret_cast<const float2*>(ho + 2 * HD * HD + nb + 8 * nt + 2 * t));
    }

  tmem_st_8x4(tm_w, wt);
  tmem_st_8x4(tm_dw, dwt);

  // the next stage (walking down) that ends a checkpoint interval, and the checkpoint that holds the state after it
  // (kept from stage to stage: no division by the runtime interval on the chain)
  int ck_idx = s_hi / p.K + 1;
  int s_ck = min(ck_idx * p.K, NS) - 1;
  if (s_ck != s_hi) {
    --ck_idx;
    s_ck = ck_idx * p.K - 1;
  }
  for (int s = s_hi; s >= s_lo; --s, ++n) {
    const int slot = n % SM::NSLOT;
    const uint32_t sl = base + slot * SM::SLOT;
    const uint32_t tq = sl + SM::OFF_Q, tk = sl + SM::OFF_K, tg = sl + SM::OFF_G, tv = sl + SM::OFF_V, tdo = sl + SM::OFF_DO;
    const uint32_t pq = tq + TF::PLANE_OFF, pk = tk + TF::PLANE_OFF, pg = tg + TF::PLANE_OFF;
    const uint8_t* gsl = gbase + slot * SM::SLOT;

    // ---- the state after this stage, out of tensor memory
    tmem_wait_st();
    tmem_ld_8x4(tm_dw, dwt);
    if (s != s_ck) tmem_ld_8x4(tm_w, wt);
    // ---- at the last stage of a checkpoint interval: exact state after the stage (= next checkpoint / final W)
    if (s == s_ck) {
      // stored by the forward as its threads held it: float4 kt of thread tid at [kt][tid]
      const float4* wc =
          reinterpret_cast<const float4*>(p.w_ckpt + ((size_t)stream * (p.NCK + 1) + ck_idx) * HD * HD);
#pragma unroll
      for (int kt = 0; kt < 8; ++kt) {
        const float4 v = __ldcg(wc + kt * NTHREADS + tid);
        wt[kt][0] = v.x * winv; wt[kt][1] = v.y * winv; wt[kt][2] = v.z * winv; wt[kt][3] = v.w * winv;
      }
      --ck_idx;
      s_ck = ck_idx * p.K - 1;  // (the last interval of the sequence may be shorter than the others)
    }

    int fail = mbar_wait_bounded(bar0 + 8 * slot, (n / SM::NSLOT) & 1) ? 0 : 1;
    bool next_issued = false;
    auto issue_next = [&]() {
      // runs right after the first CTA barrier of this stage: every thread has left the previous stage,
      // so the other slot may be overwritten
      if (!next_issued) {
        next_issued = true;
        if (tid == LOADER && s > s_lo) issue_loads(n + 1, s - 1);
        if (GATHER && s > s_lo) issue_gather(n + 1, s - 1);
      }
    };
    if constexpr (NP == 3) {
      if (!fail) {
        split_tile_f32(tk, tid);
        split_tile_f32(tq, tid);
        split_tile_f32(tg, tid);
      }
      fail = __syncthreads_or(fail);
      if (fail) {
        failed = true;
        if (tid == 0) report_timeout(p.status, 11, s);
        break;
      }
      issue_next();
    }
    // (SEG = 32: the pair's second head has its 16 values right after the first head's)
    const float lr_row[2] = {ld_as_float<T>(gsl + SM::OFF_LR, (SEG == 32 ? hsel * CS : 0) + g),
                             ld_as_float<T>(gsl + SM::OFF_LR, (SEG == 32 ? hsel * CS : 0) + g + 8)};
    const float4* stat = reinterpret_cast<const float4*>(gsl + SM::OFF_STAT);
    const float* bsv = reinterpret_cast<const float*>(gsl + SM::OFF_BS);

    // ---- 1. W_s from W_{s+1}: undo the stage's update with the saved Gp; b_s as saved
    float bias[4];
    {
      Pk<NP> agt[4];
      if (w_moves) {
        ldsm_np<NP>(agt, pg + lane_off_B_nk(lane, nb), PL, true);
        const Pk<NP> ngt[4] = {neg_pk<NP>(agt[0]), neg_pk<NP>(agt[1]), neg_pk<NP>(agt[2]), neg_pk<NP>(agt[3])};
        state_update_direct<NP>(wt, ngt, pk, lane, khalf);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float2 b2 = *reinterpret_cast<const float2*>(bsv + nb + 8 * nt + 2 * t);
        bias[2 * nt] = b2.x;
        bias[2 * nt + 1] = b2.y;
      }
    }
    // ---- 2. operand copies of W_s^T and dW^T (this warp's 16 rows) for the products that contract over n
#pragma unroll
    for (int kt = 0; kt < 8; ++kt)
#pragma unroll
      for (int rn = 0; rn < 2; ++rn) {
        st_pair_planes<NP>(tW + warp * SM::PLANES, g + 8 * rn, 8 * kt + 2 * t, wt[kt][2 * rn] * wscale,
                           wt[kt][2 * rn + 1] * wscale);
        st_pair_planes<NP>(tDW + warp * SM::PLANES, g + 8 * rn, 8 * kt + 2 * t, dwt[kt][2 * rn], dwt[kt][2 * rn + 1]);
      }
    // ---- 3. Z1 = K W + b, Zq = Q W + b, KdW = K dW, Attn = Q K^T
    float z1[2][4], zq[2][4], kdw[2][4], at[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) z1[nt][i] = zq[nt][i] = kdw[nt][i] = at[nt][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      Pk<NP> bw[2][2], bdw[2][2], ak[4], aq[4];
      bfrag_from_state<NP>(wt, ks, bw);
      bfrag_from_state<NP>(dwt, ks, bdw);
      ldsm_np<NP>(ak, pk + lane_off_A(lane, 16 * ks), PL, false);
      ldsm_np<NP>(aq, pq + lane_off_A(lane, 16 * ks), PL, false);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        mma_np<NP>(z1[nt], ak, bw[nt]);
        mma_np<NP>(zq[nt], aq, bw[nt]);
        mma_np<NP>(kdw[nt], ak, bdw[nt]);
      }
      // the A fragments of K are also the B fragments of Q K^T (the same four 8x8 blocks in another order)
      const Pk<NP> bj0[2] = {ak[0], ak[2]}, bj1[2] = {ak[1], ak[3]};
      if (SEG == 64 || (ks >> 1) == hsel) {  // Q K^T contracts over the head's own features only
        mma_np<NP>(at[0], aq, bj0);
        mma_np<NP>(at[1], aq, bj1);
      }
    }
    tmem_st_8x4(tm_w, wt);  // W_s^T: next used by the stage below (dW^T is unchanged so far: nothing to store)
    // products were taken with What: Z = wscale * acc + b
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        z1[nt][i] = fmaf(z1[nt][i], wscale, bias[2 * nt + (i & 1)]);
        zq[nt][i] = fmaf(zq[nt][i], wscale, bias[2 * nt + (i & 1)]);
      }
    // ---- 4. LN + L2 pieces of Z1 from the saved row statistics
    float mean1[2], rstd1[2], Bv1[2], mean2[2], rstd2[2];
    F2 xh[2][2], gy[2][2], gx[2][2], G[2][2];
    {
      // records of rows g and g + 8 (SEG = 32: of this warp's head; record index 2 * token + head)
      const int rg = (SEG == 32) ? 2 * g + hsel : g, rg8 = (SEG == 32) ? 2 * (g + 8) + hsel : g + 8;
      const float4 sa0 = stat[2 * rg], sb0 = stat[2 * rg + 1], sa1 = stat[2 * rg8], sb1 = stat[2 * rg8 + 1];
      mean1[0] = sa0.x; rstd1[0] = sa0.y; mean1[1] = sa1.x; rstd1[1] = sa1.y;
      const float A[2] = {sa0.z, sa1.z};
      Bv1[0] = sa0.w; Bv1[1] = sa1.w;
      mean2[0] = sb0.x; rstd2[0] = sb0.y; mean2[1] = sb1.x; rstd2[1] = sb1.y;
      F2 z1p[2][2];
      slab_pairs(z1, z1p);
      float sa[2], sb[2];
      ln_l2_pieces<T>(z1p, mean1, rstd1, gam, bet, tk, tv, L, xh, gy, gx, sa, sb);
      g_from_pieces(gx, xh, A, Bv1, rstd1, G);
    }
    // ---- 5. Zbar = Zq - M' Gp   (am holds -M')
    Pk<NP> am[4];
#pragma unroll
    for (int jt = 0; jt < 2; ++jt)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int i = g + 8 * r, jj = 8 * jt + 2 * t;
        const F2 m = f2fma(pr(at[jt], r), f2(-te_row[r]), f2(-te_row[r]));
        am[2 * jt + r] = split_pack<NP>((jj <= i) ? m.x : 0.f, (jj + 1 <= i) ? m.y : 0.f);
      }
    {
      Pk<NP> bg[4];
      ldsm_np<NP>(bg, pg + lane_off_B_kn(lane, nb), PL, true);
      const Pk<NP> b0[2] = {bg[0], bg[1]}, b1[2] = {bg[2], bg[3]};
      mma_np<NP>(zq[0], am, b0);
      mma_np<NP>(zq[1], am, b1);
    }
    // ---- 6/7. LN backward of the output (row statistics of Zbar saved by the forward) -> dZbar
    F2 dzb[2][2], dzsum[2];
    float dq[2][4];
    {
      F2 xz[2][2], tt[2][2];
      F2 p1[2] = {f2(0.f), f2(0.f)}, p2[2] = {f2(0.f), f2(0.f)};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const F2 d = ld_pair<T>(tdo, g + 8 * r, nb + 8 * nt + 2 * t);
          const F2 x = f2mul(f2sub(pr(zq[nt], r), f2(mean2[r])), f2(rstd2[r]));
          xz[nt][r] = x;
          dq[nt][2 * r] = d.x;
          dq[nt][2 * r + 1] = d.y;
          dgam[nt] = f2fma(d, x, dgam[nt]);
          dbet[nt] = f2add(dbet[nt], d);
          const F2 tv_ = f2mul(d, gam[nt]);
          tt[nt][r] = tv_;
          p1[r] = f2add(p1[r], tv_);
          p2[r] = f2fma(tv_, x, p2[r]);
        }
      float2 a0, a1;
      xch_rows2<SEG>(&xch[xsel], L, f2hsum(p1[0]), f2hsum(p2[0]), f2hsum(p1[1]), f2hsum(p2[1]), a0, a1, fail);
      xsel ^= 1;
      if (fail) {
        failed = true;
        if (tid == 0) report_timeout(p.status, 13, s);
        break;
      }
      issue_next();
      const float c1[2] = {a0.x * INV_F, a1.x * INV_F}, c2[2] = {a0.y * INV_F, a1.y * INV_F};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r)
          dzb[nt][r] = f2mul(f2fma(xz[nt][r], f2(-c2[r]), f2sub(tt[nt][r], f2(c1[r]))), f2(rstd2[r]));
      dzsum[0] = f2add(dzb[0][0], dzb[0][1]);
      dzsum[1] = f2add(dzb[1][0], dzb[1][1]);
    }
    // ---- 8. dZbar to shared memory as an operand tile; the barrier also publishes tW / tDW
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 2; ++r) st_pair_planes<NP>(tDZ, g + 8 * r, nb + 8 * nt + 2 * t, dzb[nt][r].x, dzb[nt][r].y);
    __syncthreads();

    // ---- 9. products that need dZbar
    float pp[2][4], gl[2][4], dk[2][4], dgp[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) pp[nt][i] = gl[nt][i] = dk[nt][i] = dgp[nt][i] = 0.f;
    // (bf16: the B fragments of W^T read here serve step 13 as well -- there are registers for them now that the state
    // is parked in tensor memory)
    constexpr bool KEEP_W = (NP == 1);
    Pk<NP> bw_keep[KEEP_W ? 4 : 1][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      Pk<NP> adz[4], bwt[4], ags[4], bdw[4];
      ldsm_np<NP>(adz, tDZ + lane_off_A(lane, 16 * ks), PL, false);
      ldsm_np<NP>(bwt, tW + ks * SM::PLANES + lane_off_B_kn(lane, nb), PL, true);
      if constexpr (KEEP_W) {
#pragma unroll
        for (int i = 0; i < 4; ++i) bw_keep[ks][i] = bwt[i];
      }
      ldsm_np<NP>(ags, pg + lane_off_A(lane, 16 * ks), PL, false);
      ldsm_np<NP>(bdw, tDW + ks * SM::PLANES + lane_off_B_kn(lane, nb), PL, true);
      if (SEG == 64 || (ks >> 1) == hsel) {
        // P' = dZbar Gp^T (16x16, over the head's own columns); the A fragments of Gp serve as its B fragments (same
        // 8x8 blocks, other order)
        const Pk<NP> b0[2] = {ags[0], ags[2]}, b1[2] = {ags[1], ags[3]};
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
    float dte_row[2];
    Pk<NP> ada[4];
    {
      F2 acc[2] = {f2(0.f), f2(0.f)};
#pragma unroll
      for (int jt = 0; jt < 2; ++jt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int i = g + 8 * r, jj = 8 * jt + 2 * t;
          const F2 d = f2((jj <= i) ? -pp[jt][2 * r] : 0.f, (jj + 1 <= i) ? -pp[jt][2 * r + 1] : 0.f);
          acc[r] = f2add(acc[r], f2fma(d, pr(at[jt], r), d));
          const F2 da = f2mul(d, f2(te_row[r]));
          ada[2 * jt + r] = split_pack<NP>(da.x, da.y);
        }
      dte_row[0] = quad_sum(f2hsum(acc[0]));
      dte_row[1] = quad_sum(f2hsum(acc[1]));
    }
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
    // ---- 10. gradient reaching Gp, the lr / token_eta terms, and the first pair of second-derivative sums
    F2 u[2][2], v[2][2];
    float s1t[2], s2t[2];
    {
      F2 p1[2] = {f2(0.f), f2(0.f)}, p2[2] = {f2(0.f), f2(0.f)}, pdl[2] = {f2(0.f), f2(0.f)}, prt[2] = {f2(0.f), f2(0.f)};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const F2 kk = ld_pair<T>(tk, g + 8 * r, nb + 8 * nt + 2 * t);
          const F2 glp = pr(gl[nt], r);
          // dL/dGp = -M'^T dZbar - te15 (K dW + db)
          const F2 dg = f2fma(f2add(pr(kdw[nt], r), dbias[nt]), f2(-te15), pr(dgp[nt], r));
          const F2 dkn = f2fma(glp, f2(-te15), pr(dk[nt], r));
          dk[nt][2 * r] = dkn.x;
          dk[nt][2 * r + 1] = dkn.y;
          prt[r] = f2fma(kk, glp, f2fma(f2mul(G[nt][r], f2(lr_row[r])), dbias[nt], prt[r]));
          pdl[r] = f2fma(dg, G[nt][r], pdl[r]);
          const F2 uu = f2mul(dg, f2(lr_row[r]));  // dL/dG
          const F2 vv = f2mul(uu, f2(-rstd1[r]));
          u[nt][r] = uu;
          v[nt][r] = vv;
          p1[r] = f2add(p1[r], vv);
          p2[r] = f2fma(vv, xh[nt][r], p2[r]);
        }
      float4 o0, o1;
      int f2_ = 0;
      xch_rows<SEG, false>(&xch[xsel], L, make_float4(f2hsum(p1[0]), f2hsum(p2[0]), f2hsum(pdl[0]), f2hsum(prt[0])),
                    make_float4(f2hsum(p1[1]), f2hsum(p2[1]), f2hsum(pdl[1]), f2hsum(prt[1])), o0, o1, f2_);
      xsel ^= 1;
      s1t[0] = o0.x * INV_F; s2t[0] = o0.y * INV_F;
      s1t[1] = o1.x * INV_F; s2t[1] = o1.y * INV_F;
      const float rt_all = col_sum(o0.w + o1.w);  // sum over the 16 rows
      // (every warp holds these row values; warp 2 writes them: warps 0 and 1 issue the stage's stores and loads)
      if ((SEG == 32 ? (warp & 1) == 0 : warp == 2) && t == 0) {
        // per (batch, head) stream of the caller's tensors: the pair's heads are streams 2 * stream and 2 * stream + 1
        const size_t o = (SEG == 32 ? (size_t)(2 * stream + hsel) * p.T : (size_t)row_base) + (size_t)s * MB;
        st_from_float<T>(p.d_lr, o + g, o0.z);
        if constexpr (MB == CS) {
          st_from_float<T>(p.d_lr, o + g + 8, o1.z);
          p.part_te[o + g] = dte_row[0];
          p.part_te[o + g + 8] = dte_row[1] - (g == 7 ? rt_all : 0.f);
        } else {
          p.part_te[o + g] = dte_row[0] - (g == 7 ? rt_all : 0.f);  // the last token of an 8-token mini-batch is row 7
        }
      }
    }
    // ---- 11. second derivative through LN + L2 gradient -> dZ1, dT
    F2 dz1[2][2], dT[2][2];
    {
      F2 pd[2] = {f2(0.f), f2(0.f)}, ps[2] = {f2(0.f), f2(0.f)};
      F2 dxh[2][2];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const F2 x = xh[nt][r], vv = v[nt][r];
          const F2 dgxh = f2fma(x, f2(s2t[r]), f2sub(f2(s1t[r]), vv));
          const F2 dy = f2mul(gam[nt], dgxh);
          dgam[nt] = f2fma(gy[nt][r], dgxh, f2fma(dy, x, dgam[nt]));
          dbet[nt] = f2add(dbet[nt], dy);
          const F2 dx = f2fma(dy, gam[nt], f2fma(gx[nt][r], f2(s2t[r]), f2mul(vv, f2(Bv1[r]))));
          dxh[nt][r] = dx;
          dT[nt][r] = f2neg(dy);
          pd[r] = f2add(pd[r], dx);
          ps[r] = f2fma(f2fma(dx, x, f2mul(u[nt][r], G[nt][r])), f2(-rstd1[r]), ps[r]);
        }
      float2 a0, a1;
      int f2_ = 0;
      xch_rows2<SEG, false>(&xch[xsel], L, f2hsum(pd[0]), f2hsum(ps[0]), f2hsum(pd[1]), f2hsum(ps[1]), a0, a1, f2_);
      xsel ^= 1;
      const float D[2] = {a0.x * INV_F, a1.x * INV_F}, S[2] = {a0.y * INV_F, a1.y * INV_F};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r)
          dz1[nt][r] = f2fma(f2sub(dxh[nt][r], f2(D[r])), f2(rstd1[r]), f2mul(xh[nt][r], f2(S[r])));
    }
    // ---- 12. dZ1 to shared memory as an operand tile
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 2; ++r) st_pair_planes<NP>(tDZ1, g + 8 * r, nb + 8 * nt + 2 * t, dz1[nt][r].x, dz1[nt][r].y);
    if (tid == 0) bulk_wait_read<0>();  // the previous stage's output tiles have left the staging buffers
    __syncthreads();
    // ---- 13. dk += dZ1 W^T ; dW^T += dZ1^T K ; bias gradient
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      Pk<NP> adz1[4], bwt[4];
      ldsm_np<NP>(adz1, tDZ1 + lane_off_A(lane, 16 * ks), PL, false);
      if constexpr (KEEP_W) {
#pragma unroll
        for (int i = 0; i < 4; ++i) bwt[i] = bw_keep[ks][i];
      } else {
        ldsm_np<NP>(bwt, tW + ks * SM::PLANES + lane_off_B_kn(lane, nb), PL, true);
      }
      const Pk<NP> b0[2] = {bwt[0], bwt[1]}, b1[2] = {bwt[2], bwt[3]};
      mma_np<NP>(dk[0], adz1, b0);
      mma_np<NP>(dk[1], adz1, b1);
    }
    // dW^T += dZbar^T Q, then dW^T += dZ1^T K: both here (the dZbar tile and this stage's Q tile are still in place), so
    // that dW^T is in registers for this one stretch of the stage
    tmem_ld_8x4(tm_dw, dwt);
    {
      Pk<NP> adzt[4];
      ldsm_np<NP>(adzt, tDZ + lane_off_B_nk(lane, nb), PL, true);
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {
        if (khalf >= 0 && (kp >> 1) != khalf) continue;  // paired heads: only the head's own block of dW^T
        Pk<NP> bq[4];
        ldsm_np<NP>(bq, pq + lane_off_B_kn(lane, 16 * kp), PL, true);
        const Pk<NP> b0[2] = {bq[0], bq[1]}, b1[2] = {bq[2], bq[3]};
        mma_np<NP>(dwt[2 * kp], adzt, b0);
        mma_np<NP>(dwt[2 * kp + 1], adzt, b1);
      }
    }
    {
      Pk<NP> adzt[4];
      ldsm_np<NP>(adzt, tDZ1 + lane_off_B_nk(lane, nb), PL, true);
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {
        if (khalf >= 0 && (kp >> 1) != khalf) continue;
        Pk<NP> bk[4];
        ldsm_np<NP>(bk, pk + lane_off_B_kn(lane, 16 * kp), PL, true);
        const Pk<NP> b0[2] = {bk[0], bk[1]}, b1[2] = {bk[2], bk[3]};
        mma_np<NP>(dwt[2 * kp], adzt, b0);
        mma_np<NP>(dwt[2 * kp + 1], adzt, b1);
      }
    }
    tmem_st_8x4(tm_dw, dwt);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const F2 cs = f2add(dzsum[nt], f2add(dz1[nt][0], dz1[nt][1]));
      dbias[nt] = f2add(dbias[nt], f2(col_sum(cs.x), col_sum(cs.y)));
    }
    // ---- 14. outputs: dq = d_out + ..., dk = -dT + ..., dv = dT
    {
      const uint32_t so_q = base + SM::OFF_OUT, so_k = so_q + TF::RAW_BYTES, so_v = so_k + TF::RAW_BYTES;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int row = g + 8 * r, col = nb + 8 * nt + 2 * t;
          const F2 dkk = f2sub(pr(dk[nt], r), dT[nt][r]);
          st_pair<T>(so_q, row, col, dq[nt][2 * r], dq[nt][2 * r + 1]);
          st_pair<T>(so_k, row, col, dkk.x, dkk.y);
          st_pair<T>(so_v, row, col, dT[nt][r].x, dT[nt][r].y);
        }
      fence_proxy_async_smem();
      __syncthreads();
      if constexpr (GATHER) {
        scatter_pair_tile_bf16<MB>(tm_dq.ptr, stream, s * MB, p.T, so_q, tid);
        scatter_pair_tile_bf16<MB>(tm_dk.ptr, stream, s * MB, p.T, so_k, tid);
        scatter_pair_tile_bf16<MB>(tm_dv.ptr, stream, s * MB, p.T, so_v, tid);
      } else if (tid == 0) {
        if constexpr (SEG == 64) {
          const int r0 = row_base + s * MB;
          tma_store_tile<T>(&tm_dq, r0, so_q);
          tma_store_tile<T>(&tm_dk, r0, so_k);
          tma_store_tile<T>(&tm_dv, r0, so_v);
        } else {
          tma_store_pair<T>(&tm_dq, stream, s * MB, p.T, so_q);
          tma_store_pair<T>(&tm_dk, stream, s * MB, p.T, so_k);
          tma_store_pair<T>(&tm_dv, stream, s * MB, p.T, so_v);
        }
        bulk_commit();
      }
    }
  }

    if (failed) break;
    tmem_wait_st();
    tmem_ld_8x4(tm_w, wt);
    tmem_ld_8x4(tm_dw, dwt);
    // ---- end of the item: LN partials of this (stream, chunk); then either hand the state to the earlier chunk
    // or, for the first chunk of the sequence, write the gradients w.r.t. the initial state
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float dg_[2] = {col_sum(dgam[nt].x), col_sum(dgam[nt].y)};
      const float db_[2] = {col_sum(dbet[nt].x), col_sum(dbet[nt].y)};
      if (g == 0) {
        float* pl = p.part_ln + ((size_t)stream * p.NCH + chunk) * 2 * HD;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          pl[nb + 8 * nt + 2 * t + e] = dg_[e];
          pl[HD + nb + 8 * nt + 2 * t + e] = db_[e];
        }
      }
    }
    if (chunk > 0) {
#pragma unroll
      for (int kt = 0; kt < 8; ++kt) {
        reinterpret_cast<float4*>(ho)[kt * NTHREADS + tid] = make_float4(wt[kt][0], wt[kt][1], wt[kt][2], wt[kt][3]);
        reinterpret_cast<float4*>(ho + HD * HD)[kt * NTHREADS + tid] =
            make_float4(dwt[kt][0], dwt[kt][1], dwt[kt][2], dwt[kt][3]);
      }
      if (g == 0) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) *reinterpret_cast<float2*>(ho + 2 * HD * HD + nb + 8 * nt + 2 * t) = dbias[nt];
      }
      __threadfence();
      __syncthreads();
      if (tid == 0) *reinterpret_cast<volatile int*>(p.sched + 1 + stream) = crank + 1;
    } else {
      const size_t wo = (size_t)stream * HD * HD;
#pragma unroll
      for (int kt = 0; kt < 8; ++kt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if constexpr (SEG == 64) {
            const int idx = (8 * kt + 2 * t + (i & 1)) * HD + nb + g + 8 * (i >> 1);
            st_from_float<T>(p.d_w, wo + idx, dwt[kt][i]);
            if (p.part_w != nullptr) p.part_w[(size_t)stream * (HD * HD + HD) + idx] = dwt[kt][i];
          } else if ((kt >> 2) == hsel) {
            // the head's own 32 x 32 block, at the head's place in the caller's [B, H, 32, 32] layout
            const int k = 8 * kt + 2 * t + (i & 1), nn = nb + g + 8 * (i >> 1);
            const size_t hs = (size_t)(2 * stream + hsel);
            const int idx = (k & 31) * 32 + (nn & 31);
            st_from_float<T>(p.d_w, hs * 32 * 32 + idx, dwt[kt][i]);
            if (p.part_w != nullptr) p.part_w[hs * (32 * 32 + 32) + idx] = dwt[kt][i];
          }
        }
      if (g == 0) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const float dbi[2] = {dbias[nt].x, dbias[nt].y};
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = nb + 8 * nt + 2 * t + e;
            st_from_float<T>(p.d_b, (size_t)stream * HD + c, dbi[e]);  // [B, H, 32] flat = [B, H/2, 64] flat
            if (p.part_w != nullptr) {
              if constexpr (SEG == 64) p.part_w[(size_t)stream * (HD * HD + HD) + HD * HD + c] = dbi[e];
              else p.part_w[(size_t)(2 * stream + hsel) * (32 * 32 + 32) + 32 * 32 + (c & 31)] = dbi[e];
            }
          }
        }
      }
    }
  }  // item loop
  if (tid == 0) bulk_wait_all<0>();
  if constexpr (GATHER) cp_async_wait_all();  // (an item that gave up may leave gathers in flight)
  tmem_wait_st();
  tmem_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(s_tmem, 64);
}

// ----------------------------------------------------------------------------------------------------
// Second pass: fixed-order sums of the per-stream partials.
//   d_token_eta[t]   = sum over streams of part_te[stream][t]
//   d_ln_w/b[h][f]   = sum over batch and chunks of part_ln[b*H+h][chunk][0/1][f]
//   packed (optional) = { sum_b dW[b,h], sum_b db[b,h], d_ln_w, d_ln_b, d_token_eta folded to [CS] }
//                       (the fold is a second tiny kernel over the reduced d_token_eta)
// ----------------------------------------------------------------------------------------------------
// Block = 32 consecutive outputs x 8 warps.  Warp w sums terms w, w+8, ... of each output (coalesced 128-byte
// reads), the eight partial sums meet in shared memory and are added in warp order: a fixed summation order.
template <int F>
__global__ void __launch_bounds__(256) ttt_linear_bwd_reduce_kernel(const ReduceParams p) {
  __shared__ float part[8][32];
  // H heads of F features as the caller counts them; the partials of the LayerNorm gradients are in the kernel's
  // 64-wide tiles, which hold NP = 64 / F heads side by side
  constexpr int NP = HD / F;
  const int H = p.H, B = p.B, T = p.T, NCH = p.NCH, HP = H / NP;
  const int n_te = T, n_ln = 2 * H * F, n_w = (p.packed != nullptr) ? H * (F * F + F) : 0;
  const int total = n_te + n_ln + n_w;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = blockIdx.x * 32; base < total; base += gridDim.x * 32) {
    const int i = base + lane;
    float acc = 0.f;
    if (i < n_te) {
      for (int st = warp; st < B * H; st += 8) acc += p.part_te[(size_t)st * T + i];
    } else if (i < n_te + n_ln) {
      const int k = i - n_te, which = k / (H * F), hf = k % (H * F), h = hf / F, f = hf % F;
      for (int j = warp; j < B * NCH; j += 8) {
        const int b = j / NCH, ch = j - b * NCH;
        acc += p.part_ln[(((size_t)(b * HP + h / NP) * NCH + ch) * 2 + which) * HD + (h % NP) * F + f];
      }
    } else if (i < total) {
      const int k = i - n_te - n_ln;
      const bool is_w = k < H * F * F;
      const int h = is_w ? k / (F * F) : (k - H * F * F) / F;
      const int e = is_w ? k % (F * F) : F * F + (k - H * F * F) % F;
      for (int b = warp; b < B; b += 8) acc += p.part_w[(size_t)(b * H + h) * (F * F + F) + e];
    }
    part[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && i < total) {
      float sum = part[0][lane];
#pragma unroll
      for (int w = 1; w < 8; ++w) sum += part[w][lane];
      if (i < n_te) {
        p.d_token_eta[i] = sum;
      } else if (i < n_te + n_ln) {
        const int k = i - n_te;
        (k < H * F ? p.d_ln_g : p.d_ln_b)[k % (H * F)] = sum;
        if (p.packed != nullptr) p.packed[(size_t)H * F * F + H * F + k] = sum;
      } else {
        p.packed[i - n_te - n_ln] = sum;
      }
    }
    __syncthreads();
  }
}

// token_eta gradient folded over stages into [CS] (runs after the kernel above, same stream): one warp per
// mini-batch position, lanes stride over stages, fixed-order shuffle tree.
__global__ void ttt_linear_bwd_fold_kernel(const ReduceParams p) {
  const int c = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float acc = 0.f;
  for (int s = lane; s < p.T / p.mb; s += 32) acc += p.d_token_eta[s * p.mb + c];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) p.packed[(size_t)p.H * p.F * p.F + 3 * p.H * p.F + c] = acc;
}

template <typename T, int SEG, int MB>
static cudaError_t launch_bwd_t(const CUtensorMap* m, const void* const* io, const LinBwdParams& p, int nstreams,
                                cudaStream_t st) {
  using SM = BwdSmem<T, SEG>;
  auto kfn = ttt_linear_bwd_kernel<T, SEG, MB>;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM::DYN_BYTES);
  if (e != cudaSuccess) return e;
  // Persistent grid: as many blocks as fit on the device at once, never more than there are work items.  The count
  // comes from the kernel's registers and shared memory: the occupancy calculator answers one block per SM for any
  // kernel that allocates tensor memory, whatever it allocates (which also rules out a cooperative launch of more).
  // Co-residency is not needed for progress: a block takes an item only once it runs, and the item it may wait for
  // has a smaller index, so it was taken by a block that runs or has finished; a block that is not resident yet holds
  // nothing anybody waits for.
  int dev = 0, sms = 0, regs_sm = 0, smem_sm = 0, smem_rsv = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&smem_rsv, cudaDevAttrReservedSharedMemoryPerBlock, dev)) != cudaSuccess) return e;
  cudaFuncAttributes fa;
  if ((e = cudaFuncGetAttributes(&fa, kfn)) != cudaSuccess) return e;
  const int regs_block = ((fa.numRegs + 7) & ~7) * NTHREADS;  // registers are allocated in units of 8 per thread
  const int smem_block = (int)SM::DYN_BYTES + (int)fa.sharedSizeBytes + smem_rsv;
  int per_sm = regs_sm / regs_block;
  if (smem_sm / smem_block < per_sm) per_sm = smem_sm / smem_block;
  if (per_sm > 512 / 64) per_sm = 512 / 64;  // tensor-memory columns
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  int grid = sms * per_sm;
  const int nitems = nstreams * p.NCH;
  if (grid > nitems) grid = nitems;
  if ((e = cudaMemsetAsync(p.sched, 0, sizeof(int) * (size_t)(1 + nstreams), st)) != cudaSuccess) return e;
  LinBwdParams pp = p;
  RawTensor raw[7];
  void* args[9];
  for (int i = 0; i < 7; ++i) {
    raw[i].ptr = const_cast<void*>(io[i]);
    args[i] = PairIo<T, SEG>::GATHER ? (void*)&raw[i] : (void*)&m[i];
  }
  args[7] = (void*)&m[7];
  args[8] = (void*)&pp;
  return cudaLaunchKernel((const void*)kfn, dim3(grid), dim3(NTHREADS), args, SM::DYN_BYTES, st);
}

template <typename T, int SEG>
static cudaError_t launch_bwd_mb(int mb, const CUtensorMap* m, const void* const* io, const LinBwdParams& p,
                                 int nstreams, cudaStream_t st) {
  return mb == 8 ? launch_bwd_t<T, SEG, 8>(m, io, p, nstreams, st) : launch_bwd_t<T, SEG, 16>(m, io, p, nstreams, st);
}

// mb: tokens per mini-batch, 16 or 8 (the maps' boxes then have 8 rows)
cudaError_t launch_linear_bwd(int dtype, int seg, int mb, const CUtensorMap* maps, const void* const* io,
                              const LinBwdParams& p, int nstreams, cudaStream_t st) {
  if (seg == 32) {
    if (dtype == 1) return launch_bwd_mb<__nv_bfloat16, 32>(mb, maps, io, p, nstreams, st);
    return launch_bwd_mb<float, 32>(mb, maps, io, p, nstreams, st);
  }
  if (dtype == 1) return launch_bwd_mb<__nv_bfloat16, 64>(mb, maps, io, p, nstreams, st);
  return launch_bwd_mb<float, 64>(mb, maps, io, p, nstreams, st);
}

cudaError_t launch_linear_bwd_reduce(const ReduceParams& p, cudaStream_t st) {
  const int total = p.T + 2 * p.H * p.F + (p.packed != nullptr ? p.H * (p.F * p.F + p.F) : 0);
  int blocks = (total + 31) / 32;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (p.F == 32) ttt_linear_bwd_reduce_kernel<32><<<blocks, 256, 0, st>>>(p);
  else ttt_linear_bwd_reduce_kernel<64><<<blocks, 256, 0, st>>>(p);
  if (p.packed != nullptr) ttt_linear_bwd_fold_kernel<<<1, p.mb * 32, 0, st>>>(p);
  return cudaGetLastError();
}

}  // namespace ttt
