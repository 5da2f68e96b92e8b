// Fused TTT-MLP forward scan for sm_100a (bf16 I/O): one 8-warp CTA per (batch, head) stream.
//
// The reference has no fused kernel for the 2-layer inner model; its semantics are the unfused
// `TTTMLP::forward_mini_batch` (rust/core/src/mlp.rs:127-208; PyTorch twin reference/ttt.py:1107-1229), with the
// fused-kernel conventions of the linear path (token_eta read at [0, CS) in every stage).  Per 16-token stage, with
// F = 64, E = 256, Gp = lr o G, M'[i][j] = te[i] (1 + A[i][j]) for j <= i:
//     Z1 = K W1 + b1;  X2 = gelu(Z1);  Z2 = X2 W2 + b2;  G2 = d/dZ2 0.5|LN(Z2) - (V-K)|^2;  G1 = (G2 W2^T) o gelu'(Z1)
//     Zb1 = Q W1 + b1 - M1' G1p,  A1 = Q K^T;   Xb2 = gelu(Zb1);   Zb2 = Xb2 W2 + b2 - M2' G2p,  A2 = Xb2 X2^T
//     out = Q + LN(Zb2);   W1 -= te15 K^T G1p;  b1 -= te15 colsum(G1p);  W2 -= te15 X2^T G2p;  b2 -= te15 colsum(G2p)
//
// Layout: warp w owns hidden features e in [32w, 32w+32) of every 16 x 256 tile and output features [8w, 8w+8) of
// every 16 x 64 tile, in mma accumulator layout.  W1^T[e][k] (32 x 64 per warp) and W2[e][n] (32 x 64 per warp) are
// float32 accumulator registers for the whole sequence (128 registers per thread): W1^T is directly the B operand of
// K.W1 / Q.W1, W2 directly the B operand of G2p.W2^T, and both rank-16 updates accumulate into them.  The two products
// that contract over e (X2.W2, Xb2.W2) read a bf16 copy of W2 that every warp refreshes in shared memory after its
// update; X2, Xb2 and G2p pass through shared-memory operand tiles; A2 is summed from per-warp register partials.
//
// Scheduling.  One CTA fills an SM (255 registers x 256 threads), so a launch of one CTA per stream runs in whole
// waves: 192 streams on 148 SMs cost two stream-times.  When the caller passes the backward's workspace (training),
// the kernel is launched persistently instead: blocks take work items (stream, chunk of MLP_FWD_CHUNK stages), first
// chunks of all streams first; a chunk leaves the float32 state and biases in the stream's workspace block (where
// the final state is due anyway) and the next chunk of that stream -- on whichever block takes it -- picks them up.
// An item waits only for an item of smaller index, which a resident block already holds (cooperative launch), and
// the wait is bounded.  Without a workspace (inference) there is nowhere to park 128 KB of state per stream, and the
// kernel runs one block per stream as before.
#include "ttt_kernels.h"
#include "ttt_stage.cuh"

namespace ttt {

constexpr int MLP_THREADS = 256;
constexpr int MLP_E = 256;
constexpr int MLP_NST = 2;
constexpr int MLP_FWD_CHUNK = 16;  // stages per work item of the persistent launch

struct MlpSmem {
  static constexpr uint32_t TILE = TILE_BF16_BYTES;                   // [16][64] bf16
  static constexpr uint32_t SLOT = 3 * TILE;                          // q, k, v
  static constexpr uint32_t OFF_W2 = MLP_NST * SLOT;                  // 16 sub-tiles [16 e][64 n]
  static constexpr uint32_t OFF_X2 = OFF_W2 + 16 * TILE;              // 4 sub-tiles [16 tok][64 e]
  static constexpr uint32_t OFF_XB2 = OFF_X2 + 4 * TILE;
  static constexpr uint32_t OFF_G2 = OFF_XB2 + 4 * TILE;              // [16 tok][64 n]
  static constexpr uint32_t OFF_OUT = OFF_G2 + TILE;                  // 2 staging tiles
  static constexpr uint32_t OFF_A2 = OFF_OUT + 2 * TILE;              // 8 warps x 32 lanes x 8 floats
  static constexpr uint32_t OFF_XCH = OFF_A2 + 8 * 32 * 32;           // 2 x [16 rows][10] float2 (8 warps + padding)
  static constexpr uint32_t OFF_LR = OFF_XCH + 2 * 16 * 10 * 8;       // MLP_NST x 32 bytes
  static constexpr uint32_t OFF_BAR = OFF_LR + MLP_NST * 32;
  static constexpr uint32_t TOTAL = OFF_BAR + MLP_NST * 8;
  static constexpr uint32_t DYN_BYTES = TOTAL + 1024;
};

// tanh-approximated GELU and its derivative on a column pair.  tanh(x) = 1 - 2 / (1 + e^{2x}) with the fast
// exponential and division (relative error ~1e-6; the hardware tanh.approx is only good to ~5e-4, which shows after a
// few dozen chained stages).
__device__ __forceinline__ float tanh_fast(float x) {
  return 1.f - __fdividef(2.f, 1.f + __expf(2.f * x));
}
__device__ __forceinline__ F2 gelu2(F2 z, F2* deriv) {
  const F2 c0 = f2(0.7978845608028654f), c1 = f2(0.044715f);
  const F2 z2 = f2mul(z, z);
  const F2 inner = f2mul(f2mul(z, c0), f2fma(z2, c1, f2(1.f)));
  const F2 th = f2(tanh_fast(inner.x), tanh_fast(inner.y));
  const F2 hz = f2mul(z, f2(0.5f));
  if (deriv != nullptr) {
    // 0.5 z (1 - t^2) c0 (1 + 3 c1 z^2) + 0.5 (1 + t)
    const F2 sech2 = f2fma(f2neg(th), th, f2(1.f));
    const F2 poly = f2mul(c0, f2fma(z2, f2(3.f * 0.044715f), f2(1.f)));
    *deriv = f2fma(f2mul(hz, sech2), poly, f2fma(th, f2(0.5f), f2(0.5f)));
  }
  return f2fma(hz, th, hz);
}

// row sums of two values over the 8 warps (rows g and g+8); buffer float2[16][10] (rows padded to 80 bytes so that
// the 8 rows a warp reads fall in distinct banks)
__device__ __forceinline__ void xch8(float2* xb, const Lane& L, float a0x, float a0y, float a1x, float a1y, float2& o0,
                                     float2& o1, int& flag) {
  a0x = quad_sum(a0x); a0y = quad_sum(a0y); a1x = quad_sum(a1x); a1y = quad_sum(a1y);
  if (L.t == 0) {
    xb[L.g * 10 + L.warp] = make_float2(a0x, a0y);
    xb[(L.g + 8) * 10 + L.warp] = make_float2(a1x, a1y);
  }
  flag = __syncthreads_or(flag);
  float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 p = *reinterpret_cast<const float4*>(&xb[L.g * 10 + 2 * i]);
    const float4 q = *reinterpret_cast<const float4*>(&xb[(L.g + 8) * 10 + 2 * i]);
    s0.x += p.x + p.z; s0.y += p.y + p.w;
    s1.x += q.x + q.z; s1.y += q.y + q.w;
  }
  o0 = s0;
  o1 = s1;
}

// offset of element (row, col) of a 16 x 256 operand tile stored as four [16][64] swizzled sub-tiles
__device__ __forceinline__ uint32_t off_e(int row, int col) {
  return static_cast<uint32_t>((col >> 6) * TILE_BF16_BYTES) + off_bf16(row, col & 63);
}
__device__ __forceinline__ void ldsm_x2_t(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}

__global__ void __launch_bounds__(MLP_THREADS, 1)
    ttt_mlp_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                       const MlpFwdParams p) {
  using T = __nv_bfloat16;
  using SM = MlpSmem;
  constexpr uint32_t TL = TILE_BF16_BYTES;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw_u32);
  float2* xchb = reinterpret_cast<float2*>(gbase + SM::OFF_XCH);  // 2 x [16][8]
  float4* a2b = reinterpret_cast<float4*>(gbase + SM::OFF_A2);    // [8 warps][2][32 lanes]
  const uint32_t bar0 = base + SM::OFF_BAR;
  const uint32_t tW2 = base + SM::OFF_W2, tX2 = base + SM::OFF_X2, tXB2 = base + SM::OFF_XB2, tG2 = base + SM::OFF_G2;

  const Lane L;
  const int tid = L.tid, lane = L.lane, g = L.g, t = L.t, warp = L.warp;
  const int eb = 32 * warp, fb = 8 * warp;
  const int NS = p.NS;
  const bool persistent = (p.sched != nullptr);
  const int CH = persistent ? p.CH : NS, NCH = persistent ? p.NCH : 1;
  const int nitems = persistent ? p.nstreams * NCH : (int)gridDim.x;
  __shared__ int s_item;
  int stream = 0, head = 0, row_base = 0;
  // W1^T and W2 (64 + 64 float32 words per thread) are parked in tensor memory between the places of a stage that use
  // them (see tmem_ld_8x4): 256 columns per block -- two warps share a lane quarter and take 128 columns each --
  // freed by the warp that allocated them after the work-item loop, where every way out of the loop ends.
  __shared__ uint32_t s_tmem;
  if (warp == 0) tmem_alloc(smem_u32(&s_tmem), 256);
  tmem_fence_before_sync();
  __syncthreads();
  tmem_fence_after_sync();
  const uint32_t tm_w1 = s_tmem + ((32u * (uint32_t)(warp & 3)) << 16) + 128u * (uint32_t)(warp >> 2), tm_w2 = tm_w1 + 64u;

  if (tid == 0) {
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
    prefetch_tmap(&tm_o);
    for (int i = 0; i < MLP_NST; ++i) mbar_init(bar0 + 8 * i, 1);
    fence_mbar_init();
  }
  __syncthreads();

  // Optional: the backward's per-stream workspace block (layout in ttt_kernels.h).  The lr-scaled inner gradients of
  // every stage (the bf16 operands of the state updates) and the final state go there, so that the backward can
  // start its reverse walk at once.  Set per work item.
  float* bws = nullptr;
  uint32_t* sv_g1p = nullptr;
  uint32_t* sv_g2p = nullptr;
  float* sv_bst = nullptr;

  // stage s of the current stream into ring slot n % MLP_NST (n counts the stages this block has visited)
  auto issue_loads = [&](int n, int s) {
    const int slot = n % MLP_NST;
    const uint32_t bar = bar0 + 8 * slot;
    const uint32_t tq = base + slot * SM::SLOT;
    mbar_expect_tx(bar, 3 * TL + CS * 2);
    const int r0 = row_base + s * CS;
    tma_load_2d(tq, &tm_q, 0, r0, bar);
    tma_load_2d(tq + TL, &tm_k, 0, r0, bar);
    tma_load_2d(tq + 2 * TL, &tm_v, 0, r0, bar);
    bulk_load_1d(base + SM::OFF_LR + slot * 32, static_cast<const uint8_t*>(p.lr) + (size_t)r0 * 2, CS * 2, bar);
  };

  // ---- constants: F-space column pair (fb + 2t, +1); E-space column pairs j = 0..3: (eb + 8j + 2t, +1)
  const int fc = fb + 2 * t;
  F2 gam = f2(0.f), bet = f2(0.f);
  const float te_row[2] = {ld_as_float<T>(p.token_eta, g), ld_as_float<T>(p.token_eta, g + 8)};
  const float te15 = ld_as_float<T>(p.token_eta, CS - 1);
  // both states are carried divided by wscale = -te15, so that their rank-16 updates accumulate directly by mma
  const bool w_moves = (te15 != 0.f);
  const float wscale = w_moves ? -te15 : 1.f;
  const float winv = 1.f / wscale;
  F2 b2v = f2(0.f);
  F2 b1v[4];
  // ---- state: w1t[mt][kt][2rn+e'] = W1[k = 8kt+2t+e'][e = eb+16mt+g+8rn];  w2[mt][nt][2rn+e'] = W2[e = eb+16mt+g+8rn][n = 8nt+2t+e']
  float w1t[2][8][4], w2[2][8][4];
  // bf16 copy of this warp's 32 rows of W2 -> sub-tiles 2*warp, 2*warp+1
  auto publish_w2 = [&]() {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int rn = 0; rn < 2; ++rn)
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(tW2 + (2 * warp + mt) * TL + off_bf16(g + 8 * rn, 8 * nt + 2 * t)),
                       "r"(pack_bf16(w2[mt][nt][2 * rn] * wscale, w2[mt][nt][2 * rn + 1] * wscale))
                       : "memory");
  };

  int xsel = 0;
  bool failed = false;
  int n = 0;  // stages visited by this block so far (ring slot and barrier phase)
  for (int round = 0; !failed; ++round) {
    // ---- next work item: (stream, chunk); one block per stream and a single chunk when not persistent
    int item;
    if (persistent) {
      if (tid == 0) s_item = atomicAdd(&p.sched[0], 1);
      __syncthreads();
      item = s_item;
      __syncthreads();
    } else {
      item = (round == 0) ? (int)blockIdx.x : nitems;
    }
    if (item >= nitems) break;
    const int chunk = persistent ? item / p.nstreams : 0;
    stream = persistent ? item - chunk * p.nstreams : item;
    head = stream % p.H;
    row_base = stream * p.T;
    const int s_lo = chunk * CH, s_hi = min(s_lo + CH, NS) - 1;
    bws = p.bwd_ws != nullptr ? p.bwd_ws + (size_t)stream * p.bwd_ws_stride : nullptr;
    sv_g1p = bws != nullptr ? reinterpret_cast<uint32_t*>(bws + 4 * HD * MLP_E + MLP_BWD_HANDOFF_FLOATS) : nullptr;
    sv_g2p = bws != nullptr ? sv_g1p + (size_t)NS * CS * MLP_E / 2 : nullptr;
    sv_bst = bws != nullptr ? reinterpret_cast<float*>(sv_g2p + (size_t)NS * CS * HD / 2) : nullptr;
    gam = f2(ld_as_float<T>(p.ln_g, (size_t)head * HD + fc), ld_as_float<T>(p.ln_g, (size_t)head * HD + fc + 1));
    bet = f2(ld_as_float<T>(p.ln_b, (size_t)head * HD + fc), ld_as_float<T>(p.ln_b, (size_t)head * HD + fc + 1));
    if (chunk == 0) {
      // the stream starts from the caller's initial state
      b2v = f2(ld_as_float<T>(p.b2, (size_t)stream * HD + fc), ld_as_float<T>(p.b2, (size_t)stream * HD + fc + 1));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const size_t o = (size_t)stream * MLP_E + eb + 8 * j + 2 * t;
        b1v[j] = f2(ld_as_float<T>(p.b1, o), ld_as_float<T>(p.b1, o + 1));
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int kt = 0; kt < 8; ++kt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int e = eb + 16 * mt + g + 8 * (i >> 1), c = 8 * kt + 2 * t + (i & 1);
            w1t[mt][kt][i] = ld_as_float<T>(p.w1, (size_t)stream * HD * MLP_E + (size_t)c * MLP_E + e) * winv;
            w2[mt][kt][i] = ld_as_float<T>(p.w2, (size_t)stream * HD * MLP_E + (size_t)e * HD + c) * winv;
          }
    } else {
      // wait (bounded) until the previous chunk of this stream has parked its state in the workspace block
      int ok = 1;
      if (tid == 0) {
        ok = 0;
        const volatile int* flag = p.sched + 1 + stream;
        for (uint32_t it = 0; it < p.handoff_polls; ++it) {
          if (*flag >= chunk) {
            ok = 1;
            break;
          }
          __nanosleep(100);
        }
        __threadfence();
      }
      if (__syncthreads_or(ok ? 0 : 1)) {
        failed = true;
        if (tid == 0) report_timeout(p.status, 22, item);
        break;
      }
      // raw register images (already divided by wscale), 16 float4 per thread and matrix; biases in the hand-off record
      const float4* h1 = reinterpret_cast<const float4*>(bws);
      const float4* h2 = reinterpret_cast<const float4*>(bws + HD * MLP_E);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) {
          const float4 a = __ldcg(h1 + (mt * 8 + kt) * MLP_THREADS + tid);
          const float4 b = __ldcg(h2 + (mt * 8 + kt) * MLP_THREADS + tid);
          w1t[mt][kt][0] = a.x; w1t[mt][kt][1] = a.y; w1t[mt][kt][2] = a.z; w1t[mt][kt][3] = a.w;
          w2[mt][kt][0] = b.x; w2[mt][kt][1] = b.y; w2[mt][kt][2] = b.z; w2[mt][kt][3] = b.w;
        }
      const float* ho = bws + 4 * HD * MLP_E;
#pragma unroll
      for (int j = 0; j < 4; ++j) b1v[j] = __ldcg(reinterpret_cast<const float2*>(ho + MLP_HO_B1 + eb + 8 * j + 2 * t));
      b2v = __ldcg(reinterpret_cast<const float2*>(ho + MLP_HO_B2 + fc));
    }
    if (tid == 0) {
      for (int s = s_lo; s < s_lo + MLP_NST && s <= s_hi; ++s) issue_loads(n + (s - s_lo), s);
    }
    publish_w2();
    tmem_st_8x4(tm_w1, w1t[0]);
    tmem_st_8x4(tm_w1 + 32u, w1t[1]);
    tmem_st_8x4(tm_w2, w2[0]);
    tmem_st_8x4(tm_w2 + 32u, w2[1]);

  for (int s = s_lo; s <= s_hi; ++s, ++n) {
    const int slot = n % MLP_NST;
    const uint32_t tq = base + slot * SM::SLOT, tk = tq + TL, tv = tk + TL;
    int fail = mbar_wait_bounded(bar0 + 8 * slot, (n / MLP_NST) & 1) ? 0 : 1;
    if (sv_bst != nullptr && g == 0) {  // biases at the start of the stage, for the backward
      float* const bs = sv_bst + (size_t)s * (MLP_E + HD);
#pragma unroll
      for (int j = 0; j < 4; ++j) *reinterpret_cast<float2*>(bs + eb + 8 * j + 2 * t) = b1v[j];
      *reinterpret_cast<float2*>(bs + MLP_E + fc) = b2v;
    }
    const float lr_row[2] = {ld_as_float<T>(gbase + SM::OFF_LR + slot * 32, g),
                             ld_as_float<T>(gbase + SM::OFF_LR + slot * 32, g + 8)};

    // M'[i][j] = -te[i] (1 + A[i][j]) for j <= i, as an A operand
    auto masked_operand = [&](const float (&a)[2][4], Pk<1> (&am)[4]) {
#pragma unroll
      for (int jt = 0; jt < 2; ++jt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int i = g + 8 * r, jj = 8 * jt + 2 * t;
          const F2 m = f2fma(pr(a[jt], r), f2(-te_row[r]), f2(-te_row[r]));
          am[2 * jt + r] = split_pack<1>((jj <= i) ? m.x : 0.f, (jj + 1 <= i) ? m.y : 0.f);
        }
    };

    // ---- S1. Z1 = K W1 + b1, Zq = Q W1 + b1 (columns eb..eb+31), A1 = Q K^T
    tmem_wait_st();
    tmem_ld_8x4(tm_w1, w1t[0]);
    tmem_ld_8x4(tm_w1 + 32u, w1t[1]);
    float z1[4][4], zq[4][4], at[2][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) z1[j][i] = zq[j][i] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) at[0][i] = at[1][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      Pk<1> ak[4], aq[4], bk[4];
      ldsm_np<1>(ak, tk + lane_off_A(lane, 16 * ks), TL, false);
      ldsm_np<1>(aq, tq + lane_off_A(lane, 16 * ks), TL, false);
      ldsm_np<1>(bk, tk + lane_off_B_nk(lane, 16 * ks), TL, false);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        Pk<1> bw[2][2];
        bfrag_from_state<1>(w1t[mt], ks, bw);
#pragma unroll
        for (int rn = 0; rn < 2; ++rn) {
          mma_np<1>(z1[2 * mt + rn], ak, bw[rn]);
          mma_np<1>(zq[2 * mt + rn], aq, bw[rn]);
        }
      }
      const Pk<1> bj0[2] = {bk[0], bk[1]}, bj1[2] = {bk[2], bk[3]};
      mma_np<1>(at[0], aq, bj0);
      mma_np<1>(at[1], aq, bj1);
    }
    // products were taken with W1 / wscale: Z = wscale * acc + b1
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float b = (i & 1) ? b1v[j].y : b1v[j].x;
        z1[j][i] = fmaf(z1[j][i], wscale, b);
        zq[j][i] = fmaf(zq[j][i], wscale, b);
      }
    // ---- S2. X2 = gelu(Z1), D1 = gelu'(Z1); X2 to its operand tile
    F2 x2[4][2], d1[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        x2[j][r] = gelu2(pr(z1[j], r), &d1[j][r]);
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(tX2 + off_e(g + 8 * r, eb + 8 * j + 2 * t)),
                     "r"(pack_bf16(x2[j][r].x, x2[j][r].y))
                     : "memory");
      }
    fail = __syncthreads_or(fail);  // B1: X2 tile and the refreshed W2 copy are visible; previous stage fully left
    if (fail) {
      failed = true;
      if (tid == 0) report_timeout(p.status, 21, s);
      break;
    }
    // (the first thread of warp 1: thread 0 issues the stage's stores, and a warp doing both reaches the barriers late)
    if (tid == 32 && s > s_lo && s < s_hi) issue_loads(n + 1, s + 1);

    // B fragments of W2[:, fb..fb+7] for two k-steps (32 hidden rows) from the bf16 copy
    const int m_ = lane >> 3, r_ = lane & 7;
    const uint32_t w2_lane = tW2 + (m_ >> 1) * TL + off_bf16(r_ + ((m_ & 1) << 3), fb);
    // ---- S3. Z2 = X2 W2 + b2 (columns fb..fb+7)
    float z2[4] = {b2v.x, b2v.y, b2v.x, b2v.y};
#pragma unroll
    for (int kp = 0; kp < 8; ++kp) {
      Pk<1> a0[4], a1[4];
      uint32_t bb[4];
      ldsm_np<1>(a0, tX2 + (kp >> 1) * TL + lane_off_A(lane, (kp & 1) * 32), TL, false);
      ldsm_np<1>(a1, tX2 + (kp >> 1) * TL + lane_off_A(lane, (kp & 1) * 32 + 16), TL, false);
      ldsm_x4_t(bb, w2_lane + 2 * kp * TL);
      mma_bf16(z2, a0[0].p[0], a0[1].p[0], a0[2].p[0], a0[3].p[0], bb[0], bb[1]);
      mma_bf16(z2, a1[0].p[0], a1[1].p[0], a1[2].p[0], a1[3].p[0], bb[2], bb[3]);
    }
    // ---- S4. LN + L2 gradient of Z2 against V - K; G2p = lr o G2 to its operand tile
    F2 g2p[2];
    {
      const F2 zp[2] = {pr(z2, 0), pr(z2, 1)};
      float2 a0, a1;
      int f0 = 0;
      xch8(xchb + xsel * 160, L, f2hsum(zp[0]), f2hsum(f2mul(zp[0], zp[0])), f2hsum(zp[1]), f2hsum(f2mul(zp[1], zp[1])),
           a0, a1, f0);
      xsel ^= 1;
      const float mean[2] = {a0.x * (1.f / HD), a1.x * (1.f / HD)};
      const float rstd[2] = {rsqrtf(fmaxf(a0.y * (1.f / HD) - mean[0] * mean[0], 0.f) + p.eps),
                             rsqrtf(fmaxf(a1.y * (1.f / HD) - mean[1] * mean[1], 0.f) + p.eps)};
      F2 x[2], gg[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const F2 tg = f2sub(ld_pair<T>(tv, g + 8 * r, fc), ld_pair<T>(tk, g + 8 * r, fc));
        x[r] = f2mul(f2sub(zp[r], f2(mean[r])), f2(rstd[r]));
        gg[r] = f2mul(f2fma(gam, x[r], f2sub(bet, tg)), gam);
      }
      xch8(xchb + xsel * 160, L, f2hsum(gg[0]), f2hsum(f2mul(gg[0], x[0])), f2hsum(gg[1]), f2hsum(f2mul(gg[1], x[1])),
           a0, a1, f0);
      xsel ^= 1;
      const float A[2] = {a0.x * (1.f / HD), a1.x * (1.f / HD)}, Bv[2] = {a0.y * (1.f / HD), a1.y * (1.f / HD)};
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        g2p[r] = f2mul(f2fma(x[r], f2(-Bv[r]), f2sub(gg[r], f2(A[r]))), f2(rstd[r] * lr_row[r]));
        const uint32_t pk2 = pack_bf16(g2p[r].x, g2p[r].y);
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(tG2 + off_bf16(g + 8 * r, fc)), "r"(pk2) : "memory");
        if (sv_g2p != nullptr) sv_g2p[((size_t)s * CS + g + 8 * r) * (HD / 2) + (fc >> 1)] = pk2;
      }
    }
    __syncthreads();  // B2: G2p tile visible
    // ---- S5. G1p = (G2p W2^T) o gelu'(Z1)  (columns eb..eb+31; W2 straight from registers)
    tmem_ld_8x4(tm_w2, w2[0]);
    tmem_ld_8x4(tm_w2 + 32u, w2[1]);
    F2 g1p[4][2];
    {
      float h[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) h[j][i] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        Pk<1> ag[4];
        ldsm_np<1>(ag, tG2 + lane_off_A(lane, 16 * ks), TL, false);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          Pk<1> bw[2][2];
          bfrag_from_state<1>(w2[mt], ks, bw);
          mma_np<1>(h[2 * mt], ag, bw[0]);
          mma_np<1>(h[2 * mt + 1], ag, bw[1]);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int r = 0; r < 2; ++r) g1p[j][r] = f2mul(f2mul(pr(h[j], r), f2(wscale)), d1[j][r]);
    }
    // ---- S6. Zb1 = Zq - M1' G1p (G1p transposed through movmatrix; the same fragments update W1 later)
    Pk<1> gt1[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const Pk<1> pk1 = split_pack<1>(g1p[j][r].x, g1p[j][r].y);
        if (sv_g1p != nullptr) sv_g1p[((size_t)s * CS + g + 8 * r) * (MLP_E / 2) + ((eb + 8 * j + 2 * t) >> 1)] = pk1.p[0];
        gt1[j][r] = movm_t_np<1>(pk1);
      }
    {
      Pk<1> am1[4];
      masked_operand(at, am1);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const Pk<1> bg[2] = {gt1[j][0], gt1[j][1]};
        mma_np<1>(zq[j], am1, bg);
      }
    }
    // ---- S7. Xb2 = gelu(Zb1) to its operand tile;  S8. A2 = Xb2 X2^T from per-warp register partials
    F2 xb2[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        xb2[j][r] = gelu2(pr(zq[j], r), nullptr);
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(tXB2 + off_e(g + 8 * r, eb + 8 * j + 2 * t)),
                     "r"(pack_bf16(xb2[j][r].x, xb2[j][r].y))
                     : "memory");
      }
    float a2[2][4];
    {
      float a2p[2][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a2p[0][i] = a2p[1][i] = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint32_t A0 = pack_bf16(xb2[2 * c][0].x, xb2[2 * c][0].y), A1 = pack_bf16(xb2[2 * c][1].x, xb2[2 * c][1].y);
        const uint32_t A2 = pack_bf16(xb2[2 * c + 1][0].x, xb2[2 * c + 1][0].y),
                       A3 = pack_bf16(xb2[2 * c + 1][1].x, xb2[2 * c + 1][1].y);
#pragma unroll
        for (int jt = 0; jt < 2; ++jt)
          mma_bf16(a2p[jt], A0, A1, A2, A3, pack_bf16(x2[2 * c][jt].x, x2[2 * c][jt].y),
                   pack_bf16(x2[2 * c + 1][jt].x, x2[2 * c + 1][jt].y));
      }
      a2b[(warp * 2 + 0) * 32 + lane] = make_float4(a2p[0][0], a2p[0][1], a2p[0][2], a2p[0][3]);
      a2b[(warp * 2 + 1) * 32 + lane] = make_float4(a2p[1][0], a2p[1][1], a2p[1][2], a2p[1][3]);
      __syncthreads();  // B3: partials and the Xb2 tile visible
#pragma unroll
      for (int jt = 0; jt < 2; ++jt) {
        float4 acc = a2b[jt * 32 + lane];
#pragma unroll
        for (int w = 1; w < 8; ++w) {
          const float4 v = a2b[(w * 2 + jt) * 32 + lane];
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        a2[jt][0] = acc.x; a2[jt][1] = acc.y; a2[jt][2] = acc.z; a2[jt][3] = acc.w;
      }
    }
    // ---- S9. Zb2 = Xb2 W2 + b2 - M2' G2p (columns fb..fb+7)
    float zb2[4] = {b2v.x, b2v.y, b2v.x, b2v.y};
#pragma unroll
    for (int kp = 0; kp < 8; ++kp) {
      Pk<1> a0[4], a1[4];
      uint32_t bb[4];
      ldsm_np<1>(a0, tXB2 + (kp >> 1) * TL + lane_off_A(lane, (kp & 1) * 32), TL, false);
      ldsm_np<1>(a1, tXB2 + (kp >> 1) * TL + lane_off_A(lane, (kp & 1) * 32 + 16), TL, false);
      ldsm_x4_t(bb, w2_lane + 2 * kp * TL);
      mma_bf16(zb2, a0[0].p[0], a0[1].p[0], a0[2].p[0], a0[3].p[0], bb[0], bb[1]);
      mma_bf16(zb2, a1[0].p[0], a1[1].p[0], a1[2].p[0], a1[3].p[0], bb[2], bb[3]);
    }
    {
      Pk<1> am2[4];
      masked_operand(a2, am2);
      uint32_t bg[2];
      ldsm_x2_t(bg, tG2 + off_bf16((lane & 7) + (((lane >> 3) & 1) << 3), fb));
      mma_bf16(zb2, am2[0].p[0], am2[1].p[0], am2[2].p[0], am2[3].p[0], bg[0], bg[1]);
    }
    // ---- S10. out = Q + LN(Zb2)
    {
      const F2 zp[2] = {pr(zb2, 0), pr(zb2, 1)};
      float2 a0, a1;
      int f0 = 0;
      xch8(xchb + xsel * 160, L, f2hsum(zp[0]), f2hsum(f2mul(zp[0], zp[0])), f2hsum(zp[1]), f2hsum(f2mul(zp[1], zp[1])),
           a0, a1, f0);
      xsel ^= 1;
      const float mean[2] = {a0.x * (1.f / HD), a1.x * (1.f / HD)};
      const float rstd[2] = {rsqrtf(fmaxf(a0.y * (1.f / HD) - mean[0] * mean[0], 0.f) + p.eps),
                             rsqrtf(fmaxf(a1.y * (1.f / HD) - mean[1] * mean[1], 0.f) + p.eps)};
      const uint32_t so = base + SM::OFF_OUT + (n & 1) * TL;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const F2 x = f2mul(f2sub(zp[r], f2(mean[r])), f2(rstd[r]));
        const F2 o = f2add(ld_pair<T>(tq, g + 8 * r, fc), f2fma(gam, x, bet));
        st_pair<T>(so, g + 8 * r, fc, o.x, o.y);
      }
      fence_proxy_async_smem();
      __syncthreads();  // E
      if (tid == 0) {
        tma_store_2d(&tm_o, 0, row_base + s * CS, so);
        bulk_commit();
        bulk_wait_read<1>();
      }
    }
    // ---- S11. state updates (every warp its own rows), then refresh the bf16 copy of W2
    tmem_ld_8x4(tm_w1, w1t[0]);
    tmem_ld_8x4(tm_w1 + 32u, w1t[1]);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      const Pk<1> agt[4] = {gt1[2 * mt][0], gt1[2 * mt + 1][0], gt1[2 * mt][1], gt1[2 * mt + 1][1]};
      if (w_moves) state_update_direct<1>(w1t[mt], agt, tk, lane);
    }
    tmem_st_8x4(tm_w1, w1t[0]);
    tmem_st_8x4(tm_w1 + 32u, w1t[1]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // float32 column sums, like the reference; the backward's reverse walk subtracts the sums of the bf16 operand
      // values instead, which moves the recovered biases by rounding noise only (~1e-3 of one stage's step)
      const F2 cs = f2add(g1p[j][0], g1p[j][1]);
      b1v[j] = f2fma(f2(col_sum(cs.x), col_sum(cs.y)), f2(-te15), b1v[j]);
    }
    {
      Pk<1> xt[4][2];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int r = 0; r < 2; ++r) xt[j][r] = movm_t_np<1>(split_pack<1>(x2[j][r].x, x2[j][r].y));
      tmem_ld_8x4(tm_w2, w2[0]);
      tmem_ld_8x4(tm_w2 + 32u, w2[1]);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const Pk<1> ax[4] = {xt[2 * mt][0], xt[2 * mt + 1][0], xt[2 * mt][1], xt[2 * mt + 1][1]};
        if (w_moves) state_update_direct<1>(w2[mt], ax, tG2, lane);
      }
      const F2 cs = f2add(g2p[0], g2p[1]);
      b2v = f2fma(f2(col_sum(cs.x), col_sum(cs.y)), f2(-te15), b2v);
    }
    if (s < s_hi) publish_w2();
    tmem_st_8x4(tm_w2, w2[0]);
    tmem_st_8x4(tm_w2 + 32u, w2[1]);
  }
  if (failed) break;
  tmem_wait_st();
  tmem_ld_8x4(tm_w1, w1t[0]);
  tmem_ld_8x4(tm_w1 + 32u, w1t[1]);
  tmem_ld_8x4(tm_w2, w2[0]);
  tmem_ld_8x4(tm_w2 + 32u, w2[1]);
  if (chunk < NCH - 1) {
    // ---- park the state for the next chunk of this stream: register images into the stream's workspace block
    float4* h1 = reinterpret_cast<float4*>(bws);
    float4* h2 = reinterpret_cast<float4*>(bws + HD * MLP_E);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int kt = 0; kt < 8; ++kt) {
        h1[(mt * 8 + kt) * MLP_THREADS + tid] = make_float4(w1t[mt][kt][0], w1t[mt][kt][1], w1t[mt][kt][2], w1t[mt][kt][3]);
        h2[(mt * 8 + kt) * MLP_THREADS + tid] = make_float4(w2[mt][kt][0], w2[mt][kt][1], w2[mt][kt][2], w2[mt][kt][3]);
      }
    if (g == 0) {
      float* const ho = bws + 4 * HD * MLP_E;
#pragma unroll
      for (int j = 0; j < 4; ++j) *reinterpret_cast<float2*>(ho + MLP_HO_B1 + eb + 8 * j + 2 * t) = b1v[j];
      *reinterpret_cast<float2*>(ho + MLP_HO_B2 + fc) = b2v;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) *reinterpret_cast<volatile int*>(p.sched + 1 + stream) = chunk + 1;
  } else {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int kt = 0; kt < 8; ++kt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int e = eb + 16 * mt + g + 8 * (i >> 1), c = 8 * kt + 2 * t + (i & 1);
          st_from_float<T>(p.w1_out, (size_t)stream * HD * MLP_E + (size_t)c * MLP_E + e, w1t[mt][kt][i] * wscale);
          st_from_float<T>(p.w2_out, (size_t)stream * HD * MLP_E + (size_t)e * HD + c, w2[mt][kt][i] * wscale);
        }
    if (bws != nullptr) {
      float* const M1 = bws;
      float* const M2 = bws + HD * MLP_E;
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int kt = 0; kt < 8; ++kt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int e = eb + 16 * mt + g + 8 * (i >> 1), c = 8 * kt + 2 * t + (i & 1);
            M1[mlp_state_at(c, e, MLP_E)] = w1t[mt][kt][i] * wscale;
            M2[mlp_state_at(e, c, HD)] = w2[mt][kt][i] * wscale;
          }
      if (g == 0) {
        float* const ho = bws + 4 * HD * MLP_E;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<float2*>(ho + MLP_HO_B1 + eb + 8 * j + 2 * t) = b1v[j];
        *reinterpret_cast<float2*>(ho + MLP_HO_B2 + fc) = b2v;
      }
    }
    if (g == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const size_t o = (size_t)stream * MLP_E + eb + 8 * j + 2 * t;
        st_from_float<T>(p.b1_out, o, b1v[j].x);
        st_from_float<T>(p.b1_out, o + 1, b1v[j].y);
      }
      st_from_float<T>(p.b2_out, (size_t)stream * HD + fc, b2v.x);
      st_from_float<T>(p.b2_out, (size_t)stream * HD + fc + 1, b2v.y);
    }
  }
  }  // work items
  tmem_wait_st();
  tmem_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(s_tmem, 256);
  if (tid == 0) bulk_wait_all<0>();
}

cudaError_t launch_mlp_fwd(const CUtensorMap* m, const MlpFwdParams& p, int nstreams, cudaStream_t st) {
  auto kfn = ttt_mlp_fwd_kernel;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MlpSmem::DYN_BYTES);
  if (e != cudaSuccess) return e;
  if (p.sched == nullptr) {  // no workspace to park state in: one block per stream
    kfn<<<nstreams, MLP_THREADS, MlpSmem::DYN_BYTES, st>>>(m[0], m[1], m[2], m[3], p);
    return cudaGetLastError();
  }
  // persistent: as many blocks as are co-resident (they wait on one another's hand-offs), never more than items
  int dev = 0, sms = 0, per_sm = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kfn, MLP_THREADS, MlpSmem::DYN_BYTES)) != cudaSuccess)
    return e;
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  MlpFwdParams pp = p;
  pp.nstreams = nstreams;
  pp.CH = MLP_FWD_CHUNK;
  pp.NCH = (p.NS + MLP_FWD_CHUNK - 1) / MLP_FWD_CHUNK;
  int grid = sms * per_sm;
  if (grid > nstreams * pp.NCH) grid = nstreams * pp.NCH;
  if ((e = cudaMemsetAsync(pp.sched, 0, sizeof(int) * (size_t)(1 + nstreams), st)) != cudaSuccess) return e;
  void* args[] = {(void*)&m[0], (void*)&m[1], (void*)&m[2], (void*)&m[3], (void*)&pp};
  return cudaLaunchCooperativeKernel((const void*)kfn, dim3(grid), dim3(MLP_THREADS), args, MlpSmem::DYN_BYTES, st);
}
}  // namespace ttt
