// Fused TTT-Linear forward scan, bf16 I/O, one WARP per (batch, head) stream (sm_100a).
//
// Same mathematics and the same saved state as ttt_linear_fwd.cu (reference: forward/kernel.rs:92-176, stage body
// forward/stage.rs:29-208, semantics rust/core/src/linear.rs:91-149); what differs is who does the work.  A stream is
// a chain of dependent 16-token stages, so its speed is set by the instructions on that chain, not by how many threads
// share them.  With the whole 16 x 64 tile and the whole 64 x 64 state in ONE warp
//   * every row reduction (LayerNorm statistics, the two sums of the LN gradient) is two shuffles inside the
//     4-lane group that owns the row: no shared-memory exchange, no CTA barrier anywhere in the stage loop;
//   * nothing is computed four times over (A fragments of K and Q, the 16 x 16 attention block, its mask);
//   * the A fragments of K double as the B fragments of Q.K^T (same four 8 x 8 blocks, other order).
// About 1000 warp instructions per stage instead of 2200 over four warps.  With 2.6 streams per SM each warp has a
// scheduler of its own; latency is hidden by the eight independent column tiles inside the warp.
//
// Register tile convention: x[nt][2*r + e] = element (row g + 8r, column 8*nt + 2t + e), lane = 4g + t, nt = 0..7
// (the mma.m16n8k16 accumulator layout).  State: wt[mt][kt][2*rn + e] = What[k = 8kt + 2t + e][n = 16mt + g + 8rn],
// What = W / (-te15): the rank-16 update accumulates into it by mma, and after one cvt it is the B operand of K.W, Q.W.
//
// Stage order: Z1 = K.W -> LN gradient Gp -> state update -> output.  The output uses the state AFTER the update,
// corrected exactly:  Q.W_s + b_s - M'.Gp = Q.W_{s+1} + b_{s+1} + [ (1 + Q.K^T) o (te15 - [j <= i] te_i) ] . Gp,
// so the update (which the next stage's chain waits for) is not queued behind the output products.
#include "ttt_kernels.h"
#include "ttt_stage.cuh"

namespace ttt {

constexpr int W1_NST = 4;  // TMA ring depth (stages in flight)

struct W1Smem {
  static constexpr uint32_t SLOT = 3 * TILE_BF16_BYTES;                 // q, k, v
  static constexpr uint32_t OFF_OUT = W1_NST * SLOT;                    // staging: 2 x output, 2 x Gp
  static constexpr uint32_t OFF_LR = OFF_OUT + 4 * TILE_BF16_BYTES;     // W1_NST x 32 bytes
  static constexpr uint32_t OFF_PAR = OFF_LR + W1_NST * 32;             // gamma, beta as float2[32] each
  static constexpr uint32_t OFF_BAR = OFF_PAR + 512;
  static constexpr uint32_t TOTAL = OFF_BAR + W1_NST * 8;
  static constexpr uint32_t DYN_BYTES = TOTAL + 1024;
};

__device__ __forceinline__ F2 lds_f2(uint32_t addr) {
  F2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ F2 unpack_bf16(uint32_t v) { return make_float2(bf16_lo(v), bf16_hi(v)); }

__global__ void __launch_bounds__(32, 1)
    ttt_linear_fwd_w1_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                             const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                             const __grid_constant__ CUtensorMap tm_g, const LinFwdParams p) {
  using T = __nv_bfloat16;
  using SM = W1Smem;
  constexpr uint32_t FULL = 0xffffffffu;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw_u32);
  const uint32_t bar0 = base + SM::OFF_BAR;
  const uint32_t par = base + SM::OFF_PAR;

  const int lane = threadIdx.x, g = lane >> 2, t = lane & 3;
  const int stream = blockIdx.x;
  const int head = stream % p.H;
  const int NS = p.NS;
  const int row_base = stream * p.T;

  if (lane == 0) {
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
    prefetch_tmap(&tm_o);
    prefetch_tmap(&tm_g);
    for (int i = 0; i < W1_NST; ++i) mbar_init(bar0 + 8 * i, 1);
    fence_mbar_init();
  }
  // LayerNorm weight / bias of this head as float pairs: pair i = columns 2i, 2i+1
  {
    const size_t o = (size_t)head * HD + 2 * lane;
    float2* pg = reinterpret_cast<float2*>(gbase + SM::OFF_PAR);
    pg[lane] = make_float2(ld_as_float<T>(p.ln_g, o), ld_as_float<T>(p.ln_g, o + 1));
    pg[32 + lane] = make_float2(ld_as_float<T>(p.ln_b, o), ld_as_float<T>(p.ln_b, o + 1));
  }
  __syncwarp();

  auto issue_loads = [&](int s) {
    const int slot = s % W1_NST;
    const uint32_t bar = bar0 + 8 * slot;
    const uint32_t tq = base + slot * SM::SLOT;
    mbar_expect_tx(bar, 3 * TILE_BF16_BYTES + CS * 2);
    const int r0 = row_base + s * CS;
    tma_load_2d(tq, &tm_q, 0, r0, bar);
    tma_load_2d(tq + TILE_BF16_BYTES, &tm_k, 0, r0, bar);
    tma_load_2d(tq + 2 * TILE_BF16_BYTES, &tm_v, 0, r0, bar);
    bulk_load_1d(base + SM::OFF_LR + slot * 32, static_cast<const uint8_t*>(p.lr) + (size_t)r0 * 2, CS * 2, bar);
  };
  if (lane == 0) {
    for (int s = 0; s < W1_NST && s < NS; ++s) issue_loads(s);
  }

  // ---- lane constants
  const float te_row[2] = {ld_as_float<T>(p.token_eta, g), ld_as_float<T>(p.token_eta, g + 8)};
  const float te15 = ld_as_float<T>(p.token_eta, CS - 1);
  const bool w_moves = (te15 != 0.f);
  const float wscale = w_moves ? -te15 : 1.f;
  const float winv = 1.f / wscale;
  // shared-memory lane offsets: element pair (row g, columns 8nt + 2t, +1) of a swizzled tile; row g+8 is +1024 bytes
  uint32_t xoff[8];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) xoff[nt] = off_bf16(g, 8 * nt + 2 * t);
  uint32_t offA[4], offBkn[4];  // ldmatrix lane addresses: A operand (k-step ks), transposed B operand (k pair kp)
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    offA[i] = lane_off_A(lane, 16 * i);
    offBkn[i] = lane_off_B_kn(lane, 16 * i);
  }

  // ---- state
  float wt[4][8][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int kt = 0; kt < 8; ++kt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = 8 * kt + 2 * t + (i & 1), n = 16 * mt + g + 8 * (i >> 1);
        wt[mt][kt][i] = ld_as_float<T>(p.w0, (size_t)stream * HD * HD + k * HD + n) * winv;
      }
  F2 bias[8];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    const size_t o = (size_t)stream * HD + 8 * nt + 2 * t;
    bias[nt] = f2(ld_as_float<T>(p.b0, o), ld_as_float<T>(p.b0, o + 1));
  }

  bool failed = false;
  for (int s = 0; s < NS; ++s) {
    const int slot = s % W1_NST;
    const uint32_t tq = base + slot * SM::SLOT, tk = tq + TILE_BF16_BYTES, tv = tk + TILE_BF16_BYTES;
    {
      const int bad = mbar_wait_bounded(bar0 + 8 * slot, (s / W1_NST) & 1) ? 0 : 1;
      if (__any_sync(FULL, bad)) {
        failed = true;
        if (lane == 0) report_timeout(p.status, 1, s);
        break;
      }
    }

    // ---- saved state: W before the update of every K-th stage, the bias before every stage
    if (s % p.K == 0) {
      float* wc = p.w_ckpt + ((size_t)stream * (p.NCK + 1) + s / p.K) * HD * HD;
#pragma unroll
      for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int kt = 0; kt < 8; ++kt)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            wc[(8 * kt + 2 * t + (i & 1)) * HD + 16 * mt + g + 8 * (i >> 1)] = wt[mt][kt][i] * wscale;
    }
    if (g == 0) {
      float2* bs = reinterpret_cast<float2*>(p.b_stage + ((size_t)stream * (NS + 1) + s) * HD);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) bs[4 * nt + t] = bias[nt];
    }
    const float lr_row[2] = {ld_as_float<T>(gbase + SM::OFF_LR + slot * 32, g),
                             ld_as_float<T>(gbase + SM::OFF_LR + slot * 32, g + 8)};

    // ---- Z1 = K W + b (all 64 columns)
    float z[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) z[nt][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t ak[4];
      ldsm_x4(ak, tk + offA[ks]);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int mt = nt >> 1, rn = nt & 1;
        const uint32_t b0 = pack_bf16(wt[mt][2 * ks][2 * rn], wt[mt][2 * ks][2 * rn + 1]);
        const uint32_t b1 = pack_bf16(wt[mt][2 * ks + 1][2 * rn], wt[mt][2 * ks + 1][2 * rn + 1]);
        mma_bf16(z[nt], ak[0], ak[1], ak[2], ak[3], b0, b1);
      }
    }
    // ---- LN statistics of Z1 (sum and sum of squares per row, reduced over the 4 lanes of the row)
    float mean[2], rstd[2];
    {
      F2 s1[2] = {f2(0.f), f2(0.f)}, s2[2] = {f2(0.f), f2(0.f)};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const F2 v = f2fma(pr(z[nt], r), f2(wscale), bias[nt]);
          z[nt][2 * r] = v.x;
          z[nt][2 * r + 1] = v.y;
          s1[r] = f2add(s1[r], v);
          s2[r] = f2fma(v, v, s2[r]);
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float a = quad_sum(f2hsum(s1[r])), b = quad_sum(f2hsum(s2[r]));
        mean[r] = a * (1.f / HD);
        rstd[r] = rsqrtf(fmaxf(b * (1.f / HD) - mean[r] * mean[r], 0.f) + p.eps);
      }
    }
    // ---- x_hat and gx = gamma (gamma x_hat + beta - (v - k)); their row sums; then Gp = lr (gx - A - x_hat Bv) rstd
    float4 st1[2];
    {
      F2 gx[8][2];
      F2 pa[2] = {f2(0.f), f2(0.f)}, pb[2] = {f2(0.f), f2(0.f)};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const F2 gam = lds_f2(par + 8 * (4 * nt + t)), bet = lds_f2(par + 256 + 8 * (4 * nt + t));
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const uint32_t o = xoff[nt] + 1024 * r;
          const F2 tg = f2sub(unpack_bf16(lds_u32(tv + o)), unpack_bf16(lds_u32(tk + o)));
          const F2 x = f2mul(f2sub(pr(z[nt], r), f2(mean[r])), f2(rstd[r]));
          const F2 y = f2fma(gam, x, f2sub(bet, tg));
          const F2 gg = f2mul(y, gam);
          z[nt][2 * r] = x.x;
          z[nt][2 * r + 1] = x.y;
          gx[nt][r] = gg;
          pa[r] = f2add(pa[r], gg);
          pb[r] = f2fma(gg, x, pb[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float A = quad_sum(f2hsum(pa[r])) * (1.f / HD), Bv = quad_sum(f2hsum(pb[r])) * (1.f / HD);
        const float rs = rstd[r] * lr_row[r];
        st1[r] = make_float4(mean[r], rstd[r], A, Bv);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const F2 G = f2mul(f2fma(pr(z[nt], r), f2(-Bv), f2sub(gx[nt][r], f2(A))), f2(rs));
          z[nt][2 * r] = G.x;
          z[nt][2 * r + 1] = G.y;
        }
      }
    }
    // ---- Gp as bf16: saved tile (the exact operand bits) and transposed fragments gt[nt][r] = (rows 8r.., cols 8nt..)^T
    if (lane == 0) bulk_wait_read<1>();  // the staging tiles written two stages ago have left
    __syncwarp();
    const uint32_t sg = base + SM::OFF_OUT + (2 + (s & 1)) * TILE_BF16_BYTES;
    uint32_t gt[8][2];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint32_t v = pack_bf16(z[nt][2 * r], z[nt][2 * r + 1]);
        sts_u32(sg + xoff[nt] + 1024 * r, v);
        gt[nt][r] = movm_t(v);
      }

    // ---- state update: What^T += Gp^T K ; b -= te15 colsum(Gp)
    if (w_moves) {
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {
        uint32_t bk[4];
        ldsm_x4_t(bk, tk + offBkn[kp]);
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          mma_bf16(wt[mt][2 * kp], gt[2 * mt][0], gt[2 * mt + 1][0], gt[2 * mt][1], gt[2 * mt + 1][1], bk[0], bk[1]);
          mma_bf16(wt[mt][2 * kp + 1], gt[2 * mt][0], gt[2 * mt + 1][0], gt[2 * mt][1], gt[2 * mt + 1][1], bk[2],
                   bk[3]);
        }
      }
    }
    {
      constexpr uint32_t ONES = 0x3F803F80u;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float cs[4] = {0.f, 0.f, 0.f, 0.f};
        mma_bf16(cs, ONES, ONES, ONES, ONES, gt[nt][0], gt[nt][1]);
        bias[nt] = f2fma(f2(cs[0], cs[1]), f2(-te15), bias[nt]);
      }
    }

    // ---- Zq' = Q W_{s+1} + b_{s+1}, Attn = Q K^T, Zbar = Zq' + M'' Gp with M'' = (1 + Attn) o (te15 - [j<=i] te_i)
    float at[2][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) z[nt][i] = 0.f;
#pragma unroll
    for (int jt = 0; jt < 2; ++jt)
#pragma unroll
      for (int i = 0; i < 4; ++i) at[jt][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t aq[4], ak[4];
      ldsm_x4(aq, tq + offA[ks]);
      ldsm_x4(ak, tk + offA[ks]);
      // the A fragments of K are the B fragments of Q K^T: {rows 0-7 / k-lo, rows 0-7 / k-hi}, {rows 8-15 / ...}
      mma_bf16(at[0], aq[0], aq[1], aq[2], aq[3], ak[0], ak[2]);
      mma_bf16(at[1], aq[0], aq[1], aq[2], aq[3], ak[1], ak[3]);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int mt = nt >> 1, rn = nt & 1;
        const uint32_t b0 = pack_bf16(wt[mt][2 * ks][2 * rn], wt[mt][2 * ks][2 * rn + 1]);
        const uint32_t b1 = pack_bf16(wt[mt][2 * ks + 1][2 * rn], wt[mt][2 * ks + 1][2 * rn + 1]);
        mma_bf16(z[nt], aq[0], aq[1], aq[2], aq[3], b0, b1);
      }
    }
    {
      uint32_t am[4];
#pragma unroll
      for (int jt = 0; jt < 2; ++jt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int i = g + 8 * r, j = 8 * jt + 2 * t;
          const F2 one_at = f2add(pr(at[jt], r), f2(1.f));
          const F2 coef = f2((j <= i) ? te15 - te_row[r] : te15, (j + 1 <= i) ? te15 - te_row[r] : te15);
          const F2 m = f2mul(one_at, coef);
          am[2 * jt + r] = pack_bf16(m.x, m.y);
        }
      // Zq' = wscale * acc + b, then the rank-16 correction accumulates on top
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const F2 v = f2fma(pr(z[nt], r), f2(wscale), bias[nt]);
          z[nt][2 * r] = v.x;
          z[nt][2 * r + 1] = v.y;
        }
        mma_bf16(z[nt], am[0], am[1], am[2], am[3], gt[nt][0], gt[nt][1]);
      }
    }
    // ---- out = Q + LN(Zbar)
    {
      F2 s1[2] = {f2(0.f), f2(0.f)}, s2[2] = {f2(0.f), f2(0.f)};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const F2 v = pr(z[nt], r);
          s1[r] = f2add(s1[r], v);
          s2[r] = f2fma(v, v, s2[r]);
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float a = quad_sum(f2hsum(s1[r])), b = quad_sum(f2hsum(s2[r]));
        mean[r] = a * (1.f / HD);
        rstd[r] = rsqrtf(fmaxf(b * (1.f / HD) - mean[r] * mean[r], 0.f) + p.eps);
      }
    }
    if (t == 0) {
      float4* sp = p.stats + ((size_t)row_base + (size_t)s * CS) * 2;
      sp[2 * g] = st1[0];
      sp[2 * g + 1] = make_float4(mean[0], rstd[0], 0.f, 0.f);
      sp[2 * (g + 8)] = st1[1];
      sp[2 * (g + 8) + 1] = make_float4(mean[1], rstd[1], 0.f, 0.f);
    }
    const uint32_t so = base + SM::OFF_OUT + (s & 1) * TILE_BF16_BYTES;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const F2 gam = lds_f2(par + 8 * (4 * nt + t)), bet = lds_f2(par + 256 + 8 * (4 * nt + t));
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint32_t o = xoff[nt] + 1024 * r;
        const F2 x = f2mul(f2sub(pr(z[nt], r), f2(mean[r])), f2(rstd[r]));
        const F2 ov = f2add(unpack_bf16(lds_u32(tq + o)), f2fma(gam, x, bet));
        sts_u32(so + o, pack_bf16(ov.x, ov.y));
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(&tm_o, 0, row_base + s * CS, so);
      tma_store_2d(&tm_g, 0, row_base + s * CS, sg);
      bulk_commit();
      if (s + W1_NST < NS) issue_loads(s + W1_NST);
    }
  }

  if (!failed) {
    float* wc = p.w_ckpt + ((size_t)stream * (p.NCK + 1) + p.NCK) * HD * HD;
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int kt = 0; kt < 8; ++kt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = (8 * kt + 2 * t + (i & 1)) * HD + 16 * mt + g + 8 * (i >> 1);
          const float w = wt[mt][kt][i] * wscale;
          st_from_float<T>(p.w_out, (size_t)stream * HD * HD + idx, w);
          wc[idx] = w;
        }
    if (g == 0) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int c = 8 * nt + 2 * t;
        st_from_float<T>(p.b_out, (size_t)stream * HD + c, bias[nt].x);
        st_from_float<T>(p.b_out, (size_t)stream * HD + c + 1, bias[nt].y);
        *reinterpret_cast<float2*>(p.b_stage + ((size_t)stream * (NS + 1) + NS) * HD + c) = bias[nt];
      }
    }
  }
  if (lane == 0) bulk_wait_all<0>();
}

cudaError_t launch_linear_fwd_w1(const CUtensorMap* m, const LinFwdParams& p, int nstreams, cudaStream_t st) {
  auto kfn = ttt_linear_fwd_w1_kernel;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)W1Smem::DYN_BYTES);
  if (e != cudaSuccess) return e;
  kfn<<<nstreams, 32, W1Smem::DYN_BYTES, st>>>(m[0], m[1], m[2], m[3], m[4], p);
  return cudaGetLastError();
}

}  // namespace ttt
