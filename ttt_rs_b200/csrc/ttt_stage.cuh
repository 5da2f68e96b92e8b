// Stage arithmetic shared by the forward scan and by the backward kernel's re-simulation, so that both
// walk the same state trajectory from a checkpoint (math: rust/core/src/linear.rs:91-149,
// rust/core/src/util.rs:141-182; quirks of the fused kernels: forward/kernel.rs:116-165).
//
// Register-tile convention ("slab"): float v[2][4] = v[nt][2*r + e] is element
// (row g + 8r, column 16*warp + 8*nt + 2*t + e) of a 16x64 tile; lane = 4g + t.
#pragma once

#include "ttt_tiles.cuh"

namespace ttt {

struct Lane {
  int tid, warp, lane, g, t, nb;
  __device__ __forceinline__ Lane() {
    tid = threadIdx.x;
    warp = tid >> 5;
    lane = tid & 31;
    g = lane >> 2;
    t = lane & 3;
    nb = warp * 16;
  }
};

// Exchange of up to four per-row partial sums across the four warps of the CTA.
struct __align__(16) Xch4 {
  float4 v[CS][5];  // [row][warp] with the row padded to 80 bytes: the 8 rows a warp reads fall in distinct banks
};

// Every thread contributes its two rows (g, g+8); returns the sums over the row's SEG columns: all four warps
// (SEG = 64) or the warp pair that holds this thread's 32-wide head (SEG = 32: warps 0,1 / 2,3).
// `flag` is OR-reduced over the CTA by the same barrier (used to spread a timed-out wait); with FLAG = false the
// barrier is a plain one and `flag` is left alone (a barrier that reduces costs more than one that does not).
template <int SEG = 64, bool FLAG = true>
__device__ __forceinline__ void xch_rows(Xch4* xb, const Lane& L, const float4 a0, const float4 a1, float4& o0,
                                         float4& o1, int& flag) {
  float4 p0, p1;
  p0.x = quad_sum(a0.x); p0.y = quad_sum(a0.y); p0.z = quad_sum(a0.z); p0.w = quad_sum(a0.w);
  p1.x = quad_sum(a1.x); p1.y = quad_sum(a1.y); p1.z = quad_sum(a1.z); p1.w = quad_sum(a1.w);
  if (L.t == 0) {
    xb->v[L.g][L.warp] = p0;
    xb->v[L.g + 8][L.warp] = p1;
  }
  if constexpr (FLAG) flag = __syncthreads_or(flag);
  else __syncthreads();
  const float4* r0 = &xb->v[L.g][0];
  const float4* r1 = &xb->v[L.g + 8][0];
  if constexpr (SEG == 64) {
    // (w0 + w1) + (w2 + w3) per component, two components per packed add
    auto sum4 = [](const float4* r) {
      const float4 a = r[0], b = r[1], c = r[2], d = r[3];
      const F2 lo = f2add(f2add(f2(a.x, a.y), f2(b.x, b.y)), f2add(f2(c.x, c.y), f2(d.x, d.y)));
      const F2 hi = f2add(f2add(f2(a.z, a.w), f2(b.z, b.w)), f2add(f2(c.z, c.w), f2(d.z, d.w)));
      return make_float4(lo.x, lo.y, hi.x, hi.y);
    };
    o0 = sum4(r0);
    o1 = sum4(r1);
  } else {
    auto sum2 = [](const float4* r) {
      const float4 a = r[0], b = r[1];
      const F2 lo = f2add(f2(a.x, a.y), f2(b.x, b.y)), hi = f2add(f2(a.z, a.w), f2(b.z, b.w));
      return make_float4(lo.x, lo.y, hi.x, hi.y);
    };
    o0 = sum2(r0 + (L.warp & 2));
    o1 = sum2(r1 + (L.warp & 2));
  }
}
// Two-value variant (same buffer type, half the shuffles).
template <int SEG = 64, bool FLAG = true>
__device__ __forceinline__ void xch_rows2(Xch4* xb, const Lane& L, float a0x, float a0y, float a1x, float a1y,
                                          float2& o0, float2& o1, int& flag) {
  a0x = quad_sum(a0x); a0y = quad_sum(a0y); a1x = quad_sum(a1x); a1y = quad_sum(a1y);
  // the buffer reused as float2[16][6]: four warps' pairs per row, rows padded to 48 bytes (conflict-free reads)
  float2* base = reinterpret_cast<float2*>(xb);
  if (L.t == 0) {
    base[L.g * 6 + L.warp] = make_float2(a0x, a0y);
    base[(L.g + 8) * 6 + L.warp] = make_float2(a1x, a1y);
  }
  if constexpr (FLAG) flag = __syncthreads_or(flag);
  else __syncthreads();
  const float4 p = *reinterpret_cast<const float4*>(&base[L.g * 6]);
  const float4 q = *reinterpret_cast<const float4*>(&base[L.g * 6 + 2]);
  const float4 p2 = *reinterpret_cast<const float4*>(&base[(L.g + 8) * 6]);
  const float4 q2 = *reinterpret_cast<const float4*>(&base[(L.g + 8) * 6 + 2]);
  if constexpr (SEG == 64) {
    // (w0 + w1) + (w2 + w3) for both values of a row with packed adds
    o0 = f2add(f2add(f2(p.x, p.y), f2(p.z, p.w)), f2add(f2(q.x, q.y), f2(q.z, q.w)));
    o1 = f2add(f2add(f2(p2.x, p2.y), f2(p2.z, p2.w)), f2add(f2(q2.x, q2.y), f2(q2.z, q2.w)));
  } else {
    const bool hi = (L.warp & 2) != 0;  // this thread's head: warps 0,1 or warps 2,3
    o0 = hi ? f2add(f2(q.x, q.y), f2(q.z, q.w)) : f2add(f2(p.x, p.y), f2(p.z, p.w));
    o1 = hi ? f2add(f2(q2.x, q2.y), f2(q2.z, q2.w)) : f2add(f2(p2.x, p2.y), f2(p2.z, p2.w));
  }
}

// LayerNorm row statistics of a slab: mean and 1/sqrt(var + eps) for rows g and g+8.
// bf16 I/O uses one exchange (sum, sum of squares); float32 I/O uses the two-pass variance of the reference.
// Slabs here are column pairs: F2 z[nt][r] = columns (nb + 8nt + 2t, +1) of row g + 8r.
template <bool TWO_PASS, int SEG = 64, bool FLAG = true>
__device__ __forceinline__ void ln_row_stats(const F2 (&z)[2][2], Xch4* xch, int& xsel, const Lane& L, float eps,
                                             float (&mean)[2], float (&rstd)[2], int& flag) {
  constexpr float INV = 1.f / SEG;  // features per LayerNorm row
  float s1[2], s2[2] = {0.f, 0.f};
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    s1[r] = f2hsum(f2add(z[0][r], z[1][r]));
    if constexpr (!TWO_PASS) s2[r] = f2hsum(f2fma(z[0][r], z[0][r], f2mul(z[1][r], z[1][r])));
  }
  float2 a0, a1;
  xch_rows2<SEG, FLAG>(&xch[xsel], L, s1[0], s2[0], s1[1], s2[1], a0, a1, flag);
  xsel ^= 1;
  mean[0] = a0.x * INV;
  mean[1] = a1.x * INV;
  if constexpr (!TWO_PASS) {
    rstd[0] = rsqrtf(fmaxf(a0.y * INV - mean[0] * mean[0], 0.f) + eps);
    rstd[1] = rsqrtf(fmaxf(a1.y * INV - mean[1] * mean[1], 0.f) + eps);
  } else {
    float q2[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const F2 d0 = f2sub(z[0][r], f2(mean[r])), d1 = f2sub(z[1][r], f2(mean[r]));
      q2[r] = f2hsum(f2fma(d0, d0, f2mul(d1, d1)));
    }
    int f2_ = 0;
    xch_rows2<SEG, false>(&xch[xsel], L, q2[0], 0.f, q2[1], 0.f, a0, a1, f2_);
    xsel ^= 1;
    rstd[0] = 1.0f / sqrtf(a0.x * INV + eps);
    rstd[1] = 1.0f / sqrtf(a1.x * INV + eps);
  }
}

// accumulator registers of a 16x16 slab (two n-tiles) viewed as column pairs
__device__ __forceinline__ void slab_pairs(const float (&c)[2][4], F2 (&z)[2][2]) {
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    z[nt][0] = pr(c[nt], 0);
    z[nt][1] = pr(c[nt], 1);
  }
}

// B fragments of a 64x64 matrix held transposed in accumulator registers (m[kt][2*rn+e] = M[k=8kt+2t+e][n=nb+g+8rn]),
// for products X[16 x 64(k)] . M[:, nb..nb+15]:  k-step ks, n-tile nt.
template <int NP>
__device__ __forceinline__ void bfrag_from_state(const float (&m)[8][4], int ks, Pk<NP> (&b)[2][2]) {
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    b[nt][0] = split_pack<NP>(m[2 * ks][2 * nt], m[2 * ks][2 * nt + 1]);
    b[nt][1] = split_pack<NP>(m[2 * ks + 1][2 * nt], m[2 * ks + 1][2 * nt + 1]);
  }
}

// LN + L2 gradient pieces for one slab of Z1 given its row statistics.
// Outputs x_hat, gy = gamma*x_hat + beta - (v - k), gx = gy*gamma and the per-thread partial row sums of gx, gx*x_hat.
// gam / bet: the thread's column pairs, index nt.
template <typename T>
__device__ __forceinline__ void ln_l2_pieces(const F2 (&z1)[2][2], const float (&mean)[2], const float (&rstd)[2],
                                             const F2 (&gam)[2], const F2 (&bet)[2], uint32_t tk, uint32_t tv,
                                             const Lane& L, F2 (&xh)[2][2], F2 (&gy)[2][2], F2 (&gx)[2][2],
                                             float (&sa)[2], float (&sb)[2]) {
  F2 pa[2] = {f2(0.f), f2(0.f)}, pb[2] = {f2(0.f), f2(0.f)};
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = L.g + 8 * r, col = L.nb + 8 * nt + 2 * L.t;
      const F2 tg = f2sub(ld_pair<T>(tv, row, col), ld_pair<T>(tk, row, col));
      const F2 x = f2mul(f2sub(z1[nt][r], f2(mean[r])), f2(rstd[r]));
      const F2 y = f2fma(gam[nt], x, f2sub(bet[nt], tg));
      const F2 gg = f2mul(y, gam[nt]);
      xh[nt][r] = x;
      gy[nt][r] = y;
      gx[nt][r] = gg;
      pa[r] = f2add(pa[r], gg);
      pb[r] = f2fma(gg, x, pb[r]);
    }
  sa[0] = f2hsum(pa[0]);
  sa[1] = f2hsum(pa[1]);
  sb[0] = f2hsum(pb[0]);
  sb[1] = f2hsum(pb[1]);
}

// G = (gx - A - x_hat*Bv) * rstd * scale with A = mean(gx), Bv = mean(gx*x_hat) per row (scale: e.g. lr of the row).
__device__ __forceinline__ void g_from_pieces(const F2 (&gx)[2][2], const F2 (&xh)[2][2], const float (&A)[2],
                                              const float (&Bv)[2], const float (&rs)[2], F2 (&G)[2][2]) {
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int r = 0; r < 2; ++r)
      G[nt][r] = f2mul(f2fma(xh[nt][r], f2(-Bv[r]), f2sub(gx[nt][r], f2(A[r]))), f2(rs[r]));
}

// State update of one stage from Gp = lr o G held as transposed A fragments (agt = {n-lo/tok-lo, n-hi/tok-lo,
// n-lo/tok-hi, n-hi/tok-hi}):   tmp = Gp^T K  (16 n x 64 k per warp),   W^T += coef * tmp.
// Forward uses coef = -te15; the backward's reverse walk undoes a stage with coef = +te15 and the same tmp.
template <int NP>
__device__ __forceinline__ void state_update(float (&wt)[8][4], const Pk<NP> (&agt)[4], uint32_t k_planes, int lane,
                                             float coef) {
#pragma unroll
  for (int kp = 0; kp < 4; ++kp) {
    Pk<NP> bk[4];
    ldsm_np<NP>(bk, k_planes + lane_off_B_kn(lane, 16 * kp), TILE_BF16_BYTES, true);
    const Pk<NP> b0[2] = {bk[0], bk[1]}, b1[2] = {bk[2], bk[3]};
    float t0[4] = {0.f, 0.f, 0.f, 0.f}, t1[4] = {0.f, 0.f, 0.f, 0.f};
    mma_np<NP>(t0, agt, b0);
    mma_np<NP>(t1, agt, b1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      wt[2 * kp][i] = fmaf(coef, t0[i], wt[2 * kp][i]);
      wt[2 * kp + 1][i] = fmaf(coef, t1[i], wt[2 * kp + 1][i]);
    }
  }
}

// Same rank-16 update accumulated straight into the state registers: S^T += A^T-fragments x K.  Used with the state
// kept as W / (-te15), so neither temporaries nor a scaling pass are needed; the backward's reversal passes the
// fragments with their sign bits flipped.
// `khalf`: -1 = all 64 k-columns; 0 / 1 = only k in [0,32) / [32,64) (a 32-wide head's own block when two heads share
// the tile: the other block of the state stays zero).
template <int NP>
__device__ __forceinline__ void state_update_direct(float (&wt)[8][4], const Pk<NP> (&agt)[4], uint32_t k_planes,
                                                    int lane, int khalf = -1) {
#pragma unroll
  for (int kp = 0; kp < 4; ++kp) {
    if (khalf >= 0 && (kp >> 1) != khalf) continue;
    Pk<NP> bk[4];
    ldsm_np<NP>(bk, k_planes + lane_off_B_kn(lane, 16 * kp), TILE_BF16_BYTES, true);
    const Pk<NP> b0[2] = {bk[0], bk[1]}, b1[2] = {bk[2], bk[3]};
    mma_np<NP>(wt[2 * kp], agt, b0);
    mma_np<NP>(wt[2 * kp + 1], agt, b1);
  }
}
template <int NP>
__device__ __forceinline__ Pk<NP> neg_pk(const Pk<NP>& a) {
  Pk<NP> r;
#pragma unroll
  for (int i = 0; i < NP; ++i) r.p[i] = a.p[i] ^ 0x80008000u;
  return r;
}

__device__ __forceinline__ void report_timeout(uint32_t* status, uint32_t where, uint32_t stage) {
  if (status != nullptr && atomicCAS(status, 0u, (uint32_t)KST_TIMEOUT) == 0u) {
    status[1] = where;
    status[2] = blockIdx.x;
    status[3] = stage;
  }
}

}  // namespace ttt
