// TTT-MLP backward (bf16 I/O, float32 state), first version: one 8-warp CTA per (batch, head) stream.
//
// What it computes: the gradient of the whole-sequence TTT-MLP forward (semantics rust/core/src/mlp.rs:127-208; the
// reference obtains this gradient from Burn autodiff, it has no fused MLP kernel) for loss = <grad_output, output>:
// grad_xq/xk/xv, grad_w1/b1/w2/b2 (per batch element), grad_ttt_lr_eta, and per-stream partials of grad_token_eta and
// of the LayerNorm parameter gradients (summed over streams in a fixed order by ttt_mlp_bwd_reduce_kernel).
//
// How: the stage-by-stage analytic backward (reverse walk over the mini-batches carrying dW1, db1, dW2, db2; GELU
// and LayerNorm second derivatives).  The four state matrices of a stream (W1, W2, dW1, dW2: 256 KB float32) do not
// fit on one SM next to the working tiles, so they live in the workspace (L2-resident across the stage loop) and
// every product reads / updates them there.
//   pass 1 walks forward once and saves the lr-scaled inner gradients g1p = l o g1, g2p = l o g2 of every stage;
//   pass 2 walks backward: W1_s = W1_{s+1} + K^T g1p, W2_s = W2_{s+1} + X2^T g2p recover the state of the stage,
//          the stage's forward intermediates are recomputed from it, and the gradient steps follow.
// All tile products go through one generic routine (tile_mma): operands are float32 tiles addressed by
// (pointer, row stride, column stride) in shared or global memory, converted to bf16 fragments on the fly and
// multiplied by mma.m16n8k16 with float32 accumulation -- the same operand precision as the forward kernel.  This
// version favours a direct transcription of the mathematics over speed.
#include "ttt_kernels.h"
#include "ttt_common.cuh"

namespace ttt {

constexpr int MB_THREADS = 256;
constexpr int MB_E = 256;  // hidden width of the inner MLP (4 * head_dim)
constexpr float GELU_C0 = 0.7978845608028654f, GELU_C1 = 0.044715f;

struct Mat {  // element (i, j) at p[i * rs + j * cs]
  float* p;
  int rs, cs;
};
__device__ __forceinline__ Mat mat(float* p, int rs, int cs = 1) { return Mat{p, rs, cs}; }
__device__ __forceinline__ Mat tr(const Mat& m) { return Mat{m.p, m.cs, m.rs}; }
__device__ __forceinline__ float at(const Mat& m, int i, int j) { return m.p[(size_t)i * m.rs + (size_t)j * m.cs]; }

// C[M x N] = (ACC ? C : 0) + alpha * A[M x K] . B[K x N];  M % 16 == 0, N % 8 == 0, K % 16 == 0.
// Output tiles of 16 x 8 are dealt to the warps round-robin (the same tile always goes to the same warp, so
// successive accumulations into one matrix need no barrier between them).
template <bool ACC>
__device__ void tile_mma(const Mat C, const Mat A, const Mat B, int M, int N, int K, float alpha) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int ntn = N >> 3, total = (M >> 4) * ntn;
  for (int tile = warp; tile < total; tile += MB_THREADS / 32) {
    const int mt = tile / ntn, nt = tile - mt * ntn;
    const int i0 = 16 * mt + g, j0 = 8 * nt;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < K; k0 += 16) {
      const int ka = k0 + 2 * t, kb = ka + 8;
      const uint32_t a0 = pack_bf16(at(A, i0, ka), at(A, i0, ka + 1));
      const uint32_t a1 = pack_bf16(at(A, i0 + 8, ka), at(A, i0 + 8, ka + 1));
      const uint32_t a2 = pack_bf16(at(A, i0, kb), at(A, i0, kb + 1));
      const uint32_t a3 = pack_bf16(at(A, i0 + 8, kb), at(A, i0 + 8, kb + 1));
      const uint32_t b0 = pack_bf16(at(B, ka, j0 + g), at(B, ka + 1, j0 + g));
      const uint32_t b1 = pack_bf16(at(B, kb, j0 + g), at(B, kb + 1, j0 + g));
      mma_bf16(acc, a0, a1, a2, a3, b0, b1);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int i = i0 + 8 * (q >> 1), j = j0 + 2 * t + (q & 1);
      float* c = C.p + (size_t)i * C.rs + (size_t)j * C.cs;
      *c = (ACC ? *c : 0.f) + alpha * acc[q];
    }
  }
}

__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + tanhf(GELU_C0 * x * (1.f + GELU_C1 * x * x))); }
__device__ __forceinline__ float gelu_d1(float x) {
  const float th = tanhf(GELU_C0 * x * (1.f + GELU_C1 * x * x));
  return 0.5f * x * ((1.f - th * th) * (GELU_C0 + 3.f * GELU_C0 * GELU_C1 * x * x)) + 0.5f * (1.f + th);
}
__device__ __forceinline__ float gelu_d2(float x) {
  const float th = tanhf(GELU_C0 * x * (1.f + GELU_C1 * x * x));
  const float du = GELU_C0 * (1.f + 3.f * GELU_C1 * x * x), d2u = 6.f * GELU_C0 * GELU_C1 * x;
  return (1.f - th * th) * du + 0.5f * x * (1.f - th * th) * (d2u - 2.f * th * du * du);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Shared-memory tiles (float32, row-major [16][N]).
struct MlpBwdSmem {
  float z1[CS][MB_E], x2[CS][MB_E], hm[CS][MB_E], g1[CS][MB_E], z1b[CS][MB_E], x2b[CS][MB_E];
  float t1[CS][MB_E], t2[CS][MB_E], t3[CS][MB_E], t4[CS][MB_E];  // dx2b/dz1b, dg1/dh, dx2, dz1 (+ scratch in pass 1)
  float q[CS][HD], k[CS][HD], v[CS][HD], dO[CS][HD];
  float z2[CS][HD], g2[CS][HD], z2b[CS][HD], dz2b[CS][HD], dg2[CS][HD], dz2[CS][HD], dq[CS][HD], dk[CS][HD], gl1[CS][HD];
  float eta[CS][CS], a1[CS][CS], a2[CS][CS], m1[CS][CS], m2[CS][CS], dm[CS][CS], da[CS][CS], deta[CS][CS];
  float lr[CS], te[CS], ell[CS], dell[CS], mean[CS], rstd[CS];
  float colpart[8][2 * HD];  // per-warp partial column sums (fixed-order combine)
  float dgam[HD], dbet[HD];  // this stream's LayerNorm parameter gradients
};

// mean and 1/sqrt(var + eps) of every row of a [16][64] tile (two-pass variance); warp w takes rows 2w, 2w+1
__device__ void row_stats64(const float (*x)[HD], float* mean, float* rstd, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = 2 * warp + rr;
    const float a = x[r][lane], b = x[r][lane + 32];
    const float mu = warp_sum(a + b) * (1.f / HD);
    const float var = warp_sum((a - mu) * (a - mu) + (b - mu) * (b - mu)) * (1.f / HD);
    if (lane == 0) {
      mean[r] = mu;
      rstd[r] = 1.f / sqrtf(var + eps);
    }
  }
}

// G = d/dz of 0.5 |LN(z) - (v - k)|^2 for a [16][64] tile (rust/core/src/util.rs:155-182)
__device__ void ln_l2_grad_tile(MlpBwdSmem& S, const float (*z)[HD], float (*G)[HD], const float* gam, const float* bet,
                                float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = 2 * warp + rr;
    float xv[2], gx[2];
    const float a = z[r][lane], b = z[r][lane + 32];
    const float mu = warp_sum(a + b) * (1.f / HD);
    const float var = warp_sum((a - mu) * (a - mu) + (b - mu) * (b - mu)) * (1.f / HD);
    const float rs = 1.f / sqrtf(var + eps);
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int c = lane + 32 * e;
      xv[e] = ((e ? b : a) - mu) * rs;
      gx[e] = (gam[c] * xv[e] + bet[c] - (S.v[r][c] - S.k[r][c])) * gam[c];
      s1 += gx[e];
      s2 += gx[e] * xv[e];
    }
    s1 = warp_sum(s1) * (1.f / HD);
    s2 = warp_sum(s2) * (1.f / HD);
#pragma unroll
    for (int e = 0; e < 2; ++e) G[r][lane + 32 * e] = (gx[e] - s1 - xv[e] * s2) * rs;
  }
}

// column sums of a [16][N] tile (optionally scaled per row) added, with sign, to dst[N] (global or shared)
__device__ void add_colsum(float* dst, const float* tile, int N, const float* rowscale, float sign) {
  for (int c = threadIdx.x; c < N; c += MB_THREADS) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < CS; ++r) s += tile[r * N + c] * (rowscale ? rowscale[r] : 1.f);
    dst[c] += sign * s;
  }
}

__device__ void load_tile_bf16(float (*dst)[HD], const __nv_bfloat16* src) {
  for (int e = threadIdx.x; e < CS * HD; e += MB_THREADS) dst[e / HD][e % HD] = __bfloat162float(src[e]);
}
__device__ void store_tile_bf16(__nv_bfloat16* dst, const float (*src)[HD]) {
  for (int e = threadIdx.x; e < CS * HD; e += MB_THREADS) dst[e] = __float2bfloat16_rn(src[e / HD][e % HD]);
}

__global__ void __launch_bounds__(MB_THREADS, 1) ttt_mlp_bwd_kernel(const MlpBwdParams p) {
  extern __shared__ __align__(16) uint8_t mlp_bwd_smem[];
  MlpBwdSmem& S = *reinterpret_cast<MlpBwdSmem*>(mlp_bwd_smem);
  typedef __nv_bfloat16 T;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int stream = blockIdx.x, head = stream % p.H, NS = p.NS, F = HD, E = MB_E;
  const size_t row_base = (size_t)stream * p.T;

  // per-stream workspace: W1 [F][E], W2 [E][F], dW1, dW2, b1 [E], b2 [F], db1, db2, then g1p [NS][16][E], g2p [NS][16][F]
  float* ws = p.workspace + (size_t)stream * p.ws_stride;
  float* W1 = ws;
  float* W2 = W1 + F * E;
  float* dW1 = W2 + E * F;
  float* dW2 = dW1 + F * E;
  float* b1 = dW2 + E * F;
  float* b2 = b1 + E;
  float* db1 = b2 + F;
  float* db2 = db1 + E;
  float* g1p_all = db2 + F;
  float* g2p_all = g1p_all + (size_t)NS * CS * E;

  __shared__ float gam[HD], bet[HD];
  if (tid < HD) {
    gam[tid] = ld_as_float<T>(p.ln_g, (size_t)head * HD + tid);
    bet[tid] = ld_as_float<T>(p.ln_b, (size_t)head * HD + tid);
    S.dgam[tid] = 0.f;
    S.dbet[tid] = 0.f;
  }
  if (tid < CS) S.te[tid] = ld_as_float<T>(p.token_eta, (size_t)tid);
  for (int e = tid; e < F * E; e += MB_THREADS) {
    W1[e] = ld_as_float<T>(p.w1, (size_t)stream * F * E + e);
    W2[e] = ld_as_float<T>(p.w2, (size_t)stream * F * E + e);
    dW1[e] = 0.f;
    dW2[e] = 0.f;
  }
  for (int e = tid; e < E; e += MB_THREADS) {
    b1[e] = ld_as_float<T>(p.b1, (size_t)stream * E + e);
    db1[e] = 0.f;
  }
  if (tid < F) {
    b2[tid] = ld_as_float<T>(p.b2, (size_t)stream * F + tid);
    db2[tid] = 0.f;
  }
  __syncthreads();
  const float te_last = S.te[CS - 1];

  const Mat mW1 = mat(W1, E), mW2 = mat(W2, F), mdW1 = mat(dW1, E), mdW2 = mat(dW2, F);
  const Mat mK = mat(&S.k[0][0], HD), mQ = mat(&S.q[0][0], HD);
  const Mat mz1 = mat(&S.z1[0][0], E), mx2 = mat(&S.x2[0][0], E), mh = mat(&S.hm[0][0], E), mg1 = mat(&S.g1[0][0], E);
  const Mat mz1b = mat(&S.z1b[0][0], E), mx2b = mat(&S.x2b[0][0], E);
  const Mat mt1 = mat(&S.t1[0][0], E), mt2 = mat(&S.t2[0][0], E), mt3 = mat(&S.t3[0][0], E), mt4 = mat(&S.t4[0][0], E);
  const Mat mz2 = mat(&S.z2[0][0], HD), mg2 = mat(&S.g2[0][0], HD), mz2b = mat(&S.z2b[0][0], HD);
  const Mat mdz2b = mat(&S.dz2b[0][0], HD), mdg2 = mat(&S.dg2[0][0], HD), mdz2 = mat(&S.dz2[0][0], HD);
  const Mat mdq = mat(&S.dq[0][0], HD), mdk = mat(&S.dk[0][0], HD), mgl1 = mat(&S.gl1[0][0], HD);
  const Mat ma1 = mat(&S.a1[0][0], CS), ma2 = mat(&S.a2[0][0], CS), mm1 = mat(&S.m1[0][0], CS), mm2 = mat(&S.m2[0][0], CS);
  const Mat mdm = mat(&S.dm[0][0], CS), mda = mat(&S.da[0][0], CS);

  // z1 = K W1 + b1, x2 = gelu(z1), z2 = x2 W2 + b2, g2, h = g2 W2^T, g1 = h o gelu'(z1)   (from the state in the workspace)
  auto inner_forward = [&]() {
    tile_mma<false>(mz1, mK, mW1, CS, E, F, 1.f);
    __syncthreads();
    for (int e = tid; e < CS * E; e += MB_THREADS) {
      const float z = S.z1[0][e] + b1[e % E];
      S.z1[0][e] = z;
      S.x2[0][e] = gelu_f(z);
    }
    __syncthreads();
    tile_mma<false>(mz2, mx2, mW2, CS, F, E, 1.f);
    __syncthreads();
    for (int e = tid; e < CS * F; e += MB_THREADS) S.z2[0][e] += b2[e % F];
    __syncthreads();
    ln_l2_grad_tile(S, S.z2, S.g2, gam, bet, p.eps);
    __syncthreads();
    tile_mma<false>(mh, mg2, tr(mW2), CS, E, F, 1.f);
    __syncthreads();
    for (int e = tid; e < CS * E; e += MB_THREADS) S.g1[0][e] = S.hm[0][e] * gelu_d1(S.z1[0][e]);
    __syncthreads();
  };

  // ============================== pass 1: forward walk, saving g1p and g2p ==============================
  for (int s = 0; s < NS; ++s) {
    const size_t r0 = (row_base + (size_t)s * CS) * HD;
    load_tile_bf16(S.k, static_cast<const T*>(p.xk) + r0);
    load_tile_bf16(S.v, static_cast<const T*>(p.xv) + r0);
    if (tid < CS) S.ell[tid] = te_last * ld_as_float<T>(p.lr, row_base + (size_t)s * CS + tid);
    __syncthreads();
    inner_forward();
    float* g1p = g1p_all + (size_t)s * CS * E;
    float* g2p = g2p_all + (size_t)s * CS * F;
    for (int e = tid; e < CS * E; e += MB_THREADS) {
      const float v_ = S.ell[e / E] * S.g1[0][e];
      g1p[e] = v_;
      S.t1[0][e] = v_;
    }
    for (int e = tid; e < CS * F; e += MB_THREADS) {
      const float v_ = S.ell[e / F] * S.g2[0][e];
      g2p[e] = v_;
      S.dg2[0][e] = v_;
    }
    __syncthreads();
    tile_mma<true>(mW1, tr(mK), mt1, F, E, CS, -1.f);   // W1 -= K^T g1p
    tile_mma<true>(mW2, tr(mx2), mdg2, E, F, CS, -1.f);  // W2 -= X2^T g2p
    add_colsum(b1, &S.t1[0][0], E, nullptr, -1.f);
    add_colsum(b2, &S.dg2[0][0], F, nullptr, -1.f);
    __syncthreads();
  }

  // ============================== pass 2: backward walk ==============================
  for (int s = NS - 1; s >= 0; --s) {
    const size_t r0 = (row_base + (size_t)s * CS) * HD;
    load_tile_bf16(S.q, static_cast<const T*>(p.xq) + r0);
    load_tile_bf16(S.k, static_cast<const T*>(p.xk) + r0);
    load_tile_bf16(S.v, static_cast<const T*>(p.xv) + r0);
    load_tile_bf16(S.dO, static_cast<const T*>(p.d_out) + r0);
    if (tid < CS) {
      S.lr[tid] = ld_as_float<T>(p.lr, row_base + (size_t)s * CS + tid);
      S.ell[tid] = te_last * S.lr[tid];
    }
    const float* g1p = g1p_all + (size_t)s * CS * E;
    const float* g2p = g2p_all + (size_t)s * CS * F;
    for (int e = tid; e < CS * E; e += MB_THREADS) S.t1[0][e] = g1p[e];
    for (int e = tid; e < CS * F; e += MB_THREADS) S.dg2[0][e] = g2p[e];
    __syncthreads();
    // ---- state at the start of this stage: undo the stage's updates (W1 first: X2 depends on it)
    tile_mma<true>(mW1, tr(mK), mt1, F, E, CS, 1.f);
    add_colsum(b1, &S.t1[0][0], E, nullptr, 1.f);
    __syncthreads();
    tile_mma<false>(mz1, mK, mW1, CS, E, F, 1.f);
    __syncthreads();
    for (int e = tid; e < CS * E; e += MB_THREADS) S.x2[0][e] = gelu_f(S.z1[0][e] + b1[e % E]);
    __syncthreads();
    tile_mma<true>(mW2, tr(mx2), mdg2, E, F, CS, 1.f);
    add_colsum(b2, &S.dg2[0][0], F, nullptr, 1.f);
    __syncthreads();
    // ---- forward intermediates of the stage
    inner_forward();
    for (int e = tid; e < CS * CS; e += MB_THREADS) {
      const int i = e / CS, j = e % CS;
      S.eta[i][j] = (j <= i) ? S.te[i] * S.lr[j] : 0.f;
    }
    tile_mma<false>(ma1, mQ, tr(mK), CS, CS, F, 1.f);
    __syncthreads();
    for (int e = tid; e < CS * CS; e += MB_THREADS) {
      const int i = e / CS, j = e % CS;
      const float a = (j <= i) ? S.a1[i][j] : 0.f;
      S.a1[i][j] = a;
      S.m1[i][j] = S.eta[i][j] * (1.f + a);
    }
    tile_mma<false>(mz1b, mQ, mW1, CS, E, F, 1.f);
    __syncthreads();
    tile_mma<true>(mz1b, mm1, mg1, CS, E, CS, -1.f);
    __syncthreads();
    for (int e = tid; e < CS * E; e += MB_THREADS) {
      const float z = S.z1b[0][e] + b1[e % E];
      S.z1b[0][e] = z;
      S.x2b[0][e] = gelu_f(z);
    }
    __syncthreads();
    tile_mma<false>(ma2, mx2b, tr(mx2), CS, CS, E, 1.f);
    tile_mma<false>(mz2b, mx2b, mW2, CS, F, E, 1.f);
    __syncthreads();
    for (int e = tid; e < CS * CS; e += MB_THREADS) {
      const int i = e / CS, j = e % CS;
      const float a = (j <= i) ? S.a2[i][j] : 0.f;
      S.a2[i][j] = a;
      S.m2[i][j] = S.eta[i][j] * (1.f + a);
    }
    __syncthreads();
    tile_mma<true>(mz2b, mm2, mg2, CS, F, CS, -1.f);
    __syncthreads();
    for (int e = tid; e < CS * F; e += MB_THREADS) S.z2b[0][e] += b2[e % F];
    __syncthreads();

    // ---- 1. output LayerNorm: dz2b, LN parameter gradients
    {
      float pg[2] = {0.f, 0.f}, pb[2] = {0.f, 0.f};
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int r = 2 * warp + rr;
        const float a = S.z2b[r][lane], b = S.z2b[r][lane + 32];
        const float mu = warp_sum(a + b) * (1.f / HD);
        const float var = warp_sum((a - mu) * (a - mu) + (b - mu) * (b - mu)) * (1.f / HD);
        const float rs = 1.f / sqrtf(var + p.eps);
        float xh[2], tt[2], s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = lane + 32 * e;
          xh[e] = ((e ? b : a) - mu) * rs;
          const float d = S.dO[r][c];
          pg[e] += d * xh[e];
          pb[e] += d;
          tt[e] = d * gam[c];
          s1 += tt[e];
          s2 += tt[e] * xh[e];
        }
        s1 = warp_sum(s1) * (1.f / HD);
        s2 = warp_sum(s2) * (1.f / HD);
#pragma unroll
        for (int e = 0; e < 2; ++e) S.dz2b[r][lane + 32 * e] = (tt[e] - s1 - xh[e] * s2) * rs;
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        S.colpart[warp][lane + 32 * e] = pg[e];
        S.colpart[warp][64 + lane + 32 * e] = pb[e];
      }
    }
    __syncthreads();
    if (tid < 2 * HD) {
      float s_ = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s_ += S.colpart[w][tid];
      if (tid < HD) S.dgam[tid] += s_; else S.dbet[tid - HD] += s_;
    }
    // ---- 2. z2b = x2b W2 + b2 - M2 g2
    tile_mma<false>(mt1, mdz2b, tr(mW2), CS, E, F, 1.f);         // dx2b = dz2b W2^T
    tile_mma<false>(mdm, mdz2b, tr(mg2), CS, CS, F, -1.f);        // dM2 = -tril(dz2b g2^T)
    tile_mma<false>(mdg2, tr(mm2), mdz2b, CS, F, CS, -1.f);       // dg2 = -M2^T dz2b
    __syncthreads();
    for (int e = tid; e < CS * CS; e += MB_THREADS) {
      const int i = e / CS, j = e % CS;
      const float d = (j <= i) ? S.dm[i][j] : 0.f;
      S.da[i][j] = d * S.eta[i][j];
      S.deta[i][j] = d * (1.f + S.a2[i][j]);
    }
    __syncthreads();
    tile_mma<true>(mt1, mda, mx2, CS, E, CS, 1.f);               // dx2b += dA2 x2
    tile_mma<false>(mt3, tr(mda), mx2b, CS, E, CS, 1.f);          // dx2 = dA2^T x2b
    __syncthreads();
    // ---- 3./4. dz1b = dx2b o gelu'(z1b);  z1b = Q W1 + b1 - M1 g1
    for (int e = tid; e < CS * E; e += MB_THREADS) S.t1[0][e] *= gelu_d1(S.z1b[0][e]);
    __syncthreads();
    tile_mma<false>(mdq, mt1, tr(mW1), CS, F, E, 1.f);            // dq = dz1b W1^T
    tile_mma<false>(mdm, mt1, tr(mg1), CS, CS, E, -1.f);          // dM1 = -tril(dz1b g1^T)
    tile_mma<false>(mt2, tr(mm1), mt1, CS, E, CS, -1.f);          // dg1 = -M1^T dz1b
    __syncthreads();
    for (int e = tid; e < CS * CS; e += MB_THREADS) {
      const int i = e / CS, j = e % CS;
      const float d = (j <= i) ? S.dm[i][j] : 0.f;
      S.da[i][j] = d * S.eta[i][j];
      S.deta[i][j] += d * (1.f + S.a1[i][j]);
    }
    __syncthreads();
    tile_mma<true>(mdq, mda, mK, CS, F, CS, 1.f);                 // dq += dA1 K
    tile_mma<false>(mdk, tr(mda), mQ, CS, F, CS, 1.f);            // dk = dA1^T Q
    // ---- 5. the four state updates; dW1, db1, dW2, db2 still hold the gradients w.r.t. the next stage's state
    tile_mma<false>(mgl1, mg1, tr(mdW1), CS, F, E, 1.f);          // gl1 = g1 dW1^T
    tile_mma<false>(mt4, mg2, tr(mdW2), CS, E, F, 1.f);           // gl2 = g2 dW2^T   (t4 as scratch)
    __syncthreads();
    //   dg1 -= (l o K) dW1 + l (x) db1 : l o K is built in dz2, which is free until step 7
    for (int e = tid; e < CS * F; e += MB_THREADS) S.dz2[0][e] = S.ell[e / F] * S.k[0][e];
    __syncthreads();
    tile_mma<true>(mt2, mdz2, mdW1, CS, E, F, -1.f);              // dg1 -= (l o K) dW1
    __syncthreads();
    for (int e = tid; e < CS * E; e += MB_THREADS) S.t2[0][e] -= S.ell[e / E] * db1[e % E];
    // dg2 -= (l o x2) dW2 + l (x) db2 : l o x2 into z1b (dead after step 3)
    for (int e = tid; e < CS * E; e += MB_THREADS) S.z1b[0][e] = S.ell[e / E] * S.x2[0][e];
    __syncthreads();
    tile_mma<true>(mdg2, mz1b, mdW2, CS, F, E, -1.f);
    __syncthreads();
    for (int e = tid; e < CS * F; e += MB_THREADS) {
      S.dg2[0][e] -= S.ell[e / F] * db2[e % F];
      S.dk[0][e] -= S.ell[e / F] * S.gl1[0][e];                   // dk -= l o gl1
    }
    for (int e = tid; e < CS * E; e += MB_THREADS) S.t3[0][e] -= S.ell[e / E] * S.t4[0][e];  // dx2 -= l o gl2
    __syncthreads();
    // dell[j] = -( gl1[j].K[j] + g1[j].db1 + gl2[j].x2[j] + g2[j].db2 )
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int r = 2 * warp + rr;
      float acc = 0.f;
      for (int c = lane; c < F; c += 32) acc += S.gl1[r][c] * S.k[r][c] + S.g2[r][c] * db2[c];
      for (int c = lane; c < E; c += 32) acc += S.g1[r][c] * db1[c] + S.t4[r][c] * S.x2[r][c];
      acc = warp_sum(acc);
      if (lane == 0) S.dell[r] = -acc;
    }
    __syncthreads();
    // ---- 6. g1 = (g2 W2^T) o gelu'(z1):  dh = dg1 o gelu'(z1) (in t2),  dz1 = dg1 o h o gelu''(z1) (t4)
    for (int e = tid; e < CS * E; e += MB_THREADS) {
      const float d = S.t2[0][e], z = S.z1[0][e];
      S.t4[0][e] = d * S.hm[0][e] * gelu_d2(z);
      S.t2[0][e] = d * gelu_d1(z);
    }
    __syncthreads();
    tile_mma<true>(mdg2, mt2, mW2, CS, F, E, 1.f);                // dg2 += dh W2
    tile_mma<true>(mdW2, tr(mt2), mg2, E, F, CS, 1.f);            // dW2 += dh^T g2
    __syncthreads();
    // ---- 7. second derivative through g2 = ln_l2_grad(z2, v - k): dz2, d target, LN parameter gradients
    {
      float pg[2] = {0.f, 0.f}, pb[2] = {0.f, 0.f};
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int r = 2 * warp + rr;
        const float a = S.z2[r][lane], b = S.z2[r][lane + 32];
        const float mu = warp_sum(a + b) * (1.f / HD);
        const float var = warp_sum((a - mu) * (a - mu) + (b - mu) * (b - mu)) * (1.f / HD);
        const float rs = 1.f / sqrtf(var + p.eps);
        float xh[2], gy[2], gxh[2], u[2], vv[2], sg = 0.f, sgx = 0.f, sv = 0.f, svx = 0.f;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = lane + 32 * e;
          xh[e] = ((e ? b : a) - mu) * rs;
          gy[e] = gam[c] * xh[e] + bet[c] - (S.v[r][c] - S.k[r][c]);
          gxh[e] = gy[e] * gam[c];
          u[e] = S.dg2[r][c];
          vv[e] = -u[e] * rs;
          sg += gxh[e];
          sgx += gxh[e] * xh[e];
          sv += vv[e];
          svx += vv[e] * xh[e];
        }
        sg = warp_sum(sg) * (1.f / HD);
        sgx = warp_sum(sgx) * (1.f / HD);
        sv = warp_sum(sv) * (1.f / HD);
        svx = warp_sum(svx) * (1.f / HD);
        float dxh[2], sd = 0.f, sS = 0.f;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = lane + 32 * e;
          const float G = (gxh[e] - sg - xh[e] * sgx) * rs;
          const float dgxh = u[e] * rs + sv + xh[e] * svx;
          const float dy = gam[c] * dgxh;
          pg[e] += gy[e] * dgxh + dy * xh[e];
          pb[e] += dy;
          dxh[e] = dy * gam[c] + gxh[e] * svx + vv[e] * sgx;
          sd += dxh[e];
          sS += -(dxh[e] * xh[e] + u[e] * G) * rs;
          S.gl1[r][c] = -gam[c] * dgxh;                           // d target (gl1 is dead from here on)
        }
        sd = warp_sum(sd) * (1.f / HD);
        sS = warp_sum(sS) * (1.f / HD);
#pragma unroll
        for (int e = 0; e < 2; ++e) S.dz2[r][lane + 32 * e] = dxh[e] * rs - sd * rs + xh[e] * sS;
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        S.colpart[warp][lane + 32 * e] = pg[e];
        S.colpart[warp][64 + lane + 32 * e] = pb[e];
      }
    }
    __syncthreads();
    if (tid < 2 * HD) {
      float s_ = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s_ += S.colpart[w][tid];
      if (tid < HD) S.dgam[tid] += s_; else S.dbet[tid - HD] += s_;
    }
    // ---- 8./9./10. z2 = x2 W2 + b2, x2 = gelu(z1), z1 = K W1 + b1
    tile_mma<true>(mt3, mdz2, tr(mW2), CS, E, F, 1.f);            // dx2 += dz2 W2^T
    __syncthreads();
    for (int e = tid; e < CS * E; e += MB_THREADS) S.t4[0][e] += S.t3[0][e] * gelu_d1(S.z1[0][e]);  // dz1 += dx2 o gelu'
    __syncthreads();
    tile_mma<true>(mdk, mt4, tr(mW1), CS, F, E, 1.f);             // dk += dz1 W1^T
    // ---- gradients w.r.t. this stage's state (all reads of the next-stage gradients are done)
    tile_mma<true>(mdW2, tr(mx2b), mdz2b, E, F, CS, 1.f);         // dW2 += x2b^T dz2b
    tile_mma<true>(mdW2, tr(mx2), mdz2, E, F, CS, 1.f);           // dW2 += x2^T dz2
    tile_mma<true>(mdW1, tr(mQ), mt1, F, E, CS, 1.f);             // dW1 += Q^T dz1b
    tile_mma<true>(mdW1, tr(mK), mt4, F, E, CS, 1.f);             // dW1 += K^T dz1
    add_colsum(db2, &S.dz2b[0][0], F, nullptr, 1.f);
    add_colsum(db1, &S.t1[0][0], E, nullptr, 1.f);
    __syncthreads();
    add_colsum(db2, &S.dz2[0][0], F, nullptr, 1.f);
    add_colsum(db1, &S.t4[0][0], E, nullptr, 1.f);
    // ---- 11. eta factors and outputs of the stage
    if (tid < CS) {
      const int i = tid;
      float dte = 0.f, dlr = 0.f;
      for (int j = 0; j < CS; ++j) {
        dte += S.deta[i][j] * S.lr[j];
        dlr += S.deta[j][i] * S.te[j];
      }
      if (i == CS - 1)
        for (int j = 0; j < CS; ++j) dte += S.dell[j] * S.lr[j];
      dlr += S.dell[i] * te_last;
      p.part_te[(size_t)stream * p.T + (size_t)s * CS + i] = dte;
      st_from_float<T>(p.d_lr, row_base + (size_t)s * CS + i, dlr);
    }
    __syncthreads();
    for (int e = tid; e < CS * F; e += MB_THREADS) {
      S.dq[0][e] += S.dO[0][e];
      S.dk[0][e] -= S.gl1[0][e];  // gl1 holds d target: dk -= dT, dv = dT
    }
    __syncthreads();
    store_tile_bf16(static_cast<T*>(p.d_q) + r0, S.dq);
    store_tile_bf16(static_cast<T*>(p.d_k) + r0, S.dk);
    store_tile_bf16(static_cast<T*>(p.d_v) + r0, S.gl1);
    __syncthreads();
  }

  // ---- gradients w.r.t. the initial state, per-stream LayerNorm parameter gradients
  for (int e = tid; e < F * E; e += MB_THREADS) {
    st_from_float<T>(p.d_w1, (size_t)stream * F * E + e, dW1[e]);
    st_from_float<T>(p.d_w2, (size_t)stream * F * E + e, dW2[e]);
  }
  for (int e = tid; e < E; e += MB_THREADS) st_from_float<T>(p.d_b1, (size_t)stream * E + e, db1[e]);
  if (tid < F) {
    st_from_float<T>(p.d_b2, (size_t)stream * F + tid, db2[tid]);
    p.part_ln[(size_t)stream * 2 * HD + tid] = S.dgam[tid];
    p.part_ln[(size_t)stream * 2 * HD + HD + tid] = S.dbet[tid];
  }
}

// grad_token_eta[t] = sum over streams, grad_ln_weight / grad_ln_bias [h][f] = sum over the batch; fixed order.
__global__ void ttt_mlp_bwd_reduce_kernel(const float* part_te, const float* part_ln, int B, int H, int T, float* dte,
                                          float* dg, float* db) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < T) {
    float s = 0.f;
    for (int st = 0; st < B * H; ++st) s += part_te[(size_t)st * T + i];
    dte[i] = s;
  } else if (i < T + 2 * H * HD) {
    const int j = i - T, which = j / (H * HD), hf = j % (H * HD), h = hf / HD, f = hf % HD;
    float s = 0.f;
    for (int b = 0; b < B; ++b) s += part_ln[((size_t)(b * H + h) * 2 + which) * HD + f];
    (which ? db : dg)[hf] = s;
  }
}

size_t mlp_bwd_ws_stride_floats(int T) {
  const size_t ns = (size_t)T / CS;
  return 4 * (size_t)HD * MB_E + 2 * (MB_E + HD) + ns * CS * (MB_E + HD);
}

cudaError_t launch_mlp_bwd(const MlpBwdParams& p, int B, cudaStream_t st) {
  const size_t smem = sizeof(MlpBwdSmem);
  cudaError_t e = cudaFuncSetAttribute(ttt_mlp_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  ttt_mlp_bwd_kernel<<<B * p.H, MB_THREADS, smem, st>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int n = p.T + 2 * p.H * HD;
  ttt_mlp_bwd_reduce_kernel<<<(n + 255) / 256, 256, 0, st>>>(p.part_te, p.part_ln, B, p.H, p.T, p.d_token_eta,
                                                           p.d_ln_g, p.d_ln_b);
  return cudaGetLastError();
}

}  // namespace ttt
