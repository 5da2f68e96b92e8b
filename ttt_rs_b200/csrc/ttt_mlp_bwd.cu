// TTT-MLP backward (bf16 I/O, float32 state), first version: one 16-warp CTA per (batch, head) stream.
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

constexpr int MB_THREADS = 512;
constexpr int MB_NW = MB_THREADS / 32;  // warps of the CTA
constexpr int MB_RPW = CS / MB_NW;       // tile rows a warp owns in the row-wise (LayerNorm) steps
constexpr int MB_E = 256;  // hidden width of the inner MLP (4 * head_dim)
// Row strides of the shared-memory tiles: width + 8 floats.  With a stride of 8 (mod 32) the 64-bit fragment loads of
// a half-warp (4 rows x 4 column pairs) fall in 16 distinct bank pairs; unpadded rows would put the 8 rows of a
// fragment in the same bank (8-way conflicts on every operand load).
constexpr int EP = MB_E + 8, FP = HD + 8, CP = CS + 8;
constexpr float GELU_C0 = 0.7978845608028654f, GELU_C1 = 0.044715f;

// A float32 matrix view with compile-time strides: element (i, j) at p[i * RS + j * CS_] (shared or global memory).
template <int RS, int CS_>
struct MatT {
  float* p;
  static constexpr int rs = RS, cs = CS_;
};
template <int RS, int CS_>
__device__ __forceinline__ MatT<CS_, RS> tr(const MatT<RS, CS_> m) { return MatT<CS_, RS>{m.p}; }
// the pair (i, k), (i, k+1) of an A operand / the pair (k, j), (k+1, j) of a B operand: one 64-bit load when the
// pair is contiguous in memory (k even, strides even, bases 8-byte aligned)
template <class MA>
__device__ __forceinline__ float2 pair_k_of_A(const MA m, int i, int k) {
  const float* q = m.p + i * MA::rs + k * MA::cs;
  if constexpr (MA::cs == 1) return *reinterpret_cast<const float2*>(q);
  else return make_float2(q[0], q[MA::cs]);
}
template <class MB>
__device__ __forceinline__ float2 pair_k_of_B(const MB m, int k, int j) {
  const float* q = m.p + k * MB::rs + j * MB::cs;
  if constexpr (MB::rs == 1) return *reinterpret_cast<const float2*>(q);
  else return make_float2(q[0], q[MB::rs]);
}

// C[M x N] = (ACC ? C : 0) + alpha * A[M x K] . B[K x N];  M % 16 == 0, N % 8 == 0, K in {16, 64, 256}; every
// extent and stride is a compile-time constant, so operand addresses are a lane offset plus immediates.
// Output tiles of 16 x 8 are dealt to the warps round-robin (the same tile always goes to the same warp, so
// successive accumulations into one matrix need no barrier between them).  A warp works on up to four of its tiles
// at a time with the contraction loop unrolled by two, so that the operand loads of several fragments (many of them
// from the L2-resident state in the workspace) are in flight together.
template <bool ACC, int K, int M, int N, class MC, class MA, class MB>
__device__ void tile_mma(const MC C, const MA A, const MB B, float alpha) {
  constexpr int NW = MB_THREADS / 32, ntn = N / 8, total = (M / 16) * ntn;
  // Tiles of a warp in flight together: tile0 + u * NW, u < TG.  When the tiles of a row of the output go round the
  // warps a whole number of times (ntn = NW * TG) they share their rows (one A fragment serves all of them); when NW
  // is a multiple of ntn they share their columns (one B fragment).
  constexpr int TG0 = total >= 4 * NW ? 4 : (total + NW - 1) / NW;
  constexpr int TG = (ntn % NW == 0 && ntn / NW >= 2 && ntn / NW <= 4) ? ntn / NW : TG0;
  constexpr bool SHARE_A = TG > 1 && (ntn % (NW * TG) == 0);
  constexpr bool SHARE_B = TG > 1 && !SHARE_A && (NW % ntn == 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll 1
  for (int tile0 = warp; tile0 < total; tile0 += NW * TG) {
    int i0[TG], j0[TG];
    bool on[TG];
    float acc[TG][4], cin[TG][4];
#pragma unroll
    for (int u = 0; u < TG; ++u) {
      const int tile = tile0 + u * NW;
      on[u] = tile < total;
      const int tl = on[u] ? tile : tile0, mt = tl / ntn;
      i0[u] = 16 * mt + g;
      j0[u] = 8 * (tl - mt * ntn);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[u][q] = 0.f;
        cin[u][q] = (ACC && on[u]) ? C.p[(i0[u] + 8 * (q >> 1)) * MC::rs + (j0[u] + 2 * t + (q & 1)) * MC::cs] : 0.f;
      }
    }
#pragma unroll(K >= 64 ? 2 : 1)
    for (int k0 = 0; k0 < K; k0 += 16) {
      const int ka = k0 + 2 * t, kb = ka + 8;
      uint32_t pa[TG][4], pb[TG][2];
#pragma unroll
      for (int u = 0; u < TG; ++u) {
        if (u == 0 || !SHARE_A) {
          const float2 f0 = pair_k_of_A(A, i0[u], ka), f1 = pair_k_of_A(A, i0[u] + 8, ka);
          const float2 f2_ = pair_k_of_A(A, i0[u], kb), f3 = pair_k_of_A(A, i0[u] + 8, kb);
          pa[u][0] = pack_bf16(f0.x, f0.y); pa[u][1] = pack_bf16(f1.x, f1.y);
          pa[u][2] = pack_bf16(f2_.x, f2_.y); pa[u][3] = pack_bf16(f3.x, f3.y);
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) pa[u][q] = pa[0][q];
        }
        if (u == 0 || !SHARE_B) {
          const float2 h0 = pair_k_of_B(B, ka, j0[u] + g), h1 = pair_k_of_B(B, kb, j0[u] + g);
          pb[u][0] = pack_bf16(h0.x, h0.y); pb[u][1] = pack_bf16(h1.x, h1.y);
        } else {
          pb[u][0] = pb[0][0]; pb[u][1] = pb[0][1];
        }
      }
#pragma unroll
      for (int u = 0; u < TG; ++u) mma_bf16(acc[u], pa[u][0], pa[u][1], pa[u][2], pa[u][3], pb[u][0], pb[u][1]);
    }
#pragma unroll
    for (int u = 0; u < TG; ++u)
      if (on[u]) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float* c = C.p + (i0[u] + 8 * (q >> 1)) * MC::rs + (j0[u] + 2 * t + (q & 1)) * MC::cs;
          *c = cin[u][q] + alpha * acc[u][q];
        }
      }
  }
}

// tanh(x) = 1 - 2 / (1 + e^{2x}) with the fast exponential and division (relative error ~1e-6, as in the forward kernel)
__device__ __forceinline__ float tanh_fast(float x) { return 1.f - __fdividef(2.f, 1.f + __expf(2.f * x)); }
__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + tanh_fast(GELU_C0 * x * (1.f + GELU_C1 * x * x))); }
__device__ __forceinline__ float gelu_d1(float x) {
  const float th = tanh_fast(GELU_C0 * x * (1.f + GELU_C1 * x * x));
  return 0.5f * x * ((1.f - th * th) * (GELU_C0 + 3.f * GELU_C0 * GELU_C1 * x * x)) + 0.5f * (1.f + th);
}
__device__ __forceinline__ float gelu_d2(float x) {
  const float th = tanh_fast(GELU_C0 * x * (1.f + GELU_C1 * x * x));
  const float du = GELU_C0 * (1.f + 3.f * GELU_C1 * x * x), d2u = 6.f * GELU_C0 * GELU_C1 * x;
  return (1.f - th * th) * du + 0.5f * x * (1.f - th * th) * (d2u - 2.f * th * du * du);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Shared-memory tiles (float32, [16][width + 8]).
struct MlpBwdSmem {
  float z1[CS][EP], x2[CS][EP], g1[CS][EP], z1b[CS][EP], x2b[CS][EP];
  float t1[CS][EP], t2[CS][EP], t3[CS][EP], t4[CS][EP];  // dx2b/dz1b, dg1/dh, dx2, dz1 (+ scratch)
  float q[CS][FP], k[CS][FP], v[CS][FP], dO[CS][FP];
  float z2[CS][FP], g2[CS][FP], z2b[CS][FP], dz2b[CS][FP], dg2[CS][FP], dz2[CS][FP], dk[CS][FP], gl1[CS][FP];
  float eta[CS][CP], a1[CS][CP], a2[CS][CP], m1[CS][CP], m2[CS][CP], dm[CS][CP], da[CS][CP], deta[CS][CP];
  float lr[CS], te[CS], ell[CS], dell[CS];
  float b1[MB_E], db1[MB_E], b2[HD], db2[HD];  // biases and their gradients stay on chip for the whole walk
  float dgam[HD], dbet[HD];  // this stream's LayerNorm parameter gradients
};
static_assert(sizeof(MlpBwdSmem) + 1024 <= 227 * 1024, "shared-memory tiles exceed one SM");

// G = d/dz of 0.5 |LN(z) - (v - k)|^2 for a [16][64] tile (rust/core/src/util.rs:155-182)
__device__ void ln_l2_grad_tile(MlpBwdSmem& S, const float (*z)[FP], float (*G)[FP], const float* gam, const float* bet,
                                float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int rr = 0; rr < MB_RPW; ++rr) {
    const int r = MB_RPW * warp + rr;
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

// column sums of a [16][N] tile (row stride ld) added, with sign, to dst[N]
__device__ void add_colsum(float* dst, const float* tile, int N, int ld, float sign) {
  for (int c = threadIdx.x; c < N; c += MB_THREADS) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < CS; ++r) s += tile[r * ld + c];
    dst[c] += sign * s;
  }
}

// Up to four [16][64] bf16 tiles from global memory into float32 shared tiles: every thread owns two consecutive
// elements (one 4-byte load) of each tile, and all loads are issued before the first value is used (a load that
// waits behind the previous tile's dependent stores would cost a full memory round trip per tile).
template <int NT>
__device__ void load_tiles_bf16(float (*const (&dst)[NT])[FP], const __nv_bfloat16* const (&src)[NT]) {
  static_assert(MB_THREADS * 2 == CS * HD, "two elements per thread");
  const int e = 2 * threadIdx.x, r = e / HD, c = e % HD;
  uint32_t raw[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) raw[i] = *reinterpret_cast<const uint32_t*>(src[i] + e);
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    dst[i][r][c] = bf16_lo(raw[i]);
    dst[i][r][c + 1] = bf16_hi(raw[i]);
  }
}
__device__ void store_tile_bf16(__nv_bfloat16* dst, const float (*src)[FP]) {
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
  float* g1p_all = dW2 + E * F + 2 * (E + F);  // (2 (E + F) floats of the stride are unused)
  float* const b1 = S.b1;
  float* const b2 = S.b2;
  float* const db1 = S.db1;
  float* const db2 = S.db2;
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
#ifdef TTT_MLP_TRACE
  unsigned long long tr_acc[16] = {0}, tr_last = clock64();
#define TRM(i) { __syncthreads(); const unsigned long long n_ = clock64(); tr_acc[i] += n_ - tr_last; tr_last = n_; }
#else
#define TRM(i)
#endif

  const MatT<MB_E, 1> mW1{W1}, mdW1{dW1};
  const MatT<HD, 1> mW2{W2}, mdW2{dW2};
  const MatT<FP, 1> mK{&S.k[0][0]}, mQ{&S.q[0][0]};
  const MatT<EP, 1> mz1{&S.z1[0][0]}, mx2{&S.x2[0][0]}, mg1{&S.g1[0][0]}, mz1b{&S.z1b[0][0]}, mx2b{&S.x2b[0][0]};
  const MatT<EP, 1> mt1{&S.t1[0][0]}, mt2{&S.t2[0][0]}, mt3{&S.t3[0][0]}, mt4{&S.t4[0][0]};
  const MatT<FP, 1> mz2{&S.z2[0][0]}, mg2{&S.g2[0][0]}, mz2b{&S.z2b[0][0]};
  const MatT<FP, 1> mdz2b{&S.dz2b[0][0]}, mdg2{&S.dg2[0][0]}, mdz2{&S.dz2[0][0]}, mdk{&S.dk[0][0]}, mgl1{&S.gl1[0][0]};
  const MatT<FP, 1> mdq = mz2b;  // z2b is dead once the output LayerNorm has been differentiated: its tile then holds dq
  float(*const dq)[FP] = S.z2b;
  const MatT<CP, 1> ma1{&S.a1[0][0]}, ma2{&S.a2[0][0]}, mm1{&S.m1[0][0]}, mm2{&S.m2[0][0]}, mdm{&S.dm[0][0]}, mda{&S.da[0][0]};

// element-wise loops over a [16][E] / [16][F] / [16][16] tile: r = row (token), c = column
#define FOR_E(r, c) for (int e_ = tid, r = e_ / MB_E, c = e_ % MB_E; e_ < CS * MB_E; e_ += MB_THREADS, r = e_ / MB_E, c = e_ % MB_E)
#define FOR_F(r, c) for (int e_ = tid, r = e_ / HD, c = e_ % HD; e_ < CS * HD; e_ += MB_THREADS, r = e_ / HD, c = e_ % HD)
#define FOR_C(r, c) for (int e_ = tid, r = e_ / CS, c = e_ % CS; e_ < CS * CS; e_ += MB_THREADS, r = e_ / CS, c = e_ % CS)

  // z1 = K W1 + b1, x2 = gelu(z1), z2 = x2 W2 + b2, g2, g1 = (g2 W2^T) o gelu'(z1)   (from the state in the workspace)
  auto forward_first_layer = [&]() {
    tile_mma<false, HD, CS, MB_E>(mz1, mK, mW1, 1.f);
    __syncthreads();
    FOR_E(r, c) {
      const float z = S.z1[r][c] + b1[c];
      S.z1[r][c] = z;
      S.x2[r][c] = gelu_f(z);
    }
    __syncthreads();
  };
  auto forward_second_layer = [&]() {
    tile_mma<false, MB_E, CS, HD>(mz2, mx2, mW2, 1.f);
    __syncthreads();
    FOR_F(r, c) S.z2[r][c] += b2[c];
    __syncthreads();
    ln_l2_grad_tile(S, S.z2, S.g2, gam, bet, p.eps);
    __syncthreads();
    tile_mma<false, HD, CS, MB_E>(mg1, mg2, tr(mW2), 1.f);
    __syncthreads();
    FOR_E(r, c) S.g1[r][c] *= gelu_d1(S.z1[r][c]);
    __syncthreads();
  };

  // ============================== pass 1: forward walk, saving g1p and g2p ==============================
  for (int s = 0; s < NS; ++s) {
    const size_t r0 = (row_base + (size_t)s * CS) * HD;
    {
      float(*const dst[2])[FP] = {S.k, S.v};
      const T* const src[2] = {static_cast<const T*>(p.xk) + r0, static_cast<const T*>(p.xv) + r0};
      load_tiles_bf16<2>(dst, src);
    }
    if (tid < CS) S.ell[tid] = te_last * ld_as_float<T>(p.lr, row_base + (size_t)s * CS + tid);
    __syncthreads();
    TRM(0)
    forward_first_layer();
    forward_second_layer();
    TRM(1)
    float* g1p = g1p_all + (size_t)s * CS * E;
    float* g2p = g2p_all + (size_t)s * CS * F;
    FOR_E(r, c) {
      const float v_ = S.ell[r] * S.g1[r][c];
      g1p[e_] = v_;
      S.t1[r][c] = v_;
    }
    FOR_F(r, c) {
      const float v_ = S.ell[r] * S.g2[r][c];
      g2p[e_] = v_;
      S.dg2[r][c] = v_;
    }
    __syncthreads();
    tile_mma<true, CS, HD, MB_E>(mW1, tr(mK), mt1, -1.f);   // W1 -= K^T g1p
    tile_mma<true, CS, MB_E, HD>(mW2, tr(mx2), mdg2, -1.f);  // W2 -= X2^T g2p
    add_colsum(b1, &S.t1[0][0], E, EP, -1.f);
    add_colsum(b2, &S.dg2[0][0], F, FP, -1.f);
    __syncthreads();
    TRM(2)
  }

  // ============================== pass 2: backward walk ==============================
  for (int s = NS - 1; s >= 0; --s) {
    const size_t r0 = (row_base + (size_t)s * CS) * HD;
    const float* g1p = g1p_all + (size_t)s * CS * E;
    const float* g2p = g2p_all + (size_t)s * CS * F;
    {
      // every global load of the stage's inputs is issued before the first dependent store
      constexpr int G1V = CS * MB_E / 4 / MB_THREADS;
      float4 g1v[G1V];
#pragma unroll
      for (int i = 0; i < G1V; ++i) g1v[i] = reinterpret_cast<const float4*>(g1p)[tid + MB_THREADS * i];
      const float2 g2v = reinterpret_cast<const float2*>(g2p)[tid];
      float(*const dst[4])[FP] = {S.q, S.k, S.v, S.dO};
      const T* const src[4] = {static_cast<const T*>(p.xq) + r0, static_cast<const T*>(p.xk) + r0,
                               static_cast<const T*>(p.xv) + r0, static_cast<const T*>(p.d_out) + r0};
      load_tiles_bf16<4>(dst, src);
#pragma unroll
      for (int i = 0; i < G1V; ++i) {
        const int e = 4 * (tid + MB_THREADS * i), r = e / MB_E, c = e % MB_E;
        S.t1[r][c] = g1v[i].x; S.t1[r][c + 1] = g1v[i].y; S.t1[r][c + 2] = g1v[i].z; S.t1[r][c + 3] = g1v[i].w;
      }
      const int e = 2 * tid, r = e / HD, c = e % HD;
      S.dg2[r][c] = g2v.x; S.dg2[r][c + 1] = g2v.y;
    }
    if (tid < CS) {
      S.lr[tid] = ld_as_float<T>(p.lr, row_base + (size_t)s * CS + tid);
      S.ell[tid] = te_last * S.lr[tid];
    }
    __syncthreads();
    TRM(3)
    // ---- state at the start of this stage: undo the stage's updates (W1 first: X2 depends on it)
    tile_mma<true, CS, HD, MB_E>(mW1, tr(mK), mt1, 1.f);
    add_colsum(b1, &S.t1[0][0], E, EP, 1.f);
    __syncthreads();
    forward_first_layer();  // z1 and x2 of this stage, needed to undo the second layer's update
    tile_mma<true, CS, MB_E, HD>(mW2, tr(mx2), mdg2, 1.f);
    add_colsum(b2, &S.dg2[0][0], F, FP, 1.f);
    __syncthreads();
    TRM(4)
    // ---- forward intermediates of the stage
    forward_second_layer();
    TRM(5)
    FOR_C(i, j) S.eta[i][j] = (j <= i) ? S.te[i] * S.lr[j] : 0.f;
    tile_mma<false, HD, CS, CS>(ma1, mQ, tr(mK), 1.f);
    __syncthreads();
    FOR_C(i, j) {
      const float a = (j <= i) ? S.a1[i][j] : 0.f;
      S.a1[i][j] = a;
      S.m1[i][j] = S.eta[i][j] * (1.f + a);
    }
    tile_mma<false, HD, CS, MB_E>(mz1b, mQ, mW1, 1.f);
    __syncthreads();
    tile_mma<true, CS, CS, MB_E>(mz1b, mm1, mg1, -1.f);
    __syncthreads();
    FOR_E(r, c) {
      const float z = S.z1b[r][c] + b1[c];
      S.z1b[r][c] = z;
      S.x2b[r][c] = gelu_f(z);
    }
    __syncthreads();
    tile_mma<false, MB_E, CS, CS>(ma2, mx2b, tr(mx2), 1.f);
    tile_mma<false, MB_E, CS, HD>(mz2b, mx2b, mW2, 1.f);
    __syncthreads();
    FOR_C(i, j) {
      const float a = (j <= i) ? S.a2[i][j] : 0.f;
      S.a2[i][j] = a;
      S.m2[i][j] = S.eta[i][j] * (1.f + a);
    }
    __syncthreads();
    tile_mma<true, CS, CS, HD>(mz2b, mm2, mg2, -1.f);
    __syncthreads();
    FOR_F(r, c) S.z2b[r][c] += b2[c];
    __syncthreads();

    TRM(6)
    // ---- 1. output LayerNorm: dz2b, LN parameter gradients (per-warp column partials in t4, not live yet)
    float(*colpart)[2 * HD] = reinterpret_cast<float(*)[2 * HD]>(&S.t4[0][0]);
    {
      float pg[2] = {0.f, 0.f}, pb[2] = {0.f, 0.f};
#pragma unroll
      for (int rr = 0; rr < MB_RPW; ++rr) {
        const int r = MB_RPW * warp + rr;
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
        colpart[warp][lane + 32 * e] = pg[e];
        colpart[warp][64 + lane + 32 * e] = pb[e];
      }
    }
    __syncthreads();
    if (tid < 2 * HD) {
      float s_ = 0.f;
#pragma unroll
      for (int w = 0; w < MB_NW; ++w) s_ += colpart[w][tid];
      if (tid < HD) S.dgam[tid] += s_; else S.dbet[tid - HD] += s_;
    }
    TRM(7)
    // ---- 2. z2b = x2b W2 + b2 - M2 g2
    tile_mma<false, HD, CS, MB_E>(mt1, mdz2b, tr(mW2), 1.f);         // dx2b = dz2b W2^T
    tile_mma<false, HD, CS, CS>(mdm, mdz2b, tr(mg2), -1.f);        // dM2 = -tril(dz2b g2^T)
    tile_mma<false, CS, CS, HD>(mdg2, tr(mm2), mdz2b, -1.f);        // dg2 = -M2^T dz2b
    __syncthreads();
    FOR_C(i, j) {
      const float d = (j <= i) ? S.dm[i][j] : 0.f;
      S.da[i][j] = d * S.eta[i][j];
      S.deta[i][j] = d * (1.f + S.a2[i][j]);
    }
    __syncthreads();
    tile_mma<true, CS, CS, MB_E>(mt1, mda, mx2, 1.f);                // dx2b += dA2 x2
    tile_mma<false, CS, CS, MB_E>(mt3, tr(mda), mx2b, 1.f);           // dx2 = dA2^T x2b
    __syncthreads();
    TRM(8)
    // ---- 3./4. dz1b = dx2b o gelu'(z1b);  z1b = Q W1 + b1 - M1 g1
    FOR_E(r, c) S.t1[r][c] *= gelu_d1(S.z1b[r][c]);
    __syncthreads();
    tile_mma<false, MB_E, CS, HD>(mdq, mt1, tr(mW1), 1.f);          // dq = dz1b W1^T
    tile_mma<false, MB_E, CS, CS>(mdm, mt1, tr(mg1), -1.f);        // dM1 = -tril(dz1b g1^T)
    tile_mma<false, CS, CS, MB_E>(mt2, tr(mm1), mt1, -1.f);           // dg1 = -M1^T dz1b
    __syncthreads();
    FOR_C(i, j) {
      const float d = (j <= i) ? S.dm[i][j] : 0.f;
      S.da[i][j] = d * S.eta[i][j];
      S.deta[i][j] += d * (1.f + S.a1[i][j]);
    }
    __syncthreads();
    TRM(9)
    tile_mma<true, CS, CS, HD>(mdq, mda, mK, 1.f);                 // dq += dA1 K
    tile_mma<false, CS, CS, HD>(mdk, tr(mda), mQ, 1.f);             // dk = dA1^T Q
    // ---- 5. the four state updates; dW1, db1, dW2, db2 still hold the gradients w.r.t. the next stage's state
    tile_mma<false, MB_E, CS, HD>(mgl1, mg1, tr(mdW1), 1.f);        // gl1 = g1 dW1^T
    tile_mma<false, HD, CS, MB_E>(mt4, mg2, tr(mdW2), 1.f);           // gl2 = g2 dW2^T   (t4 as scratch)
    //   dg1 -= (l o K) dW1 + l (x) db1 : l o K is built in dz2, which is free until step 7
    FOR_F(r, c) S.dz2[r][c] = S.ell[r] * S.k[r][c];
    __syncthreads();
    tile_mma<true, HD, CS, MB_E>(mt2, mdz2, mdW1, -1.f);             // dg1 -= (l o K) dW1
    //   dg2 -= (l o x2) dW2 + l (x) db2 : l o x2 goes to z1b (dead after step 3)
    FOR_E(r, c) S.z1b[r][c] = S.ell[r] * S.x2[r][c];
    __syncthreads();
    FOR_E(r, c) {
      S.t2[r][c] -= S.ell[r] * db1[c];
      S.t3[r][c] -= S.ell[r] * S.t4[r][c];                        // dx2 -= l o gl2
    }
    tile_mma<true, MB_E, CS, HD>(mdg2, mz1b, mdW2, -1.f);
    __syncthreads();
    FOR_F(r, c) {
      S.dg2[r][c] -= S.ell[r] * db2[c];
      S.dk[r][c] -= S.ell[r] * S.gl1[r][c];                       // dk -= l o gl1
    }
    // dell[j] = -( gl1[j].K[j] + g1[j].db1 + gl2[j].x2[j] + g2[j].db2 )
#pragma unroll
    for (int rr = 0; rr < MB_RPW; ++rr) {
      const int r = MB_RPW * warp + rr;
      float acc = 0.f;
      for (int c = lane; c < F; c += 32) acc += S.gl1[r][c] * S.k[r][c] + S.g2[r][c] * db2[c];
      for (int c = lane; c < E; c += 32) acc += S.g1[r][c] * db1[c] + S.t4[r][c] * S.x2[r][c];
      acc = warp_sum(acc);
      if (lane == 0) S.dell[r] = -acc;
    }
    __syncthreads();
    TRM(10)
    // ---- 6. g1 = h o gelu'(z1), h = g2 W2^T (recomputed into z1b, whose scratch use is over):
    //         dh = dg1 o gelu'(z1) (in t2),  dz1 = dg1 o h o gelu''(z1) (t4)
    tile_mma<false, HD, CS, MB_E>(mz1b, mg2, tr(mW2), 1.f);
    __syncthreads();
    FOR_E(r, c) {
      const float d = S.t2[r][c], z = S.z1[r][c];
      S.t4[r][c] = d * S.z1b[r][c] * gelu_d2(z);
      S.t2[r][c] = d * gelu_d1(z);
    }
    __syncthreads();
    tile_mma<true, MB_E, CS, HD>(mdg2, mt2, mW2, 1.f);             // dg2 += dh W2
    tile_mma<true, CS, MB_E, HD>(mdW2, tr(mt2), mg2, 1.f);            // dW2 += dh^T g2
    __syncthreads();
    TRM(11)
    // ---- 7. second derivative through g2 = ln_l2_grad(z2, v - k): dz2, d target, LN parameter gradients
    //         (column partials in t2: dh is no longer needed)
    colpart = reinterpret_cast<float(*)[2 * HD]>(&S.t2[0][0]);
    {
      float pg[2] = {0.f, 0.f}, pb[2] = {0.f, 0.f};
#pragma unroll
      for (int rr = 0; rr < MB_RPW; ++rr) {
        const int r = MB_RPW * warp + rr;
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
        colpart[warp][lane + 32 * e] = pg[e];
        colpart[warp][64 + lane + 32 * e] = pb[e];
      }
    }
    __syncthreads();
    if (tid < 2 * HD) {
      float s_ = 0.f;
#pragma unroll
      for (int w = 0; w < MB_NW; ++w) s_ += colpart[w][tid];
      if (tid < HD) S.dgam[tid] += s_; else S.dbet[tid - HD] += s_;
    }
    TRM(12)
    // ---- 8./9./10. z2 = x2 W2 + b2, x2 = gelu(z1), z1 = K W1 + b1
    tile_mma<true, HD, CS, MB_E>(mt3, mdz2, tr(mW2), 1.f);           // dx2 += dz2 W2^T
    __syncthreads();
    FOR_E(r, c) S.t4[r][c] += S.t3[r][c] * gelu_d1(S.z1[r][c]);   // dz1 += dx2 o gelu'(z1)
    __syncthreads();
    tile_mma<true, MB_E, CS, HD>(mdk, mt4, tr(mW1), 1.f);          // dk += dz1 W1^T
    TRM(13)
    // ---- gradients w.r.t. this stage's state (all reads of the next-stage gradients are done)
    tile_mma<true, CS, MB_E, HD>(mdW2, tr(mx2b), mdz2b, 1.f);         // dW2 += x2b^T dz2b
    tile_mma<true, CS, MB_E, HD>(mdW2, tr(mx2), mdz2, 1.f);           // dW2 += x2^T dz2
    tile_mma<true, CS, HD, MB_E>(mdW1, tr(mQ), mt1, 1.f);             // dW1 += Q^T dz1b
    tile_mma<true, CS, HD, MB_E>(mdW1, tr(mK), mt4, 1.f);             // dW1 += K^T dz1
    add_colsum(db2, &S.dz2b[0][0], F, FP, 1.f);
    add_colsum(db1, &S.t1[0][0], E, EP, 1.f);
    add_colsum(db2, &S.dz2[0][0], F, FP, 1.f);
    add_colsum(db1, &S.t4[0][0], E, EP, 1.f);
    TRM(14)
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
    FOR_F(r, c) {
      dq[r][c] += S.dO[r][c];
      S.dk[r][c] -= S.gl1[r][c];  // gl1 holds d target: dk -= dT, dv = dT
    }
    __syncthreads();
    store_tile_bf16(static_cast<T*>(p.d_q) + r0, dq);
    store_tile_bf16(static_cast<T*>(p.d_k) + r0, S.dk);
    store_tile_bf16(static_cast<T*>(p.d_v) + r0, S.gl1);
    __syncthreads();
    TRM(15)
  }
#ifdef TTT_MLP_TRACE
  if (tid == 0 && blockIdx.x == 0 && p.trace != nullptr)
    for (int i = 0; i < 16; ++i) p.trace[i] = (unsigned int)(tr_acc[i] / NS);
#endif
#undef FOR_E
#undef FOR_F
#undef FOR_C

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
