// TTT-MLP backward (bf16 I/O, float32 state): one 16-warp CTA per (batch, head) stream.
//
// What it computes: the gradient of the whole-sequence TTT-MLP forward (semantics rust/core/src/mlp.rs:127-208; the
// reference obtains this gradient from Burn autodiff, it has no fused MLP kernel) for loss = <grad_output, output>:
// grad_xq/xk/xv, grad_w1/b1/w2/b2 (per batch element), grad_ttt_lr_eta, and per-stream partials of grad_token_eta and
// of the LayerNorm parameter gradients (summed over streams in a fixed order by ttt_mlp_bwd_reduce_kernel).
//
// How: the stage-by-stage analytic backward (reverse walk over the mini-batches carrying dW1, db1, dW2, db2; GELU
// and LayerNorm second derivatives).
//   pass 1 walks forward once and saves the lr-scaled inner gradients g1p = lr o g1, g2p = lr o g2 of every stage
//          (bf16: exactly the operand values of the state update, so that pass 2 can undo the update); the forward
//          kernel can do this instead while it runs (it then also leaves the final state in the workspace);
//   pass 2 walks backward: W1_s = W1_{s+1} + K^T g1p, W2_s = W2_{s+1} + X2^T g2p recover the state of the stage,
//          the stage's forward intermediates are recomputed from it, and the gradient steps follow.
// Where things live: the float32 masters of W1, W2, dW1, dW2 (256 KB per stream) sit in the SM's tensor memory while a
// work item runs (each thread owns the 128 floats its accumulator fragments update, see MatM) and in the workspace
// between work items; every matrix that is an operand of a product sits in shared memory as a padded row-major bf16
// tile that ldmatrix reads directly (the 16 x 256 and 16 x 64 working tiles, and bf16 shadows of W1 and W2 refreshed
// by the same epilogue that updates the masters) -- except dW1 and dW2, for whose bf16 copies shared memory has no
// room: those are in the workspace (MatH).  Tiles that only accumulate or feed a LayerNorm (z2, z2b, dg2, dk, ...)
// are float32.  Operand precision is the forward kernel's: bf16 operands, float32 accumulation.
#include <type_traits>

#include "ttt_kernels.h"
#include "ttt_common.cuh"

namespace ttt {

constexpr int MB_THREADS = 512;
constexpr int MB_NW = MB_THREADS / 32;  // warps of the CTA
constexpr int MB_E = 256;               // hidden width of the inner MLP (4 * head_dim)
constexpr int MLP_BWD_CHUNK = 8;        // stages per work item
static_assert(MB_NW == CS, "the row-wise (LayerNorm) steps give one tile row to each warp");
// Row lengths of the shared-memory tiles: width + 8 elements.  For bf16 tiles the row stride is then an odd multiple
// of 16 bytes, so the eight 16-byte rows of an ldmatrix 8x8 block fall in distinct banks; for float32 tiles a stride
// of 8 (mod 32) words makes the 64-bit accesses of a half-warp (4 rows x 4 column pairs) conflict-free.
constexpr int EB = MB_E + 8, FB = HD + 8, CB = CS + 8;  // bf16 tiles
constexpr int FP = HD + 8, CP = CS + 8;                 // float32 tiles
constexpr float GELU_C0 = 0.7978845608028654f, GELU_C1 = 0.044715f;
typedef __nv_bfloat16 bf;

// ---- matrix views ----------------------------------------------------------------------------------------------
// float32 matrix with compile-time strides: element (i, j) at p[i * RS + j * CS_] (global or shared memory)
template <int RS, int CS_>
struct MatT {
  float* p;
  static constexpr int rs = RS, cs = CS_;
};
template <int RS, int CS_>
__device__ __forceinline__ MatT<CS_, RS> tr(const MatT<RS, CS_> m) { return MatT<CS_, RS>{m.p}; }
// bf16 tile in shared memory, rows of LD elements, given by the shared-space byte address of element (0, 0).
// TR = true: the operand is the transpose of the stored tile.
template <int LD, bool TR>
struct SB {
  uint32_t a;
};
template <int LD, bool TR>
__device__ __forceinline__ SB<LD, !TR> tr(const SB<LD, TR> m) { return SB<LD, !TR>{m.a}; }

// float32 matrix [R][C] in the workspace, stored tile by tile in accumulator-fragment order: the 16 x 8 tile
// (r / 16, c / 8) occupies 128 consecutive floats, its rows 0..7 before its rows 8..15, and inside a half the
// element (r % 8, c % 8) sits at 8 * (r % 8) + (c % 8).  A warp's read-modify-write of an output tile is then two
// contiguous 256-byte accesses instead of sixteen 32-byte row pieces, and so are the operand fetches along a row.
// TR = true: the operand is the transpose of the stored matrix.  Successive work items of a stream may run on
// different SMs, so every read of these matrices bypasses L1 (ld.global.cg).
template <int R, int C, bool TR>
struct MatG {
  float* p;
  static __device__ __forceinline__ int at(int r, int c) { return mlp_state_at(r, c, C); }
};
template <int R, int C, bool TR>
__device__ __forceinline__ MatG<R, C, !TR> tr(const MatG<R, C, TR> m) { return MatG<R, C, !TR>{m.p}; }

// bf16 copy of a float32 matrix [R][C] of the workspace, read as the B operand of a product in either orientation
// (the state gradients dW1, dW2 enter four products per stage, two of them transposed).  Stored in 8 x 8 supertiles
// of 128 bytes; inside a supertile in 2 x 2 blocks of 8 bytes, rows of a block one after the other: element (r, c)
// sits at mlp_shadow_at(r, c, C).  A B-fragment register is then one 32-bit load (pair along a row) or one 64-bit
// load and a byte permute (pair along a column), every warp-wide load is one 128-byte line in both orientations, and
// the writer's accumulator pair (r, c), (r, c + 1) is one 32-bit store (a warp's half tile = one line).
__host__ __device__ inline int mlp_shadow_at(int r, int c, int C) {
  return (((r >> 3) * (C >> 3) + (c >> 3)) << 6) + (((((r >> 1) & 3) << 2) + ((c >> 1) & 3)) << 2) + ((r & 1) << 1) + (c & 1);
}
template <int R, int C, bool TR>
struct MatH {
  bf* p;
};
template <int R, int C, bool TR>
__device__ __forceinline__ MatH<R, C, !TR> tr(const MatH<R, C, TR> m) { return MatH<R, C, !TR>{m.p}; }

// float32 master of a state matrix in tensor memory, used as a scratchpad that no tensor-core instruction touches:
// rank16_update gives the 16 x 8 output tiles of a 64 x 256 (or 256 x 64) matrix to the 16 warps, eight tiles each,
// always the same ones, so a thread only ever reads and writes its own 32 floats of a matrix -- and a warp can only
// address its own quarter of the 128 tensor-memory lanes anyway.  Thread (warp w, lane l) owns lane 32 (w % 4) + l; the four
// warps that share a lane quarter take 128 of the 512 columns each (w / 4), 32 columns per matrix (W1, W2, dW1, dW2):
// 4 matrices x 64 KB = the SM's whole 256 KB.  Column 4 u + 2 h + e of a matrix holds element (g + 8 h, 2 t + e) of the
// warp's u-th tile (g = l / 4, t = l % 4): the order of the accumulator registers.  A read-modify-write of a matrix is
// one tcgen05.ld and one tcgen05.st of 32 columns per thread instead of a round trip to L2.
template <int R, int C>
struct MatM {
  uint32_t taddr;  // lane quarter and first column of this warp's 32 columns of the matrix
};

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]),
        "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]), "=f"(r[16]),
        "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]), "=f"(r[24]),
        "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31};\n\t"
      "tcgen05.wait::st.sync.aligned;"
      ::"f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]), "f"(r[8]), "f"(r[9]),
        "f"(r[10]), "f"(r[11]), "f"(r[12]), "f"(r[13]), "f"(r[14]), "f"(r[15]), "f"(r[16]), "f"(r[17]), "f"(r[18]),
        "f"(r[19]), "f"(r[20]), "f"(r[21]), "f"(r[22]), "f"(r[23]), "f"(r[24]), "f"(r[25]), "f"(r[26]), "f"(r[27]),
        "f"(r[28]), "f"(r[29]), "f"(r[30]), "f"(r[31]), "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_t(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}

// ---- fragment loads: A fragment of rows i0..i0+15, contraction indices k0..k0+15 -------------------------------
template <int LD, bool TR>
__device__ __forceinline__ void load_A(const SB<LD, TR> A, int i0, int k0, int lane, uint32_t (&r)[4]) {
  if constexpr (!TR) {  // stored [i][k]
    ldsm_x4(r, A.a + ((i0 + (lane & 15)) * LD + k0 + 8 * (lane >> 4)) * 2);
  } else {  // stored [k][i]: the four 8x8 blocks are read transposed
    ldsm_x4_t(r, A.a + ((k0 + (lane & 7) + 8 * (lane >> 4)) * LD + i0 + 8 * ((lane >> 3) & 1)) * 2);
  }
}
template <int RS, int CS_>
__device__ __forceinline__ void load_A(const MatT<RS, CS_> A, int i0, int k0, int lane, uint32_t (&r)[4]) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float* s = A.p + (i0 + g + 8 * (q & 1)) * RS + (k0 + 2 * t + 8 * (q >> 1)) * CS_;
    if constexpr (CS_ == 1) {
      const float2 f = *reinterpret_cast<const float2*>(s);
      r[q] = pack_bf16(f.x, f.y);
    } else {
      r[q] = pack_bf16(s[0], s[CS_]);
    }
  }
}
// B fragment of contraction indices k0..k0+15, columns j0..j0+7
template <int LD, bool TR>
__device__ __forceinline__ void load_B(const SB<LD, TR> B, int k0, int j0, int lane, uint32_t (&r)[2]) {
  if constexpr (!TR) {  // stored [k][n]
    ldsm_x2_t(r, B.a + ((k0 + (lane & 15)) * LD + j0) * 2);
  } else {  // stored [n][k]
    ldsm_x2(r, B.a + ((j0 + (lane & 7)) * LD + k0 + 8 * ((lane >> 3) & 1)) * 2);
  }
}
template <int RS, int CS_>
__device__ __forceinline__ void load_B(const MatT<RS, CS_> B, int k0, int j0, int lane, uint32_t (&r)[2]) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const float* s = B.p + (k0 + 2 * t + 8 * q) * RS + (j0 + g) * CS_;
    if constexpr (RS == 1) {
      const float2 f = *reinterpret_cast<const float2*>(s);
      r[q] = pack_bf16(f.x, f.y);
    } else {
      r[q] = pack_bf16(s[0], s[RS]);
    }
  }
}
template <int R, int C, bool TR>
__device__ __forceinline__ void load_A(const MatG<R, C, TR> A, int i0, int k0, int lane, uint32_t (&r)[4]) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int i = i0 + g + 8 * (q & 1), k = k0 + 2 * t + 8 * (q >> 1);
    if constexpr (!TR) {  // stored [i][k]: the pair (k, k + 1) is adjacent
      const float2 f = __ldcg(reinterpret_cast<const float2*>(A.p + A.at(i, k)));
      r[q] = pack_bf16(f.x, f.y);
    } else {
      r[q] = pack_bf16(__ldcg(A.p + A.at(k, i)), __ldcg(A.p + A.at(k + 1, i)));
    }
  }
}
template <int R, int C, bool TR>
__device__ __forceinline__ void load_B(const MatG<R, C, TR> B, int k0, int j0, int lane, uint32_t (&r)[2]) {
  const int g = lane >> 2, t = lane & 3;
  // k0 is a multiple of 16 and j0 of 8, so the tile index and the place inside the tile separate
  if constexpr (TR) {  // stored [j][k]: the pair (k, k + 1) is adjacent; the two registers lie in neighbouring tiles
    const float* s = B.p + ((((j0 >> 4) * (C / 8) + (k0 >> 3)) << 7) + (((j0 >> 3) & 1) << 6) + (g << 3) + 2 * t);
    const float2 f0 = __ldcg(reinterpret_cast<const float2*>(s)), f1 = __ldcg(reinterpret_cast<const float2*>(s + 128));
    r[0] = pack_bf16(f0.x, f0.y);
    r[1] = pack_bf16(f1.x, f1.y);
  } else {  // stored [k][j]: rows 2t, 2t + 1 of the upper and of the lower half of one tile
    const float* s = B.p + ((((k0 >> 4) * (C / 8) + (j0 >> 3)) << 7) + (t << 4) + g);
    r[0] = pack_bf16(__ldcg(s), __ldcg(s + 8));
    r[1] = pack_bf16(__ldcg(s + 64), __ldcg(s + 72));
  }
}
template <int R, int C, bool TR>
__device__ __forceinline__ void load_B(const MatH<R, C, TR> B, int k0, int j0, int lane, uint32_t (&r)[2]) {
  const int g = lane >> 2, t = lane & 3;
  if constexpr (TR) {  // stored [j][k]: the pair (k, k + 1) is adjacent
#pragma unroll
    for (int q = 0; q < 2; ++q)
      r[q] = __ldcg(reinterpret_cast<const uint32_t*>(B.p + mlp_shadow_at(j0 + g, k0 + 2 * t + 8 * q, C)));
  } else {  // stored [k][j]: rows k, k + 1 of the 2 x 2 block that holds column j
    const uint32_t sel = (g & 1) ? 0x7632u : 0x5410u;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const uint2 w = __ldcg(reinterpret_cast<const uint2*>(B.p + mlp_shadow_at(k0 + 2 * t + 8 * q, (j0 + g) & ~1, C)));
      r[q] = __byte_perm(w.x, w.y, sel);
    }
  }
}
template <int R, int C>
__device__ __forceinline__ float2 c_load(const MatG<R, C, false> M, int i, int j) {
  return __ldcg(reinterpret_cast<const float2*>(M.p + M.at(i, j)));
}
template <int R, int C>
__device__ __forceinline__ void c_store(const MatG<R, C, false> M, int i, int j, float x, float y) {
  *reinterpret_cast<float2*>(M.p + M.at(i, j)) = make_float2(x, y);
}
// the output pair (i, j), (i, j + 1)
template <int RS>
__device__ __forceinline__ float2 c_load(const MatT<RS, 1> C, int i, int j) {
  return *reinterpret_cast<const float2*>(C.p + i * RS + j);
}
template <int RS>
__device__ __forceinline__ void c_store(const MatT<RS, 1> C, int i, int j, float x, float y) {
  *reinterpret_cast<float2*>(C.p + i * RS + j) = make_float2(x, y);
}
template <int LD>
__device__ __forceinline__ float2 c_load(const SB<LD, false> C, int i, int j) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(C.a + (i * LD + j) * 2));
  return make_float2(bf16_lo(v), bf16_hi(v));
}
template <int LD>
__device__ __forceinline__ void c_store(const SB<LD, false> C, int i, int j, float x, float y) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(C.a + (i * LD + j) * 2), "r"(pack_bf16(x, y)) : "memory");
}

struct NoEpi {};
template <int K_, class MA_, class MB_>
struct Prod {
  MA_ A;
  MB_ B;
  static constexpr int K = K_;
};
template <int K, class MA, class MB>
__device__ __forceinline__ Prod<K, MA, MB> prod(const MA a, const MB b) { return Prod<K, MA, MB>{a, b}; }

template <class X>
struct is_global_operand : std::false_type {};
template <int R, int C, bool TR>
struct is_global_operand<MatG<R, C, TR>> : std::true_type {};
template <int R, int C, bool TR>
struct is_global_operand<MatH<R, C, TR>> : std::true_type {};

// C[M x N] = (ACC ? C : 0) + alpha * sum over the given products of A[M x K] . B[K x N];  M % 16 == 0, N % 8 == 0,
// K % 16 == 0; every extent and stride is a compile-time constant.  With an epilogue functor the finished pair
// (i, j), (i, j + 1) goes to epi(i, j, x, y) instead of being stored to C.
// Output tiles of 16 x 8 are dealt to the warps round-robin (for one WOFF the same tile always goes to the same warp,
// so successive accumulations into one matrix with the same WOFF need no barrier between them).  A warp works on up to TGMAX of its tiles
// at a time: tile0 + u * NW, u < TG, so that their loads (for an accumulation into the float32 state in the
// workspace: a round trip to L2) are in flight together.  When a row of output tiles goes round the warps GA times,
// GA consecutive tiles of a warp share their rows (one A fragment serves them); when NW is a multiple of the tiles
// per row all tiles of a warp share their columns (one B fragment).
template <bool ACC, int M, int N, int TGMAX = 4, int WOFF = 0, class MC, class EPI, class... PR>
__device__ __forceinline__ void tile_mma(const MC C, const float alpha, EPI epi, const PR... pr) {
  constexpr int NW = MB_NW, ntn = N / 8, total = (M / 16) * ntn, per_warp = (total + NW - 1) / NW;
  constexpr int GA = (ntn % NW == 0) ? ntn / NW : 1;
  constexpr bool SHARE_B = (NW % ntn == 0) && per_warp > 1;
  constexpr int TG1 = per_warp < TGMAX ? per_warp : TGMAX;
  constexpr int TG = TG1 < GA ? GA : TG1 / GA * GA;
  constexpr int NA = TG / GA, NB = SHARE_B ? 1 : TG;
  static_assert(TG % GA == 0 && GA <= 4, "tile grouping");
  // WOFF: the tiles go round the warps starting at warp WOFF -- a product of 8 tiles that shares its phase with
  // another one is given to the upper eight warps, so that no warp walks both contractions one after the other
  const int warp = ((threadIdx.x >> 5) + (NW - WOFF)) & (NW - 1), lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll 1
  for (int tile0 = warp; tile0 < total; tile0 += NW * TG) {
    int i0[TG], j0[TG];
    bool on[TG];
    float acc[TG][4];
    float2 cin[TG][2];
#pragma unroll
    for (int u = 0; u < TG; ++u) {
      const int tile = tile0 + u * NW;
      on[u] = tile < total;
      const int tl = on[u] ? tile : tile0, mt = tl / ntn;
      i0[u] = 16 * mt;
      j0[u] = 8 * (tl - mt * ntn);
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[u][q] = 0.f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        cin[u][h] = make_float2(0.f, 0.f);
        if constexpr (ACC)
          if (on[u]) cin[u][h] = c_load(C, i0[u] + g + 8 * h, j0[u] + 2 * t);
      }
    }
    auto run = [&](const auto P) {
      typedef typename std::remove_cv<typename std::remove_reference<decltype(P)>::type>::type PT;
      constexpr int K = PT::K;
      // operands in the workspace: the whole contraction unrolled, so that the loads of all steps are in flight
      constexpr bool GLOBAL = is_global_operand<decltype(PT::A)>::value || is_global_operand<decltype(PT::B)>::value;
#pragma unroll(GLOBAL ? 16 : (K >= 64 ? 2 : 1))
      for (int k0 = 0; k0 < K; k0 += 16) {
        uint32_t pa[NA][4], pb[NB][2];
#pragma unroll
        for (int u = 0; u < TG; ++u) {
          if (u % GA == 0) load_A(P.A, i0[u], k0, lane, pa[u / GA]);
          if (u == 0 || !SHARE_B) load_B(P.B, k0, j0[u], lane, pb[SHARE_B ? 0 : u]);
        }
#pragma unroll
        for (int u = 0; u < TG; ++u) {
          const uint32_t(&a)[4] = pa[u / GA];
          const uint32_t(&b_)[2] = pb[SHARE_B ? 0 : u];
          mma_bf16(acc[u], a[0], a[1], a[2], a[3], b_[0], b_[1]);
        }
      }
    };
    (run(pr), ...);
#pragma unroll
    for (int u = 0; u < TG; ++u)
      if (on[u]) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int i = i0[u] + g + 8 * h, j = j0[u] + 2 * t;
          const float x = cin[u][h].x + alpha * acc[u][2 * h], y = cin[u][h].y + alpha * acc[u][2 * h + 1];
          if constexpr (std::is_same<EPI, NoEpi>::value) c_store(C, i, j, x, y);
          else epi(i, j, x, y);
        }
      }
  }
}

// M[R][C] (float32 master in tensor memory) += alpha * sum over p of A_p^T B_p for token tiles A_p [16][R] and
// B_p [16][C] (bf16, shared memory, rows of LDA / LDB elements): the rank-16 updates of the state and of its gradient.
// The warp's eight output tiles are the ones tile_mma would deal it (tile w + 16 u: for the 64 x 256 matrices row tile
// u / 2 and column tile w + 16 (u % 2), for the 256 x 64 ones row tile 2 u + w / 8 and column tile w % 8), so that the
// operand copies written by the epilogue line up with what the other products read; every shared-memory address is a
// per-thread base plus a compile-time offset.  epi(u, h, x, y) receives the finished pair (row g + 8 h of tile u,
// columns 2 t, 2 t + 1) for the copies it keeps (u and h are compile-time constants after unrolling).
template <int R, int C, int LDA, int LDB, int NP, class EPI>
__device__ __forceinline__ void rank16_update(const MatM<R, C> M, const float alpha, EPI epi,
                                              const uint32_t (&a_tiles)[NP], const uint32_t (&b_tiles)[NP]) {
  static_assert((R == HD && C == MB_E) || (R == MB_E && C == HD), "the two shapes of the state matrices");
  constexpr bool WIDE = C == MB_E;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A^T fragment of rows i0 .. i0 + 15: the four 8 x 8 blocks of the stored [token][row] tile, read transposed
  const uint32_t a_off = ((((lane & 7) + 8 * (lane >> 4)) * LDA + 8 * ((lane >> 3) & 1) + (WIDE ? 0 : 16 * (warp >> 3))) * 2);
  const uint32_t b_off = (((lane & 15) * LDB + (WIDE ? 8 * warp : 8 * (warp & 7))) * 2);
  float acc[8][4];
#pragma unroll
  for (int u = 0; u < 8; ++u)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[u][q] = 0.f;
#pragma unroll
  for (int pi = 0; pi < NP; ++pi) {
    if constexpr (WIDE) {
      uint32_t fa[4][4], fb[2][2];
#pragma unroll
      for (int m = 0; m < 4; ++m) ldsm_x4_t(fa[m], a_tiles[pi] + a_off + 16 * m * 2);
#pragma unroll
      for (int n = 0; n < 2; ++n) ldsm_x2_t(fb[n], b_tiles[pi] + b_off + 128 * n * 2);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        mma_bf16(acc[u], fa[u >> 1][0], fa[u >> 1][1], fa[u >> 1][2], fa[u >> 1][3], fb[u & 1][0], fb[u & 1][1]);
    } else {
      uint32_t fa[8][4], fb[2];
#pragma unroll
      for (int u = 0; u < 8; ++u) ldsm_x4_t(fa[u], a_tiles[pi] + a_off + 32 * u * 2);
      ldsm_x2_t(fb, b_tiles[pi] + b_off);
#pragma unroll
      for (int u = 0; u < 8; ++u) mma_bf16(acc[u], fa[u][0], fa[u][1], fa[u][2], fa[u][3], fb[0], fb[1]);
    }
  }
  float tm[32];
  tmem_ld32(M.taddr, tm);
#pragma unroll
  for (int u = 0; u < 8; ++u)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float x = tm[4 * u + 2 * h] + alpha * acc[u][2 * h], y = tm[4 * u + 2 * h + 1] + alpha * acc[u][2 * h + 1];
      tm[4 * u + 2 * h] = x;
      tm[4 * u + 2 * h + 1] = y;
      epi(u, h, x, y);
    }
  tmem_st32(M.taddr, tm);
}

// ---- element-wise helpers --------------------------------------------------------------------------------------
// tanh(x) = 1 - 2 / (1 + e^{2x}) with the fast exponential and division (relative error ~1e-6, as in the forward kernel)
__device__ __forceinline__ float tanh_fast(float x) { return 1.f - __fdividef(2.f, 1.f + __expf(2.f * x)); }
// gelu(x), gelu'(x) and (D2) gelu''(x) from one tanh
template <bool D2>
__device__ __forceinline__ void gelu_all(float x, float& f, float& d1, float& d2) {
  const float x2 = x * x, th = tanh_fast(GELU_C0 * x * (1.f + GELU_C1 * x2));
  const float hs = 0.5f * x * (1.f - th * th), du = GELU_C0 * (1.f + 3.f * GELU_C1 * x2);
  f = 0.5f * x * (1.f + th);
  d1 = hs * du + 0.5f * (1.f + th);
  if constexpr (D2) d2 = (1.f - th * th) * du + hs * (6.f * GELU_C0 * GELU_C1 * x - 2.f * th * du * du);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// a pair of adjacent bf16 elements of a tile (even column)
__device__ __forceinline__ float2 ldb2(const bf* p) {
  const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
  return make_float2(bf16_lo(v), bf16_hi(v));
}
__device__ __forceinline__ void stb2(bf* p, float x, float y) { *reinterpret_cast<uint32_t*>(p) = pack_bf16(x, y); }
__device__ __forceinline__ float ldb(const bf* p) { return __bfloat162float(*p); }

// visit the column pairs of a [16][E] tile / of a [16][F] tile (one pair per thread) / the elements of a [16][16] tile
template <class Fn>
__device__ __forceinline__ void for_e2(Fn f) {
#pragma unroll
  for (int it = 0; it < CS * MB_E / 2 / MB_THREADS; ++it) {
    const int e = threadIdx.x + it * MB_THREADS;
    f(e / (MB_E / 2), 2 * (e % (MB_E / 2)));
  }
}
template <class Fn>
__device__ __forceinline__ void for_f2(Fn f) {
  static_assert(CS * HD / 2 == MB_THREADS, "one pair per thread");
  f((int)threadIdx.x / (HD / 2), 2 * ((int)threadIdx.x % (HD / 2)));
}
template <class Fn>
__device__ __forceinline__ void for_c(Fn f) {
  if (threadIdx.x < CS * CS) f((int)threadIdx.x / CS, (int)threadIdx.x % CS);
}

struct __align__(16) MlpBwdSmem {
  // bf16 operand tiles
  bf gd1[CS][EB], gd2[CS][EB], x2[CS][EB], g1[CS][EB];  // gelu'(z1), gelu''(z1), gelu(z1), g1
  bf z1b[CS][EB], x2b[CS][EB];  // gelu'(z1b) (then scratch: l o x2, column partials), gelu(z1b)
  bf t1[CS][EB], t2[CS][EB], t3[CS][EB], t4[CS][EB];  // g1p | dz1b;  dg1, dh;  gl2;  dz1 (and column partials)
  bf q[CS][FB], k[CS][FB], v[CS][FB], dO[CS][FB], g2[CS][FB], g2p[CS][FB], dz2b[CS][FB], dz2[CS][FB];
  bf m1[CS][CB], m2[CS][CB], m1n[CS][CB], m2n[CS][CB], da1[CS][CB], da2[CS][CB];  // m*n = -m*
  bf w1[HD][EB], w2[MB_E][FB];  // bf16 shadows of the float32 state in the workspace
  // float32 tiles
  float z2[CS][FP], z2b[CS][FP], dg2[CS][FP], dk[CS][FP], gl1[CS][FP];
  float eta[CS][CP], a1[CS][CP], a2[CS][CP], dm[CS][CP], deta[CS][CP];
  float lr[CS], te[CS], ell[CS], dell[CS];
  float b1[MB_E], db1[MB_E], b2[HD], db2[HD];  // biases and their gradients stay on chip for the whole walk
  float dgam[HD], dbet[HD], gam[HD], bet[HD];  // this stream's LayerNorm parameter gradients; the parameters
};
static_assert(sizeof(MlpBwdSmem) + 1024 <= 227 * 1024, "shared-memory tiles exceed one SM");
static_assert(sizeof(bf) * CS * EB >= sizeof(float) * MB_NW * 2 * HD, "column partials alias a [16][E] tile");

// G = d/dz of 0.5 |LN(z) - (v - k)|^2 for a [16][64] tile (rust/core/src/util.rs:155-182); one row per warp, the
// lane owns columns 2 lane, 2 lane + 1
template <bool SAVE>
__device__ __forceinline__ void ln_l2_grad_tile(MlpBwdSmem& S, const float (*z)[FP], bf (*G)[FB], float eps,
                                                uint32_t* g2p_global) {
  const int r = threadIdx.x >> 5, c = 2 * (threadIdx.x & 31);
  const float2 zz = *reinterpret_cast<const float2*>(&z[r][c]);
  const float mu = warp_sum(zz.x + zz.y) * (1.f / HD);
  const float var = warp_sum((zz.x - mu) * (zz.x - mu) + (zz.y - mu) * (zz.y - mu)) * (1.f / HD);
  const float rs = 1.f / sqrtf(var + eps);
  const float2 vv = ldb2(&S.v[r][c]), kk = ldb2(&S.k[r][c]);
  const float x0 = (zz.x - mu) * rs, x1 = (zz.y - mu) * rs;
  const float gx0 = (S.gam[c] * x0 + S.bet[c] - (vv.x - kk.x)) * S.gam[c];
  const float gx1 = (S.gam[c + 1] * x1 + S.bet[c + 1] - (vv.y - kk.y)) * S.gam[c + 1];
  const float s1 = warp_sum(gx0 + gx1) * (1.f / HD);
  const float s2 = warp_sum(gx0 * x0 + gx1 * x1) * (1.f / HD);
  const float G0 = (gx0 - s1 - x0 * s2) * rs, G1 = (gx1 - s1 - x1 * s2) * rs;
  stb2(&G[r][c], G0, G1);
  if constexpr (SAVE) {  // lr o G, rounded once from the float32 value
    const uint32_t v = pack_bf16(S.lr[r] * G0, S.lr[r] * G1);
    g2p_global[(r * HD + c) >> 1] = v;
    *reinterpret_cast<uint32_t*>(&S.g2p[r][c]) = v;
  }
}

// column sums of a [16][N] bf16 tile (rows of ld elements) added, with sign, to dst[N]
__device__ __forceinline__ void add_colsum(float* dst, const bf* tile, int N, int ld, float sign) {
  for (int c = threadIdx.x; c < N; c += MB_THREADS) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < CS; ++r) s += ldb(tile + r * ld + c);
    dst[c] += sign * s;
  }
}

__global__ void __launch_bounds__(MB_THREADS, 1) ttt_mlp_bwd_kernel(const MlpBwdParams p) {
  extern __shared__ __align__(16) uint8_t mlp_bwd_smem[];
  MlpBwdSmem& S = *reinterpret_cast<MlpBwdSmem*>(mlp_bwd_smem);
  typedef __nv_bfloat16 T;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NS = p.NS;
  constexpr int F = HD, E = MB_E;
  constexpr int HO_B1 = MLP_HO_B1, HO_B2 = MLP_HO_B2, HO_DB1 = MLP_HO_DB1, HO_DB2 = MLP_HO_DB2, HO_DG = MLP_HO_DG,
                HO_DB = MLP_HO_DB;
  static_assert(HO_B2 == E && HO_DB1 == E + F && HO_DB2 == 2 * E + F && HO_DG == 2 * E + 2 * F &&
                    HO_DB == 2 * E + 3 * F && HO_DB + F == MLP_BWD_HANDOFF_FLOATS, "hand-off record");
  float* const b1 = S.b1;
  float* const b2 = S.b2;
  float* const db1 = S.db1;
  float* const db2 = S.db2;
  __shared__ int s_item;
  __shared__ uint32_t s_tmem;
  // Tensor memory, all 512 columns (shared memory keeps the block alone on its SM): the float32 masters of the state
  // and of its gradient while a work item runs (see MatM).  The warp that allocates frees it at the end of the kernel;
  // every way out of the item loop below leads there.
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&s_tmem)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_mine = s_tmem + ((32u * (uint32_t)(warp & 3)) << 16) + 128u * (uint32_t)(warp >> 2);
  // workspace <-> tensor memory, this thread's 32 floats of one matrix (MatG stores a 16 x 8 tile as 128 consecutive
  // floats in the order of the accumulator registers: tile index = the index rank16_update deals by)
  auto master_in = [&](const float* M, const uint32_t taddr) {
    float v[32];
    const float* src = M + warp * 128 + 8 * (lane >> 2) + 2 * (lane & 3);
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float2 f = __ldcg(reinterpret_cast<const float2*>(src + u * (MB_NW * 128) + 64 * h));
        v[4 * u + 2 * h] = f.x;
        v[4 * u + 2 * h + 1] = f.y;
      }
    tmem_st32(taddr, v);
  };
  auto master_out = [&](float* M, const uint32_t taddr) {
    float v[32];
    tmem_ld32(taddr, v);
    float* dst = M + warp * 128 + 8 * (lane >> 2) + 2 * (lane & 3);
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        *reinterpret_cast<float2*>(dst + u * (MB_NW * 128) + 64 * h) = make_float2(v[4 * u + 2 * h], v[4 * u + 2 * h + 1]);
  };

  // Persistent block.  A stream is a chain of 2 NCH work items: its chunks of CH stages in pass 1 (ranks 0 ..
  // NCH-1, forward), then in pass 2 (ranks NCH .. 2 NCH-1, backward).  Items are handed out rank by rank over all
  // streams, so an item only waits for an item with a smaller index (its predecessor in the chain), which is done or
  // held by a resident block: the launch cannot deadlock while all blocks are co-resident (cooperative launch).
  // Between items the stream's state lives in the workspace: the four float32 matrices anyway, the biases, their
  // gradients and the LayerNorm parameter gradients in a small hand-off record.
  // When the forward has already filled the workspace (pass1_done) the chains start at rank NCH.
  const int rank0 = p.pass1_done ? p.NCH : 0;
  const int nitems = p.nstreams * (2 * p.NCH - rank0);
#ifdef TTT_MLP_TRACE
  unsigned long long tr_acc[16] = {0}, tr_last = 0;
#endif
  while (true) {
    if (tid == 0) s_item = atomicAdd(&p.sched[0], 1);
    __syncthreads();
    const int item = s_item;
    __syncthreads();
    if (item >= nitems) break;
    const int rel = item / p.nstreams, rank = rank0 + rel, stream = item - rel * p.nstreams, head = stream % p.H;
    const bool pass1 = rank < p.NCH;
    const int chunk = pass1 ? rank : 2 * p.NCH - 1 - rank;
    const int s_lo = chunk * p.CH, s_hi = min(s_lo + p.CH, NS);
    const size_t row_base = (size_t)stream * p.T;

  // per-stream workspace: W1 [F][E], W2 [E][F], dW1, dW2 (float32, in the tile order of MatG), the hand-off record,
  // then g1p [NS][16][E], g2p [NS][16][F] (bf16), then b1 | b2 at the start of every stage [NS][E + F] (float32),
  // then the bf16 operand copies of dW1 and dW2
  float* ws = p.workspace + (size_t)stream * p.ws_stride;
  float* W1 = ws;
  float* W2 = W1 + F * E;
  float* dW1 = W2 + E * F;
  float* dW2 = dW1 + F * E;
  float* ho = dW2 + E * F;
  bf* g1p_all = reinterpret_cast<bf*>(ho + MLP_BWD_HANDOFF_FLOATS);
  bf* g2p_all = g1p_all + (size_t)NS * CS * E;
  float* bst = reinterpret_cast<float*>(g2p_all + (size_t)NS * CS * F);  // [NS][E + F]: b1, b2 at the start of a stage
  bf* dW1h = reinterpret_cast<bf*>(bst + (size_t)NS * (E + F));            // bf16 operand copies of dW1, dW2 (MatH)
  bf* dW2h = dW1h + F * E;

  if (rel > 0) {
    // wait (bounded) until the previous item of this stream has published its state
    int ok = 1;
    if (tid == 0) {
      ok = 0;
      const volatile int* flag = p.sched + 1 + stream;
      for (uint32_t it = 0; it < (1u << 24); ++it) {
        if (*flag >= rel) {
          ok = 1;
          break;
        }
        __nanosleep(100);
      }
      __threadfence();
    }
    if (__syncthreads_or(ok ? 0 : 1)) {
      if (tid == 0 && p.status != nullptr && atomicCAS(p.status, 0u, (uint32_t)KST_TIMEOUT) == 0u) {
        p.status[1] = 1u;
        p.status[2] = blockIdx.x;
        p.status[3] = (uint32_t)item;
      }
      break;
    }
  }
  if (tid < HD) {
    S.gam[tid] = ld_as_float<T>(p.ln_g, (size_t)head * HD + tid);
    S.bet[tid] = ld_as_float<T>(p.ln_b, (size_t)head * HD + tid);
    const bool fresh = rank <= p.NCH;  // the LayerNorm parameter gradients start with pass 2
    S.dgam[tid] = fresh ? 0.f : __ldcg(ho + HO_DG + tid);
    S.dbet[tid] = fresh ? 0.f : __ldcg(ho + HO_DB + tid);
  }
  if (tid < CS) S.te[tid] = ld_as_float<T>(p.token_eta, (size_t)tid);
  if (rank == 0) {
    for (int e = tid; e < F * E; e += MB_THREADS) {
      const bf a = static_cast<const bf*>(p.w1)[(size_t)stream * F * E + e];
      const bf b = static_cast<const bf*>(p.w2)[(size_t)stream * F * E + e];
      W1[MatG<F, E, false>::at(e / E, e % E)] = __bfloat162float(a);
      W2[MatG<E, F, false>::at(e / F, e % F)] = __bfloat162float(b);
      S.w1[e / E][e % E] = a;
      S.w2[e / F][e % F] = b;
    }
    for (int e = tid; e < E; e += MB_THREADS) b1[e] = ld_as_float<T>(p.b1, (size_t)stream * E + e);
    if (tid < F) b2[tid] = ld_as_float<T>(p.b2, (size_t)stream * F + tid);
  } else {
    // bf16 shadows from the float32 state the previous item left in the workspace
    for (int e = 2 * tid; e < F * E; e += 2 * MB_THREADS) {
      const float2 a = __ldcg(reinterpret_cast<const float2*>(W1 + MatG<F, E, false>::at(e / E, e % E)));
      const float2 b = __ldcg(reinterpret_cast<const float2*>(W2 + MatG<E, F, false>::at(e / F, e % F)));
      stb2(&S.w1[e / E][e % E], a.x, a.y);
      stb2(&S.w2[e / F][e % F], b.x, b.y);
    }
    for (int e = tid; e < E; e += MB_THREADS) b1[e] = __ldcg(ho + HO_B1 + e);
    if (tid < F) b2[tid] = __ldcg(ho + HO_B2 + tid);
  }
  if (!pass1) {
    const bool fresh = rank == p.NCH;  // first item of pass 2: the gradients w.r.t. the final state are zero
    if (fresh)
      for (int e = tid; e < F * E; e += MB_THREADS) {
        dW1[e] = 0.f;
        dW2[e] = 0.f;
        reinterpret_cast<uint32_t*>(dW1h)[e] = 0u;  // both bf16 copies: 2 F E elements = F E words
      }
    for (int e = tid; e < E; e += MB_THREADS) db1[e] = fresh ? 0.f : __ldcg(ho + HO_DB1 + e);
    if (tid < F) db2[tid] = fresh ? 0.f : __ldcg(ho + HO_DB2 + tid);
  }
  __syncthreads();
  // the masters of this item: W1, W2 (and in pass 2 dW1, dW2) from the workspace, where the previous item of the
  // stream (or the forward kernel, or the lines above) left them
  const uint32_t tW1a = tmem_mine, tW2a = tmem_mine + 32, tdW1a = tmem_mine + 64, tdW2a = tmem_mine + 96;
  master_in(W1, tW1a);
  master_in(W2, tW2a);
  if (!pass1) {
    master_in(dW1, tdW1a);
    master_in(dW2, tdW2a);
  }
  const float te_last = S.te[CS - 1];
// per-phase cycle counts of block 0 (instrumented builds only; written to the status words after the walk)
#ifdef TTT_MLP_TRACE
  tr_last = clock64();
#define TRM(i) { __syncthreads(); const unsigned long long n_ = clock64(); tr_acc[i] += n_ - tr_last; tr_last = n_; }
#else
#define TRM(i)
#endif

  // ---- operand / output views
  const MatM<F, E> mW1{tW1a}, mdW1{tdW1a};
  const MatM<E, F> mW2{tW2a}, mdW2{tdW2a};
  const MatH<F, E, false> hdW1{dW1h};
  const MatH<E, F, false> hdW2{dW2h};
  const MatT<1, 1> none{nullptr};
  typedef SB<EB, false> TE;
  typedef SB<FB, false> TF_;
  typedef SB<CB, false> TC;
  const TE sx2{smem_u32(S.x2)}, sg1{smem_u32(S.g1)}, sz1b{smem_u32(S.z1b)}, sx2b{smem_u32(S.x2b)};
  const TE st1{smem_u32(S.t1)}, st2{smem_u32(S.t2)}, st3{smem_u32(S.t3)}, st4{smem_u32(S.t4)}, sw1{smem_u32(S.w1)};
  const TF_ sq{smem_u32(S.q)}, sk{smem_u32(S.k)}, sg2{smem_u32(S.g2)}, sg2p{smem_u32(S.g2p)}, sdz2b{smem_u32(S.dz2b)};
  const TF_ sdz2{smem_u32(S.dz2)}, sw2{smem_u32(S.w2)};
  const TC sm1{smem_u32(S.m1)}, sm2{smem_u32(S.m2)}, sm1n{smem_u32(S.m1n)}, sm2n{smem_u32(S.m2n)};
  const TC sda1{smem_u32(S.da1)}, sda2{smem_u32(S.da2)};
  const MatT<FP, 1> mdq{&S.z2b[0][0]}, mdg2{&S.dg2[0][0]}, mdk{&S.dk[0][0]}, mgl1{&S.gl1[0][0]};
  float(*const dq)[FP] = S.z2b;  // z2b is dead once the output LayerNorm has been differentiated: its tile then holds dq
  const MatT<CP, 1> ma1{&S.a1[0][0]}, ma2{&S.a2[0][0]}, mdm{&S.dm[0][0]};
  const NoEpi noepi;

  // W += sign * A^T B with the float32 master in tensor memory and its bf16 shadow refreshed together
  // (t1 / g2p hold lr o g1 / lr o g2, the operands of the forward's update; its scale te[15] is applied here)
  // where this thread's pairs of a 64 x 256 / 256 x 64 matrix go (see rank16_update for the tiles of a warp): in the
  // bf16 shadows in shared memory and in the bf16 operand copies in the workspace (MatH), as element offsets of the
  // pair (tile u = 0, half h = 0); the other pairs follow at compile-time distances
  const int fg = lane >> 2, ft = lane & 3;
  const uint32_t w1_at = smem_u32(S.w1) + 2 * (fg * EB + 8 * warp + 2 * ft);
  const uint32_t w2_at = smem_u32(S.w2) + 2 * ((16 * (warp >> 3) + fg) * FB + 8 * (warp & 7) + 2 * ft);
  const int h_sub = ((((fg >> 1) & 3) * 4 + ft) * 4) + (fg & 1) * 2;
  bf* const dW1h_at = dW1h + warp * 64 + h_sub;
  bf* const dW2h_at = dW2h + (16 * (warp >> 3) + (warp & 7)) * 64 + h_sub;
  auto update_w1 = [&](const float sign) {  // W1 += sign * te[15] * K^T t1
    const uint32_t a[1] = {sk.a}, b[1] = {st1.a};
    rank16_update<F, E, FB, EB, 1>(mW1, sign * te_last, [&](int u, int h, float x, float y) {
      asm volatile("st.shared.b32 [%0], %1;" ::"r"(w1_at + 2 * ((16 * (u >> 1) + 8 * h) * EB + 128 * (u & 1))), "r"(pack_bf16(x, y)) : "memory");
    }, a, b);
  };
  auto update_w2 = [&](const float sign) {  // W2 += sign * te[15] * X2^T g2p
    const uint32_t a[1] = {sx2.a}, b[1] = {sg2p.a};
    rank16_update<E, F, EB, FB, 1>(mW2, sign * te_last, [&](int u, int h, float x, float y) {
      asm volatile("st.shared.b32 [%0], %1;" ::"r"(w2_at + 2 * ((32 * u + 8 * h) * FB)), "r"(pack_bf16(x, y)) : "memory");
    }, a, b);
  };
  // z1 = K W1 + b1, x2 = gelu(z1); z1 itself is only needed through gelu'(z1) and (pass 2) gelu''(z1)
  auto forward_first_layer = [&](auto d2_tag) {
    constexpr bool D2 = decltype(d2_tag)::value;
    tile_mma<false, CS, E>(none, 1.f, [&](int i, int j, float x, float y) {
      float f0, f1, a0, a1, c0 = 0.f, c1 = 0.f;
      gelu_all<D2>(x + b1[j], f0, a0, c0);
      gelu_all<D2>(y + b1[j + 1], f1, a1, c1);
      stb2(&S.x2[i][j], f0, f1);
      stb2(&S.gd1[i][j], a0, a1);
      if constexpr (D2) stb2(&S.gd2[i][j], c0, c1);
    }, prod<F>(sk, sw1));
    __syncthreads();
  };
  // z2 = x2 W2 + b2, g2 = ln_l2_grad(z2, v - k), g1 = (g2 W2^T) o gelu'(z1)
  // In pass 1 (save_tag true) l o g1 and l o g2 also go to t1 / g2p and to the workspace.
  auto forward_second_layer = [&](auto save_tag, uint32_t* g1p, uint32_t* g2p) {
    constexpr bool SAVE = decltype(save_tag)::value;
    tile_mma<false, CS, F>(none, 1.f, [&](int i, int j, float x, float y) {
      *reinterpret_cast<float2*>(&S.z2[i][j]) = make_float2(x + b2[j], y + b2[j + 1]);
    }, prod<E>(sx2, sw2));
    __syncthreads();
    ln_l2_grad_tile<SAVE>(S, S.z2, S.g2, p.eps, g2p);
    __syncthreads();
    tile_mma<false, CS, E>(none, 1.f, [&](int i, int j, float x, float y) {
      const float2 d1 = ldb2(&S.gd1[i][j]);
      x *= d1.x;
      y *= d1.y;
      stb2(&S.g1[i][j], x, y);
      if constexpr (SAVE) {
        const uint32_t v = pack_bf16(S.lr[i] * x, S.lr[i] * y);
        g1p[(i * E + j) >> 1] = v;
        *reinterpret_cast<uint32_t*>(&S.t1[i][j]) = v;
      }
    }, prod<F>(sg2, tr(sw2)));
    __syncthreads();
  };
  // one 16-byte piece per thread: [16][64] bf16 tiles from global memory (128 threads per tile)
  auto tile_piece = [&](int idx, int& r, int& c) {
    r = idx >> 3;
    c = 8 * (idx & 7);
  };

  // ============================== pass 1: forward walk, saving g1p and g2p ==============================
  if (pass1)
  for (int s = s_lo; s < s_hi; ++s) {
    const size_t r0 = (row_base + (size_t)s * CS) * HD;
    if (tid < 256) {
      int r, c;
      tile_piece(tid & 127, r, c);
      const T* src = static_cast<const T*>(tid < 128 ? p.xk : p.xv) + r0;
      bf(*dst)[FB] = tid < 128 ? S.k : S.v;
      *reinterpret_cast<uint4*>(&dst[r][c]) = *reinterpret_cast<const uint4*>(src + r * HD + c);
    } else if (tid < 256 + CS) {
      S.lr[tid - 256] = ld_as_float<T>(p.lr, row_base + (size_t)s * CS + (tid - 256));
    }
    for (int e = tid; e < E + F; e += MB_THREADS) bst[(size_t)s * (E + F) + e] = e < E ? b1[e] : b2[e - E];
    __syncthreads();
    TRM(0)
    forward_first_layer(std::false_type{});
    forward_second_layer(std::true_type{}, reinterpret_cast<uint32_t*>(g1p_all + (size_t)s * CS * E),
                         reinterpret_cast<uint32_t*>(g2p_all + (size_t)s * CS * F));
    TRM(1)
    update_w1(-1.f);
    update_w2(-1.f);
    add_colsum(b1, &S.t1[0][0], E, EB, -te_last);
    add_colsum(b2, &S.g2p[0][0], F, FB, -te_last);
    __syncthreads();
    TRM(2)
  }

  // ============================== pass 2: backward walk ==============================
  float(*const colpart)[2 * HD] = reinterpret_cast<float(*)[2 * HD]>(&S.z1b[0][0]);  // only while z1b is not live
  // The inputs of a stage (one 16-byte piece per thread and tile, the lr row, the biases at the start of the stage:
  // those were saved on the way forward, they are not recovered by undoing the update, since the forward takes its
  // column sums in float32 and the operand tiles are bf16) are fetched into registers while the previous stage
  // writes its outputs, and put in place when the stage begins.
  struct StageIn {
    uint4 g1v, in, g2v;
    float bias, lr;
  };
  auto fetch = [&](const int s) {
    StageIn v;
    const size_t r0 = (row_base + (size_t)s * CS) * HD;
    v.g1v = __ldcg(reinterpret_cast<const uint4*>(g1p_all + (size_t)s * CS * E) + tid);
    int r, c;
    tile_piece(tid & 127, r, c);
    const int which = tid >> 7;
    const T* src = static_cast<const T*>(which == 0 ? p.xq : which == 1 ? p.xk : which == 2 ? p.xv : p.d_out) + r0;
    v.in = *reinterpret_cast<const uint4*>(src + r * HD + c);
    v.g2v = make_uint4(0u, 0u, 0u, 0u);
    if (tid < 128) v.g2v = __ldcg(reinterpret_cast<const uint4*>(g2p_all + (size_t)s * CS * F) + tid);
    v.bias = tid < E + F ? __ldcg(bst + (size_t)s * (E + F) + tid) : 0.f;
    v.lr = tid < CS ? ld_as_float<T>(p.lr, row_base + (size_t)s * CS + tid) : 0.f;
    return v;
  };
  // the lines fetch(s) will read, asked into L2 a whole stage ahead (the q / k / v / d_out rows come from HBM, and
  // the fetch sits at the end of a stage with only the output stores between it and the commit that needs its data)
  auto prefetch_l2 = [&](const int s) {
    const size_t r0 = (row_base + (size_t)s * CS) * HD;
    int r, c;
    tile_piece(tid & 127, r, c);
    const int which = tid >> 7;
    const T* src = static_cast<const T*>(which == 0 ? p.xq : which == 1 ? p.xk : which == 2 ? p.xv : p.d_out) + r0;
    asm volatile("prefetch.global.L2 [%0];" ::"l"(src + r * HD + c));
    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint4*>(g1p_all + (size_t)s * CS * E) + tid));
    if (tid < 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint4*>(g2p_all + (size_t)s * CS * F) + tid));
    if (tid < E + F) asm volatile("prefetch.global.L2 [%0];" ::"l"(bst + (size_t)s * (E + F) + tid));
  };
  auto commit = [&](const StageIn& v) {
    int r, c;
    tile_piece(tid & 127, r, c);
    const int which = tid >> 7;
    bf(*dst)[FB] = which == 0 ? S.q : which == 1 ? S.k : which == 2 ? S.v : S.dO;
    *reinterpret_cast<uint4*>(&dst[r][c]) = v.in;
    *reinterpret_cast<uint4*>(&S.t1[tid >> 5][8 * (tid & 31)]) = v.g1v;
    if (tid < 128) *reinterpret_cast<uint4*>(&S.g2p[r][c]) = v.g2v;
    if (tid < E) b1[tid] = v.bias;
    else if (tid < E + F) b2[tid - E] = v.bias;
    if (tid < CS) {
      S.lr[tid] = v.lr;
      S.ell[tid] = te_last * v.lr;
    }
  };
  StageIn nxt;
  if (!pass1) nxt = fetch(s_hi - 1);
  if (!pass1)
  for (int s = s_hi - 1; s >= s_lo; --s) {
    const size_t r0 = (row_base + (size_t)s * CS) * HD;
    commit(nxt);
    if (s > s_lo) prefetch_l2(s - 1);
    __syncthreads();
    TRM(3)
    // ---- state at the start of this stage: undo the stage's updates (W1 first: X2 depends on it)
    update_w1(1.f);
    // (in the same phase, since neither depends on the state: the eta matrix and a1 = Q K^T)
    for_c([&](int i, int j) { S.eta[i][j] = (j <= i) ? S.te[i] * S.lr[j] : 0.f; });
    tile_mma<false, CS, CS>(ma1, 1.f, noepi, prod<F>(sq, tr(sk)));
    __syncthreads();
    for_c([&](int i, int j) {
      const float a = (j <= i) ? S.a1[i][j] : 0.f, m = S.eta[i][j] * (1.f + a);
      S.a1[i][j] = a;
      S.m1[i][j] = __float2bfloat16_rn(m);
      S.m1n[i][j] = __float2bfloat16_rn(-m);
    });
    forward_first_layer(std::true_type{});  // x2 (and the GELU derivatives) of this stage, needed to undo the second layer's update
    update_w2(1.f);
    __syncthreads();
    TRM(4)
    // ---- forward intermediates of the stage
    forward_second_layer(std::false_type{}, nullptr, nullptr);
    TRM(5)
    tile_mma<false, CS, E>(none, 1.f, [&](int i, int j, float x, float y) {          // z1b = Q W1 - M1 g1 + b1; x2b = gelu
      float f0, f1, a0, a1, c0, c1;
      gelu_all<false>(x + b1[j], f0, a0, c0);
      gelu_all<false>(y + b1[j + 1], f1, a1, c1);
      stb2(&S.z1b[i][j], a0, a1);  // gelu'(z1b), all that step 3 needs of z1b
      stb2(&S.x2b[i][j], f0, f1);
    }, prod<F>(sq, sw1), prod<CS>(sm1n, sg1));
    __syncthreads();
    tile_mma<false, CS, CS>(ma2, 1.f, noepi, prod<E>(sx2b, tr(sx2)));              // a2 = x2b x2^T
    tile_mma<false, CS, F, 4, 8>(mdq, 1.f, noepi, prod<E>(sx2b, sw2));             // z2b = x2b W2 ... (float32 tile)
    __syncthreads();
    for_c([&](int i, int j) {
      const float a = (j <= i) ? S.a2[i][j] : 0.f, m = S.eta[i][j] * (1.f + a);
      S.a2[i][j] = a;
      S.m2[i][j] = __float2bfloat16_rn(m);
      S.m2n[i][j] = __float2bfloat16_rn(-m);
    });
    __syncthreads();
    tile_mma<true, CS, F>(mdq, 1.f, [&](int i, int j, float x, float y) {           // ... - M2 g2 + b2
      *reinterpret_cast<float2*>(&S.z2b[i][j]) = make_float2(x + b2[j], y + b2[j + 1]);
    }, prod<CS>(sm2n, sg2));
    __syncthreads();

    TRM(6)
    // ---- 1. output LayerNorm: dz2b, LN parameter gradients (one row per warp, columns 2 lane, 2 lane + 1)
    {
      const int r = warp, c = 2 * lane;
      const float2 zz = *reinterpret_cast<const float2*>(&S.z2b[r][c]);
      const float mu = warp_sum(zz.x + zz.y) * (1.f / HD);
      const float var = warp_sum((zz.x - mu) * (zz.x - mu) + (zz.y - mu) * (zz.y - mu)) * (1.f / HD);
      const float rs = 1.f / sqrtf(var + p.eps);
      const float x0 = (zz.x - mu) * rs, x1 = (zz.y - mu) * rs;
      const float2 d = ldb2(&S.dO[r][c]);
      const float t0 = d.x * S.gam[c], t1_ = d.y * S.gam[c + 1];
      const float s1 = warp_sum(t0 + t1_) * (1.f / HD);
      const float s2 = warp_sum(t0 * x0 + t1_ * x1) * (1.f / HD);
      stb2(&S.dz2b[r][c], (t0 - s1 - x0 * s2) * rs, (t1_ - s1 - x1 * s2) * rs);
      // z1b's tile is still live: the partials of this step go through t4, which is free until step 5
      float(*cp)[2 * HD] = reinterpret_cast<float(*)[2 * HD]>(&S.t4[0][0]);
      *reinterpret_cast<float2*>(&cp[warp][c]) = make_float2(d.x * x0, d.y * x1);
      *reinterpret_cast<float2*>(&cp[warp][HD + c]) = make_float2(d.x, d.y);
    }
    __syncthreads();
    if (tid < 2 * HD) {
      const float(*cp)[2 * HD] = reinterpret_cast<const float(*)[2 * HD]>(&S.t4[0][0]);
      float s_ = 0.f;
#pragma unroll
      for (int w = 0; w < MB_NW; ++w) s_ += cp[w][tid];
      if (tid < HD) S.dgam[tid] += s_; else S.dbet[tid - HD] += s_;
    }
    TRM(7)
    // ---- 2. z2b = x2b W2 + b2 - M2 g2
    tile_mma<false, CS, CS>(mdm, -1.f, noepi, prod<F>(sdz2b, tr(sg2)));            // dM2 = -tril(dz2b g2^T)
    tile_mma<false, CS, F, 4, 8>(mdg2, 1.f, noepi, prod<CS>(tr(sm2n), sdz2b));     // dg2 = -M2^T dz2b
    __syncthreads();
    for_c([&](int i, int j) {
      const float d = (j <= i) ? S.dm[i][j] : 0.f;
      S.da2[i][j] = __float2bfloat16_rn(d * S.eta[i][j]);
      S.deta[i][j] = d * (1.f + S.a2[i][j]);
    });
    __syncthreads();
    TRM(8)
    // ---- 3. dz1b = (dz2b W2^T + dA2 x2) o gelu'(z1b)  (kept in t1)
    tile_mma<false, CS, E>(none, 1.f, [&](int i, int j, float x, float y) {
      const float2 d1 = ldb2(&S.z1b[i][j]);
      stb2(&S.t1[i][j], x * d1.x, y * d1.y);
    }, prod<F>(sdz2b, tr(sw2)), prod<CS>(sda2, sx2));
    __syncthreads();
    // ---- 4. z1b = Q W1 + b1 - M1 g1
    tile_mma<false, CS, CS>(mdm, -1.f, noepi, prod<E>(st1, tr(sg1)));              // dM1 = -tril(dz1b g1^T)
    // l o K goes to dz2 (free until step 7), l o x2 to z1b (dead after step 3)
    for_f2([&](int r, int c) {
      const float2 k_ = ldb2(&S.k[r][c]);
      stb2(&S.dz2[r][c], S.ell[r] * k_.x, S.ell[r] * k_.y);
    });
    for_e2([&](int r, int c) {
      const float2 x = ldb2(&S.x2[r][c]);
      stb2(&S.z1b[r][c], S.ell[r] * x.x, S.ell[r] * x.y);
    });
    __syncthreads();
    for_c([&](int i, int j) {
      const float d = (j <= i) ? S.dm[i][j] : 0.f;
      S.da1[i][j] = __float2bfloat16_rn(d * S.eta[i][j]);
      S.deta[i][j] += d * (1.f + S.a1[i][j]);
    });
    __syncthreads();
    tile_mma<false, CS, F>(mdq, 1.f, noepi, prod<E>(st1, tr(sw1)), prod<CS>(sda1, sk));   // dq = dz1b W1^T + dA1 K
    tile_mma<false, CS, F, 4, 8>(mdk, 1.f, noepi, prod<CS>(tr(sda1), sq));         // dk = dA1^T Q
    TRM(9)
    // ---- 5. the four state updates; dW1, db1, dW2, db2 still hold the gradients w.r.t. the next stage's state
    tile_mma<false, CS, F>(mgl1, 1.f, noepi, prod<E>(sg1, tr(hdW1)));              // gl1 = g1 dW1^T
    tile_mma<false, CS, E>(st3, 1.f, noepi, prod<F>(sg2, tr(hdW2)));               // gl2 = g2 dW2^T
    tile_mma<false, CS, E>(none, -1.f, [&](int i, int j, float x, float y) {         // dg1 = -M1^T dz1b - (l o K) dW1 - l (x) db1
      stb2(&S.t2[i][j], x - S.ell[i] * db1[j], y - S.ell[i] * db1[j + 1]);
    }, prod<CS>(tr(sm1), st1), prod<F>(sdz2, hdW1));
    tile_mma<true, CS, F, 4, 8>(mdg2, -1.f, [&](int i, int j, float x, float y) {   // dg2 -= (l o x2) dW2 + l (x) db2
      *reinterpret_cast<float2*>(&S.dg2[i][j]) = make_float2(x - S.ell[i] * db2[j], y - S.ell[i] * db2[j + 1]);
    }, prod<E>(sz1b, hdW2));
    __syncthreads();
    // dell[j] = -( gl1[j].K[j] + g1[j].db1 + gl2[j].x2[j] + g2[j].db2 )   (one row per warp)
    {
      const int r = warp;
      float acc = 0.f;
      {
        const int c = 2 * lane;
        const float2 gl = *reinterpret_cast<const float2*>(&S.gl1[r][c]), k_ = ldb2(&S.k[r][c]), g_ = ldb2(&S.g2[r][c]);
        acc += gl.x * k_.x + gl.y * k_.y + g_.x * db2[c] + g_.y * db2[c + 1];
      }
#pragma unroll
      for (int c = 2 * lane; c < E; c += 64) {
        const float2 g_ = ldb2(&S.g1[r][c]), l2 = ldb2(&S.t3[r][c]), x = ldb2(&S.x2[r][c]);
        acc += g_.x * db1[c] + g_.y * db1[c + 1] + l2.x * x.x + l2.y * x.y;
      }
      acc = warp_sum(acc);
      if (lane == 0) S.dell[r] = -acc;
    }
    for_f2([&](int r, int c) {                                                     // dk -= l o gl1
      float2* d = reinterpret_cast<float2*>(&S.dk[r][c]);
      const float2 gl = *reinterpret_cast<const float2*>(&S.gl1[r][c]);
      *d = make_float2(d->x - S.ell[r] * gl.x, d->y - S.ell[r] * gl.y);
    });
    // (no barrier: step 6 reads and writes none of what the two loops above touch)
    TRM(10)
    // ---- 6. g1 = h o gelu'(z1), h = g2 W2^T (recomputed):  dz1 = dg1 o h o gelu''(z1) (t4),  dh = dg1 o gelu'(z1) (t2)
    tile_mma<false, CS, E>(none, 1.f, [&](int i, int j, float hx, float hy) {
      const float2 d = ldb2(&S.t2[i][j]), d1 = ldb2(&S.gd1[i][j]), d2 = ldb2(&S.gd2[i][j]);
      stb2(&S.t4[i][j], d.x * hx * d2.x, d.y * hy * d2.y);
      stb2(&S.t2[i][j], d.x * d1.x, d.y * d1.y);
    }, prod<F>(sg2, tr(sw2)));
    __syncthreads();
    tile_mma<true, CS, F>(mdg2, 1.f, noepi, prod<E>(st2, sw2));                    // dg2 += dh W2
    __syncthreads();
    TRM(11)
    // ---- 7. second derivative through g2 = ln_l2_grad(z2, v - k): dz2, d target (into gl1, which is dead by now),
    //         LN parameter gradients (column partials in z1b's tile, whose scratch use is over)
    {
      const int r = warp, c = 2 * lane;
      const float2 zz = *reinterpret_cast<const float2*>(&S.z2[r][c]);
      const float mu = warp_sum(zz.x + zz.y) * (1.f / HD);
      const float var = warp_sum((zz.x - mu) * (zz.x - mu) + (zz.y - mu) * (zz.y - mu)) * (1.f / HD);
      const float rs = 1.f / sqrtf(var + p.eps);
      const float2 vv_ = ldb2(&S.v[r][c]), kk = ldb2(&S.k[r][c]);
      const float2 uu = *reinterpret_cast<const float2*>(&S.dg2[r][c]);
      const float xh[2] = {(zz.x - mu) * rs, (zz.y - mu) * rs}, tg[2] = {vv_.x - kk.x, vv_.y - kk.y}, u[2] = {uu.x, uu.y};
      float gy[2], gxh[2], vv[2], sg = 0.f, sgx = 0.f, sv = 0.f, svx = 0.f;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        gy[e] = S.gam[c + e] * xh[e] + S.bet[c + e] - tg[e];
        gxh[e] = gy[e] * S.gam[c + e];
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
      float dxh[2], pg[2], pb[2], dt[2], sd = 0.f, sS = 0.f;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float G = (gxh[e] - sg - xh[e] * sgx) * rs;
        const float dgxh = u[e] * rs + sv + xh[e] * svx;
        const float dy = S.gam[c + e] * dgxh;
        pg[e] = gy[e] * dgxh + dy * xh[e];
        pb[e] = dy;
        dxh[e] = dy * S.gam[c + e] + gxh[e] * svx + vv[e] * sgx;
        sd += dxh[e];
        sS += -(dxh[e] * xh[e] + u[e] * G) * rs;
        dt[e] = -S.gam[c + e] * dgxh;  // d target
      }
      sd = warp_sum(sd) * (1.f / HD);
      sS = warp_sum(sS) * (1.f / HD);
      *reinterpret_cast<float2*>(&S.gl1[r][c]) = make_float2(dt[0], dt[1]);
      stb2(&S.dz2[r][c], dxh[0] * rs - sd * rs + xh[0] * sS, dxh[1] * rs - sd * rs + xh[1] * sS);
      *reinterpret_cast<float2*>(&colpart[warp][c]) = make_float2(pg[0], pg[1]);
      *reinterpret_cast<float2*>(&colpart[warp][HD + c]) = make_float2(pb[0], pb[1]);
    }
    __syncthreads();
    if (tid < 2 * HD) {
      float s_ = 0.f;
#pragma unroll
      for (int w = 0; w < MB_NW; ++w) s_ += colpart[w][tid];
      if (tid < HD) S.dgam[tid] += s_; else S.dbet[tid - HD] += s_;
    }
    TRM(12)
    // ---- 8./9./10. z2 = x2 W2 + b2, x2 = gelu(z1), z1 = K W1 + b1:
    //      dx2 = dA2^T x2b + dz2 W2^T - l o gl2  (never stored);  dz1 += dx2 o gelu'(z1) (t4);  dk += dz1 W1^T
    tile_mma<false, CS, E>(none, 1.f, [&](int i, int j, float x, float y) {
      const float2 d1 = ldb2(&S.gd1[i][j]), d = ldb2(&S.t4[i][j]), gl2 = ldb2(&S.t3[i][j]);
      x -= S.ell[i] * gl2.x;
      y -= S.ell[i] * gl2.y;
      stb2(&S.t4[i][j], d.x + x * d1.x, d.y + y * d1.y);
    }, prod<CS>(tr(sda2), sx2b), prod<F>(sdz2, tr(sw2)));
    __syncthreads();
    tile_mma<true, CS, F>(mdk, 1.f, noepi, prod<E>(st4, tr(sw1)));
    TRM(13)
    // ---- gradients w.r.t. this stage's state (all reads of the next-stage gradients are done): one pass over each
    //      float32 master, the contraction running over the tokens of all the tile pairs
    {
      const uint32_t a[3] = {st2.a, sx2b.a, sx2.a}, b[3] = {sg2.a, sdz2b.a, sdz2.a};
      rank16_update<E, F, EB, FB, 3>(mdW2, 1.f, [&](int u, int h, float x, float y) {
        *reinterpret_cast<uint32_t*>(dW2h_at + (4 * u + h) * 512) = pack_bf16(x, y);
      }, a, b);
    }
    {
      const uint32_t a[2] = {sq.a, sk.a}, b[2] = {st1.a, st4.a};
      rank16_update<F, E, FB, EB, 2>(mdW1, 1.f, [&](int u, int h, float x, float y) {
        *reinterpret_cast<uint32_t*>(dW1h_at + ((2 * (u >> 1) + h) * 32 + 16 * (u & 1)) * 64) = pack_bf16(x, y);
      }, a, b);
    }
    add_colsum(db2, &S.dz2b[0][0], F, FB, 1.f);
    add_colsum(db1, &S.t1[0][0], E, EB, 1.f);
    TRM(14)
    // ---- 11. eta factors and outputs of the stage
    if (tid >= MB_THREADS - CS) {
      const int i = tid - (MB_THREADS - CS);
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
    add_colsum(db2, &S.dz2[0][0], F, FB, 1.f);
    add_colsum(db1, &S.t4[0][0], E, EB, 1.f);
    if (s > s_lo) nxt = fetch(s - 1);
    for_f2([&](int r, int c) {  // dq += dO;  dk -= dT;  dv = dT  (gl1 holds d target)
      const float2 a = *reinterpret_cast<const float2*>(&dq[r][c]), o = ldb2(&S.dO[r][c]);
      const float2 b = *reinterpret_cast<const float2*>(&S.dk[r][c]), dT = *reinterpret_cast<const float2*>(&S.gl1[r][c]);
      const size_t at = (r0 + (size_t)r * HD + c) >> 1;
      static_cast<uint32_t*>(p.d_q)[at] = pack_bf16(a.x + o.x, a.y + o.y);
      static_cast<uint32_t*>(p.d_k)[at] = pack_bf16(b.x - dT.x, b.y - dT.y);
      static_cast<uint32_t*>(p.d_v)[at] = pack_bf16(dT.x, dT.y);
    });
    __syncthreads();
    TRM(15)
  }
  __syncthreads();
  // the masters go back to the workspace: for the stream's next item, or (last item) for the output loop below
  if (rank < 2 * p.NCH - 1) {
    master_out(W1, tW1a);
    master_out(W2, tW2a);
  }
  if (!pass1) {
    master_out(dW1, tdW1a);
    master_out(dW2, tdW2a);
  }
  if (rank < 2 * p.NCH - 1) {
    // hand the stream to its next item
    for (int e = tid; e < E; e += MB_THREADS) {
      ho[HO_B1 + e] = b1[e];
      ho[HO_DB1 + e] = db1[e];
    }
    if (tid < F) {
      ho[HO_B2 + tid] = b2[tid];
      ho[HO_DB2 + tid] = db2[tid];
      ho[HO_DG + tid] = S.dgam[tid];
      ho[HO_DB + tid] = S.dbet[tid];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) *reinterpret_cast<volatile int*>(p.sched + 1 + stream) = rel + 1;
  } else {
    // ---- gradients w.r.t. the initial state, per-stream LayerNorm parameter gradients
    __syncthreads();  // dW1, dW2 are in the workspace for every thread
    for (int e = tid; e < F * E; e += MB_THREADS) {
      st_from_float<T>(p.d_w1, (size_t)stream * F * E + e, __ldcg(dW1 + MatG<F, E, false>::at(e / E, e % E)));
      st_from_float<T>(p.d_w2, (size_t)stream * F * E + e, __ldcg(dW2 + MatG<E, F, false>::at(e / F, e % F)));
    }
    for (int e = tid; e < E; e += MB_THREADS) st_from_float<T>(p.d_b1, (size_t)stream * E + e, db1[e]);
    if (tid < F) {
      st_from_float<T>(p.d_b2, (size_t)stream * F + tid, db2[tid]);
      p.part_ln[(size_t)stream * 2 * HD + tid] = S.dgam[tid];
      p.part_ln[(size_t)stream * 2 * HD + HD + tid] = S.dbet[tid];
    }
  }
  }  // item loop
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(s_tmem) : "memory");
#ifdef TTT_MLP_TRACE
  if (tid == 0 && blockIdx.x == 0 && p.trace != nullptr)
    for (int i = 0; i < 16; ++i) p.trace[i] = (unsigned int)(tr_acc[i] / NS);
#endif
#undef TRM
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

// floats of workspace per stream: the four float32 state matrices, the hand-off record, the bf16 g1p / g2p tiles of
// every stage, the float32 biases at the start of every stage, the bf16 operand copies of dW1 and dW2
size_t mlp_bwd_ws_stride_floats(int T) {
  const size_t ns = (size_t)T / CS;
  return 4 * (size_t)HD * MB_E + MLP_BWD_HANDOFF_FLOATS + ns * CS * (MB_E + HD) / 2 + ns * (MB_E + HD) + (size_t)HD * MB_E;
}

cudaError_t launch_mlp_bwd(const MlpBwdParams& p0, int B, cudaStream_t st) {
  MlpBwdParams p = p0;
  p.nstreams = B * p.H;
  p.CH = MLP_BWD_CHUNK;
  p.NCH = (p.NS + p.CH - 1) / p.CH;
  const size_t smem = sizeof(MlpBwdSmem);
  cudaError_t e = cudaFuncSetAttribute(ttt_mlp_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  // persistent grid: blocks wait on one another's hand-offs, so all of them must be resident (cooperative launch);
  // more blocks than streams would only wait (a stream's items run one after the other)
  int dev = 0, sms = 0, per_sm = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ttt_mlp_bwd_kernel, MB_THREADS, smem)) != cudaSuccess)
    return e;
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  int grid = sms * per_sm;
  if (grid > p.nstreams) grid = p.nstreams;
  if ((e = cudaMemsetAsync(p.sched, 0, sizeof(int) * (size_t)(1 + p.nstreams), st)) != cudaSuccess) return e;
  void* args[] = {(void*)&p};
  e = cudaLaunchCooperativeKernel((const void*)ttt_mlp_bwd_kernel, dim3(grid), dim3(MB_THREADS), args, smem, st);
  if (e != cudaSuccess) return e;
  const int n = p.T + 2 * p.H * HD;
  ttt_mlp_bwd_reduce_kernel<<<(n + 255) / 256, 256, 0, st>>>(p.part_te, p.part_ln, B, p.H, p.T, p.d_token_eta,
                                                           p.d_ln_g, p.d_ln_b);
  return cudaGetLastError();
}

}  // namespace ttt
