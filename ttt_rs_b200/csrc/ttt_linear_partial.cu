// One mini-batch of fewer than (or exactly) 16 tokens of the TTT-Linear inner model: the decode step (1 token) and
// the tail of a sequence whose length is not a multiple of the mini-batch.
//
// Reference semantics: `TTTInnerModel::forward` runs whole mini-batches and then calls `forward_mini_batch` once on
// the remainder, i.e. the remainder is ONE mini-batch of its own length r with eta[i][j] = token_eta[i] * lr[j]
// (rust/core/src/inner.rs:25-50, rust/core/src/linear.rs:91-149); token by token generation therefore runs with
// r = 1 (rust/layer/src/ttt.rs:253-256).  The reference's fused kernels refuse these shapes
// (rust/fused/src/linear_fused_tile/wrapper.rs:152-172); only its unfused tensor-op path covers them.
//
// Work per stream is tiny (r <= 16 rows against an F x F state, F = 64 or 32), so this is a CUDA-core kernel: one
// F-thread CTA per (batch, head) stream, thread n owns column n of W (F float registers) and column n of every 16 x F
// tile; the stream's state is read and written exactly once (the HBM traffic that bounds a decode step).
#include "ttt_kernels.h"
#include "ttt_common.cuh"

namespace ttt {

template <int FD>
struct PartialSmem {
  float q[CS][FD], k[CS][FD], v[CS][FD];
  float attn[CS][CS];
  float lr[CS], te[CS];
  float red[2][CS][2];  // cross-warp partial sums
};

// Sums over the F columns (threads) of two values per row, for rows < r.  Every thread gets the totals.
template <int RM, int FD>
__device__ __forceinline__ void row_sums(PartialSmem<FD>& sm, int r, int tid, float (&a)[RM], float (&b)[RM]) {
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    if (i < r) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        a[i] += __shfl_xor_sync(0xffffffffu, a[i], o);
        b[i] += __shfl_xor_sync(0xffffffffu, b[i], o);
      }
      if (lane == 0) {
        sm.red[warp][i][0] = a[i];
        sm.red[warp][i][1] = b[i];
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    if (i < r) {
      a[i] = (FD == 64) ? sm.red[0][i][0] + sm.red[1][i][0] : sm.red[0][i][0];
      b[i] = (FD == 64) ? sm.red[0][i][1] + sm.red[1][i][1] : sm.red[0][i][1];
    }
  }
  __syncthreads();  // red may be reused
}

// RM: compile-time bound on the number of rows (1 for the decode step, 4, or 16), so that short mini-batches do not
// pay for sixteen rows of predicated-off arithmetic.
template <typename T, int RM, int FD>
__global__ void __launch_bounds__(FD) ttt_linear_partial_kernel(const LinPartialParams p) {
  constexpr int HD = FD;  // features per head in this instantiation (shadows the 64 of the tiled kernels)
  constexpr int PT_THREADS = FD;
  __shared__ PartialSmem<FD> sm;
  const int n = threadIdx.x;
  const int stream = blockIdx.x, head = stream % p.H, r = p.R;
  const size_t row0 = (size_t)stream * r;

  // tiles (converted to float), learning rates, token coefficients
  for (int e = n; e < r * HD; e += PT_THREADS) {
    const int i = e / HD, c = e % HD;
    sm.q[i][c] = ld_as_float<T>(p.xq, (row0 + i) * HD + c);
    sm.k[i][c] = ld_as_float<T>(p.xk, (row0 + i) * HD + c);
    sm.v[i][c] = ld_as_float<T>(p.xv, (row0 + i) * HD + c);
  }
  if (n < r) {
    sm.lr[n] = ld_as_float<T>(p.lr, row0 + n);
    sm.te[n] = ld_as_float<T>(p.token_eta, (size_t)n);
  }
  float w[HD];
#pragma unroll
  for (int k = 0; k < HD; ++k) w[k] = ld_as_float<T>(p.w0, (size_t)stream * HD * HD + (size_t)k * HD + n);
  float bias = ld_as_float<T>(p.b0, (size_t)stream * HD + n);
  const float gam = ld_as_float<T>(p.ln_g, (size_t)head * HD + n), bet = ld_as_float<T>(p.ln_b, (size_t)head * HD + n);
  __syncthreads();

  // Attn[i][j] = Q[i] . K[j] for j <= i
  for (int e = n; e < r * r; e += PT_THREADS) {
    const int i = e / r, j = e % r;
    float s = 0.f;
    if (j <= i) {
#pragma unroll
      for (int k = 0; k < HD; ++k) s = fmaf(sm.q[i][k], sm.k[j][k], s);
    }
    sm.attn[i][j] = s;
  }

  // Z1 = K W + b and Zq = Q W + b, column n
  float z1[RM], zq[RM];
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    z1[i] = zq[i] = bias;
    if (i < r) {
#pragma unroll
      for (int k = 0; k < HD; ++k) {
        z1[i] = fmaf(sm.k[i][k], w[k], z1[i]);
        zq[i] = fmaf(sm.q[i][k], w[k], zq[i]);
      }
    }
  }

  // LayerNorm statistics of Z1 (two-pass variance), then G = dL/dZ1
  float a[RM], b2[RM], mean[RM], rstd[RM];
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    a[i] = z1[i];
    b2[i] = 0.f;
  }
  row_sums<RM, FD>(sm, r, n, a, b2);
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    mean[i] = a[i] * (1.f / HD);
    const float d = z1[i] - mean[i];
    a[i] = d * d;
    b2[i] = 0.f;
  }
  row_sums<RM, FD>(sm, r, n, a, b2);
  float xh[RM], gx[RM], g[RM];
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    rstd[i] = 1.f / sqrtf(a[i] * (1.f / HD) + p.eps);
    xh[i] = (z1[i] - mean[i]) * rstd[i];
    const float tgt = (i < r) ? sm.v[i][n] - sm.k[i][n] : 0.f;
    gx[i] = (gam * xh[i] + bet - tgt) * gam;
    a[i] = gx[i];
    b2[i] = gx[i] * xh[i];
  }
  row_sums<RM, FD>(sm, r, n, a, b2);
#pragma unroll
  for (int i = 0; i < RM; ++i)
    g[i] = (i < r) ? (gx[i] - a[i] * (1.f / HD) - xh[i] * b2[i] * (1.f / HD)) * rstd[i] : 0.f;

  // Zbar = Zq - sum_{j<=i} te[i] lr[j] (1 + Attn[i][j]) G[j];  out = Q + LN(Zbar)
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    if (i < r) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < RM; ++j)
        if (j <= i && j < r) s = fmaf(sm.lr[j] * (1.f + sm.attn[i][j]), g[j], s);
      zq[i] -= sm.te[i] * s;
    }
    a[i] = zq[i];
    b2[i] = 0.f;
  }
  row_sums<RM, FD>(sm, r, n, a, b2);
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    mean[i] = a[i] * (1.f / HD);
    const float d = zq[i] - mean[i];
    a[i] = d * d;
    b2[i] = 0.f;
  }
  row_sums<RM, FD>(sm, r, n, a, b2);
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    if (i < r) {
      const float rs = 1.f / sqrtf(a[i] * (1.f / HD) + p.eps);
      st_from_float<T>(p.out, (row0 + i) * HD + n, sm.q[i][n] + gam * (zq[i] - mean[i]) * rs + bet);
    }
  }

  // state update with the last row of eta: W -= (te[r-1] lr o K)^T G,  b -= sum_j te[r-1] lr[j] G[j]
  const float te_last = sm.te[r - 1];
  float gl[RM];
#pragma unroll
  for (int j = 0; j < RM; ++j) gl[j] = (j < r) ? te_last * sm.lr[j] * g[j] : 0.f;
#pragma unroll
  for (int j = 0; j < RM; ++j) {
    if (j < r) {
      bias -= gl[j];
#pragma unroll
      for (int k = 0; k < HD; ++k) w[k] = fmaf(-sm.k[j][k], gl[j], w[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < HD; ++k) st_from_float<T>(p.w_out, (size_t)stream * HD * HD + (size_t)k * HD + n, w[k]);
  st_from_float<T>(p.b_out, (size_t)stream * HD + n, bias);
}

template <typename T, int FD>
static void launch_partial_t(const LinPartialParams& p, int nstreams, cudaStream_t st) {
  if (p.R == 1)
    ttt_linear_partial_kernel<T, 1, FD><<<nstreams, FD, 0, st>>>(p);
  else if (p.R <= 4)
    ttt_linear_partial_kernel<T, 4, FD><<<nstreams, FD, 0, st>>>(p);
  else
    ttt_linear_partial_kernel<T, 16, FD><<<nstreams, FD, 0, st>>>(p);
}

cudaError_t launch_linear_partial(int dtype, int head_dim, const LinPartialParams& p, int nstreams, cudaStream_t st) {
  if (head_dim == 32) {
    if (dtype == 1) launch_partial_t<__nv_bfloat16, 32>(p, nstreams, st);
    else launch_partial_t<float, 32>(p, nstreams, st);
  } else {
    if (dtype == 1) launch_partial_t<__nv_bfloat16, 64>(p, nstreams, st);
    else launch_partial_t<float, 64>(p, nstreams, st);
  }
  return cudaGetLastError();
}

}  // namespace ttt
