// Internal interface between the C-ABI layer (ttt_abi.cu) and the kernel translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ttt {

struct LinFwdParams {
  const void* w0;         // [B,H,F,F] element type T
  const void* b0;         // [B,H,F]
  const void* token_eta;  // [T], first 16 entries read
  const void* lr;         // [B,H,T]
  const void* ln_g;       // [H,F]
  const void* ln_b;       // [H,F]
  void* w_out;            // [B,H,F,F]
  void* b_out;            // [B,H,F]
  float* w_ckpt;          // [B*H*(NCK+1), F, F] float32: state before stage c*K for c < NCK, final state at c = NCK
  float4* stats;          // [B*H*T][2]: (mean1, rstd1, A, Bv), (mean2, rstd2, 0, 0) per token
  float* b_stage;         // [B*H*(NS+1), F] float32: bias at the start of every stage, final bias last
  uint32_t* status;       // device uint32[4] or null
  int H, T, NS, K, NCK;
  float eps;
};

struct LinBwdParams {
  const void* w0;
  const void* b0;
  const void* token_eta;
  const void* lr;
  const void* ln_g;
  const void* ln_b;
  const float* w_ckpt;
  const float4* stats;
  const float* b_stage;
  const void* dw_in;  // [B,H,F,F] T: upstream gradient of the returned final weight, or null (zero)
  const void* db_in;  // [B,H,F]   T: upstream gradient of the returned final bias, or null (zero)
  void* d_w;        // [B,H,F,F] element type T (per batch element), nullable
  void* d_b;        // [B,H,F], nullable
  void* d_lr;       // [B,H,T]
  int* sched;       // workspace: [0] next work item, [1 + stream] chunks of the stream finished so far (zeroed per launch)
  float* handoff;   // workspace: [B*H][2*F*F + F] W^T, dW^T (register layout) and db handed from chunk to chunk
  int CH, NCH, nstreams;  // stages per chunk, chunks per stream, B*H
  uint32_t handoff_polls;  // iteration limit of the wait for another chunk's hand-off (each poll sleeps ~100 ns)
  int item_base;           // added to every work-item number (0 in normal use; the wait-limit test starts past the
                           // items that would publish the first hand-offs, so that a wait runs out)
  float* part_ln;   // workspace: [B*H][NCH][2][F] per-(stream, chunk) partial LN gradients (weight, bias)
  float* part_te;   // workspace: [B*H][T] per-stream token_eta gradient terms
  float* part_w;    // workspace: [B*H][F*F + F] float32 dW, db per stream (for the packed reduction)
  uint32_t* status;
  int H, T, NS, K, NCK;
  float eps;
};

struct ReduceParams {
  const float* part_ln;
  const float* part_te;
  const float* part_w;
  float* d_token_eta;  // [T] f32
  float* d_ln_g;       // [H,F] f32
  float* d_ln_b;       // [H,F] f32
  float* packed;       // nullable: [H*F*F + 3*H*F + CS] f32
  int B, H, T, NCH;
  int F;   // features per head: 64, or 32 (two heads per 64-wide tile in part_ln)
  int mb;  // tokens per mini-batch (16 or 8): d_token_eta is folded to [mb]
};

struct MlpFwdParams {
  const void* w1;         // [B,H,F,E] bf16, E = 4F
  const void* b1;         // [B,H,E]
  const void* w2;         // [B,H,E,F]
  const void* b2;         // [B,H,F]
  const void* token_eta;  // [T], first 16 entries read
  const void* lr;         // [B,H,T]
  const void* ln_g;       // [H,F]
  const void* ln_b;       // [H,F]
  void* w1_out;
  void* b1_out;
  void* w2_out;
  void* b2_out;
  uint32_t* status;
  float* bwd_ws;         // optional: the backward's workspace; the forward then leaves there what the backward's own
  size_t bwd_ws_stride;  // first pass would compute (final state, final biases, lr-scaled inner gradients per stage)
  int* sched;            // with bwd_ws: [1 + B*H] work-item counter and per-stream count of finished chunks (the
                         // persistent launch; zeroed by the launcher), else null
  int nstreams, CH, NCH; // set by the launcher: streams, stages per work item, items per stream
  uint32_t handoff_polls;  // iteration limit of the wait for the previous chunk's state
  int H, T, NS;
  float eps;
};
// Outer-layer steps either side of the inner loop (ttt_layer.cu).
struct LayerProParams {
  const void* q_src;   // projection outputs, rows = tokens (b*T + t), this head-major column block of H*F columns;
  const void* k_src;   // with the shared-QK convolutions q_src is the shared projection and k_src is unused
  const void* v_src;
  long ld_src;         // row stride of the three sources, in elements
  const void* lr_logits;  // [B*T, ld_lr], first H columns used
  long ld_lr;
  const void* lr_bias;    // [H] or null
  const void* conv_q_w;   // [H*F, conv_k] or null (no convolution)
  const void* conv_q_b;   // [H*F]
  const void* conv_k_w;
  const void* conv_k_b;
  int conv_k;
  void* xq;            // [B,H,T,F]
  void* xk;
  void* xv;
  void* lr_out;        // [B,H,T]
  int B, H, T;
  int start_idx, pos_mod, rope_mode;  // rope_mode: 0 none, 1 positions modulo pos_mod, 2 global positions
  float rope_theta, base_lr;
};
struct LayerEpiParams {
  const void* inner_out;  // [B,H,T,F]
  const void* gate;       // [B*T, ld_gate] (first H*F columns) or null
  long ld_gate;
  const void* ln_w;       // [H*F]
  const void* ln_b;
  void* y;                // [B,T,H*F]
  int B, H, T;
  float eps;
};
struct LayerProBwdParams {
  const void* dxq;  // [B,H,T,F] gradients of the prologue's outputs
  const void* dxk;
  const void* dxv;
  const void* dlr;  // [B,H,T]
  const void* lr;   // [B,H,T] the forward's ttt_lr_eta
  void* dq_dst;     // [B*T, ld_dst] column blocks of the projection-output gradient
  void* dk_dst;
  void* dv_dst;
  long ld_dst;
  void* dlogits_dst;  // [B*T, ld_dlr]: lr_cols columns written (H logit gradients, then zeros)
  long ld_dlr;
  int lr_cols;
  int B, H, T;
  int start_idx, pos_mod, rope_mode;
  float rope_theta, base_lr;
};
struct LayerEpiBwdParams {
  const void* dy;         // [B*T, H*F] gradient of the epilogue's output
  const void* inner_out;  // [B,H,T,F]
  const void* gate;       // [B*T, ld_gate] or null
  long ld_gate;
  const void* ln_w;
  const void* ln_b;
  void* d_inner;          // [B,H,T,F]
  void* dgate;            // [B*T, ld_dgate] (written when gate != null)
  long ld_dgate;
  float* d_ln_w;          // [H*F] float32
  float* d_ln_b;
  float* partials;        // workspace (float32): [B*T][2] row statistics, then [slabs][2][H*F] partial sums
  float2* row_stats;      // set by the launcher (start of the workspace)
  int B, H, T;
  float eps;
};
// Shared-QK causal depthwise convolutions as a training step of their own (ttt_layer.cu): q = conv_q(x) + bq,
// k = conv_k(x) + bk over the token axis, four taps aligned to the end (tap j multiplies token t - 3 + j; shorter
// kernels are passed zero-padded at the front), zeros before the start of the sequence.
struct LayerConvParams {
  const void* x;   // [B*T, ld_x] shared projection output, C = H*F columns used
  long ld_x;
  const void* wq;  // [C][4]
  const void* bq;  // [C]
  const void* wk;
  const void* bk;
  void* q;         // [B*T, C] (out)
  void* k;         // [B*T, C] (out)
  int B, T, C;
};
struct LayerConvBwdParams {
  const void* dq;  // [B*T, C]
  const void* dk;
  const void* x;   // as in the forward
  long ld_x;
  const void* wq;
  const void* wk;
  void* dx;        // [B*T, C] (out)
  float* partials; // [B * ceil(T / LAYER_CONV_CHUNK)][10 C] per-chunk parameter-gradient partials
  float* dparams_q;  // [5 C]: d wq as [4][C] (tap-major), then d bq [C]
  float* dparams_k;  // [5 C]
  int B, T, C;
};
constexpr int LAYER_CONV_CHUNK = 64;  // tokens a thread walks
cudaError_t launch_layer_conv(int dtype, const LayerConvParams& p, cudaStream_t st);
cudaError_t launch_layer_conv_bwd(int dtype, const LayerConvBwdParams& p, cudaStream_t st);
cudaError_t launch_layer_prologue(int dtype, int head_dim, const LayerProParams& p, cudaStream_t st);
cudaError_t launch_layer_prologue_bwd(int dtype, int head_dim, const LayerProBwdParams& p, cudaStream_t st);
cudaError_t launch_layer_epilogue_bwd(int dtype, int head_dim, const LayerEpiBwdParams& p, cudaStream_t st);
size_t layer_epilogue_bwd_workspace_bytes(int B, int H, int T, int head_dim);
cudaError_t launch_layer_epilogue(int dtype, int head_dim, const LayerEpiParams& p, cudaStream_t st);

// One mini-batch of R <= 16 tokens per stream (decode step, sequence tail): ttt_linear_partial.cu.
struct LinPartialParams {
  const void* xq;  // [B,H,R,F]
  const void* xk;
  const void* xv;
  const void* w0;         // [B,H,F,F]
  const void* b0;         // [B,H,F]
  const void* token_eta;  // [R]
  const void* lr;         // [B,H,R]
  const void* ln_g;       // [H,F]
  const void* ln_b;
  void* out;              // [B,H,R,F]
  void* w_out;            // may alias w0
  void* b_out;            // may alias b0
  int H, R;
  float eps;
};
cudaError_t launch_linear_partial(int dtype, int head_dim, const LinPartialParams& p, int nstreams, cudaStream_t st);

// TTT-MLP backward (ttt_mlp_bwd.cu), bf16 I/O.
struct MlpBwdParams {
  const void* xq;  // [B,H,T,F]
  const void* xk;
  const void* xv;
  const void* w1;  // [B,H,F,E]
  const void* b1;  // [B,H,E]
  const void* w2;  // [B,H,E,F]
  const void* b2;  // [B,H,F]
  const void* token_eta;
  const void* lr;
  const void* ln_g;
  const void* ln_b;
  const void* d_out;  // [B,H,T,F]
  void* d_q;
  void* d_k;
  void* d_v;
  void* d_w1;
  void* d_b1;
  void* d_w2;
  void* d_b2;
  void* d_lr;
  float* d_token_eta;  // [T] float32
  float* d_ln_g;       // [H,F] float32
  float* d_ln_b;
  float* workspace;    // per stream `ws_stride` floats: state, state gradients, saved inner gradients
  size_t ws_stride;
  float* part_te;      // [B*H][T]
  float* part_ln;      // [B*H][2][F]
  unsigned int* trace;  // optional 16 words (per-phase cycle counts of block 0 in instrumented builds), else null
  int* sched;           // [1 + B*H] work-item counter and per-stream count of finished items (zeroed by the launcher)
  uint32_t* status;     // optional 4 words: {TTT_ERR_TIMEOUT, where, block, item} if a hand-off wait ran out
  int H, T, NS;
  int nstreams, CH, NCH;  // set by the launcher: streams, stages per work item, items per pass
  int pass1_done;         // the forward already filled the workspace (ttt_mlp_forward with backward_workspace)
  float eps;
};
// Per-stream block of the TTT-MLP backward's workspace, in floats: W1 [64][256], W2 [256][64], dW1, dW2 (float32, each
// stored tile by tile in accumulator-fragment order, see mlp_state_at), the hand-off record between work items
// (b1, b2, db1, db2, d ln_weight, d ln_bias), then per stage the bf16 tiles lr o g1 [NS][16][256] and lr o g2
// [NS][16][64], then the float32 biases b1 | b2 at the start of every stage [NS][256 + 64], then bf16 copies of dW1 and
// dW2 (64 KB) that the backward reads as product operands.
constexpr int MLP_BWD_HANDOFF_FLOATS = 2 * 256 + 4 * 64;
constexpr int MLP_HO_B1 = 0, MLP_HO_B2 = 256, MLP_HO_DB1 = 320, MLP_HO_DB2 = 576, MLP_HO_DG = 640, MLP_HO_DB = 704;
// element (r, c) of a float32 matrix with C columns stored in accumulator-fragment order: the 16 x 8 tile
// (r / 16, c / 8) occupies 128 consecutive floats, its rows 0..7 before its rows 8..15, and inside a half the
// element (r % 8, c % 8) sits at 8 * (r % 8) + (c % 8)
__host__ __device__ inline int mlp_state_at(int r, int c, int C) {
  return (((r >> 4) * (C / 8) + (c >> 3)) << 7) + (((r >> 3) & 1) << 6) + ((r & 7) << 3) + (c & 7);
}
size_t mlp_bwd_ws_stride_floats(int T);
cudaError_t launch_mlp_bwd(const MlpBwdParams& p, int B, cudaStream_t st);

// bf16 projection GEMM C[M,N] = A[M,K] . B[N,K]^T on tcgen05 (ttt_gemm.cu).  maps: A, B (loads, box 64 x 128), C (store).
// Fused epilogue of the layer's stacked projection (ttt_layer_projections): where the column blocks of the product
// start (multiples of 64; g_col < 0 = no gate) and where their results go.
struct GemmFuse {
  int q_col, k_col, v_col, g_col, lr_col;
  int H, T;                 // heads, tokens per sequence (T % 128 == 0)
  int start_idx, pos_mod, rope_mode;  // rope_mode 0 none, 1 positions (start_idx + t) mod pos_mod, pos_mod <= 16
  float rope_theta, base_lr;
  const void* lr_bias;      // [H] bf16 or null
  void* lr_out;             // ttt_lr_eta [B,H,T] bf16
};
struct GemmParams {
  int M, N, K;
  uint32_t* status;  // optional 4 words
  GemmFuse f;        // read by the fused kernel only
};
cudaError_t launch_gemm_bf16_tn(const CUtensorMap* maps, const GemmParams& p, bool fused, bool pair, cudaStream_t st);

// bf16 only.  maps: q, k, v, out.
cudaError_t launch_mlp_fwd(const CUtensorMap* maps, const MlpFwdParams& p, int nstreams, cudaStream_t st);

// dtype: 0 = float32, 1 = bfloat16.  seg: features per head, 64 or 32 (two heads per tile).  mb: tokens per
// mini-batch, 16 or 8 (the tile maps then have boxes of 8 rows).
// maps: q, k, v, out, gp (saved lr-scaled LN gradient, [B*H*T, 64] of T); io: the plain pointers behind the first
// four maps, in the same order (used by the instantiation that gathers its tiles: seg 32 in bf16).
cudaError_t launch_linear_fwd(int dtype, int seg, int mb, const CUtensorMap* maps, const void* const* io,
                              const LinFwdParams& p, int nstreams, cudaStream_t st);
// maps: q, k, v, d_out, d_q, d_k, d_v, gp; io: the plain pointers behind the first seven.
cudaError_t launch_linear_bwd(int dtype, int seg, int mb, const CUtensorMap* maps, const void* const* io,
                              const LinBwdParams& p, int nstreams, cudaStream_t st);
cudaError_t launch_linear_bwd_reduce(const ReduceParams& p, cudaStream_t st);

}  // namespace ttt
