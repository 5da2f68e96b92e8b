/*
 * ttt_b200.h - C ABI of the B200 (sm_100a) fused TTT inner loop.
 *
 * This library replaces the *inside* of the reference's `fused-tile-multi` operator: the two host
 * functions that build launch arguments and dispatch the device kernels,
 *     forward_multi  / launch_tile_forward_multi   rust/fused/src/linear_fused_tile/forward/launch.rs:199-257,128-190
 *     backward_multi / launch_tile_backward_multi  rust/fused/src/linear_fused_tile/backward/launch.rs:332-438,234-325
 * which sit behind `TttTileMultiKernel: FusedKernel::{forward_launch, backward_launch}`
 * (rust/fused/src/linear_fused_tile/launch.rs:117-208).  Everything above that boundary (tensor bundles,
 * autodiff registration, the TTTInnerModel impl) is unchanged.
 *
 * Conventions
 *  - Every tensor pointer is a DEVICE pointer to a contiguous row-major buffer, 16-byte aligned.
 *  - The caller owns and allocates every buffer (as the reference's host wrappers do with `empty_like`);
 *    the library allocates nothing.  Apart from two documented exceptions it keeps no state between calls, so
 *    calls are re-entrant and may be issued from any thread: ttt_linear_backward_noalloc (one scratch array per
 *    device shared by all its calls, and a cached device address: see its section) and the diagnostic knob
 *    ttt_b200_debug_handoff (process-wide).  Calls enqueue work on `stream` and never synchronise.
 *  - `dtype` selects the element type of all tensors marked T below: TTT_F32 or TTT_BF16.  Arithmetic is
 *    float32 (bf16 tensor-core operands with float32 accumulation; three-plane split operands for TTT_F32).
 *  - Return value: TTT_OK or an error code; ttt_b200_last_error() gives a thread-local message.  Where the
 *    reference panics (unsupported tile config, seq_len not a multiple of the mini-batch:
 *    linear_fused_tile/mod.rs:143, forward/launch.rs:209-213) these functions return an error and launch
 *    nothing.
 *  - `status`, when non-null, points to 4 device uint32 words (16 for ttt_mlp_backward) that the caller zeroed
 *    once; a kernel whose bounded wait (on a TMA completion barrier, or on another block's hand-off) expires
 *    writes {TTT_ERR_TIMEOUT, where, block, stage} there by compare-and-swap from zero and returns early, leaving
 *    its outputs unwritten.  Launches never clear the words, so one buffer per device can serve every launch and
 *    the first report survives until the host reads and clears it.
 */
#ifndef TTT_B200_H
#define TTT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TTT_B200_ABI_VERSION 1

enum ttt_status {
  TTT_OK = 0,
  TTT_ERR_NULL = 1,        /* a required pointer is null */
  TTT_ERR_SHAPE = 2,       /* non-positive dim, seq_len % mini_batch != 0, checkpoint_interval < 1 */
  TTT_ERR_UNSUPPORTED = 3, /* tile (mini_batch, head_dim) not built (see ttt_dims); unknown dtype */
  TTT_ERR_ALIGN = 4,       /* a tensor base is not 16-byte aligned */
  TTT_ERR_CUDA = 5,        /* a CUDA runtime/driver call failed (message in ttt_b200_last_error) */
  TTT_ERR_TIMEOUT = 6,     /* written by kernels into `status`, never returned by a launch call */
  TTT_ERR_WORKSPACE = 7    /* workspace too small */
};

enum ttt_dtype { TTT_F32 = 0, TTT_BF16 = 1 };

/* Problem description.  Mirrors what the reference derives from tensor shapes plus `FusedTttConfig`
 * {mini_batch_len, head_dim, epsilon, checkpoint_interval} (rust/fused/src/lib.rs:285-328). */
typedef struct ttt_dims {
  int32_t batch;               /* B */
  int32_t heads;               /* H */
  int32_t seq_len;             /* T, multiple of mini_batch */
  int32_t head_dim;            /* F: 64; TTT-Linear forward/backward also take 32 with an even number of heads */
  int32_t mini_batch;          /* CS: 16; TTT-Linear forward/backward also take 8 */
  int32_t checkpoint_interval; /* K >= 1, in stages */
  float epsilon;               /* LayerNorm epsilon */
  int32_t dtype;               /* enum ttt_dtype */
} ttt_dims;

int ttt_b200_abi_version(void);
const char* ttt_b200_status_string(int status);
const char* ttt_b200_last_error(void);

/* Diagnostic knob for the persistent TTT-Linear backward (no counterpart in the reference, whose streaming kernels
 * spin without a limit: rust/fused/src/linear_fused_tile/streaming/d2d/kernel.rs:123-145).  Blocks of that kernel
 * wait, with an iteration limit, for the hand-off of the later chunk of their stream; when the limit is reached they
 * write {TTT_ERR_TIMEOUT, 15, block, stage} to `status` and return.  `poll_limit` replaces the limit (0 restores the
 * default, 2^24 polls of about 100 ns); `first_item` > 0 makes the launch skip that many work items, which -- set to
 * batch*heads -- leaves every remaining item waiting for a hand-off nobody publishes, so that a test can watch the
 * wait give up.  Process-wide; affects launches issued after the call.  Leave at (0, 0) in production. */
void ttt_b200_debug_handoff(uint32_t poll_limit, int32_t first_item);

/* Number of checkpoints per (batch, head) stream: ceil((T / CS) / K)  (forward/launch.rs:221-223). */
int64_t ttt_linear_num_checkpoints(const ttt_dims* d);
/* Bytes of the two saved-state buffers the forward fills and the backward reads back (the role of the reference's
 * weight_checkpoints / bias_checkpoints tensors, forward/launch.rs:221-226).  Both are opaque to the caller:
 *   weight_ckpt: float32 W before every K-th stage plus the final W, B*H*(NCK+1) blocks of 64*64 floats, each in
 *                the order the kernels' threads hold the state (not row-major);
 *   bias_ckpt:   per stage the lr-scaled LN gradient tile [B*H*T, F] of T, two float4 of row statistics per
 *                token, and the float32 bias at the start of every stage.
 * (head_dim 32, the reference's 16x32 tile, rust/fused/src/linear_fused_tile/mod.rs:32-37: the kernels run heads
 * 2j and 2j+1 of a batch element side by side in one 64-wide tile, so the saved state is laid out per PAIR of heads,
 * 64 x 64 float32 per checkpoint with the two 32 x 32 states on the diagonal.  The sizes below account for it; all
 * tensors of the caller keep the [B,H,...,32] layouts listed at the entry points.)
 * The backward walks W back from each checkpoint with the saved gradient tiles instead of re-simulating the
 * forward, so `checkpoint_interval` only sets how often W is re-read exactly. */
size_t ttt_linear_weight_ckpt_bytes(const ttt_dims* d);
size_t ttt_linear_bias_ckpt_bytes(const ttt_dims* d);

/* Forward of the whole sequence.  Replaces launch_tile_forward_multi (forward/launch.rs:128-190).
 *   xq, xk, xv      T [B,H,T,F]
 *   weight          T [B,H,F,F]   initial state W (per batch element), W[k][n]: z = x @ W
 *   bias            T [B,H,F]
 *   token_eta       T [T]         only entries [0, CS) are read, in every stage (forward/kernel.rs:152-165)
 *                                 (CS = d->mini_batch)
 *   ttt_lr_eta      T [B,H,T]
 *   ln_weight/bias  T [H,F]
 *   output          T [B,H,T,F]   (out)
 *   weight_out      T [B,H,F,F]   (out) final state
 *   bias_out        T [B,H,F]     (out)
 *   weight_ckpt, bias_ckpt        (out) opaque saved state, ttt_linear_*_ckpt_bytes bytes each; pass BOTH as NULL
 *                                 for inference: nothing is then kept for a backward (no checkpoints, gradient tiles
 *                                 or statistics are written -- about a third of the forward's HBM writes)
 */
int ttt_linear_forward(const ttt_dims* d, const void* xq, const void* xk, const void* xv, const void* weight,
                       const void* bias, const void* token_eta, const void* ttt_lr_eta, const void* ln_weight,
                       const void* ln_bias, void* output, void* weight_out, void* bias_out, void* weight_ckpt,
                       void* bias_ckpt, void* status, void* stream);

/* Scratch the backward needs (per-stream partial sums that a second, deterministic pass reduces). */
size_t ttt_linear_backward_workspace_bytes(const ttt_dims* d);

/* Backward of the whole sequence for upstream gradient `grad_output` of `output` only (gradients of the
 * returned final state are taken as zero, as launch.rs:188-194 does).  Replaces launch_tile_backward_multi
 * (backward/launch.rs:234-325).
 *   saved inputs as in forward, plus weight_ckpt / bias_ckpt written by ttt_linear_forward
 *   grad_output     T [B,H,T,F]
 *   grad_xq/xk/xv   T [B,H,T,F]   (out)
 *   grad_weight     T [B,H,F,F]   (out) per batch element (backward/launch.rs:355-362)
 *   grad_bias       T [B,H,F]     (out)
 *   grad_ttt_lr_eta T [B,H,T]     (out)
 *   grad_token_eta  float32 [T]   (out) stage s writes positions s*CS+i, summed over B and H
 *   grad_ln_weight, grad_ln_bias  float32 [H,F] (out) summed over B   (backward/launch.rs:368-385)
 *   outer_grad_packed  float32 [H*F*F + 3*H*F + CS] or null: {dW0 [H,F,F], db0 [H,F], d ln_weight, d ln_bias,
 *                   d token_eta folded to [CS]} summed over this call's batch: one buffer for one all-reduce
 *   workspace       at least ttt_linear_backward_workspace_bytes(d) bytes
 * The three float32 outputs are written (not accumulated into); the caller need not zero them.
 * The kernel is persistent (blocks take (stream, chunk of 16 mini-batches) work items; every hand-off wait is bounded,
 * see `status`) and each of its blocks holds 64 columns of the SM's tensor memory while it runs: a kernel of another
 * stream that wants more tensor memory than is left on an SM waits there until these blocks exit.
 */
int ttt_linear_backward(const ttt_dims* d, const void* xq, const void* xk, const void* xv, const void* weight,
                        const void* bias, const void* token_eta, const void* ttt_lr_eta, const void* ln_weight,
                        const void* ln_bias, const void* weight_ckpt, const void* bias_ckpt,
                        const void* grad_output, void* grad_xq, void* grad_xk, void* grad_xv, void* grad_weight,
                        void* grad_bias, void* grad_ttt_lr_eta, float* grad_token_eta, float* grad_ln_weight,
                        float* grad_ln_bias, float* outer_grad_packed, void* workspace, size_t workspace_bytes,
                        void* status, void* stream);

/* Backward that also takes upstream gradients of the returned final state (either may be null = zero):
 *   grad_weight_out  T [B,H,F,F], grad_bias_out  T [B,H,F]
 * The reference drops these gradients (launch.rs:188-194; backward/kernel.rs:293-300 starts dW_last/db_last at
 * zero); with them the operator is a complete autograd node, so a long sequence can be trained in chunks with the
 * state (and its gradient) carried from chunk to chunk.  Everything else as in ttt_linear_backward.
 */
int ttt_linear_backward_state_grads(const ttt_dims* d, const void* xq, const void* xk, const void* xv,
                                    const void* weight, const void* bias, const void* token_eta,
                                    const void* ttt_lr_eta, const void* ln_weight, const void* ln_bias,
                                    const void* weight_ckpt, const void* bias_ckpt, const void* grad_output,
                                    const void* grad_weight_out, const void* grad_bias_out, void* grad_xq,
                                    void* grad_xk, void* grad_xv, void* grad_weight, void* grad_bias,
                                    void* grad_ttt_lr_eta, float* grad_token_eta, float* grad_ln_weight,
                                    float* grad_ln_bias, float* outer_grad_packed, void* workspace,
                                    size_t workspace_bytes, void* status, void* stream);

/* Forward of the whole sequence for the 2-layer inner model (TTT-MLP, hidden width E = 4*F, GELU tanh).
 * The reference has no fused kernel for it; this replaces the loop of `TTTMLP::forward_mini_batch`
 * (rust/core/src/mlp.rs:127-208) behind `TTTInnerModel::forward` (rust/core/src/inner.rs:25-50), with the fused
 * kernels' convention that token_eta is read at [0, CS).  bf16 only (dtype must be TTT_BF16); checkpoint_interval
 * is ignored (the backward, ttt_mlp_backward, reverses the state updates instead of reloading checkpoints).
 *   xq, xk, xv      bf16 [B,H,T,F]
 *   w1, b1          bf16 [B,H,F,E], [B,H,E]   initial state, z1 = x @ w1 + b1
 *   w2, b2          bf16 [B,H,E,F], [B,H,F]
 *   token_eta [T], ttt_lr_eta [B,H,T], ln_weight / ln_bias [H,F]   bf16
 *   output          bf16 [B,H,T,F] (out);  w1_out, b1_out, w2_out, b2_out (out) final state, same shapes
 *   backward_workspace (optional, out): ttt_mlp_backward_workspace_bytes(d) bytes, 16-byte aligned.  When given, the
 *                   forward leaves there the float32 final state and the bf16 operands of every state update, which
 *                   is all the backward's own first pass would compute: pass the buffer on to ttt_mlp_backward
 *                   with workspace_from_forward = 1.  NULL (with 0 bytes) for inference.
 * One block per SM; a block holds 256 columns of the SM's tensor memory (the float32 state between its uses) while it
 * runs.
 */
int ttt_mlp_forward(const ttt_dims* d, const void* xq, const void* xk, const void* xv, const void* w1, const void* b1,
                    const void* w2, const void* b2, const void* token_eta, const void* ttt_lr_eta,
                    const void* ln_weight, const void* ln_bias, void* output, void* w1_out, void* b1_out, void* w2_out,
                    void* b2_out, void* backward_workspace, size_t backward_workspace_bytes, void* status,
                    void* stream);

/* TTT-MLP backward (bf16): gradient of ttt_mlp_forward for loss = <grad_output, output>; gradients w.r.t. the returned
 * final state are taken as zero, as for the TTT-Linear operator.  The reference has no fused counterpart: it
 * differentiates the tensor ops of rust/core/src/mlp.rs:127-208 with Burn autodiff.  Inputs are the forward's inputs
 * (nothing saved by the forward is needed: the kernel re-walks the sequence; with `workspace_from_forward` != 0 the
 * workspace is the one a ttt_mlp_forward call on the same inputs filled, and the re-walk is skipped), outputs:
 *   grad_xq, grad_xk, grad_xv [B,H,T,F]; grad_w1 [B,H,F,4F], grad_b1 [B,H,4F], grad_w2 [B,H,4F,F], grad_b2 [B,H,F]
 *   (per batch element); grad_ttt_lr_eta [B,H,T]; float32 grad_token_eta [T] (per stage position, summed over B, H),
 *   float32 grad_ln_weight / grad_ln_bias [H,F] (summed over B).  All written, never accumulated into.
 * `workspace`: ttt_mlp_backward_workspace_bytes(d) bytes, 16-byte aligned (float32 state and state gradients, a bf16
 * copy of the state gradients, the hand-off records and the saved bf16 per-stage inner gradients of every stream:
 * about B*H*(323 KB + 11 KB per mini-batch), plus the scheduler words).  The kernel is persistent: blocks take (stream,
 * chunk of 8 mini-batches) work items and hand a stream's state to one another through the workspace; it is launched
 * cooperatively (all blocks co-resident), one block per SM, and every hand-off wait is bounded.  A block allocates the
 * SM's whole tensor memory (512 columns) for the float32 state while it runs and frees it before it exits, so a kernel
 * of another stream that wants tensor memory on the same SM waits for it.  `status` (optional, 16 device words, zeroed by the
 * caller): {TTT_ERR_TIMEOUT, 1, block, item} if such a wait ran out; builds instrumented for tuning write per-phase
 * cycle counts of one block to the 16 words instead.
 */
size_t ttt_mlp_backward_workspace_bytes(const ttt_dims* d);
int ttt_mlp_backward(const ttt_dims* d, const void* xq, const void* xk, const void* xv, const void* w1, const void* b1,
                     const void* w2, const void* b2, const void* token_eta, const void* ttt_lr_eta,
                     const void* ln_weight, const void* ln_bias, const void* grad_output, void* grad_xq, void* grad_xk,
                     void* grad_xv, void* grad_w1, void* grad_b1, void* grad_w2, void* grad_b2, void* grad_ttt_lr_eta,
                     float* grad_token_eta, float* grad_ln_weight, float* grad_ln_bias, void* workspace,
                     size_t workspace_bytes, int workspace_from_forward, void* status, void* stream);

/* One mini-batch of fewer than (or exactly) mini_batch tokens: the tail of a sequence whose length is not a multiple
 * of the mini-batch, and the 1-token decode step.  Semantics: the reference's `TTTInnerModel::forward` calls
 * `forward_mini_batch` once on the remainder, i.e. the remainder is a mini-batch of its own length
 * (rust/core/src/inner.rs:25-50, rust/core/src/linear.rs:91-149); the reference's fused kernels reject such shapes
 * (rust/fused/src/linear_fused_tile/wrapper.rs:152-172), its unfused path computes them.
 *   d->seq_len = r, 1 <= r <= 16 (d->mini_batch and d->checkpoint_interval are not read); tensors as in
 *   ttt_linear_forward with T = r; token_eta holds the r coefficients of these positions.  Forward only: nothing is
 *   saved for a backward.  weight_out / bias_out may alias weight / bias (state advanced in place).
 *   head_dim 64 or 32 (here any number of heads: this kernel works head by head).
 */
int ttt_linear_forward_partial(const ttt_dims* d, const void* xq, const void* xk, const void* xv, const void* weight,
                               const void* bias, const void* token_eta, const void* ttt_lr_eta,
                               const void* ln_weight, const void* ln_bias, void* output, void* weight_out,
                               void* bias_out, void* stream);

/* ---- outer-layer steps on either side of the inner loop -------------------------------------------------------
 * These two entry points replace the tensor-op chains of the reference's `TTT` layer around `inner.forward`
 * (rust/layer/src/ttt.rs): `get_qkv` :152-197 (reshape + permute to [B,H,T,F], shared-QK causal convolutions
 * `conv_qk` :228-246, rotary embedding with the permute/undo-permute convention, rust/core/src/util.rs:284-392),
 * `get_lr` :205-227, and in `forward` :285-296 the permute back, `post_norm` and the optional gelu(tanh) gate.  The
 * projections themselves (q/k/v/g/o_proj, the per-head lr weights) stay ordinary GEMMs in the caller.
 * Only `batch`, `heads`, `seq_len`, `head_dim` (64 or 32; any number of heads, heads*head_dim <= 2048 for the
 * epilogue), `mini_batch` (rotary wrap) and `dtype` of `d` are read; seq_len need not be a multiple of mini_batch here.
 * The gradient entry points further down take the same shapes.
 */

/* Projection outputs -> inner-loop operands.
 *   q_src, k_src, v_src  [B*T, src_ld] rows = tokens; each points at the first of its H*F head-major columns (the
 *                        three may be column blocks of one fused projection output).  16-byte aligned, src_ld a
 *                        multiple of 8 elements.  With the shared-QK convolutions (conv_q_weight != NULL) q_src is
 *                        the shared projection and k_src is ignored.
 *   lr_logits            [B*T, lr_ld] x . learnable_ttt_lr_weight^T (first H columns), before the bias
 *   lr_bias              [H] or NULL
 *   conv_*_weight / bias [H*F, conv_kernel] / [H*F] depthwise causal taps (conv_kernel <= 4), or all NULL
 *   rope_mode            0 none, 1 positions (start_idx + t) mod mini_batch (`PosEncoding::Rope`), 2 global positions
 *   xq, xk, xv           (out) [B,H,T,F];   ttt_lr_eta (out) [B,H,T] = base_lr * sigmoid(logit + bias) / F
 */
int ttt_layer_prologue(const ttt_dims* d, const void* q_src, const void* k_src, const void* v_src, int64_t src_ld,
                       const void* lr_logits, int64_t lr_ld, const void* lr_bias, const void* conv_q_weight,
                       const void* conv_q_bias, const void* conv_k_weight, const void* conv_k_bias, int conv_kernel,
                       int start_idx, int rope_mode, float rope_theta, float base_lr, void* xq, void* xk, void* xv,
                       void* ttt_lr_eta, void* stream);

/* Inner-loop output [B,H,T,F] -> [B,T,H*F] with LayerNorm over H*F (biased variance, `eps` inside the root) and, when
 * `gate` != NULL, multiplied by gelu_tanh(gate) (gate = x . g_proj^T, [B*T, gate_ld], first H*F columns). */
int ttt_layer_epilogue(const ttt_dims* d, const void* inner_out, const void* gate, int64_t gate_ld,
                       const void* post_norm_weight, const void* post_norm_bias, float eps, void* y, void* stream);

/* The layer's projections as one product on the tensor cores (tcgen05, accumulators in tensor memory):
 *     c[m, n] = a[m, k] . b[n, k]^T       bf16 operands and result, float32 accumulation
 * `a` = hidden states with one token per row (row pitch lda elements), `b` = a weight matrix as the layer stores it,
 * one output feature per row (pitch ldb) -- so q/k/v/g/lr weights stacked by rows give all projections of the token
 * in one call, and o_proj is the same call on the epilogue's output.  Replaces the `Linear` forwards of
 * rust/layer/src/ttt.rs:152-227,289-299 (Burn matmul).  All pointers 16-byte aligned, pitches multiples of 8
 * elements; any m, n, k > 0 (edges are clipped / zero-filled by the tensor maps).  `status`: optional 4 words.
 * Products of 512 rows and more run as pairs of thread blocks on 256 x 256 tiles (tcgen05 cta_group::2), smaller ones
 * as single blocks on 128 x 256 tiles; TTT_GEMM_PAIR=0 / 1 in the environment forces one form (for measurements). */
int ttt_gemm_bf16_tn(int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, const void* b, int64_t ldb, void* c,
                     int64_t ldc, void* status, void* stream);

/* All projections of the layer and the step that follows them, in one launch (bf16, head_dim 64): the product
 * x . weights^T of ttt_gemm_bf16_tn with `weights` = the q | k | v | (g) | lr rows stacked, whose epilogue does what
 * `get_qkv` / `get_lr` do with the projection output (rust/layer/src/ttt.rs:152-227; this library's
 * ttt_layer_prologue without the shared-QK convolutions): q and k are rotated and written as xq / xk [B,H,T,F], v as
 * xv, the gate columns to `gate` [B*T, H*F] (pass g_col = -1 and gate = NULL when the layer has none), the logits as
 * ttt_lr_eta[b,h,t] = base_lr / F * sigmoid(logit + lr_bias[h]).  The [B*T, rows] projection output is never stored.
 *   x [B*T, x_ld] (first `hidden` columns), weights [w_rows, w_ld]; *_col: first weight row of each block (multiples
 *   of 64; q, k, v, g blocks are heads*64 rows, the lr block `heads` rows); rope_mode 0 or 1 (positions
 *   (start_idx + t) mod mini_batch, mini_batch <= 16).  seq_len must be a multiple of 128; other shapes, global
 *   rotary positions and the shared-QK layout go through ttt_gemm_bf16_tn + ttt_layer_prologue. */
int ttt_layer_projections(const ttt_dims* d, const void* x, int64_t x_ld, int64_t hidden, const void* weights,
                          int64_t w_ld, int64_t w_rows, int64_t q_col, int64_t k_col, int64_t v_col, int64_t g_col,
                          int64_t lr_col, const void* lr_bias, int start_idx, int rope_mode, float rope_theta,
                          float base_lr, void* xq, void* xk, void* xv, void* gate, void* ttt_lr_eta, void* status,
                          void* stream);

/* Gradients of the two layer steps (training; the reference gets them from Burn autodiff over the same tensor ops).
 *
 * ttt_layer_prologue_backward: gradients of XQ, XK, XV [B,H,T,F] and of ttt_lr_eta [B,H,T] -> gradient of the
 * projection output: grad_q_dst / grad_k_dst / grad_v_dst are its H*F-column blocks ([B*T, dst_ld]; inverse rotation
 * applied to q and k), grad_lr_logits its logit columns ([B*T, lr_ld]; `lr_cols` >= H columns are written, the ones
 * after the first H with zeros, so that padding columns of a fused projection are defined).  `ttt_lr_eta` is the
 * forward's output.  The shared-QK convolution layout has no backward here (TTT_ERR_UNSUPPORTED is not needed:
 * there is simply no convolution argument); its weights' gradients are not produced by this library.
 *
 * ttt_layer_epilogue_backward: grad_y [B*T, H*F] -> grad_inner_out [B,H,T,F], grad_gate ([B*T, grad_gate_ld], only
 * with a gate) and float32 grad_post_norm_weight / grad_post_norm_bias [H*F] (written, summed over all tokens in a
 * fixed order).  `workspace` must hold ttt_layer_epilogue_backward_workspace_bytes(d) bytes.
 */
int ttt_layer_prologue_backward(const ttt_dims* d, const void* grad_xq, const void* grad_xk, const void* grad_xv,
                                const void* grad_ttt_lr_eta, const void* ttt_lr_eta, int start_idx, int rope_mode,
                                float rope_theta, float base_lr, void* grad_q_dst, void* grad_k_dst,
                                void* grad_v_dst, int64_t dst_ld, void* grad_lr_logits, int64_t lr_ld, int lr_cols,
                                void* stream);
size_t ttt_layer_epilogue_backward_workspace_bytes(const ttt_dims* d);
int ttt_layer_epilogue_backward(const ttt_dims* d, const void* grad_y, const void* inner_out, const void* gate,
                                int64_t gate_ld, const void* post_norm_weight, const void* post_norm_bias,
                                float eps, void* grad_inner_out, void* grad_gate, int64_t grad_gate_ld,
                                float* grad_post_norm_weight, float* grad_post_norm_bias, void* workspace,
                                size_t workspace_bytes, void* stream);

/* Shared-QK causal depthwise convolutions as a training step of their own (the reference: `conv_qk`,
 * rust/layer/src/ttt.rs:205-227, nn.Conv1d(groups=C, padding=K-1)(x)[..., :T] in reference/ttt.py:647-663; gradients
 * there come from autodiff).  Inference applies the convolutions inside ttt_layer_prologue; for training they are a
 * step with its own gradient, whose outputs go through ttt_layer_prologue / ttt_layer_prologue_backward as separate
 * q and k blocks.  C = heads * head_dim channels; weights are [C][4] with tap j multiplying token t - 3 + j (a shorter
 * kernel is passed zero-padded at the front), biases [C]; zeros before the start of each sequence.
 *   ttt_layer_qk_conv:          x [B*T, x_ld] (first C columns) -> q, k [B*T, C]
 *   ttt_layer_qk_conv_backward: grad_q, grad_k [B*T, C] -> grad_x [B*T, C] and float32 parameter gradients
 *                               grad_q_params / grad_k_params [5*C]: d weight as [4][C] (tap-major), then d bias [C];
 *                               written, summed over all tokens in a fixed order.  `workspace`:
 *                               ttt_layer_qk_conv_backward_workspace_bytes(d) bytes, 16-byte aligned.
 */
int ttt_layer_qk_conv(const ttt_dims* d, const void* x, int64_t x_ld, const void* conv_q_weight,
                      const void* conv_q_bias, const void* conv_k_weight, const void* conv_k_bias, void* q, void* k,
                      void* stream);
size_t ttt_layer_qk_conv_backward_workspace_bytes(const ttt_dims* d);
int ttt_layer_qk_conv_backward(const ttt_dims* d, const void* grad_q, const void* grad_k, const void* x, int64_t x_ld,
                               const void* conv_q_weight, const void* conv_k_weight, void* grad_x,
                               float* grad_q_params, float* grad_k_params, void* workspace, size_t workspace_bytes,
                               void* stream);

/* Backward without a caller workspace.  (No counterpart in the reference: its host wrapper always allocates its
 * scratch itself, backward/launch.rs:389-392.)
 *
 * For hosts that cannot get device memory where the backward is issued -- an operator hook that receives only the
 * op's input and output buffers, a runtime whose pool has already claimed the device, a loop that must not call
 * cudaMalloc because it stalls every stream of the device.  Arguments and results are exactly those of
 * ttt_linear_backward minus `workspace` / `workspace_bytes`; the per-stream partial sums go to a fixed array of
 * TTT_NOALLOC_SCRATCH_BYTES bytes inside the library, which every GPU that uses the library keeps resident until
 * the process ends.  The function itself allocates nothing.
 *   - Limit: ttt_linear_backward_workspace_bytes(d) must not exceed TTT_NOALLOC_SCRATCH_BYTES
 *     (about batch*heads*(1.5*seq_len + 12420)*4 bytes; B=32 H=12 T=2048 needs 23.8 MB).  Larger problems get TTT_ERR_WORKSPACE
 *     and nothing is launched.
 *   - The first call on each device looks up the array's device address (one-time set-up, with that device
 *     current).  Make that first call outside any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels may overlap on the GPU (different
 *     streams, no ordering between them) race on it.  Issue them on one stream or order them with events.
 */
#define TTT_NOALLOC_SCRATCH_BYTES (32u << 20)
int ttt_linear_backward_noalloc(const ttt_dims* d, const void* xq, const void* xk, const void* xv,
                                const void* weight, const void* bias, const void* token_eta,
                                const void* ttt_lr_eta, const void* ln_weight, const void* ln_bias,
                                const void* weight_ckpt, const void* bias_ckpt, const void* grad_output,
                                void* grad_xq, void* grad_xk, void* grad_xv, void* grad_weight, void* grad_bias,
                                void* grad_ttt_lr_eta, float* grad_token_eta, float* grad_ln_weight,
                                float* grad_ln_bias, float* outer_grad_packed, void* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TTT_B200_H */
