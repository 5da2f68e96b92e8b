// C++ host-side mirror of the reference's `fused-tile-multi` operator over the C ABI (include/ttt_b200.h).
//
// The reference's host code is Rust: `TttTileMultiKernel: FusedKernel` with `forward_launch` / `backward_launch`
// (rust/fused/src/linear_fused_tile/launch.rs:117-208, trait rust/kernels/src/kernel.rs:32-54), tensor bundles
// `TttInputs` / `TttOutputs` (rust/fused/src/ttt/types.rs:3-13), saved state `TttSavedStateMulti`
// (launch.rs:30-41) and `FusedTttConfig` (rust/fused/src/lib.rs:285-328).  This header gives the same operator to
// compiled-code callers: same names, same argument meaning; where the reference panics these functions throw.
// Like the reference's wrappers (forward/launch.rs:217-226, backward/launch.rs:351-392) the host side allocates the
// outputs -- through an allocator the caller supplies (the role of the reference's compute client).
#pragma once

#include <cstdint>
#include <cmath>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/ttt_b200.h"

namespace ttt_b200 {

// Device memory source owned by the caller (e.g. a framework's pool).
struct Allocator {
  virtual ~Allocator() = default;
  virtual void* alloc(size_t bytes) = 0;
  virtual void free(void* p) = 0;
};

struct DeviceTensor {
  void* ptr = nullptr;
  std::vector<int64_t> shape;
  int dtype = TTT_BF16;  // enum ttt_dtype; TTT_F32 also for the float32-only tensors
  size_t numel() const {
    size_t n = 1;
    for (int64_t d : shape) n *= static_cast<size_t>(d);
    return n;
  }
  size_t bytes() const { return numel() * (dtype == TTT_BF16 ? 2u : 4u); }
};

inline DeviceTensor empty(Allocator& a, std::vector<int64_t> shape, int dtype) {
  DeviceTensor t;
  t.shape = std::move(shape);
  t.dtype = dtype;
  t.ptr = a.alloc(t.bytes());
  if (t.ptr == nullptr) throw std::runtime_error("ttt_b200: allocator returned null");
  return t;
}

struct FusedTttConfig {
  int mini_batch_len = 16;
  int head_dim = 64;
  uint32_t epsilon_scaled = 1000;  // epsilon / 1e-9 in float32, as the reference stores it
  int threads = 128;               // accepted for compatibility; the kernels always use 4 warps per stream
  int checkpoint_interval = 1;
  static FusedTttConfig make(int mini_batch_len, int head_dim, float epsilon, int threads) {
    FusedTttConfig c;
    c.mini_batch_len = mini_batch_len;
    c.head_dim = head_dim;
    c.epsilon_scaled = static_cast<uint32_t>(epsilon / 1e-9f);
    c.threads = threads;
    return c;
  }
  float epsilon() const { return static_cast<float>(epsilon_scaled) * 1e-9f; }
};

struct TttInputs {
  DeviceTensor xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias;
};
struct TttOutputs {
  DeviceTensor output, weight, bias;
};
struct TttSavedStateMulti {
  DeviceTensor xq, xk, xv, weight_init, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias;
  DeviceTensor weight_checkpoints, bias_checkpoints;
};

namespace detail {
inline void check(int rc) {
  if (rc != TTT_OK) throw std::runtime_error(std::string("ttt_b200: ") + ttt_b200_last_error());
}
inline ttt_dims dims_of(const DeviceTensor& xq, const FusedTttConfig& c) {
  if (xq.shape.size() != 4) throw std::runtime_error("ttt_b200: xq must be [batch, heads, seq_len, head_dim]");
  if (c.mini_batch_len <= 0) throw std::runtime_error("mini_batch_len must be set for TttTileMultiKernel");
  ttt_dims d;
  d.batch = static_cast<int32_t>(xq.shape[0]);
  d.heads = static_cast<int32_t>(xq.shape[1]);
  d.seq_len = static_cast<int32_t>(xq.shape[2]);
  d.head_dim = static_cast<int32_t>(xq.shape[3]);
  d.mini_batch = c.mini_batch_len;
  d.checkpoint_interval = c.checkpoint_interval;
  d.epsilon = c.epsilon();
  d.dtype = xq.dtype;
  return d;
}
}  // namespace detail

struct TttTileMultiKernel {
  // Whole-sequence forward: returns (outputs, saved state).  `status` may be null (see ttt_b200.h).
  static std::pair<TttOutputs, TttSavedStateMulti> forward_launch(const TttInputs& in, const FusedTttConfig& cfg,
                                                                  Allocator& a, void* stream, void* status = nullptr) {
    const ttt_dims d = detail::dims_of(in.xq, cfg);
    const int64_t nck = ttt_linear_num_checkpoints(&d);
    if (nck < 0) throw std::runtime_error(std::string("ttt_b200: ") + ttt_b200_last_error());
    TttOutputs out;
    out.output = empty(a, in.xq.shape, in.xq.dtype);
    out.weight = empty(a, in.weight.shape, in.weight.dtype);
    out.bias = empty(a, in.bias.shape, in.bias.dtype);
    // opaque saved state, sized by the library (float32 words)
    DeviceTensor wck = empty(a, {static_cast<int64_t>(ttt_linear_weight_ckpt_bytes(&d) / 4)}, TTT_F32);
    DeviceTensor bck = empty(a, {static_cast<int64_t>((ttt_linear_bias_ckpt_bytes(&d) + 3) / 4)}, TTT_F32);
    detail::check(ttt_linear_forward(&d, in.xq.ptr, in.xk.ptr, in.xv.ptr, in.weight.ptr, in.bias.ptr,
                                     in.token_eta.ptr, in.ttt_lr_eta.ptr, in.ln_weight.ptr, in.ln_bias.ptr,
                                     out.output.ptr, out.weight.ptr, out.bias.ptr, wck.ptr, bck.ptr, status, stream));
    TttSavedStateMulti saved{in.xq, in.xk, in.xv, in.weight, in.bias, in.token_eta, in.ttt_lr_eta,
                             in.ln_weight, in.ln_bias, wck, bck};
    return {out, saved};
  }

  // Gradients w.r.t. the nine inputs in input order.  Only grad_outputs.output is used (gradients of the returned
  // final state are ignored, as in the reference).  token_eta / ln gradients are float32 tensors.
  static TttInputs backward_launch(const TttSavedStateMulti& s, const TttOutputs& grad_outputs,
                                   const FusedTttConfig& cfg, Allocator& a, void* stream,
                                   float* outer_grad_packed = nullptr, void* status = nullptr) {
    const ttt_dims d = detail::dims_of(s.xq, cfg);
    TttInputs g;
    g.xq = empty(a, s.xq.shape, s.xq.dtype);
    g.xk = empty(a, s.xq.shape, s.xq.dtype);
    g.xv = empty(a, s.xq.shape, s.xq.dtype);
    g.weight = empty(a, s.weight_init.shape, s.weight_init.dtype);
    g.bias = empty(a, s.bias.shape, s.bias.dtype);
    g.ttt_lr_eta = empty(a, s.ttt_lr_eta.shape, s.ttt_lr_eta.dtype);
    g.token_eta = empty(a, {d.seq_len}, TTT_F32);
    g.ln_weight = empty(a, {d.heads, d.head_dim}, TTT_F32);
    g.ln_bias = empty(a, {d.heads, d.head_dim}, TTT_F32);
    const size_t ws_bytes = ttt_linear_backward_workspace_bytes(&d);
    void* ws = a.alloc(ws_bytes);
    if (ws == nullptr) throw std::runtime_error("ttt_b200: allocator returned null for the workspace");
    const int rc = ttt_linear_backward(
        &d, s.xq.ptr, s.xk.ptr, s.xv.ptr, s.weight_init.ptr, s.bias.ptr, s.token_eta.ptr, s.ttt_lr_eta.ptr,
        s.ln_weight.ptr, s.ln_bias.ptr, s.weight_checkpoints.ptr, s.bias_checkpoints.ptr, grad_outputs.output.ptr,
        g.xq.ptr, g.xk.ptr, g.xv.ptr, g.weight.ptr, g.bias.ptr, g.ttt_lr_eta.ptr,
        static_cast<float*>(g.token_eta.ptr), static_cast<float*>(g.ln_weight.ptr),
        static_cast<float*>(g.ln_bias.ptr), outer_grad_packed, ws, ws_bytes, status, stream);
    // the workspace is only read by work already enqueued on `stream`; a stream-ordered pool may recycle it now
    a.free(ws);
    detail::check(rc);
    return g;
  }
};

}  // namespace ttt_b200
