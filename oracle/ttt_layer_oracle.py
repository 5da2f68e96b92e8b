"""CPU restatement of the outer TTT layer around the inner loop (forward).  TEST INFRASTRUCTURE: only tests, the
smoke check and the CPU-baseline leg of the benchmark may import this module; the product never does.

What it restates (reference files by their path inside the reference project):

* `TTT::forward`, `get_qkv`, `get_lr`, `conv_qk`, `get_inner_loop_inputs`   rust/layer/src/ttt.rs:152-299
* rotary embedding with the permute / undo-permute convention           rust/core/src/util.rs:284-392
* the PyTorch twin `TTTBase.forward` and helpers                        reference/ttt.py:215-270,325-356,701-915

Parity: PINNED.  tests/golden/layer_linear_f64.npz holds inputs, parameters and outputs of the reference's own
`TTTLinear.forward` (float64; both the default configuration and the share_qk + gate configuration), produced by
tests/golden/make_golden.py; tests/test_layer_oracle.py checks this restatement against them.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from . import ttt_oracle as O


def rope_pairs(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotary embedding on adjacent pairs (2i, 2i+1) of the last axis of x [B,H,T,F].

    The reference permutes (evens first, odds last), applies the rotate-half form and undoes the permutation
    (reference/ttt.py:215-270, rust/layer/src/ttt.rs:176-192); the net effect is the rotation of each adjacent pair
    by angle pos * theta^(-2i/F).  Angles, cos and sin are float32 and then cast to x's dtype, as the reference does
    (reference/ttt.py:339-356).
    """
    F = x.shape[-1]
    inv_freq = 1.0 / (theta ** (torch.arange(0, F, 2, dtype=torch.int64).float() / F))
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
    x0, x1 = x[..., 0::2], x[..., 1::2]
    y0 = x0 * cos - x1 * sin
    y1 = x1 * cos + x0 * sin
    return torch.stack((y0, y1), dim=-1).flatten(-2)


def causal_depthwise_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[b,t,c] = bias[c] + sum_j weight[c,j] * x[b, t-(K-1)+j, c] with zeros before the sequence start
    (nn.Conv1d(groups=C, padding=K-1)(x)[..., :T], reference/ttt.py:647-663,747-748)."""
    B, T, C = x.shape
    K = weight.shape[-1]
    w = weight.reshape(C, K)
    xp = torch.cat((x.new_zeros(B, K - 1, C), x), dim=1)
    y = bias.reshape(1, 1, C).expand(B, T, C).clone()
    for j in range(K):
        y = y + xp[:, j:j + T, :] * w[:, j].reshape(1, 1, C)
    return y


def layer_prologue(x, p: Dict[str, torch.Tensor], *, num_heads: int, mini_batch: int = 16, base_lr: float = 1.0,
                   rope_theta: float = 10000.0, share_qk: bool = False, start_idx: int = 0):
    """Hidden states [B,T,C] -> inner-loop operands: XQ, XK, XV [B,H,T,F], ttt_lr_eta [B,H,T], token_eta [T]
    (rust/layer/src/ttt.rs:152-267)."""
    B, T, C = x.shape
    H = num_heads
    F = C // H
    xv = x @ p["v_proj"].T
    if share_qk:
        xqk = x @ p["q_proj"].T
        xq = causal_depthwise_conv(xqk, p["conv_q_weight"], p["conv_q_bias"])
        xk = causal_depthwise_conv(xqk, p["conv_k_weight"], p["conv_k_bias"])
    else:
        xq = x @ p["q_proj"].T
        xk = x @ p["k_proj"].T
    xq, xk, xv = (t.reshape(B, T, H, F).permute(0, 2, 1, 3) for t in (xq, xk, xv))
    pos = (start_idx + torch.arange(T)) % mini_batch
    xq = rope_pairs(xq, pos, rope_theta)
    xk = rope_pairs(xk, pos, rope_theta)
    logits = torch.einsum("btc,hc->bht", x, p["lr_weight"].reshape(H, C)) + p["lr_bias"].reshape(1, H, 1)
    lr = base_lr * torch.sigmoid(logits) / F
    te = torch.clamp_min(p["token_idx"] + p["learnable_token_idx"], 0.0)
    token_eta = te.repeat((T + mini_batch - 1) // mini_batch)[:T]
    return xq.contiguous(), xk.contiguous(), xv.contiguous(), lr.contiguous(), token_eta


def layer_epilogue(inner_out, x, p: Dict[str, torch.Tensor], *, use_gate: bool = False, eps: float = 1e-6):
    """Inner output [B,H,T,F] -> [B,T,C]: head merge, post LayerNorm over C, optional gelu(tanh) gate
    (rust/layer/src/ttt.rs:285-296), before the output projection."""
    B, H, T, F = inner_out.shape
    y = inner_out.permute(0, 2, 1, 3).reshape(B, T, H * F)
    mu = y.mean(dim=-1, keepdim=True)
    var = ((y - mu) ** 2).mean(dim=-1, keepdim=True)
    y = (y - mu) / torch.sqrt(var + eps) * p["post_norm_weight"] + p["post_norm_bias"]
    if use_gate:
        y = O.gelu_tanh(x @ p["g_proj"].T) * y
    return y


def ttt_layer_forward(x, p: Dict[str, torch.Tensor], *, num_heads: int, mini_batch: int = 16, base_lr: float = 1.0,
                      rope_theta: float = 10000.0, share_qk: bool = False, use_gate: bool = False,
                      start_idx: int = 0, state: Optional[Dict[str, torch.Tensor]] = None, inner: str = "linear"):
    """Whole layer.  inner = "linear": `state` = {"weight" [B,H,F,F], "bias" [B,H,F]} (defaults to the parameters W1,
    b1 repeated over the batch: rust/core/src/linear.rs:84-89); inner = "mlp": `state` = {"w1" [B,H,F,4F], "b1",
    "w2" [B,H,4F,F], "b2"} from the parameters W1, b1, W2, b2 (rust/core/src/mlp.rs:29-53; whole mini-batches only).
    Returns (output [B,T,C], new state)."""
    B, T, C = x.shape
    H = num_heads
    xq, xk, xv, lr, te = layer_prologue(x, p, num_heads=H, mini_batch=mini_batch, base_lr=base_lr,
                                        rope_theta=rope_theta, share_qk=share_qk, start_idx=start_idx)
    if inner == "mlp":
        if state is None:
            state = {"w1": p["W1"].unsqueeze(0).repeat(B, 1, 1, 1), "b1": p["b1"].reshape(1, H, -1).repeat(B, 1, 1),
                     "w2": p["W2"].unsqueeze(0).repeat(B, 1, 1, 1), "b2": p["b2"].reshape(1, H, -1).repeat(B, 1, 1)}
        r = O.ttt_mlp_forward(xq, xk, xv, state["w1"], state["b1"], state["w2"], state["b2"], te, lr,
                              p["ttt_norm_weight"], p["ttt_norm_bias"], mini_batch=mini_batch, eps=1e-6)
        new_state = {k: r[k] for k in ("w1", "b1", "w2", "b2")}
    else:
        if state is None:
            state = {"weight": p["W1"].unsqueeze(0).repeat(B, 1, 1, 1), "bias": p["b1"].reshape(1, H, -1).repeat(B, 1, 1)}
        r = O.ttt_linear_forward_any_length(xq, xk, xv, state["weight"], state["bias"], te, lr, p["ttt_norm_weight"],
                                            p["ttt_norm_bias"], mini_batch=mini_batch, eps=1e-6)
        new_state = {"weight": r["weight"], "bias": r["bias"]}
    y = layer_epilogue(r["output"], x, p, use_gate=use_gate)
    return y @ p["o_proj"].T, new_state
