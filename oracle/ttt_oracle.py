"""CPU oracle for the fused TTT inner loop (TEST INFRASTRUCTURE, not product code).

This file restates, in plain torch tensor arithmetic on the CPU, what the
reference computes on the `fused-tile-multi` path, so that the CUDA kernels can
be checked against it.  Only tests, the smoke check and the benchmark's CPU
baseline leg may import it; the product package never does.

Parity status: PINNED.  `tests/test_oracle_golden.py` checks every function here
against fixtures produced by running the reference's own PyTorch module
(`reference/ttt.py`, `TTTLinear.ttt` / `TTTMLP.ttt` plus autograd) and its
`reference/validate.py` cases; the generating script is
`tests/golden/make_golden.py`.

Reference lines each function follows (paths relative to the reference repo):

* `ln_stats`, `ln_fwd`, `ln_l2_grad`      reference/ttt.py:461-505,
                                          rust/core/src/util.rs:141-182
* `ttt_linear_forward`                    rust/core/src/linear.rs:91-149 (one stage),
                                          rust/fused/src/linear_fused_tile/forward/kernel.rs:116-175
                                          (stage loop, checkpoints *before* the update of
                                          stage s when s % K == 0, token_eta read at [0, CS)
                                          in every stage)
* `ttt_linear_backward`                   rust/fused/src/linear_fused_tile/backward/stage.rs:42-1006
                                          (analytic per-stage backward),
                                          backward/kernel.rs:254-429 (reverse stage loop; final-state
                                          gradients are taken as zero, launch.rs:188-194),
                                          backward/launch.rs:351-392 (gradient shapes: per-batch
                                          dW/db, [T] token_eta gradient, [H,F] LN gradients)
* `ttt_mlp_forward`                       rust/core/src/mlp.rs:127-208, reference/ttt.py:1107-1229
* `gelu_tanh`, `gelu_tanh_grad`           rust/thundercube/src/unary_ops.rs:147-173,
                                          reference/ttt.py:509-512

All functions take tensors laid out as the reference's operator does:
xq/xk/xv/out `[B,H,T,F]`, state weight `[B,H,F,F]`, bias `[B,H,F]`,
token_eta `[T]`, ttt_lr_eta `[B,H,T]`, LN weight/bias `[H,F]`.
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

GELU_C0 = 0.7978845608028654  # sqrt(2/pi)
GELU_C1 = 0.044715


# --------------------------------------------------------------------------
# LayerNorm pieces
# --------------------------------------------------------------------------

def ln_stats(x: torch.Tensor, eps: float):
    """Row statistics over the last dim: biased variance, eps inside the sqrt."""
    mu = x.mean(dim=-1, keepdim=True)
    xc = x - mu
    var = (xc * xc).mean(dim=-1, keepdim=True)
    sigma = torch.sqrt(var + eps)
    return xc / sigma, sigma


def ln_fwd(x, gamma, beta, eps: float):
    x_hat, _ = ln_stats(x, eps)
    return gamma * x_hat + beta


def ln_l2_grad(x, target, gamma, beta, eps: float):
    """Gradient of 0.5*||LN(x) - target||^2 w.r.t. x (summed loss, per row)."""
    F = x.shape[-1]
    x_hat, sigma = ln_stats(x, eps)
    gy = gamma * x_hat + beta - target
    gxh = gy * gamma
    g = (F * gxh - gxh.sum(-1, keepdim=True) - x_hat * (gxh * x_hat).sum(-1, keepdim=True)) / (sigma * F)
    return g


def gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(GELU_C0 * x * (1.0 + GELU_C1 * x * x)))


def gelu_tanh_grad(x):
    t = torch.tanh(GELU_C0 * x * (1.0 + GELU_C1 * x * x))
    return 0.5 * x * ((1.0 - t * t) * (GELU_C0 + 3.0 * GELU_C0 * GELU_C1 * x * x)) + 0.5 * (1.0 + t)


# --------------------------------------------------------------------------
# TTT-Linear forward
# --------------------------------------------------------------------------

def _stage_views(x: torch.Tensor, cs: int):
    B, H, T = x.shape[:3]
    return x.reshape(B, H, T // cs, cs, *x.shape[3:])


def _eta_matrices(token_eta_cs: torch.Tensor, lr_stage: torch.Tensor):
    """eta[i,j] = token_eta[i] * lr[j] for j <= i (diagonal included), else 0."""
    eta = token_eta_cs.view(1, 1, -1, 1) * lr_stage.unsqueeze(-2)  # [B,H,CS,CS]
    return torch.tril(eta)


def ttt_linear_forward(
    xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias,
    mini_batch: int = 16, eps: float = 1e-6, checkpoint_interval: int = 1,
) -> Dict[str, torch.Tensor]:
    """Whole-sequence forward scan.

    Returns dict(output [B,H,T,F], weight [B,H,F,F], bias [B,H,F],
    weight_checkpoints [B*H*ceil(NS/K),F,F], bias_checkpoints [B*H*ceil(NS/K),F]).
    """
    B, H, T, F = xq.shape
    cs = mini_batch
    if T % cs != 0:
        raise ValueError(f"seq_len ({T}) must be divisible by mini_batch_len ({cs})")
    ns = T // cs
    K = checkpoint_interval
    nck = (ns + K - 1) // K
    W = weight.clone()
    b = bias.clone()
    g_ = ln_weight.view(1, H, 1, F)
    be_ = ln_bias.view(1, H, 1, F)
    te = token_eta[:cs]
    q_s, k_s, v_s = (_stage_views(t, cs) for t in (xq, xk, xv))
    lr_s = _stage_views(ttt_lr_eta, cs)
    out = torch.empty_like(xq).reshape(B, H, ns, cs, F)
    w_ck = torch.empty(B, H, nck, F, F, dtype=W.dtype)
    b_ck = torch.empty(B, H, nck, F, dtype=W.dtype)
    for s in range(ns):
        if s % K == 0:
            w_ck[:, :, s // K] = W
            b_ck[:, :, s // K] = b
        Q, Kk, V, lr = q_s[:, :, s], k_s[:, :, s], v_s[:, :, s], lr_s[:, :, s]
        z1 = Kk @ W + b.unsqueeze(-2)
        G = ln_l2_grad(z1, V - Kk, g_, be_, eps)
        eta = _eta_matrices(te, lr)
        attn = torch.tril(Q @ Kk.transpose(-1, -2))
        zbar = Q @ W + b.unsqueeze(-2) - (eta * (1.0 + attn)) @ G
        out[:, :, s] = Q + ln_fwd(zbar, g_, be_, eps)
        last = (te[cs - 1] * lr).unsqueeze(-1)  # [B,H,CS,1]
        W = W - (last * Kk).transpose(-1, -2) @ G
        b = b - (last * G).sum(dim=-2)
    return {
        "output": out.reshape(B, H, T, F),
        "weight": W,
        "bias": b,
        "weight_checkpoints": w_ck.reshape(B * H * nck, F, F),
        "bias_checkpoints": b_ck.reshape(B * H * nck, F),
    }


# --------------------------------------------------------------------------
# TTT-Linear analytic backward
# --------------------------------------------------------------------------

def ttt_linear_forward_any_length(xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias,
                                  mini_batch: int = 16, eps: float = 1e-6) -> Dict[str, torch.Tensor]:
    """Sequences whose length is not a multiple of the mini-batch, as the inner-model trait's default `forward`
    handles them (rust/core/src/inner.rs:25-50): the whole mini-batches first, then ONE `forward_mini_batch` on the
    remainder, which is thereby a mini-batch of its own length with eta[i][j] = token_eta[L+i] * lr[L+j].
    A 1-token call (decode) is the case L = 0, remainder 1.  Returns dict(output, weight, bias)."""
    T = xq.shape[2]
    L = (T // mini_batch) * mini_batch
    outs = []
    W, b = weight, bias
    if L > 0:
        r = ttt_linear_forward(xq[:, :, :L], xk[:, :, :L], xv[:, :, :L], W, b, token_eta[:L], ttt_lr_eta[:, :, :L],
                               ln_weight, ln_bias, mini_batch=mini_batch, eps=eps)
        outs.append(r["output"])
        W, b = r["weight"], r["bias"]
    if T > L:
        r = ttt_linear_forward(xq[:, :, L:], xk[:, :, L:], xv[:, :, L:], W, b, token_eta[L:T], ttt_lr_eta[:, :, L:],
                               ln_weight, ln_bias, mini_batch=T - L, eps=eps)
        outs.append(r["output"])
        W, b = r["weight"], r["bias"]
    return {"output": torch.cat(outs, dim=2), "weight": W, "bias": b}


def _stage_states(xk, xv, weight, bias, te, lr_s, g_, be_, cs, eps):
    """Re-simulate the state (W_s, b_s) seen at the start of every stage."""
    B, H, T, F = xk.shape
    ns = T // cs
    k_s, v_s = _stage_views(xk, cs), _stage_views(xv, cs)
    W, b = weight.clone(), bias.clone()
    Ws, bs = [], []
    for s in range(ns):
        Ws.append(W)
        bs.append(b)
        Kk, V, lr = k_s[:, :, s], v_s[:, :, s], lr_s[:, :, s]
        G = ln_l2_grad(Kk @ W + b.unsqueeze(-2), V - Kk, g_, be_, eps)
        last = (te[cs - 1] * lr).unsqueeze(-1)
        W = W - (last * Kk).transpose(-1, -2) @ G
        b = b - (last * G).sum(dim=-2)
    return Ws, bs


def ttt_linear_backward(
    xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias, grad_output,
    mini_batch: int = 16, eps: float = 1e-6,
    grad_weight_out: Optional[torch.Tensor] = None, grad_bias_out: Optional[torch.Tensor] = None,
) -> Dict[str, torch.Tensor]:
    """Analytic backward of `ttt_linear_forward` for loss = <grad_output, output>
    (+ <grad_weight_out, final weight> + <grad_bias_out, final bias> when those are given).

    By default gradients w.r.t. the returned final state are taken as zero, as the
    reference's backward does (rust/fused/src/linear_fused_tile/launch.rs:188-194).  Returns dict with
    grad_xq/xk/xv [B,H,T,F], grad_weight [B,H,F,F] (per batch element),
    grad_bias [B,H,F], grad_ttt_lr_eta [B,H,T], grad_token_eta [T]
    (written per stage at stage*CS+i, summed over B and H),
    grad_ln_weight / grad_ln_bias [H,F] (summed over B).
    """
    B, H, T, F = xq.shape
    cs = mini_batch
    ns = T // cs
    g_ = ln_weight.view(1, H, 1, F)
    be_ = ln_bias.view(1, H, 1, F)
    te = token_eta[:cs]
    te_col = te.view(1, 1, cs, 1)
    q_s, k_s, v_s, do_s = (_stage_views(t, cs) for t in (xq, xk, xv, grad_output))
    lr_s = _stage_views(ttt_lr_eta, cs)
    Ws, bs = _stage_states(xk, xv, weight, bias, te, lr_s, g_, be_, cs, eps)

    dq = torch.empty_like(xq).reshape(B, H, ns, cs, F)
    dk = torch.empty_like(dq)
    dv = torch.empty_like(dq)
    dlr = torch.empty_like(ttt_lr_eta).reshape(B, H, ns, cs)
    dte = torch.zeros(T, dtype=xq.dtype)
    dgam = torch.zeros(B, H, F, dtype=xq.dtype)
    dbet = torch.zeros(B, H, F, dtype=xq.dtype)
    dW = torch.zeros_like(weight) if grad_weight_out is None else grad_weight_out.clone()
    db = torch.zeros_like(bias) if grad_bias_out is None else grad_bias_out.clone()

    for s in reversed(range(ns)):
        Q, Kk, V, lr, dO = q_s[:, :, s], k_s[:, :, s], v_s[:, :, s], lr_s[:, :, s], do_s[:, :, s]
        W, b = Ws[s], bs[s]
        # ---- recompute forward intermediates
        z1 = Kk @ W + b.unsqueeze(-2)
        xh, sig = ln_stats(z1, eps)
        gy = g_ * xh + be_ - (V - Kk)
        gxh = gy * g_
        sum_gxh = gxh.sum(-1, keepdim=True)
        sum_gxh_xh = (gxh * xh).sum(-1, keepdim=True)
        G = (F * gxh - sum_gxh - xh * sum_gxh_xh) / (sig * F)
        eta = _eta_matrices(te, lr)
        attn = torch.tril(Q @ Kk.transpose(-1, -2))
        M = eta * (1.0 + attn)
        zbar = Q @ W + b.unsqueeze(-2) - M @ G
        xhz, sigz = ln_stats(zbar, eps)
        ell = te[cs - 1] * lr  # [B,H,CS]
        ell_c = ell.unsqueeze(-1)
        # ---- 1. LN backward of the output
        dgam += (dO * xhz).sum(-2)
        dbet += dO.sum(-2)
        t = dO * g_
        dzbar = (F * t - t.sum(-1, keepdim=True) - xhz * (t * xhz).sum(-1, keepdim=True)) / (sigz * F)
        # ---- 2. direct W/b terms from Q@W + b
        dW_acc = dW + Q.transpose(-1, -2) @ dzbar
        db_acc = db + dzbar.sum(-2)
        # ---- 3. eta / attention terms
        P = dzbar @ G.transpose(-1, -2)
        dM = -torch.tril(P)
        dA = dM * eta
        deta = dM * (1.0 + attn)
        dq_inner = dzbar @ W.transpose(-1, -2) + dA @ Kk
        dk_attn = dA.transpose(-1, -2) @ Q
        # ---- 4. gradient reaching G
        dG = -(M.transpose(-1, -2) @ dzbar) - (ell_c * Kk) @ dW - ell_c * db.unsqueeze(-2)
        # ---- 5. last-eta-row terms of the state update
        Gl = G @ dW.transpose(-1, -2)
        dell = -((Gl * Kk).sum(-1) + (G * db.unsqueeze(-2)).sum(-1))  # [B,H,CS]
        dk_upd = -ell_c * Gl
        # ---- 6. eta factor gradients
        dte_stage = (deta * lr.unsqueeze(-2)).sum(-1)  # [B,H,CS] (row i)
        dte_stage[..., cs - 1] += (dell * lr).sum(-1)
        dlr_stage = (deta * te_col).sum(-2) + dell * te[cs - 1]
        dte[s * cs:(s + 1) * cs] = dte_stage.sum(dim=(0, 1))
        dlr[:, :, s] = dlr_stage
        # ---- 7. second derivative through the LN + L2 gradient
        u = dG
        v = -u / sig
        s1 = v.sum(-1, keepdim=True)
        s2 = (v * xh).sum(-1, keepdim=True)
        dgxh = u / sig + s1 / F + xh * s2 / F
        dy = g_ * dgxh
        dgam += (gy * dgxh + dy * xh).sum(-2)
        dbet += dy.sum(-2)
        dxh = dy * g_ + gxh * s2 / F + v * sum_gxh_xh / F
        S = (-(dxh * xh + u * G) / sig).sum(-1, keepdim=True)
        dz1 = dxh / sig - dxh.sum(-1, keepdim=True) / (sig * F) + xh * S / F
        dT = -g_ * dgxh
        # ---- 8. assemble
        dq[:, :, s] = dO + dq_inner
        dv[:, :, s] = dT
        dk[:, :, s] = -dT + dk_attn + dk_upd + dz1 @ W.transpose(-1, -2)
        dW = dW_acc + Kk.transpose(-1, -2) @ dz1
        db = db_acc + dz1.sum(-2)

    return {
        "grad_xq": dq.reshape(B, H, T, F),
        "grad_xk": dk.reshape(B, H, T, F),
        "grad_xv": dv.reshape(B, H, T, F),
        "grad_weight": dW,
        "grad_bias": db,
        "grad_ttt_lr_eta": dlr.reshape(B, H, T),
        "grad_token_eta": dte,
        "grad_ln_weight": dgam.sum(0),
        "grad_ln_bias": dbet.sum(0),
    }


def ttt_linear_backward_autograd(
    xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias, grad_output,
    mini_batch: int = 16, eps: float = 1e-6,
    grad_weight_out: Optional[torch.Tensor] = None, grad_bias_out: Optional[torch.Tensor] = None,
) -> Dict[str, torch.Tensor]:
    """Same contract as `ttt_linear_backward`, via torch autograd over the forward
    restatement.  Used to cross-check the analytic backward.

    `token_eta` is treated the way the layer builds it (one `[CS]` base vector
    tiled to `[T]`, rust/layer/src/ttt.rs:253-256), so its gradient is reported
    per stage position like the fused kernel writes it.
    """
    cs = mini_batch
    T = xq.shape[2]
    ns = T // cs
    leaves = [t.detach().clone().requires_grad_(True)
              for t in (xq, xk, xv, weight, bias, ttt_lr_eta, ln_weight, ln_bias)]
    q, k, v, w, b, lr, g, be = leaves
    te_full = token_eta[:cs].detach().repeat(ns).clone().requires_grad_(True)
    B, H, _, F = q.shape
    g_ = g.view(1, H, 1, F)
    be_ = be.view(1, H, 1, F)
    W, bb = w, b
    outs = []
    for s in range(ns):
        sl = slice(s * cs, (s + 1) * cs)
        Q, Kk, V, lrs, te = q[:, :, sl], k[:, :, sl], v[:, :, sl], lr[:, :, sl], te_full[sl]
        z1 = Kk @ W + bb.unsqueeze(-2)
        G = ln_l2_grad(z1, V - Kk, g_, be_, eps)
        eta = torch.tril(te.view(1, 1, cs, 1) * lrs.unsqueeze(-2))
        attn = torch.tril(Q @ Kk.transpose(-1, -2))
        zbar = Q @ W + bb.unsqueeze(-2) - (eta * (1.0 + attn)) @ G
        outs.append(Q + ln_fwd(zbar, g_, be_, eps))
        last = eta[:, :, cs - 1, :].unsqueeze(-1)
        W = W - (last * Kk).transpose(-1, -2) @ G
        bb = bb - (last * G).sum(dim=-2)
    out = torch.cat(outs, dim=2)
    roots, root_grads = [out], [grad_output]
    if grad_weight_out is not None:
        roots.append(W)
        root_grads.append(grad_weight_out)
    if grad_bias_out is not None:
        roots.append(bb)
        root_grads.append(grad_bias_out)
    grads = torch.autograd.grad(roots, leaves + [te_full], grad_outputs=root_grads)
    names = ["grad_xq", "grad_xk", "grad_xv", "grad_weight", "grad_bias",
             "grad_ttt_lr_eta", "grad_ln_weight", "grad_ln_bias", "grad_token_eta"]
    return dict(zip(names, grads))


# --------------------------------------------------------------------------
# TTT-MLP forward (2-layer inner model, GELU tanh)
# --------------------------------------------------------------------------

def ttt_mlp_forward(
    xq, xk, xv, w1, b1, w2, b2, token_eta, ttt_lr_eta, ln_weight, ln_bias,
    mini_batch: int = 16, eps: float = 1e-6,
) -> Dict[str, torch.Tensor]:
    """Whole-sequence TTT-MLP forward scan.  w1 [B,H,F,E], b1 [B,H,E],
    w2 [B,H,E,F], b2 [B,H,F]; differentiable w.r.t. every floating input."""
    B, H, T, F = xq.shape
    cs = mini_batch
    if T % cs != 0:
        raise ValueError(f"seq_len ({T}) must be divisible by mini_batch_len ({cs})")
    ns = T // cs
    g_ = ln_weight.view(1, H, 1, F)
    be_ = ln_bias.view(1, H, 1, F)
    W1, B1, W2, B2 = w1, b1, w2, b2
    outs = []
    for s in range(ns):
        sl = slice(s * cs, (s + 1) * cs)
        Q, Kk, V, lr = xq[:, :, sl], xk[:, :, sl], xv[:, :, sl], ttt_lr_eta[:, :, sl]
        te = token_eta[:cs]
        z1 = Kk @ W1 + B1.unsqueeze(-2)
        x2 = gelu_tanh(z1)
        z2 = x2 @ W2 + B2.unsqueeze(-2)
        g2 = ln_l2_grad(z2, V - Kk, g_, be_, eps)
        g1 = (g2 @ W2.transpose(-1, -2)) * gelu_tanh_grad(z1)
        eta = torch.tril(te.view(1, 1, cs, 1) * lr.unsqueeze(-2))
        attn1 = torch.tril(Q @ Kk.transpose(-1, -2))
        z1b = Q @ W1 + B1.unsqueeze(-2) - (eta * (1.0 + attn1)) @ g1
        x2b = gelu_tanh(z1b)
        attn2 = torch.tril(x2b @ x2.transpose(-1, -2))
        z2b = x2b @ W2 + B2.unsqueeze(-2) - (eta * (1.0 + attn2)) @ g2
        outs.append(Q + ln_fwd(z2b, g_, be_, eps))
        last = eta[:, :, cs - 1, :].unsqueeze(-1)
        W1 = W1 - (last * Kk).transpose(-1, -2) @ g1
        B1 = B1 - (last * g1).sum(dim=-2)
        W2 = W2 - (last * x2).transpose(-1, -2) @ g2
        B2 = B2 - (last * g2).sum(dim=-2)
    return {"output": torch.cat(outs, dim=2), "w1": W1, "b1": B1, "w2": W2, "b2": B2}


def gelu_tanh_grad2(x):
    """Second derivative of the tanh-form GELU."""
    u = GELU_C0 * x * (1.0 + GELU_C1 * x * x)
    t = torch.tanh(u)
    du = GELU_C0 * (1.0 + 3.0 * GELU_C1 * x * x)
    d2u = 6.0 * GELU_C0 * GELU_C1 * x
    return (1.0 - t * t) * du + 0.5 * x * (1.0 - t * t) * (d2u - 2.0 * t * du * du)


def _ln_l2_grad_backward(u, z, target, g_, be_, eps):
    """Backward of G = ln_l2_grad(z, target): given u = dL/dG returns (dz, dtarget, dgamma rows, dbeta rows)
    (the second-derivative formulas of rust/fused/src/linear_fused_tile/layer_norm.rs:429-709)."""
    F = z.shape[-1]
    xh, sig = ln_stats(z, eps)
    gy = g_ * xh + be_ - target
    gxh = gy * g_
    sum_gxh_xh = (gxh * xh).sum(-1, keepdim=True)
    G = (F * gxh - gxh.sum(-1, keepdim=True) - xh * sum_gxh_xh) / (sig * F)
    v = -u / sig
    s1 = v.sum(-1, keepdim=True)
    s2 = (v * xh).sum(-1, keepdim=True)
    dgxh = u / sig + s1 / F + xh * s2 / F
    dy = g_ * dgxh
    dgam = (gy * dgxh + dy * xh).sum(-2)
    dbet = dy.sum(-2)
    dxh = dy * g_ + gxh * s2 / F + v * sum_gxh_xh / F
    S = (-(dxh * xh + u * G) / sig).sum(-1, keepdim=True)
    dz = dxh / sig - dxh.sum(-1, keepdim=True) / (sig * F) + xh * S / F
    return dz, -g_ * dgxh, dgam, dbet


def ttt_mlp_backward(
    xq, xk, xv, w1, b1, w2, b2, token_eta, ttt_lr_eta, ln_weight, ln_bias, grad_output,
    mini_batch: int = 16, eps: float = 1e-6,
) -> Dict[str, torch.Tensor]:
    """Analytic backward of `ttt_mlp_forward` for loss = <grad_output, output> (gradients w.r.t. the returned final
    state taken as zero, as the reference's fused operators do).  The reference obtains this gradient from Burn
    autodiff over rust/core/src/mlp.rs:127-208; this is the stage-by-stage form a fused kernel needs: a reverse walk
    over the stages carrying (dW1, db1, dW2, db2).  Returns grad_xq/xk/xv, grad_w1/b1/w2/b2 (per batch element),
    grad_ttt_lr_eta, grad_token_eta [T] (per stage position, summed over B and H), grad_ln_weight/bias [H,F]."""
    B, H, T, F = xq.shape
    cs = mini_batch
    ns = T // cs
    g_ = ln_weight.view(1, H, 1, F)
    be_ = ln_bias.view(1, H, 1, F)
    te = token_eta[:cs]
    te_col = te.view(1, 1, cs, 1)
    q_s, k_s, v_s, do_s = (_stage_views(t, cs) for t in (xq, xk, xv, grad_output))
    lr_s = _stage_views(ttt_lr_eta, cs)
    tr = lambda m: m.transpose(-1, -2)  # noqa: E731

    # states at the start of every stage
    states = []
    W1, B1, W2, B2 = w1, b1, w2, b2
    for s in range(ns):
        states.append((W1, B1, W2, B2))
        Kk, V, lr = k_s[:, :, s], v_s[:, :, s], lr_s[:, :, s]
        z1 = Kk @ W1 + B1.unsqueeze(-2)
        x2 = gelu_tanh(z1)
        g2 = ln_l2_grad(x2 @ W2 + B2.unsqueeze(-2), V - Kk, g_, be_, eps)
        g1 = (g2 @ tr(W2)) * gelu_tanh_grad(z1)
        last = (te[cs - 1] * lr).unsqueeze(-1)
        W1 = W1 - tr(last * Kk) @ g1
        B1 = B1 - (last * g1).sum(-2)
        W2 = W2 - tr(last * x2) @ g2
        B2 = B2 - (last * g2).sum(-2)

    dq = torch.empty_like(xq).reshape(B, H, ns, cs, F)
    dk, dv = torch.empty_like(dq), torch.empty_like(dq)
    dlr = torch.empty_like(ttt_lr_eta).reshape(B, H, ns, cs)
    dte = torch.zeros(T, dtype=xq.dtype)
    dgam = torch.zeros(B, H, F, dtype=xq.dtype)
    dbet = torch.zeros(B, H, F, dtype=xq.dtype)
    dW1, dB1, dW2, dB2 = (torch.zeros_like(t) for t in (w1, b1, w2, b2))

    for s in reversed(range(ns)):
        Q, Kk, V, lr, dO = q_s[:, :, s], k_s[:, :, s], v_s[:, :, s], lr_s[:, :, s], do_s[:, :, s]
        W1, B1, W2, B2 = states[s]
        # ---- recompute the forward intermediates of the stage
        z1 = Kk @ W1 + B1.unsqueeze(-2)
        gp1 = gelu_tanh_grad(z1)
        x2 = gelu_tanh(z1)
        z2 = x2 @ W2 + B2.unsqueeze(-2)
        g2 = ln_l2_grad(z2, V - Kk, g_, be_, eps)
        hmat = g2 @ tr(W2)
        g1 = hmat * gp1
        eta = _eta_matrices(te, lr)
        a1 = torch.tril(Q @ tr(Kk))
        m1 = eta * (1.0 + a1)
        z1b = Q @ W1 + B1.unsqueeze(-2) - m1 @ g1
        x2b = gelu_tanh(z1b)
        a2 = torch.tril(x2b @ tr(x2))
        m2 = eta * (1.0 + a2)
        z2b = x2b @ W2 + B2.unsqueeze(-2) - m2 @ g2
        xhb, sigb = ln_stats(z2b, eps)
        ell_c = (te[cs - 1] * lr).unsqueeze(-1)
        # ---- 1. output LayerNorm
        dgam += (dO * xhb).sum(-2)
        dbet += dO.sum(-2)
        t_ = dO * g_
        dz2b = (F * t_ - t_.sum(-1, keepdim=True) - xhb * (t_ * xhb).sum(-1, keepdim=True)) / (sigb * F)
        # ---- 2. z2b = x2b W2 + b2 - M2 g2
        dx2b = dz2b @ tr(W2)
        nW2 = dW2 + tr(x2b) @ dz2b
        nB2 = dB2 + dz2b.sum(-2)
        dm2 = -torch.tril(dz2b @ tr(g2))
        dg2 = -(tr(m2) @ dz2b)
        da2 = dm2 * eta
        deta = dm2 * (1.0 + a2)
        dx2b = dx2b + da2 @ x2
        dx2 = tr(da2) @ x2b
        # ---- 3./4. x2b = gelu(z1b), z1b = Q W1 + b1 - M1 g1
        dz1b = dx2b * gelu_tanh_grad(z1b)
        dq_in = dz1b @ tr(W1)
        nW1 = dW1 + tr(Q) @ dz1b
        nB1 = dB1 + dz1b.sum(-2)
        dm1 = -torch.tril(dz1b @ tr(g1))
        dg1 = -(tr(m1) @ dz1b)
        da1 = dm1 * eta
        deta = deta + dm1 * (1.0 + a1)
        dq_in = dq_in + da1 @ Kk
        dk_acc = tr(da1) @ Q
        # ---- 5. the four state updates (dW1 ... are the gradients w.r.t. the NEXT stage's state here)
        gl1 = g1 @ tr(dW1)          # [cs, F]
        gl2 = g2 @ tr(dW2)          # [cs, E]
        dg1 = dg1 - (ell_c * Kk) @ dW1 - ell_c * dB1.unsqueeze(-2)
        dg2 = dg2 - (ell_c * x2) @ dW2 - ell_c * dB2.unsqueeze(-2)
        dk_acc = dk_acc - ell_c * gl1
        dx2 = dx2 - ell_c * gl2
        dell = -((gl1 * Kk).sum(-1) + (g1 * dB1.unsqueeze(-2)).sum(-1)
                 + (gl2 * x2).sum(-1) + (g2 * dB2.unsqueeze(-2)).sum(-1))
        # ---- 6. g1 = (g2 W2^T) o gelu'(z1)
        dh = dg1 * gp1
        dz1 = dg1 * hmat * gelu_tanh_grad2(z1)
        dg2 = dg2 + dh @ W2
        nW2 = nW2 + tr(dh) @ g2
        # ---- 7. g2 = d/dz2 of the LayerNorm reconstruction loss
        dz2, dT, dga, dbe = _ln_l2_grad_backward(dg2, z2, V - Kk, g_, be_, eps)
        dgam += dga
        dbet += dbe
        # ---- 8./9./10. z2 = x2 W2 + b2, x2 = gelu(z1), z1 = K W1 + b1
        dx2 = dx2 + dz2 @ tr(W2)
        nW2 = nW2 + tr(x2) @ dz2
        nB2 = nB2 + dz2.sum(-2)
        dz1 = dz1 + dx2 * gp1
        dk_acc = dk_acc + dz1 @ tr(W1)
        nW1 = nW1 + tr(Kk) @ dz1
        nB1 = nB1 + dz1.sum(-2)
        # ---- 11. eta factors
        dte_stage = (deta * lr.unsqueeze(-2)).sum(-1)
        dte_stage[..., cs - 1] += (dell * lr).sum(-1)
        dte[s * cs:(s + 1) * cs] = dte_stage.sum(dim=(0, 1))
        dlr[:, :, s] = (deta * te_col).sum(-2) + dell * te[cs - 1]
        # ---- assemble
        dq[:, :, s] = dO + dq_in
        dv[:, :, s] = dT
        dk[:, :, s] = dk_acc - dT
        dW1, dB1, dW2, dB2 = nW1, nB1, nW2, nB2

    return {
        "grad_xq": dq.reshape(B, H, T, F), "grad_xk": dk.reshape(B, H, T, F), "grad_xv": dv.reshape(B, H, T, F),
        "grad_w1": dW1, "grad_b1": dB1, "grad_w2": dW2, "grad_b2": dB2,
        "grad_ttt_lr_eta": dlr.reshape(B, H, T), "grad_token_eta": dte,
        "grad_ln_weight": dgam.sum(0), "grad_ln_bias": dbet.sum(0),
    }


def ttt_mlp_backward_autograd(
    xq, xk, xv, w1, b1, w2, b2, token_eta, ttt_lr_eta, ln_weight, ln_bias, grad_output,
    mini_batch: int = 16, eps: float = 1e-6,
) -> Dict[str, torch.Tensor]:
    """Same contract as `ttt_mlp_backward`, by torch autograd over `ttt_mlp_forward` (token_eta is a [CS] base
    vector tiled over the stages, so its gradient is reported per stage position)."""
    cs = mini_batch
    T = xq.shape[2]
    ns = T // cs
    leaves = [t.detach().clone().requires_grad_(True)
              for t in (xq, xk, xv, w1, b1, w2, b2, ttt_lr_eta, ln_weight, ln_bias)]
    q, k, v, W1, B1, W2, B2, lr, g, be = leaves
    te_full = token_eta[:cs].detach().repeat(ns).clone().requires_grad_(True)
    outs = []
    for s in range(ns):
        sl = slice(s * cs, (s + 1) * cs)
        r = ttt_mlp_forward(q[:, :, sl], k[:, :, sl], v[:, :, sl], W1, B1, W2, B2, te_full[sl], lr[:, :, sl], g, be,
                            mini_batch=cs, eps=eps)
        outs.append(r["output"])
        W1, B1, W2, B2 = r["w1"], r["b1"], r["w2"], r["b2"]
    out = torch.cat(outs, dim=2)
    grads = torch.autograd.grad(out, leaves + [te_full], grad_outputs=grad_output)
    names = ("grad_xq", "grad_xk", "grad_xv", "grad_w1", "grad_b1", "grad_w2", "grad_b2", "grad_ttt_lr_eta",
             "grad_ln_weight", "grad_ln_bias", "grad_token_eta")
    return dict(zip(names, grads))


# --------------------------------------------------------------------------
# Synthetic inputs: the seeded generator lives with the product (the benchmark
# uses it too); re-exported here because every parity test feeds the oracle and
# the kernels from it.
# --------------------------------------------------------------------------
from ttt_rs_b200.synthetic import make_inputs  # noqa: E402,F401
