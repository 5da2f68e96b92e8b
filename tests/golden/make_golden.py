#!/usr/bin/env python3
"""Generate the golden fixtures in this directory by running the reference itself.

Needs the reference checkout (its vendored PyTorch module `reference/ttt.py`) on
disk; pass its root with --reference.  It is run once where that checkout exists and the
resulting .npz files are committed, so the tests never need the checkout.

    python tests/golden/make_golden.py --reference /path/to/ttt-rs

What is produced (all by calling the reference's own `TTTLinear.ttt` /
`TTTMLP.ttt` / `ln_fwd` / `ln_fused_l2_bwd`, gradients by torch autograd):

* validate_ln.npz, validate_ttt_linear.npz, validate_ttt_mlp.npz
    the cases of reference/validate.py:69-124,156-326 (seed 42, B=2 H=4 CS=16 D=16,
    constant q/k/v = 0.1/0.2/0.3) that rust/cli/tests/validate_full.rs checks.
* linear_small_f64.npz
    B=1 H=2 T=64 F=64 CS=16, random inputs with non-trivial LN weight/bias and
    initial bias, float64: outputs, final state and all nine gradients.
* mlp_small_f64.npz
    same shape for the 2-layer inner model: outputs, final state, gradients.
* cfg0_linear_f32.npz
    the CPU-runnable benchmark configuration (B=2 H=4 T=256 F=64, seed-0 inputs
    from oracle.ttt_oracle.make_inputs): reference float32 and float64 outputs,
    stored as a strided subsample plus full-tensor sums (inputs are regenerated
    from the seed by the tests).
* layer_linear_f64.npz
    the whole outer layer (`TTTLinear.forward`: projections, optional shared-QK causal
    convolutions, rotary embedding, learning-rate gate, inner loop, post norm, optional
    gate, output projection; the analogue of reference/validate.py:338-415 at head_dim 64):
    B=2 T=48 H=2 F=64, float64, for the default configuration and for share_qk + use_gate, plus
    (tag "mlp") the default configuration with the 2-layer inner model (`TTTMLP.forward`).
    Inputs, every parameter and the expected output are stored.
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))

from oracle.ttt_oracle import make_inputs  # noqa: E402


def _module(ref, kind: str, H: int, F: int, cs: int, dtype):
    cfg = ref.TTTConfig(hidden_size=H * F, num_attention_heads=H, mini_batch_size=cs,
                        ttt_layer_type=kind, ttt_base_lr=1.0)
    cls = ref.TTTLinear if kind == "linear" else ref.TTTMLP
    m = cls(cfg, layer_idx=0)
    m.eval()
    return m.to(dtype)


def _run_ref(ref, kind, t, cs, dtype, want_grads):
    """Run reference .ttt() with per-batch initial states and (optionally) autograd."""
    B, H, T, F = t["xq"].shape
    ns = T // cs
    m = _module(ref, kind, H, F, cs, dtype)
    leaves = {k: v.detach().clone().to(dtype).requires_grad_(want_grads) for k, v in t.items()
              if k not in ("grad_output", "token_eta")}
    te_full = t["token_eta"][:cs].to(dtype).repeat(ns).clone().requires_grad_(want_grads)
    with torch.no_grad():
        pass
    # LN parameters live on the module; route our leaves through them.
    m.ttt_norm_weight = torch.nn.Parameter(leaves["ln_weight"].detach().clone())
    m.ttt_norm_bias = torch.nn.Parameter(leaves["ln_bias"].detach().clone())
    ln_w, ln_b = m.ttt_norm_weight, m.ttt_norm_bias

    def stg(x):
        return x.reshape(B, H, ns, cs, *x.shape[3:])

    token_eta = te_full.reshape(1, 1, ns, cs, 1).expand(B, H, ns, cs, 1)
    lr = stg(leaves["ttt_lr_eta"]).unsqueeze(-2)  # [B,H,ns,1,cs]
    inputs = {"XQ": stg(leaves["xq"]), "XK": stg(leaves["xk"]), "XV": stg(leaves["xv"]),
              "eta": token_eta * lr, "token_eta": token_eta, "ttt_lr_eta": lr}
    if kind == "linear":
        init = {"W1_states": leaves["weight"], "b1_states": leaves["bias"].unsqueeze(-2)}
        init["W1_grad"] = torch.zeros_like(init["W1_states"])
        init["b1_grad"] = torch.zeros_like(init["b1_states"])
    else:
        init = {"W1_states": leaves["w1"], "b1_states": leaves["b1"].unsqueeze(-2),
                "W2_states": leaves["w2"], "b2_states": leaves["b2"].unsqueeze(-2)}
        for k in ("W1", "b1", "W2", "b2"):
            init[f"{k}_grad"] = torch.zeros_like(init[f"{k}_states"])
    out, last = m.ttt(inputs, mini_batch_size=cs, last_mini_batch_params_dict=init, cache_params=None)
    out = out.reshape(B, T, H, F).transpose(1, 2)  # [B,H,T,F]
    res = {"output": out.detach()}
    for k, v in last.items():
        if k.endswith("_states"):
            vv = v.detach()
            res["final_" + k[:-7]] = vv.squeeze(-2) if k.startswith("b") else vv
    if want_grads:
        names = [k for k in leaves if k not in ("ln_weight", "ln_bias")]
        wrt = [leaves[k] for k in names] + [ln_w, ln_b, te_full]
        grads = torch.autograd.grad(out, wrt, grad_outputs=t["grad_output"].to(dtype))
        for k, gval in zip(names + ["ln_weight", "ln_bias", "token_eta"], grads):
            res["grad_" + k] = gval.detach()
    return res


def _np(d):
    return {k: v.detach().cpu().numpy() for k, v in d.items()}


def gen_validate(ref, out_dir: Path):
    """The three fixed cases of reference/validate.py (defaults: seed 42, B2 L16 H4 D16)."""
    B, H, K, D, seed = 2, 4, 16, 16, 42
    torch.manual_seed(seed)
    x = torch.randn(B, H, K, D)
    target = torch.randn(B, H, K, D)
    gamma = torch.ones(H, 1, D)
    beta = torch.zeros(H, 1, D)
    l2 = ref.ln_fused_l2_bwd(x, target, gamma, beta, eps=1e-6)
    torch.manual_seed(seed)
    x2 = torch.randn(B, H, K, D)
    fw = ref.ln_fwd(x2, gamma, beta, eps=1e-6)
    np.savez(out_dir / "validate_ln.npz", ln_fused_x=x.numpy(), ln_fused_target=target.numpy(),
             ln_fused_result=l2.numpy(), ln_fwd_x=x2.numpy(), ln_fwd_result=fw.numpy())

    for kind in ("linear", "mlp"):
        torch.manual_seed(seed)
        cfg = ref.TTTConfig(hidden_size=H * D, num_attention_heads=H, mini_batch_size=K,
                            ttt_layer_type=kind, ttt_base_lr=1.0)
        m = (ref.TTTLinear if kind == "linear" else ref.TTTMLP)(cfg, layer_idx=0)
        m.eval()
        XQ = torch.full((B, H, 1, K, D), 0.1)
        XK = torch.full((B, H, 1, K, D), 0.2)
        XV = torch.full((B, H, 1, K, D), 0.3)
        X = torch.randn(B, 1, K, H * D)
        with torch.no_grad():
            token_eta, ttt_lr_eta = m.get_eta(X, mini_batch_step_offset=0, mini_batch_size=K)
            inputs = {"XQ": XQ, "XK": XK, "XV": XV, "eta": token_eta * ttt_lr_eta,
                      "token_eta": token_eta, "ttt_lr_eta": ttt_lr_eta}
            out, last = m.ttt(inputs, mini_batch_size=K, last_mini_batch_params_dict=None, cache_params=None)
        d = {
            "xq": XQ[:, :, 0], "xk": XK[:, :, 0], "xv": XV[:, :, 0],
            "token_eta": (m.token_idx + m.learnable_token_idx).detach(),
            "ttt_lr_eta": ttt_lr_eta[:, :, 0, 0, :],
            "ln_weight": m.ttt_norm_weight.detach(), "ln_bias": m.ttt_norm_bias.detach(),
            "output_expected": out.reshape(B, K, H, D).transpose(1, 2),
        }
        names = ("W1", "b1") if kind == "linear" else ("W1", "b1", "W2", "b2")
        for n in names:
            p = getattr(m, n).detach().unsqueeze(0).expand(B, *getattr(m, n).shape)
            d[f"{n}_init"] = p.squeeze(-2) if n.startswith("b") else p
            lv = last[f"{n}_states"].detach()
            d[f"{n}_last_expected"] = lv.squeeze(-2) if n.startswith("b") else lv
        np.savez(out_dir / f"validate_ttt_{kind}.npz", **{k: v.contiguous().numpy() for k, v in d.items()})


def gen_small(ref, out_dir: Path):
    for kind in ("linear", "mlp"):
        t = make_inputs(1, 2, 64, 64, 16, seed=1234, dtype=torch.float64, inner=kind)
        g = torch.Generator().manual_seed(99)
        # non-trivial LN parameters and initial biases so every gradient path is exercised
        t["ln_weight"] = 1.0 + 0.1 * torch.randn(t["ln_weight"].shape, generator=g, dtype=torch.float64)
        t["ln_bias"] = 0.1 * torch.randn(t["ln_bias"].shape, generator=g, dtype=torch.float64)
        for bname in ("bias", "b1", "b2"):
            if bname in t:
                t[bname] = 0.05 * torch.randn(t[bname].shape, generator=g, dtype=torch.float64)
        t["grad_output"] = torch.randn(t["xq"].shape, generator=g, dtype=torch.float64)
        res = _run_ref(ref, kind, t, 16, torch.float64, want_grads=True)
        np.savez(out_dir / f"{kind}_small_f64.npz", **_np({**{"in_" + k: v for k, v in t.items()}, **res}))


def gen_cfg0(ref, out_dir: Path):
    t = make_inputs(2, 4, 256, 64, 16, seed=0, dtype=torch.float32, inner="linear")
    r32 = _run_ref(ref, "linear", t, 16, torch.float32, want_grads=False)
    r64 = _run_ref(ref, "linear", t, 16, torch.float64, want_grads=False)
    stride = 61
    d = {"stride": np.int64(stride)}
    for tag, r in (("f32", r32), ("f64", r64)):
        d[f"output_{tag}_sub"] = r["output"].reshape(-1)[::stride].numpy()
        d[f"output_{tag}_sum"] = np.float64(r["output"].double().sum().item())
        d[f"output_{tag}_sqsum"] = np.float64((r["output"].double() ** 2).sum().item())
        d[f"final_W1_{tag}_sub"] = r["final_W1"].reshape(-1)[::stride].numpy()
        d[f"final_b1_{tag}"] = r["final_b1"].numpy()
    np.savez(out_dir / "cfg0_linear_f32.npz", **d)


def gen_layer(ref, out_dir: Path):
    B, T, H, D, cs = 2, 48, 2, 64, 16
    d = {}
    for tag, share_qk, use_gate, kind in (("plain", False, False, "linear"), ("conv_gate", True, True, "linear"),
                                          ("mlp", False, False, "mlp")):
        torch.manual_seed({"plain": 5, "conv_gate": 7, "mlp": 9}[tag])
        cfg = ref.TTTConfig(hidden_size=H * D, num_attention_heads=H, mini_batch_size=cs, ttt_layer_type=kind,
                            ttt_base_lr=1.0, share_qk=share_qk, use_gate=use_gate, conv_kernel=4, pre_conv=False)
        m = (ref.TTTLinear if kind == "linear" else ref.TTTMLP)(cfg, layer_idx=0)
        m.eval()
        with torch.no_grad():  # make every parameter non-trivial
            m.ttt_norm_weight.add_(0.1 * torch.randn_like(m.ttt_norm_weight))
            m.ttt_norm_bias.add_(0.1 * torch.randn_like(m.ttt_norm_bias))
            m.post_norm.weight.add_(0.1 * torch.randn_like(m.post_norm.weight))
            m.post_norm.bias.add_(0.1 * torch.randn_like(m.post_norm.bias))
            m.learnable_ttt_lr_bias.add_(0.1 * torch.randn_like(m.learnable_ttt_lr_bias))
            m.learnable_token_idx.add_(0.05 * torch.randn_like(m.learnable_token_idx))
            m.b1.add_(0.05 * torch.randn_like(m.b1))
            if kind == "mlp":
                m.b2.add_(0.05 * torch.randn_like(m.b2))
        m = m.double()
        x = (torch.randn(B, T, H * D) * 0.5).double()
        pos = torch.arange(T).unsqueeze(0).expand(B, -1)
        with torch.no_grad():
            y = m(hidden_states=x, attention_mask=None, position_ids=pos, cache_params=None)
        t = {
            "input": x, "output_expected": y,
            "q_proj": m.q_proj.weight, "v_proj": m.v_proj.weight, "o_proj": m.o_proj.weight,
            "ttt_norm_weight": m.ttt_norm_weight, "ttt_norm_bias": m.ttt_norm_bias,
            "post_norm_weight": m.post_norm.weight, "post_norm_bias": m.post_norm.bias,
            "lr_weight": m.learnable_ttt_lr_weight, "lr_bias": m.learnable_ttt_lr_bias,
            "token_idx": m.token_idx, "learnable_token_idx": m.learnable_token_idx,
            "W1": m.W1, "b1": m.b1,
        }
        if kind == "mlp":
            t.update(W2=m.W2, b2=m.b2)
        if use_gate:
            t["g_proj"] = m.g_proj.weight
        if share_qk:
            t.update(conv_q_weight=m.conv_q.weight, conv_q_bias=m.conv_q.bias,
                     conv_k_weight=m.conv_k.weight, conv_k_bias=m.conv_k.bias)
        else:
            t["k_proj"] = m.k_proj.weight
        for k, v in t.items():
            d[f"{tag}.{k}"] = v.detach().double().contiguous().numpy()
    np.savez_compressed(out_dir / "layer_linear_f64.npz", **d)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TTT_REFERENCE_ROOT", ""))
    ap.add_argument("--out", default=str(HERE))
    a = ap.parse_args()
    if not a.reference or not (Path(a.reference) / "reference" / "ttt.py").exists():
        sys.exit("pass --reference <checkout root containing reference/ttt.py>")
    sys.path.insert(0, a.reference)
    import reference as ref  # the vendored PyTorch implementation inside the reference repo

    torch.set_grad_enabled(True)
    out_dir = Path(a.out)
    gen_validate(ref, out_dir)
    gen_small(ref, out_dir)
    gen_cfg0(ref, out_dir)
    gen_layer(ref, out_dir)
    for f in sorted(out_dir.glob("*.npz")):
        print(f"{f.name}: {f.stat().st_size} bytes")


if __name__ == "__main__":
    main()
