"""Pins the CPU oracle against fixtures produced by the reference's own PyTorch module
(tests/golden/make_golden.py).  No GPU needed."""

import numpy as np
import pytest
import torch

from oracle import ttt_oracle as O
from conftest import assert_close


def _load(path):
    z = np.load(path)
    return {k: torch.from_numpy(z[k]) for k in z.files}


def test_ln_matches_reference_validate_cases(golden_dir):
    d = _load(golden_dir / "validate_ln.npz")
    H, D = 4, 16
    gamma = torch.ones(1, H, 1, D)
    beta = torch.zeros(1, H, 1, D)
    # tolerances of rust/cli/tests/validate_full.rs:591,624 are 1e-4; the restatement is far inside
    assert_close(O.ln_fwd(d["ln_fwd_x"], gamma, beta, 1e-6), d["ln_fwd_result"], 1e-6, "ln_fwd")
    assert_close(O.ln_l2_grad(d["ln_fused_x"], d["ln_fused_target"], gamma, beta, 1e-6),
                 d["ln_fused_result"], 1e-5, "ln_fused_l2_bwd")


def test_linear_matches_reference_validate_case(golden_dir):
    d = _load(golden_dir / "validate_ttt_linear.npz")
    r = O.ttt_linear_forward(d["xq"], d["xk"], d["xv"], d["W1_init"], d["b1_init"], d["token_eta"],
                             d["ttt_lr_eta"], d["ln_weight"], d["ln_bias"], mini_batch=16, eps=1e-6)
    # reference's own tolerance for this case is 2e-3 (validate_full.rs:104-106); the case is float32 with
    # identical rows (constant q/k/v), so LN divides by a small sigma and float32 op order shows at ~1e-4
    assert_close(r["output"], d["output_expected"], 5e-4, "output")
    assert_close(r["weight"], d["W1_last_expected"], 5e-4, "W1_last")
    assert_close(r["bias"], d["b1_last_expected"], 5e-4, "b1_last")


def test_mlp_matches_reference_validate_case(golden_dir):
    d = _load(golden_dir / "validate_ttt_mlp.npz")
    r = O.ttt_mlp_forward(d["xq"], d["xk"], d["xv"], d["W1_init"], d["b1_init"], d["W2_init"], d["b2_init"],
                          d["token_eta"], d["ttt_lr_eta"], d["ln_weight"], d["ln_bias"], mini_batch=16, eps=1e-6)
    assert_close(r["output"], d["output_expected"], 5e-4, "output")
    for k, e in (("w1", "W1"), ("b1", "b1"), ("w2", "W2"), ("b2", "b2")):
        assert_close(r[k], d[f"{e}_last_expected"], 5e-4, e)


LIN_IN = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")


def test_linear_forward_and_backward_match_reference_f64(golden_dir):
    d = _load(golden_dir / "linear_small_f64.npz")
    args = [d["in_" + k] for k in LIN_IN]
    fw = O.ttt_linear_forward(*args, mini_batch=16, eps=1e-6, checkpoint_interval=2)
    assert_close(fw["output"], d["output"], 1e-11, "output")
    assert_close(fw["weight"], d["final_W1"], 1e-11, "final W")
    assert_close(fw["bias"], d["final_b1"], 1e-11, "final b")
    for fn in (O.ttt_linear_backward, O.ttt_linear_backward_autograd):
        bw = fn(*args, d["in_grad_output"], mini_batch=16, eps=1e-6)
        for name in ("xq", "xk", "xv", "weight", "bias", "ttt_lr_eta", "token_eta", "ln_weight", "ln_bias"):
            assert_close(bw["grad_" + name], d["grad_" + name], 1e-9, f"{fn.__name__}: grad_{name}")


def test_linear_checkpoint_layout():
    t = O.make_inputs(2, 3, 96, 64, 16, seed=5, dtype=torch.float64)
    args = [t[k] for k in LIN_IN]
    K = 4  # 6 stages -> checkpoints before stages 0 and 4
    fw = O.ttt_linear_forward(*args, checkpoint_interval=K)
    assert fw["weight_checkpoints"].shape == (2 * 3 * 2, 64, 64)
    assert fw["bias_checkpoints"].shape == (2 * 3 * 2, 64)
    ck = fw["weight_checkpoints"].reshape(2, 3, 2, 64, 64)
    assert torch.equal(ck[:, :, 0], t["weight"])
    # the second checkpoint is the state after 4 stages = final state of a 64-token prefix
    pre = O.ttt_linear_forward(*[a[:, :, :64] if a.dim() >= 3 and a.shape[2] == 96 else a for a in args])
    assert_close(ck[:, :, 1], pre["weight"], 1e-12, "checkpoint 1")


def test_token_eta_is_read_from_first_mini_batch_only():
    t = O.make_inputs(1, 2, 64, 64, 16, seed=6, dtype=torch.float64)
    args = {k: t[k] for k in LIN_IN}
    a = O.ttt_linear_forward(**args)
    te = args["token_eta"].clone()
    te[16:] = 123.0  # entries past the first mini-batch must not matter
    b = O.ttt_linear_forward(**{**args, "token_eta": te})
    assert torch.equal(a["output"], b["output"])


def test_mlp_forward_and_grads_match_reference_f64(golden_dir):
    d = _load(golden_dir / "mlp_small_f64.npz")
    names = ("xq", "xk", "xv", "w1", "b1", "w2", "b2", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")
    leaves = {k: d["in_" + k].clone().requires_grad_(k != "token_eta") for k in names}
    fw = O.ttt_mlp_forward(**leaves, mini_batch=16, eps=1e-6)
    # the reference's gelu derivative carries 8-digit constants (reference/ttt.py:509-512), hence 1e-8 not 1e-11
    assert_close(fw["output"], d["output"], 1e-8, "output")
    for k, e in (("w1", "W1"), ("b1", "b1"), ("w2", "W2"), ("b2", "b2")):
        assert_close(fw[k], d["final_" + e], 1e-8, "final " + e)
    wrt = [k for k in names if k != "token_eta"]
    grads = torch.autograd.grad(fw["output"], [leaves[k] for k in wrt], grad_outputs=d["in_grad_output"])
    for k, g in zip(wrt, grads):
        assert_close(g, d["grad_" + k], 1e-7, "grad_" + k)


def test_cfg0_forward_matches_reference(golden_dir):
    z = np.load(golden_dir / "cfg0_linear_f32.npz")
    stride = int(z["stride"])
    t = O.make_inputs(2, 4, 256, 64, 16, seed=0, dtype=torch.float32)
    args = [t[k] for k in LIN_IN]
    r32 = O.ttt_linear_forward(*args)
    r64 = O.ttt_linear_forward(*[a.double() for a in args])
    sub = lambda x: x.reshape(-1)[::stride]
    assert_close(sub(r64["output"]), torch.from_numpy(z["output_f64_sub"]), 1e-10, "output f64")
    assert_close(sub(r64["weight"]), torch.from_numpy(z["final_W1_f64_sub"]), 1e-10, "W f64")
    assert_close(r64["bias"], torch.from_numpy(z["final_b1_f64"]), 1e-10, "b f64")
    # float32: the restatement and the reference order their float ops differently
    assert_close(sub(r32["output"]), torch.from_numpy(z["output_f32_sub"]), 1e-4, "output f32")
    assert abs(r64["output"].sum().item() - float(z["output_f64_sum"])) < 1e-7
    # how far float32 drifts from float64 on this case bounds what a float32 kernel can be asked for
    assert_close(sub(r32["output"]).double(), torch.from_numpy(z["output_f64_sub"]), 1e-4, "output f32 vs f64")


@pytest.mark.parametrize("x", [-3.0, -0.5, 0.0, 0.7, 2.5])
def test_gelu_grad_is_derivative(x):
    xt = torch.tensor([x], dtype=torch.float64, requires_grad=True)
    (g,) = torch.autograd.grad(O.gelu_tanh(xt).sum(), xt)
    assert abs(g.item() - O.gelu_tanh_grad(xt.detach()).item()) < 1e-12
    ref = torch.nn.functional.gelu(xt.detach(), approximate="tanh")
    assert abs(ref.item() - O.gelu_tanh(xt.detach()).item()) < 1e-12


def test_linear_backward_with_final_state_gradients_matches_autograd():
    """Upstream gradients for the returned final state: analytic backward == autograd, and the gradients of a
    sequence equal those of two chunks chained through the state (backward through time in chunks)."""
    t = O.make_inputs(2, 2, 64, 64, 16, seed=8, dtype=torch.float64)
    g = torch.Generator().manual_seed(9)
    gw = torch.randn(t["weight"].shape, generator=g, dtype=torch.float64) * 0.1
    gb = torch.randn(t["bias"].shape, generator=g, dtype=torch.float64) * 0.1
    args = [t[k] for k in LIN_IN]
    a = O.ttt_linear_backward(*args, t["grad_output"], grad_weight_out=gw, grad_bias_out=gb)
    b = O.ttt_linear_backward_autograd(*args, t["grad_output"], grad_weight_out=gw, grad_bias_out=gb)
    for k in a:
        assert_close(a[k], b[k], 1e-9, k)
    # two chunks of 32 tokens
    full = O.ttt_linear_backward(*args, t["grad_output"])
    seq = ("xq", "xk", "xv", "ttt_lr_eta")
    sl = lambda k, lo, hi: t[k][:, :, lo:hi] if k in seq else t[k]
    first = {k: sl(k, 0, 32) for k in LIN_IN}
    f1 = O.ttt_linear_forward(*[first[k] for k in LIN_IN])
    second = {k: sl(k, 32, 64) for k in LIN_IN}
    second["weight"], second["bias"] = f1["weight"], f1["bias"]
    b2 = O.ttt_linear_backward(*[second[k] for k in LIN_IN], t["grad_output"][:, :, 32:])
    b1 = O.ttt_linear_backward(*[first[k] for k in LIN_IN], t["grad_output"][:, :, :32],
                               grad_weight_out=b2["grad_weight"], grad_bias_out=b2["grad_bias"])
    assert_close(torch.cat([b1["grad_xk"], b2["grad_xk"]], dim=2), full["grad_xk"], 1e-9, "chunked grad_xk")
    assert_close(b1["grad_weight"], full["grad_weight"], 1e-9, "chunked grad_weight")
    assert_close(b1["grad_ln_weight"] + b2["grad_ln_weight"], full["grad_ln_weight"], 1e-9, "chunked grad_ln_weight")


def test_mlp_analytic_backward_matches_autograd():
    """The stage-by-stage TTT-MLP backward (the form a fused kernel needs: reverse walk carrying dW1, db1, dW2, db2,
    GELU second derivative, LayerNorm second derivative) against torch autograd over the forward restatement."""
    t = O.make_inputs(2, 2, 48, 64, 16, seed=3, dtype=torch.float64, inner="mlp")
    g = torch.Generator().manual_seed(5)
    t["ln_weight"] = 1 + 0.1 * torch.randn(t["ln_weight"].shape, generator=g, dtype=torch.float64)
    t["ln_bias"] = 0.1 * torch.randn(t["ln_bias"].shape, generator=g, dtype=torch.float64)
    for k in ("b1", "b2"):
        t[k] = 0.05 * torch.randn(t[k].shape, generator=g, dtype=torch.float64)
    t["grad_output"] = torch.randn(t["xq"].shape, generator=g, dtype=torch.float64)
    names = ("xq", "xk", "xv", "w1", "b1", "w2", "b2", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias", "grad_output")
    a = O.ttt_mlp_backward(*[t[k] for k in names])
    b = O.ttt_mlp_backward_autograd(*[t[k] for k in names])
    assert set(a) == set(b)
    for k in a:
        err = (a[k] - b[k]).abs().max().item() / (b[k].abs().max().item() + 1e-300)
        assert err < 1e-11, f"{k}: {err}"
