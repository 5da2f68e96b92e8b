"""Parity of the TTT-MLP forward kernel (bf16) with the CPU oracle, through the C ABI (needs a B200)."""

import pytest
import torch

from conftest import assert_close
from oracle import ttt_oracle as O

pytestmark = pytest.mark.gpu
NAMES = ("xq", "xk", "xv", "w1", "b1", "w2", "b2", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")


@pytest.mark.parametrize("B,H,NS", [(1, 1, 1), (2, 2, 4), (1, 3, 16), (2, 12, 32)])
def test_mlp_forward_matches_oracle(B, H, NS):
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    t = O.make_inputs(B, H, NS * 16, 64, 16, seed=500 + NS, dtype=torch.bfloat16, inner="mlp", with_grad_output=False)
    g = torch.Generator().manual_seed(3)
    t["ln_weight"] = (1.0 + 0.1 * torch.randn(t["ln_weight"].shape, generator=g)).to(torch.bfloat16)
    t["ln_bias"] = (0.1 * torch.randn(t["ln_bias"].shape, generator=g)).to(torch.bfloat16)
    t["b1"] = (0.05 * torch.randn(t["b1"].shape, generator=g)).to(torch.bfloat16)
    t["b2"] = (0.05 * torch.randn(t["b2"].shape, generator=g)).to(torch.bfloat16)
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 256, 1)
    d = {k: t[k].to(dev) for k in NAMES}
    out, st = tb.fused_ttt_mlp_forward(d["xq"], d["xk"], d["xv"], tb.TTTMLPState(d["w1"], d["b1"], d["w2"], d["b2"]),
                                       d["token_eta"], d["ttt_lr_eta"], d["ln_weight"], d["ln_bias"], cfg)
    torch.cuda.synchronize()
    tb.TttTileMultiKernel.check_status()
    ref = O.ttt_mlp_forward(*[t[k].double() for k in NAMES], mini_batch=16, eps=1e-6)
    # bf16 criterion applied statistically.  The 32-stage case has one stream whose inner model is on a sensitive
    # trajectory (one output column grows stage after stage; float32 vs float64 of the oracle itself differ 10x more
    # there than elsewhere), so bf16 operand rounding shows on that column (140 of 786k elements) while every other
    # stream sits at the bf16 storage-rounding floor (relative L2 1.9e-3).
    assert_close(out, ref["output"], 2e-2, "output", max_bad_frac=3.6e-4)  # measured 1.8e-4 on B200
    for k in ("w1", "b1", "w2", "b2"):
        assert_close(getattr(st, k), ref[k], 2e-2, "final " + k, max_bad_frac=1.3e-3)  # measured 6.5e-4 (b2)


def test_mlp_rejects_float32():
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    t = O.make_inputs(1, 1, 16, 64, 16, seed=1, dtype=torch.float32, inner="mlp", with_grad_output=False)
    d = {k: t[k].to(dev) for k in NAMES}
    with pytest.raises(tb.TttError):
        tb.fused_ttt_mlp_forward(d["xq"], d["xk"], d["xv"], tb.TTTMLPState(d["w1"], d["b1"], d["w2"], d["b2"]),
                                 d["token_eta"], d["ttt_lr_eta"], d["ln_weight"], d["ln_bias"],
                                 tb.FusedTttConfig.new(16, 64, 1e-6, 256, 1))
