"""TTT-MLP backward kernel against float64 autograd over the CPU restatement of the reference's inner model."""

import pytest
import torch

from conftest import assert_close
from oracle import ttt_oracle as O

MLP_IN = ("xq", "xk", "xv", "w1", "b1", "w2", "b2", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")


def _case(B, H, T, seed):
    t = O.make_inputs(B, H, T, 64, 16, seed=seed, dtype=torch.bfloat16, inner="mlp")
    g = torch.Generator().manual_seed(seed + 1)
    t["ln_weight"] = (1 + 0.1 * torch.randn(H, 64, generator=g)).to(torch.bfloat16)
    t["ln_bias"] = (0.1 * torch.randn(H, 64, generator=g)).to(torch.bfloat16)
    t["b1"] = (0.05 * torch.randn(B, H, 256, generator=g)).to(torch.bfloat16)
    t["b2"] = (0.05 * torch.randn(B, H, 64, generator=g)).to(torch.bfloat16)
    return t


@pytest.mark.gpu
@pytest.mark.parametrize("B,H,NS", ((1, 1, 1), (2, 3, 4), (1, 2, 12)))
def test_mlp_backward_matches_autograd_of_the_restatement(B, H, NS):
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    t = _case(B, H, NS * 16, 50 + NS)
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, 1)
    d = {k: v.to(dev) for k, v in t.items()}
    g = tb.fused_ttt_mlp_backward(d["xq"], d["xk"], d["xv"], tb.TTTMLPState(d["w1"], d["b1"], d["w2"], d["b2"]),
                                  d["token_eta"], d["ttt_lr_eta"], d["ln_weight"], d["ln_bias"], d["grad_output"], cfg)
    torch.cuda.synchronize()
    want = O.ttt_mlp_backward_autograd(*[t[k].double() for k in MLP_IN], t["grad_output"].double())
    fold = lambda x: x.double().cpu().reshape(-1, 16).sum(0)  # noqa: E731  token_eta gradient per position
    for k in ("grad_xq", "grad_xk", "grad_xv", "grad_w1", "grad_b1", "grad_w2", "grad_b2", "grad_ttt_lr_eta",
              "grad_ln_weight", "grad_ln_bias"):
        assert_close(g[k], want[k], 2e-2, k, max_bad_frac=2e-3)
    assert_close(fold(g["grad_token_eta"]), fold(want["grad_token_eta"]), 2e-2, "grad_token_eta (folded)")
