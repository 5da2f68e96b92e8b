"""Parity of the CUDA forward scan with the CPU oracle, through the C ABI (needs a B200)."""

import numpy as np
import pytest
import torch

from conftest import assert_close
from oracle import ttt_oracle as O

pytestmark = pytest.mark.gpu

LIN_IN = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")
# tolerances named by the benchmark definition: 1e-4 relative for float32, 2e-2 for bfloat16
RTOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def _run(t, K, dtype):
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, K)
    ins = tb.TttInputs(*[t[k].to(dev) for k in LIN_IN])
    outs, saved = tb.TttTileMultiKernel.forward_launch(ins, cfg)
    torch.cuda.synchronize()
    tb.TttTileMultiKernel.check_status()
    return outs, saved


def _oracle(t, K):
    # the oracle consumes the (possibly bf16-rounded) operand values in float64
    args = [t[k].double() for k in LIN_IN]
    return O.ttt_linear_forward(*args, mini_batch=16, eps=1e-6, checkpoint_interval=K)


def _randomise_params(t, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    t["ln_weight"] = (1.0 + 0.1 * torch.randn(t["ln_weight"].shape, generator=g)).to(dtype)
    t["ln_bias"] = (0.1 * torch.randn(t["ln_bias"].shape, generator=g)).to(dtype)
    t["bias"] = (0.05 * torch.randn(t["bias"].shape, generator=g)).to(dtype)
    return t


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,NS,K", [(1, 1, 1, 1), (2, 2, 4, 1), (2, 2, 4, 2), (1, 3, 5, 4), (2, 4, 16, 16)])
def test_forward_matches_oracle(dtype, B, H, NS, K):
    t = O.make_inputs(B, H, NS * 16, 64, 16, seed=100 + NS, dtype=dtype, with_grad_output=False)
    t = _randomise_params(t, 7, dtype)
    outs, saved = _run(t, K, dtype)
    ref = _oracle(t, K)
    r = RTOL[dtype]
    assert_close(outs.output, ref["output"], r, "output")
    assert_close(outs.weight, ref["weight"], r, "final weight")
    assert_close(outs.bias, ref["bias"], r, "final bias")
    # saved state: float32 W before every K-th stage, then the final W, per stream
    nck = (NS + K - 1) // K
    import ttt_rs_b200 as tb
    ck = tb.unpack_weight_checkpoints(saved.weight_checkpoints).reshape(B * H, nck + 1, 64, 64)
    assert_close(ck[:, :nck].reshape(-1, 64, 64), ref["weight_checkpoints"], r, "weight checkpoints")
    assert_close(ck[:, nck], ref["weight"].reshape(B * H, 64, 64), r, "final-state checkpoint")


def test_cfg0_forward_f32_matches_reference_golden(golden_dir):
    """Benchmark configuration 0 (B=2 H=4 T=256 float32) against outputs of the reference's own module."""
    z = np.load(golden_dir / "cfg0_linear_f32.npz")
    stride = int(z["stride"])
    t = O.make_inputs(2, 4, 256, 64, 16, seed=0, dtype=torch.float32, with_grad_output=False)
    outs, _ = _run(t, 1, torch.float32)
    sub = lambda x: x.reshape(-1)[::stride].cpu()
    assert_close(sub(outs.output), torch.from_numpy(z["output_f64_sub"]), 1e-4, "output vs reference f64")
    assert_close(sub(outs.output), torch.from_numpy(z["output_f32_sub"]), 1e-4, "output vs reference f32")
    assert_close(sub(outs.weight), torch.from_numpy(z["final_W1_f64_sub"]), 1e-4, "final W")
    assert_close(outs.bias.cpu(), torch.from_numpy(z["final_b1_f64"]), 1e-4, "final b")


def test_reference_validate_case_constant_qkv(golden_dir):
    """The reference's integration-test vector is head_dim 16, which this build rejects like any other
    unsupported tile configuration; the same constant-q/k/v construction at head_dim 64 is checked instead."""
    import ttt_rs_b200 as tb
    B, H, T = 2, 4, 16
    t = O.make_inputs(B, H, T, 64, 16, seed=42, dtype=torch.float32, with_grad_output=False)
    t["xq"].fill_(0.1)
    t["xk"].fill_(0.2)
    t["xv"].fill_(0.3)
    outs, _ = _run(t, 1, torch.float32)
    ref = _oracle(t, 1)
    # identical rows make sigma tiny, so float32 rounding is amplified: the reference itself asks 2e-3 here
    assert_close(outs.output, ref["output"], 2e-3, "output")
    assert_close(outs.weight, ref["weight"], 2e-3, "final weight")


def test_token_eta_past_first_mini_batch_is_ignored():
    t = O.make_inputs(1, 2, 64, 64, 16, seed=3, dtype=torch.bfloat16, with_grad_output=False)
    a, _ = _run(t, 1, torch.bfloat16)
    t2 = dict(t)
    te = t["token_eta"].clone()
    te[16:] = 55.0
    t2["token_eta"] = te
    b, _ = _run(t2, 1, torch.bfloat16)
    assert torch.equal(a.output, b.output)


def test_forward_is_deterministic():
    t = O.make_inputs(2, 3, 128, 64, 16, seed=4, dtype=torch.bfloat16, with_grad_output=False)
    a, _ = _run(t, 4, torch.bfloat16)
    b, _ = _run(t, 4, torch.bfloat16)
    assert torch.equal(a.output, b.output) and torch.equal(a.weight, b.weight)


def test_inner_model_interface_chains_state():
    """forward() over T tokens == two forward() calls over the halves with the state carried."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    inner = tb.TTTLinear(2, 64, 16, 1e-6, 2, device=dev, dtype=torch.bfloat16)
    model = tb.FusedTileMultiTTTLinear(inner)
    assert model.name() == "FusedTileMultiTTTLinear"
    t = O.make_inputs(2, 2, 64, 64, 16, seed=9, dtype=torch.bfloat16, with_grad_output=False)
    mk = lambda sl: tb.TTTInputsInner(tb.Qkv(t["xq"][:, :, sl].to(dev), t["xk"][:, :, sl].to(dev), t["xv"][:, :, sl].to(dev)),
                                      t["token_eta"][sl].to(dev), t["ttt_lr_eta"][:, :, sl].to(dev))
    with torch.no_grad():
        s1 = model.init_state(2)
        full = model.forward(s1, mk(slice(0, 64)))
        s2 = model.init_state(2)
        a = model.forward(s2, mk(slice(0, 32)))
        b = model.forward(s2, mk(slice(32, 64)))
    assert_close(torch.cat([a, b], dim=2), full, 2e-2, "chained output")
    assert_close(s2.weight, s1.weight, 2e-2, "chained weight")
    with pytest.raises(AssertionError):
        model.forward_mini_batch(model.init_state(2), mk(slice(0, 64)), range(0, 8))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_inference_forward_keeps_no_state_and_gives_the_same_bits(dtype):
    """`save_state=False` (what `torch.no_grad()` selects): the kernel writes no checkpoints, gradient tiles or
    statistics; output and final state are bit-identical to the training forward's."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    t = O.make_inputs(2, 3, 160, 64, 16, seed=12, dtype=dtype, with_grad_output=False)
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, 4)
    ins = tb.TttInputs(*[t[k].to(dev) for k in LIN_IN])
    a, saved = tb.TttTileMultiKernel.forward_launch(ins, cfg)
    b, none = tb.TttTileMultiKernel.forward_launch(ins, cfg, save_state=False)
    tb.check_status()
    assert saved is not None and none is None
    assert torch.equal(a.output, b.output) and torch.equal(a.weight, b.weight) and torch.equal(a.bias, b.bias)
    with torch.no_grad():
        out, w, _ = tb.fused_ttt_tile_forward_multi(*[t[k].to(dev) for k in LIN_IN], cfg)
    assert torch.equal(out, a.output) and torch.equal(w, a.weight)
