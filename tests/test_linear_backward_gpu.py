"""Parity of the CUDA backward scan with the CPU oracle, through the C ABI (needs a B200).

Mirrors the reference's `test_backward_fwd` pattern (rust/core/src/test_utils.rs:303-609): same tensors into the
oracle and the kernel, loss = <grad_output, output>, compare the gradients of all nine inputs."""

import pytest
import torch

from conftest import assert_close
from oracle import ttt_oracle as O

pytestmark = pytest.mark.gpu

LIN_IN = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")
RTOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}
GRADS = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")


def _case(B, H, NS, seed, dtype, gscale=1.0):
    t = O.make_inputs(B, H, NS * 16, 64, 16, seed=seed, dtype=dtype)
    g = torch.Generator().manual_seed(seed + 1)
    t["ln_weight"] = (1.0 + 0.1 * torch.randn(t["ln_weight"].shape, generator=g)).to(dtype)
    t["ln_bias"] = (0.1 * torch.randn(t["ln_bias"].shape, generator=g)).to(dtype)
    t["bias"] = (0.05 * torch.randn(t["bias"].shape, generator=g)).to(dtype)
    t["grad_output"] = (t["grad_output"].float() * gscale).to(dtype)
    return t


def _run_gpu(t, K, packed=False):
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, K)
    ins = tb.TttInputs(*[t[k].to(dev) for k in LIN_IN])
    outs, saved = tb.TttTileMultiKernel.forward_launch(ins, cfg)
    H = t["xq"].shape[1]
    pk = torch.full((tb.packed_outer_grad_len(H),), float("nan"), device=dev) if packed else None
    grads = tb.TttTileMultiKernel.backward_launch(saved, tb.TttOutputs(t["grad_output"].to(dev), None, None), cfg,
                                                  outer_grad_packed=pk)
    torch.cuda.synchronize()
    tb.TttTileMultiKernel.check_status()
    return outs, grads, pk


def _oracle(t):
    args = [t[k].double() for k in LIN_IN]
    return O.ttt_linear_backward(*args, t["grad_output"].double(), mini_batch=16, eps=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,NS,K", [
    (1, 1, 1, 1),      # single stage
    (2, 2, 4, 1),      # a checkpoint every stage
    (2, 2, 4, 2),
    (1, 3, 5, 4),      # ragged last group
    (2, 2, 16, 16),    # one full group of 16
    (1, 2, 40, 32),    # interval larger than the stash: sub-groups + ragged tail
    (1, 2, 24, 128),   # a single checkpoint for the whole sequence
])
def test_backward_matches_oracle(dtype, B, H, NS, K):
    t = _case(B, H, NS, 300 + NS + K, dtype)
    _, grads, _ = _run_gpu(t, K)
    ref = _oracle(t)
    r = RTOL[dtype]
    frac = 1e-4 if dtype == torch.bfloat16 else 0.0
    for name in GRADS:
        assert_close(getattr(grads, name), ref["grad_" + name], r, f"grad_{name}", max_bad_frac=frac)


def test_backward_is_deterministic_and_packs_outer_grads():
    t = _case(3, 2, 8, 11, torch.bfloat16)
    _, g1, p1 = _run_gpu(t, 4, packed=True)
    _, g2, p2 = _run_gpu(t, 4, packed=True)
    for name in GRADS:
        assert torch.equal(getattr(g1, name), getattr(g2, name)), name
    assert torch.equal(p1, p2)
    H, F = 2, 64
    ref = _oracle(t)
    o = 0
    assert_close(p1[o:o + H * F * F].reshape(H, F, F), ref["grad_weight"].sum(0), 2e-2, "packed dW0"); o += H * F * F
    assert_close(p1[o:o + H * F].reshape(H, F), ref["grad_bias"].sum(0), 2e-2, "packed db0"); o += H * F
    assert_close(p1[o:o + H * F].reshape(H, F), ref["grad_ln_weight"], 2e-2, "packed d ln_weight"); o += H * F
    assert_close(p1[o:o + H * F].reshape(H, F), ref["grad_ln_bias"], 2e-2, "packed d ln_bias"); o += H * F
    assert_close(p1[o:o + 16], ref["grad_token_eta"].reshape(-1, 16).sum(0), 2e-2, "packed d token_eta")


def test_autograd_function_matches_oracle():
    """loss.backward() through the autograd-registered operator, as the layer above would call it."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    t = _case(2, 2, 6, 21, torch.float32)
    leaves = {k: t[k].to(dev).requires_grad_(True) for k in LIN_IN}
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, 4)
    out, w, b = tb.fused_ttt_tile_forward_multi(*[leaves[k] for k in LIN_IN], cfg)
    (out * t["grad_output"].to(dev)).sum().backward()
    ref = _oracle(t)
    for name in GRADS:
        assert_close(leaves[name].grad, ref["grad_" + name], 1e-4, f"grad_{name}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_backward_with_final_state_gradients(dtype):
    """Upstream gradients of the returned final state (opt-in; the reference drops them): against the oracle, and
    as backward-through-time in two chunks that must reproduce the one-shot gradients."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    t = _case(2, 2, 8, 77, dtype)
    g = torch.Generator().manual_seed(5)
    gw = (0.1 * torch.randn(t["weight"].shape, generator=g)).to(dtype)
    gb = (0.1 * torch.randn(t["bias"].shape, generator=g)).to(dtype)
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, 4)
    r = RTOL[dtype]
    frac = 1e-4 if dtype == torch.bfloat16 else 0.0

    def run(tt, go, gwo=None, gbo=None):
        ins = tb.TttInputs(*[tt[k].to(dev) for k in LIN_IN])
        outs, saved = tb.TttTileMultiKernel.forward_launch(ins, cfg)
        grads = tb.TttTileMultiKernel.backward_launch(
            saved, tb.TttOutputs(go.to(dev), None if gwo is None else gwo.to(dev), None if gbo is None else gbo.to(dev)),
            cfg, use_state_grads=True)
        torch.cuda.synchronize()
        return outs, grads

    _, grads = run(t, t["grad_output"], gw, gb)
    ref = O.ttt_linear_backward(*[t[k].double() for k in LIN_IN], t["grad_output"].double(),
                                grad_weight_out=gw.double(), grad_bias_out=gb.double())
    for name in GRADS:
        assert_close(getattr(grads, name), ref["grad_" + name], r, f"grad_{name}", max_bad_frac=frac)

    # chunked: tokens [0,64) then [64,128) with the state carried forward and its gradient carried back
    _, full = run(t, t["grad_output"])
    seq = ("xq", "xk", "xv", "ttt_lr_eta")
    first = {k: (t[k][:, :, :64] if k in seq else t[k]) for k in LIN_IN}
    first["token_eta"] = t["token_eta"][:64]  # [seq_len] of the chunk; the kernels read positions [0, 16) only
    o1, _ = run(first, t["grad_output"][:, :, :64])
    second = {k: (t[k][:, :, 64:] if k in seq else t[k]) for k in LIN_IN}
    second["token_eta"] = t["token_eta"][64:]
    second["weight"], second["bias"] = o1.weight.cpu(), o1.bias.cpu()
    _, g2 = run(second, t["grad_output"][:, :, 64:])
    _, g1 = run(first, t["grad_output"][:, :, :64], g2.weight.cpu(), g2.bias.cpu())
    tol = 2 * r  # the carried state and its gradient are rounded to the I/O type between the chunks
    assert_close(torch.cat([g1.xk, g2.xk], dim=2), full.xk.double(), tol, "chunked grad_xk", max_bad_frac=frac)
    assert_close(torch.cat([g1.xq, g2.xq], dim=2), full.xq.double(), tol, "chunked grad_xq", max_bad_frac=frac)
    assert_close(g1.weight, full.weight.double(), tol, "chunked grad_weight", max_bad_frac=frac)
