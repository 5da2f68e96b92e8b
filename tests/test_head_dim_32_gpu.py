"""head_dim 32 (the reference's 16x32 tile, rust/core/src/ttt/cubecl_kernels/linear_fused_tile/launch_multi.rs dispatch
on (mini_batch_len, head_dim)): the kernels run a pair of heads per 64-wide tile.  Forward and backward through the C
ABI against the CPU oracle, which works head by head (needs a B200)."""

import pytest
import torch

from conftest import assert_close
from oracle import ttt_oracle as O

pytestmark = pytest.mark.gpu

LIN_IN = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")
RTOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}
F = 32


def _case(B, H, NS, seed, dtype):
    t = O.make_inputs(B, H, NS * 16, F, 16, seed=seed, dtype=dtype)
    g = torch.Generator().manual_seed(seed + 1)
    t["ln_weight"] = (1.0 + 0.1 * torch.randn(t["ln_weight"].shape, generator=g)).to(dtype)
    t["ln_bias"] = (0.1 * torch.randn(t["ln_bias"].shape, generator=g)).to(dtype)
    t["bias"] = (0.05 * torch.randn(t["bias"].shape, generator=g)).to(dtype)
    return t


def _run_gpu(t, K, packed=False, save_state=True, state_grads=None):
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    cfg = tb.FusedTttConfig.new(16, F, 1e-6, 128, K)
    ins = tb.TttInputs(*[t[k].to(dev) for k in LIN_IN])
    outs, saved = tb.TttTileMultiKernel.forward_launch(ins, cfg, save_state=save_state)
    grads = pk = None
    if save_state:
        H = t["xq"].shape[1]
        pk = torch.full((tb.packed_outer_grad_len(H, F),), float("nan"), device=dev) if packed else None
        gw, gb = (None, None) if state_grads is None else (state_grads[0].to(dev), state_grads[1].to(dev))
        grads = tb.TttTileMultiKernel.backward_launch(saved, tb.TttOutputs(t["grad_output"].to(dev), gw, gb), cfg,
                                                      outer_grad_packed=pk, use_state_grads=state_grads is not None)
    torch.cuda.synchronize()
    tb.check_status()
    return outs, grads, pk


def _oracle_fwd(t, K):
    return O.ttt_linear_forward(*[t[k].double() for k in LIN_IN], mini_batch=16, eps=1e-6, checkpoint_interval=K)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,NS,K", [(1, 2, 1, 1), (2, 4, 5, 2), (1, 6, 20, 16), (3, 2, 33, 4)])
def test_forward_matches_oracle(dtype, B, H, NS, K):
    t = _case(B, H, NS, 900 + NS + K, dtype)
    outs, _, _ = _run_gpu(t, K, save_state=False)
    ref = _oracle_fwd(t, K)
    r = RTOL[dtype]
    frac = 1e-4 if dtype == torch.bfloat16 else 0.0
    assert_close(outs.output, ref["output"], r, "output (head_dim 32)", max_bad_frac=frac)
    assert_close(outs.weight, ref["weight"], r, "final weight (head_dim 32)", max_bad_frac=frac)
    assert_close(outs.bias, ref["bias"], r, "final bias (head_dim 32)", max_bad_frac=frac)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_training_forward_equals_inference_forward(dtype):
    t = _case(2, 4, 6, 31, dtype)
    a, _, _ = _run_gpu(t, 4, save_state=True)
    b, _, _ = _run_gpu(t, 4, save_state=False)
    assert torch.equal(a.output, b.output) and torch.equal(a.weight, b.weight) and torch.equal(a.bias, b.bias)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,NS,K", [(1, 2, 1, 1), (2, 4, 4, 2), (1, 2, 40, 32), (2, 6, 18, 16)])
def test_backward_matches_oracle(dtype, B, H, NS, K):
    t = _case(B, H, NS, 500 + NS + K, dtype)
    _, grads, _ = _run_gpu(t, K)
    ref = O.ttt_linear_backward(*[t[k].double() for k in LIN_IN], t["grad_output"].double(), mini_batch=16, eps=1e-6)
    r = RTOL[dtype]
    frac = 1e-4 if dtype == torch.bfloat16 else 0.0
    for name in LIN_IN:
        assert_close(getattr(grads, name), ref["grad_" + name], r, f"grad_{name} (head_dim 32)", max_bad_frac=frac)


def test_backward_packs_outer_grads_and_is_deterministic():
    t = _case(3, 4, 8, 13, torch.bfloat16)
    _, g1, p1 = _run_gpu(t, 4, packed=True)
    _, g2, p2 = _run_gpu(t, 4, packed=True)
    for name in LIN_IN:
        assert torch.equal(getattr(g1, name), getattr(g2, name)), name
    assert torch.equal(p1, p2)
    H = 4
    ref = O.ttt_linear_backward(*[t[k].double() for k in LIN_IN], t["grad_output"].double(), mini_batch=16, eps=1e-6)
    o = 0
    assert_close(p1[o:o + H * F * F].reshape(H, F, F), ref["grad_weight"].sum(0), 2e-2, "packed dW0"); o += H * F * F
    assert_close(p1[o:o + H * F].reshape(H, F), ref["grad_bias"].sum(0), 2e-2, "packed db0"); o += H * F
    assert_close(p1[o:o + H * F].reshape(H, F), ref["grad_ln_weight"], 2e-2, "packed d ln_weight"); o += H * F
    assert_close(p1[o:o + H * F].reshape(H, F), ref["grad_ln_bias"], 2e-2, "packed d ln_bias"); o += H * F
    assert_close(p1[o:o + 16], ref["grad_token_eta"].reshape(-1, 16).sum(0), 2e-2, "packed d token_eta")


def test_backward_with_final_state_gradients():
    """Upstream gradients of the final state enter the head's own 32 x 32 block."""
    dtype = torch.float32
    t = _case(2, 2, 6, 71, dtype)
    g = torch.Generator().manual_seed(5)
    gw = (0.1 * torch.randn(t["weight"].shape, generator=g)).to(dtype)
    gb = (0.1 * torch.randn(t["bias"].shape, generator=g)).to(dtype)
    _, grads, _ = _run_gpu(t, 4, state_grads=(gw, gb))
    ref = O.ttt_linear_backward(*[t[k].double() for k in LIN_IN], t["grad_output"].double(), mini_batch=16, eps=1e-6,
                                grad_weight_out=gw.double(), grad_bias_out=gb.double())
    for name in LIN_IN:
        assert_close(getattr(grads, name), ref["grad_" + name], 1e-4, f"grad_{name} (state grads, head_dim 32)")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("r", (1, 5, 16))
def test_partial_mini_batch(dtype, r):
    """Decode step / sequence tail (`ttt_linear_forward_partial`) at head_dim 32: one mini-batch of r tokens."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    t = _case(2, 3, 1, 60 + r, dtype)  # the partial kernel works head by head: odd head counts are fine
    for k in ("xq", "xk", "xv"):
        t[k] = t[k][:, :, :r].contiguous()
    t["ttt_lr_eta"] = t["ttt_lr_eta"][:, :, :r].contiguous()
    t["token_eta"] = t["token_eta"][:r].contiguous()
    cfg = tb.FusedTttConfig.new(16, F, 1e-6, 128, 1)
    outs = tb.TttTileMultiKernel.forward_partial(tb.TttInputs(*[t[k].to(dev) for k in LIN_IN]), cfg)
    torch.cuda.synchronize()
    want = O.ttt_linear_forward(*[t[k].double() for k in LIN_IN], mini_batch=r, eps=1e-6)
    assert_close(outs.output, want["output"], RTOL[dtype], "partial output (head_dim 32)")
    assert_close(outs.weight, want["weight"], RTOL[dtype], "partial weight (head_dim 32)")
    assert_close(outs.bias, want["bias"], RTOL[dtype], "partial bias (head_dim 32)")


def test_inner_model_interface_with_ragged_tail():
    """`FusedTileMultiTTTLinear.forward` over 2 full mini-batches + a 7-token tail, 4 heads of 32."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    dtype = torch.float32
    B, H, T = 2, 4, 39
    t = _case(B, H, 3, 17, dtype)
    for k in ("xq", "xk", "xv"):
        t[k] = t[k][:, :, :T].contiguous()
    t["ttt_lr_eta"] = t["ttt_lr_eta"][:, :, :T].contiguous()
    t["token_eta"] = (1.0 / (torch.arange(T) % 16 + 1)).to(dtype)
    inner = tb.TTTLinear(H, F, 16, 1e-6, 1, device=dev, dtype=dtype)
    with torch.no_grad():
        inner.ln_weight.copy_(t["ln_weight"]); inner.ln_bias.copy_(t["ln_bias"])
    m = tb.FusedTileMultiTTTLinear(inner, allow_partial=True)
    state = tb.TTTLinearState(t["weight"].to(dev), t["bias"].to(dev))
    ins = tb.TTTInputsInner(tb.Qkv(t["xq"].to(dev), t["xk"].to(dev), t["xv"].to(dev)), t["token_eta"].to(dev),
                            t["ttt_lr_eta"].to(dev))
    with torch.no_grad():
        out = m.forward(state, ins)
    torch.cuda.synchronize()
    want = O.ttt_linear_forward_any_length(*[t[k].double() for k in LIN_IN], mini_batch=16)
    assert out.shape == (B, H, T, F)
    assert_close(out, want["output"], 1e-4, "ragged output (head_dim 32)")
    assert_close(state.weight, want["weight"], 1e-4, "ragged final weight (head_dim 32)")


def test_odd_head_count_is_rejected():
    import ttt_rs_b200 as tb
    t = _case(1, 3, 2, 3, torch.bfloat16)
    with pytest.raises(tb.TttError, match="even number of heads"):
        _run_gpu(t, 1, save_state=False)
