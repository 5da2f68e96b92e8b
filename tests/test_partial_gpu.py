"""Partial mini-batches (sequence tails, 1-token decode steps): `ttt_linear_forward_partial` against the CPU
restatement of the reference's unfused inner model on the same shapes, alone, behind the host mirror, and inside the
outer layer as a prefill + decode loop."""

import pytest
import torch

from conftest import assert_close
from oracle import ttt_layer_oracle as LO
from oracle import ttt_oracle as O

LIN_IN = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")
RTOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def _inputs(B, H, T, seed, dtype):
    t = O.make_inputs(B, H, max(T, 16), 64, 16, seed=seed, dtype=dtype, with_grad_output=False)
    g = torch.Generator().manual_seed(seed + 100)
    t["ln_weight"] = (1 + 0.1 * torch.randn(H, 64, generator=g)).to(dtype)
    t["ln_bias"] = (0.1 * torch.randn(H, 64, generator=g)).to(dtype)
    t["bias"] = (0.05 * torch.randn(B, H, 64, generator=g)).to(dtype)
    for k in ("xq", "xk", "xv"):
        t[k] = t[k][:, :, :T].contiguous()
    t["ttt_lr_eta"] = t["ttt_lr_eta"][:, :, :T].contiguous()
    t["token_eta"] = t["token_eta"][:T].contiguous()
    return t


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
@pytest.mark.parametrize("r", (1, 2, 7, 15, 16))
def test_partial_forward_matches_the_unfused_semantics(dtype, r):
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    t = _inputs(2, 3, r, 40 + r, dtype)
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, 1)
    outs = tb.TttTileMultiKernel.forward_partial(tb.TttInputs(*[t[k].to(dev) for k in LIN_IN]), cfg)
    torch.cuda.synchronize()
    want = O.ttt_linear_forward(*[t[k].double() for k in LIN_IN], mini_batch=r, eps=1e-6)
    rt = RTOL[dtype]
    assert_close(outs.output, want["output"], rt, "output")
    assert_close(outs.weight, want["weight"], rt, "weight")
    assert_close(outs.bias, want["bias"], rt, "bias")


@pytest.mark.gpu
def test_in_place_state_update_equals_out_of_place():
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    t = _inputs(2, 2, 5, 3, torch.float32)
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, 1)
    a = tb.TttTileMultiKernel.forward_partial(tb.TttInputs(*[t[k].to(dev) for k in LIN_IN]), cfg)
    ins = tb.TttInputs(*[t[k].to(dev) for k in LIN_IN])
    b = tb.TttTileMultiKernel.forward_partial(ins, cfg, in_place=True)
    torch.cuda.synchronize()
    assert b.weight.data_ptr() == ins.weight.data_ptr()
    assert torch.equal(a.output, b.output) and torch.equal(a.weight, b.weight) and torch.equal(a.bias, b.bias)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
def test_host_mirror_runs_the_tail_of_a_ragged_sequence(dtype):
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    B, H, T = 2, 2, 39
    t = _inputs(B, H, T, 9, dtype)
    t["token_eta"] = (1.0 / (torch.arange(T) % 16 + 1)).to(dtype)
    inner = tb.TTTLinear(H, 64, 16, 1e-6, 1, device=dev, dtype=dtype)
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
    rt = RTOL[dtype]
    assert out.shape == (B, H, T, 64)
    assert_close(out, want["output"], rt, "output", max_bad_frac=1e-4 if dtype == torch.bfloat16 else 0.0)
    assert_close(state.weight, want["weight"], rt, "weight", max_bad_frac=1e-4 if dtype == torch.bfloat16 else 0.0)
    # the reference's fused type refuses the tail; so does the mirror unless asked otherwise
    strict = tb.FusedTileMultiTTTLinear(inner)
    with pytest.raises(AssertionError, match="mini_batch_size"), torch.no_grad():
        strict.forward(tb.TTTLinearState(t["weight"].to(dev), t["bias"].to(dev)), ins)


@pytest.mark.gpu
def test_layer_prefill_then_token_by_token_decode():
    import ttt_rs_b200 as tb
    from test_layer_gpu import _layer_from_params, _random_case
    dev = torch.device("cuda:0")
    B, H, T0, steps = 2, 2, 32, 4
    x, p = _random_case(B, T0 + steps, H, 21, False, False, torch.float32)
    m, inner = _layer_from_params(tb, p, False, False, torch.float32, dev, H)
    inner.allow_partial = True
    xs = x.float().to(dev)
    with torch.no_grad():
        state = inner.init_state(B)
        ys = [m(xs[:, :T0], inner, state, 0)]
        for i in range(steps):
            ys.append(m(xs[:, T0 + i:T0 + i + 1], inner, state, T0 + i))
    torch.cuda.synchronize()
    y, st = LO.ttt_layer_forward(x[:, :T0], p, num_heads=H, start_idx=0)
    want = [y]
    for i in range(steps):
        y, st = LO.ttt_layer_forward(x[:, T0 + i:T0 + i + 1], p, num_heads=H, start_idx=T0 + i, state=st)
        want.append(y)
    assert_close(torch.cat(ys, dim=1), torch.cat(want, dim=1), 2e-4, "prefill + decode outputs")
    assert_close(state.weight, st["weight"], 2e-4, "state after decode")


@pytest.mark.gpu
def test_decode_through_cuda_graphs_equals_eager_decode():
    """The captured decode step (one CUDA graph per rotary phase, state advanced in place) gives the same bits as
    calling the layer token by token, across two wraps of the rotary positions."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    B, H, T0, steps = 2, 2, 16, 35
    cfg = tb.TTTLayerConfig(hidden_size=H * 64, num_heads=H, use_gate=True)
    torch.manual_seed(3)
    layer = tb.TTT(cfg, device=dev, dtype=torch.bfloat16)
    x = (torch.randn(B, T0 + steps, H * 64, device=dev) * 0.5).to(torch.bfloat16)

    def run(use_graphs):
        inner = tb.new_inner(cfg, device=dev, dtype=torch.bfloat16, allow_partial=True, partial_in_place=True)
        with torch.no_grad():
            inner.inner.weight_init.copy_(torch.randn(H, 64, 64, generator=torch.Generator().manual_seed(1)) * 0.02)
            state = inner.init_state(B)
            state.weight, state.bias = state.weight.contiguous(), state.bias.contiguous()
            layer(x[:, :T0], inner, state, 0)  # prefill
            dec = tb.DecodeGraphs(layer, inner, state, B) if use_graphs else None
            outs = []
            for i in range(steps):
                xi = x[:, T0 + i:T0 + i + 1]
                y = dec.step(xi, T0 + i) if use_graphs else layer(xi.contiguous(), inner, state, T0 + i)
                outs.append(y.clone())
        torch.cuda.synchronize()
        return torch.cat(outs, dim=1), state.weight.clone()

    ye, we = run(False)
    yg, wg = run(True)
    assert torch.equal(ye, yg), "outputs differ between eager and graph decode"
    assert torch.equal(we, wg), "state differs between eager and graph decode"
