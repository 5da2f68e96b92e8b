"""Outer-layer kernels (ttt_layer_prologue / ttt_layer_epilogue) and the whole `TTT.forward` on the GPU against the
CPU restatement and against the reference's own layer outputs (tests/golden/layer_linear_f64.npz)."""

import numpy as np
import pytest
import torch

from conftest import assert_close
from oracle import ttt_layer_oracle as LO

RTOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def _golden(golden_dir, tag):
    z = np.load(golden_dir / "layer_linear_f64.npz")
    return {k.split(".", 1)[1]: torch.from_numpy(z[k]) for k in z.files if k.startswith(tag + ".")}


def _layer_from_params(tb, p, share_qk, use_gate, dtype, dev, H):
    cfg = tb.TTTLayerConfig(hidden_size=p["q_proj"].shape[0], num_heads=H, share_qk=share_qk, use_gate=use_gate)
    m = tb.TTT(cfg, device=dev, dtype=dtype)
    inner = tb.new_inner(cfg, device=dev, dtype=dtype)
    with torch.no_grad():
        def put(dst, src):
            dst.copy_(src.reshape(dst.shape).to(dtype))
        put(m.q_proj, p["q_proj"]); put(m.v_proj, p["v_proj"]); put(m.o_proj, p["o_proj"])
        if not share_qk:
            put(m.k_proj, p["k_proj"])
        else:
            put(m.q_conv_weight, p["conv_q_weight"]); put(m.q_conv_bias, p["conv_q_bias"])
            put(m.k_conv_weight, p["conv_k_weight"]); put(m.k_conv_bias, p["conv_k_bias"])
        if use_gate:
            put(m.g_proj, p["g_proj"])
        put(m.learnable_ttt_lr_weight, p["lr_weight"]); put(m.learnable_ttt_lr_bias, p["lr_bias"])
        put(m.learnable_token_idx, p["learnable_token_idx"])
        put(m.post_norm_weight, p["post_norm_weight"]); put(m.post_norm_bias, p["post_norm_bias"])
        put(inner.inner.weight_init, p["W1"]); put(inner.inner.bias_init, p["b1"])
        put(inner.inner.ln_weight, p["ttt_norm_weight"]); put(inner.inner.ln_bias, p["ttt_norm_bias"])
    m.invalidate_fused_weight()
    return m, inner


@pytest.mark.gpu
@pytest.mark.parametrize("tag,share_qk,use_gate", (("plain", False, False), ("conv_gate", True, True)))
def test_layer_forward_float32_matches_reference_golden(golden_dir, tag, share_qk, use_gate):
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    p = _golden(golden_dir, tag)
    m, inner = _layer_from_params(tb, p, share_qk, use_gate, torch.float32, dev, 2)
    x = p["input"].float().to(dev)
    with torch.no_grad():
        state = inner.init_state(x.shape[0])
        y = m(x, inner, state)
    tb.TttTileMultiKernel.check_status()
    # the projections are library float32 GEMMs (TF32 off by default); the kernels compute in float32
    assert_close(y, p["output_expected"], 2e-4, f"{tag}: layer output")
    want_state = LO.ttt_layer_forward(p["input"], p, num_heads=2, share_qk=share_qk, use_gate=use_gate)[1]
    assert_close(state.weight, want_state["weight"], 2e-4, f"{tag}: final inner weight")


def _random_case(B, T, H, seed, share_qk, use_gate, dtype, F=64):
    g = torch.Generator().manual_seed(seed)
    C = H * F
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).to(dtype).double()  # noqa: E731
    p = {"q_proj": r(C, C, sc=C ** -0.5), "v_proj": r(C, C, sc=C ** -0.5), "o_proj": r(C, C, sc=C ** -0.5),
         "lr_weight": r(H, C, 1, sc=0.02), "lr_bias": r(H, 1, sc=0.1), "token_idx": 1.0 / torch.arange(1, 17).double(),
         "learnable_token_idx": r(16, sc=0.05), "post_norm_weight": 1 + r(C, sc=0.1), "post_norm_bias": r(C, sc=0.1),
         "W1": r(H, F, F, sc=0.02), "b1": r(H, 1, F, sc=0.05), "ttt_norm_weight": 1 + r(H, F, sc=0.1),
         "ttt_norm_bias": r(H, F, sc=0.1)}
    if share_qk:
        p.update(conv_q_weight=r(C, 1, 4, sc=0.5), conv_q_bias=r(C, sc=0.1), conv_k_weight=r(C, 1, 4, sc=0.5),
                 conv_k_bias=r(C, sc=0.1))
    else:
        p["k_proj"] = r(C, C, sc=C ** -0.5)
    if use_gate:
        p["g_proj"] = r(C, C, sc=C ** -0.5)
    x = r(B, T, C)
    return x, p


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
@pytest.mark.parametrize("F,H", ((64, 3), (32, 3), (32, 12)))
@pytest.mark.parametrize("share_qk,use_gate,pos,start", ((False, False, "rope", 0), (True, True, "rope", 21),
                                                         (False, True, "rope_global", 5), (True, False, "none", 0)))
def test_prologue_and_epilogue_kernels_match_the_restatement(dtype, F, H, share_qk, use_gate, pos, start):
    """Kernel-level parity on ragged sizes (T not a multiple of the mini-batch or of the kernel's token chunk,
    heads not a multiple of the 4 or 8 a warp takes), fed with exactly the projection values the kernels see."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    B, T = 3, 83
    C = H * F
    x, p = _random_case(B, T, H, 11, share_qk, use_gate, dtype, F)
    cfg = tb.TTTLayerConfig(hidden_size=C, num_heads=H, share_qk=share_qk, use_gate=use_gate, pos_encoding=pos)
    # projection output as the layer lays it out: q | (k) | v | (g) | lr, rounded to the I/O type
    blocks = [x @ p["q_proj"].T] + ([] if share_qk else [x @ p["k_proj"].T]) + [x @ p["v_proj"].T]
    if use_gate:
        blocks.append(x @ p["g_proj"].T)
    blocks.append(torch.einsum("btc,hc->bth", x, p["lr_weight"].reshape(H, C)))
    blocks.append(torch.zeros(B, T, (-sum(b.shape[-1] for b in blocks)) % 8, dtype=torch.float64))
    proj = torch.cat(blocks, dim=-1).to(dtype)
    cols = {"q": 0, "k": 0 if share_qk else C, "v": C if share_qk else 2 * C}
    cols["g"] = cols["v"] + C
    cols["lr"] = cols["v"] + C + (C if use_gate else 0)
    conv = (p["conv_q_weight"], p["conv_q_bias"], p["conv_k_weight"], p["conv_k_bias"]) if share_qk else None
    xq, xk, xv, lr = tb.layer_prologue(proj.to(dev), cfg, q_col=cols["q"], k_col=cols["k"], v_col=cols["v"],
                                       lr_col=cols["lr"], lr_bias=p["lr_bias"].to(dev), conv=None if conv is None else
                                       tuple(t.to(dev) for t in conv), start_idx=start)
    torch.cuda.synchronize()
    # the restatement on the same rounded projection values
    pd = proj.double()
    heads = lambda t: t.reshape(B, T, H, F).permute(0, 2, 1, 3)  # noqa: E731
    qs, ks, vs = pd[..., :C], pd[..., cols["k"]:cols["k"] + C], pd[..., cols["v"]:cols["v"] + C]
    if share_qk:
        ks = LO.causal_depthwise_conv(qs, p["conv_k_weight"], p["conv_k_bias"])
        qs = LO.causal_depthwise_conv(qs, p["conv_q_weight"], p["conv_q_bias"])
    wq, wk, wv = heads(qs), heads(ks), heads(vs)
    if pos != "none":
        posv = start + torch.arange(T)
        posv = posv % 16 if pos == "rope" else posv
        wq, wk = LO.rope_pairs(wq, posv, 10000.0), LO.rope_pairs(wk, posv, 10000.0)
    wlr = torch.sigmoid(pd[..., cols["lr"]:cols["lr"] + H].permute(0, 2, 1) + p["lr_bias"].reshape(1, H, 1)) / F
    rt = RTOL[dtype]
    assert_close(xq, wq, rt, "xq"); assert_close(xk, wk, rt, "xk"); assert_close(xv, wv, rt, "xv")
    assert_close(lr, wlr, rt, "ttt_lr_eta")
    if dtype == torch.bfloat16:
        assert torch.equal(xv.cpu(), heads(proj[..., cols["v"]:cols["v"] + C]).contiguous()), "xv must be a pure copy"

    # epilogue
    inner_out = (torch.randn(B, H, T, F, generator=torch.Generator().manual_seed(3)) * 2 + 0.3).to(dtype)
    gate = gate_ld = None
    if use_gate:
        gate, gate_ld = proj.to(dev).reshape(B * T, -1)[:, cols["g"]:], proj.shape[-1]
    y = tb.layer_epilogue(inner_out.to(dev), p["post_norm_weight"].to(dev), p["post_norm_bias"].to(dev), 1e-6,
                          gate, gate_ld or 0)
    torch.cuda.synchronize()
    pw = {"post_norm_weight": p["post_norm_weight"].to(dtype).double(), "post_norm_bias": p["post_norm_bias"].to(dtype).double()}
    want = LO.layer_epilogue(inner_out.double(), None, pw, use_gate=False)
    if use_gate:
        from oracle.ttt_oracle import gelu_tanh
        want = gelu_tanh(pd[..., cols["g"]:cols["g"] + C]) * want
    assert_close(y, want, rt, "epilogue")


@pytest.mark.gpu
@pytest.mark.parametrize("F,H", ((64, 12), (32, 24)))
def test_layer_forward_bfloat16_at_a_wider_shape(F, H):
    """768 hidden features as 12 heads of 64 (one launch for projections + prologue) and as 24 heads of 32 (the
    reference's `125m-h32` split: the projection GEMM, then the prologue kernel; the inner loop packs head pairs)."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    B, T = 2, 128
    x, p = _random_case(B, T, H, 5, False, True, torch.bfloat16, F)
    m, inner = _layer_from_params(tb, p, False, True, torch.bfloat16, dev, H)
    with torch.no_grad():
        state = inner.init_state(B)
        y = m(x.to(torch.bfloat16).to(dev), inner, state)
    tb.TttTileMultiKernel.check_status()
    want, _ = LO.ttt_layer_forward(x, p, num_heads=H, use_gate=True)
    assert_close(y, want, 2e-2, "layer output", max_bad_frac=2e-4)  # measured 9.2e-5 on B200


@pytest.mark.gpu
@pytest.mark.parametrize("F,H", ((64, 3), (32, 4)))
@pytest.mark.parametrize("use_gate,share_qk", ((False, False), (True, False), (True, True)))
def test_layer_training_gradients_match_autograd_of_the_restatement(use_gate, share_qk, F, H):
    """Whole-layer backward (projection GEMM gradients by torch, every other step by this repo's gradient kernels)
    against float64 autograd through the CPU restatement."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    B, T = 2, 80 if share_qk else 48  # 80 tokens: two chunks of the convolution gradient kernel
    x, p = _random_case(B, T, H, 31, share_qk, use_gate, torch.float32, F)
    m, inner = _layer_from_params(tb, p, share_qk, use_gate, torch.float32, dev, H)
    xg = x.float().to(dev).requires_grad_(True)
    gy = torch.randn(B, T, H * F, generator=torch.Generator().manual_seed(2)).double()
    state = inner.init_state(B)
    y = m(xg, inner, state)
    y.backward(gy.float().to(dev))
    torch.cuda.synchronize()
    tb.TttTileMultiKernel.check_status()

    leaves = {k: v.clone().requires_grad_(True) for k, v in p.items() if k != "token_idx"}
    leaves["token_idx"] = p["token_idx"]
    xr = x.clone().requires_grad_(True)
    yr, _ = LO.ttt_layer_forward(xr, leaves, num_heads=H, use_gate=use_gate, share_qk=share_qk)
    yr.backward(gy)
    assert_close(y, yr, 2e-4, "output")
    rt = 1e-3
    assert_close(xg.grad, xr.grad, rt, "d input")
    pairs = {"q_proj": m.q_proj, "v_proj": m.v_proj, "o_proj": m.o_proj,
             "lr_weight": m.learnable_ttt_lr_weight, "lr_bias": m.learnable_ttt_lr_bias,
             "learnable_token_idx": m.learnable_token_idx, "post_norm_weight": m.post_norm_weight,
             "post_norm_bias": m.post_norm_bias, "W1": inner.inner.weight_init, "b1": inner.inner.bias_init,
             "ttt_norm_weight": inner.inner.ln_weight, "ttt_norm_bias": inner.inner.ln_bias}
    if use_gate:
        pairs["g_proj"] = m.g_proj
    if share_qk:
        pairs.update({"conv_q_weight": m.q_conv_weight, "conv_q_bias": m.q_conv_bias,
                      "conv_k_weight": m.k_conv_weight, "conv_k_bias": m.k_conv_bias})
    else:
        pairs["k_proj"] = m.k_proj
    for name, param in pairs.items():
        assert param.grad is not None, f"no gradient reached {name}"
        assert_close(param.grad.reshape(leaves[name].grad.shape), leaves[name].grad, rt, f"d {name}")


@pytest.mark.gpu
def test_layer_with_mlp_inner_model_forward_and_training(golden_dir):
    """The outer layer around the 2-layer inner model: forward against the reference's `TTTMLP.forward` output
    (bf16 kernels, so at bf16 tolerance), and one training step against float64 autograd of the restatement."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    p = _golden(golden_dir, "mlp")
    H, dt = 2, torch.bfloat16
    pb = {k: v.to(dt).double() for k, v in p.items()}   # what the bf16 layer actually holds
    cfg = tb.TTTLayerConfig(hidden_size=128, num_heads=H)
    m = tb.TTT(cfg, device=dev, dtype=dt)
    mlp = tb.TTTMLP(H, 64, 16, 1e-6, device=dev, dtype=dt)
    inner = tb.FusedTTTMLP(mlp)
    with torch.no_grad():
        for dst, src in ((m.q_proj, "q_proj"), (m.k_proj, "k_proj"), (m.v_proj, "v_proj"), (m.o_proj, "o_proj"),
                         (m.learnable_ttt_lr_weight, "lr_weight"), (m.learnable_ttt_lr_bias, "lr_bias"),
                         (m.learnable_token_idx, "learnable_token_idx"), (m.post_norm_weight, "post_norm_weight"),
                         (m.post_norm_bias, "post_norm_bias"), (mlp.w1_init, "W1"), (mlp.b1_init, "b1"),
                         (mlp.w2_init, "W2"), (mlp.b2_init, "b2"), (mlp.ln_weight, "ttt_norm_weight"),
                         (mlp.ln_bias, "ttt_norm_bias")):
            dst.copy_(p[src].reshape(dst.shape).to(dt))
    m.invalidate_fused_weight()
    x = p["input"].to(dt)
    with torch.no_grad():
        y = m(x.to(dev), inner, inner.init_state(x.shape[0]))
    want, _ = LO.ttt_layer_forward(x.double(), pb, num_heads=H, inner="mlp")
    assert_close(y, want, 2e-2, "layer output (mlp inner)", max_bad_frac=1e-4)  # measured 0
    assert_close(y, p["output_expected"], 5e-2, "layer output against the float64 reference", max_bad_frac=1e-4)  # measured 0

    # training step
    xg = x.to(dev).requires_grad_(True)
    gy = torch.randn(x.shape, generator=torch.Generator().manual_seed(4)).to(dt)
    m(xg, inner, inner.init_state(x.shape[0])).backward(gy.to(dev))
    torch.cuda.synchronize()
    leaves = {k: v.clone().requires_grad_(True) for k, v in pb.items() if k != "token_idx"}
    leaves["token_idx"] = pb["token_idx"]
    xr = x.double().requires_grad_(True)
    LO.ttt_layer_forward(xr, leaves, num_heads=H, inner="mlp")[0].backward(gy.double())
    assert_close(xg.grad, xr.grad, 3e-2, "d input", max_bad_frac=1e-4)  # measured 0
    for name, param in (("W1", mlp.w1_init), ("W2", mlp.w2_init), ("b1", mlp.b1_init), ("q_proj", m.q_proj),
                        ("v_proj", m.v_proj), ("o_proj", m.o_proj), ("post_norm_weight", m.post_norm_weight)):
        assert param.grad is not None, name
        assert_close(param.grad.reshape(leaves[name].grad.shape), leaves[name].grad, 3e-2, f"d {name}", max_bad_frac=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,K", ((torch.float32, 4), (torch.float32, 3), (torch.bfloat16, 4)))
def test_shared_qk_convolution_step_and_its_gradient(dtype, K):
    """`ttt_layer_qk_conv` / `ttt_layer_qk_conv_backward` on a ragged size (T not a multiple of the kernel's token
    chunk, a kernel shorter than four taps) against float64 autograd through the restatement's convolution."""
    import ttt_rs_b200 as tb
    from ttt_rs_b200.layer import _QkConvFn
    dev = torch.device("cuda:0")
    B, T, H = 2, 150, 3
    C, N = H * 64, H * 64 + 72  # the convolutions read a column block of a wider projection output
    g = torch.Generator().manual_seed(5)
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).to(dtype).double()  # noqa: E731
    proj, wq, bq, wk, bk = r(B, T, N), r(C, 1, K, sc=0.5), r(C, sc=0.1), r(C, 1, K, sc=0.5), r(C, sc=0.1)
    gq, gk = r(B, T, C), r(B, T, C)
    cfg = tb.TTTLayerConfig(hidden_size=C, num_heads=H, share_qk=True, conv_kernel_size=K)
    leaves = [t.to(dtype).to(dev).requires_grad_(True) for t in (proj, wq, bq, wk, bk)]
    q, k = _QkConvFn.apply(leaves[0], 0, C, leaves[1], leaves[2], leaves[3], leaves[4], cfg)
    torch.autograd.backward((q, k), (gq.to(dtype).to(dev), gk.to(dtype).to(dev)))
    torch.cuda.synchronize()
    ref = [t.clone().requires_grad_(True) for t in (proj, wq, bq, wk, bk)]
    qr = LO.causal_depthwise_conv(ref[0][..., :C], ref[1], ref[2])
    kr = LO.causal_depthwise_conv(ref[0][..., :C], ref[3], ref[4])
    torch.autograd.backward((qr, kr), (gq, gk))
    bf = dtype == torch.bfloat16
    rt, frac = (2e-2, 2e-3) if bf else (1e-4, 0.0)
    assert_close(q, qr, rt, "conv_q output", max_bad_frac=frac)
    assert_close(k, kr, rt, "conv_k output", max_bad_frac=frac)
    for name, a, b in zip(("d proj", "d conv_q_weight", "d conv_q_bias", "d conv_k_weight", "d conv_k_bias"), leaves, ref):
        assert_close(a.grad, b.grad, rt, name, max_bad_frac=frac)


@pytest.mark.gpu
def test_inference_forward_follows_in_place_parameter_updates(golden_dir):
    """The no_grad forward runs every projection as one GEMM over a cached concatenation of the q/k/v/g/lr weights.
    An optimizer step (an in-place update of a parameter) between two such forwards must be seen by the second:
    compare it with the restatement evaluated at the updated parameters."""
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    p = dict(_golden(golden_dir, "plain"))
    m, inner = _layer_from_params(tb, p, False, False, torch.float32, dev, 2)
    x = p["input"].float().to(dev)
    with torch.no_grad():
        y0 = m(x, inner, inner.init_state(x.shape[0]))
        m.q_proj.mul_(0.5)                      # what an optimizer does: same storage, new values
        m.learnable_ttt_lr_weight.add_(0.01)
        y1 = m(x, inner, inner.init_state(x.shape[0]))
    tb.check_status()
    p["q_proj"] = p["q_proj"] * 0.5
    p["lr_weight"] = p["lr_weight"] + 0.01
    want = LO.ttt_layer_forward(p["input"], p, num_heads=2)[0]
    assert_close(y1, want, 2e-4, "layer output after in-place parameter update")
    assert (y1 - y0).abs().max().item() > 1e-3, "the update must change the output"
