"""The projection GEMM (`ttt_gemm_bf16_tn`: tcgen05.mma, accumulators in tensor memory, TMA in and out) against a
float64 product of the same bf16 operands.  The result is rounded to bf16 once, so the bound is bf16 rounding of the
exact value: 2^-8 relative to each element plus a float32-accumulation floor."""

import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [
    (128, 128, 64),      # one tile, one k-block
    (128, 128, 768),     # the ring wraps (12 k-blocks over 3 stages)
    (256, 200, 768),     # N not a multiple of the tile: clipped store, second half-tile partly out of range
    (1000, 2320, 768),   # ragged M; the layer's fused projection width at 12 heads
    (300, 72, 104),      # ragged everything: K tail zero-filled by the tensor map, N < 128
    (4096, 768, 768),    # o_proj at the 125M layer shape
    (640, 520, 256),     # CTA-pair form (M >= 512) with an odd number of 128-row blocks: the second CTA of the last
                         # pair has no rows; last tile column 8 wide
    (1152, 288, 64),     # pair form, one k-block, last tile column 32 wide (16 columns from each CTA of the pair)
    (1024, 72, 104),     # pair form with ragged N and a K tail that the tensor maps fill with zeros
])
def test_gemm_matches_float64_product(M, N, K):
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    c = tb.gemm_bf16_tn(a.to(dev), b.to(dev))
    tb.check_status()
    want = a.double() @ b.double().t()
    assert c.shape == (M, N) and c.dtype == torch.bfloat16
    assert_close(c, want, 4e-3, f"gemm {M}x{N}x{K}")


def test_gemm_with_row_pitch_larger_than_the_row():
    """Operands and result as column blocks of wider buffers (how the layer slices its fused projection)."""
    import ctypes as C
    import ttt_rs_b200 as tb
    from ttt_rs_b200 import _lib
    dev = torch.device("cuda:0")
    M, N, K = 384, 136, 128
    g = torch.Generator().manual_seed(1)
    abuf = (torch.randn(M, K + 64, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    bbuf = (torch.randn(N, K + 8, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    cbuf = torch.full((M, N + 24), 7.0, dtype=torch.bfloat16, device=dev)
    lib = _lib.load()
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    _lib.check(lib.ttt_gemm_bf16_tn(M, N, K, p(abuf), abuf.stride(0), p(bbuf), bbuf.stride(0), p(cbuf), cbuf.stride(0),
                                    None, C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    torch.cuda.synchronize()
    want = abuf[:, :K].double().cpu() @ bbuf[:, :K].double().cpu().t()
    assert_close(cbuf[:, :N], want, 4e-3, "gemm into a column block")
    assert (cbuf[:, N:] == 7.0).all(), "columns beyond N must not be written"


def test_gemm_rejects_bad_arguments():
    import ctypes as C
    from ttt_rs_b200 import _lib
    lib = _lib.load()
    fake = C.c_void_p(0x1000)
    assert lib.ttt_gemm_bf16_tn(0, 8, 8, fake, 8, fake, 8, fake, 8, None, None) == _lib.TTT_ERR_SHAPE
    assert lib.ttt_gemm_bf16_tn(8, 8, 8, fake, 4, fake, 8, fake, 8, None, None) == _lib.TTT_ERR_SHAPE
    assert lib.ttt_gemm_bf16_tn(8, 8, 8, fake, 12, fake, 8, fake, 8, None, None) == _lib.TTT_ERR_ALIGN
    assert lib.ttt_gemm_bf16_tn(8, 8, 8, None, 8, fake, 8, fake, 8, None, None) == _lib.TTT_ERR_NULL


@pytest.mark.parametrize("use_gate,pos,start", ((False, "rope", 0), (True, "rope", 37), (True, "none", 0)))
def test_fused_projections_match_gemm_then_prologue_and_the_restatement(use_gate, pos, start):
    """`ttt_layer_projections` (GEMM with the head split, rotary rotation and learning-rate gate in its epilogue)
    against the float64 restatement on the same bf16 operands, and against the two-launch path (GEMM, then
    ttt_layer_prologue) it replaces."""
    import ttt_rs_b200 as tb
    from oracle import ttt_layer_oracle as LO
    dev = torch.device("cuda:0")
    B, T, H = (5, 128, 3) if start else (2, 256, 3)  # 5 x 128 rows: the pair form with an odd number of row blocks
    Cc = H * 64
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(B, T, Cc, generator=g) * 0.5).to(torch.bfloat16)
    blocks = {n: (torch.randn(Cc, Cc, generator=g) * Cc ** -0.5).to(torch.bfloat16) for n in ("q", "k", "v")}
    if use_gate:
        blocks["g"] = (torch.randn(Cc, Cc, generator=g) * Cc ** -0.5).to(torch.bfloat16)
    lrw = (torch.randn(H, Cc, generator=g) * 0.02).to(torch.bfloat16)
    lr_bias = (torch.randn(H, generator=g) * 0.1).to(torch.bfloat16)
    cols, off, rows = {}, 0, []
    for n, w in blocks.items():
        cols[n] = off
        off += Cc
        rows.append(w)
    cols["lr"] = off
    rows += [lrw, torch.zeros((-(off + H)) % 8, Cc, dtype=torch.bfloat16)]
    wcat = torch.cat(rows, dim=0).contiguous()
    cfg = tb.TTTLayerConfig(hidden_size=Cc, num_heads=H, use_gate=use_gate, pos_encoding=pos)
    xq, xk, xv, lr, gate = tb.layer_projections(x.to(dev), wcat.to(dev), cols, cfg, lr_bias.to(dev), start)
    tb.check_status()

    # float64 restatement on the bf16 operands
    proj = x.double() @ wcat.double().t()
    heads = lambda t: t.reshape(B, T, H, 64).permute(0, 2, 1, 3)  # noqa: E731
    wq, wk, wv = (heads(proj[..., cols[n]:cols[n] + Cc]) for n in ("q", "k", "v"))
    if pos == "rope":
        posv = (start + torch.arange(T)) % 16
        wq, wk = LO.rope_pairs(wq, posv, 10000.0), LO.rope_pairs(wk, posv, 10000.0)
    wlr = torch.sigmoid(proj[..., cols["lr"]:cols["lr"] + H].permute(0, 2, 1) + lr_bias.double().reshape(1, H, 1)) / 64
    for name, got, want in (("xq", xq, wq), ("xk", xk, wk), ("xv", xv, wv), ("ttt_lr_eta", lr, wlr)):
        assert_close(got, want, 4e-3, f"fused projections: {name}")
    if use_gate:
        assert_close(gate.reshape(B, T, Cc), proj[..., cols["g"]:cols["g"] + Cc], 4e-3, "fused projections: gate")
    else:
        assert gate is None

    # the two-launch path rounds the projection to bf16 before rotating: same values to bf16 rounding
    p2 = tb.gemm_bf16_tn(x.reshape(B * T, Cc).to(dev), wcat.to(dev)).reshape(B, T, -1)
    uq, uk, uv, ulr = tb.layer_prologue(p2, cfg, q_col=cols["q"], k_col=cols["k"], v_col=cols["v"], lr_col=cols["lr"],
                                        lr_bias=lr_bias.to(dev), start_idx=start)
    assert torch.equal(uv, xv), "v is a pure copy of the product in both paths"
    assert_close(xq, uq.double(), 1.6e-2, "fused vs two-launch: xq")
    assert_close(lr, ulr.double(), 1.6e-2, "fused vs two-launch: ttt_lr_eta")
