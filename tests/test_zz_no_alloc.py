"""`ttt_linear_backward_noalloc`: the backward for hosts that cannot provide a workspace.

Some callers of this library have no way to get device memory at the moment the backward is issued: a custom-op
hook that only receives the operator's input and output buffers, a runtime whose memory pool already owns the
device, a training loop that bans cudaMalloc on the hot path because it stalls every stream.  For them the library
keeps the per-stream partial sums in a fixed array of its own (TTT_NOALLOC_SCRATCH_BYTES) instead of a workspace.

The test calls the new entry point and the regular one through the C ABI on the same saved state and requires the
same results, twice in a row with different inputs (the array is shared by all calls and keeps the previous
call's contents, so a second call would expose anything that wrongly depended on a clean array).
"""

import ctypes as C

import pytest
import torch

from conftest import assert_close
from oracle import ttt_oracle as O

LIN_IN = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _backward_both_ways(seed, B, H, NS, K, dtype, F=64):
    import ttt_rs_b200 as tb
    from ttt_rs_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    t = O.make_inputs(B, H, NS * 16, F, 16, seed=seed, dtype=dtype)
    cfg = tb.FusedTttConfig.new(16, F, 1e-6, 128, K)
    ins = tb.TttInputs(*[t[k].to(dev) for k in LIN_IN])
    _, saved = tb.TttTileMultiKernel.forward_launch(ins, cfg)
    go = t["grad_output"].to(dev)
    T = NS * 16
    d = _lib.TttDims(B, H, T, F, 16, K, float(cfg.epsilon()), _lib.TTT_BF16 if dtype == torch.bfloat16 else _lib.TTT_F32)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def outputs():
        return dict(
            xq=torch.empty_like(saved.xq), xk=torch.empty_like(saved.xq), xv=torch.empty_like(saved.xq),
            w=torch.empty_like(saved.weight_init), b=torch.empty_like(saved.bias), lr=torch.empty_like(saved.ttt_lr_eta),
            te=torch.empty(T, device=dev), lnw=torch.empty(H, F, device=dev), lnb=torch.empty(H, F, device=dev),
            packed=torch.empty(tb.packed_outer_grad_len(H, F), device=dev))

    common = [_ptr(saved.xq), _ptr(saved.xk), _ptr(saved.xv), _ptr(saved.weight_init), _ptr(saved.bias),
              _ptr(saved.token_eta), _ptr(saved.ttt_lr_eta), _ptr(saved.ln_weight), _ptr(saved.ln_bias),
              _ptr(saved.weight_checkpoints), _ptr(saved.bias_checkpoints), _ptr(go)]

    def outs_ptrs(o):
        return [_ptr(o[k]) for k in ("xq", "xk", "xv", "w", "b", "lr", "te", "lnw", "lnb", "packed")]

    ref = outputs()
    ws_bytes = lib.ttt_linear_backward_workspace_bytes(C.byref(d))
    assert 0 < ws_bytes <= _lib.NOALLOC_SCRATCH_BYTES
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    _lib.check(lib.ttt_linear_backward(C.byref(d), *common, *outs_ptrs(ref), _ptr(ws), C.c_size_t(ws_bytes), None, stream))
    got = outputs()
    _lib.check(lib.ttt_linear_backward_noalloc(C.byref(d), *common, *outs_ptrs(got), None, stream))
    torch.cuda.synchronize()
    return got, ref


@pytest.mark.gpu
def test_noalloc_backward_matches_workspace_backward_twice_in_a_row():
    rtol = {torch.bfloat16: 2e-2, torch.float32: 1e-4}
    # two calls back to back, different sizes and data; then a third in float32; then head_dim 32 (pairs of heads)
    for seed, (B, H, NS, K), dtype, F in ((1, (3, 2, 8, 4), torch.bfloat16, 64), (2, (2, 4, 20, 16), torch.bfloat16, 64),
                                          (3, (1, 2, 5, 2), torch.float32, 64), (4, (2, 4, 6, 4), torch.bfloat16, 32)):
        got, ref = _backward_both_ways(seed, B, H, NS, K, dtype, F)
        for k in ref:
            assert_close(got[k], ref[k].double(), rtol[dtype], f"seed {seed}: {k}")
            # the kernels are deterministic, so the two entry points agree to the bit
            assert torch.equal(got[k], ref[k]), f"seed {seed}: {k} differs bitwise"


def test_noalloc_backward_rejects_problems_larger_than_its_scratch():
    """Needs no GPU: the size check comes before anything touches the device.  (The library is built first if it is
    not there yet, so the test also passes alone on a fresh checkout.)"""
    from ttt_rs_b200 import _lib
    from ttt_rs_b200.build import build
    build()
    lib = _lib.load()
    d = _lib.TttDims(64, 32, 8192, 64, 16, 16, 1e-6, _lib.TTT_BF16)  # 2048 streams x ~24,700 floats = 200 MB
    assert lib.ttt_linear_backward_workspace_bytes(C.byref(d)) > _lib.NOALLOC_SCRATCH_BYTES
    fake = C.c_void_p(0x1000)
    rc = lib.ttt_linear_backward_noalloc(C.byref(d), *([fake] * 21), None, None, None)
    assert rc == _lib.TTT_ERR_WORKSPACE
    assert "built-in scratch" in _lib.last_error()
