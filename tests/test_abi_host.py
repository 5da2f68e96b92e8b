"""CPU-only checks of the C ABI: the library loads, exports every declared symbol, and rejects bad arguments
with the documented error codes before touching a GPU (mirrors the reference's panics:
linear_fused_tile/mod.rs:143, forward/launch.rs:209-213, launch.rs:128-131)."""

import ctypes as C
import re
from pathlib import Path

import pytest

import ttt_rs_b200
from ttt_rs_b200 import _lib

REPO = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from ttt_rs_b200.build import build
    build()
    return _lib.load()


def _dims(**kw):
    d = dict(batch=2, heads=2, seq_len=64, head_dim=64, mini_batch=16, checkpoint_interval=4, epsilon=1e-6, dtype=1)
    d.update(kw)
    return _lib.TttDims(**d)


def test_every_declared_symbol_is_exported(lib):
    header = (REPO / "include" / "ttt_b200.h").read_text()
    declared = set(re.findall(r"\b(ttt_(?:b200|linear|mlp|layer|gemm)_\w+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in ttt_b200.h but not exported"
    assert declared == set(_lib.SYMBOLS), "ctypes binding and header disagree"
    assert lib.ttt_b200_abi_version() == 1


def test_checkpoint_and_workspace_sizes(lib):
    d = _dims(seq_len=80, checkpoint_interval=2)  # 5 stages -> 3 checkpoints
    assert lib.ttt_linear_num_checkpoints(C.byref(d)) == 3
    assert lib.ttt_linear_weight_ckpt_bytes(C.byref(d)) == 2 * 2 * (3 + 1) * 64 * 64 * 4
    rows, streams, ns = 2 * 2 * 80, 4, 5  # gradient tiles (bf16) + 32 B of statistics per token + per-stage biases
    assert lib.ttt_linear_bias_ckpt_bytes(C.byref(d)) == rows * 64 * 2 + rows * 32 + streams * (ns + 1) * 64 * 4
    streams = 4
    # LN partials per (stream, chunk), token_eta terms, float32 dW/db, chunk hand-off (W, dW, db), scheduler words
    assert lib.ttt_linear_backward_workspace_bytes(C.byref(d)) == 4 * (
        streams * 1 * 128 + streams * 80 + streams * (4096 + 64) + streams * (2 * 4096 + 64) + 8)


def test_sizes_for_mini_batch_8(lib):
    """8-token mini-batches: twice the stages, so twice the per-stage records; per-token records unchanged."""
    d = _dims(mini_batch=8, seq_len=80, checkpoint_interval=4)  # 10 stages -> 3 checkpoints
    assert lib.ttt_linear_num_checkpoints(C.byref(d)) == 3
    assert lib.ttt_linear_weight_ckpt_bytes(C.byref(d)) == 2 * 2 * (3 + 1) * 64 * 64 * 4
    rows, streams, ns = 2 * 2 * 80, 4, 10
    assert lib.ttt_linear_bias_ckpt_bytes(C.byref(d)) == rows * 64 * 2 + rows * 32 + streams * (ns + 1) * 64 * 4
    # the TTT-MLP kernels take 16-token mini-batches only
    assert lib.ttt_mlp_backward_workspace_bytes(C.byref(d)) == 0


def test_sizes_for_head_dim_32(lib):
    """Two 32-wide heads share a 64-wide tile: saved state is sized per pair, per-head results per head."""
    d = _dims(head_dim=32, heads=4, seq_len=80, checkpoint_interval=2)
    pairs, heads_all, ns = 2 * 2, 2 * 4, 5
    assert lib.ttt_linear_num_checkpoints(C.byref(d)) == 3
    assert lib.ttt_linear_weight_ckpt_bytes(C.byref(d)) == pairs * (3 + 1) * 64 * 64 * 4
    rows = pairs * 80
    assert lib.ttt_linear_bias_ckpt_bytes(C.byref(d)) == rows * 64 * 2 + rows * 64 + pairs * (ns + 1) * 64 * 4
    assert lib.ttt_linear_backward_workspace_bytes(C.byref(d)) == 4 * (
        pairs * 1 * 128 + heads_all * 80 + heads_all * (1024 + 32) + pairs * (2 * 4096 + 64) + 8)
    # the TTT-MLP kernels take head_dim 64 only
    assert lib.ttt_mlp_backward_workspace_bytes(C.byref(d)) == 0


@pytest.mark.parametrize("kw,code", [
    (dict(seq_len=70), _lib.TTT_ERR_SHAPE),              # not a multiple of the mini-batch
    (dict(mini_batch=32, seq_len=64), _lib.TTT_ERR_UNSUPPORTED),   # 32-token mini-batches are not built
    (dict(mini_batch=4, seq_len=64), _lib.TTT_ERR_UNSUPPORTED),
    (dict(head_dim=128), _lib.TTT_ERR_UNSUPPORTED),
    (dict(head_dim=32, heads=3), _lib.TTT_ERR_UNSUPPORTED),   # head_dim 32 pairs heads: needs an even count
    (dict(checkpoint_interval=0), _lib.TTT_ERR_SHAPE),
    (dict(batch=0), _lib.TTT_ERR_SHAPE),
    (dict(dtype=7), _lib.TTT_ERR_UNSUPPORTED),
])
def test_bad_dims_are_rejected(lib, kw, code):
    d = _dims(**kw)
    fake = C.c_void_p(0x1000)  # never dereferenced: validation fails first
    rc = lib.ttt_linear_forward(C.byref(d), *([fake] * 14), None, None)
    assert rc == code, _lib.last_error()
    assert _lib.last_error()
    assert lib.ttt_linear_num_checkpoints(C.byref(d)) == -1
    assert lib.ttt_linear_backward_workspace_bytes(C.byref(d)) == 0


def test_null_and_misaligned_pointers_are_rejected(lib):
    d = _dims()
    fake = C.c_void_p(0x1000)
    args = [fake] * 14
    args[3] = None
    assert lib.ttt_linear_forward(C.byref(d), *args, None, None) == _lib.TTT_ERR_NULL
    assert "weight" in _lib.last_error()
    args = [fake] * 14
    args[1] = C.c_void_p(0x1008)
    assert lib.ttt_linear_forward(C.byref(d), *args, None, None) == _lib.TTT_ERR_ALIGN
    assert "xk" in _lib.last_error()
    bargs = [fake] * 21 + [None, fake]
    assert lib.ttt_linear_backward(C.byref(d), *bargs, C.c_size_t(16), None, None) == _lib.TTT_ERR_WORKSPACE
    assert lib.ttt_linear_forward(None, *([fake] * 14), None, None) == _lib.TTT_ERR_NULL


def test_config_epsilon_scaling_matches_reference():
    # (1e-6f32 / 1e-9f32) as u32 == 1000 (rust/fused/src/lib.rs:298-311)
    cfg = ttt_rs_b200.FusedTttConfig.new(16, 64, 1e-6, 64)
    assert cfg.epsilon_scaled == 1000
    assert abs(cfg.epsilon() - 1e-6) < 1e-12
    assert cfg.checkpoint_interval == 1


def test_host_wrapper_refuses_cpu_tensors():
    import torch
    from oracle.ttt_oracle import make_inputs
    t = make_inputs(1, 1, 16, 64, 16, seed=0, dtype=torch.float32, with_grad_output=False)
    names = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")
    ins = ttt_rs_b200.TttInputs(*[t[k] for k in names])
    with pytest.raises(ttt_rs_b200.TttError):
        ttt_rs_b200.TttTileMultiKernel.forward_launch(ins, ttt_rs_b200.FusedTttConfig.new(16, 64, 1e-6))


def test_cpp_host_mirror_compiles(tmp_path):
    """The C++ mirror of the operator (host/fused_tile_multi.hpp) is valid C++17 against the public header."""
    import subprocess
    src = tmp_path / "t.cpp"
    src.write_text('#include "ttt_rs_b200/host/fused_tile_multi.hpp"\n'
                   'int main() { ttt_b200::FusedTttConfig c = ttt_b200::FusedTttConfig::make(16, 64, 1e-6f, 64);\n'
                   '  return c.epsilon_scaled == 1000 ? 0 : 1; }\n')
    exe = tmp_path / "t"
    r = subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", str(REPO), str(src), "-o", str(exe),
                        "-L", str(REPO / "ttt_rs_b200"), "-lttt_b200", f"-Wl,-rpath,{REPO / 'ttt_rs_b200'}"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert subprocess.run([str(exe)]).returncode == 0


def test_partial_and_layer_entry_points_validate_their_arguments(lib):
    """Argument checks of the entry points around the main path; all fail before anything touches the device."""
    fake = C.c_void_p(0x1000)
    # partial mini-batch: 1..16 tokens, head_dim 64 or 32
    for seq, code in ((0, _lib.TTT_ERR_SHAPE), (17, _lib.TTT_ERR_SHAPE)):
        assert lib.ttt_linear_forward_partial(C.byref(_dims(seq_len=seq)), *([fake] * 12), None) == code
    assert lib.ttt_linear_forward_partial(C.byref(_dims(seq_len=3, head_dim=48)), *([fake] * 12), None) == \
        _lib.TTT_ERR_UNSUPPORTED
    args = [fake] * 12
    args[9] = None
    assert lib.ttt_linear_forward_partial(C.byref(_dims(seq_len=3)), *args, None) == _lib.TTT_ERR_NULL
    assert "output" in _lib.last_error()

    # layer prologue
    d = _dims(seq_len=37)  # need not be a multiple of the mini-batch here

    def pro(src_ld=128, lr_ld=8, conv=(None, None, None, None), kc=0, start=0, mode=1, theta=10000.0, q=fake):
        return lib.ttt_layer_prologue(C.byref(d), q, fake, fake, src_ld, fake, lr_ld, None, *conv, kc, start, mode,
                                      theta, 1.0, fake, fake, fake, fake, None)

    assert pro(src_ld=120) == _lib.TTT_ERR_SHAPE          # narrower than heads * 64
    assert pro(src_ld=132) == _lib.TTT_ERR_SHAPE          # rows would lose 16-byte alignment
    assert pro(lr_ld=1) == _lib.TTT_ERR_SHAPE
    assert pro(mode=3) == _lib.TTT_ERR_UNSUPPORTED
    assert pro(theta=0.0) == _lib.TTT_ERR_SHAPE
    assert pro(start=-1) == _lib.TTT_ERR_SHAPE
    assert pro(conv=(fake, fake, fake, None), kc=4) == _lib.TTT_ERR_NULL
    assert pro(conv=(fake, fake, fake, fake), kc=5) == _lib.TTT_ERR_UNSUPPORTED
    assert pro(q=C.c_void_p(0x1004)) == _lib.TTT_ERR_ALIGN
    assert lib.ttt_layer_prologue(C.byref(_dims(head_dim=48)), *([fake] * 3), 128, fake, 8, *([None] * 5), 0, 0, 1,
                                  10000.0, 1.0, fake, fake, fake, fake, None) == _lib.TTT_ERR_UNSUPPORTED

    # layer epilogue
    def epi(dd=d, gate=None, gate_ld=0, w=fake, eps=1e-6):
        return lib.ttt_layer_epilogue(C.byref(dd), fake, gate, gate_ld, w, fake, eps, fake, None)

    assert epi(w=None) == _lib.TTT_ERR_NULL
    assert epi(gate=fake, gate_ld=64) == _lib.TTT_ERR_SHAPE
    assert epi(gate=fake, gate_ld=130) == _lib.TTT_ERR_SHAPE
    assert epi(gate=C.c_void_p(0x1004), gate_ld=128) == _lib.TTT_ERR_ALIGN
    assert epi(dd=_dims(heads=33)) == _lib.TTT_ERR_UNSUPPORTED
    assert epi(eps=-1.0) == _lib.TTT_ERR_SHAPE


def test_rust_declarations_in_the_integration_guide_match_the_header():
    """The integration guide carries the Rust `extern "C"` block a maintainer would paste; it is generated from the header.
    The committed text must equal a fresh generation, and every declaration must have as many arguments as the
    ctypes table that the tests call through."""
    import sys
    sys.path.insert(0, str(REPO / "include"))
    import gen_rust_ffi as G
    assert G.current_doc_block() == G.doc_block(), "run `python include/gen_rust_ffi.py --update`"
    decls = {name: params for _ret, name, params in G.declarations()}
    assert set(decls) == set(_lib.SYMBOLS)
    for name, (_res, argtypes) in _lib.SYMBOLS.items():
        assert len(decls[name]) == len(argtypes), f"{name}: header has {len(decls[name])} arguments, ctypes {len(argtypes)}"
    rust = G.rust_block()
    for name, params in decls.items():
        m = re.search(r"pub fn %s\((.*?)\)( ->|;)" % name, rust, flags=re.S)
        assert m is not None, name
        n_rust = 0 if not m.group(1).strip() else m.group(1).count(":")
        assert n_rust == len(params), f"{name}: Rust block has {n_rust} arguments, header {len(params)}"
