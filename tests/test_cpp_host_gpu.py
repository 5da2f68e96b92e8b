"""The C++ host mirror (host/fused_tile_multi.hpp) run as a compiled program gives the same bits as the ctypes path."""

import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import ttt_oracle as O

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent
LIN_IN = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")


def _raw(t):
    return t.contiguous().view(torch.int16).numpy().tobytes() if t.dtype == torch.bfloat16 else t.contiguous().numpy().tobytes()


def test_cpp_host_mirror_roundtrip(tmp_path):
    import ttt_rs_b200 as tb
    exe = tmp_path / "host_mirror_roundtrip"
    cuda = Path("/usr/local/cuda")
    r = subprocess.run(["g++", "-std=c++17", "-O1", "-I", str(REPO), "-I", str(cuda / "include"),
                        str(REPO / "tests" / "cpp" / "host_mirror_roundtrip.cpp"), "-o", str(exe),
                        "-L", str(REPO / "ttt_rs_b200"), "-lttt_b200", "-L", str(cuda / "lib64"), "-lcudart",
                        f"-Wl,-rpath,{REPO / 'ttt_rs_b200'}", f"-Wl,-rpath,{cuda / 'lib64'}"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    B, H, T, K = 2, 3, 96, 4
    t = O.make_inputs(B, H, T, 64, 16, seed=77, dtype=torch.bfloat16)
    for k in LIN_IN + ("grad_output",):
        (tmp_path / f"{k}.bin").write_bytes(_raw(t[k]))
    r = subprocess.run([str(exe), str(tmp_path), str(B), str(H), str(T), str(K)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr

    dev = torch.device("cuda:0")
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, K)
    outs, saved = tb.TttTileMultiKernel.forward_launch(tb.TttInputs(*[t[k].to(dev) for k in LIN_IN]), cfg)
    g = tb.TttTileMultiKernel.backward_launch(saved, tb.TttOutputs(t["grad_output"].to(dev), None, None), cfg)
    torch.cuda.synchronize()

    def bf(name, shape):
        a = np.frombuffer((tmp_path / name).read_bytes(), dtype=np.int16).reshape(shape)
        return torch.from_numpy(a.copy()).view(torch.bfloat16)

    assert torch.equal(bf("out_output.bin", (B, H, T, 64)), outs.output.cpu())
    assert torch.equal(bf("out_weight.bin", (B, H, 64, 64)), outs.weight.cpu())
    assert torch.equal(bf("out_grad_xq.bin", (B, H, T, 64)), g.xq.cpu())
    assert torch.equal(bf("out_grad_xk.bin", (B, H, T, 64)), g.xk.cpu())
    assert torch.equal(bf("out_grad_xv.bin", (B, H, T, 64)), g.xv.cpu())
    assert torch.equal(bf("out_grad_weight.bin", (B, H, 64, 64)), g.weight.cpu())
    te = torch.from_numpy(np.frombuffer((tmp_path / "out_grad_token_eta.bin").read_bytes(), dtype=np.float32).copy())
    assert torch.equal(te.to(torch.bfloat16), g.token_eta.cpu())
