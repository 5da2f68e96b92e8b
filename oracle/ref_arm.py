"""The reference's own CPU implementation of the inner loop, for the benchmark's reference arm.

TEST / MEASUREMENT INFRASTRUCTURE: only tests/, __graft_entry__ and bench.py's CPU legs may use this module; the
product package never imports it.

The reference ships a PyTorch module (`reference/ttt.py` in its repository: `TTTLinear.ttt` :925, `TTTMLP.ttt` :1081,
the mini-batch scan :431; its Rust integration tests use it as ground truth, rust/cli/tests/validate_full.rs:1-10).
`stage()` copies that file, unmodified, from a reference checkout into `oracle/_ref/reference/` (git-ignored: the
copy is never committed); `step()` runs one forward (+ autograd backward) of it on host tensors.  Where no checkout
was available at build time `available()` is False and the caller falls back to the restatement in ttt_oracle.py.
"""

from __future__ import annotations

import importlib
import shutil
import sys
from pathlib import Path
from typing import Dict

import torch

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
_FILES = ("__init__.py", "ttt.py")


def stage(reference_root) -> bool:
    """Copy the reference's PyTorch module from `<reference_root>/reference/` into oracle/_ref/reference/.
    Returns True when the copy exists afterwards."""
    src = Path(reference_root) / "reference"
    dst = REF_DIR / "reference"
    if all((src / f).exists() for f in _FILES):
        dst.mkdir(parents=True, exist_ok=True)
        for f in _FILES:
            shutil.copyfile(src / f, dst / f)
        (REF_DIR / "SOURCE.txt").write_text(
            "unmodified copies of reference/__init__.py and reference/ttt.py of the reference repository, made by "
            "oracle/ref_arm.py:stage(); not part of this repository's history\n")
    return available()


def available() -> bool:
    return all((REF_DIR / "reference" / f).exists() for f in _FILES)


_mod = None


def module():
    global _mod
    if _mod is None:
        if not available():
            raise RuntimeError("oracle/_ref/reference is missing: run __graft_entry__.build() next to a reference checkout")
        if str(REF_DIR) not in sys.path:
            sys.path.insert(0, str(REF_DIR))
        _mod = importlib.import_module("reference.ttt")
    return _mod


def step(t: Dict[str, torch.Tensor], inner: str = "linear", mini_batch: int = 16, backward: bool = True):
    """One pass of the reference's `.ttt()` over host tensors shaped like the benchmark's ([B,H,T,F] etc., float32):
    forward, and with `backward` the gradients of all inputs by autograd for upstream gradient t["grad_output"].
    token_eta enters as its first `mini_batch` entries repeated over the stages, which is what the fused kernels read
    (forward/kernel.rs:152-165)."""
    ref = module()
    B, H, T, F = t["xq"].shape
    cs, ns = mini_batch, T // mini_batch
    cfg = ref.TTTConfig(hidden_size=H * F, num_attention_heads=H, mini_batch_size=cs,
                        ttt_layer_type=inner, ttt_base_lr=1.0)
    m = (ref.TTTLinear if inner == "linear" else ref.TTTMLP)(cfg, layer_idx=0)
    m.eval()
    dtype = t["xq"].dtype
    m = m.to(dtype)
    leaves = {k: v.detach().clone().requires_grad_(backward) for k, v in t.items()
              if k not in ("grad_output", "token_eta", "ln_weight", "ln_bias")}
    m.ttt_norm_weight = torch.nn.Parameter(t["ln_weight"].detach().clone())
    m.ttt_norm_bias = torch.nn.Parameter(t["ln_bias"].detach().clone())
    te = t["token_eta"][:cs].repeat(ns).clone().requires_grad_(backward)

    def stg(x):
        return x.reshape(B, H, ns, cs, *x.shape[3:])

    token_eta = te.reshape(1, 1, ns, cs, 1).expand(B, H, ns, cs, 1)
    lr = stg(leaves["ttt_lr_eta"]).unsqueeze(-2)
    inputs = {"XQ": stg(leaves["xq"]), "XK": stg(leaves["xk"]), "XV": stg(leaves["xv"]),
              "eta": token_eta * lr, "token_eta": token_eta, "ttt_lr_eta": lr}
    if inner == "linear":
        init = {"W1_states": leaves["weight"], "b1_states": leaves["bias"].unsqueeze(-2)}
    else:
        init = {"W1_states": leaves["w1"], "b1_states": leaves["b1"].unsqueeze(-2),
                "W2_states": leaves["w2"], "b2_states": leaves["b2"].unsqueeze(-2)}
    for k in list(init):
        init[k.replace("_states", "_grad")] = torch.zeros_like(init[k])
    ctx = torch.enable_grad() if backward else torch.no_grad()
    with ctx:
        out, _ = m.ttt(inputs, mini_batch_size=cs, last_mini_batch_params_dict=init, cache_params=None)
        out = out.reshape(B, T, H, F).transpose(1, 2)
        grads = None
        if backward:
            wrt = list(leaves.values()) + [m.ttt_norm_weight, m.ttt_norm_bias, te]
            grads = torch.autograd.grad(out, wrt, grad_outputs=t["grad_output"])
    return out.detach(), grads
