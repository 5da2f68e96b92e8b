"""Seeded synthetic operands of the fused TTT inner loop (benchmark workloads and parity-test cases).

The reference benchmarks this path on synthetic tensors as well (rust/cli/src/bench.rs:112,171,
rust/core/src/test_utils.rs:126-156); no dataset is involved.
"""

from __future__ import annotations

import math
from typing import Dict

import torch


def make_inputs(B: int, H: int, T: int, F: int = 64, mini_batch: int = 16, seed: int = 0,
                dtype: torch.dtype = torch.float32, inner: str = "linear",
                with_grad_output: bool = True) -> Dict[str, torch.Tensor]:
    """Seeded synthetic operands with the benchmark's shapes and distributions.

    One CPU generator, f32, drawn in this fixed order: XQ, XK, XV ~ N(0,1)/sqrt(F);
    W0 ~ N(0,0.02) [H,F,F] repeated over B (MLP: W1 [H,F,4F], W2 [H,4F,F]); biases 0;
    LN gamma = 1, beta = 0; logits ~ N(0,1) [B,H,T], lr = (1/F)*sigmoid(logits);
    token_eta[t] = 1/((t mod CS)+1) (rust/layer/src/ttt.rs:106-110,
    rust/core/src/test_utils.rs:133-142); upstream grad ~ N(0, 1e-2).
    Values are rounded to `dtype` once and returned in `dtype`.
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    shp = (B, H, T, F)
    scale = 1.0 / math.sqrt(F)
    d: Dict[str, torch.Tensor] = {}
    d["xq"] = torch.randn(shp, generator=g) * scale
    d["xk"] = torch.randn(shp, generator=g) * scale
    d["xv"] = torch.randn(shp, generator=g) * scale
    if inner == "linear":
        w0 = torch.randn(H, F, F, generator=g) * 0.02
        d["weight"] = w0.unsqueeze(0).repeat(B, 1, 1, 1)
        d["bias"] = torch.zeros(B, H, F)
    else:
        E = 4 * F
        w1 = torch.randn(H, F, E, generator=g) * 0.02
        w2 = torch.randn(H, E, F, generator=g) * 0.02
        d["w1"] = w1.unsqueeze(0).repeat(B, 1, 1, 1)
        d["b1"] = torch.zeros(B, H, E)
        d["w2"] = w2.unsqueeze(0).repeat(B, 1, 1, 1)
        d["b2"] = torch.zeros(B, H, F)
    d["ln_weight"] = torch.ones(H, F)
    d["ln_bias"] = torch.zeros(H, F)
    logits = torch.randn(B, H, T, generator=g)
    d["ttt_lr_eta"] = (1.0 / F) * torch.sigmoid(logits)
    d["token_eta"] = 1.0 / ((torch.arange(T) % mini_batch) + 1).to(torch.float32)
    if with_grad_output:
        d["grad_output"] = torch.randn(shp, generator=g) * 1e-2
    return {k: v.to(dtype).contiguous() for k, v in d.items()}
