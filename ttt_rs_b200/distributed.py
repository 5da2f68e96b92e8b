"""Multi-GPU plumbing for the fused TTT inner loop: one process per GPU over torch.distributed.

The (batch x head) streams are independent, so ranks shard the batch and the forward needs no communication.
Training needs exactly one exchange per layer: the sum over ranks of the gradients of the parameters every stream
shares -- dW0 [H,F,F], db0 [H,F], d ln_weight [H,F], d ln_bias [H,F], d token_eta [CS] -- which the backward packs
into one float32 buffer (`outer_grad_packed`).  (The reference is single-device; these sums are what Burn's
`repeat_dim` backward and the float atomics of rust/fused/src/linear_fused_tile/backward/types.rs:28-39 produce
within one device.)
"""

from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.distributed as dist


def shard_batch(batch: int, rank: int, world: int) -> Tuple[int, int]:
    """[start, stop) of the batch rows rank `rank` owns; the first `batch % world` ranks get one extra row."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def packed_layout(heads: int, head_dim: int = 64, mini_batch: int = 16) -> Dict[str, Tuple[int, int, tuple]]:
    """name -> (offset, length, shape) inside the packed float32 buffer."""
    H, F = heads, head_dim
    out, o = {}, 0
    for name, shape in (("weight", (H, F, F)), ("bias", (H, F)), ("ln_weight", (H, F)), ("ln_bias", (H, F)),
                        ("token_eta", (mini_batch,))):
        n = 1
        for s in shape:
            n *= s
        out[name] = (o, n, shape)
        o += n
    return out


def pack_outer_grads(grad_weight, grad_bias, grad_ln_weight, grad_ln_bias, grad_token_eta,
                     mini_batch: int = 16) -> torch.Tensor:
    """Host-side equivalent of what the backward kernel writes to `outer_grad_packed`: per-batch dW/db summed over
    the batch, LN gradients as they are, the [T] token_eta gradient folded over stages to [CS]."""
    parts = [grad_weight.sum(0), grad_bias.sum(0), grad_ln_weight, grad_ln_bias,
             grad_token_eta.reshape(-1, mini_batch).sum(0)]
    return torch.cat([p.reshape(-1).float() for p in parts])


def unpack_outer_grads(packed: torch.Tensor, heads: int, head_dim: int = 64, mini_batch: int = 16):
    lay = packed_layout(heads, head_dim, mini_batch)
    if packed.numel() != sum(n for _, n, _ in lay.values()):
        raise ValueError(f"packed buffer has {packed.numel()} elements, expected {sum(n for _, n, _ in lay.values())}")
    return {k: packed[o:o + n].reshape(shape) for k, (o, n, shape) in lay.items()}


def allreduce_outer_grads(packed: torch.Tensor, group=None, async_op: bool = False):
    """Sum the packed outer-parameter gradients over the ranks (one collective per layer)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return None
    return dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
