"""World-size-2 test of the multi-rank host logic on CPU (gloo): batch sharding plus the single all-reduce of the
packed outer-parameter gradients reproduces the single-process gradients.  The per-rank compute is the CPU oracle
(no GPU here); the GPU kernels fill the same packed layout (tests/test_linear_backward_gpu.py)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ttt_oracle as O
from ttt_rs_b200 import distributed as D

LIN_IN = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")
B, H, T = 5, 2, 48  # odd batch: ranks own 3 and 2 rows


def _inputs():
    return O.make_inputs(B, H, T, 64, 16, seed=17, dtype=torch.float64)


def _packed(t):
    bw = O.ttt_linear_backward(*[t[k] for k in LIN_IN], t["grad_output"])
    return D.pack_outer_grads(bw["grad_weight"], bw["grad_bias"], bw["grad_ln_weight"], bw["grad_ln_bias"],
                              bw["grad_token_eta"]).double(), bw


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        t = _inputs()
        a, b = D.shard_batch(B, rank, world)
        mine = {k: (v[a:b] if v.dim() >= 3 else v) for k, v in t.items()}
        packed, _ = _packed(mine)
        D.allreduce_outer_grads(packed)
        ret[rank] = packed
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_batch_covers_batch_without_overlap():
    for batch in (1, 5, 32):
        for world in (1, 2, 4, 8):
            spans = [D.shard_batch(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        D.shard_batch(4, 2, 2)


def test_pack_unpack_roundtrip():
    _, bw = _packed(_inputs())
    p = D.pack_outer_grads(bw["grad_weight"], bw["grad_bias"], bw["grad_ln_weight"], bw["grad_ln_bias"],
                           bw["grad_token_eta"])
    u = D.unpack_outer_grads(p, H)
    assert u["weight"].shape == (H, 64, 64) and u["token_eta"].shape == (16,)
    assert torch.allclose(u["bias"].double(), bw["grad_bias"].sum(0), rtol=1e-6)
    assert p.numel() == H * 64 * 64 + 3 * H * 64 + 16
    with pytest.raises(ValueError):
        D.unpack_outer_grads(p[:-1], H)


def test_two_ranks_allreduce_matches_single_process():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    full, _ = _packed(_inputs())
    for r in range(world):
        # the packed buffer is float32 by definition
        assert torch.allclose(ret[r], full, rtol=1e-5, atol=1e-6 * full.abs().max().item()), f"rank {r}"


def test_benchmark_shards_are_the_batch_rows_of_the_same_tensors():
    """`bench.py --gpus N` (strong scaling) gives rank r the rows [r B/N, (r+1) B/N) of the seed-0 tensors: the shards
    tile the batch, per-stream tensors are cut, shared parameters are passed whole."""
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench
    t = O.make_inputs(8, 2, 32, 64, 16, seed=0, dtype=torch.float32)
    world = 4
    parts = [bench.shard_rows(t, *D.shard_batch(8, r, world)) for r in range(world)]
    for k, v in t.items():
        if v.dim() >= 3:
            assert torch.equal(torch.cat([p[k] for p in parts], dim=0), v), k
        else:
            assert all(p[k] is v for p in parts), k
