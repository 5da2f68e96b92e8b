"""The host-buffer runner (chunked, three streams) gives the same results as one direct call."""

import pytest
import torch

from oracle import ttt_oracle as O

pytestmark = pytest.mark.gpu
LIN_IN = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")


def test_host_runner_matches_direct_call():
    import ttt_rs_b200 as tb
    from ttt_rs_b200.host_io import HostBatchRunner, alloc_host_outputs
    dev = torch.device("cuda:0")
    B, H, T = 5, 2, 128
    t = O.make_inputs(B, H, T, 64, 16, seed=31, dtype=torch.bfloat16)
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, 4)
    ins = tb.TttInputs(*[t[k].to(dev) for k in LIN_IN])
    outs, saved = tb.TttTileMultiKernel.forward_launch(ins, cfg)
    g = tb.TttTileMultiKernel.backward_launch(saved, tb.TttOutputs(t["grad_output"].to(dev), None, None), cfg)
    torch.cuda.synchronize()

    pinned = {k: t[k].pin_memory() for k in ("xq", "xk", "xv", "ttt_lr_eta", "grad_output")}
    params = {k: t[k].to(dev) for k in ("weight", "bias", "token_eta", "ln_weight", "ln_bias")}
    host_out = alloc_host_outputs(B, H, T, 64, torch.bfloat16)
    runner = HostBatchRunner(cfg, dev, chunks=3)
    for _ in range(2):  # second run reuses the device buffers
        runner.run(pinned, params, host_out)
        torch.cuda.synchronize()
    assert torch.equal(host_out["output"], outs.output.cpu())
    for k, v in (("grad_xq", g.xq), ("grad_xk", g.xk), ("grad_xv", g.xv), ("grad_ttt_lr_eta", g.ttt_lr_eta),
                 ("grad_weight", g.weight), ("grad_bias", g.bias)):
        assert torch.equal(host_out[k], v.cpu()), k
    # batch-summed gradients are added chunk by chunk: same values up to bf16 rounding of the partial sums
    for k, v in (("grad_token_eta", g.token_eta), ("grad_ln_weight", g.ln_weight), ("grad_ln_bias", g.ln_bias)):
        a, b = host_out[k].float(), v.cpu().float()
        assert (a - b).abs().max() <= 2e-2 * (b.abs().max() + 1e-6), k
