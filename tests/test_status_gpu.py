"""Device-side status words: a bounded wait that runs out is reported, not hung on.

The persistent TTT-Linear backward hands a stream's state from block to block; every such wait has an iteration limit.
The first test shortens the limit and starts the work-item counter past the items that would publish the first
hand-offs, so the wait can never be satisfied: the launch must return, report {TTT_ERR_TIMEOUT, 15, block, stage} and
leave the context usable.  Nothing here traps, faults or spins without a limit."""

import pytest
import torch

from oracle import ttt_oracle as O

pytestmark = pytest.mark.gpu

LIN_IN = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")
GRADS = LIN_IN


def _problem(tb, dev):
    # 2 x 2 streams of 32 mini-batches = two 16-stage work items per stream
    t = O.make_inputs(2, 2, 512, 64, 16, seed=3, dtype=torch.bfloat16)
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, 4)
    ins = tb.TttInputs(*[t[k].to(dev) for k in LIN_IN])
    go = t["grad_output"].to(dev)
    return cfg, ins, go


def test_handoff_wait_that_cannot_be_satisfied_gives_up_and_is_reported():
    import ttt_rs_b200 as tb
    from ttt_rs_b200 import _lib
    dev = torch.device("cuda:0")
    lib = _lib.load()
    cfg, ins, go = _problem(tb, dev)
    outs, saved = tb.TttTileMultiKernel.forward_launch(ins, cfg)
    good = tb.TttTileMultiKernel.backward_launch(saved, tb.TttOutputs(go, None, None), cfg)
    tb.check_status()
    streams = ins.xq.shape[0] * ins.xq.shape[1]
    try:
        lib.ttt_b200_debug_handoff(2000, streams)  # 2000 polls of ~100 ns; skip the last-chunk items of all streams
        bad = tb.TttTileMultiKernel.backward_launch(saved, tb.TttOutputs(go, None, None), cfg)
        torch.cuda.synchronize()  # the launch returns: no block waits past its limit
    finally:
        lib.ttt_b200_debug_handoff(0, 0)
    words = bad.status.cpu().tolist()
    assert words[0] == _lib.TTT_ERR_TIMEOUT and words[1] == 15, words
    assert 0 <= words[2] < 296 and words[3] == 15, words  # stage = last stage of the first chunk
    with pytest.raises(tb.TttError) as ei:
        tb.check_status()
    assert ei.value.code == _lib.TTT_ERR_TIMEOUT
    tb.check_status()  # the report was cleared when it was raised
    # the context is intact: the same launch with the default limits reproduces the earlier result bit for bit
    again = tb.TttTileMultiKernel.backward_launch(saved, tb.TttOutputs(go, None, None), cfg)
    tb.check_status()
    for n in GRADS:
        assert torch.equal(getattr(again, n), getattr(good, n)), n


def test_a_report_survives_later_launches_until_it_is_checked():
    """The status words are per device and written by compare-and-swap from zero: a report made by one launch is still
    there after any number of later launches, and `check_status` raises exactly once."""
    import ttt_rs_b200 as tb
    from ttt_rs_b200 import _lib
    from ttt_rs_b200.fused import device_status
    dev = torch.device("cuda:0")
    cfg, ins, go = _problem(tb, dev)
    tb.check_status()
    st = device_status(dev)
    st.copy_(torch.tensor([_lib.TTT_ERR_TIMEOUT, 1, 7, 3] + [0] * 12, dtype=torch.int32))
    outs, saved = tb.TttTileMultiKernel.forward_launch(ins, cfg)
    g = tb.TttTileMultiKernel.backward_launch(saved, tb.TttOutputs(go, None, None), cfg)
    assert saved.status is st and g.status is st
    with pytest.raises(tb.TttError) as ei:
        tb.check_status(dev)
    assert "where=1" in str(ei.value) and "block=7" in str(ei.value)
    tb.check_status(dev)


def test_launch_on_a_device_other_than_the_current_one():
    """Tensors on cuda:1 while cuda:0 is current: the wrappers switch device for the call."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import ttt_rs_b200 as tb
    t = O.make_inputs(1, 2, 64, 64, 16, seed=0, dtype=torch.bfloat16)
    cfg = tb.FusedTttConfig.new(16, 64, 1e-6, 128, 2)
    torch.cuda.set_device(0)
    res = []
    for d in (0, 1):
        dev = torch.device("cuda", d)
        ins = tb.TttInputs(*[t[k].to(dev) for k in LIN_IN])
        outs, saved = tb.TttTileMultiKernel.forward_launch(ins, cfg)
        g = tb.TttTileMultiKernel.backward_launch(saved, tb.TttOutputs(t["grad_output"].to(dev), None, None), cfg)
        tb.check_status(dev)
        res.append((outs.output.cpu(), g.xk.cpu()))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
