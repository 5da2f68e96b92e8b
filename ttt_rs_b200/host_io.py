"""Running the operator on batches that live in (pinned) host memory.

The streams of a batch are independent, so a host-resident batch is cut into chunks of batch rows and the three
phases of each chunk -- host-to-device copy of xq/xk/xv/ttt_lr_eta/grad_output, forward + backward, device-to-host
copy of the output and gradients -- run on three CUDA streams, so that the PCIe transfers in both directions overlap
the kernels of neighbouring chunks.  Gradients that are sums over the batch (token_eta, LayerNorm weight/bias) are
accumulated on the device across chunks and copied once.  The small per-row tensors (ttt_lr_eta in; its gradient and
the state gradients out) also cross the link once per step, not once per chunk: a copy of a few hundred KB costs
about 15 us of link time whatever its size, and forty of them per step were 0.6 ms of an 11 ms step (measured).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .fused import FusedTttConfig, TttInputs, TttOutputs, TttTileMultiKernel

_IN = ("xq", "xk", "xv")  # copied chunk by chunk (+ grad_output); ttt_lr_eta is copied whole
_SMALL_OUT = ("grad_ttt_lr_eta", "grad_weight", "grad_bias")  # gathered on the device, copied whole


def chunk_bounds(batch: int, chunks: int, taper: bool = True):
    """Row boundaries of the batch chunks.  With `taper` the first and last chunks are smaller (weights 1, 2, 4, ...,
    4, 2, 1): the pipeline's fill (first copy-in + first kernels) and drain (last kernels + last copy-out) then cost a
    fraction of a full chunk, while the total number of chunks -- each costs a fixed, latency-bound kernel time --
    stays small.  Without it the chunks are as equal as the batch allows, which is what a link-bound step wants: the
    copy-out of a chunk can only start after the copy-in of the same chunk, so wherever a chunk is larger than the one
    before it the copy-out stream waits."""
    n = max(1, min(chunks, batch))
    if not taper or n < 5:
        return [(batch * c) // n for c in range(n + 1)]
    w = [1.0, 2.0] + [4.0] * (n - 4) + [2.0, 1.0]
    tot, acc, bounds = sum(w), 0.0, [0]
    for x in w:
        acc += x
        b = round(batch * acc / tot)
        bounds.append(min(batch, max(bounds[-1] + 1, b)))
    bounds[-1] = batch
    for i in range(n - 1, 0, -1):  # keep the boundaries strictly increasing if the batch is small
        bounds[i] = min(bounds[i], bounds[i + 1] - 1)
    return bounds


def auto_chunks(batch: int, heads: int, seq_len: int, head_dim: int, elem_size: int, mini_batch: int,
                backward: bool = True) -> int:
    """Number of equal chunks for a link-bound step.  A chunk's kernels are a chain of seq_len / mini_batch dependent
    stages whose time does not shrink with the chunk (about 1.5 us per forward stage and 3.3 us per backward stage on
    a B200), so a chunk must carry enough rows that copying it takes longer than that chain -- else the compute
    stream, not the link, paces the pipeline -- and no more, because the first copy-in and the last copy-out are not
    overlapped.  The link moves about 45 GB/s per direction with both directions busy."""
    chain_ms = (seq_len / mini_batch) * (4.8e-3 if backward else 1.5e-3)
    row_ms = heads * seq_len * head_dim * elem_size * (4 if backward else 3) / 45e6
    rows = max(1, -int(-1.3 * chain_ms // row_ms))
    return max(1, -(-batch // rows))


class HostBatchRunner:
    def __init__(self, config: FusedTttConfig, device: torch.device, chunks: Optional[int] = None,
                 backward: bool = True, taper: bool = False):
        """chunks: how many batch chunks to pipeline (None: `auto_chunks` of each call's shapes); taper: see
        `chunk_bounds`."""
        self.cfg, self.dev, self.backward = config, device, backward
        self.chunks = None if chunks is None else max(1, chunks)
        self.taper = taper
        self.s_in = torch.cuda.Stream(device)
        self.s_comp = torch.cuda.Stream(device)
        self.s_out = torch.cuda.Stream(device)
        self._dbuf = [None, None]
        self._whole: Dict[str, torch.Tensor] = {}

    def _buffers(self, slot: int, like: Dict[str, torch.Tensor], rows: int, capacity: int):
        """Device staging buffers of a slot: allocated once at the largest chunk size (`capacity` rows) and handed out
        as views, so that chunks of different sizes never free memory that kernels of another stream still read."""
        cur = self._dbuf[slot]
        if cur is None or next(iter(cur.values())).shape[0] < capacity:
            cur = {k: torch.empty((capacity,) + tuple(v.shape[1:]), dtype=v.dtype, device=self.dev)
                   for k, v in like.items()}
            self._dbuf[slot] = cur
        return {k: v[:rows] for k, v in cur.items()}

    def _whole_buffer(self, name: str, like: torch.Tensor):
        """A device buffer of the whole batch for one of the small tensors."""
        cur = self._whole.get(name)
        if cur is None or cur.shape != like.shape or cur.dtype != like.dtype:
            cur = torch.empty(like.shape, dtype=like.dtype, device=self.dev)
            self._whole[name] = cur
        return cur

    def run(self, host_in: Dict[str, torch.Tensor], params: Dict[str, torch.Tensor],
            host_out: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """host_in: pinned xq, xk, xv [B,H,T,F], ttt_lr_eta [B,H,T] (+ grad_output [B,H,T,F] when backward);
        params: device tensors weight [B,H,F,F], bias [B,H,F], token_eta [T], ln_weight, ln_bias [H,F];
        host_out: pinned buffers filled in place: output (+ grad_xq, grad_xk, grad_xv, grad_ttt_lr_eta, grad_weight,
        grad_bias, grad_token_eta, grad_ln_weight, grad_ln_bias).  Returns host_out after queuing all work; the
        caller synchronises (torch.cuda.synchronize or an event) before reading it."""
        names = _IN + (("grad_output",) if self.backward else ())
        B, H, T, F = host_in["xq"].shape
        chunks = self.chunks
        if chunks is None:
            chunks = auto_chunks(B, H, T, F, host_in["xq"].element_size(), self.cfg.mini_batch_len, self.backward)
        bounds = chunk_bounds(B, chunks, self.taper)
        self.last_bounds = bounds
        nchunk = len(bounds) - 1
        max_rows = max(bounds[i + 1] - bounds[i] for i in range(nchunk))
        cur = torch.cuda.current_stream(self.dev)
        for st in (self.s_in, self.s_comp, self.s_out):
            st.wait_stream(cur)
        ev_in, ev_comp, keep = [], [], []
        acc: Dict[str, Optional[torch.Tensor]] = {"token_eta": None, "ln_weight": None, "ln_bias": None}
        with torch.cuda.stream(self.s_in):
            lr_dev = self._whole_buffer("ttt_lr_eta", host_in["ttt_lr_eta"])
            lr_dev.copy_(host_in["ttt_lr_eta"], non_blocking=True)
        small = {k: self._whole_buffer(k, host_out[k]) for k in _SMALL_OUT} if self.backward else {}
        for c in range(nchunk):
            a, b = bounds[c], bounds[c + 1]
            slot = c % 2
            with torch.cuda.stream(self.s_in):
                if c >= 2:
                    self.s_in.wait_event(ev_comp[c - 2])  # the kernels of chunk c-2 have consumed this slot
                buf = self._buffers(slot, {k: host_in[k] for k in names}, b - a, max_rows)
                for k in names:
                    buf[k].copy_(host_in[k][a:b], non_blocking=True)
                e = torch.cuda.Event()
                e.record(self.s_in)
                ev_in.append(e)
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(ev_in[c])
                ins = TttInputs(buf["xq"], buf["xk"], buf["xv"], params["weight"][a:b], params["bias"][a:b],
                                params["token_eta"], lr_dev[a:b], params["ln_weight"], params["ln_bias"])
                outs, saved = TttTileMultiKernel.forward_launch(ins, self.cfg)
                res = {"output": outs.output}
                if self.backward:
                    g = TttTileMultiKernel.backward_launch(saved, TttOutputs(buf["grad_output"], None, None), self.cfg)
                    res.update(grad_xq=g.xq, grad_xk=g.xk, grad_xv=g.xv)
                    for k, v in (("grad_ttt_lr_eta", g.ttt_lr_eta), ("grad_weight", g.weight), ("grad_bias", g.bias)):
                        small[k][a:b].copy_(v)
                    for k, v in (("token_eta", g.token_eta), ("ln_weight", g.ln_weight), ("ln_bias", g.ln_bias)):
                        acc[k] = v.float() if acc[k] is None else acc[k] + v.float()
                e = torch.cuda.Event()
                e.record(self.s_comp)
                ev_comp.append(e)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_comp[c])
                for k, v in res.items():
                    host_out[k][a:b].copy_(v, non_blocking=True)
            keep.append((res, saved))
        if self.backward:
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_comp[-1])
                for k in _SMALL_OUT:
                    host_out[k].copy_(small[k], non_blocking=True)
                for k in ("token_eta", "ln_weight", "ln_bias"):
                    host_out["grad_" + k].copy_(acc[k].to(host_out["grad_" + k].dtype), non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_comp)
        self._keep = keep  # device tensors stay referenced until the next call
        return host_out


def alloc_host_outputs(B: int, H: int, T: int, F: int, dtype: torch.dtype, backward: bool = True):
    """Pinned host buffers of the shapes `HostBatchRunner.run` fills."""
    def pin(*shape):
        return torch.empty(shape, dtype=dtype, pin_memory=True)
    out = {"output": pin(B, H, T, F)}
    if backward:
        out.update(grad_xq=pin(B, H, T, F), grad_xk=pin(B, H, T, F), grad_xv=pin(B, H, T, F),
                   grad_ttt_lr_eta=pin(B, H, T), grad_weight=pin(B, H, F, F), grad_bias=pin(B, H, F),
                   grad_token_eta=pin(T), grad_ln_weight=pin(H, F), grad_ln_bias=pin(H, F))
    return out


def bind_host_thread_near(device: torch.device):
    """Restrict this process to the CPUs of the NUMA node the GPU hangs off, so that pinned buffers allocated
    afterwards land in that node's memory and host<->device copies of several ranks do not all cross one socket.
    Returns the node number, or None when the topology cannot be read (then nothing is changed)."""
    import os
    try:
        pr = torch.cuda.get_device_properties(device)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read().strip())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except (OSError, ValueError, AttributeError):
        return None
