"""Host-side mirror of the reference's `fused-tile-multi` operator, over the C ABI.

Names, argument meaning and error behaviour follow the reference so that tests read like its own:

* `FusedTttConfig`                       rust/fused/src/lib.rs:285-328
* `TttInputs` / `TttOutputs`             rust/fused/src/ttt/types.rs:3-13
* `TttSavedStateMulti`                   rust/fused/src/linear_fused_tile/launch.rs:30-41
* `TttTileMultiKernel.forward_launch / backward_launch`
                                         rust/fused/src/linear_fused_tile/launch.rs:117-208 (FusedKernel trait,
                                         rust/kernels/src/kernel.rs:32-54)
* `fused_ttt_tile_forward_multi`         rust/fused/src/linear_fused_tile/api.rs:52-83 (autodiff-registered entry,
                                         rust/kernels/src/impls/autodiff.rs:107-200)
* `TTTLinear`, `TTTLinearState`, `TTTInputsInner`, `Qkv`
                                         rust/core/src/linear.rs:18-33,84-89, rust/core/src/inner.rs:61-68,108-130
* `FusedTileMultiTTTLinear`              rust/fused/src/linear_fused_tile/wrapper.rs:81-211 (TTTInnerModel impl)

torch is used for device memory and streams only; all arithmetic happens in libttt_b200.so.
"""

from __future__ import annotations

import ctypes as C
import threading
from dataclasses import dataclass, fields
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import TttDims, TttError

_DTYPES = {torch.float32: _lib.TTT_F32, torch.bfloat16: _lib.TTT_BF16}

# --------------------------------------------------------------------------------------------
# device-side status words
# --------------------------------------------------------------------------------------------
# One 16-word int32 buffer per device, handed to every launch.  A kernel whose bounded wait runs out writes
# {TTT_ERR_TIMEOUT, where, block, stage} there by compare-and-swap from zero and returns early, so the first report
# on a device sticks until `check_status` has read (and cleared) it, however many launches follow.
_STATUS_WORDS = 16
_status_lock = threading.Lock()
_status_buffers: Dict[Tuple[str, int], torch.Tensor] = {}


def device_status(device) -> torch.Tensor:
    """The status words of `device` (created zeroed on first use).  Shared by all launches on that device."""
    device = torch.device(device)
    if device.type != "cuda":
        raise TttError(_lib.TTT_ERR_CUDA, "status words live on a CUDA device")
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (device.type, idx)
    with _status_lock:
        buf = _status_buffers.get(key)
        if buf is None:
            buf = torch.zeros(_STATUS_WORDS, dtype=torch.int32, device=torch.device("cuda", idx))
            _status_buffers[key] = buf
        return buf


def _raise_if_reported(words, what: str = "") -> None:
    if words[0] != 0:
        raise TttError(int(words[0]), f"device-side wait timed out{what} (where={words[1]}, block={words[2]}, "
                                      f"stage={words[3]}): outputs of launches since the last check are not valid")


def check_status(device=None) -> None:
    """Synchronise and raise `TttError` if any launch since the last check reported a timed-out device-side wait.
    `device` None checks every device that has run a launch.  Call it once per step, after the step's work: a kernel
    that gave up returns early and leaves its outputs unwritten.  The report is cleared when it is raised."""
    with _status_lock:
        if device is None:
            bufs = list(_status_buffers.items())
        else:
            device = torch.device(device)
            idx = device.index if device.index is not None else torch.cuda.current_device()
            bufs = [(k, v) for k, v in _status_buffers.items() if k == (device.type, idx)]
    for (kind, idx), buf in bufs:
        torch.cuda.synchronize(torch.device(kind, idx))
        words = buf.cpu().tolist()
        if words[0] != 0:
            buf.zero_()
            _raise_if_reported(words, f" on {kind}:{idx}")


# --------------------------------------------------------------------------------------------
# config and tensor bundles
# --------------------------------------------------------------------------------------------

@dataclass(frozen=True)
class FusedTttConfig:
    """Kernel configuration key.  `epsilon` travels as an integer multiple of 1e-9 like the reference's
    hashable config; `threads` is accepted for signature compatibility (the sm_100a kernels always run
    4 warps per stream)."""
    mini_batch_len: int
    head_dim: int
    epsilon_scaled: int
    threads: int = 128
    checkpoint_interval: int = 1

    @staticmethod
    def new(mini_batch_len: int, head_dim: int, epsilon: float, threads: int = 128,
            checkpoint_interval: int = 1) -> "FusedTttConfig":
        # float32 arithmetic like the reference: (1e-6f32 / 1e-9f32) as u32 == 1000
        scaled = int(np.float32(epsilon) / np.float32(1e-9))
        return FusedTttConfig(mini_batch_len, head_dim, scaled, threads, checkpoint_interval)

    def epsilon(self) -> float:
        return float(np.float32(self.epsilon_scaled) * np.float32(1e-9))

    def with_checkpoint_interval(self, k: int) -> "FusedTttConfig":
        return FusedTttConfig(self.mini_batch_len, self.head_dim, self.epsilon_scaled, self.threads, k)


@dataclass
class TttInputs:
    xq: torch.Tensor
    xk: torch.Tensor
    xv: torch.Tensor
    weight: torch.Tensor
    bias: torch.Tensor
    token_eta: torch.Tensor
    ttt_lr_eta: torch.Tensor
    ln_weight: torch.Tensor
    ln_bias: torch.Tensor
    #: set on the gradients `backward_launch` returns: the status words of the device the launch ran on
    status: Optional[torch.Tensor] = None

    def map(self, fn):
        return TttInputs(*[fn(getattr(self, f.name)) for f in fields(self) if f.name != "status"], status=self.status)


@dataclass
class TttOutputs:
    output: torch.Tensor
    weight: torch.Tensor
    bias: torch.Tensor


@dataclass
class TttSavedStateMulti:
    xq: torch.Tensor
    xk: torch.Tensor
    xv: torch.Tensor
    weight_init: torch.Tensor
    bias: torch.Tensor
    token_eta: torch.Tensor
    ttt_lr_eta: torch.Tensor
    ln_weight: torch.Tensor
    ln_bias: torch.Tensor
    weight_checkpoints: torch.Tensor
    bias_checkpoints: torch.Tensor
    #: status words of the device the forward ran on (see `check_status`)
    status: Optional[torch.Tensor] = None


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream_ptr(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _dims(xq: torch.Tensor, config: FusedTttConfig) -> TttDims:
    if xq.dim() != 4:
        raise TttError(_lib.TTT_ERR_SHAPE, f"xq must be [batch, heads, seq_len, head_dim], got {tuple(xq.shape)}")
    if xq.dtype not in _DTYPES:
        raise TttError(_lib.TTT_ERR_UNSUPPORTED, f"unsupported dtype {xq.dtype}")
    B, H, T, F = xq.shape
    if F != config.head_dim:
        raise TttError(_lib.TTT_ERR_SHAPE, f"head_dim of xq ({F}) differs from config.head_dim ({config.head_dim})")
    return TttDims(B, H, T, F, config.mini_batch_len, config.checkpoint_interval,
                   float(config.epsilon()), _DTYPES[xq.dtype])


def _expect(name: str, t: torch.Tensor, shape, dtype, device):
    if tuple(t.shape) != tuple(shape):
        raise TttError(_lib.TTT_ERR_SHAPE, f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
    if t.dtype != dtype:
        raise TttError(_lib.TTT_ERR_SHAPE, f"{name} has dtype {t.dtype}, expected {dtype}")
    if t.device != device:
        raise TttError(_lib.TTT_ERR_SHAPE, f"{name} is on {t.device}, expected {device}")


def _check_inputs(i, wname="weight"):
    xq = i.xq
    if not xq.is_cuda:
        raise TttError(_lib.TTT_ERR_CUDA, "inputs must be CUDA tensors: this operator has no CPU path")
    B, H, T, F = xq.shape
    dt, dev = xq.dtype, xq.device
    _expect("xk", i.xk, (B, H, T, F), dt, dev)
    _expect("xv", i.xv, (B, H, T, F), dt, dev)
    _expect(wname, getattr(i, wname), (B, H, F, F), dt, dev)
    _expect("bias", i.bias, (B, H, F), dt, dev)
    if i.token_eta.dim() != 1 or i.token_eta.shape[0] != T:
        raise TttError(_lib.TTT_ERR_SHAPE, f"token_eta must be [seq_len] = [{T}], got {tuple(i.token_eta.shape)}")
    _expect("token_eta", i.token_eta, (T,), dt, dev)
    _expect("ttt_lr_eta", i.ttt_lr_eta, (B, H, T), dt, dev)
    _expect("ln_weight", i.ln_weight, (H, F), dt, dev)
    _expect("ln_bias", i.ln_bias, (H, F), dt, dev)


class TttTileMultiKernel:
    """The multi-stage tiled TTT-Linear operator: one launch walks every mini-batch of the sequence."""

    @staticmethod
    def forward_launch(inputs: TttInputs, config: FusedTttConfig,
                       save_state: bool = True) -> Tuple[TttOutputs, Optional[TttSavedStateMulti]]:
        """`save_state=False` (inference): nothing is kept for a backward and the second return value is None."""
        if config.mini_batch_len <= 0:
            raise TttError(_lib.TTT_ERR_SHAPE, "mini_batch_len must be set for TttTileMultiKernel")
        lib = _lib.load()
        inputs = inputs.map(lambda t: t.contiguous())
        d = _dims(inputs.xq, config)
        _check_inputs(inputs)
        dev = inputs.xq.device
        nck = lib.ttt_linear_num_checkpoints(C.byref(d))
        if nck < 0:
            raise TttError(_lib.TTT_ERR_SHAPE, _lib.last_error())
        B, H, T, F = inputs.xq.shape
        output = torch.empty_like(inputs.xq)
        weight_out = torch.empty_like(inputs.weight)
        bias_out = torch.empty_like(inputs.bias)
        # opaque saved state, sized by the library: float32 W at every checkpoint (+ the final W), and one buffer
        # holding the per-stage lr-scaled LN gradient tiles, row statistics and biases
        w_ck = b_ck = None
        if save_state:
            w_ck = torch.empty(lib.ttt_linear_weight_ckpt_bytes(C.byref(d)) // 4, dtype=torch.float32,
                               device=dev).view(-1, 64, 64)  # head_dim 32: a pair of heads per 64 x 64 block
            b_ck = torch.empty(lib.ttt_linear_bias_ckpt_bytes(C.byref(d)), dtype=torch.uint8, device=dev)
        status = device_status(dev)
        with torch.cuda.device(dev):
            rc = lib.ttt_linear_forward(
                C.byref(d), _ptr(inputs.xq), _ptr(inputs.xk), _ptr(inputs.xv), _ptr(inputs.weight),
                _ptr(inputs.bias), _ptr(inputs.token_eta), _ptr(inputs.ttt_lr_eta), _ptr(inputs.ln_weight),
                _ptr(inputs.ln_bias), _ptr(output), _ptr(weight_out), _ptr(bias_out), _ptr(w_ck), _ptr(b_ck),
                _ptr(status), _stream_ptr(dev))
        _lib.check(rc)
        if not save_state:
            return TttOutputs(output, weight_out, bias_out), None
        saved = TttSavedStateMulti(inputs.xq, inputs.xk, inputs.xv, inputs.weight, inputs.bias, inputs.token_eta,
                                   inputs.ttt_lr_eta, inputs.ln_weight, inputs.ln_bias, w_ck, b_ck, status)
        return TttOutputs(output, weight_out, bias_out), saved

    @staticmethod
    def forward_partial(inputs: TttInputs, config: FusedTttConfig, in_place: bool = False) -> TttOutputs:
        """One mini-batch of 1..16 tokens (sequence tail, decode step): `ttt_linear_forward_partial`.  Forward only.
        With `in_place` the state tensors of `inputs` are advanced and returned."""
        lib = _lib.load()
        inputs = inputs.map(lambda t: t.contiguous())
        d = _dims(inputs.xq, config)
        _check_inputs(inputs)
        dev = inputs.xq.device
        output = torch.empty_like(inputs.xq)
        weight_out = inputs.weight if in_place else torch.empty_like(inputs.weight)
        bias_out = inputs.bias if in_place else torch.empty_like(inputs.bias)
        with torch.cuda.device(dev):
            _lib.check(lib.ttt_linear_forward_partial(
                C.byref(d), _ptr(inputs.xq), _ptr(inputs.xk), _ptr(inputs.xv), _ptr(inputs.weight),
                _ptr(inputs.bias), _ptr(inputs.token_eta), _ptr(inputs.ttt_lr_eta), _ptr(inputs.ln_weight),
                _ptr(inputs.ln_bias), _ptr(output), _ptr(weight_out), _ptr(bias_out), _stream_ptr(dev)))
        return TttOutputs(output, weight_out, bias_out)

    @staticmethod
    def backward_launch(saved: TttSavedStateMulti, grad_outputs: TttOutputs, config: FusedTttConfig,
                        outer_grad_packed: Optional[torch.Tensor] = None, use_state_grads: bool = False) -> TttInputs:
        """Gradients w.r.t. the nine inputs, in input order.  By default only `grad_outputs.output` is used: upstream
        gradients of the returned final state are ignored, as in the reference.  With `use_state_grads=True`,
        `grad_outputs.weight` / `.bias` (when not None) are taken as the gradients flowing into the final state."""
        if config.mini_batch_len <= 0:
            raise TttError(_lib.TTT_ERR_SHAPE, "mini_batch_len must be set for TttTileMultiKernel backward")
        lib = _lib.load()
        d = _dims(saved.xq, config)
        _check_inputs(saved, wname="weight_init")
        go = grad_outputs.output.contiguous()
        B, H, T, F = saved.xq.shape
        dev, dt = saved.xq.device, saved.xq.dtype
        _expect("grad_output", go, (B, H, T, F), dt, dev)
        g_xq, g_xk, g_xv = (torch.empty_like(saved.xq) for _ in range(3))
        g_w = torch.empty_like(saved.weight_init)
        g_b = torch.empty_like(saved.bias)
        g_lr = torch.empty_like(saved.ttt_lr_eta)
        g_te = torch.empty(T, dtype=torch.float32, device=dev)
        g_lnw = torch.empty((H, F), dtype=torch.float32, device=dev)
        g_lnb = torch.empty((H, F), dtype=torch.float32, device=dev)
        ws_bytes = lib.ttt_linear_backward_workspace_bytes(C.byref(d))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        status = device_status(dev)
        gw_out = gb_out = None
        if use_state_grads:
            if grad_outputs.weight is not None:
                gw_out = grad_outputs.weight.contiguous()
                _expect("grad_outputs.weight", gw_out, (B, H, F, F), dt, dev)
            if grad_outputs.bias is not None:
                gb_out = grad_outputs.bias.contiguous()
                _expect("grad_outputs.bias", gb_out, (B, H, F), dt, dev)
        with torch.cuda.device(dev):
            rc = lib.ttt_linear_backward_state_grads(
                C.byref(d), _ptr(saved.xq), _ptr(saved.xk), _ptr(saved.xv), _ptr(saved.weight_init),
                _ptr(saved.bias), _ptr(saved.token_eta), _ptr(saved.ttt_lr_eta), _ptr(saved.ln_weight),
                _ptr(saved.ln_bias), _ptr(saved.weight_checkpoints), _ptr(saved.bias_checkpoints), _ptr(go),
                _ptr(gw_out), _ptr(gb_out), _ptr(g_xq), _ptr(g_xk), _ptr(g_xv), _ptr(g_w), _ptr(g_b), _ptr(g_lr),
                _ptr(g_te), _ptr(g_lnw), _ptr(g_lnb), _ptr(outer_grad_packed), _ptr(ws), C.c_size_t(ws_bytes),
                _ptr(status), _stream_ptr(dev))
        _lib.check(rc)
        # the three reduced gradients are produced in float32 and cast back, like backward/launch.rs:423-425
        return TttInputs(g_xq, g_xk, g_xv, g_w, g_b, g_te.to(dt), g_lr, g_lnw.to(dt), g_lnb.to(dt), status)

    @staticmethod
    def check_status(device=None) -> None:
        """See the module-level `check_status`."""
        check_status(device)


def unpack_weight_checkpoints(weight_checkpoints: torch.Tensor) -> torch.Tensor:
    """The float32 state checkpoints of `TttSavedStateMulti` as plain [n, 64, 64] matrices W[k][n] (for inspection and
    tests; the kernels never need this).  The buffer holds each 64 x 64 state the way the kernels' threads hold it:
    float4 `kt` of thread `tid` at [kt][tid], whose element i is W[8 kt + 2 t + (i & 1)][16 warp + g + 8 (i >> 1)] with
    tid = 32 warp + 4 g + t -- eight coalesced 16-byte accesses per thread instead of 32 scattered ones."""
    v = weight_checkpoints.reshape(-1, 8, 4, 8, 4, 4)  # [n, kt, warp, g, t, i]
    n = v.shape[0]
    kt, warp, g, t, i = torch.meshgrid(torch.arange(8), torch.arange(4), torch.arange(8), torch.arange(4),
                                       torch.arange(4), indexing="ij")
    k = (8 * kt + 2 * t + (i & 1)).reshape(-1).to(v.device)
    col = (16 * warp + g + 8 * (i >> 1)).reshape(-1).to(v.device)
    out = torch.empty((n, 64, 64), dtype=v.dtype, device=v.device)
    out[:, k, col] = v.reshape(n, -1)
    return out


def packed_outer_grad_len(heads: int, head_dim: int = 64, mini_batch: int = 16) -> int:
    """Length of the float32 buffer `outer_grad_packed`: dW0 [H,F,F], db0 [H,F], d ln_weight [H,F],
    d ln_bias [H,F], d token_eta [CS]."""
    return heads * head_dim * head_dim + 3 * heads * head_dim + mini_batch


class _FusedTttTileMultiFn(torch.autograd.Function):
    """Registers the operator with autograd the way the reference registers its kernel with Burn's autodiff:
    one node, saved state = nine inputs + two checkpoint tensors."""

    @staticmethod
    def forward(ctx, xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias, config):
        outs, saved = TttTileMultiKernel.forward_launch(
            TttInputs(xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias), config)
        ctx.config = config
        ctx.saved = saved
        ctx.mark_non_differentiable(outs.weight, outs.bias)
        return outs.output, outs.weight, outs.bias

    @staticmethod
    def backward(ctx, g_out, _g_w, _g_b):
        g = TttTileMultiKernel.backward_launch(ctx.saved, TttOutputs(g_out, None, None), ctx.config)
        return g.xq, g.xk, g.xv, g.weight, g.bias, g.token_eta, g.ttt_lr_eta, g.ln_weight, g.ln_bias, None


def fused_ttt_tile_forward_multi(xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias,
                                 config: FusedTttConfig):
    """(output, weight_updated, bias_updated); differentiable w.r.t. the nine tensor inputs through `output`.
    Under `torch.no_grad()` the forward keeps nothing for a backward."""
    if not torch.is_grad_enabled():
        outs, _ = TttTileMultiKernel.forward_launch(
            TttInputs(xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias), config, save_state=False)
        return outs.output, outs.weight, outs.bias
    return _FusedTttTileMultiFn.apply(xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias, config)


# --------------------------------------------------------------------------------------------
# inner-model interface
# --------------------------------------------------------------------------------------------

@dataclass
class Qkv:
    xq: torch.Tensor
    xk: torch.Tensor
    xv: torch.Tensor

    def slice_seq(self, r: range) -> "Qkv":
        return Qkv(self.xq[:, :, r.start:r.stop], self.xk[:, :, r.start:r.stop], self.xv[:, :, r.start:r.stop])


@dataclass
class TTTInputsInner:
    qkv: Qkv
    token_eta: torch.Tensor   # [seq_len]
    ttt_lr_eta: torch.Tensor  # [batch, heads, seq_len]
    start_idx: int = 0

    def slice_seq(self, r: range) -> "TTTInputsInner":
        return TTTInputsInner(self.qkv.slice_seq(r), self.token_eta[r.start:r.stop],
                              self.ttt_lr_eta[:, :, r.start:r.stop], r.start)


@dataclass
class TTTLinearState:
    weight: torch.Tensor  # [batch, heads, F, F]
    bias: torch.Tensor    # [batch, heads, F]


class TTTLinear(torch.nn.Module):
    """Parameter holder of the TTT-Linear inner model: weight_init [H,F,F] ~ N(0, 0.02), bias_init [H,F] = 0,
    per-head LayerNorm weight = 1 / bias = 0."""

    def __init__(self, num_heads: int, head_dim: int, mini_batch_size: int = 16, epsilon: float = 1e-6,
                 checkpoint_interval: int = 1, device=None, dtype=torch.float32):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, head_dim
        self.mini_batch_size, self.epsilon, self.checkpoint_interval = mini_batch_size, epsilon, checkpoint_interval
        kw = dict(device=device, dtype=dtype)
        self.weight_init = torch.nn.Parameter(torch.randn(num_heads, head_dim, head_dim, **kw) * 0.02)
        self.bias_init = torch.nn.Parameter(torch.zeros(num_heads, head_dim, **kw))
        self.ln_weight = torch.nn.Parameter(torch.ones(num_heads, head_dim, **kw))
        self.ln_bias = torch.nn.Parameter(torch.zeros(num_heads, head_dim, **kw))

    def init_state(self, batch_size: int) -> TTTLinearState:
        return TTTLinearState(self.weight_init.unsqueeze(0).repeat(batch_size, 1, 1, 1),
                              self.bias_init.unsqueeze(0).repeat(batch_size, 1, 1))


class FusedTileMultiTTTLinear(torch.nn.Module):
    """`fused-tile-multi` inner model: whole-sequence forward in a single launch."""

    def __init__(self, inner: TTTLinear, allow_partial: bool = False, partial_in_place: bool = False):
        """`allow_partial`: run a remainder / decode mini-batch (fewer tokens than the mini-batch) through the
        partial-mini-batch kernel, with the semantics of the reference's unfused inner model, instead of refusing it
        as the reference's fused type does.  Inference only (no gradient is recorded for such a call).
        `partial_in_place`: such a call advances the state tensors in place (same device addresses every step, which
        a captured CUDA graph of the decode step needs) instead of binding new tensors to the state."""
        super().__init__()
        self.inner = inner
        self.allow_partial = allow_partial
        self.partial_in_place = partial_in_place

    @staticmethod
    def name() -> str:
        return "FusedTileMultiTTTLinear"

    def init_state(self, batch_size: int) -> TTTLinearState:
        return self.inner.init_state(batch_size)

    def _config(self, head_dim: int) -> FusedTttConfig:
        i = self.inner
        return FusedTttConfig.new(i.mini_batch_size, head_dim, i.epsilon, 128, i.checkpoint_interval)

    def forward(self, state: TTTLinearState, inputs: TTTInputsInner) -> torch.Tensor:
        mb = self.inner.mini_batch_size
        B, H, T, F = inputs.qkv.xv.shape
        full, rem = T // mb, T % mb
        if full == 0:
            return self.forward_mini_batch(state, inputs, range(0, T))
        L = full * mb
        q = inputs.qkv.slice_seq(range(0, L))
        out, w, b = fused_ttt_tile_forward_multi(
            q.xq, q.xk, q.xv, state.weight, state.bias, inputs.token_eta[:L], inputs.ttt_lr_eta[:, :, :L],
            self.inner.ln_weight, self.inner.ln_bias, self._config(F))
        state.weight, state.bias = w, b
        if rem == 0:
            return out
        tail = self.forward_mini_batch(state, inputs, range(L, T))
        return torch.cat([out, tail], dim=2)

    def forward_mini_batch(self, state: TTTLinearState, inputs: TTTInputsInner, r: range) -> torch.Tensor:
        if len(r) != self.inner.mini_batch_size:
            if not self.allow_partial or not 0 < len(r) < self.inner.mini_batch_size:
                raise AssertionError("Sequence length must be equal to mini_batch_size")
            if torch.is_grad_enabled():
                raise RuntimeError("a partial mini-batch runs forward only: call it under torch.no_grad()")
            sl = inputs.slice_seq(r)
            F = sl.qkv.xq.shape[-1]
            outs = TttTileMultiKernel.forward_partial(
                TttInputs(sl.qkv.xq, sl.qkv.xk, sl.qkv.xv, state.weight, state.bias, sl.token_eta, sl.ttt_lr_eta,
                          self.inner.ln_weight.detach(), self.inner.ln_bias.detach()), self._config(F),
                in_place=self.partial_in_place)
            state.weight, state.bias = outs.weight, outs.bias
            return outs.output
        sl = inputs.slice_seq(r)
        F = sl.qkv.xq.shape[-1]
        cfg = self._config(F).with_checkpoint_interval(1)
        out, w, b = fused_ttt_tile_forward_multi(
            sl.qkv.xq, sl.qkv.xk, sl.qkv.xv, state.weight, state.bias, sl.token_eta, sl.ttt_lr_eta,
            self.inner.ln_weight, self.inner.ln_bias, cfg)
        state.weight, state.bias = w, b
        return out


# --------------------------------------------------------------------------------------------
# TTT-MLP (2-layer inner model): forward only
# --------------------------------------------------------------------------------------------

@dataclass
class TTTMLPState:
    """rust/core/src/mlp.rs:29-53: w1 [B,H,F,4F], b1 [B,H,4F], w2 [B,H,4F,F], b2 [B,H,F]."""
    w1: torch.Tensor
    b1: torch.Tensor
    w2: torch.Tensor
    b2: torch.Tensor


def mlp_backward_workspace(xq: torch.Tensor, config: FusedTttConfig) -> torch.Tensor:
    """Scratch buffer of the TTT-MLP backward for inputs shaped like `xq` [B,H,T,F]; `fused_ttt_mlp_forward` can
    fill it on the way (`backward_workspace=`), which saves the backward its own forward walk."""
    lib = _lib.load()
    d = _dims(xq, config)
    n = lib.ttt_mlp_backward_workspace_bytes(C.byref(d))
    if n == 0:
        raise TttError(_lib.TTT_ERR_SHAPE, _lib.last_error() or "unsupported problem for the TTT-MLP backward")
    return torch.empty(n, dtype=torch.uint8, device=xq.device)


def fused_ttt_mlp_forward(xq, xk, xv, state: TTTMLPState, token_eta, ttt_lr_eta, ln_weight, ln_bias,
                          config: FusedTttConfig, backward_workspace: Optional[torch.Tensor] = None):
    """Whole-sequence forward of the 2-layer inner model in one launch (the loop of
    `TTTMLP::forward_mini_batch`, rust/core/src/mlp.rs:127-208).  Returns (output, new TTTMLPState).
    bf16 only.  Its gradient is `fused_ttt_mlp_backward` (no autograd node is recorded here); a buffer from
    `mlp_backward_workspace` passed as `backward_workspace` is filled for it."""
    lib = _lib.load()
    if not xq.is_cuda:
        raise TttError(_lib.TTT_ERR_CUDA, "inputs must be CUDA tensors: this operator has no CPU path")
    d = _dims(xq, config)
    B, H, T, F = xq.shape
    E = 4 * F
    dt, dev = xq.dtype, xq.device
    ts = dict(xq=xq, xk=xk, xv=xv, w1=state.w1, b1=state.b1, w2=state.w2, b2=state.b2, token_eta=token_eta,
              ttt_lr_eta=ttt_lr_eta, ln_weight=ln_weight, ln_bias=ln_bias)
    shapes = dict(xq=(B, H, T, F), xk=(B, H, T, F), xv=(B, H, T, F), w1=(B, H, F, E), b1=(B, H, E), w2=(B, H, E, F),
                  b2=(B, H, F), token_eta=(token_eta.shape[0],), ttt_lr_eta=(B, H, T), ln_weight=(H, F), ln_bias=(H, F))
    ts = {k: v.contiguous() for k, v in ts.items()}
    for k, v in ts.items():
        _expect(k, v, shapes[k], dt, dev)
    out = torch.empty_like(ts["xq"])
    new = TTTMLPState(*(torch.empty_like(ts[k]) for k in ("w1", "b1", "w2", "b2")))
    status = device_status(dev)
    with torch.cuda.device(dev):
        rc = lib.ttt_mlp_forward(
            C.byref(d), *[_ptr(ts[k]) for k in ("xq", "xk", "xv", "w1", "b1", "w2", "b2", "token_eta", "ttt_lr_eta",
                                               "ln_weight", "ln_bias")],
            _ptr(out), _ptr(new.w1), _ptr(new.b1), _ptr(new.w2), _ptr(new.b2), _ptr(backward_workspace),
            0 if backward_workspace is None else backward_workspace.numel(), _ptr(status), _stream_ptr(dev))
    _lib.check(rc)
    return out, new


def fused_ttt_mlp_backward(xq, xk, xv, state: TTTMLPState, token_eta, ttt_lr_eta, ln_weight, ln_bias, grad_output,
                           config: FusedTttConfig, workspace_from_forward: Optional[torch.Tensor] = None):
    """Gradient of `fused_ttt_mlp_forward` for loss = <grad_output, output> (`ttt_mlp_backward`; `state` is the state
    the forward started from).  Returns a dict: grad_xq, grad_xk, grad_xv, grad_w1, grad_b1, grad_w2, grad_b2 (per
    batch element), grad_ttt_lr_eta, and float32 grad_token_eta [T], grad_ln_weight, grad_ln_bias [H, F].
    `workspace_from_forward`: the buffer the forward call on the same inputs filled (`backward_workspace=`); the
    kernel then skips its own forward walk.  The buffer is consumed (the backward overwrites the state in it)."""
    lib = _lib.load()
    if not xq.is_cuda:
        raise TttError(_lib.TTT_ERR_CUDA, "inputs must be CUDA tensors: this operator has no CPU path")
    d = _dims(xq, config)
    B, H, T, F = xq.shape
    E = 4 * F
    dt, dev = xq.dtype, xq.device
    ts = dict(xq=xq, xk=xk, xv=xv, w1=state.w1, b1=state.b1, w2=state.w2, b2=state.b2, token_eta=token_eta,
              ttt_lr_eta=ttt_lr_eta, ln_weight=ln_weight, ln_bias=ln_bias, grad_output=grad_output)
    shapes = dict(xq=(B, H, T, F), xk=(B, H, T, F), xv=(B, H, T, F), w1=(B, H, F, E), b1=(B, H, E), w2=(B, H, E, F),
                  b2=(B, H, F), token_eta=(token_eta.shape[0],), ttt_lr_eta=(B, H, T), ln_weight=(H, F), ln_bias=(H, F),
                  grad_output=(B, H, T, F))
    ts = {k: v.contiguous() for k, v in ts.items()}
    for k, v in ts.items():
        _expect(k, v, shapes[k], dt, dev)
    g = {"grad_" + k: torch.empty_like(ts[k]) for k in ("xq", "xk", "xv", "w1", "b1", "w2", "b2", "ttt_lr_eta")}
    g["grad_token_eta"] = torch.empty(T, dtype=torch.float32, device=dev)
    g["grad_ln_weight"] = torch.empty(H, F, dtype=torch.float32, device=dev)
    g["grad_ln_bias"] = torch.empty(H, F, dtype=torch.float32, device=dev)
    ws_bytes = lib.ttt_mlp_backward_workspace_bytes(C.byref(d))
    if ws_bytes == 0:
        raise TttError(_lib.TTT_ERR_SHAPE, _lib.last_error() or "unsupported problem for the TTT-MLP backward")
    if workspace_from_forward is not None:
        ws = workspace_from_forward
        if ws.device != dev or ws.dtype != torch.uint8 or ws.numel() < ws_bytes:
            raise TttError(_lib.TTT_ERR_WORKSPACE, f"workspace_from_forward must be {ws_bytes} bytes on {dev}")
    else:
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    names_in = ("xq", "xk", "xv", "w1", "b1", "w2", "b2", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias",
                "grad_output")
    names_out = ("grad_xq", "grad_xk", "grad_xv", "grad_w1", "grad_b1", "grad_w2", "grad_b2", "grad_ttt_lr_eta",
                 "grad_token_eta", "grad_ln_weight", "grad_ln_bias")
    status = device_status(dev)
    with torch.cuda.device(dev):
        rc = lib.ttt_mlp_backward(C.byref(d), *[_ptr(ts[k]) for k in names_in], *[_ptr(g[k]) for k in names_out],
                                  _ptr(ws), ws_bytes, 0 if workspace_from_forward is None else 1, _ptr(status),
                                  _stream_ptr(dev))
    _lib.check(rc)
    g["_workspace"] = ws  # keeps the scratch alive until the caller drops the result
    g["_status"] = status  # the device's status words: see `check_status`
    return g


def check_mlp_status(grads) -> None:
    """Raise if a launch on the device that produced `grads` reported a device-side wait timeout (the blocks of the
    TTT-MLP backward hand the stream state to one another; every such wait is bounded).  Same as `check_status`."""
    check_status(grads["_status"].device)


class _FusedTttMlpFn(torch.autograd.Function):
    """TTT-MLP inner loop as an autograd node: forward `ttt_mlp_forward`, backward `ttt_mlp_backward`.  Like the
    TTT-Linear operator (and the reference's fused operators, launch.rs:188-194) gradients arriving at the returned
    final state are ignored."""

    @staticmethod
    def forward(ctx, xq, xk, xv, w1, b1, w2, b2, token_eta, ttt_lr_eta, ln_weight, ln_bias, config):
        # the forward fills the backward's workspace on the way (final state + the operands of every state update)
        ws = mlp_backward_workspace(xq, config)
        out, new = fused_ttt_mlp_forward(xq, xk, xv, TTTMLPState(w1, b1, w2, b2), token_eta, ttt_lr_eta, ln_weight,
                                         ln_bias, config, backward_workspace=ws)
        ctx.save_for_backward(xq, xk, xv, w1, b1, w2, b2, token_eta, ttt_lr_eta, ln_weight, ln_bias)
        ctx.config = config
        ctx.workspace = ws
        return out, new.w1, new.b1, new.w2, new.b2

    @staticmethod
    def backward(ctx, g_out, *_state_grads):
        xq, xk, xv, w1, b1, w2, b2, token_eta, lr, ln_w, ln_b = ctx.saved_tensors
        ws, ctx.workspace = ctx.workspace, None  # consumed by the backward: a second backward re-walks the sequence
        g = fused_ttt_mlp_backward(xq, xk, xv, TTTMLPState(w1, b1, w2, b2), token_eta, lr, ln_w, ln_b,
                                   g_out.contiguous(), ctx.config, workspace_from_forward=ws)
        dt = xq.dtype
        return (g["grad_xq"], g["grad_xk"], g["grad_xv"], g["grad_w1"], g["grad_b1"], g["grad_w2"], g["grad_b2"],
                g["grad_token_eta"].to(dt), g["grad_ttt_lr_eta"], g["grad_ln_weight"].to(dt), g["grad_ln_bias"].to(dt),
                None)


def fused_ttt_mlp(xq, xk, xv, state: TTTMLPState, token_eta, ttt_lr_eta, ln_weight, ln_bias, config: FusedTttConfig):
    """Differentiable whole-sequence TTT-MLP inner loop: returns (output, new TTTMLPState)."""
    out, w1, b1, w2, b2 = _FusedTttMlpFn.apply(xq, xk, xv, state.w1, state.b1, state.w2, state.b2, token_eta,
                                               ttt_lr_eta, ln_weight, ln_bias, config)
    return out, TTTMLPState(w1, b1, w2, b2)


class TTTMLP(torch.nn.Module):
    """Parameter holder of the 2-layer inner model (rust/core/src/mlp.rs:29-53): w1_init [H,F,4F], b1_init [H,4F],
    w2_init [H,4F,F], b2_init [H,F] (weights ~ N(0, 0.02), biases 0), per-head LayerNorm weight = 1 / bias = 0."""

    def __init__(self, num_heads: int, head_dim: int, mini_batch_size: int = 16, epsilon: float = 1e-6, device=None,
                 dtype=torch.bfloat16):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, head_dim
        self.mini_batch_size, self.epsilon = mini_batch_size, epsilon
        kw = dict(device=device, dtype=dtype)
        E = 4 * head_dim
        self.w1_init = torch.nn.Parameter(torch.randn(num_heads, head_dim, E, **kw) * 0.02)
        self.b1_init = torch.nn.Parameter(torch.zeros(num_heads, E, **kw))
        self.w2_init = torch.nn.Parameter(torch.randn(num_heads, E, head_dim, **kw) * 0.02)
        self.b2_init = torch.nn.Parameter(torch.zeros(num_heads, head_dim, **kw))
        self.ln_weight = torch.nn.Parameter(torch.ones(num_heads, head_dim, **kw))
        self.ln_bias = torch.nn.Parameter(torch.zeros(num_heads, head_dim, **kw))

    def init_state(self, batch_size: int) -> TTTMLPState:
        r = lambda t: t.unsqueeze(0).repeat(batch_size, *([1] * t.dim()))  # noqa: E731
        return TTTMLPState(r(self.w1_init), r(self.b1_init), r(self.w2_init), r(self.b2_init))


class FusedTTTMLP(torch.nn.Module):
    """The 2-layer inner model behind the fused kernels, with the `forward(state, inputs)` interface of the inner-model
    trait (rust/core/src/inner.rs:13-58).  Whole mini-batches only; bf16 only; differentiable."""

    def __init__(self, inner: TTTMLP):
        super().__init__()
        self.inner = inner

    @staticmethod
    def name() -> str:
        return "FusedTTTMLP"

    def init_state(self, batch_size: int) -> TTTMLPState:
        return self.inner.init_state(batch_size)

    def forward(self, state: TTTMLPState, inputs: TTTInputsInner) -> torch.Tensor:
        i = self.inner
        B, H, T, F = inputs.qkv.xv.shape
        if T % i.mini_batch_size != 0:
            raise AssertionError("Sequence length must be a multiple of mini_batch_size")
        cfg = FusedTttConfig.new(i.mini_batch_size, F, i.epsilon, 128, 1)
        fn = fused_ttt_mlp if torch.is_grad_enabled() else fused_ttt_mlp_forward
        out, new = fn(inputs.qkv.xq, inputs.qkv.xk, inputs.qkv.xv, state, inputs.token_eta, inputs.ttt_lr_eta,
                      i.ln_weight, i.ln_bias, cfg)
        state.w1, state.b1, state.w2, state.b2 = new.w1, new.b1, new.w2, new.b2
        return out
