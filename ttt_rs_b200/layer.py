"""The outer TTT layer around the fused inner loop (forward / prefill), mirroring the reference's `TTT` module
(rust/layer/src/ttt.rs:29-299; PyTorch twin reference/ttt.py:598-915): same parameters, same `forward(x, inner,
state, start_idx)`.

What runs where:
  * q/k/v(/gate) projections and the per-head learning-rate logits: ONE library GEMM over the concatenated weights
    (the reference issues one GEMM per projection plus a batched matmul for the gate logits);
  * head split + permute to [B,H,T,F], shared-QK causal convolutions, rotary embedding, sigmoid learning-rate gate:
    `ttt_layer_prologue` (one pass over the projection output);
  * inner loop: the fused kernel behind `FusedTileMultiTTTLinear`;
  * permute back + post LayerNorm + gelu gate: `ttt_layer_epilogue` (one pass);
  * output projection: library GEMM.
Under autograd the same kernels run with their gradient kernels (`ttt_layer_prologue_backward`,
`ttt_layer_epilogue_backward`) joined by torch autograd, so the layer trains end to end; with the shared-QK layout the
two convolutions are a step of their own there (`ttt_layer_qk_conv`, `ttt_layer_qk_conv_backward`) instead of being
applied inside the prologue kernel.
There is no PyTorch fallback for the layer kernels: without the CUDA library the calls raise.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import TttDims
from .fused import FusedTileMultiTTTLinear, Qkv, TTTInputsInner, TTTLinear, TTTLinearState

ROPE_NONE, ROPE_WRAPPED, ROPE_GLOBAL = 0, 1, 2
_POS = {"none": ROPE_NONE, "rope": ROPE_WRAPPED, "rope_global": ROPE_GLOBAL}


@dataclass
class TTTLayerConfig:
    """The fields of the reference's model config this layer reads (rust/config/src/train.rs:14-50,
    rust/layer/src/ttt.rs:60-145)."""
    hidden_size: int
    num_heads: int
    mini_batch_size: int = 16
    base_lr: float = 1.0
    rope_theta: float = 10000.0
    pos_encoding: str = "rope"   # "rope" (positions modulo the mini-batch), "rope_global", "none"
    conv_kernel_size: int = 4
    use_gate: bool = False
    share_qk: bool = False

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return _lib.TTT_BF16
    if dt == torch.float32:
        return _lib.TTT_F32
    raise TypeError(f"unsupported dtype {dt} (float32 or bfloat16)")


def layer_prologue(proj: torch.Tensor, cfg: TTTLayerConfig, *, q_col: int, k_col: int, v_col: int, lr_col: int,
                   lr_bias: Optional[torch.Tensor], conv=None, start_idx: int = 0):
    """proj [B,T,N]: a projection output holding, as column blocks, q at q_col, k at k_col, v at v_col (H*F columns
    each) and the H learning-rate logits at lr_col.  `conv` = (q_weight [C,1,K] or [C,K], q_bias [C], k_weight, k_bias)
    for the shared-QK layout.  Returns XQ, XK, XV [B,H,T,F] and ttt_lr_eta [B,H,T]."""
    lib = _lib.load()
    B, T, N = proj.shape
    H, F = cfg.num_heads, cfg.head_dim
    if not proj.is_cuda or not proj.is_contiguous():
        raise ValueError("proj must be a contiguous CUDA tensor")
    dt = proj.dtype
    esz = proj.element_size()
    d = TttDims(B, H, T, F, cfg.mini_batch_size, 1, 0.0, _dtype_code(dt))
    xq, xk, xv = (torch.empty(B, H, T, F, dtype=dt, device=proj.device) for _ in range(3))
    lr = torch.empty(B, H, T, dtype=dt, device=proj.device)
    base = proj.data_ptr()
    col = lambda c: C.c_void_p(base + c * esz)  # noqa: E731
    cw = [None] * 4
    kc = 0
    if conv is not None:
        cw = [t.to(dt).reshape(t.shape[0], -1).contiguous() if t.dim() > 1 else t.to(dt).contiguous() for t in conv]
        kc = cw[0].shape[1]
    bias = None if lr_bias is None else lr_bias.to(dt).reshape(-1).contiguous()
    stream = C.c_void_p(torch.cuda.current_stream(proj.device).cuda_stream)
    with torch.cuda.device(proj.device):
        _lib.check(lib.ttt_layer_prologue(
            C.byref(d), col(q_col), col(k_col), col(v_col), N, col(lr_col), N, _ptr(bias),
            _ptr(cw[0]), _ptr(cw[1]), _ptr(cw[2]), _ptr(cw[3]), kc, start_idx, _POS[cfg.pos_encoding],
            cfg.rope_theta, cfg.base_lr, _ptr(xq), _ptr(xk), _ptr(xv), _ptr(lr), stream))
    return xq, xk, xv, lr


def layer_epilogue(inner_out: torch.Tensor, ln_weight: torch.Tensor, ln_bias: torch.Tensor, eps: float = 1e-6,
                   gate: Optional[torch.Tensor] = None, gate_ld: int = 0):
    """inner_out [B,H,T,F] -> [B,T,H*F], post LayerNorm applied, times gelu_tanh(gate) when `gate` (a [B*T, gate_ld]
    view, first H*F columns) is given."""
    lib = _lib.load()
    B, H, T, F = inner_out.shape
    if not inner_out.is_cuda or not inner_out.is_contiguous():
        raise ValueError("inner_out must be a contiguous CUDA tensor")
    dt = inner_out.dtype
    d = TttDims(B, H, T, F, 16, 1, 0.0, _dtype_code(dt))
    y = torch.empty(B, T, H * F, dtype=dt, device=inner_out.device)
    w, b = ln_weight.to(dt).contiguous(), ln_bias.to(dt).contiguous()
    stream = C.c_void_p(torch.cuda.current_stream(inner_out.device).cuda_stream)
    with torch.cuda.device(inner_out.device):
        _lib.check(lib.ttt_layer_epilogue(C.byref(d), _ptr(inner_out), _ptr(gate), gate_ld, _ptr(w), _ptr(b),
                                          eps, _ptr(y), stream))
    return y


def gemm_bf16_tn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a [M, K] . b[N, K]^T -> [M, N], bf16 with float32 accumulation, on the library's tcgen05 GEMM
    (`ttt_gemm_bf16_tn`): `a` has one token per row, `b` is a weight matrix with one output feature per row, as the
    layer's projections store them.  Rows of both must be contiguous; K and N multiples of 8."""
    from .fused import device_status
    lib = _lib.load()
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise ValueError(f"gemm_bf16_tn: shapes {tuple(a.shape)} and {tuple(b.shape)} do not contract")
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or not a.is_cuda or b.device != a.device:
        raise ValueError("gemm_bf16_tn takes bf16 CUDA tensors on one device: there is no CPU path")
    if a.stride(1) != 1:
        a = a.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    M, K = a.shape
    N = b.shape[0]
    c = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    stream = C.c_void_p(torch.cuda.current_stream(a.device).cuda_stream)
    with torch.cuda.device(a.device):
        _lib.check(lib.ttt_gemm_bf16_tn(M, N, K, _ptr(a), a.stride(0), _ptr(b), b.stride(0), _ptr(c), c.stride(0),
                                        _ptr(device_status(a.device)), stream))
    return c


def layer_projections(x: torch.Tensor, wcat: torch.Tensor, cols, cfg: TTTLayerConfig, lr_bias: Optional[torch.Tensor],
                      start_idx: int = 0):
    """All projections of the layer plus the prologue in ONE launch (`ttt_layer_projections`: the tcgen05 GEMM with the
    head split, rotary rotation and learning-rate gate in its epilogue).  x [B, T, hidden] bf16, wcat the stacked
    q | k | v | (g) | lr weight rows with their starts in `cols`.  Returns xq, xk, xv [B,H,T,F], ttt_lr_eta [B,H,T] and
    the gate buffer [B*T, H*F] (None without a gate)."""
    from .fused import device_status
    lib = _lib.load()
    B, T, hidden = x.shape
    H, F = cfg.num_heads, cfg.head_dim
    dev = x.device
    x2 = x.reshape(B * T, hidden)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    xq, xk, xv = (torch.empty(B, H, T, F, dtype=x.dtype, device=dev) for _ in range(3))
    lr = torch.empty(B, H, T, dtype=x.dtype, device=dev)
    gate = torch.empty(B * T, H * F, dtype=x.dtype, device=dev) if "g" in cols else None
    d = TttDims(B, H, T, F, cfg.mini_batch_size, 1, 0.0, _dtype_code(x.dtype))
    bias = None if lr_bias is None else lr_bias.detach().reshape(-1).to(x.dtype).contiguous()
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    with torch.cuda.device(dev):
        _lib.check(lib.ttt_layer_projections(
            C.byref(d), _ptr(x2), x2.stride(0), hidden, _ptr(wcat), wcat.stride(0), wcat.shape[0], cols["q"], cols["k"],
            cols["v"], cols.get("g", -1), cols["lr"], _ptr(bias), start_idx, _POS[cfg.pos_encoding], cfg.rope_theta,
            cfg.base_lr, _ptr(xq), _ptr(xk), _ptr(xv), _ptr(gate), _ptr(lr), _ptr(device_status(dev)), stream))
    return xq, xk, xv, lr, gate


class _PrologueFn(torch.autograd.Function):
    """`ttt_layer_prologue` with its gradient `ttt_layer_prologue_backward` (layout q | k | v | lr logits | padding,
    no shared-QK convolutions)."""

    @staticmethod
    def forward(ctx, proj, lr_bias, cfg, cols, start_idx):
        xq, xk, xv, lr = layer_prologue(proj, cfg, q_col=cols["q"], k_col=cols["k"], v_col=cols["v"],
                                        lr_col=cols["lr"], lr_bias=lr_bias, start_idx=start_idx)
        ctx.save_for_backward(lr)
        ctx.meta = (cfg, cols, start_idx, proj.shape)
        return xq, xk, xv, lr

    @staticmethod
    def backward(ctx, dxq, dxk, dxv, dlr):
        (lr,) = ctx.saved_tensors
        cfg, cols, start_idx, (B, T, N) = ctx.meta
        lib = _lib.load()
        H, F = cfg.num_heads, cfg.head_dim
        dt = lr.dtype
        esz = lr.element_size()
        dproj = torch.empty(B, T, N, dtype=dt, device=lr.device)
        d = TttDims(B, H, T, F, cfg.mini_batch_size, 1, 0.0, _dtype_code(dt))
        base = dproj.data_ptr()
        col = lambda c: C.c_void_p(base + c * esz)  # noqa: E731
        stream = C.c_void_p(torch.cuda.current_stream(lr.device).cuda_stream)
        dxq, dxk, dxv, dlr = (t.contiguous() for t in (dxq, dxk, dxv, dlr))  # named: copies must outlive the launch
        with torch.cuda.device(lr.device):
            _lib.check(lib.ttt_layer_prologue_backward(
                C.byref(d), _ptr(dxq), _ptr(dxk), _ptr(dxv),
                _ptr(dlr), _ptr(lr), start_idx, _POS[cfg.pos_encoding], cfg.rope_theta, cfg.base_lr,
                col(cols["q"]), col(cols["k"]), col(cols["v"]), N, col(cols["lr"]), N, N - cols["lr"], stream))
        dbias = dproj[..., cols["lr"]:cols["lr"] + H].float().sum(dim=(0, 1)).to(dt).reshape(H, 1)
        return dproj, dbias, None, None, None


def _taps4(w: torch.Tensor, dt) -> torch.Tensor:
    """Depthwise convolution weight [C,1,K] or [C,K] (K <= 4) -> [C,4], taps aligned to the end (tap j multiplies
    token t - 3 + j)."""
    w2 = w.reshape(w.shape[0], -1).to(dt)
    K = w2.shape[1]
    if K > 4:
        raise ValueError(f"convolution kernels of up to 4 taps are supported (got {K})")
    return torch.nn.functional.pad(w2, (4 - K, 0)).contiguous()


class _QkConvFn(torch.autograd.Function):
    """Shared-QK causal depthwise convolutions as a differentiable step (`ttt_layer_qk_conv` and its gradient
    `ttt_layer_qk_conv_backward`): xqk [B,T,C] (a column block of the projection output) -> conv_q(xqk), conv_k(xqk)."""

    @staticmethod
    def forward(ctx, proj, col, C_, wq, bq, wk, bk, cfg):
        lib = _lib.load()
        B, T, N = proj.shape
        dt, dev = proj.dtype, proj.device
        d = TttDims(B, cfg.num_heads, T, cfg.head_dim, cfg.mini_batch_size, 1, 0.0, _dtype_code(dt))
        q = torch.empty(B, T, C_, dtype=dt, device=dev)
        k = torch.empty(B, T, C_, dtype=dt, device=dev)
        w4q, w4k = _taps4(wq, dt), _taps4(wk, dt)
        bqc, bkc = bq.to(dt).contiguous(), bk.to(dt).contiguous()
        x = C.c_void_p(proj.data_ptr() + col * proj.element_size())
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        with torch.cuda.device(dev):
            _lib.check(lib.ttt_layer_qk_conv(C.byref(d), x, N, _ptr(w4q), _ptr(bqc), _ptr(w4k), _ptr(bkc), _ptr(q),
                                             _ptr(k), stream))
        ctx.save_for_backward(proj, w4q, w4k)
        ctx.meta = (cfg, col, C_, wq.shape, wk.shape, wq.dtype, bq.dtype)
        return q, k

    @staticmethod
    def backward(ctx, dq, dk):
        proj, w4q, w4k = ctx.saved_tensors
        cfg, col, C_, wq_shape, wk_shape, wdt, bdt = ctx.meta
        lib = _lib.load()
        B, T, N = proj.shape
        dt, dev = proj.dtype, proj.device
        d = TttDims(B, cfg.num_heads, T, cfg.head_dim, cfg.mini_batch_size, 1, 0.0, _dtype_code(dt))
        dx = torch.empty(B, T, C_, dtype=dt, device=dev)
        gq = torch.empty(5 * C_, dtype=torch.float32, device=dev)
        gk = torch.empty(5 * C_, dtype=torch.float32, device=dev)
        ws_bytes = lib.ttt_layer_qk_conv_backward_workspace_bytes(C.byref(d))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        x = C.c_void_p(proj.data_ptr() + col * proj.element_size())
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        dq, dk = dq.contiguous(), dk.contiguous()  # named: a temporary copy must outlive the launch
        with torch.cuda.device(dev):
            _lib.check(lib.ttt_layer_qk_conv_backward(C.byref(d), _ptr(dq), _ptr(dk), x, N,
                                                      _ptr(w4q), _ptr(w4k), _ptr(dx), _ptr(gq), _ptr(gk), _ptr(ws),
                                                      ws_bytes, stream))
        dproj = torch.zeros_like(proj)
        dproj[..., col:col + C_] = dx

        def params(g, shape):
            K = 1
            for n in shape[1:]:
                K *= n
            dw = g[:4 * C_].reshape(4, C_).t()[:, 4 - K:]  # [C, K], the kernel's own taps
            return dw.reshape(shape).to(wdt), g[4 * C_:].to(bdt)

        dwq, dbq = params(gq, wq_shape)
        dwk, dbk = params(gk, wk_shape)
        return dproj, None, None, dwq, dbq, dwk, dbk, None


class _EpilogueFn(torch.autograd.Function):
    """`ttt_layer_epilogue` with its gradient `ttt_layer_epilogue_backward`."""

    @staticmethod
    def forward(ctx, inner_out, gate, ln_weight, ln_bias, eps):
        inner_out = inner_out.contiguous()
        g2d, ld = (None, 0) if gate is None else (gate.contiguous().reshape(-1, gate.shape[-1]), gate.shape[-1])
        y = layer_epilogue(inner_out, ln_weight, ln_bias, eps, g2d, ld)
        ctx.save_for_backward(inner_out, g2d, ln_weight, ln_bias)
        ctx.eps = eps
        ctx.gate_shape = None if gate is None else gate.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        inner_out, g2d, ln_weight, ln_bias = ctx.saved_tensors
        lib = _lib.load()
        B, H, T, F = inner_out.shape
        dt, dev = inner_out.dtype, inner_out.device
        d = TttDims(B, H, T, F, 16, 1, 0.0, _dtype_code(dt))
        d_inner = torch.empty_like(inner_out)
        d_gate = None if g2d is None else torch.empty_like(g2d)
        dw = torch.empty(H * F, dtype=torch.float32, device=dev)
        db = torch.empty(H * F, dtype=torch.float32, device=dev)
        ws_bytes = lib.ttt_layer_epilogue_backward_workspace_bytes(C.byref(d))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        w, b = ln_weight.to(dt).contiguous(), ln_bias.to(dt).contiguous()
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        dy = dy.contiguous()
        with torch.cuda.device(dev):
            _lib.check(lib.ttt_layer_epilogue_backward(
                C.byref(d), _ptr(dy), _ptr(inner_out), _ptr(g2d), 0 if g2d is None else g2d.shape[1],
                _ptr(w), _ptr(b), ctx.eps, _ptr(d_inner), _ptr(d_gate), 0 if d_gate is None else d_gate.shape[1],
                _ptr(dw), _ptr(db), _ptr(ws), ws_bytes, stream))
        dg = None if d_gate is None else d_gate.reshape(ctx.gate_shape)
        return d_inner, dg, dw.to(ln_weight.dtype), db.to(ln_bias.dtype), None


class TTT(torch.nn.Module):
    """Outer TTT layer.  Parameter names follow the reference (`q_proj`, `k_proj`, `v_proj`, `g_proj`, `o_proj`,
    `q_conv` / `k_conv`, `learnable_ttt_lr_weight` [H, hidden, 1], `learnable_ttt_lr_bias` [H, 1], `token_idx`,
    `learnable_token_idx`, `post_norm`)."""

    def __init__(self, config: TTTLayerConfig, device=None, dtype=torch.float32):
        super().__init__()
        c = config
        self.config = c
        kw = dict(device=device, dtype=dtype)
        hs = c.hidden_size

        def lin():
            return torch.nn.Parameter(torch.randn(hs, hs, **kw) * 0.02)

        self.q_proj = lin()
        self.k_proj = None if c.share_qk else lin()
        self.v_proj = lin()
        self.g_proj = lin() if c.use_gate else None
        self.o_proj = lin()
        if c.share_qk:
            k = c.conv_kernel_size
            self.q_conv_weight = torch.nn.Parameter(torch.randn(hs, 1, k, **kw) * (1.0 / k) ** 0.5)
            self.q_conv_bias = torch.nn.Parameter(torch.zeros(hs, **kw))
            self.k_conv_weight = torch.nn.Parameter(torch.randn(hs, 1, k, **kw) * (1.0 / k) ** 0.5)
            self.k_conv_bias = torch.nn.Parameter(torch.zeros(hs, **kw))
        self.learnable_ttt_lr_weight = torch.nn.Parameter(torch.randn(c.num_heads, hs, 1, **kw) * 0.02)
        self.learnable_ttt_lr_bias = torch.nn.Parameter(torch.zeros(c.num_heads, 1, **kw))
        self.register_buffer("token_idx", 1.0 / torch.arange(1, c.mini_batch_size + 1, **kw))
        self.learnable_token_idx = torch.nn.Parameter(torch.zeros(c.mini_batch_size, **kw))
        self.post_norm_weight = torch.nn.Parameter(torch.ones(hs, **kw))
        self.post_norm_bias = torch.nn.Parameter(torch.zeros(hs, **kw))
        self._wcat, self._wcat_key = None, None

    # ---- one GEMM for every projection of x ----------------------------------------------------------------
    def _fused_weight(self):
        """Rows: q | (k) | v | (g) | lr logits (H rows), padded to a multiple of 8 rows.  The concatenation is cached
        and rebuilt whenever one of its source parameters has changed: the cache key holds each parameter's storage
        address, in-place version counter, dtype and device, so an optimizer step, `load_state_dict`, `.to()` or a
        dtype cast all invalidate it."""
        srcs = [w for w in (self.q_proj, self.k_proj, self.v_proj, self.g_proj) if w is not None]
        srcs.append(self.learnable_ttt_lr_weight)
        key = tuple((w.data_ptr(), w._version, w.dtype, w.device) for w in srcs)
        if self._wcat is None or self._wcat_key != key:
            self._wcat_key = key
            c = self.config
            blocks, cols, off = [], {}, 0
            for name, w in (("q", self.q_proj), ("k", self.k_proj), ("v", self.v_proj), ("g", self.g_proj)):
                if w is not None:
                    blocks.append(w)
                    cols[name] = off
                    off += w.shape[0]
            blocks.append(self.learnable_ttt_lr_weight.reshape(c.num_heads, c.hidden_size))
            cols["lr"] = off
            off += c.num_heads
            pad = (-off) % 8
            if pad:
                blocks.append(torch.zeros(pad, c.hidden_size, dtype=self.q_proj.dtype, device=self.q_proj.device))
            if "k" not in cols:
                cols["k"] = cols["q"]
            self._wcat = (torch.cat([b.detach() for b in blocks], dim=0).contiguous(), cols)
        return self._wcat

    def invalidate_fused_weight(self):
        self._wcat = None

    @staticmethod
    def _project(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """x [..., K] . weight[N, K]^T -> [..., N].  bf16 on a GPU: the library's own tensor-core GEMM
        (`ttt_gemm_bf16_tn`); float32 (the parity configuration) is a float32 library product."""
        if x.dtype == torch.bfloat16 and x.is_cuda and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0:
            return gemm_bf16_tn(x.reshape(-1, x.shape[-1]), weight).reshape(*x.shape[:-1], weight.shape[0])
        return torch.matmul(x, weight.t())

    def _can_fuse_projections(self, x: torch.Tensor, cols) -> bool:
        """The one-launch projection + prologue covers bf16, sequence lengths that are multiples of 128, separate q / k
        projections, wrapped or no rotary positions with a mini-batch of at most 16 tokens, and column blocks that
        start on multiples of 64."""
        c = self.config
        return (x.dtype == torch.bfloat16 and x.is_cuda and x.shape[1] % 128 == 0 and not c.share_qk
                and c.head_dim == 64 and c.hidden_size % 8 == 0 and c.num_heads <= 64
                and c.pos_encoding in ("none", "rope") and c.mini_batch_size <= 16
                and all(v % 64 == 0 for v in cols.values()))

    def get_inner_loop_inputs(self, x: torch.Tensor, start_idx: int):
        """Hidden states -> (TTTInputsInner, gate operand, gate pitch) (rust/layer/src/ttt.rs:250-267).  The gate
        operand is a [B*T, pitch] view whose first H*F columns are x . g_proj^T (None without a gate)."""
        c = self.config
        B, T, _ = x.shape
        wcat, cols = self._fused_weight()
        te = torch.clamp_min(self.token_idx + self.learnable_token_idx, 0.0)
        token_eta = te.repeat((T + c.mini_batch_size - 1) // c.mini_batch_size)[:T].to(x.dtype)
        if self._can_fuse_projections(x, cols):
            xq, xk, xv, lr, gate = layer_projections(x, wcat, cols, c, self.learnable_ttt_lr_bias, start_idx)
            return TTTInputsInner(Qkv(xq, xk, xv), token_eta, lr, start_idx), gate, c.num_heads * c.head_dim
        proj = self._project(x, wcat)  # [B, T, N]: every projection of the token in one product
        conv = None
        if c.share_qk:
            conv = (self.q_conv_weight, self.q_conv_bias, self.k_conv_weight, self.k_conv_bias)
        xq, xk, xv, lr = layer_prologue(proj, c, q_col=cols["q"], k_col=cols["k"], v_col=cols["v"], lr_col=cols["lr"],
                                        lr_bias=self.learnable_ttt_lr_bias, conv=conv, start_idx=start_idx)
        gate = proj.reshape(B * T, -1)[:, cols["g"]:] if c.use_gate else None
        return TTTInputsInner(Qkv(xq, xk, xv), token_eta, lr, start_idx), gate, proj.shape[-1]

    def forward(self, x: torch.Tensor, inner: FusedTileMultiTTTLinear, state: TTTLinearState,
                start_idx: int = 0) -> torch.Tensor:
        """x [B, T, hidden] -> [B, T, hidden]; `state` is advanced in place (rust/layer/src/ttt.rs:269-299)."""
        if torch.is_grad_enabled():
            return self._forward_train(x, inner, state, start_idx)
        inputs, gate, gate_ld = self.get_inner_loop_inputs(x, start_idx)
        out = inner.forward(state, inputs)  # [B, H, T, F]
        y = layer_epilogue(out.contiguous(), self.post_norm_weight, self.post_norm_bias, 1e-6, gate,
                           gate_ld if gate is not None else 0)
        return self._project(y, self.o_proj.detach())


def _train_forward(self, x, inner, state, start_idx):
    """Training path: the same kernels, each with its gradient kernel, joined by torch autograd (which also supplies
    the gradients of the library GEMMs).  The gate projection is a GEMM of its own here, so that every column of the
    fused projection's gradient is written by exactly one kernel."""
    c = self.config
    B, T, _ = x.shape
    H, hs = c.num_heads, c.hidden_size
    if c.share_qk:
        # shared projection | v | lr logits, then the two convolutions as a step of their own (with its gradient
        # kernel); the prologue sees the usual q | k | v | lr layout
        pad0 = (-(2 * hs + H)) % 8
        blocks = [self.q_proj, self.v_proj, self.learnable_ttt_lr_weight.reshape(H, hs)]
        if pad0:
            blocks.append(torch.zeros(pad0, hs, dtype=x.dtype, device=x.device))
        proj0 = torch.matmul(x, torch.cat(blocks, dim=0).t())
        qc, kc = _QkConvFn.apply(proj0, 0, hs, self.q_conv_weight, self.q_conv_bias, self.k_conv_weight,
                                 self.k_conv_bias, c)
        rest = proj0[..., hs:2 * hs + H]
        pad = (-(3 * hs + H)) % 8
        parts = [qc, kc, rest]
        if pad:
            parts.append(torch.zeros(B, T, pad, dtype=x.dtype, device=x.device))
        proj = torch.cat(parts, dim=-1)
    else:
        pad = (-(3 * hs + H)) % 8
        blocks = [self.q_proj, self.k_proj, self.v_proj, self.learnable_ttt_lr_weight.reshape(H, hs)]
        if pad:
            blocks.append(torch.zeros(pad, hs, dtype=x.dtype, device=x.device))
        proj = torch.matmul(x, torch.cat(blocks, dim=0).t())
    cols = {"q": 0, "k": hs, "v": 2 * hs, "lr": 3 * hs}
    xq, xk, xv, lr = _PrologueFn.apply(proj, self.learnable_ttt_lr_bias, c, cols, start_idx)
    te = torch.clamp_min(self.token_idx + self.learnable_token_idx, 0.0)
    token_eta = te.repeat((T + c.mini_batch_size - 1) // c.mini_batch_size)[:T].to(x.dtype)
    out = inner.forward(state, TTTInputsInner(Qkv(xq, xk, xv), token_eta, lr, start_idx))
    gate = torch.matmul(x, self.g_proj.t()) if c.use_gate else None
    y = _EpilogueFn.apply(out, gate, self.post_norm_weight, self.post_norm_bias, 1e-6)
    return torch.matmul(y, self.o_proj.t())


TTT._forward_train = _train_forward


def new_inner(config: TTTLayerConfig, checkpoint_interval: int = 1, device=None, dtype=torch.float32,
              allow_partial: bool = False, partial_in_place: bool = False):
    """The `fused-tile-multi` inner model matching a layer config (`allow_partial`: also accept sequence tails and
    1-token decode steps; `partial_in_place`: advance the state in place on such calls, see FusedTileMultiTTTLinear)."""
    return FusedTileMultiTTTLinear(TTTLinear(config.num_heads, config.head_dim, config.mini_batch_size, 1e-6,
                                             checkpoint_interval, device=device, dtype=dtype), allow_partial,
                                   partial_in_place)


class DecodeGraphs:
    """Token-by-token generation through one layer with the whole step (projection GEMM, prologue, decode kernel,
    epilogue, output GEMM: five launches, launch-bound at small batch) captured once per rotary phase as a CUDA graph.

    The rotary position enters the prologue as a scalar argument, so with positions wrapped at the mini-batch there
    are `mini_batch_size` distinct steps; each is captured on first use.  The state is advanced in place, the input
    is read from `self.x` [B, 1, hidden] and the result lands in the tensor `step` returns (overwritten by the next
    step of the same phase)."""

    def __init__(self, layer: "TTT", inner: FusedTileMultiTTTLinear, state: TTTLinearState, batch: int):
        c = layer.config
        if c.pos_encoding == "rope_global":
            raise ValueError("rope_global positions never repeat: the step cannot be captured once per phase")
        if not (inner.allow_partial and inner.partial_in_place):
            raise ValueError("the inner model must be built with allow_partial=True, partial_in_place=True")
        self.layer, self.inner, self.state = layer, inner, state
        p = layer.q_proj
        self.x = torch.zeros(batch, 1, c.hidden_size, dtype=p.dtype, device=p.device)
        self.period = c.mini_batch_size if c.pos_encoding == "rope" else 1
        self._graphs, self._outs = {}, {}

    def step(self, x: torch.Tensor, start_idx: int) -> torch.Tensor:
        """One token per sequence: x [B, 1, hidden] at position `start_idx`."""
        self.x.copy_(x)
        ph = start_idx % self.period
        g = self._graphs.get(ph)
        if g is None:
            # warm-up run on a side stream (lazy initialisation of the libraries must happen outside the capture);
            # it advances the state once, so the state is saved and restored around it
            w0, b0 = self.state.weight.clone(), self.state.bias.clone()
            s = torch.cuda.Stream(self.x.device)
            s.wait_stream(torch.cuda.current_stream(self.x.device))
            with torch.cuda.stream(s), torch.no_grad():
                self.layer(self.x, self.inner, self.state, ph)
            torch.cuda.current_stream(self.x.device).wait_stream(s)
            self.state.weight.copy_(w0)
            self.state.bias.copy_(b0)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g), torch.no_grad():
                self._outs[ph] = self.layer(self.x, self.inner, self.state, ph)
            self._graphs[ph] = g
            # the capture itself does not execute: the state is still w0, b0 and the replay below does the step
        g.replay()
        return self._outs[ph]
