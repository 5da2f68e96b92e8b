#!/usr/bin/env python3
"""Benchmark of the fused TTT inner loop (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg1|cfg0|...]

One "step" is one forward + backward pass of the inner loop of one TTT layer over one batch of synthetic
input (the protocol of the reference's `ttt-bench --inner-only --backward`: rust/cli/src/bench.rs:193-234,
throughput = batch * seq_len / time, bench.rs:329).  Rank 0 prints ONE JSON line.

N > 1 is launched with torch.distributed.run, one rank per GPU.  The default is STRONG scaling: the seed-0
tensors of the workload are partitioned by batch rows (rank r owns rows [r B/N, (r+1) B/N) of the same tensors:
independent (batch x head) streams, no collective on the data path) and the value is tokens/s of the global batch.
`--scaling weak` gives every rank the full per-GPU workload instead (its own seed); with N > 1 the default run also
measures that mode and reports it under the extra key "weak".  In both modes the packed outer-parameter gradients
(dW0, db0, d ln_weight, d ln_bias, d token_eta) are all-reduced with NCCL every step, as data-parallel training
would.

`--impl reference` times the reference's own CPU implementation of the path on the host cores: its PyTorch module
(`reference/ttt.py`, forward + autograd backward), staged under oracle/_ref by the build where a reference checkout
was present, else the CPU restatement in oracle/ttt_oracle.py.  The reference's Rust/Burn CPU backend cannot be
built on this box (no Rust toolchain).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

LIN_IN = ("xq", "xk", "xv", "weight", "bias", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")
MLP_IN = ("xq", "xk", "xv", "w1", "b1", "w2", "b2", "token_eta", "ttt_lr_eta", "ln_weight", "ln_bias")

WORKLOADS = {
    # name: (B, H, T, dtype, checkpoint interval, backward?)
    "cfg0": dict(B=2, H=4, T=256, dtype="f32", K=1, backward=False,
                 desc="TTT-Linear inner loop fwd, f32, B=2 H=4 T=256 d=64 mb=16"),
    "cfg1": dict(B=32, H=12, T=2048, dtype="bf16", K=16, backward=True,
                 desc="TTT-Linear inner loop fwd+bwd, bf16, B=32 H=12 T=2048 d=64 mb=16 ckpt=16"),
    "cfg1-f32": dict(B=32, H=12, T=2048, dtype="f32", K=16, backward=True,
                     desc="TTT-Linear inner loop fwd+bwd, f32, B=32 H=12 T=2048 d=64 mb=16 ckpt=16"),
    "cfg2-fwd": dict(B=16, H=12, T=2048, dtype="bf16", K=1, backward=False, inner="mlp",
                     desc="TTT-MLP inner loop fwd (64-256-64, GELU tanh), bf16, B=16 H=12 T=2048 d=64 mb=16"),
    "cfg2": dict(B=16, H=12, T=2048, dtype="bf16", K=1, backward=True, inner="mlp",
                 desc="TTT-MLP inner loop fwd+bwd (64-256-64, GELU tanh), bf16, B=16 H=12 T=2048 d=64 mb=16"),
    # the reference's 125m-h32 preset: hidden 768 as 24 heads of 32 features (tile 16x32), two heads per kernel tile
    "cfg1-d32": dict(B=32, H=24, T=2048, F=32, dtype="bf16", K=16, backward=True,
                     desc="TTT-Linear inner loop fwd+bwd, bf16, B=32 H=24 T=2048 d=32 mb=16 ckpt=16"),
    "cfg4-8k": dict(B=8, H=32, T=8192, dtype="bf16", K=16, backward=True,
                    desc="TTT-Linear inner loop fwd+bwd, bf16, B=8 H=32 T=8192 d=64 mb=16 ckpt=16"),
    "cfg4-16k": dict(B=8, H=32, T=16384, dtype="bf16", K=16, backward=True,
                     desc="TTT-Linear inner loop fwd+bwd, bf16, B=8 H=32 T=16384 d=64 mb=16 ckpt=16"),
    "cfg4-32k": dict(B=8, H=32, T=32768, dtype="bf16", K=16, backward=True,
                     desc="TTT-Linear inner loop fwd+bwd, bf16, B=8 H=32 T=32768 d=64 mb=16 ckpt=16"),
    # the whole outer layer (projections, prologue, inner loop, epilogue, output projection), forward / prefill
    "layer-fwd": dict(kind="layer", B=8, H=12, T=2048, dtype="bf16", K=1, backward=False,
                      desc="TTT layer forward (125M layer shape: hidden 768, 12 heads x 64), bf16, B=8 T=2048 mb=16"),
    "layer-fwd-b32": dict(kind="layer", B=32, H=12, T=2048, dtype="bf16", K=1, backward=False,
                          desc="TTT layer forward (hidden 768, 12 heads x 64), bf16, B=32 T=2048 mb=16"),
    "layer-train-b32": dict(kind="layer", train=True, B=32, H=12, T=2048, dtype="bf16", K=16, backward=True,
                            desc="TTT layer forward + backward (hidden 768, 12 heads x 64), bf16, B=32 T=2048 mb=16 ckpt=16"),
    "layer-fwd-1b3": dict(kind="layer", B=8, H=32, T=8192, dtype="bf16", K=1, backward=False,
                          desc="TTT layer forward (1.3B layer shape: hidden 2048, 32 heads x 64), bf16, B=8 T=8192 mb=16"),
    # one decode step of the inner model (a mini-batch of one token per stream, state advanced in place)
    "decode": dict(kind="decode", B=8, H=12, T=1, dtype="bf16", K=1, backward=False,
                   desc="TTT-Linear inner model decode step (1 token per stream), bf16, B=8 H=12 d=64"),
    # token-by-token generation through one whole layer (projection GEMM, prologue, decode kernel, epilogue, output
    # GEMM), eager launches against one CUDA graph per rotary phase
    "decode-layer": dict(kind="decode-layer", B=8, H=12, T=1, dtype="bf16", K=1, backward=False,
                         desc="TTT layer decode step (hidden 768, 12 heads x 64), bf16, B=8, 1 token per step"),
    "decode-b256": dict(kind="decode", B=256, H=12, T=1, dtype="bf16", K=1, backward=False,
                        desc="TTT-Linear inner model decode step (1 token per stream), bf16, B=256 H=12 d=64"),
    # round-trip latency of one dependent tensor-core step: tcgen05 (descriptor operands, accumulator in tensor
    # memory) against mma.sync (operands and accumulator in registers); a measurement program, not a throughput line
    "chain-latency": dict(kind="probe", B=1, H=1, T=16, dtype="bf16", K=1, backward=False,
                          desc="dependent tensor-core step round trip, tcgen05 vs mma.sync (csrc/probe_chain_latency.cu)"),
}
F, CS = 64, 16
E2E_CHUNKS = int(os.environ.get("TTT_E2E_CHUNKS", "0")) or None  # None: chosen from the shapes (host_io.auto_chunks)


def algorithmic_bytes(w, fwd=True, bwd=True):
    """HBM bytes one launch must move: per token per head, forward reads q,k,v (3Fs) + lr (s), writes out (Fs) and
    its share of the float32 checkpoints; backward reads q,k,v,d_out (4Fs) + lr, writes dq,dk,dv (3Fs) + dlr and
    re-reads the checkpoints; per-stream constants (W0,b0,W_T,b_T; dW,db) amortise over T."""
    s = 2 if w["dtype"] == "bf16" else 4
    F = w.get("F", 64)
    tok_heads = w["B"] * w["H"] * w["T"]
    streams = w["B"] * w["H"]
    ck = (F * F + F) * s / (w["K"] * CS)  # counted at the element size; this build keeps them in float32
    fb = (4 * F * s + s + ck) * tok_heads + streams * 2 * (F * F + F) * s
    if w.get("inner") == "mlp":  # no saved state; the per-stream state is W1, b1, W2, b2 read and written once
        fb = (4 * F * s + s) * tok_heads + streams * 2 * (2 * F * 4 * F + 4 * F + F) * s
    bb = (7 * F * s + 2 * s + ck) * tok_heads + streams * (F * F + F) * s
    if w.get("inner") == "mlp":  # backward: q,k,v,d_out in, dq,dk,dv out, lr in, dlr out; state in, state gradient out
        bb = (7 * F * s + 2 * s) * tok_heads + streams * 2 * (2 * F * 4 * F + 4 * F + F) * s
    return (fb if fwd else 0) + (bb if bwd else 0), fb, bb


def measured_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_tensor_peak():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        if self._thr is not None:
            self._stop.set()
            self._thr.join()
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def make_host_inputs(w, seed):
    from ttt_rs_b200.synthetic import make_inputs
    dt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float32
    return make_inputs(w["B"], w["H"], w["T"], w.get("F", F), CS, seed=seed, dtype=dt, with_grad_output=True,
                       inner=w.get("inner", "linear"))


CPU_SAMPLE_B = 2  # batch rows of the workload that one CPU step covers (both arms use the same slice)


def cpu_kind():
    from oracle import ref_arm
    return "reference" if ref_arm.available() else "port"


def cpu_step(t, w):
    """One step on a host-resident sample (float32): the reference's own PyTorch module (forward + autograd
    backward) when it was staged under oracle/_ref, else the CPU restatement."""
    from oracle import ref_arm
    if ref_arm.available():
        return ref_arm.step(t, w.get("inner", "linear"), mini_batch=CS, backward=w["backward"])
    from oracle import ttt_oracle as O
    if w.get("inner") == "mlp":
        fw = O.ttt_mlp_forward(*[t[k] for k in MLP_IN], mini_batch=CS, eps=1e-6)
        if w["backward"]:
            O.ttt_mlp_backward(*[t[k] for k in MLP_IN], t["grad_output"], mini_batch=CS, eps=1e-6)
        return fw
    args = [t[k] for k in LIN_IN]
    fw = O.ttt_linear_forward(*args, mini_batch=CS, eps=1e-6, checkpoint_interval=w["K"])
    if w["backward"]:
        O.ttt_linear_backward(*args, t["grad_output"], mini_batch=CS, eps=1e-6)
    return fw


def time_cpu(w, steps, warmup, sample_B=CPU_SAMPLE_B):
    torch.set_num_threads(os.cpu_count() or 1)
    sample_B = min(sample_B, w["B"])
    sw = dict(w, B=sample_B)
    t = {k: v.float() for k, v in make_host_inputs(sw, seed=0).items()}
    for _ in range(warmup):
        cpu_step(t, w)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(t, w)
    dt = (time.perf_counter() - t0) / steps
    code = "reference/ttt.py (TTT%s.ttt + autograd)" % ("MLP" if w.get("inner") == "mlp" else "Linear") \
        if cpu_kind() == "reference" else "oracle/ttt_oracle.py (analytic backward)"
    return sample_B * w["T"] / dt, dt, torch.get_num_threads(), \
        f"rows [0,{sample_B}) of the workload (B={sample_B} H={w['H']} T={w['T']}), float32, {steps} step(s) after " \
        f"{warmup} warm-up, {code}"


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # each step is a 2-row slice of the workload (a second or two of host time), so K steps stay within minutes
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    val, dt, cores, sample = time_cpu(w, steps, warmup)
    kind = cpu_kind()
    line = {
        "impl": "reference", "metric": "ttt_inner_loop_tokens_per_sec", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.scaling != "weak" else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["desc"]},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": ("the reference's own PyTorch implementation of the path (reference/ttt.py, staged by the build under "
                 "oracle/_ref) on the host cores" if kind == "reference" else
                 "CPU restatement of the reference's algorithm (oracle/ttt_oracle.py) on the host cores: no reference "
                 "checkout was present at build time") +
                "; the reference's Rust/Burn CPU backend cannot be built here (no cargo/rustc)",
    }
    print(json.dumps(line), flush=True)


def time_events(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_layer(args, w):
    """Forward of one whole TTT layer on synthetic hidden states: tokens/s of the layer, the time of each piece, and
    the HBM roofline of the two layer kernels (algorithmic bytes: prologue reads q, k, v and the lr logits once and
    writes XQ, XK, XV and ttt_lr_eta once; epilogue reads the inner output once and writes the normalised rows once)."""
    import ttt_rs_b200 as tb
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        raise SystemExit("the layer workloads are single-GPU measurements")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tb.load_library()
    B, H, T = w["B"], w["H"], w["T"]
    C = H * F
    dt = torch.bfloat16
    torch.manual_seed(0)
    cfg = tb.TTTLayerConfig(hidden_size=C, num_heads=H)
    m = tb.TTT(cfg, device=dev, dtype=dt)
    inner = tb.new_inner(cfg, checkpoint_interval=w["K"], device=dev, dtype=dt)
    x = (torch.randn(B, T, C, device=dev) * 0.5).to(dt)
    state0 = inner.init_state(B)
    sampler = ClockSampler(0)

    def whole():
        with torch.no_grad():
            st = tb.TTTLinearState(state0.weight, state0.bias)
            return m(x, inner, st)

    with torch.no_grad():
        wcat, cols = m._fused_weight()
        proj = tb.gemm_bf16_tn(x.reshape(B * T, C), wcat).reshape(B, T, -1)
        inputs, _, _ = m.get_inner_loop_inputs(x, 0)
        inner_out = inner.forward(tb.TTTLinearState(state0.weight, state0.bias), inputs)
        y = tb.layer_epilogue(inner_out, m.post_norm_weight, m.post_norm_bias)
    tb.TttTileMultiKernel.check_status()

    def pro():
        return tb.layer_prologue(proj, cfg, q_col=cols["q"], k_col=cols["k"], v_col=cols["v"], lr_col=cols["lr"],
                                 lr_bias=m.learnable_ttt_lr_bias)

    def epi():
        return tb.layer_epilogue(inner_out, m.post_norm_weight, m.post_norm_bias)

    def inner_only():
        with torch.no_grad():
            return inner.forward(tb.TTTLinearState(state0.weight, state0.bias), inputs)

    train = bool(w.get("train"))
    if train:
        args.no_cpu_baseline = True  # the CPU leg of the layer workloads times the forward only
        xg = x.clone().requires_grad_(True)
        gy = (torch.randn(B, T, C, device=dev) * 1e-2).to(dt)

        def whole():  # noqa: F811  forward + backward of the layer, gradients of the input and of every parameter
            yy = m(xg, inner, inner.init_state(B))
            yy.backward(gy)
            return yy

    sampler.start()
    ms = time_events(whole, args.steps, args.warmup)
    clocks = sampler.stop()
    if train:
        tb.TttTileMultiKernel.check_status()
        from ttt_rs_b200.layer import _EpilogueFn, _PrologueFn  # the gradient kernels alone
        dxs = [torch.randn_like(inputs.qkv.xq) for _ in range(3)]
        dlr = torch.randn_like(inputs.ttt_lr_eta)
        pcols = {"q": 0, "k": C, "v": 2 * C, "lr": 3 * C}
        pproj = torch.empty(B, T, 3 * C + H + (-(3 * C + H)) % 8, device=dev, dtype=dt)

        class _Ctx:
            saved_tensors = (inputs.ttt_lr_eta,)
            meta = (cfg, pcols, 0, pproj.shape)

        class _Ctx2:
            saved_tensors = (inner_out, None, m.post_norm_weight.detach(), m.post_norm_bias.detach())
            eps = 1e-6
            gate_shape = None

        gyy = torch.randn_like(y)
        pb_ms = time_events(lambda: _PrologueFn.backward(_Ctx, *dxs, dlr), args.steps, args.warmup)
        eb_ms = time_events(lambda: _EpilogueFn.backward(_Ctx2, gyy), args.steps, args.warmup)
    fused_ok = m._can_fuse_projections(x, cols)
    pieces = {
        "projections_and_prologue_fused": time_events(
            lambda: tb.layer_projections(x, wcat, cols, cfg, m.learnable_ttt_lr_bias, 0), args.steps, args.warmup)
        if fused_ok else None,
        "projections_gemm": time_events(lambda: tb.gemm_bf16_tn(x.reshape(B * T, C), wcat), args.steps, args.warmup),
        "projections_gemm_cublas_for_comparison": time_events(lambda: torch.matmul(x, wcat.t()), args.steps, args.warmup),
        "ttt_layer_prologue_kernel": time_events(pro, args.steps, args.warmup),
        "inner_loop_forward": time_events(inner_only, args.steps, args.warmup),
        "ttt_layer_epilogue_kernel": time_events(epi, args.steps, args.warmup),
        "output_projection_gemm": time_events(lambda: tb.gemm_bf16_tn(y.reshape(B * T, C), m.o_proj.detach()), args.steps,
                                              args.warmup),
        "output_projection_gemm_cublas_for_comparison": time_events(lambda: torch.matmul(y, m.o_proj.t()), args.steps,
                                                                    args.warmup),
    }
    peak, peak_kind = measured_peaks()
    s = 2
    pro_bytes = (3 * C * s + H * s) * B * T + (3 * C * s + H * s) * B * T
    epi_bytes = 2 * C * s * B * T
    pa = pro_bytes / (pieces["ttt_layer_prologue_kernel"] * 1e-3) / 1e9
    ea = epi_bytes / (pieces["ttt_layer_epilogue_kernel"] * 1e-3) / 1e9
    tpeak, tkind = measured_tensor_peak()
    gflop = 2.0 * B * T * C * wcat.shape[0]
    gemm_tf = gflop / (pieces["projections_gemm"] * 1e-3) / 1e12
    line = {
        "metric": "ttt_layer_forward_tokens_per_sec", "value": B * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["desc"], "global_batch": B,
                   "l2": "operands of every piece exceed L2 (%.0f MB per tensor)" % (B * T * C * s / 1e6)},
        "clocks": clocks, "e2e": None, "gpu_launches": args.steps * 3,
        "pieces_ms": pieces,
        "roofline": {"bound": "hbm", "kernel": "ttt_layer_prologue_kernel", "achieved": pa, "peak": peak,
                     "unit": "GB/s", "frac": pa / peak, "traffic": None, "peak_source": f"of {peak_kind}",
                     "algorithmic_bytes_per_launch": pro_bytes,
                     "epilogue": {"kernel": "ttt_layer_epilogue_kernel", "achieved": ea, "frac": ea / peak,
                                  "algorithmic_bytes_per_launch": epi_bytes},
                     "projections_gemm": {"kernel": "ttt_gemm_bf16_tn_kernel", "bound": "tensor", "achieved": gemm_tf,
                                          "unit": "TFLOP/s", "peak": tpeak, "frac": gemm_tf / tpeak,
                                          "peak_source": f"of {tkind} (cuBLAS bf16 burst)",
                                          "flops_per_launch": gflop}},
    }
    if not args.no_cpu_baseline:
        from oracle import ttt_layer_oracle as LO
        torch.set_num_threads(os.cpu_count() or 1)
        p = {"q_proj": m.q_proj, "k_proj": m.k_proj, "v_proj": m.v_proj, "o_proj": m.o_proj,
             "lr_weight": m.learnable_ttt_lr_weight, "lr_bias": m.learnable_ttt_lr_bias, "token_idx": m.token_idx,
             "learnable_token_idx": m.learnable_token_idx, "post_norm_weight": m.post_norm_weight,
             "post_norm_bias": m.post_norm_bias, "W1": inner.inner.weight_init, "b1": inner.inner.bias_init,
             "ttt_norm_weight": inner.inner.ln_weight, "ttt_norm_bias": inner.inner.ln_bias}
        p = {k: v.detach().float().cpu() for k, v in p.items()}
        xs = x[:1].float().cpu()
        LO.ttt_layer_forward(xs[:, :256], p, num_heads=H)
        t0 = time.perf_counter()
        for _ in range(3):
            LO.ttt_layer_forward(xs, p, num_heads=H)
        dtc = (time.perf_counter() - t0) / 3
        line["cpu_baseline"] = {"value": T / dtc, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": f"B=1 T={T} slice of the workload, float32, 3 passes"}
    if train:
        line["metric"] = "ttt_layer_train_tokens_per_sec"
        line["pieces_ms"]["ttt_layer_prologue_bwd_kernel"] = pb_ms
        line["pieces_ms"]["ttt_layer_epilogue_bwd_kernels"] = eb_ms
        line["roofline"]["prologue_bwd"] = {"achieved": pro_bytes / (pb_ms * 1e-3) / 1e9,
                                            "frac": pro_bytes / (pb_ms * 1e-3) / 1e9 / peak,
                                            "algorithmic_bytes_per_launch": pro_bytes}
        eb_bytes = 3 * C * s * B * T  # dy and the inner output in, the inner-output gradient out
        line["roofline"]["epilogue_bwd"] = {"achieved": eb_bytes / (eb_ms * 1e-3) / 1e9,
                                            "frac": eb_bytes / (eb_ms * 1e-3) / 1e9 / peak,
                                            "algorithmic_bytes_per_launch": eb_bytes}
    print(json.dumps(line), flush=True)


def run_decode(args, w):
    """One-token steps of the inner model through `ttt_linear_forward_partial`, state resident and advanced in place.
    Algorithmic HBM bytes per step: the state is read and written once (2 (F^2 + F) s per stream) plus the token's
    q, k, v, output rows and lr (4 F s + s)."""
    import ttt_rs_b200 as tb
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tb.load_library()
    from ttt_rs_b200.synthetic import make_inputs
    B, H = w["B"], w["H"]
    t = make_inputs(B, H, 16, F, CS, seed=0, dtype=torch.bfloat16, with_grad_output=False)
    d = {k: v.to(dev) for k, v in t.items()}
    cfg = tb.FusedTttConfig.new(CS, F, 1e-6, 128, 1)
    ins = tb.TttInputs(d["xq"][:, :, :1].contiguous(), d["xk"][:, :, :1].contiguous(), d["xv"][:, :, :1].contiguous(),
                       d["weight"], d["bias"], d["token_eta"][:1].contiguous(), d["ttt_lr_eta"][:, :, :1].contiguous(),
                       d["ln_weight"], d["ln_bias"])
    tb.TttTileMultiKernel.forward_partial(ins, cfg, in_place=True)  # the public call, once (validates the operands)
    # the timed loop binds the same C-ABI call with prebuilt arguments: the host-side cost of a step is then the
    # foreign call alone, as it would be from the reference's Rust host
    import ctypes as C
    from ttt_rs_b200 import _lib
    lib = _lib.load()
    dd = _lib.TttDims(B, H, 1, F, CS, 1, float(cfg.epsilon()), _lib.TTT_BF16)
    out = torch.empty_like(ins.xq)
    ptr = lambda x: C.c_void_p(x.data_ptr())  # noqa: E731
    cargs = [C.byref(dd)] + [ptr(x) for x in (ins.xq, ins.xk, ins.xv, ins.weight, ins.bias, ins.token_eta,
                                                ins.ttt_lr_eta, ins.ln_weight, ins.ln_bias, out, ins.weight, ins.bias)]
    cargs.append(C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))

    def one():
        rc = lib.ttt_linear_forward_partial(*cargs)
        if rc != 0:
            raise RuntimeError(_lib.last_error())

    sampler = ClockSampler(0)
    sampler.start()
    ms = time_events(one, max(args.steps, 200), args.warmup)
    clocks = sampler.stop()
    peak, peak_kind = measured_peaks()
    s = 2
    nbytes = B * H * (2 * (F * F + F) * s + 4 * F * s + s)
    ach = nbytes / (ms * 1e-3) / 1e9
    line = {
        "metric": "ttt_inner_decode_tokens_per_sec", "value": B / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": max(args.steps, 200), "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["desc"], "global_batch": B,
                   "l2": "state of all streams: %.1f MB (L2-resident below 126 MB: the figure is an L2/launch-latency "
                         "number, not an HBM number)" % (B * H * (F * F + F) * s / 1e6)},
        "clocks": clocks, "e2e": None, "gpu_launches": max(args.steps, 200),
        "roofline": {"bound": "hbm", "kernel": "ttt_linear_partial_kernel", "achieved": ach, "peak": peak,
                     "unit": "GB/s", "frac": ach / peak, "traffic": None, "peak_source": f"of {peak_kind}",
                     "algorithmic_bytes_per_launch": nbytes},
    }
    if not args.no_cpu_baseline:
        from oracle import ttt_oracle as O
        torch.set_num_threads(os.cpu_count() or 1)
        names = LIN_IN
        c = {k: t[k].float() for k in names}
        for k in ("xq", "xk", "xv", "ttt_lr_eta"):
            c[k] = c[k][:, :, :1]
        sb = min(B, 32)
        c = {k: (v[:sb] if v.dim() >= 3 else v) for k, v in c.items()}
        O.ttt_linear_forward(*[c[k] for k in names], mini_batch=1)
        t0 = time.perf_counter()
        n = 20
        for _ in range(n):
            O.ttt_linear_forward(*[c[k] for k in names], mini_batch=1)
        dtc = (time.perf_counter() - t0) / n
        line["cpu_baseline"] = {"value": sb / dtc, "unit": "tokens/s", "cores": torch.get_num_threads(),
                                "kind": "port", "sample": f"B={sb} slice, float32, {n} steps"}
    print(json.dumps(line), flush=True)


def run_decode_layer(args, w):
    """One-token steps through the whole layer after a 64-token prefill: eager (five launches + host work per step)
    and replayed from CUDA graphs (ttt_rs_b200.layer.DecodeGraphs)."""
    import ttt_rs_b200 as tb
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tb.load_library()
    B, H = w["B"], w["H"]
    C = H * F
    dt = torch.bfloat16
    torch.manual_seed(0)
    cfg = tb.TTTLayerConfig(hidden_size=C, num_heads=H)
    layer = tb.TTT(cfg, device=dev, dtype=dt)
    steps = max(args.steps, 64)
    x = (torch.randn(B, 64 + steps + 16, C, device=dev) * 0.5).to(dt)

    def fresh():
        inner = tb.new_inner(cfg, device=dev, dtype=dt, allow_partial=True, partial_in_place=True)
        state = inner.init_state(B)
        state.weight, state.bias = state.weight.contiguous(), state.bias.contiguous()
        with torch.no_grad():
            layer(x[:, :64], inner, state, 0)
        return inner, state

    inner, state = fresh()
    pos = [64]

    def eager():
        with torch.no_grad():
            layer(x[:, pos[0]:pos[0] + 1].contiguous(), inner, state, pos[0])
        pos[0] = 64 + (pos[0] - 63) % (steps + 15)

    ms_eager = time_events(eager, steps, 16)
    inner, state = fresh()
    dec = tb.DecodeGraphs(layer, inner, state, B)
    pos[0] = 64

    def graph():
        dec.step(x[:, pos[0]:pos[0] + 1], pos[0])
        pos[0] = 64 + (pos[0] - 63) % (steps + 15)

    sampler = ClockSampler(0)
    time_events(graph, 16, 16)  # the first pass over the 16 rotary phases captures their graphs
    sampler.start()
    ms_graph = time_events(graph, steps, 0)
    clocks = sampler.stop()
    line = {
        "metric": "ttt_layer_decode_tokens_per_sec", "value": B / (ms_graph * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": 16, "ms_per_step": ms_graph, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["desc"], "global_batch": B, "l2": "launch-bound: the step moves about 8 MB"},
        "clocks": clocks, "e2e": None, "gpu_launches": steps * 3,
        "eager_ms_per_step": ms_eager, "graph_ms_per_step": ms_graph,
        "roofline": None,
    }
    print(json.dumps(line), flush=True)


def profile_traffic(kernel_workload: str):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of a kernel on a workload, read from the
    committed ncu summary `profiles/<kernel_workload>.md` (a line `dram_bytes_per_launch: <read> + <write>`), or None
    when no capture of the current kernel is on file."""
    f = REPO / "profiles" / f"{kernel_workload}.md"
    try:
        for ln in f.read_text().splitlines():
            if ln.lower().startswith("dram_bytes_per_launch:"):
                rd, wr = ln.split(":", 1)[1].split("+")
                return float(rd) + float(wr.split()[0])
    except (OSError, ValueError):
        pass
    return None


def shard_rows(t, a, b):
    """Batch rows [a, b) of every per-stream tensor of a host input dict (parameters shared by all streams stay)."""
    return {k: (v[a:b].contiguous() if v.dim() >= 3 else v) for k, v in t.items()}


def bench_inner(tb, w, host, dev, world, rank, args, name):
    """Times `args.steps` forward(+backward) passes of the inner loop on this rank's device-resident `host` tensors.
    Returns per-rank results; the caller turns them into tokens/s of the job."""
    import torch.distributed as dist
    from ttt_rs_b200.distributed import allreduce_outer_grads
    mlp = w.get("inner") == "mlp"
    cfg = tb.FusedTttConfig.new(CS, w.get("F", F), 1e-6, 128, w["K"])
    if mlp:
        md = {k: host[k].to(dev) for k in MLP_IN}
        mstate = tb.TTTMLPState(md["w1"], md["b1"], md["w2"], md["b2"])
    else:
        ins = tb.TttInputs(*[host[k].to(dev) for k in LIN_IN])
    go = host["grad_output"].to(dev)
    H = host["xq"].shape[1]
    # two packed outer-gradient buffers: the all-reduce of step i overlaps the forward of step i+1
    packed = ([torch.zeros(tb.packed_outer_grad_len(H, w.get("F", F)), device=dev) for _ in range(2)]
              if w["backward"] else None)
    pending = [None, None]
    ev_pairs = []
    step_no = [0]

    def step(record=False):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if record else None
        if record:
            e[0].record()
        if mlp:
            # training step: the forward fills the backward's workspace on the way
            mws = tb.mlp_backward_workspace(md["xq"], cfg) if w["backward"] else None
            outs = tb.fused_ttt_mlp_forward(md["xq"], md["xk"], md["xv"], mstate, md["token_eta"], md["ttt_lr_eta"],
                                            md["ln_weight"], md["ln_bias"], cfg, backward_workspace=mws)
        else:
            outs, saved = tb.TttTileMultiKernel.forward_launch(ins, cfg)
        if record:
            e[1].record()
        g = None
        if w["backward"] and mlp:
            g = tb.fused_ttt_mlp_backward(md["xq"], md["xk"], md["xv"], mstate, md["token_eta"], md["ttt_lr_eta"],
                                          md["ln_weight"], md["ln_bias"], go, cfg, workspace_from_forward=mws)
            if record:
                e[2].record()
        elif w["backward"]:
            i = step_no[0] % 2
            step_no[0] += 1
            if pending[i] is not None:
                pending[i].wait()  # the collective that last used this buffer (two steps ago)
            g = tb.TttTileMultiKernel.backward_launch(saved, tb.TttOutputs(go, None, None), cfg,
                                                      outer_grad_packed=packed[i])
            if record:
                e[2].record()
            if world > 1:
                pending[i] = allreduce_outer_grads(packed[i], async_op=True)
        if record:
            ev_pairs.append(e)
        return outs, g

    def barrier():
        for k in range(2):
            if pending[k] is not None:
                pending[k].wait()
                pending[k] = None
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    tb.check_status(dev)
    sampler = ClockSampler(dev.index)
    sampler.start()
    t_ev0, t_ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_ev0.record()
    for _ in range(args.steps):
        step(record=True)
    for k in range(2):  # the last collectives belong to the timed region
        if pending[k] is not None:
            pending[k].wait()
            pending[k] = None
    t_ev1.record()
    barrier()
    clocks = sampler.stop()
    tb.check_status(dev)  # a kernel that gave up on a wait leaves its outputs unwritten: such a run has no number
    ms = t_ev0.elapsed_time(t_ev1) / args.steps
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev_pairs)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev_pairs) if w["backward"] else None
    if world > 1:
        tmax = torch.tensor([ms, fwd_ms, bwd_ms or 0.0], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms, fwd_ms = tmax[0].item(), tmax[1].item()
        bwd_ms = tmax[2].item() if w["backward"] else None
    # per-step device time (first launch of the step to its last), for the median / minimum the reference's own
    # benchmark protocol reports (rust/cli/src/bench.rs:175-190)
    per_step = sorted(e[0].elapsed_time(e[2] if w["backward"] else e[1]) for e in ev_pairs)
    return {"ms": ms, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "clocks": clocks, "cfg": cfg, "mlp": mlp,
            "median_ms": statistics.median(per_step), "min_ms": per_step[0]}


def roofline_of(w, res, name):
    """Roofline object of a measured workload `w` (the tensors one GPU processed) from bench_inner's timings."""
    peak, peak_kind = measured_peaks()
    mlp = res["mlp"]
    ms, fwd_ms, bwd_ms = res["ms"], res["fwd_ms"], res["bwd_ms"]
    total_b, fb, bb = algorithmic_bytes(w, True, w["backward"])
    if w["backward"]:
        dom_ms, dom_bytes, dom_name = bwd_ms, bb, ("ttt_mlp_bwd_kernel" if mlp else "ttt_linear_bwd_kernel")
    else:
        dom_ms, dom_bytes, dom_name = fwd_ms, fb, ("ttt_mlp_fwd_kernel" if mlp else "ttt_linear_fwd_kernel")
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
    # DRAM bytes per launch of the dominant kernel from the committed ncu summary of this workload, when there is one
    traffic = profile_traffic(f"{dom_name}_{name}_{w['dtype']}")
    roof = {"bound": "hbm", "kernel": dom_name, "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "traffic": traffic, "peak_source": f"of {peak_kind}",
            "algorithmic_bytes_per_launch": dom_bytes, "ms_per_launch": dom_ms,
            "fwd": {"achieved": fb / (fwd_ms * 1e-3) / 1e9, "frac": fb / (fwd_ms * 1e-3) / 1e9 / peak,
                    "ms_per_launch": fwd_ms},
            "step": {"achieved": total_b / (ms * 1e-3) / 1e9, "frac": total_b / (ms * 1e-3) / 1e9 / peak,
                     "algorithmic_bytes": total_b}}
    if mlp:
        # The 2-layer inner model has ~9 times the contraction work of TTT-Linear on the same bytes: its roofline is
        # the slower of the two (north star), which here is the tensor one.  Algorithmic FLOPs per stage and stream
        # (dense contractions only, no recomputation): forward 7 products of 16 x 64 x 256 plus the four 16 x 16
        # attention-like ones = 3,997,696; backward twice that.
        tpeak, tkind = measured_tensor_peak()
        stages = w["B"] * w["H"] * (w["T"] // CS)
        f_fwd, f_bwd = 3997696.0 * stages, 7995392.0 * stages
        dom_flops = f_bwd if w["backward"] else f_fwd
        t_ach = dom_flops / (dom_ms * 1e-3) / 1e12
        if dom_flops / (tpeak * 1e12) > dom_bytes / (peak * 1e9):
            hbm = {k: roof[k] for k in ("achieved", "peak", "unit", "frac", "algorithmic_bytes_per_launch")}
            roof.update({"bound": "tensor", "achieved": t_ach, "peak": tpeak, "unit": "TFLOP/s", "frac": t_ach / tpeak,
                         "peak_source": f"of {tkind} (cuBLAS bf16 burst)", "algorithmic_flops_per_launch": dom_flops,
                         "hbm": hbm})
            tot_f = f_fwd + (f_bwd if w["backward"] else 0.0)
            roof["fwd"] = {"achieved": f_fwd / (fwd_ms * 1e-3) / 1e12, "frac": f_fwd / (fwd_ms * 1e-3) / 1e12 / tpeak,
                           "ms_per_launch": fwd_ms}
            roof["step"] = {"achieved": tot_f / (ms * 1e-3) / 1e12, "frac": tot_f / (ms * 1e-3) / 1e12 / tpeak}
    return roof


def side_workload(tb, name, dev, args):
    """A compact record of another workload measured in the same run (single GPU): per-kernel times and roofline."""
    w = WORKLOADS[name]
    host = make_host_inputs(w, seed=0)
    a2 = argparse.Namespace(**vars(args))
    a2.steps, a2.warmup = max(3, min(args.steps, 5)), 3
    res = bench_inner(tb, w, host, dev, 1, 0, a2, name)
    roof = roofline_of(w, res, name)
    out = {"workload": w["desc"], "ms_per_step": res["ms"], "fwd_ms": res["fwd_ms"], "bwd_ms": res["bwd_ms"],
           "tokens_per_s": w["B"] * w["T"] / (res["ms"] * 1e-3), "steps": a2.steps,
           "roofline": {"bound": roof["bound"], "kernel": roof["kernel"], "frac": roof["frac"],
                        "achieved": roof["achieved"], "unit": roof["unit"], "step_frac": roof["step"]["frac"],
                        "fwd_frac": roof["fwd"]["frac"]}}
    del host
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg1", choices=sorted(WORKLOADS))
    ap.add_argument("--scaling", default="auto", choices=["auto", "strong", "weak"],
                    help="N > 1: partition the workload's batch over the ranks (strong) or give every rank the whole "
                         "per-GPU workload (weak); auto = strong as the line's value plus weak as an extra key")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-side-workloads", action="store_true",
                    help="skip the compact cfg2 / cfg4-8k records a default single-GPU cfg1 run adds")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if w.get("kind") == "probe":
        import subprocess
        from ttt_rs_b200.build import build_probe
        out = subprocess.run([str(build_probe())], capture_output=True, text=True, timeout=120)
        if out.returncode != 0:
            raise SystemExit(f"probe failed ({out.returncode}): {out.stderr[-400:]}")
        line = json.loads(out.stdout.strip().splitlines()[-1])
        line.update({"metric": "dependent_tensor_core_step_cycles", "unit": "cycles/step", "higher_is_better": False,
                     "config": {"workload": w["desc"]}})
        print(json.dumps(line), flush=True)
        return
    if w.get("kind") in ("decode-layer", "decode", "layer"):
        if args.impl == "reference":
            raise SystemExit("--impl reference is defined for the inner-loop workloads")
        {"decode-layer": run_decode_layer, "decode": run_decode, "layer": run_layer}[w["kind"]](args, w)
        return
    if args.impl == "reference":
        run_reference(args, w)
        return

    import torch.distributed as dist
    import ttt_rs_b200 as tb
    from ttt_rs_b200.distributed import shard_batch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tb.load_library()
    if w["B"] % world != 0 and args.scaling != "weak":
        raise SystemExit(f"strong scaling needs the batch ({w['B']}) to be a multiple of the rank count ({world})")

    mode = "weak" if args.scaling == "weak" else "strong"
    if world == 1:
        mode = "strong"  # one GPU: the whole workload either way
    # ---- device-resident inputs: strong = this rank's batch rows of the seed-0 tensors; weak = a whole workload
    # per rank, seeded by the rank
    if mode == "strong":
        a, b = shard_batch(w["B"], rank, world)
        host = shard_rows(make_host_inputs(w, seed=0), a, b)
        w_rank = dict(w, B=b - a)
        tokens = w["B"] * w["T"]
    else:
        host = make_host_inputs(w, seed=rank)
        w_rank = w
        tokens = w["B"] * w["T"] * world
    res = bench_inner(tb, w_rank, host, dev, world, rank, args, args.workload)
    ms = res["ms"]
    value = tokens / (ms * 1e-3)
    roof = roofline_of(w_rank, res, args.workload)
    mlp = res["mlp"]

    # ---- end to end through the public operator with host buffers (pinned), copies inside the timed region
    e2e = None
    if not args.no_e2e and not mlp:
        e2e = run_e2e(tb, w_rank, host, dev, res["cfg"], world, args, tokens)

    weak = None
    if world > 1 and args.scaling == "auto":
        hostw = make_host_inputs(w, seed=rank)
        a2 = argparse.Namespace(**vars(args))
        a2.steps = max(3, min(args.steps, 10))
        rw = bench_inner(tb, w, hostw, dev, world, rank, a2, args.workload)
        weak = {"value": w["B"] * w["T"] * world / (rw["ms"] * 1e-3), "unit": "tokens/s", "ms_per_step": rw["ms"],
                "global_batch": w["B"] * world, "steps": a2.steps,
                "note": "every rank runs the whole per-GPU workload on its own seed (no data-path collective)"}
        del hostw

    if rank == 0:
        streams = w_rank["B"] * w_rank["H"]
        line = {
            "metric": "ttt_inner_loop_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": mode, "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": w["desc"], "global_batch": w["B"] * (world if mode == "weak" else 1),
                       "parallelism": f"streams-dp{world}", "streams_per_gpu": streams,
                       "l2": "inputs exceed L2: each step streams %.0f MB of operands per GPU"
                             % (roof["step"].get("algorithmic_bytes", 0) / 1e6) if not mlp else
                             "inputs exceed L2 (%.0f MB of operands per step)" % (algorithmic_bytes(w_rank)[0] / 1e6)},
            "ms_per_step_median": res["median_ms"], "ms_per_step_min": res["min_ms"],
            "clocks": res["clocks"], "e2e": e2e,
            "gpu_launches": args.steps * ((3 if mlp else 4) if w["backward"] else 1),
            "roofline": roof,
        }
        if weak is not None:
            line["weak"] = weak
        if world == 1 and args.workload == "cfg1" and not args.no_side_workloads:
            line["workloads"] = {n: side_workload(tb, n, dev, args) for n in ("cfg2", "cfg4-8k")}
        if world == 1 and not args.no_cpu_baseline:
            val, dt, cores, sample = time_cpu(w, 3, 1)
            line["cpu_baseline"] = {"value": val, "unit": "tokens/s", "cores": cores, "kind": cpu_kind(),
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def copy_ceiling(pinned, out_host, dev, world, steps):
    """Time of plain pinned-memory copies of one step's byte counts -- every input host-to-device on one stream, every
    output device-to-host on another, concurrently, on all ranks at once -- with no kernel in between: the floor the
    host link puts under the end-to-end step."""
    import torch.distributed as dist
    din = {k: torch.empty_like(v, device=dev) for k, v in pinned.items()}
    dout = {k: torch.empty_like(v, device=dev) for k, v in out_host.items()}
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def once():
        cur = torch.cuda.current_stream(dev)
        s1.wait_stream(cur)
        s2.wait_stream(cur)
        with torch.cuda.stream(s1):
            for k, v in pinned.items():
                din[k].copy_(v, non_blocking=True)
        with torch.cuda.stream(s2):
            for k, v in out_host.items():
                v.copy_(dout[k], non_blocking=True)
        cur.wait_stream(s1)
        cur.wait_stream(s2)

    once()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        once()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        tmax = torch.tensor([ms], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms = tmax.item()
    return ms


def run_e2e(tb, w, host, dev, cfg, world, args, tokens):
    """Same metric through the operator a user calls, starting from pinned HOST buffers: every step copies the
    step's inputs to the device, runs forward (+ backward), and copies output and gradients back to the host
    (ttt_rs_b200.host_io.HostBatchRunner: batch chunks pipelined over three streams).  `w` / `host` are this rank's
    share of the workload; `tokens` the job's tokens per step."""
    import torch.distributed as dist
    from ttt_rs_b200.host_io import HostBatchRunner, alloc_host_outputs, bind_host_thread_near
    numa_node = bind_host_thread_near(dev) if world > 1 else None  # pinned buffers in the GPU's own NUMA node
    names_in = ("xq", "xk", "xv", "ttt_lr_eta") + (("grad_output",) if w["backward"] else ())
    pinned = {k: host[k].pin_memory() for k in names_in}
    params = {k: host[k].to(dev) for k in ("weight", "bias", "token_eta", "ln_weight", "ln_bias")}
    out_host = alloc_host_outputs(w["B"], w["H"], w["T"], w.get("F", F), host["xq"].dtype, w["backward"])
    runner = HostBatchRunner(cfg, dev, chunks=E2E_CHUNKS, backward=w["backward"])

    for _ in range(2):
        runner.run(pinned, params, out_host)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    steps = max(3, min(args.steps, 10))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        runner.run(pinned, params, out_host)
    e1.record()
    torch.cuda.synchronize()
    tb.check_status(dev)
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        tmax = torch.tensor([ms], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms = tmax.item()
    h2d = sum(v.numel() * v.element_size() for v in pinned.values())
    d2h = sum(v.numel() * v.element_size() for v in out_host.values())
    ceiling = copy_ceiling(pinned, out_host, dev, world, steps)
    return {"value": tokens / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": steps,
            "copy_ceiling_ms": ceiling,
            "copy_ceiling_note": "the same H2D and D2H byte counts as plain pinned cudaMemcpyAsync on two streams, all "
                                 "ranks at once, no kernels: the step is bound by the host link when ms_per_step is "
                                 "close to it (bytes are per rank)",
            "how": f"pinned host buffers, {len(runner.last_bounds) - 1} equal batch chunks pipelined over copy-in / compute / "
                   "copy-out streams; the small per-row tensors cross the link once per step",
            "host_numa_node": numa_node}


if __name__ == "__main__":
    main()
