"""Builds the CUDA library (libttt_b200.so) for sm_100a with nvcc, in-tree.

    python -m ttt_rs_b200.build            # rebuild if any source is newer than the library
    python -m ttt_rs_b200.build --force
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libttt_b200.so"
PROBE_SRC = CSRC / "probe_chain_latency.cu"      # stand-alone measurement program (bench.py --workload chain-latency)
PROBE_BIN = PKG / "build" / "probe_chain_latency"
SOURCES = ["ttt_abi.cu", "ttt_linear_fwd.cu", "ttt_linear_bwd.cu", "ttt_mlp_fwd.cu", "ttt_layer.cu", "ttt_linear_partial.cu", "ttt_mlp_bwd.cu", "ttt_gemm.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or install the CUDA toolkit)")


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [p for p in CSRC.glob("*.cu") if p != PROBE_SRC] + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + \
        list((PKG.parent / "include").glob("*.h"))
    return any(p.stat().st_mtime > t for p in deps)


def build_probe(force: bool = False) -> Path:
    """The tensor-core chain-latency probe: its own executable, nothing of the library depends on it."""
    if not force and PROBE_BIN.exists() and PROBE_BIN.stat().st_mtime >= PROBE_SRC.stat().st_mtime:
        return PROBE_BIN
    PROBE_BIN.parent.mkdir(exist_ok=True)
    cmd = [find_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-o", str(PROBE_BIN), str(PROBE_SRC)]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {PROBE_SRC.name}:\n{r.stdout}")
    return PROBE_BIN


def build(force: bool = False, verbose: bool = False) -> Path:
    build_probe(force)
    if not force and not needs_build():
        return LIB
    nvcc = find_nvcc()
    objs = []
    build_dir = PKG / "build"
    build_dir.mkdir(exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = build_dir / (src + ".o")
        extra = os.environ.get("TTT_NVCC_EXTRA", "").split()
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    log = []
    for src, pr in procs:
        out, _ = pr.communicate()
        log.append(f"== {src}\n{out}")
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    cmd = [nvcc, "-shared", "-o", str(LIB), *objs]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    (build_dir / "ptxas.log").write_text("\n".join(log))
    if verbose:
        print("\n".join(log))
    return LIB


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose=True)
    print(f"built {p}")
