"""ctypes binding of libttt_b200.so (the C ABI declared in include/ttt_b200.h).

This is the binding a host language would write against the header: plain pointers and sizes, no torch types.
There is no fallback: if the library has not been built, loading raises.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Optional

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libttt_b200.so"

TTT_OK = 0
TTT_ERR_NULL = 1
TTT_ERR_SHAPE = 2
TTT_ERR_UNSUPPORTED = 3
TTT_ERR_ALIGN = 4
TTT_ERR_CUDA = 5
TTT_ERR_TIMEOUT = 6
TTT_ERR_WORKSPACE = 7

TTT_F32 = 0
TTT_BF16 = 1


class TttDims(C.Structure):
    """struct ttt_dims"""
    _fields_ = [
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq_len", C.c_int32), ("head_dim", C.c_int32),
        ("mini_batch", C.c_int32), ("checkpoint_interval", C.c_int32), ("epsilon", C.c_float),
        ("dtype", C.c_int32),
    ]


class TttError(RuntimeError):
    """Raised where the reference would panic (bad shapes, unsupported tile configuration, launch failure)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"ttt_b200 error {code}: {message}")
        self.code = code


# every symbol include/ttt_b200.h declares: name -> (restype, argtypes)
_P = C.c_void_p
_DP = C.POINTER(TttDims)
SYMBOLS = {
    "ttt_b200_abi_version": (C.c_int, []),
    "ttt_b200_status_string": (C.c_char_p, [C.c_int]),
    "ttt_b200_last_error": (C.c_char_p, []),
    "ttt_b200_debug_handoff": (None, [C.c_uint32, C.c_int32]),
    "ttt_linear_num_checkpoints": (C.c_int64, [_DP]),
    "ttt_linear_weight_ckpt_bytes": (C.c_size_t, [_DP]),
    "ttt_linear_bias_ckpt_bytes": (C.c_size_t, [_DP]),
    "ttt_linear_forward": (C.c_int, [_DP] + [_P] * 16),
    "ttt_linear_backward_workspace_bytes": (C.c_size_t, [_DP]),
    "ttt_linear_backward": (C.c_int, [_DP] + [_P] * 23 + [C.c_size_t, _P, _P]),
    "ttt_linear_backward_noalloc": (C.c_int, [_DP] + [_P] * 22 + [_P, _P]),
    "ttt_mlp_forward": (C.c_int, [_DP] + [_P] * 17 + [C.c_size_t, _P, _P]),
    "ttt_linear_backward_state_grads": (C.c_int, [_DP] + [_P] * 25 + [C.c_size_t, _P, _P]),
    "ttt_mlp_backward_workspace_bytes": (C.c_size_t, [_DP]),
    "ttt_mlp_backward": (C.c_int, [_DP] + [_P] * 24 + [C.c_size_t, C.c_int, _P, _P]),
    "ttt_linear_forward_partial": (C.c_int, [_DP] + [_P] * 13),
    "ttt_layer_prologue": (C.c_int, [_DP, _P, _P, _P, C.c_int64, _P, C.c_int64, _P, _P, _P, _P, _P, C.c_int, C.c_int,
                                     C.c_int, C.c_float, C.c_float, _P, _P, _P, _P, _P]),
    "ttt_layer_prologue_backward": (C.c_int, [_DP, _P, _P, _P, _P, _P, C.c_int, C.c_int, C.c_float, C.c_float, _P, _P,
                                              _P, C.c_int64, _P, C.c_int64, C.c_int, _P]),
    "ttt_layer_epilogue_backward_workspace_bytes": (C.c_size_t, [_DP]),
    "ttt_layer_epilogue_backward": (C.c_int, [_DP, _P, _P, _P, C.c_int64, _P, _P, C.c_float, _P, _P, C.c_int64, _P,
                                              _P, _P, C.c_size_t, _P]),
    "ttt_layer_epilogue": (C.c_int, [_DP, _P, _P, C.c_int64, _P, _P, C.c_float, _P, _P]),
    "ttt_gemm_bf16_tn": (C.c_int, [C.c_int64, C.c_int64, C.c_int64, _P, C.c_int64, _P, C.c_int64, _P, C.c_int64, _P, _P]),
    "ttt_layer_projections": (C.c_int, [_DP, _P, C.c_int64, C.c_int64, _P, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                        C.c_int64, C.c_int64, C.c_int64, _P, C.c_int, C.c_int, C.c_float, C.c_float,
                                        _P, _P, _P, _P, _P, _P, _P]),
    "ttt_layer_qk_conv": (C.c_int, [_DP, _P, C.c_int64, _P, _P, _P, _P, _P, _P, _P]),
    "ttt_layer_qk_conv_backward_workspace_bytes": (C.c_size_t, [_DP]),
    "ttt_layer_qk_conv_backward": (C.c_int, [_DP, _P, _P, _P, C.c_int64, _P, _P, _P, _P, _P, _P, C.c_size_t, _P]),
}

NOALLOC_SCRATCH_BYTES = 32 << 20  # TTT_NOALLOC_SCRATCH_BYTES

_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ttt_rs_b200.build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this operator.")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().ttt_b200_last_error().decode()


def check(rc: int) -> None:
    if rc != TTT_OK:
        raise TttError(rc, last_error() or load().ttt_b200_status_string(rc).decode())
