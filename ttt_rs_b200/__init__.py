"""B200 (sm_100a) fused TTT inner loop behind the reference's `fused-tile-multi` operator interface."""

from ._lib import TttDims, TttError, load as load_library  # noqa: F401
from .fused import (  # noqa: F401
    FusedTTTMLP,
    FusedTileMultiTTTLinear,
    FusedTttConfig,
    Qkv,
    TTTInputsInner,
    TTTLinear,
    TTTLinearState,
    TTTMLP,
    TTTMLPState,
    TttInputs,
    TttOutputs,
    TttSavedStateMulti,
    TttTileMultiKernel,
    fused_ttt_mlp,
    fused_ttt_mlp_backward,
    check_mlp_status,
    check_status,
    device_status,
    mlp_backward_workspace,
    fused_ttt_mlp_forward,
    fused_ttt_tile_forward_multi,
    packed_outer_grad_len,
    unpack_weight_checkpoints,
)
from .layer import TTT, DecodeGraphs, TTTLayerConfig, gemm_bf16_tn, layer_epilogue, layer_projections, layer_prologue, new_inner  # noqa: F401,E402
