"""The projection GEMM (`ttt_gemm_bf16_tn`: tcgen05.mma, accumulators in tensor memory, TMA in and out) against a
float64 product of the same bf16 operands.  The result is rounded to bf16 once, so the bound is bf16 rounding of the
exact value: 2^-8 relative to each element plus a float32-accumulation floor."""

import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [
    (128, 128, 64),      # one tile, one k-block
    (128, 128, 768),     # the ring wraps (12 k-blocks over 3 stages)
    (256, 200, 768),     # N not a multiple of the tile: clipped store, second half-tile partly out of range
    (1000, 2320, 768),   # ragged M; the layer's fused projection width at 12 heads
    (300, 72, 104),      # ragged everything: K tail zero-filled by the tensor map, N < 128
    (4096, 768, 768),    # o_proj at the 125M layer shape
])
def test_gemm_matches_float64_product(M, N, K):
    import ttt_rs_b200 as tb
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    c = tb.gemm_bf16_tn(a.to(dev), b.to(dev))
    tb.check_status()
    want = a.double() @ b.double().t()
    assert c.shape == (M, N) and c.dtype == torch.bfloat16
    assert_close(c, want, 4e-3, f"gemm {M}x{N}x{K}")


def test_gemm_with_row_pitch_larger_than_the_row():
    """Operands and result as column blocks of wider buffers (how the layer slices its fused projection)."""
    import ctypes as C
    import ttt_rs_b200 as tb
    from ttt_rs_b200 import _lib
    dev = torch.device("cuda:0")
    M, N, K = 384, 136, 128
    g = torch.Generator().manual_seed(1)
    abuf = (torch.randn(M, K + 64, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    bbuf = (torch.randn(N, K + 8, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    cbuf = torch.full((M, N + 24), 7.0, dtype=torch.bfloat16, device=dev)
    lib = _lib.load()
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    _lib.check(lib.ttt_gemm_bf16_tn(M, N, K, p(abuf), abuf.stride(0), p(bbuf), bbuf.stride(0), p(cbuf), cbuf.stride(0),
                                    None, C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    torch.cuda.synchronize()
    want = abuf[:, :K].double().cpu() @ bbuf[:, :K].double().cpu().t()
    assert_close(cbuf[:, :N], want, 4e-3, "gemm into a column block")
    assert (cbuf[:, N:] == 7.0).all(), "columns beyond N must not be written"


def test_gemm_rejects_bad_arguments():
    import ctypes as C
    from ttt_rs_b200 import _lib
    lib = _lib.load()
    fake = C.c_void_p(0x1000)
    assert lib.ttt_gemm_bf16_tn(0, 8, 8, fake, 8, fake, 8, fake, 8, None, None) == _lib.TTT_ERR_SHAPE
    assert lib.ttt_gemm_bf16_tn(8, 8, 8, fake, 4, fake, 8, fake, 8, None, None) == _lib.TTT_ERR_SHAPE
    assert lib.ttt_gemm_bf16_tn(8, 8, 8, fake, 12, fake, 8, fake, 8, None, None) == _lib.TTT_ERR_ALIGN
    assert lib.ttt_gemm_bf16_tn(8, 8, 8, None, 8, fake, 8, fake, 8, None, None) == _lib.TTT_ERR_NULL
