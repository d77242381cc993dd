"""tile_gemm (the tiled tcgen05 GEMM for prefill passes and large decode steps) through the C ABI against a plain
PyTorch fp32 reference of the same operation. Tolerance: the fp32 product differs from the reference only by
summation order (about 1e-6 relative), so bf16 outputs agree to one rounding step of the largest output in the row
block; the test allows one such step (at most 2^-7 relative to the largest magnitude)."""

import pytest
import torch

from nanochat_b200.native import cuda_library, pointer, stream

pytestmark = pytest.mark.gpu


def reference(x, w, resid, epilogue):
    y = x.float() @ w.float().T
    if epilogue == 3:
        return y
    y = y.bfloat16()
    if epilogue == 1:
        y = (resid.float() + y.float()).bfloat16()
    if epilogue == 2:
        y = y.float().clamp_min(0).square().bfloat16()
    return y


def run(rows, N, K, epilogue, seed=0, alias=False, form=0):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, K, generator=gen, device="cuda").bfloat16()
    w = (torch.randn(N, K, generator=gen, device="cuda") * K ** -0.5).bfloat16()
    resid = torch.randn(rows, N, generator=gen, device="cuda").bfloat16() if epilogue == 1 else None
    want = reference(x, w, resid, epilogue)
    y = torch.full((rows, N), float("nan"), dtype=torch.float32 if epilogue == 3 else torch.bfloat16, device="cuda")
    if alias:
        y.copy_(resid)
        resid = y
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib = cuda_library("tile_gemm")
    if form == 0:
        rc = lib.tile_gemm(pointer(x), pointer(w), pointer(resid), pointer(y), rows, N, K, epilogue, pointer(status), stream())
    else:
        rc = lib.tile_gemm_form(pointer(x), pointer(w), pointer(resid), pointer(y), rows, N, K, epilogue, form,
                                pointer(status), stream())
    torch.cuda.synchronize()
    assert rc == 0 and status.item() == 0
    return y, want


@pytest.mark.parametrize("rows,N,K", [(1, 128, 64), (65, 256, 256), (128, 384, 1280), (129, 768, 512), (300, 1280, 5120),
                                      (511, 3840, 1280), (4088, 1280, 1280), (1000, 128, 2048)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_tile_gemm_matches_torch(rows, N, K, epilogue):
    y, want = run(rows, N, K, epilogue, seed=rows + N + K + epilogue)
    assert torch.isfinite(y.float()).all()
    err = (y.float() - want.float()).abs()
    top = float(want.float().abs().max())
    if epilogue == 3:
        assert float(err.max()) <= 2e-5 * max(top, 1.0) * (K / 64) ** 0.5
    else:
        assert float(err.max()) <= 2 ** -7 * top + 1e-6, (float(err.max()), top)
        assert float((err > 0).float().mean()) < 0.02  # roundings flip only where the fp32 sums straddle a boundary


@pytest.mark.parametrize("rows,N,K", [(129, 256, 64), (256, 640, 64), (300, 640, 256), (700, 1280, 256), (511, 3840, 1280),
                                      (4088, 1280, 5120), (4088, 5120, 1280), (5000, 2560, 128), (9500, 2048, 192)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_block_pair_form_gives_the_single_block_form_bits(rows, N, K, epilogue):
    """tile_gemm_form: a pair of blocks per 256 x 256 or 256 x 320 tile (form 2) against one block per tile (form 1):
    the same bits (a product's k-blocks are accumulated in the same order), several tiles per pair, half-width last
    rounds, row tiles that end inside a pair's second block, and both against torch."""
    one, want = run(rows, N, K, epilogue, seed=rows + N + K + epilogue, form=1)
    two, _ = run(rows, N, K, epilogue, seed=rows + N + K + epilogue, form=2)
    auto, _ = run(rows, N, K, epilogue, seed=rows + N + K + epilogue, form=0)
    assert torch.equal(one, two) and torch.equal(one, auto)
    err = (two.float() - want.float()).abs()
    top = float(want.float().abs().max())
    assert float(err.max()) <= (2e-5 * max(top, 1.0) * (K / 64) ** 0.5 if epilogue == 3 else 2 ** -7 * top + 1e-6)


def test_block_pair_form_refuses_other_widths():
    import ctypes
    lib, p = cuda_library("tile_gemm"), ctypes.c_void_p(4096)
    assert lib.tile_gemm_form(p, p, None, p, 300, 384, 64, 0, 2, None, None) == 5   # neither a multiple of 256 nor of 640
    assert lib.tile_gemm_form(p, p, None, p, 300, 256, 64, 0, 3, None, None) == 1   # no such form


def test_tile_gemm_many_tiles_per_block_and_in_place_residual():
    """More tiles than SMs, so blocks walk over several tiles and both accumulators are in use; residual in place."""
    y, want = run(4096, 5120, 1280, 2, seed=5)  # 32 x 20 = 640 tiles
    assert float((y.float() - want.float()).abs().max()) <= 2 ** -7 * float(want.float().abs().max()) + 1e-6
    y, want = run(700, 1280, 256, 1, seed=6, alias=True)
    assert float((y.float() - want.float()).abs().max()) <= 2 ** -7 * float(want.float().abs().max()) + 1e-6


def test_tile_gemm_is_deterministic_and_validates():
    a, _ = run(1000, 2048, 2048, 0, seed=9)
    b, _ = run(1000, 2048, 2048, 0, seed=9)
    assert torch.equal(a, b)
    lib = cuda_library("tile_gemm")
    import ctypes
    p = ctypes.c_void_p(4096)
    assert lib.tile_gemm(p, p, None, p, 8, 100, 64, 0, None, None) == 1      # N not a multiple of 128
    assert lib.tile_gemm(p, p, None, p, 8, 128, 100, 0, None, None) == 1     # K not a multiple of 64
    assert lib.tile_gemm(p, p, None, p, 8, 128, 64, 1, None, None) == 1      # residual epilogue without a residual
    assert lib.tile_gemm(p, p, None, p, 0, 128, 64, 0, None, None) == 0      # nothing to do
    assert lib.tile_gemm(ctypes.c_void_p(4100), p, None, p, 8, 128, 64, 0, None, None) == 2
