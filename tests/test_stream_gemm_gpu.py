"""stream_gemm (tcgen05 weight-streaming GEMM for up to 256 rows, K split over a cluster) through the C ABI against
a plain PyTorch fp32 reference of the same operation."""

import pytest
import torch

from nanochat_b200.native import cuda_library, pointer, stream

pytestmark = pytest.mark.gpu
EPS = 1.1920928955078125e-07


def gemm(x, w, resid, norm, epilogue, split=0, status=None, next_w=None):
    rows, K = x.shape
    N = w.shape[0]
    y = torch.empty((rows, N), dtype=torch.float32 if epilogue == 3 else torch.bfloat16, device="cuda")
    if epilogue == 1:
        y.copy_(resid)  # in place, as the decoder uses it
    rc = cuda_library("stream_gemm").stream_gemm(pointer(x), pointer(w), pointer(y if epilogue == 1 else None),
                                                 pointer(y), rows, N, K, norm, epilogue, split, pointer(next_w),
                                                 0 if next_w is None else next_w.numel() * next_w.element_size(),
                                                 pointer(status), stream())
    assert rc == 0
    return y


def reference(x, w, resid, norm, epilogue):
    acc = x.float() @ w.float().T  # bf16 products are exact in fp32; only the summation order differs
    if norm:  # the kernel scales the fp32 product by the row's 1 / sqrt(mean(x^2) + eps)
        acc = acc * torch.rsqrt(x.float().square().mean(-1, keepdim=True) + EPS)
    if epilogue == 3:
        return acc
    y = acc.bfloat16()
    if epilogue == 1:
        return (resid.float() + y.float()).bfloat16()
    if epilogue == 2:
        return torch.relu(y).float().square().bfloat16()
    return y


def check(got, want):
    err = (got.float() - want.float()).abs()
    scale = want.float().abs().max().clamp(min=1.0)
    # one bf16 rounding step of difference where the fp32 sums straddle a rounding boundary, nothing more
    assert err.max() <= 2 ** -7 * scale, (float(err.max()), float(scale))
    assert err.mean() <= 2e-4 * scale


@pytest.mark.parametrize("rows", [1, 17, 32, 33, 64, 100, 128, 129, 256])
@pytest.mark.parametrize("N,K,norm", [(3072, 2048, 1), (2048, 2048, 0), (8192, 2048, 1), (2048, 8192, 0), (128, 64, 1),
                                      (1280, 5120, 0), (3840, 1280, 1), (256, 192, 0)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_stream_gemm_matches_torch(rows, N, K, norm, epilogue):
    gen = torch.Generator().manual_seed(rows * 1000 + N + K + epilogue)
    x = torch.randn(rows, K, generator=gen).bfloat16().cuda()
    w = (torch.randn(N, K, generator=gen) * 0.05).bfloat16().cuda()
    resid = torch.randn(rows, N, generator=gen).bfloat16().cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = gemm(x, w, resid, norm, epilogue, status=status)
    check(got, reference(x, w, resid, norm, epilogue))
    assert int(status.item()) == 0


@pytest.mark.parametrize("split", [1, 2, 3, 5, 8])
def test_every_split_gives_the_same_sums_up_to_order(split):
    gen = torch.Generator().manual_seed(split)
    x = torch.randn(40, 1024, generator=gen).bfloat16().cuda()
    w = (torch.randn(640, 1024, generator=gen) * 0.05).bfloat16().cuda()
    got = gemm(x, w, None, 1, 3, split=split)
    check(got, reference(x, w, None, 1, 3))


def test_a_split_is_deterministic():
    gen = torch.Generator().manual_seed(7)
    x = torch.randn(32, 2048, generator=gen).bfloat16().cuda()
    w = (torch.randn(2048, 2048, generator=gen) * 0.05).bfloat16().cuda()
    first = gemm(x, w, None, 1, 3)
    for _ in range(5):
        assert torch.equal(gemm(x, w, None, 1, 3), first)


def test_prefetching_the_next_weights_changes_nothing():
    gen = torch.Generator().manual_seed(13)
    x = torch.randn(32, 2048, generator=gen).bfloat16().cuda()
    w = (torch.randn(2048, 2048, generator=gen) * 0.05).bfloat16().cuda()
    nxt = (torch.randn(8192 * 2048 + 8, generator=gen) * 0.05).bfloat16().cuda()  # not a multiple of the block count
    plain = gemm(x, w, None, 1, 0)
    assert torch.equal(gemm(x, w, None, 1, 0, next_w=nxt), plain)
    assert torch.equal(gemm(x, w, None, 1, 0, split=1, next_w=nxt[:8]), gemm(x, w, None, 1, 0, split=1))
    lib = cuda_library("stream_gemm")
    p = pointer(x)
    assert lib.stream_gemm(p, p, None, p, 4, 128, 256, 0, 0, 0, p, 24, None, None) == 2  # not a multiple of 16 bytes


def test_head_sized_gemm_keeps_fp32_logits():
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(32, 2048, generator=gen).bfloat16().cuda()
    w = (torch.randn(65536, 2048, generator=gen) * 0.02).bfloat16().cuda()
    got = gemm(x, w, None, 1, 3)
    want = reference(x, w, None, 1, 3)
    assert got.dtype == torch.float32
    assert (got - want).abs().max() <= 1e-3 * want.abs().max()


def test_stream_gemm_rejects_unsupported_shapes():
    lib = cuda_library("stream_gemm")
    x = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    p = pointer(x)
    assert lib.stream_gemm(p, p, None, p, 257, 128, 256, 0, 0, 0, None, 0, None, None) == 1   # more than 256 rows
    assert lib.stream_gemm(p, p, None, p, 4, 100, 256, 0, 0, 0, None, 0, None, None) == 1     # N not a multiple of 128
    assert lib.stream_gemm(p, p, None, p, 4, 128, 100, 0, 0, 0, None, 0, None, None) == 1     # K not a multiple of 64
    assert lib.stream_gemm(p, p, None, p, 4, 128, 128, 0, 0, 3, None, 0, None, None) == 1     # more blocks than k-blocks
    assert lib.stream_gemm(p, p, None, p, 4, 128, 256, 0, 1, 0, None, 0, None, None) == 1     # residual epilogue, no residual
    assert lib.stream_gemm(p, p, None, p, 0, 128, 256, 0, 0, 0, None, 0, None, None) == 0     # nothing to do
    assert lib.stream_gemm_split(32, 2048, 2048) == 8 and lib.stream_gemm_split(32, 65536, 2048) == 1
    assert lib.stream_gemm_split(32, 100, 2048) == 0
