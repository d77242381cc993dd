"""The decode_step kernels (skinny GEMM with fused norm and epilogues, embedding + norm, greedy choice) through the
C ABI against plain PyTorch references of the same operations."""

import pytest
import torch
import torch.nn.functional as F

from nanochat_b200.native import cuda_library, pointer, stream

pytestmark = pytest.mark.gpu
EPS = 1.1920928955078125e-07


def gemm(x, w, resid, rows, N, K, norm, epilogue):
    y = torch.empty((rows, N), dtype=torch.float32 if epilogue == 3 else torch.bfloat16, device="cuda")
    if epilogue == 1:
        y.copy_(resid)  # in place, as the decoder uses it
    rc = cuda_library("decode_step").skinny_gemm(pointer(x), pointer(w), pointer(y if epilogue == 1 else None),
                                                 pointer(y), rows, N, K, norm, epilogue, stream())
    assert rc == 0
    return y


def reference(x, w, resid, norm, epilogue):
    xn = F.rms_norm(x, (x.size(-1),), eps=EPS) if norm else x
    acc = xn.float() @ w.float().T  # bf16 products are exact in fp32; only the summation order differs
    if epilogue == 3:
        return acc
    y = acc.bfloat16()
    if epilogue == 1:
        return (resid.float() + y.float()).bfloat16()
    if epilogue == 2:
        return F.relu(y).float().square().bfloat16()
    return y


@pytest.mark.parametrize("rows", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K,norm", [(3840, 1280, 1), (1280, 1280, 0), (5120, 1280, 1), (1280, 5120, 0), (512, 256, 1),
                                      (64, 2048, 1), (8, 768, 0)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_skinny_gemm_matches_torch(rows, N, K, norm, epilogue):
    gen = torch.Generator().manual_seed(rows * 1000 + N + K + epilogue)
    x = torch.randn(rows, K, generator=gen).bfloat16().cuda()
    w = (torch.randn(N, K, generator=gen) * 0.05).bfloat16().cuda()
    resid = torch.randn(rows, N, generator=gen).bfloat16().cuda()
    got = gemm(x, w, resid, rows, N, K, norm, epilogue)
    want = reference(x, w, resid, norm, epilogue)
    torch.cuda.synchronize()
    err = (got.float() - want.float()).abs()
    scale = want.float().abs().max().clamp(min=1.0)
    # one bf16 rounding step of difference where the fp32 sums straddle a rounding boundary, nothing more
    assert err.max() <= 2 ** -7 * scale, (float(err.max()), float(scale))
    assert err.mean() <= 2e-4 * scale


def test_skinny_gemm_rejects_unsupported_shapes():
    lib = cuda_library("decode_step")
    x = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    p = pointer(x)
    assert lib.skinny_gemm(p, p, None, p, 17, 8, 256, 0, 0, None) == 1      # more than 16 rows
    assert lib.skinny_gemm(p, p, None, p, 4, 8, 100, 0, 0, None) == 1       # K not a multiple of 256
    assert lib.skinny_gemm(p, p, None, p, 4, 8, 8192, 0, 0, None) == 5      # K above 5120
    assert lib.skinny_gemm(p, p, None, p, 4, 8, 4096, 1, 0, None) == 5      # fused norm above 2048
    assert lib.skinny_gemm(p, p, None, p, 4, 8, 256, 0, 1, None) == 1       # residual epilogue without a residual


def test_embed_norm_and_greedy_choice():
    gen = torch.Generator().manual_seed(9)
    V, C, rows = 1000, 1280, 5
    embed = torch.randn(V, C, generator=gen).bfloat16().cuda()
    tokens = torch.tensor([0, 999, 17, 17, 500], device="cuda")
    h = torch.empty((rows, C), dtype=torch.bfloat16, device="cuda")
    lib = cuda_library("decode_step")
    assert lib.embed_norm(pointer(embed), pointer(tokens), pointer(h), rows, C, V, stream()) == 0
    want = F.rms_norm(embed[tokens], (C,), eps=EPS)
    assert (h.float() - want.float()).abs().max() <= 2 ** -7 * want.float().abs().max()
    assert torch.equal(h[2], h[3])

    logits = torch.randn(rows, 65536, generator=gen).cuda()
    logits[1, 40000] = logits[1, 123] = 50.0  # a tie: the lowest id wins
    logits[2, 65535] = 60.0
    pos = torch.tensor([3, 4, 5, 6, 7], dtype=torch.int32, device="cuda")
    trace = torch.full((rows, 16), -1, dtype=torch.long, device="cuda")
    assert lib.greedy_choice(pointer(logits), pointer(tokens), pointer(pos), rows, 65536, pointer(trace), 16,
                             stream()) == 0
    torch.cuda.synchronize()
    assert tokens.tolist() == logits.argmax(-1).tolist() and tokens[1] == 123 and tokens[2] == 65535
    assert pos.tolist() == [4, 5, 6, 7, 8]
    assert [int(trace[r, pos[r]]) for r in range(rows)] == tokens.tolist() and int((trace >= 0).sum()) == rows
    # idle rows (negative position) keep their token and position and log nothing
    pos = torch.tensor([3, -1, 5, -1, 7], dtype=torch.int32, device="cuda")
    tokens.fill_(7)
    trace.fill_(-1)
    assert lib.greedy_choice(pointer(logits), pointer(tokens), pointer(pos), rows, 65536, pointer(trace), 16,
                             stream()) == 0
    torch.cuda.synchronize()
    best = logits.argmax(-1).tolist()
    assert tokens.tolist() == [best[0], 7, best[2], 7, best[4]] and pos.tolist() == [4, -1, 6, -1, 8]
    assert int((trace >= 0).sum()) == 3


@pytest.mark.parametrize("rows,C", [(1, 256), (33, 1280), (1024, 2048), (5, 4096), (7, 8)])
def test_add_rms_norm_and_relu2_match_torch(rows, C):
    gen = torch.Generator().manual_seed(rows + C)
    h = torch.randn(rows, C, generator=gen).bfloat16().cuda()
    y = torch.randn(rows, C, generator=gen).bfloat16().cuda()
    lib = cuda_library("decode_step")
    for add in (True, False):
        h1, n = h.clone(), torch.empty_like(h)
        assert lib.add_rms_norm(pointer(h1), pointer(y if add else None), pointer(n), rows, C, stream()) == 0
        want_h = (h.float() + y.float()).bfloat16() if add else h
        want_n = F.rms_norm(want_h, (C,), eps=EPS)
        torch.cuda.synchronize()
        assert torch.equal(h1, want_h)
        assert (n.float() - want_n.float()).abs().max() <= 2 ** -7 * want_n.float().abs().max()
        assert (n != want_n).float().mean() < 0.01
    u = torch.randn(rows, C, generator=gen).bfloat16().cuda()
    want = F.relu(u).float().square().bfloat16()
    assert lib.relu2_inplace(pointer(u), u.numel(), stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(u, want)
