"""decode_attn_fp8_static, the entry point for callers that cannot allocate device memory (a plug-in inside
another engine's memory plan, a host that forbids cudaMalloc after start-up): its per-chunk states live in an
8 MiB array built into the library instead of a caller workspace.

Called through the C ABI, twice in a row on different inputs (the array keeps the previous call's contents, so
the second call proves nothing stale leaks through), and compared with decode_attn_fp8 on the same inputs. Also
checks that a call that would not fit the array is refused. The file sorts last so that a run stopping at the
first failure has already run every other test."""

import ctypes

import numpy as np
import pytest
import torch

import nanochat_b200 as ncb
from nanochat_b200.attention import decode_attention_static
from nanochat_b200.native import cuda_library, pointer, stream
from tests import helpers
from tests.test_decode_attn_gpu import MAX_ABS, MEAN_ABS, SCALE, load_cache

pytestmark = pytest.mark.gpu


def both_ways(case, chunk_pages):
    cache = load_cache(case, max(case["lens"]))
    q = helpers.bits_bf16(case["q"]).cuda()
    lens = torch.tensor(case["lens"], dtype=torch.int32, device="cuda")
    B, Hq, Hkv, top = len(case["lens"]), case["Hq"], case["Hkv"], max(case["lens"])
    lib = cuda_library("decode_attn")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # the existing entry point, with a caller-allocated workspace
    need = lib.decode_attn_workspace_bytes(B, Hq, top, Hkv, chunk_pages)
    workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
    want = torch.empty_like(q)
    rc = lib.decode_attn_fp8(pointer(q), pointer(cache.pages), pointer(lens), None, pointer(workspace), need,
                             pointer(want), B, Hq, Hkv, cache.n_slots, cache.pages_per_slot, top, 0, chunk_pages,
                             SCALE, pointer(status), stream())
    assert rc == 0
    # the new one: inputs and outputs only
    got = torch.full_like(q, float("nan"))
    rc = lib.decode_attn_fp8_static(pointer(q), pointer(cache.pages), pointer(lens), None, pointer(got), B, Hq, Hkv,
                                    cache.n_slots, cache.pages_per_slot, top, 0, chunk_pages, SCALE, pointer(status),
                                    stream())
    assert rc == 0
    torch.cuda.synchronize()
    assert status.item() == 0
    return helpers.bf16_bits(got.cpu()), helpers.bf16_bits(want.cpu())


def test_static_scratch_matches_workspace_entry_on_two_calls_in_a_row():
    first = helpers.attention_case(1100, 8, 2, [700, 64, 333])
    second = helpers.attention_case(1101, 16, 4, [90, 1500])  # other shapes: states land elsewhere in the array
    for case, chunk_pages in ((first, 2), (second, 3)):
        got, want = both_ways(case, chunk_pages)
        max_abs, mean_abs = helpers.error_stats(got, want)
        assert max_abs <= MAX_ABS and mean_abs <= MEAN_ABS, (max_abs, mean_abs)
        assert np.array_equal(got, want), "same kernels, same inputs: the outputs should be identical"


def test_static_entry_point_leaves_device_memory_as_it_is():
    """What the entry point is for: after a first call (which looks up the built-in array's address), further calls
    change neither the driver's free-memory figure nor torch's allocator statistics."""
    case = helpers.attention_case(1103, 8, 2, [500, 129])
    cache = load_cache(case, 512)
    q = helpers.bits_bf16(case["q"]).cuda()
    lens = torch.tensor(case["lens"], dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    lib = cuda_library("decode_attn")
    call = lambda: lib.decode_attn_fp8_static(pointer(q), pointer(cache.pages), pointer(lens), None, pointer(out), 2, 8, 2,
                                              cache.n_slots, cache.pages_per_slot, 512, 0, 2, SCALE, None, stream())
    assert call() == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before, allocs_before = torch.cuda.memory_reserved(), torch.cuda.memory_stats()["allocation.all.allocated"]
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_reserved() == reserved_before
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocs_before


def test_static_scratch_refuses_what_does_not_fit():
    lib = cuda_library("decode_attn")
    p = ctypes.c_void_p(4096)
    # 64 x 32 rows x 8 one-page chunks x 528 bytes is just above 8 MiB
    assert lib.decode_attn_workspace_bytes(64, 32, 512, 8, 1) > 8 << 20
    assert lib.decode_attn_fp8_static(p, p, p, None, p, 64, 32, 8, 64, 8, 512, 0, 1, SCALE, None, None) == 6
    case = helpers.attention_case(1102, 32, 8, [64] * 64)
    cache = load_cache(case, 512)
    q = helpers.bits_bf16(case["q"]).cuda()
    lens = torch.tensor(case["lens"], dtype=torch.int32, device="cuda")
    with pytest.raises(ncb.NativeError):
        decode_attention_static(q, cache, lens, 512, chunk_pages=1)
    # two-page chunks halve the need and fit
    out = decode_attention_static(q, cache, lens, 512, chunk_pages=2)
    want = ncb.decode_attention(q, cache, lens, 512, chunk_pages=2)
    torch.cuda.synchronize()
    assert torch.equal(out, want)
