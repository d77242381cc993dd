"""Host logic that needs no GPU: the page layout's index arithmetic, the libraries' exported symbols against
include/nanochat_b200.h, and argument validation (entry points return a status before touching CUDA)."""

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

from nanochat_b200 import kv_cache, native
from nanochat_b200.kv_cache import HEAD_DIM, PAGE_BYTES, PAGE_TOKENS, Fp8KVCache

ROOT = Path(__file__).resolve().parent.parent


def test_page_offsets_are_a_bijection_onto_the_k_and_v_regions():
    k_off, v_off = kv_cache.page_offsets()
    assert sorted(k_off.reshape(-1).tolist()) == list(range(0, 8192))
    assert sorted(v_off.reshape(-1).tolist()) == list(range(8192, 16384))


def test_page_offsets_known_values():
    k_off, v_off = kv_cache.page_offsets()
    assert k_off[0, 0] == 0 and k_off[0, 17] == 17
    assert k_off[4, 0] == 4 * 128 + 16          # position 4 swizzles chunk 0 to chunk 1
    assert k_off[63, 127] == 63 * 128 + ((7 ^ 7) << 4) + 15
    assert v_off[0, 0] == 8192 and v_off[1, 0] == 8193 and v_off[0, 1] == 8192 + 16
    assert v_off[16, 0] == 8192 + 2048 and v_off[32, 0] == 8192 + 4096 and v_off[63, 127] == 8192 + 4096 + 2048 + 127 * 16 + 15


def test_k_rows_of_an_ldmatrix_tile_hit_distinct_banks():
    """The 8 rows one ldmatrix 8x16B matrix reads (positions 4r + c, r = 0..7) must land in 8 different 16-byte
    bank groups for every chunk."""
    k_off, _ = kv_cache.page_offsets()
    for c in range(4):
        for chunk in range(8):
            groups = {(int(k_off[4 * r + c, 16 * chunk]) // 16) % 8 for r in range(8)}
            assert len(groups) == 8


def test_cache_write_read_round_trip_cpu():
    gen = torch.Generator().manual_seed(0)
    cache = Fp8KVCache(3, 2, 200, device="cpu")
    assert cache.pages_per_slot == 4 and cache.capacity == 256
    assert cache.nbytes() == native.cuda_library("kv_append").kv_cache_bytes(3, 2, 200)
    k = torch.randint(0, 256, (2, 150, HEAD_DIM), dtype=torch.uint8, generator=gen)
    v = torch.randint(0, 256, (2, 150, HEAD_DIM), dtype=torch.uint8, generator=gen)
    ks, vs = torch.rand(2, 150, generator=gen), torch.rand(2, 150, generator=gen)
    cache.write(1, k, ks, v, vs, start=37)
    k2, ks2, v2, vs2 = cache.read(1, 150, start=37)
    assert torch.equal(k, k2) and torch.equal(v, v2) and torch.equal(ks, ks2) and torch.equal(vs, vs2)
    assert not cache.pages[0].any() and not cache.pages[2].any()
    # one K row is 128 contiguous bytes of its page, chunks permuted
    page = cache.pages[1, 0, 0]
    row = page[37 * 128:38 * 128].view(8, 16)
    swz = (37 >> 2) & 7
    for c in range(8):
        assert torch.equal(row[c ^ swz], k[0, 0, 16 * c:16 * c + 16])


def declared_functions() -> list[str]:
    """The name of every prototype in include/nanochat_b200.h."""
    text = (ROOT / "include" / "nanochat_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"^\s*(?:const\s+)?(?:int|long long|char\s*\*|void)\s*\**\s*(\w+)\s*\(", text, flags=re.M)
    assert len(names) >= 9
    return names


def test_libraries_export_every_declared_symbol():
    exported = set()
    for name in native.LIBRARIES:
        lib = native.cuda_library(name)
        for symbol in native.SIGNATURES[name]:
            assert getattr(lib, symbol) is not None
            exported.add(symbol)
    assert set(declared_functions()) == exported


def test_header_constants_match_python():
    text = (ROOT / "include" / "nanochat_b200.h").read_text()
    consts = dict(re.findall(r"#define (NCB_\w+) (\d+)", text))
    assert int(consts["NCB_PAGE_BYTES"]) == PAGE_BYTES and int(consts["NCB_PAGE_TOKENS"]) == PAGE_TOKENS
    assert int(consts["NCB_HEAD_DIM"]) == HEAD_DIM
    from nanochat_b200.attention import PART_FLOATS
    assert int(consts["NCB_PART_FLOATS"]) == PART_FLOATS


def test_argument_validation_returns_status_codes():
    app, att = native.cuda_library("kv_append"), native.cuda_library("decode_attn")
    p = ctypes.c_void_p(4096)  # a non-NULL, aligned stand-in; validation fails before any use
    nul = ctypes.c_void_p(None)
    # Hq not a multiple of Hkv
    assert app.kv_append_fp8(p, p, p, p, p, p, nul, p, p, 4, 10, 3, 16 * 128, 64, 1, 1, nul, nul) == 1
    # row stride shorter than a row
    assert app.kv_append_fp8(p, p, p, p, p, p, nul, p, p, 4, 4, 4, 100, 64, 1, 1, nul, nul) == 1
    # misaligned pointer
    assert app.kv_append_fp8(ctypes.c_void_p(4100), p, p, p, p, p, nul, p, p, 4, 4, 4, 12 * 128, 64, 1, 1, nul, nul) == 2
    # zero rows is a no-op
    assert app.kv_append_fp8(nul, nul, nul, nul, nul, nul, nul, nul, nul, 0, 4, 4, 12 * 128, 64, 1, 1, nul, nul) == 0
    # head ratio above 8
    assert att.decode_attn_fp8(p, p, p, nul, p, 1 << 30, p, 1, 16, 1, 1, 1, 64, 0, 0, 0.1, nul, nul) == 5
    # workspace too small
    need = att.decode_attn_workspace_bytes(2, 8, 640, 2, 1)
    assert need == 2 * 8 * 10 * 132 * 4
    assert att.decode_attn_fp8(p, p, p, nul, p, need - 1, p, 2, 8, 2, 2, 10, 640, 0, 1, 0.1, nul, nul) == 3
    assert att.decode_attn_merge(p, 0, 4, p, nul) == 1
    assert att.decode_attn_fp8(p, p, p, nul, p, 0, p, 0, 8, 2, 2, 10, 640, 0, 1, 0.1, nul, nul) == 0  # B == 0
    assert native.cuda_library("kv_append").ncb_status_string(3) == b"workspace too small"
    with pytest.raises(native.NativeError):
        native.check(3, "x")


def test_chunk_choice_is_positive_and_bounded():
    att = native.cuda_library("decode_attn")
    for B, Hkv, n in ((1, 10, 1024), (64, 8, 8192), (4, 8, 131072), (256, 4, 8192), (1, 1, 1)):
        c = att.decode_attn_chunk_pages(B, Hkv, n)
        assert 1 <= c <= 64


def test_stream_gemm_validates_and_chooses_its_split_on_the_host():
    lib = native.cuda_library("stream_gemm")
    p, nul = ctypes.c_void_p(4096), ctypes.c_void_p(None)
    assert lib.stream_gemm(p, p, nul, p, 257, 128, 256, 0, 0, 0, nul, 0, nul, nul) == 1   # more than 256 rows
    assert lib.stream_gemm(p, p, nul, p, 4, 100, 256, 0, 0, 0, nul, 0, nul, nul) == 1     # N not a multiple of 128
    assert lib.stream_gemm(p, p, nul, p, 4, 128, 100, 0, 0, 0, nul, 0, nul, nul) == 1     # K not a multiple of 64
    assert lib.stream_gemm(p, p, nul, p, 4, 128, 256, 0, 1, 0, nul, 0, nul, nul) == 1     # residual epilogue, no residual
    assert lib.stream_gemm(ctypes.c_void_p(4100), p, nul, p, 4, 128, 256, 0, 0, 0, nul, 0, nul, nul) == 2  # misaligned
    assert lib.stream_gemm(p, p, nul, p, 0, 128, 256, 0, 0, 0, nul, 0, nul, nul) == 0     # nothing to do
    # one wave of at most 296 blocks, powers of two, at least two k-blocks per block
    assert [lib.stream_gemm_split(32, n, k) for n, k in ((2048, 2048), (8192, 2048), (65536, 2048), (3072, 2048),
                                                        (5120, 1280), (1280, 5120), (128, 128), (100, 2048))] \
        == [8, 4, 1, 8, 4, 8, 1, 0]
    # blocks for more than 128 rows take an SM each: half as many fit
    assert [lib.stream_gemm_split(256, n, k) for n, k in ((2048, 2048), (8192, 2048), (3072, 2048))] == [8, 2, 4]


def test_planned_chunk_follows_the_block_fill_model():
    """decode_attn_plan_chunk_pages is host-only: bounded, equal to the default for uniform full-length batches, and
    it avoids the sizes that leave a nearly empty last wave of blocks."""
    att = native.cuda_library("decode_attn")
    uniform = (ctypes.c_int * 16)(*([8192] * 16))
    assert att.decode_attn_plan_chunk_pages(uniform, 16, 8, 8192, 0) == att.decode_attn_chunk_pages(16, 8, 8192)
    assert att.decode_attn_plan_chunk_pages(None, 16, 8, 8192, 0) == att.decode_attn_chunk_pages(16, 8, 8192)
    assert att.decode_attn_chunk_pages(64, 8, 8192) == 32      # 2,048 blocks of 32 pages: the measured optimum
    assert att.decode_attn_chunk_pages(8, 10, 776) == 4        # small batches: one page per warp
    short = (ctypes.c_int * 4)(100, 0, 8192, -5)               # out-of-range lengths are clipped, not trusted
    assert 4 <= att.decode_attn_plan_chunk_pages(short, 4, 2, 4096, 0) <= 32
    windowed = (ctypes.c_int * 2)(8192, 8192)
    # a 256-position window is 4 pages, one chunk whatever the bound: the largest bound launches the fewest idle blocks
    assert att.decode_attn_plan_chunk_pages(windowed, 2, 1, 8192, 256) == 32
