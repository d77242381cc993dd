"""The paged fp8 (e4m3) KV cache of one layer and the index arithmetic of its page layout.

Replaces the reference's bf16 cache `kc, vc [B][L][max_len][C]` (model/kernels/decode.cu:726, addressed at
decode.cu:562,578-579). A page is NCB_PAGE_BYTES = 16,896 bytes holding 64 positions of one (slot, kv head): K rows
with swizzled 16-byte chunks, V transposed in 16-position blocks, then the K and V fp32 scales; the exact offsets
are in include/nanochat_b200.h and restated here so that host code can fill and read caches (tests, prompt
loading). The kernels never call this module."""

import functools

import torch

from .native import cuda_library

HEAD_DIM = 128
PAGE_TOKENS = 64
PAGE_BYTES = 16896
PAGE_V = 8192
PAGE_KS = 16384
PAGE_VS = 16640


@functools.cache
def page_offsets(device: str = "cpu") -> tuple[torch.Tensor, torch.Tensor]:
    """(k_off, v_off) int64 [64, 128]: the byte offset inside a page of K's / V's byte for in-page position j
    and dim d."""
    j = torch.arange(PAGE_TOKENS)[:, None]
    d = torch.arange(HEAD_DIM)[None, :]
    k_off = j * HEAD_DIM + (((d >> 4) ^ ((j >> 2) & 7)) << 4) + (d & 15)
    v_off = PAGE_V + (j >> 5) * 4096 + ((j >> 4) & 1) * 2048 + d * 16 + (j & 15)
    return k_off.to(device), v_off.to(device)


def cache_pages(max_len: int) -> int:
    return (max_len + PAGE_TOKENS - 1) // PAGE_TOKENS


class Fp8KVCache:
    """One layer's cache: `pages` uint8 [n_slots, kv_heads, pages_per_slot, PAGE_BYTES] on `device`."""

    def __init__(self, n_slots: int, kv_heads: int, max_len: int, device: "torch.device | str" = "cuda",
                 pages: torch.Tensor | None = None):
        self.n_slots, self.kv_heads = n_slots, kv_heads
        self.pages_per_slot = cache_pages(max_len)
        self.capacity = self.pages_per_slot * PAGE_TOKENS
        shape = (n_slots, kv_heads, self.pages_per_slot, PAGE_BYTES)
        if pages is None:
            # zeros, not empty: positions past a sequence's length are masked by the kernels either way, but a
            # zeroed cache keeps read() of unwritten positions deterministic
            pages = torch.zeros(shape, dtype=torch.uint8, device=device)
        assert pages.shape == shape and pages.dtype == torch.uint8 and pages.is_contiguous()
        self.pages = pages

    @property
    def device(self) -> torch.device:
        return self.pages.device

    def nbytes(self) -> int:
        return self.pages.numel()

    def _flat(self, slot: int) -> tuple[torch.Tensor, torch.Tensor]:
        """(bytes [kv_heads, pages * PAGE_BYTES], floats [kv_heads, pages * PAGE_BYTES / 4]) views of a slot."""
        b = self.pages[slot].view(self.kv_heads, -1)
        return b, b.view(torch.float32)

    def write(self, slot: int, k_bytes: torch.Tensor, k_scale: torch.Tensor, v_bytes: torch.Tensor,
              v_scale: torch.Tensor, start: int = 0) -> None:
        """Store logical rows at positions start .. start + n: k_bytes, v_bytes uint8 [kv_heads, n, 128],
        k_scale, v_scale fp32 [kv_heads, n]."""
        n = k_bytes.shape[1]
        assert start >= 0 and start + n <= self.capacity
        dev = self.device
        k_off, v_off = page_offsets(str(dev))
        pos = torch.arange(start, start + n, device=dev)
        page, j = pos // PAGE_TOKENS, pos % PAGE_TOKENS
        flat, floats = self._flat(slot)
        base = (page * PAGE_BYTES)[:, None]
        flat[:, (base + k_off[j]).reshape(-1)] = k_bytes.to(dev).reshape(self.kv_heads, -1)
        flat[:, (base + v_off[j]).reshape(-1)] = v_bytes.to(dev).reshape(self.kv_heads, -1)
        fbase = page * (PAGE_BYTES // 4) + j
        floats[:, fbase + PAGE_KS // 4] = k_scale.to(dev)
        floats[:, fbase + PAGE_VS // 4] = v_scale.to(dev)

    def read(self, slot: int, n: int, start: int = 0) -> tuple[torch.Tensor, ...]:
        """Logical (k_bytes, k_scale, v_bytes, v_scale) of positions start .. start + n of a slot."""
        dev = self.device
        k_off, v_off = page_offsets(str(dev))
        pos = torch.arange(start, start + n, device=dev)
        page, j = pos // PAGE_TOKENS, pos % PAGE_TOKENS
        flat, floats = self._flat(slot)
        base = (page * PAGE_BYTES)[:, None]
        k = flat[:, (base + k_off[j]).reshape(-1)].view(self.kv_heads, n, HEAD_DIM)
        v = flat[:, (base + v_off[j]).reshape(-1)].view(self.kv_heads, n, HEAD_DIM)
        fbase = page * (PAGE_BYTES // 4) + j
        return k, floats[:, fbase + PAGE_KS // 4], v, floats[:, fbase + PAGE_VS // 4]


def native_cache_bytes(n_slots: int, kv_heads: int, max_len: int) -> int:
    """The library's own answer for the cache size (kv_cache_bytes of include/nanochat_b200.h)."""
    return cuda_library("kv_append").kv_cache_bytes(n_slots, kv_heads, max_len)
