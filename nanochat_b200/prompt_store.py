"""A prompt store for the paged fp8 cache: the K/V pages of prompts already prefilled, kept in pinned host memory
and copied back into a slot instead of prefilling the same prompt again.

The reference keeps prompts in registered host memory as bf16 rows [L][n][C], copied with one 2-D memcpy per cache
(model/kernels/decode.cu:933-946,1055-1075), keyed by the prompt's token tuple, stored once and never evicted
(inference/decoder.py:172-175,193-232). With the paged layout the unit of copy is a page of 64 positions: a prompt
of n positions (all but its last token) occupies ceil(n / 64) pages per layer and kv head; positions past n inside
the last page are whatever the source slot held there, which the attention kernels never read (they mask by
length) and the next append overwrites."""

import torch

from .kv_cache import PAGE_BYTES, PAGE_TOKENS, Fp8KVCache


class PromptStore:
    def __init__(self, caches: list[Fp8KVCache], store_positions: int):
        """Room for `store_positions` positions (rounded up to pages) of every layer's cache in `caches`."""
        self.caches = caches
        self.pages = (store_positions + PAGE_TOKENS - 1) // PAGE_TOKENS
        heads = caches[0].kv_heads
        self.buffer = torch.empty((len(caches), heads, self.pages, PAGE_BYTES), dtype=torch.uint8)
        if torch.cuda.is_available() and caches[0].device.type == "cuda":
            self.buffer = self.buffer.pin_memory()
        self.stored: dict[tuple[int, ...], tuple[int, int]] = {}  # prompt -> (first store page, positions)
        self.used = 0

    @staticmethod
    def pages_for(positions: int) -> int:
        return (positions + PAGE_TOKENS - 1) // PAGE_TOKENS

    def save(self, slot: int, input_ids: list[int]) -> bool:
        """Keep slot's pages for the prompt's positions 0 .. len - 2, unless already stored or out of room (a
        prompt is stored once and never evicted). Stream-ordered on the current stream."""
        key, n = tuple(input_ids), len(input_ids) - 1
        need = self.pages_for(n)
        if key in self.stored or n <= 0 or self.used + need > self.pages:
            return False
        for layer, cache in enumerate(self.caches):
            self.buffer[layer, :, self.used:self.used + need].copy_(cache.pages[slot, :, :need], non_blocking=True)
        self.stored[key] = (self.used, n)
        self.used += need
        return True

    def load(self, slot: int, input_ids: list[int]) -> bool:
        """Copy a stored prompt's pages into `slot`; False if the prompt is not in the store."""
        hit = self.stored.get(tuple(input_ids))
        if hit is None:
            return False
        at, n = hit
        need = self.pages_for(n)
        for layer, cache in enumerate(self.caches):
            cache.pages[slot, :, :need].copy_(self.buffer[layer, :, at:at + need], non_blocking=True)
        return True
