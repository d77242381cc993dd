"""Partitioning the decode path over the GPUs of one box: one process per GPU, torch.distributed for the plumbing.

Two axes, both absent from the single-GPU reference (its decoder states that a request's tokens depend on neither
the batch nor the placement, inference/decoder.py:124-125, which is what makes the first axis free):

  batch      sequences are independent units: shard_batch() assigns whole sequences to ranks, balancing the summed
             lengths; no collective on the attention path.
  KV length  for long contexts each rank holds a page-aligned contiguous slice of every sequence's positions
             (kv_slices), runs the split-KV kernel on its slice and emits one un-normalised (m, l, o) state per
             (sequence, head); the states are all-gathered (NCCL over NVLink; 528 bytes per row and rank) and merged
             by the same kernel that merges chunks inside a GPU (the rule of model/kernels/decode.cu:548,661-670
             is associative). A new token is appended by the rank that owns the tail slice (append_owner)."""

from collections.abc import Sequence

import torch
import torch.distributed as dist
from torch import Tensor

from .kv_cache import PAGE_TOKENS


def shard_batch(lens: Sequence[int], world: int) -> list[list[int]]:
    """Indices of `lens` per rank: longest-processing-time greedy on the lengths, ties to the lower rank, each
    rank's list in ascending index order. Every index appears exactly once."""
    assert world >= 1
    load = [0] * world
    shards: list[list[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(lens)), key=lambda i: (-lens[i], i)):
        r = min(range(world), key=lambda r: (load[r], len(shards[r]), r))
        shards[r].append(i)
        load[r] += lens[i]
    return [sorted(s) for s in shards]


def kv_slices(n: int, world: int) -> list[tuple[int, int]]:
    """[begin, end) positions per rank for a sequence of n positions: contiguous, page-aligned boundaries, pages
    spread as evenly as possible, earlier ranks take the remainder. Ranks past the end get empty slices."""
    pages = (n + PAGE_TOKENS - 1) // PAGE_TOKENS
    base, extra = divmod(pages, world)
    out, at = [], 0
    for r in range(world):
        take = base + (1 if r < extra else 0)
        begin, end = min(at * PAGE_TOKENS, n), min((at + take) * PAGE_TOKENS, n)
        out.append((begin, end))
        at += take
    return out


def append_owner(position: int, slices: Sequence[tuple[int, int]]) -> int:
    """The rank whose slice ends at `position` (the next position to write): the last rank with a non-empty slice,
    or the first rank whose slice can still grow within its last page."""
    for r, (begin, end) in enumerate(slices):
        if begin <= position < end:
            return r
    owners = [r for r, (begin, end) in enumerate(slices) if end > begin]
    return owners[-1] if owners else 0


def gather_states(part: Tensor, group: "dist.ProcessGroup | None" = None) -> Tensor:
    """part fp32 (B, Hq, 132) of this rank -> (world, B, Hq, 132) of every rank, in rank order. One collective."""
    world = dist.get_world_size(group)
    out = torch.empty((world * part.shape[0], *part.shape[1:]), dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(out, part.contiguous(), group=group)  # concatenated along dim 0 in rank order
    return out.view(world, *part.shape)


def attend_kv_sharded(q: Tensor, cache, local_lens: Tensor, max_local_len: int,
                      group: "dist.ProcessGroup | None" = None, **kwargs) -> Tensor:
    """Attention where this rank's `cache` holds only its slice of every sequence: local states, one all-gather,
    local merge. Every rank returns the full (B, Hq, 128) bf16 output. q is replicated."""
    from .attention import decode_attention_partial, merge_partials

    part = decode_attention_partial(q, cache, local_lens, max_local_len, **kwargs)
    return merge_partials(gather_states(part, group))
