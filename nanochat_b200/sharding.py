"""Partitioning the decode path over the GPUs of one box: one process per GPU, torch.distributed for the plumbing.

Two axes, both absent from the single-GPU reference (its decoder states that a request's tokens depend on neither
the batch nor the placement, inference/decoder.py:124-125, which is what makes the first axis free):

  batch      sequences are independent units: shard_batch() assigns whole sequences to ranks, balancing the summed
             lengths; no collective on the attention path.
  KV length  for long contexts each rank holds a page-aligned contiguous slice of every sequence's positions
             (kv_slices), runs the split-KV kernel on its slice and emits one un-normalised (m, l, o) state per
             (sequence, head); the states are all-gathered (NCCL over NVLink; 528 bytes per row and rank) and merged
             by the same kernel that merges chunks inside a GPU (the rule of model/kernels/decode.cu:548,661-670
             is associative). A new token is appended by the rank that owns the tail slice (append_owner).
             attend_kv_sharded_fused replaces the NCCL all-gather + merge by one kernel that loads the peers'
             states over NVLink itself (PeerStates)."""

import ctypes
from collections.abc import Sequence

import torch
import torch.distributed as dist
from torch import Tensor

from .attention import PART_FLOATS
from .kv_cache import PAGE_TOKENS
from .native import check, cuda_library, pointer, stream


def shard_batch(lens: Sequence[int], world: int, longest_first: bool = False) -> list[list[int]]:
    """Indices of `lens` per rank: longest-processing-time greedy on the lengths, ties to the lower rank. Every
    index appears exactly once. Each rank's list is in ascending index order, or with longest_first in descending
    length order: thread blocks are dispatched in batch order, so a ragged batch that starts with its longest
    sequences ends with short ones and leaves a shorter idle tail on the GPU."""
    assert world >= 1
    load = [0] * world
    shards: list[list[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(lens)), key=lambda i: (-lens[i], i)):
        r = min(range(world), key=lambda r: (load[r], len(shards[r]), r))
        shards[r].append(i)
        load[r] += lens[i]
    if longest_first:
        return [sorted(s, key=lambda i: (-lens[i], i)) for s in shards]
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
    """The rank that appends the token at global `position`: the rank whose slice contains it, else the last rank
    with a non-empty slice (the tail grows there), else rank 0. The owner writes at its LOCAL position
    (position - slice begin) but the rotary angle is the global position's: pass kv_append the rotary tables shifted
    by the slice's begin (cos[begin:], sin[begin:]) so that table row `local position` is the global one."""
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


class PeerStates:
    """Per-rank (m, l, o) states in memory every GPU of the group can address, for the fused exchange + merge
    kernel (decode_attn_merge_peers): no collective library on the data path, each rank's merge kernel loads the
    peers' states over NVLink itself after a bounded wait on per-rank epoch flags.

    One symmetric allocation per rank: `world` uint32 flags (padded to 256 bytes), then two buffers of
    (rows, 132) fp32 that calls alternate between, so a rank that runs one call ahead never overwrites states a
    slower peer is still reading. Construction is collective (allocation, rendezvous, barrier)."""

    FLAG_BYTES = 256

    def __init__(self, batch: int, heads: int, group: "dist.ProcessGroup | None" = None,
                 device: "torch.device | None" = None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group or dist.group.WORLD
        device = device or torch.device("cuda", torch.cuda.current_device())
        self.batch, self.heads, self.rows = batch, heads, batch * heads
        self.half_floats = self.rows * PART_FLOATS
        floats = self.FLAG_BYTES // 4 + 2 * self.half_floats
        self.buffer = symm_mem.empty(floats, dtype=torch.float32, device=device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, group)
        self.world, self.rank = self.handle.world_size, self.handle.rank
        assert self.world <= 8
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's flags are zero before anyone publishes
        self.epoch = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._flags = (ctypes.c_void_p * self.world)(*self.handle.buffer_ptrs)

    def next_part(self) -> Tensor:
        """Advance to the next call and return this rank's (batch, heads, 132) state buffer for it."""
        self.epoch += 1
        at = self.FLAG_BYTES // 4 + (self.epoch % 2) * self.half_floats
        return self.buffer[at:at + self.half_floats].view(self.batch, self.heads, PART_FLOATS)

    def merge(self, out: Tensor | None = None) -> Tensor:
        """Publish this rank's states of the current call, wait for every rank's, merge: (batch, heads, 128) bf16."""
        if out is None:
            out = torch.empty((self.batch, self.heads, 128), dtype=torch.bfloat16, device=self.buffer.device)
        offset = self.FLAG_BYTES + (self.epoch % 2) * self.half_floats * 4
        parts = (ctypes.c_void_p * self.world)(*(p + offset for p in self.handle.buffer_ptrs))
        rc = cuda_library("decode_attn").decode_attn_merge_peers(
            parts, self._flags, self.world, self.rank, self.epoch, self.rows, pointer(out), pointer(self.status),
            stream())
        check(rc, "decode_attn_merge_peers")
        return out


def attend_kv_sharded_fused(q: Tensor, cache, local_lens: Tensor, max_local_len: int, peers: PeerStates,
                            out: Tensor | None = None, **kwargs) -> Tensor:
    """attend_kv_sharded with the all-gather and the merge replaced by one kernel over peer memory."""
    from .attention import decode_attention_partial

    decode_attention_partial(q, cache, local_lens, max_local_len, part=peers.next_part(), **kwargs)
    return peers.merge(out)


def attend_kv_sharded(q: Tensor, cache, local_lens: Tensor, max_local_len: int,
                      group: "dist.ProcessGroup | None" = None, **kwargs) -> Tensor:
    """Attention where this rank's `cache` holds only its slice of every sequence: local states, one all-gather,
    local merge. Every rank returns the full (B, Hq, 128) bf16 output. q is replicated."""
    from .attention import decode_attention_partial, merge_partials

    part = decode_attention_partial(q, cache, local_lens, max_local_len, **kwargs)
    return merge_partials(gather_states(part, group))
