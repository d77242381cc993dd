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
             attend_kv_sharded_fused replaces the local merge, the NCCL all-gather and the cross-rank merge by one
             kernel that pushes the row states to the peers over NVLink itself (PeerStates)."""

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


PEER_STATE_BYTES = 1056  # NCB_PEER_STATE_BYTES: one (m, l, o) state as 8-byte (value, call number) words


class PeerStates:
    """What the fused exchange + merge (decode_attn_fp8_sharded) needs on every rank: an inbox in memory every GPU of
    the group can address, and this rank's private call counter.

    One symmetric allocation per rank: 2 * world * rows states of PEER_STATE_BYTES (two halves that calls alternate
    between). Each rank's merge kernel pushes its row states into every other rank's inbox with plain stores over
    NVLink, as 8-byte words that carry the call number and so validate themselves, then polls (bounded) its own inbox
    for the peers' states and merges: no collective library, no flags and no fences on the data path. Construction is
    collective (allocation, rendezvous, barrier); torch's symmetric memory is used for the allocation and the pointer
    exchange only."""

    def __init__(self, batch: int, heads: int, group: "dist.ProcessGroup | None" = None,
                 device: "torch.device | None" = None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group or dist.group.WORLD
        device = device or torch.device("cuda", torch.cuda.current_device())
        world = dist.get_world_size(group)
        assert world <= 8
        self.batch, self.heads, self.rows = batch, heads, batch * heads
        self.buffer = symm_mem.empty(2 * world * self.rows * PEER_STATE_BYTES // 4, dtype=torch.int32, device=device)
        self.buffer.zero_()  # call numbers start at 1: a zeroed word never passes for an arrived one
        self.handle = symm_mem.rendezvous(self.buffer, group)
        self.world, self.rank = self.handle.world_size, self.handle.rank
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)  # (calls completed, rows arrived)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's inbox is zero before anyone sends
        self._inbox = (ctypes.c_void_p * self.world)(*self.handle.buffer_ptrs)


def attend_kv_sharded_fused(q: Tensor, cache, local_lens: Tensor, max_local_len: int, peers: PeerStates,
                            out: Tensor | None = None, slot_map: Tensor | None = None, window: int = 0,
                            chunk_pages: int = 0, softmax_scale: float | None = None,
                            workspace: Tensor | None = None) -> Tensor:
    """attend_kv_sharded in two launches and without a collective: the split-KV kernel over this rank's slice, then
    one kernel that merges the local chunks, exchanges the row states over peer memory and merges across ranks.
    Every rank returns the full (B, Hq, 128) bf16 output, bit-identical across ranks. The call sequence must be the
    same on every rank; it is safe to capture in a CUDA graph (the call counter lives on the device)."""
    from .attention import workspace_bytes

    B, Hq = q.shape[0], q.shape[1]
    assert (B, Hq) == (peers.batch, peers.heads) and q.dtype == torch.bfloat16 and q.is_contiguous()
    assert local_lens.dtype == torch.int32 and local_lens.shape == (B,) and local_lens.is_contiguous()
    if workspace is None:
        need = workspace_bytes(B, Hq, cache.kv_heads, min(max_local_len, cache.capacity), chunk_pages)
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    if out is None:
        out = torch.empty_like(q)
    rc = cuda_library("decode_attn").decode_attn_fp8_sharded(
        pointer(q), pointer(cache.pages), pointer(local_lens), pointer(slot_map), pointer(workspace),
        workspace.numel(), pointer(out), B, Hq, cache.kv_heads, cache.n_slots, cache.pages_per_slot, max_local_len,
        window, chunk_pages, 128 ** -0.5 if softmax_scale is None else softmax_scale, peers._inbox, peers.world,
        peers.rank, pointer(peers.epoch), pointer(peers.status), stream())
    check(rc, "decode_attn_fp8_sharded")
    return out


def attend_kv_sharded(q: Tensor, cache, local_lens: Tensor, max_local_len: int,
                      group: "dist.ProcessGroup | None" = None, **kwargs) -> Tensor:
    """Attention where this rank's `cache` holds only its slice of every sequence: local states, one all-gather,
    local merge. Every rank returns the full (B, Hq, 128) bf16 output. q is replicated."""
    from .attention import decode_attention_partial, merge_partials

    part = decode_attention_partial(q, cache, local_lens, max_local_len, **kwargs)
    return merge_partials(gather_states(part, group))
