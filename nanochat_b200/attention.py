"""Host-side operators of the decode hot path, thin ctypes calls into the sm_100a kernels.

They keep the call style of the reference's op wrappers (model/ops/qk_prologue.py:13-21: tensors in, tensors out,
pointers + sizes + stream() passed to an extern "C" entry) and stand where inference/decoder.py's step graph
calls k_prologue and k_attn (model/kernels/decode.cu:859-863). Every function launches on the current stream and
returns without synchronising; a non-zero native status raises NativeError. There is no CPU or PyTorch fallback."""

import torch
from torch import Tensor

from .kv_cache import HEAD_DIM, Fp8KVCache
from .native import check, cuda_library, pointer, stream

PART_FLOATS = 132


class ValueEmbed:
    """The optional value-embedding mix of one layer for a pass of rows (reference model/kernels/decode.cu:482-494):
    h (rows, C) bf16, the layer's normed input rows; tokens (rows,) int64; table (vocab, Hkv * 128) bf16; gate
    (Hkv, C) fp32. C must be a multiple of 256."""

    def __init__(self, h: Tensor, tokens: Tensor, table: Tensor, gate: Tensor):
        assert h.dtype == table.dtype == torch.bfloat16 and gate.dtype == torch.float32 and tokens.dtype == torch.long
        assert h.is_contiguous() and table.is_contiguous() and gate.is_contiguous() and tokens.is_contiguous()
        assert h.shape[1] == gate.shape[1] and h.shape[1] % 256 == 0 and tokens.shape == (h.shape[0],)
        assert table.shape[1] == gate.shape[0] * HEAD_DIM
        self.h, self.tokens, self.table, self.gate = h, tokens, table, gate

    def args(self) -> list:
        return [pointer(self.h), pointer(self.tokens), pointer(self.table), pointer(self.gate), self.h.shape[1],
                self.table.shape[0]]


def rotary_table(positions: int, theta: float, device: "torch.device | str" = "cpu") -> tuple[Tensor, Tensor]:
    """cos, sin fp32 (positions, 64) of the angles t theta^(-2i/128), computed in fp64 and rounded once
    (reference model/modeling.py:169-176)."""
    exponent = torch.arange(0, HEAD_DIM, 2, dtype=torch.float64) / HEAD_DIM
    freqs = torch.arange(positions, dtype=torch.float64)[:, None] * theta ** -exponent
    return freqs.cos().float().to(device), freqs.sin().float().to(device)


def kv_append(qkv: Tensor, q_gain: Tensor, k_gain: Tensor, cos: Tensor, sin: Tensor, pos: Tensor,
              cache: Fp8KVCache, Hq: int, slot_map: Tensor | None = None, q_out: Tensor | None = None,
              status: Tensor | None = None, ve: "ValueEmbed | None" = None) -> Tensor:
    """Norm + rotate q and k, quantise k and v to e4m3 with per-(token, head) scales and append them at `pos`.
    qkv (rows, (Hq + 2 Hkv) * 128) bf16, row stride free; gains fp32 (128,); cos/sin fp32 (T, 64); pos int32
    (rows,); slot_map int32 (rows,) or None; ve: the layer's value-embedding mix on v, if it has one. Rows with a
    negative position are idle (skipped). Returns q_out (rows, Hq, 128) bf16."""
    rows, Hkv = qkv.shape[0], cache.kv_heads
    assert qkv.dtype == torch.bfloat16 and qkv.stride(-1) == 1 and qkv.shape[1] == (Hq + 2 * Hkv) * HEAD_DIM
    assert pos.dtype == torch.int32 and pos.shape == (rows,) and pos.is_contiguous()
    assert cos.shape == sin.shape and cos.shape[1] == HEAD_DIM // 2 and cos.is_contiguous() and sin.is_contiguous()
    assert q_gain.dtype == k_gain.dtype == cos.dtype == sin.dtype == torch.float32
    assert slot_map is None or (slot_map.dtype == torch.int32 and slot_map.shape == (rows,))
    if q_out is None:
        q_out = torch.empty((rows, Hq, HEAD_DIM), dtype=torch.bfloat16, device=qkv.device)
    head = [pointer(qkv), pointer(q_gain), pointer(k_gain), pointer(cos), pointer(sin), pointer(pos), pointer(slot_map),
            pointer(q_out), pointer(cache.pages), rows, Hq, Hkv, qkv.stride(0), cos.shape[0], cache.n_slots,
            cache.pages_per_slot]
    if ve is None:
        rc = cuda_library("kv_append").kv_append_fp8(*head, pointer(status), stream())
    else:
        assert ve.h.shape[0] == rows and ve.gate.shape[0] == Hkv
        rc = cuda_library("kv_append").kv_append_fp8_ve(*head, *ve.args(), pointer(status), stream())
    check(rc, "kv_append_fp8")
    return q_out


def chunk_pages_for(B: int, Hkv: int, max_kv_len: int) -> int:
    return cuda_library("decode_attn").decode_attn_chunk_pages(B, Hkv, max_kv_len)


def plan_chunk_pages(lens: list[int], Hkv: int, max_kv_len: int, window: int = 0) -> int:
    """chunk_pages for lengths the host knows: the library's model of how the split kernel's blocks fill the GPU
    picks the size that leaves no nearly empty last wave. For ragged batches whose lengths change slowly."""
    import ctypes

    arr = (ctypes.c_int * len(lens))(*lens)
    return cuda_library("decode_attn").decode_attn_plan_chunk_pages(ctypes.cast(arr, ctypes.c_void_p), len(lens), Hkv,
                                                                   max_kv_len, window)


def workspace_bytes(B: int, Hq: int, Hkv: int, max_kv_len: int, chunk_pages: int = 0) -> int:
    return cuda_library("decode_attn").decode_attn_workspace_bytes(B, Hq, max_kv_len, Hkv, chunk_pages)


def _attend(entry: str, q: Tensor, cache: Fp8KVCache, lens: Tensor, result: Tensor | None, max_kv_len: int,
            slot_map: Tensor | None, window: int, chunk_pages: int, softmax_scale: float | None,
            workspace: Tensor | None, status: Tensor | None) -> None:
    B, Hq = q.shape[0], q.shape[1]
    assert q.dtype == torch.bfloat16 and q.is_contiguous() and q.shape[2] == HEAD_DIM
    assert lens.dtype == torch.int32 and lens.shape == (B,) and lens.is_contiguous()
    assert slot_map is None or (slot_map.dtype == torch.int32 and slot_map.shape == (B,))
    need = workspace_bytes(B, Hq, cache.kv_heads, min(max_kv_len, cache.capacity), chunk_pages)
    if workspace is None:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    scale = HEAD_DIM ** -0.5 if softmax_scale is None else softmax_scale
    head = [pointer(q), pointer(cache.pages), pointer(lens), pointer(slot_map), pointer(workspace), workspace.numel()]
    if result is not None:
        head.append(pointer(result))
    rc = getattr(cuda_library("decode_attn"), entry)(
        *head, B, Hq, cache.kv_heads, cache.n_slots, cache.pages_per_slot, max_kv_len, window, chunk_pages, scale,
        pointer(status), stream())
    check(rc, entry)


def decode_attention(q: Tensor, cache: Fp8KVCache, lens: Tensor, max_kv_len: int, slot_map: Tensor | None = None,
                     window: int = 0, chunk_pages: int = 0, softmax_scale: float | None = None,
                     workspace: Tensor | None = None, out: Tensor | None = None,
                     status: Tensor | None = None) -> Tensor:
    """out[b, h] = softmax(q[b, h] . K * scale) V over the cached positions [max(0, lens[b] - window), lens[b]) of
    slot slot_map[b]. q (B, Hq, 128) bf16; lens int32 (B,) on the device; max_kv_len an upper bound of lens known
    to the host. Returns (B, Hq, 128) bf16."""
    if out is None:
        out = torch.empty_like(q)
    _attend("decode_attn_fp8", q, cache, lens, out, max_kv_len, slot_map, window, chunk_pages, softmax_scale,
            workspace, status)
    return out


def decode_step_attention(qkv: Tensor, q_gain: Tensor, k_gain: Tensor, cos: Tensor, sin: Tensor, pos: Tensor,
                          cache: Fp8KVCache, Hq: int, max_kv_len: int, slot_map: Tensor | None = None,
                          window: int = 0, chunk_pages: int = 0, softmax_scale: float | None = None,
                          workspace: Tensor | None = None, out: Tensor | None = None,
                          status: Tensor | None = None, slots: "list[int] | None" = None,
                          ve: "ValueEmbed | None" = None) -> Tensor:
    """kv_append + decode_attention for one new token per sequence in two launches instead of three: the attention
    kernel norms, rotates, quantises and stores the token's q, k, v itself, then attends over positions
    [.., pos + 1). Same cache bytes and outputs as the two calls; q is not returned. Rows must address distinct
    slots (two rows of one slot would race on its pages); a caller that has the slot list on the host passes it as
    `slots` (the host copy of slot_map, idle rows included) and gets a ValueError for duplicates. max_kv_len bounds
    pos + 1. Rows with pos < 0 are idle: nothing appended, a zero output row."""
    if slots is not None and len(set(slots)) != len(slots):
        raise ValueError(f"decode_step_attention: rows share a slot ({sorted(s for s in set(slots) if slots.count(s) > 1)}); "
                         "use kv_append + decode_attention for rows of one sequence")
    rows, Hkv = qkv.shape[0], cache.kv_heads
    assert qkv.dtype == torch.bfloat16 and qkv.stride(-1) == 1 and qkv.shape[1] == (Hq + 2 * Hkv) * HEAD_DIM
    assert pos.dtype == torch.int32 and pos.shape == (rows,) and pos.is_contiguous()
    assert cos.shape == sin.shape and cos.shape[1] == HEAD_DIM // 2 and cos.is_contiguous() and sin.is_contiguous()
    assert q_gain.dtype == k_gain.dtype == cos.dtype == sin.dtype == torch.float32
    assert slot_map is None or (slot_map.dtype == torch.int32 and slot_map.shape == (rows,))
    need = workspace_bytes(rows, Hq, Hkv, min(max_kv_len, cache.capacity), chunk_pages)
    if workspace is None:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=qkv.device)
    if out is None:
        out = torch.empty((rows, Hq, HEAD_DIM), dtype=torch.bfloat16, device=qkv.device)
    scale = HEAD_DIM ** -0.5 if softmax_scale is None else softmax_scale
    head = [pointer(qkv), pointer(q_gain), pointer(k_gain), pointer(cos), pointer(sin), pointer(pos), pointer(slot_map),
            pointer(cache.pages), pointer(workspace), workspace.numel(), pointer(out), rows, Hq, Hkv, qkv.stride(0),
            cos.shape[0], cache.n_slots, cache.pages_per_slot, max_kv_len, window, chunk_pages, scale]
    if ve is None:
        rc = cuda_library("decode_attn").decode_step_attn_fp8(*head, pointer(status), stream())
    else:
        assert ve.h.shape[0] == rows and ve.gate.shape[0] == Hkv
        rc = cuda_library("decode_attn").decode_step_attn_fp8_ve(*head, *ve.args(), pointer(status), stream())
    check(rc, "decode_step_attn_fp8")
    return out


def prefill_groups(slots, positions, limit: int) -> list[int]:
    """Group consecutive rows of a prefill pass for prefill_attention: a group is a run of rows of one slot with
    positions ascending by one, at most `limit` long. slots, positions: sequences or numpy arrays. Returns
    group_start with the end sentinel."""
    import numpy as np

    n = len(slots)
    if n == 0:
        return [0]
    s, p = np.asarray(slots, dtype=np.int64), np.asarray(positions, dtype=np.int64)
    run_start = np.ones(n, dtype=bool)  # a run: one slot, positions ascending by one
    run_start[1:] = (s[1:] != s[:-1]) | (p[1:] != p[:-1] + 1)
    first_of_run = np.flatnonzero(run_start)[np.cumsum(run_start) - 1]
    group_start = (np.arange(n) - first_of_run) % limit == 0  # runs are cut into groups of `limit` rows
    return np.flatnonzero(group_start).tolist() + [n]


def prefill_rows_per_block(Hq: int, Hkv: int) -> int:
    """Rows one block of prefill_attn_fp8 takes: 88 for Hq == Hkv, 22 for four query heads per kv head."""
    return cuda_library("decode_attn").prefill_attn_rows_per_block(Hq, Hkv)


class PrefillPlan:
    """What prefill_attention needs besides q for one pass of rows, built once per pass and shared by the layers: the
    row groups (longest first, so the blocks with the most pages start first), the rows' slots and lengths on the
    device."""

    def __init__(self, slots, positions, Hq: int, cache: Fp8KVCache, device):
        import numpy as np

        slots, positions = np.asarray(slots, dtype=np.int32), np.asarray(positions, dtype=np.int32)
        self.rows_per_block = prefill_rows_per_block(Hq, cache.kv_heads)
        starts = np.asarray(prefill_groups(slots, positions, self.rows_per_block), dtype=np.int32)
        self.rows, self.n_groups = len(slots), len(starts) - 1
        # blocks start in list order: the groups that reach furthest into their prompts (most pages) go first, so
        # the short ones fill the gaps at the end
        reach = positions[starts[1:] - 1] if self.n_groups else positions[:0]
        order = np.argsort(-reach.astype(np.int64), kind="stable")
        self.group_first = torch.from_numpy(starts[:-1][order].copy()).to(device)
        self.group_rows = torch.from_numpy((starts[1:] - starts[:-1])[order].copy()).to(device)
        self.slot_map = torch.from_numpy(slots).to(device)
        self.lens = torch.from_numpy(positions + 1).to(device)


def prefill_attention(q: Tensor, cache: Fp8KVCache, plan: PrefillPlan, softmax_scale: float | None = None,
                      out: Tensor | None = None, status: Tensor | None = None) -> Tensor:
    """Attention for a prefill pass: q (rows, Hq, 128) bf16 of the rows the plan was built for, whose k, v are
    already appended; row r attends positions [0, positions[r]] of slots[r]. Rows of one prompt should be
    consecutive and ascending: a block takes up to prefill_rows_per_block of them and reads the prompt's cache once
    for all. Returns (rows, Hq, 128) bf16."""
    rows, Hq = q.shape[0], q.shape[1]
    assert rows == plan.rows and q.dtype == torch.bfloat16 and q.is_contiguous()
    if out is None:
        out = torch.empty_like(q)
    scale = HEAD_DIM ** -0.5 if softmax_scale is None else softmax_scale
    rc = cuda_library("decode_attn").prefill_attn_fp8(
        pointer(q), pointer(cache.pages), pointer(plan.lens), pointer(plan.slot_map), pointer(plan.group_first),
        pointer(plan.group_rows), plan.n_groups, pointer(out), rows, Hq, cache.kv_heads, cache.n_slots, cache.pages_per_slot, scale,
        pointer(status), stream())
    check(rc, "prefill_attn_fp8")
    return out


def decode_attention_static(q: Tensor, cache: Fp8KVCache, lens: Tensor, max_kv_len: int,
                            slot_map: Tensor | None = None, window: int = 0, chunk_pages: int = 0,
                            softmax_scale: float | None = None, out: Tensor | None = None,
                            status: Tensor | None = None) -> Tensor:
    """decode_attention for callers that may not allocate device memory: the per-chunk states live in 8 MiB built
    into the library instead of a workspace tensor (pass `out`, and nothing here allocates). Raises NativeError
    (status 6) when the call would need more. Calls on one device share that memory, so keep them stream-ordered;
    make the first call on a device outside CUDA-graph capture."""
    B, Hq = q.shape[0], q.shape[1]
    assert q.dtype == torch.bfloat16 and q.is_contiguous() and q.shape[2] == HEAD_DIM
    assert lens.dtype == torch.int32 and lens.shape == (B,) and lens.is_contiguous()
    assert slot_map is None or (slot_map.dtype == torch.int32 and slot_map.shape == (B,))
    if out is None:
        out = torch.empty_like(q)
    scale = HEAD_DIM ** -0.5 if softmax_scale is None else softmax_scale
    rc = cuda_library("decode_attn").decode_attn_fp8_static(
        pointer(q), pointer(cache.pages), pointer(lens), pointer(slot_map), pointer(out), B, Hq, cache.kv_heads,
        cache.n_slots, cache.pages_per_slot, max_kv_len, window, chunk_pages, scale, pointer(status), stream())
    check(rc, "decode_attn_fp8_static")
    return out


def decode_attention_partial(q: Tensor, cache: Fp8KVCache, lens: Tensor, max_kv_len: int,
                             slot_map: Tensor | None = None, window: int = 0, chunk_pages: int = 0,
                             softmax_scale: float | None = None, workspace: Tensor | None = None,
                             part: Tensor | None = None, status: Tensor | None = None) -> Tensor:
    """As decode_attention but returns the un-normalised state fp32 (B, Hq, 132) = (m, l, 0, 0, o[128]) for merging
    with the states of other position slices (merge_partials)."""
    if part is None:
        part = torch.empty((q.shape[0], q.shape[1], PART_FLOATS), dtype=torch.float32, device=q.device)
    _attend("decode_attn_fp8_partial", q, cache, lens, part, max_kv_len, slot_map, window, chunk_pages,
            softmax_scale, workspace, status)
    return part


def decode_attention_split(q: Tensor, cache: Fp8KVCache, lens: Tensor, max_kv_len: int, workspace: Tensor,
                           slot_map: Tensor | None = None, window: int = 0, chunk_pages: int = 0,
                           softmax_scale: float | None = None, status: Tensor | None = None) -> None:
    """Only the split-KV launch of decode_attention; per-chunk states stay in `workspace`."""
    _attend("decode_attn_fp8_split", q, cache, lens, None, max_kv_len, slot_map, window, chunk_pages, softmax_scale,
            workspace, status)


def merge_partials(parts: Tensor, out: Tensor | None = None) -> Tensor:
    """parts fp32 (n_parts, B, Hq, 132) -> normalised bf16 (B, Hq, 128)."""
    assert parts.dtype == torch.float32 and parts.is_contiguous() and parts.shape[-1] == PART_FLOATS
    n_parts, B, Hq = parts.shape[:3]
    if out is None:
        out = torch.empty((B, Hq, HEAD_DIM), dtype=torch.bfloat16, device=parts.device)
    rc = cuda_library("decode_attn").decode_attn_merge(pointer(parts), n_parts, B * Hq, pointer(out), stream())
    check(rc, "decode_attn_merge")
    return out
