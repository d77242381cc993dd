"""One decode step of the attention path for a fixed set of slots, captured once as a CUDA graph and replayed.

The reference runs its whole step as captured graphs launched from Python through one ctypes call
(model/kernels/decode.cu:848-902,1000-1016,1107-1110; inference/decoder.py:285) because at decode sizes the step is
bound by launch latency, not by kernels. This is the same idea for the part of the step this package owns:

    pinned host qkv rows + positions --copy--> device --decode_step_attn_fp8 (append + attend)--> cache;
    the merge kernel writes the bf16 output rows straight into the pinned host buffer (it is written once and never
    re-read by the GPU, so no device copy and no copy node are needed: the stores cross PCIe as they are produced)

The rows are cut into `parts` groups that run as parallel branches of the graph (copy, then append + attention, per
group): the input copy of every group but the first crosses PCIe under the attention of the groups before it, so only
1 / parts of the copy stays in front of the kernels. Sequences never mix, so the outputs are those of one launch.

The caller writes `qkv_host` and `pos_host`, calls run(), and reads `out_host`. Sequence lengths are pos + 1 (the
new token is attended through the cache). The graph is sized for the cache's capacity, so it stays valid as the
sequences grow."""

import torch
from torch import Tensor

from . import attention as ops
from .decoder import no_collection
from .kv_cache import HEAD_DIM, Fp8KVCache


class DecodeStep:
    def __init__(self, cache: Fp8KVCache, Hq: int, cos: Tensor, sin: Tensor, q_gain: Tensor, k_gain: Tensor,
                 batch: int, slot_map: Tensor | None = None, window: int = 0, chunk_pages: int = 0,
                 softmax_scale: float | None = None, max_kv_len: int | None = None, parts: int = 0):
        dev, Hkv = cache.device, cache.kv_heads
        # the step appends inside the attention launch, which needs one row per slot: checked once, on the host
        self.slots = list(range(batch)) if slot_map is None else slot_map.tolist()
        if len(set(self.slots)) != len(self.slots):
            raise ValueError("rows of a decode step share a slot")
        self.cache, self.Hq, self.batch = cache, Hq, batch
        self.cos, self.sin, self.q_gain, self.k_gain = cos, sin, q_gain, k_gain
        self.window, self.softmax_scale = window, softmax_scale
        self.slot_map = torch.arange(batch, dtype=torch.int32, device=dev) if slot_map is None else slot_map
        self.max_kv_len = min(max_kv_len or cache.capacity, cache.capacity)
        self.chunk_pages = chunk_pages or ops.chunk_pages_for(batch, Hkv, self.max_kv_len)
        # groups of rows that run as parallel branches: at most eight, of at least eight rows each (measured at 64
        # rows of 8,192 positions: 218 us in one group, 204 in two, 199 in four, 196 in eight, 200 in sixteen)
        self.parts = parts or next((p for p in (8, 4, 2) if batch % p == 0 and batch // p >= 8), 1)
        assert batch % self.parts == 0, "the groups have equal numbers of rows"
        width = (Hq + 2 * Hkv) * HEAD_DIM
        # ONE pinned buffer and one device buffer: [positions, padded to 256 bytes | qkv rows]. The first group's copy
        # takes the positions of all rows along with its own qkv rows; the other groups copy their qkv rows only.
        self.pos_bytes = (batch * 4 + 255) // 256 * 256
        qkv_bytes = batch * width * 2
        self.in_host = torch.zeros(self.pos_bytes + qkv_bytes, dtype=torch.uint8).pin_memory()
        self.in_dev = torch.empty(self.pos_bytes + qkv_bytes, dtype=torch.uint8, device=dev)
        self.pos_host = self.in_host[:batch * 4].view(torch.int32)
        self.qkv_host = self.in_host[self.pos_bytes:].view(torch.bfloat16).view(batch, width)
        self.out_host = torch.zeros((batch, Hq, HEAD_DIM), dtype=torch.bfloat16).pin_memory()
        self.pos = self.in_dev[:batch * 4].view(torch.int32)
        self.qkv = self.in_dev[self.pos_bytes:].view(torch.bfloat16).view(batch, width)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        rows = batch // self.parts
        need = ops.workspace_bytes(rows, Hq, Hkv, self.max_kv_len, self.chunk_pages)
        self.workspaces = [torch.empty(max(need, 16), dtype=torch.uint8, device=dev) for _ in range(self.parts)]
        self.stream = torch.cuda.Stream(dev)
        self.branches = [torch.cuda.Stream(dev) for _ in range(self.parts - 1)]
        self.joins: list[torch.cuda.Event] = []
        self.graph: torch.cuda.CUDAGraph | None = None

    @property
    def h2d_bytes(self) -> int:
        return self.qkv_host.numel() * 2 + self.pos_host.numel() * 4

    @property
    def d2h_bytes(self) -> int:
        return self.out_host.numel() * 2

    def _enqueue(self) -> None:
        """On the current stream (self.stream): fork one branch per group of rows, join at the end."""
        rows, row_bytes = self.batch // self.parts, self.qkv.shape[1] * 2
        fork = torch.cuda.Event()
        fork.record()
        for part in range(self.parts):
            stream = torch.cuda.current_stream(self.cache.device) if part == 0 else self.branches[part - 1]
            with torch.cuda.stream(stream):
                if part:
                    stream.wait_event(fork)
                first = 0 if part == 0 else self.pos_bytes + part * rows * row_bytes
                last = self.pos_bytes + (part + 1) * rows * row_bytes
                self.in_dev[first:last].copy_(self.in_host[first:last], non_blocking=True)
                if part:  # the positions travel with the first group's copy
                    stream.wait_event(self.positions_there)
                else:
                    self.positions_there = torch.cuda.Event()
                    self.positions_there.record()
                r = slice(part * rows, (part + 1) * rows)
                ops.decode_step_attention(self.qkv[r], self.q_gain, self.k_gain, self.cos, self.sin, self.pos[r],
                                          self.cache, self.Hq, self.max_kv_len, slot_map=self.slot_map[r],
                                          window=self.window, chunk_pages=self.chunk_pages,
                                          softmax_scale=self.softmax_scale, workspace=self.workspaces[part],
                                          out=self.out_host[r], status=self.status, slots=self.slots[r])
                if part:
                    done = torch.cuda.Event()
                    done.record()
                    self.joins.append(done)
        for done in self.joins:
            torch.cuda.current_stream(self.cache.device).wait_event(done)
        self.joins = []

    def capture(self) -> None:
        """Run the step once eagerly (first-use set-up must happen outside capture; the token it appends is
        overwritten by the next run at the same position) and capture it."""
        self.stream.wait_stream(torch.cuda.current_stream(self.cache.device))
        with torch.cuda.stream(self.stream):
            self._enqueue()
            self.stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with no_collection(), torch.cuda.graph(self.graph, stream=self.stream):
                self._enqueue()

    def run(self) -> None:
        """Append the tokens in qkv_host at pos_host and attend; out_host holds the result on return. The graph is
        launched on the caller's current stream (ordered after the caller's earlier work there), then that stream
        is synchronised."""
        if self.graph is None:
            self.capture()
        self.graph.replay()
        torch.cuda.current_stream(self.cache.device).synchronize()

    def check(self) -> None:
        """Raise if a kernel flagged a bad position / length or a wait that ran out (reads the device word)."""
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"device status {code:#x} (NCB_DEV_* bits)")
