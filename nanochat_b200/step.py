"""One decode step of the attention path for a fixed set of slots, captured once as a CUDA graph and replayed.

The reference runs its whole step as captured graphs launched from Python through one ctypes call
(model/kernels/decode.cu:848-902,1000-1016,1107-1110; inference/decoder.py:285) because at decode sizes the step is
bound by launch latency, not by kernels. This is the same idea for the part of the step this package owns:

    pinned host qkv rows + positions --copy--> device --decode_step_attn_fp8 (append + attend)--> cache;
    the merge kernel writes the bf16 output rows straight into the pinned host buffer (it is written once and never
    re-read by the GPU, so no device copy and no copy node are needed: the stores cross PCIe as they are produced)

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
                 softmax_scale: float | None = None, max_kv_len: int | None = None):
        dev, Hkv = cache.device, cache.kv_heads
        # the step appends inside the attention launch, which needs one row per slot: checked once, on the host
        self.slots = list(range(batch)) if slot_map is None else slot_map.tolist()
        self.cache, self.Hq, self.batch = cache, Hq, batch
        self.cos, self.sin, self.q_gain, self.k_gain = cos, sin, q_gain, k_gain
        self.slot_map, self.window, self.softmax_scale = slot_map, window, softmax_scale
        self.max_kv_len = min(max_kv_len or cache.capacity, cache.capacity)
        self.chunk_pages = chunk_pages or ops.chunk_pages_for(batch, Hkv, self.max_kv_len)
        width = (Hq + 2 * Hkv) * HEAD_DIM
        # qkv rows and positions share ONE pinned buffer and one device buffer, so a step's inputs cross PCIe in a
        # single copy (a second copy node costs about as much as the 0.8 MB themselves)
        qkv_bytes = batch * width * 2
        self.in_host = torch.zeros(qkv_bytes + batch * 4, dtype=torch.uint8).pin_memory()
        self.in_dev = torch.empty(qkv_bytes + batch * 4, dtype=torch.uint8, device=dev)
        self.qkv_host = self.in_host[:qkv_bytes].view(torch.bfloat16).view(batch, width)
        self.pos_host = self.in_host[qkv_bytes:].view(torch.int32)
        self.out_host = torch.zeros((batch, Hq, HEAD_DIM), dtype=torch.bfloat16).pin_memory()
        self.qkv = self.in_dev[:qkv_bytes].view(torch.bfloat16).view(batch, width)
        self.pos = self.in_dev[qkv_bytes:].view(torch.int32)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        need = ops.workspace_bytes(batch, Hq, Hkv, self.max_kv_len, self.chunk_pages)
        self.workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
        self.stream = torch.cuda.Stream(dev)
        self.graph: torch.cuda.CUDAGraph | None = None

    @property
    def h2d_bytes(self) -> int:
        return self.qkv_host.numel() * 2 + self.pos_host.numel() * 4

    @property
    def d2h_bytes(self) -> int:
        return self.out_host.numel() * 2

    def _enqueue(self) -> None:
        self.in_dev.copy_(self.in_host, non_blocking=True)
        ops.decode_step_attention(self.qkv, self.q_gain, self.k_gain, self.cos, self.sin, self.pos, self.cache,
                                  self.Hq, self.max_kv_len, slot_map=self.slot_map, window=self.window,
                                  chunk_pages=self.chunk_pages, softmax_scale=self.softmax_scale,
                                  workspace=self.workspace, out=self.out_host, status=self.status, slots=self.slots)

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
