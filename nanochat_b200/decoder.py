"""The decode step around the fp8 attention path: a greedy decoder for nanochat-shaped models.

Stands where the reference's NativeDecoder / decode.cu step graph stands (inference/decoder.py:123-324;
model/kernels/decode.cu:848-891): per layer
    norm -> qkv GEMM -> [kv_append_fp8 -> decode_attn_fp8] -> o GEMM + residual -> norm -> up GEMM, relu^2 ->
    down GEMM + residual
then the final norm, the lm_head GEMM and an argmax. Every GEMM runs on this package's kernels (the reference's own
GEMM kernel is Hopper-only wgmma, decode.cu:232-359, and has to be replaced either way): steps of at most 16 rows on
csrc/decode_step.cu (weight-streaming mma.sync GEMMs with fused norm and epilogues), 17 to 64 rows on
csrc/stream_gemm.cu (tcgen05 weight stream, K split over a cluster), larger passes (bigger batches, prefill) on
csrc/tile_gemm.cu (tiled tcgen05 GEMM) with the norm / residual steps between them as kernels of their own. A library
GEMM (torch) is only the fallback for widths that are not a multiple of 128. The whole step is captured in one CUDA
graph per batch size, the reference's remedy for launch-bound decode steps.

Model semantics follow the reference's exported model (inference/modeling_nanochat.py:113-195): parameter-free RMS
norm with eps FLT_EPSILON, h = x0 = norm(embed), per layer h = resid_lambda h + x0_lambda x0 (fp32, rounded once),
QK-norm with per-dimension gains + the "-theta, split halves" rotary, relu^2 MLP, fp32 logits from the bf16 head.
The reference's own checkpoints also have value embeddings on alternating layers (v + 2 sigmoid(W n) ve, fused into
the append kernels) and learned resid / x0 lambdas (fused into the GEMM epilogue that writes the stream); both are
optional per layer here. Sliding windows are supported per layer; the logit cap (monotone) does not change a greedy
choice (decode.cu:195) and is applied when sampling.

Prefill runs prompt tokens as rows through the same kernels, every row attending to the positions up to its own
(decode.cu:859-863,1041-1051; inference/decoder.py:211-222); the prompt's last token is the first decode step's
input (decoder.py:196,207,215)."""

import contextlib
import gc
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import Tensor

from . import attention as ops
from .kv_cache import HEAD_DIM, Fp8KVCache
from .native import check, cuda_library, pointer, stream
from .prompt_store import PromptStore

EPS = 1.1920928955078125e-07  # FLT_EPSILON (reference model/ops/linear.py:20)


@contextlib.contextmanager
def no_collection():
    """Python's cyclic garbage collector switched off for the duration of a stream capture: a collection that
    happens to run inside the capture can finalise an old graph or memory pool, whose cudaFree invalidates the
    capture ("operation failed due to a previous error during capture" at the next launch)."""
    enabled = gc.isenabled()
    gc.collect()
    gc.disable()
    try:
        yield
    finally:
        if enabled:
            gc.enable()


@dataclass
class DecoderConfig:
    n_layers: int
    hidden: int
    n_heads: int
    n_kv_heads: int
    intermediate: int
    vocab: int
    rope_theta: float = 10000.0
    max_len: int = 1024
    windows: list[int] = field(default_factory=list)  # per layer, 0 = full attention

    @property
    def qkv_width(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * HEAD_DIM

    @staticmethod
    def from_exported(config, max_len: int | None = None) -> "DecoderConfig":
        """From the exported model's configuration (inference/modeling_nanochat.py NanochatConfig: any object or dict
        with its field names). A layer's window is the config's sliding_window where layer_types says
        "sliding_attention", else 0 (full attention)."""
        get = config.get if isinstance(config, dict) else lambda k, d=None: getattr(config, k, d)
        if get("head_dim", HEAD_DIM) != HEAD_DIM:
            raise ValueError(f"head_dim {get('head_dim')}: the kernels take {HEAD_DIM}")
        L = get("num_hidden_layers")
        types = get("layer_types") or ["full_attention"] * L
        windows = [int(get("sliding_window") or 0) if t == "sliding_attention" else 0 for t in types]
        rope = get("rope_parameters") or {}
        return DecoderConfig(n_layers=L, hidden=get("hidden_size"), n_heads=get("num_attention_heads"),
                             n_kv_heads=get("num_key_value_heads") or get("num_attention_heads"),
                             intermediate=get("intermediate_size"), vocab=get("vocab_size"),
                             rope_theta=float(rope.get("rope_theta", get("rope_theta", 10000.0))),
                             max_len=max_len or get("max_position_embeddings"),
                             windows=windows if any(windows) else [])


@dataclass
class LayerWeights:
    wqkv: Tensor   # bf16 [(Hq + 2 Hkv) 128, C]: q heads, k heads, v heads
    wo: Tensor     # bf16 [C, Hq 128]
    wup: Tensor    # bf16 [F, C]
    wdown: Tensor  # bf16 [C, F]
    q_gain: Tensor  # fp32 [128]
    k_gain: Tensor  # fp32 [128]
    resid_lambda: float = 1.0
    x0_lambda: float = 0.0
    ve_table: Tensor | None = None  # bf16 [V, Hkv 128]: the layer's value embedding (model/modeling.py:35-37), or None
    ve_gate: Tensor | None = None   # fp32 [Hkv, C]

    @property
    def mixes(self) -> bool:
        return self.resid_lambda != 1.0 or self.x0_lambda != 0.0


@dataclass
class DecoderWeights:
    embed: Tensor    # bf16 [V, C]
    lm_head: Tensor  # bf16 [V, C]
    layers: list[LayerWeights]

    @staticmethod
    def from_state_dict(state: dict, cfg: DecoderConfig, device: "torch.device | str" = "cuda") -> "DecoderWeights":
        """From a checkpoint of the exported model (the names of inference/modeling_nanochat.py: model.embed_tokens,
        lm_head, model.layers.i.self_attn.{q,k,v,o}_proj, .q_norm_weight / .k_norm_weight, .ve_gate,
        model.layers.i.mlp.{up,down}_proj, model.value_embeds.i, model.resid_lambdas / x0_lambdas). GEMM weights,
        the embedding and value-embedding tables become bf16 (the forward's rounding at use, as the reference's
        decoder takes them, inference/decoder.py:155-165); gains, gates and lambdas stay fp32."""
        def t(name: str, dtype) -> Tensor:
            return state[name].detach().to(device=device, dtype=dtype).contiguous()

        bf, f32 = torch.bfloat16, torch.float32
        resid = state["model.resid_lambdas"].float().tolist() if "model.resid_lambdas" in state else [1.0] * cfg.n_layers
        x0 = state["model.x0_lambdas"].float().tolist() if "model.x0_lambdas" in state else [0.0] * cfg.n_layers
        layers = []
        for i in range(cfg.n_layers):
            p = f"model.layers.{i}."
            wqkv = torch.cat([t(p + f"self_attn.{n}_proj.weight", bf) for n in "qkv"], 0)
            if wqkv.shape != (cfg.qkv_width, cfg.hidden):
                raise ValueError(f"layer {i}: q, k, v projections of {tuple(wqkv.shape)}, expected {(cfg.qkv_width, cfg.hidden)}")
            ve = f"model.value_embeds.{i}.weight" in state
            layers.append(LayerWeights(
                wqkv, t(p + "self_attn.o_proj.weight", bf), t(p + "mlp.up_proj.weight", bf),
                t(p + "mlp.down_proj.weight", bf), t(p + "self_attn.q_norm_weight", f32),
                t(p + "self_attn.k_norm_weight", f32), resid_lambda=float(resid[i]), x0_lambda=float(x0[i]),
                ve_table=t(f"model.value_embeds.{i}.weight", bf) if ve else None,
                ve_gate=t(p + "self_attn.ve_gate.weight", f32) if ve else None))
        return DecoderWeights(t("model.embed_tokens.weight", bf), t("lm_head.weight", bf), layers)

    @staticmethod
    def random_init(cfg: DecoderConfig, seed: int, device: "torch.device | str", std: float = 0.02,
                    on_device: bool = False) -> "DecoderWeights":
        """bf16 weights drawn from N(0, std), gains = 1. By default on the CPU generator (identical on every
        machine, which tests rely on); on_device draws with the device's generator instead, much faster for
        billion-parameter benchmark models."""
        where = device if on_device else "cpu"
        gen = torch.Generator(device=where).manual_seed(seed)
        C, Fdim = cfg.hidden, cfg.intermediate

        def w(*shape):
            return (torch.randn(*shape, generator=gen, device=where) * std).bfloat16().to(device)

        layers = [LayerWeights(w(cfg.qkv_width, C), w(C, cfg.n_heads * HEAD_DIM), w(Fdim, C), w(C, Fdim),
                               torch.ones(HEAD_DIM, device=device), torch.ones(HEAD_DIM, device=device))
                  for _ in range(cfg.n_layers)]
        return DecoderWeights(w(cfg.vocab, C), w(cfg.vocab, C), layers)


def rms_norm(x: Tensor) -> Tensor:
    return F.rms_norm(x, (x.size(-1),), eps=EPS)


MAX_SLOTS = 1024            # the reference's MAX_BATCH (model/kernels/decode.cu:29)
ALLOC_GRANULE = 2 << 20     # cudaMalloc rounds a large block up to the next 2 MiB (decode.cu:955-957)


def slot_bytes(cfg: DecoderConfig) -> int:
    """Device bytes one more slot costs a decoder of this shape: its pages in every layer's cache plus its rows of the
    step's buffers (hidden, qkv, attention output, MLP, x0, normed rows in bf16; fp32 logits and sampling
    probabilities; the int64 token trace), each rounded up to 256 bytes as the allocator rounds them. The reference
    sums its per-slot buffers the same way (slot_buffers / padded, decode.cu:977-979)."""
    from .kv_cache import PAGE_BYTES, cache_pages

    def padded(n: int) -> int:
        return (n + 255) // 256 * 256

    pages = cache_pages(cfg.max_len)
    cache = cfg.n_layers * cfg.n_kv_heads * pages * PAGE_BYTES
    rows = sum(padded(2 * n) for n in (cfg.hidden, cfg.qkv_width, cfg.n_heads * HEAD_DIM, cfg.intermediate,
                                       cfg.hidden, cfg.hidden))
    rows += 2 * padded(4 * cfg.vocab) + padded(8 * (pages * 64 + 1))
    return cache + rows


def slots_that_fit(cfg: DecoderConfig, free_bytes: int, max_slots: int = MAX_SLOTS) -> int:
    """How many slots a decoder of this shape gets out of `free_bytes` of device memory: the most (at most max_slots)
    whose block fits the free memory rounded down to the allocation granule, the reference's rule for its batch size
    (dec_create, decode.cu:983-987: `B = min(free / slot, MAX_BATCH)`, and it refuses to start with none). Measure
    `free_bytes` after the weights are on the device (torch.cuda.mem_get_info()[0]); keep what else the process
    needs (workspaces, the prefill pass's rows, CUDA graphs) out of it."""
    usable = free_bytes // ALLOC_GRANULE * ALLOC_GRANULE
    n = min(usable // slot_bytes(cfg), max_slots)
    if n < 1:
        raise MemoryError(f"not one slot of {slot_bytes(cfg)} bytes fits {free_bytes} free bytes")
    return int(n)


class Decoder:
    """Greedy decoding of up to n_slots sequences with an fp8 KV cache per layer."""

    @classmethod
    def sized_for_free_memory(cls, cfg: DecoderConfig, weights: DecoderWeights, device: "torch.device | str" = "cuda",
                              reserve_bytes: int = 2 << 30, max_slots: int = MAX_SLOTS, **kwargs) -> "Decoder":
        """A decoder with as many slots as the device's free memory holds (slots_that_fit) after `reserve_bytes` are
        set aside for workspaces, prefill rows and graphs: how the reference sizes its batch (decode.cu:983-987)."""
        free, _ = torch.cuda.mem_get_info(torch.device(device))
        return cls(cfg, weights, slots_that_fit(cfg, max(free - reserve_bytes, 0), max_slots), device, **kwargs)

    def __init__(self, cfg: DecoderConfig, weights: DecoderWeights, n_slots: int, device: "torch.device | str" = "cuda",
                 prompt_store: int = 0, softcap: float = 0.0):
        """prompt_store: positions of pinned host memory for prompts already prefilled (0: none); a prompt seen
        again is copied back into its slot instead of being prefilled (inference/decoder.py:193-232). softcap: the
        output-logit cap c applied (c tanh(z / c)) before sampling; greedy choices need none (decode.cu:195)."""
        self.softcap = float(softcap)
        self.cfg, self.w, self.n_slots, self.device = cfg, weights, n_slots, torch.device(device)
        self.caches = [Fp8KVCache(n_slots, cfg.n_kv_heads, cfg.max_len, device=device) for _ in range(cfg.n_layers)]
        self.store = PromptStore(self.caches, prompt_store) if prompt_store > 0 else None
        self.capacity = self.caches[0].capacity
        self.cos, self.sin = ops.rotary_table(self.capacity, cfg.rope_theta, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.windows = cfg.windows or [0] * cfg.n_layers
        self.use_fused = True  # decode steps of <= 64 rows run on this package's GEMM kernels when the shapes allow
        self.use_stream_gemm = True  # ... of 17 to 64 rows on the tcgen05 stream_gemm (else the row path)
        self.use_tile_gemm = True  # row passes (prefill, steps above 64 rows) on the tiled tcgen05 GEMM, not torch's
        self.chunk_pages = 0  # attention chunk size of decode steps; 0: the library's choice for full-length slots
        self.prefetch_next = True  # stream_gemm also pulls the next GEMM's weights into L2 (d32-class step: -1.3 %)
        self._graphs: dict[int, tuple] = {}
        self._graph_tensors: dict[int, tuple] = {}
        self._workspaces: dict[tuple[int, int], Tensor] = {}

    # ---- one pass over `rows` tokens -------------------------------------------------------------------------

    def _workspace(self, rows: int, max_kv_len: int) -> Tensor:
        key = (rows, max_kv_len, self.chunk_pages)
        if key not in self._workspaces:
            need = ops.workspace_bytes(rows, self.cfg.n_heads, self.cfg.n_kv_heads, max_kv_len, self.chunk_pages)
            self._workspaces[key] = torch.empty(max(need, 16), dtype=torch.uint8, device=self.device)
        return self._workspaces[key]

    def hidden_rows(self, tokens: Tensor, pos: Tensor, slot_map: Tensor, max_kv_len: int,
                    attend_last_layer: bool = True, distinct_slots: bool = False,
                    host_rows: "tuple | None" = None) -> Tensor:
        """Final-normed hidden states (rows, C) bf16 of `tokens` at positions `pos` of slots `slot_map`; appends
        every row's k, v to the caches. max_kv_len bounds pos + 1. Any number of rows: GEMMs on the tiled tcgen05 kernel, everything
        between them on this package's kernels (embedding + norm, residual add + norm, relu^2, append, attention).
        distinct_slots: no two rows share a slot (a decode step), so the attention kernel may append its own
        token; prefill passes, where rows of one sequence read each other's positions, need the separate append.
        host_rows: the rows' (slots, positions) as host lists, when the caller has them (prefill): attention then
        runs in groups of consecutive rows that read a prompt's cache once per group instead of once per row."""
        cfg, lib, s = self.cfg, cuda_library("decode_step"), stream()
        rows, C = tokens.shape[0], cfg.hidden
        layers = self.w.layers
        if C % 8 or C > 4096 or cfg.intermediate % 8 or any(l.ve_table is not None and C % 256 for l in layers):
            return self._hidden_rows_torch(tokens, pos, slot_map, max_kv_len, attend_last_layer)
        lens = pos + 1
        workspace = self._workspace(rows, max_kv_len)
        plan, grouped = None, host_rows is not None and not any(self.windows)
        h = torch.empty((rows, C), dtype=torch.bfloat16, device=self.device)
        n = torch.empty_like(h)
        # the layers run one after the other on one stream, so they share their intermediate buffers (a pass of a
        # few hundred rows is bound by the host's launches: every allocation saved is host time saved)
        qkv_buf = torch.empty((rows, cfg.qkv_width), dtype=torch.bfloat16, device=self.device)
        q_buf = torch.empty((rows, cfg.n_heads, HEAD_DIM), dtype=torch.bfloat16, device=self.device)
        att_buf = torch.empty_like(q_buf)
        u_buf = torch.empty((rows, cfg.intermediate), dtype=torch.bfloat16, device=self.device)
        mixing = any(l.mixes for l in layers)
        x0 = torch.empty_like(h) if mixing else None
        if mixing:
            check(lib.embed_norm_mix(pointer(self.w.embed), pointer(tokens), pointer(h), pointer(x0),
                                     layers[0].resid_lambda, layers[0].x0_lambda, rows, C, cfg.vocab, s), "embed_norm_mix")
        else:
            check(lib.embed_norm(pointer(self.w.embed), pointer(tokens), pointer(h), rows, C, cfg.vocab, s), "embed_norm")
        check(lib.add_rms_norm(pointer(h), None, pointer(n), rows, C, s), "add_rms_norm")
        for i, layer in enumerate(layers):
            qkv = self.gemm_rows(n, layer.wqkv, out=qkv_buf)
            ve = None if layer.ve_table is None else ops.ValueEmbed(n, tokens, layer.ve_table, layer.ve_gate)
            if distinct_slots and (attend_last_layer or i < cfg.n_layers - 1):
                att = ops.decode_step_attention(qkv, layer.q_gain, layer.k_gain, self.cos, self.sin, pos,
                                                self.caches[i], cfg.n_heads, max_kv_len, slot_map=slot_map,
                                                window=self.windows[i], chunk_pages=self.chunk_pages,
                                                workspace=workspace, out=att_buf, status=self.status, ve=ve)
            else:
                q = ops.kv_append(qkv, layer.q_gain, layer.k_gain, self.cos, self.sin, pos, self.caches[i],
                                  cfg.n_heads, slot_map=slot_map, q_out=q_buf, status=self.status, ve=ve)
                if i == cfg.n_layers - 1 and not attend_last_layer:
                    return h  # prefill: the last layer only has to fill its cache (decode.cu:862)
                if grouped and plan is None:  # built while the GPU already runs the launches above
                    plan = ops.PrefillPlan(host_rows[0], host_rows[1], cfg.n_heads, self.caches[0], self.device)
                if plan is not None:
                    att = ops.prefill_attention(q, self.caches[i], plan, out=att_buf, status=self.status)
                else:
                    att = ops.decode_attention(q, self.caches[i], lens, max_kv_len, slot_map=slot_map,
                                               window=self.windows[i], chunk_pages=self.chunk_pages,
                                               workspace=workspace, out=att_buf, status=self.status)
            self.gemm_rows(att.view(rows, -1), layer.wo, resid=h)  # h += att . wo^T in the GEMM's epilogue
            check(lib.add_rms_norm(pointer(h), None, pointer(n), rows, C, s), "add_rms_norm")
            u = self.gemm_rows(n, layer.wup, epilogue=2, out=u_buf)
            nxt = layers[i + 1] if i + 1 < len(layers) else None
            if nxt is not None and nxt.mixes:  # the next layer's stream mix rides on this add
                y = self.gemm_rows(u, layer.wdown)
                check(lib.add_rms_norm_mix(pointer(h), pointer(y), pointer(x0), nxt.resid_lambda, nxt.x0_lambda,
                                           pointer(n), rows, C, s), "add_rms_norm_mix")
            else:
                self.gemm_rows(u, layer.wdown, resid=h)
                check(lib.add_rms_norm(pointer(h), None, pointer(n), rows, C, s), "add_rms_norm")
        return n

    def gemm_rows(self, x: Tensor, w: Tensor, epilogue: int = 0, resid: "Tensor | None" = None,
                  out: "Tensor | None" = None) -> Tensor:
        """epilogue(x . w^T) for a pass of any number of rows: x bf16 (rows, K), w bf16 (N, K); epilogue 0 store,
        2 relu^2, 3 fp32 output; resid (rows, N) bf16: resid += bf16(x . w^T) in place (epilogue 1), returned; out: a
        bf16 (rows, N) buffer to write into instead of a new tensor (the result is whatever is returned).
        This package's tiled tcgen05 GEMM (csrc/tile_gemm.cu) when N is a multiple of 128 and K of 64; other shapes
        (toy models) go to torch's GEMM with the same epilogue applied afterwards."""
        rows, K, N = x.shape[0], x.shape[1], w.shape[0]
        if resid is not None:
            assert epilogue == 0 and resid.is_contiguous() and resid.shape == (rows, N)
            epilogue = 1
        if self.use_tile_gemm and N % 128 == 0 and K % 64 == 0 and x.is_contiguous() and w.is_contiguous():
            y = resid if resid is not None else out if out is not None and epilogue != 3 else torch.empty(
                (rows, N), dtype=torch.float32 if epilogue == 3 else torch.bfloat16, device=x.device)
            check(cuda_library("tile_gemm").tile_gemm(pointer(x), pointer(w), None if resid is None else pointer(resid),
                                                      pointer(y), rows, N, K, epilogue, pointer(self.status), stream()),
                  "tile_gemm")
            return y
        if epilogue == 3:
            return torch.mm(x, w.T, out_dtype=torch.float32)
        y = x @ w.T
        if epilogue == 1:
            return resid.add_(y)
        if epilogue == 2:
            check(cuda_library("decode_step").relu2_inplace(pointer(y), y.numel(), stream()), "relu2_inplace")
        return y

    def _hidden_rows_torch(self, tokens: Tensor, pos: Tensor, slot_map: Tensor, max_kv_len: int,
                           attend_last_layer: bool = True) -> Tensor:
        """hidden_rows with torch operators around the append/attention kernels, for hidden sizes the norm kernels do
        not take (not a multiple of 8, above 4096)."""
        cfg = self.cfg
        rows = tokens.shape[0]
        lens = pos + 1
        workspace = self._workspace(rows, max_kv_len)
        h = x0 = rms_norm(self.w.embed[tokens])
        for i, layer in enumerate(self.w.layers):
            if layer.resid_lambda != 1.0 or layer.x0_lambda != 0.0:
                h = (layer.resid_lambda * h.float() + layer.x0_lambda * x0.float()).to(h.dtype)
            n = rms_norm(h)
            qkv = n @ layer.wqkv.T
            ve = None if layer.ve_table is None else ops.ValueEmbed(n.contiguous(), tokens, layer.ve_table, layer.ve_gate)
            q = ops.kv_append(qkv, layer.q_gain, layer.k_gain, self.cos, self.sin, pos, self.caches[i], cfg.n_heads,
                              slot_map=slot_map, status=self.status, ve=ve)
            if i == cfg.n_layers - 1 and not attend_last_layer:
                return h  # prefill: the last layer only has to fill its cache (decode.cu:862)
            att = ops.decode_attention(q, self.caches[i], lens, max_kv_len, slot_map=slot_map, window=self.windows[i],
                                       workspace=workspace, status=self.status)
            h = h + att.view(rows, -1) @ layer.wo.T
            h = h + F.relu(rms_norm(h) @ layer.wup.T).square() @ layer.wdown.T
        return rms_norm(h)

    def logits_rows(self, tokens: Tensor, pos: Tensor, slot_map: Tensor, max_kv_len: int) -> Tensor:
        """fp32 logits (rows, V): the bf16 head's GEMM accumulated and kept in fp32."""
        return self.head(self.hidden_rows(tokens, pos, slot_map, max_kv_len))

    def head(self, hidden: Tensor) -> Tensor:
        """The bf16 head GEMM with its fp32 accumulator kept as the output (modeling_nanochat.py:190-192)."""
        return self.gemm_rows(hidden.contiguous(), self.w.lm_head, epilogue=3)

    # ---- the same pass for at most 16 rows with this package's own GEMM kernels --------------------------------

    def gemm_kernel(self, rows: int) -> str | None:
        """Which of this package's GEMM kernels runs a decode step of `rows` rows: "skinny" (decode_step.cu) for at
        most 16 rows when it takes every GEMM of the model (skinny_gemm_supported: depths it is instantiated for, the
        fused norm up to a depth of 2048), else "stream" (the tcgen05 stream_gemm) up to 64 rows when every GEMM
        width is a multiple of 128 and every depth of 64; None: the row path (tile_gemm and separate norm kernels)."""
        cfg = self.cfg
        A = cfg.n_heads * HEAD_DIM
        if any(l.ve_table is not None and cfg.hidden % 256 for l in self.w.layers):
            return None
        ok = cuda_library("decode_step").skinny_gemm_supported
        # a layer with a value embedding norms its input in a launch of its own (the append reads the normed rows)
        qkv_norm = 0 if any(l.ve_table is not None for l in self.w.layers) else 1
        if (rows <= 16 and ok(rows, cfg.qkv_width, cfg.hidden, 1) and ok(rows, cfg.qkv_width, cfg.hidden, qkv_norm)
                and ok(rows, cfg.hidden, A, 0) and ok(rows, cfg.intermediate, cfg.hidden, 1)
                and ok(rows, cfg.hidden, cfg.intermediate, 0) and ok(rows, cfg.vocab, cfg.hidden, 1)):
            return "skinny"
        if (rows <= 64 and self.use_stream_gemm  # the kernel takes 256 rows; the tiled GEMM is faster above about 64
                and all(n % 128 == 0 for n in (cfg.hidden, cfg.intermediate, cfg.qkv_width, cfg.vocab))
                and all(k % 64 == 0 for k in (cfg.hidden, cfg.intermediate, A))):
            return "stream"
        return None

    def fused_supported(self, rows: int) -> bool:
        return self.gemm_kernel(rows) is not None

    def fused_buffers(self, rows: int) -> dict[str, Tensor]:
        cfg, dev, bf = self.cfg, self.device, torch.bfloat16
        return {"h": torch.empty((rows, cfg.hidden), dtype=bf, device=dev),
                "qkv": torch.empty((rows, cfg.qkv_width), dtype=bf, device=dev),
                "att": torch.empty((rows, cfg.n_heads, HEAD_DIM), dtype=bf, device=dev),
                "u": torch.empty((rows, cfg.intermediate), dtype=bf, device=dev),
                "x0": torch.empty((rows, cfg.hidden), dtype=bf, device=dev),
                "n": torch.empty((rows, cfg.hidden), dtype=bf, device=dev),
                "trace": torch.zeros((rows, self.capacity + 1), dtype=torch.long, device=dev),
                "logits": torch.empty((rows, cfg.vocab), dtype=torch.float32, device=dev)}

    def fused_step(self, tokens: Tensor, pos: Tensor, slot_map: Tensor, max_kv_len: int, buf: dict[str, Tensor],
                   choose: bool = True, slots: "list[int] | None" = None) -> Tensor:
        """One step on this package's kernels (GEMMs: see gemm_kernel): fp32 logits in buf["logits"]; with `choose`, tokens
        become the greedy choices and pos advances by one. 6 launches per layer: qkv GEMM (norm fused), split
        attention (append fused), merge, o GEMM + residual, up GEMM (norm fused) + relu^2, down GEMM + residual."""
        cfg, lib, s = self.cfg, cuda_library("decode_step"), stream()
        rows, C, Fd, A = tokens.shape[0], cfg.hidden, cfg.intermediate, cfg.n_heads * HEAD_DIM
        workspace = self._workspace(rows, max_kv_len)
        h, qkv, att, u = buf["h"], buf["qkv"], buf["att"], buf["u"]

        wide = cuda_library("stream_gemm") if self.gemm_kernel(rows) == "stream" else None

        def gemm(x, w, resid, y, n, k, norm, epilogue, then=None, mix=None):
            """`then`: the weights of the next GEMM on the stream, prefetched into L2 meanwhile (stream_gemm only).
            `mix` = (l1, l2): the residual epilogue is followed by the next layer's stream mix with buf["x0"]."""
            if wide is not None:
                then = then if self.prefetch_next else None
                tail = [pointer(then), 0 if then is None else then.numel() * 2, pointer(self.status), s]
                if mix is None:
                    check(wide.stream_gemm(pointer(x), pointer(w), pointer(resid), pointer(y), rows, n, k, norm, epilogue,
                                           0, *tail), "stream_gemm")
                else:
                    check(wide.stream_gemm_mix(pointer(x), pointer(w), pointer(resid), pointer(buf["x0"]), mix[0], mix[1],
                                               pointer(y), rows, n, k, norm, 0, *tail), "stream_gemm_mix")
            elif mix is None:
                check(lib.skinny_gemm(pointer(x), pointer(w), pointer(resid), pointer(y), rows, n, k, norm, epilogue,
                                      s), "skinny_gemm")
            else:
                check(lib.skinny_gemm_mix(pointer(x), pointer(w), pointer(resid), pointer(buf["x0"]), mix[0], mix[1],
                                          pointer(y), rows, n, k, norm, s), "skinny_gemm_mix")

        layers = self.w.layers
        if any(l.mixes for l in layers):
            check(lib.embed_norm_mix(pointer(self.w.embed), pointer(tokens), pointer(h), pointer(buf["x0"]),
                                     layers[0].resid_lambda, layers[0].x0_lambda, rows, C, cfg.vocab, s), "embed_norm_mix")
        else:
            check(lib.embed_norm(pointer(self.w.embed), pointer(tokens), pointer(h), rows, C, cfg.vocab, s), "embed_norm")
        for i, layer in enumerate(layers):
            ve = None
            if layer.ve_table is None:
                gemm(h, layer.wqkv, None, qkv, cfg.qkv_width, C, 1, 0, then=layer.wo)
            else:  # the value-embedding gate reads the normed rows, so they are written out once
                check(lib.add_rms_norm(pointer(h), None, pointer(buf["n"]), rows, C, s), "add_rms_norm")
                gemm(buf["n"], layer.wqkv, None, qkv, cfg.qkv_width, C, 0, 0, then=layer.wo)
                ve = ops.ValueEmbed(buf["n"], tokens, layer.ve_table, layer.ve_gate)
            ops.decode_step_attention(qkv, layer.q_gain, layer.k_gain, self.cos, self.sin, pos, self.caches[i],
                                      cfg.n_heads, max_kv_len, slot_map=slot_map, window=self.windows[i],
                                      chunk_pages=self.chunk_pages, workspace=workspace, out=att, status=self.status,
                                      slots=slots, ve=ve)
            gemm(att, layer.wo, h, h, C, A, 0, 1, then=layer.wup)
            gemm(h, layer.wup, None, u, Fd, C, 1, 2, then=layer.wdown)
            nxt = layers[i + 1] if i + 1 < len(layers) else None
            gemm(u, layer.wdown, h, h, C, Fd, 0, 1, then=nxt.wqkv if nxt is not None else None,
                 mix=(nxt.resid_lambda, nxt.x0_lambda) if nxt is not None and nxt.mixes else None)
        gemm(h, self.w.lm_head, None, buf["logits"], cfg.vocab, C, 1, 3)
        if choose:
            check(lib.greedy_choice(pointer(buf["logits"]), pointer(tokens), pointer(pos), rows, cfg.vocab,
                                    pointer(buf["trace"]), buf["trace"].shape[1], s), "greedy_choice")
        return buf["logits"]

    # ---- prefill ----------------------------------------------------------------------------------------------

    @torch.no_grad()
    def prefill(self, prompts: list[list[int]], slots: list[int], rows_per_pass: int = 4096) -> None:
        """Cache positions 0 .. len - 2 of every prompt (its last token is the first decode input). Sequences are
        processed in passes of at most rows_per_pass rows; a pass holds whole position ranges in order, so every row
        finds the earlier positions of its sequence either in the cache or earlier in its own pass."""
        import numpy as np

        counts = [len(p) - 1 for p in prompts]
        total = sum(counts)
        if total == 0:
            return
        # the rows of all passes as arrays (a prompt of thousands of tokens must not cost a Python loop per row)
        slot_rows = np.repeat(np.asarray(slots, dtype=np.int32), counts)
        pos_rows = np.concatenate([np.arange(n, dtype=np.int32) for n in counts])
        token_rows = np.concatenate([np.asarray(p[:-1], dtype=np.int64) for p in prompts])
        for at in range(0, total, rows_per_pass):
            part = slice(at, min(at + rows_per_pass, total))
            n = part.stop - part.start
            # tokens, positions and slots of the pass cross to the device in ONE copy
            packed = np.empty(2 * n, dtype=np.int64)
            packed[:n] = token_rows[part]
            packed[n:].view(np.int32)[:n] = pos_rows[part]
            packed[n:].view(np.int32)[n:] = slot_rows[part]
            dev = torch.from_numpy(packed).to(self.device, non_blocking=True)
            tokens, small = dev[:n], dev[n:].view(torch.int32)
            self.hidden_rows(tokens, small[:n], small[n:], int(pos_rows[part].max()) + 1, attend_last_layer=False,
                             host_rows=(slot_rows[part], pos_rows[part]))

    # ---- decode -----------------------------------------------------------------------------------------------

    def _step_graph(self, batch: int, sampled: bool = False, chunk_pages: int = 0, masked: bool = False):
        """The captured step for `batch` slots 0 .. batch - 1: tokens, pos (device) -> chosen tokens; pos += 1; every
        choice is logged at its position in a (batch, capacity + 1) trace. `sampled` steps choose by temperature /
        nucleus / Gumbel-max (sample_choice) from per-slot controls, the others take the argmax. `chunk_pages` is
        the attention chunk size baked into the graph (0: the library's choice for full-length slots). `masked`
        (sampled steps only) adds per-slot allowed-token bit masks, ctl["allow"] int32 (batch, vocab / 32), all ones
        until a caller writes a row."""
        key = (batch, sampled, chunk_pages, masked)
        if key in self._graphs:
            return self._graphs[key]
        self.chunk_pages = chunk_pages
        dev, lib, V = self.device, cuda_library("decode_step"), self.cfg.vocab
        tokens = torch.zeros(batch, dtype=torch.long, device=dev)
        pos = torch.zeros(batch, dtype=torch.int32, device=dev)
        slot_map = torch.arange(batch, dtype=torch.int32, device=dev)
        fused = self.use_fused and self.fused_supported(batch)
        buf = self.fused_buffers(batch) if fused else {
            "logits": torch.empty((batch, V), dtype=torch.float32, device=dev),
            "trace": torch.zeros((batch, self.capacity + 1), dtype=torch.long, device=dev)}
        logits, trace = buf["logits"], buf["trace"]
        ctl = None
        if sampled:
            assert V % 32 == 0, "sampling needs a vocabulary that is a multiple of 32"
            ctl = {"temperature": torch.zeros(batch, dtype=torch.float32, device=dev),
                   "top_p": torch.ones(batch, dtype=torch.float32, device=dev),
                   "seed": torch.zeros(batch, dtype=torch.long, device=dev),
                   "first": torch.zeros(batch, dtype=torch.int32, device=dev),
                   "probs": torch.empty((batch, V), dtype=torch.float32, device=dev)}
            if masked:
                ctl["allow"] = torch.full((batch, V // 32), -1, dtype=torch.int32, device=dev)

        def body():
            if fused:
                self.fused_step(tokens, pos, slot_map, self.capacity, buf, choose=False, slots=list(range(batch)))
            else:
                logits.copy_(self.head(self.hidden_rows(tokens, pos, slot_map, self.capacity, distinct_slots=True)))
            if sampled:
                check(lib.sample_choice(pointer(logits), pointer(ctl["probs"]), pointer(ctl["temperature"]),
                                        pointer(ctl["top_p"]), pointer(ctl["seed"]), pointer(ctl["first"]),
                                        pointer(ctl.get("allow")),
                                        self.softcap, pointer(tokens), pointer(pos), batch, V, pointer(trace),
                                        trace.shape[1], stream()), "sample_choice")
            else:
                check(lib.greedy_choice(pointer(logits), pointer(tokens), pointer(pos), batch, V, pointer(trace),
                                        trace.shape[1], stream()), "greedy_choice")

        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            # eager warm-up (first-use set-up has to happen outside capture) with every slot idle: a negative position
            # appends nothing, attends nothing and advances nothing, so caches that already hold sequences (decode_from
            # with a key not captured yet) are left as they are
            pos.fill_(-1)
            body()
            pos.zero_()
            tokens.zero_()
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with no_collection(), torch.cuda.graph(graph, stream=side):
                body()
        self.chunk_pages = 0
        # the graph holds raw pointers: every tensor its kernels touch must stay alive as long as the graph does
        self._graph_tensors[key] = (slot_map, buf, ctl)
        self._graphs[key] = (graph, side, tokens, pos, logits, trace, ctl)
        return self._graphs[key]

    def planned_chunk(self, positions: list[int], steps: int) -> int:
        """The attention chunk size for `steps` decode steps starting at these positions: the library's block-fill
        model on the lengths half way through the run (they change by one per step, the choice is baked into the
        captured step)."""
        lens = [min(p + 1 + steps // 2, self.capacity) for p in positions]
        return ops.plan_chunk_pages(lens, self.cfg.n_kv_heads, self.capacity)

    @torch.no_grad()
    def decode_from(self, first_tokens: list[int], positions: list[int], steps: int, temperature: float = 0.0,
                    top_p: float = 1.0, seeds: list[int] | None = None) -> tuple[list[list[int]], float]:
        """`steps` steps for slots 0 .. B - 1 whose caches already hold positions 0 .. positions[b] - 1: slot b's
        next input is first_tokens[b] at position positions[b]. Greedy at temperature 0, else sampled as the
        reference samples (capped logits / temperature, nucleus top_p, Gumbel-max noise keyed by seeds[b] and the
        step; the cap is the decoder's `softcap`). Returns the chosen tokens and the seconds the steps took on the
        device. Stream-ordered after work queued on the current stream."""
        B = len(first_tokens)
        assert B <= self.n_slots and max(positions) + steps <= self.capacity
        sampled = temperature > 0.0
        key = (B, sampled, self.planned_chunk(positions, steps), False)
        graph, side, tokens, pos, logits, trace, ctl = self._step_graph(*key)
        # The step's rows are the slots in descending order of length: the attention kernel's blocks start in row
        # order, and a ragged batch that starts with its longest sequences leaves the shortest tail of idle SMs.
        # (A row is computed from its own slot alone, so the order changes no result.)
        order = sorted(range(B), key=lambda b: (-positions[b], b))
        row_of = {b: r for r, b in enumerate(order)}
        slot_map = self._graph_tensors[key][0]
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            slot_map.copy_(torch.tensor(order, dtype=torch.int32))
            tokens.copy_(torch.tensor([first_tokens[b] for b in order], dtype=torch.long))
            pos.copy_(torch.tensor([positions[b] for b in order], dtype=torch.int32))
            first = pos.clone()
            if sampled:
                seeds = seeds if seeds is not None else list(range(B))
                ctl["temperature"].fill_(temperature)
                ctl["top_p"].fill_(top_p)
                ctl["seed"].copy_(torch.tensor([seeds[b] for b in order], dtype=torch.long))
                ctl["first"].copy_(first)
            begin.record()
            for _ in range(steps):
                graph.replay()
            end.record()
            at = first.long()[:, None] + 1 + torch.arange(steps, device=self.device)[None, :]
            out = trace.gather(1, at)  # every choice was logged at its position: one gather at the end
        side.synchronize()
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"device status {code:#x} (NCB_DEV_* bits)")
        rows = out.tolist()
        return [rows[row_of[b]] for b in range(B)], begin.elapsed_time(end) * 1e-3

    @torch.no_grad()
    def generate(self, prompts: list[list[int]], max_new_tokens: int, temperature: float = 0.0, top_p: float = 1.0,
                 seeds: list[int] | None = None) -> tuple[list[list[int]], dict]:
        """Continuation of every prompt (slot b = prompt b), greedy or sampled (see decode_from). Returns the new
        tokens and timings: prefill seconds, decode seconds (the max_new_tokens steps), tokens per second of the
        decode phase."""
        B = len(prompts)
        assert B <= self.n_slots and all(len(p) >= 1 for p in prompts)
        assert max(len(p) for p in prompts) - 1 + max_new_tokens <= self.capacity
        # capture (and its warm-up step) before the caches are filled
        self._step_graph(B, temperature > 0.0, self.planned_chunk([len(p) - 1 for p in prompts], max_new_tokens))
        start, mid = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        missing = [b for b in range(B) if self.store is None or not self.store.load(b, prompts[b])]
        self.prefill([prompts[b] for b in missing], missing)
        if self.store is not None:
            for b in missing:
                self.store.save(b, prompts[b])
        mid.record()
        out, decode_s = self.decode_from([p[-1] for p in prompts], [len(p) - 1 for p in prompts], max_new_tokens,
                                         temperature, top_p, seeds)
        return out, {"prefill_s": start.elapsed_time(mid) * 1e-3, "decode_s": decode_s,
                     "tokens_per_s": B * max_new_tokens / decode_s}
