"""Continuous batching over the captured decode step: requests in, (index, generated ids) out in completion order.

The host loop of the reference's NativeDecoder.generate (inference/decoder.py:28-40 Request, :112-121 Slot,
:250-324 the loop) over this package's step graph: every slot of the decoder runs one request; a slot whose request
finishes (its token limit, the BOS/EOS token, or its stopping criteria) takes the next request from the queue, or
idles. An idle slot has position -1, which every kernel of the step skips silently (the reference idles slots on an
`active` bit mask, model/kernels/decode.cu:60-62,555,573), so ONE captured graph serves a batch whose slots finish
at different times. As in the reference there is one synchronisation per step (the chosen tokens, decode.cu:1120-
1124), stopping criteria of the previous token are evaluated while the GPU runs the next step, and a stopped slot's
next token is dropped (inference/decoder.py:287-289).

The loop itself (`run_requests`) only talks to a small backend (start / idle / prefill / launch / tokens / mask), so
it is tested on the CPU against a scripted backend; `NativeDecoder` is the backend over `Decoder`.

Constraints: any object with mask() -> uint32 words (bit t % 32 of word t // 32 set iff token t is allowed, the
reference's layout, inference/decoder.py:75-76) or None, and push(token). The reference's syntax engine (Rust) is
not part of this package; its product, the allowed-token mask, is what sample_choice consumes."""

import time
from collections.abc import Callable, Iterable, Iterator
from dataclasses import dataclass, field
from typing import Protocol

import numpy as np
import torch

from .decoder import Decoder


class Constraint(Protocol):
    def mask(self) -> "np.ndarray | None": ...

    def push(self, token: int) -> None: ...


def never(_: list[int]) -> bool:
    return False


@dataclass(frozen=True, kw_only=True)
class Request:
    """A continuation of input_ids (at least one token) by at most max_new_tokens (>= 1) tokens, within the
    constraint's masks, until stopping_criteria holds or the end token is chosen. temperature 0: argmax (ties to the
    lowest id); > 0: a sample drawn from (seed, generated position) alone; top_p < 1: nucleus sampling. Same fields
    as the reference's Request (inference/decoder.py:28-40)."""
    input_ids: list[int]
    max_new_tokens: int
    stopping_criteria: Callable[[list[int]], bool] = never
    constraint: "Constraint | None" = None
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0


@dataclass
class Slot:
    """A request in a slot: its index, the request, host times of its start and first token, the tokens so far."""
    index: int
    request: Request
    start: float
    first: float | None = None
    out: list[int] = field(default_factory=list)


class Backend(Protocol):
    batch: int

    def start(self, b: int, request: Request) -> None: ...      # slot b begins at the prompt's last token

    def idle(self, b: int) -> None: ...                         # slot b runs nothing from the next step on

    def prefill(self) -> None: ...                              # cache the started prompts (all but the last token)

    def set_mask(self, b: int, mask: "np.ndarray | None") -> None: ...

    def launch(self) -> None: ...                               # one step for every slot, asynchronous

    def tokens(self) -> list[int]: ...                          # the step's choices (synchronises); -1: none allowed


def run_requests(backend: Backend, requests: Iterable[Request], end_token: int,
                 timings: dict[int, tuple[float, float, float]]) -> Iterator[tuple[int, list[int]]]:
    """The continuous-batching loop. Yields (request index, generated ids) in completion order; fills `timings`
    with {index: (start, first token, end)} host times. Raises ValueError when a constraint allows no token."""
    B = backend.batch
    queue = enumerate(requests)
    slots: list[Slot | None] = [None] * B
    stopping: list[int] = []  # slots whose last token awaits its stopping criteria

    def fill(b: int) -> None:
        for i, request in queue:
            backend.start(b, request)
            slots[b] = Slot(i, request, start=time.perf_counter())
            return
        slots[b] = None
        backend.idle(b)

    for b in range(B):
        fill(b)
    while any(s is not None for s in slots):
        backend.prefill()
        active = [b for b, s in enumerate(slots) if s is not None]
        for b in active:  # this step's masks; constraints advance with every accepted token
            c = slots[b].request.constraint
            mask = c.mask() if c is not None else None
            if mask is not None and not mask.any():
                raise ValueError(f"request {slots[b].index}: its constraint allows no token at position "
                                 f"{len(slots[b].out)}")
            backend.set_mask(b, mask)
        backend.launch()
        # meanwhile: the stopping criteria of the tokens accepted last step; a stopped slot's next token is dropped
        finished = sorted(b for b in stopping if slots[b].request.stopping_criteria(slots[b].out))
        stopping = []
        chosen = backend.tokens()
        now = time.perf_counter()
        for b in active:
            if b in finished:
                continue
            s, token = slots[b], int(chosen[b])
            if token < 0:
                raise ValueError(f"request {s.index}: its constraint allows no token at position {len(s.out)}")
            if token == end_token:
                finished.append(b)
                continue
            if not s.out:
                s.first = now
            s.out.append(token)
            if s.request.constraint is not None:
                s.request.constraint.push(token)
            if len(s.out) == s.request.max_new_tokens:
                finished.append(b)
            else:
                stopping.append(b)
        for b in finished:
            done = slots[b]
            fill(b)
            timings[done.index] = (done.start, now if done.first is None else done.first, now)
            yield done.index, done.out


class NativeDecoder:
    """Continuous batching over `decoder`'s slots (its n_slots is the batch). A request's tokens depend on neither
    the other requests in the batch nor the slot it lands in: rows of a step never mix (each GEMM row, each attention
    sequence and each choice is computed from that row alone, in an order fixed by the decoder's shape), which the
    GPU tests check bit for bit. end_token: the token that ends a continuation without being emitted (the
    reference's BOS, inference/decoder.py:305-307)."""

    def __init__(self, decoder: Decoder, *, end_token: int):
        self.decoder, self.end_token, self.batch = decoder, end_token, decoder.n_slots
        self.timings: dict[int, tuple[float, float, float]] = {}
        self.pending: list[tuple[int, list[int]]] = []  # started slots whose prompts await prefill
        dev, V = decoder.device, decoder.cfg.vocab
        assert V % 32 == 0, "the allowed-token masks need a vocabulary that is a multiple of 32"
        # the sampled step serves greedy rows too (temperature 0 takes the argmax)
        graph, side, tokens, pos, logits, trace, ctl = decoder._step_graph(self.batch, True, 0, masked=True)
        self.graph, self.side, self.dev_tokens, self.dev_pos, self.ctl = graph, side, tokens, pos, ctl
        self.host_tokens = torch.zeros(self.batch, dtype=torch.long).pin_memory()
        self.host_status = torch.zeros(1, dtype=torch.int32).pin_memory()  # travels with the tokens: no second sync
        self.masked = [False] * self.batch
        with torch.cuda.stream(side):
            pos.fill_(-1)
            ctl["allow"].fill_(-1)
        side.synchronize()

    # ---- the loop's backend ----------------------------------------------------------------------------------

    def start(self, b: int, request: Request) -> None:
        n = len(request.input_ids) - 1  # the positions before the prompt's last token
        if request.max_new_tokens < 1:
            raise ValueError(f"max_new_tokens {request.max_new_tokens} < 1")
        if n < 0 or n + request.max_new_tokens > self.decoder.capacity:
            raise ValueError(f"{n + 1} prompt and {request.max_new_tokens} new tokens need {n + request.max_new_tokens} "
                             f"positions, the cache holds {self.decoder.capacity}")
        store = self.decoder.store
        with torch.cuda.stream(self.side):  # everything of this decoder is ordered on its own stream
            if store is None or not store.load(b, request.input_ids):
                self.pending.append((b, request.input_ids))
            self.dev_tokens[b:b + 1].fill_(request.input_ids[-1])
            self.dev_pos[b:b + 1].fill_(n)
            self.ctl["first"][b:b + 1].fill_(n)
            self.ctl["temperature"][b:b + 1].fill_(request.temperature)
            self.ctl["top_p"][b:b + 1].fill_(request.top_p)
            self.ctl["seed"][b:b + 1].fill_(request.seed)

    def idle(self, b: int) -> None:
        with torch.cuda.stream(self.side):
            self.dev_pos[b:b + 1].fill_(-1)

    def prefill(self) -> None:
        if not self.pending:
            return
        with torch.cuda.stream(self.side):
            self.decoder.prefill([ids for _, ids in self.pending], [b for b, _ in self.pending])
            if self.decoder.store is not None:
                for b, ids in self.pending:
                    self.decoder.store.save(b, ids)
        self.pending = []

    def set_mask(self, b: int, mask: "np.ndarray | None") -> None:
        if mask is None and not self.masked[b]:
            return
        with torch.cuda.stream(self.side):
            if mask is None:
                self.ctl["allow"][b].fill_(-1)
            else:
                words = torch.from_numpy(np.ascontiguousarray(mask, dtype=np.uint32).view(np.int32))
                self.ctl["allow"][b].copy_(words)
        self.masked[b] = mask is not None

    def launch(self) -> None:
        with torch.cuda.stream(self.side):
            self.graph.replay()
            self.host_tokens.copy_(self.dev_tokens, non_blocking=True)
            self.host_status.copy_(self.decoder.status, non_blocking=True)

    def tokens(self) -> list[int]:
        self.side.synchronize()
        code = int(self.host_status[0])
        if code:
            raise RuntimeError(f"device status {code:#x} (NCB_DEV_* bits)")
        return self.host_tokens.tolist()

    # ---- the public call ---------------------------------------------------------------------------------------

    @torch.no_grad()
    def generate(self, requests: Iterable[Request]) -> Iterator[tuple[int, list[int]]]:
        """Continuations of `requests`, consumed lazily; yields (request index, generated ids) in completion order.
        Sets timings: {request index: (start, first token, end)}, host time.perf_counter seconds."""
        self.timings = {}
        self.side.wait_stream(torch.cuda.current_stream(self.decoder.device))
        yield from run_requests(self, requests, self.end_token, self.timings)
