"""The continuous-batching loop (nanochat_b200/serving.py run_requests) against a scripted backend: no GPU. The
backend plays a 'model' whose next token is a fixed function of the slot's request, so every expectation below can
be read off the requests."""

import numpy as np
import pytest

from nanochat_b200.serving import Request, run_requests

END = 13


class ScriptedBackend:
    """Slot b running request r emits r.input_ids[0] + k as its k-th token (k = 1, 2, ...), masked to the allowed
    set if a mask is given (the lowest allowed token >= the scripted one, else -1)."""

    def __init__(self, batch):
        self.batch, self.log = batch, []
        self.running = [None] * batch  # [request, tokens emitted]
        self.masks = [None] * batch
        self.pending = []

    def start(self, b, request):
        self.running[b] = [request, 0]
        self.pending.append(b)
        self.log.append(("start", b, tuple(request.input_ids)))

    def idle(self, b):
        self.running[b] = None
        self.log.append(("idle", b))

    def prefill(self):
        if self.pending:
            self.log.append(("prefill", tuple(self.pending)))
        self.pending = []

    def set_mask(self, b, mask):
        self.masks[b] = mask

    def launch(self):
        assert not self.pending, "a step was launched before its prompts were prefilled"
        self.step = []
        for b, run in enumerate(self.running):
            if run is None:
                self.step.append(-7)  # an idle slot's token is never looked at
                continue
            run[1] += 1
            token = run[0].input_ids[0] + run[1]
            mask = self.masks[b]
            if mask is not None:
                allowed = np.flatnonzero(np.unpackbits(mask.view(np.uint8), bitorder="little"))
                later = allowed[allowed >= token]
                token = int(later[0]) if len(later) else -1
            self.step.append(token)

    def tokens(self):
        return self.step


def collect(batch, requests):
    backend, timings = ScriptedBackend(batch), {}
    done = list(run_requests(backend, requests, END, timings))
    return backend, timings, done


def test_slots_refill_in_queue_order_and_results_come_in_completion_order():
    requests = [Request(input_ids=[100, 5], max_new_tokens=3), Request(input_ids=[200], max_new_tokens=1),
                Request(input_ids=[300, 1, 2], max_new_tokens=2), Request(input_ids=[400], max_new_tokens=4)]
    backend, timings, done = collect(2, requests)
    assert done == [(1, [201]), (0, [101, 102, 103]), (2, [301, 302]), (3, [401, 402, 403, 404])]
    starts = [e for e in backend.log if e[0] == "start"]
    assert starts == [("start", 0, (100, 5)), ("start", 1, (200,)), ("start", 1, (300, 1, 2)), ("start", 0, (400,))]
    assert backend.log[-1][0] == "idle" and sorted(e[1] for e in backend.log if e[0] == "idle") == [0, 1]
    assert set(timings) == {0, 1, 2, 3} and all(s <= f <= e for s, f, e in timings.values())


def test_end_token_stops_without_being_emitted_and_stopping_criteria_drop_the_next_token():
    ends = Request(input_ids=[10], max_new_tokens=10)  # emits 11, 12, then 13 = END
    stops = Request(input_ids=[20], max_new_tokens=10, stopping_criteria=lambda out: out[-1] == 22)
    _, _, done = collect(2, [ends, stops])
    assert dict(done) == {0: [11, 12], 1: [21, 22]}  # 23 was computed while the criteria ran and is dropped


def test_masks_follow_the_constraint_and_an_empty_mask_raises():
    class Evens:
        def __init__(self, empty_after=None):
            self.seen, self.empty_after = [], empty_after

        def mask(self):
            allowed = np.zeros(64, dtype=bool)
            if self.empty_after is None or len(self.seen) < self.empty_after:
                allowed[::2] = True
            return np.packbits(allowed, bitorder="little").view("<u4")

        def push(self, token):
            self.seen.append(token)

    c = Evens()
    _, _, done = collect(1, [Request(input_ids=[13], max_new_tokens=3, constraint=c)])
    assert done == [(0, [14, 16, 16])] and c.seen == [14, 16, 16]
    with pytest.raises(ValueError, match="allows no token"):
        collect(1, [Request(input_ids=[13], max_new_tokens=3, constraint=Evens(empty_after=1))])


def test_more_slots_than_requests_idles_the_rest_and_an_empty_queue_yields_nothing():
    backend, _, done = collect(4, [Request(input_ids=[50], max_new_tokens=2)])
    assert done == [(0, [51, 52])]
    assert [e for e in backend.log if e[0] == "idle"][:3] == [("idle", 1), ("idle", 2), ("idle", 3)]
    assert collect(3, [])[2] == []
