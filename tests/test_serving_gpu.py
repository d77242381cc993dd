"""NativeDecoder (continuous batching over the captured step with idle slots) on the GPU."""

import numpy as np
import pytest
import torch

from nanochat_b200.decoder import Decoder, DecoderConfig, DecoderWeights
from nanochat_b200.serving import NativeDecoder, Request

pytestmark = pytest.mark.gpu
V = 320


def make(n_slots=4, store=0):
    cfg = DecoderConfig(n_layers=2, hidden=512, n_heads=4, n_kv_heads=2, intermediate=1024, vocab=V, max_len=192)
    w = DecoderWeights.random_init(cfg, seed=31, device="cuda", std=0.05)
    return NativeDecoder(Decoder(cfg, w, n_slots, prompt_store=store), end_token=V - 1)


def prompt(seed, n):
    return torch.randint(0, V - 1, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_a_requests_tokens_do_not_depend_on_the_batch_or_the_slot():
    """The reference's claim (inference/decoder.py:124-125): request X alone, and X queued behind short requests that
    take the first slots, finish at different times and are replaced while X runs. Bit-identical streams, greedy and
    sampled. (The other prompts have one token, hence no prefill rows: X's prefill pass is the same rows both times.)"""
    for temperature in (0.0, 0.8):
        x = Request(input_ids=prompt(1, 70), max_new_tokens=24, temperature=temperature, top_p=0.9, seed=5)
        alone = dict(make().generate([x]))[0]
        others = [Request(input_ids=prompt(10 + i, 1), max_new_tokens=1 + 3 * i, temperature=temperature, seed=i)
                  for i in range(7)]
        nd = make()
        mixed = dict(nd.generate(others[:2] + [x] + others[2:]))
        assert mixed[2] == alone and len(alone) >= 1
        assert set(mixed) == set(range(8)) and set(nd.timings) == set(range(8))
        for i, r in enumerate(others[:2] + [x] + others[2:]):
            assert 0 < len(mixed[i]) <= r.max_new_tokens or (len(mixed[i]) == 0)  # an immediate end token gives []


def test_more_requests_than_slots_match_one_request_at_a_time():
    """Eight requests of different prompt lengths through two slots against each request run alone in a one-request
    batch of the same decoder shape: the same streams, token for token. Prefill passes hold different rows in the two
    runs, but every kernel of a pass computes a row from that row alone in an order fixed by the shapes (the tiled
    GEMM accumulates a row's k-blocks in the same order wherever the row lands, the prefill attention's warps never
    mix their query slots), so a prompt's cache bytes do not depend on what else is in the pass."""
    reqs = [Request(input_ids=prompt(40 + i, n), max_new_tokens=6 + i) for i, n in enumerate((3, 65, 17, 1, 130, 64, 9, 33))]
    nd = make(2)
    together = dict(nd.generate(reqs))
    for i, r in enumerate(reqs):
        alone = dict(make(2).generate([r]))[0]
        assert alone == together[i], (i, alone, together[i])


def test_stopping_criteria_token_limits_and_masks():
    class Only:
        """Allows the tokens of a fixed set."""

        def __init__(self, allowed):
            bits = np.zeros(V, dtype=bool)
            bits[list(allowed)] = True
            self.words, self.seen = np.packbits(bits, bitorder="little").view("<u4"), []

        def mask(self):
            return self.words

        def push(self, token):
            self.seen.append(token)

    allowed = {7, 8, 200, 311}
    c = Only(allowed)
    reqs = [Request(input_ids=prompt(60, 12), max_new_tokens=9, constraint=c),
            Request(input_ids=prompt(61, 5), max_new_tokens=30, stopping_criteria=lambda out: len(out) >= 4),
            Request(input_ids=prompt(62, 2), max_new_tokens=2, temperature=1.0, seed=3)]
    out = dict(make(3).generate(reqs))
    assert len(out[0]) == 9 and set(out[0]) <= allowed and c.seen == out[0]
    assert len(out[1]) == 4
    assert len(out[2]) <= 2
    free = dict(make(3).generate([Request(input_ids=prompt(60, 12), max_new_tokens=9)]))[0]
    assert not set(free) <= allowed  # the mask did change the stream


def test_invalid_requests_are_refused_before_anything_runs():
    nd = make(2)
    with pytest.raises(ValueError):
        list(nd.generate([Request(input_ids=prompt(70, 4), max_new_tokens=0)]))
    with pytest.raises(ValueError):
        list(make(2).generate([Request(input_ids=prompt(71, 100), max_new_tokens=100)]))  # 99 + 100 > 192 positions


def test_prompts_seen_before_come_from_the_prompt_store():
    """The same prompt in several requests is prefilled once; later requests copy its pages from pinned host memory
    into whatever slot they land in and produce the same stream (inference/decoder.py:193-232)."""
    nd = make(2, store=512)
    p = prompt(80, 70)
    calls = []
    original = nd.decoder.prefill
    nd.decoder.prefill = lambda prompts, slots, **kw: (calls.append(len(prompts)), original(prompts, slots, **kw))
    reqs = [Request(input_ids=p, max_new_tokens=5), Request(input_ids=prompt(81, 3), max_new_tokens=2),
            Request(input_ids=p, max_new_tokens=5), Request(input_ids=p, max_new_tokens=5)]
    out = dict(nd.generate(reqs))
    assert out[0] == out[2] == out[3] and len(out[0]) >= 1
    assert sum(calls) == 2  # the long prompt once, the short one once
