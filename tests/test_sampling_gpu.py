"""sample_choice on the GPU through the C ABI against the numpy restatement of the reference's choice rule."""

import numpy as np
import pytest
import torch

from nanochat_b200.native import cuda_library, pointer, stream
from oracle import sampling

pytestmark = pytest.mark.gpu


def run(logits, temperature, top_p, seed, pos, first, softcap=0.0, allow=None):
    rows, V = logits.shape
    dev = "cuda"
    lg = torch.from_numpy(logits).to(dev)
    probs = torch.empty_like(lg)
    T = torch.tensor(temperature, dtype=torch.float32, device=dev)
    P = torch.tensor(top_p, dtype=torch.float32, device=dev)
    S = torch.from_numpy(np.array(seed, dtype=np.uint64).view(np.int64)).to(dev)
    F = torch.tensor(first, dtype=torch.int32, device=dev)
    pos_t = torch.tensor(pos, dtype=torch.int32, device=dev)
    tokens = torch.zeros(rows, dtype=torch.long, device=dev)
    trace = torch.full((rows, 64), -7, dtype=torch.long, device=dev)
    A = None
    if allow is not None:
        bits = allow.reshape(rows, V // 32, 32).astype(np.uint64)  # bit r % 32 of word r / 32
        words = (bits << np.arange(32, dtype=np.uint64)).sum(-1).astype(np.uint32)
        A = torch.from_numpy(words.view(np.int32).copy()).to(dev)
    rc = cuda_library("decode_step").sample_choice(pointer(lg), pointer(probs), pointer(T), pointer(P), pointer(S),
                                                   pointer(F), pointer(A), softcap, pointer(tokens), pointer(pos_t),
                                                   rows, V, pointer(trace), 64, stream())
    assert rc == 0
    torch.cuda.synchronize()
    return tokens.cpu().numpy(), pos_t.cpu().numpy(), trace.cpu().numpy()


def agrees(got, ref, tol=2e-5):
    """The kernel's choice is the checker's, or a near-tie of it (tanh/log round differently on the two machines)."""
    if got == ref["token"]:
        return True
    keys = ref["keys"]
    return got >= 0 and np.isfinite(keys[got]) and keys[ref["token"]] - keys[got] < tol


def test_argmax_temperature_sampling_and_cap():
    rng = np.random.default_rng(1)
    rows, V = 12, 4096
    logits = (rng.normal(size=(rows, V)) * 4).astype(np.float32)
    logits[3, 100] = logits[3, 2000] = 99.0  # a tie at temperature 0: the lowest id
    temperature = [0.0, 0.0, 1.0, 0.0, 0.7, 1.0, 1.3, 1.0, 0.5, 2.0, 1.0, 1.0]
    seeds = [int(x) for x in rng.integers(0, 2 ** 63, rows)]
    pos, first = list(range(10, 10 + rows)), [7] * rows
    for softcap in (0.0, 15.0):
        tokens, new_pos, trace = run(logits, temperature, [1.0] * rows, seeds, pos, first, softcap)
        assert tokens[3] == 100
        for b in range(rows):
            ref = sampling.choose(logits[b], temperature[b], 1.0, seeds[b], pos[b] - first[b], softcap)
            assert agrees(int(tokens[b]), ref), (b, int(tokens[b]), ref["token"])
            assert new_pos[b] == pos[b] + 1 and trace[b, pos[b] + 1] == tokens[b]


def test_nucleus_and_mask():
    rng = np.random.default_rng(2)
    rows, V = 16, 2048
    logits = (rng.normal(size=(rows, V)) * 2).astype(np.float32)
    top_p = [0.9, 0.5, 0.1, 0.99, 0.3, 0.7, 0.95, 0.2] * 2
    seeds = [int(x) for x in rng.integers(0, 2 ** 63, rows)]
    allow = rng.random((rows, V)) < 0.3
    allow[5] = False
    allow[5, 1234] = True   # a single allowed token
    allow[6] = False        # nothing allowed
    for mask in (None, allow):
        for step in (0, 5):
            tokens, _, trace = run(logits, [1.0] * rows, top_p, seeds, [20 + step] * rows, [20] * rows, 0.0, mask)
            for b in range(rows):
                ref = sampling.choose(logits[b], 1.0, top_p[b], seeds[b], step, 0.0, None if mask is None else mask[b])
                if ref["token"] < 0:
                    assert trace[b, 21 + step] == -1
                    continue
                got = int(tokens[b])
                if mask is not None:
                    assert mask[b, got]
                # inside the checker's nucleus, up to fp32 summation order at the boundary
                assert ref["e"][got] >= ref["least"] * (1 - 1e-4), (b, got)
                borderline = abs(ref["e"][ref["token"]] - ref["least"]) <= 1e-4 * ref["least"]
                assert agrees(got, ref) or borderline, (b, got, ref["token"])
            if mask is not None:
                assert tokens[5] == 1234


def test_sampled_frequencies_follow_the_softmax():
    """4096 rows with the same logits and different seeds: token frequencies match softmax(z / T) over the nucleus."""
    rng = np.random.default_rng(3)
    V, rows, T, top_p = 64, 4096, 0.8, 0.9
    z = (rng.normal(size=V) * 1.5).astype(np.float32)
    logits = np.tile(z, (rows, 1))
    seeds = [int(x) for x in rng.integers(0, 2 ** 63, rows)]
    tokens, _, _ = run(logits, [T] * rows, [top_p] * rows, seeds, [3] * rows, [0] * rows)
    ref = sampling.choose(z, T, top_p, 1, 0)
    p = np.where(ref["kept"], np.exp(z / T - (z / T).max()), 0.0)
    p /= p.sum()
    freq = np.bincount(tokens, minlength=V) / rows
    assert freq[~ref["kept"]].sum() == 0
    assert np.abs(freq - p).max() < 4 * np.sqrt(p.max() / rows) + 1e-3
