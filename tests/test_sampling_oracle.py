"""The sampling checker's Philox4x32-10 against the function's published known-answer vectors (Random123's
kat_vectors: counter and key all zeros, all ones, and the digits of pi), and sanity of the choice rule."""

import numpy as np

from oracle import sampling


def test_philox_known_answers():
    cases = [
        ((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
        ((0xffffffff,) * 4, (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
        ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
         (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)),
    ]
    for counter, key, want in cases:
        got = sampling.philox4x32_10(np.array([counter], dtype=np.uint32), key)[0]
        assert tuple(int(x) for x in got) == want


def test_choice_rule():
    rng = np.random.default_rng(0)
    logits = rng.normal(size=256).astype(np.float32) * 3
    assert sampling.choose(logits, 0.0, 1.0, 1, 0)["token"] == int(logits.argmax())
    allow = np.zeros(256, bool)
    allow[[5, 77]] = True
    assert sampling.choose(logits, 0.0, 1.0, 1, 0, allow=allow)["token"] in (5, 77)
    # the nucleus keeps the head of the distribution with at least top_p of the mass and drops the rest
    out = sampling.choose(logits, 1.0, 0.5, 7, 3)
    p = np.exp(logits - logits.max())
    p /= p.sum()
    kept = out["kept"]
    assert p[kept].sum() >= 0.5 and p[kept].min() >= p[~kept].max()
    assert p[kept].sum() - p[kept].min() < 0.5  # minimal: without its smallest member it falls below top_p
    assert kept[out["token"]]
    # different steps draw different noise, the same step the same
    a = [sampling.choose(logits, 1.0, 1.0, 7, s)["token"] for s in range(50)]
    assert len(set(a)) > 5 and a == [sampling.choose(logits, 1.0, 1.0, 7, s)["token"] for s in range(50)]
