"""The CPU decoder restatement (fp8 KV cache) against logits produced by the reference's own exported model
(bf16 KV cache) on a tiny random-init configuration: tests/golden/decoder_vectors.npz."""

import hashlib
from pathlib import Path

import numpy as np
import torch

from oracle.decoder import OracleDecoder
from tests import helpers

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "decoder_vectors.npz")
GOLDEN_VE = np.load(Path(__file__).resolve().parent / "golden" / "decoder_ve_vectors.npz")


def uncapped(logits: np.ndarray, cap: float) -> np.ndarray:
    """Invert the reference's c tanh(z / c)."""
    return cap * np.arctanh(np.clip(logits / cap, -0.999999, 0.999999))


def teacher_forced_logits(step, golden=GOLDEN):
    """Feed the golden run's tokens: the 12-token prompt one position at a time, then the 6 generated tokens.
    Returns logits (2, 7, V) at the last prompt position and after each generated token."""
    prompt, tokens = torch.from_numpy(golden["prompt"]), torch.from_numpy(golden["tokens"])
    feed = torch.cat([prompt, tokens], dim=1)  # (2, 18)
    keep = []
    for t in range(feed.shape[1]):
        logits = step(feed[:, t])
        if t >= prompt.shape[1] - 1:
            keep.append(logits)
    return torch.stack(keep, 1).numpy()


def test_weights_match_the_golden_run():
    _, w = helpers.tiny_decoder_weights()
    digest = hashlib.sha256()
    for t in [w["embed"], w["lm_head"]] + [lw[k] for lw in w["layers"] for k in sorted(lw)]:
        digest.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    assert np.array_equal(np.frombuffer(digest.digest(), dtype=np.uint8), GOLDEN["weights_sha256"])


def test_oracle_decoder_tracks_the_reference_model():
    cfg, w = helpers.tiny_decoder_weights()
    dec = OracleDecoder(cfg, w, n_seqs=2)
    got = teacher_forced_logits(lambda tok: dec.step(tok, [0, 1]))
    want = uncapped(GOLDEN["logits"], float(GOLDEN["softcap"]))
    err = np.abs(got - want)
    # logits have std 0.32; the fp8 cache moves them by a few 1e-3
    assert err.max() < 2e-2 and err.mean() < 3e-3, (err.max(), err.mean())
    # greedy choices agree wherever the reference's top-2 margin exceeds the error
    top2 = np.sort(want, -1)[..., -2:]
    clear = (top2[..., 1] - top2[..., 0]) > 4e-2
    assert clear.sum() >= 8
    assert (got.argmax(-1) == want.argmax(-1))[clear].all()


def test_oracle_decoder_with_value_embedding_and_stream_mix_tracks_the_reference_model():
    """The reference's own model shape: a value-embedding layer (gate 2 sigmoid(W n), v + gate ve) and per-layer
    resid / x0 lambdas away from (1, 0), against logits of the reference's exported model with the same weights."""
    cfg, w = helpers.tiny_decoder_weights_ve()
    digest = hashlib.sha256()
    for t in [w["embed"], w["lm_head"]] + [lw[k] for lw in w["layers"] for k in sorted(lw) if isinstance(lw[k], torch.Tensor)]:
        digest.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    assert np.array_equal(np.frombuffer(digest.digest(), dtype=np.uint8), GOLDEN_VE["weights_sha256"])
    dec = OracleDecoder(cfg, w, n_seqs=2)
    got = teacher_forced_logits(lambda tok: dec.step(tok, [0, 1]), GOLDEN_VE)
    want = uncapped(GOLDEN_VE["logits"], float(GOLDEN_VE["softcap"]))
    err = np.abs(got - want)
    assert err.max() < 2e-2 and err.mean() < 3e-3, (err.max(), err.mean())
    # the mix matters: without the value embedding and the lambdas the logits are far off
    plain = {**w, "layers": [{k: v for k, v in lw.items() if k not in ("ve_table", "ve_gate", "resid_lambda", "x0_lambda")}
                             for lw in w["layers"]]}
    off = np.abs(teacher_forced_logits(lambda tok, d=OracleDecoder(cfg, plain, n_seqs=2): d.step(tok, [0, 1]), GOLDEN_VE) - want)
    assert off.mean() > 10 * err.mean()

