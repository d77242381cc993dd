"""TEST INFRASTRUCTURE: numpy restatement of the reference's sampled token choice (model/kernels/decode.cu:90-120
choice keys and Gumbel noise from Philox4x32-10, :195-203 temperature and logit cap, :364-411 nucleus as
transformers' TopPLogitsWarper). The Philox function is the published one (Salmon et al., SC '11), pinned by its
known-answer vectors in tests/test_sampling_oracle.py; the reference has no test vectors of its own for sampling."""

import numpy as np

M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
MASK = 0xFFFFFFFF


def philox4x32_10(counter: np.ndarray, key: tuple[int, int]) -> np.ndarray:
    """counter uint32 (..., 4) -> uint32 (..., 4)."""
    c = counter.astype(np.uint64)
    k0, k1 = key
    for _ in range(10):
        p0, p1 = M0 * c[..., 0], M1 * c[..., 2]
        hi0, lo0, hi1, lo1 = p0 >> 32, p0 & MASK, p1 >> 32, p1 & MASK
        c = np.stack([hi1 ^ c[..., 1] ^ k0, lo1, hi0 ^ c[..., 3] ^ k1, lo0], axis=-1)
        k0, k1 = (k0 + W0) & MASK, (k1 + W1) & MASK
    return c.astype(np.uint32)


def gumbel(seed: int, step: int, tokens: np.ndarray) -> np.ndarray:
    """-log(-log(u)) as fp32, u = (2 r + 1) / 2^53 from the first two output words at counter (token, step, 0, 0)."""
    counter = np.zeros((len(tokens), 4), dtype=np.uint32)
    counter[:, 0], counter[:, 1] = tokens, step
    x = philox4x32_10(counter, (seed & MASK, (seed >> 32) & MASK)).astype(np.uint64)
    r = ((x[:, 0] << np.uint64(32)) | x[:, 1]) >> np.uint64(12)
    u = (2.0 * r.astype(np.float64) + 1.0) * 2.0 ** -53
    return (-np.log(-np.log(u))).astype(np.float32)


def scores(logits: np.ndarray, temperature: float, softcap: float) -> np.ndarray:
    """fp32 capped logits / T (the values the sampled choice works on)."""
    z = logits.astype(np.float32)
    if softcap > 0:
        z = (np.float32(softcap) * np.tanh(z / np.float32(softcap), dtype=np.float32)).astype(np.float32)
    return (z / np.float32(temperature)).astype(np.float32)


def nucleus_threshold(e: np.ndarray, top_p: float) -> float:
    """The least e with C(e) > (1 - top_p) sum(e), C(x) = sum of the e <= x (equal values kept together)."""
    drop = (1.0 - top_p) * float(e.sum(dtype=np.float64))
    values = np.sort(e.astype(np.float64))
    cum = np.cumsum(values)
    uniq, last = np.unique(values, return_index=False), None
    for v in uniq:
        if cum[np.searchsorted(values, v, side="right") - 1] > drop:
            return float(v)
    return float(values[-1])


def choose(logits: np.ndarray, temperature: float, top_p: float, seed: int, step: int, softcap: float = 0.0,
           allow: np.ndarray | None = None) -> dict:
    """One row's choice; returns the token, the noisy keys, the kept mask and (for the nucleus) e and its threshold."""
    V = logits.shape[0]
    ok = np.ones(V, bool) if allow is None else allow.astype(bool)
    if temperature <= 0:
        z = np.where(ok, logits.astype(np.float32), -np.inf)
        return {"token": int(np.argmax(z)) if ok.any() else -1, "keys": z, "kept": ok}
    if not ok.any():
        return {"token": -1, "keys": np.full(V, -np.inf, np.float32), "kept": ok}
    s = scores(logits, temperature, softcap)
    kept, e, least = ok.copy(), None, None
    if top_p < 1:
        m = s[ok].max()
        e = np.where(ok, np.exp((s - m).astype(np.float32), dtype=np.float32), np.float32(0))
        least = nucleus_threshold(e, top_p)
        kept &= e >= least
    keys = np.where(kept, (s + gumbel(seed, step, np.arange(V))).astype(np.float32), -np.inf)
    return {"token": int(np.argmax(keys)) if kept.any() else -1, "keys": keys, "kept": kept, "e": e, "least": least}
