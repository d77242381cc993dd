"""TEST INFRASTRUCTURE: CPU restatement of one decoder step with an fp8 KV cache.

The model math follows the reference's exported model op for op (inference/modeling_nanochat.py:84-100 attention
block, :105-110 MLP, :113-125 layer, :163-175 model, :188-194 head) with torch CPU bf16 operators; the two places
where the build differs from the reference go through this package's other checkers: q/k norm + rotary + fp8
quantise + append by oracle/kv_append_oracle.c, and attention over the dequantised cache in float64
(oracle/attention.py). So its logits differ from the reference's own only by the fp8 cache and the 1-ulp row-math
deviation; tests/golden/decoder_vectors.npz (made by the reference itself) bounds that difference."""

import numpy as np
import torch
import torch.nn.functional as F

from . import attention as oat
from . import kv_append as okv

EPS = float(np.finfo(np.float32).eps)


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def norm(x: torch.Tensor) -> torch.Tensor:
    return F.rms_norm(x, (x.size(-1),), eps=EPS)


class OracleDecoder:
    """cfg: dict with n_layers, hidden, n_heads, n_kv_heads, intermediate, vocab, rope_theta, max_len;
    weights: dict with embed, lm_head (bf16 [V, C]) and layers: list of dicts wqkv, wo, wup, wdown (bf16),
    q_gain, k_gain (fp32 [128]) and optionally resid_lambda, x0_lambda (floats; the per-layer stream mix of
    modeling_nanochat.py:170-171), ve_table (bf16 [V, Hkv * 128]) and ve_gate (fp32 [Hkv, C]) (the value-embedding
    mix of modeling_nanochat.py:88-90)."""

    def __init__(self, cfg: dict, weights: dict, n_seqs: int):
        self.cfg, self.w = cfg, weights
        self.cos, self.sin = okv.rotary_table(cfg["max_len"], cfg["rope_theta"])
        L, Hkv = cfg["n_layers"], cfg["n_kv_heads"]
        empty_b, empty_s = np.zeros((Hkv, 0, 128), np.uint8), np.zeros((Hkv, 0), np.float32)
        self.cache = [[{"k_bytes": empty_b, "k_scale": empty_s, "v_bytes": empty_b, "v_scale": empty_s}
                       for _ in range(n_seqs)] for _ in range(L)]

    def step(self, tokens: torch.Tensor, seqs: list[int]) -> torch.Tensor:
        """One token for each sequence in `seqs` (appended at that sequence's current length): fp32 logits
        (len(seqs), V), before any logit cap."""
        cfg, Hq, Hkv = self.cfg, self.cfg["n_heads"], self.cfg["n_kv_heads"]
        h = x0 = norm(self.w["embed"][tokens])
        for i, lw in enumerate(self.w["layers"]):
            l1, l2 = lw.get("resid_lambda", 1.0), lw.get("x0_lambda", 0.0)
            if l1 != 1.0 or l2 != 0.0:  # fp32 products and sum, rounded once
                h = (np.float32(l1) * h.float() + np.float32(l2) * x0.float()).to(h.dtype)
            n = norm(h)
            qkv = F.linear(n, lw["wqkv"])
            pos = np.array([self.cache[i][s]["k_bytes"].shape[1] for s in seqs], dtype=np.int32)
            ve = None
            if lw.get("ve_table") is not None:
                ve = {"h": _bits(n), "tokens": tokens.numpy(), "table": _bits(lw["ve_table"]),
                      "gate": lw["ve_gate"].numpy()}
            new = okv.kv_append(_bits(qkv), lw["q_gain"].numpy(), lw["k_gain"].numpy(), self.cos, self.sin, pos,
                                Hq, Hkv, ve=ve)
            att = np.zeros((len(seqs), Hq, 128), dtype=np.uint16)
            for r, s in enumerate(seqs):
                c = self.cache[i][s]
                for key in ("k_bytes", "v_bytes"):
                    c[key] = np.concatenate([c[key], new[key][r][:, None]], axis=1)
                for key in ("k_scale", "v_scale"):
                    c[key] = np.concatenate([c[key], new[key][r][:, None]], axis=1)
                att[r] = oat.decode_attention(new["q"][r:r + 1], [c["k_bytes"]], [c["k_scale"]], [c["v_bytes"]],
                                              [c["v_scale"]], 128 ** -0.5)[0]
            h = h + F.linear(_bf16(att).view(len(seqs), -1), lw["wo"])
            h = h + F.linear(F.relu(F.linear(norm(h), lw["wup"])).square(), lw["wdown"])
        return F.linear(norm(h).float(), self.w["lm_head"].float())
