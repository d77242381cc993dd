"""Seeded synthetic inputs shared by the tests: the shapes and distributions of the benchmark configurations
(q ~ N(0,1) in bf16; K, V ~ N(0,1) quantised per (token, head) with scale = amax / 448)."""

import numpy as np
import torch

from oracle import kv_append as okv

HEAD_DIM = 128


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit patterns (numpy)."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def bits_bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def randn_bf16(gen: torch.Generator, *shape: int) -> np.ndarray:
    return bf16_bits(torch.randn(*shape, generator=gen).bfloat16())


def attention_case(seed: int, Hq: int, Hkv: int, lens: list[int]) -> dict:
    """q bits (B, Hq, 128) and per sequence quantised K, V: lists of (Hkv, n, 128) u8 and (Hkv, n) fp32."""
    gen = torch.Generator().manual_seed(seed)
    B = len(lens)
    case = {"q": randn_bf16(gen, B, Hq, HEAD_DIM), "k_bytes": [], "k_scale": [], "v_bytes": [], "v_scale": [],
            "lens": list(lens), "Hq": Hq, "Hkv": Hkv}
    for n in lens:
        for name in ("k", "v"):
            b, s = okv.quant_rows(randn_bf16(gen, Hkv, n, HEAD_DIM))
            case[f"{name}_bytes"].append(b)
            case[f"{name}_scale"].append(s)
    return case


def error_stats(got_bits: np.ndarray, want_bits: np.ndarray) -> tuple[float, float]:
    """(max-abs, mean-abs) difference of two bf16 bit arrays."""
    d = np.abs(okv.bf16_to_f32(got_bits).astype(np.float64) - okv.bf16_to_f32(want_bits).astype(np.float64))
    return float(d.max()) if d.size else 0.0, float(d.mean()) if d.size else 0.0


def tiny_decoder_weights(seed: int = 21) -> tuple[dict, dict]:
    """A 2-layer, 2-head (hidden 256), vocab 512 random-init model on the CPU: bf16 weights ~ N(0, 0.02)
    (the benchmark's initialisation) and fp32 QK gains 1 + 0.1 N(0, 1). Returns (config dict, weight dict)."""
    cfg = {"n_layers": 2, "hidden": 256, "n_heads": 2, "n_kv_heads": 2, "intermediate": 1024, "vocab": 512,
           "rope_theta": 10000.0, "max_len": 256}
    gen = torch.Generator().manual_seed(seed)
    C, H, Fd, V = cfg["hidden"], cfg["n_heads"], cfg["intermediate"], cfg["vocab"]

    def w(*shape):
        return (torch.randn(*shape, generator=gen) * 0.02).bfloat16()

    layers = [{"wqkv": w(3 * H * HEAD_DIM, C), "wo": w(C, H * HEAD_DIM), "wup": w(Fd, C), "wdown": w(C, Fd),
               "q_gain": (1 + 0.1 * torch.randn(HEAD_DIM, generator=gen)).float(),
               "k_gain": (1 + 0.1 * torch.randn(HEAD_DIM, generator=gen)).float()} for _ in range(cfg["n_layers"])]
    return cfg, {"embed": w(V, C), "lm_head": w(V, C), "layers": layers}


def tiny_decoder_weights_ve(seed: int = 23) -> tuple[dict, dict]:
    """tiny_decoder_weights plus what the reference's own checkpoints have and the benchmark models lack: a value
    embedding on the last layer (table bf16 [V, H * 128] ~ N(0, 0.5), gate fp32 [H, C] ~ N(0, 2 / sqrt(C)), so gates
    spread over (0, 2)) and per-layer stream-mix lambdas away from (1, 0)."""
    cfg, w = tiny_decoder_weights(seed)
    gen = torch.Generator().manual_seed(seed + 1)
    C, H, V = cfg["hidden"], cfg["n_heads"], cfg["vocab"]
    last = w["layers"][-1]
    last["ve_table"] = (torch.randn(V, H * HEAD_DIM, generator=gen) * 0.5).bfloat16()
    last["ve_gate"] = (torch.randn(H, C, generator=gen) * 2 / C ** 0.5).float()
    for lw, (l1, l2) in zip(w["layers"], [(0.9, 0.2), (1.1, -0.15)]):
        lw["resid_lambda"], lw["x0_lambda"] = l1, l2
    return cfg, w

