"""Generate tests/golden/reference_vectors.npz by importing the reference's own CPU-runnable implementation
(inference/modeling_nanochat.py: rotary L29-34, qk_norm_rope L37-45, eager_attention_forward L48-56).

Run in the build container, where the reference checkout is mounted:
    PYTHONPATH=<reference checkout> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py
The reference cannot travel to the GPU machine, so the vectors are committed. Inputs that are cheap to store are
stored; the large attention inputs are regenerated from their seed by tests/helpers.py and pinned by checksum."""

import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from inference import modeling_nanochat as ref  # noqa: E402  (the reference, from PYTHONPATH)

from oracle import attention as oat  # noqa: E402
from oracle import kv_append as okv  # noqa: E402
from tests import helpers  # noqa: E402

FLT_EPSILON = float(np.finfo(np.float32).eps)
out: dict[str, np.ndarray] = {}

# --- rotary tables at scattered positions, both bases in play (reference 1e6, benchmark configs 1e4)
positions = torch.tensor([0, 1, 2, 63, 64, 1000, 8191, 32767, 131071])
out["rotary_positions"] = positions.numpy()
for theta in (1e4, 1e6):
    cos, sin = ref.rotary(positions, 128, theta)
    out[f"rotary_cos_{int(theta)}"] = cos.numpy()
    out[f"rotary_sin_{int(theta)}"] = sin.numpy()

# --- qk_norm_rope on a small (B, T, H, D) block
gen = torch.Generator().manual_seed(1)
x = (torch.randn(2, 7, 5, 128, generator=gen) * 3).bfloat16()
gain = (1 + 0.1 * torch.randn(128, generator=gen)).float()
pos = torch.tensor([[0, 1, 2, 3, 4, 5, 6], [100, 999, 1000, 4095, 4096, 8190, 8191]])
cos, sin = ref.rotary(pos, 128, 1e4)
y = ref.qk_norm_rope(x, gain, cos, sin, FLT_EPSILON)
out["rope_x"], out["rope_gain"], out["rope_pos"] = helpers.bf16_bits(x), gain.numpy(), pos.numpy()
out["rope_y"] = helpers.bf16_bits(y)

# --- eager_attention_forward on quantised-then-dequantised K/V (bf16, the reference's cache dtype)
for name, seed, Hq, Hkv, lens in (("cfg0", 0, 10, 10, [1024]), ("gqa", 2, 8, 2, [300, 77])):
    case = helpers.attention_case(seed, Hq, Hkv, lens)
    digest = hashlib.sha256()
    outs = []
    for b, n in enumerate(lens):
        for key in ("k_bytes", "k_scale", "v_bytes", "v_scale"):
            digest.update(case[key][b].tobytes())
        q = helpers.bits_bf16(case["q"][b])[None, :, None, :]
        k = torch.from_numpy(oat.dequant(case["k_bytes"][b], case["k_scale"][b]).astype(np.float32)).bfloat16()
        v = torch.from_numpy(oat.dequant(case["v_bytes"][b], case["v_scale"][b]).astype(np.float32)).bfloat16()
        k, v = (t.repeat_interleave(Hq // Hkv, dim=0)[None] for t in (k, v))
        o, _ = ref.eager_attention_forward(None, q, k, v, None, scaling=128 ** -0.5)
        outs.append(helpers.bf16_bits(o[0, 0]))
    digest.update(case["q"].tobytes())
    out[f"attn_{name}_out"] = np.stack(outs)
    out[f"attn_{name}_sha256"] = np.frombuffer(digest.digest(), dtype=np.uint8)

np.savez_compressed(Path(__file__).resolve().parent / "reference_vectors.npz", **out)
print({k: v.shape for k, v in out.items()})
