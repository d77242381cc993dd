"""The oracle against its pins: torch's e4m3 / bf16 conversions (exhaustive where feasible) and the committed
outputs of the reference's own functions (tests/golden/reference_vectors.npz, made by tests/golden/make_golden.py)."""

import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import attention as oat
from oracle import kv_append as okv
from tests import helpers

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_vectors.npz")


def test_e4m3_conversion_matches_torch_on_every_bf16_value():
    """All 65,536 bf16 patterns whose magnitude torch converts without overflow, at several scalings."""
    bits = np.arange(1 << 16, dtype=np.uint16)
    x = okv.bf16_to_f32(bits)
    for mul in (1.0, 0.37, 448.0 / 3.25, 2.0 ** -7):
        with np.errstate(all="ignore"):
            v = (x * np.float32(mul)).astype(np.float32)
        keep = np.isfinite(v) & (np.abs(v) < 464.0)
        want = torch.from_numpy(v[keep]).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        got = okv.f32_to_e4m3(v[keep])
        assert np.array_equal(got, want)


def test_e4m3_conversion_matches_torch_on_random_fp32():
    gen = torch.Generator().manual_seed(3)
    v = torch.randn(1 << 20, generator=gen) * torch.exp2(torch.randint(-12, 9, (1 << 20,), generator=gen).float())
    v = v[v.abs() < 464.0]
    want = v.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(okv.f32_to_e4m3(v.numpy()), want)


def test_e4m3_known_answers():
    """Ties to even, the subnormal grid and saturation."""
    x = np.array([448.0, 448.00003, 463.9, 464.0, 1e9, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9, 0.0, -0.0, -448.0, 17.0,
                  19.0], dtype=np.float32)
    want = np.array([0x7e, 0x7e, 0x7e, 0x7e, 0x7e, 0x01, 0x00, 0x02, 0x00, 0x80, 0xfe, 0x58, 0x5a], dtype=np.uint8)
    assert np.array_equal(okv.f32_to_e4m3(x), want)


def test_e4m3_decode_round_trip():
    b = np.array([i for i in range(256) if i & 0x7f != 0x7f], dtype=np.uint8)
    assert np.array_equal(okv.f32_to_e4m3(okv.e4m3_to_f32(b)), b)
    want = torch.from_numpy(b).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(okv.e4m3_to_f32(b), want)


def test_bf16_rounding_matches_torch():
    gen = torch.Generator().manual_seed(4)
    v = torch.randn(1 << 18, generator=gen) * 100
    assert np.array_equal(okv.f32_to_bf16(v.numpy()), helpers.bf16_bits(v.bfloat16()))


def test_quant_rows_rule():
    """scale = amax / 448 (one fp32 divide), byte = e4m3(x / scale), zero rows -> scale 0 and zero bytes."""
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(64, 128, generator=gen).bfloat16()
    x[3] = 0
    x[4, 1:] = 0  # a single non-zero value
    b, s = okv.quant_rows(helpers.bf16_bits(x))
    xf = x.float()
    scale = xf.abs().amax(-1) / 448.0
    assert np.array_equal(s, scale.numpy())
    safe = torch.where(scale > 0, scale, torch.ones_like(scale))
    want = (xf / safe[:, None]).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    want[3] = 0
    assert np.array_equal(b, want)
    assert s[3] == 0 and not b[3].any()
    assert b[4, 0] in (0x7e, 0xfe)


@pytest.mark.parametrize("theta", [1e4, 1e6])
def test_rotary_table_matches_reference(theta):
    cos, sin = okv.rotary_table(131072, theta)
    p = GOLDEN["rotary_positions"]
    assert np.array_equal(cos[p], GOLDEN[f"rotary_cos_{int(theta)}"])
    assert np.array_equal(sin[p], GOLDEN[f"rotary_sin_{int(theta)}"])


def test_qk_row_within_one_ulp_of_reference():
    """The oracle's individually rounded order vs the reference's torch expression (rsqrt, fused differently):
    bf16 outputs agree except for a small fraction of 1-ulp differences."""
    x, gain, pos, want = GOLDEN["rope_x"], GOLDEN["rope_gain"], GOLDEN["rope_pos"], GOLDEN["rope_y"]
    cos, sin = okv.rotary_table(8192, 1e4)
    B, T, H, D = x.shape
    rows = x.reshape(B * T, H * D)
    # treat the block as q heads only: Hq = H, and feed a dummy kv head
    qkv = np.concatenate([rows, np.zeros((B * T, 2 * D), np.uint16)], axis=1)
    got = okv.kv_append(qkv, gain, gain, cos, sin, pos.reshape(-1), H, 1)["q"].reshape(B, T, H, D)
    a, b = okv.bf16_to_f32(got).astype(np.float64), okv.bf16_to_f32(want).astype(np.float64)
    ulp = np.maximum(np.abs(b), 2.0 ** -126) * 2.0 ** -7
    assert (np.abs(a - b) <= ulp).all()
    assert (got != want).mean() < 0.01


@pytest.mark.parametrize("name,seed,Hq,Hkv,lens", [("cfg0", 0, 10, 10, [1024]), ("gqa", 2, 8, 2, [300, 77])])
def test_attention_oracles_against_reference_outputs(name, seed, Hq, Hkv, lens):
    case = helpers.attention_case(seed, Hq, Hkv, lens)
    digest = hashlib.sha256()
    for b in range(len(lens)):
        for key in ("k_bytes", "k_scale", "v_bytes", "v_scale"):
            digest.update(case[key][b].tobytes())
    digest.update(case["q"].tobytes())
    assert np.array_equal(np.frombuffer(digest.digest(), dtype=np.uint8), GOLDEN[f"attn_{name}_sha256"]), \
        "seeded inputs differ from the ones the golden outputs were made from"
    want = GOLDEN[f"attn_{name}_out"]
    # the torch port of the reference's function reproduces it exactly
    port = np.stack([oat.eager_attention_port_quantised(case["q"][b], case["k_bytes"][b], case["k_scale"][b],
                                                        case["v_bytes"][b], case["v_scale"][b], 128 ** -0.5)
                     for b in range(len(lens))])
    assert np.array_equal(port, want)
    # the float64 checker agrees with the reference within the path's tolerance (bf16 K/V and bf16 probabilities
    # in the reference account for the difference)
    got = oat.decode_attention(case["q"], case["k_bytes"], case["k_scale"], case["v_bytes"], case["v_scale"],
                               128 ** -0.5)
    max_abs, mean_abs = helpers.error_stats(got, want)
    assert max_abs <= 2e-2 and mean_abs <= 2e-3


def test_attention_oracle_merge_is_split_invariant():
    case = helpers.attention_case(7, 8, 2, [257])
    k = oat.dequant(case["k_bytes"][0], case["k_scale"][0])
    v = oat.dequant(case["v_bytes"][0], case["v_scale"][0])
    q = okv.bf16_to_f32(case["q"][0]).astype(np.float64)
    whole = oat.merge_states([oat.attention_state(q, k, v, 0.1)])
    cuts = [0, 1, 64, 64, 200, 257]  # includes an empty slice
    parts = [oat.attention_state(q, k[:, a:b], v[:, a:b], 0.1) for a, b in zip(cuts[:-1], cuts[1:])]
    assert np.allclose(oat.merge_states(parts), whole, rtol=1e-12, atol=1e-14)


def test_attention_oracle_window():
    case = helpers.attention_case(8, 4, 4, [100])
    full = oat.decode_attention(case["q"], [case["k_bytes"][0][:, 60:]], [case["k_scale"][0][:, 60:]],
                                [case["v_bytes"][0][:, 60:]], [case["v_scale"][0][:, 60:]], 0.1)
    win = oat.decode_attention(case["q"], case["k_bytes"], case["k_scale"], case["v_bytes"], case["v_scale"], 0.1,
                               window=40)
    assert np.array_equal(full, win)

