"""kv_append_fp8 on the GPU, through the C ABI, against oracle/kv_append_oracle.c: q bits, cache bytes and scales
must be bit-exact."""

import numpy as np
import pytest
import torch

import nanochat_b200 as ncb
from oracle import kv_append as okv
from tests import helpers

pytestmark = pytest.mark.gpu
HEAD_DIM = 128


def run_case(seed, rows, Hq, Hkv, max_len, n_slots, theta=1e4, pad=0, zero_rows=(), positions=None, slots=None,
             scale=1.0, ve_hidden=0, vocab=50):
    """ve_hidden > 0 adds the value-embedding mix on v with a layer input of that width."""
    gen = torch.Generator().manual_seed(seed)
    width = (Hq + 2 * Hkv) * HEAD_DIM
    qkv = (torch.randn(rows, width + pad, generator=gen) * scale).bfloat16()
    for r in zero_rows:
        qkv[r] = 0
    q_gain = (1 + 0.2 * torch.randn(HEAD_DIM, generator=gen)).float()
    k_gain = (1 + 0.2 * torch.randn(HEAD_DIM, generator=gen)).float()
    cos, sin = ncb.rotary_table(max_len, theta)
    if positions is None:
        positions = torch.randperm(max_len, generator=gen)[:rows]  # distinct, so no two rows race for a cache row
    pos = torch.as_tensor(positions, dtype=torch.int32)
    if slots is None:
        slots = torch.randint(0, n_slots, (rows,), generator=gen)
    slot_map = torch.as_tensor(slots, dtype=torch.int32)
    cache = ncb.Fp8KVCache(n_slots, Hkv, max_len)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ve = ve_ref = None
    if ve_hidden:
        h = torch.randn(rows, ve_hidden, generator=gen).bfloat16()
        tokens = torch.randint(0, vocab, (rows,), generator=gen)
        table = (torch.randn(vocab, Hkv * HEAD_DIM, generator=gen) * 0.7).bfloat16()
        gate = (torch.randn(Hkv, ve_hidden, generator=gen) * 3 / ve_hidden ** 0.5).float()  # gates all over (0, 2)
        ve = ncb.attention.ValueEmbed(h.cuda(), tokens.cuda(), table.cuda(), gate.cuda())
        ve_ref = {"h": helpers.bf16_bits(h), "tokens": tokens.numpy(), "table": helpers.bf16_bits(table),
                  "gate": gate.numpy()}
    q_out = ncb.kv_append(qkv.cuda()[:, :width], q_gain.cuda(), k_gain.cuda(), cos.cuda(),
                          sin.cuda(), pos.cuda(), cache, Hq, slot_map=slot_map.cuda(), status=status, ve=ve)
    torch.cuda.synchronize()
    assert status.item() == 0
    want = okv.kv_append(helpers.bf16_bits(qkv), q_gain.numpy(), k_gain.numpy(), cos.numpy(), sin.numpy(),
                         pos.numpy(), Hq, Hkv, ve=ve_ref)
    assert np.array_equal(helpers.bf16_bits(q_out.cpu()), want["q"]), "q bits differ"
    host = ncb.Fp8KVCache(n_slots, Hkv, max_len, device="cpu", pages=cache.pages.cpu())
    for r in range(rows):
        k, ks, v, vs = host.read(int(slot_map[r]), 1, start=int(pos[r]))
        assert np.array_equal(k[:, 0].numpy(), want["k_bytes"][r]), f"row {r}: k bytes differ"
        assert np.array_equal(v[:, 0].numpy(), want["v_bytes"][r]), f"row {r}: v bytes differ"
        assert np.array_equal(ks[:, 0].numpy(), want["k_scale"][r]), f"row {r}: k scale differs"
        assert np.array_equal(vs[:, 0].numpy(), want["v_scale"][r]), f"row {r}: v scale differs"
    return cache, want


@pytest.mark.parametrize("Hq,Hkv", [(10, 10), (32, 8), (16, 4), (8, 1), (1, 1)])
def test_bit_exact_random(Hq, Hkv):
    run_case(seed=Hq * 100 + Hkv, rows=97, Hq=Hq, Hkv=Hkv, max_len=1000, n_slots=5)


@pytest.mark.parametrize("Hq,Hkv,hidden", [(10, 10, 1280), (16, 4, 2048), (2, 2, 256), (8, 1, 768)])
def test_value_embedding_mix_is_bit_exact(Hq, Hkv, hidden):
    """kv_append_fp8_ve: v <- bf16(v + 2 sigmoid(gate . h) ve[token]) before quantising; q, k and v bytes and scales
    against the checker, which sums the gate in the reference's lane order."""
    _, plain = run_case(seed=500 + Hq, rows=61, Hq=Hq, Hkv=Hkv, max_len=512, n_slots=4)
    _, mixed = run_case(seed=500 + Hq, rows=61, Hq=Hq, Hkv=Hkv, max_len=512, n_slots=4, ve_hidden=hidden)
    assert np.array_equal(plain["k_bytes"], mixed["k_bytes"]) and not np.array_equal(plain["v_bytes"], mixed["v_bytes"])


def test_bit_exact_reference_rope_base_and_strided_rows():
    run_case(seed=11, rows=33, Hq=6, Hkv=6, max_len=4096, n_slots=3, theta=1e6, pad=64)


def test_zero_rows_and_extreme_magnitudes():
    run_case(seed=12, rows=16, Hq=4, Hkv=2, max_len=128, n_slots=16, zero_rows=(0, 7), positions=list(range(16)),
             slots=list(range(16)))
    run_case(seed=13, rows=16, Hq=4, Hkv=2, max_len=128, n_slots=16, positions=list(range(16)), slots=list(range(16)),
             scale=1e4)
    run_case(seed=14, rows=16, Hq=4, Hkv=2, max_len=128, n_slots=16, positions=list(range(16)), slots=list(range(16)),
             scale=1e-20)


def test_first_and_last_position_and_untouched_neighbours():
    cache, _ = run_case(seed=15, rows=2, Hq=2, Hkv=2, max_len=192, n_slots=2, positions=[0, 191], slots=[0, 1])
    host = ncb.Fp8KVCache(2, 2, 192, device="cpu", pages=cache.pages.cpu())
    k, ks, v, vs = host.read(0, 191, start=1)
    assert not k.any() and not v.any() and not ks.any() and not vs.any()
    k, ks, v, vs = host.read(1, 191, start=0)
    assert not k.any() and not v.any() and not ks.any() and not vs.any()


def test_default_slot_map_is_the_row():
    gen = torch.Generator().manual_seed(16)
    Hq, Hkv, rows = 4, 2, 6
    qkv = torch.randn(rows, (Hq + 2 * Hkv) * HEAD_DIM, generator=gen).bfloat16()
    ones = torch.ones(HEAD_DIM)
    cos, sin = ncb.rotary_table(64, 1e4)
    pos = torch.arange(rows, dtype=torch.int32)
    cache = ncb.Fp8KVCache(rows, Hkv, 64)
    ncb.kv_append(qkv.cuda(), ones.cuda(), ones.cuda(), cos.cuda(), sin.cuda(), pos.cuda(), cache, Hq)
    torch.cuda.synchronize()
    want = okv.kv_append(helpers.bf16_bits(qkv), ones.numpy(), ones.numpy(), cos.numpy(), sin.numpy(), pos.numpy(),
                         Hq, Hkv)
    host = ncb.Fp8KVCache(rows, Hkv, 64, device="cpu", pages=cache.pages.cpu())
    for r in range(rows):
        k, ks, v, vs = host.read(r, 1, start=r)
        assert np.array_equal(k[:, 0].numpy(), want["k_bytes"][r]) and np.array_equal(ks[:, 0].numpy(), want["k_scale"][r])


def test_out_of_range_rows_are_skipped_and_flagged():
    gen = torch.Generator().manual_seed(17)
    Hq, Hkv = 2, 1
    qkv = torch.randn(3, (Hq + 2 * Hkv) * HEAD_DIM, generator=gen).bfloat16()
    ones = torch.ones(HEAD_DIM)
    cos, sin = ncb.rotary_table(64, 1e4)
    cache = ncb.Fp8KVCache(2, Hkv, 64)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    pos = torch.tensor([5, 64, 3], dtype=torch.int32)      # row 1: position past the cache
    slots = torch.tensor([0, 0, 2], dtype=torch.int32)     # row 2: slot past the cache
    ncb.kv_append(qkv.cuda(), ones.cuda(), ones.cuda(), cos.cuda(), sin.cuda(), pos.cuda(), cache, Hq,
                  slot_map=slots.cuda(), status=status)
    torch.cuda.synchronize()
    assert status.item() == 1
    host = ncb.Fp8KVCache(2, Hkv, 64, device="cpu", pages=cache.pages.cpu())
    k, ks, _, _ = host.read(0, 64)
    assert ks[0, 5] > 0 and ks[0, :5].sum() == 0 and ks[0, 6:].sum() == 0
    assert not host.pages[1].any()


def test_idle_rows_are_skipped_silently():
    """A negative position marks an idle row (a slot without a request): nothing written, nothing flagged."""
    gen = torch.Generator().manual_seed(18)
    Hq, Hkv = 2, 1
    qkv = torch.randn(3, (Hq + 2 * Hkv) * HEAD_DIM, generator=gen).bfloat16()
    ones = torch.ones(HEAD_DIM)
    cos, sin = ncb.rotary_table(64, 1e4)
    cache = ncb.Fp8KVCache(3, Hkv, 64)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    pos = torch.tensor([5, -1, 3], dtype=torch.int32)
    ncb.kv_append(qkv.cuda(), ones.cuda(), ones.cuda(), cos.cuda(), sin.cuda(), pos.cuda(), cache, Hq, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert cache.pages[0].any() and not cache.pages[1].any() and cache.pages[2].any()


def test_native_error_on_bad_shapes():
    cache = ncb.Fp8KVCache(1, 3, 64)
    qkv = torch.zeros(1, (4 + 6) * HEAD_DIM, dtype=torch.bfloat16, device="cuda")
    ones = torch.ones(HEAD_DIM, device="cuda")
    cos, sin = ncb.rotary_table(64, 1e4, device="cuda")
    with pytest.raises(ncb.NativeError):
        ncb.kv_append(qkv, ones, ones, cos, sin, torch.zeros(1, dtype=torch.int32, device="cuda"), cache, Hq=4)


def test_prefill_runs_store_the_same_bytes_as_single_rows():
    """Rows that form runs of consecutive positions of one slot (a prefill pass): blocks whose 16 rows are an aligned
    run store V as 16-byte chunks, the ragged starts and ends and the slot changes byte by byte; every row must still
    match the checker bit for bit, and nothing else in the cache may change."""
    runs = [(0, 0, 100), (1, 5, 61), (2, 16, 48), (3, 63, 70), (1, 128, 145), (4, 32, 33)]  # (slot, first, end)
    slots = [s for s, a, b in runs for _ in range(a, b)]
    positions = [p for s, a, b in runs for p in range(a, b)]
    cache, _ = run_case(seed=21, rows=len(slots), Hq=8, Hkv=2, max_len=192, n_slots=5, positions=positions,
                        slots=slots)
    host = ncb.Fp8KVCache(5, 2, 192, device="cpu", pages=cache.pages.cpu())
    written = set(zip(slots, positions))
    for slot in range(5):
        k, ks, v, vs = host.read(slot, 192)
        for p in range(192):
            if (slot, p) not in written:
                assert not k[:, p].any() and not v[:, p].any() and not ks[:, p].any() and not vs[:, p].any(), (slot, p)
