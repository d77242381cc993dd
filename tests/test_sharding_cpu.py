"""Host-side partitioning logic and the N > 1 gather path on CPU ranks (gloo, world size 2)."""

import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nanochat_b200 import sharding
from oracle import attention as oat
from oracle import kv_append as okv
from tests import helpers


def test_shard_batch_partitions_and_balances():
    gen = torch.Generator().manual_seed(0)
    lens = torch.randint(512, 16385, (64,), generator=gen).tolist()
    for world in (1, 2, 4, 8):
        shards = sharding.shard_batch(lens, world)
        assert sorted(i for s in shards for i in s) == list(range(64))
        loads = [sum(lens[i] for i in s) for s in shards]
        assert max(loads) - min(loads) <= max(lens)  # the LPT bound
        assert max(loads) <= 1.05 * sum(lens) / world
    ordered = sharding.shard_batch(lens, 2, longest_first=True)
    assert [sorted(s) for s in ordered] == sharding.shard_batch(lens, 2)
    assert all(lens[a] >= lens[b] for s in ordered for a, b in zip(s[:-1], s[1:]))
    assert sharding.shard_batch([], 3) == [[], [], []]
    assert sharding.shard_batch([5, 5, 5], 2) == [[0, 2], [1]]


def test_kv_slices_cover_contiguously_on_page_boundaries():
    for n in (0, 1, 63, 64, 65, 1000, 131072, 131073):
        for world in (1, 2, 3, 8):
            slices = sharding.kv_slices(n, world)
            assert len(slices) == world and slices[0][0] == 0 and slices[-1][1] == n
            for (a, b), (c, d) in zip(slices[:-1], slices[1:]):
                assert b == c and a <= b
                assert b % 64 == 0 or b == n
            pages = [math.ceil((b - a) / 64) for a, b in slices]
            assert max(pages) - min(pages) <= 1


def test_append_owner():
    slices = sharding.kv_slices(1000, 4)  # 16 pages: 4 each -> [0,256) [256,512) [512,768) [768,1000)
    assert sharding.append_owner(1000, slices) == 3   # the tail grows in the last rank's slice
    assert sharding.append_owner(300, slices) == 1
    assert sharding.append_owner(0, sharding.kv_slices(0, 4)) == 0


def state_tensor(state) -> torch.Tensor:
    """(m natural-log, l, o) -> fp32 (Hq, 132) in the kernels' layout: m in log2 units, l, 0, 0, o[128]."""
    m, l, o = state
    out = np.zeros((m.shape[0], 132), dtype=np.float32)
    out[:, 0] = m / math.log(2.0)
    out[:, 1] = l
    out[:, 4:] = o
    return torch.from_numpy(out)


def merge_tensor(parts: torch.Tensor) -> np.ndarray:
    """CPU restatement of decode_attn_merge over (n_parts, rows, 132) -> (rows, 128) float64."""
    p = parts.double().numpy()
    m, l, o = p[..., 0], p[..., 1], p[..., 4:]
    top = m.max(0)
    w = np.where(np.isfinite(m), np.exp2(m - np.where(np.isfinite(top), top, 0.0)), 0.0)
    den = (w * l).sum(0)
    return np.where(den[:, None] > 0, (w[..., None] * o).sum(0) / np.where(den > 0, den, 1.0)[:, None], 0.0)


def worker(rank: int, world: int, port: int, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        Hq, Hkv, lens = 8, 2, [700, 64, 129]
        case = helpers.attention_case(77, Hq, Hkv, lens)  # same seed on every rank: q is replicated
        rows = []
        for b, n in enumerate(lens):
            a, e = sharding.kv_slices(n, world)[rank]
            k = oat.dequant(case["k_bytes"][b][:, a:e], case["k_scale"][b][:, a:e])
            v = oat.dequant(case["v_bytes"][b][:, a:e], case["v_scale"][b][:, a:e])
            q = okv.bf16_to_f32(case["q"][b]).astype(np.float64)
            rows.append(state_tensor(oat.attention_state(q, k, v, 128 ** -0.5)))
        part = torch.stack(rows)  # (B, Hq, 132), this rank's slice only
        gathered = sharding.gather_states(part)
        assert gathered.shape == (world, len(lens), Hq, 132)
        assert torch.equal(gathered[rank], part)
        merged = merge_tensor(gathered.reshape(world, -1, 132)).reshape(len(lens), Hq, 128)
        want = okv.bf16_to_f32(oat.decode_attention(case["q"], case["k_bytes"], case["k_scale"], case["v_bytes"],
                                                    case["v_scale"], 128 ** -0.5))
        err = float(np.abs(merged - want).max())
        if rank == 0:
            result.put(err)
    finally:
        dist.destroy_process_group()


def test_gather_and_merge_over_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    mp.spawn(worker, args=(2, port, result), nprocs=2, join=True)
    assert result.get(timeout=10) < 4e-3  # only the bf16 rounding of the reference output remains


def test_prefill_groups_cut_runs_into_groups_that_share_page_loads():
    """prefill_groups against a row-by-row restatement of its rule on random passes."""
    import random

    from nanochat_b200.attention import prefill_groups

    def by_rows(slots, positions, limit):
        starts = [0]
        for r in range(1, len(slots)):
            first = starts[-1]
            if r - first == limit or slots[r] != slots[first] or positions[r] != positions[r - 1] + 1:
                starts.append(r)
        return starts + [len(slots)]

    rng = random.Random(0)
    for limit in (64, 16, 8, 2, 1):
        for _ in range(20):
            slots, positions = [], []
            for _ in range(rng.randint(1, 6)):
                slot, first, count = rng.randint(0, 3), rng.randint(0, 40), rng.randint(1, 150)
                slots += [slot] * count
                positions += list(range(first, first + count))
            assert prefill_groups(slots, positions, limit) == by_rows(slots, positions, limit)
    assert prefill_groups([], [], 8) == [0]
    assert prefill_groups([3], [7], 2) == [0, 1]


def test_no_collection_restores_the_collector():
    import gc

    from nanochat_b200.decoder import no_collection

    assert gc.isenabled()
    with no_collection():
        assert not gc.isenabled()
    assert gc.isenabled()
    gc.disable()
    try:
        with no_collection():
            assert not gc.isenabled()
        assert not gc.isenabled()  # it was off before: it stays off
    finally:
        gc.enable()
    with pytest.raises(RuntimeError):
        with no_collection():
            raise RuntimeError("capture failed")
    assert gc.isenabled()


def test_decode_step_attention_refuses_rows_that_share_a_slot():
    """The fused append + attention launch needs one row per slot; a caller that passes its host-side slot list gets
    the duplicate reported before anything is launched (no GPU needed to see it)."""
    import pytest
    import torch

    from nanochat_b200 import attention as ops
    x = torch.zeros(3, 4 * 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="share a slot"):
        ops.decode_step_attention(x, None, None, None, None, None, None, 2, 64, slots=[0, 1, 0])



def test_slots_that_fit_follows_the_reference_rule():
    """The number of slots from free device memory: whole slots of the free bytes rounded down to 2 MiB, capped."""
    from nanochat_b200.decoder import ALLOC_GRANULE, MAX_SLOTS, DecoderConfig, slot_bytes, slots_that_fit
    from nanochat_b200.kv_cache import PAGE_BYTES

    cfg = DecoderConfig(n_layers=20, hidden=1280, n_heads=10, n_kv_heads=10, intermediate=5120, vocab=65536,
                        rope_theta=10000.0, max_len=2048)
    per = slot_bytes(cfg)
    assert per > 20 * 10 * 32 * PAGE_BYTES  # the cache pages of all layers, and the step's rows on top
    assert per - 20 * 10 * 32 * PAGE_BYTES < 2 << 20
    assert slots_that_fit(cfg, 10 * per + ALLOC_GRANULE) == 10
    assert slots_that_fit(cfg, 10 * per + ALLOC_GRANULE - 1) in (9, 10)
    assert slots_that_fit(cfg, per // ALLOC_GRANULE * ALLOC_GRANULE + ALLOC_GRANULE) == 1
    assert slots_that_fit(cfg, 10 ** 15) == MAX_SLOTS
    assert slots_that_fit(cfg, 10 ** 15, max_slots=64) == 64
    with pytest.raises(MemoryError):
        slots_that_fit(cfg, per - 1)


def test_weights_and_config_load_from_the_exported_model_s_names():
    """DecoderWeights.from_state_dict / DecoderConfig.from_exported against the layout the golden generator feeds the
    reference's exported model (tests/golden/make_golden_decoder.py): same tensors back, fused qkv in q, k, v order."""
    from nanochat_b200.decoder import DecoderConfig, DecoderWeights

    cfg, w = helpers.tiny_decoder_weights_ve()
    H, L = cfg["n_heads"], cfg["n_layers"]
    state = {"model.embed_tokens.weight": w["embed"], "lm_head.weight": w["lm_head"],
             "model.resid_lambdas": torch.tensor([lw["resid_lambda"] for lw in w["layers"]]),
             "model.x0_lambdas": torch.tensor([lw["x0_lambda"] for lw in w["layers"]])}
    for i, lw in enumerate(w["layers"]):
        p = f"model.layers.{i}."
        q, k, v = lw["wqkv"].split(H * 128, dim=0)
        state.update({p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k,
                      p + "self_attn.v_proj.weight": v, p + "self_attn.o_proj.weight": lw["wo"],
                      p + "mlp.up_proj.weight": lw["wup"], p + "mlp.down_proj.weight": lw["wdown"],
                      p + "self_attn.q_norm_weight": lw["q_gain"], p + "self_attn.k_norm_weight": lw["k_gain"]})
        if "ve_table" in lw:
            state.update({f"model.value_embeds.{i}.weight": lw["ve_table"], p + "self_attn.ve_gate.weight": lw["ve_gate"]})
    exported = {"vocab_size": cfg["vocab"], "hidden_size": cfg["hidden"], "intermediate_size": cfg["intermediate"],
                "num_hidden_layers": L, "num_attention_heads": H, "num_key_value_heads": H, "head_dim": 128,
                "max_position_embeddings": 256, "rope_parameters": {"rope_type": "default", "rope_theta": 10000.0},
                "sliding_window": 64, "layer_types": ["sliding_attention", "full_attention"]}
    c = DecoderConfig.from_exported(exported)
    assert (c.n_layers, c.hidden, c.n_heads, c.n_kv_heads, c.intermediate, c.vocab, c.max_len) == (L, 256, H, H, 1024, 512, 256)
    assert c.windows == [64, 0] and c.rope_theta == 10000.0
    got = DecoderWeights.from_state_dict(state, c, device="cpu")
    assert torch.equal(got.embed, w["embed"]) and torch.equal(got.lm_head, w["lm_head"])
    for lw, g in zip(w["layers"], got.layers):
        for name in ("wqkv", "wo", "wup", "wdown", "q_gain", "k_gain"):
            assert torch.equal(getattr(g, name), lw[name]), name
        assert (g.resid_lambda, g.x0_lambda) == (pytest.approx(lw["resid_lambda"]), pytest.approx(lw["x0_lambda"]))
        assert (g.ve_table is None) == ("ve_table" not in lw)
        if g.ve_table is not None:
            assert torch.equal(g.ve_table, lw["ve_table"]) and torch.equal(g.ve_gate, lw["ve_gate"])
    with pytest.raises(ValueError):
        DecoderConfig.from_exported({**exported, "head_dim": 64})
