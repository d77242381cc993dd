"""The GPU decoder (cuBLAS GEMMs + this package's append/attention kernels, CUDA-graph step) against the CPU
restatement and against logits/tokens of the reference's own exported model on the tiny golden configuration."""

from pathlib import Path

import numpy as np
import pytest
import torch

from nanochat_b200.decoder import Decoder, DecoderConfig, DecoderWeights, LayerWeights
from oracle.decoder import OracleDecoder
from tests import helpers
from tests.test_decoder_oracle import GOLDEN, GOLDEN_VE, teacher_forced_logits, uncapped

pytestmark = pytest.mark.gpu


def gpu_decoder(n_slots=2):
    cfg, w = helpers.tiny_decoder_weights()
    dcfg = DecoderConfig(cfg["n_layers"], cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["intermediate"],
                         cfg["vocab"], cfg["rope_theta"], cfg["max_len"])
    layers = [LayerWeights(*(lw[k].cuda() for k in ("wqkv", "wo", "wup", "wdown", "q_gain", "k_gain")))
              for lw in w["layers"]]
    return Decoder(dcfg, DecoderWeights(w["embed"].cuda(), w["lm_head"].cuda(), layers), n_slots), cfg, w


def gpu_decoder_ve(n_slots=2):
    """The reference's own model shape: a value embedding on the last layer, stream-mix lambdas away from (1, 0)."""
    cfg, w = helpers.tiny_decoder_weights_ve()
    dcfg = DecoderConfig(cfg["n_layers"], cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["intermediate"],
                         cfg["vocab"], cfg["rope_theta"], cfg["max_len"])
    layers = [LayerWeights(*(lw[k].cuda() for k in ("wqkv", "wo", "wup", "wdown", "q_gain", "k_gain")),
                           resid_lambda=lw["resid_lambda"], x0_lambda=lw["x0_lambda"],
                           ve_table=lw["ve_table"].cuda() if "ve_table" in lw else None,
                           ve_gate=lw["ve_gate"].cuda() if "ve_gate" in lw else None) for lw in w["layers"]]
    return Decoder(dcfg, DecoderWeights(w["embed"].cuda(), w["lm_head"].cuda(), layers), n_slots), cfg, w


@torch.no_grad()
@pytest.mark.parametrize("path", ["rows", "fused"])
def test_value_embedding_and_stream_mix_match_cpu_restatement_and_reference(path):
    """A model with a value-embedding layer and non-trivial resid / x0 lambdas, teacher-forced on the golden run of
    the reference's exported model with the same weights: the row path (cuBLAS GEMMs, add_rms_norm_mix) and the
    fused step (skinny_gemm_mix epilogue, the mix in embed_norm, the gate inside the attention launch)."""
    dec, cfg, w = gpu_decoder_ve()
    assert dec.gemm_kernel(2) == "skinny"
    slot_map = torch.arange(2, dtype=torch.int32, device="cuda")
    pos = torch.zeros(2, dtype=torch.int32, device="cuda")
    buf = dec.fused_buffers(2)

    def step(tok):
        if path == "fused":
            logits = dec.fused_step(tok.cuda(), pos, slot_map, int(pos.max()) + 1, buf, choose=False).cpu()
        else:
            logits = dec.logits_rows(tok.cuda(), pos.clone(), slot_map, int(pos.max()) + 1).cpu()
        pos.add_(1)
        return logits

    got = teacher_forced_logits(step, GOLDEN_VE)
    oracle = OracleDecoder(cfg, w, n_seqs=2)
    cpu = teacher_forced_logits(lambda tok: oracle.step(tok, [0, 1]), GOLDEN_VE)
    err = np.abs(got - cpu)
    assert err.max() < 1e-2 and err.mean() < 1.5e-3, (err.max(), err.mean())  # GEMM accumulation order only
    ref = uncapped(GOLDEN_VE["logits"], float(GOLDEN_VE["softcap"]))
    err = np.abs(got - ref)
    assert err.max() < 2.5e-2 and err.mean() < 4e-3, (err.max(), err.mean())
    assert int(dec.status.item()) == 0


@torch.no_grad()
def test_value_embedding_and_stream_mix_on_the_stream_gemm_step():
    """The same model at 24 rows: the tcgen05 step (stream_gemm_mix epilogue) against the row path with cuBLAS."""
    ours, cfg, _ = gpu_decoder_ve(24)
    ref, _, _ = gpu_decoder_ve(24)
    assert ours.gemm_kernel(24) == "stream"
    gen = torch.Generator().manual_seed(24)
    slot_map = torch.arange(24, dtype=torch.int32, device="cuda")
    pos = torch.zeros(24, dtype=torch.int32, device="cuda")
    buf = ours.fused_buffers(24)
    for t in range(3):
        tok = torch.randint(0, cfg["vocab"], (24,), generator=gen).cuda()
        got = ours.fused_step(tok.clone(), pos, slot_map, t + 1, buf, choose=False).clone()
        want = ref.logits_rows(tok, pos.clone(), slot_map, t + 1)
        pos.add_(1)
        err = (got - want).abs()
        top = max(float(want.abs().max()), 1.0)
        assert err.max() < 3e-2 * top and err.mean() < 5e-3 * top, (t, float(err.max()), float(err.mean()))
    assert int(ours.status.item()) == 0


@torch.no_grad()
def test_step_logits_match_cpu_restatement_and_reference():
    dec, cfg, w = gpu_decoder()
    slot_map = torch.arange(2, dtype=torch.int32, device="cuda")
    pos = torch.zeros(2, dtype=torch.int32, device="cuda")

    def step(tok):
        logits = dec.logits_rows(tok.cuda(), pos.clone(), slot_map, int(pos.max()) + 1)
        pos.add_(1)
        return logits.cpu()

    got = teacher_forced_logits(step)
    oracle = OracleDecoder(cfg, w, n_seqs=2)
    cpu = teacher_forced_logits(lambda tok: oracle.step(tok, [0, 1]))
    err = np.abs(got - cpu)
    assert err.max() < 1e-2 and err.mean() < 1.5e-3, (err.max(), err.mean())  # GEMM accumulation order only
    ref = uncapped(GOLDEN["logits"], float(GOLDEN["softcap"]))
    err = np.abs(got - ref)
    assert err.max() < 2.5e-2 and err.mean() < 4e-3, (err.max(), err.mean())
    assert int(dec.status.item()) == 0


@torch.no_grad()
def test_fused_step_logits_match_cpu_restatement_and_reference():
    """The same teacher-forced run on the decode_step kernels (own GEMMs with fused norm and epilogues)."""
    dec, cfg, w = gpu_decoder()
    assert dec.fused_supported(2)
    slot_map = torch.arange(2, dtype=torch.int32, device="cuda")
    pos = torch.zeros(2, dtype=torch.int32, device="cuda")
    buf = dec.fused_buffers(2)

    def step(tok):
        logits = dec.fused_step(tok.cuda(), pos, slot_map, int(pos.max()) + 1, buf, choose=False).cpu()
        pos.add_(1)
        return logits

    got = teacher_forced_logits(step)
    oracle = OracleDecoder(cfg, w, n_seqs=2)
    cpu = teacher_forced_logits(lambda tok: oracle.step(tok, [0, 1]))
    err = np.abs(got - cpu)
    assert err.max() < 1e-2 and err.mean() < 1.5e-3, (err.max(), err.mean())
    ref = uncapped(GOLDEN["logits"], float(GOLDEN["softcap"]))
    err = np.abs(got - ref)
    assert err.max() < 2.5e-2 and err.mean() < 4e-3, (err.max(), err.mean())
    assert int(dec.status.item()) == 0


def test_generate_prefill_and_graph_decode_reproduce_reference_tokens():
    dec, _, _ = gpu_decoder()
    prompts = GOLDEN["prompt"].tolist()
    tokens, timing = dec.generate(prompts, 6)
    ref = uncapped(GOLDEN["logits"], float(GOLDEN["softcap"]))[:, :6]
    top2 = np.sort(ref, -1)[..., -2:]
    clear = (top2[..., 1] - top2[..., 0]) > 1.5e-2
    # a greedy stream is only comparable up to its first near-tie
    compared = 0
    for b in range(2):
        for t in range(6):
            if not clear[b, t]:
                break
            assert tokens[b][t] == int(GOLDEN["tokens"][b, t]), (b, t)
            compared += 1
    assert compared >= 6 and timing["tokens_per_s"] > 0
    # a second call reuses the captured graph and gives the same stream
    again, _ = dec.generate(prompts, 6)
    assert again == tokens


def test_decode_from_with_an_uncaptured_key_leaves_live_caches_alone():
    """decode_from on caches that already hold the prompts, with a step graph that is captured only then: the
    capture's warm-up must not touch live positions (it runs with every slot idle). Same stream as generate(), which
    captures before it prefills."""
    dec, _, _ = gpu_decoder()
    prompts = GOLDEN["prompt"].tolist()
    want, _ = dec.generate(prompts, 6)
    other, _, _ = gpu_decoder()
    with torch.no_grad():
        other.prefill(prompts, [0, 1])
    filled = [c.pages.clone() for c in other.caches]
    assert not other._graphs
    got, _ = other.decode_from([p[-1] for p in prompts], [len(p) - 1 for p in prompts], 6)
    assert got == want
    n = len(prompts[0]) - 1  # the prefilled positions are untouched
    for cache, before in zip(other.caches, filled):
        now = ncb_cache_rows(cache, n)
        assert all(torch.equal(a, b) for a, b in zip(now, ncb_cache_rows_from(before, cache, n)))


def ncb_cache_rows(cache, n):
    return [t.clone() for slot in range(2) for t in cache.read(slot, n)]


def ncb_cache_rows_from(pages, like, n):
    from nanochat_b200.kv_cache import Fp8KVCache
    old = Fp8KVCache(like.n_slots, like.kv_heads, like.capacity, device=pages.device, pages=pages)
    return ncb_cache_rows(old, n)


def test_ragged_prompts_and_gqa_shapes_run_and_agree_with_rowwise_logits():
    """A GQA model with prompts of different lengths: generate() (prefill rows + graph decode) against the eager
    row-at-a-time path."""
    cfg = DecoderConfig(n_layers=2, hidden=512, n_heads=4, n_kv_heads=1, intermediate=1024, vocab=304, max_len=128)
    w = DecoderWeights.random_init(cfg, seed=5, device="cuda", std=0.05)
    gen = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 304, (n,), generator=gen).tolist() for n in (1, 9, 70)]
    dec = Decoder(cfg, w, 3)
    assert dec.fused_supported(3)  # generate() decodes on the decode_step kernels, the check below on torch ops
    tokens, _ = dec.generate(prompts, 5)
    ref = Decoder(cfg, w, 3)
    with torch.no_grad():
        for b, p in enumerate(prompts):
            slot = torch.tensor([b], dtype=torch.int32, device="cuda")
            seq, out = list(p), []
            for t in range(len(p) + 4):
                logits = ref.logits_rows(torch.tensor([seq[t]], device="cuda"),
                                         torch.tensor([t], dtype=torch.int32, device="cuda"), slot, t + 1)
                if t >= len(p) - 1:
                    out.append(logits[0].clone())
                    seq.append(int(logits.argmax()))
            agreed = 0
            for t, z in enumerate(out):
                if tokens[b][t] != int(z.argmax()):
                    # the two paths round their GEMMs differently: a different choice is only legitimate at a
                    # near-tie, after which the streams are no longer comparable
                    assert float(z.max() - z[tokens[b][t]]) < 5e-2, (b, t)
                    break
                agreed += 1
            assert agreed >= 2, (b, agreed)


def test_prompt_store_round_trip_gives_the_same_stream():
    """A prompt prefilled once is served from the pinned-host page store afterwards: same tokens, no prefill."""
    cfg = DecoderConfig(n_layers=2, hidden=512, n_heads=4, n_kv_heads=2, intermediate=1024, vocab=304, max_len=256)
    w = DecoderWeights.random_init(cfg, seed=7, device="cuda", std=0.05)
    gen = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 304, (n,), generator=gen).tolist() for n in (130, 2, 65)]
    dec = Decoder(cfg, w, 3, prompt_store=1024)
    first, _ = dec.generate(prompts, 6)
    assert set(dec.store.stored) == {tuple(p) for p in prompts} and dec.store.used == 3 + 1 + 1
    for cache in dec.caches:  # wipe the slots: the second run can only succeed from the store
        cache.pages.zero_()
    calls = []
    original = dec.prefill
    dec.prefill = lambda p, s, **kw: (calls.append(len(p)), original(p, s, **kw))
    second, _ = dec.generate(list(reversed(prompts)), 6)  # other slots than the first time
    assert calls == [0]
    assert second == list(reversed(first))


def test_sampled_generation_is_reproducible_and_follows_the_choice_rule():
    """Sampled decoding: the same seeds give the same stream, other seeds another; the first sampled token equals
    the checker's choice for the step's logits."""
    from oracle import sampling
    cfg = DecoderConfig(n_layers=2, hidden=512, n_heads=4, n_kv_heads=2, intermediate=1024, vocab=320, max_len=128)
    w = DecoderWeights.random_init(cfg, seed=9, device="cuda", std=0.05)
    gen = torch.Generator().manual_seed(10)
    prompts = [torch.randint(0, 320, (n,), generator=gen).tolist() for n in (5, 20)]
    dec = Decoder(cfg, w, 2, softcap=15.0)
    a, _ = dec.generate(prompts, 8, temperature=0.9, top_p=0.8, seeds=[11, 12])
    b, _ = dec.generate(prompts, 8, temperature=0.9, top_p=0.8, seeds=[11, 12])
    c, _ = dec.generate(prompts, 8, temperature=0.9, top_p=0.8, seeds=[13, 14])
    g, _ = dec.generate(prompts, 8)
    assert a == b and a != c and a != g
    # step 0 of each sequence against the checker, on the logits of the eager path
    ref = Decoder(cfg, w, 2)
    with torch.no_grad():
        ref.prefill(prompts, [0, 1])
        for s_, (p, seed) in enumerate(zip(prompts, (11, 12))):
            logits = ref.logits_rows(torch.tensor([p[-1]], device="cuda"),
                                     torch.tensor([len(p) - 1], dtype=torch.int32, device="cuda"),
                                     torch.tensor([s_], dtype=torch.int32, device="cuda"), len(p))[0].cpu().numpy()
            want = sampling.choose(logits, 0.9, 0.8, seed, 0, 15.0)
            got = a[s_][0]
            assert got == want["token"] or (want["kept"][got] and want["keys"][want["token"]] - want["keys"][got] < 5e-2)


@torch.no_grad()
@pytest.mark.parametrize("rows,intermediate", [(24, 1024), (40, 1024), (64, 1024), (8, 5248)])
def test_wide_fused_step_on_stream_gemm_matches_the_cublas_path(rows, intermediate):
    """Steps of 17 to 64 rows (and smaller ones of models the skinny kernel does not take): this package's tcgen05 GEMMs (fused norm, residual and relu^2 epilogues) against the
    same steps with cuBLAS GEMMs and separate norm kernels, three teacher-forced positions per slot."""
    cfg = DecoderConfig(n_layers=3, hidden=512, n_heads=4, n_kv_heads=2, intermediate=intermediate, vocab=384,
                        max_len=64)
    w = DecoderWeights.random_init(cfg, seed=21, device="cuda", std=0.05 if intermediate == 1024 else 0.02)
    ours, ref = Decoder(cfg, w, rows), Decoder(cfg, w, rows)
    assert ours.gemm_kernel(rows) == "stream"  # also for few rows when the MLP is too deep for the skinny kernel
    ref.use_stream_gemm = False
    assert not ref.fused_supported(rows)
    gen = torch.Generator().manual_seed(rows)
    slot_map = torch.arange(rows, dtype=torch.int32, device="cuda")
    pos = torch.zeros(rows, dtype=torch.int32, device="cuda")
    buf = ours.fused_buffers(rows)
    for t in range(3):
        tok = torch.randint(0, cfg.vocab, (rows,), generator=gen).cuda()
        got = ours.fused_step(tok.clone(), pos, slot_map, t + 1, buf, choose=False).clone()
        want = ref.logits_rows(tok, pos.clone(), slot_map, t + 1)
        pos.add_(1)
        err = (got - want).abs()
        scale = float(want.abs().max())
        # the two differ by bf16 roundings of every activation (here the norm scales the fp32 product instead of
        # rounding the normed input), which three layers turn into about 0.3 % of the largest logit
        assert err.max() < 3e-2 * max(scale, 1.0) and err.mean() < 5e-3 * max(scale, 1.0), (t, float(err.max()), scale)
    for a, b in zip(ours.caches, ref.caches):  # appended bytes only differ where a bf16 input rounded differently
        same = (a.pages == b.pages).float().mean()
        assert same > 0.98, float(same)
    assert int(ours.status.item()) == 0
