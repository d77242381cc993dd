"""The benchmark configurations at their full sizes: every sequence of configurations 2 and 3 against the float64
checker, the model shapes of configurations 1 and 4 teacher-forced against the CPU decoder restatement, and
size-independent properties:

  constant V      if every cached V row of a sequence is the same vector, the output is that vector, whatever K, q
  zero K          if every K row is zero, all scores tie and the output is the mean of the V rows
  split invariance  the result does not depend on how the positions are cut into chunks, nor on cutting them into
                    slices whose states are merged afterwards (the multi-GPU path's arithmetic on one GPU)
"""

import numpy as np
import pytest
import torch

import nanochat_b200 as ncb
from oracle import attention as oat
from oracle import kv_append as okv
from tests import helpers

pytestmark = pytest.mark.gpu
SCALE = 128 ** -0.5


def synthetic_cache(lens, Hkv, seed, max_len=None):
    """Quantised N(0, 1) keys and values generated on the device (the benchmark's data)."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    cache = ncb.Fp8KVCache(len(lens), Hkv, max_len or max(lens))
    for slot, n in enumerate(lens):
        packed = []
        for _ in range(2):
            x = torch.randn(Hkv, n, 128, generator=gen, device="cuda")
            scale = x.abs().amax(-1) / 448.0
            packed += [(x / scale[..., None]).to(torch.float8_e4m3fn).view(torch.uint8), scale]
        cache.write(slot, *packed)
    return cache


def oracle_rows(cache, q, lens, rows):
    """Float64 checker outputs for the given sequences, from the cache's own logical contents. One kv head at a
    time, so that a 131,072-position sequence stays within a few hundred MB of float64."""
    out = {}
    Hkv = cache.kv_heads
    G = q.shape[1] // Hkv
    for b in rows:
        k, ks, v, vs = (t.cpu().numpy() for t in cache.read(b, lens[b]))
        qb = helpers.bf16_bits(q[b:b + 1].cpu())
        heads = [oat.decode_attention(qb[:, h * G:(h + 1) * G], [k[h:h + 1]], [ks[h:h + 1]], [v[h:h + 1]], [vs[h:h + 1]],
                                      SCALE)[0] for h in range(Hkv)]
        out[b] = np.concatenate(heads, axis=0)
    return out


def assert_all_rows_match(cache, q, lens, out, skip=()):
    """Every sequence of the batch against the float64 checker, at the path's tolerance per sequence."""
    worst = (0.0, 0.0)
    for b, want in oracle_rows(cache, q, lens, [b for b in range(len(lens)) if b not in skip]).items():
        max_abs, mean_abs = helpers.error_stats(helpers.bf16_bits(out[b:b + 1].cpu()), want[None])
        assert max_abs <= 2e-2 and mean_abs <= 2e-3, (b, lens[b], max_abs, mean_abs)
        worst = (max(worst[0], max_abs), max(worst[1], mean_abs))
    return worst


def close(a: torch.Tensor, b: torch.Tensor, max_abs=4e-3, mean_abs=2e-4):
    d = (a.float() - b.float()).abs()
    return float(d.max()) <= max_abs and float(d.mean()) <= mean_abs


def plant_constant_v(cache, slot, n, vector_bits):
    """Make every V row of `slot` the bf16 vector `vector_bits` (quantised once, the same bytes at every position)."""
    b, s = okv.quant_rows(np.tile(vector_bits[None, None], (cache.kv_heads, 1, 1)).reshape(-1, 128))
    k, ks, _, _ = cache.read(slot, n)
    v = torch.from_numpy(b).cuda().view(cache.kv_heads, 1, 128).expand(-1, n, -1).contiguous()
    vs = torch.from_numpy(s).cuda().view(cache.kv_heads, 1).expand(-1, n).contiguous()
    cache.write(slot, k, ks, v, vs)
    return okv.e4m3_to_f32(b[0]) * s[0]  # the dequantised vector


def test_gqa_sweep_at_the_target_length():
    """Configuration 2's shapes (batch 64, 32 query / 8 KV heads) with ragged lengths up to 16,384 and the
    bandwidth-target length 8,192 in the mix."""
    gen = torch.Generator().manual_seed(0)
    lens = torch.randint(512, 16385, (64,), generator=gen).tolist()
    lens[0], lens[1], lens[2], lens[3] = 8192, 16384, 512, 8191
    cache = synthetic_cache(lens, 8, seed=1)
    q = torch.randn(64, 32, 128, generator=gen).bfloat16().cuda()
    const = helpers.randn_bf16(gen, 128)
    want_const = plant_constant_v(cache, 5, lens[5], const)
    k, ks, v, vs = cache.read(6, lens[6])
    cache.write(6, k, torch.zeros_like(ks), v, vs)  # zero K scales: every score is 0
    want_mean = (okv.e4m3_to_f32(v.cpu().numpy()).astype(np.float64) * vs.cpu().numpy()[..., None]).mean(1)  # (Hkv, 128)
    lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ncb.decode_attention(q, cache, lens_t, max(lens), status=status)
    torch.cuda.synchronize()
    assert status.item() == 0 and torch.isfinite(out.float()).all()
    # properties
    assert np.abs(out[5].float().cpu().numpy() - want_const[None]).max() <= 2 ** -8 * np.abs(want_const).max() + 1e-6
    got_mean = out[6].float().cpu().numpy().reshape(8, 4, 128)
    assert np.abs(got_mean - want_mean[:, None]).max() <= 2e-3
    for chunk_pages in (5, 64):
        other = ncb.decode_attention(q, cache, lens_t, max(lens), chunk_pages=chunk_pages)
        assert close(out, other), chunk_pages
    # all 64 sequences against the float64 checker
    assert_all_rows_match(cache, q, lens, out)


def test_long_context_and_its_length_slices():
    """Configuration 3: batch 4, 131,072 positions; also cut into 8 page-aligned slices (as 8 GPUs would hold them)
    whose states are merged."""
    from nanochat_b200 import sharding
    N, B, Hq, Hkv = 131072, 4, 32, 8
    gen = torch.Generator().manual_seed(3)
    cache = synthetic_cache([N] * B, Hkv, seed=4)
    q = torch.randn(B, Hq, 128, generator=gen).bfloat16().cuda()
    const = helpers.randn_bf16(gen, 128)
    want_const = plant_constant_v(cache, 1, N, const)
    lens_t = torch.full((B,), N, dtype=torch.int32, device="cuda")
    out = ncb.decode_attention(q, cache, lens_t, N)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert np.abs(out[1].float().cpu().numpy() - want_const[None]).max() <= 2 ** -8 * np.abs(want_const).max() + 1e-6
    assert close(out, ncb.decode_attention(q, cache, lens_t, N, chunk_pages=7))
    parts = []
    for begin, end in sharding.kv_slices(N, 8):
        n = end - begin
        piece = ncb.Fp8KVCache(B, Hkv, n)
        first = begin // 64
        piece.pages.copy_(cache.pages[:, :, first:first + piece.pages_per_slot])  # slices are page-aligned
        parts.append(ncb.decode_attention_partial(q, piece, torch.full((B,), n, dtype=torch.int32, device="cuda"), n))
    merged = ncb.merge_partials(torch.stack(parts))
    torch.cuda.synchronize()
    assert close(out, merged)
    # all 4 sequences against the float64 checker, the merged slices as well
    assert_all_rows_match(cache, q, [N] * B, out)
    assert_all_rows_match(cache, q, [N] * B, merged)


def test_batched_append_at_configuration_4_shapes():
    """256 rows of a 16 query / 4 KV head model appended at ragged positions up to 8,191: bit-exact."""
    gen = torch.Generator().manual_seed(5)
    rows, Hq, Hkv, max_len = 256, 16, 4, 8192
    qkv = torch.randn(rows, (Hq + 2 * Hkv) * 128, generator=gen).bfloat16()
    pos = torch.randint(256, 8192, (rows,), generator=gen).to(torch.int32)
    pos[0], pos[1] = 8191, 0
    cos, sin = ncb.rotary_table(max_len, 1e4)
    ones = torch.ones(128)
    cache = ncb.Fp8KVCache(rows, Hkv, max_len)
    q = ncb.kv_append(qkv.cuda(), ones.cuda(), ones.cuda(), cos.cuda(), sin.cuda(), pos.cuda(), cache, Hq)
    torch.cuda.synchronize()
    want = okv.kv_append(helpers.bf16_bits(qkv), ones.numpy(), ones.numpy(), cos.numpy(), sin.numpy(), pos.numpy(), Hq, Hkv)
    assert np.array_equal(helpers.bf16_bits(q.cpu()), want["q"])
    for r in range(0, rows, 17):
        k, ks, v, vs = (t.cpu().numpy() for t in cache.read(r, 1, start=int(pos[r])))
        assert np.array_equal(k[:, 0], want["k_bytes"][r]) and np.array_equal(v[:, 0], want["v_bytes"][r])
        assert np.array_equal(ks[:, 0], want["k_scale"][r]) and np.array_equal(vs[:, 0], want["v_scale"][r])


def test_d20_decode_is_reproducible():
    """Configuration 1's model (20 layers, d_model 1280, vocab 65,536, random init), batch 8, prompt 512: two runs of
    greedy decoding give the same tokens, all inside the vocabulary, with no device status raised."""
    from nanochat_b200.decoder import Decoder, DecoderConfig, DecoderWeights
    cfg = DecoderConfig(n_layers=20, hidden=1280, n_heads=10, n_kv_heads=10, intermediate=5120, vocab=65536, max_len=640)
    dec = Decoder(cfg, DecoderWeights.random_init(cfg, 0, "cuda", on_device=True), 8)
    gen = torch.Generator().manual_seed(6)
    prompts = torch.randint(0, 65536, (8, 512), generator=gen).tolist()
    a, timing = dec.generate(prompts, 32)
    b, _ = dec.generate(prompts, 32)
    assert a == b and all(0 <= t < 65536 for row in a for t in row) and timing["tokens_per_s"] > 0


def cpu_weights(cfg: dict, seed: int):
    """Random-init bf16 weights ~ N(0, 0.02) and gains 1 on the CPU (the checker's copy); as_gpu() uploads them."""
    gen = torch.Generator().manual_seed(seed)
    C, Fd, V = cfg["hidden"], cfg["intermediate"], cfg["vocab"]
    W = (cfg["n_heads"] + 2 * cfg["n_kv_heads"]) * 128

    def w(*shape):
        return (torch.randn(*shape, generator=gen) * 0.02).bfloat16()

    layers = [{"wqkv": w(W, C), "wo": w(C, cfg["n_heads"] * 128), "wup": w(Fd, C), "wdown": w(C, Fd),
               "q_gain": torch.ones(128), "k_gain": torch.ones(128)} for _ in range(cfg["n_layers"])]
    return {"embed": w(V, C), "lm_head": w(V, C), "layers": layers}


def as_gpu(cfg: dict, w: dict, n_slots: int):
    from nanochat_b200.decoder import Decoder, DecoderConfig, DecoderWeights, LayerWeights
    dcfg = DecoderConfig(cfg["n_layers"], cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["intermediate"],
                         cfg["vocab"], cfg["rope_theta"], cfg["max_len"])
    layers = [LayerWeights(*(lw[k].cuda() for k in ("wqkv", "wo", "wup", "wdown", "q_gain", "k_gain")))
              for lw in w["layers"]]
    return Decoder(dcfg, DecoderWeights(w["embed"].cuda(), w["lm_head"].cuda(), layers), n_slots)


@torch.no_grad()
def teacher_forced_against_the_cpu_decoder(cfg, seed, rows, steps, kernel):
    """`steps` positions of `rows` sequences through the fused step (this package's GEMM kernels, append fused into
    the attention launch) and through the CPU restatement, fed the same random tokens: fp32 logits compared. The two
    differ by bf16 roundings of activations (GEMM summation order; the tcgen05 kernel applies the norm as a scale of
    the fp32 product): a one-ulp flip of a residual-stream element is 2^-9 of its value and every layer of a
    random-init model adds and amplifies such flips, so the bound scales with depth: max 2 % + 0.2 % per layer of the
    largest logit, a sixth of that on average (measured: 3 layers 0.9 % / 0.1 %, 20 layers 3.0 % / 0.5 %)."""
    from oracle.decoder import OracleDecoder
    w = cpu_weights(cfg, seed)
    dec = as_gpu(cfg, w, rows)
    assert dec.gemm_kernel(rows) == kernel
    oracle = OracleDecoder(cfg, w, n_seqs=rows)
    gen = torch.Generator().manual_seed(seed + 1)
    slot_map = torch.arange(rows, dtype=torch.int32, device="cuda")
    pos = torch.zeros(rows, dtype=torch.int32, device="cuda")
    buf = dec.fused_buffers(rows)
    for t in range(steps):
        tok = torch.randint(0, cfg["vocab"], (rows,), generator=gen)
        got = dec.fused_step(tok.cuda(), pos, slot_map, t + 1, buf, choose=False).cpu()
        pos.add_(1)
        want = oracle.step(tok, list(range(rows)))
        err = (got - want).abs()
        top = float(want.abs().max())
        bound = (2e-2 + 2e-3 * cfg["n_layers"]) * max(top, 1.0)
        assert float(err.max()) <= bound and float(err.mean()) <= bound / 6, (t, float(err.max()), float(err.mean()), top)
    assert int(dec.status.item()) == 0
    # the appended cache rows: bit-exact wherever the bf16 qkv inputs agree, which is nearly everywhere
    host = ncb.Fp8KVCache(rows, cfg["n_kv_heads"], cfg["max_len"], device="cpu", pages=dec.caches[0].pages.cpu())
    same = total = 0
    for r in range(rows):
        k, ks, v, vs = host.read(r, steps)
        c = oracle.cache[0][r]
        same += int((k.numpy() == c["k_bytes"]).sum()) + int((v.numpy() == c["v_bytes"]).sum())
        total += 2 * k.numel()
    assert same / total > 0.97, same / total


def test_d32_class_shapes_on_stream_gemm_against_the_cpu_decoder():
    """Configuration 4's model shape (d_model 2048, 16 query / 4 KV heads, MLP 8192, vocab 65,536) at 32 rows, three
    layers, through the tcgen05 stream_gemm step."""
    cfg = {"n_layers": 3, "hidden": 2048, "n_heads": 16, "n_kv_heads": 4, "intermediate": 8192, "vocab": 65536,
           "rope_theta": 10000.0, "max_len": 64}
    teacher_forced_against_the_cpu_decoder(cfg, seed=40, rows=32, steps=3, kernel="stream")


def test_d20_first_decode_steps_against_the_cpu_decoder():
    """Configuration 1's model (20 layers, d_model 1280, 10 heads, MLP 5120, vocab 65,536), two sequences, the first
    positions, through the skinny-GEMM step."""
    cfg = {"n_layers": 20, "hidden": 1280, "n_heads": 10, "n_kv_heads": 10, "intermediate": 5120, "vocab": 65536,
           "rope_theta": 10000.0, "max_len": 64}
    teacher_forced_against_the_cpu_decoder(cfg, seed=41, rows=2, steps=4, kernel="skinny")

