"""decode_attn_fp8 on the GPU, through the C ABI, against the float64 checker (oracle/attention.py) and the
committed outputs of the reference's own attention function. Tolerance on bf16 outputs: max-abs 2e-2, mean-abs
2e-3 (the path's stated bound); the kernel is also held to a tighter internal bound against the float64 checker."""

from pathlib import Path

import numpy as np
import pytest
import torch

import nanochat_b200 as ncb
from oracle import attention as oat
from oracle import kv_append as okv
from tests import helpers

pytestmark = pytest.mark.gpu
GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_vectors.npz")
MAX_ABS, MEAN_ABS = 2e-2, 2e-3       # the path's tolerance
TIGHT_MAX, TIGHT_MEAN = 6e-3, 4e-4   # what the two-term e4m3 split should hold against the float64 checker
SCALE = 128 ** -0.5


def load_cache(case, max_len, slots=None, n_slots=None):
    B = len(case["lens"])
    slots = list(range(B)) if slots is None else slots
    cache = ncb.Fp8KVCache(n_slots or (max(slots) + 1), case["Hkv"], max_len)
    for b, slot in enumerate(slots):
        if case["lens"][b]:
            cache.write(slot, *(torch.from_numpy(case[k][b]) for k in ("k_bytes", "k_scale", "v_bytes", "v_scale")))
    return cache


def run(case, max_len=None, window=0, chunk_pages=0, slots=None, n_slots=None, poison=False):
    lens = case["lens"]
    max_len = max_len or max(max(lens), 1)
    cache = load_cache(case, max_len, slots, n_slots)
    if poison:  # bytes and scales past each sequence's end become NaN patterns: they must never reach the output
        for b, n in enumerate(lens):
            slot = b if slots is None else slots[b]
            tail = cache.capacity - n
            if tail:
                nan_b = torch.full((case["Hkv"], tail, 128), 0x7f, dtype=torch.uint8)
                nan_s = torch.full((case["Hkv"], tail), float("nan"))
                cache.write(slot, nan_b, nan_s, nan_b, nan_s, start=n)
    q = helpers.bits_bf16(case["q"]).cuda()
    lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
    slot_map = None if slots is None else torch.tensor(slots, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ncb.decode_attention(q, cache, lens_t, max_kv_len=max(lens), slot_map=slot_map, window=window,
                               chunk_pages=chunk_pages, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    return helpers.bf16_bits(out.cpu())


def check(case, got, window=0, tight=True):
    """The path's tolerance holds for outputs of magnitude <= 1 (every benchmark configuration); larger outputs
    scale both bounds, since one bf16 rounding step at magnitude 16 already exceeds 2e-2."""
    want = oat.decode_attention(case["q"], case["k_bytes"], case["k_scale"], case["v_bytes"], case["v_scale"], SCALE,
                                window=window)
    max_abs, mean_abs = helpers.error_stats(got, want)
    assert np.isfinite(max_abs), "non-finite output"
    ref = max(1.0, float(np.abs(okv.bf16_to_f32(want)).max()))
    assert max_abs <= MAX_ABS * ref and mean_abs <= MEAN_ABS * ref, (max_abs, mean_abs, ref)
    if tight:
        assert max_abs <= TIGHT_MAX * ref and mean_abs <= TIGHT_MEAN * ref, (max_abs, mean_abs, ref)
    return max_abs, mean_abs


def test_config0_against_checker_and_reference_output():
    """Batch 1, 10 heads, 1024 positions, seed 0: the reference-runnable configuration."""
    case = helpers.attention_case(0, 10, 10, [1024])
    got = run(case)
    check(case, got)
    max_abs, mean_abs = helpers.error_stats(got, GOLDEN["attn_cfg0_out"])
    assert max_abs <= MAX_ABS and mean_abs <= MEAN_ABS, (max_abs, mean_abs)


def test_gqa_against_reference_output():
    case = helpers.attention_case(2, 8, 2, [300, 77])
    got = run(case)
    check(case, got)
    max_abs, mean_abs = helpers.error_stats(got, GOLDEN["attn_gqa_out"])
    assert max_abs <= MAX_ABS and mean_abs <= MEAN_ABS, (max_abs, mean_abs)


@pytest.mark.parametrize("n", [1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 383, 384, 385, 1000])
def test_length_edges(n):
    case = helpers.attention_case(100 + n, 8, 2, [n])
    check(case, run(case, poison=True))


@pytest.mark.parametrize("Hq,Hkv", [(1, 1), (2, 2), (2, 1), (4, 1), (8, 1), (6, 2), (12, 4), (32, 8), (16, 4), (10, 10)])
def test_head_ratios(Hq, Hkv):
    case = helpers.attention_case(200 + Hq * 10 + Hkv, Hq, Hkv, [150, 64, 1, 500])
    check(case, run(case, poison=True))


@pytest.mark.parametrize("chunk_pages", [1, 2, 3, 7, 64])
def test_split_sizes_agree(chunk_pages):
    case = helpers.attention_case(300, 8, 2, [900, 64, 129, 5])
    check(case, run(case, chunk_pages=chunk_pages, poison=True))


@pytest.mark.parametrize("window", [1, 5, 63, 64, 65, 200, 10000])
def test_window_edges(window):
    case = helpers.attention_case(400 + window, 8, 2, [300, 64, 3, 129])
    check(case, run(case, window=window, chunk_pages=2, poison=True), window=window)


def test_ragged_batch_with_slot_map_and_empty_sequence():
    lens = [0, 17, 640, 64, 1, 333]
    case = helpers.attention_case(500, 16, 4, lens)
    got = run(case, max_len=700, slots=[5, 0, 3, 1, 4, 2], n_slots=6, poison=True)
    check(case, got)
    assert not got[0].any(), "an empty sequence gives a zero row"


def test_scale_extremes():
    """A zero V row, a zero K row, one dominant V scale and one tiny one."""
    case = helpers.attention_case(600, 4, 1, [200])
    case["v_bytes"][0][0, 10] = 0
    case["v_scale"][0][0, 10] = 0
    case["k_bytes"][0][0, 11] = 0
    case["k_scale"][0][0, 11] = 0
    case["v_scale"][0][0, 12] *= 1000
    case["v_scale"][0][0, 13] *= 1e-6
    case["k_scale"][0][0, 14] *= 8
    check(case, run(case), tight=False)


def test_peaked_attention():
    """One key aligned with the query dominates the softmax."""
    case = helpers.attention_case(700, 4, 1, [300])
    q = okv.bf16_to_f32(case["q"][0, 0])
    b, s = okv.quant_rows(okv.f32_to_bf16(q * 3)[None])
    case["k_bytes"][0][0, 123], case["k_scale"][0][0, 123] = b[0], s[0]
    check(case, run(case))


def test_out_of_range_length_is_flagged_and_zeroed():
    case = helpers.attention_case(800, 4, 2, [64, 64])
    cache = load_cache(case, 64)
    q = helpers.bits_bf16(case["q"]).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lens = torch.tensor([64, 65], dtype=torch.int32, device="cuda")  # 65 > capacity 64
    out = ncb.decode_attention(q, cache, lens, max_kv_len=64, status=status)
    torch.cuda.synchronize()
    assert status.item() == 4
    assert not helpers.bf16_bits(out.cpu())[1].any()
    check({**case, "lens": [64], "q": case["q"][:1], "k_bytes": case["k_bytes"][:1], "k_scale": case["k_scale"][:1],
           "v_bytes": case["v_bytes"][:1], "v_scale": case["v_scale"][:1]}, helpers.bf16_bits(out.cpu())[:1])


def test_partial_states_merge_to_the_whole():
    """A sequence cut into slices held by different caches (as ranks would hold them): per-slice states merged by
    decode_attn_merge equal attention over the whole."""
    n, cuts = 1500, [0, 400, 400, 1100, 1500]  # includes an empty slice
    case = helpers.attention_case(900, 8, 2, [n, 700])
    q = helpers.bits_bf16(case["q"]).cuda()
    parts = []
    for a, b in zip(cuts[:-1], cuts[1:]):
        sl = {**case, "lens": [max(0, min(b, L) - min(a, L)) for L in case["lens"]]}
        for key in ("k_bytes", "k_scale", "v_bytes", "v_scale"):
            sl[key] = [x[:, a:b] for x in case[key]]
        cache = load_cache(sl, max(max(sl["lens"]), 1))
        lens = torch.tensor(sl["lens"], dtype=torch.int32, device="cuda")
        parts.append(ncb.decode_attention_partial(q, cache, lens, max_kv_len=max(max(sl["lens"]), 1)))
    out = ncb.merge_partials(torch.stack(parts))
    torch.cuda.synchronize()
    check(case, helpers.bf16_bits(out.cpu()))


def test_append_then_attend():
    """The step as the decoder runs it: kv_append_fp8 writes the new token, decode_attn_fp8 reads it back. Checked
    against the oracles chained the same way."""
    gen = torch.Generator().manual_seed(1000)
    Hq, Hkv, B, T = 8, 2, 3, 70
    cos, sin = ncb.rotary_table(128, 1e4)
    ones = torch.ones(128)
    cache = ncb.Fp8KVCache(B, Hkv, 128)
    logical = {k: [[] for _ in range(B)] for k in ("k_bytes", "k_scale", "v_bytes", "v_scale")}
    for t in range(T):
        qkv = torch.randn(B, (Hq + 2 * Hkv) * 128, generator=gen).bfloat16()
        pos = torch.full((B,), t, dtype=torch.int32)
        q = ncb.kv_append(qkv.cuda(), ones.cuda(), ones.cuda(), cos.cuda(), sin.cuda(), pos.cuda(), cache, Hq)
        want = okv.kv_append(helpers.bf16_bits(qkv), ones.numpy(), ones.numpy(), cos.numpy(), sin.numpy(),
                             pos.numpy(), Hq, Hkv)
        for b in range(B):
            for key in logical:
                logical[key][b].append(want[key][b])
    lens = torch.full((B,), T, dtype=torch.int32, device="cuda")
    out = ncb.decode_attention(q, cache, lens, max_kv_len=T)
    torch.cuda.synchronize()
    assert np.array_equal(helpers.bf16_bits(q.cpu()), want["q"])
    case = {"q": want["q"], "lens": [T] * B, "Hq": Hq, "Hkv": Hkv}
    for key in logical:
        case[key] = [np.stack(logical[key][b], axis=1) for b in range(B)]
    check(case, helpers.bf16_bits(out.cpu()))


@pytest.mark.parametrize("lens,parts", [([130, 5, 64], 0), ([130, 5, 64, 200], 2), ([130, 5, 64, 200, 1, 77, 63, 128], 4)])
def test_decode_step_graph_matches_eager_operators(lens, parts):
    """DecodeStep (copies + append + attention as one CUDA graph, pinned host buffers; the rows in 1, 2 or 4 groups
    that run as parallel branches of the graph) against the same operators called one by one, over several steps of
    a growing ragged batch."""
    gen = torch.Generator().manual_seed(1200)
    Hq, Hkv = 8, 2
    B = len(lens)
    case = helpers.attention_case(1201, Hq, Hkv, lens)
    cos, sin = ncb.rotary_table(256, 1e4, device="cuda")
    gain = (1 + 0.1 * torch.randn(128, generator=gen)).cuda()
    caches = [load_cache(case, 256) for _ in range(2)]
    step = ncb.DecodeStep(caches[0], Hq, cos, sin, gain, gain, B, parts=parts)
    assert step.parts == (parts or 1)
    pos = torch.tensor(lens, dtype=torch.int32)
    for _ in range(4):
        qkv = torch.randn(B, (Hq + 2 * Hkv) * 128, generator=gen).bfloat16()
        step.qkv_host.copy_(qkv)
        step.pos_host.copy_(pos)
        step.run()
        q = ncb.kv_append(qkv.cuda(), gain, gain, cos, sin, pos.cuda(), caches[1], Hq)
        want = ncb.decode_attention(q, caches[1], (pos + 1).cuda(), max_kv_len=int(pos.max()) + 1)
        torch.cuda.synchronize()
        assert torch.equal(step.out_host, want.cpu())
        pos += 1
    step.check()
    assert torch.equal(caches[0].pages, caches[1].pages)


@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (10, 10), (8, 1)])
def test_fused_append_attention_equals_the_two_kernels(Hq, Hkv):
    """decode_step_attn_fp8 (the attention kernel appends its own token) against kv_append_fp8 + decode_attn_fp8 over
    several steps, across page and chunk boundaries, with a window and a slot map: same cache bytes, same outputs."""
    gen = torch.Generator().manual_seed(1300 + Hq)
    lens = [62, 127, 5, 300]
    B = len(lens)
    case = helpers.attention_case(1301, Hq, Hkv, lens)
    slots = [2, 0, 3, 1]
    cos, sin = ncb.rotary_table(384, 1e4, device="cuda")
    gain = (1 + 0.1 * torch.randn(128, generator=gen)).cuda()
    caches = [load_cache(case, 384, slots=slots, n_slots=4) for _ in range(2)]
    slot_map = torch.tensor(slots, dtype=torch.int32, device="cuda")
    pos = torch.tensor(lens, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    table = (torch.randn(40, Hkv * 128, generator=gen) * 0.7).bfloat16().cuda()
    gate = (torch.randn(Hkv, 512, generator=gen) * 0.1).float().cuda()
    for step in range(5):
        qkv = torch.randn(B, (Hq + 2 * Hkv) * 128, generator=gen).bfloat16().cuda()
        window = 0 if step % 2 == 0 else 100
        ve = None
        if step >= 3:  # the last steps with the value-embedding mix on v
            ve = ncb.attention.ValueEmbed(torch.randn(B, 512, generator=gen).bfloat16().cuda(),
                                          torch.randint(0, 40, (B,), generator=gen).cuda(), table, gate)
        got = ncb.decode_step_attention(qkv, gain, gain, cos, sin, pos, caches[0], Hq, int(pos.max()) + 1,
                                        slot_map=slot_map, window=window, chunk_pages=2, status=status, ve=ve)
        q = ncb.kv_append(qkv, gain, gain, cos, sin, pos, caches[1], Hq, slot_map=slot_map, status=status, ve=ve)
        want = ncb.decode_attention(q, caches[1], pos + 1, int(pos.max()) + 1, slot_map=slot_map, window=window,
                                    chunk_pages=2, status=status)
        torch.cuda.synchronize()
        assert torch.equal(caches[0].pages, caches[1].pages), f"step {step}: cache bytes differ"
        assert torch.equal(got, want), f"step {step}: outputs differ"
        pos += 1
    assert status.item() == 0
    # an out-of-range position is refused and flagged, and its row comes back as zeros
    bad = pos.clone()
    bad[1] = 384
    qkv = torch.randn(B, (Hq + 2 * Hkv) * 128, generator=gen).bfloat16().cuda()
    before = caches[0].pages.clone()
    out = ncb.decode_step_attention(qkv, gain, gain, cos, sin, bad, caches[0], Hq, 384, slot_map=slot_map, status=status)
    torch.cuda.synchronize()
    assert status.item() == 1 and not out[1].any()
    assert torch.equal(caches[0].pages[0], before[0])  # slot 0 belongs to the refused row
    # a position inside the cache but past the rotary table is refused the same way: zeros, not stale states
    status.zero_()
    bad = pos.clone()
    bad[1] = 320
    out = torch.full((B, Hq, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    ncb.decode_step_attention(qkv, gain, gain, cos[:320].contiguous(), sin[:320].contiguous(), bad, caches[0], Hq, 384,
                              slot_map=slot_map, chunk_pages=2, out=out, status=status)
    torch.cuda.synchronize()
    assert status.item() == 1 and not out[1].any() and torch.isfinite(out.float()).all()
    assert torch.equal(caches[0].pages[0], before[0])
    # idle rows (negative position): no append, a zero output row, nothing flagged; the other rows as usual
    status.zero_()
    idle = pos.clone()
    idle[0] = idle[2] = -1
    before = caches[0].pages.clone()
    out = ncb.decode_step_attention(qkv, gain, gain, cos, sin, idle, caches[0], Hq, int(pos.max()) + 1,
                                    slot_map=slot_map, chunk_pages=2, status=status)
    q = ncb.kv_append(qkv, gain, gain, cos, sin, idle, caches[1], Hq, slot_map=slot_map, status=status)
    want = ncb.decode_attention(q, caches[1], torch.where(idle < 0, idle, idle + 1), int(pos.max()) + 1,
                                slot_map=slot_map, chunk_pages=2, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0 and not out[0].any() and not out[2].any() and out[1].any() and out[3].any()
    assert torch.equal(out, want)
    for b in (0, 2):
        assert torch.equal(caches[0].pages[slots[b]], before[slots[b]])


PACKET_WORDS = 132  # NCB_PEER_STATE_BYTES / 8


def packets(states: torch.Tensor, call: int) -> torch.Tensor:
    """(rows, 132) fp32 states (m, l, 0, 0, o[128]) -> (rows, PACKET_WORDS, 2) int32 inbox words: (value bits, call
    number) for o[0..127], then m, then l; the rest stays zero."""
    rows = states.shape[0]
    out = torch.zeros((rows, PACKET_WORDS, 2), dtype=torch.int32, device=states.device)
    bits = states.view(torch.int32)
    out[:, :128, 0] = bits[:, 4:]
    out[:, 128, 0], out[:, 129, 0] = bits[:, 0], bits[:, 1]
    out[:, :130, 1] = call
    return out


class _OneGpuPeers:
    """The buffers of `world` 'ranks' of decode_attn_fp8_sharded, all on this GPU: per rank an inbox
    [2][world][rows][PACKET_WORDS] of 8-byte words, plus rank 0's call counter."""

    def __init__(self, world, rows):
        import ctypes
        self.world, self.rows = world, rows
        self.inbox = [torch.zeros((2, world, rows, PACKET_WORDS, 2), dtype=torch.int32, device="cuda") for _ in range(world)]
        self.epoch = torch.zeros(2, dtype=torch.int32, device="cuda")
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.p_inbox = (ctypes.c_void_p * world)(*(t.data_ptr() for t in self.inbox))

    def call(self, q, cache, lens, max_kv_len, rank=0, chunk_pages=2):
        from nanochat_b200.native import cuda_library, pointer, stream
        B, Hq = q.shape[0], q.shape[1]
        need = ncb.workspace_bytes(B, Hq, cache.kv_heads, max_kv_len, chunk_pages)
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        out = torch.full_like(q, float("nan"))
        rc = cuda_library("decode_attn").decode_attn_fp8_sharded(
            pointer(q), pointer(cache.pages), pointer(lens), None, pointer(workspace), workspace.numel(), pointer(out),
            B, Hq, cache.kv_heads, cache.n_slots, cache.pages_per_slot, max_kv_len, 0, chunk_pages, SCALE,
            self.p_inbox, self.world, rank, pointer(self.epoch), pointer(self.status), stream())
        return rc, out


def test_sharded_exchange_on_one_gpu_with_the_peer_already_delivered():
    """decode_attn_fp8_sharded as rank 0 of two 'ranks' whose inboxes both live on this GPU; the peer's words for the
    call are planted beforehand, so no kernel waits for another. The result equals decode_attn_merge over the two
    slices' states bit for bit, the kernel delivers its own state to the peer's inbox (not to its own), advances the
    call counter, and the next call uses the inbox's other half."""
    n, cuts = 700, [0, 320, 700]
    case = helpers.attention_case(1400, 8, 2, [n, 100])
    q = helpers.bits_bf16(case["q"]).cuda()
    parts, caches, lens_of = [], [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        sl = {**case, "lens": [max(0, min(b, L) - min(a, L)) for L in case["lens"]]}
        for key in ("k_bytes", "k_scale", "v_bytes", "v_scale"):
            sl[key] = [x[:, a:b] for x in case[key]]
        cache = load_cache(sl, max(max(sl["lens"]), 1))
        lens = torch.tensor(sl["lens"], dtype=torch.int32, device="cuda")
        parts.append(ncb.decode_attention_partial(q, cache, lens, max_kv_len=max(max(sl["lens"]), 1), chunk_pages=2))
        caches.append(cache)
        lens_of.append(lens)
    want = ncb.merge_partials(torch.stack(parts))
    rows = 2 * 8
    peers = _OneGpuPeers(2, rows)
    for call in (1, 2, 3):
        peers.inbox[0][call % 2, 1] = packets(parts[1].view(rows, 132), call)  # rank 1's states, in rank 0's inbox
        rc, out = peers.call(q, caches[0], lens_of[0], 320)
        torch.cuda.synchronize()
        assert rc == 0 and peers.status.item() == 0
        assert torch.equal(out, want), call
        assert peers.epoch.tolist() == [call, 0]
        # its own states went to the peer's inbox, into the half of the call's parity, and not into its own
        assert torch.equal(peers.inbox[1][call % 2, 0], packets(parts[0].view(rows, 132), call))
        assert not peers.inbox[0][:, 0].any()
    # a word left by call 1 in the same half must not pass for call 3: checked above (call 3 re-planted); here a stale
    # half alone makes the wait run out instead of merging old data
    check(case, helpers.bf16_bits(out.cpu()))


@pytest.mark.parametrize("world,rank", [(4, 1), (8, 0), (8, 5), (8, 7)])
def test_sharded_exchange_as_any_rank_of_a_larger_world(world, rank):
    """The same stand-in for worlds of four and eight: this GPU plays `rank`, the other ranks' words are planted in
    its inbox. The output equals decode_attn_merge over all slices' states in rank order (what every rank computes, so
    all ranks agree bit for bit), and its own state lands in every peer's inbox at its own rank's place."""
    n = 64 * 3 * world + 37
    cuts = [0] + [64 * 3 * (r + 1) for r in range(world - 1)] + [n]
    case = helpers.attention_case(1410 + world + rank, 8, 2, [n, 250])
    q = helpers.bits_bf16(case["q"]).cuda()
    parts, caches, lens_of = [], [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        sl = {**case, "lens": [max(0, min(b, L) - min(a, L)) for L in case["lens"]]}
        for key in ("k_bytes", "k_scale", "v_bytes", "v_scale"):
            sl[key] = [x[:, a:b] for x in case[key]]
        cache = load_cache(sl, max(max(sl["lens"]), 1))
        lens = torch.tensor(sl["lens"], dtype=torch.int32, device="cuda")
        parts.append(ncb.decode_attention_partial(q, cache, lens, max_kv_len=max(max(sl["lens"]), 1), chunk_pages=2))
        caches.append(cache)
        lens_of.append(lens)
    want = ncb.merge_partials(torch.stack(parts))
    rows = 2 * 8
    peers = _OneGpuPeers(world, rows)
    for call in (1, 2):
        for r in range(world):
            if r != rank:
                peers.inbox[rank][call % 2, r] = packets(parts[r].view(rows, 132), call)
        rc, out = peers.call(q, caches[rank], lens_of[rank], cuts[rank + 1] - cuts[rank], rank=rank)
        torch.cuda.synchronize()
        assert rc == 0 and peers.status.item() == 0
        assert torch.equal(out, want), call
        for r in range(world):
            if r != rank:
                assert torch.equal(peers.inbox[r][call % 2, rank], packets(parts[rank].view(rows, 132), call))
    check(case, helpers.bf16_bits(out.cpu()))


def test_sharded_exchange_wait_runs_out_and_reports():
    """A peer that never delivers, and one whose words are from an older call: the bounded wait gives up after about
    half a second, the status word carries NCB_DEV_WAIT_TIMEOUT, the call counter still advances and the context stays
    usable."""
    import time
    case = helpers.attention_case(1401, 4, 2, [70])
    cache = load_cache(case, 128)
    q = helpers.bits_bf16(case["q"]).cuda()
    lens = torch.tensor([70], dtype=torch.int32, device="cuda")
    peers = _OneGpuPeers(2, 4)
    peers.inbox[0][1, 1] = packets(torch.zeros((4, 132), device="cuda"), 7)  # stale: some other call's number
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc, _ = peers.call(q, cache, lens, 128)
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert rc == 0 and peers.status.item() == 2
    assert 0.05 < waited < 10.0
    assert peers.epoch.tolist() == [1, 0]
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0  # the device still answers


@pytest.mark.parametrize("Hq,Hkv", [(10, 10), (8, 2), (4, 1), (16, 2), (10, 2), (16, 1)])
def test_prefill_attention_groups_rows_and_matches_the_row_wise_path(Hq, Hkv):
    """prefill_attn_fp8 (a tile of a prompt's rows shares each page load; every warp owns its rows over the whole key
    range) against decode_attn_fp8 run row by row and against the float64 checker: causal prefixes of three prompts
    of different lengths in one pass, tile and warp boundaries in the middle of prompts and across page edges."""
    lens = [150, 9, 200]
    case = helpers.attention_case(1500 + Hq, Hq, Hkv, lens)
    cache = load_cache(case, 256, slots=[2, 0, 1], n_slots=3)
    for slot, n in zip([2, 0, 1], lens):  # NaN patterns past each prompt's end must never reach an output
        tail = cache.capacity - n
        cache.write(slot, torch.full((Hkv, tail, 128), 0x7f, dtype=torch.uint8), torch.full((Hkv, tail), float("nan")),
                    torch.full((Hkv, tail, 128), 0x7f, dtype=torch.uint8), torch.full((Hkv, tail), float("nan")), start=n)
    gen = torch.Generator().manual_seed(1501)
    slots, positions = [], []
    for slot, n in zip([2, 0, 1], lens):
        slots += [slot] * n
        positions += list(range(n))
    rows = len(slots)
    q = torch.randn(rows, Hq, 128, generator=gen).bfloat16().cuda()
    slot_map = torch.tensor(slots, dtype=torch.int32, device="cuda")
    lens_t = torch.tensor(positions, dtype=torch.int32, device="cuda") + 1
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    plan = ncb.attention.PrefillPlan(slots, positions, Hq, cache, "cuda")
    got = ncb.attention.prefill_attention(q, cache, plan, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    if Hq // Hkv <= 8:  # the decode kernel's limit; the two kernels round differently (f16 operands here, two-term
        # e4m3 there), so outputs may differ by one bf16 step (2^-7 relative) on top of the small absolute term
        want = ncb.decode_attention(q, cache, lens_t, max(lens), slot_map=slot_map, status=status)
        torch.cuda.synchronize()
        assert status.item() == 0
        d = (got.float() - want.float()).abs()
        assert bool((d <= 8e-3 + 2.0 ** -7 * want.float().abs()).all()) and float(d.mean()) <= 2e-4, \
            (float(d.max()), float(d.mean()))
    # a few rows against the checker: the causal prefix of each prompt
    seq_of = {2: 0, 0: 1, 1: 2}
    assert torch.isfinite(got.float()).all()
    for r in (0, 15, 16, 63, 64, 127, 128, 149, 150, 158, 159, 222, 223, 300, rows - 1):
        b, n = seq_of[slots[r]], positions[r] + 1
        ref = oat.decode_attention(helpers.bf16_bits(q[r:r + 1].cpu()), [case["k_bytes"][b][:, :n]],
                                   [case["k_scale"][b][:, :n]], [case["v_bytes"][b][:, :n]], [case["v_scale"][b][:, :n]], SCALE)
        max_abs, mean_abs = helpers.error_stats(helpers.bf16_bits(got[r:r + 1].cpu()), ref)
        assert max_abs <= 2e-2 and mean_abs <= 2e-3, (r, max_abs, mean_abs)
