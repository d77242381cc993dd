"""The KV-length-sharded path on real GPUs: two NCCL ranks each hold a slice of every sequence, attend locally
through the C ABI, all-gather the states and merge. Needs two GPUs; skipped otherwise."""

import os
import socket

import numpy as np  # noqa: F401  (used inside the spawned worker)
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import helpers

pytestmark = pytest.mark.gpu


def worker(rank: int, world: int, port: int, result):
    import nanochat_b200 as ncb
    from nanochat_b200 import sharding
    from oracle import attention as oat

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        Hq, Hkv, lens = 16, 4, [3000, 200, 64, 1]
        case = helpers.attention_case(88, Hq, Hkv, lens)
        local = [sharding.kv_slices(n, world)[rank] for n in lens]
        local_lens = [e - a for a, e in local]
        cache = ncb.Fp8KVCache(len(lens), Hkv, max(max(local_lens), 1))
        for b, (a, e) in enumerate(local):
            if e > a:
                cache.write(b, *(torch.from_numpy(case[k][b][:, a:e]) for k in ("k_bytes", "k_scale", "v_bytes", "v_scale")))
        q = helpers.bits_bf16(case["q"]).cuda()
        lens_t = torch.tensor(local_lens, dtype=torch.int32, device="cuda")
        out = sharding.attend_kv_sharded(q, cache, lens_t, max(max(local_lens), 1))
        torch.cuda.synchronize()
        want = oat.decode_attention(case["q"], case["k_bytes"], case["k_scale"], case["v_bytes"], case["v_scale"],
                                    128 ** -0.5)
        result.put((rank, *helpers.error_stats(helpers.bf16_bits(out.cpu()), want)))
        # the fused exchange + merge over peer memory, several calls in a row (the two state buffers alternate)
        peers = sharding.PeerStates(len(lens), Hq)
        for _ in range(5):
            fused = sharding.attend_kv_sharded_fused(q, cache, lens_t, max(max(local_lens), 1), peers)
        torch.cuda.synchronize()
        assert int(peers.status.item()) == 0
        result.put((rank, *helpers.error_stats(helpers.bf16_bits(fused.cpu()), helpers.bf16_bits(out.cpu()))))
        # decoding on: every step the rank that owns a sequence's tail appends the new token (at its local
        # position), then all ranks attend; the checker appends to the whole sequence
        from oracle import kv_append as okv
        gen = torch.Generator().manual_seed(99)  # the same new tokens on every rank
        cos, sin = ncb.rotary_table(4096, 1e4)
        ones = torch.ones(128)
        grown = ncb.Fp8KVCache(len(lens), Hkv, max(max(local_lens), 1) + 64)
        grown.pages[:, :, :cache.pages_per_slot].copy_(cache.pages)
        slices = [sharding.kv_slices(n, world) for n in lens]
        total = list(lens)
        for step in range(3):
            qkv = torch.randn(len(lens), (Hq + 2 * Hkv) * 128, generator=gen).bfloat16()
            pos = torch.tensor(total, dtype=torch.int32)
            want_new = okv.kv_append(helpers.bf16_bits(qkv), ones.numpy(), ones.numpy(), cos.numpy(), sin.numpy(),
                                     pos.numpy(), Hq, Hkv)
            mine = [b for b in range(len(lens)) if sharding.append_owner(total[b], slices[b]) == rank]
            if mine:
                # the owner writes at its local position but must rotate by the global one: it passes the rotary
                # table shifted by its slice's first position, so table row (local position) = global position
                for b in mine:
                    begin = slices[b][rank][0]
                    local_pos = torch.tensor([total[b] - begin], dtype=torch.int32, device="cuda")
                    ncb.kv_append(qkv[b:b + 1].cuda(), ones.cuda(), ones.cuda(), cos[begin:total[b] + 1].contiguous().cuda(),
                                  sin[begin:total[b] + 1].contiguous().cuda(), local_pos, grown, Hq,
                                  slot_map=torch.tensor([b], dtype=torch.int32, device="cuda"))
                    slices[b][rank] = (begin, total[b] + 1)
                    local_lens[b] += 1
            for b in range(len(lens)):
                total[b] += 1
                for key in ("k_bytes", "v_bytes"):
                    case[key][b] = np.concatenate([case[key][b], want_new[key][b][:, None]], axis=1)
                for key in ("k_scale", "v_scale"):
                    case[key][b] = np.concatenate([case[key][b], want_new[key][b][:, None]], axis=1)
            q_new = helpers.bits_bf16(want_new["q"]).cuda()
            lens_t = torch.tensor(local_lens, dtype=torch.int32, device="cuda")
            got = sharding.attend_kv_sharded_fused(q_new, grown, lens_t, max(local_lens), peers)
            torch.cuda.synchronize()
            want = oat.decode_attention(want_new["q"], case["k_bytes"], case["k_scale"], case["v_bytes"],
                                        case["v_scale"], 128 ** -0.5)
            result.put((rank, *helpers.error_stats(helpers.bf16_bits(got.cpu()), want)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_kv_length_sharded_attention_two_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    mp.spawn(worker, args=(2, port, result), nprocs=2, join=True)
    for _ in range(10):  # per rank: NCCL path vs checker, fused path vs NCCL path, three decode steps vs checker
        rank, max_abs, mean_abs = result.get(timeout=10)
        assert max_abs <= 2e-2 and mean_abs <= 2e-3, (rank, max_abs, mean_abs)
