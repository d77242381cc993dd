"""The KV-length-sharded path on real GPUs: two NCCL ranks each hold a slice of every sequence, attend locally
through the C ABI, all-gather the states and merge. Needs two GPUs; skipped otherwise."""

import os
import socket

import numpy as np
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
    for _ in range(4):  # per rank: NCCL path vs checker, then fused path vs NCCL path
        rank, max_abs, mean_abs = result.get(timeout=10)
        assert max_abs <= 2e-2 and mean_abs <= 2e-3, (rank, max_abs, mean_abs)
