"""Benchmark of the decode hot path: single-token attention over the paged fp8 (e4m3) KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload target8k|ragged]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

One JSON line on rank 0. A step is one decode-attention pass (split-KV kernel + merge kernel) over one batch.

  workload  target8k: batch 64 per GPU, 32 query heads, 8 KV heads, head dim 128, every sequence 8,192 positions
            (the shapes of the GQA sweep at the length the bandwidth target is stated on); ragged: the sweep
            itself, lengths uniform in [512, 16384]. With N GPUs the global batch is 64 N sequences, assigned to
            ranks by summed length (weak scaling, no collective on the data path).
  value     whole-job algorithmic GB/s with the cache, q and lens resident in HBM:
            bytes = sum_b len_b * Hkv * 264 + B * Hq * 512 per step (K + V bytes, two fp32 scales, q in, out).
  e2e       the same metric through the public operators with HOST buffers: each step copies the new token's fused
            qkv row and positions from pinned memory, runs the append + attention kernels and copies the output
            back to pinned memory, synchronising every step. The KV cache is decoder state that lives in HBM
            between steps (as in the reference's decoder), so it is not a per-step input.
  roofline  the split-KV kernel alone (CUDA events around a loop of decode_attn_fp8_split launches on the same
            inputs) against the measured HBM copy bandwidth in MEASURED_PEAKS.json.
  cpu_baseline  the reference's CPU attention (a torch restatement of inference/modeling_nanochat.py:48-56, see
            oracle/attention.py) on a bounded sample of the same workload, all host threads.

  parity    checks made inside this run, asserted before the line is printed: one sequence per rank has a constant
            V row planted, so its output must be that vector whatever q and K are (max over ranks of the error), and
            one sequence per rank is recomputed with plain torch fp32 operators on the dequantised cache.
  ragged, longctx, decoder, decoder_d32  extras in the same line: the GQA sweep itself (ragged lengths, its own
            roofline fraction); the long-context configuration (KV split by length over the ranks; fused exchange
            against the NCCL variant on the same inputs, planted-constant-V property); greedy decode tokens/s of the
            random-init d20 model (batch 8 per GPU, 512-token prompts; at N = 1 with the CPU port of the reference's
            decoder timed beside it, `decoder.cpu_baseline`) and of the d32-class model (batch 32 per GPU, ragged
            contexts).

Every timed loop runs REPEATS times inside one invocation (each repeat: exactly --steps steps between two events,
barrier and synchronize on both sides, max over ranks); the line carries the median repeat.

--impl reference times that CPU restatement alone, on the same config and metric.
Data is synthetic: q ~ N(0,1) bf16; K, V ~ N(0,1) quantised per (token, head) with scale = amax / 448."""

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HQ, HKV, D, BATCH = 32, 8, 128, 64
METRIC, UNIT = "decode_attention_hbm_gbs", "GB/s"
REPEATS = 5
PATH_MAX_ABS, PATH_MEAN_ABS = 2e-2, 2e-3  # the path's tolerance on bf16 outputs


def profiled_traffic() -> dict | None:
    """dram__bytes_read.sum + dram__bytes_write.sum of one split-kernel launch on the target8k workload, read from
    the tracked ncu summary (its `traffic_bytes_per_launch:` line, which also names the commit it was captured at)."""
    import re

    path = ROOT / "profiles" / "decode_attn_split_target8k.md"
    if not path.exists():
        return None
    m = re.search(r"traffic_bytes_per_launch:\s*([0-9_,]+)\s*\(capture of commit ([0-9a-f]+)\)", path.read_text())
    if not m:
        return None
    return {"bytes": int(m.group(1).replace("_", "").replace(",", "")), "commit": m.group(2)}


def algorithmic_bytes(lens, Hq=HQ, Hkv=HKV) -> int:
    return sum(int(n) for n in lens) * Hkv * 264 + len(lens) * Hq * 512


def workload_lens(workload: str, n_seqs: int, seed: int = 0) -> list[int]:
    if workload == "target8k":
        return [8192] * n_seqs
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(512, 16385, (n_seqs,), generator=gen).tolist()


def peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s; MEASURED_PEAKS.json is absent)"


class ClockSampler:
    """SM clock and throttle reasons of one GPU, polled through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.003):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period, self.stop_flag, self.thread = period, threading.Event(), None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    NAMES = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
             "hw_power_brake_slowdown": 0x80, "sync_boost": 0x10}

    def poll(self):
        while not self.stop_flag.is_set():
            self.sample()
            self.stop_flag.wait(self.period)

    def sample(self):
        try:
            self.samples.append(self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
            reasons = getattr(self.nvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                self.nvml.nvmlDeviceGetCurrentClocksThrottleReasons
            bits = reasons(self.handle)
            self.reasons.update(name for name, bit in self.NAMES.items() if bits & bit)
        except Exception:
            pass

    def __enter__(self):
        if self.nvml:
            self.thread = threading.Thread(target=self.poll, daemon=True)
            self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop_flag.set()
        if self.thread:
            self.thread.join()

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def cpu_sample(lens, seed: int):
    """Logical bf16 K/V (kv heads expanded to query heads, as the reference needs) and q for a few sequences."""
    gen = torch.Generator().manual_seed(seed)
    out = []
    for n in lens:
        q = torch.randn(1, HQ, 1, D, generator=gen).bfloat16()
        kv = []
        for _ in range(2):
            x = torch.randn(HKV, n, D, generator=gen)
            scale = x.abs().amax(-1, keepdim=True) / 448.0
            deq = (x / scale).to(torch.float8_e4m3fn).float() * scale
            kv.append(deq.bfloat16().repeat_interleave(HQ // HKV, dim=0)[None])
        out.append((q, kv[0], kv[1]))
    return out


def time_cpu_reference(lens, budget_s: float, seed: int = 1234) -> dict:
    """The reference's CPU attention on `lens`, repeated for about budget_s seconds; median pass time."""
    from oracle.attention import eager_attention_port

    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    sample = cpu_sample(lens, seed)
    times = []
    deadline = time.perf_counter() + budget_s
    while len(times) < 4 or time.perf_counter() < deadline:
        t0 = time.perf_counter()
        for q, k, v in sample:
            eager_attention_port(q, k, v, D ** -0.5)
        times.append(time.perf_counter() - t0)
    warm = times[1:] if len(times) > 1 else times
    t = statistics.median(warm)
    return {"value": algorithmic_bytes(lens) / t / 1e9, "unit": UNIT, "cores": threads, "cpu": cpu_model(), "kind": "port",
            "sample": f"{len(lens)} sequences of the workload ({sum(lens)} positions), bf16 K/V dequantised outside "
                      f"the timed region, {len(warm)} timed passes, median", "seconds_per_pass": t}


def quantise_rows(x: torch.Tensor):
    """(..., 128) fp32 -> (e4m3 bytes as uint8, fp32 scale = amax / 448): the cache's quantise rule, in torch."""
    scale = x.abs().amax(-1) / 448.0
    return (x / scale[..., None]).to(torch.float8_e4m3fn).view(torch.uint8), scale


def synthetic_cache(lens, max_len: int, seed: int, device, constant_v: dict | None = None):
    """A cache filled with quantised N(0,1) keys and values, generated on the device. constant_v = {slot: vector
    fp32 (128,)} plants that vector as every V row of the slot: the slot's attention output must then be the
    (dequantised) vector, whatever q and K are: a check that needs no second implementation."""
    import nanochat_b200 as ncb

    gen = torch.Generator(device=device).manual_seed(seed)
    cache = ncb.Fp8KVCache(len(lens), HKV, max_len, device=device)
    for slot, n in enumerate(lens):
        packed = []
        for which in range(2):
            x = torch.randn(HKV, n, D, generator=gen, device=device)
            if which == 1 and constant_v and slot in constant_v:
                x = constant_v[slot].to(device).expand(HKV, n, D)
            packed += list(quantise_rows(x))
        cache.write(slot, *packed)
    return cache


def dequantised(vector: torch.Tensor) -> torch.Tensor:
    b, s = quantise_rows(vector[None])
    return (b.view(torch.float8_e4m3fn).float() * s[..., None])[0]


def torch_attention_row(cache, slot: int, n: int, q_row: torch.Tensor) -> torch.Tensor:
    """One sequence recomputed with plain torch fp32 operators on the dequantised cache: q_row (Hq, 128) bf16 ->
    (Hq, 128) fp32. The check beside the planted-vector property; not an import of the CPU checker."""
    k, ks, v, vs = cache.read(slot, n)
    K = k.view(torch.float8_e4m3fn).float() * ks[..., None]
    V = v.view(torch.float8_e4m3fn).float() * vs[..., None]
    G = q_row.shape[0] // K.shape[0]
    scores = torch.einsum("kgd,knd->kgn", q_row.float().view(K.shape[0], G, D), K) * D ** -0.5
    return torch.einsum("kgn,knd->kgd", scores.softmax(-1), V).reshape(q_row.shape[0], D)


def error_of(got: torch.Tensor, want: torch.Tensor) -> tuple[float, float]:
    d = (got.float() - want.float()).abs()
    return float(d.max()), float(d.mean())


def captured(fn, device) -> torch.cuda.CUDAGraph:
    """fn's launches as a CUDA graph: one eager run first (first-use set-up happens outside capture), then the
    capture on a side stream. Replays launch on the caller's current stream."""
    from nanochat_b200.decoder import no_collection

    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        fn()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with no_collection(), torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.current_stream(device).wait_stream(side)
    return graph


def bench_longctx(rank: int, world: int, device, steps: int, warmup: int, timed) -> dict:
    """Long-context decode attention: batch 4, Hq 32, Hkv 8, 131,072 positions per sequence. With N > 1 ranks every
    sequence's positions are cut into N page-aligned slices; each rank runs the split-KV kernel over its slice and ONE
    more kernel that merges its chunks, pushes the row states to every peer over NVLink and merges across ranks
    (decode_attn_fp8_sharded; no collective library on the data path). Total work is fixed (strong scaling). The step
    is a captured CUDA graph, as a decode loop would replay it. The NCCL variant (local merge, all-gather, merge; eager
    launches) runs on the same inputs: its time is reported and its output compared. Sequence 1 has a constant V row
    planted on every rank, so its merged output is known without gathering the slices."""
    import nanochat_b200 as ncb
    from nanochat_b200 import attention as ops
    from nanochat_b200 import sharding

    B, N = 4, 131072
    begin, end = sharding.kv_slices(N, world)[rank]
    n_local = max(end - begin, 1)
    vector = 0.25 * torch.randn(D, generator=torch.Generator().manual_seed(6100))  # the same on every rank
    cache = synthetic_cache([n_local] * B, n_local, seed=5000 + rank, device=device, constant_v={1: vector})
    gen = torch.Generator(device=device).manual_seed(6000)  # q is replicated: same seed on every rank
    q = torch.randn(B, HQ, D, generator=gen, device=device).bfloat16()
    lens_t = torch.full((B,), n_local, dtype=torch.int32, device=device)
    chunk = ops.chunk_pages_for(B, HKV, n_local)
    workspace = torch.empty(max(16, ncb.workspace_bytes(B, HQ, HKV, n_local, chunk)), dtype=torch.uint8, device=device)
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    parity, ms_nccl, peers = {}, None, None
    if world == 1:
        eager = lambda: ncb.decode_attention(q, cache, lens_t, n_local, chunk_pages=chunk, workspace=workspace, out=out,
                                             status=status)
    else:
        part = torch.empty((B, HQ, 132), dtype=torch.float32, device=device)
        nccl_step = lambda: sharding.attend_kv_sharded(q, cache, lens_t, n_local, chunk_pages=chunk,
                                                       workspace=workspace, part=part, status=status)
        ms_nccl = timed(nccl_step, steps, warmup)
        out_nccl = nccl_step().clone()
        peers = sharding.PeerStates(B, HQ)
        eager = lambda: sharding.attend_kv_sharded_fused(q, cache, lens_t, n_local, peers, out=out, chunk_pages=chunk,
                                                         workspace=workspace)
    split_only = captured(lambda: ops.decode_attention_split(q, cache, lens_t, n_local, workspace, chunk_pages=chunk,
                                                             status=status), device)
    step = captured(eager, device)
    ms = timed(step.replay, steps, warmup)
    ms_split = timed(split_only.replay, steps, warmup)
    step.replay()
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device status {int(status.item())}"
    parity["property_max_abs"], parity["property_mean_abs"] = error_of(out[1], dequantised(vector).to(device).expand(HQ, D))
    if world > 1:
        assert int(peers.status.item()) == 0, "a peer wait ran out"
        parity["fused_vs_nccl_max_abs"], parity["fused_vs_nccl_mean_abs"] = error_of(out, out_nccl)
        everyone = [torch.empty_like(out) for _ in range(world)]
        torch.distributed.all_gather(everyone, out)
        parity["ranks_bit_identical"] = all(torch.equal(everyone[0], o) for o in everyone[1:])
        assert parity["ranks_bit_identical"], "ranks disagree on the merged output"
        assert parity["fused_vs_nccl_max_abs"] <= PATH_MAX_ABS and parity["fused_vs_nccl_mean_abs"] <= PATH_MEAN_ABS, parity
    else:
        ref = torch_attention_row(cache, 0, n_local, q[0])
        parity["torch_fp32_seq0_max_abs"], parity["torch_fp32_seq0_mean_abs"] = error_of(out[0], ref)
        assert parity["torch_fp32_seq0_max_abs"] <= PATH_MAX_ABS and parity["torch_fp32_seq0_mean_abs"] <= PATH_MEAN_ABS, parity
    assert parity["property_max_abs"] <= PATH_MAX_ABS and parity["property_mean_abs"] <= PATH_MEAN_ABS, parity
    parity["tolerance"] = {"max_abs": PATH_MAX_ABS, "mean_abs": PATH_MEAN_ABS}
    total = algorithmic_bytes([N] * B)
    return {"workload": "batch 4, Hq 32, Hkv 8, head_dim 128, 131072 positions per sequence, KV split by length over "
                        f"{world} GPU(s)", "value": total / (ms * 1e-3) / 1e9, "unit": UNIT,
            "ms_per_step": ms, "steps": steps, "scaling": "strong", "chunk_pages": chunk,
            "launch": "one captured CUDA graph per step (split-KV kernel, then merge" +
                      (" + exchange kernel)" if world > 1 else " kernel)"),
            "breakdown_us": {"split_kernel_alone": ms_split * 1e3, "merge_and_exchange": (ms - ms_split) * 1e3,
                             "per_gpu_slice_bytes": algorithmic_bytes([n_local] * B)},
            "collective": None if world == 1 else "none: each rank's merge kernel pushes its fp32 [4][32][132] states "
                          "into every peer's inbox over NVLink, then waits (bounded) on per-row flags",
            "nccl_variant_ms_per_step": ms_nccl, "nccl_variant_launch": None if world == 1 else "eager launches: split, "
            "merge, all_gather_into_tensor, merge", "parity": parity}


def bench_kernels(device, timed, profile_range: str) -> dict:
    """The path's other kernels on their own, each against the measured HBM bandwidth: k_kv_append on a prefill-sized
    pass (8 prompts of 2,048 positions, the d20 head shape: 209 MB per launch, larger than L2), k_merge on the target
    shape's states, and k_merge_exchange as a world of one (its local part: chunk merge, call counter; no peer to
    wait for). `profile_range` brackets one of them with cudaProfilerStart/Stop for ncu."""
    import nanochat_b200 as ncb
    from nanochat_b200 import attention as ops
    from nanochat_b200.native import cuda_library, pointer, stream

    peak, _ = peaks()
    out = {}

    def ranged(name, fn, steps):
        if profile_range == name:
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
        ms = timed(fn, steps, 3)
        if profile_range == name:
            torch.cuda.profiler.stop()
        return ms

    # ---- append: a prefill pass
    Hq, Hkv, prompts, per = 10, 10, 8, 2048
    rows = prompts * per
    gen = torch.Generator(device=device).manual_seed(7000)
    qkv = torch.randn(rows, (Hq + 2 * Hkv) * D, generator=gen, device=device).bfloat16()
    slot_map = torch.arange(prompts, dtype=torch.int32, device=device).repeat_interleave(per)
    pos = torch.arange(per, dtype=torch.int32, device=device).repeat(prompts)
    cache = ncb.Fp8KVCache(prompts, Hkv, per, device=device)
    cos, sin = ncb.rotary_table(per, 1e4, device=device)
    ones = torch.ones(D, device=device)
    q_out = torch.empty(rows, Hq, D, dtype=torch.bfloat16, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    ms = ranged("append", lambda: ncb.kv_append(qkv, ones, ones, cos, sin, pos, cache, Hq, slot_map=slot_map, q_out=q_out,
                                                status=status), 20)
    nbytes = rows * ((Hq + 2 * Hkv) * 256 + Hq * 256 + 2 * Hkv * 132)
    out["kv_append_prefill"] = {"workload": f"{rows} rows (8 prompts x 2048 positions), Hq 10, Hkv 10", "us_per_launch": ms * 1e3,
                                "algorithmic_bytes_per_launch": nbytes, "achieved": nbytes / ms / 1e6, "unit": UNIT,
                                "frac": nbytes / ms / 1e6 / peak}
    assert int(status.item()) == 0
    del qkv, cache, q_out

    # ---- prefill attention: the rows of the same pass attend their prompts' caches (d20 heads, 8 x 511 rows)
    per = 511
    rows = prompts * per
    cache = synthetic_cache([per] * prompts, per, seed=7050, device=device) if Hkv == HKV else None
    if cache is None:
        cache = ncb.Fp8KVCache(prompts, Hkv, per, device=device)
        for slot in range(prompts):
            packed = []
            for _ in range(2):
                packed += list(quantise_rows(torch.randn(Hkv, per, D, generator=gen, device=device)))
            cache.write(slot, *packed)
    slots = [s_ for s_ in range(prompts) for _ in range(per)]
    positions = [t for _ in range(prompts) for t in range(per)]
    plan = ops.PrefillPlan(slots, positions, Hq, cache, device)
    q = torch.randn(rows, Hq, D, generator=gen, device=device).bfloat16()
    att = torch.empty_like(q)
    ms = ranged("prefill_attn", lambda: ops.prefill_attention(q, cache, plan, out=att, status=status), 20)
    pages_read = sum(-(-(min(per, g0 + plan.rows_per_block)) // 64) for g0 in range(0, per, plan.rows_per_block)) * prompts * Hkv
    nbytes = pages_read * 16896 + 2 * rows * Hq * 256
    out["prefill_attention"] = {"workload": f"{rows} rows (8 prompts x 511 positions), Hq 10, Hkv 10, causal",
                                "us_per_launch": ms * 1e3, "bytes_read_per_launch": nbytes,
                                "note": "compute-bound: every cached position is scored against up to 64 query rows per block; the "
                                        "pages (10.8 MB of cache) come from L2",
                                "flops_per_launch": 4 * D * Hq * prompts * per * (per + 1) // 2,
                                "achieved_tflops": 4 * D * Hq * prompts * per * (per + 1) // 2 / ms / 1e9}
    assert int(status.item()) == 0
    ref = torch_attention_row(cache, 3, 300, q[3 * per + 299])
    err = error_of(att[3 * per + 299], ref)
    assert err[0] <= PATH_MAX_ABS and err[1] <= PATH_MEAN_ABS, err
    del cache, q, att

    # ---- the tiled tcgen05 GEMM on a prefill pass's largest projection (4,088 rows x d20's MLP up-projection)
    from nanochat_b200.native import cuda_library as _lib
    rows, N, K = 4088, 5120, 1280
    x = torch.randn(rows, K, generator=gen, device=device).bfloat16()
    w = (torch.randn(N, K, generator=gen, device=device) * 0.02).bfloat16()
    y = torch.empty(rows, N, dtype=torch.bfloat16, device=device)

    def gemm():
        rc = _lib("tile_gemm").tile_gemm(pointer(x), pointer(w), None, pointer(y), rows, N, K, 2, pointer(status), stream())
        assert rc == 0

    ms = ranged("tile_gemm", gemm, 20)
    want = (x[:64].float() @ w.float().T).bfloat16().float().clamp_min(0).square().bfloat16()
    assert float((y[:64].float() - want.float()).abs().max()) <= 2 ** -7 * float(want.float().abs().max()) + 1e-6
    flops = 2 * rows * N * K
    tensor_peak = 1610.8
    try:
        tensor_peak = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"])
    except Exception:
        pass
    out["tile_gemm_prefill"] = {"workload": f"{rows} x {K} bf16 rows times a {N} x {K} weight matrix, relu^2 epilogue",
                                "us_per_launch": ms * 1e3, "flops_per_launch": flops, "bound": "tensor",
                                "achieved": flops / ms / 1e9, "unit": "TFLOP/s", "peak": tensor_peak,
                                "frac": flops / ms / 1e9 / tensor_peak,
                                "peak_kind": "measured cuBLAS bf16 burst (MEASURED_PEAKS.json bf16_tflops), else 1610.8"}
    assert int(status.item()) == 0
    del x, w, y

    # ---- merge and the exchange kernel's local part, on states the split kernel left for the target shape
    B, chunk = BATCH, 32
    lens = [8192] * B
    cache = synthetic_cache(lens, 8192, seed=7100, device=device)
    q = torch.randn(B, HQ, D, generator=gen, device=device).bfloat16()
    lens_t = torch.tensor(lens, dtype=torch.int32, device=device)
    workspace = torch.empty(ncb.workspace_bytes(B, HQ, HKV, 8192, chunk), dtype=torch.uint8, device=device)
    ops.decode_attention_split(q, cache, lens_t, 8192, workspace, chunk_pages=chunk, status=status)
    n_chunks = 8192 // 64 // chunk
    parts = workspace.view(torch.float32).view(B * HQ, n_chunks, 132).transpose(0, 1).contiguous()  # (parts, rows, 132)
    merged = torch.empty(B, HQ, D, dtype=torch.bfloat16, device=device)
    ms = ranged("merge", lambda: ops.merge_partials(parts.view(n_chunks, B, HQ, 132), out=merged), 50)
    nbytes = B * HQ * (n_chunks * 528 + 256)
    out["merge"] = {"workload": f"{B * HQ} rows x {n_chunks} states (the target shape's split states)", "us_per_launch": ms * 1e3,
                    "algorithmic_bytes_per_launch": nbytes, "achieved": nbytes / ms / 1e6, "unit": UNIT,
                    "frac": nbytes / ms / 1e6 / peak, "note": "a launch-latency-sized kernel: 4.8 MB per launch"}
    inbox = torch.zeros(2 * B * HQ * 1056 // 4, dtype=torch.int32, device=device)
    epoch = torch.zeros(2, dtype=torch.int32, device=device)
    import ctypes
    p_inbox = (ctypes.c_void_p * 1)(inbox.data_ptr())
    lib = cuda_library("decode_attn")

    def sharded():
        rc = lib.decode_attn_fp8_sharded(pointer(q), pointer(cache.pages), pointer(lens_t), None, pointer(workspace),
                                         workspace.numel(), pointer(merged), B, HQ, HKV, cache.n_slots, cache.pages_per_slot,
                                         8192, 0, chunk, D ** -0.5, p_inbox, 1, 0, pointer(epoch), pointer(status), stream())
        assert rc == 0

    split_only = lambda: ops.decode_attention_split(q, cache, lens_t, 8192, workspace, chunk_pages=chunk, status=status)
    ms_both = ranged("exchange", sharded, 20)
    ms_split = timed(split_only, 20, 3)
    out["merge_exchange_world1"] = {"workload": "decode_attn_fp8_sharded as a world of one on the target shape: the second "
                                                "launch merges the local chunk states, has no peer to send to or wait for, "
                                                "and advances the call counter", "us_per_step": ms_both * 1e3,
                                    "us_split_alone": ms_split * 1e3, "us_merge_exchange": (ms_both - ms_split) * 1e3}
    assert int(status.item()) == 0
    return out


def bench_decoder(rank: int, world: int, device, new_tokens: int, profile: bool = False) -> dict:
    """End-to-end greedy decode of the random-init d20 model (20 layers, d_model 1280, 10 heads, vocab 65536, bf16
    weights ~ N(0, 0.02)): batch 8 per GPU, 512-token prompts, `new_tokens` generated tokens; every rank runs its own
    batch (replicated weights, no collective), tokens/s is the sum over ranks of the decode phase."""
    import torch.distributed as dist

    from nanochat_b200.decoder import Decoder, DecoderConfig, DecoderWeights

    cfg = DecoderConfig(n_layers=20, hidden=1280, n_heads=10, n_kv_heads=10, intermediate=5120, vocab=65536,
                        rope_theta=10000.0, max_len=512 + new_tokens)
    decoder = Decoder(cfg, DecoderWeights.random_init(cfg, 0, device, on_device=True), 8, device)
    gen = torch.Generator().manual_seed(100 + rank)
    prompts = torch.randint(0, 65536, (8, 512), generator=gen).tolist()
    decoder.generate(prompts, 8)  # warm-up: graph capture, cuBLAS heuristics
    if profile:
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
    _, t = decoder.generate(prompts, new_tokens)
    if profile:
        torch.cuda.profiler.stop()
    stats = torch.tensor([t["decode_s"], t["prefill_s"]], device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    decode_s, prefill_s = stats.tolist()
    return {"workload": "random-init d20, batch 8 per GPU, prompt 512, greedy, fp8 KV cache", "new_tokens": new_tokens,
            "tokens_per_s": 8 * world * new_tokens / decode_s, "ms_per_step": decode_s / new_tokens * 1e3,
            "prefill_s": prefill_s, "scaling": "weak (replicas)"}


def bench_serving(rank: int, world: int, device) -> dict:
    """Continuous batching through the public host loop (nanochat_b200.serving.NativeDecoder.generate, the shape of
    the reference's NativeDecoder.generate): the random-init d20 model with 8 slots per GPU serves 32 greedy requests
    per GPU with prompts of 32 to 512 tokens and 32 to 96 new tokens each; slots are refilled from the queue as
    requests finish, prompts of newly started requests are prefilled between steps, one host synchronisation per step.
    tokens/s counts generated tokens over the wall time of the whole call (prefill included), max over ranks."""
    import torch.distributed as dist

    from nanochat_b200.decoder import Decoder, DecoderConfig, DecoderWeights
    from nanochat_b200.serving import NativeDecoder, Request

    cfg = DecoderConfig(n_layers=20, hidden=1280, n_heads=10, n_kv_heads=10, intermediate=5120, vocab=65536,
                        rope_theta=10000.0, max_len=640)
    server = NativeDecoder(Decoder(cfg, DecoderWeights.random_init(cfg, 0, device, on_device=True), 8, device),
                           end_token=65535)
    gen = torch.Generator().manual_seed(400 + rank)

    def requests():
        lengths = torch.randint(32, 513, (32,), generator=gen).tolist()
        budgets = torch.randint(32, 97, (32,), generator=gen).tolist()
        return [Request(input_ids=torch.randint(0, 65535, (n,), generator=gen).tolist(), max_new_tokens=m)
                for n, m in zip(lengths, budgets)]

    list(server.generate(requests()))  # warm-up: every kernel form's first use, the allocator's pools
    runs = []
    for _ in range(3):  # three different request sets; the median run is reported
        batch = requests()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        done = list(server.generate(batch))
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        first = sorted(t[1] - t[0] for t in server.timings.values())
        runs.append((seconds / max(1, sum(len(ids) for _, ids in done)), seconds, sum(len(ids) for _, ids in done),
                     first[len(first) // 2]))
    runs.sort()
    _, seconds, tokens, ttft = runs[1]
    stats = torch.tensor([seconds, float(tokens)], device=device)
    if world > 1:
        worst = stats[:1].clone()
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        dist.all_reduce(stats)
        stats[0] = worst[0]
    seconds, tokens = stats.tolist()
    return {"workload": "random-init d20, 8 slots per GPU, 32 greedy requests per GPU (prompts 32-512 tokens, 32-96 new "
                        "tokens), continuous batching through NativeDecoder.generate",
            "tokens_per_s": tokens / seconds, "generated_tokens": int(tokens), "seconds": seconds,
            "median_time_to_first_token_ms": ttft * 1e3, "scaling": "weak (replicas)"}


def bench_decoder_cpu(steps: int) -> dict:
    """The CPU port of the reference's decoder (oracle/decoder.py: the exported model's operators on torch CPU
    bf16, op for op) on the d20 workload, all host threads: batch 8, 512 positions already in the caches (synthetic
    fp8 contents), `steps` greedy steps timed after one warm-up step."""
    import numpy as np

    from oracle.decoder import OracleDecoder

    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    cfg = {"n_layers": 20, "hidden": 1280, "n_heads": 10, "n_kv_heads": 10, "intermediate": 5120, "vocab": 65536,
           "rope_theta": 10000.0, "max_len": 512 + steps + 2}
    gen = torch.Generator().manual_seed(0)
    rnd = lambda *shape: (torch.randn(*shape, generator=gen) * 0.02).bfloat16()
    C, F_, W = cfg["hidden"], cfg["intermediate"], (cfg["n_heads"] + 2 * cfg["n_kv_heads"]) * D
    weights = {"embed": rnd(cfg["vocab"], C), "lm_head": rnd(cfg["vocab"], C),
               "layers": [{"wqkv": rnd(W, C), "wo": rnd(C, cfg["n_heads"] * D), "wup": rnd(F_, C), "wdown": rnd(C, F_),
                           "q_gain": torch.ones(D), "k_gain": torch.ones(D)} for _ in range(cfg["n_layers"])]}
    oracle = OracleDecoder(cfg, weights, 8)
    rng = np.random.default_rng(0)
    for layer in oracle.cache:
        for seq in layer:
            for key in ("k", "v"):
                seq[key + "_bytes"] = rng.integers(0, 120, (cfg["n_kv_heads"], 512, D), dtype=np.uint8)
                seq[key + "_scale"] = rng.uniform(1e-3, 1e-2, (cfg["n_kv_heads"], 512)).astype(np.float32)
    tokens = torch.randint(0, cfg["vocab"], (8,), generator=gen)
    seqs = list(range(8))
    tokens = oracle.step(tokens, seqs).argmax(-1)
    t0 = time.perf_counter()
    for _ in range(steps):
        tokens = oracle.step(tokens, seqs).argmax(-1)
    dt = time.perf_counter() - t0
    return {"tokens_per_s": 8 * steps / dt, "cores": threads, "cpu": cpu_model(), "kind": "port",
            "sample": f"{steps} greedy steps of batch 8 at context 512 (one warm-up step before)"}


def bench_decoder_d32(rank: int, world: int, device, new_tokens: int, profile: bool = False) -> dict:
    """Batched decode of a random-init d32-class model (32 layers, d_model 2048, 16 query / 4 KV heads, relu^2 MLP of
    8192, vocab 65536): batch 32 per GPU (256 over 8 GPUs), ragged contexts uniform in [256, 8192] already in the fp8
    caches (synthetic quantised K/V, the same pages in every layer), `new_tokens` greedy tokens. Every step appends
    and attends in every layer; at 32 rows the GEMMs run on the tcgen05 weight-stream kernel (stream_gemm)."""
    import torch.distributed as dist

    import nanochat_b200 as ncb
    from nanochat_b200.decoder import Decoder, DecoderConfig, DecoderWeights

    B = 32
    gen = torch.Generator().manual_seed(200 + rank)
    ctx = torch.randint(256, 8193, (B,), generator=gen).tolist()
    cfg = DecoderConfig(n_layers=32, hidden=2048, n_heads=16, n_kv_heads=4, intermediate=8192, vocab=65536,
                        rope_theta=10000.0, max_len=8192 + new_tokens + 8)
    decoder = Decoder(cfg, DecoderWeights.random_init(cfg, 1, device, on_device=True), B, device)
    dgen = torch.Generator(device=device).manual_seed(300 + rank)
    filled = ncb.Fp8KVCache(B, 4, cfg.max_len, device=device)
    for slot, n in enumerate(ctx):
        packed = []
        for _ in range(2):
            x = torch.randn(4, n, D, generator=dgen, device=device)
            scale = x.abs().amax(-1) / 448.0
            packed += [(x / scale[..., None]).to(torch.float8_e4m3fn).view(torch.uint8), scale]
        filled.write(slot, *packed)
    for cache in decoder.caches:
        cache.pages.copy_(filled.pages)
    del filled
    first = torch.randint(0, 65536, (B,), generator=gen).tolist()
    decoder.decode_from(first, ctx, 4)  # warm-up: graph capture, cuBLAS heuristics
    if profile:  # the same graph must not be captured inside the range: lengths half way decide its chunk size
        decoder.decode_from(first, ctx, new_tokens)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
    _, seconds = decoder.decode_from(first, ctx, new_tokens)
    if profile:
        torch.cuda.profiler.stop()
    stats = torch.tensor([seconds], device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    seconds = float(stats.item())
    kv_bytes = sum(ctx) * 4 * 264 * cfg.n_layers
    return {"workload": "random-init d32-class (32 layers, d 2048, Hq 16, Hkv 4), batch 32 per GPU, contexts uniform in "
                        "[256, 8192] (synthetic cache contents), greedy, fp8 KV cache",
            "new_tokens": new_tokens, "tokens_per_s": B * world * new_tokens / seconds,
            "ms_per_step": seconds / new_tokens * 1e3, "kv_bytes_per_step_per_gpu": kv_bytes,
            "scaling": "weak (batch-sharded replicas)"}


def pin_to_local_cores(local: int, world: int) -> str:
    """With several ranks on one host, give each rank its own slice of the cores this process may use, taken from the
    NUMA node its GPU hangs off when sysfs tells (else an even slice): the end-to-end loop is driven by the host (one
    graph launch and one synchronisation per step), and ranks that wander over each other's cores cost it more than
    the GPUs do. Returns what was done, for the JSON line."""
    try:
        allowed = sorted(os.sched_getaffinity(0))
        if world <= 1 or len(allowed) < 2 * world:
            return "not pinned"
        node_cpus = None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = int(visible.split(",")[local]) if visible and visible.split(",")[local].isdigit() else local
            bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(physical)).busId
            bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
            if len(bus.split(":")[0]) == 8:
                bus = bus[4:]
            node = int(Path(f"/sys/bus/pci/devices/{bus}/numa_node").read_text())
            if node >= 0:
                cpus = set()
                for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
                node_cpus = [c for c in allowed if c in cpus]
        except Exception:
            node_cpus = None
        per = len(allowed) // world
        mine = allowed[local * per:(local + 1) * per]
        how = "even slice of the allowed cores"
        if node_cpus and len(node_cpus) >= per:
            # ranks of one node share its cores in local-rank order
            offset = (local * per) % max(1, len(node_cpus) - per + 1)
            mine, how = node_cpus[offset:offset + per], "slice of the GPU's NUMA node"
        os.sched_setaffinity(0, mine)
        return f"{len(mine)} cores, {how}"
    except Exception as e:  # an unusual host: run unpinned
        return f"not pinned ({type(e).__name__})"


def cpu_model() -> str:
    try:
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def run_reference(args, rank: int, world: int) -> None:
    """The reference arm: the CPU port of the reference's attention on the host cores. It runs on rank 0 alone and
    does not shard (the reference has no multi-GPU or multi-process path), so its value is the same at every N."""
    if rank != 0:
        return
    lens_all = workload_lens(args.workload, BATCH * world)
    sample = lens_all[:args.cpu_sample]
    from oracle.attention import eager_attention_port

    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    data = cpu_sample(sample, 1234)
    step = lambda: [eager_attention_port(q, k, v, D ** -0.5) for q, k, v in data]
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = algorithmic_bytes(sample) * args.steps / dt / 1e9
    note = (f"each step = {len(sample)} sequences of the workload ({sum(sample)} positions; the GPU arm's step is the "
            f"whole batch of {BATCH} per GPU: the metric is a rate, so the two compare) on the host cores")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "none (one host process on rank 0; the value does not grow with N)",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_of(args, world, extra={"reference_step": note}),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "cpu": cpu_model(), "kind": "port",
                         "sample": note},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def config_of(args, world: int, extra: dict | None = None) -> dict:
    cfg = {"workload": {"target8k": "GQA sweep shapes at the bandwidth-target length: batch 64 per GPU, Hq 32, Hkv 8, "
                                    "head_dim 128, every sequence 8192 positions, e4m3 KV with per-(token, head) fp32 "
                                    "scales",
                        "ragged": "GQA sweep: batch 64 per GPU, Hq 32, Hkv 8, head_dim 128, lengths uniform in "
                                  "[512, 16384], e4m3 KV with per-(token, head) fp32 scales"}[args.workload],
           "global_batch": BATCH * world, "parallelism": f"batch-sharded x{world}", "seed": 0,
           "l2": "inputs (>= 0.5 GB of KV per GPU) exceed the 126 MB L2; no flush needed"}
    cfg.update(extra or {})
    return cfg


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="target8k", choices=["target8k", "ragged"])
    ap.add_argument("--cpu-sample", type=int, default=4, help="sequences in the CPU baseline's sample")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--chunk-pages", type=int, default=0)
    ap.add_argument("--decoder", type=int, default=1, help="also time end-to-end greedy decoding of d20 (0: skip)")
    ap.add_argument("--decoder-tokens", type=int, default=256, help="tokens generated per sequence in that run")
    ap.add_argument("--kernels", type=int, default=1, help="also time the append, merge and exchange kernels alone (N = 1; 0: skip)")
    ap.add_argument("--profile-range", default="attention",
                    choices=["attention", "decoder", "decoder_d32", "append", "prefill_attn", "tile_gemm", "merge", "exchange"],
                    help="which timed loops cudaProfilerStart/Stop bracket (for `ncu --profile-from-start off`)")
    ap.add_argument("--decoder-d32", type=int, default=1, help="also time batched decode of the d32-class model (0: skip)")
    ap.add_argument("--ragged", type=int, default=1, help="also run the ragged GQA sweep as an extra (0: skip)")
    ap.add_argument("--longctx", type=int, default=1, help="also time the KV-length-sharded long-context case (0: skip)")
    ap.add_argument("--e2e-steps", type=int, default=200, help="steps of the end-to-end loop (profiling runs shrink it)")
    ap.add_argument("--e2e-parts", type=int, default=0, help="row groups of the end-to-end step that run as parallel graph branches (0: DecodeStep's choice)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist

    import nanochat_b200 as ncb
    from nanochat_b200 import attention as ops
    from nanochat_b200.sharding import shard_batch

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    pinned = pin_to_local_cores(local, world)
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps: int, warmup: int, during=None) -> float:
        """Milliseconds per step: after `warmup` calls, REPEATS timed loops of exactly `steps` calls each, every loop
        between two CUDA events on the launching stream with a barrier and a synchronize on both sides and the max over
        ranks taken; the median loop is returned. `during` runs once per loop while its queued steps still execute."""
        for _ in range(warmup):
            fn()
        loops = []
        for _ in range(REPEATS):
            barrier()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(steps):
                fn()
            end.record()
            if during:
                during()
            barrier()
            ms = torch.tensor([start.elapsed_time(end)], device=device)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            loops.append(float(ms.item()) / steps)
        return statistics.median(loops)

    def attention_workload(workload: str, with_e2e: bool, profiled: bool) -> dict:
        """One decode-attention workload on this rank's share of the global batch: the step (split + merge), the split
        kernel alone, the checks, and (with_e2e) the step through DecodeStep with host buffers."""
        lens_all = workload_lens(workload, BATCH * world)
        mine = shard_batch(lens_all, world, longest_first=True)[rank]
        lens = [lens_all[i] for i in mine]
        B = len(lens)
        e2e_steps = max(1, min(args.steps, args.e2e_steps))
        headroom = args.warmup + e2e_steps * REPEATS + 8 if with_e2e else 0
        max_len = max(lens) + headroom
        planted = min(range(B), key=lambda b: (abs(lens[b] - 8192), b))  # the slot whose V rows are one vector
        vector = 0.25 * torch.randn(D, generator=torch.Generator().manual_seed(1500 + rank))
        cache = synthetic_cache(lens, max_len, seed=1000 + rank, device=device, constant_v={planted: vector})
        gen = torch.Generator(device=device).manual_seed(2000 + rank)
        q = torch.randn(B, HQ, D, generator=gen, device=device).bfloat16()
        lens_t = torch.tensor(lens, dtype=torch.int32, device=device)
        max_kv = max(lens)
        status = torch.zeros(1, dtype=torch.int32, device=device)
        chunk = args.chunk_pages or ops.plan_chunk_pages(lens, HKV, max_kv)  # the host knows this step's lengths
        workspace = torch.empty(ncb.workspace_bytes(B, HQ, HKV, max_kv + headroom, chunk), dtype=torch.uint8,
                                device=device)
        out = torch.empty_like(q)
        step = lambda: ncb.decode_attention(q, cache, lens_t, max_kv, chunk_pages=chunk, workspace=workspace, out=out,
                                            status=status)
        split = lambda: ops.decode_attention_split(q, cache, lens_t, max_kv, workspace, chunk_pages=chunk,
                                                   status=status)
        for _ in range(3):  # first-use costs (module load, attribute set-up) stay out of any profiled range
            step()
        torch.cuda.synchronize()
        if profiled:
            torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` see exactly the loops below
        with ClockSampler(local) as clocks:
            ms_step = timed(step, args.steps, args.warmup, during=clocks.sample if clocks.nvml else None)
        ms_split = timed(split, args.steps, 3)
        step()
        torch.cuda.synchronize()
        # ---- checks on what the timed kernels computed
        check_seq = 0 if planted != 0 else 1
        errs = torch.tensor([*error_of(out[planted], dequantised(vector).to(device).expand(HQ, D)),
                             *error_of(out[check_seq], torch_attention_row(cache, check_seq, lens[check_seq], q[check_seq]))],
                            device=device)
        res = {"lens": lens, "chunk": chunk, "ms_step": ms_step, "ms_split": ms_split, "clocks": clocks.summary()}
        if with_e2e:
            # ---- end to end through the public step object with host buffers
            cos, sin = ncb.rotary_table(max_len, 1e4, device=device)
            ones = torch.ones(D, device=device)
            host_gen = torch.Generator().manual_seed(3000 + rank)
            decode = ncb.DecodeStep(cache, HQ, cos, sin, ones, ones, B, chunk_pages=chunk, parts=args.e2e_parts)
            decode.qkv_host.copy_(torch.randn(decode.qkv_host.shape, generator=host_gen).bfloat16())
            decode.pos_host.copy_(torch.tensor(lens, dtype=torch.int32))

            def e2e_step():
                decode.run()  # pinned host in, graph replay (copies, append + attention), pinned host out, sync
                decode.pos_host.add_(1)  # the next step's token goes one position further

            for _ in range(args.warmup):
                e2e_step()
            done, loops = args.warmup, []
            for _ in range(REPEATS):
                barrier()
                # every timed step attends one position more than the one before
                nbytes = sum(algorithmic_bytes([n + done + k + 1 for n in lens]) for k in range(e2e_steps))
                t0 = time.perf_counter()
                for _ in range(e2e_steps):
                    e2e_step()
                barrier()
                t = torch.tensor([time.perf_counter() - t0, float(nbytes)], device=device)
                if world > 1:
                    seconds = t[:1].clone()
                    dist.all_reduce(seconds, op=dist.ReduceOp.MAX)
                    dist.all_reduce(t)
                    t[0] = seconds[0]
                loops.append((float(t[0]), float(t[1])))
                done += e2e_steps
            loops.sort(key=lambda x: x[0] / x[1])
            seconds, nbytes = loops[len(loops) // 2]
            decode.check()
            res["e2e"] = {"value": nbytes / seconds / 1e9, "unit": UNIT, "h2d_bytes_per_step": decode.h2d_bytes,
                          "d2h_bytes_per_step": decode.d2h_bytes, "steps": e2e_steps,
                          "ms_per_step": seconds / e2e_steps * 1e3,
                          "parts": decode.parts,
                          "what": "DecodeStep.run(): pinned-host qkv rows + positions in, decode_step_attn_fp8 (append "
                                  "+ attention; one CUDA graph with the copies, the rows in `parts` groups that run "
                                  "as parallel branches so that later groups' copies cross PCIe under earlier "
                                  "groups' attention), output to pinned host, synchronised every step; the KV cache "
                                  "is resident decoder state"}
            del decode
        if profiled:
            torch.cuda.profiler.stop()
        total_bytes = torch.tensor([float(algorithmic_bytes(lens))], device=device)
        if world > 1:
            dist.all_reduce(errs, op=dist.ReduceOp.MAX)
            dist.all_reduce(total_bytes)
        assert status.item() == 0, f"device status {status.item()}"
        res["total_bytes"] = float(total_bytes.item())
        res["parity"] = {"property_max_abs": float(errs[0]), "property_mean_abs": float(errs[1]),
                         "torch_fp32_seq_max_abs": float(errs[2]), "torch_fp32_seq_mean_abs": float(errs[3]),
                         "what": "max over ranks; property: one sequence per rank has a constant V row planted, its "
                                 "output must be that vector; torch_fp32_seq: one sequence per rank recomputed with "
                                 "plain torch fp32 operators on the dequantised cache",
                         "tolerance": {"max_abs": PATH_MAX_ABS, "mean_abs": PATH_MEAN_ABS}}
        assert errs[0] <= PATH_MAX_ABS and errs[1] <= PATH_MEAN_ABS and errs[2] <= PATH_MAX_ABS and errs[3] <= PATH_MEAN_ABS, \
            res["parity"]
        return res

    def roofline_of(res: dict, traffic) -> dict:
        peak, peak_kind = peaks()
        nbytes = algorithmic_bytes(res["lens"])
        gbs = nbytes / (res["ms_split"] * 1e-3) / 1e9
        return {"bound": "hbm", "kernel": "k_decode_attn<1> (split-KV)", "achieved": gbs, "peak": peak, "unit": UNIT,
                "frac": gbs / peak, "peak_kind": peak_kind, "traffic": traffic["bytes"] if traffic else None,
                "traffic_capture_commit": traffic["commit"] if traffic else None,
                "us_per_launch": res["ms_split"] * 1e3, "algorithmic_bytes_per_launch": nbytes}

    head = attention_workload(args.workload, True, args.profile_range == "attention")
    ragged = attention_workload("ragged", False, False) if args.ragged and args.workload != "ragged" else None
    kernels = bench_kernels(device, timed, args.profile_range) if args.kernels and world == 1 else None
    longctx = bench_longctx(rank, world, device, min(args.steps, 100), 5, timed) if args.longctx else None
    decoder = bench_decoder(rank, world, device, args.decoder_tokens, args.profile_range == "decoder") \
        if args.decoder else None
    serving = bench_serving(rank, world, device) if args.decoder else None
    d32_profiled = args.profile_range == "decoder_d32"  # two steps are enough for a launch list
    decoder_d32 = bench_decoder_d32(rank, world, device, 2 if d32_profiled else 128, d32_profiled) \
        if args.decoder_d32 else None

    if rank == 0:
        value = head["total_bytes"] / (head["ms_step"] * 1e-3) / 1e9
        traffic = profiled_traffic() if args.workload == "target8k" and not args.chunk_pages else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": head["ms_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "e4m3 operands, fp32 accumulate and softmax", "data": "synthetic",
            "config": config_of(args, world, extra={"chunk_pages": head["chunk"], "timed_loops": REPEATS,
                                                    "host_cores_per_rank": pinned,
                                                    "pct_of_8TBs_per_gpu": value / world / 80.0}),
            "clocks": head["clocks"], "e2e": head["e2e"], "gpu_launches": 2 * args.steps * REPEATS,
            "roofline": roofline_of(head, traffic), "parity": head["parity"],
        }
        if ragged:
            rvalue = ragged["total_bytes"] / (ragged["ms_step"] * 1e-3) / 1e9
            line["ragged"] = {"workload": config_of(argparse.Namespace(workload="ragged"), world)["workload"] +
                                          ", sequences longest-first inside each GPU's batch",
                              "value": rvalue, "unit": UNIT, "ms_per_step": ragged["ms_step"], "scaling": "weak",
                              "chunk_pages": ragged["chunk"], "roofline": roofline_of(ragged, None),
                              "parity": ragged["parity"]}
        if kernels:
            line["kernels"] = kernels
        if longctx:
            line["longctx"] = longctx
        if decoder:
            line["decoder"] = decoder
        if serving:
            line["serving"] = serving
        if decoder_d32:
            line["decoder_d32"] = decoder_d32
        if world == 1 and args.cpu_seconds > 0:
            line["cpu_baseline"] = time_cpu_reference(head["lens"][:args.cpu_sample], args.cpu_seconds)
            if decoder:
                decoder["cpu_baseline"] = bench_decoder_cpu(3)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
