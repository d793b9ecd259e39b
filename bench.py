#!/usr/bin/env python
"""Benchmark of the BC4 weight-linear hot path: batch-1 decode of a 27B-class dense decoder.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--model NAME]

One "step" is one decoded token: every BC4 projection of every layer (plus norms, attention over
the KV cache, lm_head and argmax) for one token.  With N > 1 the script is started once per GPU by
``torch.distributed.run`` and shards every projection tensor-parallel.  Rank 0 prints one JSON line.

``--impl reference`` times the reference's CPU arithmetic for the same path (palette-LUT dequant
followed by a dense matmul, all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# DRAM bytes moved per algorithmic byte by the decode GEMV: dram__bytes_read.sum + dram__bytes_write.sum of
# one ncu-captured gemv_tile_kernel<4,1,0,0,0> launch on a 34816x5120 matrix (89.34 MB + 3.27 MB) over its
# algorithmic 89.35 MB.  The kernel reads every payload byte once, so the ratio carries over to the other
# shapes; re-capture when the kernel's memory access pattern changes.
GEMV_DRAM_BYTES_PER_ALGORITHMIC_BYTE = (89.34 + 3.27) / 89.35

METRIC = "bc4_decode_tokens_per_second_bs1"
UNIT = "tok/s"


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.process = index, [], None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            self.rows.append([field.strip() for field in line.split(",")])

    def __exit__(self, *exc):
        if self.process:
            self.process.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if value.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# CPU baseline: the reference's CPU-side arithmetic for this path (there is no CPU operator in the
# reference; its encoder's palette gather, texelator/encoder.py:19-31, times the fp32 row scale,
# then a dense matmul), written with multi-threaded torch ops, on one projection-sized sample.
# ---------------------------------------------------------------------------------------------

def cpu_dequant(blocks: np.ndarray, scales: np.ndarray, lut: torch.Tensor) -> torch.Tensor:
    """Palette-LUT gather times the fp32 row scale, rounded to bf16: the matrix the operator multiplies by."""
    m = scales.shape[0]
    raw = torch.from_numpy(blocks).reshape(m, -1, 8)
    e0 = raw[:, :, 0].view(torch.int8).long() + 127
    e1 = raw[:, :, 1].view(torch.int8).long() + 127
    word = torch.zeros(raw.shape[:2], dtype=torch.int64)
    for byte in range(6):
        word |= raw[:, :, 2 + byte].long() << (8 * byte)
    sel = (word[:, :, None] >> (3 * torch.arange(16))[None, None, :]) & 7
    pal = lut[e1, e0]                                               # [m, nb, 8]
    w = torch.gather(pal, 2, sel).reshape(m, -1) * torch.from_numpy(scales)[:, None]
    return w.bfloat16().float()


def cpu_matmul(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return (x.float() @ w.T).bfloat16()


_CPU_CACHE: dict = {}


def cpu_baseline_sample(config, seconds: float = 10.0) -> dict:
    """Time dequantise-then-matmul on a row slab of one hidden x hidden projection sized to take about
    ``seconds`` on this host, and scale by bytes to one decoded token.  Reports the combined figure
    (``value``) and the matmul on already dequantised weights alone (``matmul_only``)."""
    from oracle import bc4_oracle as O
    k = config.hidden
    torch.set_num_threads(max(torch.get_num_threads(), os.cpu_count() or 1))   # torchrun pins OMP_NUM_THREADS=1
    if "lut" not in _CPU_CACHE:
        lut_np = O.software_palette()
        rng = np.random.default_rng(0)
        w = (rng.standard_normal((256, k)) * 0.02).astype(np.float32)
        blocks, scales = O.encode_minmax(w, lut_np)
        x = torch.randn(1, k).bfloat16()
        lut = torch.from_numpy(lut_np)
        cpu_matmul(x, cpu_dequant(blocks, scales, lut))              # warm
        start = time.perf_counter()
        cpu_matmul(x, cpu_dequant(blocks, scales, lut))
        per_row = (time.perf_counter() - start) / 256
        _CPU_CACHE.update(lut=lut, blocks=blocks, scales=scales, x=x, per_row=per_row)
    c = _CPU_CACHE
    rows = int(min(max(seconds / c["per_row"], 256), 8 * k)) // 256 * 256
    blocks = np.tile(c["blocks"].reshape(256, -1), (rows // 256, 1)).reshape(-1)
    scales = np.tile(c["scales"], rows // 256)
    start = time.perf_counter()
    weights = cpu_dequant(blocks, scales, c["lut"])
    middle = time.perf_counter()
    for _ in range(3):
        cpu_matmul(c["x"], weights)
    end = time.perf_counter()
    dequant_s, matmul_s = middle - start, (end - middle) / 3
    sample_bytes = rows * k // 2 + 4 * rows
    fraction = sample_bytes / config.bc4_bytes_per_token()
    return {"value": fraction / (dequant_s + matmul_s), "unit": UNIT, "matmul_only": fraction / matmul_s,
            "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"palette-LUT dequant ({dequant_s:.3f} s) + fp32 matmul ({matmul_s * 1e3:.1f} ms) of a {rows}x{k} BC4 slab "
                      f"({sample_bytes} B of the {config.bc4_bytes_per_token()} B read per token), scaled by bytes to one token",
            "sample_fraction_of_token": fraction, "seconds": dequant_s + matmul_s}


def workload_config(config, prompt: int, world: int, lookahead: int) -> dict:
    """The `config` object of the JSON line: the same workload description for both arms."""
    return {"workload": f"{config.name} dense decoder, batch-1 decode after a {prompt}-token random-id prompt",
            "model_shape": config.name, "hidden": config.hidden, "layers": config.layers,
            "intermediate": config.intermediate, "parallelism": f"tp{world}",
            "bc4_bytes_per_token": config.bc4_bytes_per_token(),
            "l2": "per-token weight stream (>=1.3 GB per GPU) is larger than L2; no flush needed",
            "lookahead": lookahead}


def run_reference_arm(args, config) -> None:
    """The reference's CPU arithmetic on this host.  One step = one bounded sample of the workload (a slab of
    one projection); ``ms_per_step`` is the measured time of that sample, ``value`` the tokens per second it
    corresponds to when scaled by bytes to a whole token (``cpu_baseline.sample_fraction_of_token``)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step = max(0.5, min(5.0, 150.0 / max(args.steps + args.warmup, 1)))   # whole run within minutes
    for _ in range(args.warmup):
        cpu_baseline_sample(config, per_step)
    samples = [cpu_baseline_sample(config, per_step) for _ in range(args.steps)]
    value = float(np.median([v["value"] for v in samples]))
    middle = min(samples, key=lambda v: abs(v["value"] - value))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 * float(np.median([v["seconds"] for v in samples])),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(config, args.prompt, args.gpus, args.lookahead),
            "note": "CPU dequantise-then-matmul on a bounded slab of this workload per step; value is scaled by bytes to one token",
            "cpu_baseline": dict(middle, value=value),
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def timed_steps(model, steps: int, warmup: int, world: int, e2e: bool) -> float:
    """ms per decode step, device-timed on the model's stream, max over ranks.  With ``e2e`` every step
    copies the input token id from pinned host memory and reads the produced token id back."""
    import torch.distributed as dist
    stream = model.stream
    host_in = torch.zeros(model.tok.numel(), dtype=torch.int64).pin_memory()
    host_out = torch.zeros(model.tok.numel(), dtype=torch.int64).pin_memory()

    def one():
        if e2e:
            model.tok.copy_(host_in, non_blocking=True)
        model.decode_graph()
        if e2e:
            host_out.copy_(model.next_tok, non_blocking=True)
            stream.synchronize()
            host_in.copy_(host_out)

    start_pos = model.pos.clone()
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            one()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.cudart().cudaProfilerStart()      # lets `ncu --profile-from-start off` see only the timed steps
        begin.record(stream)
        for _ in range(steps):
            one()
        end.record(stream)
        stream.synchronize()
        torch.cuda.cudart().cudaProfilerStop()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        elapsed = torch.tensor([begin.elapsed_time(end)], device=model.device)
        if world > 1:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        # rewind the position so the KV window of the next measurement is the same
        model.pos.copy_(start_pos)
        if start_pos.numel() == 1:
            model.mask[..., int(start_pos.item()):] = False
        stream.synchronize()
    return float(elapsed.item()) / steps


def gemv_roofline(model, config, world: int) -> dict:
    """All BC4 decode GEMV launches of one token (4 per layer) alone in a CUDA graph: algorithmic bytes
    (blocks + fp32 row scales + bf16 activations in and out) over the CUDA-event time."""
    ext = model.ext
    stream = model.stream
    xs, ys, total = {}, {}, 0
    jobs = []
    for handles in (model.h_qkv, model.h_o, model.h_gu, model.h_down):
        for h in handles:
            m, k = ext.handle_info(h)[:2]
            if (m, k) not in xs:
                xs[(m, k)] = torch.randn(1, k, device=model.device).bfloat16()
                ys[(m, k)] = torch.empty(1, m, device=model.device, dtype=torch.bfloat16)
            jobs.append((h, xs[(m, k)], ys[(m, k)]))
            total += m * k // 2 + 4 * m + 2 * k + 2 * m
    with torch.cuda.stream(stream):
        for h, x, y in jobs:
            ext.linear_out(h, x, y)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for h, x, y in jobs:
                ext.linear_out(h, x, y)
        for _ in range(3):
            graph.replay()
        stream.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        begin.record(stream)
        for _ in range(reps):
            graph.replay()
        end.record(stream)
        stream.synchronize()
    ms = begin.elapsed_time(end) / reps
    peak, source = measured_peaks()
    achieved = total / ms / 1e6
    traffic_ratio = GEMV_DRAM_BYTES_PER_ALGORITHMIC_BYTE
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": traffic_ratio * total, "traffic_source": "ncu capture of one 34816x5120 launch (ratio to algorithmic bytes), scaled by algorithmic bytes",
            "peak_source": source, "kernel": "gemv_tile_kernel (all %d decode GEMV launches of one token)" % len(jobs),
            "algorithmic_bytes_per_token": total, "ms_per_token_linear_only": ms, "launches": len(jobs)}


def _pack_random(ext, m: int, k: int, count: int, lut, lookahead: int) -> list[int]:
    from texelator_b200.modeling import encode_minmax_cuda
    handles = []
    for index in range(count):
        weight = torch.randn(m, k, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1000 * m + index)) * 0.02
        handles.append(ext.pack_encoded_device(*encode_minmax_cuda(weight, lut)))
        ext.set_lookahead(handles[-1], lookahead)
    return handles


def _time_calls(stream, call, repeats: int) -> float:
    """Milliseconds per call of ``call()`` (CUDA events on ``stream``, after three untimed calls)."""
    with torch.cuda.stream(stream):
        for _ in range(3):
            call()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        for _ in range(repeats):
            call()
        end.record(stream)
        stream.synchronize()
    return begin.elapsed_time(end) / repeats


def prefill_sweep(ext, stream, lookahead: int) -> list[dict]:
    """BASELINE configuration 3: T in {32, 128, 512} x {5120->5120, 5120->17408, 17408->5120}.  Every point runs
    every tile candidate over a rotating set of matrices larger than L2 and keeps the fastest (the autotuner's
    rule; all candidates are bitwise identical)."""
    from texelator_b200.autotune import CANDIDATES
    from texelator_b200.modeling import software_palette_table
    lut = software_palette_table("cuda")
    peak = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text()).get("bf16_tflops", 1590.0)) if (ROOT / "MEASURED_PEAKS.json").exists() else 1590.0
    rows = []
    for k, m in ((5120, 5120), (5120, 17408), (17408, 5120)):
        copies = max(2, int(160e6 // (m * k // 2)) + 1)
        handles = _pack_random(ext, m, k, copies, lut, lookahead)
        try:
            for tokens in (32, 128, 512):
                x = torch.randn(tokens, k, device="cuda").bfloat16()
                y = torch.empty(tokens, m, device="cuda", dtype=torch.bfloat16)
                best = None
                for name, backend in CANDIDATES.items():
                    for h in handles:
                        ext.set_prefill_backend(h, backend)
                        ext.set_prefill(h, 1, 1024)

                    def sweep():
                        for h in handles:
                            ext.linear_out(h, x, y)
                    ms = _time_calls(stream, sweep, 5) / copies
                    if best is None or ms < best[0]:
                        best = (ms, name)
                ms, name = best
                tflops = 2.0 * tokens * m * k / ms / 1e9
                weight_gbs = (m * k / 2 + 4 * m + 2 * tokens * (k + m)) / ms / 1e6
                rows.append({"T": tokens, "M": m, "K": k, "ms": ms, "tflops": tflops, "frac_of_bf16_burst": tflops / peak,
                             "hbm_gbs": weight_gbs, "tile": name})
        finally:
            for h in handles:
                ext.free(h)
    return rows


def gemv_cfg1(ext, stream, lookahead: int) -> dict:
    """BASELINE configuration 1 as a throughput point: one token through 4096x4096 matrices, a rotating set
    larger than L2 inside a CUDA graph."""
    from texelator_b200.modeling import software_palette_table
    handles = _pack_random(ext, 4096, 4096, 24, software_palette_table("cuda"), lookahead)
    try:
        x = torch.randn(1, 4096, device="cuda").bfloat16()
        y = torch.empty(1, 4096, device="cuda", dtype=torch.bfloat16)
        with torch.cuda.stream(stream):
            for h in handles:
                ext.linear_out(h, x, y)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for h in handles:
                    ext.linear_out(h, x, y)
        ms = _time_calls(stream, graph.replay, 10) / len(handles)
        peak, _ = measured_peaks()
        gbs = (4096 * 4096 / 2 + 4 * 4096 + 4 * 4096) / ms / 1e6
        return {"us_per_call": ms * 1e3, "GBps": gbs, "frac": gbs / peak, "matrices": len(handles)}
    finally:
        for h in handles:
            ext.free(h)


def tp_parity(config, device, rank: int, world: int, lookahead: int, layers: int = 4) -> dict:
    """Tensor-parallel result against one GPU, on a reduced layer count of the same shapes: rank 0 builds the
    unsharded `layers`-layer model and decodes eight tokens after a 64-token prompt; every rank then builds its
    shard from the same seed and decodes the same eight steps, fed the one-GPU run's tokens (a near-tie in one
    greedy pick would otherwise put the two runs on different sequences).  Reports whether the ranks hold identical
    bits, the lowest cosine over the eight final hidden states against the one-GPU model, and how many of the
    eight greedy picks agree."""
    import dataclasses

    import torch.distributed as dist

    from texelator_b200.modeling import BC4Decoder
    small = dataclasses.replace(config, layers=layers, name=f"{config.name}-{layers}layers")
    ids = torch.randint(0, small.vocab, (64,), generator=torch.Generator().manual_seed(7))
    steps = 8

    def decode(model, forced=None):
        model.prefill(ids)
        model.tok.fill_(int(ids[-1]))
        model.capture()
        tokens, hidden = [], []
        for step in range(steps):
            if forced is not None and step > 0:
                model.tok.fill_(int(forced[step - 1]))
                torch.cuda.synchronize()
            model.decode_graph()
            model.stream.synchronize()
            tokens.append(int(model.next_tok))
            hidden.append(model.last_hidden.float().clone())
        return tokens, torch.cat(hidden)

    expected = torch.zeros(steps, dtype=torch.int64, device=device)
    if rank == 0:
        full = BC4Decoder(small, device, 96, seed=99, lookahead=lookahead)
        full_tokens, full_hidden = decode(full)
        expected.copy_(torch.tensor(full_tokens))
        full.graph = None
        full.free()
    dist.broadcast(expected, src=0)
    shard = BC4Decoder(small, device, 96, seed=99, tp_rank=rank, tp_world=world, lookahead=lookahead)
    fused = shard.enable_peer_exchange()
    tokens, hidden = decode(shard, forced=expected.tolist())
    status = shard.ext.kernel_status(device=device.index)
    reference = hidden.clone()
    dist.broadcast(reference, src=0)
    identical = torch.tensor([int(torch.equal(reference, hidden))], device=device)
    dist.all_reduce(identical, op=dist.ReduceOp.MIN)
    shard.graph = None
    result = {"layers": layers, "fused_exchange": bool(fused), "ranks_identical": bool(identical.item()), "kernel_status": int(status)}
    if rank == 0:
        cosines = torch.nn.functional.cosine_similarity(full_hidden, hidden, dim=1)
        agree = sum(int(a == b) for a, b in zip(tokens, full_tokens))
        result.update(hidden_cosine=float(cosines.min()), tokens_agreeing=agree, tokens_compared=steps,
                      ok=bool(identical.item()) and float(cosines.min()) >= 0.999 and status == 0)
    dist.barrier()
    return result


def micro_exchange(config, device, rank: int, world: int, exchanges: int = 1000) -> dict:
    """`exchanges` back-to-back exchanges (a 64-row-tile push-linear standing in for the producer, then the
    cluster reduce + norm) in one CUDA graph: microseconds per exchange at this rank count."""
    import torch.distributed as dist

    from texelator_b200 import runtime
    from texelator_b200.modeling import encode_minmax_cuda, software_palette_table
    from texelator_b200.tp import PeerExchange
    ext = runtime.extension()
    hidden, k = config.hidden, 512
    peers = PeerExchange(hidden, device)
    handle = ext.pack_encoded_device(*encode_minmax_cuda(torch.randn(hidden, k, device=device) * 0.02, software_palette_table(device)))
    x = torch.randn(1, k, device=device).bfloat16()
    h = torch.zeros(1, hidden, device=device, dtype=torch.bfloat16)
    gamma = torch.ones(hidden, device=device, dtype=torch.bfloat16)
    y = torch.empty_like(h)
    stream = torch.cuda.Stream(device)

    def body(count):
        for _ in range(count):
            ext.linear_single_push(handle, x, peers)
            ext.peer_reduce_rmsnorm(h, gamma, 1e-6, peers=peers, y=y)

    def alone(count):
        for _ in range(count):
            ext.linear_single(handle, x, y)
            ext.peer_reduce_rmsnorm(h, gamma, 1e-6, delta=y, y=y)

    times = {}
    for name, fn in (("exchange", body), ("local", alone)):
        with torch.cuda.stream(stream):
            fn(2)
            stream.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                fn(exchanges)
            graph.replay()
            stream.synchronize()
            dist.barrier()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            graph.replay()
            end.record(stream)
            stream.synchronize()
        elapsed = torch.tensor([begin.elapsed_time(end)], device=device)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        times[name] = float(elapsed.item()) * 1e3 / exchanges
    status = ext.kernel_status(device=device.index)
    ext.free(handle)
    return {"n_gpus": world, "us_per_exchange_with_producer": times["exchange"], "us_same_kernels_without_exchange": times["local"],
            "us_exchange_only": times["exchange"] - times["local"], "hidden": hidden, "kernel_status": int(status)}


def run_gpu_arm(args, config) -> None:
    import torch.distributed as dist
    from texelator_b200.modeling import BC4Decoder
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the BC4 operator has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    device = torch.device("cuda", local)
    prompt, decode = args.prompt, args.decode
    max_len = prompt + decode + args.warmup + 16
    model = BC4Decoder(config, device, max_len, seed=1234, tp_rank=rank, tp_world=world, lookahead=args.lookahead,
                       encoder=args.encoder)
    ids = torch.randint(0, config.vocab, (prompt,), generator=torch.Generator().manual_seed(0))
    model.prefill(ids)
    model.tok.fill_(int(ids[-1]))
    fused_allreduce = world > 1 and not args.nccl_allreduce and model.enable_peer_exchange()
    model.fuse_norm = bool(args.fuse_norm)
    model.capture()
    steps, warmup = args.steps, max(args.warmup, 3)

    with ClockSampler(local) as clocks:
        ms = timed_steps(model, steps, warmup, world, e2e=False)
        # the timed region of a fast run is shorter than the sampler's period: keep the same load on (untimed,
        # the same number of steps on every rank) until about 0.6 s have been sampled
        more = int(min(args.decode - 16, 600.0 / ms) - steps)
        if more > 0:
            timed_steps(model, more, 0, world, e2e=False)
    ms_e2e = timed_steps(model, steps, warmup, world, e2e=True)
    roofline = gemv_roofline(model, config, world)
    extras = {}
    if world == 1 and not args.skip_extras:
        extras["prefill"] = prefill_sweep(model.ext, model.stream, args.lookahead)
        extras["gemv_cfg1"] = gemv_cfg1(model.ext, model.stream, args.lookahead)
    # any bounded device wait that ran out (tcgen05 pipeline, peer exchange) leaves a code here; 0 = none
    status = torch.tensor([model.ext.kernel_status()], device=device)
    if world > 1:
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
    kernel_status = int(status.item())
    model.graph = None
    if world > 1 and not args.skip_extras:
        model.free()
        extras["tp_parity"] = tp_parity(config, device, rank, world, args.lookahead)
        extras["micro_exchange"] = micro_exchange(config, device, rank, world)
        kernel_status = max(kernel_status, extras["tp_parity"]["kernel_status"], extras["micro_exchange"]["kernel_status"])
    if rank == 0:
        cpu = cpu_baseline_sample(config)
        line = {
            "metric": METRIC, "value": 1000.0 / ms, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": workload_config(config, prompt, world, args.lookahead),
            "allreduce": ("none" if world == 1 else "packets pushed from the linears' epilogues over NVLink peer memory, cluster reduce + norm"
                          if fused_allreduce else "nccl"),
            "e2e": {"value": 1000.0 / ms_e2e, "unit": UNIT, "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
            "gpu_launches": int(model.launches_per_step * steps),
            "kernel_status": kernel_status,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "clocks": clocks.summary(),
            **extras,
        }
        print(json.dumps(line), flush=True)
    sys.stdout.flush()
    # Tear down in an order that cannot block: graphs that captured NCCL kernels are gone, every rank meets at
    # a barrier, and multi-rank runs leave without destroying the communicator (its destructor can wait for
    # ever on captured work).  A bounded device wait that ran out anywhere makes the run fail.
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0 if kernel_status == 0 else 4)
    model.free()
    if kernel_status:
        raise SystemExit(f"a device-side bounded wait ran out (status {kernel_status}): the measurement is invalid")


def run_batched(args, config) -> None:
    """`--batch B`: B sequences decode one token each per step (BASELINE configuration 5 when the model is the
    70B-class one on 8 GPUs).  Every sequence gets a real prompt of `--prompt` tokens through the tensor-core
    prefill and then seeded random cache rows up to `--context` positions; prints one JSON line (tokens of all
    sequences per second, the linears' share measured alone, the weight bytes they stream)."""
    import torch.distributed as dist
    from texelator_b200.batched import BatchedBC4Decoder
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the BC4 operator has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    device = torch.device("cuda", local)
    steps, warmup = args.steps, max(args.warmup, 3)
    context = max(args.context, args.prompt)
    results = []
    model = None
    for batch in [int(v) for v in str(args.batch).split(",")]:
        if model is not None:
            model.graph = None
            model.free()
            del model
            torch.cuda.empty_cache()
        model = BatchedBC4Decoder(config, device, context + steps + 2 * warmup + 8, batch, seed=1234, tp_rank=rank, tp_world=world,
                                  lookahead=args.lookahead)
        kernels = {}
        if args.batch_kernel == "tiles":
            for handle in model.handles:
                model.ext.set_prefill(handle, 16, 1024)
        elif args.batch_kernel == "tuned":
            kernels = model.tune_decode_kernel()
        for sequence in range(batch):
            ids = torch.randint(0, config.vocab, (args.prompt,), generator=torch.Generator().manual_seed(sequence))
            model.prefill_sequence(sequence, ids)
            model.tok[sequence] = int(ids[-1])
            model.fill_context(sequence, args.prompt, context, seed=7)
        model.capture()
        with ClockSampler(local) as clocks:
            ms = timed_steps(model, steps, warmup, world, e2e=False)
        ms_e2e = timed_steps(model, steps, warmup, world, e2e=True)
        # the four linears of every layer alone, same handles, same batch, in one graph
        stream = model.stream
        with torch.cuda.stream(stream):
            def linears():
                for layer in range(config.layers):
                    model.ext.linear_out(model.h_qkv[layer], model.buf_x, model.buf_qkv)
                    model.ext.linear_out(model.h_o[layer], model.buf_attn, model.buf_o)
                    model.ext.linear_out(model.h_gu[layer], model.buf_x, model.buf_gu)
                    model.ext.linear_out(model.h_down[layer], model.buf_act, model.buf_down)
            linears()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                linears()
            for _ in range(3):
                graph.replay()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            for _ in range(8):
                graph.replay()
            end.record(stream)
            stream.synchronize()
            linear_ms = begin.elapsed_time(end) / 8
        weight_bytes = config.bc4_bytes_per_token() / world
        peak, source = measured_peaks()
        status = torch.tensor([model.ext.kernel_status()], device=device)
        if world > 1:
            dist.all_reduce(status, op=dist.ReduceOp.MAX)
        results.append({"batch": batch, "tokens_per_second": batch * 1000.0 / ms, "ms_per_step": ms,
                        "e2e_tokens_per_second": batch * 1000.0 / ms_e2e, "linears_ms_per_step": linear_ms,
                        "linears_GBps_per_gpu": weight_bytes / linear_ms / 1e6, "linears_frac_of_hbm": weight_bytes / linear_ms / 1e6 / peak,
                        "launches_per_step": int(model.launches_per_step), "kernel_status": int(status.item()),
                        "kernels": {k: {"kernel": v[0], "us": v[1], "candidates_us": v[2]} for k, v in kernels.items()},
                        "clocks": clocks.summary()})
    if rank == 0:
        print(json.dumps({"metric": "bc4_batched_decode_tokens_per_second", "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
                          "dtype": "bf16", "data": "synthetic", "peak_source": source,
                          "config": {"workload": f"{config.name} dense decoder, batched decode, {args.prompt}-token prompts + random cache rows up to "
                                                 f"{context} positions per sequence", "model_shape": config.name, "parallelism": f"tp{world}",
                                     "decode_kernel": args.batch_kernel, "lookahead": args.lookahead,
                                     "allreduce": "none" if world == 1 else "nccl inside the captured graph"},
                          "batches": results}), flush=True)
    sys.stdout.flush()
    bad = max(r["kernel_status"] for r in results)
    if world > 1:
        model.graph = None
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0 if bad == 0 else 4)
    model.free()
    if bad:
        raise SystemExit(f"a device-side bounded wait ran out (status {bad}): the measurement is invalid")


def run_micro_exchange(args, config) -> None:
    """`--micro-exchange` (under torch.distributed.run): only the tensor-parallel exchange timing of this model's
    hidden size -- 1000 back-to-back exchanges in one CUDA graph, with and without the exchange -- one JSON line."""
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("start with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N --micro-exchange")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    result = micro_exchange(config, torch.device("cuda", local), rank, world)
    if rank == 0:
        print(json.dumps({"metric": "tp_exchange_microseconds", "unit": "us", "higher_is_better": False, **result}), flush=True)
    sys.stdout.flush()
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0 if result["kernel_status"] == 0 else 4)


def run_micro(args) -> None:
    """Small single-kernel case for profilers: `--micro MxK[xT]` packs enough random BC4 matrices of that
    shape to exceed L2, runs the linear on each in turn (CUDA events) and prints one JSON line."""
    from texelator_b200 import runtime
    from texelator_b200.modeling import encode_minmax_cuda, software_palette_table
    dims = [int(v) for v in args.micro.lower().split("x")]
    m, k, tokens = dims[0], dims[1], (dims[2] if len(dims) > 2 else 1)
    torch.cuda.set_device(0)
    ext = runtime.extension()
    lut = software_palette_table("cuda")
    copies = max(2, int(200e6 // (m * k // 2)) + 1)
    handles = []
    for index in range(copies):
        weight = torch.randn(m, k, device="cuda", generator=torch.Generator(device="cuda").manual_seed(index)) * 0.02
        handles.append(ext.pack_encoded_device(*encode_minmax_cuda(weight, lut)))
        ext.set_lookahead(handles[-1], args.lookahead)
        ext.set_prefill_backend(handles[-1], args.backend)
        ext.set_prefill(handles[-1], args.threshold, 1024)
        ext.set_palette(handles[-1], args.palette)       # throughput only: the bytes are the same either way
        ext.set_decode_path(handles[-1], args.decode_path)
    x = torch.randn(tokens, k, device="cuda").bfloat16()
    y = torch.empty(tokens, m, device="cuda", dtype=torch.bfloat16)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        def sweep():
            for h in handles:
                ext.linear_out(h, x, y)
        for _ in range(max(args.warmup, 3)):
            sweep()
        stream.synchronize()
        before = ext.launch_count()
        graph = torch.cuda.CUDAGraph()          # one graph over all copies: no host time between the launches
        with torch.cuda.graph(graph, stream=stream):
            sweep()
        launches = ext.launch_count() - before
        graph.replay()
        stream.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.cudart().cudaProfilerStart()
        begin.record(stream)
        for _ in range(args.steps):
            graph.replay()
        end.record(stream)
        stream.synchronize()
        torch.cuda.cudart().cudaProfilerStop()
    us = begin.elapsed_time(end) * 1000 / (args.steps * copies)
    bytes_per_call = m * k // 2 + 4 * m + 2 * tokens * (k + m)
    print(json.dumps({"micro": args.micro, "copies": copies, "us_per_call": us, "GBps": bytes_per_call / us / 1e3,
                      "TFLOPs": 2.0 * tokens * m * k / us / 1e6, "launches_per_call": launches / copies,
                      "note": "all copies in one CUDA graph"}), flush=True)
    runtime.free(handles)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--model", default="27b-class")
    parser.add_argument("--prompt", type=int, default=2048)
    parser.add_argument("--decode", type=int, default=512)
    parser.add_argument("--lookahead", type=int, default=0,
                        help="1 KiB weight units in flight per warp; default: 3 on one GPU (measured 210.6 tok/s against 207.5 with 4), "
                             "4 tensor-parallel (what the single-token kernel was measured with)")
    parser.add_argument("--nccl-allreduce", action="store_true", help="tensor parallel: keep NCCL all-reduces (default: fused peer-memory exchange)")
    parser.add_argument("--skip-extras", action="store_true", help="only the decode measurement (no prefill sweep / cfg1 / parity / exchange timing)")
    parser.add_argument("--layers", type=int, default=0, help="override the layer count (profiling aid; not a bench result)")
    parser.add_argument("--batch", default=None, help="batched decode: B or a comma list of B (one JSON line with an entry per B)")
    parser.add_argument("--context", type=int, default=4096, help="--batch: cache positions per sequence before the timed steps")
    parser.add_argument("--batch-kernel", default="tuned", choices=["tuned", "gemv", "tiles"],
                        help="--batch: B >= 16 through the multi-token decode kernel (gemv), the tensor-core tile kernel (tiles), "
                             "or whichever measures faster per projection (tuned)")
    parser.add_argument("--threshold", type=int, default=16, help="--micro: prefill threshold (token counts below it take the decode kernel)")
    parser.add_argument("--encoder", default="minmax", choices=["minmax", "e3"],
                        help="how the synthetic weights are BC4-encoded: the encoder's min/max start, or its whole endpoint search on the GPU")
    parser.add_argument("--fuse-norm", action="store_true", help="residual add + RMSNorm inside the qkv and gate/up linears (A/B aid; default: separate norm kernels)")
    parser.add_argument("--micro-exchange", action="store_true", help="tensor parallel: time the exchange alone (1000 in one graph)")
    parser.add_argument("--micro", default=None, help="MxK[xT]: time one linear shape alone (profiling aid)")
    parser.add_argument("--backend", type=int, default=5, help="prefill backend id for --micro with T >= 16")
    parser.add_argument("--decode-path", type=int, default=0, help="--micro: 0 mma.sync ALU decode, 1 exact ALU, 2 texture")
    parser.add_argument("--palette", type=int, default=0, help="--micro: 0 software palette, 1 hardware (texture-unit) palette")
    args = parser.parse_args()
    if args.lookahead == 0:
        args.lookahead = 3 if int(os.environ.get("WORLD_SIZE", "1")) == 1 else 4
    if args.micro:
        run_micro(args)
        return
    from texelator_b200.modeling import CONFIGS
    config = CONFIGS[args.model]
    if args.layers:
        import dataclasses
        config = dataclasses.replace(config, layers=args.layers, name=f"{config.name}-{args.layers}layers")
    if args.impl == "reference":
        run_reference_arm(args, config)
    elif args.micro_exchange:
        run_micro_exchange(args, config)
    elif args.batch:
        if args.prompt == 2048:
            args.prompt = 512          # configuration 5's prompt length
        run_batched(args, config)
    else:
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if args.gpus != world:
            if world == 1 and args.gpus > 1:
                raise SystemExit("start multi-GPU runs with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
        run_gpu_arm(args, config)


if __name__ == "__main__":
    main()
