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

def cpu_dequant_matmul(blocks: np.ndarray, scales: np.ndarray, x: torch.Tensor, lut: torch.Tensor) -> torch.Tensor:
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
    return (x.float() @ w.bfloat16().float().T).bfloat16()


_CPU_CACHE: dict = {}


def cpu_baseline_sample(config, seconds: float = 10.0) -> dict:
    """Time dequantise-then-matmul on a row slab of one hidden x hidden projection sized to take
    about ``seconds`` on this host, and extrapolate linearly (bytes) to one decoded token."""
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
        cpu_dequant_matmul(blocks, scales, x, lut)                   # warm
        start = time.perf_counter()
        cpu_dequant_matmul(blocks, scales, x, lut)
        per_row = (time.perf_counter() - start) / 256
        _CPU_CACHE.update(lut=lut, blocks=blocks, scales=scales, x=x, per_row=per_row)
    c = _CPU_CACHE
    rows = int(min(max(seconds / c["per_row"], 256), 8 * k)) // 256 * 256
    blocks = np.tile(c["blocks"].reshape(256, -1), (rows // 256, 1)).reshape(-1)
    scales = np.tile(c["scales"], rows // 256)
    start = time.perf_counter()
    cpu_dequant_matmul(blocks, scales, c["x"], c["lut"])
    elapsed = time.perf_counter() - start
    sample_bytes = rows * k // 2 + 4 * rows
    return {"value": (sample_bytes / config.bc4_bytes_per_token()) / elapsed, "unit": UNIT,
            "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"palette-LUT dequant + fp32 matmul of a {rows}x{k} BC4 slab ({sample_bytes} B of the "
                      f"{config.bc4_bytes_per_token()} B read per token), extrapolated linearly to one token",
            "seconds": elapsed}


def workload_config(config, prompt: int, world: int, lookahead: int) -> dict:
    """The `config` object of the JSON line: the same workload description for both arms."""
    return {"workload": f"{config.name} dense decoder, batch-1 decode after a {prompt}-token random-id prompt",
            "model_shape": config.name, "hidden": config.hidden, "layers": config.layers,
            "intermediate": config.intermediate, "parallelism": f"tp{world}",
            "bc4_bytes_per_token": config.bc4_bytes_per_token(),
            "l2": "per-token weight stream (>=1.3 GB per GPU) is larger than L2; no flush needed",
            "lookahead": lookahead}


def run_reference_arm(args, config) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    values = []
    per_step = max(0.5, min(5.0, 150.0 / max(args.steps + args.warmup, 1)))   # whole run within minutes
    for _ in range(args.warmup):
        cpu_baseline_sample(config, per_step)
    for _ in range(args.steps):
        values.append(cpu_baseline_sample(config, per_step))
    best = max(values, key=lambda v: v["value"])
    value = float(np.median([v["value"] for v in values]))
    best = dict(best, value=value)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 / value, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(workload_config(config, args.prompt, args.gpus, args.lookahead),
                           note="reference arm: CPU dequantise-then-matmul on a bounded slab of this workload, extrapolated by bytes"),
            "cpu_baseline": best,
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
    host_in = torch.zeros(1, dtype=torch.int64).pin_memory()
    host_out = torch.zeros(1, dtype=torch.int64).pin_memory()

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
    # DRAM bytes per algorithmic byte of this kernel, from the ncu capture of one 34816x5120 launch
    # (dram__bytes_read.sum + dram__bytes_write.sum = 92.25 MB for 89.35 MB; profiles/gemv_tile_kernel_34816x5120.md),
    # scaled to the launches of one token by the bytes they process
    traffic_ratio = 92.25 / 89.35
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": traffic_ratio * total, "traffic_source": "ncu, one 34816x5120 launch, scaled by algorithmic bytes",
            "peak_source": source, "kernel": "gemv_tile_kernel (all %d decode GEMV launches of one token)" % len(jobs),
            "algorithmic_bytes_per_token": total, "ms_per_token_linear_only": ms, "launches": len(jobs)}


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
    model = BC4Decoder(config, device, max_len, seed=1234, tp_rank=rank, tp_world=world, lookahead=args.lookahead)
    ids = torch.randint(0, config.vocab, (prompt,), generator=torch.Generator().manual_seed(0))
    model.prefill(ids)
    model.tok.fill_(int(ids[-1]))
    fused_allreduce = world > 1 and not args.nccl_allreduce and model.enable_peer_exchange()
    model.capture()
    steps, warmup = args.steps, max(args.warmup, 3)

    with ClockSampler(local) as clocks:
        ms = timed_steps(model, steps, warmup, world, e2e=False)
    ms_e2e = timed_steps(model, steps, warmup, world, e2e=True)
    roofline = gemv_roofline(model, config, world)
    # any bounded device wait that ran out (tcgen05 pipeline, peer exchange) leaves a code here; 0 = none
    status = torch.tensor([model.ext.kernel_status()], device=device)
    if world > 1:
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
    kernel_status = int(status.item())
    if rank == 0:
        cpu = cpu_baseline_sample(config)
        line = {
            "metric": METRIC, "value": 1000.0 / ms, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": dict(workload_config(config, prompt, world, args.lookahead),
                           allreduce=("none" if world == 1 else
                                      "fused into the norm kernel over NVLink peer memory" if fused_allreduce else "nccl")),
            "e2e": {"value": 1000.0 / ms_e2e, "unit": UNIT, "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
            "gpu_launches": int(model.launches_per_step * steps),
            "kernel_status": kernel_status,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "clocks": clocks.summary(),
        }
        print(json.dumps(line), flush=True)
    sys.stdout.flush()
    # Tear down in an order that cannot block: graphs that captured NCCL kernels go first, every rank
    # meets at a barrier, and multi-rank runs leave without destroying the communicator (its destructor
    # can wait for ever on captured work).
    model.graph = None
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)
    model.free()


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
        ext.set_palette(handles[-1], args.palette)       # throughput only: the bytes are the same either way
        ext.set_decode_path(handles[-1], args.decode_path)
    x = torch.randn(tokens, k, device="cuda").bfloat16()
    y = torch.empty(tokens, m, device="cuda", dtype=torch.bfloat16)
    for _ in range(max(args.warmup, 3)):
        for h in handles:
            ext.linear_out(h, x, y)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.cudart().cudaProfilerStart()
    begin.record()
    for _ in range(args.steps):
        for h in handles:
            ext.linear_out(h, x, y)
    end.record()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    us = begin.elapsed_time(end) * 1000 / (args.steps * copies)
    bytes_per_call = m * k // 2 + 4 * m + 2 * tokens * (k + m)
    print(json.dumps({"micro": args.micro, "copies": copies, "us_per_call": us, "GBps": bytes_per_call / us / 1e3,
                      "TFLOPs": 2.0 * tokens * m * k / us / 1e6, "note": "eager launches: host overhead included"}), flush=True)
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
    parser.add_argument("--lookahead", type=int, default=4)
    parser.add_argument("--nccl-allreduce", action="store_true", help="tensor parallel: keep NCCL all-reduces (default: fused peer-memory exchange)")
    parser.add_argument("--layers", type=int, default=0, help="override the layer count (profiling aid; not a bench result)")
    parser.add_argument("--micro", default=None, help="MxK[xT]: time one linear shape alone (profiling aid)")
    parser.add_argument("--backend", type=int, default=5, help="prefill backend id for --micro with T >= 16")
    parser.add_argument("--decode-path", type=int, default=0, help="--micro: 0 mma.sync ALU decode, 1 exact ALU, 2 texture")
    parser.add_argument("--palette", type=int, default=0, help="--micro: 0 software palette, 1 hardware (texture-unit) palette")
    args = parser.parse_args()
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
    else:
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if args.gpus != world:
            if world == 1 and args.gpus > 1:
                raise SystemExit("start multi-GPU runs with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
        run_gpu_arm(args, config)


if __name__ == "__main__":
    main()
