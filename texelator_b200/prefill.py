"""Prefill check and benchmark.

Protocol of ``texelator/prefill.py`` of the reference: run the same prompt with the streamed
small-batch path forced (threshold ``1 << 30``, :88-90) and with the tensor-core tile path forced
(threshold 1, :91-93), require the final hidden states to agree (rel-RMS <= 0.02 on at most 32
tokens, :98-107), then time both with wall clock and CUDA events and report medians (:29-60,
:110-128).  The model is a ``modeling.BC4Decoder`` instead of the reference's stand-alone
Qwen3.8 artefact loader.
"""
from __future__ import annotations

import json
import math
import statistics
import time
from pathlib import Path

import torch

from .artifacts import environment_snapshot, write_json
from .autotune import CANDIDATES
from .runtime import PREFILL_THRESHOLD, PREFILL_TILE_ROWS, extension


def _set_prefill(handles: list[int], threshold: int, tile_rows: int) -> None:
    ext = extension()
    for handle in handles:
        ext.set_prefill(handle, threshold, tile_rows)


def _measure(model, input_ids: torch.Tensor, warmup: int, runs: int) -> dict:
    for _ in range(warmup):
        model.prefill(input_ids)
    torch.cuda.synchronize()
    wall_values, gpu_values = [], []
    for _ in range(runs):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = time.perf_counter()
        start.record()
        model.prefill(input_ids)
        stop.record()
        torch.cuda.synchronize()
        wall_values.append(time.perf_counter() - before)
        gpu_values.append(start.elapsed_time(stop) / 1000.0)
    tokens = int(input_ids.numel())
    wall_median, gpu_median = statistics.median(wall_values), statistics.median(gpu_values)
    return {"tokens": tokens, "warmup": warmup, "runs": runs, "wall_seconds": wall_values, "gpu_seconds": gpu_values,
            "wall_seconds_median": wall_median, "gpu_seconds_median": gpu_median,
            "wall_tokens_per_second": tokens / wall_median, "gpu_tokens_per_second": tokens / gpu_median}


def benchmark_prefill(model, tokens: int, warmup: int, runs: int, output: Path | None = None,
                      backend: int | None = None) -> dict:
    if not torch.cuda.is_available():
        raise RuntimeError("prefill benchmark requires a visible CUDA GPU")
    if tokens < PREFILL_THRESHOLD:
        raise ValueError(f"tokens must be at least the hybrid threshold ({PREFILL_THRESHOLD})")
    if warmup < 0 or runs < 1:
        raise ValueError("warmup must be non-negative and runs must be positive")
    ext = extension()
    handles = model.handles
    tile_backend = CANDIDATES[next(iter(CANDIDATES))] if backend is None else backend
    previous = [ext.handle_info(handle)[4] for handle in handles]
    try:
        for handle in handles:
            ext.set_prefill_backend(handle, tile_backend)
        generator = torch.Generator(device="cpu").manual_seed(0)
        input_ids = torch.randint(0, model.config.vocab, (tokens,), generator=generator, dtype=torch.int64)
        correctness_ids = input_ids[:min(tokens, 32)]
        _set_prefill(handles, 1 << 30, PREFILL_TILE_ROWS)
        reference = model.prefill(correctness_ids).float()
        _set_prefill(handles, 1, PREFILL_TILE_ROWS)
        candidate = model.prefill(correctness_ids).float()
        difference = candidate - reference
        reference_rms = float(torch.sqrt(torch.mean(reference * reference)).item())
        difference_rms = float(torch.sqrt(torch.mean(difference * difference)).item())
        cosine = float(torch.nn.functional.cosine_similarity(reference.reshape(1, -1), candidate.reshape(1, -1)).item())
        correctness = {"tokens": int(correctness_ids.numel()), "max_abs": float(difference.abs().max().item()),
                       "relative_rms": difference_rms / max(reference_rms, 1e-12), "cosine": cosine}
        if not math.isfinite(correctness["relative_rms"]) or correctness["relative_rms"] > 0.02:
            raise RuntimeError(f"hybrid prefill correctness failed: {correctness}")
        _set_prefill(handles, 1 << 30, PREFILL_TILE_ROWS)
        scalar = _measure(model, input_ids, warmup, runs)
        _set_prefill(handles, 1, PREFILL_TILE_ROWS)
        hybrid = _measure(model, input_ids, warmup, runs)
        result = {"schema_version": 1, "model": model.config.name, "prefill_backend": tile_backend,
                  "prefill_tile_rows": PREFILL_TILE_ROWS, "correctness": correctness,
                  "scalar_texture": scalar, "fused_texture_tensorcore": hybrid,
                  "speedup_wall": scalar["wall_seconds_median"] / hybrid["wall_seconds_median"],
                  "speedup_gpu": scalar["gpu_seconds_median"] / hybrid["gpu_seconds_median"],
                  "environment": environment_snapshot()}
        if output is not None:
            write_json(output, result)
        print(json.dumps(result, indent=2), flush=True)
        return result
    finally:
        _set_prefill(handles, PREFILL_THRESHOLD, PREFILL_TILE_ROWS)
        for handle, old in zip(handles, previous):
            ext.set_prefill_backend(handle, old)
