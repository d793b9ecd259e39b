"""Prefill check and benchmark of a whole model.

Protocol of the reference's ``texelator/prefill.py``: run the same prompt once with every linear forced
onto the streamed small-batch path (prefill threshold ``1 << 30``, :88-90) and once forced onto the
tensor-core tile path (threshold 1, :91-93); the final hidden states of at most 32 prompt tokens must
agree (rel-RMS <= 0.02, :98-107); then both paths are timed with the wall clock and with CUDA events
and the medians reported (:29-60, :110-128).  The result keeps the reference's JSON keys.  The model is
a ``modeling.BC4Decoder`` (anything with ``handles``, ``config`` and ``prefill(ids)``) instead of the
reference's stand-alone Qwen3.8 loader; the implementation is this build's own.
"""
from __future__ import annotations

import contextlib
import json
import math
import statistics
import time
from pathlib import Path

import torch

from .artifacts import environment_snapshot, write_json
from .autotune import BASELINE, CANDIDATES
from .runtime import PREFILL_THRESHOLD, PREFILL_TILE_ROWS, extension

STREAMED, TILES = 1 << 30, 1          # prefill thresholds that force one path or the other
AGREEMENT_LIMIT = 0.02                # rel-RMS between the two paths' final hidden states


@contextlib.contextmanager
def _borrowed(handles: list[int], backend: int):
    """Use ``backend`` on every handle for a while; thresholds and backends are put back afterwards."""
    ext = extension()
    before = [ext.handle_info(handle)[2:5] for handle in handles]
    try:
        for handle in handles:
            ext.set_prefill_backend(handle, backend)
        yield
    finally:
        for handle, (threshold, tile_rows, old_backend) in zip(handles, before):
            ext.set_prefill(handle, threshold, tile_rows)
            ext.set_prefill_backend(handle, old_backend)


def _force(handles: list[int], threshold: int) -> None:
    ext = extension()
    for handle in handles:
        ext.set_prefill(handle, threshold, PREFILL_TILE_ROWS)


def _agreement(model, ids: torch.Tensor) -> dict:
    hidden = {}
    for name, threshold in (("streamed", STREAMED), ("tiles", TILES)):
        _force(model.handles, threshold)
        hidden[name] = model.prefill(ids).double()
    gap = hidden["tiles"] - hidden["streamed"]
    scale = float(hidden["streamed"].square().mean().sqrt())
    cosine = float(torch.nn.functional.cosine_similarity(hidden["streamed"].reshape(1, -1), hidden["tiles"].reshape(1, -1)))
    return {"tokens": int(ids.numel()), "max_abs": float(gap.abs().max()),
            "relative_rms": float(gap.square().mean().sqrt()) / max(scale, 1e-12), "cosine": cosine}


def _timed(model, ids: torch.Tensor, warmup: int, runs: int) -> dict:
    for _ in range(warmup):
        model.prefill(ids)
    torch.cuda.synchronize()
    wall, device = [], []
    for _ in range(runs):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        started = time.perf_counter()
        begin.record()
        model.prefill(ids)
        end.record()
        torch.cuda.synchronize()
        wall.append(time.perf_counter() - started)
        device.append(begin.elapsed_time(end) * 1e-3)
    tokens = int(ids.numel())
    summary = {"tokens": tokens, "warmup": warmup, "runs": runs, "wall_seconds": wall, "gpu_seconds": device}
    for name, values in (("wall", wall), ("gpu", device)):
        summary[f"{name}_seconds_median"] = statistics.median(values)
        summary[f"{name}_tokens_per_second"] = tokens / summary[f"{name}_seconds_median"]
    return summary


def benchmark_prefill(model, tokens: int, warmup: int, runs: int, output: Path | None = None,
                      backend: int | None = None) -> dict:
    if not torch.cuda.is_available():
        raise RuntimeError("prefill benchmark requires a visible CUDA GPU")
    if tokens < PREFILL_THRESHOLD:
        raise ValueError(f"tokens must be at least the hybrid threshold ({PREFILL_THRESHOLD})")
    if warmup < 0 or runs < 1:
        raise ValueError("warmup must be non-negative and runs must be positive")
    tile_backend = CANDIDATES[BASELINE] if backend is None else backend
    ids = torch.randint(0, model.config.vocab, (tokens,), generator=torch.Generator().manual_seed(0), dtype=torch.int64)
    with _borrowed(model.handles, tile_backend):
        correctness = _agreement(model, ids[:min(tokens, 32)])
        if not math.isfinite(correctness["relative_rms"]) or correctness["relative_rms"] > AGREEMENT_LIMIT:
            raise RuntimeError(f"hybrid prefill correctness failed: {correctness}")
        _force(model.handles, STREAMED)
        streamed = _timed(model, ids, warmup, runs)
        _force(model.handles, TILES)
        tiles = _timed(model, ids, warmup, runs)
    result = {"schema_version": 1, "model": model.config.name, "prefill_backend": tile_backend,
              "prefill_tile_rows": PREFILL_TILE_ROWS, "correctness": correctness,
              "scalar_texture": streamed, "fused_texture_tensorcore": tiles,
              "speedup_wall": streamed["wall_seconds_median"] / tiles["wall_seconds_median"],
              "speedup_gpu": streamed["gpu_seconds_median"] / tiles["gpu_seconds_median"],
              "environment": environment_snapshot()}
    if output is not None:
        write_json(output, result)
    print(json.dumps(result, indent=2), flush=True)
    return result
