"""Prefill tile autotuner.

Protocol and profile format of ``texelator/autotune.py`` of the reference: one representative
handle per distinct (M, K) (:88-103); seeded activations ``randn(tokens, K) * 0.125`` (:139-143);
the baseline tile (backend 5) defines the expected output and a candidate is admitted only if its
output is bitwise equal (:144-168); admitted candidates are timed in rotating order with CUDA
events (:170-193); the winner per ``"tokens<=B:M=m:K=k"`` key is stored together with kernel
facts, device facts and a hash of the kernel sources (:194-242); ``apply_profile`` refuses a
profile made for another build or GPU (:247-258).

The candidates are this build's sm_100a tiles of one tcgen05 kernel (output rows x tokens x columns
per pipeline stage): 128x256x128 (baseline), 256x256x64, 128x128x128, 128x64x128, 128x192x128.  All of
them consume K in the same 16-column steps, so they pass the bitwise gate against each other.
Unlike the reference, ``apply_profile`` leaves the prefill threshold alone, so single-token decode
keeps the decode GEMV after a profile was applied.
"""
from __future__ import annotations

import hashlib
import json
import math
import statistics
from collections import Counter
from pathlib import Path

import torch

from .artifacts import safe_name, state_home
from .runtime import extension, free, pack_entry_handles

CANDIDATES = {
    "umma_128x256x128": 5,
    "umma_256x256x64": 6,
    "umma_128x128x128": 7,
    "umma_128x64x128": 8,
    "umma_128x192x128": 9,
}
BASELINE = "umma_128x256x128"
TOKEN_BUCKETS = (32, 128, 512, 2048, 8192, 16384, 32768, 65535)


def profile_path(artifact: Path) -> Path:
    metadata_hash = _sha256(Path(artifact) / "weights" / "metadata.json")
    major, minor = torch.cuda.get_device_capability()
    device = safe_name(torch.cuda.get_device_name())
    return state_home() / "profiles" / metadata_hash[:20] / f"sm_{major}{minor}-{device}-prefill.json"


def token_bucket(tokens: int) -> int:
    if tokens < 1:
        raise ValueError("tokens must be positive")
    if tokens > TOKEN_BUCKETS[-1]:
        raise ValueError(f"tokens exceeds supported CUDA grid limit: {tokens}")
    return next(value for value in TOKEN_BUCKETS if tokens <= value)


def dispatch_key(tokens: int, m: int, k: int) -> str:
    return f"tokens<={token_bucket(tokens)}:M={m}:K={k}"


def _sha256(path: Path) -> str:
    digest = hashlib.sha256()
    with Path(path).open("rb") as handle:
        for chunk in iter(lambda: handle.read(1 << 20), b""):
            digest.update(chunk)
    return digest.hexdigest()


def kernel_source_sha256() -> str:
    root = Path(__file__).resolve().parent / "cuda"
    digest = hashlib.sha256()
    for path in sorted(root.glob("*.cu")) + sorted(root.glob("*.cuh")):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def _error(reference: torch.Tensor, candidate: torch.Tensor) -> dict:
    ref, value = reference.float(), candidate.float()
    delta = value - ref
    ref_rms = torch.sqrt(torch.mean(ref.square())).item()
    denominator = math.sqrt(torch.sum(ref.square()).item() * torch.sum(value.square()).item())
    return {"max_abs": float(delta.abs().max().item()), "mean_abs": float(delta.abs().mean().item()),
            "relative_rms": float(torch.sqrt(torch.mean(delta.square())).item() / max(ref_rms, 1e-30)),
            "cosine": float(torch.sum(ref * value).item() / max(denominator, 1e-30)),
            "bitwise_equal": bool(torch.equal(reference, candidate))}


def _eligible(name: str, m: int, k: int) -> tuple[bool, str | None]:
    if k % 16:
        return False, "K is not divisible by 16"
    return True, None


def _inventory(artifact: Path):
    metadata = json.loads((Path(artifact) / "weights" / "metadata.json").read_text())
    handles: list[int] = []
    for entry in metadata["entries"]:
        handles.extend(pack_entry_handles(Path(artifact) / "weights", entry, bias=None, lookahead=1))
    ext = extension()
    representative: dict[tuple[int, int], int] = {}
    counts: Counter = Counter()
    for handle in handles:
        m, k = map(int, ext.handle_info(handle)[:2])
        counts[(m, k)] += 1
        representative.setdefault((m, k), handle)
        ext.set_prefill(handle, 1, 32768)      # force the prefill side while measuring (reference :102)
    return handles, representative, counts


def tune_handles(representative: dict, counts: Counter, tokens: list[int], warmup: int = 5, measured: int = 30,
                 seed: int = 20260827) -> tuple[dict, list]:
    """Core of the tuner on already packed handles: returns (selections, rows)."""
    ext = extension()
    selections: dict[str, dict] = {}
    rows: list[dict] = []
    for token_count in tokens:
        bucket = token_bucket(token_count)
        for shape_index, ((m, k), handle) in enumerate(sorted(representative.items())):
            generator = torch.Generator(device="cuda")
            generator.manual_seed(seed + token_count * 1009 + shape_index)
            x = torch.randn((token_count, k), device="cuda", dtype=torch.bfloat16, generator=generator)
            x.mul_(0.125)
            ext.set_prefill_backend(handle, CANDIDATES[BASELINE])
            reference = ext.linear(handle, x)
            valid, correctness, rejected = [], {}, {}
            for name, backend in CANDIDATES.items():
                supported, reason = _eligible(name, m, k)
                if not supported:
                    rejected[name] = reason or "unsupported"
                    continue
                ext.set_prefill_backend(handle, backend)
                candidate = ext.linear(handle, x)
                metrics = _error(reference, candidate)
                correctness[name] = metrics
                if metrics["bitwise_equal"]:
                    valid.append(name)
                else:
                    rejected[name] = f"correctness: rrms={metrics['relative_rms']:.6g}, cosine={metrics['cosine']:.9g}"
                del candidate
            if BASELINE not in valid:
                raise RuntimeError(f"baseline failed correctness for M={m},K={k}")
            for name in valid:
                ext.set_prefill_backend(handle, CANDIDATES[name])
                for _ in range(warmup):
                    ext.linear(handle, x)
            torch.cuda.synchronize()
            samples = {name: [] for name in valid}
            for iteration in range(measured):
                shift = iteration % len(valid)
                for name in valid[shift:] + valid[:shift]:
                    ext.set_prefill_backend(handle, CANDIDATES[name])
                    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record()
                    value = ext.linear(handle, x)
                    stop.record()
                    stop.synchronize()
                    samples[name].append(float(start.elapsed_time(stop)))
                    del value
            medians = {name: statistics.median(values) for name, values in samples.items()}
            winner = min(valid, key=lambda name: medians[name])
            key = dispatch_key(token_count, m, k)
            flops = 2.0 * token_count * m * k
            record = {"key": key, "tokens_measured": token_count, "token_bucket": bucket, "M": m, "K": k,
                      "occurrences": int(counts[(m, k)]), "winner": winner, "backend": CANDIDATES[winner],
                      "median_ms": medians[winner], "baseline_ms": medians[BASELINE],
                      "speedup_vs_baseline": medians[BASELINE] / medians[winner], "candidate_median_ms": medians,
                      "winner_tflops": flops / medians[winner] / 1e9,
                      "correctness_vs_baseline": correctness, "rejected": rejected}
            selections[key] = record
            rows.append(record)
            print(f"[autotune] tokens={token_count} M={m} K={k} winner={winner} {medians[winner]:.4f} ms "
                  f"({record['winner_tflops']:.1f} TFLOP/s) speedup={record['speedup_vs_baseline']:.3f}x", flush=True)
            del x, reference
    return selections, rows


def tune_artifact(artifact: Path, output_path: Path | None, tokens: list[int], warmup: int = 5, measured: int = 30,
                  seed: int = 20260827) -> dict:
    if warmup < 3 or measured < 10:
        raise ValueError("autotuning requires at least 3 warmups and 10 samples")
    artifact = Path(artifact).resolve()
    buckets = [token_bucket(value) for value in tokens]
    if len(buckets) != len(set(buckets)):
        raise ValueError("provide at most one representative token count per dispatch bucket")
    metadata_path = artifact / "weights" / "metadata.json"
    ext = extension()
    handles, representative, counts = _inventory(artifact)
    try:
        kernel_info = {name: list(map(int, ext.kernel_info(backend))) for name, backend in CANDIDATES.items()}
        selections, rows = tune_handles(representative, counts, tokens, warmup, measured, seed)
        properties = torch.cuda.get_device_properties(torch.cuda.current_device())
        profile = {"schema_version": 1, "status": "complete", "artifact": str(artifact),
                   "metadata_sha256": _sha256(metadata_path), "kernel_source_sha256": kernel_source_sha256(),
                   "device": {"name": torch.cuda.get_device_name(),
                              "compute_capability": list(torch.cuda.get_device_capability()),
                              "multiprocessor_count": int(properties.multi_processor_count),
                              "total_memory": int(properties.total_memory), "torch": torch.__version__,
                              "torch_cuda": torch.version.cuda},
                   "protocol": {"tokens": tokens, "warmup": warmup, "measured": measured, "seed": seed,
                                "bitwise_correctness_required": True},
                   "candidates": CANDIDATES, "kernel_info": kernel_info, "selections": selections, "rows": rows}
        target = output_path or profile_path(artifact)
        target.parent.mkdir(parents=True, exist_ok=True)
        target.write_text(json.dumps(profile, indent=2) + "\n")
        print(f"[texelator] prefill profile saved to {target}", flush=True)
        return profile
    finally:
        free(handles)


def check_profile(profile: dict, compute_capability: list[int], multiprocessor_count: int) -> None:
    """The three refusals of the reference's ``apply_profile`` (:249-258), separated from the GPU
    calls so they can be tested anywhere."""
    if profile.get("kernel_source_sha256") != kernel_source_sha256():
        raise RuntimeError("autotune profile kernel hash does not match this build")
    if profile.get("device", {}).get("compute_capability") != list(compute_capability):
        raise RuntimeError("autotune profile compute capability does not match this GPU")
    if profile.get("device", {}).get("multiprocessor_count") != int(multiprocessor_count):
        raise RuntimeError("autotune profile SM count does not match this GPU")


def apply_profile(handles: list[int], tokens: int, profile: dict) -> bool:
    ext = extension()
    properties = torch.cuda.get_device_properties(torch.cuda.current_device())
    check_profile(profile, list(torch.cuda.get_device_capability()), int(properties.multi_processor_count))
    complete = True
    for handle in handles:
        m, k = map(int, ext.handle_info(handle)[:2])
        selection = profile.get("selections", {}).get(dispatch_key(tokens, m, k))
        if selection is None:
            # profiles are finite: unknown buckets keep the baseline tile
            ext.set_prefill_backend(handle, CANDIDATES[BASELINE])
            complete = False
            continue
        ext.set_prefill_backend(handle, int(selection["backend"]))
    return complete


def selected_profile(artifact: Path) -> tuple[dict | None, Path]:
    target = profile_path(artifact)
    if not target.is_file():
        return None, target
    profile = json.loads(target.read_text())
    if profile.get("metadata_sha256") != _sha256(Path(artifact) / "weights" / "metadata.json"):
        raise RuntimeError("prefill profile does not match the encoded weights; rerun benchmark")
    if profile.get("kernel_source_sha256") != kernel_source_sha256():
        raise RuntimeError("prefill profile does not match this Texelator build; rerun benchmark")
    return profile, target
