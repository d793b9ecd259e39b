"""Prefill tile autotuner.

Protocol and profile format follow the reference's ``texelator/autotune.py``: one representative
handle per distinct (M, K) (:88-103); seeded activations ``randn(tokens, K) * 0.125`` (:139-143); the
baseline tile defines the expected output and a candidate is admitted only when its output is
bitwise equal (:144-168); admitted candidates are timed in rotating order with CUDA events
(:170-193); the winner per ``"tokens<=B:M=m:K=k"`` key goes into a JSON profile with kernel facts,
device facts and a hash of the kernel sources (:194-242); ``apply_profile`` refuses a profile made for
another build or GPU (:247-258).  The implementation is this build's own.

The candidates are the sm_100a tiles of one tcgen05 kernel (output rows x tokens x columns per pipeline
stage).  All of them consume K in the same 16-column steps, so they pass the bitwise gate against each
other.  Unlike the reference, ``apply_profile`` leaves the prefill threshold alone, so single-token
decode keeps the decode GEMV after a profile was applied.
"""
from __future__ import annotations

import hashlib
import json
import statistics
from dataclasses import dataclass
from pathlib import Path

import torch

from .artifacts import safe_name, sha256_file, state_home
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


# ---- keys, paths, hashes ---------------------------------------------------------------------------

def token_bucket(tokens: int) -> int:
    if tokens < 1:
        raise ValueError("tokens must be positive")
    for limit in TOKEN_BUCKETS:
        if tokens <= limit:
            return limit
    raise ValueError(f"tokens exceeds supported CUDA grid limit: {tokens}")


def dispatch_key(tokens: int, m: int, k: int) -> str:
    return f"tokens<={token_bucket(tokens)}:M={m}:K={k}"


def profile_path(artifact: Path) -> Path:
    capability = "".join(str(part) for part in torch.cuda.get_device_capability())
    digest = sha256_file(Path(artifact) / "weights" / "metadata.json")
    return state_home() / "profiles" / digest[:20] / f"sm_{capability}-{safe_name(torch.cuda.get_device_name())}-prefill.json"


def kernel_source_sha256() -> str:
    """Identity of the kernels a profile was measured on: every CUDA source of the library."""
    digest = hashlib.sha256()
    sources = Path(__file__).resolve().parent / "cuda"
    for path in sorted(list(sources.glob("*.cu")) + list(sources.glob("*.cuh")), key=lambda p: (p.suffix, p.name)):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


# ---- one measurement point ---------------------------------------------------------------------------

def _compare(expected: torch.Tensor, got: torch.Tensor) -> dict:
    e, g = expected.double(), got.double()
    diff = g - e
    norm_e, norm_g = float(e.square().sum().sqrt()), float(g.square().sum().sqrt())
    return {"max_abs": float(diff.abs().max()), "mean_abs": float(diff.abs().mean()),
            "relative_rms": float(diff.square().mean().sqrt()) / max(float(e.square().mean().sqrt()), 1e-30),
            "cosine": float((e * g).sum()) / max(norm_e * norm_g, 1e-30),
            "bitwise_equal": bool(torch.equal(expected, got))}


def _eligible(name: str, m: int, k: int) -> tuple[bool, str | None]:
    return (True, None) if k % 16 == 0 else (False, "K is not divisible by 16")


@dataclass
class _Point:
    """One (token count, shape) point: a handle, its activations and the tiles admitted for it."""
    handle: int
    tokens: int
    m: int
    k: int
    x: torch.Tensor

    def run(self, ext, name: str) -> torch.Tensor:
        ext.set_prefill_backend(self.handle, CANDIDATES[name])
        return ext.linear(self.handle, self.x)

    def admit(self, ext) -> tuple[list[str], dict, dict]:
        expected = self.run(ext, BASELINE)
        admitted, correctness, rejected = [], {}, {}
        for name in CANDIDATES:
            ok, reason = _eligible(name, self.m, self.k)
            if not ok:
                rejected[name] = reason or "unsupported"
                continue
            correctness[name] = _compare(expected, self.run(ext, name))
            if correctness[name]["bitwise_equal"]:
                admitted.append(name)
            else:
                rejected[name] = (f"correctness: rrms={correctness[name]['relative_rms']:.6g}, "
                                  f"cosine={correctness[name]['cosine']:.9g}")
        if BASELINE not in admitted:
            raise RuntimeError(f"baseline failed correctness for M={self.m},K={self.k}")
        return admitted, correctness, rejected

    def time(self, ext, names: list[str], warmup: int, measured: int) -> dict[str, float]:
        """Median milliseconds per call; the order of the candidates rotates from sample to sample."""
        for name in names:
            for _ in range(warmup):
                self.run(ext, name)
        torch.cuda.synchronize()
        samples = {name: [] for name in names}
        for iteration in range(measured):
            first = iteration % len(names)
            for name in names[first:] + names[:first]:
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ext.set_prefill_backend(self.handle, CANDIDATES[name])
                begin.record()
                ext.linear(self.handle, self.x)
                end.record()
                end.synchronize()
                samples[name].append(begin.elapsed_time(end))
        return {name: statistics.median(values) for name, values in samples.items()}


def tune_handles(representative: dict, counts: dict, tokens: list[int], warmup: int = 5, measured: int = 30,
                 seed: int = 20260827) -> tuple[dict, list]:
    """The tuner on already packed handles (``{(M, K): handle}``): returns (selections, rows)."""
    ext = extension()
    selections, rows = {}, []
    for token_count in tokens:
        for shape_index, ((m, k), handle) in enumerate(sorted(representative.items())):
            generator = torch.Generator(device="cuda").manual_seed(seed + token_count * 1009 + shape_index)
            x = torch.randn((token_count, k), device="cuda", dtype=torch.bfloat16, generator=generator).mul_(0.125)
            point = _Point(handle, token_count, m, k, x)
            admitted, correctness, rejected = point.admit(ext)
            medians = point.time(ext, admitted, warmup, measured)
            winner = min(admitted, key=medians.__getitem__)
            key = dispatch_key(token_count, m, k)
            record = {"key": key, "tokens_measured": token_count, "token_bucket": token_bucket(token_count), "M": m, "K": k,
                      "occurrences": int(counts[(m, k)]), "winner": winner, "backend": CANDIDATES[winner],
                      "median_ms": medians[winner], "baseline_ms": medians[BASELINE],
                      "speedup_vs_baseline": medians[BASELINE] / medians[winner], "candidate_median_ms": medians,
                      "winner_tflops": 2.0 * token_count * m * k / medians[winner] / 1e9,
                      "correctness_vs_baseline": correctness, "rejected": rejected}
            selections[key] = record
            rows.append(record)
            print(f"[autotune] tokens={token_count} M={m} K={k} winner={winner} {medians[winner]:.4f} ms "
                  f"({record['winner_tflops']:.1f} TFLOP/s) speedup={record['speedup_vs_baseline']:.3f}x", flush=True)
    return selections, rows


# ---- artefact level ------------------------------------------------------------------------------------

def _pack_all(artifact: Path) -> tuple[list[int], dict, dict]:
    """Every handle of the artefact, one representative per distinct (M, K) and how often each shape occurs;
    all handles are forced to the prefill side while measuring (the reference does the same, :102)."""
    ext = extension()
    weights = Path(artifact) / "weights"
    handles: list[int] = []
    for entry in json.loads((weights / "metadata.json").read_text())["entries"]:
        handles.extend(pack_entry_handles(weights, entry, bias=None, lookahead=1))
    representative, counts = {}, {}
    for handle in handles:
        shape = tuple(int(v) for v in ext.handle_info(handle)[:2])
        counts[shape] = counts.get(shape, 0) + 1
        representative.setdefault(shape, handle)
        ext.set_prefill(handle, 1, 32768)
    return handles, representative, counts


def _device_facts() -> dict:
    properties = torch.cuda.get_device_properties(torch.cuda.current_device())
    return {"name": torch.cuda.get_device_name(), "compute_capability": list(torch.cuda.get_device_capability()),
            "multiprocessor_count": int(properties.multi_processor_count), "total_memory": int(properties.total_memory),
            "torch": torch.__version__, "torch_cuda": torch.version.cuda}


def tune_artifact(artifact: Path, output_path: Path | None, tokens: list[int], warmup: int = 5, measured: int = 30,
                  seed: int = 20260827) -> dict:
    if warmup < 3 or measured < 10:
        raise ValueError("autotuning requires at least 3 warmups and 10 samples")
    if len({token_bucket(value) for value in tokens}) != len(tokens):
        raise ValueError("provide at most one representative token count per dispatch bucket")
    artifact = Path(artifact).resolve()
    ext = extension()
    handles, representative, counts = _pack_all(artifact)
    try:
        selections, rows = tune_handles(representative, counts, tokens, warmup, measured, seed)
        profile = {"schema_version": 1, "status": "complete", "artifact": str(artifact),
                   "metadata_sha256": sha256_file(artifact / "weights" / "metadata.json"),
                   "kernel_source_sha256": kernel_source_sha256(), "device": _device_facts(),
                   "protocol": {"tokens": tokens, "warmup": warmup, "measured": measured, "seed": seed,
                                "bitwise_correctness_required": True},
                   "candidates": CANDIDATES,
                   "kernel_info": {name: [int(v) for v in ext.kernel_info(backend)] for name, backend in CANDIDATES.items()},
                   "selections": selections, "rows": rows}
    finally:
        free(handles)
    target = output_path or profile_path(artifact)
    target.parent.mkdir(parents=True, exist_ok=True)
    target.write_text(json.dumps(profile, indent=2) + "\n")
    print(f"[texelator] prefill profile saved to {target}", flush=True)
    return profile


def check_profile(profile: dict, compute_capability: list[int], multiprocessor_count: int) -> None:
    """The three refusals of ``apply_profile`` (reference :249-258), free of GPU calls so they can be tested anywhere."""
    device = profile.get("device", {})
    refusals = ((profile.get("kernel_source_sha256") == kernel_source_sha256(), "kernel hash does not match this build"),
                (device.get("compute_capability") == list(compute_capability), "compute capability does not match this GPU"),
                (device.get("multiprocessor_count") == int(multiprocessor_count), "SM count does not match this GPU"))
    for ok, message in refusals:
        if not ok:
            raise RuntimeError(f"autotune profile {message}")


def apply_profile(handles: list[int], tokens: int, profile: dict) -> bool:
    """Set every handle's tile for a prompt of ``tokens`` tokens; False when some shape had no entry for
    that bucket (those handles get the baseline tile: profiles are finite)."""
    ext = extension()
    properties = torch.cuda.get_device_properties(torch.cuda.current_device())
    check_profile(profile, list(torch.cuda.get_device_capability()), int(properties.multi_processor_count))
    chosen = profile.get("selections", {})
    complete = True
    for handle in handles:
        m, k = (int(v) for v in ext.handle_info(handle)[:2])
        selection = chosen.get(dispatch_key(tokens, m, k))
        ext.set_prefill_backend(handle, int(selection["backend"]) if selection else CANDIDATES[BASELINE])
        complete = complete and selection is not None
    return complete


def selected_profile(artifact: Path) -> tuple[dict | None, Path]:
    target = profile_path(artifact)
    if not target.is_file():
        return None, target
    profile = json.loads(target.read_text())
    if profile.get("metadata_sha256") != sha256_file(Path(artifact) / "weights" / "metadata.json"):
        raise RuntimeError("prefill profile does not match the encoded weights; rerun benchmark")
    if profile.get("kernel_source_sha256") != kernel_source_sha256():
        raise RuntimeError("prefill profile does not match this Texelator build; rerun benchmark")
    return profile, target
