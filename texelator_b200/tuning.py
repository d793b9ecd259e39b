"""Decode look-ahead profile.

Protocol and file format are those of the reference's ``texelator/tuning.py`` (candidate set :14,
agreement check of every candidate against K=1 with ``max_abs <= 1e-3`` on the first and last four
linears :69-81, timed sweeps over every linear of the model :82-98, profile JSON under
``STATE_HOME/profiles/<sha256(metadata.json)[:20]>/sm_XY-<device>.json`` :17-21,111-129); the
implementation is this build's own.  K is the number of 1 KiB weight units each warp of the decode
GEMV keeps in flight.  One sweep (every linear of the model once, one token) is captured in a CUDA
graph per candidate, so a measurement is a handful of graph replays between two CUDA events and the
host never paces the launches.
"""
from __future__ import annotations

import json
import statistics
from dataclasses import dataclass, field
from pathlib import Path

import torch

from .artifacts import safe_name, sha256_file, state_home, write_json
from .hardware import REFERENCE_TEXTURE_PALETTE_SHA256, ensure_hardware
from .runtime import extension, free, pack_entry_handles

CANDIDATES = (1, 2, 3, 4, 6, 8)
AGREEMENT_LIMIT = 1e-3          # max |y_K - y_1| the reference tolerates (tuning.py:80)


def _profile_path(artifact: Path) -> Path:
    capability = "".join(str(part) for part in torch.cuda.get_device_capability())
    digest = sha256_file(Path(artifact) / "weights" / "metadata.json")
    return state_home() / "profiles" / digest[:20] / f"sm_{capability}-{safe_name(torch.cuda.get_device_name())}.json"


def accepted_palettes() -> set[str]:
    """Hashes of the palettes this GPU's decoders reproduce bit for bit: the software palette always; the
    texture-unit palette the reference publishes whenever this build's closed form of it (what
    ``tx_dequant`` and every decode kernel evaluate for hardware-palette handles) hashes to that value --
    the ALU paths decode such artefacts exactly whether or not the device offers BC4 texture views."""
    software = ensure_hardware()
    hashes = {sha256_file(software)}
    closed_form = software.with_name("hardware_palette.bin")
    if not closed_form.exists():
        table = extension().hardware_palette()
        closed_form.write_bytes(table.numpy().astype("<f4").tobytes())
    if sha256_file(closed_form) == REFERENCE_TEXTURE_PALETTE_SHA256:
        hashes.add(REFERENCE_TEXTURE_PALETTE_SHA256)
    return hashes


@dataclass
class _Linear:
    handles: list[int]
    x: torch.Tensor
    y: list[torch.Tensor] = field(default_factory=list)


class LookaheadTuner:
    """Packs every linear of an artefact once, then answers two questions per candidate K: do the outputs
    still agree with K=1, and how long does one sweep over the model take."""

    def __init__(self, artifact: Path):
        if not torch.cuda.is_available():
            raise RuntimeError("tuning requires a visible CUDA GPU")
        self.artifact = Path(artifact)
        self.manifest = json.loads((self.artifact / "texelator.json").read_text())
        self.dtype_name = self.manifest.get("runtime_dtype", "float16")
        if self.dtype_name != "bfloat16":
            raise RuntimeError(f"unsupported Texelator runtime dtype: {self.dtype_name!r} (this build runs bfloat16 artefacts)")
        self.palette_sha256 = self.manifest.get("hardware", {}).get("palette_sha256")
        if not self.palette_sha256 or self.palette_sha256 not in accepted_palettes():
            raise RuntimeError("model BC4 palette does not match this GPU; benchmark aborted")
        self.weights = self.artifact / self.manifest["weights"]
        self.metadata_path = self.weights / "metadata.json"
        self.entries = json.loads(self.metadata_path.read_text())["entries"]
        if not self.entries:
            raise RuntimeError("artifact contains no encoded linears")
        self.ext = extension()
        self.linears: list[_Linear] = []
        self.stream = torch.cuda.Stream()

    # -- life cycle ------------------------------------------------------------
    def __enter__(self):
        generator = torch.Generator(device="cuda").manual_seed(0)      # the reference's inputs (tuning.py:53-59)
        try:
            for entry in self.entries:
                handles = pack_entry_handles(self.weights, entry, lookahead=1)
                x = torch.randn((1, int(entry["K"])), device="cuda", dtype=torch.bfloat16, generator=generator)
                outputs = [torch.empty(1, self.ext.handle_info(h)[0], device="cuda", dtype=torch.bfloat16) for h in handles]
                self.linears.append(_Linear(handles, x, outputs))
        except Exception:
            self.__exit__(None, None, None)
            raise
        return self

    def __exit__(self, *exc):
        free([h for linear in self.linears for h in linear.handles])
        self.linears = []

    # -- the two questions -----------------------------------------------------
    def _set(self, lookahead: int) -> None:
        for linear in self.linears:
            for handle in linear.handles:
                self.ext.set_lookahead(handle, lookahead)

    def _outputs(self, linears: list[_Linear]) -> list[torch.Tensor]:
        return [torch.cat([self.ext.linear(h, linear.x) for h in linear.handles], dim=-1).float() for linear in linears]

    def probes(self) -> list[_Linear]:
        """The linears whose outputs are compared: all of a small model, else the first and last four."""
        return self.linears if len(self.linears) <= 8 else self.linears[:4] + self.linears[-4:]

    def disagreement(self, lookahead: int, expected: list[torch.Tensor]) -> float:
        self._set(lookahead)
        return max(float((got - want).abs().max()) for got, want in zip(self._outputs(self.probes()), expected))

    def sweep_times(self, lookahead: int, warmup: int, measured: int, runs: int) -> list[float]:
        """Milliseconds per sweep, one value per independent run of `measured` graph replays."""
        self._set(lookahead)

        def sweep():
            for linear in self.linears:
                for handle, y in zip(linear.handles, linear.y):
                    self.ext.linear_out(handle, linear.x, y)

        with torch.cuda.stream(self.stream):
            sweep()                                   # first use of a kernel variant sets attributes: outside capture
            self.stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream):
                sweep()
            for _ in range(warmup):
                graph.replay()
            self.stream.synchronize()
            times = []
            for _ in range(runs):
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                begin.record(self.stream)
                for _ in range(measured):
                    graph.replay()
                end.record(self.stream)
                self.stream.synchronize()
                times.append(begin.elapsed_time(end) / measured)
        return times

    # -- the protocol ------------------------------------------------------------
    def run(self, warmup: int, measured: int, runs: int) -> dict:
        self._set(1)
        expected = self._outputs(self.probes())
        rows = []
        for lookahead in CANDIDATES:
            worst = self.disagreement(lookahead, expected)
            if worst > AGREEMENT_LIMIT:
                raise RuntimeError(f"lookahead K={lookahead} failed correctness: max_abs={worst}")
            times = self.sweep_times(lookahead, warmup, measured, runs)
            rows.append({"lookahead": lookahead, "max_abs_vs_k1": worst, "sweep_ms_median": statistics.median(times),
                         "sweep_ms_min": min(times), "sweep_ms_max": max(times), "runs": times})
            print(json.dumps(rows[-1]), flush=True)
        best = min(rows, key=lambda row: row["sweep_ms_median"])
        major, minor = torch.cuda.get_device_capability()
        return {"schema_version": 1, "device": torch.cuda.get_device_name(), "compute_capability": f"{major}.{minor}",
                "weights_metadata_sha256": sha256_file(self.metadata_path), "palette_sha256": self.palette_sha256,
                "artifact": str(self.artifact.resolve()), "runtime_dtype": self.dtype_name, "linears": len(self.entries),
                "warmup_sweeps": warmup, "measured_sweeps": measured, "independent_runs": runs,
                "timing": "CUDA-graph replays of one sweep between CUDA events",
                "selected_lookahead": best["lookahead"], "candidates": rows}


def tune_artifact(artifact: Path, warmup: int = 10, measured: int = 50, runs: int = 3) -> dict:
    """Measure every candidate on ``artifact`` and store the profile (the reference's entry point)."""
    with LookaheadTuner(artifact) as tuner:
        profile = tuner.run(warmup, measured, runs)
    target = _profile_path(Path(artifact))
    write_json(target, profile)
    print(f"[texelator] selected K={profile['selected_lookahead']}; local benchmark profile saved to {target}")
    return profile


def selected_lookahead(artifact: Path) -> tuple[int, Path | None]:
    """The stored choice for this artefact on this GPU, or ``(1, None)``; a profile made for other
    weights or another palette is refused (tuning.py:134-145)."""
    artifact = Path(artifact)
    target = _profile_path(artifact)
    if not target.exists():
        return 1, None
    profile = json.loads(target.read_text())
    checks = (("weights_metadata_sha256", sha256_file(artifact / "weights" / "metadata.json"), "the encoded weights"),
              ("palette_sha256", json.loads((artifact / "texelator.json").read_text()).get("hardware", {}).get("palette_sha256"),
               "the model palette"))
    for key, current, what in checks:
        if profile.get(key) != current:
            raise RuntimeError(f"benchmark profile does not match {what}; rerun texelator benchmark")
    return int(profile["selected_lookahead"]), target
