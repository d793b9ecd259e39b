"""Files and JSON conventions of encoded BC4 artefacts.

Reads and writes what the reference's converter emits, so a reference-encoded model directory
loads unchanged: ``weights/metadata.json`` + ``<key>.bc4`` + ``<key>.scales.f32``
(texelator/converter.py:200-209, texelator/encoder.py:148-157), ``texelator.json``
(converter.py:215-230), the state directory (texelator/store.py:10-15) and the helpers of
texelator/artifacts.py (``sha256_file`` :16-21, ``write_json`` :24-28, ``environment_snapshot``
:51-73, ``validate_encoded`` :76-87).
"""
from __future__ import annotations

import datetime
import hashlib
import json
import os
import platform
import re
import sys
from pathlib import Path

import numpy as np
import torch

from .adapters import artifact_key

STATE_HOME = Path(os.environ.get("TEXELATOR_HOME", Path.home() / ".cache" / "texelator")).expanduser().resolve()
WEIGHT_FORMAT = "BC4_SNORM + one FP32 scale per output row"


def state_home() -> Path:
    """``TEXELATOR_HOME`` is read at call time so tests can redirect it."""
    return Path(os.environ.get("TEXELATOR_HOME", STATE_HOME)).expanduser().resolve()


def safe_name(value: str) -> str:
    return re.sub(r"[^A-Za-z0-9_.-]+", "-", value).strip("-").lower()


def sha256_file(path: Path) -> str:
    digest = hashlib.sha256()
    with Path(path).open("rb") as handle:
        for chunk in iter(lambda: handle.read(8 << 20), b""):
            digest.update(chunk)
    return digest.hexdigest()


def write_json(path: Path, value) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    temporary = path.with_suffix(path.suffix + ".tmp")
    temporary.write_text(json.dumps(value, indent=2, sort_keys=True) + "\n")
    temporary.replace(path)


def environment_snapshot() -> dict:
    gpu = None
    if torch.cuda.is_available():
        properties = torch.cuda.get_device_properties(torch.cuda.current_device())
        gpu = {"name": properties.name, "compute_capability": f"{properties.major}.{properties.minor}",
               "total_memory_bytes": properties.total_memory, "cuda_runtime": torch.version.cuda}
    return {"timestamp_utc": datetime.datetime.now(datetime.timezone.utc).isoformat(), "hostname": platform.node(),
            "platform": platform.platform(), "python": sys.version, "torch": torch.__version__, "gpu": gpu,
            "command": sys.argv, "cwd": os.getcwd()}


def validate_encoded(encoded: Path) -> dict:
    metadata = json.loads((Path(encoded) / "metadata.json").read_text())
    failures = []
    for entry in metadata["entries"]:
        for kind in ("blocks", "scales"):
            path = Path(encoded) / entry[f"{kind}_file"]
            actual = sha256_file(path)
            if actual != entry[f"{kind}_sha256"]:
                failures.append({"module_name": entry["module_name"], "file": str(path),
                                 "expected": entry[f"{kind}_sha256"], "actual": actual})
    return {"ok": not failures, "entries": len(metadata["entries"]), "failures": failures}


def write_encoded_entry(weights: Path, module_name: str, layer: int, blocks: np.ndarray, scales: np.ndarray,
                        bias: bool = False) -> dict:
    """Write one linear's ``.bc4`` / ``.scales.f32`` pair and return its metadata entry
    (LinearSpec fields of texelator/adapters.py:27-40 + the file fields of encoder.py:148-157)."""
    weights = Path(weights)
    weights.mkdir(parents=True, exist_ok=True)
    key = artifact_key(module_name)
    m = int(scales.shape[0])
    k = int(blocks.size // (m * 8) * 16)
    blocks_path, scales_path = weights / f"{key}.bc4", weights / f"{key}.scales.f32"
    np.ascontiguousarray(blocks, dtype=np.uint8).tofile(blocks_path)
    np.ascontiguousarray(scales, dtype="<f4").tofile(scales_path)
    return {"module_name": module_name, "artifact_key": key, "layer": layer, "op": module_name.rsplit(".", 1)[-1],
            "M": m, "K": k, "bias": bias, "supported": True, "reason": "ok",
            "blocks_file": blocks_path.name, "blocks_bytes": blocks_path.stat().st_size,
            "blocks_sha256": sha256_file(blocks_path), "scales_file": scales_path.name,
            "scales_bytes": scales_path.stat().st_size, "scales_sha256": sha256_file(scales_path)}


def write_artifact(artifact: Path, entries: list[dict], palette_sha256: str, name: str = "synthetic",
                   runtime_dtype: str = "bfloat16", encoder: str = "e3") -> Path:
    """``weights/metadata.json`` and ``texelator.json`` around already written entries."""
    artifact = Path(artifact)
    write_json(artifact / "weights" / "metadata.json", {
        "schema_version": 1, "format": WEIGHT_FORMAT, "encoder": encoder, "palette_sha256": palette_sha256,
        "entries": entries, "bc4_bytes": sum(e["blocks_bytes"] for e in entries),
        "scale_bytes": sum(e["scales_bytes"] for e in entries)})
    write_json(artifact / "texelator.json", {
        "schema_version": 1, "format": "texelator-bc4-v1", "name": name, "source": None, "inspection": None,
        "calibration": None, "hardware": {"palette": "palette.bin", "palette_sha256": palette_sha256},
        "weights": "weights", "validation": None, "linked_source": None, "runtime_dtype": runtime_dtype})
    return artifact
