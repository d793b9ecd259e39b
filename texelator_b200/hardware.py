"""Palette tables of this GPU and the palette-hash gate.

The reference measures the texture unit's BC4 palette once per GPU and caches it under
``STATE_HOME/hardware/sm_XY/palette.bin`` (texelator/hardware.py:15-60); encoded models carry the
SHA-256 of the palette they were encoded against and tools refuse to run on a mismatch
(texelator/tuning.py:38-41).  This build decodes with the *software* BC4-SNORM palette in ALU, so
``ensure_hardware`` caches two tables:

* ``palette.bin``          -- the table the library's ALU decoder produces (``tx_software_palette``);
                              this is the palette models for this build are encoded against;
* ``texture_palette.bin``  -- the table measured through a signed-BC4 CUDA texture object
                              (``tx_palette_probe``), when the device can create such views.

The texture decode path is only allowed when both hashes agree -- the reference's gate -- otherwise
the ALU path stays in force.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from .artifacts import environment_snapshot, sha256_file, state_home, write_json

# Published hash of the texture-unit palette of RTX 4060 / 4080 SUPER / 5080
# (WINDOWS_VALIDATION.md:13-14, research/results/paper/environment.json:32-36).
REFERENCE_TEXTURE_PALETTE_SHA256 = "34670bd1c521c26b14ea88ed6f2d8f16c55720f20915909ac621dcabe0f3ed47"


def ensure_hardware(force: bool = False) -> Path:
    if not torch.cuda.is_available():
        raise RuntimeError("Texelator requires CUDA-enabled PyTorch and a visible NVIDIA GPU")
    major, minor = torch.cuda.get_device_capability()
    destination = state_home() / "hardware" / f"sm_{major}{minor}"
    palette = destination / "palette.bin"
    if palette.exists() and not force:
        return palette
    from .runtime import extension
    destination.mkdir(parents=True, exist_ok=True)
    ext = extension()
    print(f"[texelator] decoding the BC4 palette on {torch.cuda.get_device_name()}...", flush=True)
    values = ext.software_palette().contiguous()
    values.numpy().astype("<f4", copy=False).tofile(palette)
    info = {"device": torch.cuda.get_device_name(), "compute_capability": f"{major}.{minor}",
            "endpoint_pairs": 255 * 255, "values_per_pair": 8, "bytes": int(values.numel() * values.element_size()),
            "source": "alu-decoder", "texture_views": bool(ext.texture_supported())}
    if ext.texture_supported():
        measured = ext.palette_probe().contiguous()
        measured.numpy().astype("<f4", copy=False).tofile(destination / "texture_palette.bin")
        info["texture_palette_sha256"] = sha256_file(destination / "texture_palette.bin")
        info["texture_matches_published_hash"] = info["texture_palette_sha256"] == REFERENCE_TEXTURE_PALETTE_SHA256
    write_json(destination / "palette.json", info)
    write_json(destination / "environment.json", environment_snapshot())
    return palette


def texture_path_allowed() -> bool:
    """True when the texture unit reproduces the decoder's palette bit for bit."""
    palette = ensure_hardware()
    measured = palette.with_name("texture_palette.bin")
    return measured.exists() and sha256_file(measured) == sha256_file(palette)


def doctor_payload(force: bool = False) -> dict:
    palette = ensure_hardware(force=force)
    metadata = json.loads(palette.with_name("palette.json").read_text())
    return {"status": "ready", "state_home": str(state_home()), "palette": str(palette),
            "palette_sha256": sha256_file(palette), "texture_path_allowed": texture_path_allowed(), **metadata}
