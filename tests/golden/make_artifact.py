"""Write the fixture ``reference_artifact/`` with the REFERENCE's own code.

Run once, in a container where the hp0303/Texelator tree is mounted:

    python tests/golden/make_artifact.py /path/to/Texelator

A three-linear toy module is discovered with the reference's ``adapters.discover_linears``, every linear is
encoded with the reference's ``encoder.encode_linear_e3`` (which writes the ``.bc4`` / ``.scales.f32`` files)
under the software palette, and ``weights/metadata.json``, ``validation.json`` and ``texelator.json`` are written
the way ``converter.py:200-231`` writes them (its ``write_json`` and ``validate_encoded``).  The fp32 weights,
biases and activation moments go to ``inputs.npz`` so that tests can re-encode them.  Nothing imports this
script and the reference tree is not needed at test time.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch
from torch import nn

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle import bc4_oracle as O  # noqa: E402  (only for the palette table)


class _Attention(nn.Module):
    def __init__(self):
        super().__init__()
        self.q_proj = nn.Linear(256, 48, bias=True)
        self.o_proj = nn.Linear(48, 256, bias=False)      # K = 48: three blocks per row


class _Mlp(nn.Module):
    def __init__(self):
        super().__init__()
        self.down_proj = nn.Linear(128, 40, bias=False)    # M = 40: not a multiple of 16


class _Layer(nn.Module):
    def __init__(self):
        super().__init__()
        self.self_attn, self.mlp = _Attention(), _Mlp()


class _Toy(nn.Module):
    def __init__(self):
        super().__init__()
        self.layers = nn.ModuleList([_Layer()])


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from texelator import adapters as A, artifacts as F, encoder as E   # the reference, unmodified

    torch.manual_seed(20260827)
    model = _Toy()
    for parameter in model.parameters():
        parameter.data.mul_(0.3)
    destination = HERE / "reference_artifact"
    weights = destination / "weights"
    weights.mkdir(parents=True, exist_ok=True)
    table = O.software_palette()
    lut = torch.from_numpy(table)
    palette_hash = O.palette_sha256(table)
    entries, inputs = [], {}
    generator = torch.Generator().manual_seed(7)
    for spec in A.discover_linears(model):
        if not spec.supported:
            continue
        module = model.get_submodule(spec.module_name)
        calibration = torch.randn(64, spec.K, generator=generator)
        hdiag = (calibration * calibration).mean(0)
        result = E.encode_linear_e3(module.weight.detach(), hdiag, lut, weights / f"{spec.artifact_key}.bc4",
                                    weights / f"{spec.artifact_key}.scales.f32", 128)
        entries.append({**spec.to_dict(), **result})
        inputs[f"{spec.artifact_key}/weight"] = module.weight.detach().numpy()
        inputs[f"{spec.artifact_key}/hdiag"] = hdiag.numpy()
        if module.bias is not None:
            inputs[f"{spec.artifact_key}/bias"] = module.bias.detach().numpy()
    F.write_json(weights / "metadata.json", {
        "schema_version": 1, "format": "BC4_SNORM + one FP32 scale per output row", "encoder": "hardware-exact activation-aware",
        "palette_sha256": palette_hash, "entries": entries, "bc4_bytes": sum(item["blocks_bytes"] for item in entries),
        "scale_bytes": sum(item["scales_bytes"] for item in entries)})
    validation = F.validate_encoded(weights)
    assert validation["ok"], validation
    F.write_json(destination / "validation.json", validation)
    F.write_json(destination / "texelator.json", {
        "schema_version": 1, "format": "texelator-bc4-v1", "name": destination.name, "source": None, "inspection": None,
        "calibration": None, "hardware": {"palette": "software", "palette_sha256": palette_hash}, "weights": "weights",
        "validation": "validation.json", "linked_source": True})
    np.savez(destination / "inputs.npz", **inputs)
    print(f"wrote {destination}: {[entry['module_name'] for entry in entries]}")


if __name__ == "__main__":
    main(sys.argv[1])
