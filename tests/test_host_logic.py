"""Host-side logic that needs no GPU: adapters, artefact files, profile validation, TP slicing."""
import json

import numpy as np
import pytest
import torch
from torch import nn

from oracle import bc4_oracle as O
from texelator_b200 import adapters, artifacts, autotune, tp


class _Block(nn.Module):
    def __init__(self, k=32):
        super().__init__()
        self.q_proj = nn.Linear(k, 16, bias=True)
        self.down_proj = nn.Linear(k, 8, bias=False)
        self.other = nn.Linear(k, 8)


class _Toy(nn.Module):
    def __init__(self, k=32):
        super().__init__()
        self.layers = nn.ModuleList([_Block(k), _Block(k)])
        self.lm_head = nn.Linear(k, 10)


def test_discover_linears_and_k_gate():
    specs = adapters.discover_linears(_Toy())
    assert [s.module_name for s in specs] == ["layers.0.down_proj", "layers.0.q_proj", "layers.1.down_proj", "layers.1.q_proj"]
    assert all(s.supported for s in specs) and specs[1].bias and not specs[0].bias
    bad = adapters.discover_linears(_Toy(k=24))
    assert not any(s.supported for s in bad) and "divisible by 16" in bad[0].reason
    assert "layers.0.other" in [s.module_name for s in adapters.discover_linears(_Toy(), include_regex=r"other$")]
    key = adapters.artifact_key("model.layers.0.self_attn.q_proj")
    assert key.startswith("model__layers__0__self_attn__q_proj--") and len(key.rsplit("--", 1)[1]) == 10
    parent, child = adapters.resolve_parent(_Toy(), "layers.1.q_proj")
    assert child == "q_proj" and isinstance(getattr(parent, child), nn.Linear)
    with pytest.raises(RuntimeError):
        adapters.resolve_parent(_Toy(), "missing")


def _entries(tmp_path, lut, shapes):
    entries = []
    rng = np.random.default_rng(0)
    for index, (name, m, k) in enumerate(shapes):
        w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
        blocks, scales = O.encode_minmax(w, lut)
        entries.append(artifacts.write_encoded_entry(tmp_path / "weights", name, index, blocks, scales))
    return entries


def test_artifact_files_follow_the_reference_format(tmp_path, lut):
    entries = _entries(tmp_path, lut, [("model.layers.0.mlp.up_proj", 32, 64), ("model.layers.1.mlp.down_proj", 16, 128)])
    artifacts.write_artifact(tmp_path, entries, O.palette_sha256(lut))
    metadata = json.loads((tmp_path / "weights" / "metadata.json").read_text())
    assert metadata["format"] == "BC4_SNORM + one FP32 scale per output row" and metadata["schema_version"] == 1
    first = metadata["entries"][0]
    assert first["blocks_bytes"] == first["M"] * first["K"] // 2 and first["scales_bytes"] == 4 * first["M"]
    assert first["blocks_file"].endswith(".bc4") and first["scales_file"].endswith(".scales.f32")
    assert artifacts.validate_encoded(tmp_path / "weights")["ok"]
    (tmp_path / "weights" / first["scales_file"]).write_bytes(b"\0" * first["scales_bytes"])
    assert not artifacts.validate_encoded(tmp_path / "weights")["ok"]
    manifest = json.loads((tmp_path / "texelator.json").read_text())
    assert manifest["format"] == "texelator-bc4-v1" and manifest["runtime_dtype"] == "bfloat16"
    assert manifest["hardware"]["palette_sha256"] == O.palette_sha256(lut)


def test_autotune_keys_and_profile_refusals():
    assert autotune.token_bucket(1) == 32 and autotune.token_bucket(33) == 128 and autotune.token_bucket(65535) == 65535
    with pytest.raises(ValueError):
        autotune.token_bucket(0)
    with pytest.raises(ValueError):
        autotune.token_bucket(70000)
    assert autotune.dispatch_key(100, 5120, 17408) == "tokens<=128:M=5120:K=17408"
    assert list(autotune.CANDIDATES.values()) == [5, 6, 7, 8, 9]
    good = {"kernel_source_sha256": autotune.kernel_source_sha256(),
            "device": {"compute_capability": [10, 0], "multiprocessor_count": 148}}
    autotune.check_profile(good, [10, 0], 148)
    with pytest.raises(RuntimeError, match="kernel hash"):
        autotune.check_profile(dict(good, kernel_source_sha256="0"), [10, 0], 148)
    with pytest.raises(RuntimeError, match="compute capability"):
        autotune.check_profile(good, [9, 0], 148)
    with pytest.raises(RuntimeError, match="SM count"):
        autotune.check_profile(good, [10, 0], 132)


def test_lookahead_profile_validation(tmp_path, lut, monkeypatch):
    from texelator_b200 import tuning
    monkeypatch.setenv("TEXELATOR_HOME", str(tmp_path / "state"))
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda *a: (10, 0))
    monkeypatch.setattr(torch.cuda, "get_device_name", lambda *a: "NVIDIA B200")
    entries = _entries(tmp_path / "art", lut, [("model.layers.0.mlp.up_proj", 32, 64)])
    artifacts.write_artifact(tmp_path / "art", entries, O.palette_sha256(lut))
    assert tuning.selected_lookahead(tmp_path / "art") == (1, None)
    target = tuning._profile_path(tmp_path / "art")
    assert target.name == "sm_100-nvidia-b200.json"
    artifacts.write_json(target, {"weights_metadata_sha256": artifacts.sha256_file(tmp_path / "art" / "weights" / "metadata.json"),
                                  "palette_sha256": O.palette_sha256(lut), "selected_lookahead": 4})
    assert tuning.selected_lookahead(tmp_path / "art")[0] == 4
    artifacts.write_json(target, {"weights_metadata_sha256": "x", "palette_sha256": O.palette_sha256(lut), "selected_lookahead": 4})
    with pytest.raises(RuntimeError, match="does not match the encoded weights"):
        tuning.selected_lookahead(tmp_path / "art")


def test_tp_shard_ranges_and_bytes(lut, golden_dir):
    z = np.load(golden_dir / "small_48x256.npz")
    m, k = 48, 256
    full = O.dequant_weights(z["blocks"], z["scales"], lut)
    for world in (2, 4):
        rows = [O.dequant_weights(*tp.shard_bytes(z["blocks"], z["scales"], m, k, "gate_proj", r, world), lut) for r in range(world)]
        assert np.array_equal(np.concatenate(rows, 0), full)
        cols = [O.dequant_weights(*tp.shard_bytes(z["blocks"], z["scales"], m, k, "down_proj", r, world), lut) for r in range(world)]
        assert np.array_equal(np.concatenate(cols, 1), full)
    assert tp.shard_ranges(5120, 17408, "down_proj", 7, 8) == ((0, 5120), (952, 1088))
    assert tp.shard_ranges(17408, 5120, "up_proj", 1, 8) == ((2176, 4352), (0, 320))
    with pytest.raises(ValueError):
        tp.shard_ranges(50, 256, "q_proj", 0, 4)
    with pytest.raises(ValueError):
        tp.shard_ranges(48, 48, "o_proj", 0, 2)
    with pytest.raises(ValueError):
        tp.shard_ranges(48, 256, "lm_head", 0, 2)


def test_model_config_byte_counts():
    from texelator_b200.modeling import CONFIGS
    assert CONFIGS["27b-class"].bc4_bytes_per_token() == 10583015424      # 10.583 GB per decoded token
    assert abs(CONFIGS["qwen2.5-3b-shaped"].bc4_bytes_per_token() / 1e9 - 1.391) < 0.002
    assert abs(CONFIGS["70b-class"].bc4_bytes_per_token() / 1e9 - 34.252) < 0.002


def test_directory_written_by_the_reference_is_read_unchanged(golden_dir, lut):
    """``reference_artifact/`` was written by the reference's own discover_linears / encode_linear_e3 / write_json
    (tests/golden/make_artifact.py): its checksums validate, its entries carry the fields this build writes, and
    the restated encoder reproduces its files byte for byte from the recorded inputs."""
    import json
    from oracle import bc4_oracle as O
    from texelator_b200 import artifacts
    root = golden_dir / "reference_artifact"
    validation = artifacts.validate_encoded(root / "weights")
    assert validation["ok"] and validation["entries"] == 3
    metadata = json.loads((root / "weights" / "metadata.json").read_text())
    assert metadata["palette_sha256"] == O.palette_sha256(lut)
    inputs = np.load(root / "inputs.npz")
    for entry in metadata["entries"]:
        assert entry["artifact_key"] == artifacts.artifact_key(entry["module_name"])
        blocks = np.fromfile(root / "weights" / entry["blocks_file"], dtype=np.uint8)
        scales = np.fromfile(root / "weights" / entry["scales_file"], dtype="<f4")
        assert blocks.size == entry["M"] * entry["K"] // 2 == entry["blocks_bytes"] and scales.size == entry["M"]
        key = entry["artifact_key"]
        again_blocks, again_scales = O.encode_linear(inputs[f"{key}/weight"], inputs[f"{key}/hdiag"], lut)
        assert np.array_equal(again_blocks, blocks) and np.array_equal(again_scales, scales)
