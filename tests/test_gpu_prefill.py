"""GPU parity of the tensor-core prefill tiles and of the tuners (run with ``-m gpu``)."""
import numpy as np
import pytest
import torch

from oracle import bc4_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from texelator_b200 import runtime
    return runtime.extension()


def _case(seed, m, k, tokens, lut, sparse=0.0, x_scale=1.0):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    if sparse:
        w[rng.random((m, k)) < sparse] = 0
    blocks, scales = O.encode_minmax(w, lut)
    x = torch.from_numpy((rng.standard_normal((tokens, k)) * x_scale).astype(np.float32)).bfloat16()
    return blocks, scales, x


def _pack(ext, blocks, scales, bias=None):
    return ext.pack_encoded(torch.from_numpy(blocks), torch.from_numpy(scales), bias)


@pytest.mark.parametrize("backend", [5, 6, 7, 8, 9])
@pytest.mark.parametrize("m,k,tokens", [(128, 128, 32), (256, 512, 40), (200, 48, 17), (1024, 1024, 128),
                                        (136, 2064, 300), (5120, 640, 512)])
def test_prefill_tiles_match_oracle(ext, lut, backend, m, k, tokens):
    blocks, scales, x = _case(m + k + tokens, m, k, tokens, lut)
    bias = torch.from_numpy(np.random.default_rng(2).standard_normal(m).astype(np.float32)).bfloat16().cuda()
    h = _pack(ext, blocks, scales, bias)
    try:
        ext.set_prefill(h, 16, 1024)
        ext.set_prefill_backend(h, backend)
        y = ext.linear(h, x.cuda())
        torch.cuda.synchronize()
        assert ext.kernel_status() == 0
        ref = O.linear_bf16(x.float().numpy(), blocks, scales, lut, bias=bias.float().cpu().numpy())
        err = O.rel_rms(y.float().cpu().numpy(), ref)
        assert err <= 1e-2, (backend, m, k, tokens, err)       # stated tolerance vs dequantise-then-matmul
    finally:
        ext.free(h)


def test_prefill_tiles_are_bitwise_identical(ext, lut):
    """The reference's admission rule (texelator/autotune.py:160-168)."""
    blocks, scales, x = _case(9, 384, 1024, 200, lut, x_scale=0.125)
    h = _pack(ext, blocks, scales)
    try:
        ext.set_prefill(h, 1, 32768)
        outs = []
        for backend in (5, 6, 7, 8, 9):
            ext.set_prefill_backend(h, backend)
            outs.append(ext.linear(h, x.cuda()))
        for other in outs[1:]:
            assert torch.equal(outs[0], other)
    finally:
        ext.free(h)


def test_prefill_low_mode_blocks(ext, lut):
    blocks, scales, x = _case(4, 256, 512, 64, lut, sparse=0.9)
    h = _pack(ext, blocks, scales)
    try:
        ext.set_prefill_backend(h, 6)
        y = ext.linear(h, x.cuda()).float().cpu().numpy()
        assert O.rel_rms(y, O.linear_bf16(x.float().numpy(), blocks, scales, lut)) <= 1e-2
    finally:
        ext.free(h)


def test_threshold_split_and_hybrid_agreement(ext, lut):
    """tokens < threshold streams through the decode GEMV, tokens >= threshold through the tile;
    both sides of the dispatcher agree within the reference's hybrid gate (rel-RMS <= 0.02,
    texelator/prefill.py:107)."""
    blocks, scales, x = _case(6, 512, 1024, 32, lut)
    h = _pack(ext, blocks, scales)
    try:
        ext.set_prefill_backend(h, 5)
        ext.set_prefill(h, 1 << 30, 1024)
        before = ext.launch_count()
        scalar = ext.linear(h, x.cuda()).float().cpu().numpy()
        ext.set_prefill(h, 1, 1024)
        hybrid = ext.linear(h, x.cuda()).float().cpu().numpy()
        assert ext.launch_count() > before
        assert O.rel_rms(hybrid, scalar) <= 0.02
    finally:
        ext.free(h)


def test_kernel_info_and_autotune_protocol(ext, lut, tmp_path, monkeypatch):
    from texelator_b200 import artifacts, autotune
    monkeypatch.setenv("TEXELATOR_HOME", str(tmp_path / "state"))
    for backend in (0, 5, 6, 7, 8, 9):
        info = ext.kernel_info(backend)
        assert len(info) == 9 and info[0] > 0 and info[8] >= 1
    entries = []
    for index, (m, k) in enumerate([(256, 512), (512, 256)]):
        blocks, scales, _ = _case(index, m, k, 1, lut)
        entries.append(artifacts.write_encoded_entry(tmp_path / "art" / "weights", f"model.layers.{index}.mlp.up_proj", index, blocks, scales))
    artifacts.write_artifact(tmp_path / "art", entries, O.palette_sha256(lut))
    profile = autotune.tune_artifact(tmp_path / "art", tmp_path / "profile.json", [32, 128], warmup=3, measured=10)
    assert profile["status"] == "complete" and len(profile["selections"]) == 4
    for record in profile["selections"].values():
        assert record["correctness_vs_baseline"][autotune.BASELINE]["bitwise_equal"]
        assert not record["rejected"]                          # every tile is bitwise identical to the baseline
    handles = []
    try:
        from texelator_b200 import runtime
        for entry in entries:
            handles.extend(runtime.pack_entry_handles(tmp_path / "art" / "weights", entry))
        assert autotune.apply_profile(handles, 100, profile) is True
        assert autotune.apply_profile(handles, 4000, profile) is False     # unknown bucket -> baseline tile
        assert ext.handle_info(handles[0])[2] == runtime.PREFILL_THRESHOLD  # threshold untouched
    finally:
        from texelator_b200 import runtime
        runtime.free(handles)


def test_lookahead_tuner_protocol(ext, lut, tmp_path, monkeypatch):
    from texelator_b200 import artifacts, tuning
    monkeypatch.setenv("TEXELATOR_HOME", str(tmp_path / "state"))
    entries = []
    for index, (m, k) in enumerate([(256, 512), (512, 256), (1024, 1024)]):
        blocks, scales, _ = _case(index, m, k, 1, lut)
        entries.append(artifacts.write_encoded_entry(tmp_path / "art" / "weights", f"model.layers.{index}.self_attn.q_proj", index, blocks, scales))
    artifacts.write_artifact(tmp_path / "art", entries, O.palette_sha256(lut))
    profile = tuning.tune_artifact(tmp_path / "art", warmup=2, measured=5, runs=2)
    assert profile["selected_lookahead"] in tuning.CANDIDATES
    assert [row["lookahead"] for row in profile["candidates"]] == list(tuning.CANDIDATES)
    assert all(row["max_abs_vs_k1"] <= 1e-3 for row in profile["candidates"])
    assert tuning.selected_lookahead(tmp_path / "art")[0] == profile["selected_lookahead"]
    # palette gate: an artefact encoded against an unknown palette is refused (texelator/tuning.py:38-41)
    artifacts.write_artifact(tmp_path / "art", entries, "0" * 64)
    with pytest.raises(RuntimeError, match="palette does not match"):
        tuning.tune_artifact(tmp_path / "art", warmup=1, measured=1, runs=1)
    # ... while the texture-unit palette the reference publishes is accepted where this GPU's texture
    # unit reproduces it, and such artefacts are packed in hardware-palette mode
    if ext.texture_supported() and O.palette_sha256(ext.palette_probe().numpy()) == O.REFERENCE_TEXTURE_PALETTE_SHA256:
        from texelator_b200 import runtime
        artifacts.write_artifact(tmp_path / "art", entries, O.REFERENCE_TEXTURE_PALETTE_SHA256)
        assert runtime.palette_of(tmp_path / "art" / "weights") == runtime.PALETTE_HARDWARE
        assert tuning.tune_artifact(tmp_path / "art", warmup=1, measured=2, runs=1)["palette_sha256"] == O.REFERENCE_TEXTURE_PALETTE_SHA256


def test_hardware_palettes_and_texture_gate(ext, lut, tmp_path, monkeypatch):
    from texelator_b200 import hardware
    monkeypatch.setenv("TEXELATOR_HOME", str(tmp_path / "state"))
    payload = hardware.doctor_payload(force=True)
    assert payload["palette_sha256"] == O.palette_sha256(lut)
    blocks, scales, x = _case(1, 64, 128, 1, lut)
    h = _pack(ext, blocks, scales)
    try:
        if payload["texture_views"] and not payload["texture_path_allowed"]:
            # texture unit palette differs from the encoder's palette -> ALU path stays in force
            with pytest.raises(RuntimeError, match="palette does not match"):
                ext.set_decode_path(h, 2)
            assert ext.handle_info(h)[5] == 0
    finally:
        ext.free(h)
