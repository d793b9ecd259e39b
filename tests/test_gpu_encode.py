"""The GPU encoder against the reference encoder's recorded output (run with ``-m gpu``)."""
import hashlib
import json

import numpy as np
import pytest
import torch

from oracle import bc4_oracle as O

pytestmark = pytest.mark.gpu

GOLDEN = ["small_48x256", "odd_24x48", "edge_32x128", "tall_130x64"]


@pytest.fixture(scope="module")
def ext():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from texelator_b200 import runtime
    return runtime.extension()


@pytest.mark.parametrize("name", GOLDEN)
def test_gpu_encoder_reproduces_the_reference_bytes(ext, lut, golden_dir, name):
    """The fixtures hold what the unmodified reference encoder wrote for these weights and moments."""
    z = np.load(golden_dir / f"{name}.npz")
    blocks, scales = ext.encode(torch.from_numpy(z["weight"]).cuda(), torch.from_numpy(z["hdiag"]).cuda(), torch.from_numpy(lut).cuda())
    assert np.array_equal(scales.cpu().numpy(), z["scales"])
    assert np.array_equal(blocks.cpu().numpy(), z["blocks"])


def test_gpu_encoder_configuration_1_hash(ext, lut, golden_dir):
    """4096 x 4096 from the pinned seed: 1 048 576 blocks, hashes recorded from the reference encoder."""
    manifest = json.loads((golden_dir / "manifest.json").read_text())["cases"]["cfg1_4096x4096"]
    g = torch.Generator().manual_seed(manifest["seed"])
    w = torch.randn(4096, 4096, generator=g) * 0.02
    xc = torch.randn(64, 4096, generator=g)
    blocks, scales = ext.encode(w.cuda(), (xc * xc).mean(0).cuda(), torch.from_numpy(lut).cuda())
    assert hashlib.sha256(blocks.cpu().numpy().tobytes()).hexdigest() == manifest["blocks_sha256"]
    assert hashlib.sha256(scales.cpu().numpy().astype("<f4").tobytes()).hexdigest() == manifest["scales_sha256"]


@pytest.mark.parametrize("palette", ["software", "hardware"])
def test_gpu_encoder_equals_restated_encoder_on_hard_inputs(ext, lut, palette):
    """Sparse rows (low-mode blocks, degenerate normal equations), constant and zero rows, +-max entries, a wide
    range of activation weights -- against the CPU restatement, under both palettes."""
    table = lut if palette == "software" else O.hardware_palette()
    rng = np.random.default_rng(5)
    m, k = 96, 512
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    w[rng.random((m, k)) < 0.7] = 0
    w[3] = 0
    w[4] = 0.125
    w[5, ::2] = w[5].max()
    w[6, 1::2] = -np.abs(w[6]).max()
    hdiag = np.exp(rng.standard_normal(k) * 3).astype(np.float32)
    want_blocks, want_scales = O.encode_linear(w, hdiag, table)
    blocks, scales = ext.encode(torch.from_numpy(w).cuda(), torch.from_numpy(hdiag).cuda(), torch.from_numpy(table).cuda())
    assert np.array_equal(scales.cpu().numpy(), want_scales)
    got = blocks.cpu().numpy()
    differing = np.flatnonzero((got.reshape(-1, 8) != want_blocks.reshape(-1, 8)).any(1))
    assert differing.size == 0, differing[:10]


def test_gpu_encoder_feeds_the_operator(ext, lut):
    """Encode on the GPU, pack without a host round trip, multiply: the whole path against the oracle."""
    rng = np.random.default_rng(8)
    m, k = 256, 1024
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    hdiag = (rng.standard_normal((64, k)) ** 2).mean(0).astype(np.float32)
    blocks, scales = ext.encode(torch.from_numpy(w).cuda(), torch.from_numpy(hdiag).cuda(), torch.from_numpy(lut).cuda())
    handle = ext.pack_encoded_device(blocks, scales)
    try:
        x = torch.from_numpy(rng.standard_normal((2, k)).astype(np.float32)).bfloat16()
        y = ext.linear(handle, x.cuda()).float().cpu().numpy()
        ref = O.linear_bf16(x.float().numpy(), blocks.cpu().numpy(), scales.cpu().numpy(), lut)
        assert O.rel_rms(y, ref) <= 1e-2
        # the encoder's point: the weighted error is no worse than the min/max start's
        start_blocks, start_scales = O.encode_minmax(w, lut)
        def weighted_error(b, s):
            return float(((O.dequant_weights(b, s, lut, round_bf16=False) - w) ** 2 * hdiag[None, :]).sum())
        assert weighted_error(blocks.cpu().numpy(), scales.cpu().numpy()) <= weighted_error(start_blocks, start_scales)
    finally:
        ext.free(handle)


def test_directory_written_by_the_reference_loads_and_runs(ext, lut, golden_dir):
    """The fixture directory written by the reference's encode_linear_e3 goes through ``pack_entry_handles``
    unchanged (bias attached like ``runtime.install`` does), multiplies like the oracle says, unpacks to the
    file's bytes, and the GPU encoder reproduces the files from the recorded fp32 inputs."""
    import json
    from texelator_b200 import runtime
    root = golden_dir / "reference_artifact"
    metadata = json.loads((root / "weights" / "metadata.json").read_text())
    inputs = np.load(root / "inputs.npz")
    rng = np.random.default_rng(11)
    for entry in metadata["entries"]:
        key = entry["artifact_key"]
        blocks = np.fromfile(root / "weights" / entry["blocks_file"], dtype=np.uint8)
        scales = np.fromfile(root / "weights" / entry["scales_file"], dtype="<f4")
        bias = torch.from_numpy(inputs[f"{key}/bias"]).bfloat16().cuda() if entry["bias"] else None
        handles = runtime.pack_entry_handles(root / "weights", entry, bias=bias, lookahead=2)
        try:
            assert len(handles) == 1 and ext.handle_info(handles[0])[:2] == [entry["M"], entry["K"]]
            assert np.array_equal(ext.unpack_blocks(handles[0]).numpy(), blocks)
            x = torch.from_numpy(rng.standard_normal((3, entry["K"])).astype(np.float32)).bfloat16()
            y = ext.linear(handles[0], x.cuda()).float().cpu().numpy()
            ref = O.linear_bf16(x.float().numpy(), blocks, scales, lut, None if bias is None else bias.float().cpu().numpy())
            assert O.rel_rms(y, ref) <= 1e-2
        finally:
            runtime.free(handles)
        got_blocks, got_scales = ext.encode(torch.from_numpy(inputs[f"{key}/weight"]).cuda(), torch.from_numpy(inputs[f"{key}/hdiag"]).cuda(),
                                            torch.from_numpy(lut).cuda())
        assert np.array_equal(got_blocks.cpu().numpy(), blocks) and np.array_equal(got_scales.cpu().numpy(), scales)
