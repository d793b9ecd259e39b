"""The CPU oracle against the fixtures recorded from the reference encoder
(tests/golden/make_golden.py) and against known answers of the format."""
import hashlib
import json

import numpy as np
import pytest
import torch

from oracle import bc4_oracle as O

CASES = ["small_48x256", "odd_24x48", "edge_32x128", "tall_130x64"]


def test_palette_is_pinned(lut, golden_dir):
    manifest = json.loads((golden_dir / "manifest.json").read_text())
    assert lut.shape == (255, 255, 8) and lut.dtype == np.float32
    assert lut.nbytes == 2_080_800                      # palette.bin size of the reference probe
    assert O.palette_sha256(lut) == manifest["palette_sha256"]
    # BC4-SNORM identities: selector 0/1 are the endpoints e/127, 6/7 are -1/+1 in the low mode
    e = np.arange(-127, 128, dtype=np.float32) / np.float32(127)
    assert np.array_equal(lut[:, :, 0], np.broadcast_to(e[None, :], (255, 255)))
    assert np.array_equal(lut[:, :, 1], np.broadcast_to(e[:, None], (255, 255)))
    low = np.arange(255)[None, :] <= np.arange(255)[:, None]       # e0 <= e1
    assert np.all(lut[:, :, 6][low] == -1) and np.all(lut[:, :, 7][low] == 1)
    assert np.abs(lut).max() == 1.0


def test_hardware_palette_reproduces_the_published_hash():
    """Known answer of the reference: the texture-unit palette hash in WINDOWS_VALIDATION.md:13-14."""
    table = O.hardware_palette()
    assert table.shape == (255, 255, 8) and table.dtype == np.float32
    assert O.palette_sha256(table) == O.REFERENCE_TEXTURE_PALETTE_SHA256
    software = O.software_palette()
    differ = int((table != software).sum())
    assert differ == 453378                                   # the paper's count of differing entries (section IV-B)
    assert abs(float(np.abs(table - software).max()) - 0.05584) < 1e-4


def test_palette_is_monotone_between_endpoints(lut):
    order8 = [0, 2, 3, 4, 5, 6, 7, 1]
    hi = lut[0, 254][order8]                                       # e1=-127, e0=127
    assert np.all(np.diff(hi) < 0)
    assert np.allclose(hi, np.linspace(1, -1, 8), atol=1e-7)


@pytest.mark.parametrize("name", CASES)
def test_unpack_and_dequant_match_reference(name, lut, golden_dir):
    z = np.load(golden_dir / f"{name}.npz")
    m = z["scales"].shape[0]
    got = O.dequant_palette(z["blocks"], m, lut)
    assert np.array_equal(got.view(np.uint32), z["palette_values"].view(np.uint32))
    e0, e1, sel = O.unpack_blocks(z["blocks"], m)
    assert np.array_equal(O.pack_blocks(e0, e1, sel).reshape(-1), z["blocks"])
    assert z["blocks"].size == m * z["weight"].shape[1] // 2       # blocks_bytes = M*K/2
    assert np.array_equal(z["scales"], O.row_scales(z["weight"]))


@pytest.mark.parametrize("name", CASES)
def test_encoder_restatement_is_bit_identical(name, lut, golden_dir):
    z = np.load(golden_dir / f"{name}.npz")
    blocks, scales = O.encode_linear(z["weight"], z["hdiag"], lut)
    manifest = json.loads((golden_dir / "manifest.json").read_text())["cases"][name]
    assert hashlib.sha256(blocks.tobytes()).hexdigest() == manifest["blocks_sha256"]
    assert hashlib.sha256(scales.tobytes()).hexdigest() == manifest["scales_sha256"]
    assert np.array_equal(blocks, z["blocks"])


def test_edge_case_exercises_low_mode(lut, golden_dir):
    z = np.load(golden_dir / "edge_32x128.npz")
    e0, e1, sel = O.unpack_blocks(z["blocks"], 32)
    low = e0 <= e1
    assert low.sum() >= 8                              # constant / zero / sparse rows
    assert ((sel == 6) & low[:, :, None]).any() or ((sel == 7) & low[:, :, None]).any()
    # all-zero row decodes to exact zeros
    assert np.all(O.dequant_palette(z["blocks"], 32, lut)[0] == 0)


def test_handcrafted_pack_matches_reference(golden_dir):
    z = np.load(golden_dir / "handcrafted_blocks.npz")
    assert np.array_equal(O.pack_blocks(z["e0"], z["e1"], z["sel"]), z["packed"])
    e0, e1, sel = O.unpack_blocks(z["packed"].reshape(-1), 1)
    assert np.array_equal(e0[0], z["e0"]) and np.array_equal(e1[0], z["e1"])
    assert np.array_equal(sel[0], z["sel"])


def test_minus128_reads_as_minus127(lut):
    blk = O.pack_blocks(np.array([-128]), np.array([127]), (np.arange(16) % 8)[None, :])
    ref = O.pack_blocks(np.array([-127]), np.array([127]), (np.arange(16) % 8)[None, :])
    assert np.array_equal(O.dequant_palette(blk.reshape(-1), 1, lut), O.dequant_palette(ref.reshape(-1), 1, lut))


def test_bf16_round_matches_torch():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 3,
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, 1e-40], dtype=np.float32)])
    assert np.array_equal(O.bf16_round(x), torch.from_numpy(x).bfloat16().float().numpy())


@pytest.mark.parametrize("name", ["small_48x256", "edge_32x128"])
def test_linear_oracle_matches_torch_dequant_matmul(name, lut, golden_dir):
    """Dequantise-then-matmul written with torch ops (the reference's CPU-side
    semantics: LUT gather, fp32 scale, bf16 weights) agrees with the oracle."""
    z = np.load(golden_dir / f"{name}.npz")
    w = torch.from_numpy(z["palette_values"]) * torch.from_numpy(z["scales"])[:, None]
    y = (torch.from_numpy(z["x_bf16"]).double() @ w.bfloat16().double().T).float().bfloat16().float().numpy()
    got = O.linear_bf16(z["x_bf16"], z["blocks"], z["scales"], lut)
    assert np.array_equal(got, y)


def test_tp_slicing_reassembles(lut, golden_dir):
    z = np.load(golden_dir / "small_48x256.npz")
    full = O.dequant_weights(z["blocks"], z["scales"], lut)
    for world in (2, 4):
        rows = [O.dequant_weights(*O.shard_rows(z["blocks"], z["scales"], r, world), lut) for r in range(world)]
        assert np.array_equal(np.concatenate(rows, 0), full)
        cols = [O.dequant_weights(*O.shard_kblocks(z["blocks"], z["scales"], r, world), lut) for r in range(world)]
        assert np.array_equal(np.concatenate(cols, 1), full)


def test_minmax_encoder_emits_valid_blocks(lut):
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((16, 64)) * 0.02).astype(np.float32)
    blocks, scales = O.encode_minmax(w, lut)
    assert blocks.size == 16 * 64 // 2
    q = O.dequant_weights(blocks, scales, lut, round_bf16=False)
    assert O.rel_rms(q, w) < 0.15


def test_cfg1_full_size_encode_hash(lut, golden_dir):
    """Configuration 1 (4096x4096, seed 20260827): the restated encoder must
    reproduce the SHA-256 of the blocks the reference encoder wrote."""
    manifest = json.loads((golden_dir / "manifest.json").read_text())["cases"]["cfg1_4096x4096"]
    g = torch.Generator().manual_seed(manifest["seed"])
    w = torch.randn(4096, 4096, generator=g) * 0.02
    xc = torch.randn(64, 4096, generator=g)
    h = (xc * xc).mean(0)
    blocks, scales = O.encode_linear(w, h, lut)
    assert blocks.size == manifest["blocks_bytes"] and scales.nbytes == manifest["scales_bytes"]
    assert blocks[:128].tobytes().hex() == manifest["first_blocks_hex"]
    assert hashlib.sha256(blocks.tobytes()).hexdigest() == manifest["blocks_sha256"]
    assert hashlib.sha256(scales.tobytes()).hexdigest() == manifest["scales_sha256"]
