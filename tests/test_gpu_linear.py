"""GPU parity of the C-ABI operator against the CPU oracle (run with ``-m gpu``)."""
import json

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


def _pack(ext, blocks, scales, bias=None):
    return ext.pack_encoded(torch.from_numpy(np.ascontiguousarray(blocks)), torch.from_numpy(np.ascontiguousarray(scales)), bias)


def _random_case(seed, m, k, tokens, lut, std=0.02, sparse=0.0):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((m, k)) * std).astype(np.float32)
    if sparse:
        w[rng.random((m, k)) < sparse] = 0
    blocks, scales = O.encode_minmax(w, lut)
    x = torch.from_numpy(rng.standard_normal((tokens, k)).astype(np.float32)).bfloat16()
    return blocks, scales, x


GOLDEN = ["small_48x256", "odd_24x48", "edge_32x128", "tall_130x64"]


@pytest.mark.parametrize("name", GOLDEN)
def test_dequant_is_bit_exact(ext, lut, golden_dir, name):
    from texelator_b200 import runtime as R
    z = np.load(golden_dir / f"{name}.npz")
    h = _pack(ext, z["blocks"], z["scales"])
    try:
        pal = ext.dequant(h, R.DEQUANT_PALETTE_F32).cpu().numpy()
        assert np.array_equal(pal.view(np.uint32), z["palette_values"].view(np.uint32))
        scaled = ext.dequant(h, R.DEQUANT_SCALED_F32).cpu().numpy()
        assert np.array_equal(scaled, O.dequant_weights(z["blocks"], z["scales"], lut, round_bf16=False))
        wb = ext.dequant(h, R.DEQUANT_SCALED_BF16).float().cpu().numpy()
        assert np.array_equal(wb, O.dequant_weights(z["blocks"], z["scales"], lut))
        assert np.array_equal(ext.unpack_blocks(h).numpy(), z["blocks"])
    finally:
        ext.free(h)


def test_software_palette_table_is_bit_exact(ext, lut, golden_dir):
    """All 65 025 x 8 palette entries through the library's ALU decoder -- the palette-hash check."""
    table = ext.software_palette().numpy().reshape(255, 255, 8)
    assert np.array_equal(table.view(np.uint32), lut.view(np.uint32))
    manifest = json.loads((golden_dir / "manifest.json").read_text())
    assert O.palette_sha256(table) == manifest["palette_sha256"]


@pytest.mark.parametrize("path", [0, 1])
@pytest.mark.parametrize("name", GOLDEN)
def test_decode_gemv_matches_oracle_on_golden(ext, lut, golden_dir, name, path):
    z = np.load(golden_dir / f"{name}.npz")
    x = torch.from_numpy(z["x_bf16"]).bfloat16().cuda()
    h = _pack(ext, z["blocks"], z["scales"])
    try:
        ext.set_decode_path(h, path)
        y = ext.linear(h, x).float().cpu().numpy()
        ref = O.linear_bf16(z["x_bf16"], z["blocks"], z["scales"], lut)
        # stated tolerance of the operator: rel-RMS <= 1e-2 against dequantise-then-matmul
        assert O.rel_rms(y, ref) <= (1e-2 if path == 0 else 4e-3), (name, path, O.rel_rms(y, ref))
    finally:
        ext.free(h)


@pytest.mark.parametrize("m,k,tokens", [(8, 16, 1), (24, 32, 2), (40, 48, 3), (16, 4096, 1), (4096, 4096, 1),
                                        (1024, 5120, 1), (5120, 5120, 1), (512, 17408, 1), (2048, 2048, 7),
                                        (2048, 2048, 8), (1000, 1024, 9), (777 * 8, 512, 15), (64, 28672, 2)])
def test_decode_gemv_shapes(ext, lut, m, k, tokens):
    blocks, scales, x = _random_case(m * 31 + k + tokens, m, k, tokens, lut)
    bias = torch.from_numpy(np.random.default_rng(1).standard_normal(m).astype(np.float32)).bfloat16().cuda()
    h = _pack(ext, blocks, scales, bias)
    try:
        ref = O.linear_bf16(x.float().numpy(), blocks, scales, lut, bias=bias.float().cpu().numpy())
        for lookahead in (1, 4, 8):
            ext.set_lookahead(h, lookahead)
            y = ext.linear(h, x.cuda()).float().cpu().numpy()
            err = O.rel_rms(y, ref)
            assert err <= 1e-2, (m, k, tokens, lookahead, err)
        first = ext.linear(h, x.cuda())
        again = ext.linear(h, x.cuda())
        assert torch.equal(first, again)              # split-K reduction is deterministic
        ext.set_decode_path(h, 1)
        exact = ext.linear(h, x.cuda()).float().cpu().numpy()
        assert O.rel_rms(exact, ref) <= 4e-3
    finally:
        ext.free(h)


def test_sparse_matrix_takes_low_mode_path(ext, lut):
    blocks, scales, x = _random_case(5, 256, 1024, 3, lut, sparse=0.9)
    e0, e1, _ = O.unpack_blocks(blocks, 256)
    assert (e0 <= e1).mean() > 0.05
    h = _pack(ext, blocks, scales)
    try:
        y = ext.linear(h, x.cuda()).float().cpu().numpy()
        ref = O.linear_bf16(x.float().numpy(), blocks, scales, lut)
        assert O.rel_rms(y, ref) <= 1e-2
    finally:
        ext.free(h)


@pytest.mark.parametrize("tokens", [1, 3, 40])
def test_subnormal_numerators(ext, lut, tokens):
    """Blocks whose endpoints are tiny: the numerators 7*e0 + g*(e1-e0) the kernels hand to the tensor
    cores are then subnormal fp16 numbers (|n| < 4 after the 2^-16 scaling).  Flushing them would cost
    about a third of the signal; the result has to match the un-rounded linear as closely as usual."""
    rng = np.random.default_rng(404)
    m, k = 64, 512
    e0 = rng.integers(-1, 2, size=(m, k // 16))
    e1 = e0 - 1
    sel = rng.integers(0, 8, size=(m, k // 16, 16))
    blocks = O.pack_blocks(e0.reshape(-1), e1.reshape(-1), sel.reshape(-1, 16)).reshape(-1)
    scales = (rng.random(m).astype(np.float32) + 0.5)
    x = torch.from_numpy(rng.standard_normal((tokens, k)).astype(np.float32)).bfloat16()
    h = _pack(ext, blocks, scales)
    try:
        ext.set_prefill_backend(h, 5)
        y = ext.linear(h, x.cuda()).float().cpu().numpy()
        weights = O.dequant_weights(blocks, scales, lut, round_bf16=False).astype(np.float64)
        ref = x.float().numpy().astype(np.float64) @ weights.T
        assert O.rel_rms(y, ref) <= 4e-3, O.rel_rms(y, ref)
    finally:
        ext.free(h)


@pytest.mark.parametrize("magnitude", [1e-30, 1e-6, 1.0, 3e4, 1e30])
def test_activation_range(ext, lut, magnitude):
    """bf16 activations far outside the fp16 range go through the exact power-of-two rescale."""
    blocks, scales, x = _random_case(11, 128, 512, 2, lut)
    x = (x.float() * magnitude).bfloat16()
    h = _pack(ext, blocks, scales)
    try:
        y = ext.linear(h, x.cuda()).float().cpu().numpy()
        ref = O.linear_bf16(x.float().numpy(), blocks, scales, lut)
        assert np.isfinite(y).all()
        assert O.rel_rms(y, ref) <= 1e-2
    finally:
        ext.free(h)


def test_prefill_side_of_dispatcher(ext, lut):
    """tokens >= threshold: same numerics contract (texelator_cuda.cu:1341)."""
    blocks, scales, x = _random_case(21, 256, 512, 40, lut)
    h = _pack(ext, blocks, scales)
    try:
        ext.set_prefill(h, 16, 1024)
        y = ext.linear(h, x.cuda()).float().cpu().numpy()
        ref = O.linear_bf16(x.float().numpy(), blocks, scales, lut)
        assert O.rel_rms(y, ref) <= 1e-2
        assert ext.handle_info(h)[:5] == [256, 512, 16, 1024, 0]
    finally:
        ext.free(h)


def test_error_behaviour(ext, lut):
    blocks, scales, x = _random_case(3, 16, 64, 1, lut)
    with pytest.raises(RuntimeError, match="invalid encoded size"):
        ext.pack_encoded(torch.from_numpy(blocks[:-8].copy()), torch.from_numpy(scales))
    with pytest.raises(RuntimeError, match="contiguous CPU uint8"):
        ext.pack_encoded(torch.from_numpy(blocks).cuda(), torch.from_numpy(scales))
    h = _pack(ext, blocks, scales)
    try:
        with pytest.raises(RuntimeError, match="lookahead must be one of"):
            ext.set_lookahead(h, 5)
        with pytest.raises(RuntimeError, match="multiple of 16"):
            ext.set_prefill(h, 16, 24)
        with pytest.raises(RuntimeError, match="threshold must be positive"):
            ext.set_prefill(h, 0, 1024)
        with pytest.raises(RuntimeError, match="backend"):
            ext.set_prefill_backend(h, 10)
        with pytest.raises(RuntimeError, match="shape/device mismatch"):
            ext.linear(h, torch.zeros(1, 32, dtype=torch.bfloat16, device="cuda"))
        with pytest.raises(RuntimeError, match="contiguous CUDA"):
            ext.linear(h, torch.zeros(1, 64, dtype=torch.float32, device="cuda"))
        assert ext.linear(h, torch.zeros(1, 64, dtype=torch.float16, device="cuda")).dtype == torch.float16
    finally:
        ext.free(h)
    with pytest.raises(RuntimeError, match="null Texelator handle"):
        ext.linear(h, x.cuda())


def test_cfg1_full_size(ext, lut, golden_dir):
    """Configuration 1: 4096x4096 weight from the pinned seed, encoded by the restated
    encoder (hash-checked against the reference's blocks), x bf16 [1,4096]."""
    import hashlib
    manifest = json.loads((golden_dir / "manifest.json").read_text())["cases"]["cfg1_4096x4096"]
    g = torch.Generator().manual_seed(manifest["seed"])
    w = torch.randn(4096, 4096, generator=g) * 0.02
    xc = torch.randn(64, 4096, generator=g)
    x = torch.randn(1, 4096, generator=g).bfloat16()
    blocks, scales = O.encode_linear(w, (xc * xc).mean(0), lut)
    assert hashlib.sha256(blocks.tobytes()).hexdigest() == manifest["blocks_sha256"]
    h = _pack(ext, blocks, scales)
    try:
        from texelator_b200 import runtime as R
        wb = ext.dequant(h, R.DEQUANT_SCALED_BF16).float().cpu().numpy()
        assert np.array_equal(wb, O.dequant_weights(blocks, scales, lut))
        y = ext.linear(h, x.cuda()).float().cpu().numpy()
        ref = O.linear_bf16(x.float().numpy(), blocks, scales, lut)
        err = O.rel_rms(y, ref)
        cosine = float((y * ref).sum() / np.sqrt((y * y).sum() * (ref * ref).sum()))
        assert err <= 1e-2 and cosine >= 0.999, (err, cosine)
    finally:
        ext.free(h)
