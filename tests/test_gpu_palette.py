"""Hardware (texture-unit) palette mode: exact tables, the palette gate, and all decode paths on a
payload encoded against the palette the reference publishes (run with ``-m gpu``)."""
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


@pytest.fixture(scope="module")
def hw_lut():
    return O.hardware_palette()


def test_hardware_palette_table_is_bit_exact(ext, hw_lut):
    table = ext.hardware_palette().numpy().reshape(255, 255, 8)
    assert np.array_equal(table.view(np.uint32), hw_lut.view(np.uint32))
    assert O.palette_sha256(table) == O.REFERENCE_TEXTURE_PALETTE_SHA256


def test_texture_unit_matches_the_published_palette(ext, hw_lut):
    if not ext.texture_supported():
        pytest.skip("device has no signed-BC4 texture views")
    measured = ext.palette_probe().numpy().reshape(255, 255, 8)
    assert O.palette_sha256(measured) == O.REFERENCE_TEXTURE_PALETTE_SHA256
    assert np.array_equal(measured.view(np.uint32), hw_lut.view(np.uint32))


def _encode(hw_lut, m, k, seed, sparse=0.0):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    if sparse:
        w[rng.random((m, k)) < sparse] = 0
    h = (rng.random(k) + 0.1).astype(np.float32)
    return O.encode_linear(torch.from_numpy(w), torch.from_numpy(h), hw_lut)     # the reference's E3 search


@pytest.mark.parametrize("m,k,sparse", [(64, 256, 0.0), (200, 1024, 0.0), (96, 512, 0.9)])
def test_hardware_mode_decode_paths(ext, hw_lut, m, k, sparse):
    from texelator_b200 import runtime as R
    blocks, scales = _encode(hw_lut, m, k, m + k, sparse)
    x = torch.from_numpy(np.random.default_rng(1).standard_normal((3, k)).astype(np.float32)).bfloat16()
    h = ext.pack_encoded(torch.from_numpy(blocks), torch.from_numpy(scales))
    try:
        ext.set_palette(h, R.PALETTE_HARDWARE)
        pal = ext.dequant(h, R.DEQUANT_PALETTE_F32).cpu().numpy()
        assert np.array_equal(pal.view(np.uint32), O.dequant_palette(blocks, m, hw_lut).view(np.uint32))
        wb = ext.dequant(h, R.DEQUANT_SCALED_BF16).float().cpu().numpy()
        assert np.array_equal(wb, O.dequant_weights(blocks, scales, hw_lut))
        ref = O.linear_bf16(x.float().numpy(), blocks, scales, hw_lut)
        paths = [0, 1] + ([2] if ext.texture_supported() else [])
        for path in paths:
            ext.set_decode_path(h, path)          # path 2 passes the gate: texture unit == this palette
            y = ext.linear(h, x.cuda()).float().cpu().numpy()
            assert O.rel_rms(y, ref) <= 1e-2, (path, O.rel_rms(y, ref))
        ext.set_decode_path(h, 0)
        ext.set_prefill(h, 1, 1024)
        ext.set_prefill_backend(h, 6)
        xp = torch.from_numpy(np.random.default_rng(2).standard_normal((48, k)).astype(np.float32)).bfloat16()
        yp = ext.linear(h, xp.cuda()).float().cpu().numpy()
        assert O.rel_rms(yp, O.linear_bf16(xp.float().numpy(), blocks, scales, hw_lut)) <= 1e-2
        # the same bytes read against the other palette are a different matrix: the modes are not interchangeable
        ext.set_palette(h, R.PALETTE_SOFTWARE)
        other = ext.dequant(h, R.DEQUANT_PALETTE_F32).cpu().numpy()
        assert not np.array_equal(other, pal)
    finally:
        ext.free(h)


def test_texture_gemv_equals_reference_arithmetic(ext, hw_lut):
    """Texture path and the exact ALU path compute the same bf16(pal*scale) weights."""
    if not ext.texture_supported():
        pytest.skip("device has no signed-BC4 texture views")
    from texelator_b200 import runtime as R
    blocks, scales = _encode(hw_lut, 128, 512, 5)
    x = torch.from_numpy(np.random.default_rng(3).standard_normal((2, 512)).astype(np.float32)).bfloat16().cuda()
    h = ext.pack_encoded(torch.from_numpy(blocks), torch.from_numpy(scales))
    try:
        ext.set_palette(h, R.PALETTE_HARDWARE)
        ext.set_decode_path(h, 1)
        exact = ext.linear(h, x).float()
        ext.set_decode_path(h, 2)
        texture = ext.linear(h, x).float()
        assert float((exact - texture).abs().max()) <= 2e-2 * float(exact.abs().max())
        with pytest.raises(RuntimeError, match="leave the texture decode path"):
            ext.set_palette(h, R.PALETTE_SOFTWARE)
    finally:
        ext.free(h)
