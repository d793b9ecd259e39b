"""Parity at the benchmark's full matrix sizes (27B-class shapes), through checks whose cost does not grow
with the matrix: oracle on a sample of rows, two independent GPU decoders against each other, round trips
and sharding identities."""
import numpy as np
import pytest
import torch

from oracle import bc4_oracle as O

pytestmark = pytest.mark.gpu

SHAPES = [(34816, 5120), (5120, 17408), (7168, 5120)]      # gate+up, down, q+k+v of the 27B-class model


@pytest.fixture(scope="module")
def ext():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from texelator_b200 import runtime
    return runtime.extension()


def _encode(m, k, seed):
    """A full-size matrix through the reference's E3 encoder (the GPU implementation, byte-identical to the
    reference's recorded output in test_gpu_encode.py; 64 rows are re-checked here against the CPU restatement)."""
    from texelator_b200 import runtime
    from texelator_b200.modeling import software_palette_table
    gen = torch.Generator(device="cuda").manual_seed(seed)
    weight = torch.randn(m, k, device="cuda", generator=gen) * 0.02
    weight[torch.rand(m, k, device="cuda", generator=gen) < 0.002] = 0       # a few low-mode blocks now and then
    calibration = torch.randn(64, k, device="cuda", generator=gen)
    hdiag = (calibration * calibration).mean(0)
    table = software_palette_table("cuda")
    blocks, scales = runtime.extension().encode(weight, hdiag, table)
    rows = np.random.default_rng(seed).choice(m, 64, replace=False)
    want_blocks, want_scales = O.encode_linear(weight[rows].cpu(), hdiag.cpu(), table.cpu().numpy())
    assert np.array_equal(blocks.cpu().numpy().reshape(m, k // 2)[rows].reshape(-1), want_blocks)
    assert np.array_equal(scales.cpu().numpy()[rows], want_scales)
    x = torch.randn(1, k, device="cuda", generator=gen).bfloat16()
    return blocks, scales, x


@pytest.mark.parametrize("m,k", SHAPES)
def test_full_size_round_trip_sample_rows_and_decoder_agreement(ext, lut, m, k):
    blocks, scales, x = _encode(m, k, m + k)
    handle = ext.pack_encoded_device(blocks, scales)
    try:
        # 1. pack -> unpack returns the encoded bytes (an endpoint of -128 comes back as -127, the same value)
        original = blocks.cpu().numpy().reshape(-1, 8).copy()
        endpoints = original[:, :2].view(np.int8)
        endpoints[endpoints == -128] = -127
        assert np.array_equal(ext.unpack_blocks(handle).numpy().reshape(-1, 8), original)
        # 2. the tensor-core decoder against the CPU oracle on 96 sampled rows
        y = ext.linear(handle, x)
        rows = np.sort(np.random.default_rng(m).choice(m, 96, replace=False))
        per_row = k // 16
        sample_blocks = original.reshape(m, per_row * 8)[rows].reshape(-1)
        sample_scales = scales.cpu().numpy()[rows]
        ref = O.linear_bf16(x.float().cpu().numpy(), sample_blocks, sample_scales, lut)
        got = y.float().cpu().numpy()[:, rows]
        assert O.rel_rms(got, ref) <= 1e-2
        # 3. ... and against the GPU kernel that uses the reference's per-weight arithmetic, on every row
        ext.set_decode_path(handle, 1)
        exact = ext.linear(handle, x)
        ext.set_decode_path(handle, 0)
        assert O.rel_rms(exact.float().cpu().numpy()[:, rows], ref) <= 4e-3
        assert O.rel_rms(y.float().cpu().numpy(), exact.float().cpu().numpy()) <= 1e-2
        # 4. determinism and look-ahead independence (summation order is fixed by the tile walk)
        for lookahead in (1, 2, 8):
            ext.set_lookahead(handle, lookahead)
            assert torch.equal(ext.linear(handle, x), y), lookahead
    finally:
        ext.free(handle)


def test_full_size_prefill_tile_agrees_with_decode_kernel(ext):
    """512 tokens through the tcgen05 tile and the same tokens one by one through the decode GEMV: both multiply
    exact integer numerators by identically rescaled activations, so only the fp32 summation order differs."""
    m, k = 17408, 5120
    blocks, scales, _ = _encode(m, k, 77)
    handle = ext.pack_encoded_device(blocks, scales)
    try:
        gen = torch.Generator(device="cuda").manual_seed(78)
        x = torch.randn(512, k, device="cuda", generator=gen).bfloat16()
        ext.set_prefill(handle, 16, 32768)
        outputs = {}
        for backend in (5, 6, 7):
            ext.set_prefill_backend(handle, backend)
            outputs[backend] = ext.linear(handle, x)
        assert torch.equal(outputs[5], outputs[6]) and torch.equal(outputs[5], outputs[7])
        for token in (0, 255, 511):
            single = ext.linear(handle, x[token:token + 1].contiguous())
            a, b = outputs[5][token].float(), single[0].float()
            assert float((a - b).norm() / b.norm()) <= 2e-3, token
        assert ext.kernel_status() == 0
    finally:
        ext.free(handle)


def test_full_size_row_shards_reassemble_bit_exactly(ext):
    """Column-parallel sharding is byte slicing: the outputs of 8 row shards concatenate to the unsharded output."""
    m, k, world = 34816, 5120, 8
    blocks, scales, x = _encode(m, k, 91)
    handle = ext.pack_encoded_device(blocks, scales)
    shards = []
    try:
        full = ext.linear(handle, x)
        host_blocks, host_scales = blocks.cpu(), scales.cpu()
        per = m // world
        for rank in range(world):
            shards.append(ext.pack_encoded_shard(host_blocks, host_scales, m, k, (rank * per, (rank + 1) * per), (0, k // 16)))
        parts = [ext.linear(h, x) for h in shards]
        assert torch.equal(torch.cat(parts, 1), full)
    finally:
        for h in shards + [handle]:
            ext.free(h)


# BASELINE configuration 3: T in {32, 128, 512} x {5120->5120, 5120->17408, 17408->5120}
CFG3_SHAPES = [(5120, 5120), (17408, 5120), (5120, 17408)]          # (M, K)


@pytest.mark.parametrize("tokens", [32, 128, 512])
@pytest.mark.parametrize("m,k", CFG3_SHAPES)
def test_prefill_sweep_points_match_oracle(ext, lut, m, k, tokens):
    """Every point of the prefill sweep through the tile the autotuner would pick for it (all candidates are
    bitwise identical, checked here on the fly), against the dequantise-then-matmul oracle on 96 sampled
    output rows.  The whole matrix is encoded by the reference's activation-weighted endpoint search (GPU
    encoder); the first 512 rows are encoded a second time by the CPU restatement and must come out the same."""
    gen = torch.Generator(device="cuda").manual_seed(3 * m + k + tokens)
    weight = torch.randn(m, k, device="cuda", generator=gen) * 0.02
    calibration = torch.randn(64, k, generator=torch.Generator().manual_seed(k))
    hdiag = (calibration * calibration).mean(0)
    blocks, scales = ext.encode(weight, hdiag.cuda(), torch.from_numpy(lut).cuda())
    real_blocks, real_scales = O.encode_linear(weight[:512].cpu(), hdiag, lut)
    assert np.array_equal(blocks[:real_blocks.size].cpu().numpy(), real_blocks.reshape(-1))
    assert np.array_equal(scales[:512].cpu().numpy(), real_scales)
    x = torch.randn(tokens, k, device="cuda", generator=gen).bfloat16()
    handle = ext.pack_encoded_device(blocks, scales)
    try:
        ext.set_prefill(handle, 16, 32768)
        outputs = []
        for backend in (5, 6, 7, 8, 9):
            ext.set_prefill_backend(handle, backend)
            outputs.append(ext.linear(handle, x))
        torch.cuda.synchronize()
        assert ext.kernel_status() == 0
        for other in outputs[1:]:
            assert torch.equal(outputs[0], other)
        rows = np.sort(np.concatenate([np.random.default_rng(m + tokens).choice(512, 48, replace=False),
                                       512 + np.random.default_rng(k + tokens).choice(m - 512, 48, replace=False)]))
        host_blocks = blocks.cpu().numpy().reshape(m, k // 2)
        ref = O.linear_bf16(x.float().cpu().numpy(), host_blocks[rows].reshape(-1), scales.cpu().numpy()[rows], lut)
        got = outputs[0].float().cpu().numpy()[:, rows]
        err = O.rel_rms(got, ref)
        assert err <= 1e-2, (m, k, tokens, err)
        cosine = float((got * ref).sum() / np.sqrt((got * got).sum() * (ref * ref).sum()))
        assert cosine >= 0.9999
    finally:
        ext.free(handle)
