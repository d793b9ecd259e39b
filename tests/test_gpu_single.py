"""Single-token decode path on the GPU: the kernel without per-weight arithmetic, K-split partial
outputs and staged activations from the norm kernel (run with ``-m gpu``)."""
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


def _case(ext, lut, m, k, seed, bias=False):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    blocks, scales = O.encode_minmax(w, lut)
    b = torch.from_numpy(rng.standard_normal(m).astype(np.float32) * 0.05).bfloat16().cuda() if bias else None
    handle = ext.pack_encoded(torch.from_numpy(blocks), torch.from_numpy(scales), b)
    x = torch.from_numpy(rng.standard_normal((1, k)).astype(np.float32)).bfloat16().cuda()
    return handle, blocks, scales, x, b


@pytest.mark.parametrize("m,k,bias", [(48, 256, False), (5120, 5120, True), (640, 17408, False), (1000, 1040, True), (16, 128, False)])
def test_single_token_kernel_matches_oracle_and_dispatcher(ext, lut, m, k, bias):
    handle, blocks, scales, x, b = _case(ext, lut, m, k, m + k, bias)
    try:
        eligible, splits, staged_bytes = ext.linear_single_info(handle)
        assert eligible and splits >= 1 and staged_bytes == 16 + ((k + 127) // 128) * 288
        y = torch.empty(1, m, device="cuda", dtype=torch.bfloat16)
        ext.linear_single(handle, x, y)
        ref = O.linear_bf16(x.float().cpu().numpy(), blocks, scales, lut, bias=None if b is None else b.float().cpu().numpy())
        assert O.rel_rms(y.float().cpu().numpy(), ref) <= 1e-2
        general = ext.linear(handle, x).float()                 # the general decode kernel: same products, other order
        assert float((general - y.float()).abs().max()) <= float(general.abs().max()) * 2 ** -7
        for lookahead in (1, 3, 8):                              # look-ahead never changes the arithmetic
            ext.set_lookahead(handle, lookahead)
            again = torch.empty_like(y)
            ext.linear_single(handle, x, again)
            assert torch.equal(again, y)
    finally:
        ext.free(handle)


@pytest.mark.parametrize("m,k,splits", [(5120, 5120, 2), (5120, 5120, 8), (320, 17408, 4), (100, 1024, 8), (64, 640, 5)])
def test_k_split_partials_add_up(ext, lut, m, k, splits):
    handle, blocks, scales, x, b = _case(ext, lut, m, k, 7 * m + k, bias=True)
    try:
        y = torch.empty(1, m, device="cuda", dtype=torch.bfloat16)
        ext.linear_single(handle, x, y)
        stride = (m + 31) // 32 * 32
        partials = torch.full((splits, stride), float("nan"), device="cuda", dtype=torch.float32)
        ext.linear_single(handle, x, None, partials=partials)
        total = partials[:, :m].sum(0)
        assert torch.isfinite(total).all()
        # same products, another summation order: the sum rounds to the same bf16 or its neighbour
        diff = (total.bfloat16().float() - y.float()[0]).abs()
        assert float(diff.max()) <= float(y.float().abs().max()) * 2 ** -7
        assert O.rel_rms(total.cpu().numpy()[None], y.float().cpu().numpy()) <= 3e-3
        with pytest.raises(RuntimeError, match="splits must divide"):
            ext.linear_single(handle, x, None, partials=torch.zeros(((k + 127) // 128) + 1, stride, device="cuda"))
    finally:
        ext.free(handle)


@pytest.mark.parametrize("hidden,m", [(5120, 7168), (2048, 512), (1000 * 8, 64)])
def test_staged_activations_from_the_norm_kernel(ext, lut, hidden, m):
    handle, blocks, scales, _, _ = _case(ext, lut, m, hidden, hidden + 3)
    try:
        gen = torch.Generator(device="cuda").manual_seed(hidden)
        h0 = torch.randn(1, hidden, device="cuda", generator=gen).bfloat16()
        delta = (torch.randn(1, hidden, device="cuda", generator=gen) * 0.3).bfloat16()
        gamma = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=gen)).bfloat16()
        # reference: the plain norm kernel, then the single-token kernel staging the bf16 row itself
        h_ref, normed = h0.clone(), torch.empty_like(h0)
        ext.add_rmsnorm(h_ref, delta, gamma, normed, 1e-6)
        want = torch.empty(1, m, device="cuda", dtype=torch.bfloat16)
        ext.linear_single(handle, normed, want)
        # delta as two fp32 partial vectors that add up to it exactly
        stride = hidden + 64
        partials = torch.zeros(2, stride, device="cuda", dtype=torch.float32)
        partials[0, :hidden] = delta.float()[0] * 0.5
        partials[1, :hidden] = delta.float()[0] * 0.5
        staged = torch.empty(ext.linear_single_info(handle)[2], dtype=torch.uint8, device="cuda")
        for kwargs in (dict(delta=delta), dict(partials=partials)):
            h, y = h0.clone(), torch.empty_like(h0)
            staged.fill_(0xAB)
            ext.add_rmsnorm_single(h, gamma, 1e-6, y=y, staged=staged, **kwargs)
            assert torch.equal(h, h_ref) and torch.equal(y, normed)
            got = torch.empty_like(want)
            ext.linear_single(handle, None, got, staged=staged)
            torch.cuda.synchronize()
            assert torch.equal(got, want)                       # staged by the producer == staged by the linear
        h = h0.clone()
        ext.add_rmsnorm_single(h, gamma, 1e-6, delta=delta, staged=staged)       # no bf16 copy requested
        got = torch.empty_like(want)
        ext.linear_single(handle, None, got, staged=staged)
        assert torch.equal(got, want)
    finally:
        ext.free(handle)


def test_single_token_path_refuses_other_payloads(ext, lut):
    from texelator_b200 import runtime as R
    handle, blocks, scales, x, _ = _case(ext, lut, 64, 256, 5)
    try:
        ext.set_palette(handle, R.PALETTE_HARDWARE)
        assert not ext.linear_single_info(handle)[0]
        with pytest.raises(RuntimeError, match="single-token kernel needs"):
            ext.linear_single(handle, x, torch.empty(1, 64, device="cuda", dtype=torch.bfloat16))
        ext.set_palette(handle, R.PALETTE_SOFTWARE)
        y = torch.empty(1, 64, device="cuda", dtype=torch.bfloat16)
        with pytest.raises(RuntimeError, match="either as bf16 or in staged form"):
            ext.linear_single(handle, None, y)
        with pytest.raises(RuntimeError, match="either a bf16 output or a partial-sum output"):
            ext.linear_single(handle, x, None)
    finally:
        ext.free(handle)
