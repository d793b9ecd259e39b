"""The fp16 activation type of the operator (the reference's texelator_bc4_kernel and fp16 prefill) against the
CPU oracle (run with ``-m gpu``)."""
import numpy as np
import pytest
import torch

from oracle import bc4_oracle as O

pytestmark = pytest.mark.gpu

TOLERANCE = 2e-3          # rel-RMS against the fp64-accumulated oracle; one fp16 rounding is 2^-11 = 4.9e-4


@pytest.fixture(scope="module")
def ext():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from texelator_b200 import runtime
    return runtime.extension()


def _case(seed, m, k, tokens, lut, sparse=0.0, bias=False):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    if sparse:
        w[rng.random((m, k)) < sparse] = 0
    blocks, scales = O.encode_minmax(w, lut)
    x = torch.from_numpy(rng.standard_normal((tokens, k)).astype(np.float32)).half()
    b = torch.from_numpy((rng.standard_normal(m) * 0.5).astype(np.float32)).half() if bias else None
    return blocks, scales, x, b


@pytest.mark.parametrize("m,k,tokens,sparse,bias", [
    (256, 1024, 1, 0.0, False), (256, 1024, 1, 0.0, True), (130, 208, 3, 0.0, True), (512, 4096, 15, 0.0, False),
    (96, 512, 2, 0.7, True), (1024, 5120, 9, 0.0, True), (64, 17408, 1, 0.0, False),
])
def test_half_decode_matches_oracle(ext, lut, m, k, tokens, sparse, bias):
    blocks, scales, x, b = _case(m + k + tokens, m, k, tokens, lut, sparse, bias)
    h = ext.pack_encoded(torch.from_numpy(blocks), torch.from_numpy(scales), None if b is None else b.cuda())
    try:
        y = ext.linear(h, x.cuda())
        assert y.dtype == torch.float16 and tuple(y.shape) == (tokens, m)
        ref = O.linear_f16(x.float().numpy(), blocks, scales, lut, None if b is None else b.float().numpy())
        assert O.rel_rms(y.float().cpu().numpy(), ref) <= TOLERANCE
        # same handle, same numbers as bf16 activations when the values are representable in both types
        if b is None:
            coarse = x.bfloat16()
            yb = ext.linear(h, coarse.cuda()).float().cpu().numpy()
            yh = ext.linear(h, coarse.half().cuda()).float().cpu().numpy()
            assert O.rel_rms(yh, yb) <= 5e-3
    finally:
        ext.free(h)


@pytest.mark.parametrize("backend", [5, 6, 7, 8, 9])
@pytest.mark.parametrize("m,k,tokens,bias", [(512, 1024, 64, True), (272, 2064, 33, False), (1024, 5120, 512, True)])
def test_half_prefill_matches_oracle(ext, lut, backend, m, k, tokens, bias):
    blocks, scales, x, b = _case(backend + m + tokens, m, k, tokens, lut, 0.0, bias)
    h = ext.pack_encoded(torch.from_numpy(blocks), torch.from_numpy(scales), None if b is None else b.cuda())
    try:
        ext.set_prefill_backend(h, backend)
        y = ext.linear(h, x.cuda())
        assert y.dtype == torch.float16
        ref = O.linear_f16(x.float().numpy(), blocks, scales, lut, None if b is None else b.float().numpy(), prefill=True)
        assert O.rel_rms(y.float().cpu().numpy(), ref) <= TOLERANCE
        ext.set_prefill(h, 1 << 30, 1024)                       # the same prompt through the decode kernel
        streamed = ext.linear(h, x[:16].cuda())
        assert O.rel_rms(streamed.float().cpu().numpy(), y[:16].float().cpu().numpy()) <= TOLERANCE
    finally:
        ext.free(h)


def test_half_values_at_the_ends_of_the_range(ext, lut):
    """fp16 activations need no rescaling: subnormal inputs and inputs near 65504 go to the tensor core as they are."""
    rng = np.random.default_rng(3)
    m, k = 128, 512
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    blocks, scales = O.encode_minmax(w, lut)
    h = ext.pack_encoded(torch.from_numpy(blocks), torch.from_numpy(scales))
    try:
        for magnitude in (3e-6, 3e4):
            x = torch.from_numpy((rng.standard_normal((2, k)) * magnitude).astype(np.float32)).clamp(-65000, 65000).half()
            ref = O.linear_f16(x.float().numpy(), blocks, scales, lut)
            got = ext.linear(h, x.cuda()).float().cpu().numpy()
            assert np.isfinite(got).all()
            assert O.rel_rms(got, ref) <= (TOLERANCE if magnitude > 1 else 2e-2)   # tiny outputs are fp16 subnormals themselves
    finally:
        ext.free(h)


def test_bias_and_activation_types_must_match(ext, lut):
    rng = np.random.default_rng(4)
    blocks, scales = O.encode_minmax((rng.standard_normal((32, 64)) * 0.02).astype(np.float32), lut)
    half_bias = torch.zeros(32, dtype=torch.float16, device="cuda")
    h = ext.pack_encoded(torch.from_numpy(blocks), torch.from_numpy(scales), half_bias)
    try:
        ext.linear(h, torch.zeros(1, 64, dtype=torch.float16, device="cuda"))
        with pytest.raises(RuntimeError, match="input and bias dtypes must match"):
            ext.linear(h, torch.zeros(1, 64, dtype=torch.bfloat16, device="cuda"))
        with pytest.raises(RuntimeError, match="input and bias dtypes must match"):
            ext.linear_static_scratch(h, torch.zeros(1, 64, dtype=torch.bfloat16, device="cuda"))
    finally:
        ext.free(h)
