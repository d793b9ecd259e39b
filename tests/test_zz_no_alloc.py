"""The allocation-free entry point against the regular one (collected last on purpose: a failure
here cannot hide the result of any other test)."""
import numpy as np
import pytest
import torch

from oracle import bc4_oracle as O

pytestmark = pytest.mark.gpu


def test_static_scratch_linear_matches_regular_linear(lut):
    """Hosts that cannot call cudaMalloc when they need the linear (memory owned by their own pool,
    a thread that must not take the allocator lock) use ``tx_linear_static_scratch``; it must give what ``tx_linear`` gives.
    Two different calls in a row also show that nothing depends on what the shared array held."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from texelator_b200 import runtime
    ext = runtime.extension()
    rng = np.random.default_rng(17)
    m, k = 1000, 2048
    blocks, scales = O.encode_minmax((rng.standard_normal((m, k)) * 0.02).astype(np.float32), lut)
    bias = torch.from_numpy(rng.standard_normal(m).astype(np.float32)).bfloat16().cuda()
    handle = ext.pack_encoded(torch.from_numpy(blocks), torch.from_numpy(scales), bias)
    try:
        for tokens, scale in ((5, 1.0), (12, 300.0)):
            x = (torch.from_numpy(rng.standard_normal((tokens, k)).astype(np.float32)) * scale).bfloat16().cuda()
            expected = ext.linear(handle, x)
            got = ext.linear_static_scratch(handle, x)
            torch.cuda.synchronize()
            # same kernel and arithmetic; tx_linear may cut K into ranges per CTA where this entry point sums whole
            # rows, so single outputs can land on the neighbouring bf16 value (2^-8 relative)
            assert O.rel_rms(got.float().cpu().numpy(), expected.float().cpu().numpy()) <= 3e-3
            assert torch.equal(got, ext.linear_static_scratch(handle, x))          # and it repeats itself bit for bit
            ref = O.linear_bf16(x.float().cpu().numpy(), blocks, scales, lut, bias=bias.float().cpu().numpy())
            assert O.rel_rms(got.float().cpu().numpy(), ref) <= 1e-2
        with pytest.raises(RuntimeError, match="1..32 tokens"):
            ext.linear_static_scratch(handle, torch.zeros(40, k, dtype=torch.bfloat16, device="cuda"))
    finally:
        ext.free(handle)
    wide = O.encode_minmax((rng.standard_normal((16, 32768)) * 0.02).astype(np.float32), lut)
    huge = ext.pack_encoded(torch.from_numpy(wide[0]), torch.from_numpy(wide[1]))
    try:
        with pytest.raises(RuntimeError, match="exceeds the built-in activation scratch"):
            ext.linear_static_scratch(huge, torch.zeros(9, 32768, dtype=torch.bfloat16, device="cuda"))
    finally:
        ext.free(huge)
