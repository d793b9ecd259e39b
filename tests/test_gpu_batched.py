"""Batched decode: the multi-token decode kernel with K ranges, the batched glue kernels and the batched model
(run with ``-m gpu``)."""
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


def _cosine(a, b):
    return float(torch.nn.functional.cosine_similarity(a.float().reshape(1, -1), b.float().reshape(1, -1)))


@pytest.mark.parametrize("m,k,tokens,bias", [
    (5120, 17408, 8, False),      # 8 rows of K = 17408 do not fit one CTA's shared memory: K ranges
    (1280, 8192, 32, True),       # few row tiles: ranges also spread the work over the SMs
    (8192, 1024, 32, False),      # short K: one range
    (272, 3584, 24, True),        # ragged rows (M % 16 != 0), three token tiles
    (512, 4112, 17, False),       # K not a multiple of 128, odd token count
    (64, 28672, 32, False),       # the longest rows of the 70B-class shapes
])
def test_multi_token_decode_matches_oracle(ext, lut, m, k, tokens, bias):
    """Reference semantics: every token count below the threshold is the decode operator, one row of x at a time
    (texelator_cuda.cu:1438-1468)."""
    rng = np.random.default_rng(m + k + tokens)
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    blocks, scales = O.encode_minmax(w, lut)
    x = torch.from_numpy(rng.standard_normal((tokens, k)).astype(np.float32)).bfloat16()
    b = torch.from_numpy((rng.standard_normal(m) * 0.3).astype(np.float32)).bfloat16() if bias else None
    h = ext.pack_encoded(torch.from_numpy(blocks), torch.from_numpy(scales), None if b is None else b.cuda())
    try:
        ext.set_prefill(h, 64, 1024)
        y = ext.linear(h, x.cuda())
        ref = O.linear_bf16(x.float().numpy(), blocks, scales, lut, None if b is None else b.float().numpy())
        assert O.rel_rms(y.float().cpu().numpy(), ref) <= 1e-2
        # the same rows one at a time: the K ranges change the order of the fp32 sums, nothing else
        single = torch.cat([ext.linear(h, x[i:i + 1].cuda()) for i in range(tokens)])
        assert O.rel_rms(y.float().cpu().numpy(), single.float().cpu().numpy()) <= 4e-3
        again = ext.linear(h, x.cuda())
        assert torch.equal(y, again)                       # deterministic: fixed ranges, fixed order
    finally:
        ext.free(h)


def test_silu_mul_pairs(ext):
    from texelator_b200.modeling import interleave_gate_up
    gen = torch.Generator(device="cuda").manual_seed(1)
    tokens, inter = 5, 264
    gate = torch.randn(tokens, inter, device="cuda", generator=gen).bfloat16()
    up = torch.randn(tokens, inter, device="cuda", generator=gen).bfloat16()
    paired = interleave_gate_up(gate.T.contiguous(), up.T.contiguous()).T.contiguous()       # [tokens, 2 * inter]
    out = torch.empty(tokens, inter, device="cuda", dtype=torch.bfloat16)
    ext.silu_mul_pairs(paired, out)
    want = torch.empty_like(out)
    ext.silu_mul(torch.cat([gate, up], 1).contiguous(), want)
    assert torch.equal(out, want)


def test_attention_step_batch_equals_per_sequence_steps(ext):
    """Sequences at different positions (one of them past the single-chunk length) in one launch."""
    from texelator_b200.modeling import CONFIGS, _rope_tables
    c = CONFIGS["toy128"]
    gen = torch.Generator(device="cuda").manual_seed(2)
    batch, q_heads, kv_heads, max_len = 5, c.q_heads, c.kv_heads, 320
    cos, sin = _rope_tables(c, max_len, torch.device("cuda"))
    k_cache = torch.randn(batch, kv_heads, max_len, 128, device="cuda", generator=gen).bfloat16()
    v_cache = torch.randn(batch, kv_heads, max_len, 128, device="cuda", generator=gen).bfloat16()
    qkv = torch.randn(batch, (q_heads + 2 * kv_heads) * 128, device="cuda", generator=gen).bfloat16()
    positions = torch.tensor([0, 7, 63, 64, 300], device="cuda", dtype=torch.int64)
    want = torch.empty(batch, q_heads * 128, device="cuda", dtype=torch.bfloat16)
    k_ref, v_ref = k_cache.clone(), v_cache.clone()
    scratch = torch.zeros(batch * ext.attention_step_scratch_floats(q_heads, max_len), dtype=torch.float32, device="cuda")
    for b in range(batch):
        ext.attention_step(qkv[b:b + 1], cos, sin, positions[b:b + 1], k_ref[b], v_ref[b], scratch, want[b:b + 1], q_heads, kv_heads, 128)
    got = torch.empty_like(want)
    ext.attention_step_batch(qkv, cos, sin, positions, k_cache, v_cache, scratch, got, q_heads, kv_heads, 128)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert torch.equal(k_cache, k_ref) and torch.equal(v_cache, v_ref)
    for _ in range(3):                                   # the arrival counters were left at zero: launch again
        ext.attention_step_batch(qkv, cos, sin, positions, k_cache, v_cache, scratch, got, q_heads, kv_heads, 128)
    assert torch.equal(got, want)


@pytest.mark.parametrize("batch", [8, 3])
def test_batch_of_sequences_equals_the_sequences_one_by_one(batch):
    """toy128: B sequences with different prompts decode together (library kernels, eagerly and from a CUDA graph)
    and one by one through PyTorch glue with the same handles; the hidden states agree at every step (the one-by-one
    run's tokens are fed to both, so a near-tie in one argmax cannot send the two runs down different sequences)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from texelator_b200.batched import BatchedBC4Decoder
    from texelator_b200.modeling import CONFIGS
    config = CONFIGS["toy128"]
    model = BatchedBC4Decoder(config, "cuda:0", max_len=160, batch=batch, seed=5)
    try:
        for sequence in range(batch):
            ids = torch.randint(0, config.vocab, (20 + 9 * sequence,), generator=torch.Generator().manual_seed(sequence))
            model.prefill_sequence(sequence, ids)
            model.tok[sequence] = int(ids[-1])
        state = (model.tok.clone(), model.pos.clone(), model.k_cache.clone(), model.v_cache.clone())

        def rewind():
            model.tok.copy_(state[0]); model.pos.copy_(state[1]); model.k_cache.copy_(state[2]); model.v_cache.copy_(state[3])

        want_hidden, want_tokens = [], []
        for _ in range(6):
            model.decode_step_reference()
            want_hidden.append(model.last_hidden.clone()); want_tokens.append(model.next_tok.clone())
        rewind()
        for step in range(6):
            model.tok.copy_(state[0] if step == 0 else want_tokens[step - 1])
            model.decode_step()
            assert _cosine(model.last_hidden, want_hidden[step]) >= 0.9995, step
        rewind()
        model.capture()
        assert model.launches_per_step > 0
        for step in range(6):
            model.tok.copy_(state[0] if step == 0 else want_tokens[step - 1])
            torch.cuda.synchronize()
            model.decode_graph()
            model.stream.synchronize()
            assert _cosine(model.last_hidden, want_hidden[step]) >= 0.9995, ("graph", step)
        assert torch.equal(model.pos, state[1] + 6)
        model.check_status()
    finally:
        model.free()
