"""Decode-loop glue kernels against PyTorch formulations (GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from texelator_b200 import runtime
    return runtime.extension()


def _reference_step(qkv, cos, sin, pos, k_cache, v_cache, q_heads, kv_heads, head_dim):
    """rotate-half RoPE of q and k, append, then softmax(q k^T / sqrt(d)) v over positions 0..pos (fp32)."""
    half = head_dim // 2
    c, s = cos[pos], sin[pos]

    def rope(x):
        x1, x2 = x[..., :half].float(), x[..., half:].float()
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(torch.bfloat16)

    q = rope(qkv[0, :q_heads * head_dim].view(q_heads, head_dim))
    k = rope(qkv[0, q_heads * head_dim:(q_heads + kv_heads) * head_dim].view(kv_heads, head_dim))
    v = qkv[0, (q_heads + kv_heads) * head_dim:].view(kv_heads, head_dim)
    k_cache[:, pos] = k
    v_cache[:, pos] = v
    group = q_heads // kv_heads
    keys = k_cache[:, :pos + 1].float().repeat_interleave(group, 0)
    values = v_cache[:, :pos + 1].float().repeat_interleave(group, 0)
    scores = torch.einsum("hd,hkd->hk", q.float(), keys) * head_dim ** -0.5
    return torch.einsum("hk,hkd->hd", torch.softmax(scores, -1), values)


@pytest.mark.parametrize("q_heads,kv_heads,max_len,positions", [
    (40, 8, 2200, [0, 1, 63, 64, 65, 1000, 2111, 2199]),     # 27B-class grouping (5 query heads per kv head)
    (8, 8, 130, [0, 64, 129]),
    (16, 2, 320, [5, 127, 128, 319]),
    (5, 1, 700, [640]),                                      # one rank of an 8-way tensor-parallel split
    (40, 8, 9000, [2367, 2368, 4500, 8999]),                 # more chunks than resident CTAs: several chunks per CTA
    (5, 1, 20000, [16383, 19999]),                           # 313 chunks on 256 CTAs
])
def test_attention_step_matches_pytorch(ext, q_heads, kv_heads, max_len, positions):
    head_dim = 128
    gen = torch.Generator(device="cuda").manual_seed(q_heads * 1000 + max_len)
    bf = dict(device="cuda", dtype=torch.bfloat16)
    k_cache = torch.randn(kv_heads, max_len, head_dim, generator=gen, **bf)
    v_cache = torch.randn(kv_heads, max_len, head_dim, generator=gen, **bf)
    angles = torch.rand(max_len, head_dim // 2, device="cuda", generator=gen) * 6.28
    cos, sin = angles.cos().contiguous(), angles.sin().contiguous()
    scratch = torch.zeros(ext.attention_step_scratch_floats(q_heads, max_len), dtype=torch.float32, device="cuda")
    out = torch.zeros(1, q_heads * head_dim, **bf)
    for pos in positions:
        qkv = torch.randn(1, (q_heads + 2 * kv_heads) * head_dim, generator=gen, **bf)
        position = torch.full((1,), pos, dtype=torch.int64, device="cuda")
        k_ref, v_ref = k_cache.clone(), v_cache.clone()
        want = _reference_step(qkv, cos, sin, pos, k_ref, v_ref, q_heads, kv_heads, head_dim)
        before = qkv.clone()
        ext.attention_step(qkv, cos, sin, position, k_cache, v_cache, scratch, out, q_heads, kv_heads, head_dim)
        torch.cuda.synchronize()
        assert torch.equal(qkv, before)                                   # q is rotated on the fly
        assert torch.equal(v_cache, v_ref), pos                           # value rows are copies
        # key rows: only row `pos` changes; fp32 contraction may move its bf16 rounding by one step
        untouched = torch.ones(max_len, dtype=torch.bool, device="cuda")
        untouched[pos] = False
        assert torch.equal(k_cache[:, untouched], k_ref[:, untouched]), pos
        assert torch.allclose(k_cache[:, pos].float(), k_ref[:, pos].float(), atol=0.04, rtol=0), pos
        k_cache[:, pos] = k_ref[:, pos]
        got = out.view(q_heads, head_dim).float()
        assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), (pos, float((got - want).abs().max()))
        cosine = torch.nn.functional.cosine_similarity(got.reshape(1, -1), want.reshape(1, -1)).item()
        assert cosine > 0.9999, (pos, cosine)


def test_attention_step_equals_two_kernel_path(ext):
    """Same inputs through rope_append + attention_decode (two sequence-split sizes, one merge order
    each): outputs agree to bf16 rounding and the caches are identical."""
    q_heads, kv_heads, head_dim, max_len, pos = 40, 8, 128, 1500, 1234
    gen = torch.Generator(device="cuda").manual_seed(7)
    bf = dict(device="cuda", dtype=torch.bfloat16)
    k1 = torch.randn(kv_heads, max_len, head_dim, generator=gen, **bf)
    v1 = torch.randn(kv_heads, max_len, head_dim, generator=gen, **bf)
    k2, v2 = k1.clone(), v1.clone()
    angles = torch.rand(max_len, head_dim // 2, device="cuda", generator=gen) * 6.28
    cos, sin = angles.cos().contiguous(), angles.sin().contiguous()
    qkv = torch.randn(1, (q_heads + 2 * kv_heads) * head_dim, generator=gen, **bf)
    position = torch.full((1,), pos, dtype=torch.int64, device="cuda")
    scratch = torch.zeros(ext.attention_step_scratch_floats(q_heads, max_len), dtype=torch.float32, device="cuda")
    a, b = torch.zeros(1, q_heads * head_dim, **bf), torch.zeros(1, q_heads * head_dim, **bf)
    ext.attention_step(qkv, cos, sin, position, k1, v1, scratch, a, q_heads, kv_heads, head_dim)
    rotated = qkv.clone()
    ext.rope_append(rotated, cos, sin, position, k2, v2, q_heads, kv_heads, head_dim)
    ext.attention_decode(rotated, k2, v2, position, scratch, b, q_heads, kv_heads, head_dim)
    torch.cuda.synchronize()
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert torch.allclose(a.float(), b.float(), atol=1e-2, rtol=1e-2)


def test_attention_step_rejects_unsupported_shapes(ext):
    bf = dict(device="cuda", dtype=torch.bfloat16)
    cache = torch.zeros(1, 64, 64, **bf)
    table = torch.zeros(64, 32, device="cuda")
    position = torch.zeros(1, dtype=torch.int64, device="cuda")
    scratch = torch.zeros(4096, dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError, match="head_dim 128"):
        ext.attention_step(torch.zeros(1, 3 * 64, **bf), table, table, position, cache, cache, scratch, torch.zeros(1, 64, **bf), 1, 1, 64)
    with pytest.raises(ValueError, match="scratch"):
        big = torch.zeros(1, 4096, 128, **bf)
        ext.attention_step(torch.zeros(1, 3 * 128, **bf), table, table, position, big, big, scratch, torch.zeros(1, 128, **bf), 1, 1, 128)


def _packed_linear(ext, m, k, seed, bias=False):
    from texelator_b200.modeling import encode_minmax_cuda, software_palette_table
    gen = torch.Generator(device="cuda").manual_seed(seed)
    weight = torch.randn(m, k, device="cuda", generator=gen) * 0.02
    blocks, scales = encode_minmax_cuda(weight, software_palette_table("cuda"))
    b = (torch.randn(m, device="cuda", generator=gen) * 0.05).bfloat16() if bias else None
    return ext.pack_encoded_device(blocks, scales, b), gen


@pytest.mark.parametrize("m,k,tokens,bias", [(512, 1024, 1, False), (17408 * 2 // 8, 5120, 1, False), (96, 272, 2, True)])
def test_fused_swiglu_epilogue_is_bit_identical_to_separate_kernels(ext, m, k, tokens, bias):
    handle, gen = _packed_linear(ext, m, k, 11, bias)
    try:
        x = torch.randn(tokens, k, device="cuda", generator=gen).bfloat16()
        full = ext.linear(handle, x).view(tokens, m // 16, 2, 8)              # (gate, up) row pairs
        gate_up = torch.cat([full[:, :, 0].reshape(tokens, -1), full[:, :, 1].reshape(tokens, -1)], 1).contiguous()
        want = torch.empty(tokens, m // 2, device="cuda", dtype=torch.bfloat16)
        ext.silu_mul(gate_up, want)
        got = torch.empty_like(want)
        ext.linear_fused_out(handle, x, got, swiglu=True)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    finally:
        ext.free(handle)


@pytest.mark.parametrize("m,k,tokens,swiglu", [(640, 5120, 1, False), (1024, 8192, 1, True), (256, 1008, 2, False)])
def test_fused_norm_prologue_matches_separate_kernels(ext, m, k, tokens, swiglu):
    handle, gen = _packed_linear(ext, m, k, 13)
    try:
        h = torch.randn(tokens, k, device="cuda", generator=gen).bfloat16()
        delta = (torch.randn(tokens, k, device="cuda", generator=gen) * 0.3).bfloat16()
        gamma = (1 + 0.1 * torch.randn(k, device="cuda", generator=gen)).bfloat16()
        for use_delta in (True, False):
            h_ref, normed = h.clone(), torch.empty_like(h)
            ext.add_rmsnorm(h_ref, delta if use_delta else None, gamma, normed, 1e-6)
            lin = ext.linear(handle, normed)
            if swiglu:
                pairs = lin.view(tokens, m // 16, 2, 8)
                want = (torch.nn.functional.silu(pairs[:, :, 0].float()) * pairs[:, :, 1].float()).bfloat16().reshape(tokens, -1)
            else:
                want = lin
            got = torch.empty_like(want)
            residual = torch.full_like(h, float("nan"))
            before = h.clone()
            ext.linear_fused_out(handle, h, got, norm_weight=gamma, delta=delta if use_delta else None, eps=1e-6,
                                 residual_out=residual, swiglu=swiglu)
            torch.cuda.synchronize()
            assert torch.equal(h, before)                       # the input stream is read-only
            assert torch.equal(residual, h_ref)                 # bf16(x + delta), element-wise exact
            # the sum of squares is reduced in a different order than add_rmsnorm's: one bf16 step at most
            # on a few normalised activations
            scale = float(want.float().abs().max())
            assert float((got.float() - want.float()).abs().max()) <= 0.02 * scale + 1e-3
            cosine = torch.nn.functional.cosine_similarity(got.float().reshape(1, -1), want.float().reshape(1, -1)).item()
            assert cosine > 0.99999
    finally:
        ext.free(handle)


def test_fused_linear_argument_checks(ext):
    handle, gen = _packed_linear(ext, 64, 256, 17)
    try:
        bf = dict(device="cuda", dtype=torch.bfloat16)
        x, y, gamma = torch.zeros(1, 256, **bf), torch.zeros(1, 64, **bf), torch.ones(256, **bf)
        with pytest.raises(RuntimeError, match="alias"):
            ext.linear_fused_out(handle, x, y, norm_weight=gamma, residual_out=x)
        delta = torch.zeros(1, 256, **bf)
        with pytest.raises(RuntimeError, match="overlap delta or y"):
            ext.linear_fused_out(handle, x, y, norm_weight=gamma, delta=delta, residual_out=delta)
        with pytest.raises(RuntimeError, match="norm weight"):
            ext.linear_fused_out(handle, x, y, delta=x)
        with pytest.raises(RuntimeError, match="at most 2 tokens"):
            ext.linear_fused_out(handle, torch.zeros(3, 256, **bf), torch.zeros(3, 64, **bf), norm_weight=gamma)
        with pytest.raises(RuntimeError, match="wrong size"):
            ext.linear_fused_out(handle, x, y, swiglu=True)
    finally:
        ext.free(handle)


class _LocalPeers:
    """Stand-in for tp.PeerExchange on one GPU: `world` inboxes that all live in this GPU's memory, so the
    test can play the other ranks' parts (write their inbox rows and flags) from the host side."""

    def __init__(self, hidden, world, rank):
        import ctypes
        self.rank, self.world, self.hidden = rank, world, hidden
        self.inboxes = [torch.zeros(2 * world * hidden, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
        self.flags = [torch.zeros(2 * world, device="cuda", dtype=torch.int32) for _ in range(world)]
        self.epoch = torch.zeros(1, device="cuda", dtype=torch.int32)
        pointers = ctypes.c_void_p * world
        self.inbox_ptrs = pointers(*[t.data_ptr() for t in self.inboxes])
        self.flag_ptrs = pointers(*[t.data_ptr() for t in self.flags])

    def deliver(self, sender, epoch, values):
        """What rank `sender` would have done for `epoch`: its row in our inbox, then its flag."""
        slot = epoch & 1
        start = (slot * self.world + sender) * self.hidden
        self.inboxes[self.rank][start:start + self.hidden] = values.reshape(-1)
        self.flags[self.rank][slot * self.world + sender] = epoch


def test_allreduce_add_rmsnorm_single_rank_equals_plain_kernel(ext):
    hidden = 5120
    gen = torch.Generator(device="cuda").manual_seed(3)
    gamma = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=gen)).bfloat16()
    peers = _LocalPeers(hidden, 1, 0)
    h = torch.randn(1, hidden, device="cuda", generator=gen).bfloat16()
    h_ref = h.clone()
    ext.kernel_status(clear=True)
    for step in range(4):                                        # both inbox slots, advancing epochs
        delta = torch.randn(1, hidden, device="cuda", generator=gen).bfloat16()
        y, y_ref = torch.empty_like(h), torch.empty_like(h)
        ext.allreduce_add_rmsnorm(h, delta, gamma, y, 1e-6, peers)
        ext.add_rmsnorm(h_ref, delta, gamma, y_ref, 1e-6)
        torch.cuda.synchronize()
        assert torch.equal(h, h_ref) and torch.equal(y, y_ref), step
        assert int(peers.epoch.item()) == step + 1
    assert ext.kernel_status() == 0


def test_allreduce_add_rmsnorm_sums_peers_in_rank_order(ext):
    """Rank 1 of 3 with the other ranks' contributions already delivered: no kernel ever waits here."""
    hidden, world, rank = 1024, 3, 1
    gen = torch.Generator(device="cuda").manual_seed(4)
    gamma = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=gen)).bfloat16()
    peers = _LocalPeers(hidden, world, rank)
    h = torch.randn(1, hidden, device="cuda", generator=gen).bfloat16()
    ext.kernel_status(clear=True)
    for epoch in (1, 2, 3):
        parts = [torch.randn(1, hidden, device="cuda", generator=gen).bfloat16() for _ in range(world)]
        for sender in range(world):
            if sender != rank:
                peers.deliver(sender, epoch, parts[sender])
        total = (parts[0].float() + parts[1].float() + parts[2].float()).bfloat16()      # rank order, one rounding
        h_ref, y_ref = h.clone(), torch.empty_like(h)
        ext.add_rmsnorm(h_ref, total, gamma, y_ref, 1e-6)
        y = torch.empty_like(h)
        ext.allreduce_add_rmsnorm(h, parts[rank], gamma, y, 1e-6, peers)
        torch.cuda.synchronize()
        assert torch.equal(h, h_ref) and torch.equal(y, y_ref), epoch
        slot = epoch & 1
        for receiver in range(world):                            # our row and flag reached every rank's inbox
            start = (slot * world + rank) * hidden
            assert torch.equal(peers.inboxes[receiver][start:start + hidden], parts[rank].reshape(-1))
            assert int(peers.flags[receiver][slot * world + rank].item()) == epoch
    assert ext.kernel_status() == 0


def test_allreduce_wait_is_bounded_and_reports(ext):
    """A flag that nobody sets: the wait runs out, the kernel finishes, the status word says 32."""
    hidden = 256
    peers = _LocalPeers(hidden, 2, 0)
    h = torch.zeros(1, hidden, device="cuda", dtype=torch.bfloat16)
    gamma = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
    ext.kernel_status(clear=True)
    ext.allreduce_add_rmsnorm(h, torch.ones_like(h), gamma, torch.empty_like(h), 1e-6, peers)
    torch.cuda.synchronize()
    assert ext.kernel_status(clear=True) == 32
    assert ext.kernel_status() == 0
    torch.zeros(1, device="cuda").add_(1)                        # the context is still usable
    torch.cuda.synchronize()
