"""Second-generation tensor-parallel exchange on ONE GPU: the other ranks' parts are played from the host
(their packets are written into inboxes that all live in this GPU's memory), so no kernel here ever waits
for another process.  Run with ``-m gpu``."""
import ctypes

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


class LocalPeers:
    """Stand-in for tp.PeerExchange: `world` packet inboxes and token inboxes in this GPU's memory."""

    def __init__(self, hidden, world, rank):
        self.rank, self.world, self.hidden = rank, world, hidden
        self.per_sender = hidden // 4
        self.inboxes = [torch.zeros(2 * world * self.per_sender, 4, device="cuda", dtype=torch.int32) for _ in range(world)]
        self.token_inboxes = [torch.zeros(2 * world, 4, device="cuda", dtype=torch.int32) for _ in range(world)]
        self.packet_inbox = self.inboxes[rank]
        self.packet_epoch = torch.zeros(1, device="cuda", dtype=torch.int32)
        self.token_epoch = torch.zeros(1, device="cuda", dtype=torch.int32)
        pointers = ctypes.c_void_p * world
        self.packet_ptrs = pointers(*[t.data_ptr() for t in self.inboxes])
        self.token_ptrs = pointers(*[t.data_ptr() for t in self.token_inboxes])

    @staticmethod
    def packets_of(values, epoch):
        """bf16 [hidden] -> int32 [hidden/4, 4] = (v0 | v1 << 16, epoch, v2 | v3 << 16, epoch)."""
        words = values.reshape(-1).view(torch.int16).to(torch.int32) & 0xFFFF
        pair = (words[0::2] | (words[1::2] << 16)).to(torch.int32)
        out = torch.empty(pair.numel() // 2, 4, device=values.device, dtype=torch.int32)
        out[:, 0], out[:, 2] = pair[0::2], pair[1::2]
        out[:, 1] = out[:, 3] = epoch
        return out

    def deliver(self, sender, epoch, values):
        start = ((epoch & 1) * self.world + sender) * self.per_sender
        self.inboxes[self.rank][start:start + self.per_sender] = self.packets_of(values, epoch)

    def sent(self, receiver, epoch):
        start = ((epoch & 1) * self.world + self.rank) * self.per_sender
        return self.inboxes[receiver][start:start + self.per_sender]


def _linear(ext, lut, m, k, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    blocks, scales = O.encode_minmax(w, lut)
    return ext.pack_encoded(torch.from_numpy(blocks), torch.from_numpy(scales))


@pytest.mark.parametrize("hidden", [256, 2048, 5120, 16384])
def test_cluster_norm_without_exchange_equals_plain_kernel(ext, lut, hidden):
    gen = torch.Generator(device="cuda").manual_seed(hidden)
    gamma = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=gen)).bfloat16()
    h = torch.randn(1, hidden, device="cuda", generator=gen).bfloat16()
    handle = _linear(ext, lut, 64, hidden, hidden)
    try:
        staged = torch.empty(ext.linear_single_info(handle)[2], dtype=torch.uint8, device="cuda")
        for delta in (None, (torch.randn(1, hidden, device="cuda", generator=gen) * 0.5).bfloat16()):
            h_ref, y_ref = h.clone(), torch.empty_like(h)
            ext.add_rmsnorm(h_ref, delta, gamma, y_ref, 1e-6)
            got_h, y = h.clone(), torch.empty_like(h)
            staged.fill_(0x5A)
            ext.peer_reduce_rmsnorm(got_h, gamma, 1e-6, delta=delta, y=y, staged=staged)
            torch.cuda.synchronize()
            assert torch.equal(got_h, h_ref)
            # the sum of squares is added in another order than the one-CTA kernel's: a bf16 step at most
            assert float((y.float() - y_ref.float()).abs().max()) <= float(y_ref.float().abs().max()) * 2 ** -7
            want, got = torch.empty(1, 64, device="cuda", dtype=torch.bfloat16), torch.empty(1, 64, device="cuda", dtype=torch.bfloat16)
            ext.linear_single(handle, y, want)
            ext.linear_single(handle, None, got, staged=staged)
            assert torch.equal(got, want)                     # staged by the cluster == staged by the linear
    finally:
        ext.free(handle)


def test_push_and_reduce_one_rank(ext, lut):
    """world = 1: the linear's packets land in its own inbox; reduce + norm equals linear + add_rmsnorm."""
    hidden, k = 1024, 2560
    handle = _linear(ext, lut, hidden, k, 1)
    gen = torch.Generator(device="cuda").manual_seed(1)
    gamma = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=gen)).bfloat16()
    peers = LocalPeers(hidden, 1, 0)
    h = torch.randn(1, hidden, device="cuda", generator=gen).bfloat16()
    h_ref = h.clone()
    ext.kernel_status(clear=True)
    try:
        for step in range(4):                                   # both slots, advancing epochs
            x = torch.randn(1, k, device="cuda", generator=gen).bfloat16()
            part = torch.empty(1, hidden, device="cuda", dtype=torch.bfloat16)
            ext.linear_single(handle, x, part)
            y_ref = torch.empty_like(h)
            ext.add_rmsnorm(h_ref, part, gamma, y_ref, 1e-6)
            ext.linear_single_push(handle, x, peers)
            y = torch.empty_like(h)
            ext.peer_reduce_rmsnorm(h, gamma, 1e-6, peers=peers, y=y)
            torch.cuda.synchronize()
            assert torch.equal(peers.sent(0, step + 1), LocalPeers.packets_of(part, step + 1)), step
            assert torch.equal(h, h_ref), step
            assert float((y.float() - y_ref.float()).abs().max()) <= float(y_ref.float().abs().max()) * 2 ** -7
            assert int(peers.packet_epoch.item()) == step + 1
        assert ext.kernel_status() == 0
    finally:
        ext.free(handle)


@pytest.mark.parametrize("world,rank", [(3, 1), (8, 5)])
def test_reduce_adds_all_ranks_in_rank_order(ext, lut, world, rank):
    hidden, k = 5120, 640
    handle = _linear(ext, lut, hidden, k, world)
    gen = torch.Generator(device="cuda").manual_seed(world)
    gamma = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=gen)).bfloat16()
    peers = LocalPeers(hidden, world, rank)
    h = torch.randn(1, hidden, device="cuda", generator=gen).bfloat16()
    ext.kernel_status(clear=True)
    try:
        for epoch in (1, 2, 3):
            x = torch.randn(1, k, device="cuda", generator=gen).bfloat16()
            mine = torch.empty(1, hidden, device="cuda", dtype=torch.bfloat16)
            ext.linear_single(handle, x, mine)
            parts = [mine if r == rank else torch.randn(1, hidden, device="cuda", generator=gen).bfloat16() for r in range(world)]
            for sender in range(world):
                if sender != rank:
                    peers.deliver(sender, epoch, parts[sender])
            total = torch.zeros(1, hidden, device="cuda")
            for r in range(world):                                # rank order, fp32, one rounding
                total += parts[r].float()
            h_ref, y_ref = h.clone(), torch.empty_like(h)
            ext.add_rmsnorm(h_ref, total.bfloat16(), gamma, y_ref, 1e-6)
            ext.linear_single_push(handle, x, peers)
            y = torch.empty_like(h)
            ext.peer_reduce_rmsnorm(h, gamma, 1e-6, peers=peers, y=y)
            torch.cuda.synchronize()
            assert torch.equal(h, h_ref), epoch
            assert float((y.float() - y_ref.float()).abs().max()) <= float(y_ref.float().abs().max()) * 2 ** -7
            for receiver in range(world):                         # our packets reached every rank's inbox
                assert torch.equal(peers.sent(receiver, epoch), LocalPeers.packets_of(mine, epoch))
        assert ext.kernel_status() == 0
    finally:
        ext.free(handle)


def test_reduce_poll_is_bounded_and_reports(ext):
    """Packets that nobody sends: the poll runs out, the kernel finishes, the status word says 32."""
    hidden = 256
    peers = LocalPeers(hidden, 2, 0)
    h = torch.zeros(1, hidden, device="cuda", dtype=torch.bfloat16)
    gamma = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
    peers.deliver(0, 1, torch.ones(1, hidden, device="cuda", dtype=torch.bfloat16))      # rank 1 never delivers
    ext.kernel_status(clear=True)
    ext.peer_reduce_rmsnorm(h, gamma, 1e-6, peers=peers, y=torch.empty_like(h))
    torch.cuda.synchronize()
    assert ext.kernel_status(clear=True) == 32
    assert ext.kernel_status() == 0
    torch.zeros(1, device="cuda").add_(1)                         # the context is still usable
    torch.cuda.synchronize()


def test_best_token_exchange(ext):
    world, rank = 4, 2
    peers = LocalPeers(64, world, rank)
    next_token = torch.zeros(1, device="cuda", dtype=torch.int64)
    ext.kernel_status(clear=True)
    cases = [([1.0, 5.0, 3.0, 2.0], [11, 22, 33, 44], 22),          # plain maximum
             ([7.5, 1.0, 7.5, 7.5], [100, 200, 300, 400], 100),     # tie: lowest rank
             ([-3.0, -2.0, -1.0, -4.0], [5, 6, 7, 8], 1000 + 7)]    # our own score wins; offset applies to ours
    for epoch, (scores, tokens, want) in enumerate(cases, start=1):
        for sender in range(world):
            if sender != rank:
                packet = torch.tensor([np.float32(scores[sender]).view(np.int32), epoch, tokens[sender], epoch], dtype=torch.int32, device="cuda")
                peers.token_inboxes[rank][(epoch & 1) * world + sender] = packet
        score = torch.tensor([scores[rank]], device="cuda", dtype=torch.float32)
        token = torch.tensor([tokens[rank]], device="cuda", dtype=torch.int64)
        offset = 1000 if want >= 1000 else 0
        ext.peer_best_token(score, token, offset, peers, next_token)
        torch.cuda.synchronize()
        assert int(next_token.item()) == want, epoch
        for receiver in range(world):                              # our packet reached every rank
            got = peers.token_inboxes[receiver][(epoch & 1) * world + rank].tolist()
            assert got[1] == epoch and got[3] == epoch and got[2] == tokens[rank] + offset
    assert ext.kernel_status() == 0
