"""The fused exchange + merge kernel of the KV-range-sharded decode (``ga_attn_exchange_merge``) on ONE GPU.

The kernel of rank r stores into its peers' buffers and waits for their flags. On one GPU the peers are plain
buffers of the same device that the test fills the way the peers' kernels would have (their rows are in
place before the launch, so the launched kernel never waits for another kernel); what is checked is the addressing
of the pushes, the (value, call number) pairs over three calls (both buffer parities), the call counter and the merge against
``ga_attn_merge``. The bounded wait is checked by rows that nothing writes: the kernel returns and leaves status 6.
The two-process form over real peer memory runs in ``bench.py --gpus N`` (its result is compared bitwise with the
NCCL path and against the oracle there).
"""

import ctypes

import pytest
import torch

from greenattention_b200 import _C

pytestmark = pytest.mark.gpu
ROWS, HD = 64, 128
N = ROWS * (HD + 1)


def partial(seed, dev, empty_rows=()):
    g = torch.Generator(device="cpu").manual_seed(seed)
    o = torch.randn(ROWS, HD, generator=g)
    lse = torch.randn(ROWS, generator=g) * 3
    for r in empty_rows:
        lse[r] = float("-inf")
        o[r] = 0
    return torch.cat([o.reshape(-1), lse]).to(dev)


def expected(parts):
    from greenattention_b200 import attn_decode

    o = torch.stack([p[: ROWS * HD].view(ROWS, HD) for p in parts])
    lse = torch.stack([p[ROWS * HD:] for p in parts])
    return attn_decode.merge_partials(o, lse)


class Peers:
    """`world` gather buffers and flag arrays on one device, as rank `rank` would see them mapped."""

    def __init__(self, world, rank, dev):
        self.world, self.rank, self.dev = world, rank, dev
        # a value and the number of the call that wrote it, side by side: [parity][source rank][element][2]
        self.bufs = [torch.zeros(2 * world * N * 2, dtype=torch.int32, device=dev) for _ in range(world)]
        self.buf_ptrs = torch.tensor([b.data_ptr() for b in self.bufs], dtype=torch.int64, device=dev)
        self.epoch = torch.zeros(2, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.out = torch.empty(ROWS, HD, dtype=torch.bfloat16, device=dev)

    def arrive(self, src, call, part):
        """What rank `src`'s kernel of call number `call` leaves in rank `rank`'s buffer and flags."""
        par = call & 1
        slot = self.bufs[self.rank].view(2, self.world, N, 2)[par, src]
        slot[:, 0].copy_(part.view(torch.int32))
        slot[:, 1].fill_(call)

    def launch(self, mine, polls=0):
        x = _C.GaExchangeParams()
        x.mine, x.peer_bufs, x.peer_flags = mine.data_ptr(), self.buf_ptrs.data_ptr(), None
        x.epoch, x.rank, x.world, x.rows, x.head_dim = self.epoch.data_ptr(), self.rank, self.world, ROWS, HD
        x.out, x.lse, x.status, x.wait_polls = self.out.data_ptr(), None, self.status.data_ptr(), polls
        _C.check(_C.lib().ga_attn_exchange_merge(ctypes.byref(x), torch.cuda.current_stream().cuda_stream), "exchange")
        torch.cuda.synchronize()


def test_single_rank_is_the_plain_merge():
    dev = torch.device("cuda")
    p = Peers(1, 0, dev)
    mine = partial(1, dev, empty_rows=(3,))
    p.launch(mine)
    assert torch.equal(p.out, expected([mine]))
    assert p.epoch.tolist() == [1, 0] and p.status.item() == 0
    assert (p.out[3] == 0).all()


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 2), (8, 5)])
def test_pushes_flags_and_merge_over_two_calls(world, rank):
    dev = torch.device("cuda")
    p = Peers(world, rank, dev)
    for call in (1, 2, 3):
        parts = [partial(100 * call + j, dev, empty_rows=(7,) if j % 2 else (7, 9)) for j in range(world)]
        for j in range(world):
            if j != rank:
                p.arrive(j, call, parts[j])
        p.launch(parts[rank])
        assert p.status.item() == 0
        assert torch.equal(p.out, expected(parts)), f"call {call}"
        assert (p.out[7] == 0).all()  # a row no rank saw a key of
        assert p.epoch.tolist() == [call, 0]
        par = call & 1
        for j in range(world):
            if j == rank:
                continue
            # my partial sits in slot [par][rank] of every peer's buffer, every value with the call number
            mine_there = p.bufs[j].view(2, world, N, 2)[par, rank]
            assert torch.equal(mine_there[:, 0].contiguous().view(torch.float32), parts[rank])
            assert (mine_there[:, 1] == call).all()
            # and nothing else of the peer's buffer was touched
            other = p.bufs[j].view(2, world, N, 2).clone()
            other[par, rank] = 0
            if call >= 2:
                other[1 - par, rank] = 0  # the call before
            assert (other == 0).all()


def test_a_wait_that_runs_out_sets_the_status_and_returns():
    dev = torch.device("cuda")
    p = Peers(2, 0, dev)
    mine = partial(5, dev)
    p.launch(mine, polls=2000)  # the peer's flag is never set: about a millisecond, then the kernel gives up
    assert p.status.item() == 6
    assert p.epoch.tolist() == [1, 0]  # the call still counts, so the next one uses the other buffer half
    # the context is fine: a complete call right after
    p.status.zero_()
    other = partial(6, dev)
    p.arrive(1, 2, other)
    p.launch(mine)
    assert p.status.item() == 0 and torch.equal(p.out, expected([mine, other]))


def test_rejects_bad_arguments():
    dev = torch.device("cuda")
    p = Peers(2, 0, dev)
    x = _C.GaExchangeParams()
    x.mine, x.peer_bufs, x.peer_flags = partial(1, dev).data_ptr(), p.buf_ptrs.data_ptr(), None
    x.epoch, x.rank, x.world, x.rows, x.head_dim = p.epoch.data_ptr(), 2, 2, ROWS, HD
    x.out, x.status = p.out.data_ptr(), p.status.data_ptr()
    assert _C.lib().ga_attn_exchange_merge(ctypes.byref(x), None) != 0
    assert b"rank" in _C.lib().ga_last_error()
    x.rank, x.world = 0, 99
    assert _C.lib().ga_attn_exchange_merge(ctypes.byref(x), None) != 0
