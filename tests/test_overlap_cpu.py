"""Weight lease of the portable path: one acquisition per pass shared by all chunks, one gradient return."""

import torch

from ep_balance_b200.parallel.overlap import (BackwardKick, LeasedExperts, WeightLease, forked, side_stream,
                                              side_streams_enabled, weight_channel)


class FakeTransport:
    """Two slots of a [2, 3] weight; slot 1 is a "replica" whose gradient goes back to the owner's parameter."""

    def __init__(self) -> None:
        self.param = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], requires_grad=True)
        self.log = []

    def acquire(self):
        self.log.append("acquire")
        return [self.param.detach().clone()]

    def give_back(self, grad_stacks):
        self.log.append("give_back")
        return [grad_stacks[0].clone()]


def test_cpu_has_no_lanes_and_forked_runs_inline():
    assert not side_streams_enabled("cpu") and side_stream("cpu") is None
    assert weight_channel(None, "cpu") is None
    ran = []
    with forked(None) as join:
        ran.append(1)
    join[0]()
    assert ran == [1]


def test_lease_is_shared_by_chunks_released_after_forward_and_returns_gradients_once():
    tr = FakeTransport()
    lease = WeightLease(tr, consumers=2, device="cpu")
    lease.start()
    lease.start()                                  # idempotent while the stacks are out
    assert tr.log == ["acquire"]

    def compute(x, stacks):
        return x @ stacks[0].t()                   # [n, 3] x [3, 2]

    xs = [torch.randn(4, 3, requires_grad=True), torch.randn(5, 3, requires_grad=True)]
    ys = [LeasedExperts.apply(x, lease, compute, tr.param) for x in xs]
    assert lease._stacks is None, "nothing may stay alive between forward and backward"
    out = BackwardKick.apply(torch.cat(ys).sum().view(1), lease)
    out.backward()
    # forward pull, backward re-pull (started by the kick, before any chunk ran), one return
    assert tr.log == ["acquire", "acquire", "give_back"]
    assert (lease.acquisitions, lease.returns) == (2, 1)
    want = torch.cat([x.detach() for x in xs]).sum(0).expand(2, 3)
    assert torch.allclose(tr.param.grad, want)
    for x in xs:
        assert torch.allclose(x.grad, tr.param.detach().sum(0).expand_as(x))
