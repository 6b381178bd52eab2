import pytest
import torch

from forgetrain_b200.data.prefetch import DataPrefetcher
from forgetrain_b200.data.synthetic import SyntheticTokenSource


class FakeEvent:
    log = []

    def __init__(self):
        self.recorded = False

    def record(self, *a):
        self.recorded = True
        FakeEvent.log.append("record")

    def wait(self):
        assert self.recorded
        FakeEvent.log.append("wait")


class FakeStream:
    pass


def _batches(n, masked=()):
    for i in range(n):
        yield {"tokens": torch.full((1, 4), i), "labels": torch.full((1, 4), i),
               "loss_mask": torch.zeros(1, 4) if i in masked else torch.ones(1, 4)}


def test_fifo_order_depth_and_events():
    FakeEvent.log = []
    pf = DataPrefetcher(_batches(5), "cpu", depth=3, stream_factory=FakeStream, event_factory=FakeEvent)
    first = next(pf)
    assert int(first["tokens"][0, 0]) == 0
    assert len(pf.queue) == 3                      # refilled to depth after the pop
    rest = [int(b["tokens"][0, 0]) for b in pf]
    assert rest == [1, 2, 3, 4]
    assert pf.recorded_tensors == 5 * 3            # every tensor handed out was stream-recorded
    assert FakeEvent.log.count("record") == 5 and FakeEvent.log.count("wait") == 5


def test_all_masked_batches_are_skipped():
    pf = DataPrefetcher(_batches(4, masked={0, 2}), "cpu", depth=1)
    got = [int(b["tokens"][0, 0]) for b in pf]
    assert got == [1, 3] and pf.skipped == 2


def test_depth_validation():
    with pytest.raises(ValueError):
        DataPrefetcher(_batches(1), "cpu", depth=0)
    with pytest.raises(ValueError):
        DataPrefetcher(_batches(1), "cpu", depth=5)


def test_synthetic_source_is_seeded_and_resumable():
    a = SyntheticTokenSource(1000, 2, 16, seed=7, dp_rank=0, pin=False)
    b = SyntheticTokenSource(1000, 2, 16, seed=7, dp_rank=0, pin=False)
    c = SyntheticTokenSource(1000, 2, 16, seed=7, dp_rank=1, pin=False)
    x, y, z = next(a), next(b), next(c)
    assert torch.equal(x["tokens"], y["tokens"]) and not torch.equal(x["tokens"], z["tokens"])
    assert torch.equal(x["tokens"][:, 1:], x["labels"][:, :-1])      # labels = inputs shifted by one
    assert x["tokens"].max() < 1000 and x["loss_mask"].sum() == 32
    next(a)
    st = a.state_dict()
    want = next(a)
    r = SyntheticTokenSource(1000, 2, 16, seed=7, dp_rank=0, pin=False)
    r.load_state_dict(st)
    assert torch.equal(next(r)["tokens"], want["tokens"])
