"""Properties of the epoch-flag protocol of the peer-memory collectives, checked on a host model
(threads as ranks): late signals, a missing rank, wrap-around of the 32-bit epoch, buffer reuse
across consecutive buckets, and the device-side epoch base that a captured graph relies on."""
import numpy as np
import pytest

from flag_protocol_model import ERR_WAIT_PEER, FlagBoards, reduce_scatter, run_ranks


def _bufs(world, n, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal(n * world).astype(np.float32) for _ in range(world)]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_reduce_scatter_with_a_late_rank(world):
    boards = FlagBoards(world)
    bufs = _bufs(world, 64)
    want = sum(b.copy() for b in bufs) / world
    ss = run_ranks(world, lambda r: reduce_scatter(boards, bufs, r, epoch=1,
                                                   delay_s=0.05 if r == world - 1 else 0.0))
    for r in range(world):
        assert np.allclose(bufs[r][r * 64:(r + 1) * 64], want[r * 64:(r + 1) * 64], atol=1e-6)
    assert sum(ss) == pytest.approx(float((want ** 2).sum()), rel=1e-5)
    assert boards.status == [0] * world


def test_a_rank_that_never_signals_gives_a_status_not_a_hang():
    world = 3
    boards = FlagBoards(world)
    bufs = _bufs(world, 16)
    before = [b.copy() for b in bufs]
    run_ranks(world, lambda r: reduce_scatter(boards, bufs, r, epoch=1, limit_s=0.05,
                                              skip_signal=(r == 2)))
    assert all(s == ERR_WAIT_PEER for s in boards.status)
    for a, b in zip(bufs, before):          # nobody reduced from a buffer that was not ready
        assert np.array_equal(a, b)


def test_consecutive_buckets_reuse_the_flags_with_growing_epochs():
    """The exit barrier keeps a fast rank from starting bucket k+1 (and overwriting data a slow
    rank still reads) before everybody has left bucket k."""
    world = 4
    boards = FlagBoards(world)
    data = [_bufs(world, 32, seed=k) for k in range(5)]
    want = [sum(b.copy() for b in d) / world for d in data]

    def rank_main(r):
        for k in range(5):
            reduce_scatter(boards, data[k], r, epoch=k + 1, delay_s=0.002 * ((r + k) % world))

    run_ranks(world, rank_main)
    for k in range(5):
        for r in range(world):
            assert np.allclose(data[k][r][r * 32:(r + 1) * 32], want[k][r * 32:(r + 1) * 32], atol=1e-6)
    assert boards.status == [0] * world


def test_epoch_comparison_survives_wrap_around():
    world = 2
    boards = FlagBoards(world)
    # flags sit just below 2^32 from earlier launches; the next epochs wrap to small numbers
    boards.flags[:] = 0xFFFFFFFE
    for epoch in (0xFFFFFFFF, 0x00000000, 0x00000001):
        bufs = _bufs(world, 8, seed=epoch & 7)
        want = (bufs[0] + bufs[1]) / 2
        run_ranks(world, lambda r: reduce_scatter(boards, bufs, r, epoch=epoch))
        assert np.allclose(bufs[0][:8], want[:8], atol=1e-6) and np.allclose(bufs[1][8:], want[8:], atol=1e-6)
    assert boards.status == [0, 0]
    # a stale flag from BEFORE the wrap must not satisfy a wait for an epoch after it
    boards.flags[0, 0, 1] = 0xFFFFFFF0
    assert boards.wait(0, 0, 5, limit_s=0.02) is False


def test_device_side_base_makes_relative_epochs_replayable():
    """A captured graph always launches with the same (relative) epochs; the base that its last
    node advances turns them into fresh absolute ones on every replay."""
    world = 2
    boards = FlagBoards(world)
    per_replay = 3                       # collectives inside the captured step
    for replay in range(4):
        for k in range(per_replay):
            bufs = _bufs(world, 8, seed=10 * replay + k)
            want = (bufs[0] + bufs[1]) / 2
            run_ranks(world, lambda r: reduce_scatter(boards, bufs, r, epoch=k + 1))
            assert np.allclose(bufs[0][:8], want[:8], atol=1e-6)
        boards.base[:, 0] += per_replay   # what the epoch-advance node does, on every rank
        boards.base[:, 1] += per_replay
    assert int(boards.flags[0, 0, 1]) == 4 * per_replay
    # without the advance a replay would find its epochs already satisfied and skip the wait:
    stale = FlagBoards(world)
    stale.signal(1, 0, 1)
    assert stale.wait(0, 0, 1, limit_s=0.01) is False      # rank 0 itself has not signalled
    stale.signal(0, 0, 1)
    assert stale.wait(0, 0, 1, limit_s=0.01) is True
    assert stale.wait(0, 0, 1, limit_s=0.01) is True       # ... and stays true: epochs must grow


def test_host_side_epoch_counter_wraps_modulo_two_to_the_32():
    """The host's per-slot counter, the int32 tensor that carries it to the device-side base
    and the value read back after graph replays all count modulo 2^32, like the device's
    signed-difference comparison: crossing 2^31 or 2^32 never yields an epoch that a stale flag
    already satisfies."""
    from forgetrain_b200.parallel.fused_dp import _as_i32, bump_epoch
    world = 2
    boards = FlagBoards(world)
    for start in (0x7FFFFFFE, 0xFFFFFFFE):
        epoch = start
        boards.flags[:] = start                      # what earlier launches left behind
        for _ in range(4):                           # the host's own increment
            epoch = bump_epoch(epoch)
            # before anyone signals, the stale flags must NOT pass for the new epoch
            assert boards.wait(0, 0, epoch, limit_s=0.005) is False
            boards.status = [0] * world
            bufs = _bufs(world, 8, seed=epoch & 7)
            want = (bufs[0] + bufs[1]) / 2
            run_ranks(world, lambda r: reduce_scatter(boards, bufs, r, epoch=epoch))
            assert np.allclose(bufs[0][:8], want[:8], atol=1e-6)
            # the device base travels through an int32 tensor and back without losing bits
            assert (_as_i32(epoch) & 0xFFFFFFFF) == epoch and -(1 << 31) <= _as_i32(epoch) < (1 << 31)
        assert boards.status == [0, 0]


def test_every_host_epoch_counter_uses_the_shared_increment():
    """The data-parallel and the tensor-parallel collectives keep separate counters; both must
    step them with ``bump_epoch`` (a private ``& 0x7FFFFFFF`` in one of them would break the
    wrap-around guarantee checked above)."""
    import inspect
    import re
    from forgetrain_b200.parallel import fused_dp, fused_tp
    assert fused_dp.bump_epoch(0x7FFFFFFF) == 0x80000000
    assert fused_dp.bump_epoch(0xFFFFFFFF) == 0
    for mod in (fused_dp, fused_tp):
        src = inspect.getsource(mod)
        assert "0x7FFFFFFF" not in src
        # every assignment to an epoch counter goes through the helper
        for m in re.finditer(r"self\.epoch(?:_[a-z]+|\[slot\]) = (.+)", src):
            rhs = m.group(1)
            assert "+ 1" not in rhs or "bump_epoch" in rhs, rhs
    assert len(re.findall(r"bump_epoch\(self\.epoch_", inspect.getsource(fused_tp))) == 3


def test_epoch_bookkeeping_of_the_symmetric_buffers_through_capture_replay_and_resync(monkeypatch):
    """The host state machine of ``SymmetricBuffers`` itself (no device: the native library is
    replaced by a stand-in whose "advance" node adds to the base tensor, as a replay would): eager
    epochs count up per slot; inside a capture the launch arguments are 1, 2, ... relative to the
    base, which starts at the eager epochs; every replay advances the base by what one step
    consumes; an eager launch after a capture is refused until ``resync_epochs`` has read the base
    back, after which eager epochs continue behind the last replay, also across 2^31."""
    import ctypes
    import torch
    from forgetrain_b200.parallel import fused_dp
    replays = []

    class FakeLib:
        def ft_comm_epoch_advance(self, base_ptr, add, stream):
            replays.append(list(add))
            return 0

    class FakeLibModule:
        @staticmethod
        def lib():
            return FakeLib()
        ptr = staticmethod(lambda t: t)
        stream = staticmethod(lambda: None)
        check_rc = staticmethod(lambda rc, what: None)

    monkeypatch.setattr(fused_dp, "_lib", FakeLibModule)
    for start in (0, 0x7FFFFFF0):
        replays.clear()
        s = object.__new__(fused_dp.SymmetricBuffers)
        s.epoch = [start] * fused_dp.NUM_FLAG_SLOTS
        s.epoch_base = torch.zeros(fused_dp.NUM_FLAG_SLOTS, dtype=torch.int32)
        s._capturing, s._graph_mode, s._used = False, False, [0] * fused_dp.NUM_FLAG_SLOTS
        # eager: absolute epochs, per slot
        assert [s.next_epoch(0), s.next_epoch(0), s.next_epoch(2)] == \
            [(start + 1) & 0xFFFFFFFF, (start + 2) & 0xFFFFFFFF, (start + 1) & 0xFFFFFFFF]
        s.set_epoch(1, s.epoch[0])
        assert s.epoch[1] == s.epoch[0]
        # capture: relative epochs, the base holds the eager ones
        s.begin_capture()
        assert [int(x) & 0xFFFFFFFF for x in s.epoch_base.tolist()] == s.epoch
        rel = [s.next_epoch(0), s.next_epoch(0), s.next_epoch(0), s.next_epoch(2)]
        assert rel == [1, 2, 3, 1]
        s.set_epoch(1, rel[2])
        s.end_capture()
        assert replays[-1][:3] == [3, 3, 1] and s._graph_mode and not s._capturing
        with pytest.raises(RuntimeError, match="resync_epochs"):
            s.next_epoch(0)
        # five replays: the graph's last node adds what one step consumes (done here by hand)
        per = torch.tensor(replays[-1], dtype=torch.int64)
        total = (torch.tensor([fused_dp._as_i32(e) for e in s.epoch], dtype=torch.int64) + 5 * per)
        s.epoch_base.copy_(((total + 2 ** 31) % 2 ** 32 - 2 ** 31).to(torch.int32))
        s.resync_epochs()
        assert not s._graph_mode and not s.epoch_base.any()
        assert s.epoch[0] == (start + 2 + 15) & 0xFFFFFFFF and s.epoch[2] == (start + 1 + 5) & 0xFFFFFFFF
        assert s.next_epoch(0) == (start + 2 + 16) & 0xFFFFFFFF      # eager again, behind the last replay
        # a second capture while in graph mode resyncs by itself
        s.begin_capture()
        s.next_epoch(0)
        s.end_capture()
        s.epoch_base += 1
        s.begin_capture()
        assert s.epoch[0] == (start + 2 + 16 + 1) & 0xFFFFFFFF and s._capturing
