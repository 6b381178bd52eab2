"""Life-cycle cases of the auxiliary subsystems on CPU: checkpoint writer, batch prefetcher, step
profiler. Same approach as the reference's CPU tests (fake events and clocks, failures injected on
the host: exports/train_engine_0.5B/tests/test_checkpoint_round_trip.py:33-572,
test_periodic_save.py:40-264, test_data_prefetcher.py:54-300, test_profiling_lifecycle.py:46-788)."""
import json
import threading

import pytest
import torch

from forgetrain_b200.ckpt import checkpoint as ck
from forgetrain_b200.data.prefetch import DataPrefetcher
from forgetrain_b200.utils.profiler import DEEP_SEGMENTS, SEGMENTS, StepProfiler


# ---------------------------------------------------------------------------------------------
# checkpoint writer
# ---------------------------------------------------------------------------------------------
def _payload(**over):
    d = dict(params={"a": torch.randn(4, 4), "b": torch.ones(3)}, param_names=["a", "b"],
             optimizer_state={"master_weights": {"a": torch.zeros(4, 4)}, "exp_avg": {}, "exp_avg_sq": {},
                              "step_count": 7, "num_samples": 70}, num_samples=70,
             dataloader_state={"kind": "synthetic", "batches_drawn": 3})
    d.update(over)
    return d


@pytest.fixture(autouse=True)
def _no_writer_left_behind():
    yield
    try:
        ck.wait_for_async_save()
    except RuntimeError:
        pass


def test_parameters_keep_dtype_shape_and_values(tmp_path):
    params = {"w": torch.randn(3, 5).to(torch.bfloat16), "n": torch.ones(7, dtype=torch.float32)}
    ck.save_checkpoint(tmp_path, 5, async_io=False, **_payload(params=params, param_names=["w", "n"]))
    st = ck.load_resume_checkpoint(tmp_path / "step_0000005" / "training_state.pt")
    assert st["params"]["w"].dtype == torch.bfloat16 and st["params"]["n"].dtype == torch.float32
    assert torch.equal(st["params"]["w"], params["w"]) and tuple(st["params"]["w"].shape) == (3, 5)
    assert list(st["params"]) == ["w", "n"]


def test_a_file_a_step_directory_and_a_save_root_all_load(tmp_path):
    ck.save_checkpoint(tmp_path, 3, async_io=False, **_payload())
    ck.save_checkpoint(tmp_path, 8, async_io=False, **_payload(num_samples=80))
    by_file = ck.load_resume_checkpoint(tmp_path / "step_0000003" / "training_state.pt")
    by_dir = ck.load_resume_checkpoint(tmp_path / "step_0000003")
    by_root = ck.load_resume_checkpoint(tmp_path)
    assert by_file["step"] == by_dir["step"] == 3 and by_root["step"] == 8 and by_root["num_samples"] == 80


def test_latest_checkpoint_orders_steps_by_number_and_skips_unfinished_directories(tmp_path):
    for step in (9_999_999, 10_000_000, 12):
        ck.save_checkpoint(tmp_path, step, async_io=False, **_payload())
    (tmp_path / "step_99999999").mkdir()                       # a writer that died before the rename
    (tmp_path / "step_99999999" / "training_state.pt.tmp").write_bytes(b"half")
    (tmp_path / "step_notanumber").mkdir()
    assert ck.latest_checkpoint(tmp_path).parent.name == "step_10000000"
    assert ck.latest_checkpoint(tmp_path / "nowhere") is None
    with pytest.raises(FileNotFoundError):
        ck.load_resume_checkpoint(tmp_path / "step_99999999")
    # the per-rank shard files of tensor-parallel runs are found the same way
    for step in (9_999_999, 10_000_000):
        (tmp_path / ck.step_dir_name(step) / "rank_0.pt").write_bytes(b"x")
    assert ck.latest_step_dir(tmp_path, "rank_*.pt").name == "step_10000000"
    assert ck.latest_step_dir(tmp_path, "rank_7.pt") is None


def test_synchronous_failure_raises_at_once_and_leaves_no_partial_file(tmp_path, monkeypatch):
    def boom(obj, f, *a, **k):
        open(f, "wb").write(b"partial")
        raise OSError("quota exceeded")
    monkeypatch.setattr(torch, "save", boom)
    with pytest.raises(OSError, match="quota"):
        ck.save_checkpoint(tmp_path, 4, async_io=False, **_payload())
    assert not list(tmp_path.rglob("*.tmp")) and not list(tmp_path.rglob("training_state.pt"))


def test_an_older_checkpoint_survives_a_failed_rewrite_of_the_same_step(tmp_path, monkeypatch):
    ck.save_checkpoint(tmp_path, 2, async_io=False, **_payload(num_samples=20))
    real = torch.save

    def boom(obj, f, *a, **k):
        real({"garbage": True}, f)
        raise OSError("lost the mount")
    monkeypatch.setattr(torch, "save", boom)
    with pytest.raises(OSError):
        ck.save_checkpoint(tmp_path, 2, async_io=False, **_payload(num_samples=99))
    monkeypatch.setattr(torch, "save", real)
    assert ck.load_resume_checkpoint(tmp_path)["num_samples"] == 20     # the rename never happened


def test_the_next_save_reports_the_failure_of_the_previous_one(tmp_path, monkeypatch):
    real = torch.save
    calls = {"n": 0}

    def flaky(obj, f, *a, **k):
        calls["n"] += 1
        if calls["n"] == 1:
            raise OSError("first write failed")
        return real(obj, f, *a, **k)
    monkeypatch.setattr(torch, "save", flaky)
    ck.save_checkpoint(tmp_path, 1, async_io=True, **_payload())
    with pytest.raises(RuntimeError, match="first write failed"):
        ck.save_checkpoint(tmp_path, 2, async_io=True, **_payload())    # auto-wait surfaces it
    ck.save_checkpoint(tmp_path, 2, async_io=True, **_payload())        # and the slot is clear again
    ck.wait_for_async_save()
    assert ck.latest_checkpoint(tmp_path).parent.name == "step_0000002"
    assert not (tmp_path / "step_0000001" / "training_state.pt").exists()


def test_only_one_writer_runs_at_a_time(tmp_path, monkeypatch):
    running, peak = [0], [0]
    lock = threading.Lock()
    real = ck._write_atomic

    def counted(payload, path):
        with lock:
            running[0] += 1
            peak[0] = max(peak[0], running[0])
        try:
            threading.Event().wait(0.02)
            real(payload, path)
        finally:
            with lock:
                running[0] -= 1
    monkeypatch.setattr(ck, "_write_atomic", counted)
    for step in range(1, 5):
        ck.save_checkpoint(tmp_path, step, async_io=True, **_payload())
    ck.wait_for_async_save()
    assert peak[0] == 1 and len(list(tmp_path.glob("step_*/training_state.pt"))) == 4


def test_wait_without_a_writer_is_a_no_op():
    ck.wait_for_async_save()
    ck.wait_for_async_save()


def test_extra_entries_and_other_file_names(tmp_path):
    p = ck.save_checkpoint(tmp_path, 6, async_io=False, extra={"tp_size": 2, "tp_rank": 1},
                           filename="rank_1.pt", **_payload())
    assert p.name == "rank_1.pt"
    st = torch.load(p, weights_only=False)
    assert st["tp_size"] == 2 and st["tp_rank"] == 1 and st["format_version"] == 1
    assert ck.latest_checkpoint(tmp_path) is None               # no training_state.pt: not a resume point


def test_save_boundaries_over_a_whole_run():
    saved = [s for s in range(0, 11) if ck.should_save_after_step(s, 10, 4)]
    assert saved == [4, 8, 10]
    assert [s for s in range(0, 11) if ck.should_save_after_step(s, 10, 0)] == [10]
    # a resumed run does not rewrite the checkpoint it started from
    assert [s for s in range(0, 11) if ck.should_save_after_step(s, 10, 4, start_step=8)] == [10]
    assert [s for s in range(0, 13) if ck.should_save_after_step(s, 12, 5, start_step=5)] == [10, 12]


# ---------------------------------------------------------------------------------------------
# prefetcher
# ---------------------------------------------------------------------------------------------
class _Event:
    def __init__(self, log):
        self.log, self.recorded, self.id = log, False, len(log)

    def record(self, *a):
        self.recorded = True
        self.log.append(("record", self.id))

    def wait(self):
        assert self.recorded, "waited for an event that was never recorded"
        self.log.append(("wait", self.id))


class _Stream:
    pass


def _batches(n, masked=(), fail_at=None, drawn=None):
    for i in range(n):
        if drawn is not None:
            drawn.append(i)
        if i == fail_at:
            raise OSError("shard unreadable")
        yield {"tokens": torch.full((2, 4), i), "labels": torch.full((2, 4), i),
               "loss_mask": torch.zeros(2, 4) if i in masked else torch.ones(2, 4), "doc": f"d{i}"}


def _pf(src, depth, log=None):
    log = [] if log is None else log
    return DataPrefetcher(src, "cpu", depth=depth, stream_factory=_Stream,
                          event_factory=lambda: _Event(log)), log


@pytest.mark.parametrize("depth", [1, 2, 3, 4])
def test_read_ahead_is_exactly_the_depth(depth):
    drawn = []
    pf, _ = _pf(_batches(10, drawn=drawn), depth)
    assert drawn == []                                          # nothing is read before the first next()
    next(pf)
    assert drawn == list(range(depth + 1)) and len(pf.queue) == depth
    next(pf)
    assert drawn == list(range(depth + 2))


def test_every_batch_is_recorded_before_it_is_waited_for_and_in_order():
    pf, log = _pf(_batches(6), 3)
    got = [int(b["tokens"][0, 0]) for b in pf]
    assert got == list(range(6))
    waits = [i for kind, i in log if kind == "wait"]
    assert len(waits) == 6 and waits == sorted(waits)
    for k, (kind, i) in enumerate(log):
        if kind == "wait":
            assert ("record", i) in log[:k]


def test_exhaustion_is_sticky_and_drains_the_queue_first():
    pf, _ = _pf(_batches(3), 4)
    assert [int(b["tokens"][0, 0]) for b in pf] == [0, 1, 2]
    assert pf.exhausted and not pf.queue
    for _ in range(3):
        with pytest.raises(StopIteration):
            next(pf)


def test_empty_source_and_fully_masked_source_stop_at_once():
    pf, _ = _pf(_batches(0), 2)
    with pytest.raises(StopIteration):
        next(pf)
    pf, _ = _pf(_batches(4, masked={0, 1, 2, 3}), 2)
    with pytest.raises(StopIteration):
        next(pf)
    assert pf.skipped == 4


def test_masked_batches_do_not_count_against_the_depth():
    drawn = []
    pf, _ = _pf(_batches(8, masked={1, 2, 5}, drawn=drawn), 2)
    first = next(pf)
    assert int(first["tokens"][0, 0]) == 0
    assert [int(q[0]["tokens"][0, 0]) for q in pf.queue] == [3, 4] and pf.skipped == 2
    assert [int(b["tokens"][0, 0]) for b in pf] == [3, 4, 6, 7] and pf.skipped == 3


def test_masked_batches_pass_when_skipping_is_off():
    pf = DataPrefetcher(_batches(3, masked={1}), "cpu", depth=1, skip_all_masked=False)
    assert [int(b["tokens"][0, 0]) for b in pf] == [0, 1, 2] and pf.skipped == 0


def test_non_tensor_entries_travel_unchanged_and_bytes_count_tensors_only():
    pf, _ = _pf(_batches(2), 1)
    b = next(pf)
    assert b["doc"] == "d0"
    assert pf.bytes_last == 2 * (2 * 4 * 8) + 2 * 4 * 4         # two int64 tensors and one fp32 mask


def test_a_failing_source_raises_where_it_is_read_and_earlier_batches_are_kept():
    pf, _ = _pf(_batches(6, fail_at=2), 1)
    assert int(next(pf)["tokens"][0, 0]) == 0                   # batch 1 is already queued
    with pytest.raises(OSError, match="unreadable"):
        next(pf)                                                # refilling after batch 1 reads item 2
    pf2, _ = _pf(_batches(6, fail_at=0), 2)
    with pytest.raises(OSError):
        next(pf2)


def test_cpu_pass_through_without_a_stream_keeps_the_order():
    pf = DataPrefetcher(_batches(5), "cpu", depth=2)
    assert pf.stream is None
    assert [int(b["tokens"][0, 0]) for b in pf] == [0, 1, 2, 3, 4]


def test_the_host_batch_of_the_last_copy_is_kept_alive():
    pf, _ = _pf(_batches(3), 1)
    next(pf)
    assert int(pf._keepalive["tokens"][0, 0]) == 0
    next(pf)
    assert int(pf._keepalive["tokens"][0, 0]) == 1


# ---------------------------------------------------------------------------------------------
# profiler
# ---------------------------------------------------------------------------------------------
class _Clock:
    def __init__(self, tick_ms=1.0):
        self.t, self.tick = 0, int(tick_ms * 1e6)

    def __call__(self):
        self.t += self.tick
        return self.t


class _FakeCudaEvent:
    """Device-event stand-in: elapsed_time is only legal once both events have been 'reached'."""
    clock = 0.0
    synced = False

    def __init__(self):
        self.t = None

    def record(self):
        _FakeCudaEvent.clock += 2.5
        self.t = _FakeCudaEvent.clock

    def elapsed_time(self, other):
        assert _FakeCudaEvent.synced, "event resolved before the step's synchronisation"
        return other.t - self.t


def _step(p, step, names=("microbatches", "reduce_scatter", "grad_norm", "optimizer", "loss_allreduce", "allgather")):
    p.begin_step(step)
    for n in names:
        p.mark(n)
    p.end_step()


def test_the_main_loop_segment_names_are_the_schema():
    assert SEGMENTS == ("step_start", "microbatches", "reduce_scatter", "grad_norm", "optimizer",
                        "loss_allreduce", "allgather")
    assert DEEP_SEGMENTS == ("mb_data", "mb_fwd", "mb_ce", "mb_bwd", "mb_accum")


def test_range_is_half_open_and_records_only_inside(tmp_path):
    p = StepProfiler(2, 5, str(tmp_path / "p.json"), use_cuda=False, clock=_Clock())
    for s in range(8):
        _step(p, s)
    assert [r["step"] for r in p.records] == [2, 3, 4]
    assert all(set(r["segments_ms"]) == set(SEGMENTS[1:]) for r in p.records)


def test_device_events_are_resolved_only_in_end_step(tmp_path):
    _FakeCudaEvent.clock, _FakeCudaEvent.synced = 0.0, False
    p = StepProfiler(0, 1, str(tmp_path / "p.json"), use_cuda=True, event_factory=_FakeCudaEvent)
    p.begin_step(0)
    p.mark("microbatches")
    p.mark("optimizer")
    _FakeCudaEvent.synced = True                                # the loop's own synchronisation
    p.end_step()
    assert p.records[0]["segments_ms"] == {"microbatches": 2.5, "optimizer": 2.5}
    assert p.records[0]["total_ms"] == 5.0


def test_repeated_marks_of_one_name_add_up(tmp_path):
    p = StepProfiler(0, 1, str(tmp_path / "p.json"), use_cuda=False, clock=_Clock(), deep=True)
    p.begin_step(0)
    for _ in range(3):                                          # three micro-batches
        for n in DEEP_SEGMENTS:
            p.deep_mark(n)
    p.mark("microbatches")
    p.end_step()
    seg = p.records[0]["segments_ms"]
    assert all(seg[n] == pytest.approx(3.0) for n in DEEP_SEGMENTS)
    assert seg["microbatches"] == pytest.approx(1.0)
    assert p.records[0]["total_ms"] == pytest.approx(16.0)
    assert sum(seg.values()) == pytest.approx(p.records[0]["total_ms"])      # segments tile the step


def test_a_step_with_no_mark_after_the_start_leaves_no_record(tmp_path):
    p = StepProfiler(0, 2, str(tmp_path / "p.json"), use_cuda=False, clock=_Clock())
    p.begin_step(0)
    p.end_step()
    assert p.records == [] and p.active is False
    _step(p, 1)
    assert [r["step"] for r in p.records] == [1]


def test_marks_outside_a_step_or_after_end_step_are_ignored(tmp_path):
    p = StepProfiler(0, 2, str(tmp_path / "p.json"), use_cuda=False, clock=_Clock())
    p.mark("microbatches")                                      # before any begin_step
    _step(p, 0)
    p.mark("optimizer")                                         # between steps
    p.deep_mark("mb_fwd")
    assert len(p.records) == 1 and "mb_fwd" not in p.records[0]["segments_ms"]
    p.end_step()                                                # a second end is harmless
    assert len(p.records) == 1


def test_begin_step_drops_the_marks_of_an_unfinished_step(tmp_path):
    p = StepProfiler(0, 3, str(tmp_path / "p.json"), use_cuda=False, clock=_Clock())
    p.begin_step(0)
    p.mark("microbatches")                                      # the step raised: no end_step
    _step(p, 1, names=("optimizer",))
    assert [r["step"] for r in p.records] == [1]
    assert set(p.records[0]["segments_ms"]) == {"optimizer"}


def test_host_timer_adds_host_intervals_next_to_the_device_ones(tmp_path):
    p = StepProfiler(0, 1, str(tmp_path / "p.json"), use_cuda=False, clock=_Clock(), host_timer=True)
    _step(p, 0, names=("microbatches", "optimizer"))
    rec = p.records[0]
    assert set(rec["host_ms"]) == {"microbatches", "optimizer"}
    assert all(v > 0 for v in rec["host_ms"].values())
    q = StepProfiler(0, 1, str(tmp_path / "q.json"), use_cuda=False, clock=_Clock())
    _step(q, 0)
    assert "host_ms" not in q.records[0]


def test_summary_statistics(tmp_path):
    class Scripted:
        def __init__(self, stamps):
            self.it = iter(stamps)

        def __call__(self):
            return next(self.it)
    # five steps, one segment of 1, 2, 3, 4 and 10 ms
    stamps = []
    t = 0
    for d in (1, 2, 3, 4, 10):
        stamps += [t, t + d * 1_000_000]
        t += 100_000_000
    p = StepProfiler(0, 5, str(tmp_path / "p.json"), use_cuda=False, clock=Scripted(stamps))
    for s in range(5):
        _step(p, s, names=("optimizer",))
    st = p.summary()["optimizer"]
    assert st["n"] == 5 and st["mean"] == pytest.approx(4.0) and st["median"] == pytest.approx(3.0)
    assert st["p90"] == pytest.approx(10.0) and st["total"] == pytest.approx(20.0)
    assert st["std"] == pytest.approx((sum((x - 4) ** 2 for x in (1, 2, 3, 4, 10)) / 5) ** 0.5)
    assert p.summary()["total"]["n"] == 5
    one = StepProfiler(0, 1, str(tmp_path / "o.json"), use_cuda=False, clock=_Clock())
    _step(one, 0, names=("optimizer",))
    assert one.summary()["optimizer"]["std"] == 0.0


def test_module_level_summaries_work_on_any_subset_of_the_records(tmp_path):
    from forgetrain_b200.utils.profiler import summarize_host_phases, summarize_segments
    p = StepProfiler(0, 4, str(tmp_path / "p.json"), use_cuda=False, clock=_Clock(), host_timer=True)
    for s in range(4):
        _step(p, s, names=("microbatches", "optimizer"))
    assert summarize_segments([]) == {} and summarize_host_phases([]) == {}
    assert summarize_segments(p.records) == p.summary()
    tail = summarize_segments(p.records[2:])                    # e.g. without the warm-up steps
    assert tail["optimizer"]["n"] == 2 and tail["total"]["n"] == 2
    host = summarize_host_phases(p.records)
    assert set(host) == {"microbatches", "optimizer"} and host["optimizer"]["n"] == 4
    doc = json.loads(open(p.write()).read())
    assert doc["host_summary"]["optimizer"]["n"] == 4
    assert summarize_host_phases([{"step": 0, "segments_ms": {"a": 1.0}, "total_ms": 1.0}]) == {}


def test_write_is_atomic_creates_directories_and_is_rank_zero_only(tmp_path):
    out = tmp_path / "a" / "b" / "prof.json"
    p = StepProfiler(0, 1, str(out), use_cuda=False, clock=_Clock(), deep=True)
    _step(p, 0)
    assert p.write() == str(out)
    doc = json.loads(out.read_text())
    assert doc["deep_mode"] is True and doc["records"][0]["step"] == 0
    assert not list(tmp_path.rglob("*.tmp"))
    p.write()                                                   # rewriting replaces the file
    assert json.loads(out.read_text())["summary"]["total"]["n"] == 1
    other = StepProfiler(0, 1, str(tmp_path / "r1.json"), use_cuda=False, rank=3)
    _step(other, 0)
    assert other.write() is None and not (tmp_path / "r1.json").exists()


def test_an_empty_profile_still_writes_a_valid_document(tmp_path):
    p = StepProfiler(5, 6, str(tmp_path / "p.json"), use_cuda=False)
    _step(p, 0)
    doc = json.loads(open(p.write()).read())
    assert doc["records"] == [] and doc["summary"] == {} and doc["range"] == [5, 6]


def test_constructor_rejects_an_empty_range(tmp_path):
    with pytest.raises(ValueError):
        StepProfiler(3, 3, str(tmp_path / "p.json"), use_cuda=False)
    with pytest.raises(ValueError):
        StepProfiler(4, 2, str(tmp_path / "p.json"), use_cuda=False)


def test_the_checkpoint_position_counts_dropped_batches_but_not_the_read_ahead():
    """A resumed source must continue right after the last batch the model saw: batches the
    prefetcher dropped on the way there have been passed, batches it has only read ahead have not."""
    pf, _ = _pf(_batches(10, masked={1, 2, 6}), 3)
    assert pf.consumed_from_source == 0
    seen = []
    for _ in range(4):
        b = next(pf)
        seen.append((int(b["tokens"][0, 0]), pf.consumed_from_source))
    #   batch 0 is item 1 of the source; batch 3 comes after two dropped ones: item 4; ...
    assert seen == [(0, 1), (3, 4), (4, 5), (5, 6)]
    assert pf.drawn > pf.consumed_from_source                   # the read-ahead is further along
