import json

import pytest

from forgetrain_b200.engine_config import EngineConfig
from forgetrain_b200.utils.profiler import StepProfiler, parse_profile_range, profiler_from_config


class Clock:
    def __init__(self):
        self.t = 0

    def __call__(self):
        self.t += 1_000_000     # 1 ms per reading
        return self.t


def test_closing_mark_segments_and_summary(tmp_path):
    out = tmp_path / "prof.json"
    p = StepProfiler(1, 3, str(out), use_cuda=False, clock=Clock())
    for step in range(4):
        p.begin_step(step)
        p.mark("microbatches")
        p.mark("reduce_scatter")
        p.mark("optimizer")
        p.end_step()
    assert [r["step"] for r in p.records] == [1, 2]
    assert set(p.records[0]["segments_ms"]) == {"microbatches", "reduce_scatter", "optimizer"}
    assert p.records[0]["segments_ms"]["optimizer"] == pytest.approx(1.0)
    assert p.records[0]["total_ms"] == pytest.approx(3.0)
    path = p.write()
    doc = json.loads(open(path).read())
    assert doc["schema_version"] == 2 and doc["range"] == [1, 3] and doc["deep_mode"] is False
    assert set(doc["summary"]["total"]) == {"n", "mean", "median", "p90", "std", "total"}
    assert doc["summary"]["total"]["n"] == 2


def test_inactive_outside_range_and_rank_filter(tmp_path):
    p = StepProfiler(5, 6, str(tmp_path / "x.json"), use_cuda=False, rank=1)
    p.begin_step(0)
    p.mark("a")
    p.end_step()
    assert p.records == [] and p.write() is None


def test_range_parsing_and_both_or_neither():
    assert parse_profile_range("2, 5") == (2, 5)
    for bad in ("3", "5,2", "-1,2", "a,b"):
        with pytest.raises(ValueError):
            parse_profile_range(bad)
    assert profiler_from_config(EngineConfig()) is None
    cfg = EngineConfig(profile_range="0,2", profile_output="o.json", profile_deep=True)
    pr = profiler_from_config(cfg)
    assert pr.deep and (pr.start, pr.end) == (0, 2)


def test_deep_marks_only_in_deep_mode(tmp_path):
    p = StepProfiler(0, 1, str(tmp_path / "d.json"), use_cuda=False, clock=Clock(), deep=False)
    p.begin_step(0)
    p.deep_mark("mb_fwd")
    p.mark("microbatches")
    p.end_step()
    assert "mb_fwd" not in p.records[0]["segments_ms"]
