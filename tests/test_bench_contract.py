"""The parts of ``bench.py`` that run without a GPU: the reference arm's "unavailable" line, the
clock record parsed from nvidia-smi's CSV, the local corpus written for the reference's command
line, and the documented defaults of the command line."""
import importlib.util
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_one_json_line_and_exits_zero():
    """Whatever the box offers, ``--impl reference`` ends with ONE JSON line that carries
    ``impl: reference`` and either a measurement or the reason it cannot be taken, and exit 0."""
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, RANK="0"))
    assert out.returncode == 0, out.stderr[-400:]
    lines = [l for l in out.stdout.strip().splitlines() if l.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference"
    assert ("unavailable" in rec and isinstance(rec["unavailable"], str) and rec["unavailable"]) or \
        (rec.get("metric") == "tokens_per_sec" and rec["value"] > 0)


def test_clock_record_from_nvidia_smi_csv():
    b = _bench()
    s = b.ClockSampler(0)
    s.proc = type("P", (), {"terminate": lambda self: None, "wait": lambda self, timeout=None: 0,
                            "kill": lambda self: None})()
    s.lines = ["0, 1650, 1965, 980.5, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "0, 1590, 1965, 991.2, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "0, 1710, 1965, 870.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active",
               "garbage line", "0, [N/A], 1965, 1, x, a, b, c, d"]
    rec = s.stop()
    assert rec["sm_mhz"] == 1650 and rec["sm_max_mhz"] == 1965 and rec["samples"] == 3
    assert rec["reasons"] == ["sw_power_cap"] and rec["power_w_max"] == 991.2
    # a thermal reason is reported by name so that the reader of the line can reject the run
    s.lines = ["0, 1200, 1965, 700, x, Not Active, Active, Not Active, Not Active"]
    assert s.stop()["reasons"] == ["hw_thermal_slowdown"]
    # no nvidia-smi at all
    t = b.ClockSampler(0)
    assert t.stop()["reasons"] == ["nvidia-smi unavailable"]


def test_reference_corpus_and_tokenizer_are_written_locally(tmp_path):
    """The reference's CLI loads its data with ``datasets.load_dataset(<--hf-dataset>, split="train")``
    and its tokenizer with ``AutoTokenizer.from_pretrained(<--tokenizer-path>)`` (0.5B
    hf_dataloader.py:28-60,228-234): both calls must work on what the arm writes."""
    import pytest
    b = _bench()
    b._write_reference_corpus(str(tmp_path), seq=32, rows=5)
    rows = [json.loads(l) for l in (tmp_path / "data" / "corpus.jsonl").read_text().splitlines()]
    assert len(rows) == 5 and all(len(r["text"].split()) == 40 for r in rows)
    assert sorted(p.name for p in (tmp_path / "data").iterdir()) == ["corpus.jsonl"]
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(str(tmp_path / "tok"), trust_remote_code=True)
    ids = tok(rows[0]["text"], add_special_tokens=False)["input_ids"]
    assert len(ids) == 40 and min(ids) >= 2          # every word is in the vocabulary
    assert tok.eos_token == "</s>" and tok.eos_token_id == 1
    datasets = pytest.importorskip("datasets")
    ds = datasets.load_dataset(str(tmp_path / "data"), name=None, split="train")
    assert len(ds) == 5 and ds.column_names == ["text"] and ds[0]["text"] == rows[0]["text"]


def test_reference_arm_uses_the_flags_of_the_reference_command_line():
    src = (ROOT / "bench.py").read_text()
    assert '"--tokenizer-path"' in src and "--hf-tokenizer" not in src
    assert '"--hf-dataset", os.path.join(work, "data")' in src


def test_command_line_defaults_match_the_documented_contract():
    """No flags: one GPU, at least three warm-up steps, a step count that ends within minutes."""
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True,
                         text=True, timeout=120)
    assert out.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--comm", "--graph", "--secondary"):
        assert flag in out.stdout
    b = _bench()
    assert b.SEQ == 4096 and b.MBS == 4 and b.METRIC == "tokens_per_sec"
    assert b.PUBLISHED_MFU["0.5b"] == 0.4413 and b.NOMINAL_BF16_TFLOPS == 2250.0
