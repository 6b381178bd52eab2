import json
import types

import pytest
import torch

from forgetrain_b200.ckpt import checkpoint as ck
from forgetrain_b200.ckpt.convert_to_hf import (convert, hf_config, merge_qkv_interleaved,
                                                  split_qkv_interleaved, to_hf_state_dict)
from forgetrain_b200.config import load_model_spec
from forgetrain_b200.data.hf_dataloader import (PackedTokenLoader, build_hf_dataloader,
                                                 pack_token_stream)
from forgetrain_b200.models.params import ParamStore
from forgetrain_b200.parallel.topology import Topology


def _spec(tie=False):
    return load_model_spec("tiny", num_layers=2, vocab_size=128, hidden_size=128, ffn_hidden_size=256,
                           num_attention_heads=4, num_query_groups=2, head_dim=32, tie_embeddings=tie)


def test_qkv_split_is_per_group_and_invertible():
    spec = _spec()
    G, g, D, H = 2, 2, 32, 128
    w = torch.arange(spec.qkv_dim * H, dtype=torch.float32).view(spec.qkv_dim, H)
    q, k, v = split_qkv_interleaved(w, spec)
    assert q.shape == (G * g * D, H) and k.shape == (G * D, H) and v.shape == (G * D, H)
    # group 1's first q row sits after group 0's (g + 2) heads
    assert torch.equal(q[g * D], w[(g + 2) * D])
    assert torch.equal(k[0], w[g * D]) and torch.equal(v[0], w[(g + 1) * D])
    assert torch.equal(merge_qkv_interleaved(q, k, v, spec), w)


@pytest.mark.parametrize("tie", [False, True])
def test_export_writes_safetensors_and_config(tmp_path, tie):
    from safetensors.torch import load_file
    spec = _spec(tie)
    st = ParamStore(spec, "cpu", torch.float32)
    st.init_random(0)
    names = [p.name for p in st.specs]
    ck.save_checkpoint(tmp_path, 5, params={n: st.params[n] for n in names}, param_names=names,
                       optimizer_state=None, async_io=False)
    spec_path = tmp_path / "spec.toml"
    spec_path.write_text(
        "[model]\nname='t'\nvocab_size=128\nhidden_size=128\nnum_layers=2\nnum_attention_heads=4\n"
        "num_query_groups=2\nhead_dim=32\nffn_hidden_size=256\nseq_length=64\n"
        "max_position_embeddings=64\nnorm_epsilon=1e-6\nrotary_base=10000.0\ninit_method_std=0.02\n")
    out = convert(str(tmp_path / "step_0000005"), str(tmp_path / "hf"), model=str(spec_path), dtype="float32")
    sd = load_file(str(out / "model.safetensors"))
    cfg = json.loads((out / "config.json").read_text())
    assert cfg["architectures"] == ["MiniCPMForCausalLM"] and cfg["tie_word_embeddings"] is tie
    assert cfg["scale_emb"] == 12.0 and cfg["dim_model_base"] == 256 and cfg["scale_depth"] == 1.4
    assert cfg["num_key_value_heads"] == 2 and cfg["rms_norm_eps"] == 1e-6
    assert "lm_head.weight" in sd                   # always written, like the reference script
    assert cfg["auto_map"]["AutoModelForCausalLM"] == "modeling_minicpm.MiniCPMForCausalLM"
    assert cfg["initializer_range"] == 0.1
    gate = sd["model.layers.1.mlp.gate_proj.weight"]
    assert torch.equal(gate, st.params["layers.1.feed_forward.wfc1.weight"][:256])
    assert torch.equal(sd["model.layers.0.self_attn.o_proj.weight"], st.params["layers.0.attention.wo.weight"])
    assert len(sd) == 2 + 9 * 2 + 1


def test_packing_and_loader_cursor():
    rows = pack_token_stream([[1, 2, 3], [4, 5], [6, 7, 8, 9]], eos_id=0, seq_length=3)
    assert rows.tolist() == [[1, 2, 3, 0], [4, 5, 0, 6], [7, 8, 9, 0]]
    ld = PackedTokenLoader(rows, 2)
    b = next(ld)
    assert b["tokens"].tolist() == [[1, 2, 3], [4, 5, 0]] and b["labels"].tolist() == [[2, 3, 0], [5, 0, 6]]
    assert b["loss_mask"].sum() == 6
    st = ld.state_dict()
    nxt = next(ld)
    ld2 = PackedTokenLoader(rows, 2)
    ld2.load_state_dict(st)
    assert torch.equal(next(ld2)["tokens"], nxt["tokens"])
    with pytest.raises(ValueError):
        pack_token_stream([[1]], eos_id=0, seq_length=8)


def test_build_loader_with_injected_tokenizer_and_rank_sharding():
    class Tok:
        eos_token_id = 9

        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [ord(c) % 50 + 10 for c in text]}
    data = [{"text": "abcdefgh" * 4} for _ in range(8)]
    args = types.SimpleNamespace(hf_text_field="text", hf_text_template=None, max_packed_rows=None,
                                 tokenizer_path=None, hf_data_files=None)
    spec = _spec()
    a = build_hf_dataloader(args, spec, 1, 16, Topology(dp_size=2, dp_rank=0), tokenizer=Tok(), dataset=data)
    b = build_hf_dataloader(args, spec, 1, 16, Topology(dp_size=2, dp_rank=1), tokenizer=Tok(), dataset=data)
    assert a.rows.shape[1] == 17 and a.rows.shape[0] == b.rows.shape[0] > 0
    assert int(a.rows.max()) < spec.vocab_size


def test_text_field_detection_and_multi_column_rendering():
    from forgetrain_b200.data.hf_dataloader import detect_text_fields, render_text

    class DS(list):
        column_names = ["id", "content", "title"]
    assert detect_text_fields(DS()) == ["content"]
    rows = [{"id": 3, "question": "q?", "answer": "a."}]
    assert detect_text_fields(rows) == ["question", "answer"]
    with pytest.raises(ValueError, match="hf-text-field"):
        detect_text_fields([{"id": 1, "n": 2}])
    assert render_text(rows[0], ["question", "answer"], None) == "q?\na."
    assert render_text({"question": "q?", "answer": ""}, ["question", "answer"], None) == "q?"
    assert render_text(rows[0], "question", None) == "q?"
    assert render_text(rows[0], None, "Q: {question} A: {answer}") == "Q: q? A: a."


@pytest.mark.parametrize("tp,heads", [(2, 4), (4, 8)])
def test_tp_shards_merge_back_to_the_full_tensors(tp, heads):
    """shard_for_tp / unshard_from_tp are inverses, also when the TP degree exceeds the number of
    KV groups (q heads split, k / v replicated) and the vocabulary shards are padded."""
    from forgetrain_b200.models.params import all_param_specs, merge_tp_shards, shard_for_tp
    spec = load_model_spec("tiny", num_layers=1, vocab_size=130, hidden_size=128, ffn_hidden_size=256,
                           num_attention_heads=heads, num_query_groups=2, head_dim=32, tie_embeddings=False)
    g = torch.Generator().manual_seed(0)
    full = {ps.name: torch.randn(ps.shape, generator=g) for ps in all_param_specs(spec)}
    shards = [{ps.name: shard_for_tp(ps, full[ps.name], spec, r, tp) for ps in all_param_specs(spec)}
              for r in range(tp)]
    assert shards[0]["output.weight"].shape[0] * tp >= 130          # padded vocabulary rows
    merged = merge_tp_shards(spec, shards)
    assert set(merged) == set(full)
    for name, t in full.items():
        assert torch.equal(merged[name], t), name


def test_export_from_tensor_parallel_rank_files(tmp_path):
    """``rank_<R>.pt`` shards of a TP run export to the same HF weights as the unsharded model."""
    from safetensors.torch import load_file
    from forgetrain_b200.models.params import shard_for_tp
    spec = _spec()
    st = ParamStore(spec, "cpu", torch.float32)
    st.init_random(0)
    d = tmp_path / "step_0000003"
    d.mkdir()
    for r in range(2):
        params = {ps.name: shard_for_tp(ps, st.params[ps.name], spec, r, 2).clone() for ps in st.specs}
        torch.save({"format_version": 1, "step": 3, "params": params, "tp_size": 2, "tp_rank": r},
                   d / f"rank_{r}.pt")
    spec_path = tmp_path / "spec.toml"
    spec_path.write_text(
        "[model]\nname='t'\nvocab_size=128\nhidden_size=128\nnum_layers=2\nnum_attention_heads=4\n"
        "num_query_groups=2\nhead_dim=32\nffn_hidden_size=256\nseq_length=64\n"
        "max_position_embeddings=64\nnorm_epsilon=1e-6\nrotary_base=10000.0\ninit_method_std=0.02\n")
    out = convert(str(d), str(tmp_path / "hf"), model=str(spec_path), dtype="float32")
    sd = load_file(str(out / "model.safetensors"))
    want, _ = to_hf_state_dict({n: st.params[n] for n in st.offsets}, spec, torch.float32)
    assert set(sd) == set(want)
    for k in want:
        assert torch.equal(sd[k], want[k]), k
    (d / "rank_1.pt").unlink()
    with pytest.raises(ValueError, match="rank files"):
        convert(str(d), str(tmp_path / "hf2"), model=str(spec_path), dtype="float32")


def test_shuffled_loader_permutes_each_pass_and_resumes_from_the_batch_count():
    rows = torch.arange(10).view(10, 1).repeat(1, 3)          # row i = [i, i, i]
    ld = PackedTokenLoader(rows, 2, shuffle=True, seed=7)
    first = [int(t) for _ in range(5) for t in next(ld)["tokens"][:, 0]]
    second = [int(t) for _ in range(5) for t in next(ld)["tokens"][:, 0]]
    assert sorted(first) == sorted(second) == list(range(10))     # every pass sees every row once
    assert first != list(range(10)) and first != second           # ... in its own order
    again = PackedTokenLoader(rows, 2, shuffle=True, seed=7)
    assert [int(t) for _ in range(5) for t in next(again)["tokens"][:, 0]] == first
    other = PackedTokenLoader(rows, 2, shuffle=True, seed=8)      # another rank: another order
    assert [int(t) for _ in range(5) for t in next(other)["tokens"][:, 0]] != first
    # resume in the middle of the second pass
    st = None
    ld = PackedTokenLoader(rows, 2, shuffle=True, seed=7)
    for _ in range(7):
        next(ld)
    st = ld.state_dict()
    want = next(ld)["tokens"]
    ld2 = PackedTokenLoader(rows, 2, shuffle=True, seed=7)
    ld2.load_state_dict(st)
    assert torch.equal(next(ld2)["tokens"], want)
    # unshuffled: sequential with wrap-around, as before
    seq = PackedTokenLoader(rows, 4)
    assert [int(t) for _ in range(3) for t in next(seq)["tokens"][:, 0]] == [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 0, 1]


def test_document_relative_positions():
    from forgetrain_b200.data.hf_dataloader import doc_position_ids
    t = torch.tensor([[5, 6, 0, 7, 8, 9, 0, 0, 4],
                      [0, 1, 2, 3, 4, 5, 6, 7, 8]])
    assert doc_position_ids(t, 0).tolist() == [[0, 1, 2, 0, 1, 2, 3, 0, 0],
                                               [0, 0, 1, 2, 3, 4, 5, 6, 7]]
    rows = torch.tensor([[5, 6, 0, 7, 8, 9, 0, 0, 4, 3]], dtype=torch.int32)
    b = next(PackedTokenLoader(rows, 1, doc_positions_eos=0))
    assert b["position_ids"].dtype == torch.int32 and b["position_ids"].shape == b["tokens"].shape
    assert "position_ids" not in next(PackedTokenLoader(rows, 1))


def test_streaming_loader_visits_every_document_each_pass_and_resumes_mid_document():
    from forgetrain_b200.data.hf_dataloader import StreamingTokenLoader
    docs = {i: [100 + i] * (3 + i % 4) for i in range(12)}          # doc i = its own id repeated
    docs[5] = []                                                     # an empty document is skipped
    mk = lambda **kw: StreamingTokenLoader(12, lambda i: docs[i], 0, 2, 7, seed=3, **kw)
    ld = mk(dp_rank=1, dp_size=2)                                    # odd documents only
    seen, stream = set(), []
    for _ in range(6):
        b = next(ld)
        assert b["tokens"].shape == (2, 7) and torch.equal(b["labels"][:, :-1], b["tokens"][:, 1:])
        stream += [int(t) for row in torch.cat([b["tokens"], b["labels"][:, -1:]], 1) for t in row]
    seen = {t - 100 for t in stream if t >= 100}
    assert seen == {1, 3, 7, 9, 11}                                  # rank's slice, 5 is empty
    first_pass = [t for t in stream if t != 0][:sum(len(docs[i]) for i in (1, 3, 7, 9, 11))]
    order = list(dict.fromkeys(first_pass))
    assert sorted(order) == [101, 103, 107, 109, 111] and order != [101, 103, 107, 109, 111]
    # resume: same continuation from the saved state, in the middle of a document
    a = mk()
    for _ in range(3):
        next(a)
    st = a.state_dict()
    want = [next(a)["tokens"] for _ in range(3)]
    b2 = mk()
    b2.load_state_dict(st)
    assert all(torch.equal(next(b2)["tokens"], w) for w in want)
    with pytest.raises(ValueError, match="no tokens"):
        next(StreamingTokenLoader(3, lambda i: [], 0, 1, 4))


def test_streaming_loader_checkpoint_ignores_prefetch_read_ahead(tmp_path):
    """A run on the streaming loader, saved while the prefetcher had drawn two batches ahead,
    resumes on exactly the batch the model would have seen next."""
    from forgetrain_b200.data.hf_dataloader import StreamingTokenLoader
    from forgetrain_b200.engine_config import from_spec
    from forgetrain_b200.trainer import run_training_loop
    spec = load_model_spec("tiny")
    g = torch.Generator().manual_seed(0)
    docs = [torch.randint(1, spec.vocab_size, (int(n),), generator=g).tolist()
            for n in torch.randint(20, 90, (40,), generator=g)]
    mk = lambda: StreamingTokenLoader(len(docs), lambda i: docs[i], 0, 1, 32, seed=1)
    cfg = from_spec(spec, dtype="fp32", comm="nccl", warmup_iters=0, data_prefetch_depth=2)
    kw = dict(spec=spec, cfg=cfg, topo=Topology(), micro_batch_size=1, seq_length=32, seed=0)
    full = run_training_loop(num_steps=4, data_source=mk(), save_dir=str(tmp_path / "ck"),
                             save_interval=2, **kw)
    rest = run_training_loop(num_steps=2, data_source=mk(), resume=str(tmp_path / "ck" / "step_0000002"),
                             **kw)
    assert [s["loss"] for s in rest["steps"]] == pytest.approx([s["loss"] for s in full["steps"]][2:],
                                                               abs=1e-6)


def test_a_huggingface_folder_loads_back_into_the_engine(tmp_path):
    """Export, then start a new trainer from the exported folder: same parameters (bf16 export of
    bf16-representable values is exact), same loss on the same batch, optimizer moments at zero;
    a folder of another architecture is refused."""
    from forgetrain_b200.ckpt import hf_import
    from forgetrain_b200.ckpt.convert_to_hf import convert
    from forgetrain_b200.engine_config import from_spec
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    spec = load_model_spec("tiny", tie_embeddings=False)
    cfg = from_spec(spec, dtype="fp32", comm="nccl")
    a = Trainer(spec, cfg, Topology(), seq_length=32, micro_batch_size=2, seed=3)
    a.store.flat_params.copy_(a.store.flat_params.to(torch.bfloat16).float())   # representable in bf16
    a.opt.sync_master_from_params()
    a.save(tmp_path / "run", 1, async_io=False)
    out = convert(str(tmp_path / "run" / "step_0000001"), str(tmp_path / "hf"), "tiny")
    assert hf_import.is_hf_folder(out) and not hf_import.is_hf_folder(tmp_path / "run")
    b = Trainer(spec, cfg, Topology(), seq_length=32, micro_batch_size=2, seed=99)
    st = b.load(out)
    assert st["step"] == 0 and not b.opt.exp_avg.any()
    for name in a.store.offsets:
        assert torch.equal(a.store.params[name], b.store.params[name]), name
    g = torch.Generator().manual_seed(0)
    c = torch.randint(0, spec.vocab_size, (2, 33), generator=g)
    batch = [{"tokens": c[:, :-1].contiguous(), "labels": c[:, 1:].contiguous(), "loss_mask": torch.ones(2, 32)}]
    assert float(a.train_step(batch)["loss"]) == float(b.train_step(batch)["loss"])
    other = load_model_spec("tiny", tie_embeddings=False, num_layers=2)
    with pytest.raises(ValueError, match="num_hidden_layers"):
        hf_import.load_hf_folder(out, other)
    # a folder whose output table differs from its embedding cannot feed a run with tied tables
    from forgetrain_b200.ckpt.convert_to_hf import to_hf_state_dict
    tied = load_model_spec("tiny", tie_embeddings=True)
    t = Trainer(tied, from_spec(tied, dtype="fp32", comm="nccl"), Topology(), seq_length=32,
                micro_batch_size=2, seed=3)
    sd, was_tied = to_hf_state_dict({n: t.store.params[n] for n in t.store.offsets}, tied, torch.float32)
    assert was_tied and "output.weight" not in hf_import.from_hf_state_dict(sd, tied)
    sd["lm_head.weight"] = sd["lm_head.weight"] + 1
    with pytest.raises(ValueError, match="ties the two tables"):
        hf_import.from_hf_state_dict(sd, tied)


def _word_tokenizer(folder, words):
    """A word-level tokenizer saved the way ``AutoTokenizer.from_pretrained`` reads it."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    vocab = {"<unk>": 0, "<s>": 1, "</s>": 2, **{w: i + 3 for i, w in enumerate(words)}}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", bos_token="<s>", eos_token="</s>")
    fast.save_pretrained(str(folder))
    return fast


def test_local_data_files_are_read_without_the_datasets_package(tmp_path):
    import json
    from forgetrain_b200.data.hf_dataloader import load_local_files
    (tmp_path / "a.jsonl").write_text("\n".join(json.dumps({"text": f"doc {i}", "id": i}) for i in range(3)) + "\n")
    (tmp_path / "b.json").write_text(json.dumps([{"text": "doc 3", "id": 3}]))
    (tmp_path / "c.txt").write_text("first line\nsecond line\n")
    (tmp_path / "d.csv").write_text("title,body\nt0,b0\nt1,b1\n")
    rows = load_local_files("json", f"{tmp_path}/a.jsonl,{tmp_path}/b.json")
    assert [r["id"] for r in rows] == [0, 1, 2, 3] and len(rows) == 4 and rows[2]["text"] == "doc 2"
    assert [r["text"] for r in load_local_files("text", str(tmp_path / "*.txt"))] == ["first line", "second line"]
    assert load_local_files("csv", str(tmp_path / "d.csv"))[1] == {"title": "t1", "body": "b1"}
    import pyarrow as pa
    import pyarrow.parquet as pq
    pq.write_table(pa.table({"text": ["p0", "p1"]}), tmp_path / "e.parquet")
    assert [r["text"] for r in load_local_files("parquet", str(tmp_path / "e.parquet"))] == ["p0", "p1"]
    with pytest.raises(FileNotFoundError):
        load_local_files("json", str(tmp_path / "nothing*.json"))
    with pytest.raises(ValueError, match="expected json"):
        load_local_files("arrow", str(tmp_path / "a.jsonl"))


def test_cli_trains_on_local_files_with_a_saved_tokenizer(tmp_path):
    """`--hf-data-files` + `--tokenizer-path` end to end on CPU, whether or not the `datasets`
    package is there: text column detected, documents tokenised, packed and trained on."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    words = [f"w{i}" for i in range(200)]
    _word_tokenizer(tmp_path / "tok", words)
    g = torch.Generator().manual_seed(0)
    with open(tmp_path / "corpus.jsonl", "w") as f:
        for _ in range(300):
            n = int(torch.randint(5, 60, (1,), generator=g))
            ids = torch.randint(0, 200, (n,), generator=g).tolist()
            f.write(json.dumps({"content": " ".join(words[i] for i in ids)}) + "\n")
    root = Path(__file__).resolve().parent.parent
    r = subprocess.run([sys.executable, "-m", "training_engine_tensor", "pretrain", "--model", "tiny", "--device", "cpu",
                        "--num-steps", "3", "--micro-batch-size", "2", "--global-batch-size", "2", "--seq-length", "64",
                        "--hf-dataset", "local", "--hf-data-files", str(tmp_path / "corpus.jsonl"),
                        "--hf-data-format", "json", "--tokenizer-path", str(tmp_path / "tok"),
                        "--random-init"], cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "text_fields=['content']" in r.stdout and "iteration        3" in r.stdout and "DONE" in r.stdout
    losses = [float(x) for x in __import__("re").findall(r"\| loss ([0-9.E+-]+)", r.stdout)]
    # 203 distinct token ids out of a 4096-entry vocabulary: the loss drops fast below ln(4096)
    assert len(losses) == 3 and losses[-1] < losses[0]


def test_per_rank_stream_states_are_packed_and_selected():
    from forgetrain_b200.data.hf_dataloader import pack_rank_states, select_rank_state
    states = [{"kind": "stream", "epoch": 1, "pos": 5 + r, "buf": [r], "batches_drawn": 9} for r in range(4)]
    packed = pack_rank_states(states)
    assert packed["kind"] == "per_rank" and packed["dp_size"] == 4
    assert select_rank_state(packed, 2, 4) == states[2]
    notes = []
    other = select_rank_state(packed, 1, 2, log=notes.append)
    assert other == {"kind": "stream", "epoch": 1, "pos": 0, "buf": [], "batches_drawn": 9}
    assert len(notes) == 1 and "4 data-parallel ranks" in notes[0]
    counted = pack_rank_states([{"kind": "packed", "batches_drawn": 7}, {"kind": "packed", "batches_drawn": 7}])
    assert select_rank_state(counted, 0, 1, log=notes.append) == {"kind": "packed", "batches_drawn": 7}
    assert len(notes) == 1                                      # no note: nothing is lost
    # states that are the same on every rank pass through untouched
    plain = {"kind": "packed", "batches_drawn": 7}
    assert select_rank_state(plain, 3, 8) is plain and select_rank_state(None, 0, 1) == {}


def test_streamed_documents_resume_on_every_data_parallel_rank(tmp_path):
    """Two ranks stream their own halves of a local corpus (`--hf-stream`); the checkpoint keeps one
    stream position per rank, so the resumed job sees exactly the batches the uninterrupted one saw
    (with rank 0's position on every rank, rank 1 would re-read other documents)."""
    import json
    import re
    import socket
    import subprocess
    import sys
    from pathlib import Path
    words = [f"w{i}" for i in range(300)]
    _word_tokenizer(tmp_path / "tok", words)
    g = torch.Generator().manual_seed(0)
    with open(tmp_path / "corpus.jsonl", "w") as f:
        for _ in range(400):
            n = int(torch.randint(5, 90, (1,), generator=g))
            f.write(json.dumps({"text": " ".join(words[i] for i in torch.randint(0, 300, (n,), generator=g).tolist())}) + "\n")
    root = Path(__file__).resolve().parent.parent

    def run(command, steps, *extra):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                            "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "training_engine_tensor",
                            command, "--model", "tiny", "--device", "cpu", "--dtype", "fp32", "--micro-batch-size", "2",
                            "--global-batch-size", "8", "--seq-length", "64", "--seed", "0", "--num-steps", str(steps),
                            "--hf-dataset", "local", "--hf-data-files", str(tmp_path / "corpus.jsonl"),
                            "--hf-data-format", "json", "--tokenizer-path", str(tmp_path / "tok"), "--hf-stream", *extra],
                           cwd=root, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        return {int(m.group(1)): float(m.group(2)) for m in re.finditer(r"iteration +(\d+) \| loss ([0-9.E+-]+)", r.stdout)}

    whole = run("pretrain", 5, "--random-init", "--save-dir", str(tmp_path / "run"), "--save-interval", "3")
    st = torch.load(tmp_path / "run" / "step_0000003" / "training_state.pt", weights_only=False)["dataloader_state"]
    assert st["kind"] == "per_rank" and st["dp_size"] == 2 and st["ranks"][0] != st["ranks"][1]
    resumed = run("train", 2, "--resume", str(tmp_path / "run" / "step_0000003"))
    assert resumed == {4: whole[4], 5: whole[5]}


def test_loader_builder_reads_local_files_itself_when_datasets_cannot_be_imported(tmp_path, monkeypatch, capsys):
    import json
    import sys

    class Tok:
        eos_token_id = 9

        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [ord(c) % 50 + 10 for c in text]}
    (tmp_path / "c.jsonl").write_text("\n".join(json.dumps({"body": "abcdefgh" * 6}) for _ in range(6)) + "\n")
    monkeypatch.setitem(sys.modules, "datasets", None)          # `import datasets` now raises ImportError
    args = types.SimpleNamespace(hf_text_field=None, hf_text_template=None, max_packed_rows=None,
                                 tokenizer_path=None, hf_data_files=str(tmp_path / "c.jsonl"),
                                 hf_data_format="json", hf_dataset="local", hf_dataset_split="train",
                                 hf_dataset_config=None)
    loader = build_hf_dataloader(args, _spec(), 1, 16, Topology(), tokenizer=Tok())
    out = capsys.readouterr().out
    assert "`datasets` is not installed: read 6 rows" in out and "text_fields=['body']" in out
    assert loader.rows.shape[1] == 17 and loader.rows.shape[0] >= 6
    args.hf_data_files = None                                   # a hub dataset does need the package
    with pytest.raises(SystemExit, match="datasets"):
        build_hf_dataloader(args, _spec(), 1, 16, Topology(), tokenizer=Tok())


def test_every_parameter_survives_shard_and_unshard_for_random_geometries():
    """Property: for any head / group / degree combination the engine accepts (also degrees above
    the KV groups, and vocabularies so small that the last ranks hold padding only), the shards have
    the advertised local shape and merge back to the full tensor exactly."""
    from hypothesis import given, settings, strategies as hst
    from forgetrain_b200.models.params import all_param_specs, local_shape, shard_for_tp, unshard_from_tp

    @settings(max_examples=120, deadline=None, derandomize=True)
    @given(groups=hst.sampled_from([1, 2, 4]), per_group=hst.sampled_from([1, 2, 4, 8]),
           tp=hst.sampled_from([1, 2, 4, 8]), vocab=hst.integers(40, 300), tie=hst.booleans())
    def check(groups, per_group, tp, vocab, tie):
        if tp > groups and (tp % groups or per_group % (tp // groups)):
            return
        if tp <= groups and groups % tp:
            return
        spec = load_model_spec("tiny", num_layers=1, vocab_size=vocab, hidden_size=32, ffn_hidden_size=16 * tp,
                               num_attention_heads=groups * per_group, num_query_groups=groups, head_dim=8,
                               tie_embeddings=tie)
        g = torch.Generator().manual_seed(0)
        for ps in all_param_specs(spec):
            full = torch.randn(ps.shape, generator=g)
            parts = [shard_for_tp(ps, full, spec, r, tp) for r in range(tp)]
            assert all(tuple(p.shape) == tuple(local_shape(ps, spec, tp)) for p in parts), ps.name
            assert torch.equal(unshard_from_tp(ps, parts, spec), full), ps.name

    check()
