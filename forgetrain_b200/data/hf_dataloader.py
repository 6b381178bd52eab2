"""HuggingFace dataset -> packed token batches.

``datasets.load_dataset`` (or local ``--hf-data-files`` in ``json`` / ``text`` / ``parquet``
format) -> tokenizer -> EOS-joined token stream -> fixed ``seq + 1`` chunks -> ``tokens =
chunk[:-1]``, ``labels = chunk[1:]``, ``loss_mask = 1``. Documents are sharded ``rank::world``
over the data-parallel ranks; the tokenizer is loaded rank by rank so a cold cache is written
once. ``max_packed_rows`` caps the pre-tokenised rows kept in memory. Behavioural spec:
exports/train_engine_0.5B/src/training_engine_tensor/hf_dataloader.py:28-269 and
exports/train_engine_8b/src/training_engine_tensor/hf_dataloader.py:42-469.
"""
from __future__ import annotations

from typing import Iterable, Iterator

import torch


def pack_token_stream(docs: Iterable[list[int]], eos_id: int, seq_length: int,
                      max_rows: int | None = None) -> torch.Tensor:
    """Join documents with EOS and cut the stream into rows of ``seq_length + 1`` tokens.

    The whole slice is tokenised once, up front, into one int32 array (4 bytes per token), so that
    drawing a batch is an index operation (the 8B engine's preload mode, hf_dataloader.py:159-237)."""
    import numpy as np
    row = seq_length + 1
    want = max_rows * row if max_rows else None
    parts: list = []
    total = 0
    for d in docs:
        a = np.empty(len(d) + 1, dtype=np.int32)
        a[:-1] = d
        a[-1] = eos_id
        parts.append(a)
        total += a.size
        if want is not None and total >= want:
            break
    n_rows = total // row
    if max_rows:
        n_rows = min(n_rows, max_rows)
    if n_rows == 0:
        raise ValueError("dataset too small: not a single full sequence could be packed")
    flat = np.concatenate(parts)[:n_rows * row]
    return torch.from_numpy(flat.reshape(n_rows, row).copy())


def doc_position_ids(tokens: torch.Tensor, eos_id: int) -> torch.Tensor:
    """Positions that restart after every EOS of a packed row (``[rows, seq]`` int32): the input
    of the document-aware RoPE (reference: ``position_ids`` in 0.5B data.py:93-107 and the
    per-(s, b) rotary branch of forward.py:97-103)."""
    S = tokens.shape[1]
    idx = torch.arange(S, dtype=torch.int64).expand_as(tokens)
    starts = torch.zeros_like(tokens, dtype=torch.bool)
    starts[:, 0] = True
    starts[:, 1:] = tokens[:, :-1] == eos_id
    last_start = torch.where(starts, idx, torch.zeros_like(idx)).cummax(dim=1).values
    return (idx - last_start).to(torch.int32)


class PackedTokenLoader:
    """Cycles over pre-packed rows in micro-batches. With ``shuffle`` every pass over the rows
    uses its own permutation, drawn from ``seed`` and the pass number (the 8B engine shuffles
    packed rows per epoch, hf_dataloader.py:93-118), so the position in the stream is a pure
    function of the number of batches drawn and that number is the only state to checkpoint."""

    def __init__(self, rows: torch.Tensor, micro_batch_size: int, pin: bool = False,
                 shuffle: bool = False, seed: int = 0, doc_positions_eos: int | None = None):
        if rows.shape[0] < micro_batch_size:
            raise ValueError(f"only {rows.shape[0]} packed rows for micro-batch {micro_batch_size}")
        self.rows, self.mbs, self.pin = rows, micro_batch_size, pin
        self.shuffle, self.seed = shuffle, seed
        self.doc_positions_eos = doc_positions_eos     # not None: add document-relative positions
        self.cursor = 0
        self.batches_drawn = 0
        self._perm_epoch = -1
        self._perm: torch.Tensor | None = None

    def __iter__(self) -> Iterator[dict]:
        return self

    def _row_index(self, k: int) -> int:
        """Row of the ``k``-th sample of the stream."""
        n = self.rows.shape[0]
        if not self.shuffle:
            return k % n
        epoch, pos = divmod(k, n)
        if epoch != self._perm_epoch:
            g = torch.Generator().manual_seed(self.seed * 1_000_003 + epoch)
            self._perm, self._perm_epoch = torch.randperm(n, generator=g), epoch
        return int(self._perm[pos])

    def __next__(self) -> dict:
        n = self.rows.shape[0]
        first = self.batches_drawn * self.mbs
        idx = [self._row_index(first + i) for i in range(self.mbs)]
        self.batches_drawn += 1
        self.cursor = (self.batches_drawn * self.mbs) % n
        chunk = self.rows[idx].long()
        b = {"tokens": chunk[:, :-1].contiguous(), "labels": chunk[:, 1:].contiguous(),
             "loss_mask": torch.ones(self.mbs, chunk.shape[1] - 1, dtype=torch.float32)}
        if self.doc_positions_eos is not None:
            b["position_ids"] = doc_position_ids(b["tokens"], self.doc_positions_eos)
        return {k: v.pin_memory() for k, v in b.items()} if self.pin else b

    def state_dict(self) -> dict:
        return {"kind": "packed", "cursor": self.cursor, "batches_drawn": self.batches_drawn,
                "shuffle": self.shuffle, "seed": self.seed}

    def load_state_dict(self, st: dict) -> None:
        if st and st.get("kind") == "packed":
            n = self.rows.shape[0]
            self.batches_drawn = int(st.get("batches_drawn", 0))
            self.cursor = (self.batches_drawn * self.mbs) % n


class StreamingTokenLoader:
    """Tokenises on demand instead of packing the whole slice up front: for corpora whose token
    array would not fit in host memory. Documents of this rank's strided slice are visited in a
    new order on every pass (seed + pass number), joined with EOS and cut into rows of
    ``seq_length + 1`` (the 0.5B engine's stream, hf_dataloader.py:148-170; the 8B engine keeps the
    same mode as ``preload=False``). The state is (pass, position in the pass, tokens left over),
    so a resumed run continues in the middle of a document."""

    def __init__(self, n_docs: int, doc_tokens, eos_id: int, micro_batch_size: int, seq_length: int,
                 dp_rank: int = 0, dp_size: int = 1, seed: int = 0, shuffle: bool = True,
                 pin: bool = False):
        self.doc_ids = list(range(dp_rank, n_docs, dp_size))
        if not self.doc_ids:
            raise ValueError(f"no documents for rank {dp_rank} of {dp_size}")
        self.doc_tokens = doc_tokens          # callable: document index -> list of token ids
        self.eos, self.mbs, self.row = eos_id, micro_batch_size, seq_length + 1
        self.seed, self.shuffle, self.pin = seed, shuffle, pin
        self.epoch, self.pos, self.buf = 0, 0, []
        self.batches_drawn = 0
        self._order_epoch, self._order = -1, None
        self._history: dict[int, dict] = {}

    # every data-parallel rank walks its own documents: a checkpoint has to keep one state per rank
    # (see pack_rank_states / select_rank_state); a packed or synthetic source is positioned by the
    # number of batches drawn alone, which is the same on every rank
    per_rank_state = True

    def __iter__(self):
        return self

    def state_dict_at(self, batches_consumed: int) -> dict:
        """State as it was when ``batches_consumed`` batches had been drawn (within the last 16):
        what a checkpoint must record when a prefetcher has already drawn further."""
        if batches_consumed == self.batches_drawn:
            return self.state_dict()
        return dict(self._history[batches_consumed])

    def _order_of(self, epoch: int) -> list[int]:
        if epoch != self._order_epoch:
            order = list(self.doc_ids)
            if self.shuffle:
                g = torch.Generator().manual_seed(self.seed * 1_000_003 + epoch)
                order = [order[i] for i in torch.randperm(len(order), generator=g).tolist()]
            self._order, self._order_epoch = order, epoch
        return self._order

    def _fill(self, n_tokens: int) -> None:
        empty_pass = 0
        while len(self.buf) < n_tokens:
            order = self._order_of(self.epoch)
            if self.pos >= len(order):
                self.epoch, self.pos = self.epoch + 1, 0
                empty_pass += 1
                if empty_pass > 1 and not self.buf:
                    raise ValueError("the documents of this rank contain no tokens")
                continue
            ids = self.doc_tokens(order[self.pos])
            self.pos += 1
            if ids:
                self.buf.extend(ids)
                self.buf.append(self.eos)
                empty_pass = 0

    def __next__(self) -> dict:
        need = self.mbs * self.row
        # a prefetcher draws ahead of what the model has consumed: remember the last few states
        self._history[self.batches_drawn] = self.state_dict()
        self._history.pop(self.batches_drawn - 16, None)
        self._fill(need)
        chunk = torch.tensor(self.buf[:need], dtype=torch.int64).view(self.mbs, self.row)
        self.buf = self.buf[need:]
        self.batches_drawn += 1
        b = {"tokens": chunk[:, :-1].contiguous(), "labels": chunk[:, 1:].contiguous(),
             "loss_mask": torch.ones(self.mbs, self.row - 1, dtype=torch.float32)}
        return {k: v.pin_memory() for k, v in b.items()} if self.pin else b

    def state_dict(self) -> dict:
        return {"kind": "stream", "epoch": self.epoch, "pos": self.pos, "buf": list(self.buf),
                "batches_drawn": self.batches_drawn}

    def load_state_dict(self, st: dict) -> None:
        if st and st.get("kind") == "stream":
            self.epoch, self.pos = int(st["epoch"]), int(st["pos"])
            self.buf = list(st.get("buf", []))
            self.batches_drawn = int(st.get("batches_drawn", 0))


def pack_rank_states(states: list[dict]) -> dict:
    """The ``dataloader_state`` entry of a checkpoint for a source with ``per_rank_state``: the
    states of all data-parallel ranks, in rank order."""
    return {"kind": "per_rank", "dp_size": len(states), "ranks": list(states)}


def select_rank_state(st: dict | None, dp_rank: int, dp_size: int, log=None) -> dict:
    """What ``source.load_state_dict`` gets on this rank. Written at another data-parallel size,
    the entry of a source that is positioned by a count of batches (synthetic, packed) is taken
    from the first rank; that of a streamed dataset cannot be mapped (the ranks' document slices
    differ): the stream then starts at the beginning of the pass the first rank was in, and
    ``log`` is told."""
    if not st or st.get("kind") != "per_rank":
        return st or {}
    if int(st["dp_size"]) == dp_size:
        return st["ranks"][dp_rank]
    if (st["ranks"][0] or {}).get("kind") != "stream":
        return st["ranks"][0] or {}      # positioned by a count of batches: any rank's state will do
    if log is not None:
        log(f"dataloader state was written by {st['dp_size']} data-parallel ranks, this run has {dp_size}: "
            f"each rank restarts its document stream at the beginning of the current pass")
    first = st["ranks"][0]
    return {"kind": first.get("kind"), "epoch": first.get("epoch", 0), "pos": 0, "buf": [],
            "batches_drawn": first.get("batches_drawn", 0)}


_COMMON_TEXT_COLUMNS = ("text", "content", "input", "sentence", "document")


def detect_text_fields(dataset) -> list[str]:
    """Pick the text column(s) of a dataset when ``--hf-text-field`` is not given: the first
    conventional name that exists, else every string-typed column, else an error that names the
    columns (reference: 0.5B hf_dataloader.py:76-103)."""
    cols = getattr(dataset, "column_names", None)
    if isinstance(cols, dict):                       # DatasetDict: columns of the first split
        cols = next(iter(cols.values()))
    if cols is None:                                 # plain iterable of dicts
        first = next(iter(dataset))
        cols = list(first)
        strings = [c for c in cols if isinstance(first[c], str)]
    else:
        feats = getattr(dataset, "features", None) or {}
        strings = [c for c in cols if getattr(feats.get(c), "dtype", None) == "string"]
    for name in _COMMON_TEXT_COLUMNS:
        if name in cols:
            return [name]
    if strings:
        return strings
    raise ValueError(f"no text column found among {list(cols)}; pass --hf-text-field")


def render_text(example: dict, text_field, template: str | None) -> str:
    """One document's text: the template filled from the row, else the non-empty named columns
    joined by newlines (a single name gives that column)."""
    if template:
        return template.format(**example)
    fields = [text_field] if isinstance(text_field, str) else list(text_field)
    if len(fields) == 1:
        return str(example[fields[0]])
    return "\n".join(str(example[f]) for f in fields if example.get(f))


class LocalRows(list):
    """Rows of local data files as a list of dicts (indexable and sized like a ``datasets.Dataset``;
    the text column is detected from the first row)."""


def load_local_files(fmt: str, files: str) -> LocalRows:
    """Read ``--hf-data-files`` (one path, a comma-separated list, or a glob) without the ``datasets``
    package: ``json`` (one object per line, or one array per file), ``text`` (one document per
    line, column ``text``), ``csv`` (header row) and ``parquet`` (through pyarrow)."""
    import csv
    import glob
    import json
    paths: list[str] = []
    for part in str(files).split(","):
        part = part.strip()
        hits = sorted(glob.glob(part)) if any(c in part for c in "*?[") else [part]
        paths += hits
    if not paths:
        raise FileNotFoundError(f"--hf-data-files {files!r} matches no file")
    rows = LocalRows()
    for path in paths:
        if fmt in ("json", "jsonl"):
            with open(path, encoding="utf-8") as f:
                head = f.read(1)
                f.seek(0)
                if head == "[":
                    rows.extend(json.load(f))
                else:
                    rows.extend(json.loads(line) for line in f if line.strip())
        elif fmt == "text":
            with open(path, encoding="utf-8") as f:
                rows.extend({"text": line.rstrip("\n")} for line in f)
        elif fmt == "csv":
            with open(path, encoding="utf-8", newline="") as f:
                rows.extend(csv.DictReader(f))
        elif fmt == "parquet":
            import pyarrow.parquet as pq
            rows.extend(pq.read_table(path).to_pylist())
        else:
            raise ValueError(f"--hf-data-format {fmt!r}: expected json, text, csv or parquet")
    return rows


def build_hf_dataloader(args, spec, micro_batch_size: int, seq_length: int, topo,
                        tokenizer=None, dataset=None) -> PackedTokenLoader:
    """Build the loader from CLI arguments. ``tokenizer`` / ``dataset`` may be injected (tests,
    offline use); otherwise ``transformers`` / ``datasets`` are imported here."""
    import torch.distributed as dist
    if tokenizer is None:
        from transformers import AutoTokenizer
        if not args.tokenizer_path:
            raise SystemExit("--hf-dataset needs --tokenizer-path")
        # rank-serialised load: rank 0 warms the cache, the others follow
        for turn in range(2):
            if (topo.rank == 0) == (turn == 0):
                tokenizer = AutoTokenizer.from_pretrained(args.tokenizer_path, trust_remote_code=True)
            if topo.world > 1 and dist.is_initialized():
                dist.barrier()
    if dataset is None:
        try:
            from datasets import load_dataset
        except ImportError:
            load_dataset = None
        if args.hf_data_files and load_dataset is None:
            # local files need no `datasets` package: read them with the standard library / pyarrow
            dataset = load_local_files(args.hf_data_format or "json", args.hf_data_files)
            if topo.rank == 0:
                print(f"[hf_dataloader] `datasets` is not installed: read {len(dataset)} rows from "
                      f"{args.hf_data_files} directly", flush=True)
        elif load_dataset is None:
            raise SystemExit("--hf-dataset needs the `datasets` package (or local files through "
                             "--hf-data-files with --hf-data-format json | text | parquet | csv)")
        elif args.hf_data_files:
            fmt = args.hf_data_format or "json"
            dataset = load_dataset(fmt, data_files=args.hf_data_files, split=args.hf_dataset_split)
        else:
            dataset = load_dataset(args.hf_dataset, args.hf_dataset_config, split=args.hf_dataset_split)
    eos = getattr(tokenizer, "eos_token_id", None)
    if eos is None:
        eos = 2
    vocab = spec.vocab_size

    fields = args.hf_text_field
    if fields is None and not args.hf_text_template:
        fields = detect_text_fields(dataset)
        if topo.rank == 0:
            print(f"[hf_dataloader] text_fields={fields}", flush=True)

    if getattr(args, "hf_stream", False):
        def doc_tokens(i: int) -> list[int]:
            text = render_text(dataset[i], fields, args.hf_text_template)
            if not text.strip():
                return []
            ids = tokenizer(text, add_special_tokens=False)["input_ids"]
            return [t if t < vocab else vocab - 1 for t in ids]
        return StreamingTokenLoader(len(dataset), doc_tokens, eos, micro_batch_size, seq_length,
                                    topo.dp_rank, topo.dp_size, seed=int(getattr(args, "seed", 0)),
                                    shuffle=bool(getattr(args, "hf_shuffle", True)),
                                    pin=topo.device.type == "cuda")

    def docs():
        for i, ex in enumerate(dataset):
            if i % topo.dp_size != topo.dp_rank:
                continue
            text = render_text(ex, fields, args.hf_text_template)
            if not text.strip():
                continue                                  # empty documents add nothing but an EOS
            ids = tokenizer(text, add_special_tokens=False)["input_ids"]
            yield [t if t < vocab else vocab - 1 for t in ids]

    rows = pack_token_stream(docs(), eos, seq_length, getattr(args, "max_packed_rows", None))
    return PackedTokenLoader(rows, micro_batch_size, pin=topo.device.type == "cuda",
                             doc_positions_eos=eos if getattr(args, "hf_doc_positions", False) else None,
                             shuffle=bool(getattr(args, "hf_shuffle", False)),
                             seed=int(getattr(args, "seed", 0)) + topo.dp_rank)
