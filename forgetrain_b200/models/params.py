"""Parameter registry, initialisation and flat-buffer storage.

* :func:`all_param_specs` is the single enumeration of trainable parameters (names, shapes,
  norm / weight-decay / muP-LR classes) in forward-registration order; the names are the
  reference's (exports/train_engine_0.5B/src/training_engine_tensor/parameters.py:76-118,
  786-844) so checkpoints stay interchangeable.
* :class:`ParamStore` owns ONE flat buffer of parameters in the compute dtype and ONE flat
  fp32 gradient buffer with identical offsets, laid out in reverse registration order
  (output head first, embedding last) so that backward fills the front of the buffer first and
  early buckets can be reduced while later layers are still running
  (reference: nccl.py:97-149). Per-parameter tensors are views into the two buffers; weight
  gradients are written in place by the wgrad GEMM, never copied.
* Tensor parallelism: column-parallel weights (wqkv, wfc1, embeddings, head) are sharded on
  rows, row-parallel weights (wo, w2) on columns; every rank initialises the full tensor from
  the same seed and keeps its shard, so results do not depend on the TP degree as long as the
  vocabulary is a multiple of ``8 * tp``; otherwise the vocabulary shards carry zero-initialised
  pad rows that take part in the softmax (Megatron's padded-vocabulary convention).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..config import ModelSpec

ALIGN_ELEMS = 128  # every parameter starts on a multiple of this many elements (TMA: 16 B)


@dataclass(frozen=True)
class ParamSpec:
    name: str
    shape: tuple[int, ...]          # full (unsharded) shape
    is_norm: bool
    has_weight_decay: bool
    mup_lr_scaled: bool             # hidden matrix: lr / width multiplier under muP
    tp_axis: int | None = None      # axis sharded under tensor parallelism (None: replicated)
    init: str = "normal"            # "normal" | "mup" | "ones"

    @property
    def numel(self) -> int:
        return math.prod(self.shape)


def mtp_layer_prefix(k: int) -> str:
    return f"mtp.layers.{k}"


def _layer_specs(prefix: str, spec: ModelSpec) -> list[ParamSpec]:
    h = spec.hidden_size
    return [
        ParamSpec(f"{prefix}.attention_norm.weight", (h,), True, False, False, None, "ones"),
        ParamSpec(f"{prefix}.attention.wqkv.weight", (spec.qkv_dim, h), False, True, True, 0, "mup"),
        ParamSpec(f"{prefix}.attention.wo.weight", (h, spec.q_dim), False, True, True, 1, "mup"),
        ParamSpec(f"{prefix}.ffn_norm.weight", (h,), True, False, False, None, "ones"),
        ParamSpec(f"{prefix}.feed_forward.wfc1.weight", (2 * spec.ffn_hidden_size, h), False, True,
                  True, 0, "mup"),
        ParamSpec(f"{prefix}.feed_forward.w2.weight", (h, spec.ffn_hidden_size), False, True, True,
                  1, "mup"),
    ]


def all_param_specs(spec: ModelSpec, mtp_num_layers: int = 0) -> list[ParamSpec]:
    """Every trainable parameter in forward-registration order."""
    h, v = spec.hidden_size, spec.vocab_size
    out = [ParamSpec("tok_embeddings.weight", (v, h), False, True, False, 0, "normal")]
    for i in range(spec.num_layers):
        out.extend(_layer_specs(f"layers.{i}", spec))
    out.append(ParamSpec("norm.weight", (h,), True, False, False, None, "ones"))
    for k in range(mtp_num_layers):
        p = mtp_layer_prefix(k)
        out.append(ParamSpec(f"{p}.enorm.weight", (h,), True, False, False, None, "ones"))
        out.append(ParamSpec(f"{p}.hnorm.weight", (h,), True, False, False, None, "ones"))
        out.append(ParamSpec(f"{p}.eh_proj.weight", (h, 2 * h), False, True, True, None, "mup"))
        out.extend(_layer_specs(p, spec))
    if not spec.tie_embeddings:
        out.append(ParamSpec("output.weight", (v, h), False, True, False, 0, "normal"))
    return out


def trainable_param_names(spec: ModelSpec, mtp_num_layers: int = 0) -> list[str]:
    return [s.name for s in all_param_specs(spec, mtp_num_layers)]


def flat_buffer_order(spec: ModelSpec, mtp_num_layers: int = 0) -> list[ParamSpec]:
    """Reverse registration order: output head, MTP, final norm, layers L-1..0 each as
    [w2, wfc1, ffn_norm, wqkv, attention_norm, wo], embedding last."""
    by_name = {s.name: s for s in all_param_specs(spec, mtp_num_layers)}
    order: list[str] = []
    if not spec.tie_embeddings:
        order.append("output.weight")
    for k in reversed(range(mtp_num_layers)):
        p = mtp_layer_prefix(k)
        order += [f"{p}.feed_forward.w2.weight",
                  f"{p}.feed_forward.wfc1.weight", f"{p}.ffn_norm.weight",
                  f"{p}.attention.wqkv.weight", f"{p}.attention_norm.weight",
                  f"{p}.attention.wo.weight", f"{p}.eh_proj.weight", f"{p}.hnorm.weight",
                  f"{p}.enorm.weight"]
    order.append("norm.weight")
    for i in reversed(range(spec.num_layers)):
        p = f"layers.{i}"
        order += [f"{p}.feed_forward.w2.weight", f"{p}.feed_forward.wfc1.weight",
                  f"{p}.ffn_norm.weight", f"{p}.attention.wqkv.weight",
                  f"{p}.attention_norm.weight", f"{p}.attention.wo.weight"]
    order.append("tok_embeddings.weight")
    assert len(order) == len(by_name) and set(order) == set(by_name)
    return [by_name[n] for n in order]


# -----------------------------------------------------------------------------------------
# tensor-parallel sharding
# -----------------------------------------------------------------------------------------
def kv_replication(spec: ModelSpec, tp: int) -> int:
    """How many TP ranks share one KV group (1 while tp <= num_query_groups)."""
    return max(1, tp // spec.num_query_groups)


def shard_for_tp(ps: ParamSpec, full: torch.Tensor, spec: ModelSpec, tp_rank: int, tp: int) -> torch.Tensor:
    """This rank's shard of a full parameter tensor."""
    if tp == 1 or ps.tp_axis is None:
        return full
    name = ps.name
    G, g, D = spec.num_query_groups, spec.heads_per_group, spec.head_dim
    if name.endswith("attention.wqkv.weight"):
        # rows: per KV group [q_0..q_{g-1} | k | v]
        w = full.view(G, g + 2, D, full.shape[1])
        if tp <= G:
            gpr = G // tp
            return w[tp_rank * gpr:(tp_rank + 1) * gpr].reshape(-1, full.shape[1])
        rep = tp // G                      # ranks per group: split q heads, replicate k / v
        grp, sub = tp_rank // rep, tp_rank % rep
        qpr = g // rep
        q = w[grp, sub * qpr:(sub + 1) * qpr]
        kv = w[grp, g:g + 2]
        return torch.cat([q, kv], dim=0).reshape(-1, full.shape[1])
    if name.endswith("attention.wo.weight"):
        # columns follow query heads in natural order
        hq = spec.num_attention_heads // tp
        return full[:, tp_rank * hq * D:(tp_rank + 1) * hq * D]
    if name.endswith("feed_forward.wfc1.weight"):
        F = spec.ffn_hidden_size
        fpr = F // tp
        gate = full[tp_rank * fpr:(tp_rank + 1) * fpr]
        up = full[F + tp_rank * fpr:F + (tp_rank + 1) * fpr]
        return torch.cat([gate, up], dim=0)
    if name.endswith("feed_forward.w2.weight"):
        fpr = spec.ffn_hidden_size // tp
        return full[:, tp_rank * fpr:(tp_rank + 1) * fpr]
    if name in ("tok_embeddings.weight", "output.weight"):
        vpr = vocab_shard_rows(spec.vocab_size, tp)
        lo = tp_rank * vpr
        hi = min(spec.vocab_size, lo + vpr)
        out = torch.zeros(vpr, full.shape[1], dtype=full.dtype, device=full.device)
        if hi > lo:
            out[:hi - lo] = full[lo:hi]
        return out
    size = full.shape[ps.tp_axis] // tp
    return full.narrow(ps.tp_axis, tp_rank * size, size)


def unshard_from_tp(ps: ParamSpec, parts: list[torch.Tensor], spec: ModelSpec) -> torch.Tensor:
    """Inverse of :func:`shard_for_tp`: the full parameter from the shards of all ``tp`` ranks
    (in rank order). Replicated parameters come from rank 0."""
    tp = len(parts)
    if tp == 1 or ps.tp_axis is None:
        return parts[0]
    name = ps.name
    G, g, D = spec.num_query_groups, spec.heads_per_group, spec.head_dim
    if name.endswith("attention.wqkv.weight"):
        if tp <= G:
            return torch.cat(parts, dim=0)
        rep = tp // G                      # q heads of a group are spread over `rep` ranks
        qpr = g // rep
        H = parts[0].shape[1]
        groups = []
        for grp in range(G):
            mine = [parts[grp * rep + sub].view(qpr + 2, D, H) for sub in range(rep)]
            groups.append(torch.cat([m[:qpr] for m in mine] + [mine[0][qpr:]], dim=0))
        return torch.cat(groups, dim=0).reshape(-1, H)
    if name.endswith("feed_forward.wfc1.weight"):
        fpr = parts[0].shape[0] // 2
        return torch.cat([x[:fpr] for x in parts] + [x[fpr:] for x in parts], dim=0)
    if name in ("tok_embeddings.weight", "output.weight"):
        return torch.cat(parts, dim=0)[:spec.vocab_size]
    axis = 1 if name.endswith(("attention.wo.weight", "feed_forward.w2.weight")) else ps.tp_axis
    return torch.cat(parts, dim=axis)


def merge_tp_shards(spec: ModelSpec, shards: list[dict[str, torch.Tensor]],
                    specs: list[ParamSpec] | None = None) -> dict[str, torch.Tensor]:
    """Full (TP = 1) named tensors from the per-rank dictionaries of a tensor-parallel run, e.g.
    the ``params`` / ``exp_avg`` entries of its ``rank_<R>.pt`` files in rank order."""
    specs = specs or all_param_specs(spec)
    out = {}
    for ps in specs:
        if ps.name in shards[0]:
            out[ps.name] = unshard_from_tp(ps, [sh[ps.name] for sh in shards], spec)
    return out


def vocab_shard_rows(vocab: int, tp: int) -> int:
    """Rows per vocabulary shard (padded so every shard has the same, 8-aligned size)."""
    per = (vocab + tp - 1) // tp
    return (per + 7) // 8 * 8


def local_shape(ps: ParamSpec, spec: ModelSpec, tp: int) -> tuple[int, ...]:
    if tp == 1 or ps.tp_axis is None:
        return ps.shape
    name = ps.name
    G, g, D = spec.num_query_groups, spec.heads_per_group, spec.head_dim
    if name.endswith("attention.wqkv.weight"):
        if tp <= G:
            return ((G // tp) * (g + 2) * D, ps.shape[1])
        rep = tp // G
        return ((g // rep + 2) * D, ps.shape[1])
    if name in ("tok_embeddings.weight", "output.weight"):
        return (vocab_shard_rows(spec.vocab_size, tp), ps.shape[1])
    s = list(ps.shape)
    s[ps.tp_axis] //= tp
    return tuple(s)


def init_std_for(ps: ParamSpec, spec: ModelSpec, scheme: str, init_std: float) -> float:
    """``spec`` scheme: embeddings / head use init_std, hidden matrices init_std/sqrt(width
    multiplier) under muP (reference parameters.py:181-262); ``normal``: N(0, init_std);
    ``mcore``: N(0, init_std) with the residual-stream projections scaled down by depth."""
    if ps.init == "ones":
        return 0.0
    if scheme == "mcore":
        # Megatron-core's scaled init of the 8B engine: the two projections that write into the
        # residual stream (attention output, FFN down) use init_std / sqrt(2 * num_layers)
        # (reference: exports/train_engine_8b/src/training_engine_tensor/parameters.py:253-358)
        if ps.name.endswith("attention.wo.weight") or ps.name.endswith("feed_forward.w2.weight"):
            return init_std / math.sqrt(2.0 * spec.num_layers)
        return init_std
    if scheme == "normal" or not spec.mup_enabled or ps.init == "normal":
        return init_std
    return init_std / math.sqrt(spec.mup_width_scale)


class ParamStore:
    """Flat parameter / gradient storage with per-parameter views."""

    def __init__(self, spec: ModelSpec, device, dtype: torch.dtype, mtp_num_layers: int = 0,
                 tp_rank: int = 0, tp_size: int = 1, pad_to: int = 1,
                 grad_buffer: torch.Tensor | None = None, align: int = ALIGN_ELEMS,
                 param_buffer: torch.Tensor | None = None):
        self.spec = spec
        self.device = torch.device(device)
        self.dtype = dtype
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.mtp_num_layers = mtp_num_layers
        self.specs = all_param_specs(spec, mtp_num_layers)
        self.by_name = {s.name: s for s in self.specs}
        self.order = flat_buffer_order(spec, mtp_num_layers)
        self.offsets: dict[str, int] = {}
        self.shapes: dict[str, tuple[int, ...]] = {}
        off = 0
        for ps in self.order:
            shp = local_shape(ps, spec, tp_size)
            self.offsets[ps.name] = off
            self.shapes[ps.name] = shp
            off += (math.prod(shp) + align - 1) // align * align
        self.raw_total = off
        self.total = (off + pad_to - 1) // pad_to * pad_to
        if param_buffer is not None:
            assert param_buffer.numel() >= self.total and param_buffer.dtype == dtype
            self.flat_params = param_buffer[:self.total]
            self.flat_params.zero_()
        else:
            self.flat_params = torch.zeros(self.total, dtype=dtype, device=self.device)
        if grad_buffer is not None:
            assert grad_buffer.numel() >= self.total and grad_buffer.dtype == torch.float32
            self.flat_grads = grad_buffer[:self.total]
            self.flat_grads.zero_()
        else:
            self.flat_grads = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        self.params: dict[str, torch.Tensor] = {}
        self.grads: dict[str, torch.Tensor] = {}
        for ps in self.order:
            o, shp = self.offsets[ps.name], self.shapes[ps.name]
            n = math.prod(shp)
            self.params[ps.name] = self.flat_params[o:o + n].view(shp)
            self.grads[ps.name] = self.flat_grads[o:o + n].view(shp)
        if spec.tie_embeddings:
            self.params["output.weight"] = self.params["tok_embeddings.weight"]
            self.grads["output.weight"] = self.grads["tok_embeddings.weight"]

    @staticmethod
    def layout_total(spec: ModelSpec, mtp_num_layers: int, tp_size: int, align: int) -> int:
        """Number of elements of the flat buffers for this layout (no allocation)."""
        off = 0
        for ps in flat_buffer_order(spec, mtp_num_layers):
            n = math.prod(local_shape(ps, spec, tp_size))
            off += (n + align - 1) // align * align
        return off

    # -- helpers -------------------------------------------------------------------------
    def entries(self) -> list[tuple[str, int, int]]:
        """(name, offset, padded numel) in flat-buffer order."""
        out = []
        names = [ps.name for ps in self.order]
        for i, n in enumerate(names):
            end = self.offsets[names[i + 1]] if i + 1 < len(names) else self.raw_total
            out.append((n, self.offsets[n], end - self.offsets[n]))
        return out

    def numel(self, name: str) -> int:
        return math.prod(self.shapes[name])

    def init_random(self, seed: int, scheme: str = "spec", init_std: float | None = None) -> None:
        """Seeded init, independent of the tensor-parallel degree: every rank draws the FULL
        tensor of each parameter from a generator keyed by (seed, parameter index) and keeps
        its shard. The draw happens on the store's device (large models initialise in seconds
        on a GPU), so CPU and GPU stores see different random streams."""
        std0 = self.spec.init_method_std if init_std is None else init_std
        gen = torch.Generator(device=self.device)
        for idx, ps in enumerate(self.specs):
            if ps.init == "ones":
                self.params[ps.name].fill_(1.0)
                continue
            std = init_std_for(ps, self.spec, scheme, std0)
            gen.manual_seed(seed * 1000003 + idx)
            full = torch.randn(ps.shape, dtype=torch.float32, generator=gen, device=self.device).mul_(std)
            shard = shard_for_tp(ps, full, self.spec, self.tp_rank, self.tp_size)
            self.params[ps.name].copy_(shard.to(self.dtype))
            del full, shard

    def load_named(self, tensors: dict[str, torch.Tensor], full_tensors: bool = True,
                   keep_missing: tuple[str, ...] = (), log=None) -> None:
        """Copy named tensors into the flat buffer, after checking that they describe THIS model.

        * A parameter whose name starts with one of ``keep_missing`` may be absent and then keeps
          its current value (the MTP head when the source is a plain language-model checkpoint).
        * ``output.weight`` absent from the source of a run with untied tables is taken from the
          embedding: that is what a checkpoint with tied tables means.
        * Anything else that is missing, a tensor the model has no parameter for (``mtp.*`` of a
          source with an MTP head excepted: the auxiliary head is dropped), or a shape that does
          not fit is an error that names the parameter, instead of a partial load.
        """
        note = log or (lambda m: None)
        own = {ps.name for ps in self.specs}
        extra = sorted(n for n in tensors if n not in own and not n.startswith("mtp."))
        if extra:
            raise ValueError(f"the checkpoint has {len(extra)} tensors this model has no parameter for "
                             f"({', '.join(extra[:4])}{', ...' if len(extra) > 4 else ''}): another "
                             f"--model, --num-layers or --tie-embeddings than the run that wrote it?")
        if any(n.startswith("mtp.") and n not in own for n in tensors):
            note("the checkpoint's MTP head is not used by this run and is dropped")
        missing, plan = [], []
        for ps in self.specs:               # first pass: everything is checked before anything is copied
            if ps.name in tensors:
                t = tensors[ps.name]
            elif keep_missing and ps.name.startswith(keep_missing):
                continue
            elif ps.name == "output.weight" and "tok_embeddings.weight" in tensors:
                note("the checkpoint ties the output table to the embedding: output.weight starts as its copy")
                t = tensors["tok_embeddings.weight"]
            else:
                missing.append(ps.name)
                continue
            if full_tensors:
                t = shard_for_tp(ps, t, self.spec, self.tp_rank, self.tp_size)
            if tuple(t.shape) != tuple(self.params[ps.name].shape):
                raise ValueError(f"{ps.name}: the checkpoint holds {tuple(t.shape)}, this model needs "
                                 f"{tuple(self.params[ps.name].shape)}")
            plan.append((ps.name, t))
        if missing:
            raise KeyError(f"the checkpoint lacks {len(missing)} parameters of this model "
                           f"({', '.join(missing[:4])}{', ...' if len(missing) > 4 else ''})")
        for name, t in plan:
            self.params[name].copy_(t.to(self.dtype))

    def named_cpu_params(self) -> dict[str, torch.Tensor]:
        return {ps.name: self.params[ps.name].detach().to("cpu").clone() for ps in self.specs}
