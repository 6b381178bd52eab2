"""MiniCPM4 decoder: hand-written forward and backward over the op layer.

There is no ``nn.Module`` and no autograd: parameters are views into the flat buffers of a
:class:`~forgetrain_b200.models.params.ParamStore`, the forward keeps what the backward needs
in plain lists, and the backward is an explicit reverse pass that writes every weight gradient
straight into the flat fp32 gradient buffer (store on the first micro-batch, accumulate
afterwards) and reports each finished parameter through ``grad_ready`` so bucket reductions
can start while earlier layers are still running. Same structure as the reference
(exports/train_engine_0.5B/src/training_engine_tensor/forward.py:81-217, backward.py:125-393)
with these differences: activations are token-major ``[B*S, H]``; q/k/v are never split out of
the projection buffer (RoPE runs in place on it and attention reads it through strided TMA
boxes); the muP residual multiplier and the logit divisor ride in GEMM epilogues.

Block (pre-norm):  h += r * Wo·attn(rope(Wqkv·rmsnorm(h)));  h += r * W2·swiglu(Wfc1·rmsnorm(h))
with r = depth_scale/sqrt(L); embedding * emb_scale; logits = Wout·(rmsnorm(h) / (H/256)).
"""
from __future__ import annotations

import os

from typing import Callable

import torch

from .. import ops
from ..config import ModelSpec
from ..parallel.tp import NO_TP, TPContext
from .params import ParamStore, vocab_shard_rows


class LayerSaved:
    __slots__ = ("h_in", "rs1", "n1_full", "qkv", "attn", "lse", "h_mid", "rs2", "n2_full", "y1",
                 "act")

    def __init__(self):
        self.attn = self.lse = self.y1 = self.act = None   # absent when they are recomputed


class MiniCPM4:
    def __init__(self, spec: ModelSpec, store: ParamStore, tp: TPContext = NO_TP,
                 max_seq_len: int | None = None, save_act: bool = True,
                 recompute_attn: bool = False, recompute_mlp: bool = False):
        """``recompute_attn`` / ``recompute_mlp``: activation recomputation, the reference's
        switches of the same names (exports/train_engine_8b/src/training_engine_tensor/
        forward.py:65-66,286-306). With ``recompute_attn`` the attention output and its
        log-sum-exp are not kept between forward and backward; the backward runs the forward
        kernel again on the saved (rotated) qkv buffer. With ``recompute_mlp`` the FC1 output
        and the SwiGLU activation (3 * ffn_hidden values per token and layer, the largest
        saved tensors) are dropped and rebuilt from the saved FFN-norm output. Both reruns use
        the kernels of the forward pass on the same inputs, so gradients are bitwise those of
        the saved-activation path."""
        self.spec = spec
        self.recompute_attn = recompute_attn
        self.recompute_mlp = recompute_mlp
        self.store = store
        self.tp = tp
        self.p = store.params
        self.g = store.grads
        self.save_act = save_act
        dev = store.device
        S = max_seq_len or max(spec.seq_length, spec.max_position_embeddings)
        self.cos, self.sin = ops.rope_tables(S, spec.head_dim, spec.rotary_base, device=dev)
        tpn = tp.size
        G = spec.num_query_groups
        if tpn <= G:
            assert G % tpn == 0, "num_query_groups must be a multiple of the TP degree"
            self.local_groups, self.local_g = G // tpn, spec.heads_per_group
        else:
            rep = tpn // G
            assert tpn % G == 0 and spec.heads_per_group % rep == 0
            self.local_groups, self.local_g = 1, spec.heads_per_group // rep
        self.vocab_rows = vocab_shard_rows(spec.vocab_size, tpn) if tpn > 1 else spec.vocab_size
        self.vocab_start = tp.rank * self.vocab_rows if tpn > 1 else 0
        self._saved: list[LayerSaved] = []
        self._head_saved = None
        # set to a dict to have the backward record a few intermediate gradients in it
        self.diagnostics: dict | None = None
        # called with a parameter-name prefix ("tok_embeddings", "layers.3", "norm", "output")
        # right before the forward first reads parameters under it: the trainer hangs the
        # per-bucket "updated and gathered" events of the previous optimizer step on it
        self.param_gate: Callable[[str], None] | None = None
        # a CUDA stream for the weight-gradient GEMMs of the decoder blocks (None: they run in
        # line). On it they overlap the tensor-parallel collective that follows the data gradient
        # of the same layer (reference backward.py:452-463,555-564); the parameter's "gradient
        # ready" call is made after the main stream has joined that GEMM.
        self.wgrad_stream = None
        self._wgrad_done: dict[str, object] = {}
        # FC1 + SwiGLU in one kernel where FC1 is a plain local GEMM (no tensor parallelism)
        self.fuse_fc1_swiglu = tpn == 1 and os.environ.get("FT_FUSE_FC1_SWIGLU", "1") != "0"
        self._ensure_rope(S)

    def _ensure_rope(self, S: int) -> None:
        if self.cos.shape[0] < S:
            self.cos, self.sin = ops.rope_tables(S, self.spec.head_dim, self.spec.rotary_base,
                                                 device=self.store.device)

    # ------------------------------------------------------------------------------ forward
    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        """Token embedding * emb_scale, returned on this rank's token shard."""
        if self.param_gate is not None:
            self.param_gate("tok_embeddings")
        w = self.p["tok_embeddings.weight"]
        e = ops.embedding_fwd(tokens, w, self.spec.emb_scale, self.vocab_start)
        if self.tp.enabled:
            e = self.tp.scatter_reduce(e)
        return e

    def layer_forward(self, prefix: str, h_prev, branch, batch: int, position_ids=None):
        """One decoder block. ``h_prev + branch`` is the block input (the add is fused into the
        first norm); returns ``(h_mid, ffn_branch, saved)`` with the output being their sum."""
        sp, p, tp = self.spec, self.p, self.tp
        if self.param_gate is not None:
            self.param_gate(prefix)
        r = sp.mup_residual_scale
        sv = LayerSaved()
        x_in = h_prev if h_prev is not None else branch
        h_in, n1, sv.rs1 = ops.add_rmsnorm_fwd(
            branch if h_prev is not None else None, x_in, p[f"{prefix}.attention_norm.weight"],
            sp.norm_epsilon, tp.gather_dest(f"{prefix}.n1", x_in.shape[0], x_in.shape[1]))
        sv.h_in = h_in
        qkv, sv.n1_full = tp.linear_gather(n1, p[f"{prefix}.attention.wqkv.weight"],
                                           key=f"{prefix}.n1")
        ops.rope_(qkv, self.cos, self.sin, batch, self.local_groups, self.local_g, sp.head_dim,
                  position_ids=position_ids)
        sv.qkv = qkv
        attn, lse = ops.attention_fwd(qkv, batch, self.local_groups, self.local_g, sp.head_dim)
        if not self.recompute_attn:
            sv.attn, sv.lse = attn, lse
        o = tp.linear_scatter(attn, p[f"{prefix}.attention.wo.weight"], alpha=r)
        del attn, lse
        sv.h_mid, n2, sv.rs2 = ops.add_rmsnorm_fwd(
            h_in, o, p[f"{prefix}.ffn_norm.weight"], sp.norm_epsilon,
            tp.gather_dest(f"{prefix}.n2", o.shape[0], o.shape[1]))
        if self.fuse_fc1_swiglu:
            # one kernel: FC1 with silu(gate) * up computed in its epilogue
            sv.n2_full = n2
            y1, act = ops.linear_swiglu_fwd(n2, p[f"{prefix}.feed_forward.wfc1.weight"])
        else:
            y1, sv.n2_full = tp.linear_gather(n2, p[f"{prefix}.feed_forward.wfc1.weight"],
                                              key=f"{prefix}.n2")
            act = ops.swiglu_fwd(y1)
        if not self.recompute_mlp:
            sv.y1, sv.act = y1, act
        f = tp.linear_scatter(act, p[f"{prefix}.feed_forward.w2.weight"], alpha=r)
        return sv.h_mid, f, sv

    def _recompute_mlp(self, prefix: str, sv: LayerSaved):
        """FC1 output and SwiGLU activation again, from the saved (gathered) FFN-norm output:
        a local GEMM, no collective."""
        w = self.p[f"{prefix}.feed_forward.wfc1.weight"]
        if self.fuse_fc1_swiglu:
            return ops.linear_swiglu_fwd(sv.n2_full, w)
        y1 = ops.linear_fwd(sv.n2_full, w)
        return y1, ops.swiglu_fwd(y1)

    def forward_hidden(self, tokens: torch.Tensor, position_ids=None):
        """Embedding + all blocks. Returns (h, branch): the final hidden state is h + branch."""
        B, S = tokens.shape
        self._ensure_rope(S)
        self._saved = []
        h, branch = None, self.embed(tokens)
        for i in range(self.spec.num_layers):
            h, branch, sv = self.layer_forward(f"layers.{i}", h, branch, B, position_ids)
            self._saved.append(sv)
        return h, branch

    def head_forward(self, h, branch):
        """Final norm, logit divisor, LM head. Returns logits of this rank's vocabulary shard."""
        sp, p = self.spec, self.p
        if self.param_gate is not None:
            self.param_gate("norm")
            self.param_gate("output")
        h_fin, nf, rsf = ops.add_rmsnorm_fwd(
            h, branch, p["norm.weight"], sp.norm_epsilon,
            self.tp.gather_dest("head.nf", branch.shape[0], branch.shape[1]))
        logits, nf_full = self.tp.linear_gather(nf, p["output.weight"],
                                                alpha=1.0 / sp.mup_width_scale, key="head.nf")
        self._head_saved = (h_fin, rsf, nf_full)
        return logits

    def forward(self, tokens: torch.Tensor, position_ids=None) -> torch.Tensor:
        h, branch = self.forward_hidden(tokens, position_ids)
        return self.head_forward(h, branch)

    # Under tensor parallelism the vocabulary shards are padded to a multiple of 8 rows; by default
    # the pad columns are part of the softmax (Megatron's padded-vocabulary convention). True:
    # their logits are set far below every real one before the loss, so they carry no probability
    # and no gradient, and the loss is the one a run without tensor parallelism computes.
    mask_vocab_padding = False
    _PAD_LOGIT = -30000.0      # finite (no inf - inf in a running maximum), exp() of it is 0 in fp32

    def loss_and_dlogits(self, logits, labels, loss_mask, loss_scale: float):
        tp = self.tp
        if self.mask_vocab_padding and tp.enabled:
            real = self.spec.vocab_size - self.vocab_start      # real columns of this rank's shard
            if real < logits.shape[1]:
                logits[:, max(real, 0):] = self._PAD_LOGIT
        return ops.cross_entropy_fwd_bwd(
            logits, labels, loss_mask, loss_scale, vocab_start=self.vocab_start,
            stats_reduce=tp.stats_reduce if tp.enabled else None,
            tp_exchange=tp if (tp.enabled and hasattr(tp, "ce_exchange")) else None)

    # ----------------------------------------------------------------------------- backward
    def head_backward(self, dlogits, accumulate: bool, emit, dnf_extra=None, emit_output=True,
                      skip_wgrad=False):
        """Backward of head + final norm. ``dnf_extra`` is added to the gradient of the final
        norm's OUTPUT (used by the MTP head, which consumes that tensor)."""
        sp, p, g, tp = self.spec, self.p, self.g, self.tp
        h_fin, rsf, nf_full = self._head_saved
        a = 1.0 / sp.mup_width_scale
        if not skip_wgrad:
            ops.linear_wgrad(dlogits, nf_full, g["output.weight"], accumulate, alpha=a)
        if not sp.tie_embeddings and emit_output:
            emit("output.weight")
        dnf = tp.dgrad_scatter(dlogits, p["output.weight"], alpha=a)
        if dnf_extra is not None:
            dnf = dnf + dnf_extra
        diag = self.diagnostics
        if diag is not None:
            diag["d_normed_final"] = dnf.detach().clone()
        dh = ops.rmsnorm_bwd(dnf, h_fin, p["norm.weight"], rsf, None, g["norm.weight"], accumulate)
        emit("norm.weight")
        if diag is not None:
            diag["d_hidden_after_norm"] = dh.detach().clone()
        self._head_saved = None
        return dh

    def _wgrad(self, dy, x, name: str, accumulate: bool, alpha: float = 1.0) -> None:
        """Weight gradient of parameter ``name``: in line, or on ``wgrad_stream`` behind an event
        of the current stream (the operands are complete there)."""
        ws = self.wgrad_stream
        if ws is None or not dy.is_cuda:
            ops.linear_wgrad(dy, x, self.g[name], accumulate, alpha=alpha)
            return
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(ws):
            ws.wait_event(ready)
            ops.linear_wgrad(dy, x, self.g[name], accumulate, alpha=alpha)
            dy.record_stream(ws)     # the caching allocator must not hand these blocks out
            x.record_stream(ws)      # again before the side stream has read them
            done = torch.cuda.Event()
            done.record()
        self._wgrad_done[name] = done

    def _emit_after_wgrad(self, emit, name: str) -> None:
        """``emit(name)`` once the current stream is behind the weight-gradient GEMM of ``name``."""
        done = self._wgrad_done.pop(name, None)
        if done is not None:
            torch.cuda.current_stream().wait_event(done)
        emit(name)

    def layer_backward(self, prefix: str, dh, sv: LayerSaved, batch: int, accumulate: bool, emit,
                       position_ids=None):
        """``dh``: gradient wrt the block output (token shard). Returns the gradient wrt the
        block input."""
        sp, p, g, tp = self.spec, self.p, self.g, self.tp
        r = sp.mup_residual_scale
        n_w2, n_fc1 = f"{prefix}.feed_forward.w2.weight", f"{prefix}.feed_forward.wfc1.weight"
        n_qkv, n_wo = f"{prefix}.attention.wqkv.weight", f"{prefix}.attention.wo.weight"
        n_fn, n_an = f"{prefix}.ffn_norm.weight", f"{prefix}.attention_norm.weight"
        # gradients of the LAST block are what a numerical comparison with another engine looks
        # at first (reference backward.py:211-252: the ``diagnostics`` dict)
        diag = self.diagnostics if prefix == f"layers.{sp.num_layers - 1}" else None
        if diag is not None:
            diag["d_hidden_into_last_layer"] = dh.detach().clone()
        # ---- feed-forward branch
        y1, act = (sv.y1, sv.act) if sv.y1 is not None else self._recompute_mlp(prefix, sv)
        sv.y1 = sv.act = None
        if diag is None:   # FC2 dgrad with the activation backward in its epilogue
            dy1, dh_full = tp.dgrad_gather_swiglu_bwd(dh, p[n_w2], y1, alpha=r, key="bwd.ffn")
        else:              # the last block keeps the intermediate gradient for the diagnostics
            dact, dh_full = tp.dgrad_gather(dh, p[n_w2], alpha=r, key="bwd.ffn")
            dy1 = ops.swiglu_bwd(dact, y1)
            diag["d_intermediate_last"] = dact.detach().clone()
            diag["d_fc1_last"] = dy1.detach().clone()
            del dact
        del y1
        self._wgrad(dh_full, act, n_w2, accumulate, alpha=r)
        del act
        self._wgrad(dy1, sv.n2_full, n_fc1, accumulate)
        dn2 = tp.dgrad_scatter(dy1, p[n_fc1])     # its collective overlaps the two GEMMs above
        del dy1
        self._emit_after_wgrad(emit, n_w2)
        self._emit_after_wgrad(emit, n_fc1)
        dh = ops.rmsnorm_bwd(dn2, sv.h_mid, p[n_fn], sv.rs2, dh, g[n_fn], accumulate)
        emit(n_fn)
        # ---- attention branch
        if sv.attn is None:   # recompute_attn: the forward kernel again, on the rotated qkv
            sv.attn, sv.lse = ops.attention_fwd(sv.qkv, batch, self.local_groups, self.local_g,
                                                sp.head_dim)
        dattn, dh_full = tp.dgrad_gather(dh, p[n_wo], alpha=r, key="bwd.attn")
        self._wgrad(dh_full, sv.attn, n_wo, accumulate, alpha=r)
        # the rotary embedding's backward rides in the attention backward's last kernel
        dqkv = ops.attention_bwd(dattn, sv.qkv, sv.attn, sv.lse, batch, self.local_groups,
                                 self.local_g, sp.head_dim,
                                 rope=(self.cos, self.sin, position_ids))
        del dattn
        sv.attn = sv.lse = None
        self._wgrad(dqkv, sv.n1_full, n_qkv, accumulate)
        dn1 = tp.dgrad_scatter(dqkv, p[n_qkv])    # its collective overlaps the GEMM above
        done = self._wgrad_done.pop(n_qkv, None)
        if done is not None:
            torch.cuda.current_stream().wait_event(done)
        emit(n_qkv)
        del dqkv
        dh = ops.rmsnorm_bwd(dn1, sv.h_in, p[n_an], sv.rs1, dh, g[n_an], accumulate)
        emit(n_an)
        self._emit_after_wgrad(emit, n_wo)
        return dh

    def finalize_grad(self, name: str) -> None:
        """The tensor-parallel collectives that complete the gradient of parameter ``name``; to be
        called ONCE per optimizer step, when the gradient has been accumulated over all
        micro-batches and before it is reduced over the data-parallel group (the trainer does so
        from its "gradient ready" callback). Two kinds of parameters need one: norm weights under
        sequence parallelism (every rank has seen its token shard only) and the k / v rows of the
        fused QKV weight when one KV group is replicated over several ranks. Summing a buffer
        that still accumulates would count the earlier micro-batches once per rank."""
        tp = self.tp
        if not tp.enabled:
            return
        ps = self.store.by_name.get(name)
        if ps is not None and ps.is_norm and tp.sequence_parallel:
            tp.all_reduce_(self.g[name])
        elif tp.replica_size > 1 and name.endswith("attention.wqkv.weight"):
            tp.replica_all_reduce_(self.g[name][self.local_g * self.spec.head_dim:])

    def embedding_backward(self, tokens, dh, accumulate: bool, emit, extra=None):
        sp, g, tp = self.spec, self.g, self.tp
        gw = g["tok_embeddings.weight"]
        if not accumulate and not sp.tie_embeddings:
            gw.zero_()
        dfull = tp.gather(dh) if tp.enabled else dh
        ops.embedding_bwd(tokens, dfull, sp.emb_scale, gw, self.vocab_start)
        for ids_x, d_x in extra or ():     # further lookups of the same table (MTP heads)
            ops.embedding_bwd(ids_x, d_x, sp.emb_scale, gw, self.vocab_start)
        emit("tok_embeddings.weight")

    def backward(self, tokens, dlogits, accumulate: bool,
                 grad_ready: Callable[[str], None] | None = None, position_ids=None,
                 dh_extra: torch.Tensor | None = None) -> None:
        """Reverse pass from ``dlogits``. ``dh_extra`` (MTP) is added to the gradient of the
        final hidden state before the blocks are walked."""
        emit = grad_ready or (lambda name: None)
        B = tokens.shape[0]
        dh = self.head_backward(dlogits, accumulate, emit)
        if dh_extra is not None:
            dh = dh + dh_extra
        for i in reversed(range(self.spec.num_layers)):
            sv = self._saved[i]
            dh = self.layer_backward(f"layers.{i}", dh, sv, B, accumulate, emit, position_ids)
            self._saved[i] = None
        self.embedding_backward(tokens, dh, accumulate, emit)
        self._saved = []

    # -------------------------------------------------------------------- one micro-batch
    def forward_backward(self, tokens, labels, loss_mask=None, loss_scale: float = 1.0,
                         accumulate: bool = False, grad_ready=None, position_ids=None):
        """Forward + loss + backward of one micro-batch; returns the (unscaled) mean loss."""
        logits = self.forward(tokens, position_ids)
        loss, dlogits = self.loss_and_dlogits(logits, labels, loss_mask, loss_scale)
        self.backward(tokens, dlogits, accumulate, grad_ready, position_ids)
        return loss
