"""Multi-token-prediction head (EAGLE style), optional and off by default.

Per extra layer k (reference: exports/train_engine_0.5B/src/training_engine_tensor/forward.py:
330-495, backward.py:521-742): token ids, labels and loss mask are rolled left by one more
position (last slot zeroed); the SHARED embedding of the rolled ids goes through ``enorm``, the
previous hidden state (the main model's final-norm output for k = 0) through ``hnorm``; the two
are concatenated and projected 2H -> H by ``eh_proj``; one full decoder block follows; the
result, divided by the muP width multiplier, feeds the SHARED output head. Each extra loss is
weighted ``mtp_loss_scaling_factor / num_layers``. Gradients of the shared tables are folded
into the main gradients: the head's weight gradient accumulates after the main head's, the
embedding lookups are scattered after the main embedding backward.
"""
from __future__ import annotations

import torch

from .. import ops
from .minicpm4 import MiniCPM4
from .params import mtp_layer_prefix


def roll_left_one(t: torch.Tensor) -> torch.Tensor:
    r = torch.roll(t, shifts=-1, dims=-1)
    r[..., -1] = 0
    return r


class MTPHead:
    def __init__(self, model: MiniCPM4, num_layers: int, loss_scaling_factor: float):
        if model.tp.enabled:
            raise NotImplementedError("the MTP head runs with tensor_parallel_size == 1")
        if model.spec.tie_embeddings:
            raise NotImplementedError("the MTP head expects untied embedding / output tables")
        self.m = model
        self.K = num_layers
        self.factor = loss_scaling_factor
        self.last_mtp_losses: list[torch.Tensor] = []

    def forward_backward(self, tokens, labels, loss_mask=None, loss_scale: float = 1.0,
                         accumulate: bool = False, grad_ready=None, position_ids=None):
        m, sp, p, g = self.m, self.m.spec, self.m.p, self.m.g
        emit = grad_ready or (lambda name: None)
        B, S = tokens.shape
        a = 1.0 / sp.mup_width_scale
        if loss_mask is None:
            loss_mask = torch.ones(B, S, dtype=torch.float32, device=tokens.device)
        # ---------------- main forward + loss
        logits = m.forward(tokens, position_ids)
        nf = m._head_saved[2]                       # final-norm output: input of the first MTP layer
        loss, dlogits = m.loss_and_dlogits(logits, labels, loss_mask, loss_scale)
        # ---------------- MTP forward
        ids, lab, msk, hidden = tokens, labels, loss_mask, nf
        saved = []
        self.last_mtp_losses = []
        for k in range(self.K):
            pre = mtp_layer_prefix(k)
            if m.param_gate is not None:
                m.param_gate(pre)
            ids, lab, msk = roll_left_one(ids), roll_left_one(lab), roll_left_one(msk)
            e = ops.embedding_fwd(ids, p["tok_embeddings.weight"], sp.emb_scale)
            _, en, rse = ops.add_rmsnorm_fwd(None, e, p[f"{pre}.enorm.weight"], sp.norm_epsilon)
            _, hn, rsh = ops.add_rmsnorm_fwd(None, hidden, p[f"{pre}.hnorm.weight"], sp.norm_epsilon)
            comb = torch.cat([en, hn], dim=-1)
            proj = ops.linear_fwd(comb, p[f"{pre}.eh_proj.weight"])
            h_mid, f, sv = m.layer_forward(pre, None, proj, B, position_ids)
            out = h_mid + f
            lg = ops.linear_fwd(out, p["output.weight"], alpha=a)
            lk, dlg = ops.cross_entropy_fwd_bwd(lg, lab, msk, loss_scale * self.factor / self.K)
            self.last_mtp_losses.append(lk)
            saved.append((pre, ids, e, rse, hidden, rsh, comb, sv, out, dlg))
            hidden = out
        # ---------------- backward: main head weight gradient first (store), then MTP (accumulate)
        ops.linear_wgrad(dlogits, nf, g["output.weight"], accumulate, alpha=a)
        d_next = None
        emb_extra = []
        for k in reversed(range(self.K)):
            pre, ids_k, e, rse, hid_in, rsh, comb, sv, out, dlg = saved[k]
            ops.linear_wgrad(dlg, out, g["output.weight"], True, alpha=a)
            d_out = ops.linear_dgrad(dlg, p["output.weight"], alpha=a)
            if d_next is not None:
                d_out = d_out + d_next
            dproj = m.layer_backward(pre, d_out, sv, B, accumulate, emit, position_ids)
            ops.linear_wgrad(dproj, comb, g[f"{pre}.eh_proj.weight"], accumulate)
            emit(f"{pre}.eh_proj.weight")
            dcomb = ops.linear_dgrad(dproj, p[f"{pre}.eh_proj.weight"])
            H = sp.hidden_size
            den, dhn = dcomb[:, :H].contiguous(), dcomb[:, H:].contiguous()
            d_next = ops.rmsnorm_bwd(dhn, hid_in, p[f"{pre}.hnorm.weight"], rsh, None,
                                     g[f"{pre}.hnorm.weight"], accumulate)
            emit(f"{pre}.hnorm.weight")
            de = ops.rmsnorm_bwd(den, e, p[f"{pre}.enorm.weight"], rse, None,
                                 g[f"{pre}.enorm.weight"], accumulate)
            emit(f"{pre}.enorm.weight")
            emb_extra.append((ids_k, de))
            saved[k] = None
        emit("output.weight")
        # ---------------- main backward with the MTP gradient entering at the final-norm output
        dh = m.head_backward(dlogits, accumulate, emit, dnf_extra=d_next, emit_output=False,
                             skip_wgrad=True)
        for i in reversed(range(sp.num_layers)):
            dh = m.layer_backward(f"layers.{i}", dh, m._saved[i], B, accumulate, emit, position_ids)
            m._saved[i] = None
        m.embedding_backward(tokens, dh, accumulate, emit, extra=emb_extra)
        m._saved = []
        return loss
