"""``training_engine_tensor.backward``: loss and the hand-derived reverse pass under the reference's
module name (0.5B backward.py:73-393, 8B backward.py:203-860)."""
from forgetrain_b200.models.minicpm4 import MiniCPM4  # noqa: F401


def cross_entropy_loss_backward(model: MiniCPM4, logits, labels, loss_mask=None, loss_scale: float = 1.0):
    """``(mean loss, d_logits)``; ``d_logits`` already carries ``loss_scale`` and overwrites the
    logits buffer on the CUDA path."""
    return model.loss_and_dlogits(logits, labels, loss_mask, loss_scale)


def backward_pass(model: MiniCPM4, tokens, dlogits, accumulate: bool = False, grad_sink=None,
                  position_ids=None) -> None:
    """Reverse pass into the flat fp32 gradient buffer. ``grad_sink(name)`` is called when the
    gradient of parameter ``name`` is complete (what lets a bucket's reduction start early)."""
    model.backward(tokens, dlogits, accumulate, grad_sink, position_ids)


manual_backward = backward_pass

__all__ = ["MiniCPM4", "cross_entropy_loss_backward", "backward_pass", "manual_backward"]
