"""``training_engine_tensor.forward``: the forward pass under the reference's module name (0.5B
forward.py:81-217, 8B forward.py:58-332). The model is an object here (:class:`MiniCPM4` over a
:class:`ParamStore`), so the reference's free functions become thin calls on it."""
from forgetrain_b200.models.minicpm4 import MiniCPM4  # noqa: F401
from forgetrain_b200.models.mtp import MTPHead  # noqa: F401


def forward_pass_with_save(model: MiniCPM4, tokens, position_ids=None):
    """Logits ``[B * S, vocab]``; the activations the reverse pass needs stay saved in ``model``."""
    return model.forward(tokens, position_ids)


forward_pass = forward_pass_with_save

__all__ = ["MiniCPM4", "MTPHead", "forward_pass_with_save", "forward_pass"]
