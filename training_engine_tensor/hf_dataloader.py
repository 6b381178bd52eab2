"""``training_engine_tensor.hf_dataloader``: tokenise + pack loader under the reference's module name
(0.5B hf_dataloader.py:28-269, 8B hf_dataloader.py:42-469)."""
from forgetrain_b200.data.hf_dataloader import (  # noqa: F401
    PackedTokenLoader, build_hf_dataloader, detect_text_fields, doc_position_ids, pack_token_stream,
    render_text)


def next_hf_batch(loader):
    """The next micro-batch dict (``tokens``, ``labels``, ``loss_mask``[, ``position_ids``])."""
    return next(loader)


__all__ = ["build_hf_dataloader", "next_hf_batch", "PackedTokenLoader", "pack_token_stream",
           "detect_text_fields", "render_text", "doc_position_ids"]
