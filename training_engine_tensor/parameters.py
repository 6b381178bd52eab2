"""``training_engine_tensor.parameters``: parameter registry, initialisation, Megatron import and
checkpoints under the reference's module name (0.5B parameters.py:9-20, 8B parameters.py:33-37)."""
from forgetrain_b200.ckpt.checkpoint import (  # noqa: F401
    latest_checkpoint, load_resume_checkpoint, save_checkpoint, should_save_after_step,
    wait_for_async_save)
from forgetrain_b200.ckpt.megatron_import import (  # noqa: F401
    is_megatron_root, load_megatron_checkpoint, load_megatron_optimizer_state, megatron_name_map)
from forgetrain_b200.models.params import (  # noqa: F401
    ParamSpec, ParamStore, all_param_specs, flat_buffer_order, merge_tp_shards, mtp_layer_prefix,
    shard_for_tp,
    trainable_param_names, unshard_from_tp)

__all__ = ["ParamSpec", "ParamStore", "all_param_specs", "trainable_param_names", "flat_buffer_order",
           "shard_for_tp", "unshard_from_tp", "merge_tp_shards", "load_megatron_checkpoint",
           "load_megatron_optimizer_state", "megatron_name_map", "is_megatron_root", "save_checkpoint",
           "load_resume_checkpoint", "latest_checkpoint", "should_save_after_step",
           "wait_for_async_save", "mtp_layer_prefix"]
