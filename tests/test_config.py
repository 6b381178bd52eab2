import math

import pytest

from forgetrain_b200 import config as C
from forgetrain_b200 import engine_config as ec


def test_builtin_specs_load():
    s05 = C.load_model_spec("0.5b")
    assert (s05.hidden_size, s05.num_layers, s05.num_attention_heads, s05.num_query_groups,
            s05.head_dim, s05.ffn_hidden_size, s05.vocab_size) == (1024, 24, 16, 2, 64, 4096, 73448)
    s8 = C.load_model_spec("8b")
    assert (s8.hidden_size, s8.num_layers, s8.head_dim, s8.ffn_hidden_size) == (4096, 32, 128, 16384)
    assert s8.tensor_model_parallel_size == 2 and s8.sequence_parallel
    t = C.load_model_spec("tiny")
    assert t.tie_embeddings and t.vocab_size == 4096


def test_mup_helpers():
    s = C.load_model_spec("0.5b")
    assert s.mup_width_scale == 4.0
    assert math.isclose(s.mup_residual_scale, 1.4 / math.sqrt(24))
    assert s.emb_scale == 12.0
    off = s.replace(mup_enabled=False)
    assert off.mup_width_scale == 1.0 and off.mup_residual_scale == 1.0 and off.emb_scale == 1.0


def test_param_count_matches_0p5b():
    s = C.load_model_spec("0.5b")
    n = s.num_parameters()
    assert 505e6 < n < 515e6


def test_flops_formulas():
    s = C.load_model_spec("0.5b")
    hw = C.compute_training_flops(s, 4096, 4096)
    std = C.compute_training_flops_standard(s, 4096, 4096)
    assert hw > std
    # attention core is the only difference: 3 * tokens * L * 2*S*q_dim
    assert math.isclose(hw - std, 3 * 4096 * s.num_layers * 2 * 4096 * s.q_dim, rel_tol=1e-9)
    # published per-token figure for seq 4096 is 3.207 GFLOP (fwd+bwd, causal attention)
    per_tok = std / 4096
    assert 3.0e9 < per_tok < 3.4e9
    with_mtp = C.compute_training_flops(s, 4096, 4096, mtp_layers=1)
    assert with_mtp > hw


def test_engine_config_singleton_and_hooks():
    calls = []
    ec.register_reset_hook(lambda: calls.append(1))
    cfg = ec.EngineConfig(max_lr=1e-2)
    ec.set_global_config(cfg)
    assert ec.get_config().max_lr == 1e-2
    with pytest.raises(RuntimeError):
        ec.set_global_config(cfg)
    ec.reset_global_config()
    assert calls and ec.get_config().max_lr == ec.EngineConfig().max_lr


def test_engine_config_from_env_and_validation():
    cfg = ec.from_env({"MAX_LR": "0.01", "WGRAD_BUCKET_TARGET_ELEMS": "4096", "SHARDED_OPTIMIZER": "0",
                       "FT_COMM": "nccl"})
    assert cfg.max_lr == 0.01 and cfg.wgrad_bucket_target_elems == 4096
    assert cfg.sharded_optimizer is False and cfg.comm == "nccl"
    with pytest.raises(ValueError):
        ec.from_env({"PROFILE_RANGE": "1,3"})
    with pytest.raises(ValueError):
        ec.from_env({"FT_COMM": "mpi"})
    with pytest.raises(ValueError):
        ec.from_env({"WGRAD_BUCKET_TARGET_ELEMS": "0"})


def test_config_is_frozen():
    cfg = ec.EngineConfig()
    with pytest.raises(Exception):
        cfg.max_lr = 1.0


def test_from_spec_takes_training_defaults():
    s = C.load_model_spec("8b")
    cfg = ec.from_spec(s)
    assert cfg.max_lr == s.lr and cfg.tensor_parallel_size == 2 and cfg.wsd_decay_iters == 0


def test_legacy_field_names_translate_or_drop():
    """Names of the reference engines (0.5B engine_config.py:141-277, 8B engine_config.py:117-192)."""
    cfg, dropped = ec.from_legacy({"lr_warmup_iters": 10, "clip_grad": 0.5, "fp32_mode": True,
                                   "step_cuda_graph_full": True, "fused_ce": True, "custom_gemm": False,
                                   "max_lr": 1e-3})
    assert (cfg.warmup_iters, cfg.max_grad_norm, cfg.dtype) == (10, 0.5, "fp32")
    assert cfg.full_step_cuda_graph and cfg.max_lr == 1e-3
    assert dropped == ["custom_gemm", "fused_ce"]
    with pytest.raises(KeyError):
        ec.from_legacy({"no_such_field": 1})
    env = ec.from_env({"CLIP_GRAD": "2.0", "STEP_CUDA_GRAPH_FULL": "1", "LR_WARMUP_ITERS": "7"})
    assert (env.max_grad_norm, env.full_step_cuda_graph, env.warmup_iters) == (2.0, True, 7)


# every field name of the reference's two EngineConfig classes (0.5B engine_config.py:132-277,
# 8B engine_config.py:107-192): the names are the contract a config written for it relies on
_REFERENCE_FIELDS_05B = """fused_ops fuse_ce fuse_swiglu fuse_rmsnorm_residual fuse_rope fuse_rope_doc_aware
fuse_adam_sync fuse_gemm_pad fuse_direct_attn fuse_inplace_residual fuse_index_add_emb_bwd use_span_based_attn
fp32_mode unfused_mode te_rope fp32_allreduce fp32_grad_accum accum_stream_overlap multi_tensor_adam custom_gemm
forward_cuda_graph_warmup forward_cuda_graph_tol forward_cuda_graph_sanity forward_cuda_graph_sample_stride
step_cuda_graph_accum step_cuda_graph_reducer step_cuda_graph_full step_cuda_graph_full_warmup
step_cuda_graph_full_tol step_cuda_graph_full_sanity step_cuda_graph_nccl_opt step_cuda_graph_nccl_opt_warmup
step_cuda_graph_optimizer step_cuda_graph_optimizer_warmup use_fused_norm_bwd norm_bwd_nan_diag vocab_size""".split()
_REFERENCE_FIELDS_8B = """fused_rope fused_rope_pack fused_residual_rmsnorm fused_rope_qkv fused_attn_rmsnorm_bwd
fused_mlp_residual_rmsnorm fused_dw_reduce fused_rope_fp32cos ag_fwd_overlap adam_ag_pipeline gpu_norm_clip
fused_ce defer_wgrad_sync fused_swiglu dw_reduce_rows_per_block direct_attn dsl_attn_fwd rope_bhsd custom_gemm
padded_vocab_size lr_warmup_iters lr_wsd_decay_iters clip_grad""".split()


def test_every_field_name_of_the_reference_that_is_not_a_field_here_is_translated_or_dropped():
    import dataclasses
    own = {f.name for f in dataclasses.fields(ec.EngineConfig)}
    for name in _REFERENCE_FIELDS_05B + _REFERENCE_FIELDS_8B:
        assert name not in own
        assert (name in ec.LEGACY_FIELD_ALIASES) != (name in ec.LEGACY_NOOP_FIELDS), name
    cfg, dropped = ec.from_legacy({"step_cuda_graph_full_warmup": 5, "step_cuda_graph_full_tol": 0.25,
                                   "step_cuda_graph_full_sanity": False,
                                   "step_cuda_graph_optimizer_warmup": 3})
    assert (cfg.step_cuda_graph_warmup, cfg.step_cuda_graph_tol, cfg.step_cuda_graph_sanity) == (5, 0.25, False)
    assert dropped == ["step_cuda_graph_optimizer_warmup"]
    env = ec.from_env({"STEP_CUDA_GRAPH_FULL_WARMUP": "7", "STEP_CUDA_GRAPH_FULL_TOL": "0.5",
                       "STEP_CUDA_GRAPH_FULL_SANITY": "0"})
    assert (env.step_cuda_graph_warmup, env.step_cuda_graph_tol, env.step_cuda_graph_sanity) == (7, 0.5, False)
    both = ec.from_env({"STEP_CUDA_GRAPH_FULL_WARMUP": "7", "STEP_CUDA_GRAPH_WARMUP": "2"})
    assert both.step_cuda_graph_warmup == 2


def test_cli_accepts_reference_spellings(capsys):
    from forgetrain_b200.cli import build_parser
    a = build_parser().parse_args(["pretrain", "--clip-grad", "0.25", "--lr-warmup-iters", "5",
                                   "--no-fused-ce", "--custom-gemm", "--rs-buckets", "4"])
    assert a.legacy_clip_grad == 0.25 and a.legacy_lr_warmup_iters == 5
    assert a.noop_fused_ce is True and a.noop_custom_gemm is True and a.cfg_rs_buckets == 4


def test_env_table_is_in_step_with_the_code():
    from pathlib import Path
    doc = Path(ec.__file__).with_name("ENV_VARS.md").read_text()
    assert doc == ec.env_table_markdown()
    # every package switch in the whitelist is explained
    own = {n for n in ec.EXTERNAL_ENV_WHITELIST if n.startswith("FT_")}
    assert own == set(ec._SWITCH_NOTES)


def test_node_layout_decides_where_peer_memory_kernels_may_run():
    from forgetrain_b200.parallel.topology import node_layout
    assert node_layout(8, 8, 2) == (False, True)        # one node: everything may be fused
    assert node_layout(8, None, 2) == (False, True)     # no launcher information: one node
    assert node_layout(16, 8, 2) == (True, True)        # two nodes: TP pairs stay inside a node
    assert node_layout(16, 8, 8) == (True, True)
    assert node_layout(12, 6, 4) == (True, False)       # a TP group would straddle two nodes
    assert node_layout(32, 8, 16) == (True, False)
