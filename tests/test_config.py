import glob
import os

import pytest
import yaml

from savanna_b200.config import ConfigError, GlobalConfig, batch_triple, expand_operator_types
from savanna_b200.config.schema import FIELDS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = os.path.join(ROOT, "configs", "baseline", "tiny_sh2_cpu.yml")


def test_tiny_config_loads():
    cfg = GlobalConfig.from_ymls([TINY], {"global_num_gpus": 1})
    assert cfg.operator_config == ["hyena_se", "hyena_mr", "hyena", "flash_v2"]
    assert cfg.ffn_size == 688
    assert cfg.train_batch_size == 2 and cfg.gradient_accumulation_steps == 1
    assert cfg.precision == "fp32" and cfg.zero_stage == 0


def test_dash_underscore_and_unknown_key(tmp_path):
    p = tmp_path / "a.yml"
    p.write_text(yaml.safe_dump({"num-layers": 2, "hidden_size": 64, "num_attention_heads": 2, "seq-length": 32,
                                 "max_position_embeddings": 32, "train_micro_batch_size_per_gpu": 1}))
    cfg = GlobalConfig.from_ymls([str(p)], {"global_num_gpus": 1})
    assert cfg.num_layers == 2 and cfg.seq_length == 32
    q = tmp_path / "b.yml"
    q.write_text(yaml.safe_dump({"not_a_key": 1}))
    with pytest.raises(ConfigError):
        GlobalConfig.from_ymls([str(p), str(q)], {"global_num_gpus": 1})


def test_duplicate_key_across_files(tmp_path):
    a, b = tmp_path / "a.yml", tmp_path / "b.yml"
    a.write_text("{num_layers: 2, train_micro_batch_size_per_gpu: 1}")
    b.write_text("{num-layers: 3}")
    with pytest.raises(ConfigError):
        GlobalConfig.from_ymls([str(a), str(b)], {"global_num_gpus": 1})


def test_type_validation():
    with pytest.raises(ConfigError):
        GlobalConfig.from_dict({"train_micro_batch_size_per_gpu": 1, "num_layers": "two", "global_num_gpus": 1})
    with pytest.raises(ConfigError):
        GlobalConfig.from_dict({"train_micro_batch_size_per_gpu": 1, "norm": "batchnorm", "global_num_gpus": 1})


def test_batch_triple():
    assert batch_triple(4, train_batch=64, micro_batch=2) == (64, 2, 8)
    assert batch_triple(4, micro_batch=2, grad_acc=3) == (24, 2, 3)
    assert batch_triple(8, train_batch=64) == (64, 8, 1)
    with pytest.raises(ConfigError):
        batch_triple(4, train_batch=10, micro_batch=3, grad_acc=1)


def test_operator_expansion():
    assert expand_operator_types([[["a", "b"], 2], [["c"], 1]], 5) == ["a", "b", "a", "b", "c"]
    assert expand_operator_types([[["a", "b"], "all"]], 5) == ["a", "b", "a", "b", "a"]


def test_parallel_sizes_and_save_iters():
    cfg = GlobalConfig.from_ymls([TINY], {"global_num_gpus": 8, "model_parallel_size": 2, "context_parallel_size": 2,
                                          "use_cp_hyena": True, "use_cp_ring": True,
                                          "operator_config": ["hyena_se", "hyena_mr", "hyena", "ring"],
                                          "checkpoint_factor": 4, "train_iters": 10, "extra_save_iters": [1]})
    assert cfg.dp_world_size == 2 and cfg.train_batch_size == 4
    assert cfg.save_iters == [1, 4, 8]
    with pytest.raises(ConfigError):   # flash_v2 has no context-parallel algorithm
        GlobalConfig.from_ymls([TINY], {"global_num_gpus": 2, "context_parallel_size": 2, "use_cp_hyena": True})


def test_encode_decode_roundtrip():
    cfg = GlobalConfig.from_ymls([TINY], {"global_num_gpus": 1})
    args = cfg.get_deepspeed_main_args() if cfg.user_script else None
    cfg.user_script = "train.py"
    args = cfg.get_deepspeed_main_args()
    i = args.index("--megatron_config")
    cfg2 = GlobalConfig.consume_global_config(["--megatron_config", args[i + 1]])
    for k in FIELDS:
        if k in ("rank", "local_rank", "world_size", "user_script"):
            continue
        assert getattr(cfg, k) == getattr(cfg2, k), k


def test_engine_config_has_zero_and_batch():
    cfg = GlobalConfig.from_ymls([os.path.join(ROOT, "configs", "baseline", "evo2_7b_8k.yml")], {"global_num_gpus": 8})
    ec = cfg.engine_config
    assert ec["zero_optimization"]["stage"] == 1 and ec["train_batch_size"] == 64 and ec["bf16"]["enabled"]
    assert cfg.ffn_size == 11264


# a checkout of the reference next to this repository (or SAVANNA_REFERENCE_DIR) provides its YAMLs
REFERENCE = os.environ.get("SAVANNA_REFERENCE_DIR", os.path.join(os.path.dirname(ROOT), "reference"))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "configs")), reason="reference configs not available")
def test_reference_model_configs_load():
    """Every current Evo 2 model YAML of the reference parses with this schema."""
    rc = os.path.join(REFERENCE, "configs")
    paths = glob.glob(os.path.join(rc, "7b-context-ext/model_configs/*.yml")) + \
        glob.glob(os.path.join(rc, "40b/model_configs/pretrain/*.yml")) + \
        glob.glob(os.path.join(rc, "quickstart/*.yml")) + glob.glob(os.path.join(rc, "test/*.yml"))
    assert paths
    bad = []
    for p in paths:
        try:
            GlobalConfig.from_ymls([p], {"global_num_gpus": 2048})
        except yaml.YAMLError:
            continue                      # a few reference files are not valid YAML
        except ConfigError as exc:
            msg = str(exc)
            if "context parallelism needs" in msg or "no context-parallel algorithm" in msg or "attention_config" in msg:
                continue                  # rejected by the reference's own validation as well
            bad.append((p, msg))
    assert not bad, bad[:5]


def test_block_scaled_fp8_recipe_key():
    from savanna_b200.config import ConfigError, GlobalConfig
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tiny = os.path.join(root, "configs", "baseline", "tiny_sh2_cpu.yml")
    cfg = GlobalConfig.from_ymls([tiny], {"global_num_gpus": 1, "fp8_recipe": "mxfp8", "use_fp8_linears": True})
    assert cfg.fp8_recipe == "mxfp8"
    assert GlobalConfig.from_ymls([tiny], {"global_num_gpus": 1}).fp8_recipe == "delayed"
    import pytest
    # with tensor + sequence parallelism the block-scaled projections run behind NCCL collectives (no fused kernel)
    tp = GlobalConfig.from_ymls([tiny], {"global_num_gpus": 2, "model_parallel_size": 2, "sequence_parallel": True,
                                         "fp8_recipe": "mxfp8", "use_fp8_linears": True})
    assert tp.fp8_recipe == "mxfp8" and tp.sequence_parallel
    with pytest.raises(ConfigError):
        GlobalConfig.from_ymls([tiny], {"global_num_gpus": 1, "fp8_recipe": "nvfp4"})
