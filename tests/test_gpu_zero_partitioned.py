"""ZeRO stages 2 and 3 on the GPU kernels: the per-block gather / release cycle around this framework's own autograd
nodes (fp8 projections with cached quantised weights, in-place weight-gradient accumulation from GEMM epilogues,
activation checkpointing).  One GPU is enough for the cycle itself (a one-rank partition group); the two-GPU run adds
the NCCL all-gathers and reduce-scatters."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0

_WIDE = {"hidden_size": 512, "num_attention_heads": 4, "num_groups_hyena": 512, "num_groups_hyena_medium": 32,
         "num_groups_hyena_short": 32, "hidden_dropout": 0.0, "gradient_accumulation_steps": 2}
_FP8 = {"use_fp8_linears": True, "use_fp8_input_projections": True, "use_fp8_output_projections": True,
        "use_fp8_mlp_projections": True}


def _losses(world, rank, over, n=5):
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.ops import cuda_ops
    from savanna_b200.parallel import state
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = {"global_num_gpus": world, "train_micro_batch_size_per_gpu": 1}
    base.update(over)
    cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_gpu.yml")], base)
    tr = Trainer(cfg, load=False)

    def it():
        i = 0
        while True:
            yield {"text": acgt_batch(1, cfg.seq_length, seed=100 * rank + i, pin=True)}
            i += 1
    d = it()
    out = [float(tr.train_step(d)) for _ in range(n)]
    cuda_ops.check_status()
    opt = tr.optimizer
    if hasattr(opt, "units"):
        blocks = [f for u in opt.units[1:] for f in u.flats]
        assert blocks and all(f.gfull.untyped_storage().size() == 0 for f in blocks)
        if opt.stage == 3:
            assert all(f.full.untyped_storage().size() == 0 for f in blocks)
            ev = tr.evaluate(d, iters=1)                      # a no-grad forward gathers and releases too
            assert ev["lm_loss"] == ev["lm_loss"]
    state.destroy_model_parallel()
    return out


def _close(got, want, tol=2e-2):
    for a, b in zip(got, want):
        assert abs(a - b) < tol * max(1.0, abs(b)), (got, want)
    assert got[-1] < got[0], got


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("stage,ckpt_layers", [(2, 0), (3, 0), (3, 2)])
def test_partitioned_stages_match_stage1_one_gpu(stage, ckpt_layers, fp8):
    over = dict(_WIDE, **(_FP8 if fp8 else {}))
    want = _losses(1, 0, dict(over, zero_optimization={"stage": 1}))
    extra = {"checkpoint_activations": True, "checkpoint_num_layers": ckpt_layers} if ckpt_layers else {}
    got = _losses(1, 0, dict(over, zero_optimization={"stage": stage}, **extra))
    _close(got, want)


def _w_two_gpus(rank, world, over, stage_over):
    want = _losses(world, rank, dict(over, zero_optimization={"stage": 1}, comm_path="nccl"))
    got = _losses(world, rank, dict(over, **stage_over))
    _close(got, want)


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("stage", [2, 3])
def test_partitioned_stages_match_stage1_two_gpus(stage):
    from test_gpu_multi import _spawn_args
    over = dict(_WIDE, **_FP8)
    _spawn_args(_w_two_gpus, 2, over, {"zero_optimization": {"stage": stage}, "checkpoint_activations": True,
                                       "checkpoint_num_layers": 2})


@pytest.mark.parametrize("over", [
    {"zero_optimization": {"stage": 1, "offload_optimizer": {"device": "cpu", "pin_memory": True}}},
    {"zero_optimization": {"stage": 3, "offload_param": {"device": "cpu"}}},
    {"zero_optimization": {"stage": 3, "offload_optimizer": {"device": "cpu"}, "offload_param": {"device": "cpu"}}},
    {"zero_optimization": {"stage": 1}, "checkpoint_activations": True, "checkpoint_num_layers": 2, "checkpoint_in_cpu": True},
], ids=["offload_optimizer", "offload_param", "offload_both_stage3", "checkpoint_in_cpu"])
def test_host_offload_paths_match_the_resident_run(over):
    """Optimizer state on the host (update on the CPU), parameter shards on the host (stage 3) and checkpointed chunk
    inputs on the host: same loss trace as the all-on-device ZeRO-1 run."""
    want = _losses(1, 0, dict(_WIDE, zero_optimization={"stage": 1}))
    got = _losses(1, 0, dict(_WIDE, **over))
    _close(got, want)


def test_fp16_precision_with_dynamic_loss_scale_on_the_gpu():
    """fp16 parameters and activations (the operators then run their PyTorch statements: the own kernels are bf16 / fp32)
    with the dynamic loss scaler: starts at the bf16 run's loss and trains."""
    want = _losses(1, 0, dict(_WIDE, zero_optimization={"stage": 1}), n=4)
    got = _losses(1, 0, dict(_WIDE, zero_optimization={"stage": 1}, precision="fp16",
                             fp16={"enabled": True, "loss_scale": 0, "initial_scale_power": 10, "loss_scale_window": 100,
                                   "hysteresis": 2}), n=4)
    assert abs(got[0] - want[0]) < 0.05, (got, want)
    assert got[-1] < got[0] - 0.2, got


def test_weight_decay_groups_with_mixed_precision_flats():
    """Weight decay on: the decayed group holds bf16 weights and fp32 filter parameters side by side, the undecayed one
    norms and biases, the Hyena-MR filter has its own learning rate.  Stage 3 reproduces stage 1 and both train."""
    over = dict(_WIDE, **_FP8, weight_decay=0.1, lr_medium_hyena=1e-4)
    want = _losses(1, 0, dict(over, zero_optimization={"stage": 1}))
    got = _losses(1, 0, dict(over, zero_optimization={"stage": 3}))
    _close(got, want)
