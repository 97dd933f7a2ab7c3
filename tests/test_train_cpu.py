"""Training-loop helpers on CPU: muP coordinate check, optional logging (activation norms, gradient noise scale,
optimizer-state norms, parameter norms under ZeRO stage 3)."""
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = os.path.join(ROOT, "configs", "baseline", "tiny_sh2_cpu.yml")

def test_mup_coord_check(tmp_path):
    """Three widths, with and without muP: every block is recorded at every step; the CSV and the slopes come out."""
    import os
    from savanna_b200.train import mup_coord_check as cc
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tiny = os.path.join(root, "configs", "baseline", "tiny_sh2_cpu.yml")
    recs = cc.coord_check([tiny], {"global_num_gpus": 1, "seq_length": 64, "max_position_embeddings": 64,
                                   "train_micro_batch_size_per_gpu": 1, "gradient_accumulation_steps": 1},
                          powers=[2, 3, 4], steps=2)
    widths = sorted({r["width"] for r in recs})
    assert len(widths) == 3 and widths[1] == 2 * widths[0]
    assert {r["mup"] for r in recs} == {0, 1} and {r["step"] for r in recs} == {0, 1}
    assert {"embedding", "block0", "logits"} <= {r["module"] for r in recs}
    cc.write_csv(recs, str(tmp_path / "cc.csv"))
    assert len(open(tmp_path / "cc.csv").read().splitlines()) == len(recs) + 1
    s = cc.summarise(recs)
    assert set(s) == {"mup", "sp"} and "logits" in s["mup"] and all(v == v for v in s["sp"].values())


@pytest.mark.parametrize("stage", [1, 3])
def test_optional_logging(monkeypatch, stage):
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.parallel import state
    from savanna_b200.train.trainer import Trainer
    from savanna_b200.utils import logging as lg
    state.destroy_model_parallel()
    cfg = GlobalConfig.from_ymls([TINY], {"global_num_gpus": 1, "log_attn_norms": True, "log_hyena_norms": True,
                                          "log_gradient_noise_scale": True, "gradient_noise_scale_n_batches": 2,
                                          "log_optimizer_states": True, "log_param_norm": True, "log_grad_norm": True,
                                          "log_interval": 1, "zero_optimization": {"stage": stage}})
    tr = Trainer(cfg, load=False)
    seen = {}
    monkeypatch.setattr(lg, "tb_wandb_log", lambda key, value, it, *a, **k: seen.__setitem__(key, value))
    logger = lg.TrainingLogger(cfg, tr)

    def it():
        i = 0
        while True:
            yield {"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i)}
            i += 1
    d = it()
    for _ in range(3):
        loss = tr.train_step(d)
        logger.log_step(loss, 0.1)
    n_layers = cfg.num_layers
    acts = [k for k in seen if k.startswith("activations/")]
    assert len(acts) == n_layers and any("hyena_output_norm" in k for k in acts) and any("attention_output_norm" in k for k in acts)
    assert any(k.startswith("optimizer_state_norms/") for k in seen)
    assert any(k.startswith("param_norm/") for k in seen)
    if stage == 1:
        assert "train/noise_scale" in seen and any(k.startswith("grad_norm/") for k in seen)
    state.destroy_model_parallel()


def test_sequence_length_curriculum_schedules_and_training():
    """The three schedules' lengths, and a tiny run whose batches grow from 128 to the full 1024 tokens."""
    import os
    import torch
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.train.curriculum import CurriculumScheduler
    from savanna_b200.train.trainer import Trainer
    lin = CurriculumScheduler({"min_difficulty": 8, "max_difficulty": 64, "schedule_type": "fixed_linear",
                               "schedule_config": {"total_curriculum_step": 7, "difficulty_step": 8}})
    assert [lin.difficulty(s) for s in (1, 2, 4, 7, 100)] == [16, 24, 40, 64, 64]
    root = CurriculumScheduler({"min_difficulty": 8, "max_difficulty": 64, "schedule_type": "fixed_root",
                                "schedule_config": {"total_curriculum_step": 16, "difficulty_step": 8, "root_degree": 2}})
    assert [root.difficulty(s) for s in (1, 4, 16)] == [16, 32, 64]          # sqrt(1/16) = 1/4, sqrt(4/16) = 1/2
    disc = CurriculumScheduler({"min_difficulty": 8, "max_difficulty": 64, "schedule_type": "fixed_discrete",
                                "schedule_config": {"difficulty": [8, 32, 64], "max_step": [2, 5]}})
    assert [disc.difficulty(s) for s in (1, 2, 3, 5, 6)] == [8, 8, 32, 32, 64]
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = GlobalConfig.from_ymls([os.path.join(here, "configs", "baseline", "tiny_sh2_cpu.yml")], {
        "global_num_gpus": 1,
        "curriculum_learning": {"enabled": True, "curriculum_type": "seqlen", "min_difficulty": 128, "max_difficulty": 1024,
                                "schedule_type": "fixed_discrete",
                                "schedule_config": {"difficulty": [128, 256, 1024], "max_step": [1, 2]}}})
    assert cfg.seq_length == 1024
    tr = Trainer(cfg, load=False)
    seen = []
    real = tr.forward_step
    tr.forward_step = lambda b, *a, **k: (seen.append(b["tokens"].shape[1]), real(b, *a, **k))[1]

    def it():
        i = 0
        while True:
            yield {"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i)}
            i += 1
    d = it()
    losses = [float(tr.train_step(d)) for _ in range(3)]
    gas = cfg.gradient_accumulation_steps
    assert seen == [128] * gas + [256] * gas + [1024] * gas
    assert all(l == l for l in losses)
    assert tr.tokens_seen == cfg.train_batch_size * (128 + 256 + 1024)


def test_dynamic_loss_scaler_policy():
    from savanna_b200.train.loss_scaler import DynamicLossScaler, LossScaler
    s = DynamicLossScaler(initial_scale_power=4, window=3, hysteresis=2, min_scale=2.0)
    assert s.scale == 16.0
    s.update(True)                       # first overflow spends the hysteresis budget
    assert s.scale == 16.0
    s.update(True)                       # second one halves
    assert s.scale == 8.0
    s.update(True); s.update(True); s.update(True)
    assert s.scale == 2.0                # floor at min_scale
    for _ in range(3):
        s.update(False)
    assert s.scale == 4.0                # doubled `window` clean steps after the last overflow
    st = s.state_dict()
    t = DynamicLossScaler(initial_scale_power=10, window=3)
    t.load_state_dict(st)
    assert t.scale == 4.0 and t.iter == s.iter
    assert s.check(float("inf")) and s.check(float("nan")) and not s.check(1.5)
    fixed = LossScaler(128.0)
    assert fixed.check(float("inf")) and fixed.scale == 128.0


@pytest.mark.parametrize("stage", [1, 2])
def test_fp16_training_scales_the_loss_and_skips_overflowed_steps(stage):
    """fp16 run of the tiny model: same updates as without scaling while the gradients are finite (the scale cancels),
    and a step whose gradients overflow changes nothing but the scale."""
    import os
    import torch
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.train.trainer import Trainer
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = GlobalConfig.from_ymls([os.path.join(here, "configs", "baseline", "tiny_sh2_cpu.yml")], {
        "global_num_gpus": 1, "precision": "fp16",
        "fp16": {"enabled": True, "loss_scale": 0, "initial_scale_power": 8, "loss_scale_window": 2, "hysteresis": 1},
        "zero_optimization": {"stage": stage}})
    tr = Trainer(cfg, load=False)
    assert tr.loss_scaler is not None and tr.loss_scaler.scale == 256.0 and tr.optimizer.loss_scaler is tr.loss_scaler

    def it():
        i = 0
        while True:
            yield {"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i)}
            i += 1
    d = it()
    l0 = float(tr.train_step(d))
    assert l0 == l0 and tr.skipped_iters == 0 and float(tr.grad_norm) < 100.0       # the norm is reported unscaled
    before = [p.detach().clone() for p in tr.model.parameters()] if stage == 1 else None
    lr_before = tr.optimizer.param_groups[0]["lr"]
    tr.loss_scaler.scale = float("inf")                       # every gradient becomes inf / nan
    tr.train_step(d)
    assert tr.skipped_iters == 1 and tr.optimizer.overflow
    assert tr.loss_scaler.scale == float("inf") / 2 or tr.loss_scaler.scale == float("inf")
    if before is not None:
        assert all(torch.equal(a, b.detach()) for a, b in zip(before, tr.model.parameters()))
    assert tr.optimizer.param_groups[0]["lr"] == lr_before    # the schedule did not advance
    tr.loss_scaler.scale = 256.0
    l2 = float(tr.train_step(d))
    assert l2 == l2 and tr.skipped_iters == 1 and not tr.optimizer.overflow
    sd = tr.optimizer.state_dict()
    assert sd["dynamic_loss_scale"] is True and sd["loss_scaler"]["cur_scale"] == tr.loss_scaler.scale


def _tag_mask_by_loop(row, eod):
    """Row-by-row statement of the tag rule: pieces between '|' / end-of-document / row ends that hold '_', ';' or ' '."""
    L = len(row)
    keep = [1] * L
    cuts = sorted({0, L - 1} | {i for i, t in enumerate(row) if t in (124, eod)})
    for a, b in zip(cuts[:-1], cuts[1:]):
        if any(t in (95, 59, 32) for t in row[a:b]):
            lo = a + 1 if row[a] == eod else a
            hi = b - 1 if row[b] == eod else b
            for i in range(lo, hi + 1):
                keep[i] = 0
    for i, t in enumerate(row):
        if t in (64, 35):
            keep[i] = 0
    return keep


def test_control_and_phylogenetic_tag_loss_mask():
    import torch
    from savanna_b200.train.batch import mask_control_tags
    enc = lambda s: [0 if c == "$" else ord(c) for c in s]             # '$' stands for end-of-document (token 0)
    rows = [
        "ACGT|d__Bacteria;p__Firmicutes|ACGTACGT$ACGT@ACGT",            # a whole tag, a control character
        "teria;s__coli|ACGTACGTACGT#ACGT|d__Archaea;p__Eury",            # tags cut by both sample boundaries
        "ACGTACGTACGTACGTACGTACGTACGTACGTACGTACGTACGTACGTAC",            # plain sequence
        "ACGT$|d__B;c__X|ACGT$ACGT|r__Z|$ACGTACGTACGTACGT|ACG",          # tags next to end-of-document tokens, a lone bar
    ]
    L = max(len(r) for r in rows)
    rows = [r.ljust(L, "A") for r in rows]
    tok = torch.tensor([enc(r) for r in rows])
    got = mask_control_tags(tok, torch.ones(tok.shape), eod=0)
    want = torch.tensor([_tag_mask_by_loop(enc(r), 0) for r in rows], dtype=torch.float32)
    assert torch.equal(got, want), (got - want).nonzero().tolist()
    assert got[0, :4].sum() == 4 and got[0, 4:31].sum() == 0 and got[0, 31:39].sum() == 8      # DNA kept, tag dropped
    assert got[1, :14].sum() == 0 and got[1, 14] == 1                                           # leading partial tag
    assert got[2].sum() == L


def test_masked_strategies_follow_their_rules_and_train():
    import math
    import os
    import torch
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.train import batch as bm
    from savanna_b200.train.trainer import Trainer
    g = torch.Generator().manual_seed(0)
    clean = acgt_batch(4, 199, seed=3)[:, :200]
    clean[:, 50] = 0                                                     # an end-of-document token per row
    out, sel = bm._mlm_corrupt(clean, 512, eod=0, eod_mask_loss=True, gen=g)
    n = math.ceil(0.15 * 200)
    assert all(n - 1 <= int(s) <= n for s in sel.sum(1)) and float(sel[:, 50].sum()) == 0
    changed = out != clean
    assert bool((changed <= sel.bool()).all()) and float((out[sel.bool()] == bm.MASK_TOKEN_ID).float().mean()) > 0.6
    out, sel = bm._span_corrupt(clean.clone(), 512, randomize=False, gen=g)
    assert all(10 <= int(s) <= 30 for s in sel.sum(1)) and bool((out[sel.bool()] == bm.MASK_TOKEN_ID).all())
    assert bool((out[~sel.bool()] == bm._dna_only(clean)[~sel.bool()]).all())
    runs = (sel[:, 1:] > sel[:, :-1]).sum(1) + sel[:, 0]
    assert all(int(r) >= 2 for r in runs)                                # several spans, not one block
    out, sel, t = bm._oadm_corrupt(clean, gen=g)
    assert torch.equal(sel.sum(1).long(), (200 - t + 1).clamp(max=200)) and bool((out[sel.bool()] == bm.MASK_TOKEN_ID).all())
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for strategy in ("MLM", "SPAN", "SPAN_R", "OADM"):
        cfg = GlobalConfig.from_ymls([os.path.join(here, "configs", "baseline", "tiny_sh2_cpu.yml")],
                                     {"global_num_gpus": 1, "pretraining_strategy": strategy, "mask_loss_control_tags": True})
        assert cfg.causal is False
        tr = Trainer(cfg, load=False)
        d = iter([{"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i)} for i in range(64)])
        losses = [float(tr.train_step(d)) for _ in range(4)]
        assert all(l == l for l in losses) and losses[-1] < losses[0], (strategy, losses)


def test_annealing_lr_values_including_the_saturated_tail():
    import math
    from savanna_b200.train.lr import AnnealingLR

    class Opt:
        param_groups = [{"lr": 0.0}, {"lr": 0.0, "fixed_lr": True, "lr_mult": 0.5}]
    s = AnnealingLR(Opt, start_lr=1.0, warmup_iter=10, total_iters=100, decay_style="cosine", min_lr=0.1)

    def want(i):
        n = min(i, 90)
        if i <= 10:
            return max(n / 10, 0.0) if i else 0.0
        return max(0.5 * (math.cos(math.pi * (n - 10) / 100) + 1), 0.1)
    for i in (0, 1, 5, 10, 11, 50, 90, 95, 100, 150):
        s.step(i)
        got = Opt.param_groups[0]["lr"]
        ref = want(i) if i > 10 else i / 10
        assert abs(got - ref) < 1e-12, (i, got, ref)
        own = 0.5 * s.factor()
        assert abs(Opt.param_groups[1]["lr"] - (own if i <= 10 else max(own, 0.1))) < 1e-12
    s.step(95)
    a = Opt.param_groups[0]["lr"]
    s.step(100)
    assert Opt.param_groups[0]["lr"] == a                     # held over the last `warmup_iter` steps
    for style, f in (("linear", lambda n: (100 - n) / 100), ("exponential", lambda n: math.exp(-0.693 * n / 100)),
                     ("constant", lambda n: 1.0)):
        t = AnnealingLR(Opt, 2.0, 10, 100, style, min_lr=0.0)
        t.step(60)
        assert abs(Opt.param_groups[0]["lr"] - 2.0 * f(50)) < 1e-12


def test_fp16_loss_scale_survives_checkpoint_resume(tmp_path):
    """The dynamic scaler's state travels in the optimizer checkpoint: a resumed run continues at the saved scale."""
    import os
    from savanna_b200.ckpt import save_checkpoint
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.parallel import state
    from savanna_b200.train.trainer import Trainer
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    save = str(tmp_path / "ck")
    over = {"global_num_gpus": 1, "precision": "fp16", "save": save, "load": save,
            "fp16": {"enabled": True, "loss_scale": 0, "initial_scale_power": 8, "loss_scale_window": 2, "hysteresis": 1}}
    cfg = GlobalConfig.from_ymls([os.path.join(here, "configs", "baseline", "tiny_sh2_cpu.yml")], over)
    tr = Trainer(cfg, load=False)
    d = iter([{"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i)} for i in range(16)])
    for _ in range(4):
        tr.train_step(d)                                   # two clean windows: 256 -> 512 -> 1024
    scale, it = tr.loss_scaler.scale, tr.loss_scaler.iter
    assert scale > 256.0
    save_checkpoint(tr)
    state.destroy_model_parallel()
    t2 = Trainer(GlobalConfig.from_ymls([os.path.join(here, "configs", "baseline", "tiny_sh2_cpu.yml")], over), load=True)
    assert t2.iteration == 4 and t2.loss_scaler.scale == scale and t2.loss_scaler.iter == it


def test_curriculum_continues_after_resume(tmp_path):
    """The curriculum length depends on the iteration only: a resumed run picks the schedule up where it stopped."""
    import os
    from savanna_b200.ckpt import save_checkpoint
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.parallel import state
    from savanna_b200.train.trainer import Trainer
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    save = str(tmp_path / "ck")
    over = {"global_num_gpus": 1, "save": save, "load": save,
            "curriculum_learning": {"enabled": True, "curriculum_type": "seqlen", "min_difficulty": 128, "max_difficulty": 1024,
                                    "schedule_type": "fixed_discrete",
                                    "schedule_config": {"difficulty": [128, 512, 1024], "max_step": [2, 4]}}}
    yml = [os.path.join(here, "configs", "baseline", "tiny_sh2_cpu.yml")]
    cfg = GlobalConfig.from_ymls(yml, over)
    tr = Trainer(cfg, load=False)
    d = iter([{"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i)} for i in range(32)])
    for _ in range(3):
        tr.train_step(d)
    assert cfg.curriculum_seqlen == 512 and tr.tokens_seen == cfg.train_batch_size * (128 + 128 + 512)
    save_checkpoint(tr)
    state.destroy_model_parallel()
    cfg2 = GlobalConfig.from_ymls(yml, over)
    t2 = Trainer(cfg2, load=True)
    assert t2.iteration == 3 and t2.tokens_seen == tr.tokens_seen
    t2.train_step(d)
    assert cfg2.curriculum_seqlen == 512
    t2.train_step(d)
    assert cfg2.curriculum_seqlen == 1024
