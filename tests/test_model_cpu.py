"""Tiny StripedHyena 2 on CPU (configs/baseline/tiny_sh2_cpu.yml): trains, is deterministic, checkpoints and resumes."""
import os

import pytest
import torch

from savanna_b200.config import GlobalConfig
from savanna_b200.data.synthetic import acgt_batch
from savanna_b200.train.trainer import Trainer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = os.path.join(ROOT, "configs", "baseline", "tiny_sh2_cpu.yml")


def _cfg(**over):
    base = {"global_num_gpus": 1}
    base.update(over)
    return GlobalConfig.from_ymls([TINY], base)


def _iter(cfg, start=0):
    def it():
        i = start
        while True:
            yield {"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i)}
            i += 1
    return it()


def test_state_dict_keys_follow_reference_layout():
    cfg = _cfg()
    tr = Trainer(cfg, load=False)
    keys = set(tr.model.state_dict().keys())
    for k in ("sequential.0.word_embeddings.weight", "sequential.2.input_layernorm.weight",
              "sequential.2.mixer.dense_projection.weight", "sequential.2.mixer.hyena_proj_conv.short_conv_weight",
              "sequential.2.mixer.mixer.short_conv.short_conv_weight", "sequential.3.mixer.mixer.filter.h",
              "sequential.3.mixer.mixer.filter.decay", "sequential.3.mixer.mixer.conv_bias",
              "sequential.4.mixer.mixer.filter.gamma", "sequential.4.mixer.mixer.filter.R", "sequential.4.mixer.mixer.filter.p",
              "sequential.5.mixer.dense.weight", "sequential.5.mixer.dense.bias", "sequential.2.mlp.w1.weight",
              "sequential.2.mlp.w2.weight", "sequential.2.mlp.w3.weight", "sequential.7.norm.weight"):
        assert k in keys, k


def test_loss_decreases_and_is_deterministic():
    losses = []
    for _ in range(2):
        cfg = _cfg()
        tr = Trainer(cfg, load=False)
        d = _iter(cfg)
        losses.append([float(tr.train_step(d)) for _ in range(10)])
    assert losses[0] == losses[1]
    assert losses[0][-1] < losses[0][0] - 1.5
    assert 5.5 < losses[0][0] < 6.6          # ~ln(512) at initialisation


def test_golden_loss_trace():
    """The 10-step loss trace of the tiny CPU model (seed 0) stays what it was when first recorded."""
    cfg = _cfg()
    tr = Trainer(cfg, load=False)
    d = _iter(cfg)
    got = [float(tr.train_step(d)) for _ in range(10)]
    golden_path = os.path.join(ROOT, "tests", "golden", "tiny_sh2_cpu_loss.txt")
    golden = [float(x) for x in open(golden_path).read().split()]
    for a, b in zip(got, golden):
        assert abs(a - b) < 5e-3 * max(1.0, abs(b)), (got, golden)


def test_gradient_accumulation_matches_large_batch():
    cfg1 = _cfg(train_micro_batch_size_per_gpu=2, gradient_accumulation_steps=1)
    t1 = Trainer(cfg1, load=False)
    full = acgt_batch(2, cfg1.seq_length, seed=0)
    l1 = float(t1.train_step(iter([{"text": full}])))
    cfg2 = _cfg(train_micro_batch_size_per_gpu=1, gradient_accumulation_steps=2)
    t2 = Trainer(cfg2, load=False)
    l2 = float(t2.train_step(iter([{"text": full[:1]}, {"text": full[1:]}])))
    assert abs(l1 - l2) < 1e-4
    # the first Adam step moves every weight by ~lr*sign(grad): rounding can flip the sign of a near-zero gradient,
    # so compare on average instead of element-wise
    for a, b in zip(t1.model.parameters(), t2.model.parameters()):
        assert (a - b).abs().mean() < 2e-5, "parameters differ after one step"


def test_activation_checkpointing_same_result():
    ca, cb = _cfg(), _cfg(checkpoint_activations=True, checkpoint_num_layers=2)
    ta, tb = Trainer(ca, load=False), Trainer(cb, load=False)
    la = [float(ta.train_step(_iter(ca))) for _ in range(2)]
    lb = [float(tb.train_step(_iter(cb))) for _ in range(2)]
    assert all(abs(a - b) < 1e-5 for a, b in zip(la, lb))


def test_checkpoint_in_cpu_same_result_and_inputs_leave_through_the_hooks(monkeypatch):
    """`checkpoint_in_cpu`: the chunk inputs pass through the host-offload hooks (counted) and training is unchanged."""
    seen = []
    real = torch.autograd.graph.save_on_cpu

    class Counting(real):
        def __init__(self, *a, **k):
            super().__init__(*a, **k)
            pack = self.pack_hook

            def counted(t):
                seen.append(tuple(t.shape))
                return pack(t)
            self.pack_hook = counted
    monkeypatch.setattr(torch.autograd.graph, "save_on_cpu", Counting)
    ca, cb = _cfg(), _cfg(checkpoint_activations=True, checkpoint_num_layers=2, checkpoint_in_cpu=True)
    ta, tb = Trainer(ca, load=False), Trainer(cb, load=False)
    la = [float(ta.train_step(_iter(ca))) for _ in range(2)]
    lb = [float(tb.train_step(_iter(cb))) for _ in range(2)]
    assert all(abs(a - b) < 1e-5 for a, b in zip(la, lb))
    assert any(len(sh) == 3 and sh[-1] == cb.hidden_size for sh in seen), seen


def test_checkpoint_resume_bit_exact(tmp_path):
    save = str(tmp_path / "ckpt")
    cfg = _cfg(save=save, train_iters=6)
    tr = Trainer(cfg, load=False)
    d = _iter(cfg)
    ref = [float(tr.train_step(d)) for _ in range(6)]
    # second run: 3 steps, save, new trainer resumes and runs 3 more
    cfg_a = _cfg(save=save, train_iters=6)
    ta = Trainer(cfg_a, load=False)
    da = _iter(cfg_a)
    first = [float(ta.train_step(da)) for _ in range(3)]
    from savanna_b200.ckpt import read_global_step, save_checkpoint
    save_checkpoint(ta)
    assert read_global_step(save) == 3
    assert os.path.isfile(os.path.join(save, "global_step3", "mp_rank_00_model_states.pt"))
    assert os.path.isfile(os.path.join(save, "global_step3", "zero_pp_rank_0_mp_rank_00_optim_states.pt"))
    assert open(os.path.join(save, "latest")).read() == "global_step3"
    cfg_b = _cfg(save=save, load=save, train_iters=6)
    tb = Trainer(cfg_b, load=True)
    assert tb.iteration == 3
    db = _iter(cfg_b, start=3)
    second = [float(tb.train_step(db)) for _ in range(3)]
    assert first + second == ref


def test_checkpoint_file_contents(tmp_path):
    save = str(tmp_path / "ckpt")
    cfg = _cfg(save=save)
    tr = Trainer(cfg, load=False)
    tr.train_step(_iter(cfg))
    from savanna_b200.ckpt import save_checkpoint
    d = save_checkpoint(tr)
    ms = torch.load(os.path.join(d, "mp_rank_00_model_states.pt"), weights_only=False)
    for k in ("module", "param_shapes", "buffer_names", "shared_params", "ds_config", "ds_version", "dp_world_size",
              "mp_world_size", "iteration", "args", "data_loading", "lr_scheduler", "torch_rng_state"):
        assert k in ms, k
    assert ms["iteration"] == 1 and ms["data_loading"]["train_data_token_index"] == cfg.train_batch_size * cfg.seq_length
    osd = torch.load(os.path.join(d, "zero_pp_rank_0_mp_rank_00_optim_states.pt"), weights_only=False)["optimizer_state_dict"]
    assert osd["zero_stage"] == 1 and "single_partition_of_fp32_groups" in osd and "base_optimizer_state" in osd
    assert os.path.isfile(os.path.join(d, "configs", "tiny_sh2_cpu.yml"))


def test_read_global_step_prefers_older(tmp_path):
    from savanna_b200.ckpt import read_global_step
    root = tmp_path
    (root / "global_step10").mkdir()
    (root / "global_step20").mkdir()
    (root / "latest").write_text("global_step20")
    assert read_global_step(str(root)) == 20
    (root / "latest").write_text("global_step30")      # latest points past what is on disk
    assert read_global_step(str(root)) == 20
    (root / "latest").write_text("global_step10")      # a newer, possibly half-written directory exists
    assert read_global_step(str(root)) == 10


def test_keep_last_n(tmp_path):
    save = str(tmp_path / "c")
    cfg = _cfg(save=save, keep_last_n_checkpoints=2)
    tr = Trainer(cfg, load=False)
    from savanna_b200.ckpt import save_checkpoint
    d = _iter(cfg)
    for _ in range(3):
        tr.train_step(d)
        save_checkpoint(tr)
    dirs = sorted(p for p in os.listdir(save) if p.startswith("global_step"))
    assert dirs == ["global_step2", "global_step3"]


def test_save_retain_interval_selects_the_uploaded_checkpoints(tmp_path):
    """Every save lands on the local disk; only iterations that are multiples of `save_retain_interval` reach the stores."""
    save, mirror = str(tmp_path / "c"), str(tmp_path / "mirror")
    cfg = _cfg(save=save, save_retain_interval=2, checkpoint_stores=[{"storage_type": "posix", "location": mirror}])
    tr = Trainer(cfg, load=False)
    from savanna_b200.ckpt import save_checkpoint
    d = _iter(cfg)
    for _ in range(4):
        tr.train_step(d)
        save_checkpoint(tr)
    assert sorted(p for p in os.listdir(save) if p.startswith("global_step")) == [f"global_step{i}" for i in (1, 2, 3, 4)]
    assert sorted(os.listdir(mirror)) == ["global_step2", "global_step4"]


def test_checkpoint_validation_with_forward_pass(tmp_path):
    """The logits of a fixed input are stored with the checkpoint and reproduced after loading; a checkpoint whose
    stored logits do not belong to its weights is refused."""
    from savanna_b200.ckpt import load_checkpoint, save_checkpoint
    save = str(tmp_path / "c")
    cfg = _cfg(save=save, load=save, checkpoint_validation_with_forward_pass=True)
    tr = Trainer(cfg, load=False)
    tr.train_step(_iter(cfg))
    d = save_checkpoint(tr)
    path = os.path.join(d, "mp_rank_00_model_states.pt")
    ms = torch.load(path, weights_only=False)
    assert ms["checkpoint_validation_logits"].shape == (cfg.seq_length, cfg.padded_vocab_size)
    t2 = Trainer(cfg, load=True)                                  # validates while loading
    assert t2.iteration == 1
    ms["checkpoint_validation_logits"] = ms["checkpoint_validation_logits"] + 1.0      # what another model would have stored
    torch.save(ms, path)
    with pytest.raises(RuntimeError, match="does not reproduce"):
        Trainer(cfg, load=True)


def test_finetune_loads_module_only(tmp_path):
    save = str(tmp_path / "c")
    cfg = _cfg(save=save)
    tr = Trainer(cfg, load=False)
    d = _iter(cfg)
    tr.train_step(d)
    from savanna_b200.ckpt import save_checkpoint
    save_checkpoint(tr)
    cfg2 = _cfg(load=save, finetune=True)
    t2 = Trainer(cfg2, load=True)
    assert t2.iteration == 0
    for a, b in zip(tr.model.parameters(), t2.model.parameters()):
        assert torch.equal(a, b)
    assert t2.optimizer.step_count == 0


def test_warmstart_loads_state_but_restarts_the_count(tmp_path):
    """`warmstart`: module and optimizer state come from the checkpoint, the iteration and the data cursor start at 0."""
    save = str(tmp_path / "c")
    cfg = _cfg(save=save)
    tr = Trainer(cfg, load=False)
    d = _iter(cfg)
    for _ in range(2):
        tr.train_step(d)
    from savanna_b200.ckpt import save_checkpoint
    save_checkpoint(tr)
    t2 = Trainer(_cfg(load=save, warmstart=True), load=True)
    assert t2.iteration == 0 and t2.tokens_seen == 0
    for a, b in zip(tr.model.parameters(), t2.model.parameters()):
        assert torch.equal(a, b)
    assert t2.optimizer.step_count == tr.optimizer.step_count == 2
    for ga, gb in zip(tr.optimizer.groups, t2.optimizer.groups):
        assert torch.equal(ga.exp_avg, gb.exp_avg) and torch.equal(ga.master, gb.master)


def test_score_bias_position_embeddings_on_the_global_operator():
    """`pos_emb: alibi` and `pos_emb: rpe` add a per-head bias to the attention scores of the legacy `global` operator:
    bucket law of the relative-position table, head split over tensor-parallel ranks, and a model step."""
    from savanna_b200.models.rope import AliBi, RelativePositionBias
    rpe = RelativePositionBias(2.0, causal=True, num_buckets=32, max_distance=128, heads=4)
    rel = torch.tensor([[0, -1, -15, -16, -64, -127, -128, -5000, 3]])
    b = rpe.bucket(rel)[0].tolist()
    assert b[:3] == [0, 1, 15]                       # exact below num_buckets / 2
    assert b[3] == 16 and b[4] > b[3] and b[5] <= 31 and b[6] == 31 and b[7] == 31
    assert b[8] == 0                                 # future positions collapse to bucket 0 in the causal form
    bias = rpe(6, 6)
    assert bias.shape == (4, 6, 6)
    assert torch.allclose(bias[:, 3, 1], rpe.weight[2].float() * 2.0)
    half = RelativePositionBias(1.0, heads=4, mp_size=2, mp_rank=1)
    assert half.weight.shape == (32, 2)
    ali = AliBi(8)
    assert torch.allclose(ali.bias(torch.arange(4), torch.arange(4))[0, 3, 1], ali.slopes[0] * -2.0)
    for pe in ("alibi", "rpe"):
        cfg = _cfg(operator_config=[[["global"], 2]], num_layers=2, pos_emb=pe)
        tr = Trainer(cfg, load=False)
        d = _iter(cfg)
        losses = [float(tr.train_step(d)) for _ in range(4)]
        assert losses[-1] < losses[0], (pe, losses)
    with pytest.raises(NotImplementedError, match="global"):
        Trainer(_cfg(operator_config=[[["flash_v2"], 2]], num_layers=2, pos_emb="alibi"), load=False)


def test_tokentype_embeddings_can_be_added_after_construction():
    from savanna_b200.models.embedding import Embedding
    from savanna_b200.models.init_functions import get_init_methods
    cfg = _cfg()
    Trainer(cfg, load=False)                                   # brings up the (single-rank) parallel state
    init, _ = get_init_methods(cfg)
    emb = Embedding(cfg, init, dtype=torch.float32)
    ids = torch.randint(0, 512, (2, 8))
    pos = torch.arange(8)
    base = emb(ids, pos)
    with pytest.raises(RuntimeError):
        emb(ids, pos, torch.zeros(2, 8, dtype=torch.long))
    emb.add_tokentype_embeddings(3)
    tt = torch.randint(0, 3, (2, 8))
    emb.eval()
    assert torch.allclose(emb(ids, pos, tt), emb(ids, pos) + emb.tokentype_embeddings(tt))
    assert "tokentype_embeddings.weight" in emb.state_dict()
    with pytest.raises(RuntimeError):
        emb.add_tokentype_embeddings(2)
    assert base.shape == (2, 8, cfg.hidden_size)


def test_mup_optimizer_groups_scale_matrix_like_learning_rates():
    """`use_mup`: projection / MLP weights get lr / mup_width_scale under Adam (MuAdam), vector-like parameters get
    lr * mup_width_scale under SGD (MuSGD); every parameter stays in exactly one group."""
    from savanna_b200.models.backbone import param_groups
    cfg = _cfg(use_mup=True, mup_width_scale=4, weight_decay=0.1)
    tr = Trainer(cfg, load=False)
    groups = param_groups(tr.model, cfg)
    names = {g["name"] for g in groups}
    assert "decay_matrix" in names
    n_params = sum(len(g["params"]) for g in groups)
    assert n_params == len([p for p in tr.model.parameters() if p.requires_grad])
    mat = next(g for g in groups if g["name"] == "decay_matrix")
    assert abs(mat["lr"] - cfg.lr / 4) < 1e-12 and all(p.dim() == 2 for p in mat["params"])
    vec = next(g for g in groups if g["name"] == "no_decay")
    assert "lr" not in vec or vec["lr"] == cfg.lr
    # the optimizer carries the ratio through the schedule
    zg = [g for g in tr.optimizer.param_groups if g["name"] == "decay_matrix"][0]
    assert abs(zg["lr_mult"] - 0.25) < 1e-9 and zg["fixed_lr"]
    cfg2 = _cfg(use_mup=True, mup_width_scale=4, weight_decay=0.1, optimizer={"type": "sgd", "params": {"lr": 1e-3}})
    assert cfg2.optimizer_type == "sgd"
    tr2 = Trainer(cfg2, load=False)
    g2 = param_groups(tr2.model, cfg2)
    vec2 = next(g for g in g2 if g["name"] == "no_decay")
    assert abs(vec2["lr"] - cfg2.lr * 4) < 1e-12
    assert "lr" not in next(g for g in g2 if g["name"] == "decay_matrix")


@pytest.mark.parametrize("over", [
    {"bidirectional": True, "hyena_filter_cls": "implicit_freeform", "hyena_filter_emb_dim": 5, "hyena_filter_order": 16},
    {"use_slow_heads": True, "num_groups_hyena": 16},
    {"hyena_filter_cls": "implicit_freeform", "hyena_pos_emb": "random_fourier", "hyena_filter_emb_dim": 8,
     "hyena_filter_order": 16, "normalize_hyena_filters": True},
])
def test_long_operator_variants_train(over):
    """Two-sided filters, outer-product heads and the free-form filter's options: the tiny model builds with them, trains,
    and the loss falls."""
    cfg = _cfg(**over)
    tr = Trainer(cfg, load=False)
    d = _iter(cfg)
    losses = [float(tr.train_step(d)) for _ in range(6)]
    assert all(l == l for l in losses) and losses[-1] < losses[0], losses
    if over.get("use_slow_heads"):
        li = [m for m in tr.model.modules() if getattr(m, "slow_heads", False)]
        assert li and li[0].conv_bias.shape == (li[0].num_groups,)
    if over.get("bidirectional"):
        li = [m for m in tr.model.modules() if getattr(m, "bidirectional", False)]
        assert li and li[0].filter(8).shape[0] == 2 * li[0].num_groups


def test_grouped_and_tied_in_projections():
    """`proj_groups` narrows the attention layers' in-projection to D + 2 D / groups (second and third stream repeated
    over the groups); `tie_projection_weights` narrows every in-projection to D (the three streams are equal)."""
    D = _cfg().hidden_size
    cfg = _cfg(proj_groups=2)
    tr = Trainer(cfg, load=False)
    widths = {n: p.shape[0] for n, p in tr.model.named_parameters() if n.endswith("dense_projection.weight")}
    attn = [n for n in widths if cfg.operator_config[int(n.split(".")[1]) - 2] in ("flash_v2", "flash", "global", "ring")]
    assert attn and all(widths[n] == 2 * D for n in attn)
    assert all(w == 3 * D for n, w in widths.items() if n not in attn)
    d = _iter(cfg)
    l = [float(tr.train_step(d)) for _ in range(4)]
    assert l[-1] < l[0]
    # the repeated streams: the second half of the expanded projection equals the first
    mixer = tr.model.get_submodule(".".join(attn[0].split(".")[:3]))
    x = torch.randn(1, cfg.seq_length, D)
    proj, _ = mixer.dense_projection(x)
    own = proj.shape[-1] * 2 // 4
    wide = torch.cat([proj[..., :own], proj[..., own:].repeat(1, 1, 2)], dim=-1)
    assert wide.shape[-1] == 3 * D and torch.equal(wide[..., D:2 * D], wide[..., 2 * D:])
    cfg = _cfg(tie_projection_weights=True)
    tr = Trainer(cfg, load=False)
    assert all(p.shape[0] == D for n, p in tr.model.named_parameters() if n.endswith("dense_projection.weight"))
    d = _iter(cfg)
    l = [float(tr.train_step(d)) for _ in range(4)]
    assert l[-1] < l[0]


def test_mup_base_shapes_file_drives_the_groups(tmp_path):
    """Base shapes from two meta-device models; a model twice as wide as the base then gets multiplier 2 on exactly the
    parameters with two growing dimensions."""
    from savanna_b200.models.backbone import build_model, param_groups
    from savanna_b200.train import mup_shapes
    cfg = _cfg(use_mup=True, mup_width_scale=2, base_shapes_file=str(tmp_path / "shapes"))
    cfg.build_tokenizer()
    shapes = mup_shapes.save_base_shapes(cfg, str(tmp_path / "shapes") + ".0")
    D = cfg.hidden_size
    assert shapes["sequential.2.mixer.dense_projection.weight"] == {"shape": [3 * D, D], "infinite": [True, True]}
    assert shapes["sequential.0.word_embeddings.weight"]["infinite"] == [False, True]
    wide = _cfg(use_mup=True, mup_width_scale=7, hidden_size=2 * D, base_shapes_file=str(tmp_path / "shapes"),
                weight_decay=0.1, optimizer={"type": "Adam", "params": {"lr": 1e-3}})
    wide.build_tokenizer()
    model = build_model(wide, device=torch.device("cpu"))
    w = mup_shapes.width_multipliers(model, mup_shapes.load_base_shapes(str(tmp_path / "shapes") + ".0"))
    assert w["sequential.2.mixer.dense_projection.weight"] == (2, 2.0) and w["sequential.0.word_embeddings.weight"][0] == 1
    groups = param_groups(model, wide)
    mat = [g for g in groups if g["name"].endswith("_matrix")]
    assert mat and all(abs(g["lr"] - 1e-3 / 2.0) < 1e-12 for g in mat)          # 2 from the file, not mup_width_scale = 7


def test_block_sparse_layouts_follow_their_rules():
    from savanna_b200.models.sparse_layouts import additive_mask, block_layout
    nb = 8
    loc = block_layout("local", 2, nb, {"num_sliding_window_blocks": 5})[0]
    for r in range(nb):
        for c in range(nb):
            assert bool(loc[r, c]) == (r - 2 <= c <= r), (r, c)
    fx = block_layout("sparse_fixed", 1, nb, {"num_local_blocks": 4, "num_global_blocks": 1})[0]
    assert bool(fx[2, 0]) and bool(fx[3, 3]) and not bool(fx[1, 2])           # inside window 0, lower triangle
    assert bool(fx[6, 4]) and not bool(fx[6, 2])                              # window 1 sees itself, not window 0 ...
    assert bool(fx[6, 3]) and bool(fx[7, 3]) and bool(fx[7, 7])               # ... except the global column 3 (and 7)
    var = block_layout("sparse_variable", 1, nb, {"local_window_blocks": [2, 3], "global_block_indices": [1]})[0]
    assert bool(var[1, 0]) and not bool(var[2, 0]) and bool(var[4, 2]) and bool(var[7, 5]) and not bool(var[5, 4])
    assert all(bool(var[r, 1]) for r in range(1, nb))
    bb = block_layout("bigbird", 1, nb, {"num_random_blocks": 1, "num_sliding_window_blocks": 3, "num_global_blocks": 1})[0]
    assert all(bool(bb[r, 0]) and bool(bb[r, r]) and (r == 0 or bool(bb[r, r - 1])) for r in range(nb))
    assert int(bb.sum()) >= int(block_layout("bigbird", 1, nb, {"num_random_blocks": 0})[0].sum())
    lf = block_layout("bslongformer", 1, nb, {"num_sliding_window_blocks": 3, "global_block_indices": [0, 4],
                                               "global_block_end_indices": [1, 6]})[0]
    assert bool(lf[7, 4]) and bool(lf[7, 5]) and not bool(lf[7, 3]) and bool(lf[7, 0]) and bool(lf[7, 6])
    for lay in (loc, fx, var, bb, lf):
        assert not bool(torch.triu(lay, 1).any()) and bool(torch.diagonal(lay).all())
    heads = block_layout("sparse_fixed", 4, nb, {"num_local_blocks": 4, "num_global_blocks": 1, "different_layout_per_head": True,
                                                  "num_different_global_patterns": 2})
    assert not torch.equal(heads[0], heads[1]) and torch.equal(heads[0], heads[2])
    m = additive_mask("local", 2, 64, {"block": 16, "num_sliding_window_blocks": 3})
    assert m.shape == (2, 64, 64) and m[0, 40, 20] == 0 and m[0, 40, 10] == float("-inf")
    with pytest.raises(ValueError):
        additive_mask("local", 2, 60, {"block": 16})


def test_block_sparse_attention_operators_train_and_match_a_masked_softmax():
    cfg = _cfg(operator_config=[[["hyena_se", "local", "hyena_mr", "bigbird"], 1]], num_layers=4,
               sparsity_config={"block": 16, "num_sliding_window_blocks": 3, "num_random_blocks": 1})
    tr = Trainer(cfg, load=False)
    d = _iter(cfg)
    losses = [float(tr.train_step(d)) for _ in range(5)]
    assert losses[-1] < losses[0], losses
    layer = [m for m in tr.model.modules() if getattr(m, "sparse", False) and m.operator_type == "local"][0]
    B, L, H, hd = 1, 64, layer.heads, layer.hd
    torch.manual_seed(0)
    qkv = torch.randn(B, L, H * 3 * hd)
    pos = torch.arange(L)
    got = layer(qkv, pos).view(B, L, H, hd)
    q3 = qkv.view(B, L, H, 3 * hd)
    q, k, v = q3[..., :hd], q3[..., hd:2 * hd], q3[..., 2 * hd:]
    if layer._rotary:
        from savanna_b200 import ops
        cos, sin = layer._rotary[0](pos)
        q, k = ops.apply_rope(q, cos, sin), ops.apply_rope(k, cos, sin)
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) / hd ** 0.5
    blk = torch.arange(L) // 16
    keep = (blk[None, :] >= blk[:, None] - 1) & (pos[None, :] <= pos[:, None])
    s = s.masked_fill(~keep[None, None], float("-inf"))
    want = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v)
    assert torch.allclose(got, want, atol=1e-5), (got - want).abs().max()


def test_attention_dropout_is_applied_in_training_only():
    cfg = _cfg(attention_dropout=0.5, hidden_dropout=0.0)
    tr = Trainer(cfg, load=False)
    layer = [m for m in tr.model.modules() if hasattr(m, "attn_dropout")][0]
    assert layer.attn_dropout == 0.5
    torch.manual_seed(0)
    qkv = torch.randn(1, 64, layer.heads * 3 * layer.hd)
    pos = torch.arange(64)
    layer.train()
    a, b = layer(qkv, pos), layer(qkv, pos)
    assert not torch.allclose(a, b)                       # two draws of the dropout mask
    layer.eval()
    c, d = layer(qkv, pos), layer(qkv, pos)
    assert torch.equal(c, d)
    losses = [float(tr.train_step(_iter(cfg))) for _ in range(3)]
    assert all(l == l for l in losses)


def test_hyena_width_expansion_widens_the_operators_not_the_stream():
    """`hyena_mlp_expansion_factor` 2 on the short-Hyena MLP and `hyena_width_expansion` 2 on the mixers: projections go
    D -> 3 H -> D with H a multiple of 32, groups scale with the width, and the model trains."""
    cfg = _cfg(mlp_type="short_hyena", hyena_mlp_expansion_factor=2, hyena_width_expansion=2, num_groups_hyena=256,
               num_groups_hyena_medium=16, num_groups_hyena_short=16, num_groups_hyena_mlp=16)
    D = cfg.hidden_size
    tr = Trainer(cfg, load=False)
    shapes = {n: tuple(p.shape) for n, p in tr.model.named_parameters()}
    Hm, Hx = 2 * D, 32 * ((int(2 * D) + 31) // 32)
    assert shapes["sequential.2.mlp.dense_projection.weight"] == (3 * Hm, D)
    assert shapes["sequential.2.mlp.dense.weight"] == (D, Hm)
    assert shapes["sequential.2.mixer.dense_projection.weight"] == (3 * Hx, D)
    assert shapes["sequential.2.mixer.dense.weight"] == (D, Hx)
    attn = [n for n in shapes if n.endswith("mixer.dense_projection.weight")
            and cfg.operator_config[int(n.split(".")[1]) - 2] == "flash_v2"]
    assert attn and all(shapes[n] == (3 * D, D) for n in attn)           # attention keeps the stream's width
    se = tr.model.get_submodule("sequential.2.mlp.mixer")
    assert se.width == Hm and se.num_groups == int(int(16 * 2) * 2) and se.width % se.num_groups == 0
    losses = [float(tr.train_step(_iter(cfg))) for _ in range(4)]
    assert losses[-1] < losses[0], losses


@pytest.mark.parametrize("over", [{"postnorm": True, "pre_mlp_norm": False}, {"outer_mlp_norm": True},
                                  {"prenorm": False, "pre_mlp_norm": False, "postnorm": True}])
def test_block_norm_placements_follow_the_reference_order(over):
    """Post-norm on the MLP output, outer norm on (residual + gated-MLP output), written out with the block's own
    sub-modules."""
    cfg = _cfg(hidden_dropout=0.0, **over)
    tr = Trainer(cfg, load=False)
    blk = tr.model.blocks()[0]
    blk.eval()
    torch.manual_seed(0)
    x = torch.randn(1, cfg.seq_length, cfg.hidden_size)
    pos = torch.arange(cfg.seq_length)
    with torch.no_grad():
        got = blk(x, pos)
        u = blk.input_layernorm(x) if cfg.prenorm else x
        m, mb = blk.mixer(u, pos)
        a = x + (m + mb if mb is not None else m)
        u = blk.pre_mlp_layernorm(a) if cfg.pre_mlp_norm else a
        f, _ = blk.mlp(u, None)
        if cfg.postnorm:
            f = blk.post_attention_layernorm(f)
        want = a + f
        if cfg.outer_mlp_norm:
            want = blk.outer_mlp_layernorm(want)
    assert torch.allclose(got, want, atol=1e-5), (got - want).abs().max()
    losses = [float(tr.train_step(_iter(cfg))) for _ in range(3)]
    assert losses[-1] < losses[0]
