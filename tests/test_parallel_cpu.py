"""Host-side logic of the parallel runtime on CPU processes (gloo): topology, zigzag sharding, the
context-parallel all-to-all and halo exchange, ring attention, ZeRO-1 partitioning and tensor /
sequence / context-parallel equivalence of the whole model."""
import os

import pytest
import torch
import torch.distributed as dist

from savanna_b200.parallel.topology import build_topology
from savanna_b200.parallel.zigzag import inverse_zigzag_permutation, zigzag_indices, zigzag_merge, zigzag_split
from tests.dist_utils import run_distributed

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = os.path.join(ROOT, "configs", "baseline", "tiny_sh2_cpu.yml")


def test_topology_rank_order():
    topo = build_topology(16, pp=1, cp=2, tp=2)
    assert topo.get_coord(0) == {"pipe": 0, "data": 0, "context": 0, "model": 0}
    assert topo.get_coord(1)["model"] == 1 and topo.get_coord(2)["context"] == 1 and topo.get_coord(4)["data"] == 1
    assert topo.get_axis_comm_lists("model")[0] == [0, 1]
    assert topo.get_axis_comm_lists("context")[0] == [0, 2]
    assert topo.get_axis_comm_lists("data")[0] == [0, 4, 8, 12]
    assert topo.get_multi_axis_comm_lists(["data", "context"])[0] == [0, 2, 4, 6, 8, 10, 12, 14]


def test_zigzag_roundtrip():
    x = torch.arange(2 * 32 * 3).view(2, 32, 3)
    for cp in (1, 2, 4):
        parts = [zigzag_split(x, cp, r) for r in range(cp)]
        assert torch.equal(zigzag_merge(parts), x)
    idx = zigzag_indices(16, 2, 0)
    assert idx.tolist() == [0, 1, 2, 3, 12, 13, 14, 15]
    inv = inverse_zigzag_permutation(16, 2)
    order = torch.cat([zigzag_indices(16, 2, r) for r in range(2)])
    assert torch.equal(order[inv], torch.arange(16))


# ----------------------------------------------------------------------------- multi-process workers


def _w_groups(rank, world):
    from savanna_b200.parallel import state
    state.initialize_model_parallel(2, 2, 1)
    assert state.get_model_parallel_world_size() == 2 and state.get_context_parallel_world_size() == 2
    assert state.get_data_parallel_world_size() == world // 4
    assert state.get_sequence_data_parallel_world_size() == world // 2
    t = torch.ones(1)
    dist.all_reduce(t, group=state.get_model_parallel_group())
    assert t.item() == 2
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=state.get_context_parallel_group())
    coord = state.get_topology().get_coord(rank)
    partner = state.get_topology().get_rank(**{**coord, "context": 1 - coord["context"]})
    assert t.item() == rank + partner


def test_process_groups():
    run_distributed(_w_groups, 8)


def _w_a2a_halo(rank, world):
    from savanna_b200.parallel import a2a, halo, state
    state.initialize_model_parallel(1, world, 1)
    torch.manual_seed(0)
    B, L, D = 2, 16 * world, 4 * world
    full = torch.randn(B, L, D, dtype=torch.float64)
    local = zigzag_split(full, world, rank).clone().requires_grad_()
    # split_to_full gives the natural-order sequence with this rank's channel block
    sf = a2a.split_to_full(local)
    d = D // world
    assert torch.allclose(sf, full[..., rank * d:(rank + 1) * d])
    back = a2a.full_to_split(sf)
    assert torch.allclose(back, local)
    back.sum().backward()
    assert torch.allclose(local.grad, torch.ones_like(local))
    # halo rows equal the rows that precede each chunk in the full sequence
    H = 3
    h = halo.zigzag_halo(local.detach(), H)
    c = L // (2 * world)
    a_id, b_id = rank, 2 * world - 1 - rank
    exp_a = full[:, a_id * c - H:a_id * c] if a_id > 0 else torch.zeros(B, H, D, dtype=torch.float64)
    exp_b = full[:, b_id * c - H:b_id * c]
    assert torch.allclose(h[:, 0], exp_a) and torch.allclose(h[:, 1], exp_b)


def test_a2a_and_halo():
    run_distributed(_w_a2a_halo, 4)


def _w_halo_grad(rank, world):
    """Gradient of a causal conv through the halo exchange equals the gradient on the full sequence."""
    from savanna_b200.ops import reference as ref
    from savanna_b200.parallel import halo, state
    state.initialize_model_parallel(1, world, 1)
    torch.manual_seed(1)
    B, L, C, K = 1, 8 * 2 * world, 6, 4
    full = torch.randn(B, L, C, dtype=torch.float64, requires_grad=True)
    w = torch.randn(C, K, dtype=torch.float64)
    g = torch.randn(B, L, C, dtype=torch.float64)
    ref.causal_conv1d(full, w).backward(g)
    local = zigzag_split(full.detach(), world, rank).clone().requires_grad_()
    h = halo.zigzag_halo(local, K - 1)
    y = ref.causal_conv1d(local.reshape(B * 2, -1, C), w, h.reshape(B * 2, K - 1, C)).reshape(B, -1, C)
    y.backward(zigzag_split(g, world, rank))
    assert torch.allclose(local.grad, zigzag_split(full.grad, world, rank), atol=1e-10)


def test_halo_gradient():
    run_distributed(_w_halo_grad, 4)


def _w_ring_attention(rank, world):
    from savanna_b200.ops import reference as ref
    from savanna_b200.parallel import state
    from savanna_b200.parallel.ring_attention import ring_attention
    state.initialize_model_parallel(1, world, 1)
    torch.manual_seed(2)
    B, L, H, hd = 1, 8 * 2 * world, 2, 8
    q, k, v = (torch.randn(B, L, H, hd, dtype=torch.float64, requires_grad=True) for _ in range(3))
    g = torch.randn(B, L, H, hd, dtype=torch.float64)
    o = ref.attention(q, k, v, causal=True)
    o.backward(g)
    ql, kl, vl = (zigzag_split(t.detach(), world, rank).clone().requires_grad_() for t in (q, k, v))
    pos = zigzag_indices(L, world, rank)
    ol = ring_attention(ql, kl, vl, pos, causal=True)
    assert torch.allclose(ol, zigzag_split(o.detach(), world, rank), atol=2e-5)
    ol.backward(zigzag_split(g, world, rank))
    for a, b in ((ql, q), (kl, k), (vl, v)):
        assert torch.allclose(a.grad, zigzag_split(b.grad, world, rank), atol=5e-5)


def test_ring_attention():
    run_distributed(_w_ring_attention, 4)


def _tiny_cfg(world, **over):
    from savanna_b200.config import GlobalConfig
    base = {"global_num_gpus": world, "hidden_dropout": 0.0, "train_micro_batch_size_per_gpu": 2}
    base.update(over)
    cfg = GlobalConfig.from_ymls([TINY], base)
    return cfg


def _run_steps(cfg, n=3, seed_offset=0, global_batch=None):
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.parallel import state
    from savanna_b200.train.trainer import Trainer
    tr = Trainer(cfg, load=False)
    dp, dr = state.get_data_parallel_world_size(), state.get_data_parallel_rank()
    mb = cfg.train_micro_batch_size_per_gpu

    def it():
        i = 0
        while True:
            full = acgt_batch(mb * dp, cfg.seq_length, seed=i)
            yield {"text": full[dr * mb:(dr + 1) * mb]}
            i += 1
    d = it()
    losses, norms = [], []
    for _ in range(n):
        losses.append(float(tr.train_step(d)))
        norms.append(float(tr.grad_norm))
    tr.grad_norms = norms
    return tr, losses


def _w_equiv(rank, world, over, ref_losses, ref_norms=None):
    cfg = _tiny_cfg(world, **over)
    tr, losses = _run_steps(cfg)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    if ref_norms is not None:
        # Adam is invariant to the gradient's scale, so equal loss traces do not show a mis-scaled gradient:
        # the logged global norm (what clipping acts on) must match the single-process value too
        for a, b in zip(tr.grad_norms, ref_norms):
            assert abs(a - b) < 2e-3 * max(1.0, abs(b)), (tr.grad_norms, ref_norms)


def _reference_losses(mb=2, with_norms=False, **over):
    cfg = _tiny_cfg(1, train_micro_batch_size_per_gpu=mb, **over)
    tr, losses = _run_steps(cfg)
    from savanna_b200.parallel import state
    state.destroy_model_parallel()
    return (losses, tr.grad_norms) if with_norms else losses


@pytest.mark.slow
def test_tensor_parallel_equivalence():
    ref_losses = _reference_losses()
    run_distributed(_w_equiv, 2, {"model_parallel_size": 2}, ref_losses)


def _w_partition_activations(rank, world, ref_losses):
    """tp = 2 with checkpointed chunks whose saved inputs are cut to 1 / tp and gathered back for the recomputation."""
    import savanna_b200.models.backbone as bb
    stored = []
    real = bb._partitioned_saved_tensors

    def spy(tp, r, group):
        ctx = real(tp, r, group)
        pack = ctx.pack_hook

        def counted(t):
            out = pack(t)
            stored.append((out[0], tuple(t.shape), tuple(out[1].shape)))
            return out
        ctx.pack_hook = counted
        return ctx
    bb._partitioned_saved_tensors = spy
    cfg = _tiny_cfg(world, model_parallel_size=2, checkpoint_activations=True, checkpoint_num_layers=2,
                    partition_activations=True)
    tr, losses = _run_steps(cfg)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    parts = [s for s in stored if s[0] == "part"]
    assert parts and all(p[2][1] * 2 == p[1][1] for p in parts), stored


@pytest.mark.slow
def test_partition_activations_over_tensor_parallel_ranks():
    ref_losses = _reference_losses()
    run_distributed(_w_partition_activations, 2, ref_losses)


@pytest.mark.slow
def test_sequence_parallel_equivalence():
    ref_losses = _reference_losses()
    run_distributed(_w_equiv, 2, {"model_parallel_size": 2, "sequence_parallel": True}, ref_losses)


@pytest.mark.slow
def test_context_parallel_equivalence_a2a():
    ref_losses, ref_norms = _reference_losses(with_norms=True)
    over = {"context_parallel_size": 2, "use_cp_hyena": True, "use_cp_ring": True,
            "operator_config": ["hyena_se", "hyena_mr", "hyena", "ring"]}
    run_distributed(_w_equiv, 2, over, ref_losses, ref_norms)


@pytest.mark.slow
@pytest.mark.parametrize("optimizer", ["adam", "sgd"])
def test_context_parallel_gradient_scale_with_clipping(optimizer):
    """cp=2 with clipping active (threshold far below the norm) and, for SGD, an optimizer whose step depends on
    the gradient's scale: loss trace and gradient norm equal the single-process run."""
    extra = {"gradient_clipping": 0.5}
    if optimizer == "sgd":
        extra["optimizer"] = {"type": "sgd", "params": {"lr": 0.05, "momentum": 0.0}}
        extra["lr"] = 0.05
    ref_losses, ref_norms = _reference_losses(with_norms=True, **extra)
    assert min(ref_norms) > 1.0                      # clipping really is active
    over = {"context_parallel_size": 2, "use_cp_hyena": True, "use_cp_ring": True,
            "operator_config": ["hyena_se", "hyena_mr", "hyena", "ring"], **extra}
    run_distributed(_w_equiv, 2, over, ref_losses, ref_norms)


@pytest.mark.slow
def test_context_parallel_equivalence_p2p_state():
    ref_losses = _reference_losses()
    over = {"context_parallel_size": 2, "use_cp_hyena": True, "use_cp_ring": True, "cp_hyena_mr_algo": "p2p",
            "cp_hyena_li_algo": "state", "operator_config": ["hyena_se", "hyena_mr", "hyena", "ring"]}
    run_distributed(_w_equiv, 2, over, ref_losses)


@pytest.mark.slow
@pytest.mark.parametrize("algo", ["a2a", "p2p_state"])
def test_context_parallel_equivalence_cp4(algo):
    """cp=4: distinct previous / next neighbours in the halo exchange, three ring steps, four-way all-to-all."""
    ref_losses, ref_norms = _reference_losses(with_norms=True)
    over = {"context_parallel_size": 4, "use_cp_hyena": True, "use_cp_ring": True,
            "operator_config": ["hyena_se", "hyena_mr", "hyena", "ring"]}
    if algo == "p2p_state":
        over.update({"cp_hyena_mr_algo": "p2p", "cp_hyena_li_algo": "state"})
    run_distributed(_w_equiv, 4, over, ref_losses, ref_norms)


@pytest.mark.slow
@pytest.mark.parametrize("comm", ["a2a", "all_gather"])
def test_context_parallel_attention_comm_types(comm):
    """`flash_te` layers with the head-exchange and the key/value all-gather forms of context-parallel attention at
    cp=2 reproduce the single-process loss trace and gradient norm."""
    ref_losses, ref_norms = _reference_losses(with_norms=True)
    over = {"context_parallel_size": 2, "use_cp_hyena": True, "use_cp_flash_te": True, "flash_te_comm_type": comm,
            "operator_config": ["hyena_se", "hyena_mr", "hyena", "flash_te"]}
    run_distributed(_w_equiv, 2, over, ref_losses, ref_norms)


@pytest.mark.slow
def test_zero1_data_parallel_equivalence():
    """dp=2 with micro batch 1 and ZeRO-1 partitioning == one process with micro batch 2."""
    ref_losses = _reference_losses(mb=2)
    run_distributed(_w_equiv, 2, {"train_micro_batch_size_per_gpu": 1, "zero_optimization": {"stage": 1}}, ref_losses)


@pytest.mark.slow
@pytest.mark.parametrize("stage", [1, 3])
def test_zero_with_weight_decay_groups_matches_one_process(stage):
    """With weight decay on there are several parameter groups (decayed weights incl. the fp32 modal filter parameters,
    undecayed norms and biases, the Hyena-MR filter at its own learning rate): partitioned training still reproduces
    the single-process trace and gradient norms."""
    over = {"weight_decay": 0.1, "lr_medium_hyena": 1e-4}
    ref_losses, ref_norms = _reference_losses(mb=2, with_norms=True, **over)
    run_distributed(_w_equiv, 2, dict(over, train_micro_batch_size_per_gpu=1, zero_optimization={"stage": stage}),
                    ref_losses, ref_norms)


def _w_partitioned(rank, world, over, ref_losses, tmp):
    """Stage 2 / 3 training reproduces the loss trace; between steps a stage-3 rank holds no whole block; a checkpoint
    written from shards reloads into an identical model."""
    import os
    from savanna_b200.ckpt import load_checkpoint, save_checkpoint
    cfg = _tiny_cfg(world, **over)
    tr, losses = _run_steps(cfg)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    opt = tr.optimizer
    assert opt.stage == over["zero_optimization"]["stage"]
    blocks = [f for u in opt.units[1:] for f in u.flats]
    assert blocks and all(f.gfull.untyped_storage().size() == 0 for f in blocks)
    if opt.stage == 3:
        assert all(f.full.untyped_storage().size() == 0 for f in blocks)
    with opt.full_params():
        before = {k: v.detach().clone() for k, v in tr.model.state_dict().items()}
    cfg.save = os.path.join(tmp, "ck")
    save_checkpoint(tr)
    with opt.full_params(writeback=True):
        for q in tr.model.parameters():
            q.data.zero_()
    cfg.load = cfg.save
    load_checkpoint(tr)
    with opt.full_params():
        for k, v in tr.model.state_dict().items():
            assert torch.equal(v, before[k]), k


@pytest.mark.slow
@pytest.mark.parametrize("stage,ckpt_layers", [(2, 0), (3, 0), (3, 1), (3, 2)])
def test_zero23_data_parallel_equivalence(stage, ckpt_layers, tmp_path):
    """dp=2, micro batch 1, two accumulation steps, gradients (stage 2) and parameters (stage 3) partitioned per block
    == one process with micro batch 2 and two accumulation steps; with activation checkpointing over 1 or 2 blocks."""
    cfg = _tiny_cfg(1, train_micro_batch_size_per_gpu=2, gradient_accumulation_steps=2)
    _, ref_losses = _run_steps(cfg)
    from savanna_b200.parallel import state
    state.destroy_model_parallel()
    over = {"train_micro_batch_size_per_gpu": 1, "gradient_accumulation_steps": 2, "zero_optimization": {"stage": stage}}
    if ckpt_layers:
        over.update({"checkpoint_activations": True, "checkpoint_num_layers": ckpt_layers})
    run_distributed(_w_partitioned, 2, over, ref_losses, str(tmp_path))


def _w_offload_param(rank, world, over, ref_losses):
    cfg = _tiny_cfg(world, **over)
    tr, losses = _run_steps(cfg)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    off = [f for f in tr.optimizer.groups if f.param_offloaded]
    keep = [f for f in tr.optimizer.groups if not f.param_offloaded]
    assert off and keep                       # block units are offloaded; the resident root unit and fp32 flats are not
    assert all(f.free_params and f.param_shard.device.type == "cpu" for f in off)
    rep = tr.optimizer.memory_report()
    assert rep["persistent_bytes"] < sum(f.shard * 12 + f.shard * 2 + f.shard * 4 for f in tr.optimizer.groups) + 2 * sum(
        f.nbytes for f in tr.optimizer.units[0].flats)
    # the host copies follow the update: gathering from them reproduces the masters
    with tr.optimizer.full_params():
        for f in off:
            assert torch.allclose(f.shard_slice(f.full).float(), f.master.to(f.full.dtype).float())


def _w_write_losses(rank, world, over, out):
    import json
    cfg = _tiny_cfg(world, **over)
    _, losses = _run_steps(cfg)
    if rank == 0:
        with open(out, "w") as fh:
            json.dump(losses, fh)


def _w_offload_optimizer_partitioned(rank, world, over, ref_losses):
    cfg = _tiny_cfg(world, **over)
    tr, losses = _run_steps(cfg)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    opt = tr.optimizer
    assert opt.offload_optimizer and all(f.optimizer_offloaded and f.master.device.type == "cpu" and not f.master_is_view
                                         for f in opt.groups)
    with opt.full_params():
        for f in opt.groups:
            assert torch.allclose(f.shard_slice(f.full).float(), f.master.to(f.full.dtype).float())


@pytest.mark.slow
@pytest.mark.parametrize("stage", [2, 3])
def test_zero23_optimizer_offload_matches(stage, tmp_path):
    """`offload_optimizer.device: cpu` with the partitioned optimizer (fp32 and bf16 flats alike): same loss trace."""
    import json
    over = {"train_micro_batch_size_per_gpu": 1, "gradient_accumulation_steps": 2, "zero_optimization": {"stage": stage}}
    out = str(tmp_path / "ref.json")
    run_distributed(_w_write_losses, 2, over, out)
    ref_losses = json.load(open(out))
    over2 = dict(over, zero_optimization={"stage": stage, "offload_optimizer": {"device": "cpu"}})
    run_distributed(_w_offload_optimizer_partitioned, 2, over2, ref_losses)
    if stage == 3:                                         # ... and with the state arrays as mapped files
        nv = str(tmp_path / "nv")
        over3 = dict(over, zero_optimization={"stage": stage, "offload_optimizer": {"device": "nvme", "nvme_path": nv}})
        run_distributed(_w_offload_optimizer_partitioned, 2, over3, ref_losses)
        files = os.listdir(nv)
        assert files and len(files) % 3 == 0 and any(f.startswith("zero_state_rank1_") for f in files)


@pytest.mark.slow
def test_zero3_parameter_offload_matches(tmp_path):
    """`offload_param.device: cpu` with stage 3 in bf16: the shards of released units live on the host, the loss trace
    equals the run without offload."""
    import json
    over = {"train_micro_batch_size_per_gpu": 1, "gradient_accumulation_steps": 2, "precision": "bfloat16",
            "zero_optimization": {"stage": 3}}
    out = str(tmp_path / "ref.json")
    run_distributed(_w_write_losses, 2, over, out)
    ref_losses = json.load(open(out))
    over2 = dict(over, zero_optimization={"stage": 3, "offload_param": {"device": "cpu"}})
    run_distributed(_w_offload_param, 2, over2, ref_losses)


@pytest.mark.slow
@pytest.mark.parametrize("stage", [2, 3])
def test_zero_mics_subgroup_sharding(stage, tmp_path):
    """4 replicas, optimizer state sharded over sub-groups of 2 (MiCS) and replicated across the two sub-groups: the loss
    trace equals the single-process run, and the checkpoint holds one set of shards (2 optimizer files), which reloads."""
    ref_losses = _reference_losses(mb=4)
    over = {"train_micro_batch_size_per_gpu": 1, "zero_use_mics": True,
            "zero_optimization": {"stage": stage, "mics_shard_size": 2}}
    run_distributed(_w_mics, 4, over, ref_losses, str(tmp_path))


def _w_mics(rank, world, over, ref_losses, tmp):
    import os
    from savanna_b200.ckpt import load_checkpoint, save_checkpoint
    cfg = _tiny_cfg(world, save=tmp, **over)
    tr, losses = _run_steps(cfg)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    opt = tr.optimizer
    assert opt.world == 2 and opt.replica_world == 2 and opt.reduce_world == 4
    d = save_checkpoint(tr)
    dist.barrier()
    files = sorted(f for f in os.listdir(d) if f.endswith("optim_states.pt"))
    assert files == ["zero_pp_rank_0_mp_rank_00_optim_states.pt", "zero_pp_rank_1_mp_rank_00_optim_states.pt"], files
    before = [p.detach().clone() for p in tr.model.parameters()] if opt.stage == 2 else None
    cfg.load = tmp
    load_checkpoint(tr)
    if before is not None:
        for a, b in zip(before, tr.model.parameters()):
            assert torch.equal(a, b)


@pytest.mark.slow
def test_zero3_with_tensor_parallel():
    """Stage 3 over a one-rank partition group beside tp=2 + sequence parallelism (replicated-parameter gradients are
    summed per unit) reproduces the loss trace."""
    ref_losses = _reference_losses()
    run_distributed(_w_equiv, 2, {"model_parallel_size": 2, "sequence_parallel": True,
                                  "zero_optimization": {"stage": 3}}, ref_losses)


@pytest.mark.slow
def test_pipeline_parallel_equivalence():
    """Two pipeline stages (tied embedding on both ends) reproduce the single-process loss trace."""
    ref_losses = _reference_losses()
    run_distributed(_w_equiv, 2, {"pipe_parallel_size": 2, "gradient_accumulation_steps": 1}, ref_losses)


def _w_pipeline_1f1b(rank, world, ref_losses):
    cfg = _tiny_cfg(world, pipe_parallel_size=world, gradient_accumulation_steps=4, train_micro_batch_size_per_gpu=1)
    tr, losses = _run_steps(cfg, n=2)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    # 1F1B bound on live activations: stages - stage, not the accumulation depth
    assert tr.pipeline_peak_live == world - rank, (rank, tr.pipeline_peak_live)


@pytest.mark.slow
@pytest.mark.parametrize("stages", [2, 3])
def test_pipeline_1f1b_schedule(stages):
    """4 micro-batches through 2 and 3 stages: same loss trace as one process accumulating the same 4 micro-batches,
    with the number of live micro-batch activations per stage bounded by the schedule."""
    cfg = _tiny_cfg(1, gradient_accumulation_steps=4, train_micro_batch_size_per_gpu=1)
    _, ref_losses = _run_steps(cfg, n=2)
    from savanna_b200.parallel import state
    state.destroy_model_parallel()
    run_distributed(_w_pipeline_1f1b, stages, ref_losses)


def _w_pipeline_ckpt(rank, world, ref_losses, tmp):
    """Two stages: 2 steps, save, fresh trainers load and run 2 more steps; the 4 losses equal the single-process trace."""
    from savanna_b200.ckpt import load_checkpoint, save_checkpoint
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.parallel import state
    from savanna_b200.train.trainer import Trainer
    over = {"pipe_parallel_size": 2, "gradient_accumulation_steps": 1, "save": tmp, "checkpoint_strict_load": True}
    cfg = _tiny_cfg(world, **over)
    tr = Trainer(cfg, load=False)
    mb = cfg.train_micro_batch_size_per_gpu

    def it(start):
        i = start
        while True:
            yield {"text": acgt_batch(mb, cfg.seq_length, seed=i)}
            i += 1
    d = it(0)
    first = [float(tr.train_step(d)) for _ in range(2)]
    ck = save_checkpoint(tr)
    names = sorted(os.listdir(ck))
    if rank == 0:
        # per-layer module files and one engine + optimizer file per stage: no path is shared by two stages
        assert "mp_rank_00_model_states.pt" in names and "mp_rank_01_model_states.pt" in names, names
        assert "zero_pp_rank_0_mp_rank_00_optim_states.pt" in names and "zero_pp_rank_0_mp_rank_01_optim_states.pt" in names, names
        layers = [n for n in names if n.startswith("layer_")]
        assert len(layers) == len(set(layers)) and "layer_00-model_00-model_states.pt" in layers, names
        assert len(layers) == cfg.num_layers + 2, layers      # embedding + blocks + final norm
    cfg2 = _tiny_cfg(world, load=tmp, **over)
    state.destroy_model_parallel()
    t2 = Trainer(cfg2, load=True)
    assert t2.iteration == 2
    d2 = it(2)
    second = [float(t2.train_step(d2)) for _ in range(2)]
    for a, b in zip(first + second, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (first + second, ref_losses)


@pytest.mark.slow
def test_pipeline_checkpoint_save_load_continue(tmp_path):
    cfg = _tiny_cfg(1)
    _, ref_losses = _run_steps(cfg, n=4)
    from savanna_b200.parallel import state
    state.destroy_model_parallel()
    run_distributed(_w_pipeline_ckpt, 2, ref_losses, str(tmp_path))
    # the per-layer files of the two stages load into one whole model (single process, for inference and the tools)
    from savanna_b200.inference.load import load_for_inference
    from savanna_b200.tools.reshard_model_parallel import load_shards
    step = os.path.join(str(tmp_path), "global_step2")
    shards = load_shards(step)
    assert len(shards) == 1 and "sequential.0.word_embeddings.weight" in shards[0]["module"]
    model, tok, cfg1 = load_for_inference(step, device="cpu")
    sd = model.state_dict()
    for k, v in shards[0]["module"].items():
        if k in sd:
            assert torch.equal(sd[k], v.to(sd[k].dtype)), k
    ids = torch.tensor([list(tok.tokenize("ACGTACGT"))], dtype=torch.long)
    with torch.no_grad():
        logits = model(ids, torch.arange(ids.shape[1]))
    assert logits.shape[:2] == ids.shape and torch.isfinite(logits).all()
    state.destroy_model_parallel()


def test_ring_block_plan_covers_the_causal_mask():
    """The (query part, key part, causal) blocks of every ring step add up to exactly the causal mask between the local
    zigzag query chunks and each rank's zigzag key chunks."""
    import torch
    from savanna_b200.parallel.ring_attention import _block_plan
    cp, c = 4, 3                                   # 8 chunks of 3 positions
    L = 2 * cp * c

    def positions(rank):
        return list(range(rank * c, (rank + 1) * c)) + list(range((2 * cp - 1 - rank) * c, (2 * cp - rank) * c))

    def rows(part):
        return {"lo": range(0, c), "hi": range(c, 2 * c), "all": range(0, 2 * c)}[part]
    for me in range(cp):
        for src in range(cp):
            qpos, kpos = positions(me), positions(src)
            want = torch.tensor([[int(kp <= qp) for kp in kpos] for qp in qpos])
            got = torch.zeros_like(want)
            for qp, kp, causal in _block_plan(me, src, True):
                for i_local, i in enumerate(rows(qp)):
                    for j_local, j in enumerate(rows(kp)):
                        visible = (j_local <= i_local) if causal else True
                        got[i, j] += int(visible)
            assert torch.equal(got, want), (me, src, got, want)
    # without causality a step is one dense block
    assert _block_plan(1, 2, False) == [("all", "all", False)]


def test_symmetric_memory_door_reports_a_moved_api(monkeypatch):
    """The private PyTorch API behind every peer mapping is checked in one place: a module without `rendezvous` (or no
    module at all) gives one clear error, and the ZeRO allocator answers None so that the NCCL path runs."""
    import sys
    import types
    from savanna_b200.parallel import fused_zero, symm
    fake = types.ModuleType("fake_symm_without_rendezvous")
    fake.empty = lambda *a, **k: None
    sys.modules[fake.__name__] = fake
    with pytest.raises(symm.SymmetricMemoryUnavailable, match="lacks rendezvous"):
        symm.load(fake.__name__)
    with pytest.raises(symm.SymmetricMemoryUnavailable, match="no importable"):
        symm.load("savanna_b200_no_such_module")
    handle = types.SimpleNamespace(buffer_ptrs=[16, 0])
    with pytest.raises(symm.SymmetricMemoryUnavailable):
        symm.peer_pointers(handle, 2)
    assert symm.peer_pointers(types.SimpleNamespace(buffer_ptrs=[16, 32]), 2) == [16, 32]
    assert symm.multicast_pointer(types.SimpleNamespace()) == 0
    monkeypatch.setattr(symm, "_MODULE", fake.__name__)
    monkeypatch.setattr(symm.load, "__defaults__", (fake.__name__,))
    assert fused_zero.make_allocator(None) is None


@pytest.mark.slow
@pytest.mark.parametrize("ckpt_layers", [0, 1])
def test_zero3_hpz_secondary_partition(ckpt_layers):
    """Stage 3 over 4 ranks with `zero_hpz_partition_size: 2`: after a unit's forward gather every rank keeps its half of
    the whole parameters, and the backward (and recomputation) gathers run inside the sub-group of 2; the loss trace
    equals the single-process run and the secondary gathers are counted."""
    ref_losses = _reference_losses(mb=4)
    over = {"train_micro_batch_size_per_gpu": 1, "zero_optimization": {"stage": 3, "zero_hpz_partition_size": 2}}
    if ckpt_layers:
        over.update({"checkpoint_activations": True, "checkpoint_num_layers": ckpt_layers})
    run_distributed(_w_hpz, 4, over, ref_losses)


def _w_hpz(rank, world, over, ref_losses):
    cfg = _tiny_cfg(world, **over)
    tr, losses = _run_steps(cfg)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    opt = tr.optimizer
    assert opt.stage == 3 and opt.world == 4 and opt.hpz_world == 2
    freed = [f for f in opt.groups if f.free_params]
    assert freed and all(f.hpz_gathers > 0 for f in freed), [f.hpz_gathers for f in freed]
    assert all(f.hpz_shard.numel() == f.padded // 2 for f in freed)
    assert all(not f.hpz_fresh for f in freed)                  # stale after the optimizer step


def test_zero_offload_keeps_state_on_the_host_and_matches():
    """`zero_optimization.offload_optimizer.device: cpu`: the loss trace equals the run without offload (same Adam
    arithmetic, fp32), master weights and moments are host tensors, and the optimizer state survives a state-dict
    round trip."""
    from savanna_b200.parallel import state
    cfg = _tiny_cfg(1)
    _, ref_losses = _run_steps(cfg)
    state.destroy_model_parallel()
    cfg2 = _tiny_cfg(1, zero_optimization={"stage": 1, "offload_optimizer": {"device": "cpu", "pin_memory": True}})
    tr, losses = _run_steps(cfg2)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-5 * max(1.0, abs(b)), (losses, ref_losses)
    opt = tr.optimizer
    assert opt.offload_optimizer and opt.fused is None
    for g in opt.groups:
        assert g.master.device.type == "cpu" and g.exp_avg.device.type == "cpu" and not g.master_is_view
        assert torch.allclose(g.master.to(g.flat_param.dtype), g.shard_slice(g.flat_param).cpu())
    import copy
    sd = copy.deepcopy(opt.state_dict())
    m0 = [g.master.clone() for g in opt.groups]
    for g in opt.groups:
        g.master.zero_()
    opt.load_state_dict(sd)
    for a, g in zip(m0, opt.groups):
        assert torch.equal(a, g.master)
    state.destroy_model_parallel()


def test_zero_offload_to_files_matches_and_persists_on_disk(tmp_path):
    """`offload_optimizer.device: nvme`: same loss trace as without offload; master weights and moments are mapped
    files of shard * 4 bytes under `nvme_path` whose contents follow the update."""
    import numpy as np
    from savanna_b200.parallel import state
    cfg = _tiny_cfg(1)
    _, ref_losses = _run_steps(cfg)
    state.destroy_model_parallel()
    cfg2 = _tiny_cfg(1, zero_optimization={"stage": 1, "offload_optimizer": {"device": "nvme", "nvme_path": str(tmp_path / "nv")}})
    tr, losses = _run_steps(cfg2)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-5 * max(1.0, abs(b)), (losses, ref_losses)
    files = sorted(os.listdir(tmp_path / "nv"))
    assert len(files) == 3 * len(tr.optimizer.groups) and all(f.startswith("zero_state_rank0_buf") for f in files)
    g = tr.optimizer.groups[0]
    on_disk = np.fromfile(tmp_path / "nv" / "zero_state_rank0_buf0_master.bin", dtype=np.float32)
    assert on_disk.shape[0] == g.shard and np.array_equal(on_disk, g.master.numpy())
    moments = np.fromfile(tmp_path / "nv" / "zero_state_rank0_buf0_exp_avg_sq.bin", dtype=np.float32)
    assert moments.max() > 0.0
    state.destroy_model_parallel()
    with pytest.raises(ValueError):
        _run_steps(_tiny_cfg(1, zero_optimization={"stage": 1, "offload_optimizer": {"device": "nvme"}}))
    state.destroy_model_parallel()


def test_pipeline_partition_methods():
    """Even block counts for `type:` / `uniform`; `parameters` balances the parameter count with the embedding on the
    first and the head on the last stage."""
    from savanna_b200.parallel.pipeline import balanced_layer_ranges, partition_layers
    r = balanced_layer_ranges([1, 1, 1, 1, 1, 1], 3)
    assert [list(x) for x in r] == [[0, 1], [2, 3], [4, 5]]
    r = balanced_layer_ranges([1, 1, 1, 1, 1, 1], 2, first_extra=2.0)          # a heavy embedding: fewer blocks up front
    assert [len(x) for x in r] == [2, 4]
    r = balanced_layer_ranges([5, 1, 1, 1, 1, 1], 2)
    assert [len(x) for x in r] == [1, 5]
    with pytest.raises(ValueError):
        balanced_layer_ranges([1, 1], 3)
    cfg = _tiny_cfg(1)
    cfg.build_tokenizer()
    even = partition_layers(cfg, 2)
    assert [len(x) for x in even] == [cfg.num_layers // 2, cfg.num_layers - cfg.num_layers // 2] or sum(len(x) for x in even) == cfg.num_layers
    cfg.pipe_partition_method = "parameters"
    by_params = partition_layers(cfg, 2)
    assert by_params[0].start == 0 and by_params[-1].stop == cfg.num_layers and by_params[0].stop == by_params[1].start
    cfg.pipe_partition_method = "nonsense"
    with pytest.raises(ValueError):
        partition_layers(cfg, 2)
