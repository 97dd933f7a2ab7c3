"""Straggler detection, collective logging and the allocation watcher, on CPU (gloo ranks, injected slow rank)."""
import time

import torch
import torch.distributed as dist

from savanna_b200.utils.observability import AllocStats, CommsLogger, StragglerDetector, bus_bandwidth_factor
from tests.dist_utils import run_distributed


def _w_straggler(rank, world):
    lines = []
    det = StragglerDetector(world, rank, interval=4, minmax_count=2, rel_threshold=0.7, use_cuda_events=False, printer=lines.append)
    rep = None
    for step in range(4):
        with det.section("TRAIN_STEP_FORWARD"):
            time.sleep(0.06 if rank == 2 else 0.02)          # rank 2 is three times slower in this section
        with det.section("TRAIN_STEP_BACKWARD"):
            time.sleep(0.02)
        rep = det.step()
        dist.barrier()
    assert rep is not None and rep["steps"] == 4
    fwd = rep["sections"]["host/TRAIN_STEP_FORWARD"]
    assert fwd["slowest_ranks"][0] == 2 and rep["stragglers"]["host/TRAIN_STEP_FORWARD"] == [2], rep
    assert "host/TRAIN_STEP_BACKWARD" not in rep["stragglers"]
    assert abs(fwd["relative_perf_scores"][0] - 1.0) < 0.3 and fwd["relative_perf_scores"][2] < 0.5
    if rank == 0:
        assert any("ranks [2]" in ln for ln in lines), lines


def test_straggler_detector_names_the_slow_rank():
    run_distributed(_w_straggler, 4)


def test_straggler_individual_score_flags_a_rank_that_slows_down():
    lines = []
    det = StragglerDetector(1, 0, interval=2, use_cuda_events=False, individual_threshold=0.7, printer=lines.append)
    for delay in (0.01, 0.01, 0.04, 0.04):
        with det.section("step"):
            time.sleep(delay)
        rep = det.step()
    assert rep["individual_perf_scores"]["host/step"] < 0.5 and "host/step" in rep["individual_stragglers"]


def _w_comms(rank, world):
    lines = []
    lg = CommsLogger(rank, ops=["all_reduce", "broadcast"], rank_stride=2, world=world, printer=lines.append)
    lg.install()
    try:
        lg.enabled = True
        x = torch.ones(1024)
        for _ in range(3):
            dist.all_reduce(x)
        dist.broadcast(x[:16].clone(), 0)
        dist.all_gather([torch.empty(4) for _ in range(world)], torch.ones(4))       # not in the op list: not recorded
        lg.enabled = False
        dist.all_reduce(x)                                                             # disabled: not recorded
        summ = lg.summary()
        assert summ["all_reduce"][4096]["count"] == 3 and summ["broadcast"][64]["count"] == 1 and "all_gather" not in summ
        assert summ["all_reduce"][4096]["busbw_gbs"] == summ["all_reduce"][4096]["algbw_gbs"] * bus_bandwidth_factor("all_reduce", world)
        out = lg.serialize()
        assert any(ln.startswith(f"COMMS:all_reduce,{rank},4096,") and ln.count(",") == 5 for ln in out), out
        assert (len(lines) > 0) == (rank % 2 == 0)            # only every second rank prints
    finally:
        lg.uninstall()
    assert not hasattr(dist.all_reduce, "_sb_comms_original")


def test_comms_logger_records_selected_collectives():
    run_distributed(_w_comms, 2)


def test_alloc_stats_warns_when_the_allocator_goes_back_to_the_driver():
    counters = {"num_alloc_retries": 0, "num_device_alloc": 10, "num_device_free": 2}
    lines = []
    w = AllocStats(rank=3, warmup_steps=7, reader=lambda: dict(counters), printer=lines.append)
    for it in range(1, 10):
        assert w.step(it) is False
    counters["num_device_alloc"] = 12
    assert w.step(10) is True and w.changes == 1 and "rank=3" in lines[0]
    assert w.step(11) is False


def test_torch_profiler_records_the_step_marks_with_expected_counts(tmp_path):
    """A short CPU run under `profiler_type: torch`: one trace per schedule cycle is written, the key-averages table
    exists, and the three training marks appear once per micro-batch / optimizer step of the active window
    (role of the reference's tests/functional/test_profiler.py)."""
    import glob
    import gzip
    import json
    import os
    import torch
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "prof")
    active, gas = 2, 2
    cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_cpu.yml")], {
        "global_num_gpus": 1, "train_iters": 5, "gradient_accumulation_steps": gas, "should_profile": True,
        "profiler_type": "torch", "profiler_output_dir": out, "profile_cpu": True, "profile_cuda": False,
        "profiler_schedule_wait": 1, "profiler_schedule_warmup": 1, "profiler_schedule_active": active,
        "profiler_schedule_repeat": 1, "log_interval": 100, "eval_interval": 1000, "save": None, "load": None})
    tr = Trainer(cfg, load=False)

    def it():
        i = 0
        while True:
            yield {"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i)}
            i += 1
    tr.train(it())
    traces = glob.glob(os.path.join(out, "rank0_step*.pt.trace.json.gz"))
    assert len(traces) == 1, os.listdir(out)
    assert glob.glob(os.path.join(out, "key_averages_step*.txt"))
    with gzip.open(traces[0], "rt") as fh:
        events = json.load(fh)["traceEvents"]
    names = [e.get("name") for e in events if e.get("cat") in ("user_annotation", "cpu_op") or e.get("ph") == "X"]
    count = lambda n: sum(1 for x in names if x == n)          # noqa: E731
    assert count("TRAIN_STEP_FORWARD") == active * gas
    assert count("TRAIN_STEP_BACKWARD") == active * gas
    assert count("TRAIN_STEP_OPTIMIZER_STEP") == active


def test_cuda_profiler_window_and_nsys_command():
    """The capture-range profiler opens its window after `nsys_warmup_steps` steps and closes it `nsys_num_steps` later;
    the nsys command line wraps the training command with the capture-range flags."""
    import types
    from savanna_b200.utils.profiler import CudaProfiler, EmptyProfiler, build_nsys_command, setup_profiler
    cfg = types.SimpleNamespace(disable_autograd_multithreading=False, nsys_warmup_steps=2, nsys_num_steps=3, emit_nvtx=False,
                                profile_record_shapes=False, should_profile=True, profiler_type="nsys", profile_ranks=[0],
                                rank=0, nsys_stop_on_exit=True)
    p = setup_profiler(cfg)
    assert isinstance(p, CudaProfiler)
    states = []
    for _ in range(7):
        p.step()
        states.append(p.running)
    assert states == [False, True, True, True, False, False, False]
    cfg.rank = 1
    assert type(setup_profiler(cfg)) is EmptyProfiler            # not a profiled rank
    cmd = build_nsys_command(cfg, ["python", "train.py"], "out")
    assert cmd[0] == "nsys" and "--capture-range=cudaProfilerApi" in cmd and "--capture-range-end=stop" in cmd
    assert cmd[-2:] == ["python", "train.py"]


def test_native_library_proxy_opens_an_nvtx_range_per_entry_point(monkeypatch):
    """While NVTX is on (the capture-range profiler's window) every native entry point runs inside a range named after it;
    off, the raw C function objects are returned unchanged, and attribute writes reach the underlying library."""
    import types
    import torch
    from savanna_b200.ops import cuda_ops
    calls = []
    raw = types.SimpleNamespace(sb_demo=lambda a, b: a + b, other=lambda: 7)
    lib = cuda_ops._Library(raw)
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: calls.append(("push", name)))
    monkeypatch.setattr(torch.cuda.nvtx, "range_pop", lambda: calls.append(("pop",)))
    cuda_ops.set_nvtx(False)
    assert lib.sb_demo is raw.sb_demo and lib.sb_demo(1, 2) == 3 and calls == []
    lib.flag = 5
    assert raw.flag == 5 and lib.flag == 5
    cuda_ops.set_nvtx(True)
    try:
        assert lib.sb_demo(2, 3) == 5
        assert calls == [("push", "sb_demo"), ("pop",)]
        assert lib.other() == 7 and len(calls) == 2            # only sb_* entry points are wrapped
        raw.sb_fail = lambda: (_ for _ in ()).throw(ValueError("x"))
        try:
            lib.sb_fail()
        except ValueError:
            pass
        assert calls[-1] == ("pop",)                             # the range is closed on exceptions too
    finally:
        cuda_ops.set_nvtx(False)


def test_memory_snapshotter_writes_every_freq_steps_and_on_oom(tmp_path):
    """The snapshot schedule, file layout and the out-of-memory dump, with the two allocator calls replaced."""
    import pickle
    from savanna_b200.utils.memory_stats import MemorySnapshotter
    calls = []
    snap = MemorySnapshotter(str(tmp_path), rank=3, step=10, freq=2, max_entries=77,
                             recorder=lambda **kw: calls.append(kw), snapshot=lambda: {"segments": [1, 2]},
                             printer=lambda *_: None)
    assert calls == [{"max_entries": 77}]
    for _ in range(4):
        snap.step()                                   # steps 11 .. 14: snapshots at 12 and 14
    snap.on_oom()
    snap.close()
    assert calls[-1] == {"enabled": None}
    rel = [p.replace(str(tmp_path), "") for p in snap.written]
    assert rel == ["/rank3/iteration_12/rank3_memory_snapshot.pickle", "/rank3/iteration_14/rank3_memory_snapshot.pickle",
                   "/rank3/iteration_14_exit/rank3_memory_snapshot.pickle"]
    with open(snap.written[0], "rb") as fh:
        assert pickle.load(fh) == {"segments": [1, 2]}

    class Cfg:
        enable_memory_snapshot = False
        memory_snapshot_rank0_only = True
    assert MemorySnapshotter.from_config(Cfg, 0) is None


def test_alloc_stats_reporting_ranks_and_gradient_zero_share(tmp_path):
    """`mem_alloc_stats_ranks` picks every n-th rank; `log_grad_pct_zeros` logs the share of zero gradient entries."""
    import os
    from savanna_b200.config import GlobalConfig
    from savanna_b200.utils import observability
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_cpu.yml")],
                                 {"global_num_gpus": 1, "print_mem_alloc_stats": True, "mem_alloc_stats_ranks": 4,
                                  "log_grad_pct_zeros": True, "log_interval": 1})
    assert observability.build_from_config(cfg, 0, 8)[2] is not None
    assert observability.build_from_config(cfg, 4, 8)[2] is not None
    assert observability.build_from_config(cfg, 5, 8)[2] is None
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.train.trainer import Trainer
    from savanna_b200.utils.logging import TrainingLogger
    tr = Trainer(cfg, load=False)
    logged = {}
    lg = TrainingLogger(cfg, tr)
    lg._log = lambda k, v, it: logged.__setitem__(k, v)

    def it():
        i = 0
        while True:
            yield {"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i)}
            i += 1
    loss = tr.train_step(it())
    lg.log_step(loss, 0.1)
    keys = [k for k in logged if k.startswith("pct_grad_zeros/")]
    assert keys and all(0.0 <= logged[k] <= 100.0 for k in keys)


def test_weight_decay_groups_follow_the_reference_rules():
    """Module-by-module grouping: norms and `bias` parameters are never decayed; the explicit Hyena-MR filter is free of
    decay only while `hyena_filter_wd` is 0 (then in its own group when `lr_medium_hyena` differs); the modal Hyena-LI
    filter, `conv_bias` and the depthwise convolution weights are decayed, as the reference's class list leaves them;
    with `weight_decay` 0 there is one group."""
    import os
    from savanna_b200.config import GlobalConfig
    from savanna_b200.models.backbone import param_groups
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    yml = [os.path.join(root, "configs", "baseline", "tiny_sh2_cpu.yml")]

    def groups_of(**over):
        cfg = GlobalConfig.from_ymls(yml, {"global_num_gpus": 1, **over})
        tr = Trainer(cfg, load=False)
        names = {id(p): n for n, p in tr.model.named_parameters()}
        out = {g["name"]: sorted(names[id(p)] for p in g["params"]) for g in param_groups(tr.model, cfg)}
        assert sum(len(v) for v in out.values()) == len(names)            # every parameter in exactly one group
        return out
    g = groups_of(weight_decay=0.1)
    assert any(n.endswith("filter.h") for n in g["no_decay"]) and not any(n.endswith("filter.h") for n in g["decay"])
    assert all(("layernorm" not in n and not n.endswith(".bias") and not n.endswith("norm.weight")) for n in g["decay"])
    for tail in ("filter.gamma", "filter.R", "filter.p", "mixer.conv_bias", "short_conv_weight", "word_embeddings.weight"):
        assert any(n.endswith(tail) for n in g["decay"]), tail
    assert any(n.endswith("mixer.dense.bias") for n in g["no_decay"])
    g = groups_of(weight_decay=0.1, hyena_filter_wd=0.1)
    assert any(n.endswith("filter.h") for n in g["decay"])
    g = groups_of(weight_decay=0.1, lr_medium_hyena=1e-5)
    assert all(n.endswith("filter.h") for n in g["medium_hyena"]) and g["medium_hyena"]
    g = groups_of(weight_decay=0.0)
    assert set(g) == {"no_decay"}
