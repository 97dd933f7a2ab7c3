"""Failure detection is exercised on the host only: a step that never finishes trips the watchdog, a
rank that raises is reported by the launcher harness, a truncated checkpoint is rejected on load."""
import os
import time

import pytest
import torch

from savanna_b200.utils.watchdog import OverflowMonitor, Watchdog
from tests.dist_utils import run_distributed


def test_watchdog_fires_and_writes_poison(tmp_path):
    fired = []
    wd = Watchdog(0.3, str(tmp_path), rank=2, on_timeout=fired.append, poll=0.05)
    wd.start()
    wd.beat(5)
    time.sleep(0.1)
    assert not wd.fired
    time.sleep(0.6)
    wd.stop()
    assert wd.fired and fired == [5]
    assert os.path.exists(tmp_path / "poison.rank2")
    other = Watchdog(10.0, str(tmp_path), rank=0)
    with pytest.raises(RuntimeError):
        other.beat(6)                      # sees rank 2's poison file at its next heartbeat


def test_watchdog_quiet_when_beating(tmp_path):
    wd = Watchdog(0.4, str(tmp_path), rank=0, on_timeout=lambda it: None, poll=0.05)
    wd.start()
    for i in range(8):
        time.sleep(0.1)
        wd.beat(i)
    wd.stop()
    assert not wd.fired


def test_overflow_monitor():
    m = OverflowMonitor(3)
    m.check(True); m.check(False); m.check(True); m.check(True)
    with pytest.raises(RuntimeError):
        m.check(True)


def _w_rank_raises(rank, world):
    import torch.distributed as dist
    if rank == 1:
        raise ValueError("injected failure on rank 1")
    t = torch.ones(1)
    dist.all_reduce(t)          # the peers' collective ends with an error once rank 1 is gone


def test_rank_failure_is_reported():
    with pytest.raises(RuntimeError) as e:
        run_distributed(_w_rank_raises, 2, timeout=60)
    assert "injected failure on rank 1" in str(e.value)


def test_truncated_checkpoint_is_rejected(tmp_path):
    from savanna_b200.ckpt import load_checkpoint, save_checkpoint
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_cpu.yml")],
                                 {"global_num_gpus": 1, "save": str(tmp_path)})
    tr = Trainer(cfg, load=False)
    tr.train_step(iter([{"text": acgt_batch(2, cfg.seq_length, 0)}]))
    d = save_checkpoint(tr)
    path = os.path.join(d, "mp_rank_00_model_states.pt")
    data = open(path, "rb").read()
    open(path, "wb").write(data[: len(data) // 2])
    cfg.load = str(tmp_path)
    with pytest.raises(Exception):
        load_checkpoint(tr)
