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
    assert os.path.exists(tmp_path / "poison.rank2.gen0")
    other = Watchdog(10.0, str(tmp_path), rank=0)
    other._started_wall -= 5.0             # a peer of the same launch: it started before the stall was reported
    with pytest.raises(RuntimeError):
        other.beat(6)                      # sees rank 2's poison file at its next heartbeat


def test_stale_poison_is_ignored_after_restart(tmp_path, monkeypatch):
    """A relaunch into the same heartbeat directory must not be stopped by the previous attempt's poison files."""
    fired = []
    wd = Watchdog(0.2, str(tmp_path), rank=1, on_timeout=fired.append, poll=0.05)
    wd.start()
    time.sleep(0.5)
    wd.stop()
    assert wd.fired and os.path.exists(tmp_path / "poison.rank1.gen0")
    time.sleep(1.2)
    # same generation number (a relaunch outside torchrun): the file predates the new watchdog and is ignored
    again = Watchdog(10.0, str(tmp_path), rank=0)
    again.start()
    again.beat(1)
    again.stop()
    # rank 1's own relaunch removes its leftover
    own = Watchdog(10.0, str(tmp_path), rank=1)
    own.start()
    own.stop()
    assert not os.path.exists(tmp_path / "poison.rank1.gen0")
    # a torchrun restart carries a new generation: files of generation 0 are not this launch's
    wd2 = Watchdog(0.2, str(tmp_path), rank=3, on_timeout=fired.append, poll=0.05)
    wd2.start(); time.sleep(0.5); wd2.stop()
    monkeypatch.setenv("TORCHELASTIC_RESTART_COUNT", "1")
    nxt = Watchdog(10.0, str(tmp_path), rank=0)
    nxt._started_wall -= 5.0
    nxt.beat(1)


def test_paused_watchdog_does_not_fire_during_long_host_phase(tmp_path):
    fired = []
    wd = Watchdog(0.2, str(tmp_path), rank=0, on_timeout=fired.append, poll=0.05)
    wd.start()
    with wd.paused():                      # stands for a checkpoint save or an evaluation longer than the deadline
        time.sleep(0.7)
    time.sleep(0.1)
    assert not wd.fired
    time.sleep(0.5)                        # outside the pause the deadline applies again
    wd.stop()
    assert wd.fired


def test_status_word_aborts_the_training_loop(tmp_path):
    """A non-zero device status word (a kernel gave up on a bounded wait) stops `Trainer.train` at the next
    logging interval and before any checkpoint is written.  The word is set on the host; no GPU is involved."""
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_cpu.yml")],
                                 {"global_num_gpus": 1, "save": str(tmp_path / "ck"), "train_iters": 6, "log_interval": 2,
                                  "save_iters": [4], "eval_interval": 0})
    tr = Trainer(cfg, load=False)
    word = {"v": 0}
    tr.status_reader = lambda: word["v"]

    def it():
        i = 0
        while True:
            if i == 2 * cfg.gradient_accumulation_steps:
                word["v"] = (3 << 24) | 7     # "peer wait timed out", detail 7, raised during the third step
            yield {"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, i)}
            i += 1
    with pytest.raises(RuntimeError, match="bounded wait: code 3, detail 7"):
        tr.train(it())
    assert tr.iteration == 4                 # stopped at the first logging interval after the word was set
    assert not os.path.exists(tmp_path / "ck" / "global_step4")


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
