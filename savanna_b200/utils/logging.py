"""Training log line, sinks (stdout / TensorBoard / wandb), Tee, and the approximate-FLOPs helper.

Per step: lr, loss, gradient norm; every `log_interval` steps additionally samples/s, iteration time,
tokens/s per GPU, tokens consumed, model and hardware FLOP/s, MFU and HFU against the measured B200
peak, allocator statistics and skipped / NaN counters (reference: savanna/logging.py:150-521; its MFU is
silently skipped on Blackwell because its peak table has no entry — here the peak comes from
utils/mfu.py).
"""
from __future__ import annotations

import contextlib
import math
import os
import sys
import time
from typing import Dict, Optional

import torch
import torch.distributed as dist

from .. import print_rank_0
from . import memory_stats as mem
from .mfu import mfu as mfu_fn


class Tee:
    """Duplicate a stream into a file (per-host log files, logging.py:77-111)."""

    def __init__(self, path: str, err: bool = False):
        self.file = open(path, "w")
        self.err = err
        self.std = sys.stderr if err else sys.stdout
        if err:
            sys.stderr = self
        else:
            sys.stdout = self

    def write(self, data):
        try:
            self.file.write(data)
        except OSError:
            pass
        self.std.write(data)

    def flush(self):
        try:
            self.file.flush()
        except OSError:
            pass
        self.std.flush()

    def close(self):
        if self.err:
            sys.stderr = self.std
        else:
            sys.stdout = self.std
        self.file.close()


def human_readable_flops(f: float) -> str:
    for unit in ("", "K", "M", "G", "T", "P", "E"):
        if abs(f) < 1000.0:
            return f"{f:.2f} {unit}FLOPS"
        f /= 1000.0
    return f"{f:.2f} ZFLOPS"


def approx_flops_per_token(num_params: int, cfg) -> float:
    """The reference's quick estimate: 6*params + 60*L*D*layers*? folded per token (logging.py:131-140);
    kept for comparable log lines — the MFU figures use the per-operator model in utils/mfu.py."""
    ckpt_factor = 4 if cfg.checkpoint_activations else 3
    return ckpt_factor * 2 * (num_params + 2 * cfg.num_layers * cfg.seq_length * cfg.hidden_size)


def tb_wandb_log(key: str, value, iteration: int, use_wandb: bool, tensorboard_writer=None) -> None:
    if tensorboard_writer is not None:
        try:
            tensorboard_writer.add_scalar(key, value, iteration)
        except Exception:
            pass
    if use_wandb:
        try:
            import wandb
            wandb.log({key: value}, step=iteration)
        except Exception:
            pass


def init_wandb(cfg) -> bool:
    if not cfg.use_wandb:
        return False
    if (cfg.rank or 0) != 0 and not cfg.wandb_init_all_ranks:
        cfg.use_wandb = False
        return False
    try:
        import wandb
        wandb.init(project=cfg.wandb_project, group=cfg.wandb_group, name=cfg.wandb_run_name, entity=cfg.wandb_team,
                   config=cfg.to_dict(only_non_default=True), save_code=False, force=False)
        return True
    except Exception as exc:
        print_rank_0(f"wandb unavailable ({exc}); continuing without it")
        cfg.use_wandb = False
        return False


class ActivationNormRecorder:
    """Per-layer activation norms of the sequence mixers (`log_attn_norms`, `log_hyena_norms`; the reference logs
    `x.norm(2, -1).max(1).mean(0)` of the attention / Hyena outputs from rank 0, savanna/model/block.py:60-79,
    1122-1192, operators/hyena/hyena.py:383-402).  Forward hooks keep the latest value per layer as a device scalar;
    the logger reads them at the logging interval only."""

    def __init__(self, model, cfg):
        self.values: Dict[str, torch.Tensor] = {}
        self.handles = []
        if not (cfg.log_attn_norms or cfg.log_hyena_norms) or not hasattr(model, "blocks"):
            return
        for b in model.blocks():
            op = getattr(b, "operator_type", "")
            hyena = op.startswith("hyena")
            if (hyena and not cfg.log_hyena_norms) or (not hyena and not cfg.log_attn_norms):
                continue
            key = f"{'hyena' if hyena else 'attention'}_output_norm_{b.layer_number}" if hasattr(b, "layer_number") \
                else f"{'hyena' if hyena else 'attention'}_output_norm_{len(self.handles)}"
            self.handles.append(b.mixer.register_forward_hook(self._hook(key)))

    def _hook(self, key):
        def fn(_m, _a, out):
            t = out[0] if isinstance(out, (tuple, list)) else out
            if isinstance(t, torch.Tensor) and t.dim() == 3:
                with torch.no_grad():
                    self.values[key] = t.detach().float().norm(2, dim=-1).max(1).values.mean(0)
        return fn

    def read(self) -> Dict[str, float]:
        return {k: float(v) for k, v in self.values.items()}


class TrainingLogger:
    def __init__(self, cfg, trainer):
        self.cfg, self.trainer = cfg, trainer
        self.act_norms = ActivationNormRecorder(trainer.model, cfg)
        self.interval = max(1, cfg.log_interval or 1)
        self.t_acc, self.n_acc, self.loss_acc = 0.0, 0, 0.0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.use_wandb = init_wandb(cfg)
        self.tb = cfg.tensorboard_writer
        self.tee = None
        if cfg.log_dir:
            os.makedirs(cfg.log_dir, exist_ok=True)
            if (cfg.local_rank or 0) == 0:
                self.tee = Tee(os.path.join(cfg.log_dir, f"{os.uname().nodename}_stdout.txt"))

    def _log(self, key, value, it):
        if (self.cfg.rank or 0) == 0:
            tb_wandb_log(key, value, it, self.use_wandb, self.tb)

    def log_step(self, loss: torch.Tensor, step_time: float) -> None:
        cfg, tr = self.cfg, self.trainer
        it = tr.iteration
        self.t_acc += step_time
        self.n_acc += 1
        if it % self.interval != 0:
            return
        lossv = float(loss)                      # the only host read of the step, at the logging interval
        gn = float(tr.grad_norm) if getattr(tr, "grad_norm", None) is not None else float("nan")
        if math.isnan(lossv) or math.isinf(lossv):
            tr.nan_iters += 1
        dt = self.t_acc / self.n_acc
        self.t_acc, self.n_acc = 0.0, 0
        tokens_per_step = cfg.train_batch_size * cfg.seq_length
        tps = tokens_per_step / dt
        tps_gpu = tps / self.world
        m = mfu_fn(tps_gpu, cfg, recompute=cfg.checkpoint_activations)
        lr = tr.optimizer.param_groups[0]["lr"]
        self._log("train/lm_loss", lossv, it)
        self._log("train/learning_rate", lr, it)
        self._log("train/grad_norm", gn, it)
        self._log("runtime/iteration_time", dt, it)
        self._log("runtime/samples_per_sec", cfg.train_batch_size / dt, it)
        self._log("runtime/tokens_per_sec_per_gpu", tps_gpu, it)
        self._log("runtime/model_flops_per_sec_per_gpu", m["model_flops_per_sec"], it)
        if m["mfu"] is not None:
            self._log("runtime/mfu", m["mfu"], it)
            self._log("runtime/hfu", m["hfu"], it)
        self._log("train/tokens", tr.tokens_seen, it)
        if getattr(tr, "loss_scaler", None) is not None:
            self._log("train/loss_scale", tr.loss_scaler.scale, it)
        if getattr(tr, "curriculum", None) is not None:
            self._log("train/curriculum_seqlen", cfg.curriculum_seqlen, it)
        line = (f" iteration {it:8d}/{cfg.train_iters:8d} | elapsed per iteration (ms): {dt * 1e3:.1f} | "
                f"lr: {lr:.3E} | lm_loss: {lossv:.6E} | grad norm: {gn:.3f} | tokens/s/gpu: {tps_gpu:,.0f} | "
                f"tokens: {tr.tokens_seen:,} | model {human_readable_flops(m['model_flops_per_sec'])}/gpu")
        if m["mfu"] is not None:
            line += f" | MFU {100 * m['mfu']:.1f}% HFU {100 * m['hfu']:.1f}%"
        line += f" | skipped: {tr.skipped_iters} | nan: {tr.nan_iters}"
        if getattr(tr, "loss_scaler", None) is not None:
            line += f" | loss scale: {tr.loss_scaler.scale:.1f}"
        if cfg.log_memory_stats and torch.cuda.is_available():
            st = mem.memory_stats()
            line += " | " + mem.format_memory_stats(st)
            for k, v in st.items():
                self._log(f"memory/{k}", v, it)
        if cfg.log_memory_alloc_counts and torch.cuda.is_available():
            line += f" | alloc counts {mem.gather_alloc_counts()}"
        for k, v in self.act_norms.read().items():
            self._log(f"activations/{k}", v, it)
        ns = getattr(tr, "noise_scale", None)
        if cfg.log_gradient_noise_scale and ns is not None and ns.noise_scale is not None:
            self._log("train/noise_scale", ns.noise_scale, it)
            line += f" | noise scale: {ns.noise_scale:.3E}"
        if cfg.log_optimizer_states and hasattr(tr.optimizer, "groups"):
            for i, g in enumerate(tr.optimizer.groups):
                name = getattr(g, "name", None) or g.hyper.get("name", str(i))
                self._log(f"optimizer_state_norms/{name}_{i}/exp_avg", float(g.exp_avg.float().norm()), it)
                self._log(f"optimizer_state_norms/{name}_{i}/exp_avg_sq", float(g.exp_avg_sq.float().norm()), it)
        if cfg.log_param_norm or cfg.log_grad_norm or cfg.log_grad_pct_zeros:
            # ZeRO stage 2 / 3 keep no whole gradients after the step and (stage 3) no whole parameters: gather the
            # parameters for the read, skip the per-parameter gradient norms
            part = getattr(tr, "partitioned", False)
            ctx = tr.optimizer.full_params() if part else contextlib.nullcontext()
            with ctx:
                for name, p in tr.model.named_parameters():
                    if cfg.log_param_norm:
                        self._log(f"param_norm/{name}", float(p.detach().float().norm()), it)
                    if cfg.log_grad_norm and not part and p.grad is not None:
                        self._log(f"grad_norm/{name}", float(p.grad.detach().float().norm()), it)
                    if cfg.log_grad_pct_zeros and not part and p.grad is not None:
                        # share of exactly-zero gradient entries: dead units, saturated gates, underflow in low precision
                        self._log(f"pct_grad_zeros/{name}", float((p.grad.detach() == 0).float().mean()) * 100.0, it)
        print_rank_0(line)

    def log_eval(self, results: Dict[str, float], it: int, prefix: str = "validation") -> None:
        s = f" {prefix} results at iteration {it} | " + " | ".join(f"{k} value: {v:.6E}" for k, v in results.items())
        print_rank_0("-" * len(s))
        print_rank_0(s)
        print_rank_0("-" * len(s))
        for k, v in results.items():
            self._log(f"{prefix}/{k}", v, it)
