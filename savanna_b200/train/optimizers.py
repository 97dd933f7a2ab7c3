"""Optimizers other than the ZeRO-partitioned Adam: SGD, SophiaG, SM3, MADGRAD-WD, schedule-free AdamW
(reference: savanna/training.py:1065-1185, savanna/optimizers/{sophia,sm3,madgrad,adam_schedulefree}.py).

They run un-partitioned: gradients are averaged over the data-parallel (x context-parallel) group with one
flat all-reduce, clipped by global norm and handed to the update rule.  `DataParallelOptimizer` gives them
the interface the trainer expects (zero_grad / step -> grad norm / param_groups / state_dict).
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch
import torch.distributed as dist

from ..parallel import state


class SophiaG(torch.optim.Optimizer):
    """Sophia with the Gauss-Newton-Bartlett Hessian estimate: m <- b1 m + (1-b1) g;
    update = clip(m / max(rho * bs * h, 1e-15), 1); `update_hessian()` refreshes h <- b2 h + (1-b2) g*g from
    gradients of a sampled-label loss every k steps."""

    def __init__(self, params, lr=1e-4, betas=(0.965, 0.99), rho=0.04, weight_decay=1e-1, bs=5120):
        super().__init__(params, dict(lr=lr, betas=betas, rho=rho, weight_decay=weight_decay))
        self.bs = bs

    @torch.no_grad()
    def update_hessian(self):
        for g in self.param_groups:
            _, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "hessian" not in st:
                    st["hessian"] = torch.zeros_like(p, dtype=torch.float32)
                st["hessian"].mul_(b2).addcmul_(p.grad.float(), p.grad.float(), value=1 - b2)

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, _ = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "exp_avg" not in st:
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st.setdefault("hessian", torch.zeros_like(p, dtype=torch.float32))
                m, h = st["exp_avg"], st["hessian"]
                m.mul_(b1).add_(p.grad.float(), alpha=1 - b1)
                pf = p.float()
                pf.mul_(1 - g["lr"] * g["weight_decay"])
                ratio = (m.abs() / (g["rho"] * self.bs * h + 1e-15)).clamp(max=1.0)
                pf.addcmul_(m.sign(), ratio, value=-g["lr"])
                p.copy_(pf)


class SM3(torch.optim.Optimizer):
    """Memory-efficient adaptive optimizer: one accumulator per tensor axis instead of per element."""

    def __init__(self, params, lr=0.1, momentum=0.0, beta=0.0, eps=1e-30):
        super().__init__(params, dict(lr=lr, momentum=momentum, beta=beta, eps=eps))

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float()
                st = self.state[p]
                shape = grad.shape
                if not st:
                    st["step"] = 0
                    st["acc"] = [torch.zeros([s if i == d else 1 for i, s in enumerate(shape)], device=p.device)
                                 for d in range(max(1, grad.dim()))] if grad.dim() > 0 else [torch.zeros((), device=p.device)]
                    if g["momentum"] > 0:
                        st["mom"] = torch.zeros_like(grad)
                st["step"] += 1
                acc = st["acc"][0]
                for a in st["acc"][1:]:
                    acc = torch.min(acc, a)
                if g["beta"] > 0:
                    acc = acc * g["beta"] + grad * grad * (1 - g["beta"])
                else:
                    acc = acc + grad * grad
                for d, a in enumerate(st["acc"]):
                    if grad.dim() > 0:
                        dims = [i for i in range(grad.dim()) if i != d]
                        a.copy_(torch.max(a, acc.amax(dim=dims, keepdim=True) if dims else acc))
                    else:
                        a.copy_(acc)
                upd = grad / (acc.sqrt() + g["eps"])
                if g["momentum"] > 0:
                    st["mom"].mul_(g["momentum"]).add_(upd, alpha=1 - g["momentum"])
                    upd = st["mom"]
                p.add_(upd.to(p.dtype), alpha=-g["lr"])


class MadgradWD(torch.optim.Optimizer):
    """MADGRAD (momentumised dual averaging with cube-root denominator) with decoupled weight decay."""

    def __init__(self, params, lr=1e-2, momentum=0.9, weight_decay=0.0, eps=1e-6):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, eps=eps, k=0))

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            k, lr, mom = g["k"], g["lr"] + g["eps"], g["momentum"]
            lamb = lr * math.sqrt(k + 1)
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float()
                st = self.state[p]
                if not st:
                    st["sum_sq"] = torch.zeros_like(grad)
                    st["s"] = torch.zeros_like(grad)
                    st["x0"] = p.detach().float().clone()
                if g["weight_decay"] != 0:
                    # decoupled decay of the iterate only, with the eps-shifted rate; the anchor x0 is left alone
                    # (reference: savanna/optimizers/madgrad.py:131-133)
                    p.mul_(1 - lr * g["weight_decay"])
                if mom > 0:
                    x0 = st["x0"]
                else:                                   # without momentum the anchor is recovered from the iterate
                    x0 = p.float() + st["s"] / st["sum_sq"].pow(1 / 3).add_(g["eps"])
                st["sum_sq"].addcmul_(grad, grad, value=lamb)
                st["s"].add_(grad, alpha=lamb)
                rms = st["sum_sq"].pow(1 / 3).add_(g["eps"])
                z = x0 - st["s"] / rms
                p.copy_((p.float() * mom + z * (1 - mom)).to(p.dtype)) if mom > 0 else p.copy_(z.to(p.dtype))
            g["k"] = k + 1


class AdamWScheduleFree(torch.optim.Optimizer):
    """Schedule-free AdamW (interpolated iterates y = (1-b1) z + b1 x; call train()/eval() to switch)."""

    def __init__(self, params, lr=2.5e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, warmup_steps=0, r=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, warmup_steps=warmup_steps,
                                      r=r, k=0, train_mode=True, weight_sum=0.0))

    @torch.no_grad()
    def eval(self):
        for g in self.param_groups:
            if g["train_mode"]:
                b1, _ = g["betas"]
                for p in g["params"]:
                    st = self.state[p]
                    if "z" in st:
                        p.lerp_(st["z"].to(p.dtype), 1 - 1 / b1)
                g["train_mode"] = False

    @torch.no_grad()
    def train(self):
        for g in self.param_groups:
            if not g["train_mode"]:
                b1, _ = g["betas"]
                for p in g["params"]:
                    st = self.state[p]
                    if "z" in st:
                        p.lerp_(st["z"].to(p.dtype), 1 - b1)
                g["train_mode"] = True

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            k = g["k"]
            sched = min(1.0, (k + 1) / g["warmup_steps"]) if g["warmup_steps"] > 0 else 1.0
            bc2 = 1 - b2 ** (k + 1)
            lr = g["lr"] * sched * math.sqrt(bc2)
            w = (k + 1) ** g["r"] * lr * lr
            g["weight_sum"] += w
            ck = w / g["weight_sum"] if g["weight_sum"] > 0 else 0.0
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["z"] = p.detach().float().clone()
                    st["v"] = torch.zeros_like(st["z"])
                grad = p.grad.float()
                st["v"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                den = st["v"].sqrt().add_(g["eps"])
                gn = grad / den
                y = p.float()
                if g["weight_decay"] != 0:
                    gn = gn + g["weight_decay"] * y
                y = y.lerp(st["z"], ck)
                y.add_(gn, alpha=lr * (b1 * (1 - ck) - 1))
                st["z"].sub_(gn, alpha=lr)
                p.copy_(y.to(p.dtype))
            g["k"] = k + 1


class DataParallelOptimizer:
    """Adapter: gradient averaging over the replica group + global-norm clipping around a torch-style optimizer."""

    def __init__(self, inner: torch.optim.Optimizer, clip_grad: float, group, world: int, sum_ranks: int = 1):
        self.inner, self.clip_grad, self.group, self.world = inner, clip_grad or 0.0, group, world
        # `sum_ranks` ranks of the group (the context-parallel ranks of one replica) hold partial gradients that are
        # summed; the remaining factor of the group (data-parallel replicas) is averaged
        self.sum_ranks = sum_ranks if (sum_ranks and world % sum_ranks == 0) else 1
        self.param_groups = inner.param_groups
        for g in self.param_groups:
            g.setdefault("lr_mult", 1.0)
        self.fused = None
        self.step_count = 0
        self.last_grad_norm = None

    def zero_grad(self, set_to_none: bool = False):
        self.inner.zero_grad(set_to_none=False)

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        self.step_count += 1
        params = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
        if self.world > 1 and params:
            flat = torch.cat([p.grad.reshape(-1).float() for p in params])
            dist.all_reduce(flat, group=self.group)
            flat.mul_(float(self.sum_ranks) / float(self.world))
            off = 0
            for p in params:
                p.grad.copy_(flat[off:off + p.numel()].view_as(p.grad))
                off += p.numel()
        tp = state.get_model_parallel_world_size()
        sq = torch.zeros((), dtype=torch.float32, device=params[0].device if params else "cpu")
        for p in params:
            w = 1.0 if (tp == 1 or getattr(p, "model_parallel", False)) else 1.0 / tp
            sq += w * p.grad.float().pow(2).sum()
        if tp > 1:
            dist.all_reduce(sq, group=state.get_model_parallel_group())
        norm = sq.sqrt()
        if self.clip_grad > 0:
            coef = torch.clamp(self.clip_grad / (norm + 1e-6), max=1.0)
            for p in params:
                p.grad.mul_(coef.to(p.grad.dtype))
        self.inner.step()
        self.last_grad_norm = norm
        return norm

    def state_dict(self) -> Dict:
        return {"inner": self.inner.state_dict(), "step_count": self.step_count}

    def load_state_dict(self, sd: Dict, load_master: bool = True) -> None:
        self.inner.load_state_dict(sd["inner"])
        self.step_count = sd.get("step_count", 0)


def build_generic_optimizer(kind: str, groups: List[Dict], cfg, params: Dict) -> DataParallelOptimizer:
    lr = cfg.lr
    tgroups = [{"params": g["params"], "weight_decay": g.get("weight_decay", 0.0), "lr": g.get("lr", lr)} for g in groups]
    if kind == "sgd":
        inner = torch.optim.SGD(tgroups, lr=lr, momentum=params.get("momentum", 0.0))
    elif kind == "sophia":
        inner = SophiaG(tgroups, lr=lr, betas=tuple(params.get("betas", (0.965, 0.99))), rho=params.get("rho", 0.04),
                        weight_decay=cfg.weight_decay, bs=cfg.train_batch_size * cfg.seq_length)
    elif kind == "sm3":
        inner = SM3(tgroups, lr=lr, momentum=params.get("momentum", 0.0), beta=params.get("beta", 0.0))
    elif kind == "madgrad_wd":
        inner = MadgradWD(tgroups, lr=lr, momentum=params.get("momentum", 0.9), weight_decay=cfg.weight_decay)
    elif kind == "adamw_schedulefree":
        inner = AdamWScheduleFree(tgroups, lr=lr, betas=tuple(params.get("betas", (0.9, 0.999))), weight_decay=cfg.weight_decay)
    else:
        raise ValueError(f"optimizer type {kind!r} is not implemented")
    ranks = state.get_sequence_data_parallel_ranks()
    return DataParallelOptimizer(inner, cfg.gradient_clipping, state.get_sequence_data_parallel_group(), len(ranks),
                                 sum_ranks=state.get_context_parallel_world_size())
