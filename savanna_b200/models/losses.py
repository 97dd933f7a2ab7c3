"""Training losses (reference: savanna/model/backbone.py:57-206).

cross_entropy          masked mean of the per-token CE; under context parallelism numerator and
                       denominator are summed over the context-parallel group.
reweighted_cross_entropy   lowercase tokens (soft-masked DNA) weigh `lowercase_weight`; weights are
                       renormalised so they sum to the number of unmasked tokens.
oadm_loss / dpo_loss   order-agnostic diffusion and direct-preference objectives.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import ops
from ..parallel import state
from ..parallel.cross_entropy import vocab_parallel_cross_entropy


class _CPSum(torch.autograd.Function):
    """Sum over the context-parallel group; the gradient passes through unchanged (every rank holds the
    same summed loss and back-propagates its own share)."""

    @staticmethod
    def forward(ctx, x):
        y = x.clone()
        dist.all_reduce(y, group=state.get_context_parallel_group())
        return y

    @staticmethod
    def backward(ctx, g):
        return g


def _masked_mean(losses, weights, mask):
    num = (losses.float() * weights.float()).sum()
    den = mask.float().sum()
    if state.get_context_parallel_world_size() > 1:
        num, den = _CPSum.apply(num), _CPSum.apply(den)
    return num / den.clamp(min=1.0)


def cross_entropy(logits, labels, loss_mask, vocab_parallel: bool = False):
    losses = vocab_parallel_cross_entropy(logits, labels) if vocab_parallel else ops.cross_entropy(logits, labels)
    return _masked_mean(losses, loss_mask, loss_mask)


def lowercase_weights(labels, loss_mask, lowercase_weight: float = 0.1):
    """Weights 1 for upper-case / non-letter byte tokens, `lowercase_weight` for a..z, renormalised."""
    lower = (labels >= 97) & (labels <= 122)
    w = torch.where(lower, torch.full_like(loss_mask, lowercase_weight, dtype=torch.float32), torch.ones_like(loss_mask, dtype=torch.float32))
    w = w * loss_mask.float()
    num, den = loss_mask.float().sum(), w.sum()
    if state.get_context_parallel_world_size() > 1:
        num, den = _CPSum.apply(num), _CPSum.apply(den)
    return w * (num / den.clamp(min=1e-8))


def reweighted_cross_entropy(logits, labels, loss_mask, lowercase_weight: float = 0.1, normalize_per_batch: bool = True,
                             vocab_parallel: bool = False):
    # the target is the upper-case letter (the model never sees case); the case of the label only sets the weight
    lower = (labels >= 97) & (labels <= 122)
    target = torch.where(lower, labels - 32, labels)
    losses = vocab_parallel_cross_entropy(logits, target) if vocab_parallel else ops.cross_entropy(logits, target)
    if normalize_per_batch:
        w = lowercase_weights(labels, loss_mask, lowercase_weight)
    else:
        w = torch.where(lower, lowercase_weight, 1.0) * loss_mask.float()
    return _masked_mean(losses, w, loss_mask)


def oadm_loss(logits, labels, loss_mask, t_frac=None, pad_token: int = 1):
    """Order-agnostic autoregressive diffusion (reference: savanna/model/backbone.py:151-171): the cross-entropy of a
    row's masked positions is weighted by (non-pad tokens of the row) / (masked positions of the row), the term of the
    diffusion bound for the row's time step, and the batch is normalised by its number of masked positions."""
    mask = loss_mask.float()
    losses = ops.cross_entropy(logits, labels).float() * mask
    n_masked = mask.sum(-1).clamp(min=1.0)
    non_pad = (labels != pad_token).sum(-1).float()
    return ((non_pad / n_masked)[:, None] * losses).sum() / mask.sum().clamp(min=1.0)


def dpo_loss(policy_chosen_logps, policy_rejected_logps, ref_chosen_logps, ref_rejected_logps, beta: float = 1.0):
    pi = policy_chosen_logps - policy_rejected_logps
    rf = ref_chosen_logps - ref_rejected_logps
    losses = -F.logsigmoid(beta * (pi - rf))
    chosen_r = beta * (policy_chosen_logps - ref_chosen_logps).detach()
    rejected_r = beta * (policy_rejected_logps - ref_rejected_logps).detach()
    return losses.mean(), chosen_r, rejected_r


def sequence_logps(logits, labels, loss_mask, positions=None):
    """Per-row log-probability as the reference's preference loss measures it (savanna/model/backbone.py:190-197): the
    masked token log-probabilities summed and divided by the number of label positions (a mean over all positions, the
    masked-out ones counting as zero).  `positions` is that count; the reference's preference batches hold
    seq_length - 1 labels (training.py:680-712: rows are padded to seq_length, then shifted), which is what the trainer
    passes so that stored reference log-probabilities are on the same scale.  Default: the row length."""
    lp = -ops.cross_entropy(logits, labels)
    return (lp * loss_mask.float()).sum(-1) / float(positions or lp.shape[-1])
