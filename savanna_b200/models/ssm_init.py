"""State-space initialisers for modal / diagonal long-convolution filters: HiPPO transition matrices, their
normal-plus-low-rank (NPLR) diagonalisation and diagonal-plus-low-rank (DPLR) pole layouts.

    transition(measure, N)            (A [N, N], B [N, 1]) of the HiPPO operator for `legs`, `legt`, `lagt`, `fourier`
    rank_correction(measure, N, rank) P [rank, N] with A + P^T P normal (skew-symmetric plus a multiple of I)
    nplr(measure, N, rank)            (w [N/2], P [rank, N/2], B [N/2], V [N, N/2]): eigenvalues of the normal part
                                      (one of each conjugate pair) and P, B in that eigenbasis
    dplr(scaling, N, rank, H, ...)    closed-form pole layouts (`linear`: -1/2 + i pi n, `inverse`, `quadratic`, `real`,
                                      `random`, `legs`: imaginary parts of the HiPPO-LegS spectrum) for H filter copies
    ssm(measure, N, R, H)             dispatcher (`dplr`, `diag-<scaling>`, or a HiPPO measure repeated H times)
    combination(measures, N, R, S)    S copies split evenly over several measures ("hippo", "diag", "all" or a list)

`models/filters.py:ComplexModalFilter` starts from `dplr("linear")`; the other layouts are alternative starting points
for the same parametrisation.  Role of the reference's savanna/model/operators/hyena/parametrization/utils.py:33-399
(the S4 initialisation toolbox), restated with plain tensor algebra.
"""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple, Union

import torch


def embed_c2r(A: torch.Tensor) -> torch.Tensor:
    """Complex [..., m, n] -> real [..., 2m, 2n] with every entry a + ib replaced by the block [[a, -b], [b, a]]."""
    re, im = A.real, A.imag
    top = torch.stack([re, -im], dim=-1).flatten(-2)            # [..., m, 2n]
    bot = torch.stack([im, re], dim=-1).flatten(-2)
    return torch.stack([top, bot], dim=-2).flatten(-3, -2)


def transition(measure: str, N: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """HiPPO (A, B) in float64: x' = A x + B u projects the input history onto N basis functions of the measure."""
    n = torch.arange(N, dtype=torch.float64)
    if measure in ("legs", "legsd"):
        r = torch.sqrt(2 * n + 1)
        A = -torch.tril(r[:, None] * r[None, :], -1) - torch.diag(n + 1)
        B = r[:, None].clone()
    elif measure == "legt":
        r = torch.sqrt(2 * n + 1)
        i, j = torch.meshgrid(n, n, indexing="ij")
        sign = torch.where(i < j, (-1.0) ** (i - j), torch.ones_like(i))
        A = -0.5 * (r[:, None] * sign * r[None, :])
        B = 0.5 * r[:, None]
    elif measure == "lagt":
        A = -0.5 * torch.eye(N, dtype=torch.float64) - torch.tril(torch.ones(N, N, dtype=torch.float64), -1)
        B = torch.ones(N, 1, dtype=torch.float64)
    elif measure == "fourier":
        f = torch.arange(N // 2, dtype=torch.float64)
        d = torch.stack([torch.zeros_like(f), f], dim=-1).reshape(-1)[1:]
        A = math.pi * (-torch.diag(d, 1) + torch.diag(d, -1))
        b = torch.zeros(N, dtype=torch.float64)
        b[0::2] = math.sqrt(2.0)
        b[0] = 1.0
        A = A - b[:, None] * b[None, :]
        B = b[:, None]
    else:
        raise NotImplementedError(f"measure {measure!r}")
    return A, B


def rank_correction(measure: str, N: int, rank: int = 1, dtype=torch.float64) -> torch.Tensor:
    """P [rank, N] such that A + P^T P is normal."""
    n = torch.arange(N, dtype=dtype)
    if measure in ("legs", "legsd"):
        P = torch.sqrt(0.5 + n)[None]
    elif measure == "legt":
        p = torch.sqrt(1 + 2 * n)
        p0, p1 = p.clone(), p.clone()
        p0[0::2] = 0.0
        p1[1::2] = 0.0
        P = torch.stack([p0, p1]) * 2 ** -0.5
    elif measure == "lagt":
        P = math.sqrt(0.5) * torch.ones(1, N, dtype=dtype)
    elif measure == "fourier":
        p = torch.zeros(N, dtype=dtype)
        p[0::2] = math.sqrt(2.0)
        p[0] = 1.0
        P = p[None]
    else:
        raise NotImplementedError(f"measure {measure!r}")
    if rank < P.shape[0]:
        raise ValueError(f"measure {measure!r} needs rank >= {P.shape[0]}")
    if rank > P.shape[0]:
        P = torch.cat([P, torch.zeros(rank - P.shape[0], N, dtype=dtype)])
    return P


def nplr(measure: str, N: int, rank: int = 1, dtype=torch.float32):
    """Diagonalise the normal part of a HiPPO matrix.  Returns (w, P, B, V) in the complex dtype matching `dtype`, keeping
    one eigenvalue of every conjugate pair (non-negative imaginary part, ascending): A = V diag(w) V^H - P P^H on the
    kept half together with its conjugate."""
    cdtype = torch.complex64 if dtype == torch.float32 else torch.complex128
    A, B = transition(measure, N)
    B = B[:, 0]
    P = rank_correction(measure, N, rank)
    AP = A + (P[:, :, None] * P[:, None, :]).sum(0)
    # AP = (skew-symmetric) + c I: the real part of every eigenvalue is the mean of the diagonal
    w_re = torch.diagonal(AP).mean()
    skew = AP - w_re * torch.eye(N, dtype=AP.dtype)
    w_im, V = torch.linalg.eigh((skew * -1j).to(torch.complex128))     # -i * skew is Hermitian
    order = torch.argsort(w_im)
    w_im, V = w_im[order], V[:, order]
    keep = slice(N - N // 2, N)                                       # the half with non-negative imaginary part
    w = (w_re + 1j * w_im)[keep]
    V = V[:, keep]
    Vh = V.conj().t()
    Bc = Vh @ B.to(torch.complex128)
    Pc = (Vh @ P.to(torch.complex128).t()).t()
    if measure == "legsd":
        Pc = torch.zeros_like(Pc)
    return w.to(cdtype), Pc.to(cdtype), Bc.to(cdtype), V.to(cdtype)


def dplr(scaling: str = "linear", N: int = 64, rank: int = 1, H: int = 1, dtype=torch.float32, real_scale: float = 1.0,
         imag_scale: float = 1.0, random_real: bool = False, random_imag: bool = False, normalize: bool = False,
         diagonal: bool = True, random_B: bool = False):
    """Closed-form pole layouts for H copies of an order-N (N/2 conjugate pairs) diagonal state-space filter:
    w [H, N/2] = -real + i imag, P [rank, H, N/2] (zero when `diagonal`), B [H, N/2], V [H, N, N/2]."""
    cdtype = torch.complex64 if dtype == torch.float32 else torch.complex128
    half = N // 2
    real = torch.rand(H, half) if random_real else 0.5 * torch.ones(H, half)
    imag = half * torch.rand(H, half) if random_imag else torch.arange(half, dtype=torch.float32).expand(H, half).clone()
    real = real_scale * real
    if scaling == "random":
        imag = torch.randn(H, half)
    elif scaling == "real":
        imag = torch.zeros(H, half)
        real = 1 + torch.arange(half, dtype=torch.float32).expand(H, half).clone()
    elif scaling in ("linear", "lin"):
        imag = math.pi * imag
    elif scaling in ("inverse", "inv"):
        imag = 1 / math.pi * N * (N / (1 + 2 * imag) - 1)
    elif scaling in ("inverse2", "inv2"):
        imag = 1 / math.pi * N * (N / (1 + imag) - 1)
    elif scaling in ("quadratic", "quad"):
        imag = 1 / math.pi * (1 + 2 * imag) ** 2
    elif scaling in ("legs", "hippo"):
        w, _, _, _ = nplr("legsd", N)
        imag = w.imag.float().expand(H, half).clone()
    else:
        raise NotImplementedError(f"scaling {scaling!r}")
    imag = imag_scale * imag
    w = torch.complex(-real.float(), imag.float()).to(cdtype)
    B = torch.randn(H, half, dtype=cdtype) if random_B else torch.ones(H, half, dtype=cdtype)
    if normalize:
        zeta = 2 * ((-B / w).abs() ** 2).sum(-1, keepdim=True)
        B = B / zeta ** 0.5
    P = torch.randn(rank, H, half, dtype=cdtype)
    if diagonal:
        P = P * 0.0
    V = torch.eye(N, dtype=cdtype)[:, :half].expand(H, N, half).clone()
    return w, P, B, V


def ssm(measure: str, N: int, R: int, H: int, **ssm_args):
    """One initialisation for H independent copies: `dplr`, `diag-<scaling>`, or a HiPPO measure (repeated H times)."""
    if measure == "dplr":
        return dplr(N=N, rank=R, H=H, **ssm_args)
    if measure.startswith("diag"):
        parts = measure.split("-")
        if len(parts) < 2:
            raise ValueError("diagonal initialisations are named diag-<scaling>")
        return dplr(scaling=parts[1], N=N, rank=R, H=H, diagonal=True, **ssm_args)
    w, P, B, V = nplr(measure, N, R, **ssm_args)
    return (w[None].expand(H, -1).clone(), P[:, None].expand(-1, H, -1).clone(), B[None].expand(H, -1).clone(),
            V[None].expand(H, -1, -1).clone())


COMBINATIONS = {"hippo": ["legs", "fourier"], "diag": ["diag-inv", "diag-lin"], "all": ["legs", "fourier", "diag-inv", "diag-lin"]}


def combination(measures: Union[str, Sequence[str]], N: int, R: int, S: int, **ssm_args):
    """S copies split evenly over several measures; results concatenated along the copy dimension."""
    if isinstance(measures, str):
        measures = COMBINATIONS.get(measures, [measures])
    measures = list(measures)
    if S % len(measures):
        raise ValueError(f"{S} copies cannot be split evenly over {len(measures)} measures")
    parts: List = [ssm(m, N, R, S // len(measures), **ssm_args) for m in measures]
    w, P, B, V = zip(*parts)
    return torch.cat(w, 0), torch.cat(P, 1), torch.cat(B, 0), torch.cat(V, 0)
