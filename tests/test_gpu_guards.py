"""Out-of-bounds stores: every operator of the library runs forward and backward with its output buffers allocated
inside guard margins (ops/cuda_ops.py `guarded_allocations`); a kernel that stores outside its output - a wrong tile
bound, an off-by-one row, a bad leading dimension - damages a margin and `check_guards()` names the buffer.  Shapes are
chosen NOT to be multiples of the kernels' tile sizes, so that every partial-tile path runs.  This is the stand-in for
a memory checker: stray stores that land in memory the process owns raise no fault, but they do change the margins."""
import math

import pytest
import torch

from savanna_b200 import ops
from savanna_b200.ops import cuda_ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _run(fn, *leaves):
    with cuda_ops.guarded_allocations():
        out = fn(*leaves)
        out = out[0] if isinstance(out, tuple) else out
        out.backward(torch.randn_like(out))
        n = cuda_ops.check_guards()
    cuda_ops.check_status()
    assert n > 0
    return n


def test_guard_detects_a_stray_store():
    with cuda_ops.guarded_allocations():
        t = cuda_ops._alloc((4, 8), dtype=BF, device=DEV)
        assert cuda_ops.check_guards() == 1
        t.view(-1)[-1:].data_ptr()
        whole = cuda_ops._GUARDED[0][0]
        whole[cuda_ops.GUARD + 32] = 1.0                      # one element past the window
        with pytest.raises(RuntimeError, match="outside its output buffer"):
            cuda_ops.check_guards()


@pytest.mark.parametrize("M,N,K", [(300, 264, 136), (129, 520, 72)])
def test_linear_partial_tiles(M, N, K):
    x = torch.randn(M, K, device=DEV, dtype=BF, requires_grad=True)
    w = torch.randn(N, K, device=DEV, dtype=BF, requires_grad=True)
    b = torch.randn(N, device=DEV, dtype=BF, requires_grad=True)
    _run(lambda a, c, d: ops.linear(a, c, d), x, w, b)


def test_linear_fp8_partial_tiles():
    x = torch.randn(300, 144, device=DEV, dtype=BF, requires_grad=True)
    w = torch.randn(272, 144, device=DEV, dtype=BF, requires_grad=True)
    _run(lambda a, c: ops.linear(a, c, None, fp8=True), x, w)


@pytest.mark.parametrize("K,C,L", [(3, 192, 301), (4, 72, 130)])
def test_featuriser_conv(K, C, L):
    x = torch.randn(2, L, C, device=DEV, dtype=BF, requires_grad=True)
    w = torch.randn(C, K, device=DEV, requires_grad=True)
    h = torch.randn(2, K - 1, C, device=DEV, dtype=BF, requires_grad=True)
    _run(lambda a, c, d: ops.causal_conv1d(a, c, d), x, w, h)


@pytest.mark.parametrize("D,G,L", [(256, 16, 203), (96, 6, 130)])
def test_hyena_se(D, G, L):
    feat = torch.randn(2, L, 3 * D, device=DEV, dtype=BF, requires_grad=True)
    w = torch.randn(G, 7, device=DEV, requires_grad=True)
    _run(lambda a, c: ops.hyena_se_inner(a, c), feat, w)


@pytest.mark.parametrize("K,L", [(128, 333), (37, 70)])
def test_hyena_mr(K, L):
    D, G = 256, 16
    feat = torch.randn(2, L, 3 * D, device=DEV, dtype=BF, requires_grad=True)
    h = (torch.randn(G, K, device=DEV) / math.sqrt(K)).requires_grad_()
    bias = torch.randn(D, device=DEV, requires_grad=True)
    halo = torch.randn(2, K - 1, 3 * D, device=DEV, dtype=BF, requires_grad=True)
    _run(lambda a, c, d, e: ops.hyena_mr_inner(a, c, d, e), feat, h, bias, halo)


@pytest.mark.parametrize("L,D", [(300, 128), (1300, 160)])
def test_hyena_li(L, D):
    O = 16
    feat = (torch.randn(2, L, 3 * D, device=DEV) * 0.7).to(BF).requires_grad_()
    gamma = (torch.rand(D, O, device=DEV) * 0.09 + 0.01).log().requires_grad_()
    R = (0.1 * torch.randn(D, O, device=DEV) / 4).requires_grad_()
    p = (-torch.ones(D, O, device=DEV)).requires_grad_()
    bias = torch.randn(D, device=DEV, requires_grad=True)
    _run(lambda a, c, d, e, f: ops.hyena_li_modal(a, c, d, e, f), feat, gamma, R, p, bias)


def test_norm_gate_loss():
    x = torch.randn(3, 50, 264, device=DEV, dtype=BF, requires_grad=True)
    w = torch.ones(264, device=DEV, dtype=BF, requires_grad=True)
    _run(lambda a, c: ops.rmsnorm(a, c, 1e-6, "te"), x, w)
    ab = torch.randn(5, 33, 2 * 688, device=DEV, dtype=BF, requires_grad=True)
    _run(lambda a: ops.glu_act_packed(a, "silu"), ab)
    logits = torch.randn(3, 37, 512, device=DEV, dtype=BF, requires_grad=True)
    labels = torch.randint(0, 512, (3, 37), device=DEV)
    _run(lambda a: ops.cross_entropy(a, labels), logits)


@pytest.mark.parametrize("L", [384, 520])
def test_attention(L):
    q, k, v = (torch.randn(1, L, 2, 128, device=DEV, dtype=BF, requires_grad=True) for _ in range(3))
    _run(lambda a, c, d: ops.attention(a, c, d, causal=True), q, k, v)
