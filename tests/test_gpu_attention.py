"""tcgen05 flash attention (csrc/attn_sm100.cu) against the fp32 PyTorch statement of the op: forward, log-sum-exp and
all three gradients; causal and full; lengths that are not multiples of the tile sizes; q/k/v as strided slices of one
fused projection output; a gradient arriving at the log-sum-exp output (the ring-attention merge)."""
import pytest
import torch

from savanna_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _rel(a, b, tol, what):
    a, b = a.float(), b.float()
    err = (a - b).norm() / b.norm().clamp_min(1e-12)
    assert err < tol, f"{what}: relative error {err.item():.3e} (tolerance {tol})"


def _status_ok():
    from savanna_b200.ops import cuda_ops
    cuda_ops.check_status()


def _case(B, Lq, Lk, H, causal, fused_qkv=False, lse_grad=False, seed=0):
    from savanna_b200.ops import flash_sm100
    torch.manual_seed(seed)
    if fused_qkv:
        assert Lq == Lk
        qkv = torch.randn(B, Lq, 3, H, 128, device=DEV, dtype=BF, requires_grad=True)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    else:
        q = torch.randn(B, Lq, H, 128, device=DEV, dtype=BF, requires_grad=True)
        k = torch.randn(B, Lk, H, 128, device=DEV, dtype=BF, requires_grad=True)
        v = torch.randn(B, Lk, H, 128, device=DEV, dtype=BF, requires_grad=True)
    assert flash_sm100.supported(q, k, v, causal)
    o, lse = flash_sm100.attention(q, k, v, causal, return_lse=True)
    go = torch.randn_like(o)
    gl = torch.randn_like(lse) if lse_grad else None
    loss = (o.float() * go.float()).sum() + ((lse * gl).sum() if lse_grad else 0.0)
    leaves = (qkv,) if fused_qkv else (q, k, v)
    grads = torch.autograd.grad(loss, leaves)
    _status_ok()

    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf, lser = ref.attention(qr, kr, vr, causal, return_lse=True)
    lossr = (orf * go.float()).sum() + ((lser * gl).sum() if lse_grad else 0.0)
    gr = torch.autograd.grad(lossr, (qr, kr, vr))
    _rel(o, orf, 1e-2, "out")
    assert (lse - lser).abs().max() < 2e-2, (lse - lser).abs().max()
    if fused_qkv:
        got = (grads[0][:, :, 0], grads[0][:, :, 1], grads[0][:, :, 2])
    else:
        got = grads
    for name, a, b in zip(("dq", "dk", "dv"), got, gr):
        _rel(a, b, 2e-2, name)


@pytest.mark.parametrize("L", [256, 1024, 333])
def test_flash_causal(L):
    _case(2, L, L, 3, True, seed=L)


@pytest.mark.parametrize("Lq,Lk", [(256, 256), (192, 448), (100, 130)])
def test_flash_full(Lq, Lk):
    _case(1, Lq, Lk, 2, False, seed=Lq + Lk)


def test_flash_backward_variant_shared_memory_p():
    """The backward variant that passes P^T through shared memory (two Q/dO stages) gives the same gradients."""
    from savanna_b200.ops import flash_sm100
    flash_sm100.set_backward_variant(False)
    try:
        _case(1, 640, 640, 2, True, seed=21)
        _case(1, 200, 328, 2, False, seed=22)
    finally:
        flash_sm100.set_backward_variant(True)


@pytest.mark.parametrize("pingpong", [False, True])
@pytest.mark.parametrize("Lq,Lk,causal", [(1024, 1024, True), (333, 333, True), (128, 128, True), (640, 896, False),
                                           (130, 130, True)])
def test_flash_forward_variants(pingpong, Lq, Lk, causal):
    """Both forward schedules (softmax warpgroups taking turns on the exponentials, or free running) on shapes where
    the two query tiles of a CTA see equal and unequal numbers of key blocks, and where the second tile is empty."""
    from savanna_b200.ops import flash_sm100
    flash_sm100.set_forward_variant(pingpong)
    try:
        _case(2, Lq, Lk, 2, causal, seed=5)
    finally:
        flash_sm100.set_forward_variant(False)


def test_flash_fused_qkv_strides():
    _case(2, 512, 512, 4, True, fused_qkv=True, seed=7)


def test_flash_lse_gradient():
    _case(1, 384, 384, 2, True, lse_grad=True, seed=8)
    _case(1, 128, 256, 2, False, lse_grad=True, seed=9)


@pytest.mark.parametrize("rotary_dim", [None, 128, 64])
@pytest.mark.parametrize("L", [256, 333])
def test_packed_projection_attention(L, rotary_dim):
    """The one-function form on the packed projection [B, L, H, 3*128] (rotary embedding inside, gradients written
    straight into one packed buffer) against slicing, rotating and attending in fp32."""
    from savanna_b200 import ops
    torch.manual_seed(21)
    B, H = 2, 2
    qkv = torch.randn(B, L, H, 384, device=DEV, dtype=BF, requires_grad=True)
    cos = sin = None
    if rotary_dim:
        cos, sin = ref.rope_tables(torch.arange(L, device=DEV), rotary_dim)
    o = ops.attention_packed(qkv, cos, sin, True)
    assert o is not None
    go = torch.randn_like(o)
    (g,) = torch.autograd.grad((o.float() * go.float()).sum(), (qkv,))
    _status_ok()
    qr = qkv.detach().float().requires_grad_()
    q, k, v = qr[..., :128], qr[..., 128:256], qr[..., 256:]
    if rotary_dim:
        q, k = ref.apply_rope(q, cos, sin), ref.apply_rope(k, cos, sin)
    orf = ref.attention(q, k, v, True)
    (gr,) = torch.autograd.grad((orf * go.float()).sum(), (qr,))
    _rel(o, orf, 1e-2, "out")
    for name, sl in (("dq", slice(0, 128)), ("dk", slice(128, 256)), ("dv", slice(256, 384))):
        _rel(g[..., sl], gr[..., sl], 2e-2, name)


@pytest.mark.parametrize("shape", [(1, 256, 256, 2, True), (2, 1024, 1024, 2, True), (1, 333, 333, 2, True),
                                   (1, 384, 640, 2, False), (1, 2048, 2048, 4, True)])
def test_flash_forward_with_probabilities_through_shared_memory(shape):
    """The forward variant that stages P in shared memory (the default feeds it to the P V product from tensor memory):
    same cases, same tolerances."""
    from savanna_b200.ops import flash_sm100
    B, Lq, Lk, H, causal = shape
    flash_sm100.set_forward_p_in_tmem(False)
    try:
        _case(B, Lq, Lk, H, causal, seed=31)
    finally:
        flash_sm100.set_forward_p_in_tmem(True)


def test_flash_long_sequence_statistics():
    """Scores with a large spread exercise the lazy rescaling of the output accumulator."""
    from savanna_b200.ops import flash_sm100
    torch.manual_seed(11)
    B, L, H = 1, 2048, 2
    q = (torch.randn(B, L, H, 128, device=DEV) * 3).to(BF)
    k = (torch.randn(B, L, H, 128, device=DEV) * 3).to(BF)
    v = torch.randn(B, L, H, 128, device=DEV, dtype=BF)
    o, lse = flash_sm100.attention(q, k, v, True, return_lse=True)
    _status_ok()
    orf, lser = ref.attention(q.float(), k.float(), v.float(), True, return_lse=True)
    _rel(o, orf, 1.5e-2, "out")
    assert (lse - lser).abs().max() < 5e-2


def test_model_training_own_attention_tracks_library_attention():
    """A small StripedHyena with 128-wide heads: the loss trace with the tcgen05 attention kernels stays on the trace
    obtained with the library flash kernels (same seeds, same data)."""
    import os
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.ops import attention_cuda, cuda_ops
    from savanna_b200.parallel import state
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    traces = []
    try:
        for own in (False, True):
            attention_cuda.set_own_kernels(own)
            cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_gpu.yml")],
                                         {"global_num_gpus": 1, "hidden_size": 512, "num_attention_heads": 4,
                                          "num_groups_hyena": 512, "num_groups_hyena_medium": 32,
                                          "num_groups_hyena_short": 32,
                                          "operator_config": ["hyena_se", "flash_v2", "hyena_mr", "flash_v2"]})
            tr = Trainer(cfg, load=False)
            before = cuda_ops.launch_count()
            batches = iter([{"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i).cuda()}
                            for i in range(12)])
            traces.append([float(tr.train_step(batches)) for _ in range(12)])
            cuda_ops.check_status()
            assert cuda_ops.launch_count() > before
            state.destroy_model_parallel()
    finally:
        attention_cuda.set_own_kernels(True)
    a, b = traces
    assert max(abs(x - y) for x, y in zip(a, b)) < 0.05, (a, b)


def test_merge_partials_matches_pairwise_merge():
    """Fused merge of partial attention results (and its backward) against the pairwise log-sum-exp merge in PyTorch,
    with partials that are strided slices of larger tensors."""
    from savanna_b200.ops import flash_sm100
    from savanna_b200.parallel.ring_attention import _merge
    torch.manual_seed(70)
    B, L, H, S = 2, 96, 3, 5
    big_o = [torch.randn(B, 2 * L, H, 128, device=DEV, dtype=BF, requires_grad=True) for _ in range(S)]
    big_l = [(torch.randn(B, H, 2 * L, device=DEV) * 3).requires_grad_() for _ in range(S)]
    os_ = [t[:, L:] if i % 2 else t[:, :L] for i, t in enumerate(big_o)]
    ls_ = [t[..., L:] if i % 2 else t[..., :L] for i, t in enumerate(big_l)]
    assert flash_sm100.merge_supported(os_, ls_)
    out, lse = flash_sm100.merge_partials(os_, ls_)
    g = torch.randn_like(out)
    grads = torch.autograd.grad((out.float() * g.float()).sum(), big_o + big_l)
    ro = [t.detach().float().requires_grad_() for t in big_o]
    rl = [t.detach().clone().requires_grad_() for t in big_l]
    oa = la = None
    for i in range(S):
        o_i = ro[i][:, L:] if i % 2 else ro[i][:, :L]
        l_i = rl[i][..., L:] if i % 2 else rl[i][..., :L]
        oa, la = _merge(oa, la, o_i, l_i)
    rgrads = torch.autograd.grad((oa * g.float()).sum(), ro + rl)
    _rel(out, oa, 1e-2, "merged output")
    assert (lse - la).abs().max() < 1e-4
    for i, (a, b) in enumerate(zip(grads, rgrads)):
        _rel(a, b, 2e-2, f"merge grad {i}")
