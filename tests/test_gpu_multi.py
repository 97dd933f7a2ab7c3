"""Multi-GPU tests (skipped with fewer than 2 GPUs): the fused peer-memory ZeRO-1 step against the NCCL
path, and a short data-parallel training run.  Ranks are child processes, one per GPU, NCCL with NVLS off
(a rank that exits while bound to a multicast object can fault its peers)."""
import os
import socket
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0
needs2 = pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, errq, args=()):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world),
                       "LOCAL_RANK": str(rank), "NCCL_NVLS_ENABLE": "0"})
    import torch.distributed as dist
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        fn(rank, world, *args)
        torch.cuda.synchronize()
        dist.barrier()
    except Exception:  # noqa: BLE001
        # Report, then stay alive and idle: this rank's memory stays mapped for peers whose kernels may still read it, and
        # tearing the process group down would wait for peers that are themselves waiting for this rank inside a
        # collective.  The parent ends all ranks together once it has the report.
        errq.put((rank, traceback.format_exc()))
        import time
        try:
            torch.cuda.synchronize()
        except Exception:  # noqa: BLE001
            pass
        time.sleep(3600)
    if dist.is_initialized():
        dist.destroy_process_group()


def _spawn_args(fn, world, *args):
    _spawn(fn, world, args)


def _spawn(fn, world, args=(), timeout=300.0):
    import time
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, errq, args)) for r in range(world)]
    for p in procs:
        p.start()
    deadline = time.time() + timeout
    failed = False
    while time.time() < deadline and any(p.is_alive() for p in procs):
        if not errq.empty() or any(p.exitcode not in (None, 0) for p in procs):
            failed = True                      # a rank failed: the others wait for it inside a collective
            time.sleep(4.0)                    # bounded device waits run out, in-flight kernels drain
            break
        time.sleep(0.2)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.terminate()
    for p in procs:
        p.join(10)
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    errs.sort()
    assert not errs, "\n".join(f"[rank {r}]\n{t}" for r, t in errs)
    assert not hung or failed, "worker hung"
    assert not failed and all(p.exitcode == 0 for p in procs), f"worker exit codes {[p.exitcode for p in procs]}"


def _w_fused_zero(rank, world, use_nvls=False):
    import torch.distributed as dist
    from savanna_b200.parallel import fused_zero, state
    from savanna_b200.parallel.zero import ZeroOptimizer
    state.initialize_model_parallel(1, 1, 1)
    dev = torch.device("cuda", rank)
    torch.manual_seed(0)
    shapes = [(512, 384), (1000, 77), (4096,), (333, 129)]

    def make(alloc):
        torch.manual_seed(1)
        ps = [torch.nn.Parameter(torch.randn(s, device=dev).to(torch.bfloat16)) for s in shapes]
        opt = ZeroOptimizer([{"params": ps, "weight_decay": 0.1}], lr=1e-2, betas=(0.9, 0.95), clip_grad=1.0,
                            group=state.get_sequence_data_parallel_group(),
                            group_ranks=state.get_sequence_data_parallel_ranks(), allocator=alloc)
        return ps, opt
    alloc = fused_zero.make_allocator(state.get_sequence_data_parallel_group())
    assert alloc is not None
    pa, oa = make(alloc)
    assert fused_zero.attach(oa, alloc, use_nvls=use_nvls), "fused path did not come up"
    if use_nvls and not oa.fused.nvls:
        print("no NVLink multicast mapping on this box: the multimem variant was not exercised", flush=True)
    pb, ob = make(None)
    for step in range(3):
        g = torch.Generator(device=dev).manual_seed(100 * step + rank)
        for a, b in zip(pa, pb):
            gr = torch.randn(a.shape, device=dev, generator=g).to(torch.bfloat16)
            a.grad.copy_(gr)
            b.grad.copy_(gr)
        na, nb = oa.step(), ob.step()
        torch.cuda.synchronize()
        assert abs(float(na) - float(nb)) <= 2e-3 * float(nb), (float(na), float(nb))
        for a, b in zip(pa, pb):
            # the NCCL path rounds the reduced gradient to bf16 before Adam, the fused one keeps fp32 partial sums
            # only inside the kernel and stores bf16 too: both see the same bf16 gradient except for summation order
            diff = (a.float() - b.float()).abs().max()
            assert diff <= 2e-2, f"step {step}: params differ by {diff}"
        # every rank holds the same parameters after the peer-store all-gather
        flat = oa.groups[0].flat_param.float()
        ref = flat.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(flat, ref)


@needs2
def test_fused_zero_matches_nccl():
    _spawn(_w_fused_zero, 2)


@needs2
def test_fused_zero_nvls_multimem_matches_nccl():
    """Same step with the NVLS kernels (multimem.ld_reduce reduce-scatter, multimem.st all-gather) where the symmetric
    buffers have a multicast mapping; falls back to plain peer access (and says so) where they do not."""
    _spawn_args(_w_fused_zero, 2, True)


def _w_dp_train(rank, world):
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.ops import cuda_ops
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_gpu.yml")],
                                 {"global_num_gpus": world, "zero_optimization": {"stage": 1}})
    tr = Trainer(cfg, load=False)
    assert tr.optimizer.fused is not None

    def it():
        i = 0
        while True:
            yield {"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=1000 * rank + i, pin=True)}
            i += 1
    d = it()
    losses = [float(tr.train_step(d)) for _ in range(8)]
    cuda_ops.check_status()
    assert losses[-1] < losses[0] - 0.5, losses


@needs2
def test_data_parallel_training_fused_zero():
    _spawn(_w_dp_train, 2)


def _w_zero_overlap(rank, world, checkpointing):
    """ZeRO-1 with the reduce-scatter launched from the last micro-batch's backward (side stream, device barrier per
    block boundary) against the same run with the whole reduce-scatter inside the optimizer step: identical loss traces
    and gradient norms (the same kernels reduce the same ranges; only the order of the squared-norm partials differs)."""
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.ops import cuda_ops
    from savanna_b200.parallel import state
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run(overlap):
        cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_gpu.yml")],
                                     {"global_num_gpus": world, "gradient_accumulation_steps": 2, "gradient_clipping": 0.3,
                                      "checkpoint_activations": checkpointing, "checkpoint_num_layers": 2,
                                      "use_nvls": False,
                                      "zero_optimization": {"stage": 1, "overlap_comm": overlap}})
        state.destroy_model_parallel()
        tr = Trainer(cfg, load=False)
        fused = tr.optimizer.fused
        assert fused is not None and (tr._zero_overlap is not None) == overlap

        def it():
            i = 0
            while True:
                yield {"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=1000 * rank + i, pin=True)}
                i += 1
        d = it()
        out = []
        for _ in range(5):
            loss = float(tr.train_step(d))
            out.append((loss, float(tr.grad_norm)))
        cuda_ops.check_status()
        launches = torch.tensor([float(fused.overlap_launches)], device="cuda")
        torch.distributed.all_reduce(launches)                 # a reported range may lie entirely in another rank's shard
        return out, (fused.overlap_rounds, int(launches.item()))

    base, n0 = run(False)
    over, n1 = run(True)
    assert n0 == (0, 0) and n1[0] > 0 and n1[1] > 0, (n0, n1)
    for (la, na), (lb, nb) in zip(base, over):
        assert abs(la - lb) < 1e-3 * max(1.0, abs(la)), (base, over)
        assert abs(na - nb) < 2e-3 * max(1.0, abs(na)), (base, over)


@needs2
@pytest.mark.parametrize("checkpointing", [False, True])
def test_zero_reduce_scatter_overlapped_with_backward(checkpointing):
    _spawn_args(_w_zero_overlap, 2, checkpointing)


def _w_fused_tp(rank, world):
    import torch.distributed as dist
    from savanna_b200 import ops
    from savanna_b200.ops import cuda_ops
    from savanna_b200.parallel import fused_tp, mappings, state
    state.initialize_model_parallel(world, 1, 1)
    dev = torch.device("cuda", rank)
    assert fused_tp.setup(), "fused tensor-parallel workspace did not come up"
    l, K, N = 512, 384, 640
    torch.manual_seed(7)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    wr = (torch.randn(K, N, device=dev) * 0.05).to(torch.bfloat16)          # row-parallel weight [out=K, in=N]
    bias = torch.randn(N, device=dev).to(torch.bfloat16)
    torch.manual_seed(100 + rank)
    x = torch.randn(1, l, K, device=dev).to(torch.bfloat16)
    g = torch.randn(1, l * world, N, device=dev).to(torch.bfloat16)

    def rel(a, b, tol, what):
        r = (a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-9)
        assert r <= tol, f"{what}: rel err {r.item():.4g}"

    for rep in range(3):                                                      # repeated calls exercise the double buffering
        # ---- all-gather -> GEMM
        xa, wa, ba = x.clone().requires_grad_(), w.clone().requires_grad_(), bias.clone().requires_grad_()
        ya = ops.linear_allgather(xa, wa, ba, 1)
        ya.backward(g)
        ws = fused_tp._WS
        fused_tp._WS = None                                                   # reference: NCCL all-gather + GEMM
        xb, wb, bb = x.clone().requires_grad_(), w.clone().requires_grad_(), bias.clone().requires_grad_()
        yb = ops.linear_allgather(xb, wb, bb, 1)
        yb.backward(g)
        fused_tp._WS = ws
        torch.cuda.synchronize()
        cuda_ops.check_status()
        rel(ya, yb, 1e-2, "ag-gemm fwd"); rel(xa.grad, xb.grad, 2e-2, "ag-gemm dx"); rel(wa.grad, wb.grad, 2e-2, "ag-gemm dw")
        rel(ba.grad, bb.grad, 2e-2, "ag-gemm dbias")
        # ---- GEMM -> reduce-scatter
        xin = torch.randn(1, l * world, N, device=dev, generator=torch.Generator(device=dev).manual_seed(5 + rank + rep)).to(torch.bfloat16)
        g2 = torch.randn(1, l, K, device=dev, generator=torch.Generator(device=dev).manual_seed(9 + rank)).to(torch.bfloat16)
        xa, wa = xin.clone().requires_grad_(), wr.clone().requires_grad_()
        ya = ops.linear_reducescatter(xa, wa, 1)
        ya.backward(g2)
        fused_tp._WS = None
        xb, wb = xin.clone().requires_grad_(), wr.clone().requires_grad_()
        yb = ops.linear_reducescatter(xb, wb, 1)
        yb.backward(g2)
        fused_tp._WS = ws
        torch.cuda.synchronize()
        cuda_ops.check_status()
        rel(ya, yb, 1e-2, "gemm-rs fwd"); rel(xa.grad, xb.grad, 2e-2, "gemm-rs dx"); rel(wa.grad, wb.grad, 2e-2, "gemm-rs dw")


@needs2
def test_fused_tp_matches_nccl():
    _spawn(_w_fused_tp, 2)


def _w_fused_tp_fp8_batched(rank, world):
    """Fused projections with fp8 operands and a micro-batch of two sequences in one launch, against (a) the NCCL
    collective + fp8 GEMM path and (b) the exact bf16 result, forward and all gradients."""
    from savanna_b200 import ops
    from savanna_b200.ops import cuda_ops
    from savanna_b200.parallel import fused_tp, state
    state.initialize_model_parallel(world, 1, 1)
    dev = torch.device("cuda", rank)
    assert fused_tp.setup(), "fused tensor-parallel workspace did not come up"
    cuda_ops.set_fp8_history(0)                                              # current scaling on both paths: comparable scales
    Bn, l, K, N = 2, 256, 384, 640
    torch.manual_seed(7)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    wr = (torch.randn(K, N, device=dev) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device=dev).to(torch.bfloat16)
    torch.manual_seed(100 + rank)
    x = torch.randn(Bn, l, K, device=dev).to(torch.bfloat16)
    g = torch.randn(Bn, l * world, N, device=dev).to(torch.bfloat16)
    xin = torch.randn(Bn, l * world, N, device=dev).to(torch.bfloat16)
    g2 = torch.randn(Bn, l, K, device=dev).to(torch.bfloat16)

    def rel(a, b, tol, what):
        r = (a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-9)
        assert r <= tol, f"{what}: rel err {r.item():.4g}"

    def run(fn, fp8, fused, *leaves):
        ws = fused_tp._WS
        if not fused:
            fused_tp._WS = None
        try:
            ls = [t.clone().requires_grad_() for t in leaves]
            y = fn(*ls, fp8)
            return y, ls
        finally:
            fused_tp._WS = ws

    for rep in range(2):
        outs = {}
        for name, fp8, fused in (("fused_fp8", True, True), ("nccl_fp8", True, False), ("fused_bf16", False, True), ("nccl_bf16", False, False)):
            y, ls = run(lambda a, b, c, f: ops.linear_allgather(a, b, c, 1, fp8=f), fp8, fused, x, w, bias)
            y.backward(g)
            outs[name] = (y, ls[0].grad, ls[1].grad, ls[2].grad)
        torch.cuda.synchronize(); cuda_ops.check_status()
        for i, what in enumerate(("fwd", "dx", "dw", "dbias")):
            rel(outs["fused_bf16"][i], outs["nccl_bf16"][i], 2e-2, f"batched bf16 ag-gemm {what}")
            rel(outs["fused_fp8"][i], outs["nccl_bf16"][i], 8e-2, f"fp8 ag-gemm {what} vs exact")
            rel(outs["fused_fp8"][i], outs["nccl_fp8"][i], 6e-2, f"fp8 ag-gemm {what} vs nccl fp8")
        outs = {}
        for name, fp8, fused in (("fused_fp8", True, True), ("nccl_fp8", True, False), ("fused_bf16", False, True), ("nccl_bf16", False, False)):
            y, ls = run(lambda a, b, f: ops.linear_reducescatter(a, b, 1, fp8=f), fp8, fused, xin, wr)
            y.backward(g2)
            outs[name] = (y, ls[0].grad, ls[1].grad)
        torch.cuda.synchronize(); cuda_ops.check_status()
        for i, what in enumerate(("fwd", "dx", "dw")):
            rel(outs["fused_bf16"][i], outs["nccl_bf16"][i], 2e-2, f"batched bf16 gemm-rs {what}")
            rel(outs["fused_fp8"][i], outs["nccl_bf16"][i], 8e-2, f"fp8 gemm-rs {what} vs exact")
            rel(outs["fused_fp8"][i], outs["nccl_fp8"][i], 6e-2, f"fp8 gemm-rs {what} vs nccl fp8")
    assert fused_tp.FP8_CALLS > 0 and fused_tp.fp8_active() is True


@needs2
def test_fused_tp_fp8_and_batched_matches_nccl():
    _spawn(_w_fused_tp_fp8_batched, 2)


def _w_tp_train(rank, world):
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.ops import cuda_ops
    from savanna_b200.parallel import fused_tp
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_gpu.yml")],
                                 {"global_num_gpus": world, "model_parallel_size": world, "sequence_parallel": True,
                                  "train_micro_batch_size_per_gpu": 1})
    tr = Trainer(cfg, load=False)
    assert fused_tp._WS is not None

    def it():
        i = 0
        while True:
            yield {"text": acgt_batch(1, cfg.seq_length, seed=i, pin=True)}
            i += 1
    d = it()
    before = cuda_ops.launch_count()
    losses = [float(tr.train_step(d)) for _ in range(8)]
    cuda_ops.check_status()
    assert losses[-1] < losses[0] - 0.5, losses
    assert cuda_ops.launch_count() > before


@needs2
def test_tensor_sequence_parallel_training_fused():
    _spawn(_w_tp_train, 2)


def _w_tp_train_mx(rank, world):
    """Block-scaled fp8 projections under tensor + sequence parallelism: NCCL all-gather / reduce-scatter around the
    MXFP8 GEMMs (the fused peer-memory projections take per-tensor scales only)."""
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.ops import cuda_ops
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_gpu.yml")],
                                 {"global_num_gpus": world, "model_parallel_size": world, "sequence_parallel": True,
                                  "train_micro_batch_size_per_gpu": 1, "use_fp8_linears": True, "fp8_recipe": "mxfp8",
                                  "use_fp8_input_projections": True, "use_fp8_output_projections": True,
                                  "use_fp8_mlp_projections": True})
    tr = Trainer(cfg, load=False)
    assert cuda_ops.FP8_RECIPE == "mxfp8"
    calls = []
    real = cuda_ops.gemm_mx
    cuda_ops.gemm_mx = lambda *a, **k: (calls.append(1), real(*a, **k))[1]

    def it():
        i = 0
        while True:
            yield {"text": acgt_batch(1, cfg.seq_length, seed=i, pin=True)}
            i += 1
    d = it()
    try:
        losses = [float(tr.train_step(d)) for _ in range(8)]
    finally:
        cuda_ops.gemm_mx = real
        cuda_ops.set_fp8_recipe("delayed")
    cuda_ops.check_status()
    assert calls, "no block-scaled GEMM ran"
    assert losses[-1] < losses[0] - 0.5, losses


@needs2
def test_tensor_sequence_parallel_training_block_scaled_fp8():
    _spawn(_w_tp_train_mx, 2)


# ------------------------------------------------------------------------------------------ context parallelism
# 128-wide heads so that the tcgen05 attention kernels and the peer-memory ring are the ones that run
_WIDE = {"hidden_size": 512, "num_attention_heads": 4, "num_groups_hyena": 512, "num_groups_hyena_medium": 32,
         "num_groups_hyena_short": 32, "hidden_dropout": 0.0}
_CP_OVER = dict(_WIDE, context_parallel_size=2, use_cp_hyena=True, use_cp_ring=True,
                operator_config=["hyena_se", "ring", "hyena_mr", "hyena", "ring"], num_layers=5)


def _cp_losses(world, over, n=4):
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = {"global_num_gpus": world, "train_micro_batch_size_per_gpu": 1}
    base.update(over)
    cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_gpu.yml")], base)
    tr = Trainer(cfg, load=False)

    def it():
        i = 0
        while True:
            yield {"text": acgt_batch(1, cfg.seq_length, seed=i, pin=True)}
            i += 1
    d = it()
    return [float(tr.train_step(d)) for _ in range(n)]


def _w_cp_train(rank, world, over, want):
    from savanna_b200.ops import cuda_ops
    from savanna_b200.parallel import halo
    got = _cp_losses(world, over, len(want))
    assert halo._PEER_WS is not None, "the peer-memory halo exchange was not brought up"
    from savanna_b200.parallel import ring_attention
    assert ring_attention._SIDE, "the peer-memory ring attention did not run"
    from savanna_b200.parallel import halo_fused
    assert halo_fused.CALLS > 0, "the convolutions did not read their halo rows from peer memory themselves"
    if over.get("cp_hyena_li_algo", "a2a") == "a2a":
        from savanna_b200.parallel import a2a
        assert a2a.PEER_CALLS > 0, "the peer-memory all-to-all did not run"
    cuda_ops.check_status()
    for a, b in zip(got, want):
        assert abs(a - b) < 2e-2 * max(1.0, abs(b)), (got, want)


def _cp_reference():
    from savanna_b200.parallel import state
    want = _cp_losses(1, dict(_WIDE, operator_config=["hyena_se", "flash_v2", "hyena_mr", "hyena", "flash_v2"], num_layers=5))
    state.destroy_model_parallel()
    return want


@needs2
def test_context_parallel_training_a2a_matches_single_gpu():
    """cp=2 (zigzag split, all-to-all Hyena, ring attention) reproduces the single-GPU loss trace in bf16."""
    want = _cp_reference()
    _spawn_args(_w_cp_train, 2, dict(_CP_OVER), want)


@needs2
def test_context_parallel_training_halo_state_matches_single_gpu():
    """cp=2 with the halo exchange (Hyena-SE/MR) and the modal-state hand-off (Hyena-LI)."""
    want = _cp_reference()
    over = dict(_CP_OVER, cp_hyena_mr_algo="p2p", cp_hyena_li_algo="state")
    _spawn_args(_w_cp_train, 2, over, want)


needs4 = pytest.mark.skipif(NGPU < 4, reason="needs 4 GPUs")


@needs4
@pytest.mark.parametrize("li_algo", ["a2a", "state"])
def test_context_parallel_training_cp4_matches_single_gpu(li_algo):
    """cp=4: distinct previous / next neighbours in the halo exchange, two staging buffers with the side-stream prefetch
    in the ring attention, four-way pulls in the all-to-all and the per-owner dK/dV reduction."""
    want = _cp_reference()
    over = dict(_CP_OVER, context_parallel_size=4)
    if li_algo == "state":
        over.update(cp_hyena_mr_algo="p2p", cp_hyena_li_algo="state")
    _spawn_args(_w_cp_train, 4, over, want)
