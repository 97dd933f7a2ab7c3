"""Fused tensor/sequence-parallel projection benchmark (roofline rows F1 / F2): all-gather->GEMM and
GEMM->reduce-scatter on the Evo-2-7B projection shapes, fused peer-memory kernels vs NCCL collective + GEMM.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench_tp.py [--seq 8192] [--iters 10]
    python bench_tp.py --emulate-world 2        # one GPU, all rank slots in local memory: for ncu captures

Per measurement: CUDA events on each rank, 3 warm-ups, L2 flush between launches, MAX over ranks.  Roofline time =
max(FLOPs / measured cuBLAS burst peak, bytes that must cross NVLink per GPU / 770 GB/s); one JSON line each.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from savanna_b200 import ops  # noqa: E402
from savanna_b200.parallel import fused_tp, state  # noqa: E402
from savanna_b200.utils.mfu import measured_peaks  # noqa: E402

NVLINK_GBS = 770.0


def emulate(a):
    """One GPU, one process: the fused kernels run with `--emulate-world` rank slots whose buffers all live in this
    GPU's memory (the peer pointers point at local buffers), as ONE launch per measurement.  NVLink is not exercised; the
    run exists so that the kernels can be captured by ncu (tensor-pipe activity of the GEMM CTAs beside the copy CTAs,
    DRAM throughput of the ZeRO kernels) and gives the kernel-side upper bound of the multi-GPU numbers."""
    import ctypes
    from savanna_b200.ops import cuda_ops
    lib = cuda_ops.require()
    P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.sb_gemm_tp.restype = I
    lib.sb_gemm_tp.argtypes = [P, I, P, I, I, P, I, P, I, I, I, I, I, P, P, I, I, I, I, P, P, P, I, I, I, I, P, P, P]
    lib.sb_zero_reduce_scatter.restype = I
    lib.sb_zero_reduce_scatter.argtypes = [P, I, I, LL, LL, P, P, P, P]
    lib.sb_zero_adam_allgather.restype = I
    lib.sb_zero_adam_allgather.argtypes = [P, P, P, P, P, P, I, I, LL, LL, F, F, F, F, F, F, F, I, P, P]
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    world, D, F_, L = a.emulate_world, 4096, 11264, a.seq
    l = L // world
    peak = float((measured_peaks() or {}).get("bf16_tflops", 1590.0)) * 1e12
    hbm = float((measured_peaks() or {}).get("hbm_gbs", 6650.0)) * 1e9
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    st = lambda: torch.cuda.current_stream().cuda_stream
    status = cuda_ops.status_word(dev)
    flags = torch.zeros(8192, dtype=torch.int32, device=dev)
    epoch = [0]

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]

    for name, N, K in (() if a.only_zero else (("in_proj", 3 * D, D), ("mlp_w12", 2 * F_, D))):
        shards = [torch.randn(l, K, device=dev).to(torch.bfloat16) for _ in range(world)]
        w = (torch.randn(N // world, K, device=dev) * 0.02).to(torch.bfloat16)
        gather = torch.empty(L * K, dtype=torch.bfloat16, device=dev)
        out = torch.empty(L, N // world, dtype=torch.bfloat16, device=dev)
        ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in shards])

        def run():
            epoch[0] += 1
            rc = lib.sb_gemm_tp(shards[0].data_ptr(), K, w.data_ptr(), K, 0, out.data_ptr(), N // world, None, L, N // world, K,
                                1, 2, None, None, 0, 0,
                                world, 0, ptrs, gather.data_ptr(), flags.data_ptr(), epoch[0], 16, 0, 0, None,
                                status.data_ptr(), st())
            assert rc == 0, rc
        ms = timed(run)
        cuda_ops.check_status()
        want = torch.cat(shards).float() @ w.float().t()
        err = ((out.float() - want).norm() / want.norm()).item()
        fl = 2.0 * L * (N // world) * K
        print(json.dumps({"op": f"F1.ag_gemm.{name}.emulated_1gpu", "slots": world, "ms": round(ms, 4),
                          "tflops": round(fl / ms / 1e9, 1), "frac_of_gemm_peak": round(fl / (ms / 1e3) / peak, 3),
                          "rel_err": round(err, 5)}), flush=True)
    for name, N, K in (() if a.only_zero else (("in_proj", 3 * D, D), ("mlp_w12", 2 * F_, D))):
        # the same projection on one-byte e4m3 operands (unit scales: the timing does not depend on them)
        shards = [torch.randint(0, 120, (l, K), device=dev, dtype=torch.uint8) for _ in range(world)]
        w = torch.randint(0, 120, (N // world, K), device=dev, dtype=torch.uint8)
        gather = torch.empty(L * K, dtype=torch.uint8, device=dev)
        out = torch.empty(L, N // world, dtype=torch.bfloat16, device=dev)
        ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in shards])
        one = torch.ones(1, device=dev)

        def run():
            epoch[0] += 1
            rc = lib.sb_gemm_tp(shards[0].data_ptr(), K, w.data_ptr(), K, 0, out.data_ptr(), N // world, None, L, N // world, K,
                                1, 1, one.data_ptr(), one.data_ptr(), 0, 0,
                                world, 0, ptrs, gather.data_ptr(), flags.data_ptr(), epoch[0], 16, 0, 0, None,
                                status.data_ptr(), st())
            assert rc == 0, rc
        ms = timed(run)
        cuda_ops.check_status()
        fl = 2.0 * L * (N // world) * K
        print(json.dumps({"op": f"F1.ag_gemm.{name}.fp8.emulated_1gpu", "slots": world, "ms": round(ms, 4),
                          "tflops": round(fl / ms / 1e9, 1), "frac_of_bf16_gemm_peak": round(fl / (ms / 1e3) / peak, 3)}), flush=True)
    for name, N, K in (() if a.only_zero else (("out_proj", D, D), ("mlp_w3", D, F_))):
        x = torch.randn(L, K // world, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, K // world, device=dev) * 0.02).to(torch.bfloat16)
        stages = [torch.empty(world * l * N, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        sp = (ctypes.c_void_p * world)(*[t.data_ptr() for t in stages])

        def run():
            rc = lib.sb_gemm_tp(x.data_ptr(), K // world, w.data_ptr(), K // world, 0, None, 0, None, L, N, K // world,
                                1, 2, None, None, 0, 0,
                                0, 0, None, None, flags.data_ptr(), 0, 16, world, 0, sp, status.data_ptr(), st())
            assert rc == 0, rc
        ms = timed(run)
        cuda_ops.check_status()
        fl = 2.0 * L * N * (K // world)
        print(json.dumps({"op": f"F2.gemm_rs.{name}.emulated_1gpu", "slots": world, "ms": round(ms, 4),
                          "tflops": round(fl / ms / 1e9, 1), "frac_of_gemm_peak": round(fl / (ms / 1e3) / peak, 3)}), flush=True)
    # ZeRO-1 step kernels on a flat group (512M elements by default): every slot's gradient / parameter buffer is local
    n = (a.zero_elems // (8 * world)) * 8 * world
    shard = n // world
    grads = [torch.randn(n, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    params = [torch.empty(n, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    gp = (ctypes.c_void_p * world)(*[t.data_ptr() for t in grads])
    pp = (ctypes.c_void_p * world)(*[t.data_ptr() for t in params])
    red = torch.empty(shard, device=dev, dtype=torch.bfloat16)
    sq = torch.zeros((), device=dev)
    master, m1, m2 = (torch.zeros(shard, device=dev) for _ in range(3))
    coef = torch.ones(1, device=dev)

    def rs():
        assert lib.sb_zero_reduce_scatter(gp, world, 0, 0, shard, red.data_ptr(), None, sq.data_ptr(), st()) == 0

    def adam():
        assert lib.sb_zero_adam_allgather(master.data_ptr(), m1.data_ptr(), m2.data_ptr(), red.data_ptr(), pp, None, world, 0,
                                          0, shard, 1e-3, 0.9, 0.95, 1e-8, 0.0, 0.1, 0.05, 1, coef.data_ptr(), st()) == 0
    ms = timed(rs)
    by = shard * 2 * (world + 1)
    print(json.dumps({"op": "F6.zero_reduce_scatter.emulated_1gpu", "slots": world, "ms": round(ms, 4),
                      "gbs": round(by / ms / 1e6, 1), "frac_of_copy_bw": round(by / (ms / 1e3) / hbm, 3)}), flush=True)
    ms = timed(adam)
    by = shard * (2 + 24 + 2 * world)
    print(json.dumps({"op": "F7.zero_adam_allgather.emulated_1gpu", "slots": world, "ms": round(ms, 4),
                      "gbs": round(by / ms / 1e6, 1), "frac_of_copy_bw": round(by / (ms / 1e3) / hbm, 3)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--batch", type=int, default=1, help="sequences per launch (micro-batch)")
    ap.add_argument("--hidden", type=int, default=4096, help="model width (8192 with --ffn 21888 = the 40B shapes)")
    ap.add_argument("--ffn", type=int, default=11264)
    ap.add_argument("--zero-elems", type=int, default=512 * 1024 * 1024,
                    help="elements of the flat group of the emulated ZeRO kernels (smaller for profiler captures)")
    ap.add_argument("--only-zero", action="store_true", help="emulation: run the ZeRO kernels only")
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="single-GPU emulation with this many rank slots in local memory (for ncu captures)")
    a = ap.parse_args()
    if a.emulate_world > 1:
        return emulate(a)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    state.initialize_model_parallel(world, 1, 1)
    assert fused_tp.setup()
    peak = float((measured_peaks() or {}).get("bf16_tflops", 1590.0)) * 1e12
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    D, F, L = a.hidden, a.ffn, a.seq
    l = L // world

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def report(name, ms, flops, nvbytes, fp8=False):
        # compute roofline: the measured cuBLAS bf16 burst peak; for one-byte operands twice that (the hardware ratio)
        roof = max(flops / (peak * (2.0 if fp8 else 1.0)), nvbytes / (NVLINK_GBS * 1e9)) * 1e3
        if rank == 0:
            print(json.dumps({"op": name, "tp": world, "ms": round(ms, 4), "roofline_ms": round(roof, 4),
                              "frac_of_roofline": round(roof / ms, 3), "tflops_per_gpu": round(flops / ms / 1e9, 1),
                              "nvlink_bytes_per_gpu": nvbytes}), flush=True)

    ws = fused_tp._WS
    Bn = a.batch
    for name, N, K in (("in_proj", 3 * D, D), ("mlp_w12", 2 * F, D)):
        x = torch.randn(Bn, l, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(N // world, K, device=dev) * 0.02).to(torch.bfloat16)
        fl = 2.0 * Bn * L * (N // world) * K
        for fp8 in (False, True):
            nb = (world - 1) * Bn * l * K * (1 if fp8 else 2)
            tag = ".fp8" if fp8 else ""
            with torch.no_grad():
                fused_tp._WS = ws
                report(f"F1.ag_gemm.{name}{tag}.fused", timed(lambda: ops.linear_allgather(x, w, None, 1, fp8=fp8)), fl, nb, fp8)
                fused_tp._WS = None
                nbn = (world - 1) * Bn * l * K * 2                     # the NCCL path gathers bf16
                report(f"F1.ag_gemm.{name}{tag}.nccl", timed(lambda: ops.linear_allgather(x, w, None, 1, fp8=fp8)), fl, nbn, fp8)
    for name, N, K in (("out_proj", D, D), ("mlp_w3", D, F)):
        x = torch.randn(Bn, L, K // world, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, K // world, device=dev) * 0.02).to(torch.bfloat16)
        fl = 2.0 * Bn * L * N * (K // world)
        nb = (world - 1) * Bn * l * N * 2
        for fp8 in (False, True):
            tag = ".fp8" if fp8 else ""
            with torch.no_grad():
                fused_tp._WS = ws
                report(f"F2.gemm_rs.{name}{tag}.fused", timed(lambda: ops.linear_reducescatter(x, w, 1, fp8=fp8)), fl, nb, fp8)
                fused_tp._WS = None
                report(f"F2.gemm_rs.{name}{tag}.nccl", timed(lambda: ops.linear_reducescatter(x, w, 1, fp8=fp8)), fl, nb, fp8)
    fused_tp._WS = ws
    from savanna_b200.ops import cuda_ops
    cuda_ops.check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
