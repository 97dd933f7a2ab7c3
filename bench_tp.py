"""Fused tensor/sequence-parallel projection benchmark (roofline rows F1 / F2): all-gather->GEMM and
GEMM->reduce-scatter on the Evo-2-7B projection shapes, fused peer-memory kernels vs NCCL collective + GEMM.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench_tp.py [--seq 8192] [--iters 10]

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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    state.initialize_model_parallel(world, 1, 1)
    assert fused_tp.setup()
    peak = float((measured_peaks() or {}).get("bf16_tflops", 1590.0)) * 1e12
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    D, F, L = 4096, 11264, a.seq
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

    def report(name, ms, flops, nvbytes):
        roof = max(flops / peak, nvbytes / (NVLINK_GBS * 1e9)) * 1e3
        if rank == 0:
            print(json.dumps({"op": name, "tp": world, "ms": round(ms, 4), "roofline_ms": round(roof, 4),
                              "frac_of_roofline": round(roof / ms, 3), "tflops_per_gpu": round(flops / ms / 1e9, 1),
                              "nvlink_bytes_per_gpu": nvbytes}), flush=True)

    ws = fused_tp._WS
    for name, N, K in (("in_proj", 3 * D, D), ("mlp_w12", 2 * F, D)):
        x = torch.randn(1, l, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(N // world, K, device=dev) * 0.02).to(torch.bfloat16)
        fl = 2.0 * L * (N // world) * K
        nb = (world - 1) * l * K * 2
        with torch.no_grad():
            fused_tp._WS = ws
            report(f"F1.ag_gemm.{name}.fused", timed(lambda: ops.linear_allgather(x, w, None, 1)), fl, nb)
            fused_tp._WS = None
            report(f"F1.ag_gemm.{name}.nccl", timed(lambda: ops.linear_allgather(x, w, None, 1)), fl, nb)
    for name, N, K in (("out_proj", D, D), ("mlp_w3", D, F)):
        x = torch.randn(1, L, K // world, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, K // world, device=dev) * 0.02).to(torch.bfloat16)
        fl = 2.0 * L * N * (K // world)
        nb = (world - 1) * l * N * 2
        with torch.no_grad():
            fused_tp._WS = ws
            report(f"F2.gemm_rs.{name}.fused", timed(lambda: ops.linear_reducescatter(x, w, 1)), fl, nb)
            fused_tp._WS = None
            report(f"F2.gemm_rs.{name}.nccl", timed(lambda: ops.linear_reducescatter(x, w, 1)), fl, nb)
    fused_tp._WS = ws
    from savanna_b200.ops import cuda_ops
    cuda_ops.check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
