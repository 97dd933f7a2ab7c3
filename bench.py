"""Headline benchmark: training tokens/s of the Evo-2-7B-style StripedHyena 2 at sequence length 8192,
ZeRO-1 data parallel, bf16 (BASELINE.json config 3: 32 layers, hidden 4096, 32 heads, byte vocab 512,
SwiGLU inner 11264, attention at layers 3/10/17/24/31, SE/MR/LI elsewhere; global batch 64 sequences on
8 GPUs).  Weak scaling: every GPU processes 8 sequences of 8192 tokens per optimizer step (micro-batch 1,
8 accumulation steps), so the global batch is 8 * N sequences.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched with torch.distributed.run)
    python bench.py --impl reference ...                   (the unmodified reference, when installable)

Two timed regions, each bracketed by barrier + synchronize:
  * device-timed (`value`): K optimizer steps on batches already resident on the GPU, CUDA events, max over ranks;
  * end to end (`e2e`): K calls of the public `Trainer.train_step` whose iterator yields pinned host batches
    (host->device copy inside the step) followed by a device->host read of the loss.
Synthetic data: uniform random bytes of A, C, G, T; weights: random init of the named architecture.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--config", type=str, default=os.path.join(ROOT, "configs", "baseline", "evo2_7b_8k.yml"))
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (result is then not the named config)")
    ap.add_argument("--accum", type=int, default=None, help="debug only: accumulation steps per optimizer step")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--bf16-only", action="store_true", help="measure only the all-bf16 recipe (no fp8 projection GEMMs)")
    ap.add_argument("--skip-second", action="store_true", help="do not also measure the all-bf16 recipe")
    ap.add_argument("--comm", type=str, default=None, choices=["symm", "nccl"], help="ZeRO collective path (default: config)")
    ap.add_argument("--override", action="append", default=[], metavar="KEY=VALUE",
                    help="debug only: override a config key (YAML value); the result is then not the named config")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML queries from a thread of this process
    (three cheap reads every 250 ms).  An `nvidia-smi -lms 200` child, the first implementation, cost 6-10 % of the step
    time it was meant to observe; it remains only as the fallback when the NVML binding is missing, at 1 s intervals."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.samples = []           # (sm_mhz, reasons bitmask) from NVML
        self.max_mhz = None
        self.handle = None
        self.stop_flag = threading.Event()
        self.thread = None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            import torch
            pr = torch.cuda.get_device_properties(self.gpu)
            bus = "%08X:%02X:%02X.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
            return pynvml, pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu)

    def _poll(self):
        nv, h = self.nv, self.handle
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop_flag.is_set():
            try:
                self.samples.append((float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), int(reasons_fn(h))))
            except Exception:
                pass
            self.stop_flag.wait(0.25)

    def start(self):
        try:
            self.nv, self.handle = self._nvml_handle()
            self.max_mhz = float(self.nv.nvmlDeviceGetMaxClockInfo(self.handle, self.nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.handle = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "1000", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.handle is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            sm = [s for s, _ in self.samples]
            bits = 0
            for _, r in self.samples:
                bits |= r
            reasons = sorted(n for n, b in self.REASON_BITS.items() if bits & b)
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz, "reasons": reasons,
                    "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


def reference_arm(args):
    """The reference needs DeepSpeed (engine, pipeline module, activation checkpointing), TransformerEngine
    (imported unconditionally by its norm layer) and lazy_import_plus; none is installed or present in the
    offline wheelhouse, so `import savanna` fails and its training entry point cannot run."""
    why = None
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import savanna  # noqa: F401
        import deepspeed  # noqa: F401
        import transformer_engine  # noqa: F401
    except Exception as exc:  # noqa: BLE001
        why = f"reference not runnable offline: {type(exc).__name__}: {exc}".replace("\n", " ")[:300]
    if why is None:
        why = "reference imports resolved but no driver for its DeepSpeed launcher is wired on this box"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    if args.impl == "torch":
        os.environ["SAVANNA_B200_BACKEND"] = "torch"
    import torch
    import torch.distributed as dist
    from savanna_b200 import ops
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import ACGT
    from savanna_b200.train.trainer import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}; using WORLD_SIZE", file=sys.stderr)
    over = {"global_num_gpus": world}
    if args.layers:
        over["num_layers"] = args.layers
    if args.accum:
        over["gradient_accumulation_steps"] = args.accum
    if args.comm:
        over["comm_path"] = args.comm
    for kv in args.override:
        import yaml
        k, _, v = kv.partition("=")
        over[k.replace("-", "_")] = yaml.safe_load(v)
    if args.layers:
        import yaml
        doc = yaml.load(open(args.config), Loader=yaml.FullLoader)
        from savanna_b200.config import expand_operator_types
        full = expand_operator_types(doc["operator-config"], doc["num_layers"])
        over["operator_config"] = full[: args.layers]
    fp8_over = {"use_fp8_linears": True, "use_fp8_input_projections": True, "use_fp8_output_projections": True,
                "use_fp8_mlp_projections": True}
    acgt = torch.from_numpy(ACGT)

    def measure(extra_over, with_e2e):
        """Build the trainer for one precision recipe and time it; returns a dict of results."""
        o = dict(over)
        o.update(extra_over)
        cfg = GlobalConfig.from_ymls([args.config], o)
        trainer = Trainer(cfg, load=False)
        dev = trainer.device
        B, L, gas = cfg.train_micro_batch_size_per_gpu, cfg.seq_length, cfg.gradient_accumulation_steps
        tokens_per_step = cfg.train_batch_size * L
        gen = torch.Generator().manual_seed(1234 + rank)

        def host_batch():
            t = acgt[torch.randint(0, 4, (B, L + 1), generator=gen)]
            return t.pin_memory() if dev.type == "cuda" else t

        def device_iter(n):
            batches = [host_batch().to(dev) for _ in range(n)]
            def it():
                i = 0
                while True:
                    yield {"text": batches[i % n]}
                    i += 1
            return it()

        def host_iter():
            while True:
                yield {"text": host_batch()}

        def sync():
            if dist.is_initialized():
                dist.barrier()
            if dev.type == "cuda":
                torch.cuda.synchronize()

        own = args.impl == "ours" and dev.type == "cuda"
        dit = device_iter(gas * 2)
        for _ in range(args.warmup):
            loss = trainer.train_step(dit)
        sync()
        if own:
            from savanna_b200.ops import cuda_ops
            cuda_ops.check_status()
        sampler = ClockSampler(local)
        launches0 = ops.kernel_launch_count() if own else 0
        sampler.start()
        sync()
        if dev.type == "cuda":
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            loss = trainer.train_step(dit)
        if dev.type == "cuda":
            e1.record()
        sync()
        wall = time.perf_counter() - t0
        ms = e0.elapsed_time(e1) if dev.type == "cuda" else wall * 1e3
        clocks = sampler.stop()
        launches = (ops.kernel_launch_count() - launches0) if own else 0
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if dist.is_initialized():
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step = float(t.item()) / args.steps
        from savanna_b200.parallel import state as pstate
        par = "".join(f"{n}{v} " for n, v in (("pp", pstate.get_pipe_parallel_world_size()),
                                               ("tp", pstate.get_model_parallel_world_size()),
                                               ("cp", pstate.get_context_parallel_world_size())) if v > 1)
        par += f"dp{pstate.get_data_parallel_world_size()} zero{cfg.zero_stage}" + (" sp" if cfg.sequence_parallel else "")
        res = {"value": tokens_per_step / (ms_per_step / 1e3), "ms_per_step": ms_per_step, "loss": float(loss),
               "parallelism": par,
               "clocks": clocks, "gpu_launches": launches, "cfg": cfg, "e2e": None,
               "zero_path": (("fused peer-memory kernels" + (" (NVLS multimem)" if getattr(trainer.optimizer.fused, "nvls", False) else ""))
                             if getattr(trainer.optimizer, "fused", None) is not None
                             else ("nccl" if world > 1 else "single rank"))}
        if with_e2e:
            hit = host_iter()
            sync()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                loss = trainer.train_step(hit)
                _ = float(loss)                     # device -> host read of the step's result
            sync()
            dt = time.perf_counter() - t0
            tt = torch.tensor([dt], dtype=torch.float64, device=dev)
            if dist.is_initialized():
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            res["e2e"] = {"value": tokens_per_step / (float(tt.item()) / args.steps), "unit": "tokens/s",
                          "h2d_bytes_per_step": gas * B * (L + 1) * 8, "d2h_bytes_per_step": 4}
        if own:
            cuda_ops.check_status()
        # release this recipe's model before the next one is built
        del trainer, dit
        import gc
        gc.collect()
        if dev.type == "cuda":
            torch.cuda.empty_cache()
        return res

    # Headline recipe = the named configuration: bf16 with fp8 projection GEMMs (what the reference's Evo 2 7B configs
    # enable through use_fp8_linears).  The all-bf16 recipe is measured in the same run and reported beside it.
    use_fp8 = not args.bf16_only and args.impl == "ours" and torch.cuda.is_available()
    main_res = measure(fp8_over if use_fp8 else {}, not args.no_e2e)
    other = measure({}, False) if (use_fp8 and not args.skip_second) else None
    cfg = main_res["cfg"]
    L, B, gas = cfg.seq_length, cfg.train_micro_batch_size_per_gpu, cfg.gradient_accumulation_steps
    value, ms_per_step, final_loss = main_res["value"], main_res["ms_per_step"], main_res["loss"]
    clocks, launches, e2e = main_res["clocks"], main_res["gpu_launches"], main_res["e2e"]
    zero_path = main_res["zero_path"]
    from savanna_b200.utils.mfu import model_flops_per_token, peak_flops
    fpt = model_flops_per_token(cfg)
    peak = peak_flops(cfg)
    mfu = value * fpt / (world * peak) if peak else None
    if rank == 0:
        out = {
            "metric": "train tokens/sec (Evo2-7B-style StripedHyena 2 @8K, ZeRO-1 DP)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 + fp8 (e4m3/e5m2, per-tensor scaling) projection GEMMs" if use_fp8 else "bf16",
            "data": "synthetic uniform ACGT bytes; random-init weights", "impl": args.impl,
            "config": {"model": (f"{cfg.num_layers}L D{cfg.hidden_size} {cfg.num_attention_heads} heads ffn {cfg.ffn_size} vocab {cfg.padded_vocab_size} ({os.path.basename(args.config)})") if not args.layers
                       else f"DEBUG {args.layers}-layer truncation (not the named config)",
                       "global_batch": cfg.train_batch_size, "seq_len": L, "micro_batch": B, "grad_accum": gas,
                       "parallelism": main_res["parallelism"], "zero_path": zero_path, "l2": "inputs larger than L2 (per-step working set >> 126 MB)"},
            "mfu_of_measured_bf16_peak": mfu, "mfu_note": "model FLOPs/s over the measured sustained cuBLAS bf16 peak; fp8 projection GEMMs can exceed 1.0 of a bf16 denominator", "model_flops_per_token": fpt, "loss": final_loss,
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
            "bf16_only": None if other is None else {"value": other["value"], "ms_per_step": other["ms_per_step"],
                                                     "loss": other["loss"], "dtype": "bf16",
                                                     "mfu_of_measured_peak": (other["value"] * fpt / (world * peak)) if peak else None},
        }
        print(json.dumps(out))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
