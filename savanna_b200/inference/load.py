"""Load a trained model for inference (reference: savanna/inference/load.py, savanna/loading.py).

    model, tokenizer, cfg = load_for_inference("<save>/global_step100")            # configs stored in the checkpoint
    model, tokenizer, cfg = load_for_inference(ckpt_dir, config_files=["model.yml"])

Only the model states are read (no optimizer shards); tensor-parallel shards are merged when the checkpoint was written
with more than one model-parallel rank and this process runs alone.  Command line: prints completions for prompts.

    python -m savanna_b200.inference.load <save>/global_step100 --prompt ACGTTGCA --tokens 64 [--temperature 0.8]
"""
from __future__ import annotations

import argparse
import glob
import os
from typing import List, Optional

import torch


def load_for_inference(step_dir: str, config_files: Optional[List[str]] = None, device: Optional[str] = None,
                       overrides: Optional[dict] = None):
    from ..config import GlobalConfig
    from ..models import build_model
    from ..tools.reshard_model_parallel import load_shards, merge_module
    if os.path.isfile(os.path.join(step_dir, "latest")):          # a save root: follow `latest`
        with open(os.path.join(step_dir, "latest")) as fh:
            step_dir = os.path.join(step_dir, fh.read().strip())
    if config_files is None:
        config_files = sorted(glob.glob(os.path.join(step_dir, "configs", "*.yml")))
        if not config_files:
            raise FileNotFoundError(f"{step_dir} holds no configs/*.yml: pass config_files")
    over = {"global_num_gpus": 1, "model_parallel_size": 1, "pipe_parallel_size": 0, "context_parallel_size": 1,
            "sequence_parallel": False, "checkpoint_activations": False, "hidden_dropout": 0.0, "attention_dropout": 0.0}
    over.update(overrides or {})
    cfg = GlobalConfig.from_ymls(config_files, over)
    cfg.build_tokenizer()
    from ..parallel import state
    if not state.model_parallel_is_initialized():
        state.initialize_model_parallel(1, 1, 1)
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    model = build_model(cfg, device=dev)
    shards = load_shards(step_dir)
    module = merge_module([s["module"] for s in shards]) if len(shards) > 1 else shards[0]["module"]
    missing, unexpected = model.load_state_dict(module, strict=False)
    bad = [k for k in list(missing) + list(unexpected) if not k.endswith("_extra_state") and not k.endswith("filter.t")]
    if bad:
        raise RuntimeError(f"checkpoint and model disagree on {len(bad)} keys, e.g. {bad[:4]}")
    model.eval()
    return model, cfg.tokenizer, cfg


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("checkpoint")
    ap.add_argument("--config", nargs="*", default=None)
    ap.add_argument("--prompt", action="append", default=[])
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=0.0)
    a = ap.parse_args(argv)
    from .generation import generate
    model, tok, _ = load_for_inference(a.checkpoint, a.config)
    for rec in generate(model, tok, a.prompt or ["ACGT"], maximum_tokens=a.tokens, temperature=a.temperature,
                        top_k=a.top_k, top_p=a.top_p):
        print(rec)


if __name__ == "__main__":
    main()
