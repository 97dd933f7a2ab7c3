"""Model-FLOPs accounting and MFU / HFU.

FLOP model per token and layer (forward; x3 for forward+backward, x4 with full activation recompute = HFU),
after the reference's savanna/mfu.py:182-294, with its layer-type parsing fixed (it counts every Hyena
layer as an FFT long convolution, mfu.py:313-342):
    in-projection 2*D*3D, out-projection 2*D*D, gated MLP 6*D*F (plain MLP 16*D*D),
    attention 4*L*D, featuriser conv 2*k_f*3D, Hyena-SE 2*k*D, Hyena-MR 2*k*D,
    Hyena-LI as the reference counts it: FFT 10*log2(L)*D  (this framework's modal scan does less work),
    logits 2*D*V once per token.
The peak comes from the measured cuBLAS bf16 throughput of this pool's B200 (MEASURED_PEAKS.json at the
repository root, key bf16_tflops_sustained) when present, else from the table below.  The reference has
no Blackwell entry and silently skips MFU (mfu.py:542-657).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional

# dense bf16 tensor-core peaks, FLOP/s
DEVICE_PEAKS = {
    "B200": 2.25e15,
    "H100 SXM": 989.4e12, "H100": 989.4e12, "H100 PCIe": 756e12, "H200": 989.4e12,
    "A100": 312e12,
}
FALLBACK_MEASURED = 1.59e15


def layer_flops_per_token(cfg, op: str, executed: bool = False) -> float:
    """`executed=False` reproduces the reference's accounting (full L x L attention, Hyena-LI as an FFT).
    `executed=True` counts what a causal model has to do: attention over the lower triangle only (2*L*D) and
    Hyena-LI as the order-`hyena_filter_order` modal recurrence (state update + read-out, 4*order*D)."""
    D, L = cfg.hidden_size, cfg.seq_length
    f = 2 * D * 3 * D + 2 * D * D
    if cfg.identity_mlp:
        pass
    elif cfg.mlp_type == "regular":
        f += 16 * D * D
    elif cfg.mlp_type == "short_hyena":
        k = cfg.hyena_mlp_len or cfg.hyena_se_len
        f += 2 * D * 3 * D + 2 * D * D + 2 * cfg.short_conv_L * 3 * D + 2 * k * D
    else:
        f += 6 * D * cfg.ffn_size
    if op.startswith("hyena"):
        f += 2 * cfg.short_conv_L * 3 * D
        if op == "hyena_se":
            f += 2 * cfg.hyena_se_len * D
        elif op == "hyena_mr":
            f += 2 * min(cfg.hyena_mr_len, L) * D
        elif executed:
            f += 4 * (cfg.hyena_filter_order or 16) * D
        else:
            f += 10 * math.log2(max(2, L)) * D
    else:
        f += (2 if executed else 4) * L * D
    return float(f)


def model_flops_per_token(cfg, backward: bool = True, recompute: bool = False, executed: bool = False) -> float:
    fwd = sum(layer_flops_per_token(cfg, op, executed) for op in cfg.operator_config)
    fwd += 2 * cfg.hidden_size * (cfg.padded_vocab_size or 512)
    mult = 1 + (2 if backward else 0) + (1 if recompute else 0)
    return fwd * mult


def measured_peaks() -> Optional[Dict]:
    here = os.path.dirname(os.path.abspath(__file__))
    for up in (os.path.join(here, "..", ".."), os.getcwd()):
        p = os.path.join(up, "MEASURED_PEAKS.json")
        if os.path.exists(p):
            try:
                return json.load(open(p))
            except Exception:
                return None
    return None


def peak_flops(cfg=None, device_name: Optional[str] = None, sustained: bool = True) -> Optional[float]:
    """Denominator of MFU, FLOP/s per GPU: configured > measured on this pool > datasheet table."""
    if cfg is not None and getattr(cfg, "peak_tflops", None):
        return cfg.peak_tflops * 1e12
    m = measured_peaks()
    if m:
        key = "bf16_tflops_sustained" if sustained and "bf16_tflops_sustained" in m else "bf16_tflops"
        if key in m:
            return float(m[key]) * 1e12
    if device_name is None:
        try:
            import torch
            device_name = torch.cuda.get_device_name() if torch.cuda.is_available() else None
        except Exception:
            device_name = None
    if device_name:
        for k in sorted(DEVICE_PEAKS, key=len, reverse=True):
            if k.lower() in device_name.lower():
                return DEVICE_PEAKS[k]
    return None


def mfu(tokens_per_sec_per_gpu: float, cfg, recompute: bool = False) -> Dict[str, Optional[float]]:
    peak = peak_flops(cfg)
    model = tokens_per_sec_per_gpu * model_flops_per_token(cfg, True, False)
    hw = tokens_per_sec_per_gpu * model_flops_per_token(cfg, True, recompute)
    return {"model_flops_per_sec": model, "hardware_flops_per_sec": hw,
            "mfu": model / peak if peak else None, "hfu": hw / peak if peak else None}
