"""Generation with cached state: one token per step in constant time, instead of re-running the model on the growing context.

Every operator of a StripedHyena 2 block has a small recurrent form:

    featuriser conv (k_f taps)        the last k_f - 1 rows of the in-projection output
    Hyena-SE / Hyena-MR (K taps)      the last K - 1 rows of u = x2 v           (a FIR filter needs nothing older)
    Hyena-LI (modal filter, order O)  the O modal states per channel, s <- lam s + u, y = R . s + bias u
    attention                         the keys (rotary embedding applied) and values of all previous tokens

`CachedDecoder.prefill(tokens)` runs the model's ordinary parallel forward over the prompt once and collects those states
from the layers' inputs (forward pre-hooks; the Hyena-LI state comes from the scan kernel's `return_state`);
`CachedDecoder.step(token)` then advances all layers by one position.  Role of the reference's cached inference path
(savanna/text_generation_utils.py:173-365 `stream_tokens` with `InferenceParams`, :672-774 the interactive driver; its
recurrent Hyena inference lives in the separate vortex project).  Decode steps are matrix-vector work on one token and
use plain PyTorch operations on the model's own parameters.  Supported: one device (no tensor / context / pipeline
parallelism), pre-norm blocks with the gated MLP, rotary or no position embedding, implicit-modal Hyena-LI filters; any
other configuration raises and the caller falls back to `stream_tokens` (recompute).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..models.filters import ImplicitModalFilter
from ..models.hyena import HyenaOperator, ShortHyenaOperator
from ..models.mixer import SelfAttention
from ..models.mlp import ParallelGLU
from ..ops import reference as ref
from ..parallel import state


def _rms(x, norm):
    return ref.rmsnorm(x, norm.gain, norm.eps, norm.form) if hasattr(norm, "gain") else norm(x)


def _act(name: str):
    return {"silu": F.silu, "gelu": F.gelu, "relu": F.relu, "identity": lambda t: t}[name]


class CachedDecoder:
    def __init__(self, model):
        cfg = model.cfg
        if state.get_model_parallel_world_size() > 1 or state.get_context_parallel_world_size() > 1 or \
                getattr(model, "is_pipeline_stage", False):
            raise NotImplementedError("cached generation runs on one device")
        if not cfg.prenorm or cfg.postnorm or cfg.outer_mlp_norm or cfg.gpt_j_residual:
            raise NotImplementedError("cached generation supports pre-norm blocks")
        if cfg.pos_emb not in ("rotary", "rotary_linear_scaled", "rotary_ntk_scaled", "rotary2", "none", None):
            raise NotImplementedError(f"cached generation does not support pos_emb={cfg.pos_emb!r}")
        self.model, self.cfg = model, cfg
        self.blocks = model.blocks()
        for b in self.blocks:
            if not isinstance(b.mlp, ParallelGLU):
                raise NotImplementedError("cached generation supports the gated MLP")
            if getattr(b.mixer, "tie_projections", False) or getattr(b.mixer, "proj_groups", 1) > 1:
                raise NotImplementedError("cached generation expects the full-width (3 x hidden) in-projection")
            m = b.mixer.mixer
            if isinstance(m, HyenaOperator) and not m.is_mr and not isinstance(m.filter, ImplicitModalFilter):
                raise NotImplementedError("cached generation needs the implicit modal filter for Hyena-LI")
            if getattr(m, "sparse", False):
                raise NotImplementedError("cached generation does not cover the block-sparse attention operators")
            if isinstance(m, HyenaOperator) and (m.bidirectional or m.slow_heads):
                raise NotImplementedError("cached generation does not cover two-sided filters or outer-product heads")
        self.states: List[Dict] = []
        self.pos = 0

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, T] -> logits of the last position [B, V]; leaves every layer's state at position T."""
        from .. import ops
        model = self.model
        B, T = tokens.shape
        self.states = [dict() for _ in self.blocks]
        hooks = []

        def tail(x, n):
            """Last n rows of x [B, T, C], zero-padded on the left when the prompt is shorter."""
            if n <= 0:
                return x[:, :0]
            if x.shape[1] >= n:
                return x[:, -n:].clone()
            return F.pad(x, (0, 0, n - x.shape[1], 0))

        for st, blk in zip(self.states, self.blocks):
            mixer = blk.mixer
            inner = mixer.mixer
            if isinstance(inner, SelfAttention):
                def grab_kv(mod, args, st=st):
                    qkv, positions = args[0], args[1]
                    Bq, L, _ = qkv.shape
                    qkv = qkv.view(Bq, L, mod.heads, 3 * mod.hd)
                    k, v = qkv[..., mod.hd: 2 * mod.hd], qkv[..., 2 * mod.hd:]
                    if mod._rotary:
                        cos, sin = mod._rotary[0](positions)
                        k = ref.apply_rope(k.float(), cos, sin).to(qkv.dtype)
                    st["k"], st["v"] = k.clone(), v.clone()
                hooks.append(inner.register_forward_pre_hook(grab_kv))
            else:
                kf = mixer.short_conv_L

                def grab_proj(mod, args, st=st, kf=kf):
                    st["proj_tail"] = tail(args[0], kf - 1)
                hooks.append(mixer.hyena_proj_conv.register_forward_pre_hook(grab_proj))

                def grab_feat(mod, args, st=st):
                    feat = args[0]
                    u = feat[..., 1::3] * feat[..., 2::3]
                    if isinstance(mod, ShortHyenaOperator):
                        st["u_tail"] = tail(u if mod.pregate else feat[..., 2::3], mod.kernel_size - 1)
                    elif mod.is_mr:
                        st["u_tail"] = tail(u, min(mod.hyena_mr_len, 1 << 30) - 1)
                    else:
                        g, R, p = mod._modal()
                        _, s = ops.hyena_li_modal(feat, g, R, p, mod.conv_bias, None, True)
                        st["s"] = s.float()
                hooks.append(inner.register_forward_pre_hook(grab_feat))
        was_training = model.training
        model.eval()
        try:
            logits = model(tokens)[:, -1].float()
        finally:
            for h in hooks:
                h.remove()
            model.train(was_training)
        self.pos = T
        return logits

    # ------------------------------------------------------------------ one decode step
    def _hyena_step(self, blk, st, proj):
        """proj [B, 3D] (in-projection of the new token) -> z [B, D]."""
        mixer, inner = blk.mixer, blk.mixer.mixer
        conv = mixer.hyena_proj_conv
        w = conv.taps().float()
        if conv.group_dim > 1:
            w = w.repeat_interleave(conv.group_dim, dim=0)
        window = torch.cat([st["proj_tail"].float(), proj[:, None].float()], dim=1)          # [B, kf, 3D], oldest first
        feat = torch.einsum("bkc,ck->bc", window, w)
        st["proj_tail"] = window[:, 1:].to(proj.dtype)
        feat = feat.to(proj.dtype).float()                 # the parallel path rounds the featuriser output to the model dtype
        x1, x2, v = feat[:, 0::3], feat[:, 1::3], feat[:, 2::3]
        u = x2 * v
        if isinstance(inner, ShortHyenaOperator):
            un = u if inner.pregate else v
            w = inner.short_conv.taps().float().repeat_interleave(inner.group_dim, dim=0)    # [D, K] correlation order
            window = torch.cat([st["u_tail"].float(), un[:, None]], dim=1)
            y = torch.einsum("bkc,ck->bc", window, w)
            st["u_tail"] = window[:, 1:]
            return (x1 * y) if inner.postgate else y
        if inner.is_mr:
            K = st["u_tail"].shape[1] + 1
            h = inner.filter(K).float().repeat_interleave(inner.group_dim, dim=0)            # [D, K] convolution order
            window = torch.cat([st["u_tail"].float(), u[:, None]], dim=1)
            y = torch.einsum("bkc,ck->bc", window, h.flip(-1)) + inner.conv_bias.float() * u
            st["u_tail"] = window[:, 1:]
            return x1 * y
        g, R, p = inner._modal()
        lam = torch.exp(-torch.exp(p.float()) * torch.exp(g.float()))                         # [D, O]
        s = lam * st["s"] + u[..., None]
        st["s"] = s
        y = (R.float() * s).sum(-1) + inner.conv_bias.float() * u
        return x1 * y

    def _attention_step(self, blk, st, proj):
        inner = blk.mixer.mixer
        B = proj.shape[0]
        qkv = proj.view(B, 1, inner.heads, 3 * inner.hd)
        q, k, v = qkv[..., : inner.hd], qkv[..., inner.hd: 2 * inner.hd], qkv[..., 2 * inner.hd:]
        if inner._rotary:
            pos = torch.tensor([self.pos], device=proj.device)
            cos, sin = ref.rope_tables(pos, inner._rotary[0].dim, inner._rotary[0].base, inner._rotary[0].scaling_factor)
            q = ref.apply_rope(q.float(), cos, sin).to(proj.dtype)
            k = ref.apply_rope(k.float(), cos, sin).to(proj.dtype)
        st["k"] = torch.cat([st["k"], k], dim=1)
        st["v"] = torch.cat([st["v"], v], dim=1)
        scores = torch.einsum("bqhd,bkhd->bhqk", q.float(), st["k"].float()) / math.sqrt(inner.hd)
        o = torch.einsum("bhqk,bkhd->bqhd", scores.softmax(-1), st["v"].float())
        return o.reshape(B, inner.heads * inner.hd)

    @torch.no_grad()
    def step(self, token: torch.Tensor) -> torch.Tensor:
        """token [B] -> logits of the next position [B, V]; advances every layer's state by one token."""
        model, cfg = self.model, self.cfg
        dtype = cfg.params_dtype
        pos = torch.tensor([self.pos], device=token.device)
        was_training = model.training
        model.eval()
        try:
            x = model.embedding(token[:, None], pos)[:, 0]                                   # [B, D]
        finally:
            model.train(was_training)
        for blk, st in zip(self.blocks, self.states):
            mixer = blk.mixer
            u = _rms(x.float(), blk.input_layernorm).to(dtype)
            proj = F.linear(u, mixer.dense_projection.weight)
            if isinstance(mixer.mixer, SelfAttention):
                z = self._attention_step(blk, st, proj)
            else:
                z = self._hyena_step(blk, st, proj)
            a = F.linear(z.to(dtype), mixer.dense.weight, mixer.dense.bias).float() + x.float()
            a = a.to(dtype)
            h = _rms(a.float(), blk.pre_mlp_layernorm).to(dtype) if blk.pre_mlp_norm else a
            mlp = blk.mlp
            ab = F.linear(h, mlp.w12)
            g, b = ab.float().chunk(2, dim=-1)
            hid = (_act(mlp.act)(g) * b).to(dtype)
            y = F.linear(hid, mlp.w3.weight, mlp.w3.bias).float() + a.float()
            x = y.to(dtype)
        self.pos += 1
        return model.logits(x[:, None])[:, 0].float()


@torch.no_grad()
def stream_tokens_cached(model, context_tokens: List[List[int]], eos_token_id: Optional[int] = None, maximum_tokens: int = 64,
                         temperature: float = 0.0, top_k: int = 0, top_p: float = 0.0, generator=None):
    """Cached counterpart of `generation.stream_tokens` for prompts of equal length: one prefill, then one `step` per
    generated token.  Yields (tokens [B, T], logits of the step, finished mask)."""
    from .generation import sample_tokens
    lens = {len(c) for c in context_tokens}
    if len(lens) != 1:
        raise ValueError("cached generation takes prompts of equal length (pad or group them by length)")
    device = next(model.parameters()).device
    toks = torch.tensor(context_tokens, dtype=torch.long, device=device)
    dec = CachedDecoder(model)
    logits = dec.prefill(toks)
    done = torch.zeros(toks.shape[0], dtype=torch.bool, device=device)
    for _ in range(maximum_tokens):
        nxt = sample_tokens(logits, temperature, top_k, top_p, generator)
        if eos_token_id is not None:
            nxt = torch.where(done, torch.full_like(nxt, eos_token_id), nxt)
            done |= nxt == eos_token_id
        toks = torch.cat([toks, nxt[:, None]], dim=1)
        yield toks, logits, done
        if bool(done.all()):
            break
        logits = dec.step(nxt)
