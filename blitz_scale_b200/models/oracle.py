"""Eager PyTorch Llama forward used as the numerical oracle (CPU or GPU, any float dtype).

It reads the same weight segment as the fused engine, keeps a dense (non-paged) KV list per
sequence and applies the rotate-half RoPE convention to q and k.  The reference admits its own
kernels emit wrong tokens (README.md:61-62), so this forward, not the reference, defines
correctness: the fused kernels must stay within 1e-2 relative error of it in bf16.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .config import ModelConfig
from .weights import WeightSegment


def rms_norm_ref(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def rope_ref(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """x: [T, heads, hd]; pos: [T]. Rotate-half convention, computed in fp32."""
    hd = x.shape[-1]
    half = hd // 2
    inv = theta ** (-torch.arange(0, half, dtype=torch.float32, device=x.device) * 2.0 / hd)
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)


class LlamaOracle:
    def __init__(self, seg: WeightSegment, compute_dtype: Optional[torch.dtype] = None):
        assert seg.tp == 1, "the oracle runs the unsharded model"
        self.cfg: ModelConfig = seg.cfg
        self.dt = compute_dtype or seg.dtype
        self.w = {n: seg[n].to(self.dt) for n in seg.names()}
        self.kv: List[List[Tuple[torch.Tensor, torch.Tensor]]] = []  # [seq][layer] -> (k, v)

    def _layer(self, l: int, x: torch.Tensor, pos: torch.Tensor, past):
        c, w = self.cfg, self.w
        p = f"layers.{l}."
        h = rms_norm_ref(x, w[p + "input_ln"], c.rms_eps)
        qkv = h @ w[p + "qkv"]
        Q, K = c.q_heads * c.head_dim, c.kv_heads * c.head_dim
        T = x.shape[0]
        q = rope_ref(qkv[:, :Q].view(T, c.q_heads, c.head_dim), pos, c.rope_theta)
        k = rope_ref(qkv[:, Q:Q + K].view(T, c.kv_heads, c.head_dim), pos, c.rope_theta)
        v = qkv[:, Q + K:].view(T, c.kv_heads, c.head_dim)
        if past is not None:
            k = torch.cat([past[0], k], 0)
            v = torch.cat([past[1], v], 0)
        S = k.shape[0]
        g = c.q_heads // c.kv_heads
        kk = k.repeat_interleave(g, dim=1).float()
        vv = v.repeat_interleave(g, dim=1).float()
        scores = torch.einsum("thd,shd->hts", q.float(), kk) * (c.head_dim ** -0.5)
        qpos = torch.arange(S - T, S, device=x.device)
        mask = torch.arange(S, device=x.device)[None, :] > qpos[:, None]
        scores = scores.masked_fill(mask[None], float("-inf"))
        att = torch.einsum("hts,shd->thd", scores.softmax(-1), vv).to(x.dtype).reshape(T, Q)
        x = x + att @ w[p + "o"]
        h = rms_norm_ref(x, w[p + "post_ln"], c.rms_eps)
        gu = h @ w[p + "gate_up"]
        it = c.inter
        act = (torch.nn.functional.silu(gu[:, :it].float()) * gu[:, it:].float()).to(x.dtype)
        x = x + act @ w[p + "down"]
        return x, (k, v)

    def run_layers(self, x: torch.Tensor, pos: torch.Tensor, past, lo: int = 0, hi: Optional[int] = None):
        hi = self.cfg.layers if hi is None else hi
        new = []
        for l in range(lo, hi):
            x, kv = self._layer(l, x, pos, None if past is None else past[l])
            new.append(kv)
        return x, new

    def logits(self, x_last: torch.Tensor) -> torch.Tensor:
        h = rms_norm_ref(x_last, self.w["final_norm"], self.cfg.rms_eps)
        return h @ self.w["lm_head"]

    @torch.no_grad()
    def generate(self, prompts: List[List[int]], max_new: int, return_logits: bool = False):
        """Greedy generation; returns token lists (and the per-step logits of every sequence)."""
        dev = self.w["embed"].device
        outs, all_logits = [], []
        for prompt in prompts:
            ids = torch.tensor(prompt, device=dev, dtype=torch.long)
            x = self.w["embed"][ids]
            pos = torch.arange(len(prompt), device=dev)
            x, past = self.run_layers(x, pos, None)
            toks, lgs = [], []
            lg = self.logits(x[-1:])
            for step in range(max_new):
                t = int(lg.float().argmax(-1))
                toks.append(t)
                lgs.append(lg[0].float().cpu())
                if step == max_new - 1:
                    break
                x = self.w["embed"][torch.tensor([t], device=dev)]
                pos = torch.tensor([len(prompt) + step], device=dev)
                x, past = self.run_layers(x, pos, past)
                lg = self.logits(x)
            outs.append(toks)
            all_logits.append(lgs)
        return (outs, all_logits) if return_logits else outs
