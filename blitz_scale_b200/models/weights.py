"""Weight segment: one contiguous buffer per TP rank with named tensor views.

The flat file format is the segment itself (byte-identical, like the reference's
``dangertensors.<tp_rank>.bin``, src/blitz/model_loader.cc:48-49) plus a JSON sidecar
carrying shapes, dtype and a layout hash so a stale file is rejected instead of
silently mis-sliced.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Optional

import torch

from .config import ModelConfig, SegmentLayout, build_layout

_ELEM = {torch.float16: 2, torch.bfloat16: 2, torch.float32: 4}


class WeightSegment:
    def __init__(self, cfg: ModelConfig, tp: int = 1, tp_rank: int = 0, dtype=torch.bfloat16, device="cpu",
                 buffer: Optional[torch.Tensor] = None):
        self.cfg, self.tp, self.tp_rank, self.dtype = cfg, tp, tp_rank, dtype
        self.layout: SegmentLayout = build_layout(cfg, tp, _ELEM[dtype])
        if buffer is None:
            buffer = torch.empty(self.layout.total_bytes, dtype=torch.uint8, device=device)
        assert buffer.dtype == torch.uint8 and buffer.numel() >= self.layout.total_bytes
        self.buffer = buffer
        self._views: Dict[str, torch.Tensor] = {}
        for name, spec in self.layout.tensors.items():
            self._views[name] = buffer[spec.offset:spec.offset + spec.nbytes].view(dtype).view(*spec.shape)

    def __getitem__(self, name: str) -> torch.Tensor:
        return self._views[name]

    def names(self):
        return list(self._views)

    def unit_bytes(self, name: str) -> torch.Tensor:
        off, nb = self.layout.unit(name)
        return self.buffer[off:off + nb]

    def layout_hash(self) -> str:
        desc = json.dumps({"model": self.cfg.name, "tp": self.tp, "dtype": str(self.dtype),
                           "tensors": [(n, list(s.shape), s.offset) for n, s in self.layout.tensors.items()]})
        return hashlib.sha256(desc.encode()).hexdigest()[:16]

    # ------------------------------------------------------------------ init / io
    def random_init_(self, seed: int = 0) -> "WeightSegment":
        """Deterministic random weights with activations of order one (norm gains near 1, matrices ~ N(0, 1/in))."""
        gen = torch.Generator(device="cpu").manual_seed(seed * 1000003 + self.tp_rank)
        shared = torch.Generator(device="cpu").manual_seed(seed * 1000003 + 7919)   # replicated tensors: same on every rank
        for name, v in self._views.items():
            if v.dim() == 1:
                val = 1.0 + 0.05 * torch.randn(v.shape, generator=shared)
            elif name == "embed":
                val = torch.randn(v.shape, generator=gen)
            else:
                val = torch.randn(v.shape, generator=gen) * (v.shape[0] ** -0.5)
            v.copy_(val.to(self.dtype))
        return self

    def random_init_fast_(self, seed: int = 0) -> "WeightSegment":
        """Random fill generated on the segment's own device (for multi-GB models)."""
        gen = torch.Generator(device=self.buffer.device).manual_seed(seed * 1000003 + self.tp_rank)
        # norm gains are replicated across the TP ranks of a replica: they must not depend on the rank
        shared = torch.Generator(device=self.buffer.device).manual_seed(seed * 1000003 + 7919)
        for name, v in self._views.items():
            if v.dim() == 1:
                v.copy_((1.0 + 0.05 * torch.randn(v.shape, generator=shared, device=v.device)).to(self.dtype))
            else:
                scale = 1.0 if name == "embed" else v.shape[0] ** -0.5
                rows = max(1, (64 << 20) // max(1, v.shape[1] * 4))
                for r0 in range(0, v.shape[0], rows):
                    blk = v[r0:r0 + rows]
                    blk.copy_((torch.randn(blk.shape, generator=gen, device=v.device) * scale).to(self.dtype))
        return self

    def save(self, directory) -> Path:
        d = Path(directory)
        d.mkdir(parents=True, exist_ok=True)
        path = d / f"segment.{self.tp_rank}.bin"
        self.buffer[:self.layout.total_bytes].cpu().numpy().tofile(path)
        (d / f"segment.{self.tp_rank}.json").write_text(json.dumps({
            "model": self.cfg.name, "tp": self.tp, "tp_rank": self.tp_rank, "dtype": str(self.dtype),
            "total_bytes": self.layout.total_bytes, "layout_hash": self.layout_hash()}))
        return path

    @staticmethod
    def check_sidecar(directory, cfg: ModelConfig, tp: int, tp_rank: int, dtype) -> Path:
        d = Path(directory)
        meta = json.loads((d / f"segment.{tp_rank}.json").read_text())
        probe = WeightSegment(cfg, tp, tp_rank, dtype, device="meta")
        if meta["layout_hash"] != probe.layout_hash() or meta["total_bytes"] != probe.layout.total_bytes:
            raise ValueError("segment file does not match the model layout")
        return d / f"segment.{tp_rank}.bin"


def shard_from_full(full: WeightSegment, tp: int, tp_rank: int, device=None) -> WeightSegment:
    """Slice a tp=1 segment into the segment of ``tp_rank`` (heads / inter / vocab split, Megatron style;
    cf. scripts/util/make_dangertensors.py:90-188)."""
    cfg = full.cfg
    assert full.tp == 1
    out = WeightSegment(cfg, tp, tp_rank, full.dtype, device=device or full.buffer.device)
    hd = cfg.head_dim
    qh, kvh, it, vs = cfg.q_heads // tp, cfg.kv_heads // tp, cfg.inter // tp, cfg.vocab // tp
    r = tp_rank
    out["embed"].copy_(full["embed"][r * vs:(r + 1) * vs])
    for l in range(cfg.layers):
        p = f"layers.{l}."
        out[p + "input_ln"].copy_(full[p + "input_ln"])
        out[p + "post_ln"].copy_(full[p + "post_ln"])
        w = full[p + "qkv"]
        Q, K = cfg.q_heads * hd, cfg.kv_heads * hd
        q = w[:, r * qh * hd:(r + 1) * qh * hd]
        k = w[:, Q + r * kvh * hd:Q + (r + 1) * kvh * hd]
        v = w[:, Q + K + r * kvh * hd:Q + K + (r + 1) * kvh * hd]
        out[p + "qkv"].copy_(torch.cat([q, k, v], dim=1))
        out[p + "o"].copy_(full[p + "o"][r * qh * hd:(r + 1) * qh * hd])
        gu = full[p + "gate_up"]
        out[p + "gate_up"].copy_(torch.cat([gu[:, r * it:(r + 1) * it],
                                            gu[:, cfg.inter + r * it:cfg.inter + (r + 1) * it]], dim=1))
        out[p + "down"].copy_(full[p + "down"][r * it:(r + 1) * it])
    out["final_norm"].copy_(full["final_norm"])
    out["lm_head"].copy_(full["lm_head"][:, r * vs:(r + 1) * vs])
    return out
