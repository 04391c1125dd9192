"""Fused-kernel Llama forward over the weight segment and the paged KV cache.

Per layer on one GPU (tp = 1) the launch sequence is::

    rms_norm -> tcgen05 GEMM (fused qkv) -> rope_kv_store -> attention (prefill: tcgen05 ragged causal,
    decode: paged split-KV) -> tcgen05 GEMM (o_proj, residual add in the epilogue) -> rms_norm
    -> tcgen05 GEMM (gate||up, SiLU*mul in the epilogue) -> tcgen05 GEMM (down_proj, residual add in the epilogue)

i.e. 8 launches against the reference's ~9 kernels + 2 collectives (src/layer/attn.h:98-236,
src/layer/glu.h:86-164), with no standalone activation or residual kernels.  Layers can be run
one at a time (`run_layer`) so the live-scaling scheduler can execute exactly the layers whose
parameters have arrived (src/blitz/zigzag_manager.h:355-431), and `embed` / `head` are separate
steps like the reference's prologue/epilogue.

With tp > 1 the row-parallel GEMMs store partial sums, a `TPComm` sums them across the
replica's ranks and the fused add+RMSNorm kernel applies the residual (Megatron layout,
src/layer/attn.h:217-233, src/layer/glu.h:138-154); the LM head exchanges one
(max, index) pair per row instead of gathering logits (src/layer/lm_head.h:100-115).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

from .. import ops
from .config import ModelConfig
from .weights import WeightSegment


@dataclass
class StepMeta:
    """Device-side inputs of one forward step (all int32)."""
    ids: torch.Tensor            # [T] token ids
    pos: torch.Tensor            # [T] positions
    slot: torch.Tensor           # [T] cache slot = page_id * page_size + offset (-1: do not write)
    page_indices: torch.Tensor   # CSR page ids
    page_indptr: torch.Tensor    # [B + 1]
    last_page_len: torch.Tensor  # [B]
    tok_indptr: Optional[torch.Tensor] = None  # [B + 1] token offsets (prefill)
    seq_lens_host: List[int] = field(default_factory=list)  # rows per sequence in this pass (prefill)
    kv_lens_host: List[int] = field(default_factory=list)   # tokens cached per sequence after this pass (prefill)
    prefill_work: Optional[torch.Tensor] = None             # work records of the prefill attention (heaviest first)
    is_prefill: bool = False
    batch: int = 0
    num_tokens: int = 0
    num_splits: int = 1


class TPComm:
    """Sum / exchange across the tensor-parallel ranks of one replica. The NCCL implementation is the
    comparison baseline; the fused peer-memory kernels plug in through the same interface."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        self.dist.all_reduce(t, group=self.group)
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.size,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        self.dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out


class LlamaRunner:
    def __init__(self, seg: WeightSegment, kv_cache: torch.Tensor, max_tokens: int, max_batch: int,
                 comm: Optional[TPComm] = None):
        cfg = seg.cfg
        self.cfg: ModelConfig = cfg
        self.seg, self.kv, self.comm = seg, kv_cache, comm
        self.tp = seg.tp
        self.qh, self.kvh, self.hd = cfg.q_heads // self.tp, cfg.kv_heads // self.tp, cfg.head_dim
        self.inter = cfg.inter // self.tp
        self.page_size = kv_cache.shape[3]
        assert kv_cache.shape[0] == cfg.layers and kv_cache.shape[4] == self.kvh and kv_cache.shape[5] == self.hd
        dev, dt = seg.buffer.device, seg.dtype
        H = cfg.hidden
        self.max_tokens, self.max_batch = max_tokens, max_batch
        e = lambda *s: torch.empty(*s, dtype=dt, device=dev)
        self.res = e(max_tokens, H)
        self.normed = e(max_tokens, H)
        self.qkv = e(max_tokens, (self.qh + 2 * self.kvh) * self.hd)
        self.attn = e(max_tokens, self.qh * self.hd)
        self.act = e(max_tokens, self.inter)
        self.tmp = e(max_tokens, H) if self.tp > 1 else None
        self.last = e(max_batch, H)
        self.logits = e(max_batch, cfg.vocab // self.tp)
        self.tokens = torch.empty(max_batch, dtype=torch.int32, device=dev)
        self.maxval = torch.empty(max_batch, dtype=torch.float32, device=dev)
        self._ws = {}

    # ------------------------------------------------------------------ pieces
    def _w(self, l: int, name: str) -> torch.Tensor:
        return self.seg[f"layers.{l}.{name}"]

    def embed(self, m: StepMeta) -> None:
        T = m.num_tokens
        vs = self.cfg.vocab // self.tp
        ops.embedding(m.ids[:T], self.seg["embed"], self.res[:T], vocab_start=self.seg.tp_rank * vs,
                      zero_missing=True)
        if self.tp > 1:
            self.comm.all_reduce_(self.res[:T])

    def _workspace(self, B: int, splits: int) -> Optional[torch.Tensor]:
        if splits <= 1:
            return None
        n = ops.attn_decode_workspace_bytes(B, self.qh, self.hd, splits)
        ws = self._ws.get("dec")
        if ws is None or ws.numel() < n:
            ws = torch.empty(n, dtype=torch.uint8, device=self.res.device)
            self._ws["dec"] = ws
        return ws

    def attention_block(self, l: int, m: StepMeta) -> None:
        T, c = m.num_tokens, self.cfg
        ops.rms_norm(self.res[:T], self._w(l, "input_ln"), c.rms_eps, out=self.normed[:T])
        ops.gemm(self.normed[:T], self._w(l, "qkv"), static_b=True, out=self.qkv[:T])
        ops.rope_kv_store(self.qkv[:T], m.pos[:T], m.slot[:T], self.kv[l], q_heads=self.qh, kv_heads=self.kvh,
                          head_dim=self.hd, page_size=self.page_size, rope_theta=c.rope_theta)
        if m.is_prefill:
            self._prefill_attention(l, m)
        else:
            ops.attn_decode(self.qkv[:T], self.kv[l], m.page_indices, m.page_indptr, m.last_page_len,
                            q_heads=self.qh, kv_heads=self.kvh, head_dim=self.hd, page_size=self.page_size,
                            num_splits=m.num_splits, workspace=self._workspace(m.batch, m.num_splits),
                            out=self.attn[:T])
        if self.tp == 1:
            ops.gemm(self.attn[:T], self._w(l, "o"), static_b=True, out=self.res[:T], residual=self.res[:T], epilogue="add")
        else:
            ops.gemm(self.attn[:T], self._w(l, "o"), static_b=True, out=self.tmp[:T])
            self.comm.all_reduce_(self.tmp[:T])

    def _prefill_attention(self, l: int, m: StepMeta) -> None:
        """The pass's rows against everything the cache holds for their sequences (rope_kv_store has just added the
        rows' own keys and values): earlier chunks of a long prompt are simply a longer page list."""
        T = m.num_tokens
        if m.prefill_work is None:      # a caller that built the step by hand
            m.prefill_work = ops.prefill_work_list(m.seq_lens_host, m.kv_lens_host or m.seq_lens_host, self.page_size,
                                                   self.qkv.device)
        ops.attn_prefill_paged(self.qkv[:T], self.kv[l], m.page_indices, m.prefill_work, q_heads=self.qh,
                               kv_heads=self.kvh, head_dim=self.hd, page_size=self.page_size, out=self.attn[:T])

    def last_rows(self, m: StepMeta) -> torch.Tensor:
        """[batch, hidden]: the state `head` starts from, for the last row of every sequence of a prefill pass."""
        ops.gather_last(self.res[:m.num_tokens], m.tok_indptr, out=self.last[:m.batch])
        return self.last[:m.batch]

    def head_from_rows(self, rows: torch.Tensor) -> torch.Tensor:
        """First tokens from states collected with `last_rows` over several passes (a prompt prefetched in chunks)."""
        B = rows.shape[0]
        self.res[:B].copy_(rows)
        return self.head(StepMeta(ids=None, pos=None, slot=None, page_indices=None, page_indptr=None, last_page_len=None,
                                  is_prefill=False, batch=B, num_tokens=B))

    def ffn_block(self, l: int, m: StepMeta) -> None:
        T, c = m.num_tokens, self.cfg
        if self.tp == 1:
            ops.rms_norm(self.res[:T], self._w(l, "post_ln"), c.rms_eps, out=self.normed[:T])
        else:
            ops.add_rms_norm(self.tmp[:T], self.res[:T], self._w(l, "post_ln"), c.rms_eps, out=self.normed[:T])
        ops.gemm(self.normed[:T], self._w(l, "gate_up"), static_b=True, out=self.act[:T], epilogue="silu_mul")
        if self.tp == 1:
            ops.gemm(self.act[:T], self._w(l, "down"), static_b=True, out=self.res[:T], residual=self.res[:T], epilogue="add")
        else:
            ops.gemm(self.act[:T], self._w(l, "down"), static_b=True, out=self.tmp[:T])
            self.comm.all_reduce_(self.tmp[:T])
            ops.add_residual(self.res[:T], self.tmp[:T])

    def run_layer(self, l: int, m: StepMeta) -> None:
        self.attention_block(l, m)
        self.ffn_block(l, m)

    def head(self, m: StepMeta) -> torch.Tensor:
        B, T, c = m.batch, m.num_tokens, self.cfg
        if m.is_prefill:
            ops.gather_last(self.res[:T], m.tok_indptr, out=self.last[:B])
            src = self.last[:B]
        else:
            src = self.res[:B]
        ops.rms_norm(src, self.seg["final_norm"], c.rms_eps, out=self.normed[:B])
        ops.gemm(self.normed[:B], self.seg["lm_head"], static_b=True, out=self.logits[:B])
        vs = c.vocab // self.tp
        if self.tp == 1:
            ops.argmax(self.logits[:B], out=self.tokens[:B])
        else:
            ops.argmax(self.logits[:B], out=self.tokens[:B], out_val=self.maxval[:B], idx_offset=self.seg.tp_rank * vs)
            vals = self.comm.all_gather(self.maxval[:B])            # [tp, B]
            idxs = self.comm.all_gather(self.tokens[:B])            # [tp, B]
            best = vals.argmax(0, keepdim=True)
            self.tokens[:B].copy_(idxs.gather(0, best)[0])
        return self.tokens[:B]

    def forward(self, m: StepMeta, lo: int = 0, hi: Optional[int] = None, with_embed: bool = True,
                with_head: bool = True, after_layer=None) -> Optional[torch.Tensor]:
        """`after_layer(l)` is called once layer l's kernels are in the stream (its K/V stores among them): the hook
        of a layer-progressive KV migration."""
        hi = self.cfg.layers if hi is None else hi
        if with_embed:
            self.embed(m)
        for l in range(lo, hi):
            self.run_layer(l, m)
            if after_layer is not None:
                after_layer(l)
        return self.head(m) if with_head else None
