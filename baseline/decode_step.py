"""Stand-in reference decode step: the reference's model loop on the libraries it serves with.

The reference cannot be built here (empty submodules, no MPI / gRPC C++ / cargo), so its decode iteration
(src/model/llama.h:268-416: per layer RMSNorm -> qkv GEMM -> paged decode attention with RoPE and KV append ->
o GEMM + residual -> RMSNorm -> gate/up GEMM -> SiLU*mul -> down GEMM + residual; then final norm, LM head, arg-max)
is re-stated on library kernels only: cuBLAS through ``torch.matmul`` / ``torch.addmm`` for every GEMM
(src/util/cublas_wrapper.h:31-141), and a library paged decode attention where the reference calls FlashInfer
(src/kernel/attention_decode.cu:13-40).  The attention library is the first of these that runs on the box:

  1. ``flash_attn.flash_attn_with_kvcache`` with a block table (RoPE, KV append and attention in one call; its paged
     cache wants blocks of 256 tokens, so this arm pages in 256-token blocks),
  2. ``flashinfer.BatchDecodeWithPagedKVCacheWrapper`` (RoPE and append by torch ops),
  3. ``torch.nn.functional.scaled_dot_product_attention`` over a dense per-sequence cache.

The step is captured in a CUDA graph, like the product's.  Nothing here imports the product's kernels or engine, and
nothing in the product path imports this module.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn.functional as F

from blitz_scale_b200.models.config import ModelConfig, get_config


class BaselineDecoder:
    """Random-init Llama-shaped model + KV cache for `batch` sequences of `ctx` tokens, decoding one token per step."""

    def __init__(self, model: str, batch: int, ctx: int, max_new: int, device: torch.device, seed: int = 0,
                 attention: Optional[str] = None):
        self.cfg: ModelConfig = get_config(model)
        c = self.cfg
        self.B, self.ctx, self.dev = batch, ctx, device
        dt = torch.bfloat16
        g = torch.Generator(device=device).manual_seed(seed)

        def w(*shape, scale):
            return (torch.randn(*shape, device=device, dtype=torch.float32, generator=g) * scale).to(dt)

        qkv_out = (c.q_heads + 2 * c.kv_heads) * c.head_dim
        self.embed = w(c.vocab, c.hidden, scale=0.02)
        self.layers = []
        for _ in range(c.layers):
            self.layers.append(dict(
                ln1=torch.ones(c.hidden, device=device, dtype=dt), ln2=torch.ones(c.hidden, device=device, dtype=dt),
                qkv=w(c.hidden, qkv_out, scale=c.hidden ** -0.5), o=w(c.q_heads * c.head_dim, c.hidden, scale=c.hidden ** -0.5),
                gate_up=w(c.hidden, 2 * c.inter, scale=c.hidden ** -0.5), down=w(c.inter, c.hidden, scale=c.inter ** -0.5)))
        self.norm = torch.ones(c.hidden, device=device, dtype=dt)
        self.lm_head = w(c.hidden, c.vocab, scale=c.hidden ** -0.5)

        self.max_len = ctx + max_new + 1
        self.attention = attention or self._pick_attention()
        self._alloc_cache()
        rope_len = max(self.max_len + 8, getattr(self, "pages_per_seq", 0) * getattr(self, "page", 0))
        # per-step inputs live in fixed device buffers (the graph reads them); a pinned host mirror feeds them
        self.ids = torch.zeros(batch, dtype=torch.int64, device=device)
        self.lens = torch.full((batch,), ctx, dtype=torch.int32, device=device)       # tokens already cached
        self.tokens = torch.zeros(batch, dtype=torch.int64, device=device)
        self.h_in = torch.zeros(2, batch, dtype=torch.int64).pin_memory()
        self.h_out = torch.zeros(batch, dtype=torch.int64).pin_memory()
        self.d_in = torch.zeros(2, batch, dtype=torch.int64, device=device)
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=device, dtype=torch.float32) / c.head_dim))
        ang = torch.arange(rope_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos().to(dt), ang.sin().to(dt)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.h2d_bytes = self.h_in.numel() * 8
        self.d2h_bytes = self.h_out.numel() * 8

    # ------------------------------------------------------------------ attention back ends
    def _pick_attention(self) -> str:
        c = self.cfg
        q = torch.randn(2, 1, c.q_heads, c.head_dim, device=self.dev, dtype=torch.bfloat16)
        try:
            from flash_attn import flash_attn_with_kvcache
            kc = torch.zeros(4, 256, c.kv_heads, c.head_dim, device=self.dev, dtype=torch.bfloat16)
            bt = torch.tensor([[0, 1], [2, 3]], dtype=torch.int32, device=self.dev)
            flash_attn_with_kvcache(q, kc, kc.clone(), cache_seqlens=torch.tensor([300, 7], dtype=torch.int32, device=self.dev),
                                    block_table=bt, causal=True)
            torch.cuda.synchronize()
            return "flash_attn"
        except Exception:
            pass
        try:
            import flashinfer
            ws = torch.empty(128 << 20, dtype=torch.uint8, device=self.dev)
            wr = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
            kv = torch.zeros(4, 2, 64, c.kv_heads, c.head_dim, device=self.dev, dtype=torch.bfloat16)
            wr.plan(torch.tensor([0, 2, 4], dtype=torch.int32, device=self.dev),
                    torch.tensor([0, 1, 2, 3], dtype=torch.int32, device=self.dev),
                    torch.tensor([5, 64], dtype=torch.int32, device=self.dev), c.q_heads, c.kv_heads, c.head_dim, 64,
                    q_data_type=torch.bfloat16)
            wr.run(q[:, 0], kv)
            torch.cuda.synchronize()
            return "flashinfer"
        except Exception:
            return "sdpa"

    def _alloc_cache(self) -> None:
        c, B = self.cfg, self.B
        dt = torch.bfloat16
        if self.attention == "flash_attn":
            self.page = 256
            self.pages_per_seq = (self.max_len + self.page - 1) // self.page
            n = B * self.pages_per_seq
            self.kcache = [torch.randn(n, self.page, c.kv_heads, c.head_dim, device=self.dev, dtype=dt) for _ in range(c.layers)]
            self.vcache = [torch.randn(n, self.page, c.kv_heads, c.head_dim, device=self.dev, dtype=dt) for _ in range(c.layers)]
            perm = torch.randperm(n, device=self.dev).to(torch.int32)
            self.block_table = perm.view(B, self.pages_per_seq).contiguous()
        elif self.attention == "flashinfer":
            import flashinfer
            self.page = 64
            self.pages_per_seq = (self.max_len + self.page - 1) // self.page
            n = B * self.pages_per_seq
            self.kv = [torch.randn(n, 2, self.page, c.kv_heads, c.head_dim, device=self.dev, dtype=dt) for _ in range(c.layers)]
            perm = torch.randperm(n, device=self.dev).to(torch.int32)
            self.block_table = perm.view(B, self.pages_per_seq).contiguous()
            self.fi_ws = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)
            self.fi_indptr = (torch.arange(B + 1, device=self.dev, dtype=torch.int32) * self.pages_per_seq)
            self.fi_wrapper = flashinfer.BatchDecodeWithPagedKVCacheWrapper(
                self.fi_ws, "NHD", use_cuda_graph=True, paged_kv_indptr_buffer=self.fi_indptr.clone(),
                paged_kv_indices_buffer=self.block_table.view(-1).clone(),
                paged_kv_last_page_len_buffer=torch.ones(B, dtype=torch.int32, device=self.dev))
        else:
            self.kdense = [torch.randn(B, c.kv_heads, self.max_len, c.head_dim, device=self.dev, dtype=dt) for _ in range(c.layers)]
            self.vdense = [torch.randn(B, c.kv_heads, self.max_len, c.head_dim, device=self.dev, dtype=dt) for _ in range(c.layers)]

    def _plan(self, cur_len: int) -> None:
        """flashinfer only: the wrapper plans page counts on the host before every step (as the reference's
        flashinfer_types.cu:52-80 does)."""
        if self.attention != "flashinfer":
            return
        n_pages = (cur_len + 1 + self.page - 1) // self.page
        indptr = torch.arange(self.B + 1, dtype=torch.int32) * n_pages
        indices = self.block_table[:, :n_pages].reshape(-1)
        last = torch.full((self.B,), cur_len + 1 - (n_pages - 1) * self.page, dtype=torch.int32)
        c = self.cfg
        self.fi_wrapper.plan(indptr, indices, last, c.q_heads, c.kv_heads, c.head_dim, self.page,
                             q_data_type=torch.bfloat16)

    def _rope(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        cos, sin = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
        x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)

    def _attend(self, li: int, q, k, v):
        c, B = self.cfg, self.B
        if self.attention == "flash_attn":
            from flash_attn import flash_attn_with_kvcache
            o = flash_attn_with_kvcache(q.view(B, 1, c.q_heads, c.head_dim), self.kcache[li], self.vcache[li],
                                        k=k.view(B, 1, c.kv_heads, c.head_dim), v=v.view(B, 1, c.kv_heads, c.head_dim),
                                        rotary_cos=self.cos, rotary_sin=self.sin, cache_seqlens=self.lens,
                                        block_table=self.block_table, causal=True, rotary_interleaved=False)
            return o.view(B, c.q_heads * c.head_dim)
        pos = self.lens.long()
        q = self._rope(q.view(B, c.q_heads, c.head_dim), pos)
        k = self._rope(k.view(B, c.kv_heads, c.head_dim), pos)
        v = v.view(B, c.kv_heads, c.head_dim)
        if self.attention == "flashinfer":
            page = self.block_table.gather(1, (pos // self.page)[:, None]).squeeze(1).long()
            slot = pos % self.page
            self.kv[li][page, 0, slot] = k
            self.kv[li][page, 1, slot] = v
            return self.fi_wrapper.run(q.contiguous(), self.kv[li]).view(B, c.q_heads * c.head_dim)
        ar = torch.arange(B, device=self.dev)
        self.kdense[li][ar, :, pos] = k
        self.vdense[li][ar, :, pos] = v
        mask = (torch.arange(self.max_len, device=self.dev)[None, :] <= pos[:, None])[:, None, None, :]
        o = F.scaled_dot_product_attention(q[:, :, None, :], self.kdense[li], self.vdense[li], attn_mask=mask, enable_gqa=True)
        return o.reshape(B, c.q_heads * c.head_dim)

    # ------------------------------------------------------------------ one decode step
    def _forward(self) -> None:
        c = self.cfg
        qd, kd = c.q_heads * c.head_dim, c.kv_heads * c.head_dim
        x = self.embed[self.ids]
        for li, L in enumerate(self.layers):
            h = F.rms_norm(x, (c.hidden,), L["ln1"], c.rms_eps)
            qkv = h @ L["qkv"]
            a = self._attend(li, qkv[:, :qd], qkv[:, qd:qd + kd], qkv[:, qd + kd:])
            x = torch.addmm(x, a, L["o"])
            h = F.rms_norm(x, (c.hidden,), L["ln2"], c.rms_eps)
            gu = h @ L["gate_up"]
            x = torch.addmm(x, F.silu(gu[:, :c.inter]) * gu[:, c.inter:], L["down"])
        h = F.rms_norm(x, (c.hidden,), self.norm, c.rms_eps)
        self.tokens.copy_(torch.argmax(h @ self.lm_head, dim=-1))

    def capture(self) -> None:
        self._plan(self.ctx)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self._forward()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._forward()

    def replay(self) -> None:
        self.graph.replay()

    def step(self, cur_len: int, ids_host: torch.Tensor) -> List[int]:
        """End-to-end step as a serving loop makes it: inputs from pinned host memory, the captured step, tokens back."""
        self.h_in[0].copy_(ids_host)
        self.h_in[1].fill_(cur_len)
        self._plan(cur_len)
        self.d_in.copy_(self.h_in, non_blocking=True)
        self.ids.copy_(self.d_in[0])
        self.lens.copy_(self.d_in[1])
        self.graph.replay()
        self.h_out.copy_(self.tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.h_out.tolist()


def run(model: str, batch: int, ctx: int, steps: int, warmup: int, device: torch.device, seed: int = 0,
        barrier=lambda: torch.cuda.synchronize()) -> dict:
    """Time `steps` decode steps: device-only (graph replays between CUDA events) and end to end.  Returns seconds."""
    dec = BaselineDecoder(model, batch, ctx, 2 * (warmup + steps) + 8, device, seed)
    dec.capture()
    vocab = dec.cfg.vocab
    ids = torch.randint(0, vocab, (batch,), dtype=torch.int64)
    cur = ctx
    for _ in range(warmup):
        ids = torch.tensor(dec.step(cur, ids), dtype=torch.int64) % vocab
        cur += 1
    barrier()
    import time
    t0 = time.perf_counter()
    for _ in range(steps):
        ids = torch.tensor(dec.step(cur, ids), dtype=torch.int64) % vocab
        cur += 1
    barrier()
    e2e_s = time.perf_counter() - t0
    dec.lens.fill_(ctx + warmup + steps)
    for _ in range(warmup):
        dec.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        dec.replay()
    e1.record()
    barrier()
    out = dict(dev_s=e0.elapsed_time(e1) * 1e-3, e2e_s=e2e_s, attention=dec.attention, page=getattr(dec, "page", 0),
               h2d_bytes_per_step=dec.h2d_bytes, d2h_bytes_per_step=dec.d2h_bytes)
    del dec
    torch.cuda.empty_cache()
    return out
