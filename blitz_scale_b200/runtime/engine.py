"""Per-GPU serving engine: weight segment + paged KV pool + batches + the fused forward.

This is the counterpart of the reference's engine facade (src/blitz/stub.h:68-291 constructor,
:1283-1364 `forward`): it owns the model memory, the page allocator and the cached batches, stages
the per-step page table through pinned memory, and runs prefill / decode steps.  Differences that
matter for speed: the decode step is replayed from a CUDA graph per padded batch size (the
reference relaunches ~9 kernels per layer per token on the default stream and synchronises after
every prefill layer, src/model/llama.h:345-355), attention needs no host-side plan, and there is
exactly one H2D copy (inputs + page table) and one D2H copy (sampled tokens) per step.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..models.config import ModelConfig, get_config
from ..models.llama import LlamaRunner, StepMeta, TPComm
from ..models.weights import WeightSegment
from ..utils.tracing import nvtx_range
from . import core

_BUCKETS = [1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512, 768, 1024]


def _bucket(n: int) -> int:
    for b in _BUCKETS:
        if n <= b:
            return b
    return n


class Engine:
    def __init__(self, model: str | ModelConfig, *, num_pages: int, page_size: int = 64, max_batch: int = 256,
                 max_batch_tokens: int = 8192, tp: int = 1, tp_rank: int = 0, dtype=torch.bfloat16,
                 device: Optional[torch.device] = None, comm: Optional[TPComm] = None, use_graphs: bool = True,
                 seg_buffer: Optional[torch.Tensor] = None, kv_buffer: Optional[torch.Tensor] = None,
                 ready: bool = True, seed: int = 0, fused_tp: bool = True, oneshot_max_rows: int = 1024,
                 tp_contexts: int = 1, use_switch: bool = True):
        self.cfg = get_config(model) if isinstance(model, str) else model
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.dtype, self.tp, self.tp_rank = dtype, tp, tp_rank
        self.page_size, self.num_pages = page_size, num_pages
        self.max_batch, self.max_batch_tokens = max_batch, max_batch_tokens
        c = self.cfg
        self.seg = WeightSegment(c, tp, tp_rank, dtype, device=self.device, buffer=seg_buffer)
        kvh = c.kv_heads // tp
        kv_shape = (c.layers, num_pages, 2, page_size, kvh, c.head_dim)
        if kv_buffer is None:
            # zero-filled: the attention kernels require finite values in every slot of an allocated page
            self.kv = torch.zeros(kv_shape, dtype=dtype, device=self.device)
        else:
            self.kv = kv_buffer.view(dtype)[:int(np.prod(kv_shape))].view(kv_shape)
        self.fused = None
        if tp > 1 and comm is not None and fused_tp:
            # tensor-parallel layers through the fused peer-memory kernels (GEMM -> reduce-scatter push, reduce + norm +
            # all-gather push, flag-gated GEMM); the NCCL all-reduce runner is the baseline (`fused_tp=False`)
            from ..parallel.tp import FusedTP, LlamaRunnerTP
            self.fused = FusedTP(comm.group, c.hidden, max(max_batch_tokens, max_batch), dtype=dtype,
                                 contexts=tp_contexts)
            self.runner = LlamaRunnerTP(self.seg, self.kv, max(max_batch_tokens, max_batch), max_batch, comm, self.fused,
                                        oneshot_max_rows=oneshot_max_rows)
            self.runner.use_switch = use_switch
        else:
            self.runner = LlamaRunner(self.seg, self.kv, max_tokens=max(max_batch_tokens, max_batch), max_batch=max_batch,
                                      comm=comm)
        self.pool = core.PagePool(num_pages, page_size)
        self.layout = core.MetaLayout.make(max(max_batch_tokens, max_batch), max_batch, num_pages)
        self.host = torch.zeros(self.layout.total, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.layout.total, dtype=torch.int32, device=self.device)
        self.tok_host = torch.zeros(max_batch, dtype=torch.int32, pin_memory=True)
        self.status = core.ModelStatus(c.layers)
        if ready:
            self.seg.random_init_fast_(seed)
            self.status.set_ready()
        self.batches: Dict[int, "core.Batch"] = {}
        self.use_graphs = use_graphs
        self._graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self.stream = torch.cuda.Stream(device=self.device)
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.launches_per_decode_step = 0

    # ------------------------------------------------------------------ meta views
    def _views(self, T: int, B: int, P: int, prefill: bool, seq_lens: Sequence[int] = (), splits: int = 1,
               kv_lens: Sequence[int] = (), work: Optional[torch.Tensor] = None) -> StepMeta:
        L, d = self.layout, self.dev
        kv_lens = list(kv_lens) if kv_lens else list(seq_lens)
        if prefill and work is None:
            work = ops.prefill_work_list(seq_lens, kv_lens, self.page_size, self.device)
        return StepMeta(kv_lens_host=kv_lens, prefill_work=work,
                        ids=d[L.ids:L.ids + T], pos=d[L.pos:L.pos + T], slot=d[L.slot:L.slot + T],
                        page_indices=d[L.page_indices:L.page_indices + max(P, 1)],
                        page_indptr=d[L.page_indptr:L.page_indptr + B + 1],
                        last_page_len=d[L.last_page_len:L.last_page_len + B],
                        tok_indptr=d[L.tok_indptr:L.tok_indptr + B + 1] if prefill else None,
                        seq_lens_host=list(seq_lens), is_prefill=prefill, batch=B, num_tokens=T, num_splits=splits)

    def _h2d(self, hi: int) -> None:
        self.dev[:hi].copy_(self.host[:hi], non_blocking=True)
        self.h2d_bytes = hi * 4

    def _tokens_to_host(self, toks: torch.Tensor, B: int) -> List[int]:
        self.tok_host[:B].copy_(toks[:B], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes = B * 4
        return self.tok_host[:B].tolist()

    # ------------------------------------------------------------------ batches
    def new_batch(self, batch_id: int, specs) -> Optional["core.Batch"]:
        b = core.Batch(batch_id, self.pool)
        if not b.add_prompts(specs):
            return None
        return b

    def choose_splits(self, B: int, max_len: int) -> int:
        ctas = B * (self.cfg.kv_heads // self.tp)
        if ctas >= 2 * 148 or max_len <= 256:
            return 1
        want = (2 * 148 + ctas - 1) // ctas
        cap = max(1, max_len // 256)
        s = 1
        while s * 2 <= min(want, cap, 32):
            s *= 2
        return s

    # ------------------------------------------------------------------ steps
    @torch.no_grad()
    def prefill(self, batch: "core.Batch", after_layer=None) -> List[int]:
        """Run the prompt of every request in `batch`, cache its K/V and return the first token of each.

        `after_layer(l)` is called when every K/V row of layer l is in the stream that runs the pass (in a prefill of
        several windows: during the last window), so that a caller can send the layer away while the next ones run."""
        if not self.status.fully_loaded():
            raise RuntimeError("model parameters are not loaded")
        if batch.size > self.max_batch:
            raise ValueError(f"prefill batch of {batch.size} sequences exceeds max_batch={self.max_batch}")
        if batch.num_prompt_tokens() > self.max_batch_tokens:
            toks = self._prefill_in_chunks(batch, after_layer)
            toks = self._sample_rows(batch, batch.size, toks)
            out = self._tokens_to_host(toks, batch.size)
            batch.mark_prefilled()
            batch.append_tokens(out, False)
            batch.decode = True
            return out
        T, P = batch.fill_prefill(self.host_np, self.layout)
        self._h2d(self.layout.page_indices + P)
        lens = batch.prompt_lens()
        m = self._views(T, batch.size, P, True, lens)
        with nvtx_range("prefill"):
            toks = self.runner.forward(m, after_layer=after_layer)
        toks = self._sample_rows(batch, batch.size, toks)
        out = self._tokens_to_host(toks, batch.size)
        batch.mark_prefilled()
        batch.append_tokens(out, False)
        batch.decode = True
        return out

    def _prefill_in_chunks(self, batch: "core.Batch", after_layer=None) -> torch.Tensor:
        """Prompts that together exceed `max_batch_tokens` (one prompt alone may): passes over windows of that many
        tokens of the prompts laid end to end.  A window's rows attend to the cache, which holds what earlier windows
        stored for the same sequence; the state of every sequence's last token is kept when its prompt ends, and the
        head runs once over all of them.  The reference stops packing at the token budget and cannot split a prompt
        (router_v2/src/queue.rs:279-286)."""
        total, B = batch.num_prompt_tokens(), batch.size
        runner = self.runner
        forced = getattr(runner, "force_switch", None)
        if forced is not None:
            runner.force_switch = True          # tensor parallel: keep the residual stream replicated in every pass
        try:
            states = torch.empty(B, self.cfg.hidden, dtype=self.dtype, device=self.device)
            tok0 = 0
            while tok0 < total:
                T, P, rows, s0, q_lens, kv_lens, ended = batch.fill_prefill_chunk(self.host_np, self.layout, tok0,
                                                                                  self.max_batch_tokens)
                self._h2d(self.layout.page_indices + P)
                m = self._views(T, rows, P, True, q_lens, kv_lens=kv_lens)
                with nvtx_range("prefill_chunk"):
                    runner.forward(m, with_head=False, after_layer=after_layer if tok0 + T >= total else None)
                    if any(ended):
                        last = runner.last_rows(m)
                        for r, e in enumerate(ended):
                            if e:
                                states[s0 + r].copy_(last[r])
                # the staging arrays are reused by the next window
                torch.cuda.current_stream().synchronize()
                tok0 += T
            return runner.head_from_rows(states)
        finally:
            if forced is not None:
                runner.force_switch = forced

    @torch.no_grad()
    def decode(self, batch: "core.Batch") -> List[int]:
        """One decode step for every request in `batch` (already extended if several were merged).  Requests that
        have already finished stay in their rows as padding (no cache write; their returned token is meaningless and
        is not recorded): callers normally filter them out between steps."""
        if not self.status.fully_loaded():
            raise RuntimeError("model parameters are not loaded")
        B = batch.size
        if B > self.max_batch:
            raise ValueError(f"decode batch of {B} sequences exceeds max_batch={self.max_batch}")
        Bp = _bucket(B) if self.use_graphs else B
        Bp = min(Bp, self.max_batch)
        splits = self.choose_splits(Bp, batch.max_seq_len())
        P = batch.fill_decode(self.host_np, self.layout, Bp)
        self._h2d(self.layout.page_indices + P)
        if self.use_graphs:
            key = (Bp, splits)
            g = self._graphs.get(key)
            if g is None:
                g = self._capture(Bp, splits)
            g.replay()
            toks = self.runner.tokens
        else:
            toks = self.runner.forward(self._views(Bp, Bp, self.num_pages, False, splits=splits))
        toks = self._sample_rows(batch, B, toks)
        out = self._tokens_to_host(toks, B)
        batch.append_tokens(out, True)
        return out

    def _sample_rows(self, batch: "core.Batch", B: int, toks: torch.Tensor) -> torch.Tensor:
        """Rows whose request asked for sampling (`do_sample` with temperature / top-k / top-p / seed) draw their token
        from this step's logits with the sampling kernel; all other rows keep the arg-max.  One extra small launch,
        outside the CUDA graph, and only when such a row exists.  With tp > 1 every rank holds a vocabulary shard of
        the logits; the shards of the sampled rows are gathered first (the reference serves greedily only)."""
        rows, temp, top_k, top_p, seeds = batch.sampling_rows()
        if not rows:
            return toks
        dev = self.device
        idx = torch.tensor(rows, dtype=torch.long, device=dev)
        logits = self.runner.logits[:B].index_select(0, idx)
        if self.tp > 1:
            # every rank holds a vocabulary shard of the rows: gather the shards of the (few) sampled rows, so that
            # every rank draws from the same full distribution with the same seed and gets the same token
            logits = self._gather_vocab_shards(logits)
        drawn = ops.sample(logits, torch.tensor(temp, dtype=torch.float32, device=dev),
                           torch.tensor(top_k, dtype=torch.int32, device=dev),
                           torch.tensor(top_p, dtype=torch.float32, device=dev),
                           torch.tensor(seeds, dtype=torch.int64, device=dev), 0)
        toks = toks[:B].clone()
        toks[idx] = drawn.to(toks.dtype)
        return toks

    def _gather_vocab_shards(self, shard_rows: torch.Tensor) -> torch.Tensor:
        """[n, vocab / tp] on every rank -> [n, vocab] on every rank, through the peer-memory all-gather of the fused
        runner (a few rows per call, bounded by its slot size) or the collective library of the comparison runner."""
        n, vs = shard_rows.shape
        if self.fused is None:
            full = self.runner.comm.all_gather(shard_rows)                       # [tp, n, vs]
            return full.permute(1, 0, 2).reshape(n, self.tp * vs).contiguous()
        per_call = max(1, self.fused.gather_bytes // (vs * shard_rows.element_size()))
        parts = []
        for r0 in range(0, n, per_call):
            g = self.fused.all_gather(shard_rows[r0:r0 + per_call])             # [tp, k, vs]
            parts.append(g.permute(1, 0, 2).reshape(g.shape[1], self.tp * vs))
        return torch.cat(parts, 0).contiguous()

    def _capture(self, Bp: int, splits: int) -> torch.cuda.CUDAGraph:
        m = self._views(Bp, Bp, self.num_pages, False, splits=splits)
        # warm up outside capture: first-use work (attribute setup, descriptor cache, workspace allocation)
        self.runner.forward(m)
        torch.cuda.current_stream().synchronize()
        g = torch.cuda.CUDAGraph()
        # thread-local capture: transfer and RPC threads of a worker keep making CUDA calls (small copies, flag reads)
        # on their own streams while this thread captures; under the default global mode those calls invalidate
        # the capture ("operation not permitted when stream is capturing")
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            self.runner.forward(m)
        self._graphs[(Bp, splits)] = g
        return g

    def precapture(self, max_batch: Optional[int] = None, contexts: Sequence[int] = (64, 1024, 4096, 16384)) -> int:
        """Capture the decode graphs of every batch bucket up to `max_batch` (default: the engine's) and of the
        split-KV choices that contexts of the given lengths select, so that no request pays for a capture later.
        The captures run on padded rows only (an empty batch): graph topology and buffer addresses do not depend
        on the parameters' values, so this also works on a replica whose parameters have not arrived.  With tp > 1
        every rank of the replica must call it (the captures contain the collectives).  Returns the number captured."""
        if not self.use_graphs:
            return 0
        limit = min(max_batch or self.max_batch, self.max_batch)
        empty = core.Batch((1 << 62), self.pool)
        n = 0
        for Bp in _BUCKETS:
            if Bp > limit:
                break
            for ctx in contexts:
                splits = self.choose_splits(Bp, ctx)
                if (Bp, splits) in self._graphs:
                    continue
                P = empty.fill_decode(self.host_np, self.layout, Bp)      # Bp padded rows: no page, no cache write
                self._h2d(self.layout.page_indices + P)
                self._capture(Bp, splits)
                n += 1
        torch.cuda.current_stream().synchronize()
        return n

    def release_graphs(self) -> None:
        """Drop every captured decode graph (first step of an orderly exit: the graphs hold kernel arguments that
        name peer memory and, with the NCCL runner, collectives of its communicator)."""
        self._graphs.clear()

    def close_regions(self) -> None:
        """Drop the symmetric regions this engine owns (the fused tensor-parallel state); see parallel/teardown.py."""
        if self.fused is not None:
            self.fused.close_regions()

    def decode_launch_count(self) -> int:
        """Kernels of this library launched by one decode step at tp = 1 (for the bench's launch accounting)."""
        per_layer = 8  # rms_norm, qkv gemm, rope_kv_store, attention, o gemm, rms_norm, gate_up gemm, down gemm
        return 1 + per_layer * self.cfg.layers + 3  # embedding + layers + final norm, lm_head gemm, argmax

    # ------------------------------------------------------------------ parameters
    def set_status_ready(self) -> None:
        self.status.set_ready()

    def reset_status(self) -> None:
        self.status.reset()

    def load_params_from_host(self, host_mirror: torch.Tensor, chunk_bytes: int = 256 << 20) -> float:
        """Chunked H2D of a pinned host mirror on two streams; returns seconds."""
        n = self.seg.layout.total_bytes
        assert host_mirror.numel() >= n and host_mirror.dtype == torch.uint8
        t0 = time.perf_counter()
        streams = [torch.cuda.Stream(device=self.device) for _ in range(2)]
        for i, off in enumerate(range(0, n, chunk_bytes)):
            hi = min(n, off + chunk_bytes)
            with torch.cuda.stream(streams[i % 2]):
                self.seg.buffer[off:hi].copy_(host_mirror[off:hi], non_blocking=True)
        for s in streams:
            s.synchronize()
        self.status.set_ready()
        return time.perf_counter() - t0

    def load_params_from_disk(self, directory, host_mirror: Optional[torch.Tensor] = None) -> dict:
        """Disk -> pinned host (O_DIRECT, threaded) -> device.  Returns timings."""
        path = WeightSegment.check_sidecar(directory, self.cfg, self.tp, self.tp_rank, self.dtype)
        n = self.seg.layout.total_bytes
        if host_mirror is None:
            host_mirror = torch.empty(n, dtype=torch.uint8, pin_memory=True)
        res = core.load_file_to_host(str(path), host_mirror.data_ptr(), n)
        h2d = self.load_params_from_host(host_mirror)
        return {"disk_s": res.seconds, "h2d_s": h2d, "bytes": n, "direct_io": res.direct_io, "host_mirror": host_mirror}
