"""Fused tensor-parallel layer path: GEMM -> reduce-scatter and all-gather -> GEMM over peer memory.

`FusedTP` owns the symmetric buffers of one replica's TP group (two staging areas for the partial
results of the row-parallel GEMMs, two gathered-activation buffers, the flag words, and a slot area
for the one-shot all-reduce of the vocab-sharded embedding) and exposes the three launches of the
data flow described in csrc/comm/tp_fused.cu:

    gemm_rs(a, w, which)                      tcgen05 GEMM whose epilogue pushes partial rows to their owner rank
    reduce_norm(which, residual, w, which_x)  owner sums partials + residual, RMSNorm, pushes rows to every rank
    ag_gemm(which_x, w, ...)                  tcgen05 GEMM whose TMA producer waits for the gathered rows

`LlamaRunnerTP` runs the Llama forward with those launches: the residual stream is sharded by rows
between the row-parallel and column-parallel GEMMs (Megatron-style sequence parallelism falls out of
the push model), and no collective library is called in the layer loop.  It replaces the
AllReduce-after-GEMM structure of src/layer/attn.h:217-233 and src/layer/glu.h:138-154; the NCCL
version of the same forward (`LlamaRunner` with `TPComm`) is kept as the comparison baseline.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import ops
from ..models.llama import LlamaRunner, StepMeta, TPComm
from ..ops import _lib as _L
from ..ops import _check, _dt, _p, _stream, gemm_workspace, status_word
from .symm import SymmRegion


class _GemmTp(ctypes.Structure):
    _fields_ = [("push_base", ctypes.c_void_p * 8), ("push_flags", ctypes.c_void_p * 8), ("tp", ctypes.c_int),
                ("tp_rank", ctypes.c_int), ("rows_per_rank", ctypes.c_int), ("wait_flags", ctypes.c_void_p),
                ("n_wait", ctypes.c_int), ("wait_value", ctypes.c_uint32)]


_EPI = {"store": 0, "add": 1, "silu_mul": 2, "push": 3}


class FusedTP:
    LANES = 2
    FLAG_WORDS = 128  # rs0: 0..15, rs1: 16..31, ag0: 32..39, ag1: 40..47, one-shot all-reduce: 48..56 and 64..72

    def __init__(self, group, hidden: int, max_rows: int, dtype=torch.bfloat16, device=None, contexts: int = 1,
                 gather_bytes: int = 1 << 20):
        import torch.distributed as dist
        self.group = group
        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.hidden, self.dtype = hidden, dtype
        self.max_rows = (max_rows + self.tp * 8 - 1) // (self.tp * 8) * (self.tp * 8)
        self.elem = 2
        self.buf_bytes = self.max_rows * hidden * self.elem
        # layout of the symmetric region
        self.o_stage = [0, self.buf_bytes]
        self.o_xg = [2 * self.buf_bytes, 3 * self.buf_bytes]
        self.o_emb = 4 * self.buf_bytes                       # one-shot all-reduce slots: [parity 2][tp][max_rows * hidden]
        self.o_flags = self.o_emb + 2 * self.tp * self.buf_bytes
        self._ar_parity = 0
        self.fused_allreduce = True                           # one-kernel all-reduce (per-block rendezvous)
        self.o_cflags = self.o_flags + self.FLAG_WORDS * 4    # per-block counters of it: [parity 2][tp 8][64 blocks]
        # switch-reduced path (all-reduce + add + RMSNorm in one kernel): partial results [lane][parity], and `contexts`
        # copies of the replicated residual stream and of the normalised activations (one per interleaved task).
        # A lane is an independent sequence of calls with its own partial buffers, counters and parity: lane 0 is the
        # ordinary forward pass (parity restarts with every pass, which is what a captured graph bakes in), lane 1 is
        # live execution, whose steps of several tasks interleave and whose parity therefore just keeps alternating.
        self.contexts = contexts
        L2 = 2 * self.LANES
        o = self.o_cflags + 2 * 8 * 64 * 4
        self.o_in = [o + i * self.buf_bytes for i in range(L2)]            # index lane * 2 + parity
        self.o_res = o + L2 * self.buf_bytes
        self.o_xn = self.o_res + contexts * self.buf_bytes
        self.o_nflags = self.o_xn + contexts * self.buf_bytes  # [lane][parity][32 words]: ready[8] | done[8] | ticket
        self.gather_bytes = gather_bytes                       # per rank and call of the small all-gather
        self.o_gather = self.o_nflags + L2 * 32 * 4            # [lane][parity][tp][gather_bytes]
        self.o_gflags = self.o_gather + L2 * self.tp * gather_bytes  # [lane][parity][16 words]
        # reduce-scatter arrival counters of the two staging areas: [64 blocks of 128 rows][8 sources] + a ticket word
        self.RS_FLAG_WORDS = 64 * 8 + 8
        self.o_rsflags = self.o_gflags + L2 * 16 * 4
        total = self.o_rsflags + 2 * self.RS_FLAG_WORDS * 4
        self._in_parity = [0] * self.LANES
        self._g_parity = [0] * self.LANES
        self.lane = 0
        self.ctx = 0
        self.region = SymmRegion(total, group, device)
        self.region.local[self.o_flags:].zero_()
        torch.cuda.synchronize()
        self.region.barrier()
        self.ptrs = self.region.ptrs
        self.device = self.region.local.device
        self.budget_ns = int(2e9)
        # the switch-reduced kernels need the region's multicast address (NVLS); without it the push kernels serve
        self.has_mc = bool(self.region.mc_ptr) and hidden <= 8192

    def close_regions(self) -> None:
        self.region.close_regions()

    # ------------------------------------------------------------------ views / pointers
    def xg(self, which: int, rows: int) -> torch.Tensor:
        off = self.o_xg[which]
        return self.region.local[off:off + rows * self.hidden * self.elem].view(self.dtype).view(rows, self.hidden)

    def _flag_ptr(self, rank: int, word: int) -> int:
        return self.ptrs[rank] + self.o_flags + word * 4

    def _rs_flag_ptr(self, rank: int, which: int) -> int:
        return self.ptrs[rank] + self.o_rsflags + which * self.RS_FLAG_WORDS * 4

    def _tp_struct(self) -> _GemmTp:
        s = _GemmTp()
        s.tp, s.tp_rank = self.tp, self.rank
        return s

    def _gemm(self, a, w, out, epi, tp_struct, residual=None, N=None):
        M, K = a.shape
        bcols = w.shape[1]
        n_out = bcols // 2 if epi == 2 else bcols
        ws, tickets = gemm_workspace(a.device)
        rc = _L.lib().blitz_gemm_tp(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0) if out is not None else n_out,
                                    _p(residual), M, n_out, K, 0, epi, n_out if epi == 2 else 0, _dt(a), 0, 0,
                                    _p(ws), ws.numel(), _p(tickets), tickets.numel(), _p(status_word(a.device)),
                                    ctypes.byref(tp_struct), _stream())
        _check(rc, "blitz_gemm_tp")

    # ------------------------------------------------------------------ the three launches
    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, which: int) -> int:
        """Partial result of a row-parallel GEMM pushed to the owners' staging area `which`.  a: [M, K_local] with
        M a multiple of tp.  Returns the number of tiles per 128 rows that every source pushes (what `reduce_norm`
        waits for, block of rows by block of rows)."""
        M = a.shape[0]
        assert M % self.tp == 0 and M <= self.max_rows
        rpr = M // self.tp
        s = self._tp_struct()
        s.rows_per_rank = rpr
        for r in range(self.tp):
            s.push_base[r] = self.ptrs[r] + self.o_stage[which]
            s.push_flags[r] = self._rs_flag_ptr(r, which)
        self._gemm(a, w, None, 3, s)
        bn = int(_L.lib().blitz_gemm_tile_n(M, w.shape[1], 3, 0))
        return (w.shape[1] + bn - 1) // bn

    def reduce_norm(self, which: int, tiles_n: int, rows_per_rank: int, residual: Optional[torch.Tensor],
                    norm_w: torch.Tensor, which_x: int, eps: float) -> None:
        """Owner side: sum the partials of staging area `which` (+ residual shard, updated in place), RMSNorm, push the
        normalised rows into gathered buffer `which_x` of every rank.  A row is processed as soon as the tiles of its
        own block of 128 rows have arrived from every source (`tiles_n` each, from `gemm_rs`)."""
        xg = (ctypes.c_void_p * self.tp)(*[self.ptrs[r] + self.o_xg[which_x] for r in range(self.tp)])
        fl = (ctypes.c_void_p * self.tp)(*[self._flag_ptr(r, 32 + 8 * which_x) for r in range(self.tp)])
        rc = _L.lib().blitz_rs_reduce_norm(
            ctypes.c_void_p(self.ptrs[self.rank] + self.o_stage[which]), ctypes.c_void_p(self._rs_flag_ptr(self.rank, which)),
            tiles_n, _p(residual), _p(norm_w), xg, fl, self.tp, self.rank, rows_per_rank, rows_per_rank,
            rows_per_rank * self.tp, self.hidden, eps, self.budget_ns, _p(status_word(self.device)), 1 if self.dtype == torch.bfloat16 else 0, _stream())
        _check(rc, "blitz_rs_reduce_norm")

    def ag_gemm(self, which_x: int, rows: int, w: torch.Tensor, out: torch.Tensor, epilogue: str = "store",
                wait: bool = True) -> torch.Tensor:
        """Column-parallel GEMM on the gathered activations; waits in-kernel for every source's rows, then re-arms the flags."""
        a = self.xg(which_x, rows)
        s = self._tp_struct()
        s.rows_per_rank = rows
        if wait:
            s.wait_flags = self._flag_ptr(self.rank, 32 + 8 * which_x)
            s.n_wait = self.tp
            s.wait_value = rows // self.tp
        self._gemm(a, w, out, _EPI[epilogue], s)
        if wait:
            _check(_L.lib().blitz_flags_zero(ctypes.c_void_p(self._flag_ptr(self.rank, 32 + 8 * which_x)), self.tp, _stream()),
                   "blitz_flags_zero")
        return out

    def wait_gathered(self, which_x: int, rows: int) -> None:
        """Stream-ordered wait for gathered buffer `which_x` (for consumers that are not GEMMs), then re-arm."""
        for sidx in range(self.tp):
            _check(_L.lib().blitz_flag_wait(ctypes.c_void_p(self._flag_ptr(self.rank, 32 + 8 * which_x + sidx)),
                                            rows // self.tp, self.budget_ns, _p(status_word(self.device)), _stream()),
                   "blitz_flag_wait")
        _check(_L.lib().blitz_flags_zero(ctypes.c_void_p(self._flag_ptr(self.rank, 32 + 8 * which_x)), self.tp, _stream()),
               "blitz_flags_zero")

    def reset_allreduce_parity(self) -> None:
        """Call at the same point of the program on every rank (the runner does it at the start of a forward)."""
        if self.lane == 0:
            self._ar_parity = 0
            self._in_parity[0] = 0
            self._g_parity[0] = 0

    # ------------------------------------------------------------------ switch-reduced path
    def use_context(self, i: int) -> None:
        """Select which copy of (residual stream, normalised activations) the next calls work on; interleaved
        live-execution tasks each keep their own.  Every rank of the group must select the same one."""
        assert 0 <= i < self.contexts
        self.ctx = i

    def use_lane(self, i: int) -> None:
        """Select the call sequence (partial buffers, counters, parity) the next calls belong to.  Every rank of the
        group must make the same calls in the same order within a lane; the lanes are independent of each other."""
        assert 0 <= i < self.LANES
        self.lane = i

    def next_partial(self, rows: int) -> torch.Tensor:
        """Buffer for the next row-parallel GEMM's partial result (alternates between two, like the counters)."""
        off = self.o_in[self.lane * 2 + self._in_parity[self.lane]]
        return self.region.local[off:off + rows * self.hidden * self.elem].view(self.dtype).view(rows, self.hidden)

    def res(self, rows: int) -> torch.Tensor:
        off = self.o_res + self.ctx * self.buf_bytes
        return self.region.local[off:off + rows * self.hidden * self.elem].view(self.dtype).view(rows, self.hidden)

    def xn(self, rows: int) -> torch.Tensor:
        off = self.o_xn + self.ctx * self.buf_bytes
        return self.region.local[off:off + rows * self.hidden * self.elem].view(self.dtype).view(rows, self.hidden)

    def ar_add_norm(self, rows: int, norm_w: torch.Tensor, eps: float, add_residual: bool = True) -> None:
        """residual (+)= sum over ranks of the partial written to `next_partial`; normalised rows = RMSNorm(residual) * w.
        One kernel: the switch sums the partials (multimem.ld_reduce), every rank finalises its share of the rows and
        writes them into every rank's copies (multimem.st).  Both results are valid on every rank afterwards."""
        assert self.has_mc and rows <= self.max_rows
        par = self.lane * 2 + self._in_parity[self.lane]
        self._in_parity[self.lane] ^= 1
        mc = self.region.mc_ptr
        fl = (ctypes.c_void_p * self.tp)(*[self.ptrs[r] + self.o_nflags + par * 32 * 4 for r in range(self.tp)])
        res_off = self.o_res + self.ctx * self.buf_bytes
        rc = _L.lib().blitz_ar_add_norm_mm(
            ctypes.c_void_p(mc + self.o_in[par]),
            ctypes.c_void_p(self.ptrs[self.rank] + res_off if add_residual else 0),
            ctypes.c_void_p(mc + res_off), ctypes.c_void_p(mc + self.o_xn + self.ctx * self.buf_bytes), _p(norm_w), fl,
            self.tp, self.rank, rows, self.hidden, eps, self.budget_ns, _p(status_word(self.device)),
            1 if self.dtype == torch.bfloat16 else 0, _stream())
        _check(rc, "blitz_ar_add_norm_mm")

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[tp, *t.shape] with every rank's `t`, exchanged by peer stores (no collective library): for the (value,
        index) pairs of the sharded arg-max and the logit rows of sampled requests."""
        t = t.contiguous()
        nbytes = (t.numel() * t.element_size() + 15) // 16 * 16
        assert nbytes <= self.gather_bytes, "piece too large for the small all-gather"
        par = self.lane * 2 + self._g_parity[self.lane]
        self._g_parity[self.lane] ^= 1
        base = self.o_gather + par * self.tp * self.gather_bytes
        src = t
        if t.numel() * t.element_size() != nbytes:          # pad to whole 16-byte vectors
            src = torch.zeros(nbytes, dtype=torch.uint8, device=t.device)
            src[:t.numel() * t.element_size()].copy_(t.view(torch.uint8).view(-1))
        slots = (ctypes.c_void_p * self.tp)(*[self.ptrs[r] + base for r in range(self.tp)])
        fl = (ctypes.c_void_p * self.tp)(*[self.ptrs[r] + self.o_gflags + par * 16 * 4 for r in range(self.tp)])
        rc = _L.lib().blitz_peer_allgather(_p(src), slots, fl, self.tp, self.rank, nbytes, self.budget_ns,
                                           _p(status_word(self.device)), _stream())
        _check(rc, "blitz_peer_allgather")
        # the slots of this parity are rewritten two calls later: hand out a copy
        out = torch.empty((self.tp,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        raw = self.region.local[base:base + self.tp * nbytes].view(self.tp, nbytes)      # the kernel packs slots by nbytes
        out.view(self.tp, -1).view(torch.uint8).copy_(raw[:, :t.numel() * t.element_size()])
        return out

    def allreduce_oneshot(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out = sum over ranks of x (out may be x).  Every rank stores its contribution into every rank's slot and
        sums the tp slots in rank order.  Consecutive calls alternate between two slot / counter sets, so a rank
        that runs one call ahead never overwrites data its peer is still summing."""
        n = x.numel()
        assert n * self.elem <= self.buf_bytes and x.is_contiguous()
        par = self._ar_parity
        self._ar_parity ^= 1
        base = self.o_emb + par * self.tp * self.buf_bytes
        slots = (ctypes.c_void_p * self.tp)(*[self.ptrs[r] + base for r in range(self.tp)])
        if self.fused_allreduce:
            cf = (ctypes.c_void_p * self.tp)(*[self.ptrs[r] + self.o_cflags + par * 8 * 64 * 4 for r in range(self.tp)])
            rc = _L.lib().blitz_allreduce_fused(_p(x), slots, cf, _p(out), self.tp, self.rank, n, self.budget_ns,
                                                _p(status_word(self.device)), 1 if self.dtype == torch.bfloat16 else 0,
                                                _stream())
            _check(rc, "blitz_allreduce_fused")
            return out
        fl = (ctypes.c_void_p * self.tp)(*[self._flag_ptr(r, 48 + 16 * par) for r in range(self.tp)])
        rc = _L.lib().blitz_allreduce_oneshot(_p(x), slots, fl, _p(out), self.tp, self.rank, n, self.budget_ns,
                                              _p(status_word(self.device)), 1 if self.dtype == torch.bfloat16 else 0, _stream())
        _check(rc, "blitz_allreduce_oneshot")
        return out


class _PeerAllReduce:
    """The collective interface of `TPComm` on the peer-memory kernels: one-shot all-reduce and small all-gather."""

    def __init__(self, comm: TPComm, fused: FusedTP):
        self.comm, self.fused = comm, fused
        self.size, self.rank, self.group = comm.size, comm.rank, comm.group

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        return self.fused.allreduce_oneshot(t, t)

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        return self.fused.all_gather(t)


class LlamaRunnerTP(LlamaRunner):
    """Llama forward on one TP rank with the fused peer-memory path (no collective library in the layer loop)."""

    def __init__(self, seg, kv_cache, max_tokens, max_batch, comm: TPComm, fused: FusedTP, oneshot_max_rows: int = 0):
        super().__init__(seg, kv_cache, max_tokens, max_batch, comm=comm)
        self.fused = fused
        # Steps of at most this many rows skip the reduce-scatter / all-gather split: every partial sum goes through
        # the one-shot peer-memory all-reduce (each rank pushes its partial rows into every rank's slot and sums),
        # which is one hop instead of two dependent ones; the row-sharded pipeline wins once rows are many.
        self.oneshot_max_rows = oneshot_max_rows
        self._nccl_comm = comm
        self._peer_comm = _PeerAllReduce(comm, fused)
        self.use_switch = True
        self.force_switch = False     # live execution: every step takes the switch-reduced path, whatever its size
        # Where the fabric reduces in the switch, passes of any size take that path: the row-parallel GEMMs then run
        # at their plain speed and one kernel does all-reduce + add + norm.  Measured at 8192 rows (Mistral-24B shape,
        # two ranks): 183.8 ms per prefill pass against 211.1 ms for the row-sharded pipeline, whose GEMM with the
        # push epilogue runs at half the speed of the plain one, and 183.9 ms for the NCCL runner.  The row-sharded
        # pipeline serves fabrics without in-switch reduction.
        self.switch_all = True
        self.res_shard = torch.empty(fused.max_rows // fused.tp, self.cfg.hidden, dtype=seg.dtype, device=self.res.device)
        self._pad_ids = torch.zeros(fused.max_rows, dtype=torch.int32, device=self.res.device)

    def _rows(self, m: StepMeta):
        tp = self.fused.tp
        Tp = (m.num_tokens + tp - 1) // tp * tp
        return Tp, Tp // tp

    def _small(self, m: StepMeta) -> bool:
        return m.num_tokens <= self.oneshot_max_rows

    def _switch(self, m: StepMeta) -> bool:
        """Steps of a few hundred rows on a fabric with in-switch reduction: all-reduce, residual add and RMSNorm are
        one kernel (`FusedTP.ar_add_norm`), the residual stream and the normalised rows live in symmetric memory."""
        return (self._small(m) or self.force_switch or self.switch_all) and self.fused.has_mc and self.use_switch

    def load_residual(self, T: int, src: torch.Tensor, layer: int) -> None:
        """Continue a batch whose first `layer` layers ran elsewhere: `src` [T, hidden] is the residual stream after
        them (every shard holds all rows on the switch-reduced path).  The normalised rows that layer `layer` reads are
        rebuilt from it here."""
        f, c = self.fused, self.cfg
        f.reset_allreduce_parity()
        self.comm = self._peer_comm
        f.res(T).copy_(src[:T])
        nw = self._w(layer, "input_ln") if layer < c.layers else self.seg["final_norm"]
        ops.rms_norm(f.res(T), nw, c.rms_eps, out=f.xn(T))

    def embed(self, m: StepMeta) -> None:
        self.fused.reset_allreduce_parity()
        self.comm = self._peer_comm
        if self._switch(m):
            T, f = m.num_tokens, self.fused
            vs = self.cfg.vocab // self.tp
            ops.embedding(m.ids[:T], self.seg["embed"], f.next_partial(T), vocab_start=self.seg.tp_rank * vs,
                          zero_missing=True)
            f.ar_add_norm(T, self._w(0, "input_ln"), self.cfg.rms_eps, add_residual=False)
            return
        if self._small(m):
            return LlamaRunner.embed(self, m)
        self.comm = self._nccl_comm
        T = m.num_tokens
        Tp, rpr = self._rows(m)
        vs = self.cfg.vocab // self.tp
        self._pad_ids[:Tp].zero_()
        self._pad_ids[:T].copy_(m.ids[:T])
        ops.embedding(self._pad_ids[:Tp], self.seg["embed"], self.tmp[:Tp], vocab_start=self.seg.tp_rank * vs,
                      zero_missing=True)
        self.fused.allreduce_oneshot(self.tmp[:Tp], self.res[:Tp])
        r = self.fused.rank
        self.res_shard[:rpr].copy_(self.res[r * rpr:(r + 1) * rpr])
        # first layer's input norm: every rank has the full rows, no exchange needed
        ops.rms_norm(self.res[:Tp], self._w(0, "input_ln"), self.cfg.rms_eps, out=self.fused.xg(0, Tp))
        self._first = True

    def attention_block(self, l: int, m: StepMeta) -> None:
        if self._switch(m):
            T, c, f = m.num_tokens, self.cfg, self.fused
            ops.gemm(f.xn(T), self._w(l, "qkv"), static_b=True, out=self.qkv[:T])
            ops.rope_kv_store(self.qkv[:T], m.pos[:T], m.slot[:T], self.kv[l], q_heads=self.qh, kv_heads=self.kvh,
                              head_dim=self.hd, page_size=self.page_size, rope_theta=c.rope_theta)
            if m.is_prefill:
                self._prefill_attention(l, m)
            else:
                ops.attn_decode(self.qkv[:T], self.kv[l], m.page_indices, m.page_indptr, m.last_page_len,
                                q_heads=self.qh, kv_heads=self.kvh, head_dim=self.hd, page_size=self.page_size,
                                num_splits=m.num_splits, workspace=self._workspace(m.batch, m.num_splits),
                                out=self.attn[:T])
            ops.gemm(self.attn[:T], self._w(l, "o"), static_b=True, out=f.next_partial(T))
            f.ar_add_norm(T, self._w(l, "post_ln"), c.rms_eps)
            return
        if self._small(m):
            return LlamaRunner.attention_block(self, l, m)
        T, c, f = m.num_tokens, self.cfg, self.fused
        Tp, rpr = self._rows(m)
        f.ag_gemm(0, Tp, self._w(l, "qkv"), self.qkv[:Tp], wait=not self._first)
        self._first = False
        ops.rope_kv_store(self.qkv[:T], m.pos[:T], m.slot[:T], self.kv[l], q_heads=self.qh, kv_heads=self.kvh,
                          head_dim=self.hd, page_size=self.page_size, rope_theta=c.rope_theta)
        if m.is_prefill:
            self._prefill_attention(l, m)
        else:
            ops.attn_decode(self.qkv[:T], self.kv[l], m.page_indices, m.page_indptr, m.last_page_len,
                            q_heads=self.qh, kv_heads=self.kvh, head_dim=self.hd, page_size=self.page_size,
                            num_splits=m.num_splits, workspace=self._workspace(m.batch, m.num_splits), out=self.attn[:T])
        if Tp > T:
            self.attn[T:Tp].zero_()
        exp = f.gemm_rs(self.attn[:Tp], self._w(l, "o"), 0)
        f.reduce_norm(0, exp, rpr, self.res_shard, self._w(l, "post_ln"), 1, c.rms_eps)

    def ffn_block(self, l: int, m: StepMeta) -> None:
        if self._switch(m):
            T, c, f = m.num_tokens, self.cfg, self.fused
            ops.gemm(f.xn(T), self._w(l, "gate_up"), static_b=True, out=self.act[:T], epilogue="silu_mul")
            ops.gemm(self.act[:T], self._w(l, "down"), static_b=True, out=f.next_partial(T))
            nw = self._w(l + 1, "input_ln") if l + 1 < c.layers else self.seg["final_norm"]
            f.ar_add_norm(T, nw, c.rms_eps)       # the normalised rows are the next layer's (or the head's) input
            return
        if self._small(m):
            return LlamaRunner.ffn_block(self, l, m)
        c, f = self.cfg, self.fused
        Tp, rpr = self._rows(m)
        f.ag_gemm(1, Tp, self._w(l, "gate_up"), self.act[:Tp], epilogue="silu_mul")
        exp = f.gemm_rs(self.act[:Tp], self._w(l, "down"), 1)
        nw = self._w(l + 1, "input_ln") if l + 1 < c.layers else self.seg["final_norm"]
        f.reduce_norm(1, exp, rpr, self.res_shard, nw, 0, c.rms_eps)

    def head(self, m: StepMeta) -> torch.Tensor:
        if self._switch(m):
            B, T, c, f = m.batch, m.num_tokens, self.cfg, self.fused
            xn = f.xn(T)                           # already normalised with the final norm's weight
            if m.is_prefill:
                ops.gather_last(xn, m.tok_indptr, out=self.last[:B])
                src = self.last[:B]
            else:
                src = xn[:B]
            ops.gemm(src, self.seg["lm_head"], static_b=True, out=self.logits[:B])
            return self._pick_tokens(B)
        if self._small(m):
            return LlamaRunner.head(self, m)
        B, T, c, f = m.batch, m.num_tokens, self.cfg, self.fused
        Tp, _ = self._rows(m)
        f.wait_gathered(0, Tp)     # final-norm rows of every rank are in gathered buffer 0
        xn = f.xg(0, Tp)
        if m.is_prefill:
            ops.gather_last(xn[:T], m.tok_indptr, out=self.last[:B])
            src = self.last[:B]
        else:
            src = xn[:B]
        ops.gemm(src, self.seg["lm_head"], static_b=True, out=self.logits[:B])
        return self._pick_tokens(B)

    def last_rows(self, m: StepMeta) -> torch.Tensor:
        if not self._switch(m):
            raise NotImplementedError("a prompt prefetched in chunks runs on the switch-reduced path at tp > 1")
        # already normalised with the final norm's weight (see ffn_block)
        ops.gather_last(self.fused.xn(m.num_tokens), m.tok_indptr, out=self.last[:m.batch])
        return self.last[:m.batch]

    def head_from_rows(self, rows: torch.Tensor) -> torch.Tensor:
        B = rows.shape[0]
        self.fused.xn(B).copy_(rows)
        saved, self.force_switch = self.force_switch, True
        try:
            return self.head(StepMeta(ids=None, pos=None, slot=None, page_indices=None, page_indptr=None,
                                      last_page_len=None, is_prefill=False, batch=B, num_tokens=B))
        finally:
            self.force_switch = saved

    def _pick_tokens(self, B: int) -> torch.Tensor:
        """Arg-max over the vocabulary shards: every rank's (value, index) candidates travel by peer stores."""
        vs = self.cfg.vocab // self.tp
        ops.argmax(self.logits[:B], out=self.tokens[:B], out_val=self.maxval[:B], idx_offset=self.seg.tp_rank * vs)
        pair = torch.stack([self.maxval[:B], self.tokens[:B].view(torch.float32)], dim=1)      # [B, 2] x 4 bytes
        both = self.fused.all_gather(pair)                                                     # [tp, B, 2]
        best = both[:, :, 0].argmax(0, keepdim=True)
        self.tokens[:B].copy_(both[:, :, 1].view(torch.int32).gather(0, best)[0])
        return self.tokens[:B]
