"""GPU worker backend: the engine plus the peer-memory data paths behind the RPC surface.

One instance per process / GPU.  Counterpart of the reference's engine facade and managers
(src/blitz/stub.h:68-1604, migration_manager.h, activation_manager.h, zigzag_manager.h,
nccl_bcastor.h), with every inter-GPU transfer done by this GPU's own kernels over symmetric
memory (`parallel/symm.py`) instead of RDMA / NCCL calls:

* parameters: a source streams `embed | layer i | head` units into the destinations' weight
  segments and bumps per-unit flags; a destination only polls its flag pad and marks units
  ready in order, so it can serve layers as they land (live execution);
* KV migration: `Immigrate` reserves pages on the decode GPU and publishes their ids in its
  control region; `Migrate` on the prefill GPU waits for that, then stores the prompt pages
  straight into the decode GPU's paged pool (all layers, or the first k / the remaining ones);
* live execution: ZagPrefill tasks run layer by layer under the native scheduler; `Relay` ships the
  residual stream of the head task into the old instance's mailbox slot, which continues from
  that layer inside `PrefillV2(NAIVE_PP | IMMIGRATE)`.
"""
from __future__ import annotations

import logging
import threading
import time
from concurrent.futures import Future
from typing import Dict, List, Optional

import torch

from .. import ops
from ..models.config import get_config
from ..models.llama import TPComm
from ..models.weights import WeightSegment
from ..parallel import symm
from ..parallel.agreement import LoadAgreement, StepLog
from ..pb.schema import pb
from ..runtime import core
from ..runtime.engine import Engine
from .service import Backend, seq_spec_from_request
from .stopping import StopSequences

CTL_SLOT_WORDS = 16384  # page ids one transfer slot can publish
log = logging.getLogger("blitz.worker")


class GpuBackend(Backend):
    def __init__(self, rank: int, world: int, model: str, *, tp: int = 1, num_pages: int = 2048, page_size: int = 64,
                 max_batch: int = 256, max_batch_tokens: int = 8192, ready: bool = True, use_fabric: bool = True,
                 tp_group=None, model_path: str = "", seed: int = 0, use_multimem: bool = False, copy_ctas: int = 128,
                 fused_tp: bool = True, precapture: bool = False, eos_token: Optional[int] = None,
                 tokenizer_path: str = ""):
        self.rank, self.world, self.tp = rank, world, tp
        self.cfg = get_config(model)
        self.eos_token = self.cfg.eos_token if eos_token is None else int(eos_token)
        self.stopper = StopSequences.from_tokenizer_file(tokenizer_path)
        self.model, self.model_path = model, model_path
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.lock = threading.RLock()
        self.use_multimem, self.copy_ctas = use_multimem, copy_ctas
        dt = torch.bfloat16
        probe = WeightSegment(self.cfg, tp, rank % tp, dt, device="meta")
        kvh = self.cfg.kv_heads // tp
        self.page_bytes = 2 * page_size * kvh * self.cfg.head_dim * 2
        self.kv_layer_stride = num_pages * self.page_bytes
        kv_bytes = self.cfg.layers * self.kv_layer_stride
        self.slot_bytes = max_batch_tokens * self.cfg.hidden * 2
        self.fabric: Optional[symm.PeerFabric] = None
        seg_buf = kv_buf = None
        self.multimem_min_dests = 2       # fewer destinations than this: plain peer stores are faster
        if use_fabric and world > 1:
            column = None
            if tp > 1:
                import torch.distributed as dist
                # one group per shard index (every rank creates all of them, in the same order): parameters of shard
                # t only ever move between the ranks t, t + tp, t + 2 tp, ...
                for t in range(tp):
                    g_ = dist.new_group([r for r in range(world) if r % tp == t])
                    if rank % tp == t:
                        column = g_
            self.fabric = symm.PeerFabric(symm.FabricSizes(weight_bytes=probe.layout.total_bytes, kv_bytes=kv_bytes,
                                                           mailbox_slots=4, mailbox_slot_bytes=self.slot_bytes),
                                          weight_group=column)
            seg_buf, kv_buf = self.fabric.weights.local, self.fabric.kv.local
            self.ctl = symm.SymmRegion(symm.KV_SLOTS * CTL_SLOT_WORDS * 4 + symm.KV_SLOTS * 4)  # id lists, then tags
            self.ctl.local.zero_()
        comm = TPComm(tp_group) if tp > 1 else None
        self.engine = Engine(self.cfg, num_pages=num_pages, page_size=page_size, max_batch=max_batch,
                             max_batch_tokens=max_batch_tokens, tp=tp, tp_rank=rank % tp, dtype=dt, comm=comm,
                             seg_buffer=seg_buf, kv_buffer=kv_buf, ready=ready, seed=seed, fused_tp=fused_tp,
                             tp_contexts=5 if tp > 1 else 1)     # context 0 + one per live-execution slot
        self.units = [(n, o, b) for n, o, b in self.engine.seg.layout.units]
        if precapture:
            # every decode graph is captured now, whether or not the parameters are here yet, so that neither a
            # running replica nor one that has just been scaled out stops to capture when a new batch size shows up
            t0 = time.perf_counter()
            n = self.engine.precapture()
            log.info("captured %d decode graphs in %.2f s", n, time.perf_counter() - t0)
        self.batches: Dict[int, "core.Batch"] = {}
        self.param_expected = 0      # cumulative flag value that means "all stripes of the current transfer landed"
        self.host_mirror: Optional[torch.Tensor] = None
        # live execution
        L = self.cfg.layers
        self.zag = core.ZigzagScheduler(L, 4)
        self._zag_layers_seen = 0
        self.zag_tasks: Dict[int, dict] = {}
        self.zag_slots = torch.empty(4, max_batch_tokens, self.cfg.hidden, dtype=dt, device=self.device)
        self.zag_cv = threading.Condition(self.lock)
        self._stop = False
        # transfers (parameter copies, KV push / arrival waits, relays) run on their own high-priority stream so that
        # they overlap the serving kernels of the default stream instead of queueing between decode steps
        self.side = torch.cuda.Stream(device=self.device, priority=-1)
        self.xfer_lock = threading.Lock()      # one transfer at a time uses the side stream and the ticket words
        self.progressive_push_ctas = 16        # CTAs of one layer's push while the prefill pass goes on beside it
        self._poll_stream = torch.cuda.Stream(device=self.device)
        self._kv_slot_busy = [False] * symm.KV_SLOTS   # incoming KV transfers: slot reserved until the push has completed
        self._kv_done_want = [0] * symm.KV_SLOTS       # pushes started per slot = value its completion counter will reach
        # TP shards of a replica act on the minimum of their loaded-unit counts
        self.agree: Optional[LoadAgreement] = None
        self.steplog: Optional[StepLog] = None          # order of live-execution steps, decided by the first shard
        self._agreed_full = False
        self._relay_waiters: List[tuple] = []           # relay calls waiting for the leading shard's choice
        if tp > 1 and self.fabric is not None:
            first = rank - rank % tp
            self.agree = LoadAgreement(self.fabric, list(range(first, first + tp)), rank, symm.AGREE_FLAG0, L)
            self.agree.publish(L + 2 if ready else 0)
            self.steplog = StepLog(self.fabric, list(range(first, first + tp)), rank, symm.ZAG_LOG_FLAG0, symm.ZAG_LOG)
        self.zag_thread = threading.Thread(target=self._zag_loop, daemon=True)
        self.zag_thread.start()
        self.transfer_thread: Optional[threading.Thread] = None
        self.transfer_log: List[dict] = []     # one entry per parameter transfer this GPU took part in
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ helpers
    def thread_init(self) -> None:
        # the CUDA current device is per thread and defaults to device 0
        torch.cuda.set_device(self.device)

    def info(self) -> dict:
        return {"ready": self.engine.status.fully_loaded(), "dtype": "bfloat16", "device_type": "cuda",
                "ranks": {"rank": self.rank, "world": self.world, "tp": self.tp}}

    def _specs(self, batch, track: bool = True) -> List["core.SeqSpec"]:
        if track:
            self.stopper.add(batch)     # the requests are about to live here: remember their stop sequences
        return [seq_spec_from_request(r, eos_token=self.eos_token) for r in batch.requests]

    def _cached(self, b):
        ids = b.unfinished_ids()
        return pb.CachedBatch(id=b.id, request_ids=ids, size=len(ids), max_tokens=b.max_tokens()) if ids else None

    def _emit(self, b, toks):
        # wire bytes built natively: touching `b.seqs` here would copy every prompt and token history per step, and
        # building the messages one by one costs ~4 us each
        return b.encode_generations(toks)

    def _finish_step(self, b, toks):
        self.stopper.check(b)          # a request whose text now holds one of its stop sequences ends with this token
        gens = self._emit(b, toks)
        b.filter(b.unfinished_ids())
        if b.size:
            self.batches[b.id] = b
        else:
            self.batches.pop(b.id, None)
        return gens, (self._cached(b) if b.size else None)

    # ------------------------------------------------------------------ inference
    def prefill(self, batch, forward_case, pp_info, pipe_peer):
        with self.lock:
            if not self.engine.status.fully_loaded():
                raise RuntimeError("model parameters are not loaded")
            b = self.engine.new_batch(batch.id, self._specs(batch))
            if b is None:
                raise RuntimeError("out of KV pages")
            if forward_case & pb.PREFILL_CASE_NAIVE_PP:
                start = 0
                if pp_info is not None and pp_info.WhichOneof("start_layer") == "tfm_layer":
                    start = int(pp_info.tfm_layer)
                toks = self._continue_relayed(b, start)
            elif forward_case & pb.PREFILL_CASE_MIGRATE_PROGRESSIVE and pipe_peer:
                if self.fabric is None:
                    b.clear()
                    raise RuntimeError("a layer-progressive migration needs the peer fabric")
                try:
                    toks = self._prefill_pushing(b, batch, list(pipe_peer))
                    ops.check_status()
                    gens, _ = self._finish_step(b, toks)
                finally:
                    # every layer has left for the decode replica (or the call failed): nothing of the batch stays
                    self.batches.pop(b.id, None)
                    b.clear()
                return gens, None, None
            else:
                toks = self.engine.prefill(b)
            ops.check_status()
            gens, cb = self._finish_step(b, toks)
            return gens, cb, None

    def _prefill_pushing(self, b, batch, dst) -> List[int]:
        """Prefill with a layer-progressive migration (`PREFILL_CASE_MIGRATE_PROGRESSIVE`, proto/generate.proto:315-326;
        the reference declares the case and never runs it): layer l's pages are stored into the decode replica's pool
        on the transfer stream as soon as layer l has run, so only the last layer's push is left when the pass ends.
        The decode replica's `immigrate` runs at the same time and publishes its page ids under the transfer's tag,
        as for a migration of all layers; shard i pushes to shard i."""
        peer = dst[self.rank % self.tp]
        slot = batch.id % symm.KV_SLOTS
        src_ids = self._rpc_page_list(b, batch)
        L = self.cfg.layers
        main = torch.cuda.current_stream()
        # same event names as a migration of all layers, so that a log check of "every batch migrated once" holds
        log.info("batch %d migrate start, layer by layer while the prefill runs, layers [0,%d) -~> rank %d", batch.id, L, peer)
        with self.xfer_lock:
            with torch.cuda.stream(self.side):
                src_pages = torch.tensor(src_ids, dtype=torch.int32, device=self.device)
                # the first push waits (on the transfer stream only) until the destination has published its page ids
                tag_ptr = self.ctl.ptrs[peer] + (symm.KV_SLOTS * CTL_SLOT_WORDS + slot) * 4
                self.fabric.wait_flag_eq(tag_ptr, self._kv_tag(batch.id, 0), budget_ms=10000)
            count_ptr = self.ctl.ptrs[peer] + slot * CTL_SLOT_WORDS * 4

            def after_layer(l: int) -> None:
                ran = torch.cuda.Event()
                ran.record(main)
                self.side.wait_event(ran)
                with torch.cuda.stream(self.side):
                    self.fabric.kv_push(peer, src_pages, None, l, l + 1, self.page_bytes, self.kv_layer_stride,
                                        self.kv_layer_stride, self.engine.num_pages, self.engine.num_pages,
                                        flag_slot=slot, dst_pages_ptr=count_ptr + 4, dst_count_ptr=count_ptr,
                                        done=(l == L - 1), ctas_per_layer=self.progressive_push_ctas)
            try:
                toks = self.engine.prefill(b, after_layer=after_layer if src_ids else None)
            finally:
                self.side.synchronize()
            log.info("batch %d migrate done", batch.id)
            return toks

    def _continue_relayed(self, b, start_layer: int) -> List[int]:
        """Old-instance half of a relayed batch: take the residual stream from the mailbox and run layers [k, L)."""
        eng = self.engine
        if b.num_prompt_tokens() > eng.max_batch_tokens:
            raise RuntimeError(f"a relayed batch takes at most {eng.max_batch_tokens} prompt tokens")
        T, P = b.fill_prefill(eng.host_np, eng.layout)
        eng._h2d(eng.layout.page_indices + P)
        m = eng._views(T, b.size, P, True, b.prompt_lens())
        if start_layer > 0:
            slot = b.id % 4
            self.fabric.wait_flag(symm.MAILBOX_FLAG0 + slot, int(b.id) + 1, budget_ms=5000)
            src = self.fabric.mailbox.local[slot * self.slot_bytes:(slot + 1) * self.slot_bytes]
            rows = src.view(torch.bfloat16).view(-1, self.cfg.hidden)
            if eng.fused is not None:
                # tensor parallel: every shard received all rows from its counterpart; the rest of the pass keeps the
                # residual stream replicated (switch-reduced path), whatever the number of rows
                if not eng.fused.has_mc:
                    raise RuntimeError("continuing a relayed batch with tp > 1 needs in-switch reduction")
                eng.runner.load_residual(T, rows, start_layer)
            else:
                eng.runner.res[:T].copy_(rows[:T])
            # the slot is consumed: re-arm its flag (stream-ordered after the copy) so that a later batch with a
            # smaller id cannot pass the wait on a stale value
            self.fabric.set_flag(self.rank, symm.MAILBOX_FLAG0 + slot, 0, add=False)
            eng.runner.force_switch = eng.fused is not None
            try:
                toks = eng.runner.forward(m, lo=start_layer, with_embed=False)
            finally:
                eng.runner.force_switch = False
        else:
            toks = eng.runner.forward(m)
        out = eng._tokens_to_host(toks, b.size)
        b.mark_prefilled()
        b.append_tokens(out, False)
        b.decode = True
        return out

    def decode(self, batches, last_iter_tokens, steps: int = 1):
        """One decode step of the merged batches; with `steps` > 1 up to that many steps back to back (the generations
        of all steps come back in step order), which takes the router's round trip out of the time between steps.
        The lock is released between steps so that other calls (a prefill here, the set-up of a migration) get in."""
        with self.lock:
            for i, cb in enumerate(batches):
                ids = list(last_iter_tokens[i].ids) if i < len(last_iter_tokens) else []
                bi = self.batches[cb.id]
                if ids and len(ids) == bi.size and bi.none_generated():
                    bi.append_tokens(ids, False)
            b = self.batches[batches[0].id]
            for cb in batches[1:]:
                b.extend(self.batches.pop(cb.id))
            toks = self.engine.decode(b)
            gens, cb = self._finish_step(b, toks)
        for _ in range(1, max(1, steps)):
            if cb is None:
                break
            with self.lock:
                if self.batches.get(b.id) is not b:       # cleared or migrated away in between
                    break
                toks = self.engine.decode(b)
                more, cb = self._finish_step(b, toks)
            gens += more
        return gens, cb

    def clear_cache(self, batch_id):
        with self.lock:
            for i in ([batch_id] if batch_id is not None else list(self.batches)):
                b = self.batches.pop(i, None)
                if b is not None:
                    b.clear()

    def filter_batch(self, batch_id, request_ids):
        with self.lock:
            b = self.batches[batch_id]
            b.filter(list(request_ids))
            return pb.CachedBatch(id=b.id, request_ids=b.unfinished_ids(), size=b.size, max_tokens=b.max_tokens())

    def warmup(self, req) -> int:
        return self.engine.pool.total_pages * self.engine.page_size

    # ------------------------------------------------------------------ live execution (ZigZag)
    def zag_prefill(self, batch, forward_case, pp_info, zag_layers, zag_seq):
        if self.engine.fused is not None and not self.engine.fused.has_mc:
            # tensor-parallel live execution keeps one residual stream per task in symmetric memory and updates it
            # through the switch-reduced kernel, which needs the fabric's multicast address
            raise RuntimeError("live execution with tp > 1 needs in-switch reduction (or workers started with --no-fused-tp)")
        if self.tp > 1 and self.steplog is None:
            raise RuntimeError("live execution with tp > 1 needs the peer fabric")
        fut: Future = Future()
        with self.lock:
            b = self.engine.new_batch(batch.id, self._specs(batch))
            if b is None:
                raise RuntimeError("out of KV pages")
            if b.num_prompt_tokens() > self.engine.max_batch_tokens:
                # a layer-interleaved task keeps its whole residual stream in one activation slot
                b.clear()
                raise RuntimeError(f"live execution takes at most {self.engine.max_batch_tokens} prompt tokens per batch")
            slot = self.zag.add_task(batch.id, zag_seq, b.num_prompt_tokens())
            if slot < 0:
                b.clear()
                raise RuntimeError("no activation slot free")
            self.zag_tasks[batch.id] = {"batch": b, "future": fut, "slot": slot, "meta": None, "seq": int(zag_seq)}
            self.zag_cv.notify_all()
        return fut.result(timeout=120)

    def _zag_loop(self) -> None:
        torch.cuda.set_device(self.device)
        while not self._stop:
            try:
                self._zag_turn()
            except Exception:  # noqa: BLE001  (this thread serves every later live-execution task: it must survive)
                log.exception("live-execution step failed")
                with self.lock:
                    for t in list(self.zag_tasks.values()):
                        if not t["future"].done():
                            t["future"].set_exception(RuntimeError("live-execution step failed"))
                time.sleep(0.01)

    def _zag_loaded(self):
        """(embedding, layers, head) this replica may use now: what every tensor-parallel shard holds."""
        st = self.engine.status
        if self.agree is not None and not self._agreed_full:
            loaded = self.agree.agreed_state()
            self._agreed_full = loaded[2] and loaded[1] >= self.cfg.layers
            return loaded
        return st.embed_ready, st.layers_ready, st.head_ready

    def _zag_turn(self) -> None:
        with self.lock:
            if self.steplog is not None and not self.steplog.leader:
                d = self._zag_follow()
                if d is None:
                    return
            else:
                loaded = self._zag_loaded()
                if loaded[1] < self._zag_layers_seen:
                    self.zag.reset()    # a replica that was emptied and is being loaded again starts from no layers
                self.zag.set_loaded(*loaded)
                self._zag_layers_seen = loaded[1]
                d = self.zag.next()
                if d.step in (core.ZagStep.Idle, core.ZagStep.Blocked):
                    # nothing to run: sleep until a task or a parameter unit arrives (both notify the condition); the
                    # short timeout only bounds the wait while layers are still landing
                    self.zag_cv.wait(0.0005 if d.step == core.ZagStep.Blocked else 0.05)
                    return
                if self.steplog is not None:
                    self.steplog.publish(StepLog.STEP, int(d.step), max(0, d.layer), d.slot, self.zag.seq_of(d.batch_id))
            self._zag_run(d)

    def _zag_follow(self):
        """A shard other than the leading one: the next entry of the leader's log, as a decision to run here.  Returns
        None after having waited a little when there is nothing to do yet (no entry, or an entry about a request or a
        relay call that has not reached this shard)."""
        e = self.steplog.peek()
        if e is None:
            self.zag_cv.wait(0.0003 if (self.zag.pending() or self._relay_waiters) else 0.02)
            return None
        if e["kind"] == StepLog.RELAY_NONE:
            if not self._relay_waiters:
                self.zag_cv.wait(0.0003)
                return None
            self.steplog.consume()
            self._relay_waiters.pop(0)[1].set_result(None)
            return None
        seq = self._zag_seq_full(e["seq_num"])
        if seq is None:
            self.zag_cv.wait(0.0003)      # the request itself is still on its way here
            return None
        if e["kind"] == StepLog.RELAY:
            if not self._relay_waiters:
                self.zag_cv.wait(0.0003)
                return None
            self.steplog.consume()
            rank, fut = self._relay_waiters.pop(0)
            r = self.zag.relay_task(seq)
            assert r is not None and r.next_layer == e["layer"] - 1, "shards disagree about a relayed task"
            fut.set_result(self._relay_task(r, rank, e["slot"]))
            return None
        self.steplog.consume()
        d = core.ZagDecision()
        d.step, d.batch_id, d.slot = core.ZagStep(e["step"]), self.zag.batch_of(seq), e["slot"]
        d.layer = e["layer"] if d.step == core.ZagStep.Layer else -1
        return d

    def _zag_seq_full(self, low8: int):
        """Sequence number of the queued task whose low 8 bits are `low8` (at most a handful are in flight)."""
        for t in self.zag_tasks.values():
            if (t["seq"] & 0xFF) == low8:
                return t["seq"]
        return None

    def _zag_run(self, d) -> None:
        """Run one step (embedding, one layer, or the head) of one live-execution task.  Lock held."""
        task = self.zag_tasks[d.batch_id]
        eng, b = self.engine, task["batch"]
        if task["meta"] is None:
            T, P = b.fill_prefill(eng.host_np, eng.layout)
            eng._h2d(eng.layout.page_indices + P)
            # the staging arrays are shared: keep a private device copy of this task's inputs
            dev_copy = eng.dev[:eng.layout.page_indices + P].clone()
            task["meta"] = (T, P, dev_copy)
        T, P, dev_copy = task["meta"]
        eng.dev[:dev_copy.numel()].copy_(dev_copy)
        m = eng._views(T, b.size, P, True, b.prompt_lens(), work=task.get("work"))
        task["work"] = m.prefill_work          # the attention's CTA order is the same for every step of the task
        saved = eng.runner.res
        fused = eng.fused
        if fused is not None:
            # tensor parallel: the residual stream and the normalised rows of each task live in a context of the
            # symmetric region (context 0 belongs to ordinary passes); live steps form their own call sequence
            fused.use_lane(1)
            fused.use_context(1 + d.slot)
            eng.runner.force_switch = True
        else:
            eng.runner.res = self.zag_slots[task["slot"]]
        try:
            if d.step == core.ZagStep.Embed:
                log.debug("zag embed batch=%d", d.batch_id)
                eng.runner.embed(m)
            elif d.step == core.ZagStep.Layer:
                log.debug("zag layer batch=%d layer=%d", d.batch_id, d.layer)
                eng.runner.run_layer(d.layer, m)
            else:
                log.debug("zag head batch=%d", d.batch_id)
                toks = eng._tokens_to_host(eng.runner.head(m), b.size)
            torch.cuda.current_stream().synchronize()
        finally:
            eng.runner.res = saved
            if fused is not None:
                fused.use_lane(0)
                fused.use_context(0)
                eng.runner.force_switch = False
        done = self.zag.complete(d)
        if done:
            b.mark_prefilled()
            b.append_tokens(toks, False)
            b.decode = True
            gens, cb = self._finish_step(b, toks)
            self.zag_tasks.pop(d.batch_id)["future"].set_result((gens, cb, None))

    def relay(self, rank, relax_not_head):
        if self.steplog is not None and not self.steplog.leader:
            # the leading shard chooses the task and the layer; this shard's live-execution thread acts when it reads
            # that choice in the log
            fut: Future = Future()
            with self.lock:
                self._relay_waiters.append((rank, fut))
                self.zag_cv.notify_all()
            return fut.result(timeout=60)
        with self.lock:
            r = self.zag.relay(bool(relax_not_head))
            if self.steplog is not None:
                if r is None:
                    self.steplog.publish(StepLog.RELAY_NONE)
                else:
                    self.steplog.publish(StepLog.RELAY, 0, r.next_layer + 1, r.slot, r.seq_num)
            if r is None:
                return None
            return self._relay_task(r, rank, r.slot)

    def _relay_task(self, r, rank, ctx_slot):
        """Hand a task over to the old instance's shard `rank`: ship its residual stream, release its slot, answer its
        ZagPrefill call with the layer to resume from.  Lock held."""
        task = self.zag_tasks.pop(r.batch_id)
        b = task["batch"]
        k = max(0, r.next_layer)
        log.info("zag relay batch=%d layer=%d +>+> rank %d", r.batch_id, k, rank)
        if k > 0:
            # ship the residual stream [T, hidden] into the old instance's mailbox slot and flag it
            T = r.num_tokens
            nbytes = T * self.cfg.hidden * 2
            nbytes = (nbytes + 15) // 16 * 16
            slot = r.batch_id % 4
            fused = self.engine.fused
            if fused is not None:
                fused.use_context(1 + ctx_slot)
                resid = fused.res(T)
                fused.use_context(0)
            else:
                resid = self.zag_slots[task["slot"]]
            with self.xfer_lock, torch.cuda.stream(self.side):
                stage = self.fabric.mailbox.local[slot * self.slot_bytes:slot * self.slot_bytes + nbytes]
                stage.copy_(resid.view(torch.uint8).view(-1)[:nbytes])
                self.fabric.copy_units(self.fabric.mailbox, [rank], [slot * self.slot_bytes], [nbytes],
                                       symm.MAILBOX_FLAG0 + slot, num_ctas=16)
                # the flag is a counter; publish the batch tag on top so the reader can wait for ">= id + 1"
                self.fabric.set_flag(rank, symm.MAILBOX_FLAG0 + slot, int(r.batch_id) + 1, add=False)
                self.side.synchronize()
        self.zag.release_slot(task["slot"])
        pp = pb.PipeParaInfo()
        if r.next_layer <= 0:
            pp.embedding_layer = 1
        else:
            pp.tfm_layer = k
        # layers [0, k) of this batch's KV stay here until MigratePartial(FIRST) moves them
        b.mark_prefilled()
        self.batches[b.id] = b
        cb = pb.CachedBatch(id=b.id, request_ids=b.request_ids(), size=b.size, max_tokens=b.max_tokens())
        task["future"].set_result(([], cb, pp))
        return r.batch_id, r.seq_num

    # ------------------------------------------------------------------ KV migration
    def _layer_range(self, partial, num_layer):
        L = self.cfg.layers
        if partial == pb.PARTIAL_CASE_FIRST:
            return 0, min(num_layer, L)
        if partial == pb.PARTIAL_CASE_SECOND:
            return min(num_layer, L), L
        return 0, L

    # Handshake of one transfer (all layers, or one half of a relayed batch).  Control region of every GPU:
    # KV_SLOTS slots of CTL_SLOT_WORDS words (word 0 = number of page ids, then the ids) followed by one tag word per
    # slot.  The destination reserves slot `batch id mod KV_SLOTS` (a second transfer that maps to the same slot waits
    # until the first has completed), writes count and ids, then publishes the transfer's tag: a value unique to
    # (batch, half), matched exactly by the source, so a tag left by any other transfer can never satisfy the wait.
    # The source pushes every layer and then, in stream order, bumps the slot's completion counter on the
    # destination; only then does the destination clear the tag and free the slot, so no CTA of the push can still
    # be reading the id list when the next transfer overwrites it.  Both page lists follow the requests of the RPC,
    # in its order, with -1 entries for requests one side no longer holds (see Batch::prompt_page_ids_for).
    @staticmethod
    def _kv_tag(batch_id: int, partial: int) -> int:
        return (((int(batch_id) + 1) & 0x0FFFFFFF) << 2) | (int(partial) & 3)

    def _rpc_page_list(self, b, batch) -> List[int]:
        specs = self._specs(batch, track=False)
        ids = b.prompt_page_ids_for([sp.id for sp in specs], [len(sp.prompt) for sp in specs])
        if len(ids) + 1 > CTL_SLOT_WORDS:
            raise RuntimeError(f"batch {batch.id}: {len(ids)} KV pages exceed the {CTL_SLOT_WORDS - 1} a transfer slot holds")
        return ids

    def immigrate(self, batch, src, dst, partial=0, num_layer=0):
        lo, hi = self._layer_range(partial, num_layer)
        half = {pb.PARTIAL_CASE_FIRST: " first half", pb.PARTIAL_CASE_SECOND: " second half"}.get(partial, "")
        slot = batch.id % symm.KV_SLOTS
        keep = [r.id for r in batch.requests]
        reserved = False
        with self.lock:
            b = self.batches.get(batch.id)
            if b is None:
                b = self.engine.new_batch(batch.id, self._specs(batch))
                if b is None:
                    raise RuntimeError("out of KV pages")
                b.mark_prefilled()
                b.decode = True
                if b.size:
                    self.batches[batch.id] = b
            elif partial == pb.PARTIAL_CASE_SECOND:
                # the second half names the requests that are still alive after the prefill; the ones that ended at
                # their first token were part of the first half only and leave the batch (and their pages) here
                b.filter([i for i in b.request_ids() if i in set(keep)])
            log.info("batch %d immigrate start%s layers [%d,%d) <~- rank %s", batch.id, half, lo, hi, list(src))
            ids = None
            if hi > lo and self.fabric is not None:
                ids = self._rpc_page_list(b, batch) or None
            if ids is not None:
                deadline = time.monotonic() + 30.0
                while self._kv_slot_busy[slot]:
                    if not self.zag_cv.wait(max(0.0, deadline - time.monotonic())) and time.monotonic() >= deadline:
                        raise RuntimeError(f"batch {batch.id}: transfer slot {slot} stayed busy")
                self._kv_slot_busy[slot] = reserved = True
                self._kv_done_want[slot] += 1
                done_want = self._kv_done_want[slot]
        try:
            if ids is not None:
                tag_index = symm.KV_SLOTS * CTL_SLOT_WORDS + slot
                with self.xfer_lock, torch.cuda.stream(self.side):
                    words = self.ctl.local.view(torch.int32)
                    words[slot * CTL_SLOT_WORDS:slot * CTL_SLOT_WORDS + 1 + len(ids)].copy_(
                        torch.tensor([len(ids)] + ids, dtype=torch.int32), non_blocking=False)
                    self._ctl_set(self.rank, tag_index, self._kv_tag(batch.id, partial))
                    self.side.synchronize()
                # the layers land without this GPU doing anything: poll the completion counter from the host, with no
                # stream or lock held, so that decode steps and other transfers go on meanwhile
                deadline = time.monotonic() + 10.0
                with torch.cuda.stream(self._poll_stream):
                    while self.fabric.read_flags(symm.KV_DONE_FLAG0 + slot, 1)[0] < done_want:
                        if time.monotonic() > deadline:
                            raise RuntimeError(f"batch {batch.id}: KV push did not complete{half}")
                        time.sleep(0.0001)
                    self.ctl.local.view(torch.int32)[tag_index:tag_index + 1].zero_()
                    self._poll_stream.synchronize()
                ops.check_status()
        finally:
            if reserved:
                with self.lock:
                    self._kv_slot_busy[slot] = False
                    self.zag_cv.notify_all()
        with self.lock:
            cb = pb.CachedBatch(id=b.id, request_ids=b.request_ids(), size=b.size, max_tokens=b.max_tokens())
        log.info("batch %d immigrate done%s", batch.id, half)
        return cb

    def _ctl_set(self, rank, word_index, value):
        import ctypes
        ptr = self.ctl.ptrs[rank] + word_index * 4
        symm._check(symm._L.lib().blitz_flag_set(ctypes.c_void_p(ptr), value, 0, symm._stream()), "blitz_flag_set")

    def migrate(self, batch, src, dst, partial=0, num_layer=0):
        with self.lock:
            b = self.batches.get(batch.id)
            if b is None:
                raise KeyError(f"batch {batch.id} not cached on rank {self.rank}")
            lo, hi = self._layer_range(partial, num_layer)
            my = src.index(self.rank) if self.rank in src else self.rank % self.tp
            peer = dst[my]
            slot = batch.id % symm.KV_SLOTS
            half = {pb.PARTIAL_CASE_FIRST: " first half", pb.PARTIAL_CASE_SECOND: " second half"}.get(partial, "")
            log.info("batch %d migrate start%s layers [%d,%d) -~> rank %d", batch.id, half, lo, hi, peer)
            src_ids = self._rpc_page_list(b, batch)
        # the push itself runs outside the lock, on the transfer stream: this batch is parked until it has migrated,
        # and prefills of other batches continue meanwhile
        if hi > lo and src_ids:
            with self.xfer_lock, torch.cuda.stream(self.side):
                src_pages = torch.tensor(src_ids, dtype=torch.int32, device=self.device)
                # wait until the destination has published its page ids for exactly this transfer
                tag_ptr = self.ctl.ptrs[peer] + (symm.KV_SLOTS * CTL_SLOT_WORDS + slot) * 4
                self.fabric.wait_flag_eq(tag_ptr, self._kv_tag(batch.id, partial), budget_ms=10000)
                count_ptr = self.ctl.ptrs[peer] + slot * CTL_SLOT_WORDS * 4
                self.fabric.kv_push(peer, src_pages, None, lo, hi, self.page_bytes, self.kv_layer_stride,
                                    self.kv_layer_stride, self.engine.num_pages, self.engine.num_pages,
                                    flag_slot=slot, dst_pages_ptr=count_ptr + 4, dst_count_ptr=count_ptr)
                self.side.synchronize()
            ops.check_status()
        with self.lock:
            cb = pb.CachedBatch(id=b.id, request_ids=b.request_ids(), size=b.size, max_tokens=b.max_tokens())
            log.info("batch %d migrate done%s", batch.id, half)
            self.batches.pop(batch.id, None)
            b.clear()
            return cb

    # ------------------------------------------------------------------ parameters
    def _shard_peers(self, ranks):
        t = self.rank % self.tp
        return [r for r in ranks if r % self.tp == t]

    def broadcast(self, kind, src_ranks, dst_ranks):
        sources, dests = self._shard_peers(src_ranks), self._shard_peers(dst_ranks)
        if self.rank in sources:
            offs = [o for _, o, _ in self.units]
            lens = [(b + 15) // 16 * 16 for _, _, b in self.units]
            # one destination: plain peer stores are the fastest (92 % of the measured link rate); several: one
            # multimem store per 16 bytes keeps the source's egress at 1x whatever the fan-out
            # (the multicast address covers the GPUs that hold this shard, in every replica: the ones that are not
            # destinations already hold the same bytes)
            mm = self.use_multimem and len(dests) >= self.multimem_min_dests and bool(self.fabric.weights.mc_ptr)
            with self.xfer_lock:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                with torch.cuda.stream(self.side):
                    e0.record()
                    self.fabric.copy_units(self.fabric.weights, dests, offs, lens, symm.PARAM_FLAG0,
                                           stripe=sources.index(self.rank), n_stripes=len(sources), use_multimem=mm,
                                           num_ctas=self.copy_ctas)
                    e1.record()
                self.side.synchronize()
                # device time of this source's share (first store to last flag), for reports beside the router's clock
                self.transfer_log.append({"role": "source", "rank": self.rank, "device_ms": e0.elapsed_time(e1),
                                          "bytes": sum(lens) // len(sources) * len(dests), "dests": list(dests),
                                          "sources": list(sources), "multimem": bool(mm)})
        elif self.rank in dests:
            self._receive_params(len(sources))

    def _receive_params(self, n_stripes: int, timeout_s: float = 120.0) -> None:
        """Poll this GPU's own flag pad and mark units ready in arrival order."""
        torch.cuda.set_device(self.device)
        with self.lock:
            self.engine.status.reset()
            if self.agree is not None:
                self.agree.publish(0)
                self._agreed_full = False
            base = self.param_expected
            self.param_expected += n_stripes
        want, n_units, nxt = base + n_stripes, len(self.units), 0
        t0 = time.monotonic()
        side = torch.cuda.Stream(device=self.device)
        while nxt < n_units:
            with torch.cuda.stream(side):
                flags = self.fabric.read_flags(symm.PARAM_FLAG0, n_units)
            while nxt < n_units and flags[nxt] >= want:
                with self.lock:
                    self.engine.status.unit_arrived(nxt)
                    if self.agree is not None:
                        self.agree.publish(nxt + 1)
                    self.zag_cv.notify_all()
                nxt += 1
            if nxt < n_units:
                if time.monotonic() - t0 > timeout_s:
                    raise RuntimeError(f"parameter transfer stalled at unit {nxt}")
                time.sleep(0.0002)
        self.transfer_log.append({"role": "destination", "rank": self.rank, "host_ms": (time.monotonic() - t0) * 1e3,
                                  "units": n_units, "stripes": n_stripes})

    def send_params(self, dst):
        self.broadcast("p2p", [self.rank], [dst])

    def recv_params(self, src):
        self.transfer_thread = threading.Thread(target=self._receive_params, args=(1,), daemon=True)
        self.transfer_thread.start()

    def wait_transfer_done(self):
        if self.transfer_thread is not None:
            self.transfer_thread.join()
            self.transfer_thread = None

    def load_params(self, load_case, model_name, model_path):
        path = model_path or self.model_path
        with self.lock:
            if load_case == pb.LOAD_FROM_HOST_MEM and self.host_mirror is not None:
                self.engine.load_params_from_host(self.host_mirror)
            else:
                res = self.engine.load_params_from_disk(path, self.host_mirror)
                self.host_mirror = res["host_mirror"]

    def reset_status(self):
        with self.lock:
            self.engine.reset_status()

    def set_status_ready(self):
        with self.lock:
            self.engine.set_status_ready()

    def release_graphs(self) -> None:
        self.engine.release_graphs()

    def close_regions(self) -> None:
        """Symmetric regions of this worker: engine (fused TP), fabric, control words.  See parallel/teardown.py."""
        self.engine.close_regions()
        if self.fabric is not None:
            self.fabric.close_regions()
            self.ctl.close_regions()

    def close(self):
        """Stop the live-execution thread and wait for it: a thread that is still inside a native call when the
        interpreter shuts down takes the process down with it."""
        self._stop = True
        with self.lock:
            self.zag_cv.notify_all()
        if self.zag_thread.is_alive() and threading.current_thread() is not self.zag_thread:
            self.zag_thread.join(timeout=5.0)
