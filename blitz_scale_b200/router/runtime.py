"""Router runtime: the asyncio shell around the native orchestrator core.

The core (`blitz_core.Controller`) decides; this module performs the IO: it turns each `Action` into
the matching RPCs on every tensor-parallel rank of the replica (the reference's `join_all` over
stubs, router_v2/src/replica/disaggregation.rs:944-963), reports completions back, and streams
tokens to the per-request queues the HTTP layer reads.  A failed RPC is reported as a lost replica
(the reference `unwrap()`s the result and dies, disaggregation.rs:960-963).  Transition and metric
log lines keep the reference's grep-able formats (`Replica<i> A => B`,
`System Metrics: prefill_tokens: .., decode_tokens: ..`, scripts/batch/utils.py:391-424).
"""
from __future__ import annotations

import asyncio
import logging
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..pb.schema import pb
from ..runtime import core
from ..utils.tracing import child_traceparent, new_traceparent
from .stub import CURRENT_TRACE, WorkerStub, encode_prefill_case

log = logging.getLogger("blitz.router")


class RankFailure(Exception):
    """An RPC to `rank` failed while carrying out an action."""

    def __init__(self, rank: int, cause: BaseException):
        super().__init__(f"rank {rank}: {type(cause).__name__}: {cause}")
        self.rank = rank


def _is_unreachable(e: BaseException) -> bool:
    code = getattr(e, "code", None)
    try:
        import grpc
        return callable(code) and code() in (grpc.StatusCode.UNAVAILABLE, grpc.StatusCode.DEADLINE_EXCEEDED)
    except Exception:  # noqa: BLE001
        return False


A = core.ActionType


@dataclass
class LiveRequest:
    id: int
    proto: object                      # pb.Request
    queue: asyncio.Queue = field(default_factory=asyncio.Queue)
    t_submit: float = 0.0
    tokens: List[int] = field(default_factory=list)
    texts: List[str] = field(default_factory=list)
    times: List[float] = field(default_factory=list)   # router clock at the delivery of each token
    # stream = True: every token is also put on `queue` as ("token", id, final) / ("error", text), waking the consumer
    # once per token.  stream = False: tokens only accumulate in `tokens` / `times` and `done` resolves at the end
    # (None, or the error text): one wake-up per request instead of one per token.
    stream: bool = True
    done: Optional[asyncio.Future] = None
    entry: object = None               # the core's record of the request (queue and token times), set when it finishes
    finish_reason: str = ""            # "length" | "eos_token" | "stop_sequence", set with the last token
    # stop sequences (text): checked here, where the text of a request can be known, after every token.  `detok` turns
    # token ids into text; `stop_window` = how many trailing tokens can contain the longest stop sequence.
    stop: tuple = ()
    detok: object = None
    stop_window: int = 0
    stopped: bool = False              # ended by a stop sequence; the worker's later tokens are dropped


FINISH_REASONS = {1: "length", 2: "eos_token", 3: "stop_sequence"}   # the `final` code of a delivery


class RouterRuntime:
    def __init__(self, cfg: "core.ControllerConfig", worker_urls: List[str], model_layers: int = 32,
                 model_path: str = "", stat_csv: str = "", health_interval_s: float = 0.0, health_misses: int = 2,
                 rpc_timeout_s: float = 300.0, exporter=None, decode_steps: int = 1):
        self.cfg = cfg
        # decode steps a worker runs per DecodeV2 call.  1: every token makes the round trip through the router (the
        # reference's behaviour).  k > 1: the round trip is paid once per k steps; tokens then arrive k at a time, and
        # a batch that migrates in joins the running one up to k steps later.
        self.decode_steps = max(1, int(decode_steps))
        # optional span sink (`utils.otlp.SpanExporter`): one span per dispatched operation and one per request
        self.exporter = exporter
        # failure detector: every `health_interval_s` each active replica's ranks are pinged with the Health RPC;
        # `health_misses` consecutive misses (error or no answer within the interval) declare the replica lost.
        # The reference has no detector (its Health is a stub and a failed RPC panics the replica task).
        self.health_interval_s, self.health_misses = health_interval_s, max(1, health_misses)
        self._missed: Dict[int, int] = {}
        # 500 ms CSV of prefill / decode token deltas (router_v2/src/statistic.rs:26-63)
        self.stat_csv = open(stat_csv, "w", buffering=1) if stat_csv else None
        if self.stat_csv:
            self.stat_csv.write("time_s,prefill_tokens,decode_tokens\n")
        self._stat_last = (0.0, 0, 0)
        self.ctl = core.Controller(cfg)
        self.ctl.set_compact_deliveries(True)       # tokens come back as (request, token, final) tuples, not Actions
        # deadline of every worker RPC: a reply that never comes fails the operation (and the replica that owed it)
        # instead of leaving it in flight for ever; generous, a cold load of a large model from disk must fit
        self.stubs = [WorkerStub(u, rpc_timeout_s) for u in worker_urls]
        self.tp = cfg.tp
        self.layers = model_layers
        self.model_path = model_path
        self.requests: Dict[int, LiveRequest] = {}
        self.cached: Dict[tuple, object] = {}        # (replica, batch_id) -> pb.CachedBatch
        self.first_tokens: Dict[int, Dict[int, int]] = {}  # batch_id -> {request_id: first token} until first decode
        self.wake = asyncio.Event()
        self._loop_turns = 0
        self.stopped = False
        self.t0 = time.monotonic()
        self.root_trace = new_traceparent()
        self._next_id = 0
        self._tasks: set = set()
        self.transitions: "deque[tuple]" = deque(maxlen=50000)   # (router time, log line) of recent state transitions
        self._zag_pp: Dict[int, int] = {}            # batch_id -> layer at which a relayed batch was handed over

    # ------------------------------------------------------------------ submission
    def now(self) -> float:
        return time.monotonic() - self.t0

    def submit(self, input_tokens: List[int], max_new_tokens: int, *, inputs: str = "", parameters=None,
               ignore_eos: bool = True, stream: bool = True, stop=(), detok=None) -> LiveRequest:
        """Queue a request.  `ignore_eos` = False lets the worker end it at the model's end-of-sequence token.  `stop`:
        texts that end the request when the generated text contains one (needs `detok`, ids -> text); the reference
        carries both in the contract and applies neither (src/blitz/stopping.h:21 stops on length only)."""
        rid = self._next_id
        self._next_id += 1
        r = pb.Request(id=rid, inputs=inputs, prefill_logprobs=False, top_n_tokens=0)
        r.input_tokens.extend(input_tokens)
        r.stopping_parameters.max_new_tokens = max_new_tokens
        r.stopping_parameters.ignore_eos_token = ignore_eos
        stop = tuple(s for s in stop if s)
        if stop and detok is None:
            raise ValueError("stop sequences need a detokenizer")
        r.stopping_parameters.stop_sequences.extend(stop)
        if parameters is not None:
            r.parameters.CopyFrom(parameters)
        lr = LiveRequest(rid, r, t_submit=self.now(), stream=stream, done=asyncio.get_running_loop().create_future(),
                         stop=stop, detok=detok, stop_window=max((len(s.encode()) for s in stop), default=0) + 1)
        self.requests[rid] = lr
        self.ctl.submit(core.RequestEntry(rid, len(input_tokens), max_new_tokens, lr.t_submit))
        self.wake.set()
        return lr

    def client_gone(self, rid: int) -> None:
        """The consumer of request `rid` went away: stop spending work on it."""
        if self.ctl.client_gone(rid):                 # still queued: nothing will ever be delivered for it
            lr = self.requests.pop(rid, None)
            if lr is not None and not lr.done.done():
                lr.done.set_result("client gone")
        self.wake.set()

    # ------------------------------------------------------------------ main loop
    async def _ping(self, rep: int) -> bool:
        """True when every rank of the replica answers Health within one interval."""
        try:
            await asyncio.wait_for(asyncio.gather(*[self.stubs[r].health(timeout=self.health_interval_s)
                                                    for r in self._ranks(rep)]), timeout=self.health_interval_s)
            return True
        except Exception:  # noqa: BLE001 - any failure to answer counts as a miss
            return False

    async def _health_loop(self) -> None:
        while not self.stopped:
            await asyncio.sleep(self.health_interval_s)
            # replicas in service, and lost ones that may have come back (a restarted worker); all pinged at once, so
            # one that is away does not delay the verdict on the others
            reps = [rep for rep in range(self.ctl.num_replicas)
                    if self.ctl.state_name(rep) != "Inactive" or not self.ctl.reachable(rep)]
            answers = await asyncio.gather(*[self._ping(rep) for rep in reps])
            for rep, ok in zip(reps, answers):
                if self.ctl.state_name(rep) == "Inactive":
                    self._missed.pop(rep, None)
                    if ok and not self.ctl.reachable(rep):
                        log.info("replica %d answers again", rep)
                        self.ctl.set_reachable(rep, True)     # only now may the planner load into it
                    continue
                if ok:
                    self._missed[rep] = 0
                    continue
                self._missed[rep] = self._missed.get(rep, 0) + 1
                if self._missed[rep] >= self.health_misses:
                    log.error("replica %d missed %d heartbeats: declared lost", rep, self._missed[rep])
                    self.ctl.on_replica_unhealthy(rep, self.now())
                    self.ctl.set_reachable(rep, False)
                    self._purge_replica(rep)
                    self._missed[rep] = 0
                    self.wake.set()

    async def _warmup(self) -> None:
        """Ask every worker how many KV tokens it can hold (the Warmup call of the contract; the reference's router
        does the same at start, router_v2/src/replica/disaggregation.rs:679) and never plan for more pages per replica
        than the smallest answer, less a little headroom.  Workers that do not answer are left to the failure handling."""
        async def ask(r):
            try:
                return (await self.stubs[r].warmup()).max_supported_total_tokens
            except Exception:  # noqa: BLE001
                return 0
        tokens = [t for t in await asyncio.gather(*[ask(r) for r in range(len(self.stubs))]) if t > 0]
        if tokens:
            blocks = min(tokens) // max(1, self.cfg.block_size)
            before = self.ctl.max_blocks_per_replica
            self.ctl.limit_blocks_per_replica(max(1, blocks - max(1, blocks // 64)))
            if self.ctl.max_blocks_per_replica != before:
                log.warning("workers hold %d KV pages: the limit per replica is lowered from %d to %d", blocks, before,
                            self.ctl.max_blocks_per_replica)

    async def run(self) -> None:
        await self._warmup()
        last_metrics = 0.0
        if self.health_interval_s > 0:
            self._spawn(self._health_loop())
        while not self.stopped:
            now = self.now()
            self._loop_turns += 1
            actions = self.ctl.step(now)
            for line in self.ctl.drain_log():
                log.info(line)
                if " => " in line:
                    self.transitions.append((now, line))
            for a in actions:
                self._dispatch(a)
            self._deliver(now)
            if self.stat_csv is not None and now - self._stat_last[0] >= 0.5:
                p_tok, d_tok = self.ctl.token_counts()
                self.stat_csv.write(f"{now:.3f},{p_tok - self._stat_last[1]},{d_tok - self._stat_last[2]}\n")
                self._stat_last = (now, p_tok, d_tok)
            if now - last_metrics >= 1.0:
                last_metrics = now
                log.info(self.ctl.system_metrics_line())
                log.info("Waiting migration token num: %d", self.ctl.waiting_migration_tokens())
                for rep, mb_in, mb_out in self.ctl.take_flows():
                    log.info("Replica[%d]: Flow in: %dMB, Flow out: %dMB", rep, round(mb_in), round(mb_out))
                # the loop that plans and dispatches must keep turning (the reference asserts the same once a second)
                if self._loop_turns == 0 and now > 2.0:
                    log.error("Control loop stuck!")
                self._loop_turns = 0
                if log.isEnabledFor(logging.DEBUG):
                    for r in range(self.ctl.num_replicas):
                        m = self.ctl.metric(r)
                        log.debug("Replica<%d> state=%s used_blocks=%d model_loaded=%s", r, self.ctl.state_name(r),
                                  m.used_blocks, m.model_loaded)
            if not actions:
                self.wake.clear()
                try:
                    await asyncio.wait_for(self.wake.wait(), timeout=0.002)
                except asyncio.TimeoutError:
                    pass
            else:
                await asyncio.sleep(0)

    async def stop(self) -> None:
        self.stopped = True
        self.wake.set()
        for t in list(self._tasks):
            t.cancel()
        for s in self.stubs:
            await s.close()

    def _spawn(self, coro) -> None:
        t = asyncio.get_running_loop().create_task(coro)
        self._tasks.add(t)
        t.add_done_callback(self._tasks.discard)

    async def _all(self, ranks, calls) -> list:
        """Await one call per rank; if any fails, raise `RankFailure` naming the rank to blame.  A migration or a
        broadcast spans several replicas and a healthy participant's call can fail merely because its peer went
        away (a bounded wait that ran out), so a rank that cannot be reached at all is blamed before one that
        answered with an error."""
        res = await asyncio.gather(*calls, return_exceptions=True)
        bad = [(r, e) for r, e in zip(ranks, res) if isinstance(e, BaseException)]
        if not bad:
            return res
        for r, e in bad:
            if isinstance(e, asyncio.CancelledError):
                raise e
        unreachable = [(r, e) for r, e in bad if _is_unreachable(e)]
        r, e = (unreachable or bad)[0]
        raise RankFailure(r, e) from e

    def _ranks(self, replica: int) -> List[int]:
        return [replica * self.tp + i for i in range(self.tp)]

    def _batch_proto(self, a) -> object:
        b = pb.Batch(id=a.batch_id, size=len(a.request_ids), max_tokens=a.max_tokens)
        for rid in a.request_ids:
            lr = self.requests.get(rid)
            if lr is not None:
                b.requests.append(lr.proto)
        return b

    def _dispatch(self, a) -> None:
        t = a.type
        if t == A.Fail:
            lr = self.requests.pop(a.request_id, None)
            if lr is not None:
                if lr.stream:
                    lr.queue.put_nowait(("error", "replica lost"))
                if not lr.done.done():
                    lr.done.set_result("replica lost")
            return
        if t == A.Deliver:     # only when compact deliveries are off
            self._deliver_one(a.request_id, a.token, 1 + a.finish_reason if a.final else 0, self.now())
            return
        handler = {A.Prefill: self._do_prefill, A.ZagPrefill: self._do_prefill, A.PrefillPP: self._do_prefill,
                   A.Decode: self._do_decode, A.Migrate: self._do_migrate, A.MigratePartial: self._do_migrate,
                   A.Relay: self._do_relay, A.NvlBroadcast: self._do_params, A.TanzBroadcast: self._do_params,
                   A.RdmaBroadcast: self._do_params, A.LoadParams: self._do_params, A.ResetStatus: self._do_simple,
                   A.SetStatusReady: self._do_simple, A.ClearCache: self._do_simple, A.FilterBatch: self._do_filter}[t]
        self._spawn(self._guard(a, handler))

    def _purge_replica(self, rep: int) -> None:
        """Forget what the runtime remembers about batches on a replica that was lost."""
        for k in [k for k in self.cached if k[0] == rep]:
            del self.cached[k]
        held = {k[1] for k in self.cached}
        for b in [b for b in self.first_tokens if b not in held]:
            del self.first_tokens[b]

    def _remember(self, replica: int, batch) -> None:
        """Keep a worker's handle of a resident batch, unless the replica was lost while the call was in flight."""
        if self.ctl.state_name(replica) != "Inactive":
            self.cached[(replica, batch.id)] = batch

    def _deliver_one(self, rid: int, token: int, final: int, now: float) -> None:
        """`final`: 0 while the request goes on, else a key of FINISH_REASONS."""
        lr = self.requests.get(rid)
        if lr is None:
            return
        final = int(final)
        if lr.stopped:
            # ended at a stop sequence: what the worker produced after it is dropped, and the core's record goes when
            # the core ends the request (it filters it out of the worker's batch at the next step)
            if final:
                del self.requests[rid]
                self.ctl.pop_finished(rid)
            return
        lr.tokens.append(token)
        lr.times.append(now)
        if not final and lr.stop and self._stop_hit(lr):
            # every token is at least one byte of text, so the last `stop_window` tokens hold any stop sequence that
            # this token completed; an earlier occurrence would have ended the request already
            final, lr.stopped = 3, True
            self.ctl.client_gone(rid)                 # nobody wants its next tokens
            self.wake.set()
        if lr.stream:
            lr.queue.put_nowait(("token", token, final))
        if final:
            lr.finish_reason = FINISH_REASONS.get(final, "length")
            if lr.stopped:
                lr.entry = self.ctl.request(rid)      # a copy: the core still holds the request for one more step
            else:
                del self.requests[rid]
                lr.entry = self.ctl.pop_finished(rid)     # out of the core: its map of finished requests stays empty
            if self.exporter is not None:
                end = time.time()
                self.exporter.span("generate", child_traceparent(self.root_trace), end - (now - lr.t_submit), end,
                                   request_id=rid, input_tokens=len(lr.proto.input_tokens), generated_tokens=len(lr.tokens),
                                   first_token_s=lr.times[0] - lr.t_submit, parent_span_id=self.root_trace.split("-")[2])
            if not lr.done.done():
                lr.done.set_result(None)

    @staticmethod
    def _stop_hit(lr: LiveRequest) -> bool:
        try:
            text = lr.detok(lr.tokens[-lr.stop_window:])
        except Exception as e:  # noqa: BLE001 - a detokenizer that fails must not look like a failed worker call
            log.warning("request %d: detokenizer failed (%s); its stop sequences are ignored from here on", lr.id, e)
            lr.stop = ()
            return False
        return any(s in text for s in lr.stop)

    def _deliver(self, now: float) -> None:
        """Hand the tokens the core has released since the last call to their requests."""
        for rid, token, final in self.ctl.take_deliveries():
            self._deliver_one(rid, token, final, now)

    async def _guard(self, a, handler) -> None:
        tp = child_traceparent(self.root_trace)       # one span per dispatched operation
        t0, ok = time.time(), True
        try:
            CURRENT_TRACE.set(tp)
            await handler(a)
        except asyncio.CancelledError:
            raise
        except Exception as e:  # noqa: BLE001  an RPC failed: the replica is gone
            ok = False
            blamed = e.rank // self.tp if isinstance(e, RankFailure) else a.replica
            log.error("RPC for %s on replica %d failed (replica %d is taken as lost): %s", a.type.name, a.replica, blamed, e)
            if a.op_id:
                self.ctl.on_failure(a.op_id, self.now(), blamed)
                for rep in range(self.ctl.num_replicas):
                    if self.ctl.state_name(rep) == "Inactive":
                        self._purge_replica(rep)
                if self.health_interval_s > 0 and isinstance(e, RankFailure) and self.ctl.state_name(blamed) == "Inactive":
                    self.ctl.set_reachable(blamed, False)       # the detector will say when it answers again
        if self.exporter is not None:
            self.exporter.span(a.type.name, tp, t0, time.time(), replica=a.replica, peer=a.peer, batch_id=int(a.batch_id),
                               requests=len(a.request_ids), ok=ok, parent_span_id=self.root_trace.split("-")[2])
        self.wake.set()

    # ------------------------------------------------------------------ handlers
    async def _do_prefill(self, a) -> None:
        batch = self._batch_proto(a)
        ranks = self._ranks(a.replica)
        holder = a.replica          # the replica that holds the batch's KV when the call returns
        if a.type == A.Prefill and a.peer >= 0:
            # layer-progressive migration: the decode replica reserves and publishes its pages while the prefill
            # replica runs the pass and pushes each layer behind it; shard i pushes to shard i
            src, dst = list(a.src_ranks), list(a.dst_ranks)
            case = encode_prefill_case(pb.PREFILL_CASE_NORMAL, pb.PREFILL_CASE_MIGRATE_PROGRESSIVE)
            calls = [self.stubs[r].prefill_v2(batch, case, None, dst) for r in src] + \
                    [self.stubs[r].immigrate(batch, src, dst, 0, 0) for r in dst]
            ranks, holder = src + dst, a.peer
        elif a.type == A.Prefill:
            calls = [self.stubs[r].prefill_v2(batch, pb.PREFILL_CASE_NORMAL) for r in ranks]
        elif a.type == A.ZagPrefill:
            calls = [self.stubs[r].zag_prefill(batch, a.zag_seq, self.layers, pb.PREFILL_CASE_NAIVE_PP) for r in ranks]
        else:
            pp = pb.PipeParaInfo()
            if a.num_layer <= 0:
                pp.embedding_layer = 1
            else:
                pp.tfm_layer = a.num_layer
            case = encode_prefill_case(pb.PREFILL_CASE_NAIVE_PP, pb.PREFILL_CASE_IMMIGRATE)
            calls = [self.stubs[r].prefill_v2(batch, case, pp, a.dst_ranks) for r in ranks]
        answers = await self._all(ranks, calls)
        res = answers[0]
        if a.type == A.ZagPrefill and not res.generations and res.HasField("pp_info"):
            # taken over by a relay: the relay completion reports the hand-over to the core
            which = res.pp_info.WhichOneof("start_layer")
            self._zag_pp[a.batch_id] = res.pp_info.tfm_layer if which == "tfm_layer" else 0
            return
        if holder != a.replica:
            self._remember(holder, answers[-1].batch)
        elif res.HasField("batch"):
            self._remember(a.replica, res.batch)
        ids, toks, fins, reasons = core.parse_generations_full(res.raw)
        if (holder, a.batch_id) in self.cached:      # somebody will decode this batch: its first tokens travel with the first step
            self.first_tokens[a.batch_id] = {i: t for i, t in zip(ids, toks) if t >= 0}
        now = self.now()
        self.ctl.on_prefill_done_lists(a.op_id, ids, toks, fins, now, reasons)
        self._deliver(now)

    async def _do_decode(self, a) -> None:
        batches, lasts = [], []
        for bid in a.batch_ids:
            cb = self.cached.get((a.replica, bid))
            if cb is None:
                continue
            batches.append(cb)
            t = pb.Tokens()
            ft = self.first_tokens.pop(bid, None)
            if ft is not None:  # first decode step of this batch here: hand over the tokens prefill produced
                t.ids.extend(ft.get(rid, 0) for rid in cb.request_ids)
            lasts.append(t)
        ranks = self._ranks(a.replica)
        res = (await self._all(ranks, [self.stubs[r].decode_v2(batches, lasts, self.decode_steps) for r in ranks]))[0]
        for bid in a.batch_ids:
            self.cached.pop((a.replica, bid), None)
        if res.HasField("batch"):
            self._remember(a.replica, res.batch)
        now = self.now()
        self.ctl.on_decode_done_wire(a.op_id, res.raw, now)
        self._deliver(now)          # straight away: the next step of the loop may be a tick away

    async def _do_filter(self, a) -> None:
        """Drop the requests whose client went away from a worker's resident batch (`a.request_ids` stay)."""
        ranks = self._ranks(a.replica)
        res = (await self._all(ranks, [self.stubs[r].filter_batch(a.batch_id, list(a.request_ids)) for r in ranks]))[0]
        if res.HasField("batch"):
            self._remember(a.replica, res.batch)
        self.ctl.on_filter_done(a.op_id, self.now())

    async def _do_migrate(self, a) -> None:
        batch = self._batch_proto(a)
        partial = a.partial if a.type == A.MigratePartial else 0
        src, dst = list(a.src_ranks), list(a.dst_ranks)
        calls = [self.stubs[r].migrate(batch, src, dst, partial, a.num_layer) for r in src] + \
                [self.stubs[r].immigrate(batch, src, dst, partial, a.num_layer) for r in dst]
        res = await self._all(src + dst, calls)
        self.cached.pop((a.replica, a.batch_id), None)
        self._remember(a.peer, res[-1].batch)
        self.ctl.on_migrate_done(a.op_id, self.now())

    async def _do_relay(self, a) -> None:
        new_ranks = self._ranks(a.replica)
        # shard i of the new replica hands its copy of the activations to shard i of the old one
        old = list(a.src_ranks)
        res = (await self._all(new_ranks, [self.stubs[r].relay(old[i % len(old)], a.final)
                                           for i, r in enumerate(new_ranks)]))[0]
        has = res.HasField("batch_id")
        next_layer = 0
        if has:
            # the hand-over layer travels in the ZagPrefill response of that batch (bounded wait for it)
            for _ in range(4000):
                if res.batch_id in self._zag_pp:
                    next_layer = self._zag_pp.pop(res.batch_id)
                    break
                await asyncio.sleep(0.0005)
        self.ctl.on_relay_done(a.op_id, has, res.batch_id if has else 0, next_layer, self.now())

    async def _do_params(self, a) -> None:
        if a.mock:
            await asyncio.sleep(self.cfg.mock_load_ms * 1e-3)
            await self._all(list(a.dst_ranks), [self.stubs[r].set_status_ready() for r in a.dst_ranks])
        elif a.type == A.LoadParams:
            await self._all(list(a.dst_ranks), [self.stubs[r].load_params(a.load_case, self.cfg.model_name, self.model_path)
                                                for r in a.dst_ranks])
        else:
            kind = {A.NvlBroadcast: "nvl", A.TanzBroadcast: "tanz", A.RdmaBroadcast: "rdma"}[a.type]
            # every participant receives the same request and derives its role (src/service/service.cc:1341-1347)
            ranks = list(a.src_ranks) + list(a.dst_ranks)
            await self._all(ranks, [self.stubs[r].broadcast(kind, a.src_ranks, a.dst_ranks) for r in ranks])
        self.ctl.on_params_done(a.op_id, self.now())

    async def _do_simple(self, a) -> None:
        if self.ctl.state_name(a.replica) == "Inactive" and a.type in (A.ClearCache, A.ResetStatus):
            # housekeeping on a replica that is out of service (lost, or just unloaded): some of its ranks may be
            # gone, which is no reason to declare anything else lost
            if a.type == A.ClearCache and a.final:
                self._purge_replica(a.replica)
                calls = [self.stubs[r].clear_cache(None) for r in self._ranks(a.replica)]
            elif a.type == A.ClearCache:
                self.cached.pop((a.replica, a.batch_id), None)
                calls = [self.stubs[r].clear_cache(a.batch_id) for r in self._ranks(a.replica)]
            else:
                calls = [self.stubs[r].reset_status() for r in a.dst_ranks]
            for res in await asyncio.gather(*calls, return_exceptions=True):
                if isinstance(res, Exception):
                    log.debug("%s on inactive replica %d: %s", a.type.name, a.replica, res)
            return
        if a.type == A.ClearCache:
            self.cached.pop((a.replica, a.batch_id), None)
            if not any(k[1] == a.batch_id for k in self.cached):
                self.first_tokens.pop(a.batch_id, None)
            await asyncio.gather(*[self.stubs[r].clear_cache(a.batch_id) for r in self._ranks(a.replica)])
        elif a.type == A.ResetStatus:
            await asyncio.gather(*[self.stubs[r].reset_status() for r in a.dst_ranks])
        elif a.type == A.SetStatusReady:
            await asyncio.gather(*[self.stubs[r].set_status_ready() for r in a.dst_ranks])
