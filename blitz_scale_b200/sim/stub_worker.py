"""GPU-less worker backend: the full RPC surface with seeded pseudo-random tokens.

It keeps real batch / page bookkeeping (the native PagePool and Batch), so FilterBatch, ClearCache,
Migrate / Immigrate and block accounting behave like a GPU worker, and it models parameter state
(ready flags, per-unit arrival during a broadcast) with sleeps, which is what the reference's
`mock_transfer` feature and its SetStatusReady / ResetStatus RPCs are for
(router_v2/src/replica/disaggregation.rs:454-518, proto/generate.proto:46-49).  Tokens depend only on
(seed, request id, position), so a replayed trace yields identical token streams.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional

from ..pb.schema import pb
from ..runtime import core
from ..worker.service import Backend, seq_spec_from_request
from ..worker.stopping import StopSequences


def stub_token(seed: int, request_id: int, position: int, vocab: int = 32000) -> int:
    z = (seed * 0x9E3779B97F4A7C15 + request_id * 0xBF58476D1CE4E5B9 + position * 0x94D049BB133111EB) & (2 ** 64 - 1)
    z ^= z >> 31
    z = (z * 0xD6E8FEB86659FD93) & (2 ** 64 - 1)
    z ^= z >> 29
    return int(z % vocab)


class StubBackend(Backend):
    def __init__(self, rank: int = 0, world: int = 1, *, seed: int = 0, layers: int = 2, vocab: int = 32000,
                 num_pages: int = 4096, page_size: int = 64, ready: bool = True, prefill_tokens_per_s: float = 2e5,
                 decode_step_s: float = 0.002, load_s: float = 0.2, peers: Optional[Dict[int, "StubBackend"]] = None,
                 eos_token: int = -1):
        self.rank, self.world, self.seed, self.layers, self.vocab = rank, world, seed, layers, vocab
        self.eos_token = eos_token
        self.stopper = StopSequences()        # no tokenizer here: stop sequences match the `<id>` text of the generations
        self.pool = core.PagePool(num_pages, page_size)
        self.status = core.ModelStatus(layers)
        if ready:
            self.status.set_ready()
        self.batches: Dict[int, "core.Batch"] = {}
        self.lock = threading.RLock()
        self.prefill_rate, self.decode_step_s, self.load_s = prefill_tokens_per_s, decode_step_s, load_s
        self.zag = core.ZigzagScheduler(layers, 16)
        self.zag_events: Dict[int, threading.Event] = {}
        self.zag_relayed: Dict[int, int] = {}
        self.transfer_done = threading.Event()
        self.transfer_done.set()
        self.counters = {"prefill": 0, "decode": 0, "migrate": 0, "immigrate": 0, "migrate_progressive": 0}

    # ------------------------------------------------------------------ helpers
    def info(self) -> dict:
        return {"ready": self.status.fully_loaded(), "dtype": "float32", "device_type": "cpu",
                "ranks": {"rank": self.rank, "world": self.world}}

    def _specs(self, batch) -> List["core.SeqSpec"]:
        self.stopper.add(batch)
        return [seq_spec_from_request(r, [1] * max(1, len(r.inputs.split())), self.eos_token) for r in batch.requests]

    def _cached(self, b) -> Optional[object]:
        ids = b.unfinished_ids()
        if not ids:
            return None
        return pb.CachedBatch(id=b.id, request_ids=ids, size=len(ids), max_tokens=b.max_tokens())

    def _emit(self, b, new_tokens: List[int]):
        return b.encode_generations(new_tokens)

    def _step(self, b, prefill: bool):
        toks = [stub_token(self.seed, rid, pl + n, self.vocab) for (rid, _, n), pl in zip(b.emit_info(), b.prompt_lens())]
        rows, _temp, top_k, _top_p, seeds = b.sampling_rows()
        for row, k, sd in zip(rows, top_k, seeds):      # stand-in for sampling: a function of the (mixed) seed, within top-k
            toks[row] = (sd & 0x7FFFFFFF) % (k if k > 0 else self.vocab)
        if prefill:
            b.mark_prefilled()
        b.append_tokens(toks, not prefill)
        self.stopper.check(b)
        return toks

    # ------------------------------------------------------------------ inference
    def prefill(self, batch, forward_case, pp_info, pipe_peer):
        if not self.status.fully_loaded():
            raise RuntimeError("model not loaded")
        with self.lock:
            if forward_case & pb.PREFILL_CASE_NAIVE_PP and batch.id in self.batches:
                b = self.batches[batch.id]  # continuation of a relayed batch whose pages were reserved here
            else:
                b = core.Batch(batch.id, self.pool)
                if not b.add_prompts(self._specs(batch)):
                    raise RuntimeError("out of KV pages")
            frac = 1.0
            if pp_info is not None and pp_info.WhichOneof("start_layer") == "tfm_layer":
                frac = 1.0 - pp_info.tfm_layer / max(1, self.layers)
        time.sleep(frac * b.num_prompt_tokens() / self.prefill_rate)
        with self.lock:
            toks = self._step(b, True)
            gens = self._emit(b, toks)
            b.filter(b.unfinished_ids())
            b.decode = True
            self.counters["prefill"] += 1
            if forward_case & pb.PREFILL_CASE_MIGRATE_PROGRESSIVE and pipe_peer:
                # every layer's KV went to the decode replica as the layer ran: nothing of the batch stays here
                self.counters["migrate_progressive"] += 1
                self.batches.pop(b.id, None)
                b.clear()
                return gens, None, None
            if b.size:
                self.batches[b.id] = b
            else:
                self.batches.pop(b.id, None)
            return gens, self._cached(b) if b.size else None, None

    def zag_prefill(self, batch, forward_case, pp_info, zag_layers, zag_seq):
        """Serve while loading: run as far as the loaded layers allow; a relay may take the batch away."""
        with self.lock:
            b = core.Batch(batch.id, self.pool)
            if not b.add_prompts(self._specs(batch)):
                raise RuntimeError("out of KV pages")
            self.batches[batch.id] = b
            slot = self.zag.add_task(batch.id, zag_seq, b.num_prompt_tokens())
            if slot < 0:
                raise RuntimeError("no activation slot")
            ev = self.zag_events[batch.id] = threading.Event()
        per_layer = b.num_prompt_tokens() / self.prefill_rate / max(1, self.layers)
        while True:
            with self.lock:
                if batch.id in self.zag_relayed:
                    k = self.zag_relayed.pop(batch.id)
                    pp = pb.PipeParaInfo()
                    if k < 0:
                        pp.embedding_layer = 1
                    else:
                        pp.tfm_layer = k
                    return [], pb.CachedBatch(id=b.id, request_ids=b.unfinished_ids(), size=b.size,
                                              max_tokens=b.max_tokens()), pp
                self.zag.set_loaded(self.status.embed_ready, self.status.layers_ready, self.status.head_ready)
                d = self.zag.next()
                mine = d.step in (core.ZagStep.Embed, core.ZagStep.Layer, core.ZagStep.Head) and d.batch_id == batch.id
                if mine:
                    done = self.zag.complete(d)
                    if done:
                        toks = self._step(b, True)
                        gens = self._emit(b, toks)
                        b.filter(b.unfinished_ids())
                        b.decode = True
                        if not b.size:
                            self.batches.pop(b.id, None)
                        self.zag_events.pop(batch.id, None)
                        return gens, self._cached(b) if b.size else None, None
            if mine and d.step == core.ZagStep.Layer:
                time.sleep(per_layer)
            else:
                ev.wait(0.001)

    def relay(self, rank, relax_not_head):
        with self.lock:
            r = self.zag.relay(bool(relax_not_head))
            if r is None:
                return None
            self.zag.release_slot(r.slot)
            self.zag_relayed[r.batch_id] = r.next_layer
            ev = self.zag_events.get(r.batch_id)
            if ev:
                ev.set()
            return r.batch_id, r.seq_num

    def decode(self, batches, last_iter_tokens, steps: int = 1):
        gens, cb = self._decode_once(batches, last_iter_tokens)
        for _ in range(1, max(1, steps)):
            if cb is None:
                break
            more, cb = self._decode_once([cb], [])
            gens += more
        return gens, cb

    def _decode_once(self, batches, last_iter_tokens):
        with self.lock:
            # tokens produced by prefill elsewhere travel with a migrated batch and are appended before the
            # first decode step here (src/service/service.cc:657-679); then all batches merge into the first
            for i, cb in enumerate(batches):
                ids = list(last_iter_tokens[i].ids) if i < len(last_iter_tokens) else []
                bi = self.batches[cb.id]
                if ids and len(ids) == bi.size and bi.none_generated():
                    bi.append_tokens(ids, False)
            first = self.batches[batches[0].id]
            for cb in batches[1:]:
                other = self.batches.pop(cb.id)
                first.extend(other)
            b = first
        time.sleep(self.decode_step_s)
        with self.lock:
            toks = self._step(b, False)
            gens = self._emit(b, toks)
            b.filter(b.unfinished_ids())
            self.counters["decode"] += 1
            if not b.size:
                self.batches.pop(b.id, None)
                return gens, None
            return gens, self._cached(b)

    def clear_cache(self, batch_id):
        with self.lock:
            ids = [batch_id] if batch_id is not None else list(self.batches)
            for i in ids:
                b = self.batches.pop(i, None)
                if b is not None:
                    b.clear()

    def filter_batch(self, batch_id, request_ids):
        with self.lock:
            b = self.batches[batch_id]
            b.filter(list(request_ids))
            return pb.CachedBatch(id=b.id, request_ids=b.unfinished_ids(), size=b.size, max_tokens=b.max_tokens())

    # ------------------------------------------------------------------ KV migration
    def migrate(self, batch, src, dst, partial=0, num_layer=0):
        with self.lock:
            b = self.batches.get(batch.id)
            ntok = b.num_prompt_tokens() if b is not None else 0
        time.sleep(ntok / 5e6)
        with self.lock:
            self.counters["migrate"] += 1
            cb = pb.CachedBatch(id=batch.id, request_ids=[r.id for r in batch.requests], size=len(batch.requests),
                                max_tokens=batch.max_tokens)
            # this worker's share of the batch (all layers, or its half of a relayed batch) has left: free it
            if b is not None:
                self.batches.pop(batch.id, None)
                b.clear()
            return cb

    def immigrate(self, batch, src, dst, partial=0, num_layer=0):
        with self.lock:
            b = self.batches.get(batch.id)
            if b is None:
                b = core.Batch(batch.id, self.pool)
                if not b.add_prompts(self._specs(batch)):
                    raise RuntimeError("out of KV pages")
                b.mark_prefilled()
                b.decode = True
                if b.size:
                    self.batches[batch.id] = b
            self.counters["immigrate"] += 1
            return pb.CachedBatch(id=b.id, request_ids=b.request_ids(), size=b.size, max_tokens=b.max_tokens())

    # ------------------------------------------------------------------ parameters
    def _arrive(self, total_s: float):
        self.transfer_done.clear()
        n = self.layers + 2

        def run():
            for u in range(n):
                time.sleep(total_s / n)
                with self.lock:
                    self.status.unit_arrived(u)
            self.transfer_done.set()
        threading.Thread(target=run, daemon=True).start()

    def broadcast(self, kind, src_ranks, dst_ranks):
        if self.rank in dst_ranks:
            with self.lock:
                self.status.reset()
            self._arrive(self.load_s)
            self.transfer_done.wait()
        else:
            time.sleep(self.load_s)

    def send_params(self, dst):
        time.sleep(self.load_s)

    def recv_params(self, src):
        with self.lock:
            self.status.reset()
        self._arrive(self.load_s)

    def wait_transfer_done(self):
        self.transfer_done.wait()

    def load_params(self, load_case, model_name, model_path):
        time.sleep(self.load_s * (1.0 if load_case == pb.LOAD_FROM_HOST_MEM else 4.0))
        with self.lock:
            self.status.set_ready()

    def reset_status(self):
        with self.lock:
            self.status.reset()
            self.zag.reset()

    def set_status_ready(self):
        with self.lock:
            self.status.set_ready()

    def warmup(self, req) -> int:
        return self.pool.total_pages * self.pool.page_size


def main(argv=None) -> None:
    """`python -m blitz_scale_b200.sim.stub_worker --rank R --world N --port P --config cluster.json`"""
    import argparse
    import asyncio
    import json
    import signal

    from ..worker.service import serve
    ap = argparse.ArgumentParser("blitz-stub-worker")
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--world", type=int, default=1)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, required=True)
    ap.add_argument("--config", default="")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--load-seconds", type=float, default=0.2)
    ap.add_argument("--decode-step-ms", type=float, default=2.0, help="simulated duration of one decode step")
    ap.add_argument("--prefill-tokens-per-s", type=float, default=2e5, help="simulated prefill rate")
    a = ap.parse_args(argv)
    ready = True
    if a.config:
        ready = json.load(open(a.config))["init_states"][a.rank] != "Inactive"
    backend = StubBackend(a.rank, a.world, seed=a.seed, layers=a.layers, ready=ready, load_s=a.load_seconds,
                          decode_step_s=a.decode_step_ms * 1e-3, prefill_tokens_per_s=a.prefill_tokens_per_s)

    async def run():
        stop = asyncio.Event()
        loop = asyncio.get_running_loop()
        for sig in (signal.SIGINT, signal.SIGTERM):
            loop.add_signal_handler(sig, stop.set)
        await serve(backend, a.host, a.port, stop_event=stop)
    asyncio.run(run())


if __name__ == "__main__":
    main()
