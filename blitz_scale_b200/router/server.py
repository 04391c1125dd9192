"""HTTP front of the router (TGI-compatible surface of router_v2/src/server.rs:892-947).

Routes: POST `/`, `/generate`, `/invocations` (JSON in, JSON out, timing headers), POST `/generate_stream`
(server-sent events), GET `/info`, `/health`, `/ping`, `/metrics` (Prometheus text), `/docs` (OpenAPI
summary), POST `/modify_cluster_state` (manual scaling, `manually_scale` feature only).  The timing
headers are the ones the trace client consumes (router_v2/src/server.rs:252-349): x-first-token-time,
x-queue-time, x-inference-time, x-{max,avg,p90,p95,p99}-time-between-tokens, x-first-decode-token-time,
x-input-length, x-output-length, ...; TTFT is measured to the prefill-done event and the first
inter-token interval is excluded from the TBT statistics (router_v2/src/infer.rs:324-333).

Tokenization: without a tokenizer file the router uses a deterministic word-hash tokenizer (one id
per whitespace-separated word), enough for trace replay; `input_tokens` may also be posted directly.
"""
from __future__ import annotations

import argparse
import asyncio
import bisect
from concurrent.futures import ThreadPoolExecutor
import json
import logging
import os
import signal
import time
import zlib
from typing import List, Optional

from aiohttp import web

from ..pb.schema import pb
from ..runtime import core
from .runtime import FINISH_REASONS, RouterRuntime

log = logging.getLogger("blitz.router.http")


class WordHashTokenizer:
    def __init__(self, vocab: int = 32000):
        self.vocab = vocab

    def encode(self, text: str) -> List[int]:
        return [zlib.crc32(w.encode()) % self.vocab for w in text.split()]

    def decode(self, ids: List[int]) -> str:
        return " ".join(f"<{i}>" for i in ids)

    def piece(self, tid: int) -> str:
        return f"<{tid}>"

    def special(self, tid: int) -> bool:
        return False


class NativeTokenizer:
    """tokenizer.json through the native BPE tokenizer (the reference runs a pool of tokenizer workers,
    router_v2/src/validation.rs:152-305; here `encode` releases the GIL and runs on the router's thread pool)."""

    def __init__(self, path: str):
        self.t = core.Tokenizer.from_file(path)
        self.vocab = self.t.num_ids()

    def encode(self, text: str) -> List[int]:
        return list(self.t.encode(text))

    def decode(self, ids: List[int]) -> str:
        return self.t.decode(list(ids), True)

    def piece(self, tid: int) -> str:
        return self.t.decode([tid], False)

    def special(self, tid: int) -> bool:
        return bool(self.t.is_special(tid))


def _pct(xs: List[float], q: float) -> float:
    if not xs:
        return 0.0
    s = sorted(xs)
    return s[min(len(s) - 1, int(q * len(s)))]


class Metrics:
    """Prometheus exposition with the reference's metric names (router_v2/src/server.rs:811-857)."""
    BUCKETS = [0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10, 30]

    SIZE_BUCKETS = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384]
    _SIZES = ("blitz_request_generated_tokens", "blitz_request_input_length", "blitz_request_max_new_tokens",
              "blitz_batch_next_size")

    def __init__(self):
        self.counters = {"blitz_request_count": 0, "blitz_request_success": 0, "blitz_request_failure": 0}
        names = ("blitz_request_duration", "blitz_request_validation_duration", "blitz_request_queue_duration",
                 "blitz_request_inference_duration", "blitz_request_mean_time_per_token_duration",
                 "blitz_request_skipped_tokens") + self._SIZES
        # fixed-size state per histogram: [bucket upper bounds, count per bucket (last = overflow), sum, count]
        self.hist = {n: [self.SIZE_BUCKETS if n in self._SIZES else self.BUCKETS, None, 0.0, 0] for n in names}
        for h in self.hist.values():
            h[1] = [0] * (len(h[0]) + 1)

    def observe(self, name: str, v: float) -> None:
        h = self.hist[name]
        h[1][bisect.bisect_left(h[0], v)] += 1
        h[2] += v
        h[3] += 1

    def render(self, rt: RouterRuntime) -> str:
        out = []
        ctl = rt.ctl
        merged = dict(self.counters)
        for k, v in ctl.counters().items():
            merged[k] = merged.get(k, 0) + v if k not in ("blitz_request_count",) else v
        for k, v in sorted(merged.items()):
            out += [f"# TYPE {k} counter", f"{k} {v}"]
        gauges = dict(ctl.gauges())
        gauges["blitz_queue_size"] = ctl.queue_size
        for k, v in sorted(gauges.items()):
            out += [f"# TYPE {k} gauge", f"{k} {v}"]
        for name, (bounds, counts, total, n) in sorted(self.hist.items()):
            out.append(f"# TYPE {name} histogram")
            acc = 0
            for b, c in zip(bounds, counts):
                acc += c
                out.append(f'{name}_bucket{{le="{b}"}} {acc}')
            out.append(f'{name}_bucket{{le="+Inf"}} {n}')
            out.append(f"{name}_sum {total}")
            out.append(f"{name}_count {n}")
        return "\n".join(out) + "\n"


class RouterApp:
    def __init__(self, rt: RouterRuntime, *, model_name: str = "llama3_8b", max_input_length: int = 4095,
                 max_total_tokens: int = 4096, max_concurrent: int = 4096, vocab: int = 32000,
                 tokenizer_path: str = "", tokenizer_workers: int = 2, max_best_of: int = 2, max_stop_sequences: int = 4,
                 max_top_n_tokens: int = 5, cors_allow_origin: Optional[List[str]] = None):
        self.rt = rt
        self.tok = NativeTokenizer(tokenizer_path) if tokenizer_path else WordHashTokenizer(vocab)
        self.tok_pool = ThreadPoolExecutor(max_workers=max(1, tokenizer_workers), thread_name_prefix="tokenizer")
        self.limits = core.ValidationLimits()
        self.limits.max_input_length, self.limits.max_total_tokens = max_input_length, max_total_tokens
        self.limits.max_best_of, self.limits.max_stop_sequences = max_best_of, max_stop_sequences
        self.limits.max_top_n_tokens = max_top_n_tokens
        self.cors = list(cors_allow_origin or [])
        self.model_name = model_name
        try:
            from ..models.config import get_config
            self.model_vocab = get_config(model_name).vocab
        except Exception:  # noqa: BLE001 - unknown model name: no id range to enforce
            self.model_vocab = 0
        if not tokenizer_path and self.model_vocab:
            self.tok = WordHashTokenizer(min(vocab, self.model_vocab))
        self.sem = asyncio.Semaphore(max_concurrent)
        self.max_concurrent, self.tokenizer_workers = max_concurrent, max(1, tokenizer_workers)
        self._worker_info = None          # dtype / device of the workers, asked once (the Info RPC of the contract)
        self.metrics = Metrics()
        self.app = web.Application(client_max_size=64 << 20, middlewares=[self._cors_middleware] if self.cors else [])
        r = self.app.router
        r.add_post("/generate", self.generate)
        for path in ("/", "/invocations"):
            r.add_post(path, self.compat_generate)
        r.add_post("/generate_stream", self.generate_stream)
        r.add_get("/info", self.info)
        r.add_get("/health", self.health)
        r.add_get("/", self.health)
        r.add_get("/ping", self.health)
        r.add_get("/metrics", self.prom)
        r.add_get("/docs", self.docs)
        r.add_post("/modify_cluster_state", self.modify_cluster_state)

    @web.middleware
    async def _cors_middleware(self, req: web.Request, handler):
        """Cross-origin access for the origins given with --cors-allow-origin ("*" allows any)."""
        origin = req.headers.get("Origin", "")
        allowed = origin and ("*" in self.cors or origin in self.cors)
        if req.method == "OPTIONS" and allowed:
            resp = web.Response(status=204)
        else:
            resp = await handler(req)
        if allowed:
            resp.headers["Access-Control-Allow-Origin"] = "*" if "*" in self.cors else origin
            resp.headers["Access-Control-Allow-Methods"] = "GET, POST, OPTIONS"
            resp.headers["Access-Control-Allow-Headers"] = req.headers.get("Access-Control-Request-Headers", "Content-Type")
            resp.headers["Vary"] = "Origin"
        return resp

    # ------------------------------------------------------------------ request parsing
    async def _parse(self, body):
        """(token ids, parameters, error text).  Anything in the body that has the wrong type or shape is a validation
        error (HTTP 422), as a typed request structure makes it in the reference, never a server error."""
        t0 = time.perf_counter()
        try:
            toks, g, err = await self._parse_checked(body)
        except (TypeError, ValueError, AttributeError, KeyError, OverflowError) as e:
            return None, None, f"invalid request body: {e}"
        if g is not None:
            g.validation_s = time.perf_counter() - t0      # tokenization + checks (the reference's validation stage)
        return toks, g, err

    async def _parse_checked(self, body):
        if not isinstance(body, dict):
            raise TypeError("a JSON object is expected")
        p = body.get("parameters")
        if p is not None and not isinstance(p, dict):
            raise TypeError("`parameters` must be an object")
        p = p or {}
        if "input_tokens" in body:
            if not isinstance(body["input_tokens"], list) or not all(isinstance(t, int) and not isinstance(t, bool)
                                                                     for t in body["input_tokens"]):
                raise TypeError("`input_tokens` must be a list of integers")
            toks = [int(t) for t in body["input_tokens"]]
            if self.model_vocab and any(t < 0 or t >= self.model_vocab for t in toks):
                # an id outside the embedding table would make the worker's lookup fail the whole batch
                return toks, None, f"input_tokens must lie in [0, {self.model_vocab})"
        else:
            if not isinstance(body.get("inputs", ""), str):
                raise TypeError("`inputs` must be a string")
            toks = await asyncio.get_running_loop().run_in_executor(self.tok_pool, self.tok.encode, body.get("inputs", ""))
        g = core.GenerateParams()
        g.input_len = len(toks)
        g.max_new_tokens = int(p.get("max_new_tokens", 20))
        g.best_of = int(p.get("best_of") or 1)
        g.do_sample = bool(p.get("do_sample", False))
        g.temperature = float(p.get("temperature") or 1.0)
        g.repetition_penalty = float(p.get("repetition_penalty") or 1.0)
        g.top_p = float(p.get("top_p") or 1.0)
        g.typical_p = float(p.get("typical_p") or 1.0)
        g.top_k = int(p.get("top_k") or 0)
        g.top_n_tokens = int(p.get("top_n_tokens") or 0)
        if not isinstance(p.get("stop") or [], list) or not all(isinstance(x, str) for x in p.get("stop") or []):
            raise TypeError("`stop` must be a list of strings")
        g.stop = [x for x in (p.get("stop") or []) if x]
        g.num_stop_sequences = len(g.stop)
        # the end-of-sequence token ends a request unless the request opts out (trace replays that fix output lengths do)
        g.ignore_eos = bool(p.get("ignore_eos_token", False))
        if p.get("truncate") is not None:
            if int(p["truncate"]) <= 0:
                raise ValueError("`truncate` must be strictly positive")
            g.truncate = int(p["truncate"])
            toks = toks[-int(p["truncate"]):]
            g.input_len = len(toks)
        g.has_seed = p.get("seed") is not None
        err = core.validate_request(g, self.limits)
        if not err and g.best_of > 1:
            # candidates would have to be ranked by sequence log-probability, which the workers do not return
            # (Generation.logprobs is always 0, as in the reference's workers): refuse instead of ignoring the field
            err = "`best_of` > 1 is not supported: the workers return no log-probabilities to rank candidates by"
        if not err and g.do_sample:
            # carried to the worker in the request's NextTokenChooserParameters; greedy requests carry none
            seed = int(p["seed"]) if g.has_seed else zlib.crc32(repr((toks[:16], time.time_ns())).encode())
            g.chooser = pb.NextTokenChooserParameters(
                temperature=g.temperature, top_k=g.top_k, top_p=g.top_p, typical_p=g.typical_p, do_sample=True,
                seed=seed & 0xFFFFFFFFFFFFFFFF, repetition_penalty=g.repetition_penalty, watermark=False)
        return toks, g, err

    def _finish(self, lr, toks, g):
        """Timing headers and metrics of a finished request, from the router-clock time of each token delivery."""
        times, out = lr.times, lr.tokens
        t_start = lr.t_submit
        total = (times[-1] if times else self.rt.now()) - t_start
        validation = float(getattr(g, "validation_s", 0.0))
        t_first = times[0] if times else t_start
        t_first_dec = times[1] if len(times) > 1 else t_first
        # the interval between the prefill token and the first decode token contains the KV migration: it is reported
        # on its own and is not a time-between-tokens sample
        tbt = [b - a for a, b in zip(times[1:], times[2:])]
        e = lr.entry
        queue_s = (e.t_batched - e.t_arrival) if e is not None and e.t_batched >= 0 else 0.0
        stats = {
            "x-compute-type": "gpu+optimized", "x-total-time": int((total + validation) * 1e3),
            "x-validation-time": int(validation * 1e3),
            "x-queue-time": int(queue_s * 1e3), "x-inference-time": int((total - queue_s) * 1e3),
            "x-first-token-time": int((t_first - t_start) * 1e3),
            "x-first-decode-token-time": int((t_first_dec - t_start) * 1e3),
            "x-time-per-token": int(total * 1e3 / max(1, len(out))),
            "x-max-time-between-tokens": int(max(tbt, default=0.0) * 1e3),
            "x-avg-time-between-tokens": int((sum(tbt) / len(tbt) if tbt else 0.0) * 1e3),
            "x-p90-time-between-tokens": int(_pct(tbt, 0.90) * 1e3), "x-p95-time-between-tokens": int(_pct(tbt, 0.95) * 1e3),
            "x-p99-time-between-tokens": int(_pct(tbt, 0.99) * 1e3),
            "x-input-length": len(toks), "x-output-length": len(out), "x-generated-tokens": len(out),
        }
        m = self.metrics
        m.observe("blitz_request_duration", total + validation)
        m.observe("blitz_request_validation_duration", validation)
        m.observe("blitz_request_queue_duration", queue_s)
        m.observe("blitz_request_inference_duration", total - queue_s)
        m.observe("blitz_request_mean_time_per_token_duration", total / max(1, len(out)))
        m.observe("blitz_request_generated_tokens", len(out))
        m.observe("blitz_request_input_length", len(toks))
        m.observe("blitz_request_max_new_tokens", g.max_new_tokens)
        m.observe("blitz_request_skipped_tokens", 0.0)     # no speculation: a token is never skipped
        return list(out), stats, (lr.finish_reason or "length")

    @staticmethod
    def _unavailable(text):
        return web.HTTPServiceUnavailable(text=json.dumps({"error": text, "error_type": "generation"}),
                                          content_type="application/json")

    async def _collect(self, toks, g):
        """Whole response at once: the handler sleeps until the last token instead of waking for every token."""
        lr = self.rt.submit(toks, g.max_new_tokens, stream=False, parameters=getattr(g, "chooser", None),
                            ignore_eos=g.ignore_eos, stop=g.stop, detok=self.tok.decode)
        try:
            err = await lr.done
        except asyncio.CancelledError:        # the client closed the connection: stop generating for it
            self.rt.client_gone(lr.id)
            raise
        if err:
            raise self._unavailable(err)
        return self._finish(lr, toks, g)

    async def _run(self, toks, g):
        """Token by token (server-sent events); the last item carries (tokens, timing headers)."""
        lr = self.rt.submit(toks, g.max_new_tokens, parameters=getattr(g, "chooser", None), ignore_eos=g.ignore_eos,
                            stop=g.stop, detok=self.tok.decode)
        try:
            while True:
                ev = await lr.queue.get()
                if ev[0] == "error":
                    raise self._unavailable(ev[1])
                _, tok, final = ev
                yield tok, final, None
                if final:
                    break
        except (asyncio.CancelledError, GeneratorExit, ConnectionResetError):
            if not lr.done.done():
                self.rt.client_gone(lr.id)    # the consumer left before the last token: stop generating for it
            raise
        yield None, True, self._finish(lr, toks, g)

    # ------------------------------------------------------------------ handlers
    async def compat_generate(self, req: web.Request) -> web.StreamResponse:
        """`/` and `/invocations`: `stream` in the body picks the event stream; otherwise the generation comes back
        inside a one-element list (router_v2/src/server.rs:66-86)."""
        try:
            body = await req.json()
        except Exception:  # noqa: BLE001
            return web.json_response({"error": "invalid JSON", "error_type": "validation"}, status=422)
        if isinstance(body, dict) and body.get("stream"):
            return await self.generate_stream(req)
        return await self.generate(req, wrap=True)

    async def generate(self, req: web.Request, wrap: bool = False) -> web.Response:
        try:
            body = await req.json()
        except Exception:  # noqa: BLE001
            return web.json_response({"error": "invalid JSON", "error_type": "validation"}, status=422)
        toks, g, err = await self._parse(body)
        if err:
            self.metrics.counters["blitz_request_failure"] += 1
            return web.json_response({"error": err, "error_type": "validation"}, status=422)
        if self.sem.locked():
            return web.json_response({"error": "Model is overloaded", "error_type": "overloaded"}, status=429)
        async with self.sem:
            out, stats, reason = await self._collect(toks, g)
        details = None
        if (body.get("parameters") or {}).get("details"):
            chooser = getattr(g, "chooser", None)
            details = {"finish_reason": reason, "generated_tokens": len(out), "prefill": [],
                       "seed": int(chooser.seed) if chooser is not None else None,
                       "tokens": [{"id": t, "text": self.tok.piece(t), "logprob": 0.0, "special": self.tok.special(t)} for t in out]}
        text = self.tok.decode(out)
        if (body.get("parameters") or {}).get("return_full_text") and isinstance(body.get("inputs"), str):
            text = body["inputs"] + text
        payload = {"generated_text": text, "details": details}
        return web.json_response([payload] if wrap else payload,
                                 headers={k: str(v) for k, v in stats.items()})

    async def generate_stream(self, req: web.Request) -> web.StreamResponse:
        try:
            body = await req.json()
        except Exception:  # noqa: BLE001
            return web.json_response({"error": "invalid JSON", "error_type": "validation"}, status=422)
        toks, g, err = await self._parse(body)
        if err:
            return web.json_response({"error": err, "error_type": "validation"}, status=422)
        resp = web.StreamResponse(headers={"Content-Type": "text/event-stream", "Cache-Control": "no-cache"})
        await resp.prepare(req)
        ids: List[int] = []
        agen = self._run(toks, g)
        try:
            async for tok, final, done in agen:
                if done is not None:
                    continue
                ids.append(tok)
                ev = {"token": {"id": tok, "text": self.tok.piece(tok), "logprob": 0.0, "special": self.tok.special(tok)},
                      "generated_text": None, "details": None}
                if final:
                    # the last event carries the whole text and why the request ended
                    ev["generated_text"] = self.tok.decode(ids)
                    ev["details"] = {"finish_reason": FINISH_REASONS.get(int(final), "length"), "generated_tokens": len(ids)}
                await resp.write(f"data:{json.dumps(ev)}\n\n".encode())
            await resp.write_eof()
        except (ConnectionResetError, asyncio.CancelledError):
            pass  # the client went away
        finally:
            await agen.aclose()      # an unfinished stream tells the core that its client is gone
        return resp

    async def info(self, req):
        """Model and router parameters, with the fields of the reference's answer (router_v2/src/lib.rs:99-137; it
        hard-codes the shard part, here the first worker that answers `Info` is asked once) plus the replica states."""
        if self._worker_info is None:
            for stub in self.rt.stubs:
                try:
                    wi = await stub.info()
                    self._worker_info = (wi.dtype, wi.device_type)
                    break
                except Exception:  # noqa: BLE001 - that worker is away; the next one may answer
                    continue
        dtype, device = self._worker_info or ("unknown", "unknown")
        cfg = self.rt.cfg
        return web.json_response({
            "model_id": self.model_name, "model_sha": None, "model_dtype": dtype, "model_device_type": device,
            "model_pipeline_tag": "text-generation", "max_concurrent_requests": self.max_concurrent,
            "max_best_of": self.limits.max_best_of, "max_stop_sequences": self.limits.max_stop_sequences,
            "max_input_length": self.limits.max_input_length, "max_total_tokens": self.limits.max_total_tokens,
            "max_batch_prefill_tokens": cfg.max_prefill_tokens, "max_batch_total_tokens": cfg.max_total_tokens,
            "validation_workers": self.tokenizer_workers, "version": "0.1.0", "sha": None, "docker_label": None,
            "replicas": [self.rt.ctl.state_name(i) for i in range(self.rt.ctl.num_replicas)]})

    async def health(self, req):
        """Healthy when at least one replica is in service and every replica in service answers (replicas that are
        out of service, parked or lost, do not count against the router)."""
        ctl = self.rt.ctl
        serving = [r for r in range(ctl.num_replicas) if ctl.state_name(r) != "Inactive"]
        if not serving:
            return web.json_response({"error": "unhealthy: no replica in service", "error_type": "healthcheck"}, status=503)
        try:
            await asyncio.gather(*[self.rt.stubs[k].health() for r in serving for k in self.rt._ranks(r)])
            return web.Response(text="ok")
        except Exception as e:  # noqa: BLE001
            return web.json_response({"error": f"unhealthy: {e}", "error_type": "healthcheck"}, status=503)

    async def prom(self, req):
        return web.Response(text=self.metrics.render(self.rt), content_type="text/plain")

    def openapi(self) -> dict:
        """The API as an OpenAPI 3 document (the reference generates one from its handler types,
        router_v2/src/server.rs:704-780)."""
        num, integer, boolean, string = {"type": "number"}, {"type": "integer"}, {"type": "boolean"}, {"type": "string"}
        params = {"type": "object", "properties": {
            "max_new_tokens": dict(integer, default=20, minimum=1), "do_sample": dict(boolean, default=False),
            "temperature": dict(num, exclusiveMinimum=0), "top_k": dict(integer, minimum=1),
            "top_p": dict(num, exclusiveMinimum=0, maximum=1), "typical_p": dict(num, exclusiveMinimum=0, maximum=1),
            "repetition_penalty": dict(num, exclusiveMinimum=0), "seed": dict(integer, minimum=0),
            "best_of": dict(integer, minimum=1, description="only 1 is served"),
            "stop": {"type": "array", "items": string, "maxItems": self.limits.max_stop_sequences},
            "ignore_eos_token": dict(boolean, default=False), "truncate": dict(integer, minimum=1),
            "return_full_text": dict(boolean, default=False), "details": dict(boolean, default=False),
            "top_n_tokens": dict(integer, minimum=0, maximum=self.limits.max_top_n_tokens), "watermark": boolean,
            "decoder_input_details": boolean}}
        token = {"type": "object", "properties": {"id": integer, "text": string, "logprob": num, "special": boolean}}
        details = {"type": "object", "nullable": True, "properties": {
            "finish_reason": {"type": "string", "enum": ["length", "eos_token", "stop_sequence"]}, "generated_tokens": integer,
            "seed": dict(integer, nullable=True), "prefill": {"type": "array", "items": token},
            "tokens": {"type": "array", "items": token}}}
        schemas = {
            "GenerateParameters": params,
            "GenerateRequest": {"type": "object", "properties": {
                "inputs": dict(string, description="prompt text (tokenized by the router)"),
                "input_tokens": {"type": "array", "items": integer, "description": "prompt as token ids, instead of `inputs`"},
                "stream": dict(boolean, description="only on `/` and `/invocations`: answer as an event stream"),
                "parameters": {"$ref": "#/components/schemas/GenerateParameters"}}},
            "Token": token, "Details": details,
            "GenerateResponse": {"type": "object", "properties": {"generated_text": string, "details": {"$ref": "#/components/schemas/Details"}}},
            "StreamResponse": {"type": "object", "properties": {"token": {"$ref": "#/components/schemas/Token"},
                                                                 "generated_text": dict(string, nullable=True),
                                                                 "details": {"$ref": "#/components/schemas/Details"}}},
            "ErrorResponse": {"type": "object", "properties": {"error": string, "error_type": string}},
            "ClusterStateChange": {"type": "object", "required": ["replica", "state"], "properties": {
                "replica": integer, "state": {"type": "string", "enum": ["Prefill", "Decode", "Inactive"]}}},
            "Info": {"type": "object", "properties": {k: {} for k in (
                "model_id", "model_dtype", "model_device_type", "max_concurrent_requests", "max_best_of", "max_stop_sequences",
                "max_input_length", "max_total_tokens", "max_batch_prefill_tokens", "max_batch_total_tokens",
                "validation_workers", "version", "replicas")}}}

        def ref(name):
            return {"content": {"application/json": {"schema": {"$ref": f"#/components/schemas/{name}"}}}}
        errors = {"422": dict(ref("ErrorResponse"), description="the request does not validate"),
                  "429": dict(ref("ErrorResponse"), description="too many requests in flight"),
                  "503": dict(ref("ErrorResponse"), description="the replica that served the request was lost")}
        timing = {h: {"schema": integer, "description": "milliseconds"} for h in (
            "x-total-time", "x-queue-time", "x-inference-time", "x-first-token-time", "x-first-decode-token-time",
            "x-time-per-token", "x-max-time-between-tokens", "x-avg-time-between-tokens", "x-p99-time-between-tokens")}
        gen = {"post": {"summary": "generate the whole answer", "requestBody": ref("GenerateRequest"), "responses": dict(
            errors, **{"200": dict(ref("GenerateResponse"), description="the generation; timing in the headers", headers=timing)})}}
        stream = {"post": {"summary": "generate token by token (server-sent events)", "requestBody": ref("GenerateRequest"),
                           "responses": dict(errors, **{"200": {"description": "one `data:` event per token", "content": {
                               "text/event-stream": {"schema": {"$ref": "#/components/schemas/StreamResponse"}}}}})}}
        compat = {"post": dict(gen["post"], summary="as /generate inside a one-element list, or as /generate_stream when `stream` is set")}
        plain = {"200": {"description": "ok"}}
        return {"openapi": "3.0.3", "info": {"title": "blitz_scale_b200 router", "version": "0.1.0"},
                "paths": {"/generate": gen, "/generate_stream": stream, "/": dict(compat, get={"summary": "health", "responses": plain}),
                          "/invocations": compat,
                          "/info": {"get": {"summary": "model and router parameters, replica states",
                                            "responses": {"200": dict(ref("Info"), description="ok")}}},
                          "/health": {"get": {"summary": "every replica in service answers", "responses": dict(
                              plain, **{"503": dict(ref("ErrorResponse"), description="no replica in service, or one does not answer")})}},
                          "/ping": {"get": {"summary": "as /health", "responses": plain}},
                          "/metrics": {"get": {"summary": "Prometheus text format", "responses": plain}},
                          "/modify_cluster_state": {"post": {
                              "summary": "bring a replica into a role or take it out (feature manually_scale)",
                              "requestBody": ref("ClusterStateChange"),
                              "responses": {"200": {"description": "accepted"}, "403": {"description": "manually_scale is off"},
                                            "409": {"description": "not possible in the replica's current state"},
                                            "422": dict(ref("ErrorResponse"), description="malformed body")}}}},
                "components": {"schemas": schemas}}

    async def docs(self, req):
        return web.json_response(self.openapi())

    async def modify_cluster_state(self, req):
        if not self.rt.ctl.has_feature("manually_scale"):
            return web.json_response({"error": "manually_scale is not enabled"}, status=403)
        try:
            body = await req.json()
            replica, state = body["replica"], body["state"]
            if not isinstance(replica, int) or isinstance(replica, bool) or not isinstance(state, str):
                raise TypeError("`replica` must be an integer and `state` a string")
        except Exception as e:  # noqa: BLE001 - not JSON, not an object, or a field missing / of the wrong type
            return web.json_response({"error": f"expected {{\"replica\": int, \"state\": str}}: {e}",
                                      "error_type": "validation"}, status=422)
        ok = self.rt.ctl.manual_scale(replica, state, self.rt.now())
        self.rt.wake.set()
        return web.json_response({"ok": bool(ok)}, status=200 if ok else 409)


def controller_config_from_cluster(cluster: dict, tp: int, features: str, **overrides) -> "core.ControllerConfig":
    """Cluster JSON {init_states, replicas, machines} -> controller config (src/server/disaggregate.cc:31-50)."""
    cfg = core.ControllerConfig()
    from ..utils.cluster_config import check_cluster
    states = check_cluster(cluster, tp)
    cfg.init_states = list(states)
    cfg.num_ranks = len(cfg.init_states)
    cfg.tp = tp
    cfg.machines = list(cluster.get("machines") or [0] * cfg.num_ranks)
    cfg.features = features
    planner = cfg.planner
    for k, v in overrides.items():
        if hasattr(cfg, k):
            setattr(cfg, k, v)
        elif hasattr(planner, k):
            setattr(planner, k, v)
    cfg.planner = planner
    return cfg


async def serve_router(rt: RouterRuntime, host: str, port: int, stop: Optional[asyncio.Event] = None, **kw) -> None:
    app = RouterApp(rt, **kw)
    # a handler is cancelled when its client closes the connection: that is how a collected `/generate` learns
    # that nobody waits for the answer any more
    runner = web.AppRunner(app.app, access_log=None, handler_cancellation=True)
    await runner.setup()
    site = web.TCPSite(runner, host, port)
    await site.start()
    loop_task = asyncio.get_running_loop().create_task(rt.run())
    print(f"Router listening on {host}:{port}", flush=True)
    try:
        if stop is not None:
            await stop.wait()
        else:
            await asyncio.Event().wait()
    finally:
        await rt.stop()
        loop_task.cancel()
        await runner.cleanup()


def build_parser() -> argparse.ArgumentParser:
    """Flags of the router binary (router_v2/src/main.rs:40-155; what does not apply to one NVSwitch box is accepted
    and ignored).  Every flag can also be given through the environment, as FLAG_NAME in upper case."""
    ap = argparse.ArgumentParser("blitz-router")
    ap.add_argument("--hostname", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=3000)
    ap.add_argument("--client-config", required=True, help="JSON list of worker URLs (host:port), rank order")
    ap.add_argument("--deployment-config-path", required=True, help="cluster JSON {init_states, replicas, machines}")
    ap.add_argument("--features", default="impl_blitz,impl_fast_pro,impl_live_pro")
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--model-name", default="llama3_8b")
    ap.add_argument("--model-path", default="")
    ap.add_argument("--tokenizer-path", default="", help="tokenizer.json; without it words are hashed to ids")
    ap.add_argument("--validation-workers", type=int, default=2)
    ap.add_argument("--max-input-length", type=int, default=4095)
    ap.add_argument("--max-total-tokens", type=int, default=4096)
    ap.add_argument("--max-batch-prefill-tokens", type=int, default=8192)
    ap.add_argument("--max-blocks-per-replica", type=int, default=4000,
                    help="KV pages the router lets one replica hold; keep it a little below the workers' --num-total-blocks "
                         "(default 4096) or a worker runs out of pages")
    ap.add_argument("--planner-horizon-ms", type=float, default=1000.0,
                    help="how much queued prefill work per replica the planner tolerates before it adds one, as time: the "
                         "capacity it plans with is tokens-prefilled-per-sec x horizon.  1000 = the per-second rule of the "
                         "reference; with a ~25 ms scale-out 100 keeps p99 TTFT far lower under bursts")
    ap.add_argument("--planner-arrival-window-ms", type=float, default=0.0, help="also size the prefill side by the rate "
                    "at which prompt tokens arrived during the last W ms against --tokens-prefilled-per-sec (a utilisation "
                    "band on the arrival rate: reacts before a backlog has built up, uses more replicas; a window that holds only a few "
                    "arrivals makes replicas come and go, 200 is a sensible start).  0 = off")
    ap.add_argument("--block-size", type=int, default=64, help="tokens per KV page; must equal the workers' --page-size")
    ap.add_argument("--tokens-prefilled-per-sec", type=int, default=15000)
    ap.add_argument("--tokens-transferred-per-sec", type=int, default=96000)
    for n, d in (("prefill-lower-bound", .5), ("prefill-upper-bound", .7), ("decode-lower-bound", .75),
                 ("decode-upper-bound", .95), ("migration-lower-bound", .4), ("migration-upper-bound", .8)):
        ap.add_argument("--" + n, type=float, default=d)
    for n in ("min-prefill-num", "min-decode-num"):
        ap.add_argument("--" + n, type=int, default=1)
    for n in ("max-prefill-num", "max-decode-num"):
        ap.add_argument("--" + n, type=int, default=8)
    ap.add_argument("--scale-down-threshold-millis", type=float, default=333)
    ap.add_argument("--mock-load-millis", type=float, default=0)
    ap.add_argument("--log-level", default=None, help="default: the LOG_LEVEL environment variable, else INFO")
    ap.add_argument("--health-interval-ms", type=float, default=0.0, help="ping every active replica this often (0 = off)")
    ap.add_argument("--health-misses", type=int, default=2, help="consecutive missed pings that declare a replica lost")
    ap.add_argument("--rpc-timeout-ms", type=float, default=300000.0,
                    help="deadline of every worker RPC; a reply that never comes then counts as a failed replica (0 = none)")
    ap.add_argument("--no-chunked-prefill", action="store_true",
                    help="never admit a prompt longer than --max-batch-prefill-tokens (by default it gets a batch of its own, "
                         "which the worker prefills in chunks; raise --max-input-length / --max-total-tokens to let such "
                         "prompts through validation)")
    ap.add_argument("--max-batch-size", type=int, default=256,
                    help="sequences one worker step can carry; must equal the workers' --max-batch-size (0 = no limit)")
    ap.add_argument("--decode-steps-per-call", type=int, default=1,
                    help="decode steps a worker runs per DecodeV2 call (1 = one round trip per token, as the reference)")
    ap.add_argument("--max-incoming-migrations", type=int, default=1,
                    help="KV migrations in flight towards one decode replica at a time (1 = one at a time, as the reference)")
    ap.add_argument("--quarantine-ms", type=float, default=5000.0,
                    help="a replica declared lost is not chosen for scale-up again before this much time has passed")
    ap.add_argument("--statistic-csv", "--statistic-path", dest="statistic_csv", default="",
                    help="write prefill/decode token deltas every 500 ms to this file")
    ap.add_argument("--json-output", action="store_true", help="log lines as JSON objects")
    ap.add_argument("--log-path", default="", help="write the log to this file (through a background writer) instead of stderr")
    ap.add_argument("--otlp-endpoint", default="", help="OTLP/HTTP collector, e.g. http://127.0.0.1:4318: spans of every "
                    "dispatched operation and request are exported there as service blitz.router")
    ap.add_argument("--otlp-service-name", default="blitz.router")
    ap.add_argument("--cors-allow-origin", action="append", default=[], help="origin allowed for cross-origin requests (repeatable, * = any)")
    # the reference can publish its port through an ngrok tunnel (router_v2/src/main.rs:83-89); there is no tunnel
    # client here, so the flags are recognised and refused with a message instead of being unknown
    ap.add_argument("--ngrok", action="store_true", help="not available: no tunnel client in this build")
    ap.add_argument("--ngrok-authtoken", default="", help="not available (see --ngrok)")
    ap.add_argument("--ngrok-edge", default="", help="not available (see --ngrok)")
    ap.add_argument("--max-concurrent-requests", type=int, default=4096)
    ap.add_argument("--max-best-of", type=int, default=2)
    ap.add_argument("--max-stop-sequences", type=int, default=4)
    ap.add_argument("--max-top-n-tokens", type=int, default=5)
    # accepted so that the reference's launch scripts run unchanged; what they configure is either derived from the
    # model registry here (layers, parameter size), fixed by the one-box deployment, or has no counterpart
    for name, kw in (("--num-hidden-layers", dict(type=int)), ("--parameter-size", dict(type=float)),
                     ("--num-gpus-per-node", dict(type=int)), ("--mock-transfer-millis", dict(type=float)),
                     ("--waiting-served-ratio", dict(type=float)), ("--max-waiting-tokens", dict(type=int)),
                     ("--max-batch-total-tokens", dict(type=int)), ("--tokenizer-name", {}), ("--revision", {}),
                     ("--deployment", {}), ("--use-tokenizer", dict(action="store_true"))):
        ap.add_argument(name, help="accepted for command-line compatibility", **({"default": None} | kw if "action" not in kw else kw))
    # every flag can also be given through the environment (FLAG_NAME in upper case), as with the reference's CLI
    for act in ap._actions:
        env = os.environ.get(act.dest.upper())
        # HOSTNAME is set by most shells and containers to the machine's name: not a request to listen there
        if env is None or not act.option_strings or act.dest in ("help", "hostname"):
            continue
        if isinstance(act, argparse._StoreTrueAction):
            act.default = env.lower() not in ("", "0", "false", "no")
        elif isinstance(act, argparse._AppendAction):
            act.default = [x for x in env.split(",") if x]
        else:
            act.default = act.type(env) if act.type else env
            act.required = False
    return ap


def main(argv=None) -> None:
    a = build_parser().parse_args(argv)
    if a.ngrok or a.ngrok_authtoken or a.ngrok_edge:
        raise SystemExit("--ngrok: no tunnel client in this build; publish the port with a reverse proxy instead")
    from ..utils.otlp import SpanExporter, init_logging
    log_listener = init_logging(a.log_level, a.json_output, a.log_path)
    from ..models.config import get_config
    try:
        cluster = json.load(open(a.deployment_config_path))
        urls = json.loads(a.client_config) if a.client_config.strip().startswith("[") else json.load(open(a.client_config))
        if not isinstance(urls, list) or not all(isinstance(u, str) for u in urls):
            raise ValueError("--client-config must be a JSON list of worker addresses (or a file that holds one)")
        if isinstance(cluster, dict) and isinstance(cluster.get("init_states"), list) and len(cluster["init_states"]) != len(urls):
            raise ValueError(f"{len(urls)} worker addresses for {len(cluster['init_states'])} ranks in the cluster config")
        if a.tokenizer_path:
            try:
                core.Tokenizer.from_file(a.tokenizer_path)
            except RuntimeError as e:
                raise ValueError(f"--tokenizer-path: {e}")
    except (OSError, ValueError) as e:
        raise SystemExit(f"router: {e}")
    try:
        core.FeatureSet.parse(a.features)
    except Exception as e:  # noqa: BLE001 - unknown feature or a combination the feature rules forbid
        raise SystemExit(f"router: --features {a.features}: {e}")
    try:
        controller_config_from_cluster(cluster, a.tensor_parallel_size, a.features)      # shape of the cluster description
        get_config(a.model_name)
    except (ValueError, KeyError) as e:
        raise SystemExit(f"router: {e}")
    arrival = {}
    if a.planner_arrival_window_ms > 0:
        # the planner also sizes the prefill side by the rate at which prompt tokens arrive (feature planner_arrival_rate)
        a.features = a.features + ",planner_arrival_rate"
        arrival = dict(prefill_rate_per_sec=float(a.tokens_prefilled_per_sec), arrival_window_ms=float(a.planner_arrival_window_ms))
    cfg = controller_config_from_cluster(
        cluster, a.tensor_parallel_size, a.features, model_name=a.model_name, **arrival,
        max_prefill_tokens=a.max_batch_prefill_tokens, max_total_tokens=max(a.max_total_tokens, 16000),
        max_blocks_per_replica=a.max_blocks_per_replica, block_size=a.block_size, mock_load_ms=a.mock_load_millis,
        tokens_prefilled_per_sec=max(1, int(a.tokens_prefilled_per_sec * a.planner_horizon_ms * 1e-3)),
        tokens_transferred_per_sec=a.tokens_transferred_per_sec,
        prefill_lower=a.prefill_lower_bound, prefill_upper=a.prefill_upper_bound, decode_lower=a.decode_lower_bound,
        decode_upper=a.decode_upper_bound, migration_lower=a.migration_lower_bound,
        migration_upper=a.migration_upper_bound, min_prefill=a.min_prefill_num, max_prefill=a.max_prefill_num,
        min_decode=a.min_decode_num, max_decode=a.max_decode_num, scale_down_threshold_ms=a.scale_down_threshold_millis)
    cfg.quarantine_ms = a.quarantine_ms
    cfg.max_batch_seqs = max(0, a.max_batch_size)
    cfg.chunked_prefill = not a.no_chunked_prefill
    cfg.max_incoming_migrations = max(1, a.max_incoming_migrations)
    layers = get_config(a.model_name).layers
    try:
        from ..runtime import core as _core
        cfg.param_gb = _core.build_segment_layout(a.model_name, a.tensor_parallel_size, 2).total_bytes * a.tensor_parallel_size / 1e9
        cfg.kv_mb_per_token = get_config(a.model_name).kv_bytes_per_token(1, 2) / 1e6
    except Exception:  # noqa: BLE001 - only feeds a metric
        pass
    async def amain():
        # the gRPC channels of the runtime belong to the event loop that creates them: build it inside the loop
        exporter = SpanExporter(a.otlp_endpoint, a.otlp_service_name) if a.otlp_endpoint else None
        if exporter is not None:
            exporter.start()
        rt = RouterRuntime(cfg, urls, model_layers=layers, model_path=a.model_path, stat_csv=a.statistic_csv,
                           health_interval_s=a.health_interval_ms * 1e-3, health_misses=a.health_misses,
                           rpc_timeout_s=a.rpc_timeout_ms * 1e-3, exporter=exporter, decode_steps=a.decode_steps_per_call)
        stop = asyncio.Event()
        for sig in (signal.SIGINT, signal.SIGTERM):
            asyncio.get_running_loop().add_signal_handler(sig, stop.set)
        try:
            await serve_router(rt, a.hostname, a.port, stop=stop, model_name=a.model_name, max_input_length=a.max_input_length,
                               max_total_tokens=a.max_total_tokens, tokenizer_path=a.tokenizer_path,
                               tokenizer_workers=a.validation_workers, max_concurrent=a.max_concurrent_requests,
                               max_best_of=a.max_best_of, max_stop_sequences=a.max_stop_sequences,
                               max_top_n_tokens=a.max_top_n_tokens, cors_allow_origin=a.cors_allow_origin)
        finally:
            if exporter is not None:
                await exporter.stop()           # flushes what is buffered

    try:
        asyncio.run(amain())
    finally:
        if log_listener is not None:
            log_listener.stop()


if __name__ == "__main__":
    main()
