"""gRPC service `generate.v2.TextGenerationService` of one worker (one process per GPU).

The 25 RPCs of the contract (proto/generate.proto:5-58) are served by a generic handler built from
the runtime schema, on top of a `Backend` (the GPU engine or the GPU-less stub).  Behavioural
notes carried over from the reference implementation (src/service/service.cc): cached batches live
in a map keyed by batch id (:101-145, :147-208); `DecodeV2` first appends the tokens of the previous
iteration that travelled with a migrated batch, then merges all named batches into the first one
(:610-757); `ZagPrefill` calls are executed strictly in `zag_seq_num` order (:798-818); `Prefill` /
`Decode` (v1) are rejected (:276-304).  `Health` and `Info`, unimplemented in the reference
(:72-78, :308-317), answer properly here.
"""
from __future__ import annotations

import asyncio
import logging
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Optional

import grpc

from ..pb.schema import FULL_SERVICE, RPCS, pb


log = logging.getLogger("blitz.worker.rpc")


class Backend:
    """What a worker must be able to do; see gpu_backend.GpuBackend and sim.stub_worker.StubBackend."""

    rank = 0
    world = 1

    def thread_init(self) -> None:
        """Runs once in every handler thread (a GPU backend binds the thread to its device)."""

    def info(self) -> dict: ...
    def prefill(self, batch, forward_case: int, pp_info, pipe_peer): ...
    def zag_prefill(self, batch, forward_case: int, pp_info, zag_layers: int, zag_seq: int): ...
    def decode(self, batches, last_iter_tokens): ...
    def clear_cache(self, batch_id: Optional[int]): ...
    def filter_batch(self, batch_id: int, request_ids): ...
    def migrate(self, batch, src, dst, partial: int = 0, num_layer: int = 0): ...
    def immigrate(self, batch, src, dst, partial: int = 0, num_layer: int = 0): ...
    def send_params(self, dst: int): ...
    def recv_params(self, src: int): ...
    def wait_transfer_done(self): ...
    def load_params(self, load_case: int, model_name: str, model_path: str): ...
    def broadcast(self, kind: str, src_ranks, dst_ranks): ...
    def relay(self, rank: int, relax_not_head: bool): ...
    def reset_status(self): ...
    def set_status_ready(self): ...
    def warmup(self, req) -> int: ...


class TextGenerationService:
    def __init__(self, backend: Backend, urls=None):
        self.b = backend
        self.urls = list(urls or [])
        self.pool = ThreadPoolExecutor(max_workers=32, thread_name_prefix=f"worker{backend.rank}",
                                       initializer=backend.thread_init)
        self._zag_next = 0
        self._zag_cv = asyncio.Condition()

    async def _call(self, fn, *a):
        return await asyncio.get_running_loop().run_in_executor(self.pool, fn, *a)

    @staticmethod
    def _abort(context, e: Exception):
        code = grpc.StatusCode.FAILED_PRECONDITION if isinstance(e, (RuntimeError, KeyError)) else grpc.StatusCode.INTERNAL
        return context.abort(code, f"{type(e).__name__}: {e}")

    # ------------------------------------------------------------------ status
    async def Health(self, req, ctx):
        return pb.HealthResponse(state="ready" if self.b.info().get("ready", True) else "loading")

    async def Info(self, req, ctx):
        i = self.b.info()
        return pb.InfoResponse(requires_padding=False, dtype=i.get("dtype", "bfloat16"),
                               device_type=i.get("device_type", "cuda"), speculate=0)

    async def ServiceDiscovery(self, req, ctx):
        import json
        return pb.ServiceDiscoveryResponse(urls=self.urls, ranks_view_in_json=json.dumps(self.b.info().get("ranks", {})))

    async def Warmup(self, req, ctx):
        return pb.WarmupResponse(max_supported_total_tokens=await self._call(self.b.warmup, req))

    async def ResetStatus(self, req, ctx):
        await self._call(self.b.reset_status)
        self._zag_next = 0
        return pb.ResetStatusResponse()

    async def SetStatusReady(self, req, ctx):
        await self._call(self.b.set_status_ready)
        return pb.SetStatusReadyResponse()

    # ------------------------------------------------------------------ batch cache
    async def ClearCache(self, req, ctx):
        await self._call(self.b.clear_cache, req.id if req.HasField("id") else None)
        return pb.ClearCacheResponse()

    async def FilterBatch(self, req, ctx):
        try:
            cb = await self._call(self.b.filter_batch, req.batch_id, list(req.request_ids))
        except Exception as e:  # noqa: BLE001
            return await self._abort(ctx, e)
        return pb.FilterBatchResponse(batch=cb)

    # ------------------------------------------------------------------ inference
    async def Prefill(self, req, ctx):
        await ctx.abort(grpc.StatusCode.UNIMPLEMENTED, "use PrefillV2")

    async def Decode(self, req, ctx):
        await ctx.abort(grpc.StatusCode.UNIMPLEMENTED, "use DecodeV2")

    async def PrefillV2(self, req, ctx):
        t0 = time.perf_counter_ns()
        try:
            gens, cb, pp = await self._call(self.b.prefill, req.batch, req.forward_case,
                                            req.pp_info if req.HasField("pp_info") else None, list(req.pipe_peer))
        except Exception as e:  # noqa: BLE001
            return await self._abort(ctx, e)
        dt = time.perf_counter_ns() - t0
        r = _response(pb.PrefillV2Response, gens, forward_ns=dt, decode_ns=0, total_ns=dt)
        if cb is not None:
            r.batch.CopyFrom(cb)
        if pp is not None:
            r.pp_info.CopyFrom(pp)
        return r

    async def ZagPrefill(self, req, ctx):
        t0 = time.perf_counter_ns()
        async with self._zag_cv:  # strictly in sequence-number order
            await self._zag_cv.wait_for(lambda: self._zag_next == req.zag_seq_num)
            self._zag_next += 1
            self._zag_cv.notify_all()
        try:
            gens, cb, pp = await self._call(self.b.zag_prefill, req.batch, req.forward_case,
                                            req.pp_info if req.HasField("pp_info") else None, req.zag_layers,
                                            req.zag_seq_num)
        except Exception as e:  # noqa: BLE001
            return await self._abort(ctx, e)
        dt = time.perf_counter_ns() - t0
        r = _response(pb.PrefillV2Response, gens, forward_ns=dt, decode_ns=0, total_ns=dt)
        if cb is not None:
            r.batch.CopyFrom(cb)
        if pp is not None:
            r.pp_info.CopyFrom(pp)
        return r

    async def DecodeV2(self, req, ctx):
        t0 = time.perf_counter_ns()
        if not req.batches:
            await ctx.abort(grpc.StatusCode.INVALID_ARGUMENT, "DecodeV2 needs at least one cached batch")
        try:
            # "x-decode-steps: k" in the call's metadata asks for up to k steps in this one call
            steps = 1
            for k, v in (ctx.invocation_metadata() or ()):
                if k == "x-decode-steps":
                    steps = max(1, min(64, int(v)))
            if steps > 1:
                gens, cb = await self._call(self.b.decode, list(req.batches), list(req.last_iter_tokens), steps)
            else:
                gens, cb = await self._call(self.b.decode, list(req.batches), list(req.last_iter_tokens))
        except Exception as e:  # noqa: BLE001
            return await self._abort(ctx, e)
        r = _response(pb.DecodeV2Response, gens, total_ns=time.perf_counter_ns() - t0)
        if cb is not None:
            r.batch.CopyFrom(cb)
        return r

    async def Relay(self, req, ctx):
        try:
            res = await self._call(self.b.relay, req.rank, req.relax_not_head)
        except Exception as e:  # noqa: BLE001
            return await self._abort(ctx, e)
        r = pb.RelayResponse()
        if res is not None:
            r.batch_id, r.seq_num = res
        return r

    # ------------------------------------------------------------------ KV migration
    async def _mig(self, fn, req, ctx, partial=0, num_layer=0, resp=None):
        try:
            cb = await self._call(fn, req.batch, list(req.src), list(req.dst), partial, num_layer)
        except Exception as e:  # noqa: BLE001
            return await self._abort(ctx, e)
        return resp(batch=cb)

    async def Migrate(self, req, ctx):
        return await self._mig(self.b.migrate, req, ctx, resp=pb.MigrateResponse)

    async def Immigrate(self, req, ctx):
        return await self._mig(self.b.immigrate, req, ctx, resp=pb.ImmigrateResponse)

    async def MigratePartial(self, req, ctx):
        return await self._mig(self.b.migrate, req, ctx, req.fst_or_snd, req.num_layer, pb.MigrateResponse)

    async def ImmigratePartial(self, req, ctx):
        return await self._mig(self.b.immigrate, req, ctx, req.fst_or_snd, req.num_layer, pb.ImmigrateResponse)

    # ------------------------------------------------------------------ parameters
    async def SendParams(self, req, ctx):
        await self._call(self.b.send_params, req.dst)
        return pb.SendParamsResponse()

    async def RecvParams(self, req, ctx):
        await self._call(self.b.recv_params, req.src)
        return pb.RecvParamsResponse()

    async def WaitRdmaDone(self, req, ctx):
        await self._call(self.b.wait_transfer_done)
        return pb.WaitRdmaDoneResponse()

    async def LoadParams(self, req, ctx):
        try:
            await self._call(self.b.load_params, req.load_case, req.model_name,
                             req.model_path if req.HasField("model_path") else "")
        except Exception as e:  # noqa: BLE001
            return await self._abort(ctx, e)
        return pb.LoadParamsResponse()

    async def _bcast(self, kind, req, ctx):
        try:
            await self._call(self.b.broadcast, kind, list(req.src_ranks), list(req.dst_ranks))
        except Exception as e:  # noqa: BLE001
            return await self._abort(ctx, e)
        return pb.BroadcastResponse()

    async def NvlBroadcast(self, req, ctx):
        return await self._bcast("nvl", req, ctx)

    async def RdmaBroadcast(self, req, ctx):
        return await self._bcast("rdma", req, ctx)

    async def TanzBroadcast(self, req, ctx):
        return await self._bcast("tanz", req, ctx)

    # ------------------------------------------------------------------ wiring
    def generic_handler(self) -> grpc.GenericRpcHandler:
        handlers = {}
        def traced(rpc, fn):
            # the router sends a W3C traceparent with every call; one debug line per RPC lets merged logs follow a
            # request across processes
            async def call(req, ctx):
                if log.isEnabledFor(logging.DEBUG):
                    tp = dict(ctx.invocation_metadata() or ()).get("traceparent", "")
                    log.debug("rpc %s rank=%d traceparent=%s", rpc, self.b.rank, tp)
                return await fn(req, ctx)
            return call

        for rpc, (req, res) in RPCS.items():
            handlers[rpc] = grpc.unary_unary_rpc_method_handler(
                traced(rpc, getattr(self, rpc)), request_deserializer=getattr(pb, req).FromString,
                response_serializer=getattr(pb, res).SerializeToString)
        return grpc.method_handlers_generic_handler(FULL_SERVICE, handlers)


async def serve(backend: Backend, host: str, port: int, urls=None, ready_event: Optional[asyncio.Event] = None,
                stop_event: Optional[asyncio.Event] = None) -> None:
    """Start the gRPC server on host:port (the launcher uses port = base + rank, src/server/disaggregate.cc:330)."""
    server = grpc.aio.server(options=[("grpc.max_receive_message_length", 256 << 20),
                                      ("grpc.max_send_message_length", 256 << 20)])
    svc = TextGenerationService(backend, urls)
    server.add_generic_rpc_handlers((svc.generic_handler(),))
    server.add_insecure_port(f"{host}:{port}")
    await server.start()
    print(f"Start gRPC server on {host}:{port} (rank {backend.rank})", flush=True)
    if ready_event is not None:
        ready_event.set()
    try:
        if stop_event is not None:
            await stop_event.wait()
        else:
            await server.wait_for_termination()
    finally:
        await server.stop(grace=1.0)


def seq_spec_from_request(r, default_tokens=None, eos_token: int = -1) -> "core.SeqSpec":
    """The engine's view of one `Request` of the contract: prompt ids, stopping rule (token budget, and the model's
    end-of-sequence id `eos_token` unless the request ignores it) and, when the request asks for it
    (`parameters.do_sample`), the sampling parameters."""
    from ..runtime import core
    s = core.SeqSpec(r.id, list(r.input_tokens) or list(default_tokens or [1]), r.stopping_parameters.max_new_tokens,
                     r.stopping_parameters.ignore_eos_token, int(eos_token))
    if r.HasField("parameters") and r.parameters.do_sample:
        p = r.parameters
        s.do_sample, s.temperature, s.top_k, s.top_p, s.seed = True, float(p.temperature), int(p.top_k), float(p.top_p), int(p.seed)
    return s


def _response(cls, gens, **fields):
    """Response of class `cls` whose `generations` (field 1 in both response types) come either as a list of
    messages or as the wire bytes a backend encoded natively (`Batch.encode_generations`)."""
    if isinstance(gens, (bytes, bytearray)):
        r = cls.FromString(bytes(gens))
        for k, v in fields.items():
            setattr(r, k, v)
        return r
    return cls(generations=gens, **fields)


def make_generation(request_id: int, token: int, text: str = "", finished: Optional[int] = None, n_generated: int = 0):
    g = pb.Generation(request_id=request_id)
    g.tokens.ids.append(token)
    g.tokens.logprobs.append(0.0)
    g.tokens.texts.append(text)
    g.tokens.is_special.append(False)
    if finished is not None:
        g.generated_text.text = text
        g.generated_text.generated_tokens = n_generated
        g.generated_text.finish_reason = finished
    return g
