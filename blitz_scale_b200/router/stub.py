"""Async gRPC client of one worker: one coroutine per RPC of the contract
(the role of router_v2/src/stub.rs:34-487).  Requests and responses are the runtime-built
protobuf classes; no generated code is involved."""
from __future__ import annotations

import contextvars
from typing import Iterable, Optional, Sequence

import grpc

from ..pb.schema import RPCS, method_path, pb
from ..utils.tracing import grpc_metadata

CURRENT_TRACE: contextvars.ContextVar = contextvars.ContextVar("blitz_traceparent", default=None)


def encode_prefill_case(*cases: int) -> int:
    """Bit-or of PrefillCase values (router_v2/src/stub.rs:20-30)."""
    v = 0
    for c in cases:
        v |= int(c)
    return v


class WireResponse:
    """A parsed response that also keeps its wire bytes (the router core reads the generations from them natively
    instead of walking the message object token by token).  Attribute access goes to the message."""
    __slots__ = ("msg", "raw")

    def __init__(self, msg, raw: bytes):
        self.msg, self.raw = msg, raw

    def __getattr__(self, name):
        return getattr(self.msg, name)


_KEEP_WIRE = ("PrefillV2", "ZagPrefill", "DecodeV2")


def _wire_deserializer(cls):
    return lambda data: WireResponse(cls.FromString(data), data)


class WorkerStub:
    def __init__(self, url: str, default_timeout: Optional[float] = None):
        """`default_timeout` (seconds) is the deadline of every call that does not pass its own: a worker that never
        answers then surfaces as DEADLINE_EXCEEDED instead of an operation that stays in flight for ever."""
        self.url = url
        self.default_timeout = default_timeout if default_timeout and default_timeout > 0 else None
        # short reconnect back-off: a worker that was restarted is reachable again within a second, while calls to
        # one that is away still fail at once (no wait-for-ready), which is what the failure handling relies on
        self.channel = grpc.aio.insecure_channel(url, options=[("grpc.max_receive_message_length", 256 << 20),
                                                               ("grpc.max_send_message_length", 256 << 20),
                                                               ("grpc.initial_reconnect_backoff_ms", 100),
                                                               ("grpc.min_reconnect_backoff_ms", 100),
                                                               ("grpc.max_reconnect_backoff_ms", 1000)])
        self._m = {}
        for rpc, (req, res) in RPCS.items():
            des = _wire_deserializer(getattr(pb, res)) if rpc in _KEEP_WIRE else getattr(pb, res).FromString
            self._m[rpc] = self.channel.unary_unary(method_path(rpc),
                                                    request_serializer=getattr(pb, req).SerializeToString,
                                                    response_deserializer=des)

    async def call(self, rpc: str, request, timeout: Optional[float] = None, metadata=None):
        if not request.IsInitialized():
            # the transport would swallow the encoding error and send an empty message instead
            raise ValueError(f"{rpc}: request is missing required fields: {request.FindInitializationErrors()}")
        if metadata is None:
            # trace context of the operation this call belongs to (set by the router runtime per dispatched op)
            metadata = grpc_metadata(CURRENT_TRACE.get())
        return await self._m[rpc](request, timeout=timeout if timeout is not None else self.default_timeout,
                                  metadata=metadata)

    async def close(self):
        await self.channel.close()

    # ---- convenience wrappers
    async def health(self, timeout=2.0):
        return await self.call("Health", pb.HealthRequest(), timeout)

    async def info(self):
        return await self.call("Info", pb.InfoRequest())

    async def clear_cache(self, batch_id: Optional[int] = None):
        r = pb.ClearCacheRequest()
        if batch_id is not None:
            r.id = batch_id
        return await self.call("ClearCache", r)

    async def filter_batch(self, batch_id: int, request_ids: Iterable[int]):
        return await self.call("FilterBatch", pb.FilterBatchRequest(batch_id=batch_id, request_ids=list(request_ids)))

    async def warmup(self, max_input_length=2048, max_prefill_tokens=4096, max_total_tokens=4096):
        return await self.call("Warmup", pb.WarmupRequest(max_input_length=max_input_length,
                                                          max_prefill_tokens=max_prefill_tokens,
                                                          max_total_tokens=max_total_tokens))

    async def prefill_v2(self, batch, forward_case: int = 0, pp_info=None, pipe_peer: Sequence[int] = ()):
        r = pb.PrefillV2Request(batch=batch, forward_case=forward_case, pipe_peer=list(pipe_peer))
        if pp_info is not None:
            r.pp_info.CopyFrom(pp_info)
        return await self.call("PrefillV2", r)

    async def zag_prefill(self, batch, zag_seq_num: int, zag_layers: int, forward_case: int = 4, pp_info=None):
        r = pb.ZagPrefillRequest(batch=batch, forward_case=forward_case, zag_layers=zag_layers, zag_seq_num=zag_seq_num)
        if pp_info is None:
            r.pp_info.embedding_layer = 1
        else:
            r.pp_info.CopyFrom(pp_info)
        return await self.call("ZagPrefill", r)

    async def decode_v2(self, batches, last_iter_tokens, steps: int = 1):
        """`steps` > 1: the worker runs up to that many decode steps in this call (asked for in the call's metadata;
        the request message of the contract stays as it is) and returns every step's generations in order."""
        req = pb.DecodeV2Request(batches=list(batches), last_iter_tokens=list(last_iter_tokens))
        if steps <= 1:
            return await self.call("DecodeV2", req)
        md = tuple(grpc_metadata(CURRENT_TRACE.get()) or ()) + (("x-decode-steps", str(int(steps))),)
        return await self.call("DecodeV2", req, metadata=md)

    async def relay(self, rank: int, relax_not_head: bool):
        return await self.call("Relay", pb.RelayRequest(rank=rank, relax_not_head=relax_not_head))

    async def migrate(self, batch, src, dst, partial: int = 0, num_layer: int = 0):
        if partial:
            return await self.call("MigratePartial", pb.MigratePartialRequest(batch=batch, fst_or_snd=partial,
                                                                              num_layer=num_layer, src=src, dst=dst))
        return await self.call("Migrate", pb.MigrateRequest(batch=batch, src=src, dst=dst))

    async def immigrate(self, batch, src, dst, partial: int = 0, num_layer: int = 0):
        if partial:
            return await self.call("ImmigratePartial", pb.ImmigratePartialRequest(batch=batch, fst_or_snd=partial,
                                                                                  num_layer=num_layer, src=src, dst=dst))
        return await self.call("Immigrate", pb.ImmigrateRequest(batch=batch, src=src, dst=dst))

    async def broadcast(self, kind: str, src_ranks, dst_ranks):
        rpc = {"nvl": "NvlBroadcast", "rdma": "RdmaBroadcast", "tanz": "TanzBroadcast"}[kind]
        return await self.call(rpc, pb.BroadcastRequest(src_ranks=list(src_ranks), dst_ranks=list(dst_ranks)))

    async def load_params(self, load_case: int, model_name: str, model_path: str = ""):
        r = pb.LoadParamsRequest(load_case=load_case, model_name=model_name)
        if model_path:
            r.model_path = model_path
        return await self.call("LoadParams", r)

    async def send_params(self, dst: int):
        return await self.call("SendParams", pb.SendParamsRequest(dst=dst))

    async def recv_params(self, src: int):
        return await self.call("RecvParams", pb.RecvParamsRequest(src=src))

    async def wait_rdma_done(self):
        return await self.call("WaitRdmaDone", pb.WaitRdmaDoneRequest())

    async def reset_status(self):
        return await self.call("ResetStatus", pb.ResetStatusRequest())

    async def set_status_ready(self):
        return await self.call("SetStatusReady", pb.SetStatusReadyRequest())
