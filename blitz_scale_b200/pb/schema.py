"""The ``generate.v2`` wire contract, built at import time without protoc.

Neither ``protoc`` nor ``grpc_tools`` exists in the target image, so the schema is declared
here as data (message -> [(field number, label, type, name)]) and turned into a
``FileDescriptorProto`` + message classes with the protobuf runtime.  Package, service,
RPC, message and field names and numbers follow the reference contract
(proto/generate.proto:5-58 service, :60-462 messages) so either side can talk to the other.
``render_proto()`` prints the same schema as ``.proto`` text for documentation and for
generating stubs in other languages.
"""
from __future__ import annotations

from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

PACKAGE = "generate.v2"
SERVICE = "TextGenerationService"

O, R, P = "optional", "required", "repeated"

ENUMS = {
    "FinishReason": [("FINISH_REASON_LENGTH", 0), ("FINISH_REASON_EOS_TOKEN", 1), ("FINISH_REASON_STOP_SEQUENCE", 2)],
    "LoadParamCase": [("LOAD_FROM_HOST_MEM", 0), ("LOAD_FROM_DISK", 1)],
    "PrefillCase": [("PREFILL_CASE_NORMAL", 0), ("PREFILL_CASE_MIGRATE", 1), ("PREFILL_CASE_MIGRATE_PROGRESSIVE", 2),
                    ("PREFILL_CASE_NAIVE_PP", 4), ("PREFILL_CASE_IMMIGRATE", 8)],
    "PartialCase": [("PARTIAL_CASE_FIRST", 1), ("PARTIAL_CASE_SECOND", 2)],
}

# message -> list of (number, label, type, name[, oneof])
MESSAGES = {
    "HealthRequest": [], "HealthResponse": [(1, R, "string", "state")],
    "RelayRequest": [(1, R, "int32", "rank"), (2, R, "bool", "relax_not_head")],
    "RelayResponse": [(1, O, "uint64", "batch_id"), (2, O, "uint32", "seq_num")],
    "BroadcastRequest": [(1, P, "int32", "src_ranks"), (2, P, "int32", "dst_ranks")], "BroadcastResponse": [],
    "ResetStatusRequest": [], "ResetStatusResponse": [], "SetStatusReadyRequest": [], "SetStatusReadyResponse": [],
    "InfoRequest": [],
    "InfoResponse": [(1, R, "bool", "requires_padding"), (2, R, "string", "dtype"), (3, R, "string", "device_type"),
                     (4, O, "uint32", "window_size"), (5, R, "uint32", "speculate")],
    "ServiceDiscoveryRequest": [],
    "ServiceDiscoveryResponse": [(1, P, "string", "urls"), (2, R, "string", "ranks_view_in_json")],
    "ClearCacheRequest": [(1, O, "uint64", "id")], "ClearCacheResponse": [],
    "NextTokenChooserParameters": [(1, R, "float", "temperature"), (2, R, "uint32", "top_k"), (3, R, "float", "top_p"),
                                   (4, R, "float", "typical_p"), (5, R, "bool", "do_sample"), (6, R, "uint64", "seed"),
                                   (7, R, "float", "repetition_penalty"), (8, R, "bool", "watermark")],
    "StoppingCriteriaParameters": [(1, R, "uint32", "max_new_tokens"), (2, P, "string", "stop_sequences"),
                                   (3, R, "bool", "ignore_eos_token")],
    "Request": [(1, R, "uint64", "id"), (2, R, "string", "inputs"), (3, O, "uint32", "truncate"),
                (4, O, "NextTokenChooserParameters", "parameters"),
                (5, R, "StoppingCriteriaParameters", "stopping_parameters"), (6, R, "bool", "prefill_logprobs"),
                (7, R, "uint32", "top_n_tokens"), (8, P, "uint32", "input_tokens")],
    "Batch": [(1, R, "uint64", "id"), (2, P, "Request", "requests"), (3, R, "uint32", "size"),
              (4, R, "uint32", "max_tokens")],
    "CachedBatch": [(1, R, "uint64", "id"), (2, P, "uint64", "request_ids"), (3, R, "uint32", "size"),
                    (4, R, "uint32", "max_tokens")],
    "GeneratedText": [(1, R, "string", "text"), (2, R, "uint32", "generated_tokens"),
                      (3, R, "FinishReason", "finish_reason"), (4, O, "uint64", "seed")],
    "Tokens": [(1, P, "uint32", "ids"), (2, P, "float", "logprobs"), (3, P, "string", "texts"),
               (4, P, "bool", "is_special")],
    "Generation": [(1, R, "uint64", "request_id"), (2, O, "Tokens", "prefill_tokens"), (3, R, "Tokens", "tokens"),
                   (4, O, "GeneratedText", "generated_text"), (5, P, "Tokens", "top_tokens")],
    "FilterBatchRequest": [(1, R, "uint64", "batch_id"), (2, P, "uint64", "request_ids")],
    "FilterBatchResponse": [(1, R, "CachedBatch", "batch")],
    "PrefillRequest": [(1, R, "Batch", "batch")],
    "PrefillResponse": [(1, P, "Generation", "generations"), (2, O, "CachedBatch", "batch"),
                        (3, R, "uint64", "forward_ns"), (4, R, "uint64", "decode_ns"), (5, R, "uint64", "total_ns")],
    "DecodeRequest": [(1, P, "CachedBatch", "batches")],
    "DecodeResponse": [(1, P, "Generation", "generations"), (2, O, "CachedBatch", "batch"),
                       (3, R, "uint64", "forward_ns"), (4, R, "uint64", "decode_ns"), (5, R, "uint64", "total_ns"),
                       (6, O, "uint64", "concat_ns")],
    "WarmupRequest": [(1, O, "Batch", "batch"), (2, O, "uint32", "max_input_length"),
                      (3, O, "uint32", "max_prefill_tokens"), (4, O, "uint32", "max_total_tokens")],
    "WarmupResponse": [(1, O, "uint32", "max_supported_total_tokens")],
    "SendParamsRequest": [(1, R, "int32", "dst")], "SendParamsResponse": [],
    "RecvParamsRequest": [(1, R, "int32", "src")], "RecvParamsResponse": [],
    "LoadParamsRequest": [(1, R, "LoadParamCase", "load_case"), (2, R, "string", "model_name"),
                          (3, O, "string", "model_path")],
    "LoadParamsResponse": [],
    "PipeParaInfo": [(1, O, "uint32", "embedding_layer", "start_layer"), (2, O, "uint32", "lm_head", "start_layer"),
                     (3, O, "uint32", "tfm_layer", "start_layer"), (4, P, "uint32", "num_layer_per_rank")],
    "PrefillV2Request": [(1, R, "Batch", "batch"), (2, R, "uint32", "forward_case"), (3, O, "PipeParaInfo", "pp_info"),
                         (4, P, "int32", "pipe_peer")],
    "PrefillV2Response": [(1, P, "Generation", "generations"), (2, O, "CachedBatch", "batch"),
                          (3, O, "PipeParaInfo", "pp_info"), (4, R, "uint64", "forward_ns"),
                          (5, R, "uint64", "decode_ns"), (6, R, "uint64", "total_ns")],
    "ZagPrefillRequest": [(1, R, "Batch", "batch"), (2, R, "uint32", "forward_case"),
                          (3, O, "PipeParaInfo", "pp_info"), (4, R, "uint32", "zag_layers"),
                          (5, R, "uint32", "zag_seq_num")],
    "DecodeV2Request": [(1, P, "CachedBatch", "batches"), (2, P, "Tokens", "last_iter_tokens")],
    "DecodeV2Response": [(1, P, "Generation", "generations"), (2, O, "CachedBatch", "batch"),
                         (3, R, "uint64", "total_ns")],
    "MigrateRequest": [(1, R, "Batch", "batch"), (2, P, "int32", "src"), (3, P, "int32", "dst")],
    "MigratePartialRequest": [(1, R, "Batch", "batch"), (2, R, "PartialCase", "fst_or_snd"),
                              (3, R, "uint32", "num_layer"), (4, P, "int32", "src"), (5, P, "int32", "dst")],
    "MigrateResponse": [(1, R, "CachedBatch", "batch")],
    "ImmigrateRequest": [(1, R, "Batch", "batch"), (2, P, "int32", "src"), (3, P, "int32", "dst")],
    "ImmigratePartialRequest": [(1, R, "Batch", "batch"), (2, R, "PartialCase", "fst_or_snd"),
                                (3, R, "uint32", "num_layer"), (4, P, "int32", "src"), (5, P, "int32", "dst")],
    "ImmigrateResponse": [(1, R, "CachedBatch", "batch")],
    "WaitRdmaDoneRequest": [], "WaitRdmaDoneResponse": [],
}

# rpc name -> (request, response); 26 methods
RPCS = {
    "Info": ("InfoRequest", "InfoResponse"),
    "ServiceDiscovery": ("ServiceDiscoveryRequest", "ServiceDiscoveryResponse"),
    "ClearCache": ("ClearCacheRequest", "ClearCacheResponse"),
    "FilterBatch": ("FilterBatchRequest", "FilterBatchResponse"),
    "Warmup": ("WarmupRequest", "WarmupResponse"),
    "Prefill": ("PrefillRequest", "PrefillResponse"),
    "Decode": ("DecodeRequest", "DecodeResponse"),
    "Health": ("HealthRequest", "HealthResponse"),
    "SendParams": ("SendParamsRequest", "SendParamsResponse"),
    "RecvParams": ("RecvParamsRequest", "RecvParamsResponse"),
    "LoadParams": ("LoadParamsRequest", "LoadParamsResponse"),
    "PrefillV2": ("PrefillV2Request", "PrefillV2Response"),
    "DecodeV2": ("DecodeV2Request", "DecodeV2Response"),
    "ZagPrefill": ("ZagPrefillRequest", "PrefillV2Response"),
    "Migrate": ("MigrateRequest", "MigrateResponse"),
    "Immigrate": ("ImmigrateRequest", "ImmigrateResponse"),
    "MigratePartial": ("MigratePartialRequest", "MigrateResponse"),
    "ImmigratePartial": ("ImmigratePartialRequest", "ImmigrateResponse"),
    "WaitRdmaDone": ("WaitRdmaDoneRequest", "WaitRdmaDoneResponse"),
    "ResetStatus": ("ResetStatusRequest", "ResetStatusResponse"),
    "SetStatusReady": ("SetStatusReadyRequest", "SetStatusReadyResponse"),
    "Relay": ("RelayRequest", "RelayResponse"),
    "NvlBroadcast": ("BroadcastRequest", "BroadcastResponse"),
    "RdmaBroadcast": ("BroadcastRequest", "BroadcastResponse"),
    "TanzBroadcast": ("BroadcastRequest", "BroadcastResponse"),
}

_SCALAR = {
    "double": 1, "float": 2, "int64": 3, "uint64": 4, "int32": 5, "bool": 8, "string": 9, "uint32": 13,
}
_LABEL = {O: 1, R: 2, P: 3}


def _build_file() -> descriptor_pb2.FileDescriptorProto:
    f = descriptor_pb2.FileDescriptorProto()
    f.name = "generate.proto"
    f.package = PACKAGE
    f.syntax = "proto2"
    for ename, vals in ENUMS.items():
        e = f.enum_type.add()
        e.name = ename
        for n, v in vals:
            ev = e.value.add()
            ev.name, ev.number = n, v
    for mname, fields in MESSAGES.items():
        m = f.message_type.add()
        m.name = mname
        oneofs = {}
        for fld in fields:
            num, label, typ, name = fld[:4]
            fd = m.field.add()
            fd.name, fd.number, fd.label = name, num, _LABEL[label]
            if typ in _SCALAR:
                fd.type = _SCALAR[typ]
            elif typ in ENUMS:
                fd.type = 14
                fd.type_name = f".{PACKAGE}.{typ}"
            else:
                fd.type = 11
                fd.type_name = f".{PACKAGE}.{typ}"
            if len(fld) == 5:
                if fld[4] not in oneofs:
                    oneofs[fld[4]] = len(m.oneof_decl)
                    m.oneof_decl.add().name = fld[4]
                fd.oneof_index = oneofs[fld[4]]
    s = f.service.add()
    s.name = SERVICE
    for rpc, (req, res) in RPCS.items():
        md = s.method.add()
        md.name = rpc
        md.input_type = f".{PACKAGE}.{req}"
        md.output_type = f".{PACKAGE}.{res}"
    return f


_pool = descriptor_pool.DescriptorPool()
_file_proto = _build_file()
_file = _pool.Add(_file_proto) if hasattr(_pool, "Add") else None
if _file is None:
    _pool.AddSerializedFile(_file_proto.SerializeToString())


def _cls(name: str):
    return message_factory.GetMessageClass(_pool.FindMessageTypeByName(f"{PACKAGE}.{name}"))


class _Namespace:
    pass


pb = _Namespace()
for _m in MESSAGES:
    setattr(pb, _m, _cls(_m))
for _e, _vals in ENUMS.items():
    for _n, _v in _vals:
        setattr(pb, _n, _v)

FULL_SERVICE = f"{PACKAGE}.{SERVICE}"


def method_path(rpc: str) -> str:
    return f"/{FULL_SERVICE}/{rpc}"


def render_proto() -> str:
    """The schema as .proto text."""
    out = ['syntax = "proto2";', "", f"package {PACKAGE};", "", f"service {SERVICE} {{"]
    for rpc, (req, res) in RPCS.items():
        out.append(f"  rpc {rpc}({req}) returns ({res});")
    out.append("}")
    for e, vals in ENUMS.items():
        out += ["", f"enum {e} {{"] + [f"  {n} = {v};" for n, v in vals] + ["}"]
    for m, fields in MESSAGES.items():
        out += ["", f"message {m} {{"]
        groups = {}
        for fld in fields:
            if len(fld) == 5:
                groups.setdefault(fld[4], []).append(fld)
            else:
                out.append(f"  {fld[1]} {fld[2]} {fld[3]} = {fld[0]};")
        for g, fl in groups.items():
            out.append(f"  oneof {g} {{")
            out += [f"    {x[2]} {x[3]} = {x[0]};" for x in fl]
            out.append("  }")
        out.append("}")
    return "\n".join(out) + "\n"


def main() -> int:
    """`python -m blitz_scale_b200.pb.schema > generate.proto`: the contract as text, for clients in other languages."""
    print(render_proto(), end="")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
