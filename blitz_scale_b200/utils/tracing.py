"""Tracing helpers: NVTX ranges behind a flag, W3C trace context for the control plane, Chrome-trace export.

* `nvtx_range(name)`  a context manager that pushes an NVTX range when BLITZ_NVTX=1 (so a profiler timeline shows
  prefill / decode / per-layer / transfer phases) and costs one attribute lookup otherwise.
* `new_traceparent()` / `child_traceparent()`  W3C `traceparent` values; the router attaches one to every worker RPC
  as gRPC metadata (the reference injects its OpenTelemetry context the same way, rust-grpc/src/lib.rs:45-63) and
  the worker logs it at debug level, which lets `logtools merge` follow one request across processes.
* `chrome_trace(...)`  router state transitions, scale-out intervals and (optionally) per-request spans from
  `client.jsonl` as a Chrome / Perfetto trace-event JSON.

    python -m blitz_scale_b200.utils.tracing router.log [--client client.jsonl] -o trace.json
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import secrets
from typing import Dict, Iterable, List, Optional

from .analysis import load_jsonl, parse_router_log, replica_timeline, scale_out_latencies

_NVTX = os.environ.get("BLITZ_NVTX", "0") not in ("", "0")


def nvtx_enabled() -> bool:
    return _NVTX


def set_nvtx(on: bool) -> None:
    global _NVTX
    _NVTX = bool(on)


@contextlib.contextmanager
def nvtx_range(name: str):
    if not _NVTX:
        yield
        return
    import torch
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


# ---------------------------------------------------------------------------------------------- trace context
def new_traceparent() -> str:
    return f"00-{secrets.token_hex(16)}-{secrets.token_hex(8)}-01"


def child_traceparent(parent: str) -> str:
    parts = parent.split("-")
    if len(parts) != 4 or len(parts[1]) != 32:
        return new_traceparent()
    return f"{parts[0]}-{parts[1]}-{secrets.token_hex(8)}-{parts[3]}"


def trace_id(traceparent: str) -> str:
    parts = traceparent.split("-")
    return parts[1] if len(parts) == 4 else ""


def grpc_metadata(traceparent: Optional[str]):
    return (("traceparent", traceparent),) if traceparent else None


# ---------------------------------------------------------------------------------------------- Chrome trace
def chrome_trace(router_log: Iterable[str], client_records: Optional[List[dict]] = None) -> Dict:
    parsed = parse_router_log(router_log)
    tr = parsed["transitions"]
    t_end = (max((t or 0.0) for t, *_ in tr) if tr else 0.0) + 1.0
    ev: List[dict] = [{"ph": "M", "pid": 1, "name": "process_name", "args": {"name": "replicas"}}]
    for rid, spans in sorted(replica_timeline(tr, t_end).items()):
        ev.append({"ph": "M", "pid": 1, "tid": rid, "name": "thread_name", "args": {"name": f"replica {rid}"}})
        for a, b, st in spans:
            if st != "Inactive":
                ev.append({"ph": "X", "pid": 1, "tid": rid, "name": st, "cat": "state", "ts": a * 1e6, "dur": max(1.0, (b - a) * 1e6)})
    for rid, lat in scale_out_latencies(tr):
        ev.append({"ph": "i", "pid": 1, "tid": rid, "name": f"scale-out {lat * 1e3:.0f} ms", "cat": "scale", "s": "t",
                   "ts": next(((t or 0.0) for t, r, a, _b in tr if r == rid and a == "Inactive"), 0.0) * 1e6})
    for t, p, d in parsed["signals"]:
        ev.append({"ph": "i", "pid": 1, "tid": 0, "name": f"control P{p:+d} D{d:+d}", "cat": "planner", "s": "p", "ts": (t or 0.0) * 1e6})
    for t, p, d in parsed["metrics"]:
        ev.append({"ph": "C", "pid": 1, "name": "tokens", "ts": (t or 0.0) * 1e6, "args": {"prefill": p, "decode": d}})
    if client_records:
        ev.append({"ph": "M", "pid": 2, "name": "process_name", "args": {"name": "requests"}})
        t0 = parsed["client_start"] or 0.0
        for i, r in enumerate(client_records):
            start = t0 + float(r.get("start_s", r.get("t_submit", 0.0)))
            ttft = float(r.get("ttft_ms", 0.0)) / 1e3
            total = float(r.get("latency_ms", r.get("total_ms", ttft * 1e3))) / 1e3
            lane = i % 64
            ev.append({"ph": "X", "pid": 2, "tid": lane, "name": "queue+prefill", "cat": "request", "ts": start * 1e6,
                       "dur": max(1.0, ttft * 1e6), "args": {"input": r.get("input_length"), "id": r.get("id", i)}})
            if total > ttft:
                ev.append({"ph": "X", "pid": 2, "tid": lane, "name": "decode", "cat": "request", "ts": (start + ttft) * 1e6,
                           "dur": (total - ttft) * 1e6, "args": {"output": r.get("output_length")}})
    return {"traceEvents": ev, "displayTimeUnit": "ms"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("router_log")
    ap.add_argument("--client", default="")
    ap.add_argument("-o", "--out", required=True)
    a = ap.parse_args(argv)
    tr = chrome_trace(open(a.router_log), load_jsonl(a.client) if a.client else None)
    with open(a.out, "w") as f:
        json.dump(tr, f)
    print(f"{len(tr['traceEvents'])} events -> {a.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
