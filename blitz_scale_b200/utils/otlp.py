"""OpenTelemetry span export over OTLP/HTTP with the JSON encoding, and the router's logging set-up.

The reference's router can ship its spans to an OTLP collector (`--otlp-endpoint`, service name `blitz.router`,
router_v2/src/main.rs:497-522) and formats its log as text or JSON, to stdout or through a non-blocking file
writer, filtered by the `LOG_LEVEL` environment variable (:465-533).  This module provides the same without an
OpenTelemetry SDK: spans are plain records, batched and POSTed to `<endpoint>/v1/traces` as an
`ExportTraceServiceRequest` in OTLP's JSON mapping (hex trace / span ids, times in unix nanoseconds as strings).
Export never blocks the caller: `SpanExporter.add` appends to a bounded buffer, a background task flushes it
every `interval_s`, and spans are dropped (and counted) when the collector is away.
"""
from __future__ import annotations

import asyncio
import json
import logging
import logging.handlers
import os
import queue
import secrets
import time
from typing import Dict, List, Optional

log = logging.getLogger("blitz.otlp")


def span_record(name: str, traceparent: str, start_ns: int, end_ns: int, attributes: Optional[Dict[str, object]] = None,
                parent_span_id: str = "", ok: bool = True) -> dict:
    """One span in OTLP's JSON mapping.  `traceparent` names the trace and THIS span (its third field)."""
    parts = (traceparent or "").split("-")
    tid, sid = (parts[1], parts[2]) if len(parts) == 4 else (secrets.token_hex(16), secrets.token_hex(8))
    attrs = []
    for k, v in (attributes or {}).items():
        if isinstance(v, bool):
            val = {"boolValue": v}
        elif isinstance(v, int):
            val = {"intValue": str(v)}
        elif isinstance(v, float):
            val = {"doubleValue": v}
        else:
            val = {"stringValue": str(v)}
        attrs.append({"key": k, "value": val})
    return {"traceId": tid, "spanId": sid, "parentSpanId": parent_span_id, "name": name, "kind": 1,
            "startTimeUnixNano": str(int(start_ns)), "endTimeUnixNano": str(int(end_ns)), "attributes": attrs,
            "status": {"code": 1 if ok else 2}}


def export_request(spans: List[dict], service_name: str) -> dict:
    return {"resourceSpans": [{
        "resource": {"attributes": [{"key": "service.name", "value": {"stringValue": service_name}}]},
        "scopeSpans": [{"scope": {"name": "blitz_scale_b200"}, "spans": spans}]}]}


class SpanExporter:
    def __init__(self, endpoint: str, service_name: str = "blitz.router", interval_s: float = 1.0, max_buffer: int = 8192,
                 max_batch: int = 512):
        self.url = endpoint.rstrip("/") + ("" if endpoint.rstrip("/").endswith("/v1/traces") else "/v1/traces")
        self.service_name, self.interval_s, self.max_buffer, self.max_batch = service_name, interval_s, max_buffer, max_batch
        self.buf: List[dict] = []
        self.exported = self.dropped = 0
        self._task: Optional[asyncio.Task] = None
        self._session = None

    def add(self, span: dict) -> None:
        if len(self.buf) >= self.max_buffer:
            self.dropped += 1
            return
        self.buf.append(span)

    def span(self, name: str, traceparent: str, start_s: float, end_s: float, **attributes) -> None:
        """Record a finished span from wall-clock seconds (`time.time()` values)."""
        ok = bool(attributes.pop("ok", True))
        parent = str(attributes.pop("parent_span_id", ""))
        self.add(span_record(name, traceparent, int(start_s * 1e9), int(end_s * 1e9), attributes, parent, ok))

    async def flush(self) -> int:
        import aiohttp
        sent = 0
        while self.buf:
            batch, self.buf = self.buf[:self.max_batch], self.buf[self.max_batch:]
            try:
                if self._session is None:
                    self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=5))
                async with self._session.post(self.url, data=json.dumps(export_request(batch, self.service_name)),
                                              headers={"Content-Type": "application/json"}) as r:
                    if r.status >= 300:
                        raise RuntimeError(f"collector answered {r.status}")
                self.exported += len(batch)
                sent += len(batch)
            except Exception as e:  # noqa: BLE001  the collector is optional: count, say it once in a while, go on
                self.dropped += len(batch)
                if self.dropped == len(batch) or self.dropped % 4096 < len(batch):
                    log.warning("span export to %s failed (%s); %d spans dropped so far", self.url, e, self.dropped)
        return sent

    async def run(self) -> None:
        try:
            while True:
                await asyncio.sleep(self.interval_s)
                await self.flush()
        except asyncio.CancelledError:
            await self.flush()
            raise
        finally:
            await self.close()

    async def close(self) -> None:
        if self._session is not None:
            await self._session.close()
            self._session = None

    def start(self) -> None:
        self._task = asyncio.get_running_loop().create_task(self.run())

    async def stop(self) -> None:
        if self._task is not None:
            self._task.cancel()
            try:
                await self._task
            except asyncio.CancelledError:
                pass
            self._task = None
        await self.close()


# ---------------------------------------------------------------------------------------------- logging
class JsonFormatter(logging.Formatter):
    """One JSON object per line with the event's fields flattened into it."""

    def format(self, record: logging.LogRecord) -> str:
        out = {"timestamp": time.strftime("%Y-%m-%dT%H:%M:%S", time.gmtime(record.created)) + f".{int(record.msecs):03d}Z",
               "level": record.levelname, "target": record.name, "filename": record.filename, "line_number": record.lineno,
               "message": record.getMessage()}
        if record.exc_info:
            out["exception"] = self.formatException(record.exc_info)
        return json.dumps(out)


def init_logging(level: Optional[str] = None, json_output: bool = False, log_path: str = "") -> Optional[logging.handlers.QueueListener]:
    """Root logger set-up of the router: level from the argument or the `LOG_LEVEL` environment variable (default
    info), text or JSON lines, stdout or a file written by a background thread (the caller never waits for the
    disk).  Returns the listener of the file writer (call `.stop()` at exit to drain it), else None."""
    lvl = (level or os.environ.get("LOG_LEVEL") or "INFO").upper()
    fmt: logging.Formatter = JsonFormatter() if json_output else logging.Formatter(
        "%(asctime)s %(levelname)s %(name)s %(filename)s:%(lineno)d %(message)s")
    root = logging.getLogger()
    for h in list(root.handlers):
        root.removeHandler(h)
    root.setLevel(getattr(logging, lvl, logging.INFO))
    if not log_path:
        h = logging.StreamHandler()
        h.setFormatter(fmt)
        root.addHandler(h)
        return None
    fh = logging.FileHandler(log_path, mode="w")
    fh.setFormatter(fmt)
    q: "queue.Queue" = queue.Queue(-1)
    root.addHandler(logging.handlers.QueueHandler(q))
    listener = logging.handlers.QueueListener(q, fh, respect_handler_level=False)
    listener.start()
    return listener
