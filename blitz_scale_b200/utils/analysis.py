"""Log analytics and sizing helpers (text only, no plotting library needed).

* `parse_router_log`: state transitions (`Replica<i> A => B`), control signals, `System Metrics` token lines and
  the `>>= unload` marker, the grep-able protocol the reference's tools rely on (scripts/batch/utils.py:387-502,
  scripts/debug/awesome_grep.py:6-13).
* `replica_timeline`: per-replica state intervals (the data behind the reference's stacked GPU-usage chart,
  scripts/debug/pipe_gpu_usage.py).
* `slo_table`: TTFT / TBT violation rates with the reference's thresholds (TTFT > max(300 ms, 0.375 ms x input
  length), max-TBT bar 100 ms; scripts/batch/plot.py:8-12,116-119).
* `kv_sizing`: KV bytes per token / per block, blocks that fit in a memory budget, tokens/s a link sustains
  (scripts/util/calculate_hyper_params.py:61-87), with B200 defaults.
"""
from __future__ import annotations

import json
import re
from typing import Dict, Iterable, List, Tuple

from ..models.config import get_config

_TRANS = re.compile(r"Replica<(\d+)> (\w+) => (\w+)")
_METRIC = re.compile(r"System Metrics: prefill_tokens: (\d+), decode_tokens: (\d+)")
_FLOW = re.compile(r"Replica\[(\d+)\]: Flow in: (\d+)MB, Flow out: (\d+)MB")
_SIGNAL = re.compile(r"Control signal: P([+-]\d+) D([+-]\d+)")
_STAMP = re.compile(r"^\[?\s*(\d+\.\d+)\]?")


_ISO = re.compile(r"^\[?(\d{4}-\d{2}-\d{2})[T ](\d{2}):(\d{2}):(\d{2})(?:[.,](\d+))?")


def line_time(ln: str):
    """Seconds from a log line's stamp: `[  12.345]` / `12.345 ...` (seconds) or `2024-01-01 10:00:00,123` (the
    `logging` default; also the "timestamp" field of a JSON log line; returned as seconds since midnight of the line's own date plus the day number * 86400)."""
    ln = ln.strip()
    if ln.startswith("{"):               # a JSON log line: its "timestamp" field is an ISO stamp
        m = re.search(r'"timestamp"\s*:\s*"([^"]+)"', ln)
        return line_time(m.group(1)) if m else None
    m = _STAMP.match(ln)
    if m and not _ISO.match(ln):
        return float(m.group(1))
    m = _ISO.match(ln)
    if m:
        import datetime
        day = datetime.date.fromisoformat(m.group(1)).toordinal()
        frac = float("0." + m.group(5)) if m.group(5) else 0.0
        return day * 86400.0 + int(m.group(2)) * 3600 + int(m.group(3)) * 60 + int(m.group(4)) + frac
    return None


def parse_router_log(lines: Iterable[str]) -> dict:
    """Times are relative to the first stamped line when the log carries wall-clock stamps."""
    out = {"transitions": [], "signals": [], "metrics": [], "unloads": [], "flows": [], "client_start": None}
    t0 = None
    for ln in lines:
        t = line_time(ln)
        if t is not None and t > 1e6:          # wall-clock stamp: make it relative
            t0 = t if t0 is None else t0
            t -= t0
        tr = _TRANS.search(ln)
        if tr:
            out["transitions"].append((t, int(tr.group(1)), tr.group(2), tr.group(3)))
        sg = _SIGNAL.search(ln)
        if sg:
            out["signals"].append((t, int(sg.group(1)), int(sg.group(2))))
        me = _METRIC.search(ln)
        if me:
            out["metrics"].append((t, int(me.group(1)), int(me.group(2))))
        fl = _FLOW.search(ln)
        if fl:
            out["flows"].append((t, int(fl.group(1)), int(fl.group(2)), int(fl.group(3))))   # (t, replica, MB in, MB out)
        if ">>= unload" in ln:
            out["unloads"].append(t)
        if "Client start" in ln and out["client_start"] is None:
            out["client_start"] = t
    return out


def replica_timeline(transitions: List[Tuple[float, int, str, str]], t_end: float) -> Dict[int, List[Tuple[float, float, str]]]:
    cur: Dict[int, Tuple[float, str]] = {}
    spans: Dict[int, List[Tuple[float, float, str]]] = {}
    for t, r, _a, b in transitions:
        t = 0.0 if t is None else t
        if r in cur:
            spans.setdefault(r, []).append((cur[r][0], t, cur[r][1]))
        cur[r] = (t, b)
    for r, (t0, s) in cur.items():
        spans.setdefault(r, []).append((t0, t_end, s))
    return spans


def scale_out_latencies(transitions) -> List[Tuple[int, float]]:
    """(replica, seconds) from leaving Inactive to reaching Prefill or Decode."""
    start, out = {}, []
    for t, r, a, b in transitions:
        if a == "Inactive":
            start[r] = t
        if b in ("Prefill", "Decode") and r in start and t is not None and start[r] is not None:
            out.append((r, t - start.pop(r)))
    return out


def slo_table(records: Iterable[dict]) -> dict:
    ok = [r for r in records if r.get("status") == "ok"]
    n = max(1, len(ok))
    pct = lambda xs, q: sorted(xs)[min(len(xs) - 1, int(q * len(xs)))] if xs else 0.0
    ttft = [r["first_token_time"] for r in ok]
    tbt = [r["max_time_between_tokens"] for r in ok]
    # prefill token -> first decode token: contains the KV migration, reported apart from the time between tokens
    gap = [r["first_decode_token_time"] - r["first_token_time"] for r in ok
           if r.get("first_decode_token_time", 0) > r.get("first_token_time", 0)]
    return {
        "requests": len(ok),
        "ttft_ms": {"p50": pct(ttft, .5), "p90": pct(ttft, .9), "p99": pct(ttft, .99)},
        "max_tbt_ms": {"p50": pct(tbt, .5), "p90": pct(tbt, .9), "p99": pct(tbt, .99)},
        "first_decode_gap_ms": {"p50": pct(gap, .5), "p90": pct(gap, .9), "p99": pct(gap, .99)},
        "ttft_violation_rate": sum(1 for r in ok if r["first_token_time"] > max(300.0, 0.375 * r["input_length"])) / n,
        "tbt_violation_rate": sum(1 for x in tbt if x > 100.0) / n,
    }


def load_jsonl(path: str) -> List[dict]:
    return [json.loads(l) for l in open(path) if l.strip()]


def kv_sizing(model: str, tp: int = 1, page_size: int = 64, mem_budget_gb: float = 150.0, link_gbs: float = 770.0,
              elem_bytes: int = 2) -> dict:
    c = get_config(model)
    per_token = c.kv_bytes_per_token(tp, elem_bytes)
    block = per_token * page_size
    weights_gb = c.param_gb / tp
    free = max(0.0, mem_budget_gb - weights_gb) * 1e9
    return {"kv_bytes_per_token": per_token, "block_bytes": block, "blocks_in_budget": int(free // block),
            "tokens_in_budget": int(free // per_token), "tokens_per_sec_at_link": link_gbs * 1e9 / per_token}
