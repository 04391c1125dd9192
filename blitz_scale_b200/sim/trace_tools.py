"""Trace files for the request simulator: `timestamp(ms),prefill,decode` CSV rows.

Slicing, time scaling, concatenation and summary of traces, and comparison of SLO-violation tables between runs
(the reference's dataset utilities: scripts/figure/process_dataset_v2.py:40-55, scripts/util/concat_dataset.py,
scripts/util/compare_violation.py).

    python -m blitz_scale_b200.sim.trace_tools slice in.csv out.csv --start-s 60 --length-s 120
    python -m blitz_scale_b200.sim.trace_tools scale in.csv out.csv --rate 2.0 --max-prefill 4095
    python -m blitz_scale_b200.sim.trace_tools concat a.csv b.csv out.csv --gap-s 5
    python -m blitz_scale_b200.sim.trace_tools stats in.csv
    python -m blitz_scale_b200.sim.trace_tools compare runA/client.jsonl runB/client.jsonl
"""
from __future__ import annotations

import argparse
import csv
import json
from typing import Iterable, List, Tuple

Row = Tuple[float, int, int]     # (ms, prompt tokens, output tokens)


def read_trace(path: str) -> List[Row]:
    rows: List[Row] = []
    with open(path, newline="") as f:
        for r in csv.reader(f):
            if not r or not r[0].strip() or not r[0].strip()[0].isdigit():
                continue                                # header or comment
            rows.append((float(r[0]), int(float(r[1])), int(float(r[2]))))
    rows.sort(key=lambda x: x[0])
    return rows


def write_trace(path: str, rows: Iterable[Row]) -> None:
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["timestamp", "prefill", "decode"])
        for t, p, d in rows:
            w.writerow([f"{t:.3f}", p, d])


def slice_trace(rows: List[Row], start_s: float, length_s: float) -> List[Row]:
    a, b = start_s * 1e3, (start_s + length_s) * 1e3
    return [(t - a, p, d) for t, p, d in rows if a <= t < b]


def scale_trace(rows: List[Row], rate: float = 1.0, max_prefill: int = 0, max_decode: int = 0) -> List[Row]:
    """`rate` > 1 compresses time (more requests per second); lengths are clamped, not dropped."""
    out = []
    for t, p, d in rows:
        out.append((t / rate, min(p, max_prefill) if max_prefill else p, min(d, max_decode) if max_decode else d))
    return out


def concat_traces(parts: List[List[Row]], gap_s: float = 0.0) -> List[Row]:
    out, base = [], 0.0
    for rows in parts:
        out += [(t + base, p, d) for t, p, d in rows]
        if rows:
            base = out[-1][0] + gap_s * 1e3
    return out


def trace_stats(rows: List[Row], window_s: float = 10.0) -> dict:
    if not rows:
        return {"requests": 0}
    dur = max(1e-9, (rows[-1][0] - rows[0][0]) / 1e3)
    buckets = {}
    for t, p, d in rows:
        buckets[int(t / 1e3 / window_s)] = buckets.get(int(t / 1e3 / window_s), 0) + 1
    rates = [n / window_s for n in buckets.values()]
    return {"requests": len(rows), "duration_s": dur, "mean_rps": len(rows) / dur, "peak_rps": max(rates),
            "burstiness": max(rates) / (len(rows) / dur), "mean_prefill": sum(p for _, p, _ in rows) / len(rows),
            "mean_decode": sum(d for _, _, d in rows) / len(rows), "prefill_tokens_per_s": sum(p for _, p, _ in rows) / dur}


def compare_violations(a_path: str, b_path: str) -> dict:
    from ..utils.analysis import load_jsonl, slo_table
    a, b = slo_table(load_jsonl(a_path)), slo_table(load_jsonl(b_path))
    keys = [k for k in a if isinstance(a[k], (int, float)) and k in b]
    return {"a": a, "b": b, "delta": {k: b[k] - a[k] for k in keys}}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("slice"); s.add_argument("src"); s.add_argument("dst")
    s.add_argument("--start-s", type=float, default=0.0); s.add_argument("--length-s", type=float, required=True)
    c = sub.add_parser("scale"); c.add_argument("src"); c.add_argument("dst"); c.add_argument("--rate", type=float, default=1.0)
    c.add_argument("--max-prefill", type=int, default=0); c.add_argument("--max-decode", type=int, default=0)
    k = sub.add_parser("concat"); k.add_argument("files", nargs="+"); k.add_argument("--gap-s", type=float, default=0.0)
    t = sub.add_parser("stats"); t.add_argument("src")
    v = sub.add_parser("compare"); v.add_argument("a"); v.add_argument("b")
    a = ap.parse_args(argv)
    if a.cmd == "slice":
        write_trace(a.dst, slice_trace(read_trace(a.src), a.start_s, a.length_s))
    elif a.cmd == "scale":
        write_trace(a.dst, scale_trace(read_trace(a.src), a.rate, a.max_prefill, a.max_decode))
    elif a.cmd == "concat":
        *srcs, dst = a.files
        write_trace(dst, concat_traces([read_trace(f) for f in srcs], a.gap_s))
    elif a.cmd == "stats":
        print(json.dumps(trace_stats(read_trace(a.src)), indent=1))
    else:
        print(json.dumps(compare_violations(a.a, a.b), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
