"""Log debuggers for the router and worker logs (the reference's scripts/debug/{awesome_grep,stp_lck_chk,bsight,
pipe_gpu_usage}.py).

    python -m blitz_scale_b200.utils.logtools merge router.log worker0.log worker1.log      # one stream, by time stamp
    python -m blitz_scale_b200.utils.logtools grep transitions router.log                   # arrow-glyph filters
    python -m blitz_scale_b200.utils.logtools zigzag worker2.log                            # per-layer ZigZag timeline
    python -m blitz_scale_b200.utils.logtools usage router.log --width 100                  # replica-state chart
    python -m blitz_scale_b200.utils.logtools migrations router.log                         # every batch migrated once?

Lines are expected to start with a time stamp: seconds as a float (`[  12.345]`, `12.345 ...`) or ISO
`2024-01-01T10:00:00.123`.  Lines without one keep the stamp of the line before them.
"""
from __future__ import annotations

import argparse
import heapq
import re
from datetime import datetime
from typing import Dict, Iterable, Iterator, List, Optional, Tuple

from .analysis import parse_router_log, replica_timeline

_TS_FLOAT = re.compile(r"^\s*\[?\s*(\d+\.\d+)\]?")
_TS_ISO = re.compile(r"^\s*\[?(\d{4}-\d{2}-\d{2}[T ]\d{2}:\d{2}:\d{2}(?:[.,]\d+)?)")

# glyphs used by the router / worker logs
FILTERS = {
    "transitions": re.compile(r"Replica<\d+>.*=>"),        # state machine: `Replica<2> Inactive => NewPrefill`
    "migrations": re.compile(r"-~>|migrat", re.I),          # KV migration: `batch 7 -~> replica 1`
    "relay": re.compile(r"\+>\+>|relay", re.I),             # ZigZag hand-off
    "zigzag": re.compile(r"~\+~|zag", re.I),                # live-execution scheduler decisions
    "scale": re.compile(r"scale|planner|control signal", re.I),
    "errors": re.compile(r"error|fail|timed out|stall", re.I),
}


def timestamp(line: str) -> Optional[float]:
    m = _TS_FLOAT.match(line)
    if m:
        return float(m.group(1))
    m = _TS_ISO.match(line)
    if m:
        s = m.group(1).replace(" ", "T").replace(",", ".")
        return datetime.fromisoformat(s).timestamp()
    return None


def stamped(lines: Iterable[str], tag: str = "") -> Iterator[Tuple[float, int, str]]:
    last, n = 0.0, 0
    for line in lines:
        t = timestamp(line)
        last = t if t is not None else last
        n += 1
        yield last, n, (f"{tag}| " if tag else "") + line.rstrip("\n")


def merge_logs(named: Dict[str, Iterable[str]]) -> Iterator[str]:
    """K-way merge of already time-ordered logs; ties keep file order, then line order."""
    streams = [((t, i, n), s) for i, (name, lines) in enumerate(named.items()) for t, n, s in stamped(lines, name)]
    for _, s in heapq.merge(*[[x for x in streams if x[0][1] == i] for i in range(len(named))], key=lambda x: x[0]):
        yield s


def grep(lines: Iterable[str], which: str) -> List[str]:
    rx = FILTERS[which]
    return [l.rstrip("\n") for l in lines if rx.search(l)]


_ZAG = re.compile(r"zag\s+(?P<ev>embed|layer|head|relay|yield)\s+batch=(?P<b>\d+)(?:\s+layer=(?P<l>\d+))?", re.I)


def zigzag_timeline(lines: Iterable[str], layers: Optional[int] = None) -> str:
    """One row per batch, one column per scheduler step: E embed, digits/letters = layer (base 36), H head,
    > relayed to the old instance, . waiting.  Shows at a glance how the live scheduler interleaved batches."""
    steps: List[Tuple[int, str]] = []
    for l in lines:
        m = _ZAG.search(l)
        if not m:
            continue
        ev, b = m.group("ev").lower(), int(m.group("b"))
        if ev == "layer":
            k = int(m.group("l") or 0)
            ch = "0123456789abcdefghijklmnopqrstuvwxyz"[k % 36]
        else:
            ch = {"embed": "E", "head": "H", "relay": ">", "yield": "."}[ev]
        steps.append((b, ch))
    batches = sorted({b for b, _ in steps})
    rows = {b: [] for b in batches}
    for b, ch in steps:
        for o in batches:
            rows[o].append(ch if o == b else " ")
    return "\n".join(f"batch {b:>6} |{''.join(r)}|" for b, r in rows.items())


_GLYPH = {"Inactive": " ", "Prefill": "P", "Decode": "D", "NewPrefill": "n", "OldPrefill": "o", "Refractory": "r",
          "LoadingPrefill": "l", "LoadingDecode": "L", "MutatingToDecode": "m", "ShuttingNull": "_"}


def usage_chart(lines: Iterable[str], width: int = 100) -> str:
    """Replica state over time, one row per replica (P prefill, D decode, l/L loading, n/o/r live scaling...)."""
    parsed = parse_router_log(lines)
    tr = parsed["transitions"]
    if not tr:
        return "(no transitions)"
    t_end = max((t or 0.0) for t, *_ in tr) * 1.02 + 1e-6
    tl = replica_timeline(tr, t_end)
    out = []
    for rid in sorted(tl):
        row = [" "] * width
        for a, b, st in tl[rid]:
            g = _GLYPH.get(st, st[:1].lower() if st.startswith("Shutting") else "?")
            for x in range(int(a / t_end * width), min(width, max(int(a / t_end * width) + 1, int(b / t_end * width)))):
                row[x] = g
        out.append(f"replica {rid:>2} |{''.join(row)}|")
    out.append(f"            0{' ' * (width - 8)}{t_end:7.2f}s")
    return "\n".join(out)


_MIG = re.compile(r"batch[ =](?P<b>\d+).*?(?P<ev>migrate start|migrate done|immigrate start|immigrate done|first half|second half)",
                  re.I)


def check_migrations(lines: Iterable[str]) -> Dict[str, List[int]]:
    """Every migrated batch must log `migrate start/done` on the source ranks and `immigrate start/done` on the
    destination ranks the same number of times (once per TP rank, twice when the batch moved in two halves after a
    ZigZag hand-off); returns the batches that do not."""
    seen: Dict[int, Dict[str, int]] = {}
    for l in lines:
        m = _MIG.search(l)
        if m:
            d = seen.setdefault(int(m.group("b")), {})
            ev = m.group("ev").lower()
            d[ev] = d.get(ev, 0) + 1
    bad, ok = [], []
    for b, d in sorted(seen.items()):
        counts = {d.get(k, 0) for k in ("migrate start", "migrate done", "immigrate start", "immigrate done")}
        good = len(counts) == 1 and 0 not in counts
        (ok if good else bad).append(b)
    return {"complete": ok, "incomplete": bad}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    m = sub.add_parser("merge"); m.add_argument("files", nargs="+")
    g = sub.add_parser("grep"); g.add_argument("which", choices=sorted(FILTERS)); g.add_argument("file")
    z = sub.add_parser("zigzag"); z.add_argument("file")
    u = sub.add_parser("usage"); u.add_argument("file"); u.add_argument("--width", type=int, default=100)
    c = sub.add_parser("migrations"); c.add_argument("file")
    a = ap.parse_args(argv)
    if a.cmd == "merge":
        for s in merge_logs({f: open(f) for f in a.files}):
            print(s)
    elif a.cmd == "grep":
        print("\n".join(grep(open(a.file), a.which)))
    elif a.cmd == "zigzag":
        print(zigzag_timeline(open(a.file)))
    elif a.cmd == "usage":
        print(usage_chart(open(a.file), a.width))
    else:
        r = check_migrations(open(a.file))
        print(f"{len(r['complete'])} complete, {len(r['incomplete'])} incomplete: {r['incomplete'][:50]}")
        return 1 if r["incomplete"] else 0
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
