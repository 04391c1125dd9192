"""Figures of one run as a self-contained HTML file with inline SVG (no plotting library needed).

    python -m blitz_scale_b200.utils.plots --router-log router.log --client client.jsonl -o report.html

Four panels, the ones the reference's harness draws after every run (scripts/batch/plot.py:91-184, 263-280;
scripts/debug/pipe_gpu_usage.py):

* TTFT of every request over its send time, coloured by whether it violates the SLO
  `ttft > max(300 ms, 0.375 ms x input_len)`;
* the largest time between tokens of every request against the 100 ms bar;
* replica states over time (one lane per replica, one colour per state), with scale-out intervals marked;
* prefill and decode tokens per second from the router's `System Metrics` lines.
"""
from __future__ import annotations

import argparse
import html
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from .analysis import load_jsonl, parse_router_log, replica_timeline, scale_out_latencies, slo_table

W, H, ML, MR, MT, MB = 860, 240, 64, 16, 28, 34      # panel size and margins

STATE_COLOURS = {
    "Prefill": "#3b7dd8", "Decode": "#d9822b", "NewPrefill": "#7fb3f5", "OldPrefill": "#1f4e8c", "RefractoryPrefill": "#a5c8f7",
    "LoadingPrefill": "#b8c4d6", "LoadingDecode": "#e6c9a8", "AusPrefill": "#5c9ae6", "AusDecode": "#e8a35c",
    "MutatingToDecode": "#8e6bbf", "ShuttingPrefill": "#9aa5b1", "ShuttingDecode": "#b19a8a", "ShuttingNull": "#cfd4da",
}


def _ticks(lo: float, hi: float, n: int = 5) -> List[float]:
    if hi <= lo:
        return [lo]
    raw = (hi - lo) / n
    mag = 10 ** int(f"{raw:e}".split("e")[1])
    step = min((s * mag for s in (1, 2, 5, 10) if s * mag >= raw), default=raw)
    t, out = (int(lo / step)) * step, []
    while t <= hi + 1e-9:
        if t >= lo - 1e-9:
            out.append(round(t, 10))
        t += step
    return out


class Panel:
    def __init__(self, title: str, xlabel: str, ylabel: str, xr: Tuple[float, float], yr: Tuple[float, float]):
        self.title, self.xlabel, self.ylabel = title, xlabel, ylabel
        self.x0, self.x1 = xr[0], xr[1] if xr[1] > xr[0] else xr[0] + 1.0
        self.y0, self.y1 = yr[0], yr[1] if yr[1] > yr[0] else yr[0] + 1.0
        self.items: List[str] = []

    def sx(self, x: float) -> float:
        return ML + (x - self.x0) / (self.x1 - self.x0) * (W - ML - MR)

    def sy(self, y: float) -> float:
        return H - MB - (y - self.y0) / (self.y1 - self.y0) * (H - MT - MB)

    def dot(self, x: float, y: float, colour: str, r: float = 2.2) -> None:
        self.items.append(f'<circle cx="{self.sx(x):.1f}" cy="{self.sy(min(y, self.y1)):.1f}" r="{r}" fill="{colour}" fill-opacity="0.75"/>')

    def hline(self, y: float, colour: str, label: str = "") -> None:
        yy = self.sy(y)
        self.items.append(f'<line x1="{ML}" x2="{W - MR}" y1="{yy:.1f}" y2="{yy:.1f}" stroke="{colour}" stroke-dasharray="5,4"/>')
        if label:
            self.items.append(f'<text x="{W - MR - 4}" y="{yy - 4:.1f}" text-anchor="end" font-size="10" fill="{colour}">{html.escape(label)}</text>')

    def line(self, pts: Sequence[Tuple[float, float]], colour: str) -> None:
        if len(pts) >= 2:
            d = " ".join(f"{self.sx(x):.1f},{self.sy(y):.1f}" for x, y in pts)
            self.items.append(f'<polyline points="{d}" fill="none" stroke="{colour}" stroke-width="1.6"/>')

    def rect(self, xa: float, xb: float, ya: float, yb: float, colour: str, tip: str = "") -> None:
        x, w = self.sx(xa), max(0.8, self.sx(xb) - self.sx(xa))
        y, h = self.sy(yb), max(0.8, self.sy(ya) - self.sy(yb))
        t = f"<title>{html.escape(tip)}</title>" if tip else ""
        self.items.append(f'<rect x="{x:.1f}" y="{y:.1f}" width="{w:.1f}" height="{h:.1f}" fill="{colour}">{t}</rect>')

    def legend(self, entries: Sequence[Tuple[str, str]]) -> None:
        x = ML + 4
        for label, colour in entries:
            self.items.append(f'<rect x="{x}" y="{MT - 18}" width="9" height="9" fill="{colour}"/>')
            self.items.append(f'<text x="{x + 12}" y="{MT - 10}" font-size="10">{html.escape(label)}</text>')
            x += 20 + 6 * len(label)

    def svg(self, ylabels: Optional[Dict[float, str]] = None) -> str:
        out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" font-family="sans-serif">',
               f'<rect x="{ML}" y="{MT}" width="{W - ML - MR}" height="{H - MT - MB}" fill="#fafafa" stroke="#999"/>',
               f'<text x="{W - MR}" y="{MT - 10}" text-anchor="end" font-size="12" font-weight="bold">{html.escape(self.title)}</text>',
               f'<text x="{(ML + W - MR) / 2}" y="{H - 6}" text-anchor="middle" font-size="11">{html.escape(self.xlabel)}</text>',
               f'<text x="12" y="{(MT + H - MB) / 2}" text-anchor="middle" font-size="11" transform="rotate(-90 12 {(MT + H - MB) / 2})">{html.escape(self.ylabel)}</text>']
        for t in _ticks(self.x0, self.x1, 8):
            out.append(f'<line x1="{self.sx(t):.1f}" x2="{self.sx(t):.1f}" y1="{H - MB}" y2="{H - MB + 4}" stroke="#666"/>')
            out.append(f'<text x="{self.sx(t):.1f}" y="{H - MB + 15}" text-anchor="middle" font-size="10">{t:g}</text>')
        if ylabels is None:
            ylabels = {t: f"{t:g}" for t in _ticks(self.y0, self.y1, 5)}
        for t, lab in ylabels.items():
            out.append(f'<line x1="{ML - 4}" x2="{ML}" y1="{self.sy(t):.1f}" y2="{self.sy(t):.1f}" stroke="#666"/>')
            out.append(f'<text x="{ML - 6}" y="{self.sy(t) + 3:.1f}" text-anchor="end" font-size="10">{html.escape(lab)}</text>')
        return "\n".join(out + self.items + ["</svg>"])


def _pct(xs: List[float], q: float) -> float:
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(q * len(xs)))] if xs else 0.0


def ttft_panel(recs: List[dict]) -> str:
    ok = [r for r in recs if r.get("status") == "ok"]
    t_end = max((r.get("s_time", 0.0) for r in ok), default=1.0)
    cap = max(400.0, 1.15 * _pct([r["first_token_time"] for r in ok], 0.995))
    p = Panel("time to first token", "send time (s)", "TTFT (ms)", (0.0, t_end), (0.0, cap))
    for r in ok:
        bad = r["first_token_time"] > max(300.0, 0.375 * r.get("input_length", 0))
        p.dot(r.get("s_time", 0.0), r["first_token_time"], "#d6453d" if bad else "#2e8b57")
    p.hline(300.0, "#d6453d", "300 ms")
    p.legend([("within SLO", "#2e8b57"), ("violation: > max(300 ms, 0.375 ms x input)", "#d6453d")])
    return p.svg()


def tbt_panel(recs: List[dict]) -> str:
    ok = [r for r in recs if r.get("status") == "ok"]
    t_end = max((r.get("s_time", 0.0) for r in ok), default=1.0)
    cap = max(150.0, 1.15 * _pct([r.get("max_time_between_tokens", 0.0) for r in ok], 0.995))
    p = Panel("largest time between tokens", "send time (s)", "max TBT (ms)", (0.0, t_end), (0.0, cap))
    for r in ok:
        v = r.get("max_time_between_tokens", 0.0)
        p.dot(r.get("s_time", 0.0), v, "#d6453d" if v > 100.0 else "#3b7dd8")
    p.hline(100.0, "#d6453d", "100 ms")
    return p.svg()


def replica_panel(transitions, t_end: float) -> str:
    spans = replica_timeline(transitions, t_end)
    reps = sorted(spans)
    n = max(1, len(reps))
    p = Panel("replica states", "router time (s)", "replica", (0.0, t_end), (0.0, float(n)))
    used = []
    for lane, r in enumerate(reps):
        for a, b, st in spans[r]:
            if st == "Inactive":
                continue
            c = STATE_COLOURS.get(st, "#888888")
            p.rect(a or 0.0, b, n - lane - 0.85, n - lane - 0.15, c, f"replica {r}: {st} {a:.3f}-{b:.3f} s")
            if st not in used:
                used.append(st)
    p.legend([(s, STATE_COLOURS.get(s, "#888888")) for s in used[:8]])
    return p.svg({n - i - 0.5: str(r) for i, r in enumerate(reps)})


def throughput_panel(metrics) -> str:
    pts_p, pts_d = [], []
    for (t0, p0, d0), (t1, p1, d1) in zip(metrics, metrics[1:]):
        if t0 is None or t1 is None or t1 <= t0:
            continue
        pts_p.append((t1, (p1 - p0) / (t1 - t0)))
        pts_d.append((t1, (d1 - d0) / (t1 - t0)))
    top = max([v for _, v in pts_p + pts_d] + [1.0])
    t_end = max([t for t, _ in pts_p] + [1.0])
    p = Panel("tokens per second", "router time (s)", "tokens/s", (0.0, t_end), (0.0, 1.1 * top))
    p.line(pts_p, "#3b7dd8")
    p.line(pts_d, "#d9822b")
    p.legend([("prefill", "#3b7dd8"), ("decode", "#d9822b")])
    return p.svg()


def report(router_log: Iterable[str], client_records: Optional[List[dict]] = None, title: str = "run") -> str:
    parsed = parse_router_log(router_log)
    tr = parsed["transitions"]
    t_end = max([(t or 0.0) for t, *_ in tr] + [(m[0] or 0.0) for m in parsed["metrics"]] + [1.0])
    recs = client_records or []
    parts = [f"<html><head><meta charset='utf-8'><title>{html.escape(title)}</title></head><body style='font-family:sans-serif'>",
             f"<h2>{html.escape(title)}</h2>"]
    if recs:
        s = slo_table(recs)
        parts.append("<p>" + ", ".join(f"{html.escape(str(k))}: {v:.4g}" if isinstance(v, float) else f"{html.escape(str(k))}: {html.escape(str(v))}"
                                       for k, v in s.items()) + "</p>")
        parts += [ttft_panel(recs), "<br>", tbt_panel(recs), "<br>"]
    so = scale_out_latencies(tr)
    if so:
        parts.append("<p>scale-out: " + ", ".join(f"replica {r} in {1e3 * dt:.1f} ms" for r, dt in so) + "</p>")
    parts += [replica_panel(tr, t_end), "<br>", throughput_panel(parsed["metrics"]), "</body></html>"]
    return "\n".join(parts)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="figures of one run as HTML with inline SVG")
    ap.add_argument("--router-log", required=True)
    ap.add_argument("--client", default="", help="client.jsonl of the trace client")
    ap.add_argument("-o", "--output", default="report.html")
    ap.add_argument("--title", default="")
    a = ap.parse_args(argv)
    recs = load_jsonl(a.client) if a.client else None
    with open(a.router_log, errors="ignore") as f:
        doc = report(f, recs, a.title or a.router_log)
    with open(a.output, "w") as f:
        f.write(doc)
    print(a.output)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
