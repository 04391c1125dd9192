"""Trace-replay client ("request-sim").

Replays a synthetic or CSV trace against the router's `/generate` endpoint in open loop (each request is
sent at its trace timestamp regardless of earlier responses), reads the timing headers of every
response and writes one JSON line per request to `client.jsonl`.  Flags and output fields follow what
the reference's harness passes to and expects from its trace client (scripts/batch/runner.py:471-492,
scripts/batch/utils.py:345-357): `--endpoint --protocol st --replay-mode --scale-factor --dataset-type
--dataset-path --time-in-secs --truncate --output-path`; it prints a line containing `Client start`
(scripts/batch/runner.py:30) when the replay begins.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import time
from typing import List, Optional

import aiohttp

from ..runtime import core


def make_mock_trace(rate: float, duration: float, seed: int = 0, cv: float = 1.0, input_rng=(32, 512),
                    output_rng=(16, 128), max_requests: int = 10 ** 9, rate_step=None, lognormal=None):
    """Synthetic traces of the benchmark configurations: Poisson / Gamma arrivals, uniform or lognormal lengths."""
    s = core.TraceSpec()
    phases = [core.RatePhase(0.0, rate)]
    if rate_step is not None:
        phases.append(core.RatePhase(rate_step[0], rate_step[1]))
    s.phases, s.duration, s.seed, s.cv, s.max_requests = phases, duration, seed, cv, max_requests
    if lognormal is not None:
        (imed, imax), (omed, omax) = lognormal
        s.input.kind, s.input.a, s.input.b, s.input.max_len = core.LengthDist.Kind.LogNormal, imed, 1.0, imax
        s.output.kind, s.output.a, s.output.b, s.output.max_len = core.LengthDist.Kind.LogNormal, omed, 1.0, omax
    else:
        s.input.kind, s.input.a, s.input.b = core.LengthDist.Kind.Uniform, input_rng[0], input_rng[1]
        s.output.kind, s.output.a, s.output.b = core.LengthDist.Kind.Uniform, output_rng[0], output_rng[1]
    return core.generate_trace(s)


def token_ids_for(item, vocab: int = 32000) -> List[int]:
    """Uniform token ids, a deterministic function of the trace item's seed."""
    r = core.Rng(item.seed)
    return [int(r.uniform_int(0, vocab - 1)) for _ in range(item.input_len)]


async def _one(session, endpoint: str, idx: int, item, t0: float, out: list, vocab: int, record_tokens: bool):
    s_time = time.monotonic() - t0
    body = {"input_tokens": token_ids_for(item, vocab),
            # a replayed trace fixes every output length: the end-of-sequence token must not cut a request short
            "parameters": {"max_new_tokens": int(item.output_len), "details": record_tokens, "ignore_eos_token": True}}
    rec = {"request_id": idx, "status": "error", "s_time": s_time, "input_length": int(item.input_len),
           "output_length": int(item.output_len)}
    try:
        async with session.post(endpoint, json=body) as resp:
            data = await resp.json()
            h = resp.headers
            rec["status"] = "ok" if resp.status == 200 else f"http_{resp.status}"
            if resp.status == 200:
                g = lambda k: float(h.get(k, 0))
                rec.update(first_token_time=g("x-first-token-time"), inference_time=g("x-inference-time"),
                           queue_time=g("x-queue-time"), max_time_between_tokens=g("x-max-time-between-tokens"),
                           avg_time_between_tokens=g("x-avg-time-between-tokens"),
                           p95_time_between_tokens=g("x-p95-time-between-tokens"),
                           p99_time_between_tokens=g("x-p99-time-between-tokens"),
                           first_decode_token_time=g("x-first-decode-token-time"), total_time=g("x-total-time"),
                           generated_tokens=int(g("x-generated-tokens")))
                if record_tokens and data.get("details"):
                    rec["tokens"] = [t["id"] for t in data["details"]["tokens"]]
                    rec["finish_reason"] = data["details"].get("finish_reason")
            else:
                rec["error"] = data.get("error")
    except Exception as e:  # noqa: BLE001
        rec["error"] = f"{type(e).__name__}: {e}"
    rec["e_time"] = time.monotonic() - t0
    out.append(rec)


async def replay(endpoint: str, trace, output_path: Optional[str] = None, scale_factor: float = 1.0,
                 time_in_secs: Optional[float] = None, vocab: int = 32000, record_tokens: bool = False) -> list:
    out, tasks = [], []
    conn = aiohttp.TCPConnector(limit=0)
    async with aiohttp.ClientSession(connector=conn, timeout=aiohttp.ClientTimeout(total=None)) as session:
        print("Client start", flush=True)
        t0 = time.monotonic()
        for i, item in enumerate(trace):
            t = item.t / scale_factor
            if time_in_secs is not None and t > time_in_secs:
                break
            delay = t - (time.monotonic() - t0)
            if delay > 0:
                await asyncio.sleep(delay)
            tasks.append(asyncio.create_task(_one(session, endpoint, i, item, t0, out, vocab, record_tokens)))
        await asyncio.gather(*tasks)
    out.sort(key=lambda r: r["request_id"])
    if output_path:
        with open(output_path, "w") as f:
            for r in out:
                f.write(json.dumps(r) + "\n")
    return out


def summarize(records: list) -> dict:
    ok = [r for r in records if r["status"] == "ok"]
    pct = lambda xs, q: sorted(xs)[min(len(xs) - 1, int(q * len(xs)))] if xs else 0.0
    ttft = [r["first_token_time"] for r in ok]
    tbt = [r["max_time_between_tokens"] for r in ok]
    # TTFT SLO of the reference's plots: violated if TTFT > max(300 ms, 0.375 ms * input_len) (scripts/batch/plot.py:116-119)
    viol = sum(1 for r in ok if r["first_token_time"] > max(300.0, 0.375 * r["input_length"]))
    gap = [r["first_decode_token_time"] - r["first_token_time"] for r in ok
           if r.get("first_decode_token_time", 0) > r.get("first_token_time", 0)]
    return {"requests": len(records), "ok": len(ok), "ttft_p50_ms": pct(ttft, .5), "ttft_p99_ms": pct(ttft, .99),
            "first_decode_gap_p50_ms": pct(gap, .5), "first_decode_gap_p99_ms": pct(gap, .99),
            "max_tbt_p50_ms": pct(tbt, .5), "max_tbt_p99_ms": pct(tbt, .99),
            "ttft_slo_violation_rate": viol / max(1, len(ok)),
            "tbt_slo_violation_rate": sum(1 for x in tbt if x > 100.0) / max(1, len(ok)),
            "output_tokens": sum(r.get("generated_tokens", 0) for r in ok)}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser("request-sim")
    ap.add_argument("--endpoint", default="http://127.0.0.1:3000/generate")
    ap.add_argument("--protocol", default="st")
    ap.add_argument("--replay-mode", action="store_true")
    ap.add_argument("--scale-factor", type=float, default=1.0)
    ap.add_argument("--dataset-type", default="mock", choices=["mock", "csv"])
    ap.add_argument("--dataset-path", default="")
    ap.add_argument("--time-in-secs", type=float, default=None)
    ap.add_argument("--truncate", type=int, default=4095)
    ap.add_argument("--output-path", default="client.jsonl")
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--rate", type=float, default=4.0)
    ap.add_argument("--cv", type=float, default=1.0)
    ap.add_argument("--duration", type=float, default=50.0)
    ap.add_argument("--num-requests", type=int, default=200)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--vocab", type=int, default=32000, help="synthetic token ids are drawn from [0, vocab)")
    a = ap.parse_args(argv)
    if a.dataset_type == "csv" or a.dataset_path:
        trace = core.load_trace_csv(a.dataset_path, 1.0, a.truncate)
    else:
        trace = make_mock_trace(a.rate, a.duration, a.seed, a.cv, max_requests=a.num_requests)
    recs = asyncio.run(replay(a.endpoint, trace, a.output_path, a.scale_factor, a.time_in_secs, vocab=a.vocab))
    print(json.dumps(summarize(recs)))


if __name__ == "__main__":
    main()
