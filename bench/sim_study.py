"""Autoscaling study in virtual time: the real controller (planner, executors, migration, live scaling) driven by a
cost model calibrated with this repository's B200 measurements, replaying bursty traces.  No GPU involved: this is
a model of the cluster, not a measurement of it; it shows how the policies compare once the measured transfer and
step times are plugged in.

    python bench/sim_study.py [--model llama3_8b|mistral_24b] [--horizon-ms 100] [--json out.json]

Calibration (B200, bf16; numbers measured with bench.py, bench/comm_bench.py and bench/cluster_bench.py):
  llama3_8b    prefill 1024 tokens in ~17 ms; decode step 4.2 / 5.1 / 6.3 / 9.5 ms at batch 16 / 64 / 128 / 256;
               16.06 GB per replica; striped multicast 630 GB/s into every destination; pinned host 55 GB/s;
               KV push 690 GB/s = 5.3 M tokens/s.
  mistral_24b  TP2: decode step 6.8 ms at batch 16, 13.0 ms at batch 256 (measured); prefill and sizes scaled by
               parameter count.  (A TP4 model leaves two replicas on an 8-GPU box, so there is nothing to scale out to.)
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from blitz_scale_b200.runtime import core  # noqa: E402

MODELS = {
    # replicas of tp GPUs on one 8-GPU box
    "llama3_8b": dict(tp=1, replicas=8, param_gb=16.06, prefill_tps=65000, dec_base=0.0040, dec_per_seq=0.0000215, kv_bytes=131072),
    "mistral_24b": dict(tp=2, replicas=4, param_gb=23.6, prefill_tps=42000, dec_base=0.0064, dec_per_seq=0.0000258, kv_bytes=81920),
}
POLICIES = {
    "multicast, stop-the-world load (impl_blitz,impl_nvl)": "impl_blitz,impl_nvl",
    "multicast + live execution (impl_blitz,impl_nvl,impl_live)": "impl_blitz,impl_nvl,impl_live",
    "multicast + arrival-rate signal (impl_blitz,impl_nvl,planner_arrival_rate)": "impl_blitz,impl_nvl,planner_arrival_rate",
    "host-cache load (impl_sllm,cache_all_hit)": "impl_sllm,cache_all_hit",
    "disk load (impl_sllm,cache_all_miss)": "impl_sllm,cache_all_miss",
}


def pct(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(q * len(xs)))] if xs else 0.0


def run(model: str, burst_factor: float, horizon_ms: float, seed: int = 0):
    m = MODELS[model]
    R, tp = m["replicas"], m["tp"]
    cm = core.CostModel()
    cm.prefill_tokens_per_s, cm.prefill_overhead_s = m["prefill_tps"], 0.002
    cm.decode_step_base_s, cm.decode_step_per_seq_s = m["dec_base"], m["dec_per_seq"]
    cm.kv_tokens_per_s, cm.migrate_overhead_s = 690e9 / m["kv_bytes"], 0.0003
    cm.param_gb, cm.nvlink_gbs, cm.host_gbs, cm.disk_gbs = m["param_gb"], 630.0, 55.0, 6.0
    # a trace that one prefill replica handles at the base rate and cannot handle in the burst
    base = 0.35 * m["prefill_tps"] / 1024.0
    spec = core.TraceSpec()
    spec.phases = [core.RatePhase(0.0, base), core.RatePhase(5.0, base * burst_factor), core.RatePhase(11.0, base)]
    spec.duration, spec.seed, spec.cv = 18.0, seed, 2.0
    spec.input.kind, spec.input.a, spec.input.b = core.LengthDist.Kind.Uniform, 256, 1792
    spec.output.kind, spec.output.a, spec.output.b = core.LengthDist.Kind.Uniform, 16, 128
    trace = core.generate_trace(spec)
    rows = []
    for name, feats in POLICIES.items():
        cfg = core.ControllerConfig()
        cfg.num_ranks, cfg.tp = R * tp, tp
        cfg.init_states = sum([[s] * tp for s in ["Prefill", "Decode"] + ["Inactive"] * (R - 2)], [])
        cfg.features = feats
        cfg.max_blocks_per_replica = 30000
        p = cfg.planner
        # The planner adds a prefill replica when the queued prompt tokens exceed (upper bound x capacity); the
        # reference states capacity per second, i.e. it tolerates most of a second of queue before it reacts, which
        # suits transfers that take seconds.  With a 26 ms scale-out the same rule can run on a much shorter horizon.
        p.tokens_prefilled_per_sec = max(1, int(m["prefill_tps"] * horizon_ms * 1e-3))
        p.tokens_transferred_per_sec = int(cm.kv_tokens_per_s)
        p.max_prefill, p.max_decode = R - 1, R - 1
        # only read with the feature planner_arrival_rate: prompt tokens arrived in the last 200 ms against the rate of
        # one replica, as a second lower bound on the prefill side
        p.prefill_rate_per_sec, p.arrival_window_ms = float(m["prefill_tps"]), 200.0
        cfg.planner = p
        rep = core.ClusterSim(cfg, cm).run(trace)
        burst = [r for r in rep.requests if 5.0 <= r.t_arrival < 11.0]
        ttft = [r.ttft for r in burst]
        viol = sum(1 for r in burst if r.ttft > max(0.3, 0.000375 * r.input_len)) / max(1, len(burst))

        def mean_count(samples, t_lo=5.0, t_hi=11.0):      # time-weighted replicas of a role during the burst
            area, t_prev, n_prev = 0.0, t_lo, 0
            for t, n in samples:                           # (time, count) whenever the count changed
                if t <= t_lo:
                    n_prev = n
                    continue
                if t >= t_hi:
                    break
                area += (t - t_prev) * n_prev
                t_prev, n_prev = t, n
            return (area + (t_hi - t_prev) * n_prev) / (t_hi - t_lo)
        rows.append({"policy": name, "requests": len(rep.requests), "failed": rep.failed,
                     "scale_outs": len(rep.scale_up_latency),
                     "gpus_in_burst": round((mean_count(rep.prefill_replicas) + mean_count(rep.decode_replicas)) * tp, 2),
                     "scale_out_latency_ms": round(1e3 * (sum(rep.scale_up_latency.values()) / max(1, len(rep.scale_up_latency))), 1),
                     "ttft_ms_p50": round(1e3 * pct(ttft, 0.5), 1), "ttft_ms_p99": round(1e3 * pct(ttft, 0.99), 1),
                     "max_tbt_ms_p99": round(1e3 * pct([r.max_tbt for r in burst], 0.99), 1),
                     "ttft_violation_rate": round(viol, 4)})
    return {"model": model, "tp": tp, "replicas": R, "planner_horizon_ms": horizon_ms, "base_rps": round(base, 1), "burst_rps": round(base * burst_factor, 1),
            "trace_requests": len(trace), "rows": rows, "kind": "virtual-time simulation, calibrated cost model"}


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="all")
    ap.add_argument("--burst", type=float, default=6.0, help="burst rate as a multiple of the base rate")
    ap.add_argument("--horizon-ms", type=float, default=1000.0, help="queue the planner tolerates per replica, as time "
                    "(1000 = the reference's per-second capacity rule)")
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    out = [run(m, a.burst, a.horizon_ms) for m in (MODELS if a.model == "all" else [a.model])]
    for o in out:
        print(f"\n{o['model']} (tp {o['tp']}, {o['replicas']} replicas): {o['base_rps']} -> {o['burst_rps']} req/s, "
              f"{o['trace_requests']} requests, planner horizon {o['planner_horizon_ms']:.0f} ms  [{o['kind']}]")
        print(f"{'policy':76s} {'ups':>3s} {'GPUs':>5s} {'scale-out ms':>12s} {'TTFT p50':>9s} {'TTFT p99':>9s} {'maxTBT p99':>10s} {'SLO viol':>8s}")
        for r in o["rows"]:
            print(f"{r['policy']:76s} {r['scale_outs']:3d} {r['gpus_in_burst']:5.2f} {r['scale_out_latency_ms']:12.1f} {r['ttft_ms_p50']:9.1f} "
                  f"{r['ttft_ms_p99']:9.1f} {r['max_tbt_ms_p99']:10.1f} {r['ttft_violation_rate']:8.4f}")
    if a.json:
        json.dump(out, open(a.json, "w"), indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
