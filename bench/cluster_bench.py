"""Whole-system benchmark on real GPUs: scale-out latency and TTFT / TBT under a burst, one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 bench/cluster_bench.py \
        --model llama3_8b --mode live --json out.json

Every rank runs a GPU worker (gRPC service over `GpuBackend`) in a background thread; rank 0 also runs the router
runtime in-process and replays a synthetic trace through it: a base load on 1 prefill + 1 decode replica, then a
burst, at the start of which the remaining GPUs are scaled out as prefill replicas.  `--mode`:

    stop   parameters are multicast into the new GPUs, which serve once everything has arrived (impl_blitz + impl_nvl)
    live   the new GPUs serve while loading (ZigZag: layers they hold run there, the rest on the old instance)
    sllm   the stand-in for the ServerlessLLM baseline: the new GPUs load the weights from pinned host memory (host-cache
           hit, the baseline's best case) or, with --model-path, from the segment file on disk

With --autoscale nothing is triggered by hand: the planner sees the queue grow and scales out (and back in) itself;
the latencies are then measured from the start of the burst.

Reported (rank 0, one JSON line): scale-out latency per new replica (manual trigger -> replica takes work; in
`live` mode that is before its parameters have arrived) and the time until it is fully loaded, router clock,
parameter bytes per replica, TTFT p50/p99 and TBT p50/p99 over the burst, decode tokens/s.
Weights are random (same seed everywhere); prompts are random token ids.
"""
import argparse
import asyncio
import json
import os
import sys
import threading

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pct(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(q * len(xs)))] if xs else 0.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3_8b")
    ap.add_argument("--mode", default="stop", choices=["stop", "live", "sllm"])
    ap.add_argument("--base-rate", type=float, default=4.0)
    ap.add_argument("--burst-rate", type=float, default=24.0)
    ap.add_argument("--base-s", type=float, default=2.0)
    ap.add_argument("--burst-s", type=float, default=4.0)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=32)
    ap.add_argument("--pages", type=int, default=4096)
    ap.add_argument("--model-path", default="")
    ap.add_argument("--multimem", action="store_true")
    ap.add_argument("--precapture", action="store_true", help="capture every decode graph at start-up instead of on first use")
    ap.add_argument("--autoscale", action="store_true", help="let the planner decide when and how far to scale (no manual trigger)")
    ap.add_argument("--prefill-rate", type=float, default=60000.0, help="autoscale: prefill tokens/s one replica sustains")
    ap.add_argument("--horizon-ms", type=float, default=100.0, help="autoscale: queue the planner tolerates, as time")
    ap.add_argument("--decode-steps", type=int, default=1, help="decode steps per DecodeV2 call")
    ap.add_argument("--max-incoming-migrations", type=int, default=1, help="KV migrations in flight per decode replica")
    ap.add_argument("--scale-down-ms", type=float, default=0.0,
                    help="autoscale: how long demand must stay below capacity before a replica is released (0 = the default)")
    ap.add_argument("--max-decode", type=int, default=1, help="autoscale: decode replicas the planner may use")
    ap.add_argument("--arrival-window-ms", type=float, default=0.0, help="autoscale: also size the prefill side by the "
                    "arrival rate over this window (feature planner_arrival_rate); 0 = off")
    ap.add_argument("--extra-features", default="", help="comma-separated router features added to the mode's set "
                    "(e.g. migrate_progressive)")
    ap.add_argument("--trace", default="fixed", choices=["fixed", "gamma"],
                    help="fixed: evenly spaced requests of --prompt-len / --new-tokens; gamma: Gamma inter-arrivals (CV 4) whose "
                         "rate steps from --base-rate to --burst-rate at --base-s, lognormal prompt lengths (median "
                         "--prompt-len, at most 4096) and output lengths (median --new-tokens, at most 1024)")
    ap.add_argument("--trace-sigma", type=float, default=0.8, help="gamma trace: sigma of the two lognormal length laws")
    ap.add_argument("--port", type=int, default=50600)
    ap.add_argument("--json", default="")
    a = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    host_group = dist.new_group(backend="gloo")
    from blitz_scale_b200.models.config import get_config
    from blitz_scale_b200.worker.gpu_backend import GpuBackend
    from blitz_scale_b200.worker.service import serve
    cfg_model = get_config(a.model)
    states = ["Prefill", "Decode"] + ["Inactive"] * (world - 2)
    backend = GpuBackend(rank, world, a.model, tp=1, num_pages=a.pages, page_size=64, max_batch=256, max_batch_tokens=8192,
                         ready=states[rank] != "Inactive", seed=0, use_multimem=a.multimem, model_path=a.model_path,
                         precapture=a.precapture)
    if states[rank] == "Inactive":
        if a.mode == "sllm" and not a.model_path:
            # best case of the host-cache baseline: the weights already sit in pinned host memory on this machine
            n = backend.engine.seg.layout.total_bytes
            backend.host_mirror = torch.empty(n, dtype=torch.uint8, pin_memory=True)
            backend.host_mirror.copy_(backend.engine.seg.buffer[:n])
        backend.engine.seg.buffer.zero_()
    if a.mode == "sllm" and a.model_path and rank == 0:
        backend.engine.seg.save(a.model_path)          # the file the cold replicas will load
    torch.cuda.synchronize()
    dist.barrier()

    holder, started = {}, threading.Event()

    def serve_thread():
        async def run():
            holder["loop"] = asyncio.get_running_loop()
            holder["stop"] = asyncio.Event()
            ready = asyncio.Event()
            t = asyncio.create_task(serve(backend, "127.0.0.1", a.port + rank, stop_event=holder["stop"], ready_event=ready))
            await ready.wait()
            started.set()
            await t
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        asyncio.run(run())

    th = threading.Thread(target=serve_thread, daemon=True)
    th.start()
    started.wait(120)
    dist.barrier(group=host_group)

    result = None
    if rank == 0:
        try:
            result = run_router(a, world, states, cfg_model, backend)
        except Exception:  # noqa: BLE001
            import traceback
            traceback.print_exc()
    flag = torch.tensor([1 if result else 0])
    dist.broadcast(flag, 0, group=host_group)
    logs = [None] * world
    dist.all_gather_object(logs, backend.transfer_log, group=host_group)
    if rank == 0 and result:
        src = [e for l in logs for e in (l or []) if e["role"] == "source"]
        dst = [e for l in logs for e in (l or []) if e["role"] == "destination"]
        result["param_transfer"] = {
            "device_ms_max_over_sources": round(max((e["device_ms"] for e in src), default=0.0), 3),
            "gbs_into_each_destination": round(sum(e["bytes"] / max(1, len(e["dests"])) for e in src) / 1e9 /
                                               max(1e-9, max((e["device_ms"] for e in src), default=0.0) * 1e-3), 1) if src else 0.0,
            "sources": sorted({e["rank"] for e in src}), "destinations": sorted({e["rank"] for e in dst}),
            "destination_host_ms": {str(e["rank"]): round(e["host_ms"], 2) for e in dst},
            "timing": "CUDA events around the copy kernels on every source GPU (first store to last flag), max over sources"}
    holder["loop"].call_soon_threadsafe(holder["stop"].set)
    th.join(10)
    backend.close()
    dist.barrier(group=host_group)
    if rank == 0 and result:
        print(json.dumps(result), flush=True)
        if a.json:
            os.makedirs(os.path.dirname(os.path.abspath(a.json)), exist_ok=True)
            json.dump(result, open(a.json, "w"), indent=1)
    sys.stdout.flush()
    sys.stderr.flush()
    from blitz_scale_b200.parallel.teardown import shutdown
    shutdown([backend])      # graphs, then symmetric regions, then process groups, with barriers in between
    sys.exit(0 if int(flag) else 1)


def run_router(a, world, states, cfg_model, backend):
    from blitz_scale_b200.router.runtime import RouterRuntime
    from blitz_scale_b200.router.server import controller_config_from_cluster
    feats = {"stop": "impl_blitz,impl_nvl,manually_scale", "live": "impl_blitz,impl_nvl,impl_live,manually_scale",
             "sllm": "impl_sllm,manually_scale" if a.model_path else "impl_sllm,cache_all_hit,manually_scale"}[a.mode]
    extra = {}
    if getattr(a, "autoscale", False):
        feats = feats.replace(",manually_scale", "")
        extra = dict(tokens_prefilled_per_sec=max(1, int(a.prefill_rate * a.horizon_ms * 1e-3)),
                     tokens_transferred_per_sec=5000000, max_prefill=world - 1, max_decode=max(1, a.max_decode), min_prefill=1,
                     min_decode=1)
        if a.arrival_window_ms > 0:
            feats += ",planner_arrival_rate"
            extra.update(prefill_rate_per_sec=float(a.prefill_rate), arrival_window_ms=float(a.arrival_window_ms))
        if a.scale_down_ms > 0:
            # a CV-4 arrival process has long gaps inside a burst: the patience has to cover them, or replicas are
            # released and reloaded between two clusters of arrivals
            extra["scale_down_threshold_ms"] = a.scale_down_ms
    if a.extra_features:
        feats += "," + a.extra_features.strip(",")
    cfg = controller_config_from_cluster({"init_states": states, "machines": [0] * world}, 1, feats,
                                         max_blocks_per_replica=a.pages - 64, block_size=64, max_prefill_tokens=8192,
                                         model_layers=cfg_model.layers, max_batch_seqs=256, **extra)
    cfg.max_incoming_migrations = max(1, a.max_incoming_migrations)
    g = torch.Generator().manual_seed(5)
    if a.trace == "gamma":
        # the bursty synthetic trace of the second benchmark configuration, from the native generator (seeded)
        from blitz_scale_b200.runtime import core
        spec = core.TraceSpec()
        spec.phases = [core.RatePhase(0.0, a.base_rate), core.RatePhase(a.base_s, a.burst_rate)]
        spec.cv, spec.duration, spec.seed = 4.0, a.base_s + a.burst_s, 0
        spec.input.kind, spec.input.a, spec.input.b, spec.input.max_len, spec.input.min_len = \
            core.LengthDist.Kind.LogNormal, float(a.prompt_len), a.trace_sigma, 4096, 8
        spec.output.kind, spec.output.a, spec.output.b, spec.output.max_len, spec.output.min_len = \
            core.LengthDist.Kind.LogNormal, float(a.new_tokens), a.trace_sigma, 1024, 2
        items = core.generate_trace(spec)
        arrivals = [it.t for it in items]
        in_lens, out_lens = [int(it.input_len) for it in items], [int(it.output_len) for it in items]
    else:
        n_base, n_burst = int(a.base_rate * a.base_s), int(a.burst_rate * a.burst_s)
        arrivals = [i / a.base_rate for i in range(n_base)] + [a.base_s + i / a.burst_rate for i in range(n_burst)]
        in_lens, out_lens = [a.prompt_len] * len(arrivals), [a.new_tokens] * len(arrivals)
    prompts = [torch.randint(0, cfg_model.vocab, (n,), generator=g).tolist() for n in in_lens]

    async def go():
        rt = RouterRuntime(cfg, [f"127.0.0.1:{a.port + r}" for r in range(world)], model_layers=cfg_model.layers,
                           model_path=a.model_path, decode_steps=a.decode_steps)
        loop_task = asyncio.create_task(rt.run())
        # warm both serving replicas (graph capture, first-use work) outside the measurement
        warm = rt.submit(prompts[0], 4)
        while True:
            ev = await asyncio.wait_for(warm.queue.get(), timeout=300)
            if ev[0] == "error" or ev[2]:
                break
        records = []

        async def one(i, t_arr):
            await asyncio.sleep(max(0.0, t_arr - (rt.now() - t_start)))
            t0 = rt.now()
            # whole response at once (what POST /generate does): the token times are the router's delivery times
            lr = rt.submit(prompts[i], out_lens[i], stream=False)
            if await asyncio.wait_for(lr.done, timeout=300):
                records.append({"i": i, "ok": False})
                return
            times = list(lr.times)
            tbt = [b - c for b, c in zip(times[1:], times[:-1])]
            records.append({"i": i, "ok": True, "burst": t_arr >= a.base_s, "ttft": times[0] - t0, "tbt": tbt,
                            "tokens": len(times), "done": times[-1]})

        t_start = rt.now()
        tasks = [asyncio.create_task(one(i, t)) for i, t in enumerate(arrivals)]
        await asyncio.sleep(a.base_s)
        t_trigger = rt.now()
        if not getattr(a, "autoscale", False):
            for r in range(2, world):
                assert rt.ctl.manual_scale(r, "Prefill", rt.now())
            rt.wake.set()
        await asyncio.gather(*tasks)
        t_end = rt.now()
        scale, loaded, decided = {}, {}, {}
        for t, line in rt.transitions:
            for r in range(2, world):
                if f"Replica<{r}>" not in line or t < t_trigger:
                    continue
                if r not in decided and f"Replica<{r}> Inactive =>" in line:
                    decided[r] = t - t_trigger            # the planner's (or the manual) decision: the replica leaves Inactive
                if r not in scale and line.rstrip().endswith(("=> Prefill", "=> NewPrefill")):
                    scale[r] = t - t_trigger              # first moment the replica takes work
                if r not in loaded and line.rstrip().endswith("=> Prefill"):
                    loaded[r] = t - t_trigger             # all parameters resident, ordinary prefill replica
        scale = {"serving": scale, "loaded": loaded, "decided": decided}
        await rt.stop()
        loop_task.cancel()
        return records, scale, t_start, t_end, [l for _, l in rt.transitions if "boot" not in l]

    records, scale, t_start, t_end, transitions = asyncio.run(go())
    ok = [r for r in records if r["ok"]]
    burst = [r for r in ok if r["burst"]]
    # as in the reference's statistics, the interval between the prefill token and the first decode token (which
    # contains the KV migration) is not a time-between-tokens sample; it is reported on its own
    tbt_all = [x for r in burst for x in r["tbt"][1:]]
    first_gap = [r["tbt"][0] for r in burst if r["tbt"]]
    seg_bytes = backend.engine.seg.layout.total_bytes
    out = {"bench": "cluster_scale_out", "model": a.model, "mode": a.mode + ("+autoscale" if getattr(a, "autoscale", False) else ""),
           "gpus": world, "requests": len(records), "trace": a.trace,
           "input_len_p50_max": [sorted(in_lens)[len(in_lens) // 2], max(in_lens)],
           "output_len_p50_max": [sorted(out_lens)[len(out_lens) // 2], max(out_lens)],
           "failed": len(records) - len(ok), "prompt_len": a.prompt_len, "new_tokens": a.new_tokens,
           "base_rate": a.base_rate, "burst_rate": a.burst_rate, "decode_steps_per_call": a.decode_steps,
           "max_incoming_migrations": a.max_incoming_migrations, "precapture": bool(a.precapture),
           "scale_out_latency_ms": {str(r): round(v * 1e3, 2) for r, v in sorted(scale["serving"].items())},
           "fully_loaded_ms": {str(r): round(v * 1e3, 2) for r, v in sorted(scale["loaded"].items())},
           # with --autoscale the clock starts when the burst begins, so the figures above contain the time the planner
           # needed to see the burst; these two split it off
           "decision_ms": {str(r): round(v * 1e3, 2) for r, v in sorted(scale["decided"].items())},
           "serving_after_decision_ms": {str(r): round((v - scale["decided"].get(r, 0.0)) * 1e3, 2)
                                         for r, v in sorted(scale["serving"].items())},
           "loaded_after_decision_ms": {str(r): round((v - scale["decided"].get(r, 0.0)) * 1e3, 2)
                                        for r, v in sorted(scale["loaded"].items())},
           "param_gb_per_replica": round(seg_bytes / 1e9, 3),
           "effective_gbs_per_replica": {str(r): round(seg_bytes / v / 1e9, 1) for r, v in sorted(scale["loaded"].items()) if v > 0},
           "ttft_ms_p50": round(pct([r["ttft"] for r in burst], 0.5) * 1e3, 2),
           "ttft_ms_p99": round(pct([r["ttft"] for r in burst], 0.99) * 1e3, 2),
           "tbt_ms_p50": round(pct(tbt_all, 0.5) * 1e3, 2), "tbt_ms_p99": round(pct(tbt_all, 0.99) * 1e3, 2),
           "first_decode_gap_ms_p50": round(pct(first_gap, 0.5) * 1e3, 2),
           "first_decode_gap_ms_p99": round(pct(first_gap, 0.99) * 1e3, 2),
           "tokens_per_s": round(sum(r["tokens"] for r in ok) / max(1e-9, t_end - t_start), 1),
           "transitions": transitions[:24], "timing": "router wall clock (host), one box"}
    return out


if __name__ == "__main__":
    main()
