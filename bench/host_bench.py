"""Host-side (CPU) microbenchmarks of the control plane and IO paths.  No GPU involved.

    python bench/host_bench.py [--json out.json] [--quick]

Measures, on the machine it runs on:
  * controller: cost of one `step()` of the router core with many replicas and a deep queue, and how much simulated
    cluster time the virtual-time simulator covers per wall second (the planner runs inside `step()`, so "a scale
    decision within one tick" holds when a step costs far less than the tick);
  * queue: requests batched per second by the native batch queue;
  * tokenizer: encode / decode throughput of the native BPE tokenizer (and of the `tokenizers` library on the same
    model when it is installed);
  * loader: throughput of the native multi-threaded segment-file reader (page cache warm);
  * RPC: round-trip latency of worker RPCs over loopback gRPC against a stub worker (what the transport adds to a
    decode step), router-level requests/s with stub workers, and the same through the HTTP API (`POST /generate`) with
    the router started from its command line.
"""
import argparse
import asyncio
import json
import os
import socket
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from blitz_scale_b200.runtime import core  # noqa: E402


def _pct(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(q * len(xs)))] if xs else 0.0


def bench_controller(quick: bool) -> dict:
    out = {}
    for reps in (8, 64):
        cfg = core.ControllerConfig()
        states = ["Prefill"] * (reps // 2) + ["Decode"] * (reps // 2)
        cfg.num_ranks, cfg.tp, cfg.init_states = reps, 1, states
        cfg.features = "impl_blitz,impl_nvl"
        ctl = core.Controller(cfg)
        n_req = 2000 if quick else 20000
        for i in range(n_req):
            e = core.RequestEntry()
            e.id, e.input_len, e.max_new_tokens, e.t_arrival = i, 512, 64, 0.0
            ctl.submit(e)
        # steps with every replica busy (nothing completes): the per-tick cost of scanning replicas, queue and planner
        ctl.step(0.0)
        n = 2000 if quick else 20000
        t0 = time.perf_counter()
        for k in range(n):
            ctl.step(0.001 * (k + 1))
        dt = time.perf_counter() - t0
        out[f"step_us_{reps}_replicas_queue_{n_req}"] = round(dt / n * 1e6, 2)
    # simulator speed on a bursty trace with autoscaling
    spec = core.TraceSpec()
    spec.phases = [core.RatePhase(0.0, 8.0), core.RatePhase(5.0, 60.0), core.RatePhase(10.0, 8.0)]
    spec.duration, spec.seed, spec.cv = (8.0 if quick else 30.0), 1, 2.0
    spec.input.kind, spec.input.a, spec.input.b = core.LengthDist.Kind.Uniform, 64, 1024
    spec.output.kind, spec.output.a, spec.output.b = core.LengthDist.Kind.Uniform, 16, 128
    trace = core.generate_trace(spec)
    cfg = core.ControllerConfig()
    cfg.num_ranks, cfg.tp = 8, 1
    cfg.init_states = ["Prefill", "Decode"] + ["Inactive"] * 6
    cfg.features = "impl_blitz,impl_nvl,impl_live"
    t0 = time.perf_counter()
    rep = core.ClusterSim(cfg, core.CostModel()).run(trace)
    dt = time.perf_counter() - t0
    out["sim_requests"] = len(trace)
    out["sim_seconds_per_wall_second"] = round(rep.end_time / dt, 1)
    out["sim_ticks_per_second"] = round(rep.end_time / 0.001 / dt)
    return out


def bench_queue(quick: bool) -> dict:
    q = core.BatchQueue(64)
    n = 20000 if quick else 200000
    t0 = time.perf_counter()
    for i in range(n):
        e = core.RequestEntry()
        e.id, e.input_len, e.max_new_tokens = i, 100 + i % 400, 32
        q.append(e)
    t_app = time.perf_counter() - t0
    got = 0
    t0 = time.perf_counter()
    while True:
        nb = q.next_batch(None, 8192, 10 ** 9)
        if nb is None:
            break
        got += len(nb.entries)
    t_bat = time.perf_counter() - t0
    assert got == n
    return {"append_per_s": round(n / t_app), "batched_requests_per_s": round(n / t_bat)}


def bench_tokenizer(quick: bool) -> dict:
    try:
        from tokenizers import Tokenizer, models, pre_tokenizers, decoders, trainers
    except Exception:  # noqa: BLE001
        return {"skipped": "tokenizers library not installed (needed to train a vocabulary)"}
    import random
    rng = random.Random(0)
    words = ["".join(rng.choice("abcdefghijklmnopqrstuvwxyz") for _ in range(rng.randint(2, 9))) for _ in range(3000)]
    corpus = [" ".join(rng.choice(words) for _ in range(40)) + "." for _ in range(2000)]
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=4000, special_tokens=["<s>", "</s>"],
                                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                                        show_progress=False))
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "tokenizer.json")
        tok.save(path)
        nat = core.Tokenizer.from_file(path)
        text = " ".join(corpus[: (100 if quick else 1000)])
        nbytes = len(text.encode())
        t0 = time.perf_counter()
        ids = nat.encode(text)
        t_nat = time.perf_counter() - t0
        t0 = time.perf_counter()
        ref = tok.encode(text).ids
        t_ref = time.perf_counter() - t0
        assert list(ids) == list(ref)
        t0 = time.perf_counter()
        back = nat.decode(ids)
        t_dec = time.perf_counter() - t0
        assert back == text
        # request-sized inputs: latency per call
        prompts = corpus[:200]
        t0 = time.perf_counter()
        for p in prompts:
            nat.encode(p)
        per_call = (time.perf_counter() - t0) / len(prompts)
    return {"encode_mb_per_s": round(nbytes / t_nat / 1e6, 2), "library_encode_mb_per_s": round(nbytes / t_ref / 1e6, 2),
            "decode_mtok_per_s": round(len(ids) / t_dec / 1e6, 2), "encode_us_per_200_char_prompt": round(per_call * 1e6, 1),
            "tokens": len(ids)}


def bench_loader(quick: bool) -> dict:
    import numpy as np
    n = (64 if quick else 1024) << 20
    out = {}
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "seg.bin")
        src = np.random.default_rng(0).integers(0, 255, n, dtype=np.uint8)
        src.tofile(path)
        dst = np.zeros(n, dtype=np.uint8)
        for threads in (1, 2, 4, 8):
            core.load_file_to_host(path, dst.ctypes.data, n, threads, 64 << 20)      # warm
            t0 = time.perf_counter()
            res = core.load_file_to_host(path, dst.ctypes.data, n, threads, 64 << 20)
            dt = time.perf_counter() - t0
            out[f"read_gbs_{threads}_threads"] = round(res.bytes / dt / 1e9, 2)
        assert (dst == src).all()
    out["bytes"] = n
    return out


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def bench_rpc(quick: bool) -> dict:
    from blitz_scale_b200.pb.schema import pb
    from blitz_scale_b200.router.runtime import RouterRuntime
    from blitz_scale_b200.router.server import controller_config_from_cluster
    from blitz_scale_b200.router.stub import WorkerStub

    import subprocess
    ports = [_free_port() for _ in range(2)]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    # the workers run as processes of their own, as in a deployment (sharing one event loop with the client would
    # charge the client's turn-taking to the transport)
    procs = [subprocess.Popen([sys.executable, "-m", "blitz_scale_b200.sim.stub_worker", "--rank", str(r), "--world", "2",
                               "--port", str(ports[r]), "--decode-step-ms", "0", "--prefill-tokens-per-s", "1e12"],
                              cwd=root, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) for r in range(2)]

    async def go():
        for p in ports:
            probe = WorkerStub(f"127.0.0.1:{p}")
            for _ in range(200):
                try:
                    await probe.health(timeout=0.5)
                    break
                except Exception:  # noqa: BLE001
                    await asyncio.sleep(0.1)
            await probe.close()
        out = {}
        stub = WorkerStub(f"127.0.0.1:{ports[0]}")
        for _ in range(20):
            await stub.health()
        lat = []
        for _ in range(200 if quick else 2000):
            t0 = time.perf_counter()
            await stub.health()
            lat.append(time.perf_counter() - t0)
        out["health_rtt_us_p50"], out["health_rtt_us_p99"] = round(_pct(lat, .5) * 1e6, 1), round(_pct(lat, .99) * 1e6, 1)
        # a decode-sized exchange: prefill a batch of 64 requests once, then time DecodeV2 round trips
        batch = pb.Batch(id=1, size=64, max_tokens=64 * 128)
        for i in range(64):
            r = batch.requests.add()
            r.id, r.inputs, r.prefill_logprobs, r.top_n_tokens = i, "", False, 0
            r.input_tokens.extend(range(32))
            r.stopping_parameters.max_new_tokens = 100000
            r.stopping_parameters.ignore_eos_token = True
        res = await stub.prefill_v2(batch, pb.PREFILL_CASE_NORMAL)
        cached = res.batch
        lat = []
        for _ in range(100 if quick else 1000):
            t0 = time.perf_counter()
            res = await stub.decode_v2([cached], [pb.Tokens()])
            lat.append(time.perf_counter() - t0)
            cached = res.batch
        out["decode_rpc_batch64_us_p50"] = round(_pct(lat, .5) * 1e6, 1)
        out["decode_rpc_batch64_us_p99"] = round(_pct(lat, .99) * 1e6, 1)
        await stub.clear_cache(1)
        await stub.close()
        # router level: requests through the runtime (queue -> prefill -> migrate -> decode) with stub workers
        cfg = controller_config_from_cluster({"init_states": ["Prefill", "Decode"], "machines": [0, 0]}, 1,
                                             "impl_blitz,impl_nvl", max_blocks_per_replica=200000, autoscale=False)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2)
        lt = asyncio.create_task(rt.run())
        n_req = 100 if quick else 600

        async def one(n_tok, stream):
            lr = rt.submit(list(range(64)), n_tok, stream=stream)
            if not stream:                                  # what POST /generate does: one wake-up per request
                return (await asyncio.wait_for(lr.done, timeout=120)) is None
            while True:                                     # what /generate_stream does: one wake-up per token
                ev = await asyncio.wait_for(lr.queue.get(), timeout=120)
                if ev[0] == "error" or ev[2]:
                    return ev[0] != "error"
        await asyncio.gather(*[one(4, False) for _ in range(8)])
        for label, n_tok, stream in (("short", 8, False), ("long", 64, False), ("long_streamed", 64, True)):
            t0 = time.perf_counter()
            oks = await asyncio.gather(*[one(n_tok, stream) for _ in range(n_req)])
            dt = time.perf_counter() - t0
            assert all(oks)
            out[f"router_{label}_requests_per_s"] = round(n_req / dt, 1)
            out[f"router_{label}_tokens_per_s"] = round(n_req * n_tok / dt, 1)
        await rt.stop()
        lt.cancel()
        return out
    try:
        return asyncio.run(go())
    finally:
        for p in procs:
            p.terminate()
        for p in procs:
            p.wait(timeout=10)


def bench_decode_steps(quick: bool) -> dict:
    """What the router's round trip costs a decode replica, and what several steps per call give back: stub workers
    whose decode step sleeps 5 ms (a stand-in for the GPU time of one step), 64 requests decoding together."""
    import subprocess
    from blitz_scale_b200.router.runtime import RouterRuntime
    from blitz_scale_b200.router.server import controller_config_from_cluster
    from blitz_scale_b200.router.stub import WorkerStub
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ports = [_free_port() for _ in range(2)]
    step_ms = 5.0
    procs = [subprocess.Popen([sys.executable, "-m", "blitz_scale_b200.sim.stub_worker", "--rank", str(r), "--world", "2",
                               "--port", str(ports[r]), "--decode-step-ms", str(step_ms), "--prefill-tokens-per-s", "1e12"],
                              cwd=root, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) for r in range(2)]

    async def go():
        for p in ports:
            probe = WorkerStub(f"127.0.0.1:{p}")
            for _ in range(200):
                try:
                    await probe.health(timeout=0.5)
                    break
                except Exception:  # noqa: BLE001
                    await asyncio.sleep(0.1)
            await probe.close()
        out = {"simulated_step_ms": step_ms, "batch": 64}
        n_tok = 48 if quick else 160
        for k in (1, 2, 4, 8):
            cfg = controller_config_from_cluster({"init_states": ["Prefill", "Decode"], "machines": [0, 0]}, 1,
                                                 "impl_blitz,impl_nvl", max_blocks_per_replica=200000, autoscale=False)
            rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2, decode_steps=k)
            lt = asyncio.create_task(rt.run())
            lrs = [rt.submit(list(range(64)), n_tok, stream=False) for _ in range(64)]
            for lr in lrs:
                assert (await asyncio.wait_for(lr.done, timeout=300)) is None
            # steady state: from the moment all 64 decode together to the last token
            t_a = max(lr.times[1] for lr in lrs)
            t_b = max(lr.times[-1] for lr in lrs)
            toks = sum(sum(1 for t in lr.times if t > t_a) for lr in lrs)
            out[f"ms_per_step_{k}_steps_per_call"] = round((t_b - t_a) * 1e3 / max(1, toks / 64), 3)
            out[f"tokens_per_s_{k}_steps_per_call"] = round(toks / max(1e-9, t_b - t_a), 1)
            await rt.stop()
            lt.cancel()
            await asyncio.sleep(0.2)
        return out
    try:
        return asyncio.run(go())
    finally:
        for p in procs:
            p.terminate()
        for p in procs:
            p.wait(timeout=10)


def bench_http(quick: bool) -> dict:
    """The user-facing path: POST /generate against the router started from its command line (own process), two
    stub workers (own processes, zero simulated compute), a client with many requests in flight."""
    import subprocess

    import aiohttp
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    wports, rport = [_free_port() for _ in range(2)], _free_port()
    with tempfile.TemporaryDirectory() as d:
        json.dump({"init_states": ["Prefill", "Decode"], "machines": [0, 0]}, open(os.path.join(d, "cluster.json"), "w"))
        procs = [subprocess.Popen([sys.executable, "-m", "blitz_scale_b200.sim.stub_worker", "--rank", str(r), "--world", "2",
                                   "--port", str(wports[r]), "--decode-step-ms", "0", "--prefill-tokens-per-s", "1e12"],
                                  cwd=root, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) for r in range(2)]
        procs.append(subprocess.Popen(
            [sys.executable, "-m", "blitz_scale_b200.router.server", "--port", str(rport), "--client-config",
             json.dumps([f"127.0.0.1:{p}" for p in wports]), "--deployment-config-path", os.path.join(d, "cluster.json"),
             "--features", "impl_blitz,impl_nvl,manually_scale", "--model-name", "tiny", "--max-blocks-per-replica", "2000000",
             "--log-level", "WARNING"], cwd=root, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL))

        async def go():
            url = f"http://127.0.0.1:{rport}/generate"
            out = {}
            async with aiohttp.ClientSession(connector=aiohttp.TCPConnector(limit=0)) as sess:
                for _ in range(300):
                    try:
                        async with sess.get(f"http://127.0.0.1:{rport}/health") as r:
                            if r.status == 200:
                                break
                    except Exception:  # noqa: BLE001
                        pass
                    await asyncio.sleep(0.1)

                async def one(n_tok):
                    body = {"input_tokens": list(range(64)), "parameters": {"max_new_tokens": n_tok}}
                    async with sess.post(url, json=body) as r:
                        await r.json()
                        return r.status == 200
                assert all(await asyncio.gather(*[one(4) for _ in range(16)]))
                n_req = 200 if quick else 1500
                for label, n_tok in (("8_tokens", 8), ("64_tokens", 64)):
                    t0 = time.perf_counter()
                    oks = await asyncio.gather(*[one(n_tok) for _ in range(n_req)])
                    dt = time.perf_counter() - t0
                    assert all(oks)
                    out[f"http_generate_{label}_requests_per_s"] = round(n_req / dt, 1)
                    out[f"http_generate_{label}_tokens_per_s"] = round(n_req * n_tok / dt, 1)
            return out
        try:
            return asyncio.run(go())
        finally:
            for p in procs:
                p.terminate()
            for p in procs:
                p.wait(timeout=10)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", default="", help="comma list of: controller,queue,tokenizer,loader,rpc,decode_steps,http")
    a = ap.parse_args()
    parts = {"controller": bench_controller, "queue": bench_queue, "tokenizer": bench_tokenizer, "loader": bench_loader,
             "rpc": bench_rpc, "decode_steps": bench_decode_steps, "http": bench_http}
    want = [p for p in a.only.split(",") if p] or list(parts)
    res = {"bench": "host", "cpus": os.cpu_count()}
    for name in want:
        res[name] = parts[name](a.quick)
        print(name, json.dumps(res[name]), flush=True)
    if a.json:
        os.makedirs(os.path.dirname(os.path.abspath(a.json)), exist_ok=True)
        json.dump(res, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
