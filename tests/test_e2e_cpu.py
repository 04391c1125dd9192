"""CPU plumbing end to end: router (HTTP + native core) + trace client + two GPU-less workers over real gRPC.

A scaled-down version of the first benchmark configuration: Poisson arrivals with uniform input/output lengths,
one serving instance, a second one scaled out during the run.  Checks: every request completes with the
right number of tokens, token streams are identical across two runs with the same seeds, the scale-out is
visible in the transition log, /metrics and the timing headers are present, a worker that dies is detected.
"""
import asyncio
import os
import json
import socket

import pytest

from blitz_scale_b200.pb.schema import RPCS, pb, render_proto
from blitz_scale_b200.router.runtime import RouterRuntime
from blitz_scale_b200.router.server import controller_config_from_cluster, serve_router
from blitz_scale_b200.router.stub import WorkerStub
from blitz_scale_b200.sim import request_sim
from blitz_scale_b200.sim.stub_worker import StubBackend
from blitz_scale_b200.worker.service import serve


def _free_ports(n):
    socks = [socket.socket() for _ in range(n)]
    for s in socks:
        s.bind(("127.0.0.1", 0))
    ports = [s.getsockname()[1] for s in socks]
    for s in socks:
        s.close()
    return ports


def _free_port_run(n):
    """First port of a run of n consecutive free ports."""
    for _ in range(200):
        base = _free_ports(1)[0]
        if base + n >= 65536:
            continue
        socks = []
        try:
            for i in range(n):
                s = socket.socket()
                socks.append(s)
                s.bind(("127.0.0.1", base + i))
            return base
        except OSError:
            continue
        finally:
            for s in socks:
                s.close()
    raise RuntimeError("no run of free ports found")


def test_proto_contract_roundtrip():
    assert len(RPCS) == 25
    for rpc, (req, res) in RPCS.items():
        for name in (req, res):
            cls = getattr(pb, name)
            m = cls()
            # fill required scalar fields so serialisation is legal, then round-trip
            for f in cls.DESCRIPTOR.fields:
                if f.label == f.LABEL_REQUIRED and f.message_type is None:
                    setattr(m, f.name, {f.TYPE_STRING: "x", f.TYPE_BOOL: True}.get(f.type, 1))
            data = m.SerializeToString(deterministic=True) if m.IsInitialized() else None
            if data is not None:
                assert cls.FromString(data) == m
    r = pb.PrefillV2Request(forward_case=pb.PREFILL_CASE_NAIVE_PP | pb.PREFILL_CASE_IMMIGRATE)
    assert r.forward_case == 12
    text = render_proto()
    assert "service TextGenerationService" in text and "rpc TanzBroadcast(BroadcastRequest)" in text
    assert "oneof start_layer" in text and "repeated uint32 input_tokens = 8;" in text


async def _cluster(n_workers, states, features, seed=0, **kw):
    ports = _free_ports(n_workers + 1)
    stop = asyncio.Event()
    backends = [StubBackend(r, n_workers, seed=seed, ready=(states[r] != "Inactive"), load_s=0.15) for r in range(n_workers)]
    tasks = []
    for r, b in enumerate(backends):
        ready = asyncio.Event()
        tasks.append(asyncio.create_task(serve(b, "127.0.0.1", ports[r], stop_event=stop, ready_event=ready)))
        await ready.wait()
    cfg = controller_config_from_cluster({"init_states": states, "machines": [0] * n_workers}, 1, features,
                                         max_blocks_per_replica=4000, **kw)
    rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports[:n_workers]], model_layers=2)
    tasks.append(asyncio.create_task(serve_router(rt, "127.0.0.1", ports[-1], stop=stop)))
    await asyncio.sleep(0.2)
    return rt, backends, ports[-1], stop, tasks


async def _shutdown(stop, tasks):
    stop.set()
    await asyncio.wait(tasks, timeout=5)


async def _run_config1(seed):
    rt, backends, port, stop, tasks = await _cluster(2, ["Normal", "Inactive"], "impl_blitz,impl_nvl,manually_scale", seed)
    trace = request_sim.make_mock_trace(rate=40.0, duration=3.0, seed=0, input_rng=(32, 512), output_rng=(16, 64),
                                        max_requests=80)

    async def scale_later():
        await asyncio.sleep(1.0)
        import aiohttp
        async with aiohttp.ClientSession() as s:
            async with s.post(f"http://127.0.0.1:{port}/modify_cluster_state", json={"replica": 1, "state": "Prefill"}) as r:
                assert r.status == 200
    sc = asyncio.create_task(scale_later())
    recs = await request_sim.replay(f"http://127.0.0.1:{port}/generate", trace, record_tokens=True)
    await sc
    import aiohttp
    async with aiohttp.ClientSession() as s:
        async with s.get(f"http://127.0.0.1:{port}/metrics") as r:
            metrics = await r.text()
        async with s.get(f"http://127.0.0.1:{port}/info") as r:
            info = await r.json()
        async with s.get(f"http://127.0.0.1:{port}/health") as r:
            assert r.status == 200
    transitions = [l for _, l in rt.transitions]
    used = rt.ctl.total_used_blocks()
    pages = [b.pool.used_pages for b in backends]
    await _shutdown(stop, tasks)
    return trace, recs, metrics, info, transitions, used, pages, backends


def test_config1_cpu_plumbing_scale_out_and_determinism():
    trace, recs, metrics, info, transitions, used, pages, backends = asyncio.run(_run_config1(seed=0))
    assert len(recs) == len(trace) and all(r["status"] == "ok" for r in recs), [r for r in recs if r["status"] != "ok"][:3]
    for r, item in zip(recs, trace):
        assert r["generated_tokens"] == item.output_len and len(r["tokens"]) == item.output_len
        assert r["first_token_time"] >= 0 and r["total_time"] >= r["first_token_time"]
    assert any("Replica<1> Inactive => LoadingPrefill" in l for l in transitions)
    assert any("Replica<1> LoadingPrefill => Prefill" in l for l in transitions)
    assert backends[1].counters["prefill"] > 0, "the scaled-out instance must serve requests"
    assert "blitz_request_count 80" in metrics and "blitz_request_duration_count 80" in metrics
    # histograms are cumulative and end at the count; sizes have buckets of their own
    assert 'blitz_request_duration_bucket{le="+Inf"} 80' in metrics and 'blitz_request_input_length_bucket{le="16384"} 80' in metrics
    cum = [int(l.rsplit(" ", 1)[1]) for l in metrics.splitlines() if l.startswith("blitz_request_generated_tokens_bucket")]
    assert cum == sorted(cum) and cum[-1] == 80 and cum[0] < 80
    # every metric name of the reference's list is exported (router_v2/src/server.rs:1084-1207)
    for name in ("blitz_queue_size", "blitz_relay_queue_size", "blitz_migration_queue_size", "blitz_used_blocks",
                 "blitz_scale_up_times", "blitz_nvbroadcast_times", "blitz_waiting_full_batches",
                 "blitz_waiting_partial_batches", "blitz_shutting_replica", "blitz_prefill_replica", "blitz_decode_replica",
                 "blitz_request_success", "blitz_request_validation_duration", "blitz_batch_next_size"):
        assert f"\n{name}" in "\n" + metrics, name
    assert "blitz_scale_up_times 1" in metrics and "blitz_nvbroadcast_times 1" in metrics and "blitz_used_blocks 0" in metrics
    assert info["replicas"] == ["Prefill", "Prefill"]
    # the reference's fields; dtype and device come from the workers' Info RPC
    assert info["model_dtype"] == "float32" and info["model_device_type"] == "cpu" and info["max_stop_sequences"] == 4
    assert info["max_batch_prefill_tokens"] > 0 and info["max_concurrent_requests"] > 0 and info["max_best_of"] >= 1
    assert used == 0 and pages == [0, 0]
    s = request_sim.summarize(recs)
    assert s["ok"] == 80 and s["output_tokens"] == sum(i.output_len for i in trace)
    # same seeds -> identical token streams (tokens depend on request id and position only)
    _, recs2, *_ = asyncio.run(_run_config1(seed=0))
    assert [r["tokens"] for r in recs] == [r["tokens"] for r in recs2]
    _, recs3, *_ = asyncio.run(_run_config1(seed=1))
    assert [r["tokens"] for r in recs] != [r["tokens"] for r in recs3]


def test_pd_disaggregation_with_autoscaling_over_grpc():
    async def go():
        rt, backends, port, stop, tasks = await _cluster(
            4, ["Prefill", "Decode", "Inactive", "Inactive"], "impl_blitz,impl_fast_pro,impl_live_pro",
            tokens_prefilled_per_sec=3000, max_prefill=3, max_decode=2)
        for b in backends:
            b.prefill_rate = 20000.0
        trace = request_sim.make_mock_trace(rate=6.0, duration=4.0, seed=2, input_rng=(256, 1024), output_rng=(8, 24),
                                            rate_step=(1.0, 50.0), max_requests=120)
        recs = await request_sim.replay(f"http://127.0.0.1:{port}/generate", trace)
        transitions = [l for _, l in rt.transitions]
        counters = [dict(b.counters) for b in backends]
        await _shutdown(stop, tasks)
        return trace, recs, transitions, counters
    trace, recs, transitions, counters = asyncio.run(go())
    assert all(r["status"] == "ok" for r in recs), [r for r in recs if r["status"] != "ok"][:3]
    assert sum(r["generated_tokens"] for r in recs) == sum(i.output_len for i in trace)
    assert counters[0]["migrate"] > 0 and counters[1]["immigrate"] > 0        # KV moved prefill -> decode
    assert any("Inactive => NewPrefill" in l or "Inactive => LoadingPrefill" in l for l in transitions)


def test_worker_failure_is_detected_not_hung():
    async def go():
        rt, backends, port, stop, tasks = await _cluster(2, ["Prefill", "Decode"], "impl_blitz,impl_nvl", autoscale=False)

        def boom(*a, **k):
            raise RuntimeError("injected worker fault")
        backends[1].decode = boom       # the decode worker fails every step (host-side fault injection)
        trace = request_sim.make_mock_trace(rate=20.0, duration=0.5, seed=3, input_rng=(16, 64), output_rng=(4, 8), max_requests=6)
        recs = await asyncio.wait_for(request_sim.replay(f"http://127.0.0.1:{port}/generate", trace), timeout=30)
        state = rt.ctl.state_name(1)
        await _shutdown(stop, tasks)
        return recs, state
    recs, state = asyncio.run(go())
    assert state == "Inactive"
    assert any(r["status"] != "ok" for r in recs)      # surfaced as an error, not a hang


def test_direct_rpcs_against_stub_worker():
    async def go():
        port = _free_ports(1)[0]
        stop, ready = asyncio.Event(), asyncio.Event()
        b = StubBackend(0, 1, ready=False)
        t = asyncio.create_task(serve(b, "127.0.0.1", port, stop_event=stop, ready_event=ready))
        await ready.wait()
        s = WorkerStub(f"127.0.0.1:{port}")
        assert (await s.health()).state == "loading"
        await s.set_status_ready()
        assert (await s.health()).state == "ready"
        assert (await s.info()).dtype == "float32"
        batch = pb.Batch(id=5, size=2, max_tokens=128)
        for i, n in enumerate((7, 20)):
            r = batch.requests.add()
            r.id, r.inputs, r.prefill_logprobs, r.top_n_tokens = i, "", False, 0
            r.input_tokens.extend(range(n))
            r.stopping_parameters.max_new_tokens = 3 if i == 0 else 2
            r.stopping_parameters.ignore_eos_token = True
        res = await s.prefill_v2(batch)
        assert len(res.generations) == 2 and res.batch.request_ids == [0, 1] and res.total_ns > 0
        d1 = await s.decode_v2([res.batch], [pb.Tokens()])
        assert [g.request_id for g in d1.generations] == [0, 1]
        assert d1.generations[1].HasField("generated_text") and d1.batch.request_ids == [0]
        f = await s.filter_batch(5, [0])
        assert f.batch.request_ids == [0]
        d2 = await s.decode_v2([d1.batch], [pb.Tokens()])
        assert d2.generations[0].generated_text.generated_tokens == 3 and not d2.HasField("batch")
        assert b.pool.used_pages == 0
        with pytest.raises(Exception):
            await s.call("Prefill", pb.PrefillRequest(batch=batch))     # v1 RPCs are rejected
        await s.reset_status()
        with pytest.raises(Exception):
            await s.prefill_v2(batch)                                    # parameters not loaded
        await s.close()
        stop.set()
        await asyncio.wait([t], timeout=5)
    asyncio.run(go())


def test_experiment_runner_expansion_and_dry_run(tmp_path):
    import subprocess
    import sys
    import tomllib
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench"))
    import experiment
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tpl = tomllib.load(open(os.path.join(root, "bench/templates/llama3_8b_pd.toml"), "rb"))
    inst = experiment.expand(tpl)
    assert len(inst) == 3 * 2     # three feature sets x two scale-down thresholds
    assert {i["router"]["scale_down_threshold_millis"] for i in inst} == {333, 1500}
    cj = experiment.cluster_json(inst[0])
    assert cj["init_states"] == ["Prefill", "Decode", "Inactive", "Inactive"] and cj["replicas"] == [[0], [1], [2], [3]]
    res = subprocess.run([sys.executable, os.path.join(root, "bench/experiment.py"), "--template",
                          os.path.join(root, "bench/templates/cpu_plumbing.toml"), "--out", str(tmp_path), "--dry-run"],
                         capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stderr[-2000:]
    d = next(p for p in tmp_path.iterdir() if p.is_dir())
    cmds = json.load(open(d / "commands.json"))
    assert len(cmds["workers"]) == 3 and "request_sim" in cmds["client"] and "--features" in cmds["router"]
    assert json.load(open(d / "config-server.json"))["init_states"] == ["Prefill", "Decode", "Inactive"]
    # waiting for the GPUs of a finished instance: a fake device query that frees up on the third poll
    polls = []

    def fake(i):
        polls.append(i)
        return 1 if len(polls) <= 4 and i == 1 else 0
    assert experiment.wait_gpus_released(2, timeout=10.0, query=fake) and len(polls) >= 6
    assert not experiment.wait_gpus_released(1, timeout=0.2, query=lambda i: 3)
    experiment.record_provenance(tmp_path / "prov")
    assert (tmp_path / "prov" / "git-info.txt").read_text()


def test_log_analysis_and_sizing():
    from blitz_scale_b200.utils import analysis
    log = ["[0.000000] Replica<0> boot => Prefill", "[1.5] Replica<2> Inactive => LoadingPrefill",
           "[1.9] Replica<2> LoadingPrefill => Prefill", "[2.0] Control signal: P+1 D+0 | x",
           "[3.0] System Metrics: prefill_tokens: 100, decode_tokens: 7", "[4.0] Replica<2> >>= unload", "Client start",
           "[4.5] Replica[2]: Flow in: 16061MB, Flow out: 0MB"]
    p = analysis.parse_router_log(log)
    assert p["transitions"][1] == (1.5, 2, "Inactive", "LoadingPrefill") and p["signals"] == [(2.0, 1, 0)]
    assert p["metrics"] == [(3.0, 100, 7)] and p["unloads"] == [4.0] and p["flows"] == [(4.5, 2, 16061, 0)]
    assert analysis.scale_out_latencies(p["transitions"]) == [(2, pytest.approx(0.4))]
    tl = analysis.replica_timeline(p["transitions"], 5.0)
    assert tl[2] == [(1.5, 1.9, "LoadingPrefill"), (1.9, 5.0, "Prefill")]
    recs = [{"status": "ok", "first_token_time": 100.0, "max_time_between_tokens": 20.0, "input_length": 100},
            {"status": "ok", "first_token_time": 900.0, "max_time_between_tokens": 150.0, "input_length": 1000}]
    s = analysis.slo_table(recs)
    assert s["ttft_violation_rate"] == 0.5 and s["tbt_violation_rate"] == 0.5
    z = analysis.kv_sizing("llama3_8b", tp=1, page_size=64)
    assert z["kv_bytes_per_token"] == 2 * 8 * 128 * 2 * 32 and z["block_bytes"] == z["kv_bytes_per_token"] * 64


def test_experiment_runs_processes_end_to_end(tmp_path):
    """The deployment path as separate processes: two stub workers, the router CLI, the trace client CLI."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tpl = open(os.path.join(root, "bench/templates/cpu_plumbing.toml")).read()
    p0, p2 = _free_port_run(3), _free_ports(1)[0]            # the workers listen on p0, p0 + 1, p0 + 2
    tpl = tpl.replace("worker_port = 50151", f"worker_port = {p0}").replace("port = 3100", f"port = {p2}")
    tpl = tpl.replace("duration = 50", "duration = 4").replace("num_requests = 200", "num_requests = 16")
    (tmp_path / "t.toml").write_text(tpl)
    run = subprocess.Popen([sys.executable, os.path.join(root, "bench/experiment.py"), "--template", str(tmp_path / "t.toml"),
                            "--out", str(tmp_path / "out"), "--force"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        out, _ = run.communicate(timeout=240)
    except subprocess.TimeoutExpired:
        run.terminate()                                     # SIGTERM: the runner stops the processes it started
        out, _ = run.communicate(timeout=60)
        raise AssertionError("experiment runner timed out:\n" + out[-3000:])
    assert run.returncode == 0, out[-4000:]
    d = next(p for p in (tmp_path / "out").iterdir() if p.is_dir())
    recs = [json.loads(l) for l in open(d / "client.jsonl")]
    assert len(recs) >= 8 and all(r.get("status") == "ok" for r in recs), recs[:2]
    summary = json.load(open(d / "summary.json"))
    assert "slo" in summary
    assert "attached to a different loop" not in open(d / "router.log").read()
    prov = tmp_path / "out" / "provenance"
    assert (prov / "git-info.txt").exists()


def test_heartbeat_failure_detector_marks_idle_replica_lost():
    """A worker that stops answering Health is declared lost although no operation was in flight on it; traffic
    then goes to the surviving prefill replica only (host-side failure: the worker's server is shut down)."""
    async def go():
        ports = _free_ports(3)
        stops, tasks = [], []
        states = ["Prefill", "Decode", "Prefill"]
        backends = [StubBackend(r, 3, ready=True) for r in range(3)]
        for r, b in enumerate(backends):
            ready, stop = asyncio.Event(), asyncio.Event()
            tasks.append(asyncio.create_task(serve(b, "127.0.0.1", ports[r], stop_event=stop, ready_event=ready)))
            await ready.wait()
            stops.append(stop)
        cfg = controller_config_from_cluster({"init_states": states, "machines": [0] * 3}, 1, "impl_blitz,impl_nvl,manually_scale",
                                             max_blocks_per_replica=4000)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2, health_interval_s=0.1, health_misses=2)
        lt = asyncio.create_task(rt.run())
        await asyncio.sleep(0.35)
        assert rt.ctl.state_name(2) == "Prefill"          # healthy so far
        stops[2].set()                                     # the third worker goes away while idle
        for _ in range(60):
            await asyncio.sleep(0.1)
            if rt.ctl.state_name(2) == "Inactive":
                break
        assert rt.ctl.state_name(2) == "Inactive" and dict(rt.ctl.counters()).get("blitz_replica_lost") == 1
        # the cluster keeps serving on the remaining replicas
        lr = rt.submit(list(range(40)), 4)
        toks = []
        while True:
            ev = await asyncio.wait_for(lr.queue.get(), timeout=10)
            assert ev[0] != "error"
            toks.append(ev[1])
            if ev[2]:
                break
        assert len(toks) == 4 and rt.ctl.state_name(0) == "Prefill" and rt.ctl.state_name(1) == "Decode"
        await rt.stop()
        lt.cancel()
        for s in stops:
            s.set()
        await asyncio.wait(tasks, timeout=5)
    asyncio.run(go())


def test_migration_to_dead_decode_replica_blames_the_destination():
    """The only decode worker's server is shut down (host-side failure).  The next request's KV migration fails on
    the destination's RPC: that replica is declared lost, the prefill replica stays in service, takes over both
    phases, and later requests complete."""
    async def go():
        ports = _free_ports(2)
        stops, tasks = [], []
        states = ["Prefill", "Decode"]
        backends = [StubBackend(r, 2, ready=True) for r in range(2)]
        for r, b in enumerate(backends):
            ready, stop = asyncio.Event(), asyncio.Event()
            tasks.append(asyncio.create_task(serve(b, "127.0.0.1", ports[r], stop_event=stop, ready_event=ready)))
            await ready.wait()
            stops.append(stop)
        cfg = controller_config_from_cluster({"init_states": states, "machines": [0] * 2}, 1, "impl_blitz,impl_nvl",
                                             max_blocks_per_replica=4000)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2)
        lt = asyncio.create_task(rt.run())

        async def run_one(n_new):
            lr = rt.submit(list(range(40)), n_new)
            evs = []
            while True:
                ev = await asyncio.wait_for(lr.queue.get(), timeout=20)
                evs.append(ev)
                if ev[0] == "error" or ev[2]:
                    return evs
        assert len(await run_one(4)) == 4                       # healthy pair: prefill on 0, decode on 1
        stops[1].set()
        await asyncio.wait([tasks[1]], timeout=5)
        evs = await run_one(4)                                  # prefill answers, then the migration finds nobody
        assert evs[0][0] == "token" and evs[-1][0] == "error"
        assert rt.ctl.state_name(1) == "Inactive" and rt.ctl.state_name(0) == "Prefill"
        evs = await run_one(5)                                  # the survivor now serves both phases
        assert [e[0] for e in evs] == ["token"] * 5 and evs[-1][2]
        assert rt.ctl.total_used_blocks() == 0
        await rt.stop()
        lt.cancel()
        stops[0].set()
        await asyncio.wait(tasks, timeout=5)
    asyncio.run(go())


def test_progressive_migration_to_dead_decode_replica_serves_the_prompt_again():
    """As above with `migrate_progressive`: the decode replica is already part of the prefill call, so its loss is
    noticed while the prompt has produced nothing; the prompt is queued again and the prefill replica, now alone,
    serves it completely (no token is lost, nothing fails)."""
    async def go():
        ports = _free_ports(2)
        stops, tasks = [], []
        backends = [StubBackend(r, 2, ready=True) for r in range(2)]
        for r, b in enumerate(backends):
            ready, stop = asyncio.Event(), asyncio.Event()
            tasks.append(asyncio.create_task(serve(b, "127.0.0.1", ports[r], stop_event=stop, ready_event=ready)))
            await ready.wait()
            stops.append(stop)
        cfg = controller_config_from_cluster({"init_states": ["Prefill", "Decode"], "machines": [0] * 2}, 1,
                                             "impl_blitz,impl_nvl,migrate_progressive", max_blocks_per_replica=4000)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2)
        lt = asyncio.create_task(rt.run())

        async def run_one(n_new):
            lr = rt.submit(list(range(40)), n_new)
            evs = []
            while True:
                ev = await asyncio.wait_for(lr.queue.get(), timeout=20)
                evs.append(ev)
                if ev[0] == "error" or ev[2]:
                    return evs
        assert len(await run_one(4)) == 4
        assert backends[0].counters["migrate_progressive"] == 1 and backends[0].counters["migrate"] == 0
        stops[1].set()
        await asyncio.wait([tasks[1]], timeout=5)
        evs = await run_one(4)
        assert [e[0] for e in evs] == ["token"] * 4 and evs[-1][2]
        assert rt.ctl.state_name(1) == "Inactive" and rt.ctl.state_name(0) == "Prefill"
        for _ in range(100):
            if rt.ctl.idle() and not backends[0].batches:
                break
            await asyncio.sleep(0.02)
        assert rt.ctl.total_used_blocks() == 0 and backends[0].pool.used_pages == 0
        await rt.stop()
        lt.cancel()
        stops[0].set()
        await asyncio.wait(tasks, timeout=5)
    asyncio.run(go())


def test_dropped_immigrate_reply_fails_the_operation_not_the_router():
    """A decode worker accepts the Immigrate call and never answers (host-side fault: its handler blocks).  The RPC
    deadline turns that into a failed operation: the silent replica is declared lost, its batch fails, and the next
    request migrates to the other decode replica."""
    import threading
    release = threading.Event()

    async def go():
        ports = _free_ports(3)
        stop, tasks = asyncio.Event(), []
        states = ["Prefill", "Decode", "Decode"]
        backends = [StubBackend(r, 3, ready=True) for r in range(3)]
        backends[1].immigrate = lambda *a, **k: release.wait(30)          # reply withheld
        for r, b in enumerate(backends):
            ready = asyncio.Event()
            tasks.append(asyncio.create_task(serve(b, "127.0.0.1", ports[r], stop_event=stop, ready_event=ready)))
            await ready.wait()
        cfg = controller_config_from_cluster({"init_states": states, "machines": [0] * 3}, 1, "impl_blitz,impl_nvl",
                                             max_blocks_per_replica=4000, autoscale=False)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2, rpc_timeout_s=1.0)
        lt = asyncio.create_task(rt.run())

        async def run_one(n_new):
            lr = rt.submit(list(range(40)), n_new)
            evs = []
            while True:
                ev = await asyncio.wait_for(lr.queue.get(), timeout=20)
                evs.append(ev)
                if ev[0] == "error" or ev[2]:
                    return evs
        evs = await run_one(4)
        assert evs[0][0] == "token" and evs[-1][0] == "error"
        assert rt.ctl.state_name(1) == "Inactive" and rt.ctl.state_name(0) == "Prefill"
        evs = await run_one(4)
        assert [e[0] for e in evs] == ["token"] * 4 and rt.ctl.state_name(2) == "Decode"
        assert rt.ctl.total_used_blocks() == 0 and rt.ctl.inflight_ops() == 0
        release.set()
        await rt.stop()
        lt.cancel()
        stop.set()
        await asyncio.wait(tasks, timeout=5)
    try:
        asyncio.run(go())
    finally:
        release.set()


def test_nothing_is_left_behind_after_many_requests():
    """Soak: after a few hundred requests of mixed lengths (some finish with their first token) every map of the
    router runtime and of the core is empty again and the workers hold no batch and no page."""
    async def go():
        rt, backends, port, stop, tasks = await _cluster(3, ["Prefill", "Decode", "Decode"], "impl_blitz,impl_nvl", autoscale=False)
        for b in backends:
            b.decode_step_s, b.prefill_rate = 0.0, 1e12

        async def one(i):
            lr = rt.submit(list(range(8 + i % 50)), 1 + (i * 7) % 12, stream=bool(i % 2))
            assert (await asyncio.wait_for(lr.done, timeout=60)) is None
            assert len(lr.tokens) == 1 + (i * 7) % 12 and lr.entry is not None
            if lr.stream:
                assert lr.queue.qsize() == len(lr.tokens)
        for wave in range(3):
            await asyncio.gather(*[one(wave * 100 + i) for i in range(100)])
        for _ in range(100):                                   # trailing ClearCache actions
            if rt.ctl.idle() and not rt.cached and all(not b.batches for b in backends):
                break
            await asyncio.sleep(0.05)
        state = (len(rt.requests), len(rt.cached), len(rt.first_tokens), len(rt.ctl.finished()), rt.ctl.inflight_ops(),
                 rt.ctl.total_used_blocks(), rt.ctl.idle(), [len(b.batches) for b in backends],
                 [b.pool.used_pages for b in backends])
        await _shutdown(stop, tasks)
        return state
    assert asyncio.run(go()) == (0, 0, 0, 0, 0, 0, True, [0, 0, 0], [0, 0, 0])


def test_progressive_migration_over_grpc_gives_the_same_tokens_and_leaves_nothing_behind():
    """`migrate_progressive`: the prefill call and the decode replica's immigrate run side by side, the batch decodes on
    the decode replica without a Migrate round, requests that end at their first token are filtered out there, and the
    tokens are the ones the ordinary path gives."""
    async def go(features):
        rt, backends, port, stop, tasks = await _cluster(3, ["Prefill", "Decode", "Decode"], features, autoscale=False)
        for b in backends:
            b.decode_step_s, b.prefill_rate = 0.0, 1e12

        async def one(i):
            lr = rt.submit(list(range(8 + i % 50)), 1 + (i * 7) % 12)
            assert (await asyncio.wait_for(lr.done, timeout=60)) is None
            return list(lr.tokens)
        toks = []
        for wave in range(2):
            toks += await asyncio.gather(*[one(wave * 60 + i) for i in range(60)])
        for _ in range(100):
            if rt.ctl.idle() and not rt.cached and all(not b.batches for b in backends):
                break
            await asyncio.sleep(0.05)
        state = (len(rt.requests), len(rt.cached), len(rt.first_tokens), rt.ctl.inflight_ops(), rt.ctl.total_used_blocks(),
                 [len(b.batches) for b in backends], [b.pool.used_pages for b in backends])
        counters = dict(rt.ctl.counters()), [dict(b.counters) for b in backends]
        await _shutdown(stop, tasks)
        return toks, state, counters
    plain, state0, _ = asyncio.run(go("impl_blitz,impl_nvl"))
    prog, state1, (ctl_counters, worker_counters) = asyncio.run(go("impl_blitz,impl_nvl,migrate_progressive"))
    assert prog == plain
    assert state0 == state1 == (0, 0, 0, 0, 0, [0, 0, 0], [0, 0, 0])
    assert ctl_counters["blitz_progressive_kv_cache_times"] > 0
    assert worker_counters[0]["migrate_progressive"] == ctl_counters["blitz_progressive_kv_cache_times"]
    assert worker_counters[0]["migrate"] == ctl_counters["blitz_kv_cache_times"] - ctl_counters["blitz_progressive_kv_cache_times"]
    assert ctl_counters.get("blitz_filtered_batches", 0) > 0      # some requests ask for one token only


def test_several_decode_steps_per_call_give_the_same_tokens():
    """With k decode steps per DecodeV2 call the token streams are those of one step per call; tokens arrive up to k
    at a time, requests still stop at their own length, and nothing is left behind."""
    async def run(k):
        ports = _free_ports(2)
        stop, tasks = asyncio.Event(), []
        backends = [StubBackend(r, 2, ready=True, seed=5) for r in range(2)]
        for r, b in enumerate(backends):
            ready = asyncio.Event()
            tasks.append(asyncio.create_task(serve(b, "127.0.0.1", ports[r], stop_event=stop, ready_event=ready)))
            await ready.wait()
        cfg = controller_config_from_cluster({"init_states": ["Prefill", "Decode"], "machines": [0, 0]}, 1, "impl_blitz,impl_nvl",
                                             max_blocks_per_replica=4000, autoscale=False)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2, decode_steps=k)
        lt = asyncio.create_task(rt.run())
        lrs = [rt.submit(list(range(10 + i)), 3 + 2 * i, stream=False) for i in range(6)]     # lengths 3, 5, ..., 13
        for lr in lrs:
            assert (await asyncio.wait_for(lr.done, 30)) is None
        for _ in range(100):
            if rt.ctl.idle() and not rt.cached and all(not b.batches for b in backends):
                break
            await asyncio.sleep(0.05)
        left = (len(rt.cached), rt.ctl.total_used_blocks(), [len(b.batches) for b in backends], [b.pool.used_pages for b in backends])
        await rt.stop()
        lt.cancel()
        stop.set()
        await asyncio.wait(tasks, timeout=5)
        return [list(lr.tokens) for lr in lrs], [list(lr.times) for lr in lrs], left
    one, _, left1 = asyncio.run(run(1))
    four, times4, left4 = asyncio.run(run(4))
    assert [len(t) for t in one] == [3, 5, 7, 9, 11, 13] and four == one
    assert left1 == left4 == (0, 0, [0, 0], [0, 0])
    bursts = max(sum(1 for a, b in zip(ts, ts[1:]) if a == b) for ts in times4)
    assert bursts >= 6                                   # the longest request got most of its tokens in groups


def test_restarted_stub_worker_is_readmitted():
    """A worker goes away, is declared lost by the heartbeat detector, comes back on the same port (a restart) and is
    scaled in again: the router's channel reconnects and the replica serves."""
    async def go():
        ports = _free_ports(3)
        stops, tasks = [], []
        states = ["Prefill", "Decode", "Prefill"]

        async def start(r, ready_flag):
            ready, stop = asyncio.Event(), asyncio.Event()
            t = asyncio.create_task(serve(StubBackend(r, 3, ready=ready_flag, load_s=0.05), "127.0.0.1", ports[r],
                                          stop_event=stop, ready_event=ready))
            await ready.wait()
            return stop, t
        for r in range(3):
            s, t = await start(r, True)
            stops.append(s)
            tasks.append(t)
        cfg = controller_config_from_cluster({"init_states": states, "machines": [0] * 3}, 1, "impl_blitz,impl_nvl,manually_scale",
                                             max_blocks_per_replica=4000)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2, health_interval_s=0.1, health_misses=2)
        lt = asyncio.create_task(rt.run())
        stops[2].set()
        await asyncio.wait([tasks[2]], timeout=5)
        for _ in range(80):
            await asyncio.sleep(0.1)
            if rt.ctl.state_name(2) == "Inactive":
                break
        assert rt.ctl.state_name(2) == "Inactive" and not rt.ctl.reachable(2)
        stops[2], tasks[2] = await start(2, False)               # the restarted worker: same port, no parameters yet
        for _ in range(100):                                     # the detector keeps pinging; the channel reconnects (<= 1 s)
            if rt.ctl.reachable(2):
                break
            await asyncio.sleep(0.1)
        assert rt.ctl.reachable(2)
        assert rt.ctl.manual_scale(2, "Prefill", rt.now())
        rt.wake.set()
        for _ in range(80):
            await asyncio.sleep(0.1)
            if rt.ctl.state_name(2) == "Prefill":
                break
        assert rt.ctl.state_name(2) == "Prefill"
        served = set()
        for i in range(8):                                       # both prefill replicas take work again
            lr = rt.submit(list(range(30)), 2, stream=False)
            assert (await asyncio.wait_for(lr.done, 20)) is None
        served = {l.split(">")[0][-1] for _, l in rt.transitions}
        await rt.stop()
        lt.cancel()
        for s in stops:
            s.set()
        await asyncio.wait(tasks, timeout=5)
        return served
    assert "2" in asyncio.run(go())


@pytest.mark.parametrize("features", ["impl_blitz,impl_nvl", "impl_blitz,impl_nvl,migrate_progressive"])
def test_chaos_workers_fail_and_return_while_requests_flow(features):
    """Workers are stopped and restarted at random while requests flow (host-side failures only).  Every request
    either completes with exactly its tokens or fails with an error, nothing hangs, and once things are quiet the
    runtime, the core and the surviving workers hold nothing."""
    import random
    features = os.environ.get("BLITZ_CHAOS_FEATURES", features)
    rng = random.Random(int(os.environ.get("BLITZ_CHAOS_SEED", "7")))

    async def go():
        n = 4
        ports = _free_ports(n)
        states = ["Prefill", "Decode", "Prefill", "Decode"]
        backends, stops, tasks = [None] * n, [None] * n, [None] * n

        async def start(r, ready_flag):
            ready, stop = asyncio.Event(), asyncio.Event()
            backends[r] = StubBackend(r, n, ready=ready_flag, load_s=0.02, decode_step_s=0.001)
            tasks[r] = asyncio.create_task(serve(backends[r], "127.0.0.1", ports[r], stop_event=stop, ready_event=ready))
            stops[r] = stop
            await ready.wait()
        for r in range(n):
            await start(r, True)
        cfg = controller_config_from_cluster({"init_states": states, "machines": [0] * n}, 1,
                                             features,
                                             max_blocks_per_replica=4000, tokens_prefilled_per_sec=2000, min_prefill=1,
                                             min_decode=1, max_prefill=3, max_decode=3)
        cfg.quarantine_ms = 200.0
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2, health_interval_s=0.05, health_misses=2,
                           rpc_timeout_s=2.0)
        lt = asyncio.create_task(rt.run())
        results = []

        async def client(i):
            await asyncio.sleep(rng.random() * 3.0)
            want = 1 + i % 9
            lr = rt.submit(list(range(5 + i % 40)), want, stream=False)
            err = await asyncio.wait_for(lr.done, timeout=60)
            results.append((err, len(lr.tokens), want))

        async def chaos():
            down = None
            for _ in range(6):
                await asyncio.sleep(0.4)
                if down is None:
                    down = rng.choice([1, 2, 3])
                    stops[down].set()
                    await asyncio.wait([tasks[down]], timeout=5)
                else:
                    await start(down, False)
                    down = None
            if down is not None:
                await start(down, False)
        await asyncio.gather(chaos(), *[client(i) for i in range(120)])
        for _ in range(200):
            if rt.ctl.idle() and not rt.requests:
                break
            await asyncio.sleep(0.05)
        await asyncio.sleep(0.3)
        alive = [r for r in range(n) if rt.ctl.state_name(r) != "Inactive"]
        left = {"requests": len(rt.requests), "cached": len(rt.cached), "first_tokens": len(rt.first_tokens),
                "finished": len(rt.ctl.finished()), "ops": rt.ctl.inflight_ops(), "blocks": rt.ctl.total_used_blocks(),
                "idle": rt.ctl.idle(), "worker_batches": [len(backends[r].batches) for r in alive],
                "worker_pages": [backends[r].pool.used_pages for r in alive]}
        await rt.stop()
        lt.cancel()
        for s in stops:
            s.set()
        await asyncio.wait([t for t in tasks if t is not None], timeout=5)
        return results, left, alive
    results, left, alive = asyncio.run(go())
    assert len(results) == 120
    done = [r for r in results if r[0] is None]
    assert all(got == want for _, got, want in done) and len(done) >= 60
    assert all(err == "replica lost" for err, _, _ in results if err is not None)
    assert left == {"requests": 0, "cached": 0, "first_tokens": 0, "finished": 0, "ops": 0, "blocks": 0, "idle": True,
                    "worker_batches": [0] * len(alive), "worker_pages": [0] * len(alive)}, left


def test_new_replica_dies_while_serving_during_its_load():
    """Live scaling: the new prefill replica serves while its parameters stream in, then its worker goes away in the
    middle.  Prompts it held go back to the queue and finish elsewhere, relayed batches fail cleanly, the helper
    replica returns to ordinary prefill, nothing hangs."""
    async def go():
        n = 3
        ports = _free_ports(n)
        states = ["Prefill", "Decode", "Inactive"]
        backends, stops, tasks = [], [], []
        for r in range(n):
            ready, stop = asyncio.Event(), asyncio.Event()
            b = StubBackend(r, n, ready=states[r] != "Inactive", load_s=1.5, decode_step_s=0.001, prefill_tokens_per_s=20000)
            backends.append(b)
            tasks.append(asyncio.create_task(serve(b, "127.0.0.1", ports[r], stop_event=stop, ready_event=ready)))
            stops.append(stop)
            await ready.wait()
        cfg = controller_config_from_cluster({"init_states": states, "machines": [0] * n}, 1,
                                             "impl_blitz,impl_nvl,impl_live,manually_scale", max_blocks_per_replica=4000)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2, rpc_timeout_s=3.0)
        lt = asyncio.create_task(rt.run())
        results = []

        async def client(i):
            await asyncio.sleep(0.02 * i)
            lr = rt.submit(list(range(200 + i)), 3, stream=False)
            err = await asyncio.wait_for(lr.done, timeout=60)
            results.append((err, len(lr.tokens)))
        cl = [asyncio.create_task(client(i)) for i in range(60)]
        await asyncio.sleep(0.1)
        assert rt.ctl.manual_scale(2, "Prefill", rt.now())
        rt.wake.set()
        await asyncio.sleep(0.4)
        seen_new = rt.ctl.state_name(2)
        stops[2].set()                                           # the new replica's worker goes away mid-load
        await asyncio.gather(*cl)
        for _ in range(100):
            if rt.ctl.idle() and not rt.requests:
                break
            await asyncio.sleep(0.05)
        final = ([rt.ctl.state_name(r) for r in range(n)], rt.ctl.idle(), rt.ctl.total_used_blocks(), len(rt.cached),
                 [len(backends[r].batches) for r in (0, 1)], [backends[r].pool.used_pages for r in (0, 1)])
        await rt.stop()
        lt.cancel()
        for s in stops:
            s.set()
        await asyncio.wait(tasks, timeout=5)
        return results, seen_new, final
    results, seen_new, final = asyncio.run(go())
    assert seen_new == "NewPrefill"
    assert len(results) == 60 and all((err is None and k == 3) or err == "replica lost" for err, k in results)
    assert sum(1 for err, _ in results if err is None) >= 40
    assert final == (["Prefill", "Decode", "Inactive"], True, 0, 0, [0, 0], [0, 0]), final


def test_client_disconnect_stops_generation_for_that_request():
    """A client closes its connection in the middle of a long generation (and another one while still queued): the
    router tells the worker to drop the request, the others go on, and nothing is left behind."""
    import aiohttp

    async def go():
        rt, backends, port, stop, tasks = await _cluster(2, ["Prefill", "Decode"], "impl_blitz,impl_nvl", autoscale=False)
        for b in backends:
            b.decode_step_s = 0.01
        url = f"http://127.0.0.1:{port}"
        async with aiohttp.ClientSession() as s:
            async def full(n):
                async with s.post(url + "/generate", json={"input_tokens": list(range(30)), "parameters": {"max_new_tokens": n}}) as r:
                    return r.status, r.headers.get("x-generated-tokens")
            keep = asyncio.create_task(full(60))
            gone = asyncio.create_task(full(2000))               # 20 s of decoding if nobody stops it
            await asyncio.sleep(0.3)
            gone.cancel()                                        # closes that connection
            streamed = 0
            async with s.post(url + "/generate_stream", json={"input_tokens": list(range(30)), "parameters": {"max_new_tokens": 2000}}) as r:
                async for line in r.content:
                    if line.startswith(b"data:"):
                        streamed += 1
                        if streamed == 3:
                            break                                # leave in the middle of the stream
            status, n = await asyncio.wait_for(keep, timeout=30)
        assert status == 200 and n == "60"
        for _ in range(100):
            if rt.ctl.idle() and not rt.requests and all(not b.batches for b in backends):
                break
            await asyncio.sleep(0.05)
        state = (len(rt.requests), rt.ctl.idle(), rt.ctl.total_used_blocks(), [len(b.batches) for b in backends],
                 [b.pool.used_pages for b in backends], dict(rt.ctl.counters()).get("blitz_filtered_batches", 0),
                 backends[1].counters["decode"])
        await _shutdown(stop, tasks)
        return state
    state = asyncio.run(go())
    assert state[:5] == (0, True, 0, [0, 0], [0, 0]), state
    assert state[5] >= 1 and state[6] < 400                      # filtered; nowhere near the 2000 steps asked for


@pytest.mark.parametrize("progressive", [False, True])
def test_tensor_parallel_replicas_over_grpc_and_loss_of_one_shard(progressive):
    """Replicas of two ranks each: every action goes to both ranks of a replica; when one shard's worker goes away the
    whole replica is lost (the failing rank maps to its replica), and the survivor takes over both phases.  With
    layer-progressive migration the prefill call spans both shards of both replicas; a decode shard that is gone is
    then noticed before the prompt has produced anything, so the prompt is served again instead of failing."""
    async def go():
        n, tp = 4, 2
        ports = _free_ports(n)
        states = ["Prefill", "Prefill", "Decode", "Decode"]          # per rank: replica 0 = ranks 0-1, replica 1 = ranks 2-3
        backends, stops, tasks = [], [], []
        for r in range(n):
            ready, stop = asyncio.Event(), asyncio.Event()
            backends.append(StubBackend(r, n, ready=True, seed=3))
            tasks.append(asyncio.create_task(serve(backends[r], "127.0.0.1", ports[r], stop_event=stop, ready_event=ready)))
            stops.append(stop)
            await ready.wait()
        cfg = controller_config_from_cluster({"init_states": states, "machines": [0] * n}, tp,
                                             "impl_blitz,impl_nvl" + (",migrate_progressive" if progressive else ""),
                                             max_blocks_per_replica=4000)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2)
        assert rt.ctl.num_replicas == 2
        lt = asyncio.create_task(rt.run())

        async def one(k):
            lr = rt.submit(list(range(25)), k, stream=False)
            return await asyncio.wait_for(lr.done, 30), list(lr.tokens)
        err, toks = await one(5)
        assert err is None and len(toks) == 5
        counts = [dict(b.counters) for b in backends]
        assert counts[0]["prefill"] == counts[1]["prefill"] == 1 and counts[2]["decode"] == counts[3]["decode"] >= 4
        moved = "migrate_progressive" if progressive else "migrate"
        assert counts[0][moved] == counts[1][moved] == 1 and counts[2]["immigrate"] == counts[3]["immigrate"] == 1
        stops[3].set()                                            # one shard of the decode replica goes away
        await asyncio.wait([tasks[3]], timeout=5)
        err, toks_lost = await one(5)
        if progressive:
            assert err is None and len(toks_lost) == 5            # nothing had been delivered: served again by replica 0
        else:
            assert err == "replica lost"
        assert rt.ctl.state_name(1) == "Inactive" and rt.ctl.state_name(0) == "Prefill"
        for _ in range(40):                                       # the surviving shard of the lost replica drops its state
            if not backends[2].batches:
                break
            await asyncio.sleep(0.05)
        assert not backends[2].batches and backends[2].pool.used_pages == 0
        err, toks2 = await one(5)                                 # replica 0 now serves both phases, on both of its ranks
        assert err is None and len(toks2) == 5
        assert backends[0].counters["decode"] == backends[1].counters["decode"] >= 4
        await rt.stop()
        lt.cancel()
        for s in stops:
            s.set()
        await asyncio.wait(tasks, timeout=5)
    asyncio.run(go())


def test_sampling_parameters_reach_the_worker():
    """`do_sample` with temperature / top-k / seed travels from the HTTP request through the router into the worker's
    sequence state: the same seed reproduces the same tokens, another seed gives others, top-k bounds the draw, and
    greedy requests in the same batch are unaffected (the stub draws a function of the seed instead of sampling)."""
    import aiohttp

    async def go():
        rt, backends, port, stop, tasks = await _cluster(2, ["Prefill", "Decode"], "impl_blitz,impl_nvl", autoscale=False)
        url = f"http://127.0.0.1:{port}/generate"
        async with aiohttp.ClientSession() as s:
            async def gen(params):
                body = {"input_tokens": list(range(12)), "parameters": dict({"max_new_tokens": 6, "details": True}, **params)}
                async with s.post(url, json=body) as r:
                    data = await r.json()
                    assert r.status == 200, data
                    return [t["id"] for t in data["details"]["tokens"]]
            greedy, a1, a2, b, k = await asyncio.gather(
                gen({}), gen({"do_sample": True, "temperature": 0.7, "seed": 11}), gen({"do_sample": True, "temperature": 0.7, "seed": 11}),
                gen({"do_sample": True, "temperature": 0.7, "seed": 12}), gen({"do_sample": True, "top_k": 5, "seed": 3}))
            greedy2 = await gen({})
            async with s.post(url, json={"input_tokens": [1, 2], "parameters": {"do_sample": True, "temperature": -1.0}}) as r:
                bad = r.status
            # best_of > 1 is refused, not silently ignored
            async with s.post(url, json={"input_tokens": [1, 2], "parameters": {"do_sample": True, "best_of": 2}}) as r:
                assert r.status == 422 and "best_of" in (await r.text())
        await _shutdown(stop, tasks)
        return greedy, greedy2, a1, a2, b, k, bad
    greedy, greedy2, a1, a2, b, k, bad = asyncio.run(go())
    assert len(greedy) == 6 and len(greedy2) == 6          # greedy requests next to sampled ones run as usual
    assert a1 == a2 and a1 != b and a1 != greedy           # the seed decides
    assert len(set(a1)) > 1                                # a fresh draw at every step
    assert all(0 <= t < 5 for t in k)                      # top-k bounds the draw
    assert bad == 422


def test_end_of_sequence_token_and_stop_sequences_end_a_request():
    """Stopping rules beyond the token budget, over HTTP: the worker ends a request at the model's end-of-sequence token
    (finish_reason eos_token) unless the request sets ignore_eos_token; the router ends it when the generated text
    contains a stop sequence (finish_reason stop_sequence), drops what the worker produced after it and has the request
    filtered out of the worker's batch.  Other requests of the same batch are unaffected and nothing is left behind."""
    import aiohttp
    from blitz_scale_b200.sim.stub_worker import stub_token

    async def go():
        rt, backends, port, stop, tasks = await _cluster(2, ["Prefill", "Decode"], "impl_blitz,impl_nvl", autoscale=False)
        url = f"http://127.0.0.1:{port}/generate"
        async with aiohttp.ClientSession() as s:
            async def gen(params, stream=False):
                body = {"input_tokens": list(range(12)), "parameters": dict({"max_new_tokens": 8, "details": True}, **params)}
                if not stream:
                    async with s.post(url, json=body) as r:
                        data = await r.json()
                        assert r.status == 200, data
                        return [t["id"] for t in data["details"]["tokens"]], data["details"]["finish_reason"]
                toks, reason = [], None
                async with s.post(url + "_stream", json=body) as r:
                    assert r.status == 200
                    async for line in r.content:
                        if line.startswith(b"data:"):
                            ev = json.loads(line[5:])
                            toks.append(ev["token"]["id"])
                            if ev["details"]:
                                reason = ev["details"]["finish_reason"]
                return toks, reason
            def expected(rid):             # the stub's tokens are a function of (seed, request id, position)
                return [stub_token(0, rid, 12 + n) for n in range(8)]
            full = expected(rt._next_id)
            assert await gen({}) == (full, "length")
            # the worker's end-of-sequence id is the 4th token of the next request
            nxt = expected(rt._next_id)
            for b in backends:
                b.eos_token = nxt[3]
            cut = await gen({})
            assert cut == (nxt[:4], "eos_token")
            nxt = expected(rt._next_id)
            for b in backends:
                b.eos_token = nxt[3]
            assert await gen({"ignore_eos_token": True}) == (nxt, "length")
            for b in backends:
                b.eos_token = -1
            # a stop sequence that the 3rd token completes (two tokens long; streamed and not), next to a request
            # that runs to its budget: the two are submitted together, so either may get the lower id
            for rnd, stream in enumerate((False, True, False)):
                for b in backends:
                    b.stopper.enabled = rnd != 1         # second round: only the router checks the stop sequences
                if rnd == 2:
                    rt.decode_steps = 4     # third round: the worker runs 4 decode steps per call, so tokens it produced
                                            # after the stop sequence arrive in the same answer and must be dropped
                e0, e1 = expected(rt._next_id), expected(rt._next_id + 1)
                stops = [f"<{e[1]}> <{e[2]}>" for e in (e0, e1)] + ["never"]
                (st, why_st), (other, why_other) = await asyncio.gather(gen({"stop": stops}, stream=stream), gen({}))
                assert (st, other) in ((e0[:3], e1), (e1[:3], e0)), (st, other, e0, e1)
                assert (why_st, why_other) == ("stop_sequence", "length")
            async with s.post(url, json={"input_tokens": [1], "parameters": {"stop": ["a", "b", "c", "d", "e"]}}) as r:
                too_many = r.status
            # the compatibility route: a one-element list, or the event stream when the body asks for it
            root = f"http://127.0.0.1:{port}/"
            want = expected(rt._next_id)[:3]
            async with s.post(root, json={"input_tokens": list(range(12)), "parameters": {"max_new_tokens": 3, "details": True}}) as r:
                data = await r.json()
                assert r.status == 200 and isinstance(data, list) and len(data) == 1
                assert [t["id"] for t in data[0]["details"]["tokens"]] == want and "x-first-token-time" in r.headers
            async with s.post(root, json={"input_tokens": list(range(12)), "stream": True, "parameters": {"max_new_tokens": 3}}) as r:
                assert r.status == 200 and r.headers["Content-Type"].startswith("text/event-stream")
                events = [json.loads(l[5:]) async for l in r.content if l.startswith(b"data:")]
                assert len(events) == 3 and events[-1]["details"]["finish_reason"] == "length"
                assert events[0]["generated_text"] is None                       # the last event carries the whole text
                assert events[-1]["generated_text"] == " ".join(f"<{e['token']['id']}>" for e in events)
        for _ in range(100):
            if rt.ctl.idle() and not rt.requests and not rt.cached and all(not b.batches for b in backends):
                break
            await asyncio.sleep(0.05)
        state = (len(rt.requests), len(rt.cached), len(rt.ctl.finished()), rt.ctl.total_used_blocks(),
                 [len(b.batches) for b in backends], [b.pool.used_pages for b in backends])
        await _shutdown(stop, tasks)
        return too_many, state
    too_many, state = asyncio.run(go())
    assert too_many == 422
    assert state == (0, 0, 0, 0, [0, 0], [0, 0])


def test_worker_applies_stop_sequences_of_the_contract_by_itself():
    """A worker called directly (no router) ends a request when its generated text contains one of the request's
    `stop_sequences`, reports FinishReason 2 and frees the pages; other requests of the batch go on."""
    from blitz_scale_b200.runtime import core
    from blitz_scale_b200.sim.stub_worker import stub_token
    b = StubBackend(0, 1, ready=True)
    b.prefill_rate, b.decode_step_s = 1e12, 0.0
    exp = [stub_token(0, 7, 5 + n) for n in range(8)]
    batch = pb.Batch(id=1, size=2, max_tokens=256)
    for rid, stops in ((7, [f"<{exp[2]}> <{exp[3]}>", "never"]), (8, [])):
        r = batch.requests.add()
        r.id, r.inputs, r.prefill_logprobs, r.top_n_tokens = rid, "", False, 0
        r.input_tokens.extend(range(5))
        r.stopping_parameters.max_new_tokens, r.stopping_parameters.ignore_eos_token = 8, True
        r.stopping_parameters.stop_sequences.extend(stops)
    out, reasons = {7: [], 8: []}, {}

    def take(raw):
        for i, t, f, why in zip(*core.parse_generations_full(raw)):
            out[i].append(t)
            if f:
                reasons[i] = why
    gens, cb, _ = b.prefill(batch, 0, None, [])
    take(gens)
    while cb is not None:
        gens, cb = b.decode([cb], [pb.Tokens()])
        take(gens)
    assert out[7] == exp[:4] and reasons == {7: 2, 8: 0} and len(out[8]) == 8
    assert b.pool.used_pages == 0 and not b.batches and not b.stopper.stops
    # the pieces: the tail of a request's tokens, and ending it for a reason found outside the batch
    nb = core.Batch(3, b.pool)
    assert nb.add_prompts([core.SeqSpec(1, [1, 2, 3], 9)])
    nb.mark_prefilled()
    for t in (4, 5, 6):
        nb.append_tokens([t], True)
    assert nb.generated_tail(1, 2) == [5, 6] and nb.generated_tail(1, 10) == [4, 5, 6] and nb.generated_tail(99, 2) == []
    assert nb.finish_request(1, 2) and not nb.finish_request(1, 0) and not nb.finish_request(99, 2)
    assert nb.unfinished_ids() == [] and core.parse_generations_full(nb.encode_generations([6]))[3] == [2]
    nb.clear()


def test_malformed_request_bodies_are_validation_errors():
    """Bodies with wrong types or shapes answer 422 on every generation route (a typed request structure does that in
    the reference), never 5xx; well-formed edge cases still work."""
    import aiohttp

    async def go():
        rt, backends, port, stop, tasks = await _cluster(2, ["Prefill", "Decode"], "impl_blitz,impl_nvl,manually_scale",
                                                         autoscale=False)
        url = f"http://127.0.0.1:{port}"
        bad_bodies = [[1, 2, 3], "text", None, {"inputs": 123}, {"input_tokens": "abc"}, {"input_tokens": [1.5]},
                      {"inputs": "a", "parameters": []}, {"inputs": "a", "parameters": {"max_new_tokens": "x"}},
                      {"inputs": "a", "parameters": {"max_new_tokens": 0}}, {"inputs": "a", "parameters": {"stop": "word"}},
                      {"inputs": "a", "parameters": {"stop": [1]}}, {"inputs": "a", "parameters": {"truncate": -1}},
                      {"inputs": "a", "parameters": {"temperature": "hot", "do_sample": True}},
                      {"inputs": "a", "parameters": {"seed": "s", "do_sample": True}}, {"inputs": ""}, {"input_tokens": []}]
        out = []
        async with aiohttp.ClientSession() as s:
            for path in ("/generate", "/generate_stream", "/"):
                for b in bad_bodies:
                    async with s.post(url + path, json=b) as r:
                        out.append((path, b, r.status))
                async with s.post(url + path, data=b"{not json", headers={"Content-Type": "application/json"}) as r:
                    out.append((path, "raw", r.status))
            for b in ({}, [], "x", {"replica": "a", "state": "Prefill"}, {"replica": 1}, {"state": "Decode"}, {"replica": 1.5, "state": "Decode"}):
                async with s.post(url + "/modify_cluster_state", json=b) as r:
                    out.append(("/modify_cluster_state", b, r.status))
            async with s.post(url + "/modify_cluster_state", json={"replica": 7, "state": "Decode"}) as r:
                assert r.status == 409                       # well-formed, but there is no such replica
            # the API description: every route, and every schema reference resolves
            async with s.get(url + "/docs") as r:
                api = await r.json()
            import re
            assert {"/generate", "/generate_stream", "/", "/invocations", "/info", "/health", "/metrics",
                    "/modify_cluster_state"} <= set(api["paths"])
            assert set(re.findall(r"#/components/schemas/(\w+)", json.dumps(api))) <= set(api["components"]["schemas"])
            assert "stop" in api["components"]["schemas"]["GenerateParameters"]["properties"]
            async with s.post(url + "/generate", json={"inputs": "a b c d e", "parameters": {"truncate": 2, "max_new_tokens": 2}}) as r:
                ok = (r.status, r.headers.get("x-input-length"))
        await _shutdown(stop, tasks)
        return out, ok
    out, ok = asyncio.run(go())
    assert [o for o in out if o[2] != 422] == []
    assert ok == (200, "2")


@pytest.mark.parametrize("worker_stops", [True, False])
def test_stop_sequences_leaving_clients_and_progressive_migration_together(worker_stops):
    """Soak of the ways a request can end before its budget, mixed at random on a 2 + 2 cluster with layer-progressive
    migration and three decode steps per worker call: every request gets exactly the tokens up to its stop sequence
    (or all of them), clients that leave are forgotten, and nothing is left behind anywhere."""
    import random
    from blitz_scale_b200.sim.stub_worker import stub_token

    async def go():
        rng = random.Random(3)
        rt, backends, port, stop, tasks = await _cluster(4, ["Prefill", "Decode", "Prefill", "Decode"],
                                                         "impl_blitz,impl_nvl,migrate_progressive", autoscale=False)
        rt.decode_steps = 3
        for b in backends:
            b.decode_step_s, b.prefill_rate = 0.0005, 1e7
            # workers apply stop sequences themselves; with that off the router's own check is what ends the requests
            # (the case of a router and workers that do not share a tokenizer)
            b.stopper.enabled = worker_stops

        def detok(ids):
            return " ".join(f"<{i}>" for i in ids)

        async def one(i):
            await asyncio.sleep(rng.random())
            n_in, n_new = 5 + rng.randrange(60), 1 + rng.randrange(20)
            exp = [stub_token(0, rt._next_id, n_in + n) for n in range(n_new)]
            mode = rng.choice(["plain", "stop", "gone", "stop_at_last"])
            stops, want = (), exp
            if mode in ("stop", "stop_at_last") and n_new >= 3:
                k = rng.randrange(1, n_new - 1) if mode == "stop" else n_new - 1
                stops, want = (f"<{exp[k]}>",), exp[:k + 1]
            lr = rt.submit(list(range(n_in)), n_new, stream=False, stop=stops, detok=detok)
            if mode == "gone":
                await asyncio.sleep(rng.random() * 0.05)
                rt.client_gone(lr.id)
                await asyncio.wait_for(lr.done, 30)
                return None
            assert (await asyncio.wait_for(lr.done, 30)) is None
            if list(lr.tokens) != want:
                return (mode, lr.tokens, want)
            if len(want) < len(exp) and lr.finish_reason != "stop_sequence":
                return (mode, lr.finish_reason)
            return None
        wrong = [r for r in await asyncio.gather(*[one(i) for i in range(150)]) if r]
        for _ in range(200):
            if rt.ctl.idle() and not rt.requests and not rt.cached and all(not b.batches for b in backends):
                break
            await asyncio.sleep(0.05)
        state = (len(rt.requests), len(rt.cached), len(rt.first_tokens), len(rt.ctl.finished()), rt.ctl.inflight_ops(),
                 rt.ctl.total_used_blocks(), [len(b.batches) for b in backends], [b.pool.used_pages for b in backends])
        progressive = rt.ctl.counters().get("blitz_progressive_kv_cache_times", 0)
        await _shutdown(stop, tasks)
        return wrong, state, progressive
    wrong, state, progressive = asyncio.run(go())
    assert wrong == []
    assert state == (0, 0, 0, 0, 0, 0, [0, 0, 0, 0], [0, 0, 0, 0])
    assert progressive > 0


def test_router_learns_the_workers_kv_capacity_at_start():
    async def go():
        ports = _free_ports(2)
        stop, tasks = asyncio.Event(), []
        for r in range(2):
            ready = asyncio.Event()
            b = StubBackend(r, 2, ready=True, num_pages=512 if r == 0 else 300, page_size=64)
            tasks.append(asyncio.create_task(serve(b, "127.0.0.1", ports[r], stop_event=stop, ready_event=ready)))
            await ready.wait()
        cfg = controller_config_from_cluster({"init_states": ["Prefill", "Decode"], "machines": [0, 0]}, 1, "impl_blitz,impl_nvl",
                                             max_blocks_per_replica=30000, block_size=64)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2)
        lt = asyncio.create_task(rt.run())
        lr = rt.submit(list(range(20)), 3, stream=False)
        assert (await asyncio.wait_for(lr.done, 20)) is None
        limit = rt.ctl.max_blocks_per_replica
        await rt.stop()
        lt.cancel()
        stop.set()
        await asyncio.wait(tasks, timeout=5)
        return limit
    assert asyncio.run(go()) == 300 - 300 // 64          # the smaller pool, less headroom; not the configured 30000
