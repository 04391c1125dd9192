"""CPU tests of the operator tools: worker client (REPL, load latency, broadcast bench), log and trace tools, topology."""
import asyncio
import io
import json
import os
import socket

import pytest

from blitz_scale_b200.sim import trace_tools
from blitz_scale_b200.utils import logtools, topology


def _free_ports(n):
    socks = [socket.socket() for _ in range(n)]
    for s in socks:
        s.bind(("127.0.0.1", 0))
    ports = [s.getsockname()[1] for s in socks]
    for s in socks:
        s.close()
    return ports


def test_worker_client_against_stub_workers(tmp_path):
    from blitz_scale_b200.router.stub import WorkerStub
    from blitz_scale_b200.sim.stub_worker import StubBackend
    from blitz_scale_b200.utils import worker_client as wc
    from blitz_scale_b200.worker.service import serve

    async def go():
        ports = _free_ports(3)
        stops, tasks, backends = [], [], []
        for r, p in enumerate(ports):
            stop, ready = asyncio.Event(), asyncio.Event()
            b = StubBackend(r, 3, ready=(r == 0))
            backends.append(b)
            tasks.append(asyncio.create_task(serve(b, "127.0.0.1", p, stop_event=stop, ready_event=ready)))
            await ready.wait()
            stops.append(stop)
        stubs = [WorkerStub(f"127.0.0.1:{p}") for p in ports]
        # cold start of rank 1 by a transfer from rank 0, then of rank 2 from "disk"
        r = await wc.load_latency(stubs, "p2p", src=0, dst=1, prompt_len=64)
        assert r["ttft_s"] >= r["load_s"] > 0 and (await stubs[1].health()).state == "ready"
        r = await wc.load_latency(stubs, "disk", dst=2, prompt_len=32)
        assert r["mode"] == "disk" and (await stubs[2].health()).state == "ready"
        b = await wc.benchmark_broadcast(stubs, "nvl", [0], [1, 2], repeats=2, param_bytes=16e9)
        assert b["median_s"] > 0 and b["gbs_per_dst"] > 0
        # scripted REPL session touching the main RPC families
        out = io.StringIO()
        repl = wc.Repl(stubs, out=out)
        script = ["help", "health 0", "info 0", "prefill 0 11 16,40 3", "decode 0 11", "decode 0 11", "clear 0",
                  "reset 1", "health 1", "bcast nvl 0 1", "ready 1", "health 1", "bogus", "decode 0 999", "quit"]
        await repl.loop(iter(script))
        text = out.getvalue()
        assert "commands" in text and "loading" in text and "unknown command" in text and "error: KeyError" in text
        assert text.count("'tokens'") == 3
        for s in stubs:
            await s.close()
        for st in stops:
            st.set()
        await asyncio.wait(tasks, timeout=5)
    asyncio.run(go())


def test_logtools(tmp_path):
    router = ["[   0.001] boot Replica<0> Inactive => Prefill", "[   0.002] boot Replica<1> Inactive => Decode",
              "[   1.500] scale: planner wants 2 prefill", "[   1.501] Replica<2> Inactive => LoadingPrefill",
              "  continuation without a stamp", "[   2.750] Replica<2> LoadingPrefill => Prefill",
              "[   3.000] batch 7 migrate start -~> replica 1", "[   3.010] batch 7 immigrate start",
              "[   3.050] batch 7 migrate done", "[   3.051] batch 7 immigrate done", "[   3.100] batch 8 migrate start"]
    worker = ["[   1.600] zag embed batch=3", "[   1.610] zag layer batch=3 layer=0", "[   1.620] zag layer batch=4 layer=0",
              "[   1.630] zag layer batch=3 layer=1", "[   1.640] zag relay batch=3", "[   1.650] zag head batch=4"]
    merged = list(logtools.merge_logs({"router": router, "w2": worker}))
    stamps = [logtools.timestamp(l.split("| ", 1)[1]) for l in merged]
    known = [s for s in stamps if s is not None]
    assert known == sorted(known) and len(merged) == len(router) + len(worker)
    assert merged[4].startswith("w2|") or merged[5].startswith("w2|")
    assert len(logtools.grep(router, "transitions")) == 4 and len(logtools.grep(router, "migrations")) == 5
    tl = logtools.zigzag_timeline(worker)
    rows = tl.splitlines()
    assert rows[0].endswith("|E0 1> |") and rows[1].endswith("|  0  H|")
    chart = logtools.usage_chart(router, width=40)
    assert "replica  2" in chart and "l" in chart and "P" in chart and "D" in chart
    res = logtools.check_migrations(router)
    assert res == {"complete": [7], "incomplete": [8]}
    assert logtools.timestamp("2024-05-01T10:00:00.250 INFO x") == pytest.approx(
        logtools.timestamp("2024-05-01 10:00:00.250 x"))
    p = tmp_path / "r.log"
    p.write_text("\n".join(router))
    assert logtools.main(["migrations", str(p)]) == 1 and logtools.main(["usage", str(p), "--width", "30"]) == 0


def test_trace_tools(tmp_path):
    rows = [(i * 100.0, 100 + i, 10 + i % 3) for i in range(100)]          # 10 req/s for 10 s
    src = tmp_path / "t.csv"
    trace_tools.write_trace(str(src), rows)
    assert trace_tools.read_trace(str(src)) == rows
    s = trace_tools.slice_trace(rows, 2.0, 3.0)
    assert len(s) == 30 and s[0][0] == 0.0 and s[-1][0] == pytest.approx(2900.0)
    sc = trace_tools.scale_trace(rows, rate=2.0, max_prefill=150)
    assert sc[-1][0] == pytest.approx(rows[-1][0] / 2) and max(p for _, p, _ in sc) == 150
    cc = trace_tools.concat_traces([rows[:10], rows[:10]], gap_s=1.0)
    assert len(cc) == 20 and cc[10][0] == pytest.approx(900.0 + 1000.0)
    st = trace_tools.trace_stats(rows, window_s=1.0)
    assert st["requests"] == 100 and st["mean_rps"] == pytest.approx(100 / 9.9) and st["peak_rps"] == 10
    assert trace_tools.main(["scale", str(src), str(tmp_path / "o.csv"), "--rate", "4"]) == 0
    assert len(trace_tools.read_trace(str(tmp_path / "o.csv"))) == 100
    recs = [{"ttft_ms": 100 + 10 * i, "input_length": 200, "tbt_ms": [20, 30], "ok": True} for i in range(30)]
    for name in ("a", "b"):
        with open(tmp_path / f"{name}.jsonl", "w") as f:
            for r in recs:
                f.write(json.dumps(r) + "\n")
    cmp = trace_tools.compare_violations(str(tmp_path / "a.jsonl"), str(tmp_path / "b.jsonl"))
    assert all(v == 0 for v in cmp["delta"].values())


TOPO = """\tGPU0\tGPU1\tGPU2\tGPU3\tNIC0\tCPU Affinity\tNUMA Affinity\tGPU NUMA ID
GPU0\t X \tNV18\tNV18\tNV18\tPIX\t0-3,8-11\t0\t\tN/A
GPU1\tNV18\t X \tNV18\tNV18\tSYS\t0-3,8-11\t0\t\tN/A
GPU2\tNV18\tNV18\t X \tNV18\tSYS\t4-7\t1\t\tN/A
GPU3\tNV18\tNV18\tNV18\t X \tSYS\t4-7\t1\t\tN/A
NIC0\tPIX\tSYS\tSYS\tSYS\t X \t\t\t\t

Legend:
  X    = Self
"""


def test_topology_parser():
    t = topology.parse_topo_matrix(TOPO)
    assert sorted(t.links) == [0, 1, 2, 3] and t.all_nvlink() and t.nvlink_count(0, 3) == 18
    assert t.cpu_affinity[0] == [0, 1, 2, 3, 8, 9, 10, 11] and t.cpu_affinity[3] == [4, 5, 6, 7]
    assert t.numa_node == {0: 0, 1: 0, 2: 1, 3: 1}
    bad = topology.parse_topo_matrix(TOPO.replace("GPU1\tNV18", "GPU1\tSYS"))
    assert not bad.all_nvlink()
    assert topology.parse_topo_matrix("no gpus here").links == {}
    assert topology.bind_to_gpu_cpus(0, topology.GpuTopology()) == []


def test_tracing_helpers(tmp_path):
    from blitz_scale_b200.utils import tracing
    root = tracing.new_traceparent()
    kid = tracing.child_traceparent(root)
    assert tracing.trace_id(root) == tracing.trace_id(kid) and root != kid and len(kid.split("-")) == 4
    assert tracing.grpc_metadata(None) is None and tracing.grpc_metadata(kid) == (("traceparent", kid),)
    with tracing.nvtx_range("noop"):          # flag off: no CUDA needed
        pass
    log = ["[   0.001] boot Replica<0> Inactive => Prefill", "[   0.002] boot Replica<1> Inactive => Decode",
           "[   1.000] Control signal: P+1 D+0", "[   1.001] Replica<2> Inactive => LoadingPrefill",
           "[   1.400] Replica<2> LoadingPrefill => Prefill", "[   2.000] System Metrics: prefill_tokens: 1200, decode_tokens: 340",
           "[   0.500] Client start"]
    recs = [{"id": 0, "start_s": 0.1, "ttft_ms": 120.0, "latency_ms": 900.0, "input_length": 300, "output_length": 20}]
    tr = tracing.chrome_trace(log, recs)
    names = [e["name"] for e in tr["traceEvents"]]
    assert "LoadingPrefill" in names and "Prefill" in names and "decode" in names and "tokens" in names
    assert any(n.startswith("scale-out 399") or n.startswith("scale-out 400") for n in names)
    p = tmp_path / "r.log"
    p.write_text("\n".join(log))
    assert tracing.main([str(p), "-o", str(tmp_path / "t.json")]) == 0
    assert json.loads((tmp_path / "t.json").read_text())["traceEvents"]


def test_tp_load_agreement():
    """Shards of a replica act on the minimum of their published loaded-unit counts."""
    from blitz_scale_b200.parallel.agreement import LoadAgreement

    class FakeFabric:
        def __init__(self, world, rank, pads):
            self.rank, self.pads = rank, pads
        def set_flag(self, rank, index, value, add=False):
            self.pads[rank][index] = self.pads[rank].get(index, 0) + value if add else value
        def read_flags(self, start, count):
            return [self.pads[self.rank].get(start + i, 0) for i in range(count)]

    pads = {r: {} for r in range(4)}
    L, F0 = 4, 1000
    a = [LoadAgreement(FakeFabric(4, r, pads), [2, 3], r, F0, L) for r in (2, 3)]
    for x in a:
        x.publish(0)
    assert a[0].agreed_state() == (False, 0, False)
    a[0].publish(3)                      # shard 0 has embed + 2 layers, shard 1 nothing yet
    assert a[0].agreed_units() == 0 and a[1].agreed_units() == 0
    a[1].publish(2)
    assert a[0].agreed_state() == (True, 1, False) and a[1].agreed_state() == (True, 1, False)
    a[0].publish(L + 2)
    a[1].publish(L + 1)
    assert a[1].agreed_state() == (True, L, False)
    a[1].publish(L + 2)
    assert a[0].agreed_state() == (True, L, True)
    assert 0 not in pads[0] and F0 not in pads[0]          # nothing leaks to other replicas' pads


def test_tp_step_log_orders_live_execution_steps():
    """The leading shard's decisions reach the other shard in order, one word each, through a ring that is reused; the
    follower's scheduler applies them by task sequence number although its queue filled in a different order."""
    from blitz_scale_b200.parallel.agreement import StepLog
    from blitz_scale_b200.runtime import core

    class FakeFabric:
        def __init__(self, rank, pads):
            self.rank, self.pads = rank, pads
        def set_flag(self, rank, index, value, add=False):
            self.pads[rank][index] = value
        def read_flags(self, start, count):
            return [self.pads[self.rank].get(start + i, 0) for i in range(count)]

    pads = {r: {} for r in range(2)}
    lead = StepLog(FakeFabric(0, pads), [0, 1], 0, 500, 16)
    fol = StepLog(FakeFabric(1, pads), [0, 1], 1, 500, 16)
    assert lead.leader and not fol.leader and fol.peek() is None
    L = 3
    zl, zf = core.ZigzagScheduler(L, 4), core.ZigzagScheduler(L, 4)
    zl.add_task(70, 1, 10)
    zl.add_task(71, 2, 20)
    zl.set_loaded(True, 1, False)
    applied = []
    fol_tasks_added = False
    for turn in range(60):
        if turn == 3:
            zl.set_loaded(True, 2, False)
        if turn == 6:
            zl.set_loaded(True, L, True)
        d = zl.next()
        if d.step in (core.ZagStep.Idle, core.ZagStep.Blocked):
            if turn > 6:
                break
            continue
        lead.publish(StepLog.STEP, int(d.step), max(0, d.layer), d.slot, zl.seq_of(d.batch_id))
        zl.complete(d)
        if turn == 1 and not fol_tasks_added:
            # the follower hears about the requests late, and in one go
            zf.add_task(70, 1, 10)
            zf.add_task(71, 2, 20)
            fol_tasks_added = True
        while fol_tasks_added:
            e = fol.peek()
            if e is None:
                break
            fol.consume()
            fd = core.ZagDecision()
            fd.step, fd.batch_id, fd.slot = core.ZagStep(e["step"]), zf.batch_of(e["seq_num"]), e["slot"]
            fd.layer = e["layer"] if fd.step == core.ZagStep.Layer else -1
            zf.complete(fd)
            applied.append((int(fd.step), fd.batch_id, fd.layer))
    assert zl.pending() == 0 and zf.pending() == 0
    assert len(applied) == 2 * (L + 2) and lead.pos == fol.pos == len(applied)
    # a hand-over names the task by sequence number
    zf.add_task(80, 5, 7)
    zf.add_task(81, 6, 9)
    lead.publish(StepLog.RELAY, 0, 0, 2, 6)
    e = fol.peek()
    assert e["kind"] == StepLog.RELAY and e["seq_num"] == 6 and e["layer"] == 0
    r = zf.relay_task(e["seq_num"])
    assert r.batch_id == 81 and r.next_layer == -1 and zf.pending() == 1 and zf.relay_task(99) is None


def test_otlp_span_export_logging_and_cors(tmp_path):
    """Spans of dispatched operations and requests reach an OTLP/HTTP collector (a local stand-in) in the JSON
    mapping; the log set-up writes JSON lines through the background file writer; CORS headers follow the allow list."""
    import asyncio
    import json
    import logging
    import socket

    from aiohttp import web

    from blitz_scale_b200.router.runtime import RouterRuntime
    from blitz_scale_b200.router.server import RouterApp, controller_config_from_cluster
    from blitz_scale_b200.sim.stub_worker import StubBackend
    from blitz_scale_b200.utils import analysis
    from blitz_scale_b200.utils.otlp import SpanExporter, init_logging, span_record
    from blitz_scale_b200.worker.service import serve

    rec = span_record("x", "00-" + "ab" * 16 + "-" + "cd" * 8 + "-01", 10, 20, {"n": 3, "f": 0.5, "s": "t", "b": True}, "ee" * 8, ok=False)
    assert rec["traceId"] == "ab" * 16 and rec["spanId"] == "cd" * 8 and rec["parentSpanId"] == "ee" * 8
    assert rec["startTimeUnixNano"] == "10" and rec["status"]["code"] == 2
    assert {a["key"]: list(a["value"])[0] for a in rec["attributes"]} == {"n": "intValue", "f": "doubleValue", "s": "stringValue", "b": "boolValue"}

    cport, aport, *worker_ports = _free_ports(4)

    async def go():
        got = []

        async def collect(req):
            got.append(await req.json())
            return web.json_response({})
        capp = web.Application()
        capp.router.add_post("/v1/traces", collect)
        crun = web.AppRunner(capp, access_log=None)
        await crun.setup()
        await web.TCPSite(crun, "127.0.0.1", cport).start()

        ports = worker_ports
        stop, tasks = asyncio.Event(), []
        for r in range(2):
            ready = asyncio.Event()
            tasks.append(asyncio.create_task(serve(StubBackend(r, 2, ready=True), "127.0.0.1", ports[r], stop_event=stop, ready_event=ready)))
            await ready.wait()
        exp = SpanExporter(f"http://127.0.0.1:{cport}", "blitz.router", interval_s=0.1)
        exp.start()
        cfg = controller_config_from_cluster({"init_states": ["Prefill", "Decode"], "machines": [0, 0]}, 1, "impl_blitz,impl_nvl",
                                             max_blocks_per_replica=4000, autoscale=False)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{p}" for p in ports], model_layers=2, exporter=exp)
        lt = asyncio.create_task(rt.run())
        lr = rt.submit(list(range(20)), 3, stream=False)
        assert (await asyncio.wait_for(lr.done, 20)) is None
        # CORS on the HTTP app
        app = RouterApp(rt, model_name="tiny", cors_allow_origin=["http://ui.example"])
        arun = web.AppRunner(app.app, access_log=None)
        await arun.setup()
        await web.TCPSite(arun, "127.0.0.1", aport).start()
        import aiohttp
        async with aiohttp.ClientSession() as s:
            async with s.get(f"http://127.0.0.1:{aport}/info", headers={"Origin": "http://ui.example"}) as r:
                assert r.status == 200 and r.headers["Access-Control-Allow-Origin"] == "http://ui.example"
            async with s.get(f"http://127.0.0.1:{aport}/info", headers={"Origin": "http://other.example"}) as r:
                assert r.status == 200 and "Access-Control-Allow-Origin" not in r.headers
            async with s.options(f"http://127.0.0.1:{aport}/generate", headers={"Origin": "http://ui.example",
                                                                                "Access-Control-Request-Headers": "content-type"}) as r:
                assert r.status == 204 and r.headers["Access-Control-Allow-Headers"] == "content-type"
            async with s.get(f"http://127.0.0.1:{aport}/metrics") as r:
                assert "blitz_request_skipped_tokens_count" in await r.text()
        await exp.stop()                                        # flushes
        await rt.stop()
        lt.cancel()
        stop.set()
        await asyncio.wait(tasks, timeout=5)
        await arun.cleanup()
        await crun.cleanup()
        # the collector is gone now: export fails quietly and counts the loss
        exp2 = SpanExporter(f"http://127.0.0.1:{cport}", interval_s=0.1)
        exp2.span("late", "", 1.0, 2.0)
        assert await exp2.flush() == 0 and exp2.dropped == 1
        await exp2.close()
        return got, exp
    got, exp = asyncio.run(go())
    spans = [s for g in got for rs in g["resourceSpans"] for ss in rs["scopeSpans"] for s in ss["spans"]]
    assert got[0]["resourceSpans"][0]["resource"]["attributes"][0]["value"]["stringValue"] == "blitz.router"
    names = [s["name"] for s in spans]
    assert {"Prefill", "Migrate", "Decode", "generate"} <= set(names) and exp.exported == len(spans) and exp.dropped == 0
    assert len({s["traceId"] for s in spans}) == 1 and len({s["spanId"] for s in spans}) == len(spans)
    gen = [s for s in spans if s["name"] == "generate"][0]
    attrs = {a["key"]: a["value"] for a in gen["attributes"]}
    assert attrs["generated_tokens"] == {"intValue": "3"} and attrs["input_tokens"] == {"intValue": "20"}
    assert int(gen["endTimeUnixNano"]) > int(gen["startTimeUnixNano"])

    # logging: JSON lines through the background file writer, level from LOG_LEVEL
    saved = logging.getLogger().handlers[:], logging.getLogger().level
    try:
        os.environ["LOG_LEVEL"] = "warning"
        listener = init_logging(None, True, str(tmp_path / "router.log"))
        logging.getLogger("blitz.router").info("dropped by the filter")
        logging.getLogger("blitz.router").warning("Replica<%d> Inactive => LoadingPrefill", 2)
        listener.stop()
        lines = [json.loads(l) for l in open(tmp_path / "router.log")]
        assert len(lines) == 1 and lines[0]["level"] == "WARNING" and lines[0]["target"] == "blitz.router"
        assert lines[0]["message"] == "Replica<2> Inactive => LoadingPrefill" and lines[0]["filename"].endswith(".py")
        p = analysis.parse_router_log(open(tmp_path / "router.log"))
        assert p["transitions"][0][1:] == (2, "Inactive", "LoadingPrefill") and p["transitions"][0][0] is not None
    finally:
        os.environ.pop("LOG_LEVEL", None)
        root = logging.getLogger()
        for h in root.handlers[:]:
            root.removeHandler(h)
        for h in saved[0]:
            root.addHandler(h)
        root.setLevel(saved[1])


def test_router_flags_from_the_environment(monkeypatch):
    from blitz_scale_b200.router.server import build_parser
    monkeypatch.setenv("CLIENT_CONFIG", '["127.0.0.1:1"]')
    monkeypatch.setenv("DEPLOYMENT_CONFIG_PATH", "/tmp/cluster.json")
    monkeypatch.setenv("MAX_BEST_OF", "3")
    monkeypatch.setenv("JSON_OUTPUT", "true")
    monkeypatch.setenv("CORS_ALLOW_ORIGIN", "http://a,http://b")
    monkeypatch.setenv("HOSTNAME", "some-container-name")
    a = build_parser().parse_args(["--max-stop-sequences", "7", "--num-hidden-layers", "32", "--parameter-size", "16.0"])
    assert a.client_config == '["127.0.0.1:1"]' and a.deployment_config_path == "/tmp/cluster.json"   # required ones too
    assert a.max_best_of == 3 and a.json_output is True and a.cors_allow_origin == ["http://a", "http://b"]
    assert a.max_stop_sequences == 7 and a.hostname == "127.0.0.1"          # the command line wins; HOSTNAME is ignored
    monkeypatch.setenv("MAX_BEST_OF", "9")
    assert build_parser().parse_args(["--max-best-of", "4"]).max_best_of == 4


def test_run_report_figures(tmp_path):
    from blitz_scale_b200.utils import plots
    log = ["[0.000] Replica<0> boot => Prefill", "[0.000] Replica<1> boot => Decode",
           "[1.500] Replica<2> Inactive => LoadingPrefill", "[1.530] Replica<2> LoadingPrefill => Prefill",
           "[1.0] System Metrics: prefill_tokens: 0, decode_tokens: 0", "[2.0] System Metrics: prefill_tokens: 9000, decode_tokens: 700",
           "[3.0] System Metrics: prefill_tokens: 30000, decode_tokens: 2100", "[3.2] Replica<2> Prefill => ShuttingPrefill"]
    recs = [{"status": "ok", "s_time": 0.1 * i, "first_token_time": 40.0 + (500.0 if i == 7 else 0.0), "input_length": 200,
             "max_time_between_tokens": 12.0 + (120.0 if i == 3 else 0.0)} for i in range(20)] + [{"status": "error", "s_time": 1.0}]
    doc = plots.report(log, recs, "tiny <run>")
    assert doc.count("<svg") == 4 and "tiny &lt;run&gt;" in doc
    assert doc.count('fill="#d6453d" fill-opacity') == 2          # one TTFT violation, one TBT violation
    assert "replica 2 in 30.0 ms" in doc and "replica 2: LoadingPrefill" in doc and "prefill" in doc
    import xml.dom.minidom
    for part in doc.split("<svg")[1:]:
        xml.dom.minidom.parseString("<svg" + part.split("</svg>")[0] + "</svg>")      # every panel is well-formed
    (tmp_path / "router.log").write_text("\n".join(log))
    assert plots.main(["--router-log", str(tmp_path / "router.log"), "-o", str(tmp_path / "r.html")]) == 0
    assert (tmp_path / "r.html").read_text().count("<svg") == 2   # without client records: states and token rates
    assert plots._ticks(0.0, 10.0, 5) == [0.0, 2.0, 4.0, 6.0, 8.0, 10.0]


def test_package_command_dispatcher():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = lambda *a: subprocess.run([sys.executable, "-m", "blitz_scale_b200", *a], cwd=root, capture_output=True, text=True, timeout=120)
    r = run("--help")
    assert r.returncode == 0 and "stub-worker" in r.stdout and "report" in r.stdout
    assert run("no-such-command").returncode == 2
    r = run("trace", "--help")
    assert r.returncode == 0 and "usage" in r.stdout.lower()
    r = run("report", "--help")
    assert r.returncode == 0 and "--router-log" in r.stdout


def test_router_cli_reports_configuration_mistakes_in_one_line(tmp_path):
    """A cluster description or flag the router cannot work with ends the start-up with one line that names the
    mistake, not a traceback."""
    import json
    import subprocess
    import sys
    good = tmp_path / "good.json"
    good.write_text(json.dumps({"init_states": ["Prefill", "Decode"], "machines": [0, 0]}))
    mixed = tmp_path / "mixed.json"
    mixed.write_text(json.dumps({"init_states": ["Prefill", "Decode"], "machines": [0, 0]}))
    nostates = tmp_path / "nostates.json"
    nostates.write_text(json.dumps({"machines": [0, 0]}))
    two = '["127.0.0.1:1", "127.0.0.1:2"]'

    def run(*args):
        cmd = [sys.executable, "-m", "blitz_scale_b200.router.server", "--model-name", "tiny", "--model-path", "x",
               "--parameter-size", "1", *args]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=60,
                           cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        assert r.returncode != 0 and "Traceback" not in r.stderr, r.stderr
        return r.stderr.strip().splitlines()[-1]
    assert "init_states" in run("--client-config", two, "--deployment-config-path", str(nostates))
    assert "must share a state" in run("--client-config", two, "--deployment-config-path", str(mixed), "--tensor-parallel-size", "2")
    assert "3 worker addresses for 2 ranks" in run("--client-config", '["a:1", "b:2", "c:3"]', "--deployment-config-path", str(good))
    assert "unknown feature: bogus" in run("--client-config", two, "--deployment-config-path", str(good), "--features", "impl_blitz,bogus")
    assert "No such file" in run("--client-config", two, "--deployment-config-path", str(tmp_path / "none.json"))
    assert "tunnel" in run("--client-config", two, "--deployment-config-path", str(good), "--ngrok")


def test_worker_launcher_checks_the_cluster_description_before_touching_a_gpu(tmp_path, monkeypatch):
    import json

    from blitz_scale_b200.worker import launcher
    good = tmp_path / "good.json"
    good.write_text(json.dumps({"init_states": ["Prefill", "Decode"]}))
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"init_states": ["Prefill", "Sleeping"]}))

    def run(world, *args):
        # the checks come first in `main`: it leaves with one line before any device, log file or process group is touched
        monkeypatch.setenv("WORLD_SIZE", str(world))
        monkeypatch.setenv("RANK", "0")
        monkeypatch.setenv("LOCAL_RANK", "0")
        with pytest.raises(SystemExit) as e:
            launcher.main(list(args))
        assert isinstance(e.value.code, str)
        return e.value.code
    assert "lists 2 ranks, world size is 1" in run(1, "--config", str(good), "--model-name", "tiny")
    assert "init_states" in run(2, "--config", str(bad), "--model-name", "tiny")
    assert "must share a state" in run(2, "--config", str(good), "--model-name", "tiny", "-TP", "2")
    assert "unknown model" in run(2, "--config", str(good), "--model-name", "nope")
    assert "tokenizer file" in run(2, "--config", str(good), "--model-name", "tiny", "-T", str(tmp_path / "none.json"))
    assert "pipeline parallelism" in run(2, "--config", str(good), "--model-name", "tiny", "-PP", "2")
