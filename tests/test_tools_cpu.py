"""CPU tests of the operator tools: worker client (REPL, load latency, broadcast bench), log and trace tools, topology."""
import asyncio
import io
import json
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
