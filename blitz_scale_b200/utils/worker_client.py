"""Direct gRPC drivers of a worker group, without the router.

* `load_latency`  time-to-first-token of a cold instance: parameters from disk / the host cache, or streamed
  from a running instance (`SendParams`/`RecvParams`, or an NVLink broadcast), followed by one prefill
  (the reference's microtest, scripts/batch/test_load_latency.py:267-381).
* `benchmark_broadcast`  time the parameter-transfer RPCs for a list of destination sets
  (scripts/debug/bcast_test.py:700-811: benchmark_{rdma_chain,nccl,tanz,tanz_nccl}).
* `repl`  an interactive client with one command per RPC (scripts/debug/bcast_test.py:228-251).

    python -m blitz_scale_b200.utils.worker_client repl --workers 127.0.0.1:50051,127.0.0.1:50052
    python -m blitz_scale_b200.utils.worker_client load-latency --workers ... --mode disk --model-path /data/llama3_8b
    python -m blitz_scale_b200.utils.worker_client bcast --workers ... --kind nvl --src 0 --dst 1,2,3
"""
from __future__ import annotations

import argparse
import asyncio
import json
import shlex
import sys
import time
from typing import Dict, List, Sequence

from ..pb.schema import pb
from ..router.stub import WorkerStub


def make_batch(batch_id: int, prompt_lens: Sequence[int], max_new_tokens: int = 2, first_id: int = 0, vocab: int = 1000):
    b = pb.Batch(id=batch_id, size=len(prompt_lens), max_tokens=sum(prompt_lens) + max_new_tokens * len(prompt_lens))
    for i, n in enumerate(prompt_lens):
        r = b.requests.add()
        r.id, r.inputs, r.prefill_logprobs, r.top_n_tokens = first_id + i, "", False, 0
        r.input_tokens.extend((7 * j + i) % vocab for j in range(n))
        r.stopping_parameters.max_new_tokens = max_new_tokens
        r.stopping_parameters.ignore_eos_token = True
    return b


async def load_latency(stubs: List[WorkerStub], mode: str, *, src: int = 0, dst: int = 1, model_name: str = "",
                       model_path: str = "", prompt_len: int = 512) -> Dict[str, float]:
    """One cold start of worker `dst`; returns seconds for the load, the first prefill and their sum."""
    d = stubs[dst]
    await d.reset_status()
    t0 = time.perf_counter()
    if mode == "disk":
        await d.load_params(pb.LOAD_FROM_DISK, model_name, model_path)
    elif mode == "host":
        await d.load_params(pb.LOAD_FROM_HOST_MEM, model_name, model_path)
    elif mode == "p2p":
        await d.recv_params(src)
        await stubs[src].send_params(dst)
        await d.wait_rdma_done()
    elif mode == "nvl":
        await asyncio.gather(stubs[src].broadcast("nvl", [src], [dst]), d.broadcast("nvl", [src], [dst]))
    else:
        raise ValueError(f"unknown mode {mode}")
    await d.set_status_ready()
    t1 = time.perf_counter()
    res = await d.prefill_v2(make_batch(900001, [prompt_len]))
    t2 = time.perf_counter()
    await d.clear_cache(900001)
    assert len(res.generations) == 1
    return {"mode": mode, "load_s": t1 - t0, "prefill_s": t2 - t1, "ttft_s": t2 - t0}


async def benchmark_broadcast(stubs: List[WorkerStub], kind: str, src: Sequence[int], dst: Sequence[int],
                              repeats: int = 3, param_bytes: float = 0.0) -> Dict[str, float]:
    """Every involved rank gets the same broadcast RPC (sources push, destinations poll their flags)."""
    times = []
    for _ in range(repeats):
        for r in dst:
            await stubs[r].reset_status()
        t0 = time.perf_counter()
        await asyncio.gather(*[stubs[r].broadcast(kind, list(src), list(dst)) for r in list(src) + list(dst)])
        times.append(time.perf_counter() - t0)
        for r in dst:
            await stubs[r].set_status_ready()
    times.sort()
    out = {"kind": kind, "src": list(src), "dst": list(dst), "median_s": times[len(times) // 2], "min_s": times[0]}
    if param_bytes:
        out["gbs_per_dst"] = param_bytes / out["median_s"] / 1e9
    return out


HELP = """commands (rank = index into --workers):
  info R | health R | warmup R | clear R [BATCH] | ready R | reset R
  prefill R BATCH_ID LEN[,LEN...] [NEW]      one PrefillV2 with synthetic prompts
  decode R BATCH_ID                          one DecodeV2 on the cached batch returned by the last prefill/decode
  load R disk|host [PATH]                    LoadParams
  send SRC DST | recv DST SRC | wait R       SendParams / RecvParams / WaitRdmaDone
  bcast KIND SRC[,SRC..] DST[,DST..]         KIND = nvl | tanz | rdma (all map to the NVLink unit copy here)
  migrate SRC DST BATCH_ID                   Immigrate on DST and Migrate on SRC
  bench KIND SRC DST[,DST..] [REPEATS]       timed broadcasts
  latency MODE [SRC] DST [PATH]              cold-start TTFT; MODE = disk | host | p2p | nvl
  help | quit"""


class Repl:
    def __init__(self, stubs: List[WorkerStub], out=sys.stdout):
        self.s, self.out = stubs, out
        self.cached: Dict[int, object] = {}

    def p(self, *a):
        print(*a, file=self.out, flush=True)

    async def run_line(self, line: str) -> bool:
        a = shlex.split(line)
        if not a:
            return True
        c, ints = a[0], lambda x: [int(v) for v in x.split(",") if v != ""]
        try:
            if c in ("quit", "exit"):
                return False
            elif c == "help":
                self.p(HELP)
            elif c == "info":
                r = await self.s[int(a[1])].info()
                self.p({"dtype": r.dtype, "device_type": r.device_type})
            elif c == "health":
                self.p((await self.s[int(a[1])].health()).state)
            elif c == "warmup":
                self.p((await self.s[int(a[1])].warmup()).max_supported_total_tokens)
            elif c == "clear":
                await self.s[int(a[1])].clear_cache(int(a[2]) if len(a) > 2 else None)
            elif c == "ready":
                await self.s[int(a[1])].set_status_ready()
            elif c == "reset":
                await self.s[int(a[1])].reset_status()
            elif c == "prefill":
                b = make_batch(int(a[2]), ints(a[3]), int(a[4]) if len(a) > 4 else 4)
                t0 = time.perf_counter()
                r = await self.s[int(a[1])].prefill_v2(b)
                if r.HasField("batch"):
                    self.cached[b.id] = r.batch
                self.p({"ms": round((time.perf_counter() - t0) * 1e3, 3), "tokens": [g.tokens.ids[0] for g in r.generations]})
            elif c == "decode":
                cb = self.cached[int(a[2])]
                t0 = time.perf_counter()
                r = await self.s[int(a[1])].decode_v2([cb], [pb.Tokens()])
                if r.HasField("batch"):
                    self.cached[int(a[2])] = r.batch
                else:
                    self.cached.pop(int(a[2]), None)
                self.p({"ms": round((time.perf_counter() - t0) * 1e3, 3), "tokens": [g.tokens.ids[0] for g in r.generations]})
            elif c == "load":
                case = pb.LOAD_FROM_DISK if a[2] == "disk" else pb.LOAD_FROM_HOST_MEM
                t0 = time.perf_counter()
                await self.s[int(a[1])].load_params(case, "", a[3] if len(a) > 3 else "")
                self.p({"s": round(time.perf_counter() - t0, 4)})
            elif c == "send":
                await self.s[int(a[1])].send_params(int(a[2]))
            elif c == "recv":
                await self.s[int(a[1])].recv_params(int(a[2]))
            elif c == "wait":
                await self.s[int(a[1])].wait_rdma_done()
            elif c == "bcast":
                src, dst = ints(a[2]), ints(a[3])
                t0 = time.perf_counter()
                await asyncio.gather(*[self.s[r].broadcast(a[1], src, dst) for r in src + dst])
                self.p({"s": round(time.perf_counter() - t0, 4)})
            elif c == "migrate":
                src, dst, bid = int(a[1]), int(a[2]), int(a[3])
                cb = self.cached[bid]
                b = pb.Batch(id=bid, size=cb.size, max_tokens=cb.max_tokens)
                await asyncio.gather(self.s[dst].immigrate(b, [src], [dst]), self.s[src].migrate(b, [src], [dst]))
                self.p("migrated")
            elif c == "bench":
                self.p(await benchmark_broadcast(self.s, a[1], ints(a[2]), ints(a[3]), int(a[4]) if len(a) > 4 else 3))
            elif c == "latency":
                rest = a[2:]
                if a[1] in ("disk", "host"):
                    self.p(await load_latency(self.s, a[1], dst=int(rest[0]), model_path=rest[1] if len(rest) > 1 else ""))
                else:
                    self.p(await load_latency(self.s, a[1], src=int(rest[0]), dst=int(rest[1])))
            else:
                self.p(f"unknown command {c!r}; try help")
        except Exception as e:  # noqa: BLE001 - a REPL reports and carries on
            self.p(f"error: {type(e).__name__}: {e}")
        return True

    async def loop(self, lines=None):
        loop = asyncio.get_running_loop()
        while True:
            if lines is not None:
                line = next(lines, None)
            else:
                line = await loop.run_in_executor(None, lambda: sys.stdin.readline())
            if not line or not await self.run_line(line.strip()):
                break


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("cmd", choices=["repl", "load-latency", "bcast"])
    ap.add_argument("--workers", required=True, help="comma-separated host:port list in rank order")
    ap.add_argument("--mode", default="disk")
    ap.add_argument("--kind", default="nvl")
    ap.add_argument("--src", default="0")
    ap.add_argument("--dst", default="1")
    ap.add_argument("--model-path", default="")
    ap.add_argument("--model-name", default="")
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--script", default="", help="repl: read commands from this file instead of stdin")
    a = ap.parse_args(argv)

    async def go():
        stubs = [WorkerStub(u) for u in a.workers.split(",")]
        try:
            if a.cmd == "repl":
                lines = iter(open(a.script).read().splitlines()) if a.script else None
                await Repl(stubs).loop(lines)
            elif a.cmd == "load-latency":
                print(json.dumps(await load_latency(stubs, a.mode, src=int(a.src), dst=int(a.dst), model_name=a.model_name,
                                                    model_path=a.model_path, prompt_len=a.prompt_len)))
            else:
                print(json.dumps(await benchmark_broadcast(stubs, a.kind, [int(x) for x in a.src.split(",")],
                                                           [int(x) for x in a.dst.split(",")], a.repeats)))
        finally:
            for s in stubs:
                await s.close()
    asyncio.run(go())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
