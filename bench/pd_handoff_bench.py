"""Prefill -> decode hand-off between two GPU workers: migration of all layers after the pass against the
layer-progressive migration that pushes each layer's KV while the next layers run.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29561 \
        bench/pd_handoff_bench.py [--model llama3_8b] [--prompt-len 2048] [--prompts 2] [--push-ctas 16 4] [--json out.json]

Rank 0 is the prefill worker, rank 1 the decode worker; both are `GpuBackend`s called directly (no gRPC in between, so
the two extra round trips of the ordinary path are not in its figure: the router learns that the prefill ended, then
issues Migrate and Immigrate).  Per iteration both ranks leave a host barrier together; the figure of merit is the
host time from that barrier until `immigrate` returns on the decode worker, i.e. until the batch can join a decode
step there.  Random-init weights of the model's shape, synthetic prompts, bf16.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from blitz_scale_b200 import ops  # noqa: E402
from blitz_scale_b200.pb.schema import pb  # noqa: E402
from blitz_scale_b200.worker.gpu_backend import GpuBackend  # noqa: E402


def make_batch(bid: int, prompts) -> "pb.Batch":
    b = pb.Batch(id=bid, size=len(prompts), max_tokens=sum(len(p) + 64 for p in prompts))
    for i, p in enumerate(prompts):
        r = b.requests.add()
        r.id, r.inputs, r.prefill_logprobs, r.top_n_tokens = bid * 64 + i, "", False, 0
        r.input_tokens.extend(p)
        r.stopping_parameters.max_new_tokens = 8
        r.stopping_parameters.ignore_eos_token = True
    return b


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3_8b")
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--prompts", type=int, default=2)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--push-ctas", type=int, nargs="+", default=[16], help="CTAs per layer of the progressive push")
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    assert world == 2, "one prefill worker and one decode worker"
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    host = dist.new_group(backend="gloo")
    ps = 64
    pages = 2 * a.prompts * (a.prompt_len // ps + 2) + 8
    backend = GpuBackend(rank, world, a.model, num_pages=pages, page_size=ps, max_batch=max(8, a.prompts),
                         max_batch_tokens=8192, ready=True, seed=0)
    backend.thread_init()
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, backend.cfg.vocab, (a.prompt_len,), generator=g).tolist() for _ in range(a.prompts)]
    progressive = pb.PREFILL_CASE_NORMAL | pb.PREFILL_CASE_MIGRATE_PROGRESSIVE
    out = {"kind": "pd_handoff", "model": a.model, "prompt_len": a.prompt_len, "prompts": a.prompts, "iters": a.iters}
    bid = 0
    modes = ["after_the_pass"] + [f"progressive_{c}ctas" for c in a.push_ctas]
    for mode in modes:
        total, prefill = [], []
        if mode.startswith("progressive"):
            backend.progressive_push_ctas = int(mode.split("_")[1][:-4])
        for it in range(a.warmup + a.iters):
            bid += 1
            batch = make_batch(bid, prompts)
            torch.cuda.synchronize()
            dist.barrier(group=host)
            t0 = time.perf_counter()
            t_pf = t0
            if rank == 0:
                if mode.startswith("progressive"):
                    backend.prefill(batch, progressive, None, [1])
                    t_pf = time.perf_counter()
                else:
                    backend.prefill(batch, pb.PREFILL_CASE_NORMAL, None, [])
                    t_pf = time.perf_counter()
                    dist.barrier(group=host)          # the prefill has answered: both halves of the migration are issued
                    backend.migrate(batch, [0], [1])
            else:
                if not mode.startswith("progressive"):
                    dist.barrier(group=host)
                backend.immigrate(batch, [0], [1])
            t1 = time.perf_counter()
            if rank == 1:
                backend.clear_cache(bid)
            if it >= a.warmup:
                total.append((t1 - t0) * 1e3)
                prefill.append((t_pf - t0) * 1e3)
        ops.check_status()
        both = [None, None]
        dist.all_gather_object(both, {"total": total, "prefill": prefill}, group=host)
        out[f"{mode}_prefill_ms"] = statistics.median(both[0]["prefill"])
        out[f"{mode}_source_done_ms"] = statistics.median(both[0]["total"])
        out[f"{mode}_resident_on_decode_ms"] = statistics.median(both[1]["total"])
    # what the hand-off adds to the pass itself (the pass timed without any push beside it)
    for mode in modes:
        out[f"handoff_{mode}_ms"] = out[f"{mode}_resident_on_decode_ms"] - out["after_the_pass_prefill_ms"]
    if rank == 0:
        print(json.dumps(out), flush=True)
        if a.json:
            os.makedirs(os.path.dirname(os.path.abspath(a.json)), exist_ok=True)
            json.dump(out, open(a.json, "w"), indent=1)
    backend.close()
    dist.barrier(group=host)
    from blitz_scale_b200.parallel.teardown import shutdown
    shutdown([backend])


if __name__ == "__main__":
    main()
