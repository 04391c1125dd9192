"""Prefill throughput of one tensor-parallel replica: fused peer-memory runner against the NCCL all-reduce runner.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node TP --master-addr 127.0.0.1 --master-port 29551 \
        bench/tp_prefill_bench.py [--model mistral_24b] [--prompt-len 2048] [--prompts 4] [--json out.json]

Every rank builds the same engine twice (fused_tp on / off, random-init weights of the model's shape, same seed), prefills
`--prompts` prompts of `--prompt-len` tokens in one pass (up to 8192 tokens) and reports prompt tokens per second.  The
fused runner takes the switch-reduced path (plain GEMMs, then all-reduce + add + norm in one multimem kernel) where the
fabric reduces in the switch; `--pipeline` also times its row-sharded pipeline (GEMM -> reduce-scatter push, reduce +
norm + all-gather push, gated GEMM), which is what it uses elsewhere.  The other runner calls NCCL all-reduce after the
o-proj and down-proj GEMMs.

Timing: CUDA events around `iters` prefill passes (each on fresh KV pages of the same batch), after a warm-up pass,
barrier + synchronize on both sides, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from blitz_scale_b200 import ops  # noqa: E402
from blitz_scale_b200.models.llama import TPComm  # noqa: E402
from blitz_scale_b200.runtime import core  # noqa: E402
from blitz_scale_b200.runtime.engine import Engine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mistral_24b")
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--prompts", type=int, default=4)
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--pipeline", action="store_true", help="also time the fused runner's row-sharded pipeline")
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    rank, tp = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    comm = TPComm(dist.group.WORLD)
    tokens = a.prompt_len * a.prompts
    assert tokens <= 8192, "one pass takes at most 8192 tokens"
    ps = 64
    pages = (a.iters + 2) * a.prompts * (a.prompt_len // ps + 2) + 8
    out = {"kind": "tp_prefill", "tp": tp, "model": a.model, "prompt_len": a.prompt_len, "prompts": a.prompts}
    owners = []
    modes = [("fused", True, True), ("nccl", False, True)] + ([("fused_pipeline", True, False)] if a.pipeline else [])
    for name, fused, switch in modes:
        eng = Engine(a.model, num_pages=pages, page_size=ps, max_batch=max(a.prompts, 8), max_batch_tokens=8192, seed=0, tp=tp,
                     tp_rank=rank, comm=comm, fused_tp=fused, use_switch=switch)
        owners.append(eng)
        g = torch.Generator().manual_seed(5)
        prompts = [torch.randint(0, eng.cfg.vocab, (a.prompt_len,), generator=g).tolist() for _ in range(a.prompts)]

        def one_pass(bid):
            b = eng.new_batch(bid, [core.SeqSpec(bid * 100 + i, p, 2) for i, p in enumerate(prompts)])
            assert b is not None, "KV pool too small"
            toks = eng.prefill(b)
            b.clear()
            return toks

        first = one_pass(0)
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(a.iters):
            one_pass(1 + i)
        e.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([s.elapsed_time(e) * 1e-3], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ops.check_status()
        out[f"{name}_ms_per_pass"] = float(t) / a.iters * 1e3
        out[f"{name}_prompt_tokens_per_s"] = tokens * a.iters / float(t)
        out[f"{name}_first_tokens"] = first[:4]
        eng.release_graphs()
    out["fused_vs_nccl"] = out["nccl_ms_per_pass"] / out["fused_ms_per_pass"]
    if a.pipeline:
        out["fused_pipeline_vs_nccl"] = out["nccl_ms_per_pass"] / out["fused_pipeline_ms_per_pass"]
    if rank == 0:
        print(json.dumps(out), flush=True)
        if a.json:
            os.makedirs(os.path.dirname(os.path.abspath(a.json)), exist_ok=True)
            json.dump(out, open(a.json, "w"), indent=1)
    dist.barrier()
    from blitz_scale_b200.parallel.teardown import shutdown
    shutdown(owners)


if __name__ == "__main__":
    main()
