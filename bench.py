"""Headline benchmark: aggregate decode tokens/s of Llama-3-8B-shaped replicas (bf16, TP1) on N B200s.

    python bench.py --gpus N --steps K --warmup W          # N = 1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Each rank is one serving replica (the reference's unit of scaling: N independent instances behind
the router) holding a full random-init Llama-3-8B-shaped model and a decode batch of `--batch`
sequences whose `--ctx`-token prompts were prefilled through the engine before timing (synthetic
token ids).  One step = one decode iteration of the whole batch = `batch` tokens per replica.

Two numbers are reported:
  * value  : kernel-only.  K replays of the captured decode step, CUDA events on the launching
             stream, barrier + synchronize on both sides, max over ranks.
  * e2e    : K real `Engine.decode()` calls (the call a worker makes per DecodeV2 RPC): every step
             fills the pinned staging buffer, copies it host->device, replays the step, copies the
             sampled tokens device->host, updates the page tables on the host.
Per step each replica touches all weights (~15 GB) and its KV working set (batch x ctx x 128 KB),
far beyond the 126 MB L2, so no explicit flush is needed between iterations.

`vs_baseline`: the reference publishes no numbers and cannot be built here, so the anchor is a stand-in
measured in the same run, before the product's own numbers and on the same GPUs: the reference's decode
iteration on cuBLAS GEMMs and a library paged decode attention (`baseline/decode_step.py`), same model
shape, batch, context, CUDA-graph timing and end-to-end definition.  `--impl baseline` prints that arm
alone; `--no-baseline` skips it (vs_baseline is then null).  With --tp > 1 the stand-in is the NCCL
all-reduce runner (`--no-fused-tp`), which this script does not run by itself.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def reference_arm():
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is a C++/Rust/CMake project with empty submodules: pip reports "
                                     "'Directory is not installable. Neither setup.py nor pyproject.toml found'"}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read-only)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        sm = sorted(float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for i, n in enumerate(names):
                if len(r) > 4 + i and r[4 + i].lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None,
                "reasons": sorted(reasons), "samples": len(self.rows)}


def measure_tp_replica(args, world, rank, barrier, owners):
    """One replica spanning all `world` GPUs (tensor parallel), decode step timed on the device for the fused
    peer-memory runner and for the NCCL all-reduce runner: a number in the record that depends on NVLink."""
    import torch
    import torch.distributed as dist
    from blitz_scale_b200.models.llama import TPComm
    from blitz_scale_b200.runtime import core
    from blitz_scale_b200.runtime.engine import Engine, _BUCKETS
    from blitz_scale_b200 import ops
    B, ctx, ps = args.batch, args.ctx, args.page_size
    steps, warmup = args.steps, args.warmup
    comm = TPComm(dist.group.WORLD)
    out = {"tp": world, "model": args.model, "batch": B, "seq_len": ctx}
    for name, fused in (("fused", True), ("nccl", False)):
        eng = Engine(args.model, num_pages=B * ((ctx + warmup + steps + 16 + ps) // ps + 1) + 8, page_size=ps,
                     max_batch=max(B, 8), max_batch_tokens=8192, seed=0, tp=world, tp_rank=rank, comm=comm,
                     fused_tp=fused, oneshot_max_rows=args.oneshot_max_rows)
        owners.append(eng)
        g = torch.Generator().manual_seed(77)          # every rank of the replica sees the same prompts
        per, batch, bid = max(1, 8192 // ctx), None, 0
        for s0 in range(0, B, per):
            n = min(per, B - s0)
            nb = eng.new_batch(bid, [core.SeqSpec(s0 + i, torch.randint(0, eng.cfg.vocab, (ctx,), generator=g).tolist(),
                                                  warmup + steps + 12) for i in range(n)])
            bid += 1
            eng.prefill(nb)
            if batch is None:
                batch = nb
            else:
                batch.extend(nb)
        for _ in range(warmup):
            eng.decode(batch)
        Bp = min(b for b in _BUCKETS if b >= B)
        splits = eng.choose_splits(Bp, batch.max_seq_len())
        graph = eng._graphs.get((Bp, splits)) or eng._capture(Bp, splits)
        for _ in range(warmup):
            graph.replay()
        barrier()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record()
        for _ in range(steps):
            graph.replay()
        k1.record()
        barrier()
        t = torch.tensor([k0.elapsed_time(k1) * 1e-3], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ops.check_status()
        out[f"{name}_ms_per_step"] = float(t[0]) / steps * 1e3
        out[f"{name}_tokens_per_s"] = B * steps / float(t[0])
        del graph, batch
        eng.release_graphs()
    out["fused_vs_nccl"] = out["nccl_ms_per_step"] / out["fused_ms_per_step"]
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="llama3_8b")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree of every replica (GPUs / tp replicas)")
    ap.add_argument("--oneshot-max-rows", type=int, default=1024, help="tp > 1: steps of at most this many rows use the one-shot "
                    "peer-memory all-reduce instead of the reduce-scatter / all-gather pipeline")
    ap.add_argument("--no-fused-tp", action="store_true", help="tp > 1: NCCL all-reduce layers (the baseline) instead of the "
                    "fused peer-memory kernels")
    ap.add_argument("--no-baseline", action="store_true", help="do not run the stand-in baseline arm first")
    ap.add_argument("--no-extra-tp", action="store_true", help="N > 1: do not add the tensor-parallel record "
                    "(one replica over all N GPUs, fused peer-memory runner against the NCCL runner)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from blitz_scale_b200.runtime.engine import Engine
    from blitz_scale_b200.runtime import core
    from blitz_scale_b200 import ops

    B, ctx, ps = args.batch, args.ctx, args.page_size

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(*vals):
        if world == 1:
            return list(vals)
        t = torch.tensor(list(vals), device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t]

    # ---------------- stand-in baseline arm (library kernels only), same GPUs, before the product's own run
    base = None
    if args.impl == "baseline" or (not args.no_baseline and args.tp <= 1):
        r, err = None, ""
        try:
            from baseline import decode_step
            r = decode_step.run(args.model, B, ctx, args.steps, args.warmup, torch.device("cuda", local),
                                seed=rank, barrier=barrier)
        except Exception as e:  # noqa: BLE001  (the product's number must not depend on the stand-in)
            err = f"{type(e).__name__}: {e}"[:300]
        # every rank takes part in the reduction whether or not its own arm worked
        dev_b, e2e_b, failed = max_over_ranks(r["dev_s"] if r else 0.0, r["e2e_s"] if r else 0.0, 0.0 if r else 1.0)
        if r is not None and failed == 0.0:
            tokens_b = world * B * args.steps
            base = {"value": tokens_b / dev_b, "ms_per_step": dev_b / args.steps * 1e3,
                    "e2e_value": tokens_b / e2e_b, "e2e_ms_per_step": e2e_b / args.steps * 1e3,
                    "gemm": "cuBLAS (torch.matmul / addmm)", "attention": r["attention"], "kv_block": r["page"],
                    "h2d_bytes_per_step": r["h2d_bytes_per_step"], "d2h_bytes_per_step": r["d2h_bytes_per_step"]}
        else:
            base = {"error": err or "the arm failed on another rank"}
    if args.impl == "baseline":
        if rank == 0:
            ok = base is not None and "value" in base
            print(json.dumps({"impl": "baseline", "metric": "decode_tokens_per_s", "value": base["value"] if ok else None,
                              "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                              "ms_per_step": base["ms_per_step"] if ok else None, "higher_is_better": True,
                              "scaling": "weak", "dtype": "bf16", "data": "synthetic token ids, random-init weights",
                              "config": {"model": args.model, "global_batch": world * B, "seq_len": ctx,
                                         "parallelism": f"dp{world}"}, "detail": base}))
        if world > 1:
            from blitz_scale_b200.parallel.teardown import shutdown
            shutdown([])
        return 0

    total_steps = args.warmup + args.steps + 8
    pages_per_seq = (ctx + total_steps + ps) // ps + 1
    tp = max(1, args.tp)
    assert world % tp == 0, "--gpus must be a multiple of --tp"
    comm = None
    if tp > 1:
        from blitz_scale_b200.models.llama import TPComm
        group = None
        for r0 in range(0, world, tp):          # every rank creates every group, in the same order
            g_ = dist.new_group(list(range(r0, r0 + tp)))
            if r0 <= rank < r0 + tp:
                group = g_
        comm = TPComm(group)
    eng = Engine(args.model, num_pages=B * pages_per_seq + 8, page_size=ps, max_batch=max(B, 8),
                 max_batch_tokens=8192, seed=rank // tp, tp=tp, tp_rank=rank % tp, comm=comm,
                 fused_tp=not args.no_fused_tp, oneshot_max_rows=args.oneshot_max_rows)
    # synthetic prompts, prefilled through the engine in chunks that fit the activation workspace
    g = torch.Generator().manual_seed(1234 + rank // tp)      # the ranks of one replica see the same prompts
    per = max(1, 8192 // ctx)
    batch = None
    bid = 0
    for s0 in range(0, B, per):
        n = min(per, B - s0)
        specs = [core.SeqSpec(s0 + i, torch.randint(0, eng.cfg.vocab, (ctx,), generator=g).tolist(),
                              total_steps + 4) for i in range(n)]
        nb = eng.new_batch(bid, specs)
        assert nb is not None, "KV pool too small"
        bid += 1
        eng.prefill(nb)
        if batch is None:
            batch = nb
        else:
            batch.extend(nb)
    ops.check_status()

    # ---------------- e2e: real decode steps through the public engine API
    for _ in range(args.warmup):
        eng.decode(batch)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        eng.decode(batch)
    e1.record()
    barrier()
    e2e_s = max(time.perf_counter() - t0, e0.elapsed_time(e1) * 1e-3)
    h2d, d2h = eng.h2d_bytes, eng.d2h_bytes

    # ---------------- kernel-only: replay the captured step
    Bp = min(b for b in __import__("blitz_scale_b200.runtime.engine", fromlist=["_BUCKETS"])._BUCKETS if b >= B)
    splits = eng.choose_splits(Bp, batch.max_seq_len())
    graph = eng._graphs.get((Bp, splits)) or eng._capture(Bp, splits)
    for _ in range(args.warmup):
        graph.replay()
    barrier()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(args.steps):
        graph.replay()
    k1.record()
    barrier()
    dev_s = k0.elapsed_time(k1) * 1e-3
    clocks = sampler.stop() if rank == 0 else None
    ops.check_status()

    dev_s, e2e_s = max_over_ranks(dev_s, e2e_s)
    owners = [eng]
    extra = None
    if world > 1 and tp == 1 and not args.no_extra_tp and world in (2, 4, 8):
        del graph, batch
        eng.release_graphs()
        try:
            extra = {"tp": measure_tp_replica(args, world, rank, barrier, owners)}
        except Exception as e:  # noqa: BLE001  (the headline line must not depend on the extra record)
            extra = {"tp": {"error": f"{type(e).__name__}: {e}"[:300]}}
        graph = None
    if rank == 0:
        replicas = world // tp
        tokens = replicas * B * args.steps
        have_base = base is not None and "value" in base
        out = {
            "metric": "decode_tokens_per_s", "value": tokens / dev_s, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_s / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (tokens / dev_s) / base["value"] if have_base else None, "dtype": "bf16",
            "data": "synthetic token ids, random-init weights",
            "config": {"model": args.model, "global_batch": replicas * B, "seq_len": ctx,
                       "parallelism": f"dp{replicas}" + (f"xtp{tp}" + ("" if eng.fused is not None else "-nccl") if tp > 1 else ""),
                       "tp": tp, "page_size": ps, "l2": "per-step working set (weights + KV) >> 126 MB L2, no flush",
                       "timing": "CUDA events around K graph replays, max over ranks"},
            "clocks": clocks,
            "e2e": {"value": tokens / e2e_s, "unit": "tokens/s", "ms_per_step": e2e_s / args.steps * 1e3,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "vs_baseline": (tokens / e2e_s) / base["e2e_value"] if have_base else None},
            "baseline": ({**base, "what": "stand-in for the reference (not buildable here): its decode iteration on "
                          "library kernels, measured in this run on the same GPUs"} if base is not None else None),
            "gpu_launches": eng.decode_launch_count() * args.steps,
        }
        if extra is not None:
            out["extra"] = extra
        print(json.dumps(out))
    if world > 1:
        sys.stdout.flush()
        from blitz_scale_b200.parallel.teardown import shutdown
        graph = None
        shutdown(owners)     # graphs, then symmetric regions, then process groups, with barriers in between
    return 0


if __name__ == "__main__":
    sys.exit(main())
