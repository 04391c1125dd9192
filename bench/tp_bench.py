"""Microbenchmark of the fused tensor-parallel pair against NCCL + torch.matmul.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node TP --master-addr 127.0.0.1 --master-port 29541 \
        bench/tp_bench.py [--json out.json]

For M in {16, 256, 4096} and K = N = 8192 (per-rank K = 8192 / TP for the row-parallel GEMM, per-rank
N = 8192 / TP for the column-parallel one) it times one row-parallel -> column-parallel hand-off:

  fused   : gemm_rs (tcgen05 GEMM, epilogue pushes partial rows to their owner over NVLink)
            -> reduce_norm (owner sums, adds residual, RMSNorm, pushes rows to every rank)
            -> ag_gemm (tcgen05 GEMM whose TMA producer waits for the gathered rows)
  nccl    : torch.matmul -> reduce_scatter -> add + rms norm (torch) -> all_gather -> torch.matmul

Timing: one pass captured in a CUDA graph and replayed (no host launch cost inside the interval), CUDA events,
barrier + synchronize on both sides, max over ranks.  Roofline per GPU: the slower of the two GEMMs' FLOPs at
the measured cuBLAS bf16 peak and the bytes every GPU must send over NVLink at 770 GB/s measured (900 nominal).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from baseline import nccl_paths  # noqa: E402
from blitz_scale_b200 import ops  # noqa: E402
from blitz_scale_b200.parallel.tp import FusedTP  # noqa: E402


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["bf16_tflops"] * 1e12, "measured"
    return 1.59e15, "fallback"


def graph_time(fn, iters=5):
    fn()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    best = None
    for _ in range(iters + 1):
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) * 1e-3], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        best = float(t) if best is None else min(best, float(t))
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--small-only", action="store_true", help="only the decode-size all-reduce + add + norm comparison")
    a = ap.parse_args()
    rank, tp = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    H = a.hidden
    flops_peak, src = peaks()
    fused = FusedTP(dist.group.WORLD, H, 4096)
    out = []
    for M in ((16, 256, 4096) if not a.small_only else ()):
        torch.manual_seed(rank)
        x = torch.randn(M, H // tp, device="cuda", dtype=torch.bfloat16)             # row-parallel input (K sharded)
        w_row = torch.randn(H // tp, H, device="cuda", dtype=torch.bfloat16) * H ** -0.5
        w_col = torch.randn(H, H // tp, device="cuda", dtype=torch.bfloat16) * H ** -0.5
        norm_w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        rpr = M // tp
        res = torch.randn(rpr, H, device="cuda", dtype=torch.bfloat16)
        y = torch.empty(M, H // tp, device="cuda", dtype=torch.bfloat16)

        def run_fused():
            exp = fused.gemm_rs(x, w_row, 0)
            fused.reduce_norm(0, exp, rpr, res, norm_w, 1, 1e-5)
            fused.ag_gemm(1, M, w_col, y)

        def run_nccl():
            part = nccl_paths.matmul_reduce_scatter(x, w_row)
            r2 = part + res
            n = (r2.float() * torch.rsqrt(r2.float().pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16) * norm_w
            return nccl_paths.allgather_matmul(n, w_col)

        # numerics of the fused chain against the NCCL chain (same inputs, residual restored in between)
        res0 = res.clone()
        run_fused()
        torch.cuda.synchronize()
        ops.check_status()
        res.copy_(res0)
        ref = run_nccl()
        err = float((y.float() - ref.float()).norm() / ref.float().norm())
        t_f = graph_time(run_fused)
        ops.check_status()
        # where the fused chain spends its time: events between the three launches (eager, so each stage carries a
        # host launch; meaningful for the large case)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        dist.barrier()
        torch.cuda.synchronize()
        ev[0].record()
        exp = fused.gemm_rs(x, w_row, 0)
        ev[1].record()
        fused.reduce_norm(0, exp, rpr, res, norm_w, 1, 1e-5)
        ev[2].record()
        fused.ag_gemm(1, M, w_col, y)
        ev[3].record()
        torch.cuda.synchronize()
        stages = torch.tensor([ev[i].elapsed_time(ev[i + 1]) * 1e3 for i in range(3)], device="cuda", dtype=torch.float64)
        dist.all_reduce(stages, op=dist.ReduceOp.MAX)
        stages = [round(float(v), 1) for v in stages]
        t_n = graph_time(run_nccl)
        fl = 2.0 * M * H * (H // tp) * 2            # two GEMMs per rank
        wire = (M * H * 2) * (tp - 1) / tp * 2      # reduce-scatter out + all-gather out, bytes each GPU sends
        roof = max(fl / flops_peak, wire / 770e9)
        if rank == 0:
            row = dict(kind="tp_pair", tp=tp, M=M, K=H, N=H, fused_us=t_f * 1e6, nccl_us=t_n * 1e6, speedup=t_n / t_f,
                       roofline_us=roof * 1e6, fused_frac_of_roofline=roof / t_f, rel_err_vs_nccl=err, peaks=src,
                       stage_us_gemm_rs_reduce_norm_ag_gemm=stages)
            out.append(row)
            print(json.dumps(row), flush=True)
    # Decode-size all-reduce + residual add + RMSNorm: the switch-reduced one-kernel form, the one-shot push form
    # followed by the add+norm kernel, and NCCL all-reduce followed by the add+norm kernel.  Eight dependent
    # rounds per graph replay, so the time per round includes the launch gap a layer loop sees.
    for Hs in (4096, 8192):
        f2 = fused if Hs == H else FusedTP(dist.group.WORLD, Hs, 1024)
        for M in (16, 256, 1024):
            nw = torch.ones(Hs, device="cuda", dtype=torch.bfloat16)
            xin = torch.randn(M, Hs, device="cuda", dtype=torch.bfloat16)
            resid = torch.zeros(M, Hs, device="cuda", dtype=torch.bfloat16)
            tmp = torch.empty(M, Hs, device="cuda", dtype=torch.bfloat16)
            normed = torch.empty(M, Hs, device="cuda", dtype=torch.bfloat16)
            rounds = 8

            def run_switch():
                for _ in range(rounds):
                    f2.next_partial(M).copy_(xin)
                    f2.ar_add_norm(M, nw, 1e-5)

            def run_oneshot():
                for _ in range(rounds):
                    tmp.copy_(xin)
                    f2.allreduce_oneshot(tmp, tmp)
                    ops.add_rms_norm(tmp, resid, nw, 1e-5, out=normed)

            def run_nccl2():
                for _ in range(rounds):
                    tmp.copy_(xin)
                    dist.all_reduce(tmp)
                    ops.add_rms_norm(tmp, resid, nw, 1e-5, out=normed)

            def run_copy():
                for _ in range(rounds):
                    tmp.copy_(xin)

            row = dict(kind="ar_add_norm", tp=tp, M=M, H=Hs, has_switch=bool(f2.has_mc))
            t_c = graph_time(run_copy) / rounds
            f2.reset_allreduce_parity()
            if f2.has_mc:
                f2.res(M).zero_()
                row["switch_us"] = (graph_time(run_switch) / rounds - t_c) * 1e6
            f2.reset_allreduce_parity()
            row["oneshot_us"] = (graph_time(run_oneshot) / rounds - t_c) * 1e6
            row["nccl_us"] = (graph_time(run_nccl2) / rounds - t_c) * 1e6
            ops.check_status()
            if rank == 0:
                out.append(row)
                print(json.dumps(row), flush=True)
    if rank == 0 and a.json:
        os.makedirs(os.path.dirname(os.path.abspath(a.json)), exist_ok=True)
        json.dump(out, open(a.json, "w"), indent=1)
    dist.barrier()
    sys.stdout.flush()
    from blitz_scale_b200.parallel.teardown import shutdown
    shutdown([fused])      # graphs (local to the timing helpers, already gone), symmetric regions, process groups


if __name__ == "__main__":
    main()
