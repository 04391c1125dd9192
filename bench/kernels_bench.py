"""Single-GPU kernel microbenchmarks: tcgen05 GEMM vs torch.matmul (cuBLAS), decode attention vs the HBM roofline.

Timing: CUDA events on the launching stream, >= 3 warm-up iterations.  Cold-cache behaviour is obtained by
rotating every timed launch over enough independent copies of its large operand (weights, KV pool) that the
copies together exceed twice the 126 MB L2 ("inputs larger than L2"); attention cases whose KV pool alone is
far larger than L2 just repeat.  A write-flush of L2 is deliberately not used for the GEMMs: the dirty lines
it leaves behind are written back during the timed kernel and halve the DRAM bandwidth it sees.  Peaks come from MEASURED_PEAKS.json at the repository
root when present, else the fallback figures (6.65 TB/s, 1.59 PFLOP/s).

    python bench/kernels_bench.py [--quick] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from blitz_scale_b200 import ops  # noqa: E402


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def timeit(fn, iters=7, warmup=3, copies=1):
    """fn(i) runs the launch on operand copy i % copies.

    One pass over all copies is captured in a CUDA graph and replayed, so the host cost of a launch (tens of
    microseconds through Python) never sits inside the timed interval even for 10 us kernels; the reported
    time is (event time of one replay) / (launches in the graph), median over `iters` replays, and therefore
    includes the device-side launch gap between dependent kernels, as inside a model step."""
    n = max(copies, 4)
    for i in range(max(warmup, n)):
        fn(i % copies)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n):
            fn(i % copies)
    g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) / n)
    times.sort()
    return times[len(times) // 2] * 1e-3


def n_copies(nbytes: int) -> int:
    return max(2, -(-(256 << 20) // max(1, nbytes)) + 1)


def bench_gemm(shapes, out):
    hbm, flops_peak, src = peaks()
    for (M, N, K, epi) in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        bcols = 2 * N if epi == "silu_mul" else N
        nc = n_copies(K * bcols * 2)
        bs = [torch.randn(K, bcols, device="cuda", dtype=torch.bfloat16) * K ** -0.5 for _ in range(nc)]
        r = torch.randn(M, N, device="cuda", dtype=torch.bfloat16) if epi == "add" else None
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        extra = {}
        if M <= 256:
            # decode sizes: weight-streaming kernel as the model runs it (weights static -> prefetched under the
            # previous kernel's tail), the same without that promise, and the general tiled kernel
            t = timeit(lambda i: ops.gemm(a, bs[i], out=c, residual=r, epilogue=epi, static_b=True), copies=nc)
            t_ns = timeit(lambda i: ops.gemm(a, bs[i], out=c, residual=r, epilogue=epi), copies=nc)
            t_gen = timeit(lambda i: ops.gemm(a, bs[i], out=c, residual=r, epilogue=epi, decode_path=False), copies=nc)
            extra = dict(kernel="decode", us_no_prefetch=t_ns * 1e6, us_general_kernel=t_gen * 1e6)
        else:
            t = timeit(lambda i: ops.gemm(a, bs[i], out=c, residual=r, epilogue=epi), copies=nc)
        ops.check_status()
        cref = torch.empty(M, bcols, device="cuda", dtype=torch.bfloat16)
        t_ref = timeit(lambda i: torch.matmul(a, bs[i], out=cref), copies=nc)
        fl = 2.0 * M * bcols * K
        by = 2.0 * (M * K + K * bcols + M * N)
        roof = max(fl / flops_peak, by / hbm)
        row = dict(kind="gemm", M=M, N=N, K=K, epilogue=epi, us=t * 1e6, cublas_us=t_ref * 1e6,
                   tflops=fl / t / 1e12, gbs=by / t / 1e9, roofline_frac=roof / t, vs_cublas=t_ref / t, peaks=src,
                   **extra)
        out.append(row)
        print(json.dumps(row), flush=True)


def bench_decode_attn(cases, out):
    hbm, _, src = peaks()
    for (B, ctx, qh, kvh, hd, page, splits) in cases:
        npg = (ctx + page - 1) // page
        total = B * npg
        kv = torch.randn(total, 2, page, kvh, hd, device="cuda", dtype=torch.bfloat16)
        idx = torch.randperm(total, device="cuda").to(torch.int32)
        indptr = (torch.arange(B + 1, device="cuda") * npg).to(torch.int32)
        last = torch.full((B,), ctx - (npg - 1) * page, device="cuda", dtype=torch.int32)
        q = torch.randn(B, qh * hd, device="cuda", dtype=torch.bfloat16)
        o = torch.empty(B, qh * hd, device="cuda", dtype=torch.bfloat16)
        ws = torch.empty(max(1, ops.attn_decode_workspace_bytes(B, qh, hd, splits)), dtype=torch.uint8, device="cuda")
        nc = n_copies(kv.numel() * 2)
        kvs = [kv] + [torch.randn_like(kv) for _ in range(nc - 1)] if kv.numel() * 2 < (512 << 20) else [kv]
        t = timeit(lambda i: ops.attn_decode(q, kvs[i], idx, indptr, last, q_heads=qh, kv_heads=kvh, head_dim=hd,
                                             page_size=page, num_splits=splits, workspace=ws, out=o), copies=len(kvs))
        ops.check_status()
        by = 2.0 * B * ctx * 2 * kvh * hd
        row = dict(kind="attn_decode", B=B, ctx=ctx, q_heads=qh, kv_heads=kvh, page=page, splits=splits, us=t * 1e6,
                   gbs=by / t / 1e9, hbm_frac=by / t / hbm, peaks=src)
        out.append(row)
        print(json.dumps(row), flush=True)


def bench_prefill_attn(cases, out):
    _, flops_peak, src = peaks()
    for (B, n, qh, kvh) in cases:
        hd = 128
        qkv = torch.randn(B * n, (qh + 2 * kvh) * hd, device="cuda", dtype=torch.bfloat16)
        o = torch.empty(B * n, qh * hd, device="cuda", dtype=torch.bfloat16)
        fl = 4.0 * B * qh * hd * n * n / 2
        # through the paged pool (persistent grid, two ping-ponged query tiles per work item, keys and values read from
        # 64-token pages), with and without a share of the exponentials on the FMA pipe
        ps = 64
        npg = n // ps
        pool = torch.randn(B * npg, 2, ps, kvh, hd, device="cuda", dtype=torch.bfloat16)
        ids = torch.randperm(B * npg, device="cuda").to(torch.int32)
        work = ops.prefill_work_list([n] * B, [n] * B, ps, "cuda")
        for poly in (False, True):
            t = timeit(lambda i: ops.attn_prefill_paged(qkv, pool, ids, work, q_heads=qh, kv_heads=kvh, head_dim=hd,
                                                         page_size=ps, out=o, poly_exp=poly))
            ops.check_status()
            row = dict(kind="attn_prefill_paged", B=B, n=n, q_heads=qh, kv_heads=kvh, poly_exp=poly, us=t * 1e6,
                       tflops=fl / t / 1e12, frac_of_gemm_peak=fl / t / flops_peak, peaks=src)
            out.append(row)
            print(json.dumps(row), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", default="", help="run only one group: gemm, decode_attn, prefill_attn")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    out = []
    # Llama-3-8B layer GEMMs at decode (M = batch) and prefill (M = tokens) sizes
    ms = [16, 128, 256] if args.quick else [16, 64, 128, 256, 1024, 4096, 8192]
    shapes = []
    for M in ms:
        shapes += [(M, 6144, 4096, "store"), (M, 4096, 4096, "add"), (M, 14336, 4096, "silu_mul"),
                   (M, 4096, 14336, "add")]
    shapes += [(256, 128256, 4096, "store"), (8192, 8192, 8192, "store")]
    if args.only in ("", "gemm"):
        bench_gemm(shapes, out)
    cases = [(64, 1024, 32, 8, 128, 64, 1), (256, 1024, 32, 8, 128, 64, 1), (256, 1024, 32, 8, 128, 16, 1),
             (8, 8192, 32, 8, 128, 64, 8), (1, 16384, 32, 8, 128, 64, 32)]
    if args.only in ("", "decode_attn"):
        bench_decode_attn(cases[:2] if args.quick else cases, out)
    if args.only in ("", "prefill_attn"):
        bench_prefill_attn([(4, 2048, 32, 8)] if args.quick else [(8, 512, 32, 8), (4, 2048, 32, 8), (1, 8192, 32, 8)], out)
    if args.json:
        os.makedirs(os.path.dirname(os.path.abspath(args.json)), exist_ok=True)
        json.dump(out, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
