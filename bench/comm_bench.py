"""Multi-GPU microbenchmarks of the peer-memory data paths against the NCCL stand-in baseline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29531 \
        bench/comm_bench.py [--what multicast,kv_push] [--total-gb 4] [--json out.json]

(a) parameter multicast: one source streams `total-gb` of bf16 weights in 256 MB units to 1..N-1 destinations
    with peer stores, with NVLS multimem stores (if the fabric offers a multicast address), with two sources
    striping (Tanz-style), and with the NCCL chain (256 MB chunks) and `ncclBroadcast` baselines.
(b) KV-block push: prompt pages (16-token and 64-token pages, 8 KV heads x 128 dims, 32 layers) of 1K-64K
    tokens, pushed by the kv_push kernel vs one NCCL send/recv per (page, layer).

Timing: CUDA events on each rank's stream around the whole transfer (a destination's interval ends when its
last readiness flag has been observed by a device-side wait), barrier + synchronize on both sides, the
reported time is the max over ranks.  Link roofline: 900 GB/s nominal per direction per GPU; 770 GB/s measured
for a peer copy on B200 / NVSwitch.
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
from blitz_scale_b200.parallel import symm  # noqa: E402

LINK_NOMINAL = 900e9
LINK_MEASURED = 770e9


def timed(fn, rank_world, iters=3, warmup=1):
    """max-over-ranks event time of fn() (seconds), best of `iters`."""
    best = None
    for i in range(warmup + iters):
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) * 1e-3], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if i >= warmup:
            best = float(t) if best is None else min(best, float(t))
    return best


def bench_multicast(fab, rank, world, total_bytes, out, ctas_list=(64, 128, 256), dst_list=None):
    unit = 256 << 20
    n_units = max(1, total_bytes // unit)
    offs = [u * unit for u in range(n_units)]
    lens = [unit] * n_units
    epoch = [0]

    def run(n_dst, mode, ctas=64, n_src=1):
        dsts = list(range(n_src, n_src + n_dst))
        epoch[0] += n_src

        def go():
            if rank < n_src:
                fab.copy_units(fab.weights, dsts, offs, lens, symm.PARAM_FLAG0, stripe=rank, n_stripes=n_src,
                               use_multimem=(mode == "multimem"), num_ctas=ctas)
            elif rank in dsts:
                fab.wait_flag(symm.PARAM_FLAG0 + n_units - 1, go.want, budget_ms=20000)
        go.want = 0
        # flags are cumulative counters: compute the value after this run's iterations one at a time
        def once():
            go.want += n_src
            go()
        return timed(once, (rank, world))

    fab.reset_param_flags()
    torch.cuda.synchronize()
    dist.barrier()
    for n_dst in (dst_list or range(1, world)):
        for mode in ("peer_st", "multimem"):
            if mode == "multimem" and not fab.weights.mc_ptr:
                continue
            for ctas in ctas_list:
                fab.reset_param_flags()
                torch.cuda.synchronize()
                dist.barrier()
                t = run(n_dst, mode, ctas)
                ops.check_status()
                if rank == 0:
                    per_dst = total_bytes / t
                    row = dict(kind="multicast", mode=mode, n_dst=n_dst, ctas=ctas, gb=total_bytes / 1e9, ms=t * 1e3,
                               gbs_per_dst=per_dst / 1e9, frac_of_900=per_dst / LINK_NOMINAL,
                               frac_of_measured_770=per_dst / LINK_MEASURED, src_egress_gbs=(per_dst * (1 if mode == "multimem" else n_dst)) / 1e9)
                    out.append(row)
                    print(json.dumps(row), flush=True)
        if world >= 3 and n_dst <= world - 2:
            fab.reset_param_flags()
            torch.cuda.synchronize()
            dist.barrier()
            for mode, name in (("peer_st", "two_source_stripes"), ("multimem", "two_source_multimem")):
                if mode == "multimem" and not fab.weights.mc_ptr:
                    continue
                fab.reset_param_flags()
                torch.cuda.synchronize()
                dist.barrier()
                t = run(n_dst, mode, 128, n_src=2)
                ops.check_status()
                if rank == 0:
                    row = dict(kind="multicast", mode=name, n_dst=n_dst, ctas=128, gb=total_bytes / 1e9,
                               ms=t * 1e3, gbs_per_dst=total_bytes / t / 1e9, frac_of_900=total_bytes / t / LINK_NOMINAL,
                               frac_of_measured_770=total_bytes / t / LINK_MEASURED)
                    out.append(row)
                    print(json.dumps(row), flush=True)
        # baselines on the same buffer
        buf = fab.weights.local[:total_bytes]
        chain = list(range(0, n_dst + 1))
        t = timed(lambda: nccl_paths.chain_broadcast(buf, chain), (rank, world))
        if rank == 0:
            row = dict(kind="multicast", mode="nccl_chain_256MB", n_dst=n_dst, gb=total_bytes / 1e9, ms=t * 1e3,
                       gbs_per_dst=total_bytes / t / 1e9, frac_of_900=total_bytes / t / LINK_NOMINAL)
            out.append(row)
            print(json.dumps(row), flush=True)
    t = timed(lambda: nccl_paths.nccl_broadcast(fab.weights.local[:total_bytes], 0), (rank, world))
    if rank == 0:
        row = dict(kind="multicast", mode="nccl_broadcast", n_dst=world - 1, gb=total_bytes / 1e9, ms=t * 1e3,
                   gbs_per_dst=total_bytes / t / 1e9, frac_of_900=total_bytes / t / LINK_NOMINAL)
        out.append(row)
        print(json.dumps(row), flush=True)


def bench_kv_push(fab, rank, world, out, layers=32, kvh=8, hd=128):
    for page in (16, 64):
        page_bytes = 2 * page * kvh * hd * 2
        pages_total = fab.kv.nbytes // (layers * page_bytes)
        stride = pages_total * page_bytes
        kv3 = fab.kv.local[:layers * stride].view(layers, pages_total, page_bytes)
        for tokens in (1024, 4096, 16384, 65536):
            n = tokens // page
            if n * 2 > pages_total:
                continue
            g = torch.Generator().manual_seed(tokens + page)
            src_pages = torch.randperm(pages_total, generator=g)[:n].to(torch.int32).cuda()
            dst_pages = torch.randperm(pages_total, generator=g)[:n].to(torch.int32).cuda()
            count = [0]

            def push():
                count[0] += 1
                if rank == 0:
                    fab.kv_push(1, src_pages, dst_pages, 0, layers, page_bytes, stride, stride, pages_total,
                                pages_total, flag_slot=0)
                elif rank == 1:
                    fab.wait_flag(symm.KV_FLAG0 + layers - 1, count[0], budget_ms=20000)
            fab.flag_view()[symm.KV_FLAG0:symm.KV_FLAG0 + symm.MAX_LAYERS].zero_()
            torch.cuda.synchronize()
            dist.barrier()
            t = timed(push, (rank, world))
            ops.check_status()
            sp, dp = src_pages.tolist(), dst_pages.tolist()
            t_ref = timed(lambda: nccl_paths.kv_migrate_per_page(kv3, sp, dp, 0, 1, range(layers)), (rank, world), iters=1) \
                if tokens <= 16384 else float("nan")
            if rank == 0:
                by = n * page_bytes * layers
                row = dict(kind="kv_push", page=page, tokens=tokens, mb=by / 1e6, us=t * 1e6, gbs=by / t / 1e9,
                           frac_of_900=by / t / LINK_NOMINAL, nccl_per_page_us=t_ref * 1e6,
                           speedup_vs_nccl_per_page=t_ref / t)
                out.append(row)
                print(json.dumps(row), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="multicast,kv_push")
    ap.add_argument("--total-gb", type=float, default=4.0)
    ap.add_argument("--json", default="")
    ap.add_argument("--dst-list", default="", help="destination counts to run (default: 1..world-1)")
    ap.add_argument("--ctas", default="64,128,256")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    total = int(a.total_gb * (1 << 30)) // (256 << 20) * (256 << 20)
    kv_bytes = 32 * 8192 * 32768  # 8 GB pool: 8192 pages of 16 tokens (2048 pages of 64 tokens) x 32 layers
    fab = symm.PeerFabric(symm.FabricSizes(weight_bytes=total, kv_bytes=kv_bytes, mailbox_slots=1, mailbox_slot_bytes=1 << 20))
    if rank == 0:
        fab.weights.local.view(torch.int32).random_()
        print(json.dumps(dict(kind="info", world=world, multicast_ptr=bool(fab.weights.mc_ptr), total_gb=total / 1e9)), flush=True)
    out = []
    if "multicast" in a.what:
        bench_multicast(fab, rank, world, total, out, tuple(int(x) for x in a.ctas.split(",")),
                        [int(x) for x in a.dst_list.split(",") if x and int(x) < world] or None)
    if "kv_push" in a.what and world >= 2:
        bench_kv_push(fab, rank, world, out)
    if rank == 0 and a.json:
        os.makedirs(os.path.dirname(os.path.abspath(a.json)), exist_ok=True)
        json.dump(out, open(a.json, "w"), indent=1)
    dist.barrier()
    sys.stdout.flush()
    from blitz_scale_b200.parallel.teardown import shutdown
    shutdown([fab])      # graphs (local to the timing helpers, already gone), symmetric regions, process groups


if __name__ == "__main__":
    main()
