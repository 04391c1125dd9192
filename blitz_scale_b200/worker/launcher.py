"""Worker launcher: one process per GPU, gRPC port = base port + rank.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m blitz_scale_b200.worker.launcher \
        --model-name llama3_8b --config cluster.json --port 50051 -TP 1 --num-total-blocks 4096

Flags follow the reference's worker CLI (src/server/args.h:39-97: --model-path --model-name -T -V -P --host
--config --port -PP -TP -A --num-total-blocks --log-dir --time-to-live) and the cluster JSON it reads
({init_states, replicas, machines}, src/server/disaggregate.cc:31-50, :97-120).  Ranks whose initial state is
not "Inactive" start with parameters marked ready (random-init weights, as in the reference where active ranks
never load from disk at boot, src/blitz/stub.h:284-287); inactive ranks wait for a broadcast or LoadParams.
torch.distributed (TCP store + NCCL) replaces the MPI bootstrap; NUMA binding is left to the process launcher.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import logging
import os
import signal
import sys

import torch
import torch.distributed as dist


def parse_args(argv=None):
    ap = argparse.ArgumentParser("blitz-worker")
    ap.add_argument("--model-path", default="")
    ap.add_argument("--model-name", default="llama3_8b")
    ap.add_argument("-T", "--tokenizer", default="", help="tokenizer.json: text of generated tokens, which the worker "
                    "needs to apply the stop sequences of a request (without it they match the <id> text of its generations)")
    ap.add_argument("-V", "--vocab-json", default="")
    ap.add_argument("-P", "--precision", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--config", required=True, help="cluster JSON: init_states, replicas, machines")
    ap.add_argument("--port", type=int, default=50051)
    ap.add_argument("-PP", "--pipeline-parallel", type=int, default=1)
    ap.add_argument("-TP", "--tensor-parallel", type=int, default=1)
    ap.add_argument("-A", "--activation-slots", type=int, default=4)
    ap.add_argument("--num-total-blocks", type=int, default=4096)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--max-batch-size", type=int, default=256)
    ap.add_argument("--max-batch-tokens", type=int, default=8192)
    ap.add_argument("--log-dir", default="")
    ap.add_argument("--time-to-live", type=float, default=0.0, help="exit after this many seconds (0 = run until signalled)")
    ap.add_argument("--multimem", action="store_true", help="multicast parameter stores through NVLS when available")
    ap.add_argument("--ibv-rate", type=int, default=0, help="accepted for command-line compatibility; an NVSwitch box has "
                    "no NIC to rate-limit")
    ap.add_argument("--no-fused-tp", action="store_true", help="tensor-parallel layers through NCCL all-reduce instead of the "
                    "fused peer-memory kernels (needed for live execution with tp > 1)")
    ap.add_argument("--precapture-graphs", action="store_true", help="capture the decode CUDA graphs of every batch bucket "
                    "at start-up instead of on first use")
    ap.add_argument("--eos-token-id", type=int, default=None, help="end-of-sequence token id (default: the model "
                    "family's; -1: none).  A request stops there unless it sets ignore_eos_token")
    ap.add_argument("--no-numa-bind", action="store_true", help="do not pin host threads to the CPU cores next to the GPU")
    return ap.parse_args(argv)


def main(argv=None) -> int:
    a = parse_args(argv)
    if a.pipeline_parallel != 1:
        raise SystemExit("static pipeline parallelism is not supported (the reference asserts pp == 1 as well)")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    try:        # before anything touches a GPU: a description the job cannot run with ends it with one line
        from ..models.config import get_config
        from ..utils.cluster_config import check_cluster
        cluster = json.load(open(a.config))
        states = check_cluster(cluster, a.tensor_parallel)
        get_config(a.model_name)
        if a.tokenizer and not os.path.isfile(a.tokenizer):
            raise ValueError(f"tokenizer file {a.tokenizer} does not exist")
        if len(states) != world:
            raise ValueError(f"cluster config lists {len(states)} ranks, world size is {world}")
    except (OSError, ValueError, KeyError) as e:
        raise SystemExit(f"worker launcher: {e}")
    if a.log_dir:
        os.makedirs(a.log_dir, exist_ok=True)
        f = open(os.path.join(a.log_dir, f"rank-{rank}.log"), "a", buffering=1)
        os.dup2(f.fileno(), 1)
        os.dup2(f.fileno(), 2)
    logging.basicConfig(level=os.environ.get("LOG_LEVEL", "INFO").upper(), format="%(asctime)s %(name)s %(message)s")
    torch.cuda.set_device(local)
    if not a.no_numa_bind:
        # host threads, pinned staging buffers and the disk loader should live on the GPU's NUMA node (the reference
        # binds ranks 0-3 / 4-7 to node 0 / 1, src/server/disaggregate.cc)
        from ..utils.topology import bind_to_gpu_cpus
        cpus = bind_to_gpu_cpus(local)
        logging.getLogger("blitz.worker").info("rank %d bound to %d CPU cores next to GPU %d", rank, len(cpus), local)
    tp = a.tensor_parallel
    tp_group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        if tp > 1:
            for r0 in range(0, world, tp):
                g = dist.new_group(list(range(r0, r0 + tp)))
                if r0 <= rank < r0 + tp:
                    tp_group = g
    from .gpu_backend import GpuBackend
    from .service import serve
    backend = GpuBackend(rank, world, a.model_name, tp=tp, num_pages=a.num_total_blocks, page_size=a.page_size,
                         max_batch=a.max_batch_size, max_batch_tokens=a.max_batch_tokens,
                         ready=states[rank] != "Inactive", tp_group=tp_group, model_path=a.model_path,
                         seed=0, use_multimem=a.multimem, fused_tp=not a.no_fused_tp, precapture=a.precapture_graphs,
                         eos_token=a.eos_token_id, tokenizer_path=a.tokenizer)
    urls = [f"{a.host}:{a.port + r}" for r in range(world)]

    async def run():
        stop = asyncio.Event()
        loop = asyncio.get_running_loop()
        for sig in (signal.SIGINT, signal.SIGTERM, signal.SIGQUIT):
            loop.add_signal_handler(sig, stop.set)
        if a.time_to_live > 0:
            loop.call_later(a.time_to_live, stop.set)
        await serve(backend, a.host, a.port + rank, urls=urls, stop_event=stop)

    asyncio.run(run())
    backend.close()
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        from ..parallel.teardown import shutdown
        shutdown([backend])      # graphs, then symmetric regions, then process groups, with barriers in between
    return 0


if __name__ == "__main__":
    sys.exit(main())
