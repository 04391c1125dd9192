"""Whole-system check on real GPUs: GPU workers (gRPC) + router runtime + trace, one rank per GPU.

Launched by test_multi_gpu.py through torch.distributed.run.  Every rank builds a GpuBackend on its GPU
(tiny Llama shape, same weight seed everywhere) and serves the RPC contract from a background thread;
rank 0 also runs the router runtime in-process and replays a small trace through it:

  pd        1 prefill + 1 decode replica: KV pages are pushed into the decode GPU's pool by the kv_push
            kernel; greedy tokens must match a single-engine run of the same prompts.
  scale     as above plus an inactive replica brought up by in-kernel parameter multicast from the decode
            replica (byte-exact weights -> same tokens), then used for prefill.
  live      the new replica serves while loading (ZigZag): batches are relayed to the old prefill replica
            through the activation mailbox; tokens again match.
  pd_tp2    (4 GPUs) the pd case with two tensor-parallel replicas of two shards each: every RPC goes to both shards of
            a replica, KV pages move shard to shard (rank i of the prefill replica pushes into rank i of the decode
            replica); the expected tokens come from the prefill replica's own engine, run by its two shards together
            before serving starts.
"""
import asyncio
import os
import sys
import threading

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_requests():
    g = torch.Generator().manual_seed(11)
    n_req = 12
    lens = [int(x) for x in torch.randint(20, 300, (n_req,), generator=g)]
    news = [int(x) for x in torch.randint(3, 9, (n_req,), generator=g)]
    prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in lens]
    return prompts, news


def reference_tokens(prompts, new_tokens, eng=None):
    """Greedy tokens of every request, one request at a time: on a fresh single-GPU engine, or on `eng` (all shards of
    a tensor-parallel engine call this together)."""
    from blitz_scale_b200.runtime import core
    from blitz_scale_b200.runtime.engine import Engine
    own = eng is None
    if own:
        eng = Engine("tiny_gpu", num_pages=256, page_size=16, max_batch=8, max_batch_tokens=2048, seed=0, use_graphs=False)
    out = []
    for i, (p, n) in enumerate(zip(prompts, new_tokens)):
        b = eng.new_batch(1000 + i, [core.SeqSpec(i, p, n)])
        toks = eng.prefill(b)
        seq = list(toks)
        while b.unfinished_ids():
            seq += eng.decode(b)
        b.clear()
        out.append(seq)
    if own:
        del eng
        torch.cuda.empty_cache()
    return out


def main():
    case = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    host_group = dist.new_group(backend="gloo")     # host-side rendezvous that keeps no kernel spinning on the GPUs
    from blitz_scale_b200.worker.gpu_backend import GpuBackend
    from blitz_scale_b200.worker.service import serve
    tp = 2 if case.endswith("_tp2") else 1
    case = case[:-4] if tp == 2 else case
    replica_states = {"pd": ["Prefill", "Decode"], "pd_progressive": ["Prefill", "Decode"],
                      "scale": ["Prefill", "Decode", "Inactive"],
                      "live": ["Prefill", "Decode", "Inactive"]}[case][:world // tp]
    states = [s for s in replica_states for _ in range(tp)]          # one entry per rank
    tp_group = None
    if tp > 1:
        for r0 in range(0, world, tp):
            g_ = dist.new_group(list(range(r0, r0 + tp)))
            if r0 <= rank < r0 + tp:
                tp_group = g_
    base_port = 50400 + (os.getpid() % 50) * 0
    backend = GpuBackend(rank, world, "tiny_gpu", tp=tp, tp_group=tp_group, num_pages=256, page_size=16, max_batch=16,
                         max_batch_tokens=2048, ready=states[rank] != "Inactive", seed=0, copy_ctas=16)
    if states[rank] == "Inactive":
        backend.engine.seg.buffer.zero_()          # a fresh replica holds no parameters
    torch.cuda.synchronize()
    dist.barrier()
    ref = None
    if tp > 1 and rank < tp:
        # the expected tokens of a sharded model come from the first replica's own engine, before it serves
        ref = reference_tokens(*make_requests(), eng=backend.engine)
        assert backend.engine.pool.used_pages == 0
    dist.barrier(group=host_group)

    stop_holder = {}
    started = threading.Event()

    def serve_thread():
        async def run():
            stop_holder["loop"] = asyncio.get_running_loop()
            stop_holder["stop"] = asyncio.Event()
            ready = asyncio.Event()
            t = asyncio.create_task(serve(backend, "127.0.0.1", base_port + rank, stop_event=stop_holder["stop"], ready_event=ready))
            await ready.wait()
            started.set()
            await t
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        asyncio.run(run())

    th = threading.Thread(target=serve_thread, daemon=True)
    th.start()
    started.wait(60)
    dist.barrier()

    ok = 1
    if rank == 0:
        try:
            ok = run_router(case, world, states, base_port, tp, ref)
        except Exception as e:  # noqa: BLE001
            import traceback
            traceback.print_exc()
            ok = 0
    flag = torch.tensor([ok])
    dist.broadcast(flag, 0, group=host_group)      # blocks on the host: the other ranks keep serving until rank 0 is done
    stop_holder["loop"].call_soon_threadsafe(stop_holder["stop"].set)
    th.join(10)
    backend.close()
    dist.barrier(group=host_group)
    good = int(flag) == 1
    if rank == 0 and good:
        print(f"cluster {case}{'_tp2' if tp == 2 else ''}: OK on {world} GPUs", flush=True)
    sys.stdout.flush()
    sys.stderr.flush()
    from blitz_scale_b200.parallel.teardown import shutdown
    shutdown([backend])          # graphs, then symmetric regions, then process groups, with barriers in between
    sys.exit(0 if good else 1)


def run_router(case, world, states, base_port, tp=1, ref=None) -> int:
    from blitz_scale_b200.router.runtime import RouterRuntime
    from blitz_scale_b200.router.server import controller_config_from_cluster
    prompts, news = make_requests()
    n_req = len(prompts)
    if ref is None:
        ref = reference_tokens(prompts, news)
    feats = {"pd": "impl_blitz,impl_nvl,manually_scale", "scale": "impl_blitz,impl_nvl,manually_scale",
             "pd_progressive": "impl_blitz,impl_nvl,manually_scale,migrate_progressive",
             "live": "impl_blitz,impl_nvl,impl_live,manually_scale"}[case]
    cfg = controller_config_from_cluster({"init_states": states, "machines": [0] * world}, tp, feats,
                                         max_blocks_per_replica=200, block_size=16, max_prefill_tokens=1024,
                                         model_layers=2, zigzag_req_limit=2, zigzag_req_floor=2, max_batch_seqs=16)

    async def go():
        rt = RouterRuntime(cfg, [f"127.0.0.1:{base_port + r}" for r in range(world)], model_layers=2)
        loop_task = asyncio.create_task(rt.run())
        reqs = []

        async def collect(lr):
            toks = []
            while True:
                ev = await asyncio.wait_for(lr.queue.get(), timeout=120)
                if ev[0] == "error":
                    return None
                toks.append(ev[1])
                if ev[2]:
                    return toks
        half = n_req // 2
        for i in range(half):
            reqs.append(asyncio.create_task(collect(rt.submit(prompts[i], news[i]))))
        if case in ("scale", "live") and world >= 3:
            assert rt.ctl.manual_scale(2, "Prefill", rt.now())
            rt.wake.set()
        for i in range(half, n_req):
            await asyncio.sleep(0.01)
            reqs.append(asyncio.create_task(collect(rt.submit(prompts[i], news[i]))))
        got = await asyncio.gather(*reqs)
        if case in ("scale", "live") and world >= 3:
            for _ in range(2000):          # let the transfer finish, then push more work through the new replica
                if rt.ctl.state_name(2) == "Prefill":
                    break
                await asyncio.sleep(0.005)
            extra = [asyncio.create_task(collect(rt.submit(prompts[i], news[i]))) for i in range(n_req)]
            got += await asyncio.gather(*extra)
        trans = [l for _, l in rt.transitions]
        used = rt.ctl.total_used_blocks()
        counters = dict(rt.ctl.counters())
        await rt.stop()
        loop_task.cancel()
        return got, trans, used, counters

    got, trans, used, counters = asyncio.run(go())
    want = ref + (ref if len(got) > n_req else [])
    total = agree = 0
    for gtoks, w in zip(got, want):
        assert gtoks is not None and len(gtoks) == len(w), (gtoks, w)
        total += len(w)
        agree += sum(int(a == b) for a, b in zip(gtoks, w))
    print(f"token agreement {agree}/{total}; transitions: {[t for t in trans if 'boot' not in t]}")
    assert agree >= 0.9 * total, (agree, total)
    assert used == 0
    if case == "pd_progressive":
        # batches whose KV left the prefill replica layer by layer while they ran
        print(f"kv transfers {counters.get('blitz_kv_cache_times', 0):.0f}, of which layer-progressive "
              f"{counters.get('blitz_progressive_kv_cache_times', 0):.0f}")
        assert counters.get("blitz_progressive_kv_cache_times", 0) > 0
    if case == "scale":
        assert any("Replica<2> LoadingPrefill => Prefill" in t for t in trans)
    if case == "live":
        assert any("Replica<2> Inactive => NewPrefill" in t for t in trans)
        assert any("=> Prefill" in t and "Replica<2>" in t for t in trans)
    return 1


if __name__ == "__main__":
    main()
