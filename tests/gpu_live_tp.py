"""Live execution (layer-interleaved prefill while parameters arrive) on tensor-parallel replicas, on real GPUs.

Launched by test_multi_gpu.py through torch.distributed.run with 4 ranks (2 ranks: no hand-over part).  Ranks 0-1 are
the two shards of a new replica, ranks 2-3 the shards of an old, fully loaded one; all hold the same weights.

  0. (4 ranks) the new replica's weights are cleared and come back from the old replica: shard t of the old replica
     stores into shard t of the new one through the multicast address of their shard column (the weight region of a
     tensor-parallel worker spans only the ranks that hold the same shard).
  1. every replica prefills three prompts the ordinary way: the expected first tokens.
  2. the new replica forgets that it is loaded; a thread per shard then marks one unit after the other as arrived, the
     second shard later than the first, so that only the agreed minimum keeps a shard from running a layer its
     sibling lacks.
  3. the three prompts go to the new replica as live-execution tasks.  The leading shard decides the order of the
     interleaved steps and the other follows its log; both must produce the expected tokens.
  4. (4 ranks) meanwhile the head task is handed over: each shard of the new replica ships its copy of the residual
     stream to its counterpart, and the old replica runs the remaining layers on the switch-reduced path.
"""
import os
import sys
import threading
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_batch(pb, bid, prompts):
    b = pb.Batch(id=bid, size=len(prompts), max_tokens=sum(len(p) for p in prompts) + 8 * len(prompts))
    for i, p in enumerate(prompts):
        r = b.requests.add()
        r.id, r.inputs, r.prefill_logprobs, r.top_n_tokens = bid * 100 + i, "", False, 0
        r.input_tokens.extend(p)
        r.stopping_parameters.max_new_tokens = 4
        r.stopping_parameters.ignore_eos_token = True
    return b


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    tp = 2
    assert world in (2, 4)
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    host = dist.new_group(backend="gloo")
    tp_group = None
    for r0 in range(0, world, tp):
        g = dist.new_group(list(range(r0, r0 + tp)))
        if r0 <= rank < r0 + tp:
            tp_group = g
    from blitz_scale_b200 import ops
    from blitz_scale_b200.pb.schema import pb
    from blitz_scale_b200.runtime import core
    from blitz_scale_b200.worker.gpu_backend import GpuBackend
    backend = GpuBackend(rank, world, "tiny_gpu_deep", tp=tp, num_pages=256, page_size=16, max_batch=8,
                         max_batch_tokens=1024, ready=True, seed=0, tp_group=tp_group, copy_ctas=16)
    L = backend.cfg.layers
    new_replica = rank < tp
    has_switch = torch.tensor([1 if backend.engine.fused.has_mc else 0])
    dist.all_reduce(has_switch, op=dist.ReduceOp.MIN, group=host)
    if int(has_switch) == 0:
        if rank == 0:
            print("SKIP: no in-switch reduction on this fabric", flush=True)
        backend.close()
        from blitz_scale_b200.parallel.teardown import shutdown
        shutdown([backend])
        return 0

    if world == 4:
        seg = backend.engine.seg.buffer
        before = int(seg.view(torch.int32).sum(dtype=torch.int64))
        assert backend.fabric.weights.world == world // tp and backend.fabric.weights.job_ranks == [rank % tp, rank % tp + tp]
        if new_replica:
            seg.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=host)
        backend.use_multimem, backend.multimem_min_dests = True, 1
        backend.broadcast("nvl", [2, 3], [0, 1])          # sources store, destinations wait for every unit
        torch.cuda.synchronize()
        ops.check_status()
        assert int(seg.view(torch.int32).sum(dtype=torch.int64)) == before, "shard differs after the transfer"
        assert backend.engine.status.fully_loaded()
        if not new_replica:
            assert backend.transfer_log and backend.transfer_log[-1]["multimem"] == bool(backend.fabric.weights.mc_ptr)
        dist.barrier(group=host)

    g = torch.Generator().manual_seed(21)
    prompts = [[torch.randint(0, 4096, (n,), generator=g).tolist() for n in lens] for lens in ((70, 33), (150,), (9, 40, 21))]

    def first_tokens(raw):
        return [t for _, t, _ in zip(*core.parse_generations(raw))]

    # 1. expected tokens: ordinary prefill on every replica
    want = []
    for i, ps in enumerate(prompts):
        gens, cb, _ = backend.prefill(make_batch(pb, 50 + i, ps), 0, None, [])
        want.append(first_tokens(gens))
        backend.clear_cache(50 + i)
    ops.check_status()
    dist.barrier(group=host)

    got, errors = {}, []
    relayed = [None]
    if new_replica:
        # 2. forget the parameters; the loader threads bring them "back" unit by unit
        with backend.lock:
            backend.engine.status.reset()
            backend.agree.publish(0)
            backend._agreed_full = False

        def loader():
            torch.cuda.set_device(backend.device)
            time.sleep(0.05)
            for unit in range(L + 2):
                time.sleep(0.03 + 0.02 * (rank % tp))
                with backend.lock:
                    backend.engine.status.unit_arrived(unit)
                    backend.agree.publish(unit + 1)
                    backend.zag_cv.notify_all()

        def task(i):
            torch.cuda.set_device(backend.device)
            try:
                gens, cb, pp = backend.zag_prefill(make_batch(pb, 10 + i, prompts[i]), pb.PREFILL_CASE_NAIVE_PP, None, 0, i + 1)
                if pp is not None:
                    relayed[0] = (10 + i, int(pp.tfm_layer) if pp.WhichOneof("start_layer") == "tfm_layer" else 0)
                else:
                    got[i] = first_tokens(gens)
            except Exception as e:  # noqa: BLE001
                errors.append(repr(e))

        threads = [threading.Thread(target=task, args=(i,)) for i in range(len(prompts))]
        for t in threads:
            t.start()
            time.sleep(0.005)
        ld = threading.Thread(target=loader)
        ld.start()
        if world == 4:
            # 4. hand the head task over once a few layers are here (each shard notices at its own time)
            while backend.engine.status.layers_ready < 3:
                time.sleep(0.002)
            res = backend.relay(rank + tp, False)
            assert res is not None, "nothing was handed over"
        for t in threads:
            t.join(120)
        ld.join(30)
    info = [relayed[0]]
    dist.broadcast_object_list(info, 0, group=host)
    if world == 4 and not new_replica:
        bid, k = info[0]
        pp = pb.PipeParaInfo()
        pp.tfm_layer = k
        gens, cb, _ = backend.prefill(make_batch(pb, bid, prompts[bid - 10]), pb.PREFILL_CASE_NAIVE_PP, pp, [])
        got[bid - 10] = first_tokens(gens)
    ops.check_status()
    ok = not errors
    for i, toks in got.items():
        if toks != want[i]:
            ok = False
            errors.append(f"rank {rank} task {i}: {toks} != {want[i]}")
    if new_replica:
        expect_local = len(prompts) - (1 if world == 4 else 0)
        if len(got) != expect_local:
            ok = False
            errors.append(f"rank {rank}: {len(got)} tasks finished here, expected {expect_local}")
        if world == 4 and not (relayed[0] and 1 <= relayed[0][1] < L):
            ok = False
            errors.append(f"rank {rank}: hand-over {relayed[0]} is not in the middle of the model")
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=host)
    if errors:
        print(f"rank {rank}: {errors}", flush=True)
    if rank == 0 and int(flag) == 1:
        print(f"live tp: OK on {world} ranks; handed over {info[0]}", flush=True)
    sys.stdout.flush()
    backend.close()
    from blitz_scale_b200.parallel.teardown import shutdown
    shutdown([backend])
    return 0 if int(flag) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
