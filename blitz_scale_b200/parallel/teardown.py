"""Orderly exit of a multi-GPU process: CUDA graphs, then symmetric regions, then process groups.

At interpreter exit Python drops objects in no particular order.  For a rank of a multi-GPU job that order matters:
a captured CUDA graph keeps launching kernels' arguments alive (peer pointers into other ranks' symmetric regions,
and, for the NCCL comparison runner, collectives of an NCCL communicator); a symmetric region is mapped into every
peer, so a rank that unmaps it while a peer still holds graphs or queued kernels that name it pulls memory from
under them; and destroying an NCCL communicator that captured graphs still reference, or whose peers have already
left, blocks in the library until its own timeout.  None of these libraries defines the order for us, so the exit
path does it explicitly, with a barrier between the phases so that every rank is past a phase before any rank
starts the next:

    1. synchronize the device; drop every captured graph (engines first);
    2. barrier: no rank will launch, or wait on a peer's flag, again;
    3. drop the symmetric regions (handles and local tensors), synchronize;
    4. barrier: every rank has unmapped;
    5. destroy the process groups.

A watchdog bounds the whole sequence: if a phase does not finish within `timeout_s` the phase is named on stderr
and the process leaves with `os._exit`, so a teardown fault cannot turn into a job that never ends.  The reference
leaves through `MPI_Finalize` after joining its server thread (src/service/service.cc:1408-1436).
"""
from __future__ import annotations

import gc
import os
import sys
import threading
import time
from typing import Iterable


def shutdown(owners: Iterable[object] = (), timeout_s: float = 60.0, exit_code_on_timeout: int = 0) -> float:
    """Tear down in the order above.  `owners`: objects with any of `release_graphs()`, `close_regions()` (engines,
    fused-TP state, peer fabrics, single regions).  Returns the seconds it took."""
    import torch
    import torch.distributed as dist

    owners = [o for o in owners if o is not None]
    phase = ["start"]
    done = threading.Event()
    t0 = time.monotonic()

    def watchdog():
        if not done.wait(timeout_s):
            sys.stderr.write(f"teardown: phase '{phase[0]}' did not finish within {timeout_s:.0f} s; leaving\n")
            sys.stderr.flush()
            sys.stdout.flush()
            os._exit(exit_code_on_timeout)

    threading.Thread(target=watchdog, daemon=True).start()
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    phase[0] = "synchronize"
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    phase[0] = "graphs"
    for o in owners:
        fn = getattr(o, "release_graphs", None)
        if fn is not None:
            fn()
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if multi:
        phase[0] = "barrier after graphs"
        dist.barrier()
    phase[0] = "symmetric regions"
    for o in owners:
        fn = getattr(o, "close_regions", None)
        if fn is not None:
            fn()
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if multi:
        phase[0] = "barrier after regions"
        dist.barrier()
        torch.cuda.synchronize()
    if dist.is_available() and dist.is_initialized():
        phase[0] = "process groups"
        dist.destroy_process_group()
    done.set()
    return time.monotonic() - t0
