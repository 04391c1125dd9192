"""Stand-in reference data plane: the reference's algorithms on NCCL / torch.matmul, for comparison only.

The reference cannot be built here (empty submodules, no MPI / gRPC C++ / cargo), so its data-plane algorithms are
re-stated on the libraries it uses, with its chunk sizes:

* parameter broadcast: chain src -> d1 -> d2 -> ... in 256 MB chunks, double buffered (src/blitz/nccl_bcastor.h:286-373),
  and plain `ncclBroadcast`;
* KV migration: one send/recv per (page, layer) (src/blitz/migration_manager.h:436-536);
* tensor-parallel layers: `torch.matmul` + AllReduce after the row-parallel GEMMs (src/layer/attn.h:217-233,
  src/layer/glu.h:138-154), ReduceScatter / AllGather variants for the fused-kernel microbenchmark.

Nothing in the product path imports this module.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
import torch.distributed as dist

CHAIN_CHUNK = 256 << 20


def chain_broadcast(buf: torch.Tensor, chain: Sequence[int], chunk_bytes: int = CHAIN_CHUNK) -> None:
    """Store-and-forward pipeline along `chain` (ranks); every rank of the chain calls this with its own buffer."""
    rank = dist.get_rank()
    if rank not in chain:
        return
    i = list(chain).index(rank)
    prev_r = chain[i - 1] if i > 0 else None
    next_r = chain[i + 1] if i + 1 < len(chain) else None
    n = buf.numel()
    pending = []
    for off in range(0, n, chunk_bytes):
        piece = buf[off:min(n, off + chunk_bytes)]
        if prev_r is not None:
            dist.recv(piece, src=prev_r)
        if next_r is not None:
            pending.append(dist.isend(piece, dst=next_r))
    for w in pending:
        w.wait()


def nccl_broadcast(buf: torch.Tensor, src: int, group=None) -> None:
    dist.broadcast(buf, src=src, group=group)


def kv_migrate_per_page(kv: torch.Tensor, src_pages: List[int], dst_pages: List[int], src: int, dst: int,
                        layers: Sequence[int], window: int = 64) -> None:
    """kv: [layers, pages, page_bytes] uint8 on every rank.  One message per (page, layer), `window` in flight."""
    rank = dist.get_rank()
    ops = []
    for sp, dp in zip(src_pages, dst_pages):
        for l in layers:
            if rank == src:
                ops.append(dist.P2POp(dist.isend, kv[l, sp], dst))
            elif rank == dst:
                ops.append(dist.P2POp(dist.irecv, kv[l, dp], src))
            if len(ops) >= window:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
                ops = []
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()


def matmul_allreduce(x: torch.Tensor, w: torch.Tensor, group=None) -> torch.Tensor:
    y = torch.matmul(x, w)
    dist.all_reduce(y, group=group)
    return y


def matmul_reduce_scatter(x: torch.Tensor, w: torch.Tensor, group=None) -> torch.Tensor:
    y = torch.matmul(x, w)
    tp = dist.get_world_size(group)
    out = torch.empty(y.shape[0] // tp, y.shape[1], dtype=y.dtype, device=y.device)
    dist.reduce_scatter_tensor(out, y, group=group)
    return out


def allgather_matmul(x_shard: torch.Tensor, w: torch.Tensor, group=None) -> torch.Tensor:
    tp = dist.get_world_size(group)
    full = torch.empty(x_shard.shape[0] * tp, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
    dist.all_gather_into_tensor(full, x_shard.contiguous(), group=group)
    return torch.matmul(full, w)
