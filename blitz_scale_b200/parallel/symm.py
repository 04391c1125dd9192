"""Symmetric (peer-mapped) memory regions and the in-kernel NVLink data paths built on them.

Every GPU of the NVSwitch domain allocates the same set of regions at boot (weight segment, KV
pool, activation mailbox, flag pad, scratch) through ``torch.distributed._symmetric_memory``;
after the rendezvous each rank holds the peer pointers of every other rank's copy and, when the
fabric supports NVLS, one multicast pointer that addresses all copies at once.  The hand-written
kernels take those raw pointers.  This replaces the reference's registered RDMA memory regions and
queue pairs (src/blitz/blitz_tccl.cpp:51-221, src/blitz/stub.h:387-462) and its NCCL warm-up of
every p2p connection (src/blitz/nccl_bcastor.h:71-90): one rendezvous at boot, no per-transfer setup.

Flag pad layout (uint32 counters, all zero at boot):
    [0, 128)                      parameter units: embed | layer 0.. | head   (+1 per source stripe)
    [128, 128 + 16)               activation mailbox slots                    (value = sequence tag)
    [256, 256 + KV_SLOTS*LAYERS)  KV push: per (transfer slot, layer)         (+1 per push)
    [AGREE_FLAG0, +16)            loaded-unit counts published by the TP shards of the replica (plain stores)
    [KV_DONE_FLAG0, +KV_SLOTS)    KV push: per transfer slot, +1 after the last layer of a push
    [ZAG_LOG_FLAG0, +ZAG_LOG)     live execution at tp > 1: ring of step decisions the leading shard publishes
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import _lib as _L
from ..ops import status_word, _check

PARAM_FLAG0 = 0
MAILBOX_FLAG0 = 128
KV_FLAG0 = 256
KV_SLOTS = 8
MAX_LAYERS = 128
AGREE_FLAG0 = KV_FLAG0 + KV_SLOTS * MAX_LAYERS    # loaded-unit count of every TP shard of this replica (<= 16)
KV_DONE_FLAG0 = AGREE_FLAG0 + 16                  # per transfer slot: +1 when a whole push (all its layers) has landed
ZAG_LOG_FLAG0 = KV_DONE_FLAG0 + KV_SLOTS           # ring of decisions of the leading TP shard (see parallel/agreement.py)
ZAG_LOG = 16
FLAG_WORDS = ZAG_LOG_FLAG0 + ZAG_LOG


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class SymmRegion:
    """nbytes allocated identically on every rank of `group`."""

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.nbytes = int(nbytes)
        dev = device or torch.device("cuda", torch.cuda.current_device())
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=dev)
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        # the region may live on a sub-group (one tensor-parallel shard column): callers name ranks of the whole job
        self.job_ranks: List[int] = list(dist.get_process_group_ranks(self.group))
        mc = 0
        try:
            if self.handle.has_multicast_support(dev.type, dev.index):
                mc = int(self.handle.multicast_ptr)
        except Exception:
            mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.mc_ptr = mc

    def ptr_of(self, job_rank: int) -> int:
        """Address of `job_rank`'s copy (a rank of the whole job, which must belong to this region's group)."""
        return self.ptrs[self.job_ranks.index(job_rank)]

    def peer_tensor(self, rank: int, dtype=torch.uint8) -> torch.Tensor:
        return self.handle.get_buffer(rank, (self.nbytes // torch.empty((), dtype=dtype).element_size(),), dtype)

    def barrier(self) -> None:
        self.handle.barrier()

    def close_regions(self) -> None:
        """Drop the mapping (local tensor and rendezvous handle).  Call on every rank, between two barriers, after
        everything that names this region's pointers (kernels, captured graphs) is gone."""
        self.handle = None
        self.local = None
        self.ptrs = []
        self.mc_ptr = 0


@dataclass
class FabricSizes:
    weight_bytes: int
    kv_bytes: int
    mailbox_slots: int = 16
    mailbox_slot_bytes: int = 0
    scratch_bytes: int = 1 << 20


class PeerFabric:
    """The per-GPU set of symmetric regions plus launch helpers for the peer-memory kernels."""

    def __init__(self, sizes: FabricSizes, group=None, device: Optional[torch.device] = None, weight_group=None):
        """`weight_group`: the ranks that hold the same weight shard as this one (with tensor parallelism: the same
        shard index in every replica).  Parameters only ever move within it, so the weight region and with it the
        multicast address are made over that group alone: one `multimem.st` then reaches the replicas of this shard
        and nothing else, and a scale-out costs the source one copy per shard whatever the number of new replicas
        (the reference builds one broadcast chain per shard, src/service/service.cc:1339-1347)."""
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.group = group if group is not None else dist.group.WORLD
        self.weights = SymmRegion(sizes.weight_bytes, weight_group if weight_group is not None else self.group,
                                  self.device)
        self.kv = SymmRegion(sizes.kv_bytes, self.group, self.device)
        self.mailbox = SymmRegion(max(16, sizes.mailbox_slots * sizes.mailbox_slot_bytes), self.group, self.device)
        self.flags = SymmRegion(FLAG_WORDS * 4, self.group, self.device)
        self.flags.local.zero_()
        self.kv.local.zero_()
        self.sizes = sizes
        self.rank, self.world = self.flags.rank, self.flags.world
        # local scratch: tickets for the "last CTA publishes" protocol
        self.tickets = torch.zeros(4096, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        self.flags.barrier()

    def close_regions(self) -> None:
        for r in (self.weights, self.kv, self.mailbox, self.flags):
            r.close_regions()

    # ------------------------------------------------------------------ flags
    def flag_view(self) -> torch.Tensor:
        return self.flags.local.view(torch.int32)

    def read_flags(self, start: int, count: int) -> List[int]:
        """Host read of this GPU's own flag words (synchronises a small D2H copy on a side stream)."""
        return self.flag_view()[start:start + count].tolist()

    def reset_param_flags(self) -> None:
        self.flag_view()[PARAM_FLAG0:PARAM_FLAG0 + 128].zero_()

    def wait_flag(self, index: int, want: int, budget_ms: float = 1000.0) -> None:
        """Enqueue a bounded device-side wait on flag `index` of this GPU (timeout -> status word, no trap)."""
        ptr = self.flags.ptrs[self.rank] + index * 4
        _check(_L.lib().blitz_flag_wait(ctypes.c_void_p(ptr), want, int(budget_ms * 1e6),
                                        ctypes.c_void_p(status_word(self.device).data_ptr()), _stream()),
               "blitz_flag_wait")

    def wait_flag_eq(self, ptr: int, want: int, budget_ms: float = 1000.0) -> None:
        """Bounded device-side wait until the word at `ptr` (any rank's memory) equals `want` exactly."""
        _check(_L.lib().blitz_flag_wait_eq(ctypes.c_void_p(ptr), want, int(budget_ms * 1e6),
                                           ctypes.c_void_p(status_word(self.device).data_ptr()), _stream()),
               "blitz_flag_wait_eq")

    def set_flag(self, rank: int, index: int, value: int, add: bool = False) -> None:
        ptr = self.flags.ptrs[rank] + index * 4
        _check(_L.lib().blitz_flag_set(ctypes.c_void_p(ptr), value, int(add), _stream()), "blitz_flag_set")

    # ------------------------------------------------------------------ unit copies (parameters / activations)
    def copy_units(self, region: SymmRegion, dst_ranks: Sequence[int], unit_offsets: Sequence[int],
                   unit_nbytes: Sequence[int], flag_index0: int, *, stripe: int = 0, n_stripes: int = 1,
                   use_multimem: bool = False, num_ctas: int = 64) -> None:
        """Stream byte ranges of `region` from this GPU to the same offsets on `dst_ranks`, bumping
        flag `flag_index0 + u` on each destination when unit u has landed."""
        n = len(unit_offsets)
        assert n == len(unit_nbytes) and 1 <= len(dst_ranks) <= 8
        lib = _L.lib()
        for u0 in range(0, n, 96):
            u1 = min(n, u0 + 96)
            k = u1 - u0
            offs = (ctypes.c_int64 * k)(*unit_offsets[u0:u1])
            lens = (ctypes.c_int64 * k)(*unit_nbytes[u0:u1])
            bases = (ctypes.c_void_p * len(dst_ranks))(*[region.ptr_of(r) for r in dst_ranks])
            flags = (ctypes.c_void_p * len(dst_ranks))(*[self.flags.ptrs[r] for r in dst_ranks])
            tick = self.tickets[:k]
            tick.zero_()
            mc = ctypes.c_void_p(region.mc_ptr if (use_multimem and region.mc_ptr) else 0)
            rc = lib.blitz_peer_copy_units(ctypes.c_void_p(region.ptrs[region.rank]), bases, flags, len(dst_ranks), mc,
                                           offs, lens, k, flag_index0 + u0, stripe, n_stripes,
                                           ctypes.c_void_p(tick.data_ptr()), num_ctas, _stream())
            _check(rc, "blitz_peer_copy_units")

    # ------------------------------------------------------------------ KV push
    def kv_push(self, dst_rank: int, src_pages: torch.Tensor, dst_pages: torch.Tensor, layer_begin: int,
                layer_end: int, page_bytes: int, src_layer_stride: int, dst_layer_stride: int, src_max_pages: int,
                dst_max_pages: int, flag_slot: Optional[int] = None, ctas_per_layer: int = 0,
                dst_pages_ptr: int = 0, dst_count_ptr: int = 0, n_pages: Optional[int] = None,
                done: bool = True) -> None:
        """Store prompt pages of layers [layer_begin, layer_end) into `dst_rank`'s pool using its page ids.

        ``dst_pages`` is a local int32 tensor, or None with ``dst_pages_ptr`` the address (possibly in the peer's
        memory) of the ids the destination published; ``dst_count_ptr`` then names the count it published, which
        the kernel compares with the number of source pages.  With a ``flag_slot`` the slot's completion counter
        on the destination is bumped after the push (stream order: after every layer has been stored); a transfer
        made of several calls passes ``done=False`` on all but its last one."""
        assert src_pages.dtype == torch.int32 and (dst_pages is None or dst_pages.dtype == torch.int32)
        nl = layer_end - layer_begin
        tick = self.tickets[1024:1024 + nl]
        tick.zero_()
        flags = 0
        if flag_slot is not None:
            flags = self.flags.ptrs[dst_rank] + (KV_FLAG0 + flag_slot * MAX_LAYERS) * 4
        dptr = dst_pages.data_ptr() if dst_pages is not None else dst_pages_ptr
        n = src_pages.numel() if n_pages is None else n_pages
        rc = _L.lib().blitz_kv_push(ctypes.c_void_p(self.kv.ptrs[self.rank]), ctypes.c_void_p(self.kv.ptrs[dst_rank]),
                                    ctypes.c_void_p(src_pages.data_ptr()), ctypes.c_void_p(dptr),
                                    n, layer_begin, layer_end, page_bytes, src_layer_stride,
                                    dst_layer_stride, src_max_pages, dst_max_pages, ctypes.c_void_p(flags),
                                    ctypes.c_void_p(tick.data_ptr()), ctas_per_layer, ctypes.c_void_p(dst_count_ptr),
                                    ctypes.c_void_p(status_word(self.device).data_ptr()), _stream())
        _check(rc, "blitz_kv_push")
        if flag_slot is not None and done:
            self.set_flag(dst_rank, KV_DONE_FLAG0 + flag_slot, 1, add=True)
