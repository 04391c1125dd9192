"""Build the per-step device inputs (token ids, positions, cache slots, page-table CSR) from host lists.

One pinned staging buffer per builder is filled on the host and copied to the device with a
single asynchronous H2D copy per step, the role of the pinned page-table slots and token
staging buffer of the reference (src/blitz/cache_manager.h:198-253, src/blitz/stub.h:1288-1338).
Static device buffers keep their addresses so a captured CUDA graph can be replayed after the
copy.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..models.llama import StepMeta


class MetaBuilder:
    def __init__(self, max_tokens: int, max_batch: int, max_pages_per_step: int, page_size: int, device="cuda"):
        self.max_tokens, self.max_batch, self.page_size = max_tokens, max_batch, page_size
        self.max_pages = max_pages_per_step
        # layout of the single int32 staging array
        self.o_ids = 0
        self.o_pos = self.o_ids + max_tokens
        self.o_slot = self.o_pos + max_tokens
        self.o_tokptr = self.o_slot + max_tokens
        self.o_pgptr = self.o_tokptr + max_batch + 1
        self.o_last = self.o_pgptr + max_batch + 1
        self.o_idx = self.o_last + max_batch
        total = self.o_idx + max_pages_per_step
        pin = torch.cuda.is_available()
        self.host = torch.zeros(total, dtype=torch.int32, pin_memory=pin)
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        self.h2d_bytes = 0

    def _views(self, T: int, B: int, P: int):
        d = self.dev
        return (d[self.o_ids:self.o_ids + T], d[self.o_pos:self.o_pos + T], d[self.o_slot:self.o_slot + T],
                d[self.o_tokptr:self.o_tokptr + B + 1], d[self.o_pgptr:self.o_pgptr + B + 1],
                d[self.o_last:self.o_last + B], d[self.o_idx:self.o_idx + max(P, 1)])

    def _flush(self, used_ranges):
        # one copy covering the used prefix of each field would need several copies; the array is small
        # (a few hundred KB at most), so one copy of the whole used span is cheaper than many launches.
        hi = max(e for _, e in used_ranges)
        self.dev[:hi].copy_(self.host[:hi], non_blocking=True)
        self.h2d_bytes = hi * 4

    def prefill(self, prompts: Sequence[Sequence[int]], page_tables: Sequence[Sequence[int]]) -> StepMeta:
        """Positions start at 0; page_tables[b] must hold ceil((len + 1) / page) page ids."""
        B = len(prompts)
        T = sum(len(p) for p in prompts)
        assert T <= self.max_tokens and B <= self.max_batch
        h, ps = self.host, self.page_size
        t = 0
        idx: List[int] = []
        h[self.o_tokptr] = 0
        h[self.o_pgptr] = 0
        for b, (pr, pt) in enumerate(zip(prompts, page_tables)):
            n = len(pr)
            h[self.o_ids + t:self.o_ids + t + n] = torch.as_tensor(pr, dtype=torch.int32)
            ar = torch.arange(n, dtype=torch.int32)
            h[self.o_pos + t:self.o_pos + t + n] = ar
            pages = torch.as_tensor(pt, dtype=torch.int32)
            h[self.o_slot + t:self.o_slot + t + n] = pages[(ar // ps).long()] * ps + ar % ps
            t += n
            used = (n + ps - 1) // ps
            idx += list(pt[:used])
            h[self.o_tokptr + b + 1] = t
            h[self.o_pgptr + b + 1] = len(idx)
            h[self.o_last + b] = n - (used - 1) * ps if n else 0
        assert len(idx) <= self.max_pages
        h[self.o_idx:self.o_idx + len(idx)] = torch.as_tensor(idx, dtype=torch.int32)
        self._flush([(0, self.o_idx + len(idx))])
        ids, pos, slot, tokptr, pgptr, last, pidx = self._views(T, B, len(idx))
        return StepMeta(ids=ids, pos=pos, slot=slot, page_indices=pidx, page_indptr=pgptr, last_page_len=last,
                        tok_indptr=tokptr, seq_lens_host=[len(p) for p in prompts], is_prefill=True, batch=B,
                        num_tokens=T)

    def decode(self, last_tokens, seq_lens, page_tables, pad_to: int = 0, num_splits: int = 1) -> StepMeta:
        """seq_lens[b] = tokens already in the cache; the new token is written at that position.
        ``page_tables`` is a list of page-id lists or an int32 matrix [B, W] (rows padded arbitrarily).
        ``pad_to`` pads the batch with empty sequences (no pages, slot -1) up to a captured graph size.
        Vectorised with numpy: the host cost is a few tens of microseconds at batch 256."""
        import numpy as np
        B = len(last_tokens)
        Bp = max(B, pad_to)
        assert Bp <= self.max_batch and Bp <= self.max_tokens
        ps = self.page_size
        h = self.host.numpy()
        n = np.asarray(seq_lens, dtype=np.int64)
        if isinstance(page_tables, np.ndarray):
            pt = page_tables
        else:
            W = max(len(r) for r in page_tables) if B else 1
            pt = np.zeros((B, W), dtype=np.int32)
            for b, r in enumerate(page_tables):
                pt[b, :len(r)] = r
        used = n // ps + 1
        h[self.o_ids:self.o_ids + B] = np.asarray(last_tokens, dtype=np.int32)
        h[self.o_pos:self.o_pos + B] = n
        h[self.o_slot:self.o_slot + B] = pt[np.arange(B), n // ps].astype(np.int64) * ps + n % ps
        h[self.o_last:self.o_last + B] = n + 1 - (used - 1) * ps
        h[self.o_pgptr] = 0
        h[self.o_pgptr + 1:self.o_pgptr + 1 + B] = np.cumsum(used)
        mask = np.arange(pt.shape[1])[None, :] < used[:, None]
        idx = pt[mask]
        if Bp > B:
            h[self.o_ids + B:self.o_ids + Bp] = 0
            h[self.o_pos + B:self.o_pos + Bp] = 0
            h[self.o_slot + B:self.o_slot + Bp] = -1
            h[self.o_last + B:self.o_last + Bp] = 0
            h[self.o_pgptr + 1 + B:self.o_pgptr + 1 + Bp] = len(idx)
        assert len(idx) <= self.max_pages
        h[self.o_idx:self.o_idx + len(idx)] = idx
        self._flush([(0, self.o_idx + len(idx))])
        ids, pos, slot, tokptr, pgptr, last, pidx = self._views(Bp, Bp, self.max_pages)
        return StepMeta(ids=ids, pos=pos, slot=slot, page_indices=pidx, page_indptr=pgptr, last_page_len=last,
                        tok_indptr=None, seq_lens_host=[], is_prefill=False, batch=Bp, num_tokens=Bp,
                        num_splits=num_splits)
