"""Python entry points of the hand-written sm_100a kernels.

Each function takes CUDA tensors, launches on the current stream and returns
the output tensor.  Shapes follow the serving data layouts: activations
``[tokens, features]`` row-major, weights ``[in, out]`` row-major (the layout
the reference loads, scripts/util/make_dangertensors.py:9-30), the paged KV
cache ``[page][K|V][token][kv_head][head_dim]`` per layer.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ._lib import lib, available, KernelLibraryMissing  # noqa: F401

_DT = {torch.float16: 0, torch.bfloat16: 1}
_status = {}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"kernels take fp16/bf16 tensors, got {t.dtype}") from None


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}" + (
            " (argument not supported by the kernel)" if rc == -1 else
            " (TMA descriptor encoder unavailable)" if rc == -2 else ""))


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 word the kernels write a non-zero code into when a bounded wait or an index check fails."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.type, dev.index)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status[key]


def check_status(device=None, reset: bool = True) -> int:
    """Read the status word (synchronises). Raises on a non-zero code."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        if reset:
            w.zero_()
            for _, tickets in _gemm_ws.values():  # an aborted split-K GEMM may leave tickets behind
                tickets.zero_()
            for _, flags in _pair_ws.values():
                flags.zero_()
        names = {1: "TMA producer wait timed out", 2: "MMA wait timed out", 3: "epilogue wait timed out",
                 4: "flag wait timed out", 5: "index out of range", 6: "size beyond the supported maximum"}
        raise RuntimeError(f"kernel status {code}: {names.get(code, 'unknown')}")
    return code


# ---------------------------------------------------------------------------------------------- GEMM
_EPI = {"store": 0, "add": 1, "silu_mul": 2}


_gemm_ws = {}
_pair_ws = {}
GEMM_TICKETS = 4096
PAIR_FLAGS = 65536
DECODE_GEMM_MAX_M = 128
PAIR_GEMM_MAX_M = 256


def gemm_workspace(device=None):
    """Per-device scratch of the split-K path: (fp32 partials as bytes, zeroed uint32 tickets)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.type, dev.index)
    if key not in _gemm_ws:
        n = int(lib().blitz_gemm_workspace_bytes(148))
        _gemm_ws[key] = (torch.empty(n, dtype=torch.uint8, device=dev),
                         torch.zeros(GEMM_TICKETS, dtype=torch.int32, device=dev))
    return _gemm_ws[key]


def pair_gemm_workspace(device=None):
    """Per-device scratch of the paired-SM GEMM: (fp32 partials as bytes, zeroed uint32 counters, eight per tile)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.type, dev.index)
    if key not in _pair_ws:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        n = int(lib().blitz_gemm_pair_workspace_bytes(sms))
        _pair_ws[key] = (torch.empty(n, dtype=torch.uint8, device=dev),
                         torch.zeros(PAIR_FLAGS, dtype=torch.int32, device=dev))
    return _pair_ws[key]


def gemm(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, *, residual=None,
         epilogue: str = "store", b_layout: str = "kn", bn: int = 0, split_k: int = 0, static_b: bool = False,
         decode_path: Optional[bool] = None, decode_split: int = 0, pair_path: Optional[bool] = None,
         pair_bnf: int = 0, pair_upp: int = 0, pair_nacc: int = 0) -> torch.Tensor:
    """``out = a @ b`` on tcgen05 with a fused epilogue.

    a: [M, K].  b: [K, N] when ``b_layout == 'kn'`` (weights stored in,out) or [N, K] for ``'nk'``.
    epilogue 'add' adds ``residual`` ([M, N], same pitch as out); 'silu_mul' treats b as [gate | up] with
    N_out = b_cols / 2 and returns silu(a@gate) * (a@up).  ``split_k``: 0 lets the kernel split K when the
    GEMM is too skinny to fill the GPU, 1 forbids it, n > 1 forces n splits.

    Up to 256 rows of ``a`` with 'kn' weights go to the weight-streaming decode kernel (operands swapped on
    the tensor core, K split over a thread-block cluster with the reduction in distributed shared memory);
    ``decode_path`` forces (True) or forbids (False) that choice and ``decode_split`` caps its cluster size.  ``static_b=True`` promises that ``b`` is not written by kernels still
    running in this stream (model weights), so the decode kernel may start streaming it before its
    predecessor has finished.

    129..256 rows with 'kn' weights go to the paired-SM kernel (two CTAs issue one 256-row
    ``tcgen05.mma.cta_group::2``, stream-K over CTA pairs); ``pair_path`` forces (True) or forbids (False) it for
    any M, ``pair_bnf`` / ``pair_nacc`` / ``pair_upp`` override its tile width, tiles per pair and units per pair.
    """
    assert a.is_cuda and a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = a.shape
    if b_layout == "kn":
        assert b.shape[0] == K
        bcols = b.shape[1]
    else:
        assert b.shape[1] == K
        bcols = b.shape[0]
    epi = _EPI[epilogue]
    N = bcols // 2 if epi == 2 else bcols
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1
    if epi == 1:
        assert residual is not None and residual.shape == (M, N) and residual.stride(0) == out.stride(0)
    ws, tickets = gemm_workspace(a.device)
    # the decode kernel re-reads the activation tile with every weight tile, which the SM's load path cannot keep up
    # with beyond ~128 rows; from there on the tiled kernel is faster
    use_dec = M <= DECODE_GEMM_MAX_M and bn == 0 and split_k == 0 and \
        bool(lib().blitz_gemm_decode_supported(M, N, K, 0 if b_layout == "kn" else 1, epi))
    if decode_path is not None:
        assert not decode_path or lib().blitz_gemm_decode_supported(M, N, K, 0 if b_layout == "kn" else 1, epi)
        use_dec = decode_path
    pair_ok = bool(lib().blitz_gemm_pair_supported(M, N, K, 0 if b_layout == "kn" else 1, epi))
    use_pair = (not use_dec and DECODE_GEMM_MAX_M < M <= PAIR_GEMM_MAX_M and bn == 0 and split_k == 0 and pair_ok)
    if pair_path is not None:
        assert not pair_path or pair_ok
        use_pair = pair_path
    if use_pair:
        pws, pflags = pair_gemm_workspace(a.device)
        rc = lib().blitz_gemm_pair(_p(a), a.stride(0), _p(b), b.stride(0), _p(out), out.stride(0), _p(residual), M, N,
                                   K, epi, N if epi == 2 else 0, _dt(a), int(static_b), pair_bnf, pair_nacc, pair_upp,
                                   _p(pws), pws.numel(), _p(pflags), pflags.numel(), _p(status_word(a.device)),
                                   _stream())
        _check(rc, "blitz_gemm_pair")
        return out
    if use_dec:
        rc = lib().blitz_gemm_decode(_p(a), a.stride(0), _p(b), b.stride(0), _p(out), out.stride(0), _p(residual), M, N,
                                     K, epi, N if epi == 2 else 0, _dt(a), int(static_b), decode_split,
                                     _p(status_word(a.device)), _stream())
        _check(rc, "blitz_gemm_decode")
        return out
    rc = lib().blitz_gemm(_p(a), a.stride(0), _p(b), b.stride(0), _p(out), out.stride(0), _p(residual), M, N, K,
                          0 if b_layout == "kn" else 1, epi, N if epi == 2 else 0, _dt(a), bn, split_k,
                          _p(ws), ws.numel(), _p(tickets), tickets.numel(), _p(status_word(a.device)), _stream())
    _check(rc, "blitz_gemm")
    return out


# ---------------------------------------------------------------------------------------------- elementwise
def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, *, vocab_start: int = 0,
              zero_missing: bool = True, dst_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    assert ids.dtype == torch.int32
    T, H = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    _check(lib().blitz_embedding(_p(ids), _p(table), _p(out), T, H, vocab_start, table.shape[0], int(zero_missing),
                                 _p(dst_rows), _dt(table), _stream()), "blitz_embedding")
    return out


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    T, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    _check(lib().blitz_rms_norm(_p(x), _p(w), _p(out), T, H, eps, _dt(x), _stream()), "blitz_rms_norm")
    return out


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float = 1e-5,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual += x; returns RMSNorm(residual) * w (written to ``out``, which may be ``x``)."""
    T, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    _check(lib().blitz_add_rms_norm(_p(x), _p(residual), _p(w), _p(out), T, H, eps, _dt(x), _stream()),
           "blitz_add_rms_norm")
    return out


def silu_mul(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    T, two_i = x.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty((T, inter), dtype=x.dtype, device=x.device)
    _check(lib().blitz_silu_mul(_p(x), _p(out), T, inter, x.stride(0), _dt(x), _stream()), "blitz_silu_mul")
    return out


def add_residual(residual: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    assert residual.is_contiguous() and x.is_contiguous() and residual.numel() == x.numel()
    _check(lib().blitz_add_residual(_p(residual), _p(x), residual.numel(), _dt(x), _stream()), "blitz_add_residual")
    return residual


def gather_last(x: torch.Tensor, indptr: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    B, H = indptr.numel() - 1, x.shape[1]
    if out is None:
        out = torch.empty((B, H), dtype=x.dtype, device=x.device)
    _check(lib().blitz_gather_last(_p(x), _p(indptr), _p(out), B, H, _dt(x), _stream()), "blitz_gather_last")
    return out


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, out_val: Optional[torch.Tensor] = None,
           idx_offset: int = 0) -> torch.Tensor:
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _check(lib().blitz_argmax(_p(logits), B, V, logits.stride(0), _p(out), _p(out_val), idx_offset, _dt(logits),
                              _stream()), "blitz_argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seeds: torch.Tensor, step: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    assert temperature.dtype == torch.float32 and top_k.dtype == torch.int32 and top_p.dtype == torch.float32
    assert seeds.dtype in (torch.int64, torch.uint64)
    _check(lib().blitz_sample(_p(logits), B, V, logits.stride(0), _p(temperature), _p(top_k), _p(top_p), _p(seeds),
                              step, _p(out), _dt(logits), _stream()), "blitz_sample")
    return out


def rope_kv_store(qkv: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, kv_layer: torch.Tensor, *, q_heads: int,
                  kv_heads: int, head_dim: int, page_size: int, rope_theta: float) -> None:
    """Rotate q and k of ``qkv`` in place and write rotated k and v to ``kv_layer`` ([pages, 2, page, kvh, hd])."""
    T = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (q_heads + 2 * kv_heads) * head_dim
    assert pos.dtype == torch.int32 and slot.dtype == torch.int32
    max_pages = kv_layer.shape[0]
    _check(lib().blitz_rope_kv_store(_p(qkv), _p(pos), _p(slot), _p(kv_layer), T, q_heads, kv_heads, head_dim,
                                     page_size, max_pages, rope_theta, _p(status_word(qkv.device)), _dt(qkv),
                                     _stream()), "blitz_rope_kv_store")


# ---------------------------------------------------------------------------------------------- attention
def attn_decode_workspace_bytes(batch: int, q_heads: int, head_dim: int, num_splits: int) -> int:
    return int(lib().blitz_attn_decode_workspace_bytes(batch, q_heads, head_dim, num_splits))


def attn_decode(q: torch.Tensor, kv_layer: torch.Tensor, indices: torch.Tensor, indptr: torch.Tensor,
                last_page_len: torch.Tensor, *, q_heads: int, kv_heads: int, head_dim: int, page_size: int,
                num_splits: int = 1, workspace: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                sm_scale: Optional[float] = None) -> torch.Tensor:
    """q: [batch, >= q_heads*head_dim] (row pitch free, e.g. a view of the fused qkv buffer)."""
    B = indptr.numel() - 1
    if out is None:
        out = torch.empty((B, q_heads * head_dim), dtype=q.dtype, device=q.device)
    if num_splits > 1 and workspace is None:
        workspace = torch.empty(attn_decode_workspace_bytes(B, q_heads, head_dim, num_splits), dtype=torch.uint8,
                                device=q.device)
    if sm_scale is None:
        sm_scale = head_dim ** -0.5
    _check(lib().blitz_attn_decode(_p(q), q.stride(0), _p(kv_layer), _p(indices), _p(indptr), _p(last_page_len),
                                   _p(out), out.stride(0), _p(workspace), B, q_heads, kv_heads, head_dim, page_size,
                                   kv_layer.shape[0], num_splits, sm_scale, _p(status_word(q.device)), _dt(q),
                                   _stream()), "blitz_attn_decode")
    return out


def prefill_work_list(q_lens, kv_lens, page_size: int, device) -> torch.Tensor:
    """Work records of `attn_prefill_paged`, one per (sequence, 256 rows of it): first row of the sequence in the
    activation, its rows in this pass, index of its first page id, number of its pages, tokens cached for it (this
    pass included), which 256-row pair.  Ordered by the number of key blocks the pair walks, heaviest first; the kernel
    deals the list back and forth over its CTAs."""
    items = []
    row0 = pg0 = 0
    for n, kv in zip(q_lens, kv_lens):
        n, kv = int(n), int(kv)
        npages = (kv + page_size - 1) // page_size
        for pair in range((n + 255) // 256):
            items.append((min(kv, kv - n + 256 * (pair + 1)), row0, n, pg0, npages, kv, pair))
        row0 += n
        pg0 += npages
    items.sort(key=lambda x: -x[0])
    rec = [[r0, n, p0, np_, kv, pair, 0, 0] for _, r0, n, p0, np_, kv, pair in items]
    return torch.tensor(rec, dtype=torch.int32).reshape(-1, 8).to(device, non_blocking=True)


def attn_prefill_paged(qkv: torch.Tensor, kv_layer: torch.Tensor, page_indices: torch.Tensor, work: torch.Tensor, *,
                       q_heads: int, kv_heads: int, head_dim: int, page_size: int, out: Optional[torch.Tensor] = None,
                       sm_scale: Optional[float] = None, poly_exp: bool = False) -> torch.Tensor:
    """Causal attention of the pass's rows over the paged cache (which already holds the rows' own keys and values,
    after whatever earlier passes stored).  ``qkv`` rotated (rope_kv_store); ``page_indices``: the sequences' page
    ids back to back, covering prefix + rows; ``work`` from `prefill_work_list` for the same sequences."""
    T = qkv.shape[0]
    if out is None:
        out = torch.empty((T, q_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    if sm_scale is None:
        sm_scale = head_dim ** -0.5
    assert work.dtype == torch.int32 and work.dim() == 2 and work.shape[1] == 8 and work.is_contiguous()
    max_pages = kv_layer.shape[0]
    _check(lib().blitz_attn_prefill_paged(_p(qkv), _p(kv_layer), _p(out), out.stride(0), _p(page_indices), _p(work),
                                          work.shape[0], T, q_heads, kv_heads, head_dim, page_size, max_pages, sm_scale,
                                          1 if poly_exp else 0, _p(status_word(qkv.device)), _dt(qkv), _stream()),
           "blitz_attn_prefill_paged")
    return out
