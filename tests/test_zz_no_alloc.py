"""The allocation-free decode-attention entry point against the ordinary one.

Some hosts of this library cannot allocate device memory at the point where they call it (the GPU is
fully owned by their own pool, or the call sits inside a callback that must not allocate), so
`blitz_attn_decode_noalloc` keeps the split-KV scratch inside the library.  The test calls it through the
exported C symbol, twice in a row on different inputs (the built-in scratch keeps the first call's
contents), and compares with `blitz_attn_decode` fed a caller-allocated workspace.  It sits in its own
file, collected last, so a failure here cannot hide any other test's result.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = torch.bfloat16
SCRATCH_BYTES = 16 << 20
TOO_LARGE = -3


def _case(seed, lens, page, kvh, hd, dt=DT):
    g = torch.Generator().manual_seed(seed)
    npages = [(n + page - 1) // page for n in lens]
    total = sum(npages) + 2
    perm = torch.randperm(total, generator=g).tolist()
    kv = torch.zeros(total, 2, page, kvh, hd, dtype=dt)
    idx, indptr, last, cur = [], [0], [], 0
    for n, npg in zip(lens, npages):
        pg = perm[cur:cur + npg]
        cur += npg
        for i, p in enumerate(pg):
            m = min(n, (i + 1) * page) - i * page
            kv[p, :, :m] = torch.randn(2, m, kvh, hd, generator=g).to(dt)
        idx += pg
        indptr.append(len(idx))
        last.append(n - (npg - 1) * page)
    ti = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    return kv.cuda(), ti(idx), ti(indptr), ti(last)


def _entry():
    from blitz_scale_b200 import ops
    fn = ops.lib().blitz_attn_decode_noalloc
    c_i, c_i64, c_p, c_f = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float
    fn.argtypes = [c_p, c_i64, c_p, c_p, c_p, c_p, c_p, c_i64, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_f, c_p, c_i, c_p]
    fn.restype = c_i
    return ops, fn


def _allocations():
    """(free bytes on the device, allocations torch's caching allocator has made so far)."""
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0], torch.cuda.memory_stats().get("allocation.all.allocated", 0)


@pytest.mark.parametrize("dt,code,qh,kvh,hd,splits", [(torch.bfloat16, 1, 32, 8, 128, 4),
                                                      (torch.bfloat16, 1, 32, 8, 128, 1),
                                                      (torch.float16, 0, 16, 4, 64, 3)])
def test_noalloc_entry_matches_workspace_entry(dt, code, qh, kvh, hd, splits):
    ops, fn = _entry()
    page = 16
    c_p = ctypes.c_void_p
    stream = lambda: c_p(torch.cuda.current_stream().cuda_stream)
    status = ops.status_word()
    for seed, lens in ((1, [700, 33, 1, 2048]), (2, [64, 1500, 257])):    # two calls in a row, different shapes
        kv, idx, indptr, last = _case(seed, lens, page, kvh, hd, dt)
        B = len(lens)
        torch.manual_seed(seed)
        q = torch.randn(B, qh * hd, device="cuda", dtype=dt)
        ref = ops.attn_decode(q, kv, idx, indptr, last, q_heads=qh, kv_heads=kvh, head_dim=hd, page_size=page,
                              num_splits=splits)
        out = torch.full_like(ref, float("nan"))
        args = (q.data_ptr(), q.stride(0), kv.data_ptr(), idx.data_ptr(), indptr.data_ptr(), last.data_ptr(),
                out.data_ptr(), out.stride(0), B, qh, kvh, hd, page, kv.shape[0], splits, hd ** -0.5,
                status.data_ptr(), code, stream())
        # the first call on a device does the one-time set-up (symbol address, kernel attributes); the property in the
        # entry point's name is checked on the call after it: no device memory is taken, from the driver or from torch
        assert fn(*args) == 0
        before = _allocations()
        out.fill_(float("nan"))
        rc = fn(*args)
        assert rc == 0, rc
        after = _allocations()
        assert after == before, (before, after)
        ops.check_status()
        err = float((out.float() - ref.float()).norm() / ref.float().norm())
        assert err < 1e-2, err


def test_noalloc_entry_refuses_more_than_its_scratch():
    ops, fn = _entry()
    qh, kvh, hd, page = 32, 8, 128, 16
    kv, idx, indptr, last = _case(3, [64, 5], page, kvh, hd)
    q = torch.randn(2, qh * hd, device="cuda", dtype=DT)
    out = torch.empty_like(q)
    # a request beyond the built-in scratch is refused, and nothing is launched
    big_b = SCRATCH_BYTES // (qh * 32 * (hd + 1) * 4) + 1
    rc = fn(q.data_ptr(), q.stride(0), kv.data_ptr(), idx.data_ptr(), indptr.data_ptr(), last.data_ptr(),
            out.data_ptr(), out.stride(0), big_b, qh, kvh, hd, page, kv.shape[0], 32, hd ** -0.5, None, 1,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == TOO_LARGE
    torch.cuda.synchronize()
