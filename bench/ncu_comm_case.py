"""Single-process cases of the NVLink kernels for ncu captures (one process, two GPUs, no process group).

ncu replays a captured kernel many times, so a multi-rank job cannot be profiled: a replayed kernel would wait for
a peer that has moved on.  Here one process owns both GPUs: the kernel under study runs on GPU 0 and its peer
pointers name buffers this process allocated on GPU 1.  Producer kernels (unit copy, KV push, GEMM with the push
epilogue) need nothing else.  Kernels that wait for a peer (reduce + norm + all-gather push, one-kernel all-reduce)
get their arrival counters set beforehand, as if the peer had already delivered; the counters are local memory of
the profiled GPU, so the profiler restores them between passes, and the wait budget is 10 ms in case it does not.
The switch-reduced kernels (multimem) need a multicast object, which only a process group can set up: they are
timed with CUDA events in bench/tp_bench.py instead.

    python bench/ncu_comm_case.py peer_copy [MB]        # peer_copy_units_kernel<false>, default 256 MB
    python bench/ncu_comm_case.py kv_push [TOKENS]      # kv_push_kernel, 32 layers x 8 KV heads x 128, default 2048 tokens
    python bench/ncu_comm_case.py push_gemm [M]         # gemm_tcgen05_kernel<..., push epilogue>, K = 4096, N = 8192
    python bench/ncu_comm_case.py reduce_norm [M]       # rs_reduce_norm_kernel, hidden 8192
    python bench/ncu_comm_case.py allreduce [M]         # allreduce_fused_kernel, hidden 8192
"""
import ctypes
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from blitz_scale_b200 import ops  # noqa: E402
from blitz_scale_b200.ops import _lib as _L  # noqa: E402


def vp(x):
    return ctypes.c_void_p(x.data_ptr() if isinstance(x, torch.Tensor) else int(x))


def main():
    kind = sys.argv[1]
    arg = int(sys.argv[2]) if len(sys.argv) > 2 else 0
    assert torch.cuda.device_count() >= 2, "needs two GPUs in one process"
    d0, d1 = torch.device("cuda", 0), torch.device("cuda", 1)
    torch.cuda.set_device(0)
    # peer access in both directions (torch enables it on the first cross-device copy)
    a, b = torch.zeros(16, device=d0), torch.zeros(16, device=d1)
    b.copy_(a)
    a.copy_(b)
    torch.cuda.synchronize()
    lib = ops.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = ops.status_word(d0)
    bf = torch.bfloat16
    pp = ctypes.c_void_p * 8

    if kind == "peer_copy":
        mb = arg or 256
        n = mb << 20
        src = torch.empty(n, dtype=torch.uint8, device=d0).random_()
        dst = torch.zeros(n, dtype=torch.uint8, device=d1)
        flags = torch.zeros(128, dtype=torch.int32, device=d1)
        tickets = torch.zeros(128, dtype=torch.int32, device=d0)
        units = 4
        offs = (ctypes.c_int64 * units)(*[i * (n // units) for i in range(units)])
        lens = (ctypes.c_int64 * units)(*[n // units] * units)
        bases = (ctypes.c_void_p * 1)(dst.data_ptr())
        fl = (ctypes.c_void_p * 1)(flags.data_ptr())
        for _ in range(3):
            tickets.zero_()
            rc = lib.blitz_peer_copy_units(vp(src), bases, fl, 1, ctypes.c_void_p(0), offs, lens, units, 0, 0, 1, vp(tickets),
                                           128, stream)
            assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.equal(dst.cpu()[:1 << 20], src.cpu()[:1 << 20])
    elif kind == "kv_push":
        tokens = arg or 2048
        layers, kvh, hd, page = 32, 8, 128, 64
        pages = tokens // page
        page_bytes = 2 * page * kvh * hd * 2
        pool_pages = pages + 8
        stride = pool_pages * page_bytes
        src = torch.empty(layers * stride, dtype=torch.uint8, device=d0).random_()
        dst = torch.zeros(layers * stride, dtype=torch.uint8, device=d1)
        sp = torch.randperm(pool_pages, device=d0)[:pages].to(torch.int32)
        dp = torch.randperm(pool_pages, device=d0)[:pages].to(torch.int32)
        flags = torch.zeros(256, dtype=torch.int32, device=d1)
        tickets = torch.zeros(layers, dtype=torch.int32, device=d0)
        for _ in range(3):
            tickets.zero_()
            rc = lib.blitz_kv_push(vp(src), vp(dst), vp(sp), vp(dp), pages, 0, layers, page_bytes, stride, stride, pool_pages,
                                   pool_pages, vp(flags), vp(tickets), 0, ctypes.c_void_p(0), vp(status), stream)
            assert rc == 0, rc
        torch.cuda.synchronize()
    elif kind == "push_gemm":
        from blitz_scale_b200.parallel.tp import _GemmTp
        M = arg or 4096
        K, N, tp = 4096, 8192, 2
        x = torch.randn(M, K, device=d0, dtype=bf)
        w = torch.randn(K, N, device=d0, dtype=bf) * K ** -0.5
        rpr = M // tp
        stage0 = torch.zeros(tp * rpr * N, dtype=bf, device=d0)
        stage1 = torch.zeros(tp * rpr * N, dtype=bf, device=d1)
        f0 = torch.zeros(32, dtype=torch.int32, device=d0)
        f1 = torch.zeros(32, dtype=torch.int32, device=d1)
        s = _GemmTp()
        s.tp, s.tp_rank, s.rows_per_rank = tp, 0, rpr
        s.push_base[0], s.push_base[1] = stage0.data_ptr(), stage1.data_ptr()
        s.push_flags[0], s.push_flags[1] = f0.data_ptr(), f1.data_ptr()
        ws, tickets = ops.gemm_workspace(d0)
        for _ in range(3):
            rc = lib.blitz_gemm_tp(vp(x), x.stride(0), vp(w), w.stride(0), ctypes.c_void_p(0), N, ctypes.c_void_p(0), M, N, K, 0,
                                   3, 0, 1, 0, 0, vp(ws), ws.numel(), vp(tickets), tickets.numel(), vp(status),
                                   ctypes.byref(s), stream)
            assert rc == 0, rc
        torch.cuda.synchronize()
    elif kind == "reduce_norm":
        M = arg or 4096
        H, tp = 8192, 2
        rpr = M // tp
        stage = torch.randn(tp * rpr * H, device=d0, dtype=bf)
        flag_rs = torch.zeros(64 * 8 + 8, dtype=torch.int32, device=d0)        # [block of 128 rows][source] + ticket
        res = torch.randn(rpr, H, device=d0, dtype=bf)
        nw = torch.ones(H, device=d0, dtype=bf)
        xg0 = torch.zeros(M, H, device=d0, dtype=bf)
        xg1 = torch.zeros(M, H, device=d1, dtype=bf)
        fa0 = torch.zeros(16, dtype=torch.int32, device=d0)
        fa1 = torch.zeros(16, dtype=torch.int32, device=d1)
        xg = (ctypes.c_void_p * tp)(xg0.data_ptr(), xg1.data_ptr())
        fl = (ctypes.c_void_p * tp)(fa0.data_ptr(), fa1.data_ptr())
        tiles_n = 7
        for _ in range(3):
            flag_rs[:64 * 8] = tiles_n     # as if both sources had pushed all their tiles of every block
            rc = lib.blitz_rs_reduce_norm(vp(stage), vp(flag_rs), tiles_n, vp(res), vp(nw), xg, fl, tp, 0, rpr, rpr, M, H,
                                          1e-5, int(10e6), vp(status), 1, stream)
            assert rc == 0, rc
        torch.cuda.synchronize()
    elif kind == "allreduce":
        M = arg or 256
        H, tp = 8192, 2
        n = M * H
        x = torch.randn(n, device=d0, dtype=bf)
        out = torch.empty(n, device=d0, dtype=bf)
        slots0 = torch.zeros(tp * n, device=d0, dtype=bf)
        slots1 = torch.zeros(tp * n, device=d1, dtype=bf)
        c0 = torch.zeros(8 * 64, dtype=torch.int32, device=d0)
        c1 = torch.zeros(8 * 64, dtype=torch.int32, device=d1)
        sl = (ctypes.c_void_p * tp)(slots0.data_ptr(), slots1.data_ptr())
        cf = (ctypes.c_void_p * tp)(c0.data_ptr(), c1.data_ptr())
        for _ in range(3):
            c0[64:128] = 1                 # as if rank 1 had delivered every block's chunk
            rc = lib.blitz_allreduce_fused(vp(x), sl, cf, vp(out), tp, 0, n, int(10e6), vp(status), 1, stream)
            assert rc == 0, rc
        torch.cuda.synchronize()
    else:
        raise SystemExit(f"unknown case {kind}")
    torch.cuda.synchronize()
    ops.check_status(d0)
    print("ok")


if __name__ == "__main__":
    main()
