"""Small single-kernel cases for ncu captures (inputs larger than L2, a few hundred MB on the device).

    python bench/ncu_case.py gemm M N K [epilogue]       # 3 launches of the tcgen05 GEMM
    python bench/ncu_case.py attn_decode B CTX            # 3 launches of the paged decode attention
    python bench/ncu_case.py attn_prefill_paged B N       # 3 launches of the paged prefill attention (64-token pages)
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from blitz_scale_b200 import ops  # noqa: E402


def main():
    kind = sys.argv[1]
    if kind == "gemm":
        M, N, K = map(int, sys.argv[2:5])
        epi = sys.argv[5] if len(sys.argv) > 5 else "store"
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(K, 2 * N if epi == "silu_mul" else N, device="cuda", dtype=torch.bfloat16)
        r = torch.randn(M, N, device="cuda", dtype=torch.bfloat16) if epi == "add" else None
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            ops.gemm(a, b, out=c, residual=r, epilogue=epi)
    elif kind == "attn_decode":
        B, ctx = map(int, sys.argv[2:4])
        qh, kvh, hd, page = 32, 8, 128, 64
        npg = (ctx + page - 1) // page
        kv = torch.randn(B * npg, 2, page, kvh, hd, device="cuda", dtype=torch.bfloat16)
        idx = torch.randperm(B * npg, device="cuda").to(torch.int32)
        indptr = (torch.arange(B + 1, device="cuda") * npg).to(torch.int32)
        last = torch.full((B,), ctx - (npg - 1) * page, device="cuda", dtype=torch.int32)
        q = torch.randn(B, qh * hd, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            ops.attn_decode(q, kv, idx, indptr, last, q_heads=qh, kv_heads=kvh, head_dim=hd, page_size=page)
    elif kind == "attn_prefill_paged":
        B, n = map(int, sys.argv[2:4])
        qh, kvh, hd, ps = 32, 8, 128, 64
        qkv = torch.randn(B * n, (qh + 2 * kvh) * hd, device="cuda", dtype=torch.bfloat16)
        npg = n // ps
        pool = torch.randn(B * npg, 2, ps, kvh, hd, device="cuda", dtype=torch.bfloat16)
        ids = torch.randperm(B * npg, device="cuda").to(torch.int32)
        work = ops.prefill_work_list([n] * B, [n] * B, ps, "cuda")
        for _ in range(3):
            ops.attn_prefill_paged(qkv, pool, ids, work, q_heads=qh, kv_heads=kvh, head_dim=hd, page_size=ps)
    elif kind == "decode_step":
        # two eager decode steps of the full model (no CUDA graph), for a per-kernel launch list of one step:
        #   ncu --metrics gpu__time_duration.sum -k regex:"blitz|gemm|attn|rms|rope|argmax|embedding|sample" ...
        # The KV pool stays zero (no prefill): the step does the same work on any data.
        from blitz_scale_b200.runtime import core
        from blitz_scale_b200.runtime.engine import Engine
        model = sys.argv[2]
        B, ctx = map(int, sys.argv[3:5])
        ps = 64
        eng = Engine(model, num_pages=B * ((ctx + 16 + ps) // ps + 1) + 8, page_size=ps, max_batch=max(B, 8),
                     max_batch_tokens=8192, seed=0, use_graphs=False)
        batch = eng.new_batch(0, [core.SeqSpec(i, [1] * ctx, 16) for i in range(B)])
        batch.mark_prefilled()
        batch.append_tokens([1] * B, False)
        batch.decode = True
        for _ in range(2):
            eng.decode(batch)
    torch.cuda.synchronize()
    ops.check_status()
    print("ok")


if __name__ == "__main__":
    main()
