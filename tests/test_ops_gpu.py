"""GPU numerics of every hand-written kernel against a plain PyTorch fp32 reference of the same op."""

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = torch.bfloat16


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


@pytest.fixture(scope="module")
def ops():
    from blitz_scale_b200 import ops as o
    o.lib()  # must load the in-tree kernel library; no fallback
    return o


@pytest.fixture(autouse=True)
def _status(ops):
    yield
    ops.check_status()


# ------------------------------------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 256), (16, 512, 128), (200, 384, 320),
                                   (256, 4096, 4096), (1000, 1024, 2048)])
@pytest.mark.parametrize("layout", ["kn", "nk"])
def test_gemm_store(ops, M, N, K, layout):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=DT)
    b = torch.randn(K, N, device="cuda", dtype=DT) * K ** -0.5
    ref = a.float() @ b.float()
    bb = b if layout == "kn" else b.t().contiguous()
    for bn in (0, 64, 128, 256):
        out = ops.gemm(a, bb, b_layout=layout, bn=bn)
        torch.cuda.synchronize()
        assert rel_err(out, ref) < 1e-2, (bn, rel_err(out, ref))


@pytest.mark.parametrize("M,N,K", [(64, 256, 128), (300, 1408, 512)])
def test_gemm_add_and_silu(ops, M, N, K):
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda", dtype=DT)
    b = torch.randn(K, N, device="cuda", dtype=DT) * K ** -0.5
    r = torch.randn(M, N, device="cuda", dtype=DT)
    ref = a.float() @ b.float() + r.float()
    out = ops.gemm(a, b, residual=r, epilogue="add")
    assert rel_err(out, ref) < 1e-2
    # in-place residual update
    r2 = r.clone()
    ops.gemm(a, b, out=r2, residual=r2, epilogue="add")
    assert rel_err(r2, ref) < 1e-2
    gu = torch.randn(K, 2 * N, device="cuda", dtype=DT) * K ** -0.5
    acc = a.float() @ gu.float()
    ref2 = torch.nn.functional.silu(acc[:, :N]) * acc[:, N:]
    for bn in (0, 128, 256):
        out2 = ops.gemm(a, gu, epilogue="silu_mul", bn=bn)
        assert rel_err(out2, ref2) < 1e-2, bn
    out3 = ops.gemm(a, gu.t().contiguous(), epilogue="silu_mul", b_layout="nk")
    assert rel_err(out3, ref2) < 1e-2


@pytest.mark.parametrize("M,N,K", [(16, 4096, 4096), (256, 4096, 14336), (40, 1408, 1024)])
def test_gemm_split_k(ops, M, N, K):
    """Skinny GEMMs split K across CTAs and reduce in-kernel; every split count gives the same result."""
    torch.manual_seed(11)
    a = torch.randn(M, K, device="cuda", dtype=DT)
    b = torch.randn(K, N, device="cuda", dtype=DT) * K ** -0.5
    r = torch.randn(M, N, device="cuda", dtype=DT)
    ref = a.float() @ b.float()
    base = ops.gemm(a, b, split_k=1)
    assert rel_err(base, ref) < 1e-2
    for s in (0, 2, 5, 16):
        out = ops.gemm(a, b, split_k=s)
        assert rel_err(out, ref) < 1e-2, s
        again = ops.gemm(a, b, split_k=s)
        assert torch.equal(out, again), "split-K reduction must be deterministic"
    assert rel_err(ops.gemm(a, b, residual=r, epilogue="add", split_k=0), ref + r.float()) < 1e-2
    gu = torch.randn(K, 2 * N, device="cuda", dtype=DT) * K ** -0.5
    acc = a.float() @ gu.float()
    ref2 = torch.nn.functional.silu(acc[:, :N]) * acc[:, N:]
    assert rel_err(ops.gemm(a, gu, epilogue="silu_mul", split_k=4), ref2) < 1e-2


@pytest.mark.parametrize("M", [1, 7, 16, 33, 100, 128, 200, 256])
@pytest.mark.parametrize("N,K", [(4096, 4096), (1088, 520), (6144, 1024)])
def test_gemm_decode_path(ops, M, N, K):
    """Weight-streaming decode GEMM (swapped operands, cluster split-K with the reduction in distributed shared
    memory): every cluster size gives the right result, and the same one on every run."""
    torch.manual_seed(13)
    a = torch.randn(M, K, device="cuda", dtype=DT)
    b = torch.randn(K, N, device="cuda", dtype=DT) * K ** -0.5
    r = torch.randn(M, N, device="cuda", dtype=DT)
    ref = a.float() @ b.float()
    gu = torch.randn(K, 2 * N, device="cuda", dtype=DT) * K ** -0.5
    acc = a.float() @ gu.float()
    ref2 = torch.nn.functional.silu(acc[:, :N]) * acc[:, N:]
    for split in (0, 1, 2, 3, 8):
        out = ops.gemm(a, b, decode_path=True, decode_split=split)
        assert rel_err(out, ref) < 1e-2, (split, rel_err(out, ref))
        assert torch.equal(out, ops.gemm(a, b, decode_path=True, decode_split=split, static_b=True)), "must be deterministic"
        r2 = r.clone()
        ops.gemm(a, b, out=r2, residual=r2, epilogue="add", decode_path=True, decode_split=split)
        assert rel_err(r2, ref + r.float()) < 1e-2, split
        assert rel_err(ops.gemm(a, gu, epilogue="silu_mul", decode_path=True, decode_split=split), ref2) < 1e-2, split
    ops.check_status()


@pytest.mark.parametrize("M", [129, 200, 256, 640])
@pytest.mark.parametrize("N,K", [(4096, 4096), (1088, 520), (6144, 1024)])
def test_gemm_pair_path(ops, M, N, K):
    """Paired-SM GEMM (one 256-row tcgen05.mma over two CTAs, stream-K over CTA pairs): every tile width and every
    cut of the unit range gives the right result, and the same one on every run (partials are summed in pair order)."""
    torch.manual_seed(17)
    a = torch.randn(M, K, device="cuda", dtype=DT)
    b = torch.randn(K, N, device="cuda", dtype=DT) * K ** -0.5
    r = torch.randn(M, N, device="cuda", dtype=DT)
    ref = a.float() @ b.float()
    gu = torch.randn(K, 2 * N, device="cuda", dtype=DT) * K ** -0.5
    acc = a.float() @ gu.float()
    ref2 = torch.nn.functional.silu(acc[:, :N]) * acc[:, N:]
    nkb = (K + 63) // 64
    for bnf, nacc in ((0, 0), (128, 1), (128, 2), (256, 1), (256, 2)):
        for upp in (0, nkb, max(1, nkb // 2), (nkb + 2) // 3 + 1, 3 * nkb + 1, -2, -3, -4):
            kw = dict(pair_path=True, pair_bnf=bnf, pair_nacc=nacc, pair_upp=upp)
            out = ops.gemm(a, b, **kw)
            assert rel_err(out, ref) < 1e-2, (bnf, nacc, upp, rel_err(out, ref))
            assert torch.equal(out, ops.gemm(a, b, static_b=True, **kw)), "must be deterministic"
            r2 = r.clone()
            ops.gemm(a, b, out=r2, residual=r2, epilogue="add", **kw)
            assert rel_err(r2, ref + r.float()) < 1e-2, (bnf, nacc, upp)
            out2 = ops.gemm(a, gu, epilogue="silu_mul", **kw)
            assert rel_err(out2, ref2) < 1e-2, (bnf, nacc, upp)
    ops.check_status()


def test_gemm_pair_fp16_and_pdl_chain(ops):
    torch.manual_seed(18)
    a = torch.randn(192, 768, device="cuda", dtype=torch.float16)
    w1 = torch.randn(768, 1536, device="cuda", dtype=torch.float16) / 28
    w2 = torch.randn(1536, 768, device="cuda", dtype=torch.float16) / 39
    torch.cuda.synchronize()
    # back-to-back dependent launches share the partial scratch: the second waits for the first before it writes
    h = ops.gemm(a, w1, pair_path=True, static_b=True, pair_upp=5)
    y = ops.gemm(h, w2, pair_path=True, static_b=True, pair_upp=7)
    ref_h = (a.float() @ w1.float()).to(torch.float16)
    assert rel_err(h, a.float() @ w1.float()) < 5e-3
    assert rel_err(y, ref_h.float() @ w2.float()) < 5e-3
    ops.check_status()


def test_gemm_decode_fp16_and_pdl_chain(ops):
    torch.manual_seed(14)
    a = torch.randn(48, 768, device="cuda", dtype=torch.float16)
    w1 = torch.randn(768, 1536, device="cuda", dtype=torch.float16) / 28
    w2 = torch.randn(1536, 768, device="cuda", dtype=torch.float16) / 39
    torch.cuda.synchronize()
    # back-to-back dependent launches: the second GEMM prefetches its weights before the first has finished
    h = ops.gemm(a, w1, decode_path=True, static_b=True)
    y = ops.gemm(h, w2, decode_path=True, static_b=True)
    ref_h = (a.float() @ w1.float()).to(torch.float16)
    assert rel_err(h, a.float() @ w1.float()) < 5e-3
    assert rel_err(y, ref_h.float() @ w2.float()) < 5e-3
    ops.check_status()


def test_gemm_fp16(ops):
    torch.manual_seed(2)
    a = torch.randn(96, 256, device="cuda", dtype=torch.float16)
    b = torch.randn(256, 320, device="cuda", dtype=torch.float16) / 16
    assert rel_err(ops.gemm(a, b), a.float() @ b.float()) < 5e-3


# ------------------------------------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("T,H", [(7, 256), (33, 4096), (5, 8192)])
def test_norms(ops, T, H):
    torch.manual_seed(3)
    x = torch.randn(T, H, device="cuda", dtype=DT)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(DT)
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert rel_err(ops.rms_norm(x, w, 1e-5), ref) < 1e-2
    res = torch.randn(T, H, device="cuda", dtype=DT)
    s = (res.float() + x.float()).to(DT)
    ref2 = s.float() * torch.rsqrt(s.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    res2 = res.clone()
    out = ops.add_rms_norm(x, res2, w, 1e-5)
    assert rel_err(res2, s) < 1e-3 and rel_err(out, ref2) < 1e-2


def test_silu_add_embed_gather(ops):
    torch.manual_seed(4)
    x = torch.randn(9, 2 * 688, device="cuda", dtype=DT)
    ref = torch.nn.functional.silu(x[:, :688].float()) * x[:, 688:].float()
    assert rel_err(ops.silu_mul(x), ref) < 1e-2
    a = torch.randn(9, 512, device="cuda", dtype=DT)
    b = torch.randn(9, 512, device="cuda", dtype=DT)
    ref = a.float() + b.float()
    assert rel_err(ops.add_residual(a, b), ref) < 1e-2
    table = torch.randn(1000, 256, device="cuda", dtype=DT)
    ids = torch.randint(0, 1000, (37,), device="cuda", dtype=torch.int32)
    assert torch.equal(ops.embedding(ids, table), table[ids.long()])
    # vocab shard [500, 1000): rows owned elsewhere are zero
    shard = table[500:]
    out = ops.embedding(ids, shard, vocab_start=500)
    exp = torch.where((ids >= 500)[:, None], table[ids.long()], torch.zeros_like(table[ids.long()]))
    assert torch.equal(out, exp)
    indptr = torch.tensor([0, 3, 10, 37], device="cuda", dtype=torch.int32)
    xs = torch.randn(37, 256, device="cuda", dtype=DT)
    assert torch.equal(ops.gather_last(xs, indptr), xs[[2, 9, 36]])


def test_argmax_and_sampling(ops):
    torch.manual_seed(5)
    lg = torch.randn(6, 128256, device="cuda", dtype=DT)
    lg[2, 77] = lg[2, 90001] = 50.0  # tie -> smallest index
    out = ops.argmax(lg)
    assert torch.equal(out.long(), lg.float().argmax(-1)) or int(out[2]) == 77
    assert int(out[2]) == 77
    vals = torch.empty(6, device="cuda")
    out2 = ops.argmax(lg, out_val=vals, idx_offset=1000)
    assert torch.equal(out2, out + 1000) and torch.allclose(vals, lg.float().max(-1).values)
    # sampling: top_k = 1 is greedy; draws stay inside the top-k set; frequencies follow the softmax
    B, V = 4, 4096
    lg = torch.randn(B, V, device="cuda", dtype=DT) * 2
    temp = torch.ones(B, device="cuda")
    topp = torch.ones(B, device="cuda")
    seeds = torch.arange(B, device="cuda", dtype=torch.int64) + 11
    k1 = torch.ones(B, device="cuda", dtype=torch.int32)
    s1 = ops.sample(lg, temp, k1, topp, seeds, 0).long()
    # top_k = 1 keeps the maximum (all tokens tied at the maximum stay eligible)
    assert torch.equal(lg.float().gather(1, s1[:, None])[:, 0], lg.float().max(-1).values)
    k8 = torch.full((B,), 8, device="cuda", dtype=torch.int32)
    top8 = lg.float().topk(8, -1).indices
    counts = torch.zeros(B, V)
    for step in range(300):
        s = ops.sample(lg, temp, k8, topp, seeds, step).long()
        assert all(int(s[i]) in top8[i].tolist() for i in range(B))
        counts[torch.arange(B), s.cpu()] += 1
    p = torch.softmax(lg.float().cpu().gather(1, top8.cpu()), -1)
    f = counts.gather(1, top8.cpu()) / 300
    assert float((p - f).abs().max()) < 0.12
    # top_p small keeps only the head of the distribution
    sharp = torch.zeros(1, V, device="cuda", dtype=DT)
    sharp[0, 5] = 10.0
    tp = torch.full((1,), 0.5, device="cuda")
    k0 = torch.zeros(1, device="cuda", dtype=torch.int32)
    for step in range(20):
        assert int(ops.sample(sharp, temp[:1], k0, tp, seeds[:1], step)) == 5


def _rope_ref(x, pos, theta):
    from blitz_scale_b200.models.oracle import rope_ref
    return rope_ref(x, pos, theta)


@pytest.mark.parametrize("hd,page", [(128, 16), (64, 64)])
def test_rope_kv_store(ops, hd, page):
    torch.manual_seed(6)
    T, qh, kvh, pages = 50, 4, 2, 12
    qkv = torch.randn(T, (qh + 2 * kvh) * hd, device="cuda", dtype=DT)
    pos = torch.randint(0, 3000, (T,), device="cuda", dtype=torch.int32)
    perm = torch.randperm(pages * page)[:T]
    slot = perm.to(device="cuda", dtype=torch.int32)
    slot[3] = -1
    kv = torch.zeros(pages, 2, page, kvh, hd, device="cuda", dtype=DT)
    orig = qkv.clone()
    ops.rope_kv_store(qkv, pos, slot, kv, q_heads=qh, kv_heads=kvh, head_dim=hd, page_size=page, rope_theta=5e5)
    q_ref = _rope_ref(orig[:, :qh * hd].view(T, qh, hd), pos, 5e5)
    k_ref = _rope_ref(orig[:, qh * hd:(qh + kvh) * hd].view(T, kvh, hd), pos, 5e5)
    v_ref = orig[:, (qh + kvh) * hd:].view(T, kvh, hd)
    assert rel_err(qkv[:, :qh * hd].view(T, qh, hd), q_ref) < 1e-2
    assert rel_err(qkv[:, qh * hd:(qh + kvh) * hd].view(T, kvh, hd), k_ref) < 1e-2
    flat = kv.view(pages, 2, page, kvh, hd)
    for t in range(T):
        s = int(slot[t])
        if s < 0:
            continue
        assert rel_err(flat[s // page, 0, s % page], k_ref[t]) < 1e-2
        assert torch.equal(flat[s // page, 1, s % page], v_ref[t])


# ------------------------------------------------------------------------------------------------ attention
def _paged_setup(B, lens, page, kvh, hd, seed):
    g = torch.Generator().manual_seed(seed)
    npages = [(n + page - 1) // page for n in lens]
    total = sum(npages) + 3
    perm = torch.randperm(total, generator=g)
    kv = torch.zeros(total, 2, page, kvh, hd, dtype=DT)
    ks, vs, idx, indptr, last = [], [], [], [0], []
    cur = 0
    for b, n in enumerate(lens):
        k = torch.randn(n, kvh, hd, generator=g).to(DT)
        v = torch.randn(n, kvh, hd, generator=g).to(DT)
        pg = perm[cur:cur + npages[b]].tolist()
        cur += npages[b]
        for i, p in enumerate(pg):
            seg = slice(i * page, min(n, (i + 1) * page))
            kv[p, 0, :seg.stop - seg.start] = k[seg]
            kv[p, 1, :seg.stop - seg.start] = v[seg]
        ks.append(k); vs.append(v); idx += pg; indptr.append(len(idx)); last.append(n - (npages[b] - 1) * page if n else 0)
    ti = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    return kv.cuda(), ks, vs, ti(idx), ti(indptr), ti(last)


@pytest.mark.parametrize("hd,qh,kvh,page", [(128, 32, 8, 16), (128, 8, 8, 64), (64, 4, 2, 64), (128, 16, 2, 64)])
@pytest.mark.parametrize("splits", [1, 3])
def test_attn_decode(ops, hd, qh, kvh, page, splits):
    lens = [1, 17, 64, 200, 1031, 5]
    B = len(lens)
    kv, ks, vs, idx, indptr, last = _paged_setup(B, lens, page, kvh, hd, 7)
    torch.manual_seed(8)
    q = torch.randn(B, qh * hd, device="cuda", dtype=DT)
    out = ops.attn_decode(q, kv, idx, indptr, last, q_heads=qh, kv_heads=kvh, head_dim=hd, page_size=page,
                          num_splits=splits)
    g = qh // kvh
    for b in range(B):
        k = ks[b].cuda().float().repeat_interleave(g, 1)
        v = vs[b].cuda().float().repeat_interleave(g, 1)
        s = torch.einsum("hd,shd->hs", q[b].view(qh, hd).float(), k) * hd ** -0.5
        ref = torch.einsum("hs,shd->hd", s.softmax(-1), v).reshape(-1)
        assert rel_err(out[b], ref) < 1e-2, (b, rel_err(out[b], ref))


def test_attn_decode_simt_matches_tc(ops):
    """The CUDA-core kernel (kept as a cross-check) and the tensor-core kernel agree."""
    import ctypes
    lens = [33, 400, 64]
    kv, ks, vs, idx, indptr, last = _paged_setup(3, lens, 16, 2, 128, 21)
    q = torch.randn(3, 8 * 128, device="cuda", dtype=DT)
    a = ops.attn_decode(q, kv, idx, indptr, last, q_heads=8, kv_heads=2, head_dim=128, page_size=16)
    b = torch.empty_like(a)
    L = ops.lib()
    L.blitz_attn_decode_simt.argtypes = L.blitz_attn_decode.argtypes
    rc = L.blitz_attn_decode_simt(q.data_ptr(), q.stride(0), kv.data_ptr(), idx.data_ptr(), indptr.data_ptr(),
                                  last.data_ptr(), b.data_ptr(), b.stride(0), None, 3, 8, 2, 128, 16, kv.shape[0], 1,
                                  128 ** -0.5, None, 1, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0 and rel_err(a, b) < 1e-2


@pytest.mark.parametrize("qh,kvh,hd,ps,dt,cases", [
    (8, 2, 128, 16, torch.bfloat16, [(300, 0), (128, 0), (1, 0), (77, 200), (513, 256)]),
    (4, 4, 128, 64, torch.float16, [(256, 0), (257, 129), (40, 1000)]),
    (6, 2, 64, 64, torch.bfloat16, [(700, 0), (130, 64), (5, 0)]),
    (8, 1, 64, 8, torch.bfloat16, [(260, 24)]),
])
@pytest.mark.parametrize("poly", [False, True])
def test_attn_prefill_paged(ops, qh, kvh, hd, ps, dt, cases, poly):
    """Chunk rows against prefix + chunk in the paged pool, two ping-ponged query tiles per CTA, against fp32 math.
    (q_len, prefix) per sequence; pages are scattered over the pool; stale pool contents are finite garbage."""
    torch.manual_seed(5)
    T = sum(n for n, _ in cases)
    qkv = torch.randn(T, (qh + 2 * kvh) * hd, device="cuda", dtype=dt)
    need = sum((n + pre + ps - 1) // ps for n, pre in cases)
    pool_pages = need + 7
    pool = (torch.randn(pool_pages, 2, ps, kvh, hd, device="cuda") * 3).to(dt)      # garbage where nothing is stored
    perm = torch.randperm(pool_pages).tolist()
    tok_indptr, page_indptr, page_ids, last = [0], [0], [], []
    full = []
    o = 0
    for n, pre in cases:
        kv_len = n + pre
        npg = (kv_len + ps - 1) // ps
        mine = [perm.pop() for _ in range(npg)]
        k = torch.randn(kv_len, kvh, hd, device="cuda", dtype=dt)
        v = torch.randn(kv_len, kvh, hd, device="cuda", dtype=dt)
        # the chunk's own keys and values are what its qkv rows carry
        k[pre:] = qkv[o:o + n, qh * hd:(qh + kvh) * hd].view(n, kvh, hd)
        v[pre:] = qkv[o:o + n, (qh + kvh) * hd:].view(n, kvh, hd)
        for t in range(kv_len):
            pool[mine[t // ps], 0, t % ps] = k[t]
            pool[mine[t // ps], 1, t % ps] = v[t]
        full.append((k, v))
        page_ids += mine
        tok_indptr.append(tok_indptr[-1] + n)
        page_indptr.append(page_indptr[-1] + npg)
        last.append(kv_len - (npg - 1) * ps)
        o += n
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    q_lens = [n for n, _ in cases]
    kv_lens = [n + pre for n, pre in cases]
    work = ops.prefill_work_list(q_lens, kv_lens, ps, "cuda")
    assert work.shape == (sum((n + 255) // 256 for n in q_lens), 8)
    out = ops.attn_prefill_paged(qkv, pool, dev(page_ids), work, q_heads=qh, kv_heads=kvh, head_dim=hd, page_size=ps,
                                 poly_exp=poly)
    # the order of the work list does not matter
    out2 = ops.attn_prefill_paged(qkv, pool, dev(page_ids), work.flip(0).contiguous(), q_heads=qh, kv_heads=kvh,
                                  head_dim=hd, page_size=ps, poly_exp=poly)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(out, out2)
    g = qh // kvh
    o = 0
    for (n, pre), (k, v) in zip(cases, full):
        q = qkv[o:o + n, :qh * hd].view(n, qh, hd).float()
        kk = k.float().repeat_interleave(g, 1)
        vv = v.float().repeat_interleave(g, 1)
        s_ = torch.einsum("thd,shd->hts", q, kk) * hd ** -0.5
        mask = torch.arange(n + pre, device="cuda")[None, :] > (pre + torch.arange(n, device="cuda"))[:, None]
        s_ = s_.masked_fill(mask[None], float("-inf"))
        ref = torch.einsum("hts,shd->thd", s_.softmax(-1), vv).reshape(n, qh * hd)
        assert rel_err(out[o:o + n], ref) < 1e-2, (n, pre, rel_err(out[o:o + n], ref))
        o += n


def test_attn_prefill_paged_rescales_when_the_maximum_grows(ops):
    """Scores that grow steeply along the sequence force the in-place rescaling of the output rows in tensor memory."""
    torch.manual_seed(6)
    qh = kvh = 1
    hd, ps, n = 128, 64, 512
    qkv = torch.zeros(n, 3 * hd, device="cuda", dtype=torch.bfloat16)
    q = torch.zeros(n, hd, device="cuda")
    k = torch.zeros(n, hd, device="cuda")
    q[:, 0] = 8.0
    k[:, 0] = torch.arange(n, device="cuda") * 0.25          # score of key s = 2 s / sqrt(128) * ... grows by far more than 2^8 in all
    v = torch.randn(n, hd, device="cuda")
    qkv[:, :hd], qkv[:, hd:2 * hd], qkv[:, 2 * hd:] = q.bfloat16(), k.bfloat16(), v.bfloat16()
    pool = torch.zeros(n // ps, 2, ps, 1, hd, device="cuda", dtype=torch.bfloat16)
    pool[:, 0] = qkv[:, hd:2 * hd].view(n // ps, ps, 1, hd)
    pool[:, 1] = qkv[:, 2 * hd:].view(n // ps, ps, 1, hd)
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    out = ops.attn_prefill_paged(qkv, pool, dev(list(range(n // ps))), ops.prefill_work_list([n], [n], ps, "cuda"),
                                 q_heads=qh, kv_heads=kvh, head_dim=hd, page_size=ps)
    torch.cuda.synchronize()
    ops.check_status()
    qf, kf, vf = (qkv[:, i * hd:(i + 1) * hd].float() for i in range(3))
    s_ = (qf @ kf.T) * hd ** -0.5
    s_ = s_.masked_fill(torch.ones(n, n, device="cuda").triu(1).bool(), float("-inf"))
    ref = s_.softmax(-1) @ vf
    assert float((s_.max(-1).values[-1] - s_.max(-1).values[0]) * 1.4427) > 32     # far beyond one rescale threshold
    assert rel_err(out, ref) < 1e-2, rel_err(out, ref)
