"""CPU tests of the native runtime core: model shape table, weight-segment layout (closed form), segment files and
the native loader (byte-exact reload), batch metadata for the attention kernels, the ZigZag layer scheduler
(deterministic cases plus a randomised interleaving of parameter arrival, execution and relays), and the PyTorch
oracle's KV-cache consistency.  No GPU."""
import random

import numpy as np
import pytest
import torch

from blitz_scale_b200.models.config import ALIGN_BYTES, REGISTRY, build_layout, get_config
from blitz_scale_b200.models.oracle import LlamaOracle
from blitz_scale_b200.models.weights import WeightSegment, shard_from_full
from blitz_scale_b200.runtime import core


# ------------------------------------------------------------------------------------------------ shape table
def test_native_and_python_shape_tables_agree():
    names = set(core.model_names())
    assert names == set(REGISTRY)
    for fam in ("opt_125m", "opt_30b", "llama2_7b", "llama2_70b", "llama3_8b", "mistral_13b", "mistral_24b", "qwen_72b"):
        assert fam in names
    for n in names:
        c, p = core.get_model(n), get_config(n)
        assert (c.vocab, c.hidden, c.layers, c.q_heads, c.kv_heads, c.head_dim, c.inter) == \
               (p.vocab, p.hidden, p.layers, p.q_heads, p.kv_heads, p.head_dim, p.inter), n
        assert c.rope_theta == pytest.approx(p.rope_theta) and c.rms_eps == pytest.approx(p.rms_eps)
        for tp in (1, 2):
            if p.kv_heads % tp == 0:
                assert c.kv_bytes_per_token(tp, 2) == p.kv_bytes_per_token(tp, 2)
    l3 = core.get_model("llama3_8b")
    assert (l3.vocab, l3.hidden, l3.layers, l3.q_heads, l3.kv_heads, l3.head_dim, l3.inter) == (128256, 4096, 32, 32, 8, 128, 14336)
    assert l3.kv_bytes_per_token(1, 2) == 2 * 8 * 128 * 2 * 32      # 128 KiB per token, as the sizing tools assume
    with pytest.raises(Exception):
        core.get_model("no_such_model")


# ------------------------------------------------------------------------------------------------ segment layout
def _closed_form_elements(cfg, tp):
    """Elements of one TP rank's segment: vocab-sharded embedding and head, per layer two norms, fused QKV, O, fused
    gate/up and down; one final norm (the head unit)."""
    h, hd = cfg.hidden, cfg.head_dim
    qh, kvh, it = cfg.q_heads // tp, cfg.kv_heads // tp, cfg.inter // tp
    per_layer = 2 * h + h * (qh + 2 * kvh) * hd + qh * hd * h + h * 2 * it + it * h
    return (cfg.vocab // tp) * h, per_layer, h + h * (cfg.vocab // tp)


@pytest.mark.parametrize("name,tp", [("tiny", 1), ("tiny", 2), ("llama3_8b", 1), ("llama3_8b", 4), ("mistral_24b", 2),
                                     ("qwen_72b", 8), ("llama2_70b", 4)])
def test_segment_layout_matches_closed_form_and_native_layout(name, tp):
    cfg = get_config(name)
    py = build_layout(cfg, tp, 2)
    nat = core.build_segment_layout(name, tp, 2)
    assert nat.total_bytes == py.total_bytes
    assert [(u.name, u.offset, u.nbytes) for u in nat.units] == [tuple(u) for u in py.units]
    assert {t.name: (t.offset, t.nbytes, tuple(t.shape)) for t in nat.tensors} == \
           {t.name: (t.offset, t.nbytes, tuple(t.shape)) for t in py.tensors.values()}
    # units: embed | layer 0..L-1 | head, contiguous, aligned, covering the whole segment
    assert [u[0] for u in py.units] == ["embed"] + [f"layer.{i}" for i in range(cfg.layers)] + ["head"]
    end = 0
    for _, off, nb in py.units:
        assert off == end and off % ALIGN_BYTES == 0 and nb % ALIGN_BYTES == 0
        end = off + nb
    assert end == py.total_bytes
    # tensors: aligned, inside their unit, never overlapping
    spans = sorted((t.offset, t.offset + t.nbytes) for t in py.tensors.values())
    for (a0, a1), (b0, _) in zip(spans, spans[1:]):
        assert a1 <= b0
    assert all(t.offset % ALIGN_BYTES == 0 for t in py.tensors.values())
    # payload equals the closed form; what remains is alignment padding, less than one unit of it per tensor
    e_embed, e_layer, e_head = _closed_form_elements(cfg, tp)
    payload = sum(t.nbytes for t in py.tensors.values())
    assert payload == 2 * (e_embed + cfg.layers * e_layer + e_head)
    assert 0 <= py.total_bytes - payload < ALIGN_BYTES * len(py.tensors)
    # every layer unit has the same size, so a layer's offset is a closed form of its index
    l0 = py.unit("layer.0")
    for i in (1, cfg.layers - 1):
        assert py.unit(f"layer.{i}") == (l0[0] + i * l0[1], l0[1])


def test_tp_shards_partition_the_full_weights():
    cfg = get_config("tiny")
    full = WeightSegment(cfg, 1, 0, dtype=torch.float32).random_init_(3)
    shards = [shard_from_full(full, 2, r) for r in range(2)]
    hd, qh, kvh = cfg.head_dim, cfg.q_heads, cfg.kv_heads
    wqkv = full["layers.0.qkv"]                      # [hidden, (qh + 2 kvh) * hd]
    q, k, v = wqkv[:, :qh * hd], wqkv[:, qh * hd:(qh + kvh) * hd], wqkv[:, (qh + kvh) * hd:]
    for r, s in enumerate(shards):
        sq, sk = qh // 2 * hd, kvh // 2 * hd
        want = torch.cat([q[:, r * sq:(r + 1) * sq], k[:, r * sk:(r + 1) * sk], v[:, r * sk:(r + 1) * sk]], dim=1)
        assert torch.equal(s["layers.0.qkv"], want)                            # column-parallel by heads
        assert torch.equal(s["layers.0.o"], full["layers.0.o"][r * sq:(r + 1) * sq])   # row-parallel
        assert torch.equal(s["layers.0.input_ln"], full["layers.0.input_ln"])           # replicated
    assert torch.equal(torch.cat([s["embed"] for s in shards], 0), full["embed"])   # vocab-parallel


# ------------------------------------------------------------------------------------------------ files + loader
def test_segment_file_reloads_byte_exactly_through_the_native_loader(tmp_path):
    cfg = get_config("tiny")
    seg = WeightSegment(cfg, 1, 0).random_init_(11)
    path = seg.save(tmp_path)
    assert path.stat().st_size == seg.layout.total_bytes
    WeightSegment.check_sidecar(tmp_path, cfg, 1, 0, torch.bfloat16)
    with pytest.raises(Exception):
        WeightSegment.check_sidecar(tmp_path, get_config("tiny_gpu"), 1, 0, torch.bfloat16)      # wrong model: refused
    dst = torch.zeros(seg.layout.total_bytes, dtype=torch.uint8)
    for threads, chunk in ((1, 1 << 16), (3, 1 << 12)):
        dst.zero_()
        res = core.load_file_to_host(str(path), dst.data_ptr(), seg.layout.total_bytes, threads, chunk)
        assert res.bytes == seg.layout.total_bytes and res.seconds >= 0
        assert torch.equal(dst, seg.buffer.view(torch.uint8)[:seg.layout.total_bytes].cpu())
    with pytest.raises(Exception):
        core.load_file_to_host(str(path), dst.data_ptr(), seg.layout.total_bytes + 4096)           # size mismatch
    with pytest.raises(Exception):
        core.load_file_to_host(str(tmp_path / "missing.bin"), dst.data_ptr(), -1)


# ------------------------------------------------------------------------------------------------ batch metadata
def test_batch_metadata_for_prefill_and_decode():
    ps = 16
    pool = core.PagePool(32, ps)
    b = core.Batch(7, pool)
    lens = [5, 16, 33]
    assert b.add_prompts([core.SeqSpec(i, list(range(100 * i, 100 * i + n)), 4) for i, n in enumerate(lens)])
    assert b.size == 3 and b.num_prompt_tokens() == sum(lens) and b.max_seq_len() == 33
    pages = [list(s.pages) for s in b.seqs]
    assert [len(p) for p in pages] == [(n + 1 + ps - 1) // ps for n in lens]     # room for the first new token
    L = core.MetaLayout.make(64, 4, 32)
    h = np.full(L.total, -7, dtype=np.int32)
    T, P = b.fill_prefill(h, L)
    used = [(n + ps - 1) // ps for n in lens]
    assert (T, P) == (sum(lens), sum(used))
    assert list(h[L.tok_indptr:L.tok_indptr + 4]) == [0, 5, 21, 54]
    assert list(h[L.ids:L.ids + 5]) == [0, 1, 2, 3, 4] and list(h[L.ids + 5:L.ids + 8]) == [100, 101, 102]
    assert list(h[L.pos:L.pos + 5]) == [0, 1, 2, 3, 4] and list(h[L.pos + 21:L.pos + 24]) == [0, 1, 2]
    assert list(h[L.page_indptr:L.page_indptr + 4]) == [0, 1, 2, 5]
    assert list(h[L.page_indices:L.page_indices + P]) == [p for ps_, u in zip(pages, used) for p in ps_[:u]]
    assert list(h[L.last_page_len:L.last_page_len + 3]) == [5, 16, 1]
    # KV slot of token t of a sequence = page(t // ps) * ps + t % ps
    assert h[L.slot + 4] == pages[0][0] * ps + 4 and h[L.slot + 5 + 15] == pages[1][0] * ps + 15
    assert h[L.slot + 21 + 32] == pages[2][2] * ps + 0
    b.mark_prefilled()
    b.append_tokens([9, 9, 9], False)
    h[:] = -7
    P = b.fill_decode(h, L, 4)
    assert list(h[L.ids:L.ids + 4]) == [9, 9, 9, 0] and list(h[L.pos:L.pos + 4]) == lens + [0]
    assert list(h[L.last_page_len:L.last_page_len + 4]) == [(n % ps) + 1 for n in lens] + [0]
    assert h[L.slot + 1] == pages[1][1] * ps + 0                                  # token 16 opens the second page
    assert h[L.slot + 3] == -1                                                    # padded row: cache write skipped
    assert P == sum(n // ps + 1 for n in lens) and list(h[L.page_indptr:L.page_indptr + 5]) == [0, 1, 3, 6, 6]
    # filter keeps order and returns pages; extend merges and empties the donor
    used = pool.used_pages
    b.filter([0, 2])
    assert [s.spec.id for s in b.seqs] == [0, 2] and pool.used_pages == used - len(pages[1])
    c = core.Batch(8, pool)
    assert c.add_prompts([core.SeqSpec(10, [1, 2, 3], 2)])
    c.mark_prefilled()
    b.extend(c)
    assert [s.spec.id for s in b.seqs] == [0, 2, 10] and c.size == 0
    # generation ends at max_new_tokens; finished sequences leave with filter(unfinished_ids)
    c2 = core.Batch(9, pool)
    assert c2.add_prompts([core.SeqSpec(20, [1, 2], 2), core.SeqSpec(21, [1, 2], 3)])
    c2.mark_prefilled()
    c2.append_tokens([5, 5], False)
    c2.append_tokens([5, 5], True)
    assert c2.unfinished_ids() == [21]
    c2.filter(c2.unfinished_ids())
    assert c2.size == 1
    for x in (b, c2):
        x.clear()
    assert pool.used_pages == 0


def test_prefill_in_chunks_covers_every_token_once_with_growing_page_lists():
    """Windows over the prompts laid end to end: the rows of all windows are exactly the prompts, positions continue
    across windows, and a row's page list reaches to the end of what the window adds for its sequence."""
    ps = 16
    pool = core.PagePool(64, ps)
    b = core.Batch(3, pool)
    lens = [5, 70, 33, 1]
    assert b.add_prompts([core.SeqSpec(i, list(range(1000 * i, 1000 * i + n)), 4) for i, n in enumerate(lens)])
    pages = [list(s.pages) for s in b.seqs]
    L = core.MetaLayout.make(32, 4, 64)
    h = np.full(L.total, -7, dtype=np.int32)
    seen = {i: [] for i in range(len(lens))}
    tok0, windows, ended_at = 0, 0, {}
    while tok0 < sum(lens):
        T, P, rows, s0, q_lens, kv_lens, ended = b.fill_prefill_chunk(h, L, tok0, 32)
        assert 0 < T <= 32 and rows == len(q_lens) == len(kv_lens) == len(ended) and sum(q_lens) == T
        assert list(h[L.tok_indptr:L.tok_indptr + rows + 1]) == [0] + list(np.cumsum(q_lens))
        off = pg = 0
        for r in range(rows):
            sq = s0 + r
            n, kv = q_lens[r], kv_lens[r]
            ids = list(h[L.ids + off:L.ids + off + n])
            pos = list(h[L.pos + off:L.pos + off + n])
            assert pos == list(range(kv - n, kv)) and ids == [1000 * sq + x for x in pos]
            assert list(h[L.slot + off:L.slot + off + n]) == [pages[sq][x // ps] * ps + x % ps for x in pos]
            used = (kv + ps - 1) // ps
            assert list(h[L.page_indices + pg:L.page_indices + pg + used]) == pages[sq][:used]
            assert h[L.page_indptr + r + 1] == pg + used and h[L.last_page_len + r] == kv - (used - 1) * ps
            seen[sq] += pos
            if ended[r]:
                assert kv == lens[sq]
                ended_at[sq] = windows
            off += n
            pg += used
        assert P == pg
        tok0 += T
        windows += 1
    assert windows == 4 and all(seen[i] == list(range(n)) for i, n in enumerate(lens))
    assert ended_at == {0: 0, 1: 2, 2: 3, 3: 3}
    b.clear()


def test_prefill_attention_work_list_covers_every_row_pair_heaviest_first():
    """One record per (sequence, 256 rows of it): offsets follow the packed rows and page lists of the pass, pairs that
    walk more key blocks come first, and a later chunk (prefix already cached) counts its prefix."""
    from blitz_scale_b200 import ops
    q_lens, kv_lens, ps = [300, 128, 1, 77, 513], [300, 128, 1, 277, 769], 16
    w = ops.prefill_work_list(q_lens, kv_lens, ps, "cpu").tolist()
    assert len(w) == sum((n + 255) // 256 for n in q_lens)
    row0 = np.concatenate([[0], np.cumsum(q_lens)])
    pg0 = np.concatenate([[0], np.cumsum([(kv + ps - 1) // ps for kv in kv_lens])])
    seen = set()
    weights = []
    for r0, n, p0, npg, kv, pair, z0, z1 in w:
        b = int(np.searchsorted(row0, r0, side="right")) - 1
        assert (r0, n, p0, npg, kv) == (row0[b], q_lens[b], pg0[b], (kv_lens[b] + ps - 1) // ps, kv_lens[b]) and z0 == z1 == 0
        assert 0 <= pair < (n + 255) // 256 and (b, pair) not in seen
        seen.add((b, pair))
        weights.append(min(kv, kv - n + 256 * (pair + 1)))
    assert weights == sorted(weights, reverse=True) and weights[0] == 769


def test_batch_admission_is_all_or_nothing_and_eos_stops():
    pool = core.PagePool(4, 16)
    b = core.Batch(1, pool)
    assert not b.add_prompts([core.SeqSpec(0, list(range(40)), 4), core.SeqSpec(1, list(range(40)), 4)])
    assert pool.used_pages == 0 and b.size == 0
    s = core.SeqSpec(2, [1, 2, 3], 10)
    s.eos_token, s.ignore_eos = 42, False       # benchmark traces ignore EOS by default, like the reference's harness
    assert b.add_prompts([s])
    b.mark_prefilled()
    b.append_tokens([7], False)
    assert b.unfinished_ids() == [2]
    assert core.parse_generations_full(b.encode_generations([7])) == ([2], [7], [False], [-1])
    b.append_tokens([42], True)
    assert b.unfinished_ids() == []
    # the finish reason travels in the generation (proto FinishReason: 0 length, 1 EOS token) and the native reader
    # hands it to the router core
    assert core.parse_generations_full(b.encode_generations([42])) == ([2], [42], [True], [1])
    b.clear()
    s = core.SeqSpec(3, [1, 2, 3], 1)
    assert b.add_prompts([s])
    b.mark_prefilled()
    b.append_tokens([9], False)
    raw = b.encode_generations([9])
    assert core.parse_generations_full(raw) == ([3], [9], [True], [0]) and core.parse_generations(raw) == ([3], [9], [True])
    b.clear()


# ------------------------------------------------------------------------------------------------ ZigZag scheduler
def test_zigzag_preemption_yield_and_blocking():
    z = core.ZigzagScheduler(4, 2)
    assert z.next().step == core.ZagStep.Idle
    assert z.add_task(100, 0, 8) >= 0 and z.add_task(101, 1, 8) >= 0
    assert z.add_task(102, 2, 8) == -1                       # no activation slot left
    with pytest.raises(Exception):
        z.add_task(99, 1, 8)                                 # sequence numbers only grow
    assert z.next().step == core.ZagStep.Blocked             # nothing has arrived
    z.set_loaded(True, 0, False)
    d = z.next()
    assert (d.step, d.batch_id) == (core.ZagStep.Embed, 100)
    z.complete(d)
    d = z.next()                                             # head waits for layer 0: the second task advances (yield)
    assert (d.step, d.batch_id) == (core.ZagStep.Embed, 101)
    z.complete(d)
    assert z.next().step == core.ZagStep.Blocked
    z.set_loaded(True, 2, False)
    order = []
    while z.next().step == core.ZagStep.Layer:
        d = z.next()
        order.append((d.batch_id, d.layer))
        z.complete(d)
    assert order == [(100, 0), (100, 1), (101, 0), (101, 1)]  # head first whenever it can run (preemption)
    with pytest.raises(Exception):
        z.set_loaded(True, 1, False)                         # the layer counter is monotonic
    z.set_loaded(True, 4, True)
    done = []
    while z.next().step not in (core.ZagStep.Idle, core.ZagStep.Blocked):
        d = z.next()
        if z.complete(d):
            done.append(d.batch_id)
    assert done == [100, 101] and z.pending() == 0 and z.free_slots() == 2


def test_zigzag_relay_head_and_second_task():
    z = core.ZigzagScheduler(6, 4)
    for i in range(3):
        z.add_task(200 + i, i, 4)
    z.set_loaded(True, 2, False)
    for _ in range(3):                                        # task 200: embedded + layers 0, 1
        z.complete(z.next())
    r = z.relay(False)
    assert (r.batch_id, r.seq_num, r.next_layer) == (200, 0, 2)   # the old instance resumes at layer 2
    z.release_slot(r.slot)
    r2 = z.relay(True)                                        # draining: the head keeps running, the second task leaves
    assert (r2.batch_id, r2.next_layer) == (202, -1)          # never embedded: restarts from the embedding
    z.release_slot(r2.slot)
    assert z.pending() == 1 and z.free_slots() == 3
    assert z.relay(True) is None                              # no second task
    assert z.relay(False).batch_id == 201 and z.relay(False) is None


def test_zigzag_random_interleavings_run_every_layer_once_in_order():
    rng = random.Random(0)
    for trial in range(200):
        L = rng.randint(1, 6)
        z = core.ZigzagScheduler(L, 3)
        arrived, embed, head = 0, False, False
        trace, relayed, finished, seq = {}, {}, [], 0
        live = []
        for _ in range(400):
            ev = rng.random()
            if ev < 0.15 and len(live) < 3:
                slot = z.add_task(1000 + seq, seq, rng.randint(1, 9))
                assert slot >= 0
                live.append(1000 + seq)
                trace[1000 + seq] = []
                seq += 1
            elif ev < 0.35:
                if not embed:
                    embed = True
                elif arrived < L:
                    arrived += 1
                else:
                    head = True
                z.set_loaded(embed, arrived, head)
            elif ev < 0.42 and live:
                r = z.relay(rng.random() < 0.5)
                if r is not None:
                    steps = trace[r.batch_id]
                    assert r.next_layer == (-1 if not steps else len(steps) - 1)
                    relayed[r.batch_id] = r.next_layer
                    live.remove(r.batch_id)
                    z.release_slot(r.slot)
            else:
                d = z.next()
                if d.step in (core.ZagStep.Idle, core.ZagStep.Blocked):
                    assert (d.step == core.ZagStep.Idle) == (not live)
                    continue
                # the chosen task is the first one in admission order that can advance
                for b in live:
                    n = len(trace[b])
                    can = (n == 0 and embed) or (0 < n <= L and n - 1 < arrived) or (n == L + 1 and head)
                    if can:
                        assert b == d.batch_id
                        break
                steps = trace[d.batch_id]
                want = "E" if not steps else (len(steps) - 1 if len(steps) <= L else "H")
                got = {core.ZagStep.Embed: "E", core.ZagStep.Layer: d.layer, core.ZagStep.Head: "H"}[d.step]
                assert got == want, (trial, d.batch_id, steps, got)
                steps.append(got)
                if z.complete(d):
                    finished.append(d.batch_id)
                    live.remove(d.batch_id)
        for b in finished:
            assert trace[b] == ["E"] + list(range(L)) + ["H"]
        assert z.pending() == len(live) and z.free_slots() == 3 - len(live)
        assert not set(finished) & set(relayed)


# ------------------------------------------------------------------------------------------------ oracle
def test_oracle_kv_cache_matches_recomputation_and_tp_shards_sum_to_full():
    cfg = get_config("tiny")
    seg = WeightSegment(cfg, 1, 0, dtype=torch.float32).random_init_(5)
    o = LlamaOracle(seg)
    prompts = [[3, 1, 4, 1, 5, 9, 2, 6], [2, 7, 1, 8]]
    toks = o.generate(prompts, 5)
    assert [len(t) for t in toks] == [5, 5]
    # greedy continuation is self-consistent: feeding prompt + first k tokens reproduces token k+1 (KV cache == recompute)
    for p, t in zip(prompts, toks):
        again = o.generate([p + t[:3]], 2)[0]
        assert again == t[3:5]
    assert o.generate(prompts, 5) == toks                      # deterministic


def test_native_generation_encoding_equals_the_message_built_one():
    from blitz_scale_b200.pb.schema import pb
    from blitz_scale_b200.worker.service import _response, make_generation
    pool = core.PagePool(64, 16)
    b = core.Batch(3, pool)
    specs = [core.SeqSpec(2 ** 40 + 5, [1, 2, 3], 1), core.SeqSpec(7, [4] * 20, 5), core.SeqSpec(300, [9], 2)]
    assert b.add_prompts(specs)
    b.mark_prefilled()
    toks = [0, 131071, 127]
    b.append_tokens(toks, False)                       # the first request reaches max_new_tokens = 1 and finishes
    info = b.emit_info()
    assert [i[0] for i in info] == [2 ** 40 + 5, 7, 300] and [i[1] for i in info] == [0, -1, -1] and [i[2] for i in info] == [1, 1, 1]
    want = pb.DecodeV2Response(generations=[make_generation(rid, t, f"<{t}>", None if fin < 0 else fin, n)
                                            for (rid, fin, n), t in zip(info, toks)])
    raw = b.encode_generations(toks)
    assert raw == want.SerializePartialToString()
    got = _response(pb.DecodeV2Response, raw, total_ns=5)
    assert got.total_ns == 5 and got.generations == want.generations and got.IsInitialized()
    assert got.generations[0].generated_text.finish_reason == 0 and not got.generations[1].HasField("generated_text")
    pre = _response(pb.PrefillV2Response, raw, forward_ns=1, decode_ns=0, total_ns=1)
    assert [g.tokens.ids[0] for g in pre.generations] == toks and [g.tokens.texts[0] for g in pre.generations] == ["<0>", "<131071>", "<127>"]
    assert b.request_ids() == [2 ** 40 + 5, 7, 300] and b.prompt_lens() == [3, 20, 1] and not b.none_generated()
    assert b.prompt_page_ids() == [s.pages[0] for s in b.seqs[:1]] + list(b.seqs[1].pages[:2]) + [b.seqs[2].pages[0]]
    with pytest.raises(Exception):
        b.encode_generations([1])
    b.clear()


def test_migration_page_lists_stay_aligned_when_one_side_has_filtered():
    """Both ends of a KV migration list pages per request of the RPC, in its order; a request one side no longer holds
    keeps its entries as -1, so entry i always faces entry i (a relayed batch whose request ended at its first token)."""
    from blitz_scale_b200.runtime import core
    src_pool, dst_pool = core.PagePool(64, 16), core.PagePool(64, 16)
    specs = [core.SeqSpec(11, [1] * 40, 1), core.SeqSpec(12, [2] * 16, 8), core.SeqSpec(13, [3] * 5, 8)]
    src, dst = core.Batch(9, src_pool), core.Batch(9, dst_pool)
    assert src.add_prompts(specs) and dst.add_prompts(list(reversed(specs)))      # the destination allocated in another order
    ids, lens = [11, 12, 13], [40, 16, 5]
    a, b = src.prompt_page_ids_for(ids, lens), dst.prompt_page_ids_for(ids, lens)
    assert len(a) == len(b) == 3 + 1 + 1 and -1 not in a and -1 not in b
    by_req = {s.spec.id: list(s.pages) for s in dst.seqs}
    assert b == by_req[11][:3] + by_req[12][:1] + by_req[13][:1]
    # request 11 finished at its first token on the source: its batch was filtered, the destination still holds all
    src.mark_prefilled()
    src.append_tokens([5, 6, 7], False)
    src.filter(src.unfinished_ids())
    a2 = src.prompt_page_ids_for(ids, lens)
    assert a2[:3] == [-1, -1, -1] and a2[3:] == a[3:] and len(a2) == len(b)
    # the second half names the survivors only: both sides list exactly those
    assert len(src.prompt_page_ids_for([12, 13], [16, 5])) == len(dst.prompt_page_ids_for([12, 13], [16, 5])) == 2
    with pytest.raises(Exception):
        src.prompt_page_ids_for([12], [16, 5])
    # a finished request left in a decode batch is carried as a padded row instead of indexing past its pages
    d = core.Batch(1, dst_pool)
    assert d.add_prompts([core.SeqSpec(1, [1] * 16, 1), core.SeqSpec(2, [1] * 3, 4)])
    d.mark_prefilled()
    d.append_tokens([9, 9], False)
    L = core.MetaLayout.make(64, 8, 64)
    h = np.zeros(L.total, dtype=np.int32)
    P = d.fill_decode(h, L, 4)
    assert h[L.slot + 0] == -1 and h[L.last_page_len + 0] == 0 and h[L.slot + 1] >= 0 and P == 1


def test_native_generation_reader_agrees_with_the_protobuf_library():
    from blitz_scale_b200.pb.schema import pb
    from blitz_scale_b200.worker.service import make_generation
    rng = random.Random(1)
    for trial in range(50):
        gens = []
        for _ in range(rng.randint(0, 40)):
            tok = rng.choice([0, 1, 127, 128, 300, 131071, 2 ** 31 - 1])
            fin = rng.choice([None, 0, 1, 2])
            g = make_generation(rng.choice([0, 5, 2 ** 33, 2 ** 63 + 1]), tok, f"<{tok}>", fin, rng.randint(0, 9))
            if rng.random() < 0.3:                         # fields the reader must skip
                g.prefill_tokens.ids.extend([1, 2, 3])
                g.prefill_tokens.logprobs.extend([0.5, 0.25, 0.0])
            if rng.random() < 0.2:
                g.tokens.ids.append(9)                     # only the first token id counts
                g.tokens.logprobs.append(0.0)
                g.tokens.texts.append("x")
                g.tokens.is_special.append(True)
            gens.append(g)
        r = pb.DecodeV2Response(generations=gens, total_ns=rng.randint(0, 2 ** 40))
        if gens and rng.random() < 0.5:
            r.batch.CopyFrom(pb.CachedBatch(id=3, request_ids=[1, 2], size=2, max_tokens=128))
        ids, toks, fins = core.parse_generations(r.SerializeToString())
        assert ids == [g.request_id for g in gens]
        assert toks == [g.tokens.ids[0] for g in gens]
        assert fins == [g.HasField("generated_text") for g in gens]
    # a prefill response carries the same field 1, plus fields the decode response does not have
    p = pb.PrefillV2Response(generations=[make_generation(4, 77)], forward_ns=1, decode_ns=2, total_ns=3)
    p.pp_info.tfm_layer = 5
    assert core.parse_generations(p.SerializeToString()) == ([4], [77], [False])
    assert core.parse_generations(b"") == ([], [], [])
    for bad in (b"\x0a\x05\x08", b"\x0a\xff\xff\xff\xff\xff\xff\xff\xff\xff\xff\xff", b"\x0b\x00", b"\x0a\x03\x1a\x05\x08"):
        with pytest.raises(Exception):
            core.parse_generations(bad)                    # truncated or malformed input is refused, never read past


def test_sampling_rows_of_a_batch():
    pool = core.PagePool(16, 16)
    b = core.Batch(1, pool)
    specs = [core.SeqSpec(i, [1, 2, 3], 4) for i in range(4)]
    specs[1].do_sample, specs[1].temperature, specs[1].top_k, specs[1].top_p, specs[1].seed = True, 0.5, 40, 0.9, 7
    specs[3].do_sample, specs[3].temperature, specs[3].top_p, specs[3].seed = True, 0.0, 2.0, 2 ** 63 + 5   # out-of-range values
    assert b.add_prompts(specs)
    rows, temp, top_k, top_p, seeds = b.sampling_rows()
    assert rows == [1, 3] and temp == [0.5, 1.0] and top_k == [40, 0] and top_p == pytest.approx([0.9, 1.0])
    assert all(-2 ** 63 <= s < 2 ** 63 for s in seeds) and seeds[0] != seeds[1]
    b.mark_prefilled()
    b.append_tokens([5, 5, 5, 5], False)
    assert b.sampling_rows()[4] != seeds                       # another draw at the next step
    b.filter([0, 2])
    assert b.sampling_rows() == ([], [], [], [], [])           # greedy batch: nothing to do
    b.clear()
