"""Capturing every decode graph up front gives the same tokens as capturing on first use.  (Named to run after the
other GPU tests.)"""
import pytest

pytestmark = pytest.mark.gpu


def _run(precapture: bool):
    import torch
    from blitz_scale_b200 import ops
    from blitz_scale_b200.runtime import core
    from blitz_scale_b200.runtime.engine import Engine
    torch.cuda.set_device(0)
    eng = Engine("tiny_gpu", num_pages=96, page_size=16, max_batch=8, max_batch_tokens=512, seed=0)
    captured = eng.precapture() if precapture else 0
    ops.check_status()
    before = len(eng._graphs)
    batch = eng.new_batch(0, [core.SeqSpec(i, list(range(3 + i, 40 + 7 * i)), 8) for i in range(3)])
    steps = [eng.prefill(batch)]
    for _ in range(5):
        steps.append(eng.decode(batch))
    ops.check_status()
    return steps, captured, before, len(eng._graphs)


def test_precaptured_graphs_serve_the_same_tokens():
    lazy, _, _, n_lazy = _run(False)
    eager, captured, before, after = _run(True)
    assert captured >= 4 and before == captured          # buckets 1, 2, 4, 8 (at least one split choice each)
    assert after == before                               # serving found its graph: nothing captured on the way
    assert n_lazy >= 1 and eager == lazy
