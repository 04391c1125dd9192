"""Sampling in the engine's serving steps: rows that ask for it draw from the step's logits, the others keep the
arg-max.  (Named to run after the other GPU tests.)"""
import pytest

pytestmark = pytest.mark.gpu


def _generate(seeds, top_k=0, temperature=0.8):
    """Prefill + 4 decode steps of 4 requests; `seeds[i]` = None for a greedy request, else its sampling seed."""
    import torch
    from blitz_scale_b200 import ops
    from blitz_scale_b200.runtime import core
    from blitz_scale_b200.runtime.engine import Engine
    torch.cuda.set_device(0)
    eng = Engine("tiny_gpu", num_pages=64, page_size=16, max_batch=8, max_batch_tokens=512, seed=0)
    specs = []
    for i in range(4):
        s = core.SeqSpec(i, list(range(3 + i, 40 + 7 * i)), 6)
        if seeds[i] is not None:
            s.do_sample, s.temperature, s.top_k, s.top_p, s.seed = True, temperature, top_k, 1.0, seeds[i]
        specs.append(s)
    batch = eng.new_batch(0, specs)
    steps = [eng.prefill(batch)]
    for _ in range(4):
        steps.append(eng.decode(batch))
    ops.check_status()
    assert all(0 <= t < eng.cfg.vocab for st in steps for t in st)
    return [[st[i] for st in steps] for i in range(4)]


def test_sampled_rows_draw_and_greedy_rows_keep_the_argmax():
    greedy = _generate([None, None, None, None])
    mixed = _generate([None, 11, None, 12], temperature=1.5)
    again = _generate([None, 11, None, 12], temperature=1.5)
    assert mixed == again                                        # same seeds: same tokens
    # a greedy row next to sampled rows sees the same history as in the all-greedy run
    assert mixed[0] == greedy[0] and mixed[2] == greedy[2]
    other = _generate([None, 13, None, 14], temperature=1.5)
    assert (mixed[1], mixed[3]) != (other[1], other[3])          # other seeds: other draws (random-init logits are flat)
    assert (mixed[1], mixed[3]) != (greedy[1], greedy[3])        # and not simply the arg-max
