"""Several decode steps per worker call on the GPU backend give the tokens of one step per call, including a request
that finishes in the middle of a call.  (Named to run after the other GPU tests.)"""
import pytest

pytestmark = pytest.mark.gpu


def test_multi_step_decode_equals_single_steps():
    import torch
    from blitz_scale_b200 import ops
    from blitz_scale_b200.pb.schema import pb
    from blitz_scale_b200.runtime import core
    from blitz_scale_b200.worker.gpu_backend import GpuBackend
    torch.cuda.set_device(0)
    backend = GpuBackend(0, 1, "tiny_gpu", num_pages=128, page_size=16, max_batch=8, max_batch_tokens=512)

    def batch(bid, new_tokens):
        b = pb.Batch(id=bid, size=len(new_tokens), max_tokens=len(new_tokens) * 128)
        for i, n in enumerate(new_tokens):
            r = b.requests.add()
            r.id, r.inputs, r.prefill_logprobs, r.top_n_tokens = i, "", False, 0
            r.input_tokens.extend(range(3 + i, 30 + 5 * i))
            r.stopping_parameters.max_new_tokens = n
            r.stopping_parameters.ignore_eos_token = True
        return b

    def toks(raw):
        return list(zip(*core.parse_generations(raw)))

    def run(bid, steps):
        gens, cb, _ = backend.prefill(batch(bid, [9, 4, 7]), 0, None, [])
        out, calls = toks(gens), 0
        while cb is not None:
            g, cb = backend.decode([cb], [pb.Tokens()], steps) if steps > 1 else backend.decode([cb], [pb.Tokens()])
            out += toks(g)
            calls += 1
        return out, calls
    single, calls1 = run(1, 1)
    multi, calls4 = run(2, 4)
    ops.check_status()
    assert calls1 == 8 and calls4 == 2                       # 8 decode steps for the longest request: 8 calls or 2
    assert multi == single and len(single) == 9 + 4 + 7
    assert [t for t in single if t[0] == 1][-1][2] is True   # request 1 finished on its 4th token, inside a call
    assert not backend.batches and backend.engine.pool.used_pages == 0
    backend.close()
