"""Property tests of the controller in the virtual-time simulator: whatever the trace, the feature set and the
failure injected, every request is accounted for and no KV block is left behind (hypothesis, CPU)."""
import os

import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st  # noqa: E402

from blitz_scale_b200.runtime import core  # noqa: E402

FEATURES = ["impl_blitz,impl_nvl", "impl_blitz,impl_nvl,impl_live", "impl_blitz,impl_fast_pro,impl_live_pro",
            "impl_blitz,impl_nvl,impl_tanz", "impl_blitz,impl_nvl,mutate", "impl_sllm,cache_replace",
            "impl_sllm,cache_all_miss", "impl_blitz,impl_nvl,unidirect", "impl_blitz,impl_nvl,prefill_share_idle",
            "impl_blitz,impl_nvl,impl_live,decode_first_fit", "impl_blitz,impl_nvl,migrate_progressive",
            "impl_blitz,impl_fast_pro,impl_live_pro,migrate_progressive", "impl_blitz,impl_nvl,mutate,migrate_progressive",
            "impl_blitz,impl_nvl,planner_arrival_rate", "impl_blitz,impl_fast_pro,impl_live_pro,planner_arrival_rate"]


@settings(max_examples=int(os.environ.get("BLITZ_PROPERTY_EXAMPLES", "25")), deadline=None)
@given(feat=st.sampled_from(FEATURES), seed=st.integers(0, 10 ** 6), n_inactive=st.integers(0, 4),
       burst=st.floats(4.0, 60.0), cv=st.sampled_from([1.0, 2.0, 4.0]), kill=st.booleans(), kill_replica=st.integers(0, 2), kill_at=st.sampled_from([0.5, 1.2, 2.0, 3.5]),
       prefill_rate=st.sampled_from([8000.0, 30000.0, 120000.0]), tp=st.sampled_from([1, 2]),
       max_incoming=st.sampled_from([1, 2, 4]), gone_every=st.sampled_from([0, 0, 3, 7]))
def test_requests_and_blocks_are_conserved(feat, seed, n_inactive, burst, cv, kill, kill_replica, kill_at, prefill_rate,
                                           tp, max_incoming, gone_every):
    states = ["Prefill", "Decode"] + ["Inactive"] * n_inactive
    cfg = core.ControllerConfig()
    cfg.num_ranks, cfg.tp = len(states) * tp, tp
    cfg.init_states = sum([[s] * tp for s in states], [])
    cfg.features = feat
    cfg.max_blocks_per_replica = 3000
    cfg.max_incoming_migrations = max_incoming
    cfg.max_batch_seqs = [0, 6, 256][seed % 3]          # a worker step's sequence cap, sometimes tight
    p = cfg.planner
    p.tokens_prefilled_per_sec, p.tokens_transferred_per_sec = int(prefill_rate * 0.2), 500000
    p.max_prefill, p.max_decode = len(states) - 1, len(states) - 1
    p.prefill_rate_per_sec, p.arrival_window_ms = prefill_rate, 50.0      # read only with the feature planner_arrival_rate
    cfg.planner = p
    cm = core.CostModel()
    cm.prefill_tokens_per_s = prefill_rate
    spec = core.TraceSpec()
    spec.phases = [core.RatePhase(0.0, 2.0), core.RatePhase(1.0, burst), core.RatePhase(3.0, 1.0)]
    spec.duration, spec.seed, spec.cv = 5.0, seed, cv
    spec.input.kind, spec.input.a, spec.input.b = core.LengthDist.Kind.Uniform, 16, 1500
    spec.output.kind, spec.output.a, spec.output.b = core.LengthDist.Kind.Uniform, 1, 48
    trace = core.generate_trace(spec)
    sim = core.ClusterSim(cfg, cm)
    kill_replica = min(kill_replica, len(states) - 1)
    rep = sim.run(trace, 0.001, 120.0, kill_replica if kill else -1, kill_at if kill else -1.0, gone_every)
    assert rep.submitted == len(trace)
    # a client that leaves while its request waits is forgotten; one that leaves later gets a shortened answer
    assert rep.completed + rep.failed + rep.gone_in_queue == len(trace), (rep.completed, rep.failed, rep.gone_in_queue, len(trace))
    assert rep.leftover_blocks == 0
    want = sum(x.output_len for x in trace)
    if not kill:
        assert rep.failed == 0
        assert rep.delivered_tokens == want if gone_every == 0 else rep.delivered_tokens <= want
    if gone_every == 0:
        assert rep.gone_in_queue == rep.gone_in_service == 0
    for r in rep.requests:
        assert r.ttft >= 0 and r.t_done >= r.t_arrival
