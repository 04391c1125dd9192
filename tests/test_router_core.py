"""CPU tests of the native orchestrator core: queue budgets, validation, feature flags, planner,
state machine, steersman, and whole-cluster virtual-time simulations (scaling, live scaling,
ServerlessLLM baseline, replica failure)."""
import math

import pytest

from blitz_scale_b200.runtime import core


def E(i, inp, new, t=0.0):
    return core.RequestEntry(i, inp, new, t)


# ------------------------------------------------------------------------------------------------ queue
def test_queue_empty_and_fifo():
    q = core.BatchQueue(block_size=1)
    assert q.next_batch(None, 1, 1) is None and q.next_batch(1, 1, 1) is None
    q.append(E(0, 0, 1))
    q.append(E(1, 0, 1))
    nb = q.next_batch(None, 2, 2)
    assert nb.batch.id == 0 and nb.batch.request_ids == [0, 1] and nb.batch.size == 2
    q.append(E(2, 0, 1))
    nb = q.next_batch(None, 2, 2)
    assert nb.batch.id == 1 and nb.batch.request_ids == [2]


def test_queue_min_size_restores_entries_and_waiting_tokens():
    q = core.BatchQueue(block_size=1)
    q.append(E(0, 5, 1))
    q.append(E(1, 7, 1))
    assert q.next_batch(3, 100, 100) is None      # fewer queued than min_size
    assert q.waiting_prefill_tokens == 12
    # budget admits only the first entry -> below min_size -> everything restored
    assert q.next_batch(2, 5, 100) is None
    assert len(q) == 2 and q.waiting_prefill_tokens == 12
    nb = q.next_batch(2, 100, 100)
    assert nb.batch.size == 2 and q.waiting_prefill_tokens == 0


def test_queue_token_and_block_budgets():
    q = core.BatchQueue(block_size=16)
    for i in range(3):
        q.append(E(i, 20, 12))      # 32 tokens = 2 blocks each
    nb = q.next_batch(None, 1000, 1000, block_budget=5)
    assert nb.batch.size == 2 and nb.batch.max_tokens == 64 and nb.batch.prompt_tokens == 40
    assert len(q) == 1
    # prefill budget: a 20-token prompt does not fit in 19
    assert q.next_batch(None, 19, 1000) is None
    # ... unless long prompts may be split by the worker: then it gets a batch of its own (and only the first one does)
    q.append(E(7, 20, 12))
    q.set_split_long_prompts(True)
    nb = q.next_batch(None, 19, 1000)
    assert nb.batch.size == 1 and nb.batch.prompt_tokens == 20 and len(q) == 1
    q.set_split_long_prompts(False)
    # a single request larger than the total-token budget is never admitted
    assert q.next_batch(None, 1000, 31) is None
    assert q.next_batch(None, 1000, 32).batch.size == 1


def test_queue_speculate_and_dropped_client():
    q = core.BatchQueue(block_size=1, speculate=2)
    q.append(E(0, 1, 1))
    assert q.next_batch(None, 10, 3) is None           # 2 + speculate(2) > 3
    assert q.next_batch(None, 10, 4).batch.size == 1
    q.append(E(1, 4, 1))
    q.append(E(2, 4, 1))
    q.mark_client_gone(1)
    nb = q.next_batch(None, 100, 100)
    assert nb.batch.request_ids == [2] and q.dropped == 1 and q.waiting_prefill_tokens == 0


# ------------------------------------------------------------------------------------------------ validation / features
def test_validation_rules():
    lim = core.ValidationLimits()
    p = core.GenerateParams()
    p.input_len, p.max_new_tokens = 10, 20
    assert core.validate_request(p, lim) == ""
    p.max_new_tokens = 0
    assert "max_new_tokens" in core.validate_request(p, lim)
    p.max_new_tokens = 5000
    assert "must be <=" in core.validate_request(p, lim)
    p.max_new_tokens, p.input_len = 10, 5000
    assert "inputs" in core.validate_request(p, lim)
    p.input_len, p.best_of = 10, 2
    assert "sampling" in core.validate_request(p, lim)
    p.do_sample = True
    assert core.validate_request(p, lim) == ""
    p.best_of, p.top_p = 1, 1.5
    assert "top_p" in core.validate_request(p, lim)
    p.top_p, p.top_n_tokens = 1.0, 9
    assert "top_n_tokens" in core.validate_request(p, lim)
    p.top_n_tokens, p.temperature = 0, 0.0
    assert "temperature" in core.validate_request(p, lim)


def test_feature_flags():
    f = core.FeatureSet.parse("impl_blitz,impl_fast_pro,impl_live_pro")
    for name in ("impl_rdma", "mutate", "fast", "impl_tanz", "impl_nvl", "live"):
        assert f.has(name)
    assert set(core.FeatureSet.parse("eval_all").list()) - {"eval_all"} == set(f.list())
    s = core.FeatureSet.parse("impl_sllm,cache_replace")
    assert s.has("impl_sllm") and not s.has("fast")
    for bad in ("impl_blitz,impl_sllm,cache_replace", "impl_sllm", "impl_blitz,cache_all_hit", "impl_sllm,cache_replace,fast",
                "nonsense", ""):
        with pytest.raises(ValueError):
            core.FeatureSet.parse(bad)


# ------------------------------------------------------------------------------------------------ planner / states / steersman
def test_planner_equations():
    c = core.PlannerConfig()
    c.tokens_prefilled_per_sec, c.tokens_transferred_per_sec, c.max_blocks_per_replica, c.block_size = 15000, 96000, 1000, 64
    v = core.PlannerView()
    v.num_prefill, v.num_decode = 1, 1
    t = core.plan_scale(c, v)
    assert (t.d_prefill, t.d_decode) == (0, 0)
    # prefill demand: 40000 waiting tokens -> [ceil(40000/.7/15000), ceil(40000/.5/15000)] = [4, 6] -> midpoint 5
    v.waiting_prefill_tokens = 40000
    t = core.plan_scale(c, v)
    assert (t.bands.prefill_thpt_min, t.bands.prefill_thpt_max) == (4, 6) and t.d_prefill == (4 + 6 + 1) // 2 - 1
    # decode memory: 2500 used blocks -> [ceil(2500/.95/1000), ceil(2500/.75/1000)] = [3, 4] -> up to 4
    v.waiting_prefill_tokens, v.decode_used_blocks = 0, 2500
    t = core.plan_scale(c, v)
    assert (t.bands.decode_mem_min, t.bands.decode_mem_max) == (3, 4) and t.d_decode == 3
    # scale down by at most one, never below one, clamped to the configured maximum
    v.decode_used_blocks, v.num_decode, v.num_prefill = 0, 4, 3
    t = core.plan_scale(c, v)
    assert (t.d_prefill, t.d_decode) == (-1, -1)
    v.num_decode = v.num_prefill = 1
    assert core.plan_scale(c, v).d_decode == 0
    v.decode_used_blocks, c.max_decode = 100000, 3
    assert core.plan_scale(c, v).d_decode == 2
    # KV bandwidth: tokens parked on prefill replicas
    v.decode_used_blocks, v.prefill_used_blocks, c.max_decode = 0, 3000, 8     # 192000 tokens
    t = core.plan_scale(c, v)
    assert (t.bands.decode_kv_min, t.bands.decode_kv_max) == (math.ceil(192000 / .8 / 96000), math.ceil(192000 / .4 / 96000))


def test_state_machine_table():
    names = core.replica_state_names()
    assert len(names) == 20 and names[0] == "Inactive"
    ok = [("Inactive", "LoadingPrefill"), ("LoadingPrefill", "Prefill"), ("Inactive", "NewPrefill"),
          ("NewPrefill", "RefractoryPrefill"), ("RefractoryPrefill", "Prefill"), ("Prefill", "OldPrefill"),
          ("OldPrefill", "Prefill"), ("Prefill", "MutatingToDecode"), ("MutatingToDecode", "Decode"),
          ("Prefill", "ShuttingPrefill"), ("ShuttingPrefill", "ShuttingNull"), ("Decode", "ShuttingDecode"),
          ("ShuttingDecode", "ShuttingNull"), ("ShuttingNull", "Inactive"), ("ShuttingNull", "Prefill"),
          ("ShuttingPrefill", "Prefill"), ("LoadingDecode", "AusDecode"), ("AusDecode", "Decode")]
    for a, b in ok:
        assert core.transition_allowed(a, b), (a, b)
    for a, b in [("Inactive", "Prefill"), ("Inactive", "Decode"), ("Decode", "Prefill"), ("NewPrefill", "Decode"),
                 ("ShuttingNull", "NewPrefill"), ("OldPrefill", "Decode")]:
        assert not core.transition_allowed(a, b), (a, b)


def test_steersman():
    s = core.Steersman([0, 0, 0, 0, 1, 1, 1, 1], 2, 30.0)
    assert s.ranks_of_replica(1) == [2, 3] and s.replica_of_rank(5) == 2
    s.record_model_loaded(0)
    s.record_model_loaded(2)
    plan = s.assign_nvlink_chains([0, 2], [1, 3])
    assert plan == {0: [1], 2: [3]}           # same-machine sources only
    s.set_nvlink_busy(0, True)
    assert s.assign_nvlink_chains([0, 2], [1, 3]) == {2: [3]}
    s.set_nvlink_busy(0, False)
    assert s.assign_tanz_chains([0, 2], [1]) == [([0], [1])]
    # host cache TTL (ServerlessLLM baseline)
    s.record_model_unloaded(0, 100.0)
    assert s.host_cache_hit(0, 120.0) and not s.host_cache_hit(0, 131.0) and not s.host_cache_hit(1, 120.0)
    s.register_model("llama3_8b", "/models/l3", 16.0)
    assert s.model_info("llama3_8b") == ("/models/l3", 16.0) and s.model_info("x") is None


# ------------------------------------------------------------------------------------------------ traces
def test_trace_generators_are_seeded_and_calibrated():
    spec = core.TraceSpec()
    spec.phases = [core.RatePhase(0.0, 4.0)]
    spec.duration, spec.seed = 500.0, 0
    spec.input.kind, spec.input.a, spec.input.b = core.LengthDist.Kind.Uniform, 32, 512
    spec.output.kind, spec.output.a, spec.output.b = core.LengthDist.Kind.Uniform, 16, 128
    a, b = core.generate_trace(spec), core.generate_trace(spec)
    assert [(x.t, x.input_len, x.output_len) for x in a] == [(x.t, x.input_len, x.output_len) for x in b]
    assert abs(len(a) / 500.0 - 4.0) < 0.4
    assert all(32 <= x.input_len <= 512 and 16 <= x.output_len <= 128 for x in a)
    gaps = [a[i + 1].t - a[i].t for i in range(len(a) - 1)]
    mean = sum(gaps) / len(gaps)
    cv = (sum((g - mean) ** 2 for g in gaps) / len(gaps)) ** 0.5 / mean
    assert abs(cv - 1.0) < 0.15                      # Poisson
    spec.cv, spec.seed = 4.0, 1
    spec.phases = [core.RatePhase(0.0, 2.0), core.RatePhase(250.0, 16.0)]
    spec.input.kind, spec.input.a, spec.input.b, spec.input.max_len = core.LengthDist.Kind.LogNormal, 512, 1.0, 4096
    g = core.generate_trace(spec)
    early = sum(1 for x in g if x.t < 250) / 250.0
    late = sum(1 for x in g if x.t >= 250) / 250.0
    assert 0.8 < early < 3.5 and 10 < late < 22     # the rate step is visible
    gaps = [g[i + 1].t - g[i].t for i in range(len(g) - 1) if g[i].t >= 250]
    mean = sum(gaps) / len(gaps)
    cv = (sum((x - mean) ** 2 for x in gaps) / len(gaps)) ** 0.5 / mean
    assert cv > 2.5                                  # bursty
    lens = sorted(x.input_len for x in g)
    assert 380 < lens[len(lens) // 2] < 680 and lens[-1] <= 4096


def test_csv_trace(tmp_path):
    p = tmp_path / "t.csv"
    p.write_text("timestamp,prefill,decode\n1000,100,20\n500,9000,5\n")
    tr = core.load_trace_csv(str(p), 2.0, 4095)
    assert [(x.t, x.input_len, x.output_len) for x in tr] == [(0.25, 4095, 5), (0.5, 100, 20)]
    # rows that are not three sane numbers are skipped, like the header
    p.write_text("t,in,out\n1e300,99999999999999999999,5\n1e999,5,5\n5,0,4\nx,y,z\n1,2\n1000,64,8\n")
    assert [(x.t, x.input_len, x.output_len) for x in core.load_trace_csv(str(p), 1.0, 4095)] == [(1.0, 64, 8)]


# ------------------------------------------------------------------------------------------------ whole-cluster simulations
def _cfg(states, features, **kw):
    c = core.ControllerConfig()
    c.num_ranks, c.tp = len(states), 1
    c.init_states = states
    c.features = features
    c.max_blocks_per_replica = kw.get("blocks", 4000)
    p = c.planner
    p.tokens_prefilled_per_sec, p.tokens_transferred_per_sec = 15000, 96000
    p.max_prefill, p.max_decode = kw.get("max_p", 4), kw.get("max_d", 4)
    c.planner = p
    for k, v in kw.items():
        if hasattr(c, k):
            setattr(c, k, v)
    return c


def _trace(rate_phases, duration, seed=0, cv=1.0, n=10 ** 9, inp=(32, 512), out=(16, 128)):
    s = core.TraceSpec()
    s.phases = [core.RatePhase(t, r) for t, r in rate_phases]
    s.duration, s.seed, s.cv, s.max_requests = duration, seed, cv, n
    s.input.kind, s.input.a, s.input.b = core.LengthDist.Kind.Uniform, inp[0], inp[1]
    s.output.kind, s.output.a, s.output.b = core.LengthDist.Kind.Uniform, out[0], out[1]
    return core.generate_trace(s)


def _check_conservation(rep, trace):
    assert rep.submitted == len(trace)
    assert rep.completed + rep.failed == len(trace)
    assert rep.leftover_blocks == 0
    want = sum(x.output_len for x in trace)
    if rep.failed == 0:
        assert rep.delivered_tokens == want
        by_id = {r.id: r for r in rep.requests}
        for i, x in enumerate(trace):
            assert by_id[i].output_len == x.output_len and by_id[i].ttft > 0


def test_sim_static_pd_pair_serves_everything():
    cfg = _cfg(["Prefill", "Decode"], "impl_blitz,impl_nvl", autoscale=False)
    trace = _trace([(0, 4.0)], 50.0, n=200)
    rep = core.ClusterSim(cfg, core.CostModel()).run(trace)
    _check_conservation(rep, trace)
    assert any("Replica<0> boot => Prefill" in l for l in rep.log)


def test_sim_is_deterministic():
    cfg = _cfg(["Prefill", "Decode", "Inactive", "Inactive"], "impl_blitz,impl_fast_pro,impl_live_pro")
    trace = _trace([(0, 2.0), (5.0, 40.0)], 12.0, seed=3, cv=4.0, inp=(256, 2048))
    a = core.ClusterSim(cfg, core.CostModel()).run(trace)
    b = core.ClusterSim(cfg, core.CostModel()).run(trace)
    assert a.log == b.log and [(r.id, r.ttft) for r in a.requests] == [(r.id, r.ttft) for r in b.requests]


@pytest.mark.parametrize("features", ["impl_blitz,impl_nvl", "impl_blitz,impl_fast_pro", "impl_blitz,impl_fast_pro,impl_live_pro",
                                      "impl_sllm,cache_replace", "impl_sllm,cache_all_hit,mutate"])
def test_sim_burst_triggers_scale_out_and_conserves_requests(features):
    cfg = _cfg(["Prefill", "Decode", "Inactive", "Inactive", "Inactive", "Inactive"], features)
    cm = core.CostModel()
    cm.prefill_tokens_per_s = 20000
    trace = _trace([(0, 2.0), (4.0, 30.0), (10.0, 1.0)], 16.0, seed=1, inp=(512, 2048), out=(16, 64))
    rep = core.ClusterSim(cfg, cm).run(trace)
    _check_conservation(rep, trace)
    ups = [l for l in rep.log if "Inactive =>" in l]
    assert ups, "the burst must trigger a scale-out"
    assert rep.scale_up_latency and all(v > 0 for v in rep.scale_up_latency.values())
    if "live" in features or "impl_live_pro" in features:
        assert any("=> NewPrefill" in l for l in rep.log) and any("=> OldPrefill" in l for l in rep.log)
        assert any("RefractoryPrefill => Prefill" in l for l in rep.log)
    if "impl_sllm" in features:
        assert not any("NewPrefill" in l for l in rep.log)
    # after the burst the planner parks replicas and later unloads them
    assert any("=> ShuttingNull" in l for l in rep.log)


def test_sim_live_scaling_serves_on_the_loading_replica():
    states = ["Prefill", "Decode", "Inactive", "Inactive"]
    cm = core.CostModel()
    cm.prefill_tokens_per_s, cm.nvlink_gbs = 20000, 8.0       # slow transfer: 2 s per model
    trace = _trace([(0, 1.0), (2.0, 25.0), (8.0, 1.0)], 12.0, seed=5, inp=(1024, 2048), out=(8, 16))
    live = core.ClusterSim(_cfg(states, "impl_blitz,impl_fast_pro,impl_live_pro"), cm).run(trace)
    stop = core.ClusterSim(_cfg(states, "impl_blitz,impl_fast_pro"), cm).run(trace)
    _check_conservation(live, trace)
    _check_conservation(stop, trace)
    t_of = lambda rep, pat: min(float(l[1:l.index("]")]) for l in rep.log if pat in l)
    # the new replica takes requests the moment scaling is triggered, not when its parameters have landed
    assert t_of(live, "Inactive => NewPrefill") + 1.0 < t_of(live, "RefractoryPrefill => Prefill")
    assert any("Prefill => OldPrefill" in l for l in live.log) and any("OldPrefill => Prefill" in l for l in live.log)
    assert not any("NewPrefill" in l for l in stop.log)
    mean = lambda rep: sum(r.ttft for r in rep.requests) / len(rep.requests)
    assert mean(live) < 1.5 * mean(stop)


def test_sim_sllm_host_cache_policy():
    states = ["Prefill", "Decode", "Inactive"]
    trace = _trace([(0, 1.0), (2.0, 30.0), (6.0, 0.5)], 9.0, seed=2, inp=(512, 2048), out=(8, 32))
    cm = core.CostModel()
    cm.prefill_tokens_per_s = 8000
    miss = core.ClusterSim(_cfg(states, "impl_sllm,cache_all_miss"), cm).run(trace)
    hit = core.ClusterSim(_cfg(states, "impl_sllm,cache_all_hit"), cm).run(trace)
    _check_conservation(miss, trace)
    _check_conservation(hit, trace)
    assert min(hit.scale_up_latency.values()) < min(miss.scale_up_latency.values())


def test_sim_replica_failure_requeues_or_fails_but_never_hangs():
    cfg = _cfg(["Prefill", "Prefill", "Decode", "Decode"], "impl_blitz,impl_nvl", autoscale=False)
    trace = _trace([(0, 20.0)], 6.0, seed=4, inp=(256, 1024), out=(8, 32))
    rep = core.ClusterSim(cfg, core.CostModel()).run(trace, kill_replica=0, kill_at=2.0)
    assert rep.submitted == len(trace) and rep.completed + rep.failed == len(trace)
    assert rep.completed > 0.9 * len(trace)           # prefill work is re-queued, not lost
    assert any("Replica<0> Prefill => Inactive" in l for l in rep.log)
    assert rep.leftover_blocks == 0
    rep = core.ClusterSim(cfg, core.CostModel()).run(trace, kill_replica=2, kill_at=2.0)
    assert rep.completed + rep.failed == len(trace) and rep.failed > 0 and rep.leftover_blocks == 0


def test_mutation_prefill_to_decode():
    # a prompt burst keeps two prefill replicas busy; when it ends the long outputs still fill the single
    # decode replica: prefill surplus + decode shortage with no spare GPU -> one prefill replica mutates
    cfg = _cfg(["Prefill", "Prefill", "Decode"], "impl_blitz,impl_nvl", blocks=250, max_p=2)
    cm = core.CostModel()
    cm.prefill_tokens_per_s = 6000
    trace = _trace([(0, 10.0), (3.0, 0.01)], 20.0, seed=6, inp=(1024, 2048), out=(400, 500))
    rep = core.ClusterSim(cfg, cm).run(trace)
    _check_conservation(rep, trace)
    assert any("Prefill => MutatingToDecode" in l for l in rep.log)
    assert any("MutatingToDecode => Decode" in l for l in rep.log)


def test_manual_scale_and_log_lines():
    cfg = _cfg(["Prefill", "Decode", "Inactive"], "impl_blitz,impl_nvl,manually_scale")
    ctl = core.Controller(cfg)
    assert ctl.manual_scale(2, "Decode", 0.0)
    acts = ctl.step(0.0)
    bc = [a for a in acts if a.type == core.ActionType.NvlBroadcast]
    assert len(bc) == 1 and bc[0].dst_ranks == [2] and bc[0].src_ranks == [1]
    assert ctl.state_name(2) == "LoadingDecode" and ctl.metric(1).marker == "NvlCasting"
    ctl.on_params_done(bc[0].op_id, 0.05)
    assert ctl.state_name(2) == "Decode" and ctl.metric(1).marker == "" and not ctl.metric(2).dst_busy
    log = ctl.drain_log()
    assert "Replica<2> Inactive => LoadingDecode" in log and "Replica<2> AusDecode => Decode" in log
    assert ctl.system_metrics_line().startswith("System Metrics: prefill_tokens: 0, decode_tokens: 0")


def test_simultaneous_scale_ups_share_one_multicast():
    """Scale-ups requested together become ONE striped multicast: two sources, every new replica a destination."""
    cfg = _cfg(["Prefill", "Decode"] + ["Inactive"] * 4, "impl_blitz,impl_nvl,manually_scale")
    ctl = core.Controller(cfg)
    for r in (2, 3, 4):
        assert ctl.manual_scale(r, "Prefill", 0.0)
    assert ctl.manual_scale(5, "Decode", 0.0) and ctl.manual_scale(5, "Decode", 0.0)      # repeated request: once
    acts = [a for a in ctl.step(0.0) if a.type in (core.ActionType.NvlBroadcast, core.ActionType.TanzBroadcast)]
    assert len(acts) == 1
    a = acts[0]
    assert a.type == core.ActionType.TanzBroadcast and sorted(a.src_ranks) == [0, 1] and a.dst_ranks == [2, 3, 4, 5]
    assert [ctl.state_name(r) for r in range(2, 6)] == ["LoadingPrefill"] * 3 + ["LoadingDecode"]
    assert ctl.metric(0).marker == "TanzCasting" and ctl.metric(1).marker == "TanzCasting"
    assert not [x for x in ctl.step(0.01) if x.type == core.ActionType.TanzBroadcast]              # nothing is re-issued
    ctl.on_params_done(a.op_id, 0.03)
    assert [ctl.state_name(r) for r in range(2, 6)] == ["Prefill"] * 3 + ["Decode"]
    g, c = dict(ctl.gauges()), dict(ctl.counters())
    assert g["blitz_last_scale_out_seconds"] == pytest.approx(0.03) and g["blitz_last_scale_out_fanout"] == 4
    assert c["blitz_scale_out_total"] == 4 and c["blitz_scale_out_seconds_sum"] == pytest.approx(0.03)
    assert ctl.metric(0).marker == "" and ctl.metric(1).marker == ""
    # live variant: every new prefill replica serves at once; one old prefill replica is paired as the helper
    cfg = _cfg(["Prefill", "Decode"] + ["Inactive"] * 2, "impl_blitz,impl_nvl,impl_live,manually_scale")
    ctl = core.Controller(cfg)
    for r in (2, 3):
        assert ctl.manual_scale(r, "Prefill", 0.0)
    acts = [a for a in ctl.step(0.0) if a.type == core.ActionType.TanzBroadcast]
    assert len(acts) == 1 and acts[0].live and acts[0].dst_ranks == [2, 3]
    assert ctl.state_name(2) == "NewPrefill" and ctl.state_name(3) == "NewPrefill" and ctl.state_name(0) == "OldPrefill"


def _prefill_one(ctl, rid, t=0.0, new_tokens=8):
    """Submit one request and carry it through prefill on whichever replica takes it; returns that replica."""
    ctl.submit(E(rid, 100, new_tokens, t))
    pf = [a for a in ctl.step(t) if a.type == core.ActionType.Prefill]
    assert len(pf) == 1
    ctl.on_prefill_done(pf[0].op_id, [core.TokenOut(rid, 7, False)], t + 0.01)
    return pf[0].replica


def test_lost_migration_destination_is_blamed_not_the_source():
    """A migration spans two replicas: when its destination dies the batch fails, the source gets its pages back and
    stays in service, and the late answer of the cancelled operation is ignored."""
    cfg = _cfg(["Prefill", "Decode", "Decode"], "impl_blitz,impl_nvl", autoscale=False)
    ctl = core.Controller(cfg)
    src = _prefill_one(ctl, 1)
    mig = [a for a in ctl.step(0.02) if a.type == core.ActionType.Migrate]
    assert len(mig) == 1 and mig[0].replica == src
    dst = mig[0].peer
    assert ctl.metric(src).used_blocks > 0 and ctl.metric(dst).used_blocks > 0
    ctl.on_failure(mig[0].op_id, 0.03, dst)                   # the destination's RPC was the one that failed
    assert ctl.state_name(dst) == "Inactive" and ctl.state_name(src) == "Prefill"
    acts = ctl.step(0.03)
    assert [a.request_id for a in acts if a.type == core.ActionType.Fail] == [1]
    assert any(a.type == core.ActionType.ClearCache and a.replica == src for a in acts)
    assert ctl.total_used_blocks() == 0 and ctl.inflight_ops() == 0
    ctl.on_migrate_done(mig[0].op_id, 0.05)                   # the source's RPC still answers: ignored, cache cleared again
    assert any(a.type == core.ActionType.ClearCache and a.replica == src for a in ctl.step(0.05))
    assert ctl.idle()
    # the survivors keep serving: the next request migrates to the other decode replica
    src = _prefill_one(ctl, 2, 0.1)
    mig = [a for a in ctl.step(0.12) if a.type == core.ActionType.Migrate]
    assert len(mig) == 1 and mig[0].peer not in (dst, src)
    # the failure detector's verdict while a migration is in flight settles it the same way
    ctl.on_replica_unhealthy(mig[0].peer, 0.13)
    assert [a.request_id for a in ctl.step(0.13) if a.type == core.ActionType.Fail] == [2]
    assert ctl.total_used_blocks() == 0 and ctl.inflight_ops() == 0


def test_lost_role_is_restored_and_lost_replica_is_quarantined():
    # the only decode replica dies: the spare becomes the decode side and the queued migration goes there
    cfg = _cfg(["Prefill", "Decode", "Inactive"], "impl_blitz,impl_nvl", quarantine_ms=1000.0)
    ctl = core.Controller(cfg)
    assert _prefill_one(ctl, 1) == 0
    ctl.on_replica_unhealthy(1, 0.02)
    acts = ctl.step(0.05)
    loads = [a for a in acts if a.type in (core.ActionType.NvlBroadcast, core.ActionType.RdmaBroadcast)]
    assert len(loads) == 1 and loads[0].dst_ranks == [2] and loads[0].src_ranks == [0]   # never the lost replica
    assert ctl.state_name(2) == "LoadingDecode" and ctl.state_name(1) == "Inactive"
    ctl.on_params_done(loads[0].op_id, 0.1)
    assert ctl.state_name(2) == "Decode"
    mig = [a for a in ctl.step(0.11) if a.type == core.ActionType.Migrate]
    assert len(mig) == 1 and (mig[0].replica, mig[0].peer) == (0, 2)    # request 1 waited for the new decode side
    # with no spare at all the surviving replica serves both phases instead of waiting for ever
    cfg = _cfg(["Prefill", "Decode"], "impl_blitz,impl_nvl", quarantine_ms=1000.0)
    ctl = core.Controller(cfg)
    ctl.on_replica_unhealthy(0, 0.0)
    ctl.submit(E(5, 64, 3, 0.0))
    acts = ctl.step(0.02)
    assert ctl.state_name(1) == "Prefill" and ctl.state_name(0) == "Inactive"
    pf = [a for a in acts + ctl.step(0.03) if a.type == core.ActionType.Prefill]
    assert len(pf) == 1 and pf[0].replica == 1
    ctl.on_prefill_done(pf[0].op_id, [core.TokenOut(5, 1, False)], 0.05)
    dec = [a for a in ctl.step(0.06) if a.type == core.ActionType.Decode]
    assert len(dec) == 1 and dec[0].replica == 1
    # after the quarantine the lost replica may be tried again, unless a failure detector says it is still away
    assert not [a for a in ctl.step(0.5) if a.type == core.ActionType.NvlBroadcast]
    ctl.set_reachable(0, False)
    assert not [a for a in ctl.step(1.1) if a.type in (core.ActionType.NvlBroadcast, core.ActionType.RdmaBroadcast)]
    ctl.set_reachable(0, True)
    again = [a for a in ctl.step(1.2) if a.type in (core.ActionType.NvlBroadcast, core.ActionType.RdmaBroadcast)]
    assert len(again) == 1 and again[0].dst_ranks == [0]


def test_prompt_longer_than_the_prefill_budget_gets_a_batch_of_its_own():
    """Workers prefill long prompts in chunks, so the controller admits such a prompt alone instead of leaving it at the
    head of the queue for ever; with chunked prefill switched off it is never admitted (the reference's rule)."""
    for chunked, want in ((True, 1), (False, 0)):
        cfg = _cfg(["Prefill", "Decode"], "impl_blitz,impl_nvl,manually_scale", max_prefill_tokens=64, chunked_prefill=chunked)
        ctl = core.Controller(cfg)
        ctl.submit(E(1, 300, 4, 0.0))
        ctl.submit(E(2, 20, 4, 0.0))
        pf = [a for a in ctl.step(0.01) + ctl.step(0.02) if a.type == core.ActionType.Prefill]
        assert len(pf) == want
        if want:
            assert list(pf[0].request_ids) == [1]            # alone: the short request behind it waits for the next batch


def test_lost_participant_aborts_a_shared_parameter_transfer():
    cfg = _cfg(["Prefill", "Decode"] + ["Inactive"] * 2, "impl_blitz,impl_nvl,manually_scale")
    ctl = core.Controller(cfg)
    assert ctl.manual_scale(2, "Prefill", 0.0) and ctl.manual_scale(3, "Prefill", 0.0)
    bc = [a for a in ctl.step(0.0) if a.type == core.ActionType.TanzBroadcast]
    assert len(bc) == 1 and bc[0].dst_ranks == [2, 3]
    ctl.on_failure(bc[0].op_id, 0.01, 3)
    acts = ctl.step(0.01)
    assert ctl.state_name(2) == "Inactive" and ctl.state_name(3) == "Inactive"
    assert [a.dst_ranks for a in acts if a.type == core.ActionType.ResetStatus] == [[2]]   # the healthy one starts over
    assert ctl.metric(0).marker == "" and ctl.metric(1).marker == "" and ctl.inflight_ops() == 0
    ctl.on_params_done(bc[0].op_id, 0.02)                     # late answer of the aborted transfer
    assert ctl.state_name(2) == "Inactive"
    assert ctl.manual_scale(2, "Prefill", 0.03)               # the healthy replica can be scaled again at once
    assert [a.dst_ranks for a in ctl.step(0.03) if a.type == core.ActionType.NvlBroadcast] == [[2]]


def test_concurrent_incoming_migrations_respect_limit_and_transfer_slots():
    def start(max_in, slots):
        cfg = _cfg(["Prefill", "Prefill", "Prefill", "Decode"], "impl_blitz,impl_nvl", autoscale=False,
                   max_incoming_migrations=max_in, kv_transfer_slots=slots)
        ctl = core.Controller(cfg)
        for i in range(3):
            ctl.submit(E(i, 6000, 8))            # one request per batch (prefill token budget 8192)
        pf = [a for a in ctl.step(0.0) if a.type == core.ActionType.Prefill]
        assert sorted(a.replica for a in pf) == [0, 1, 2]
        for a in pf:
            ctl.on_prefill_done(a.op_id, [core.TokenOut(a.request_ids[0], 1, False)], 0.01)
        return ctl, [a for a in ctl.step(0.02) if a.type == core.ActionType.Migrate]
    ctl, mig = start(1, 8)
    assert len(mig) == 1 and ctl.metric(3).dst_busy          # one at a time (the reference's destination mutex)
    ctl.on_migrate_done(mig[0].op_id, 0.03)
    assert len([a for a in ctl.step(0.04) if a.type == core.ActionType.Migrate]) == 1
    ctl, mig = start(2, 8)
    assert len(mig) == 2 and ctl.metric(3).dst_busy          # two in flight, the third waits
    assert not [a for a in ctl.step(0.03) if a.type == core.ActionType.Migrate]
    ctl.on_migrate_done(mig[0].op_id, 0.04)
    assert len([a for a in ctl.step(0.05) if a.type == core.ActionType.Migrate]) == 1
    ctl, mig = start(3, 1)
    assert len(mig) == 1                                     # a single transfer slot: never two at once, whatever the limit
    ctl, mig = start(3, 8)
    assert len(mig) == 3 and len({a.batch_id % 8 for a in mig}) == 3


def test_network_flow_accounting():
    cfg = _cfg(["Prefill", "Decode", "Inactive"], "impl_blitz,impl_nvl,manually_scale", param_gb=16.0, kv_mb_per_token=0.125)
    ctl = core.Controller(cfg)
    assert ctl.manual_scale(2, "Decode", 0.0)
    bc = [a for a in ctl.step(0.0) if a.type == core.ActionType.NvlBroadcast][0]
    ctl.on_params_done(bc.op_id, 0.03)
    assert ctl.take_flows() == [(1, 0.0, 16000.0), (2, 16000.0, 0.0)]       # decode replica 1 was the source
    assert ctl.take_flows() == []                                             # reported once
    ctl.submit(E(1, 1000, 4))
    pf = [a for a in ctl.step(0.1) if a.type == core.ActionType.Prefill][0]
    ctl.on_prefill_done(pf.op_id, [core.TokenOut(1, 5, False)], 0.12)
    assert ctl.waiting_migration_tokens() == 1000
    mig = [a for a in ctl.step(0.13) if a.type == core.ActionType.Migrate][0]
    assert ctl.waiting_migration_tokens() == 0
    ctl.on_migrate_done(mig.op_id, 0.14)
    assert ctl.take_flows() == [(0, 0.0, 125.0), (mig.peer, 125.0, 0.0)]


def test_calibrated_autoscaling_study_orders_the_policies():
    """Virtual-time replay with the measured B200 cost model: faster parameter delivery -> lower p99 TTFT."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench"))
    import sim_study
    out = sim_study.run("llama3_8b", 6.0, 100.0)
    rows = {r["policy"].split(" (")[0]: r for r in out["rows"]}
    mc, host, disk = rows["multicast, stop-the-world load"], rows["host-cache load"], rows["disk load"]
    assert all(r["failed"] == 0 and r["requests"] == out["trace_requests"] for r in out["rows"])
    assert mc["scale_outs"] >= 2 and mc["scale_out_latency_ms"] < host["scale_out_latency_ms"] < disk["scale_out_latency_ms"]
    assert mc["ttft_ms_p99"] < host["ttft_ms_p99"] < disk["ttft_ms_p99"]
    assert mc["ttft_violation_rate"] <= host["ttft_violation_rate"] <= disk["ttft_violation_rate"]


def test_client_gone_is_forgotten_in_the_queue_and_filtered_out_of_a_running_batch():
    cfg = _cfg(["Prefill", "Decode"], "impl_blitz,impl_nvl", autoscale=False)
    ctl = core.Controller(cfg)
    ctl.set_compact_deliveries(True)
    for i in range(3):
        ctl.submit(E(i, 100, 50))
    ctl.submit(E(9, 9000, 5))                               # does not fit the first prefill batch: stays queued
    pf = [a for a in ctl.step(0.0) if a.type == core.ActionType.Prefill][0]
    assert sorted(pf.request_ids) == [0, 1, 2]
    assert ctl.client_gone(9) is True and ctl.queue_size in (0, 1)      # forgotten at once
    ctl.on_prefill_done(pf.op_id, [core.TokenOut(i, 7, False) for i in range(3)], 0.01)
    mig = [a for a in ctl.step(0.02) if a.type == core.ActionType.Migrate][0]
    ctl.on_migrate_done(mig.op_id, 0.03)
    dec = [a for a in ctl.step(0.04) if a.type == core.ActionType.Decode][0]
    assert ctl.client_gone(1) is False                      # being served: ends with its next token
    ctl.on_decode_done(dec.op_id, [core.TokenOut(i, 8, False) for i in range(3)], 0.05)
    assert (1, 8, True) in ctl.take_deliveries()
    acts = ctl.step(0.06)
    flt = [a for a in acts if a.type == core.ActionType.FilterBatch]
    assert len(flt) == 1 and sorted(flt[0].request_ids) == [0, 2] and flt[0].replica == 1
    assert not [a for a in acts if a.type == core.ActionType.Decode]          # no step before the batch is filtered
    ctl.on_filter_done(flt[0].op_id, 0.07)
    dec = [a for a in ctl.step(0.08) if a.type == core.ActionType.Decode]
    assert len(dec) == 1
    # everybody leaves: the batch is cleared instead of filtered
    ctl.client_gone(0), ctl.client_gone(2)
    ctl.on_decode_done(dec[0].op_id, [core.TokenOut(0, 8, False), core.TokenOut(2, 8, False)], 0.09)
    acts = ctl.step(0.1)
    assert [a.type for a in acts if a.type in (core.ActionType.FilterBatch, core.ActionType.ClearCache)] == [core.ActionType.ClearCache]
    for _ in range(3):
        ctl.step(0.2)
    assert ctl.idle() and ctl.total_used_blocks() == 0 and ctl.inflight_ops() == 0


def test_migrations_are_served_oldest_first_across_replicas():
    """With one destination and several prefill replicas holding finished batches, the free destination goes to the
    batch that has waited longest, not to the replica with the lowest index."""
    cfg = _cfg(["Prefill", "Prefill", "Prefill", "Decode"], "impl_blitz,impl_nvl", autoscale=False)
    ctl = core.Controller(cfg)
    for i in range(3):
        ctl.submit(E(i, 6000, 8))
    pf = {a.replica: a for a in ctl.step(0.0) if a.type == core.ActionType.Prefill}
    assert sorted(pf) == [0, 1, 2]
    # replica 2 finishes first, then 1, then 0
    for t, r in ((0.010, 2), (0.011, 1), (0.012, 0)):
        ctl.on_prefill_done(pf[r].op_id, [core.TokenOut(pf[r].request_ids[0], 1, False)], t)
    order = []
    t = 0.02
    for _ in range(3):
        mig = [a for a in ctl.step(t) if a.type == core.ActionType.Migrate]
        assert len(mig) == 1
        order.append(mig[0].replica)
        ctl.on_migrate_done(mig[0].op_id, t + 0.005)
        t += 0.01
    assert order == [2, 1, 0]
    # under sustained load the tail of the prefill-to-first-decode gap stays close to its median (no starved replica)
    cfg = _cfg(["Prefill"] * 4 + ["Decode"], "impl_blitz,impl_nvl", autoscale=False, blocks=300000)
    cm = core.CostModel()
    cm.kv_tokens_per_s, cm.migrate_overhead_s, cm.rpc_overhead_s = 250000.0, 0.004, 0.003
    trace = _trace([(0, 180.0)], 6.0, seed=3, cv=2.0, inp=(900, 1100), out=(16, 32))
    sim = core.ClusterSim(cfg, cm)
    rep = sim.run(trace)
    _check_conservation(rep, trace)
    gaps = sorted(e.t_first_decode_token - e.t_first_token for e in sim.controller().finished().values() if e.t_first_decode_token > 0)
    assert gaps[int(0.99 * len(gaps))] < 3.0 * gaps[len(gaps) // 2]


def test_decode_placement_prefers_the_least_loaded_replica():
    def tbt_p99(features):
        cfg = _cfg(["Prefill"] * 3 + ["Decode"] * 3, features, autoscale=False, blocks=30000, max_batch_seqs=0)
        cm = core.CostModel()
        cm.decode_step_per_seq_s = 4e-5
        trace = _trace([(0, 150.0)], 4.0, seed=3, cv=2.0, inp=(400, 600), out=(100, 300))
        rep = core.ClusterSim(cfg, cm).run(trace)
        _check_conservation(rep, trace)
        xs = sorted(r.avg_tbt for r in rep.requests)
        return xs[int(0.99 * len(xs))]
    balanced, first_fit = tbt_p99("impl_blitz,impl_nvl"), tbt_p99("impl_blitz,impl_nvl,decode_first_fit")
    assert balanced < 0.6 * first_fit          # the reference's first-fit scan piles everything on one decode replica


def test_sequence_cap_of_a_worker_step():
    # the queue never forms a batch with more requests than one worker step carries
    q = core.BatchQueue(64)
    for i in range(10):
        q.append(E(i, 8, 4))
    nb = q.next_batch(None, 8192, 16000, None, 4)
    assert nb.batch.request_ids == [0, 1, 2, 3] and len(q) == 6
    assert len(q.next_batch(None, 8192, 16000).batch.request_ids) == 6          # no cap: everything that fits the budgets
    # a decode replica is not handed more sequences than it can step; the batch waits and goes elsewhere or later
    cfg = _cfg(["Prefill", "Prefill", "Decode", "Decode"], "impl_blitz,impl_nvl,decode_first_fit", autoscale=False, max_batch_seqs=4)
    ctl = core.Controller(cfg)
    for i in range(8):
        ctl.submit(E(i, 8, 50))
    pf = [a for a in ctl.step(0.0) if a.type == core.ActionType.Prefill]
    assert [len(a.request_ids) for a in pf] == [4, 4]                          # capped prefill batches
    for a in pf:
        ctl.on_prefill_done(a.op_id, [core.TokenOut(i, 1, False) for i in a.request_ids], 0.01)
    first = [a for a in ctl.step(0.02) if a.type == core.ActionType.Migrate]
    assert len(first) == 2 and sorted(a.peer for a in first) == [2, 3]         # first fit would have sent both to replica 2
    for a in first:
        ctl.on_migrate_done(a.op_id, 0.03)
    # a third batch finds both decode replicas full and waits
    for i in range(8, 10):
        ctl.submit(E(i, 8, 50))
    acts = ctl.step(0.04)
    pf = [a for a in acts if a.type == core.ActionType.Prefill]
    ctl.on_prefill_done(pf[0].op_id, [core.TokenOut(i, 1, False) for i in pf[0].request_ids], 0.05)
    assert not [a for a in ctl.step(0.06) if a.type == core.ActionType.Migrate]
    assert ctl.waiting_migration_tokens() == 16
    # when a request of a decode replica finishes, room opens up
    dec = [a for a in ctl.step(0.07) + acts if a.type == core.ActionType.Decode]
    d2 = [a for a in dec if a.replica == 2][0]
    ids = list(d2.request_ids)
    ctl.on_decode_done(d2.op_id, [core.TokenOut(ids[0], 2, True), core.TokenOut(ids[1], 2, True)] + [core.TokenOut(i, 2, False) for i in ids[2:]], 0.08)
    mig = [a for a in ctl.step(0.09) if a.type == core.ActionType.Migrate]
    assert len(mig) == 1 and mig[0].peer == 2


def test_planner_adds_a_decode_replica_when_the_sequence_cap_is_reached():
    """Many short requests fill a decode replica's step long before its KV memory: the planner scales the decode side on
    that signal too, and everything completes."""
    cfg = _cfg(["Prefill", "Decode"] + ["Inactive"] * 3, "impl_blitz,impl_nvl", blocks=30000, max_batch_seqs=64, max_p=2, max_d=3)
    trace = _trace([(0, 120.0)], 5.0, seed=3, inp=(32, 128), out=(100, 200))
    rep = core.ClusterSim(cfg, core.CostModel()).run(trace)
    _check_conservation(rep, trace)
    assert sum(1 for l in rep.log if l.endswith("=> LoadingDecode")) >= 1


def test_colocated_replica_never_exceeds_its_step_size():
    cfg = _cfg(["Normal"], "impl_blitz,impl_nvl", autoscale=False, max_batch_seqs=8)
    trace = _trace([(0, 200.0)], 2.0, seed=1, inp=(16, 64), out=(30, 60))
    sim = core.ClusterSim(cfg, core.CostModel())
    rep = sim.run(trace)
    _check_conservation(rep, trace)
    # driving the core by hand: what the replica holds never exceeds the cap, and new prompts come in as others finish
    ctl = core.Controller(cfg)
    for i in range(30):
        ctl.submit(E(i, 16, 10))
    held, t, peak, prefills = set(), 0.0, 0, 0
    for _ in range(300):
        t += 0.001
        for a in ctl.step(t):
            if a.type == core.ActionType.Deliver and a.final:
                held.discard(a.request_id)
            elif a.type == core.ActionType.Prefill:
                held |= set(a.request_ids)
                prefills += 1
                assert len(held) <= 8
                ctl.on_prefill_done(a.op_id, [core.TokenOut(i, 1, False) for i in a.request_ids], t)
            elif a.type == core.ActionType.Decode:
                assert len(a.request_ids) <= 8
                ctl.on_decode_done(a.op_id, [core.TokenOut(i, 2, False) for i in a.request_ids], t)
        peak = max(peak, len(held))
    assert peak == 8 and prefills >= 4 and ctl.idle() and not held


def test_progressive_migration_places_the_batch_at_prefill_dispatch():
    """With `migrate_progressive` the decode replica is chosen and locked when the prefill is issued; when the prefill
    answers, the batch is on the decode replica (no Migrate action), the prefill replica holds nothing, and requests
    that ended at their first token are filtered out of the received batch before its first decode step."""
    A = core.ActionType
    cfg = _cfg(["Prefill", "Decode"], "impl_blitz,impl_nvl,migrate_progressive", autoscale=False)
    ctl = core.Controller(cfg)
    ctl.set_compact_deliveries(True)
    for i in range(3):
        ctl.submit(E(i, 100, 1 if i == 1 else 20))
    pf = [a for a in ctl.step(0.0) if a.type == A.Prefill]
    assert len(pf) == 1 and pf[0].replica == 0 and pf[0].peer == 1
    assert list(pf[0].src_ranks) == [0] and list(pf[0].dst_ranks) == [1]
    assert ctl.metric(0).used_blocks > 0 and ctl.metric(0).used_blocks == ctl.metric(1).used_blocks
    # a second batch finds the only decode replica locked and takes the ordinary path (after the first has answered)
    ctl.submit(E(7, 64, 4))
    assert not [a for a in ctl.step(0.005) if a.type == A.Prefill]
    ctl.on_prefill_done(pf[0].op_id, [core.TokenOut(0, 5, False), core.TokenOut(1, 5, True), core.TokenOut(2, 5, False)], 0.01)
    assert ctl.metric(0).used_blocks == 0
    acts = ctl.step(0.02)
    assert not [a for a in acts if a.type == A.Migrate]
    flt = [a for a in acts if a.type == A.FilterBatch]
    assert len(flt) == 1 and flt[0].replica == 1 and sorted(flt[0].request_ids) == [0, 2]
    assert not [a for a in acts if a.type == A.Decode]                 # not before the filter has been applied
    nxt = [a for a in acts if a.type == A.Prefill]
    assert len(nxt) == 1 and nxt[0].peer == -1                         # the decode replica is still locked by the first batch
    ctl.on_filter_done(flt[0].op_id, 0.03)
    dec = [a for a in ctl.step(0.04) if a.type == A.Decode]
    assert len(dec) == 1 and dec[0].replica == 1 and sorted(dec[0].request_ids) == [0, 2]
    assert ctl.counters()["blitz_progressive_kv_cache_times"] == 1
    # nothing finished at the first token: the batch joins the decode replica as soon as the prefill answers
    ctl.on_prefill_done(nxt[0].op_id, [core.TokenOut(7, 5, False)], 0.05)
    ctl.on_decode_done(dec[0].op_id, [core.TokenOut(0, 6, False), core.TokenOut(2, 6, False)], 0.05)
    acts = ctl.step(0.06)
    mig = [a for a in acts if a.type == A.Migrate]
    assert len(mig) == 1                                               # the ordinary path for the second batch
    ctl.on_migrate_done(mig[0].op_id, 0.07)
    ctl.submit(E(8, 64, 4))
    pf = [a for a in ctl.step(0.08) if a.type == A.Prefill]
    assert len(pf) == 1 and pf[0].peer == 1
    ctl.on_prefill_done(pf[0].op_id, [core.TokenOut(8, 5, False)], 0.09)
    assert not [a for a in ctl.step(0.1) if a.type in (A.FilterBatch, A.Migrate)]
    assert ctl.metric(0).used_blocks == 0 and ctl.metric(1).used_blocks > 0


@pytest.mark.parametrize("lost", ["source", "destination"])
def test_progressive_migration_survives_the_loss_of_either_side(lost):
    A = core.ActionType
    cfg = _cfg(["Prefill", "Decode", "Prefill", "Decode"], "impl_blitz,impl_nvl,migrate_progressive", autoscale=False)
    ctl = core.Controller(cfg)
    ctl.submit(E(1, 100, 8))
    pf = [a for a in ctl.step(0.0) if a.type == A.Prefill][0]
    src, dst = pf.replica, pf.peer
    assert dst >= 0
    gone, kept = (src, dst) if lost == "source" else (dst, src)
    ctl.on_failure(pf.op_id, 0.01, gone)
    assert ctl.state_name(gone) == "Inactive" and ctl.state_name(kept) != "Inactive"
    acts = ctl.step(0.01)
    assert not [a for a in acts if a.type == A.Fail]                   # nothing was delivered: the prompt is served again
    assert any(a.type == A.ClearCache and a.replica == kept for a in acts)
    again = [a for a in acts if a.type == A.Prefill]
    assert len(again) == 1 and again[0].replica not in (gone,) and again[0].peer != gone
    assert ctl.metric(kept).used_blocks == (0 if kept not in (again[0].replica, again[0].peer) else ctl.metric(kept).used_blocks)
    ctl.on_prefill_done(pf.op_id, [core.TokenOut(1, 5, False)], 0.02)   # the late answer of the cancelled call is ignored
    ctl.on_prefill_done(again[0].op_id, [core.TokenOut(1, 5, False)], 0.03)
    acts = ctl.step(0.04)
    holder = again[0].peer if again[0].peer >= 0 else again[0].replica
    if again[0].peer < 0:
        mig = [a for a in acts if a.type == A.Migrate]
        assert len(mig) == 1
        ctl.on_migrate_done(mig[0].op_id, 0.05)
        holder = mig[0].peer
        acts = ctl.step(0.06)
    dec = [a for a in acts if a.type == A.Decode]
    assert len(dec) == 1 and dec[0].replica == holder


def test_sim_progressive_migration_conserves_requests_and_pages():
    cfg = _cfg(["Prefill", "Decode", "Prefill", "Decode"], "impl_blitz,impl_nvl,migrate_progressive", autoscale=False)
    trace = _trace([(0, 6.0)], 40.0, n=240, seed=2, out=(1, 64))
    sim = core.ClusterSim(cfg, core.CostModel())
    rep = sim.run(trace)
    _check_conservation(rep, trace)
    c = sim.controller().counters()
    assert c["blitz_progressive_kv_cache_times"] > 0 and c["blitz_kv_cache_times"] >= c["blitz_progressive_kv_cache_times"]


def test_deliveries_carry_the_finish_reason():
    """The last delivery of a request says why it ended: 1 token budget (also when the router ends it itself), 2 the
    worker met the end-of-sequence token, 3 a stop sequence; 0 while it goes on."""
    A = core.ActionType
    cfg = _cfg(["Normal"], "impl_blitz,impl_nvl", autoscale=False)
    ctl = core.Controller(cfg)
    ctl.set_compact_deliveries(True)
    ctl.submit(E(1, 50, 8))
    ctl.submit(E(2, 50, 2))
    ctl.submit(E(3, 50, 8))
    pf = [a for a in ctl.step(0.0) if a.type == A.Prefill][0]
    ctl.on_prefill_done(pf.op_id, [core.TokenOut(1, 5, True, 1), core.TokenOut(2, 5, False), core.TokenOut(3, 5, False)], 0.01)
    assert ctl.take_deliveries() == [(1, 5, 2), (2, 5, 0), (3, 5, 0)]
    dec = [a for a in ctl.step(0.02) if a.type == A.Decode][0]
    ctl.on_decode_done(dec.op_id, [core.TokenOut(2, 6, False), core.TokenOut(3, 6, True, 2)], 0.03)
    assert ctl.take_deliveries() == [(2, 6, 1), (3, 6, 3)]      # request 2 reached its budget in the router's count
    # without compact deliveries the reason rides on the Deliver action
    ctl = core.Controller(cfg)
    ctl.submit(E(1, 50, 8))
    pf = [a for a in ctl.step(0.0) if a.type == A.Prefill][0]
    ctl.on_prefill_done(pf.op_id, [core.TokenOut(1, 5, True, 1)], 0.01)
    d = [a for a in ctl.step(0.02) if a.type == A.Deliver]
    assert len(d) == 1 and d[0].final and d[0].finish_reason == 1


def test_planner_arrival_rate_signal():
    """With the feature planner_arrival_rate the prefill side is also sized by the rate at which prompt tokens arrive:
    a utilisation band on that rate, which asks for replicas before a backlog exists."""
    c = core.PlannerConfig()
    c.prefill_lower, c.prefill_upper, c.max_prefill = 0.5, 0.7, 8
    c.tokens_prefilled_per_sec, c.prefill_rate_per_sec = 1000, 10000.0
    v = core.PlannerView()
    v.num_prefill, v.num_decode = 1, 1
    assert core.plan_scale(c, v).d_prefill == 0                      # nothing waits, nothing arrives
    v.arrival_tokens_per_sec = 30000.0                               # 3 replicas' worth at full utilisation
    t = core.plan_scale(c, v)
    assert (t.bands.prefill_rate_min, t.bands.prefill_rate_max) == (5, 6) and t.d_prefill == 5   # to the middle of [5, 6]
    c.prefill_rate_per_sec = 0.0
    assert core.plan_scale(c, v).d_prefill == 0                      # not configured: the view's rate is not read
    # in the controller: a burst of arrivals inside the window asks for replicas although the queue is still short
    cfg = _cfg(["Prefill", "Decode", "Inactive", "Inactive"], "impl_blitz,impl_nvl,planner_arrival_rate")
    p = cfg.planner
    p.tokens_prefilled_per_sec, p.prefill_rate_per_sec, p.arrival_window_ms = 10 ** 6, 20000.0, 50.0   # the queue rule never fires
    cfg.planner = p
    ctl = core.Controller(cfg)
    for i in range(6):
        ctl.submit(E(i, 500, 4, 0.001 * i))                          # 3000 tokens in 6 ms = 60 k tokens/s over the window
    acts = []
    for k in range(30):
        acts += ctl.step(0.006 + 0.001 * k)
    assert any(a.type in (core.ActionType.NvlBroadcast, core.ActionType.TanzBroadcast) for a in acts)
    same = _cfg(["Prefill", "Decode", "Inactive", "Inactive"], "impl_blitz,impl_nvl")
    same.planner = p
    ctl = core.Controller(same)
    for i in range(6):
        ctl.submit(E(i, 500, 4, 0.001 * i))
    acts = []
    for k in range(30):
        acts += ctl.step(0.006 + 0.001 * k)
    assert not any(a.type in (core.ActionType.NvlBroadcast, core.ActionType.TanzBroadcast) for a in acts)
