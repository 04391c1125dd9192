#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include "router/controller.h"
#include "util/pbwire.h"
namespace py = pybind11;
using namespace blitz;

void bind_router(py::module_& m) {
  py::class_<RequestEntry>(m, "RequestEntry").def(py::init<>())
      .def(py::init([](uint64_t id, uint32_t input_len, uint32_t max_new, double t) {
             RequestEntry e; e.id = id; e.input_len = input_len; e.max_new_tokens = max_new; e.t_arrival = t; return e; }),
           py::arg("id"), py::arg("input_len"), py::arg("max_new_tokens"), py::arg("t_arrival") = 0.0)
      .def_readwrite("id", &RequestEntry::id).def_readwrite("input_len", &RequestEntry::input_len)
      .def_readwrite("max_new_tokens", &RequestEntry::max_new_tokens).def_readwrite("client_alive", &RequestEntry::client_alive)
      .def_readwrite("t_arrival", &RequestEntry::t_arrival).def_readonly("t_batched", &RequestEntry::t_batched)
      .def_readonly("t_first_token", &RequestEntry::t_first_token).def_readonly("t_last_token", &RequestEntry::t_last_token)
      .def_readonly("t_first_decode_token", &RequestEntry::t_first_decode_token)
      .def_readonly("generated", &RequestEntry::generated).def_readonly("tbt", &RequestEntry::tbt);
  py::class_<RouterBatch>(m, "RouterBatch").def_readonly("id", &RouterBatch::id)
      .def_readonly("request_ids", &RouterBatch::request_ids).def_readonly("max_tokens", &RouterBatch::max_tokens)
      .def_readonly("prompt_tokens", &RouterBatch::prompt_tokens).def_property_readonly("size", &RouterBatch::size);
  py::class_<BatchQueue::Next>(m, "NextBatch").def_readonly("batch", &BatchQueue::Next::batch)
      .def_readonly("entries", &BatchQueue::Next::entries);
  py::class_<BatchQueue>(m, "BatchQueue")
      .def(py::init<uint32_t, uint32_t, std::optional<uint32_t>>(), py::arg("block_size") = 64, py::arg("speculate") = 0,
           py::arg("window") = std::nullopt)
      .def("set_split_long_prompts", &BatchQueue::set_split_long_prompts)
      .def("append", &BatchQueue::append).def("__len__", &BatchQueue::size)
      .def_property_readonly("waiting_prefill_tokens", &BatchQueue::waiting_prefill_tokens)
      .def("mark_client_gone", &BatchQueue::mark_client_gone).def_property_readonly("dropped", &BatchQueue::dropped)
      .def("next_batch", &BatchQueue::next_batch, py::arg("min_size"), py::arg("prefill_token_budget"),
           py::arg("token_budget"), py::arg("block_budget") = std::nullopt, py::arg("max_size") = 0);

  py::class_<GenerateParams>(m, "GenerateParams", py::dynamic_attr()).def(py::init<>())
      .def_readwrite("input_len", &GenerateParams::input_len).def_readwrite("max_new_tokens", &GenerateParams::max_new_tokens)
      .def_readwrite("best_of", &GenerateParams::best_of).def_readwrite("do_sample", &GenerateParams::do_sample)
      .def_readwrite("temperature", &GenerateParams::temperature)
      .def_readwrite("repetition_penalty", &GenerateParams::repetition_penalty).def_readwrite("top_p", &GenerateParams::top_p)
      .def_readwrite("typical_p", &GenerateParams::typical_p).def_readwrite("top_k", &GenerateParams::top_k)
      .def_readwrite("top_n_tokens", &GenerateParams::top_n_tokens)
      .def_readwrite("num_stop_sequences", &GenerateParams::num_stop_sequences)
      .def_readwrite("truncate", &GenerateParams::truncate).def_readwrite("has_seed", &GenerateParams::has_seed);
  py::class_<ValidationLimits>(m, "ValidationLimits").def(py::init<>())
      .def_readwrite("max_best_of", &ValidationLimits::max_best_of)
      .def_readwrite("max_stop_sequences", &ValidationLimits::max_stop_sequences)
      .def_readwrite("max_top_n_tokens", &ValidationLimits::max_top_n_tokens)
      .def_readwrite("max_input_length", &ValidationLimits::max_input_length)
      .def_readwrite("max_total_tokens", &ValidationLimits::max_total_tokens);
  m.def("validate_request", &validate_request);

  py::class_<FeatureSet>(m, "FeatureSet").def_static("parse", &FeatureSet::parse).def("has", &FeatureSet::has)
      .def("list", &FeatureSet::list);

  m.def("transition_allowed", [](const std::string& a, const std::string& b) {
    auto x = rstate_from_name(a), y = rstate_from_name(b);
    if (!x || !y) throw std::invalid_argument("unknown state");
    return transition_allowed(*x, *y); });
  m.def("replica_state_names", [] {
    std::vector<std::string> v;
    for (int i = 0; i <= static_cast<int>(RState::TanzCasting); ++i) v.push_back(rstate_name(static_cast<RState>(i)));
    return v; });

  py::class_<PlannerConfig>(m, "PlannerConfig").def(py::init<>())
      .def_readwrite("prefill_lower", &PlannerConfig::prefill_lower).def_readwrite("prefill_upper", &PlannerConfig::prefill_upper)
      .def_readwrite("decode_lower", &PlannerConfig::decode_lower).def_readwrite("decode_upper", &PlannerConfig::decode_upper)
      .def_readwrite("migration_lower", &PlannerConfig::migration_lower).def_readwrite("migration_upper", &PlannerConfig::migration_upper)
      .def_readwrite("min_prefill", &PlannerConfig::min_prefill).def_readwrite("max_prefill", &PlannerConfig::max_prefill)
      .def_readwrite("min_decode", &PlannerConfig::min_decode).def_readwrite("max_decode", &PlannerConfig::max_decode)
      .def_readwrite("tokens_prefilled_per_sec", &PlannerConfig::tokens_prefilled_per_sec)
      .def_readwrite("tokens_transferred_per_sec", &PlannerConfig::tokens_transferred_per_sec)
      .def_readwrite("max_blocks_per_replica", &PlannerConfig::max_blocks_per_replica)
      .def_readwrite("block_size", &PlannerConfig::block_size)
      .def_readwrite("scale_down_threshold_ms", &PlannerConfig::scale_down_threshold_ms)
      .def_readwrite("prefill_rate_per_sec", &PlannerConfig::prefill_rate_per_sec)
      .def_readwrite("arrival_window_ms", &PlannerConfig::arrival_window_ms);
  py::class_<PlannerView>(m, "PlannerView").def(py::init<>())
      .def_readwrite("num_prefill", &PlannerView::num_prefill).def_readwrite("num_decode", &PlannerView::num_decode)
      .def_readwrite("arrival_tokens_per_sec", &PlannerView::arrival_tokens_per_sec)
      .def_readwrite("decode_used_blocks", &PlannerView::decode_used_blocks)
      .def_readwrite("prefill_used_blocks", &PlannerView::prefill_used_blocks)
      .def_readwrite("waiting_prefill_tokens", &PlannerView::waiting_prefill_tokens);
  py::class_<ScaleBands>(m, "ScaleBands")
      .def_readonly("prefill_thpt_min", &ScaleBands::prefill_thpt_min).def_readonly("prefill_thpt_max", &ScaleBands::prefill_thpt_max)
      .def_readonly("prefill_kv_min", &ScaleBands::prefill_kv_min).def_readonly("prefill_kv_max", &ScaleBands::prefill_kv_max)
      .def_readonly("decode_mem_min", &ScaleBands::decode_mem_min).def_readonly("decode_mem_max", &ScaleBands::decode_mem_max)
      .def_readonly("decode_kv_min", &ScaleBands::decode_kv_min).def_readonly("decode_kv_max", &ScaleBands::decode_kv_max)
      .def_readonly("prefill_rate_min", &ScaleBands::prefill_rate_min).def_readonly("prefill_rate_max", &ScaleBands::prefill_rate_max);
  py::class_<ScaleTarget>(m, "ScaleTarget").def_readonly("d_prefill", &ScaleTarget::d_prefill)
      .def_readonly("d_decode", &ScaleTarget::d_decode).def_readonly("bands", &ScaleTarget::bands);
  m.def("plan_scale", &plan_scale);

  py::class_<Steersman>(m, "Steersman")
      .def(py::init<std::vector<int>, int, double>(), py::arg("machine_of_rank"), py::arg("tp"), py::arg("host_cache_ttl_s") = 30.0)
      .def("replica_of_rank", &Steersman::replica_of_rank).def("ranks_of_replica", &Steersman::ranks_of_replica)
      .def("machine_of", &Steersman::machine_of).def("register_model", &Steersman::register_model)
      .def("model_info", &Steersman::model_info).def("record_model_loaded", &Steersman::record_model_loaded)
      .def("record_model_unloaded", &Steersman::record_model_unloaded).def("model_on_gpu", &Steersman::model_on_gpu)
      .def("host_cache_hit", &Steersman::host_cache_hit).def("touch_host_cache", &Steersman::touch_host_cache)
      .def("nvlink_busy", &Steersman::nvlink_busy).def("set_nvlink_busy", &Steersman::set_nvlink_busy)
      .def("assign_nvlink_chains", &Steersman::assign_nvlink_chains, py::arg("sources"), py::arg("targets"), py::arg("fanout") = 7)
      .def("assign_tanz_chains", [](const Steersman& s, const std::vector<int>& a, const std::vector<int>& b) {
        std::vector<std::pair<std::vector<int>, std::vector<int>>> out;
        for (auto& p : s.assign_tanz_chains(a, b)) out.push_back({p.sources, p.targets});
        return out; });

  py::enum_<ActionType>(m, "ActionType")
      .value("Prefill", ActionType::Prefill).value("ZagPrefill", ActionType::ZagPrefill).value("PrefillPP", ActionType::PrefillPP)
      .value("Decode", ActionType::Decode).value("Migrate", ActionType::Migrate).value("MigratePartial", ActionType::MigratePartial)
      .value("Relay", ActionType::Relay).value("NvlBroadcast", ActionType::NvlBroadcast).value("TanzBroadcast", ActionType::TanzBroadcast)
      .value("RdmaBroadcast", ActionType::RdmaBroadcast).value("LoadParams", ActionType::LoadParams)
      .value("ResetStatus", ActionType::ResetStatus).value("SetStatusReady", ActionType::SetStatusReady)
      .value("ClearCache", ActionType::ClearCache).value("Deliver", ActionType::Deliver).value("Fail", ActionType::Fail)
      .value("FilterBatch", ActionType::FilterBatch);
  py::class_<Action>(m, "Action").def_readonly("type", &Action::type).def_readonly("op_id", &Action::op_id)
      .def_readonly("replica", &Action::replica).def_readonly("peer", &Action::peer).def_readonly("batch_id", &Action::batch_id)
      .def_readonly("batch_ids", &Action::batch_ids).def_readonly("request_ids", &Action::request_ids)
      .def_readonly("max_tokens", &Action::max_tokens).def_readonly("src_ranks", &Action::src_ranks)
      .def_readonly("dst_ranks", &Action::dst_ranks).def_readonly("load_case", &Action::load_case)
      .def_readonly("partial", &Action::partial).def_readonly("num_layer", &Action::num_layer)
      .def_readonly("zag_seq", &Action::zag_seq).def_readonly("live", &Action::live).def_readonly("mock", &Action::mock)
      .def_readonly("request_id", &Action::request_id).def_readonly("token", &Action::token).def_readonly("final", &Action::final)
      .def_readonly("finish_reason", &Action::finish_reason);
  py::class_<ControllerConfig>(m, "ControllerConfig").def(py::init<>())
      .def_readwrite("num_ranks", &ControllerConfig::num_ranks).def_readwrite("tp", &ControllerConfig::tp)
      .def_readwrite("machines", &ControllerConfig::machines).def_readwrite("init_states", &ControllerConfig::init_states)
      .def_readwrite("block_size", &ControllerConfig::block_size)
      .def_readwrite("max_prefill_tokens", &ControllerConfig::max_prefill_tokens)
      .def_readwrite("max_total_tokens", &ControllerConfig::max_total_tokens)
      .def_readwrite("max_blocks_per_replica", &ControllerConfig::max_blocks_per_replica)
      .def_readwrite("zigzag_req_limit", &ControllerConfig::zigzag_req_limit)
      .def_readwrite("zigzag_req_floor", &ControllerConfig::zigzag_req_floor)
      .def_readwrite("zigzag_decay_ms", &ControllerConfig::zigzag_decay_ms)
      .def_readwrite("planner_interval_ms", &ControllerConfig::planner_interval_ms)
      .def_readwrite("model_layers", &ControllerConfig::model_layers).def_readwrite("model_name", &ControllerConfig::model_name)
      .def_readwrite("planner", &ControllerConfig::planner).def_readwrite("features", &ControllerConfig::features)
      .def_readwrite("param_gb", &ControllerConfig::param_gb).def_readwrite("quarantine_ms", &ControllerConfig::quarantine_ms).def_readwrite("max_batch_seqs", &ControllerConfig::max_batch_seqs).def_readwrite("chunked_prefill", &ControllerConfig::chunked_prefill).def_readwrite("kv_mb_per_token", &ControllerConfig::kv_mb_per_token).def_readwrite("max_incoming_migrations", &ControllerConfig::max_incoming_migrations).def_readwrite("kv_transfer_slots", &ControllerConfig::kv_transfer_slots).def_readwrite("autoscale", &ControllerConfig::autoscale).def_readwrite("mock_load_ms", &ControllerConfig::mock_load_ms);
  m.def("parse_generations", [](py::bytes raw) {
    auto g = pbwire::parse_generations(static_cast<std::string>(raw));
    return py::make_tuple(g.request_ids, g.tokens, g.finished); },
    "(request ids, first token ids, finished flags) of the `generations` of a serialized prefill / decode response");
  m.def("parse_generations_full", [](py::bytes raw) {
    auto g = pbwire::parse_generations(static_cast<std::string>(raw));
    std::vector<int> reasons(g.reasons.begin(), g.reasons.end());
    return py::make_tuple(g.request_ids, g.tokens, g.finished, reasons); },
    "as parse_generations, plus the finish reason of every generation (-1 while it is unfinished)");
  py::class_<Controller::TokenOut>(m, "TokenOut")
      .def(py::init([](uint64_t id, int32_t tok, bool fin, int reason) {
             return Controller::TokenOut{id, tok, fin, static_cast<int8_t>(reason)}; }),
           py::arg("request_id"), py::arg("token"), py::arg("finished"), py::arg("reason") = 0);
  py::class_<ReplicaMetric>(m, "ReplicaMetric")
      .def_property_readonly("state", [](const ReplicaMetric& r) { return std::string(rstate_name(r.state)); })
      .def_property_readonly("marker", [](const ReplicaMetric& r) { return r.marker ? std::string(rstate_name(*r.marker)) : std::string(); })
      .def_readonly("used_blocks", &ReplicaMetric::used_blocks).def_readonly("model_loaded", &ReplicaMetric::model_loaded)
      .def_readonly("dst_busy", &ReplicaMetric::dst_busy).def_readonly("flying_partial", &ReplicaMetric::flying_partial)
      .def_readonly("loop_cnt", &ReplicaMetric::loop_cnt);
  py::class_<Controller>(m, "Controller").def(py::init<const ControllerConfig&>())
      .def("submit", &Controller::submit).def("client_gone", &Controller::client_gone)
      .def("on_prefill_done", &Controller::on_prefill_done).def("on_decode_done", &Controller::on_decode_done)
      .def("on_migrate_done", &Controller::on_migrate_done).def("on_params_done", &Controller::on_params_done)
      .def("on_relay_done", &Controller::on_relay_done).def("on_filter_done", &Controller::on_filter_done).def("on_failure", &Controller::on_failure, py::arg("op_id"), py::arg("now"), py::arg("failed_replica") = -1)
      .def("step", &Controller::step).def("manual_scale", &Controller::manual_scale)
      // completion straight from the wire bytes of the worker's response: the generations are read natively
      .def("on_prefill_done_wire", [](Controller& c, uint64_t op, py::bytes raw, double now) {
        auto g = pbwire::parse_generations(static_cast<std::string>(raw));
        std::vector<Controller::TokenOut> t;
        t.reserve(g.request_ids.size());
        for (size_t i = 0; i < g.request_ids.size(); ++i)
          t.push_back({g.request_ids[i], g.tokens[i], g.finished[i], static_cast<int8_t>(std::max<int>(0, g.reasons[i]))});
        c.on_prefill_done(op, t, now); })
      .def("on_decode_done_wire", [](Controller& c, uint64_t op, py::bytes raw, double now) {
        auto g = pbwire::parse_generations(static_cast<std::string>(raw));
        std::vector<Controller::TokenOut> t;
        t.reserve(g.request_ids.size());
        for (size_t i = 0; i < g.request_ids.size(); ++i)
          t.push_back({g.request_ids[i], g.tokens[i], g.finished[i], static_cast<int8_t>(std::max<int>(0, g.reasons[i]))});
        c.on_decode_done(op, t, now); })
      .def("limit_blocks_per_replica", &Controller::limit_blocks_per_replica)
      .def_property_readonly("max_blocks_per_replica", &Controller::max_blocks_per_replica)
      .def("set_reachable", &Controller::set_reachable).def("reachable", &Controller::reachable)
      .def("take_flows", &Controller::take_flows).def("waiting_migration_tokens", &Controller::waiting_migration_tokens)
      .def("set_compact_deliveries", &Controller::set_compact_deliveries)
      .def("take_deliveries", [](Controller& c) {
        // (request id, token, final) with final = 0 while the request goes on, else 1 + finish reason
        // (1 length, 2 EOS token, 3 stop sequence)
        std::vector<std::tuple<uint64_t, int32_t, int>> out;
        for (auto& d : c.take_deliveries()) out.emplace_back(d.request_id, d.token, d.final ? 1 + d.reason : 0);
        return out; })
      // completions given as three parallel lists (request ids, tokens, finished flags): cheaper to build than one
      // TokenOut object per token
      .def("on_prefill_done_lists", [](Controller& c, uint64_t op, const std::vector<uint64_t>& ids, const std::vector<int32_t>& toks,
                                       const std::vector<bool>& fins, double now, const std::vector<int>& reasons) {
        if (ids.size() != toks.size() || ids.size() != fins.size() || (!reasons.empty() && reasons.size() != ids.size()))
          throw std::invalid_argument("lists differ in length");
        std::vector<Controller::TokenOut> t;
        t.reserve(ids.size());
        for (size_t i = 0; i < ids.size(); ++i)
          t.push_back({ids[i], toks[i], fins[i], static_cast<int8_t>(reasons.empty() ? 0 : std::max(0, reasons[i]))});
        c.on_prefill_done(op, t, now); },
        py::arg("op_id"), py::arg("request_ids"), py::arg("tokens"), py::arg("finished"), py::arg("now"),
        py::arg("reasons") = std::vector<int>{})
      .def("on_decode_done_lists", [](Controller& c, uint64_t op, const std::vector<uint64_t>& ids, const std::vector<int32_t>& toks,
                                      const std::vector<bool>& fins, double now) {
        if (ids.size() != toks.size() || ids.size() != fins.size()) throw std::invalid_argument("lists differ in length");
        std::vector<Controller::TokenOut> t;
        t.reserve(ids.size());
        for (size_t i = 0; i < ids.size(); ++i) t.push_back({ids[i], toks[i], fins[i]});
        c.on_decode_done(op, t, now); })
      .def_property_readonly("num_replicas", &Controller::num_replicas).def("metric", &Controller::metric)
      .def("state_name", &Controller::state_name).def_property_readonly("queue_size", &Controller::queue_size)
      .def_property_readonly("waiting_prefill_tokens", &Controller::waiting_prefill_tokens)
      .def("counters", &Controller::counters).def("gauges", &Controller::gauges).def("drain_log", &Controller::drain_log)
      .def("system_metrics_line", &Controller::system_metrics_line).def("idle", &Controller::idle)
      .def("token_counts", &Controller::token_counts).def("on_replica_unhealthy", &Controller::on_replica_unhealthy)
      .def("inflight_ops", &Controller::inflight_ops).def("total_used_blocks", &Controller::total_used_blocks)
      .def("request", [](const Controller& c, uint64_t id) -> py::object {
        const RequestEntry* e = c.request(id); if (!e) return py::none(); return py::cast(*e); })
      .def("finished", &Controller::finished).def("pop_finished", &Controller::pop_finished).def("last_target", &Controller::last_target)
      .def("has_feature", [](const Controller& c, const std::string& f) { return c.features().has(f); });
}
