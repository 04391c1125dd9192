#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include "sim/cluster_sim.h"
namespace py = pybind11;
using namespace blitz;

void bind_sim(py::module_& m) {
  py::class_<Rng>(m, "Rng").def(py::init<uint64_t>()).def("uniform", &Rng::uniform).def("exponential", &Rng::exponential)
      .def("normal", &Rng::normal).def("gamma", &Rng::gamma).def("uniform_int", &Rng::uniform_int).def("next_u64", &Rng::next_u64);
  py::class_<LengthDist> ld(m, "LengthDist");
  py::enum_<LengthDist::Kind>(ld, "Kind").value("Fixed", LengthDist::Fixed).value("Uniform", LengthDist::Uniform)
      .value("LogNormal", LengthDist::LogNormal);
  ld.def(py::init<>()).def_readwrite("kind", &LengthDist::kind).def_readwrite("a", &LengthDist::a).def_readwrite("b", &LengthDist::b)
      .def_readwrite("max_len", &LengthDist::max_len).def_readwrite("min_len", &LengthDist::min_len).def("sample", &LengthDist::sample);
  py::class_<RatePhase>(m, "RatePhase").def(py::init([](double t, double r) { return RatePhase{t, r}; }))
      .def_readwrite("t_start", &RatePhase::t_start).def_readwrite("rate", &RatePhase::rate);
  py::class_<TraceItem>(m, "TraceItem").def(py::init([](double t, int64_t i, int64_t o, uint64_t s) { return TraceItem{t, i, o, s}; }))
      .def_readonly("t", &TraceItem::t).def_readonly("input_len", &TraceItem::input_len)
      .def_readonly("output_len", &TraceItem::output_len).def_readonly("seed", &TraceItem::seed);
  py::class_<TraceSpec>(m, "TraceSpec").def(py::init<>()).def_readwrite("phases", &TraceSpec::phases)
      .def_readwrite("cv", &TraceSpec::cv).def_readwrite("duration", &TraceSpec::duration)
      .def_readwrite("max_requests", &TraceSpec::max_requests).def_readwrite("input", &TraceSpec::input)
      .def_readwrite("output", &TraceSpec::output).def_readwrite("seed", &TraceSpec::seed);
  m.def("generate_trace", &generate_trace);
  m.def("load_trace_csv", &load_trace_csv, py::arg("path"), py::arg("scale_factor") = 1.0, py::arg("truncate") = 4095);

  py::class_<CostModel>(m, "CostModel").def(py::init<>())
      .def_readwrite("prefill_tokens_per_s", &CostModel::prefill_tokens_per_s)
      .def_readwrite("prefill_overhead_s", &CostModel::prefill_overhead_s)
      .def_readwrite("decode_step_base_s", &CostModel::decode_step_base_s)
      .def_readwrite("decode_step_per_seq_s", &CostModel::decode_step_per_seq_s)
      .def_readwrite("kv_tokens_per_s", &CostModel::kv_tokens_per_s).def_readwrite("migrate_overhead_s", &CostModel::migrate_overhead_s)
      .def_readwrite("param_gb", &CostModel::param_gb).def_readwrite("nvlink_gbs", &CostModel::nvlink_gbs)
      .def_readwrite("host_gbs", &CostModel::host_gbs).def_readwrite("disk_gbs", &CostModel::disk_gbs)
      .def_readwrite("rpc_overhead_s", &CostModel::rpc_overhead_s).def_readwrite("layers", &CostModel::layers);
  py::class_<SimRequestResult>(m, "SimRequestResult").def_readonly("id", &SimRequestResult::id)
      .def_readonly("t_arrival", &SimRequestResult::t_arrival).def_readonly("ttft", &SimRequestResult::ttft)
      .def_readonly("max_tbt", &SimRequestResult::max_tbt).def_readonly("avg_tbt", &SimRequestResult::avg_tbt)
      .def_readonly("t_done", &SimRequestResult::t_done).def_readonly("input_len", &SimRequestResult::input_len)
      .def_readonly("output_len", &SimRequestResult::output_len);
  py::class_<SimReport>(m, "SimReport").def_readonly("requests", &SimReport::requests).def_readonly("log", &SimReport::log)
      .def_readonly("submitted", &SimReport::submitted).def_readonly("completed", &SimReport::completed)
      .def_readonly("failed", &SimReport::failed).def_readonly("gone_in_queue", &SimReport::gone_in_queue)
      .def_readonly("gone_in_service", &SimReport::gone_in_service).def_readonly("delivered_tokens", &SimReport::delivered_tokens)
      .def_readonly("end_time", &SimReport::end_time).def_readonly("leftover_blocks", &SimReport::leftover_blocks)
      .def_readonly("prefill_replicas", &SimReport::prefill_replicas).def_readonly("decode_replicas", &SimReport::decode_replicas)
      .def_readonly("scale_up_latency", &SimReport::scale_up_latency);
  py::class_<ClusterSim>(m, "ClusterSim").def(py::init<const ControllerConfig&, const CostModel&>())
      .def("run", &ClusterSim::run, py::arg("trace"), py::arg("tick_s") = 0.001, py::arg("drain_s") = 120.0,
           py::arg("kill_replica") = -1, py::arg("kill_at") = -1.0, py::arg("gone_every") = 0)
      .def("controller", &ClusterSim::controller, py::return_value_policy::reference_internal);
}
