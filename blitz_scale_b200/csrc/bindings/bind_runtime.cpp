#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <pybind11/numpy.h>
#include "runtime/hyper.h"
#include "runtime/kv_pool.h"
#include "runtime/zigzag.h"
#include "runtime/model_loader.h"
namespace py = pybind11;
using namespace blitz;

void bind_runtime(py::module_& m) {
  py::class_<ModelShape>(m, "ModelShape")
      .def_readonly("name", &ModelShape::name).def_readonly("vocab", &ModelShape::vocab)
      .def_readonly("hidden", &ModelShape::hidden).def_readonly("layers", &ModelShape::layers)
      .def_readonly("q_heads", &ModelShape::q_heads).def_readonly("kv_heads", &ModelShape::kv_heads)
      .def_readonly("head_dim", &ModelShape::head_dim).def_readonly("inter", &ModelShape::inter)
      .def_readonly("rope_theta", &ModelShape::rope_theta).def_readonly("rms_eps", &ModelShape::rms_eps)
      .def_readonly("param_gb", &ModelShape::param_gb)
      .def("kv_bytes_per_token", &ModelShape::kv_bytes_per_token);
  m.def("get_model", &get_model, py::return_value_policy::copy);
  m.def("model_names", [] { std::vector<std::string> v; for (auto& kv : model_registry()) v.push_back(kv.first); return v; });
  py::class_<TensorSlot>(m, "TensorSlot").def_readonly("name", &TensorSlot::name).def_readonly("shape", &TensorSlot::shape)
      .def_readonly("offset", &TensorSlot::offset).def_readonly("nbytes", &TensorSlot::nbytes);
  py::class_<UnitSlot>(m, "UnitSlot").def_readonly("name", &UnitSlot::name).def_readonly("offset", &UnitSlot::offset)
      .def_readonly("nbytes", &UnitSlot::nbytes);
  py::class_<SegmentLayout>(m, "SegmentLayout").def_readonly("tensors", &SegmentLayout::tensors)
      .def_readonly("units", &SegmentLayout::units).def_readonly("total_bytes", &SegmentLayout::total_bytes);
  m.def("build_segment_layout", [](const std::string& name, int tp, int elem) {
    return build_segment_layout(get_model(name), tp, elem); });
  py::class_<ModelStatus>(m, "ModelStatus").def(py::init([](int layers) { ModelStatus s; s.total_layers = layers; return s; }))
      .def_readwrite("embed_ready", &ModelStatus::embed_ready).def_readwrite("layers_ready", &ModelStatus::layers_ready)
      .def_readwrite("head_ready", &ModelStatus::head_ready).def_readonly("total_layers", &ModelStatus::total_layers)
      .def("fully_loaded", &ModelStatus::fully_loaded).def("empty", &ModelStatus::empty)
      .def("set_ready", &ModelStatus::set_ready).def("reset", &ModelStatus::reset)
      .def("unit_arrived", &ModelStatus::unit_arrived);

  py::class_<PagePool>(m, "PagePool").def(py::init<int, int>(), py::arg("num_pages"), py::arg("page_size"))
      .def_property_readonly("page_size", &PagePool::page_size).def_property_readonly("total_pages", &PagePool::total_pages)
      .def_property_readonly("free_pages", &PagePool::free_pages).def_property_readonly("used_pages", &PagePool::used_pages)
      .def("allocate", [](PagePool& p, int n) -> py::object {
        std::vector<int32_t> out; if (!p.allocate(n, out)) return py::none(); return py::cast(out); })
      .def("release", &PagePool::release).def("is_used", &PagePool::is_used);

  py::class_<SeqSpec>(m, "SeqSpec").def(py::init<>())
      .def(py::init([](uint64_t id, std::vector<int32_t> prompt, int max_new, bool ignore_eos, int eos) {
             SeqSpec s; s.id = id; s.prompt = std::move(prompt); s.max_new_tokens = max_new; s.ignore_eos = ignore_eos;
             s.eos_token = eos; return s; }),
           py::arg("id"), py::arg("prompt"), py::arg("max_new_tokens") = 16, py::arg("ignore_eos") = true,
           py::arg("eos_token") = -1)
      .def_readwrite("id", &SeqSpec::id).def_readwrite("prompt", &SeqSpec::prompt)
      .def_readwrite("max_new_tokens", &SeqSpec::max_new_tokens).def_readwrite("ignore_eos", &SeqSpec::ignore_eos)
      .def_readwrite("eos_token", &SeqSpec::eos_token).def_readwrite("do_sample", &SeqSpec::do_sample)
      .def_readwrite("temperature", &SeqSpec::temperature).def_readwrite("top_p", &SeqSpec::top_p)
      .def_readwrite("top_k", &SeqSpec::top_k).def_readwrite("seed", &SeqSpec::seed);
  py::class_<SeqState>(m, "SeqState").def_readonly("spec", &SeqState::spec).def_readonly("generated", &SeqState::generated)
      .def_readonly("pages", &SeqState::pages).def_readonly("cached_tokens", &SeqState::cached_tokens)
      .def_property_readonly("finish", [](const SeqState& s) { return static_cast<int>(s.finish); })
      .def("total_len", &SeqState::total_len);
  py::class_<MetaLayout>(m, "MetaLayout").def_static("make", &MetaLayout::make)
      .def_readonly("ids", &MetaLayout::ids).def_readonly("pos", &MetaLayout::pos).def_readonly("slot", &MetaLayout::slot)
      .def_readonly("tok_indptr", &MetaLayout::tok_indptr).def_readonly("page_indptr", &MetaLayout::page_indptr)
      .def_readonly("last_page_len", &MetaLayout::last_page_len).def_readonly("page_indices", &MetaLayout::page_indices)
      .def_readonly("total", &MetaLayout::total);
  py::class_<Batch>(m, "Batch").def(py::init<uint64_t, PagePool*>(), py::keep_alive<1, 3>())
      .def_property_readonly("id", &Batch::id).def_property_readonly("size", &Batch::size)
      .def_property_readonly("seqs", &Batch::seqs, py::return_value_policy::reference_internal)
      .def_property("decode", &Batch::is_decode, &Batch::set_decode)
      .def("max_tokens", &Batch::max_tokens).def("num_pages", &Batch::num_pages)
      .def("num_prompt_tokens", &Batch::num_prompt_tokens).def("max_seq_len", &Batch::max_seq_len)
      .def("add_prompts", &Batch::add_prompts).def("mark_prefilled", &Batch::mark_prefilled)
      .def("append_tokens", &Batch::append_tokens, py::arg("tokens"), py::arg("count_cached") = true)
      .def("filter", &Batch::filter).def("unfinished_ids", &Batch::unfinished_ids)
      .def("generated_tail", &Batch::generated_tail).def("finish_request", &Batch::finish_request)
      .def("extend", &Batch::extend).def("clear", &Batch::clear)
      .def("request_ids", &Batch::request_ids).def("prompt_lens", &Batch::prompt_lens).def("emit_info", &Batch::emit_info)
      .def("encode_generations", [](const Batch& b, const std::vector<int32_t>& toks) { return py::bytes(b.encode_generations(toks)); })
      .def("sampling_rows", [](const Batch& b) {
        auto r = b.sampling_rows();
        return py::make_tuple(r.rows, r.temperature, r.top_k, r.top_p, r.seeds); })
      .def("none_generated", &Batch::none_generated).def("prompt_page_ids", &Batch::prompt_page_ids)
      .def("prompt_page_ids_for", &Batch::prompt_page_ids_for)
      .def("fill_prefill", [](const Batch& b, py::array_t<int32_t, py::array::c_style> h, const MetaLayout& L) {
        if (h.size() < L.total) throw std::invalid_argument("staging array too small");
        return b.fill_prefill(h.mutable_data(), L); })
      .def("fill_prefill_chunk", [](const Batch& b, py::array_t<int32_t, py::array::c_style> h, const MetaLayout& L,
                                    int64_t tok0, int max_tokens) {
        if (h.size() < L.total) throw std::invalid_argument("staging array too small");
        auto c = b.fill_prefill_chunk(h.mutable_data(), L, tok0, max_tokens);
        return py::make_tuple(c.tokens, c.pages, c.rows, c.first_seq, c.q_lens, c.kv_lens, c.ended); })
      .def("fill_decode", [](const Batch& b, py::array_t<int32_t, py::array::c_style> h, const MetaLayout& L, int pad_to) {
        if (h.size() < L.total) throw std::invalid_argument("staging array too small");
        return b.fill_decode(h.mutable_data(), L, pad_to); });

  bind_zigzag(m);
  bind_loader(m);
}
