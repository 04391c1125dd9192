// Bindings and C ABI of the tokenizer and the safetensors reader.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include "runtime/safetensors.h"
#include "runtime/tokenizer.h"
#include "util/log.h"
namespace py = pybind11;
using namespace blitz;

// ---- C ABI (same five operations as the reference's tokenizer binding; handles are opaque) -------------------
#define BLITZ_EXPORT extern "C" __attribute__((visibility("default")))

BLITZ_EXPORT void* blitz_tokenizer_create_from_file(const char* path) {
  try {
    return new Tokenizer(Tokenizer::from_file(path));
  } catch (...) {
    return nullptr;
  }
}
BLITZ_EXPORT void blitz_tokenizer_free(void* h) { delete static_cast<Tokenizer*>(h); }
BLITZ_EXPORT int32_t blitz_tokenizer_num_ids(void* h) { return static_cast<Tokenizer*>(h)->num_ids(); }
BLITZ_EXPORT int32_t blitz_tokenizer_get_id(void* h, const char* token) { return static_cast<Tokenizer*>(h)->get_id(token); }
// Writes at most `cap` ids to `out`; returns the number of ids the text encodes to (call again with a larger buffer
// if it exceeds `cap`).
BLITZ_EXPORT int64_t blitz_tokenizer_encode(void* h, const char* text, int64_t len, int32_t* out, int64_t cap) {
  const std::vector<int32_t> ids = static_cast<Tokenizer*>(h)->encode(std::string_view(text, static_cast<size_t>(len)));
  const int64_t n = static_cast<int64_t>(ids.size());
  if (out && cap > 0) std::memcpy(out, ids.data(), sizeof(int32_t) * static_cast<size_t>(n < cap ? n : cap));
  return n;
}
// Writes at most `cap` bytes (no terminator) to `out`; returns the byte length of the decoded text.
BLITZ_EXPORT int64_t blitz_tokenizer_decode(void* h, const int32_t* ids, int64_t n, int skip_special, char* out, int64_t cap) {
  const std::string s = static_cast<Tokenizer*>(h)->decode(std::vector<int32_t>(ids, ids + n), skip_special != 0);
  const int64_t len = static_cast<int64_t>(s.size());
  if (out && cap > 0) std::memcpy(out, s.data(), static_cast<size_t>(len < cap ? len : cap));
  return len;
}

void bind_text(py::module_& m) {
  // native logger and contract macros (the Python shells log through `logging`; this is for the C++ side and tests)
  m.def("native_log", [](int level, const std::string& msg) {
    ::blitz::log::emit(static_cast<::blitz::log::Level>(level), "python", 0, "%s", msg.c_str()); });
  m.def("set_native_log_level", [](const std::string& name) { ::blitz::log::set_threshold(::blitz::log::parse_level(name.c_str())); });
  m.def("native_log_enabled", [](int level) { return ::blitz::log::enabled(static_cast<::blitz::log::Level>(level)); });
  m.def("check_precondition", [](bool ok) { Precondition(ok); });
  py::class_<Tokenizer>(m, "Tokenizer")
      .def_static("from_file", [](const std::string& p) { return new Tokenizer(Tokenizer::from_file(p)); },
                  py::return_value_policy::take_ownership)
      .def_static("from_json", [](const std::string& s) { return new Tokenizer(Tokenizer::from_json(s)); },
                  py::return_value_policy::take_ownership)
      .def("encode", [](const Tokenizer& t, const std::string& s) {
             py::gil_scoped_release rel;
             return t.encode(s); })
      // byte-level tokens can end in the middle of a character (a model may emit any id): such bytes become U+FFFD,
      // as in the `tokenizers` library, instead of an exception
      .def("decode", [](const Tokenizer& t, const std::vector<int32_t>& ids, bool skip) {
             const std::string s = t.decode(ids, skip);
             PyObject* u = PyUnicode_DecodeUTF8(s.data(), static_cast<Py_ssize_t>(s.size()), "replace");
             if (!u) throw py::error_already_set();
             return py::reinterpret_steal<py::str>(u); },
           py::arg("ids"), py::arg("skip_special_tokens") = true)
      .def("decode_bytes", [](const Tokenizer& t, const std::vector<int32_t>& ids, bool skip) { return py::bytes(t.decode(ids, skip)); },
           py::arg("ids"), py::arg("skip_special_tokens") = true)
      .def("num_ids", &Tokenizer::num_ids)
      .def("is_special", &Tokenizer::is_special)
      .def("get_id", &Tokenizer::get_id)
      .def("token", &Tokenizer::token);

  py::class_<SafeTensorInfo>(m, "SafeTensorInfo")
      .def_readonly("name", &SafeTensorInfo::name).def_readonly("dtype", &SafeTensorInfo::dtype)
      .def_readonly("shape", &SafeTensorInfo::shape)
      .def_property_readonly("nbytes", [](const SafeTensorInfo& t) { return t.end - t.begin; });
  py::class_<SafeTensorsFile>(m, "SafeTensorsFile")
      .def(py::init<const std::string&>())
      .def("tensors", &SafeTensorsFile::tensors)
      .def("metadata", &SafeTensorsFile::metadata)
      .def("names", [](const SafeTensorsFile& f) { std::vector<std::string> v; for (auto& t : f.tensors()) v.push_back(t.name); return v; })
      .def("info", [](const SafeTensorsFile& f, const std::string& n) {
             const SafeTensorInfo* t = f.find(n);
             if (!t) throw py::key_error(n);
             return *t; })
      // read-only view of the mapped bytes; the file object stays alive as long as the view does
      .def("view", [](py::object self, const std::string& n) {
             const SafeTensorsFile& f = self.cast<const SafeTensorsFile&>();
             const SafeTensorInfo* t = f.find(n);
             if (!t) throw py::key_error(n);
             py::object mv = py::memoryview::from_memory(const_cast<uint8_t*>(f.data(*t)), static_cast<py::ssize_t>(t->end - t->begin), true);
             return py::make_tuple(mv, self); });
}
