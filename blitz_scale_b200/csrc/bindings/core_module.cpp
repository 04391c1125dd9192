// pybind11 module `blitz_core`: the native runtime (page pool, batches, shapes), router core and
// simulator exposed to the Python shells.
#include <pybind11/pybind11.h>
namespace py = pybind11;
void bind_runtime(py::module_& m);
void bind_router(py::module_& m);
void bind_sim(py::module_& m);
void bind_text(py::module_& m);

PYBIND11_MODULE(blitz_core, m) {
  m.doc() = "native cores of blitz_scale_b200";
  bind_runtime(m);
  bind_router(m);
  bind_sim(m);
  bind_text(m);
}
