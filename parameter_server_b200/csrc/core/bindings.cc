// pybind11 module `_core`: the host runtime of the parameter server.
#include "bind_common.h"

namespace PS {
void BindSystem(py::module& m);
void BindUtil(py::module& m);
void BindApp(py::module& m);
}  // namespace PS

PYBIND11_MODULE(_core, m) {
  m.doc() = "Host runtime: messages, executor DAG engine, van, manager, shared parameters, filters, parsers";
  py::register_exception<PS::CheckError>(m, "CheckError");
  PS::BindSystem(m);
  PS::BindUtil(m);
  PS::BindApp(m);
}
