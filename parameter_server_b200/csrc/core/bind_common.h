// Shared helpers of the pybind11 bindings.
#pragma once
#include <memory>
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include "sarray.h"

namespace py = pybind11;

namespace PS {

template <typename T>
SArray<T> FromNumpy(const py::array_t<T, py::array::c_style | py::array::forcecast>& a) {
  SArray<T> out;
  out.CopyFrom(a.data(), (size_t)a.size());
  return out;
}
template <typename T>
py::array_t<T> ToNumpy(const SArray<T>& a) {
  py::array_t<T> out((py::ssize_t)a.size());
  if (a.size()) memcpy(out.mutable_data(), a.data(), a.size() * sizeof(T));
  return out;
}

// A Python callable kept alive by C++ objects (message callbacks, failure handlers) whose last owner may
// be a runtime thread: the reference is dropped with the interpreter lock held (and simply leaked once
// the interpreter is gone).
inline std::shared_ptr<py::object> HoldPython(py::object f) {
  return std::shared_ptr<py::object>(new py::object(std::move(f)), [](py::object* p) {
    if (Py_IsInitialized()) {
      py::gil_scoped_acquire g;
      delete p;
    }
  });
}

}  // namespace PS
