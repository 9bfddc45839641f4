// Conversions shared by the binding translation units (Python object -> Tensor view, Handle, Config).
#ifndef INFINI_OPS_BINDING_UTILS_H_
#define INFINI_OPS_BINDING_UTILS_H_

#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>
#include <memory>
#include <optional>
#include <string>

#include "infini/ops.h"

namespace py = pybind11;
using namespace infini::ops;


inline Device::Type DeviceTypeFromString(const std::string& name) {
  if (name == "cuda" || name == "nvidia") return Device::Type::kNvidia;
  if (name == "cpu") return Device::Type::kCpu;
  throw py::value_error("unsupported device `" + name + "`: this build supports cuda / nvidia only");
}

inline Tensor ToTensor(const py::handle& obj) {
  auto* data = reinterpret_cast<void*>(obj.attr("data_ptr")().cast<std::uintptr_t>());
  auto shape = obj.attr("shape").cast<Tensor::Shape>();
  auto strides = obj.attr("stride")().cast<Tensor::Strides>();
  DataType dtype;
  const std::string dtype_name = py::str(obj.attr("dtype")).cast<std::string>();
  if (!infini::rt::DataTypeFromString(dtype_name, dtype)) throw py::value_error("unsupported dtype `" + dtype_name + "`");
  const py::object device = obj.attr("device");
  const py::object index = device.attr("index");
  return Tensor{data, std::move(shape), dtype,
                Device{DeviceTypeFromString(device.attr("type").cast<std::string>()), index.is_none() ? 0 : index.cast<int>()},
                std::move(strides)};
}

inline std::optional<Tensor> ToOptional(const py::object& obj) {
  if (obj.is_none()) return std::nullopt;
  return ToTensor(obj);
}

inline Handle MakeHandle(std::uintptr_t stream) {
  Handle handle;
  handle.set_stream(reinterpret_cast<void*>(stream));
  return handle;
}

inline Config MakeConfig(const py::object& implementation_index) {
  Config config;
  if (!implementation_index.is_none()) config.set_implementation_index(implementation_index.cast<std::size_t>());
  return config;
}

// Owning wrapper behind the PascalCase classes.
template <typename Key>
struct Descriptor {
  std::unique_ptr<Operator<Key>> op;
};

template <typename Key, typename Class>
void AddStatics(Class& cls) {
  cls.def_static("active_implementation_indices",
                 [](const std::string& device) { return Key::active_implementation_indices(DeviceTypeFromString(device)); })
      .def_static("clear_cache", [] { Key::clear_cache(); });
}

#define KW py::kw_only(), py::arg("stream") = 0, py::arg("implementation_index") = py::none()



#endif
