// Minimal stand-in for the InfiniRT public types the operator API is written against.
//
// The reference aliases `infini::ops::Tensor`, `Device` and `DataType` to InfiniRT types
// (src/tensor.h:8, src/device.h:10, src/data_type.h:11 of the reference); InfiniRT itself is a
// separate library.  This header provides the same names, members and semantics for the parts
// the operators of this library use: a non-owning tensor view, a device tag and the element
// type enumeration.
#ifndef INFINI_RT_H_
#define INFINI_RT_H_

#include <cstddef>
#include <cstdint>
#include <functional>
#include <string_view>
#include <utility>
#include <vector>

namespace infini::rt {

enum class DataType : int {
  kInt8, kInt16, kInt32, kInt64, kUInt8, kUInt16, kUInt32, kUInt64, kFloat16, kBFloat16, kFloat32, kFloat64,
};

inline constexpr std::size_t kDataTypeSizes[] = {1, 2, 4, 8, 1, 2, 4, 8, 2, 2, 4, 8};
inline constexpr std::string_view kDataTypeNames[] = {"int8",   "int16",  "int32",   "int64",    "uint8",   "uint16",
                                                      "uint32", "uint64", "float16", "bfloat16", "float32", "float64"};

inline std::size_t SizeOf(DataType t) { return kDataTypeSizes[static_cast<int>(t)]; }
inline std::string_view NameOf(DataType t) { return kDataTypeNames[static_cast<int>(t)]; }

// Parses "float16", "torch.float16", "bool" (carried as uint8, as the reference's binding layer does,
// src/pybind11_utils.h:106-111).  Returns false for an unknown name.
inline bool DataTypeFromString(std::string_view name, DataType& out) {
  const auto dot = name.rfind('.');
  if (dot != std::string_view::npos) name.remove_prefix(dot + 1);
  if (name == "bool") {
    out = DataType::kUInt8;
    return true;
  }
  if (name == "half") name = "float16";
  if (name == "float") name = "float32";
  if (name == "double") name = "float64";
  if (name == "int") name = "int32";
  if (name == "long") name = "int64";
  for (int i = 0; i < 12; ++i) {
    if (kDataTypeNames[i] == name) {
      out = static_cast<DataType>(i);
      return true;
    }
  }
  return false;
}

class Device {
 public:
  enum class Type : int { kCpu, kNvidia, kCambricon, kAscend, kMetax, kMoore, kIluvatar, kHygon, kCount };

  Device() = default;
  Device(Type type, int index = 0) : type_{type}, index_{index} {}

  Type type() const { return type_; }
  int index() const { return index_; }

  static std::string_view StringFromType(Type type) {
    constexpr std::string_view names[] = {"cpu", "nvidia", "cambricon", "ascend", "metax", "moore", "iluvatar",
                                          "hygon", "unknown"};
    return names[static_cast<int>(type)];
  }

  bool operator==(const Device& o) const { return type_ == o.type_ && index_ == o.index_; }
  bool operator!=(const Device& o) const { return !(*this == o); }

 private:
  Type type_{Type::kCpu};
  int index_{0};
};

// Non-owning view of a strided tensor: pointer, shape, element type, device, strides (in elements).
class TensorView {
 public:
  using Size = std::size_t;
  using Stride = std::ptrdiff_t;
  using Index = std::ptrdiff_t;
  using Shape = std::vector<Size>;
  using Strides = std::vector<Stride>;

  TensorView() = default;
  TensorView(void* data, Shape shape, DataType dtype = DataType::kFloat32, Device device = Device{})
      : data_{data}, shape_{std::move(shape)}, dtype_{dtype}, device_{device}, strides_{Contiguous(shape_)} {}
  TensorView(void* data, Shape shape, DataType dtype, Device device, Strides strides)
      : data_{data}, shape_{std::move(shape)}, dtype_{dtype}, device_{device}, strides_{std::move(strides)} {}
  TensorView(void* data, Shape shape, Device device) : TensorView(data, std::move(shape), DataType::kFloat32, device) {}

  void* data() const { return data_; }
  const Shape& shape() const { return shape_; }
  const Strides& strides() const { return strides_; }
  DataType dtype() const { return dtype_; }
  const Device& device() const { return device_; }
  Size ndim() const { return shape_.size(); }
  Size size(Index i) const { return shape_[Wrap(i)]; }
  Stride stride(Index i) const { return strides_[Wrap(i)]; }
  Size element_size() const { return SizeOf(dtype_); }
  Size numel() const {
    Size n = 1;
    for (Size s : shape_) n *= s;
    return n;
  }
  bool IsContiguous() const {
    Stride expect = 1;
    for (Index d = static_cast<Index>(shape_.size()) - 1; d >= 0; --d) {
      if (shape_[d] != 1 && strides_[d] != expect) return false;
      expect *= static_cast<Stride>(shape_[d]);
    }
    return true;
  }

  static Strides Contiguous(const Shape& shape) {
    Strides s(shape.size());
    Stride run = 1;
    for (Index d = static_cast<Index>(shape.size()) - 1; d >= 0; --d) {
      s[d] = run;
      run *= static_cast<Stride>(shape[d]);
    }
    return s;
  }

 private:
  std::size_t Wrap(Index i) const { return static_cast<std::size_t>(i < 0 ? i + static_cast<Index>(shape_.size()) : i); }

  void* data_{nullptr};
  Shape shape_;
  DataType dtype_{DataType::kFloat32};
  Device device_;
  Strides strides_;
};

}  // namespace infini::rt

// Hash and equality over METADATA only (shape, strides, element type, device) -- never the data
// pointer: operator descriptors are cached per geometry and reused with other buffers.
template <>
struct std::hash<infini::rt::TensorView> {
  std::size_t operator()(const infini::rt::TensorView& t) const {
    std::size_t h = static_cast<std::size_t>(t.dtype()) * 1315423911u + static_cast<std::size_t>(t.device().type()) * 31u +
                    static_cast<std::size_t>(t.device().index());
    for (auto s : t.shape()) h = h * 1099511628211ull + s;
    for (auto s : t.strides()) h = h * 1099511628211ull + static_cast<std::size_t>(s);
    return h;
  }
};
template <>
struct std::equal_to<infini::rt::TensorView> {
  bool operator()(const infini::rt::TensorView& a, const infini::rt::TensorView& b) const {
    return a.dtype() == b.dtype() && a.device() == b.device() && a.shape() == b.shape() && a.strides() == b.strides();
  }
};

#endif  // INFINI_RT_H_
