// Operator front end: descriptor construction, per-thread descriptor cache, call forwarding.
//
// Same public surface as the reference's src/operator.h:205-468 -- `Op::Call(handle, config,
// args...)`, `Op::Call(tensor, args...)`, `Op::Make([config,] args...)`, `(*op)([handle,]
// args...)`, `Op::active_implementation_indices(device_type)`, `Op::clear_cache()`, and the
// `INFINI_OPS_TRACE_CALLS` line per dispatched call (src/operator.h:126-171) -- but with a single
// back end: an operator `Key` is implemented by the specialisation
// `Operator<Key, Device::Type::kNvidia, 0>` (plus, for the Marlin GEMMs, slot 16) or not at all.  A request for any other device or
// slot prints a message and aborts, like a dispatcher miss in the reference
// (src/dispatcher.h:44-49).
#ifndef INFINI_OPS_OPERATOR_H_
#define INFINI_OPS_OPERATOR_H_

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <optional>
#include <string>
#include <type_traits>
#include <unordered_map>
#include <utility>
#include <vector>

#include "config.h"
#include "handle.h"
#include "tensor.h"

namespace infini::ops {

// Validation failure: message on stderr, then abort -- the reference validates with `assert`, and
// its tests look for these texts in the stderr of a child process.  Always on here.
[[noreturn]] inline void CheckFailed(const char* expr, const char* message, const char* file, int line) {
  std::fprintf(stderr, "%s:%d: Assertion `%s && \"%s\"' failed.\n", file, line, expr, message);
  std::fflush(stderr);
  std::abort();
}
#define INFINI_OPS_CHECK(cond, message) \
  ((cond) ? static_cast<void>(0) : ::infini::ops::CheckFailed(#cond, message, __FILE__, __LINE__))

class OperatorBase {
 public:
  virtual ~OperatorBase() = default;
  virtual std::size_t workspace_size_in_bytes() const { return 0; }

  void set_handle(const Handle& handle) { handle_ptr_ = handle.Clone(); }
  void set_config(const Config& config) { config_ptr_ = config.Clone(); }
  void set_stream(void* stream) { stream_ = stream; }
  void set_workspace(void* workspace) { workspace_ = workspace; }
  void set_workspace_size_in_bytes(std::size_t bytes) { workspace_size_in_bytes_ = bytes; }

 protected:
  std::unique_ptr<Handle> handle_ptr_;
  std::unique_ptr<Config> config_ptr_;
  void* stream_{nullptr};
  void* workspace_{nullptr};
  std::size_t workspace_size_in_bytes_{0};
};

namespace detail {

// Cache key: implementation index, then the metadata of every tensor argument (never its data
// pointer) and the value of every scalar argument, serialised into one byte string.
class KeyBytes {
 public:
  void Add(const Tensor& t) {
    Raw(static_cast<int>(t.dtype()));
    Raw(static_cast<int>(t.device().type()));
    Raw(t.device().index());
    Raw(t.ndim());
    for (auto s : t.shape()) Raw(s);
    for (auto s : t.strides()) Raw(s);
  }
  void Add(const std::optional<Tensor>& t) {
    Raw(static_cast<char>(t.has_value()));
    if (t) Add(*t);
  }
  void Add(const std::vector<Tensor>& ts) {
    Raw(ts.size());
    for (const auto& t : ts) Add(t);
  }
  template <typename T, typename = std::enable_if_t<std::is_arithmetic_v<T> || std::is_enum_v<T>>>
  void Add(const T& v) {
    Raw(v);
  }
  std::string Take() { return std::move(bytes_); }

 private:
  template <typename T>
  void Raw(const T& v) {
    bytes_.append(reinterpret_cast<const char*>(&v), sizeof(T));
  }
  std::string bytes_;
};

inline bool TraceCalls() {
  static const bool enabled = [] {
    const char* v = std::getenv("INFINI_OPS_TRACE_CALLS");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  return enabled;
}

inline const Tensor* FirstTensor() { return nullptr; }
template <typename First, typename... Rest>
const Tensor* FirstTensor(const First& first, const Rest&... rest) {
  if constexpr (std::is_same_v<std::decay_t<First>, Tensor>) {
    return &first;
  } else {
    return FirstTensor(rest...);
  }
}

}  // namespace detail

// Implementations specialise this for (Key, Device::Type::kNvidia, 0) and derive from Key.
template <typename Key, Device::Type device_type = Device::Type::kCount, std::size_t implementation_index = 0>
class Operator {};

template <typename Key, Device::Type device_type, std::size_t implementation_index>
inline constexpr bool kIsImplemented = std::is_base_of_v<Key, Operator<Key, device_type, implementation_index>>;

// Slot 16 is where the reference registers a linked provider (vLLM) implementation
// (docs/linked-operators.md:106-110 of the reference).  Operators whose provider takes tensors in
// a layout of its own -- the Marlin GEMMs' permuted scales and zero points -- register a second
// implementation there that reads exactly those layouts, so a caller that selects the provider
// slot keeps working with the tensors it prepared for it.
inline constexpr std::size_t kProviderSlot = 16;

template <typename Key>
class Operator<Key, Device::Type::kCount, 0> : public OperatorBase {
 public:
  using Front = Operator<Key, Device::Type::kCount, 0>;

  // Drops every cached descriptor of this operator at the next Call (test isolation).
  static void clear_cache() { cache_generation_.fetch_add(1, std::memory_order_relaxed); }

  static std::vector<std::size_t> active_implementation_indices(Device::Type type) {
    std::vector<std::size_t> slots;
    if (type == Device::Type::kNvidia && kIsImplemented<Key, Device::Type::kNvidia, 0>) slots.push_back(0);
    if (type == Device::Type::kNvidia && kIsImplemented<Key, Device::Type::kNvidia, kProviderSlot>) slots.push_back(kProviderSlot);
    return slots;
  }

  template <typename... Args>
  static std::unique_ptr<Front> Make(const Config& config, const Tensor tensor, Args&&... args) {
    RequireBackend(tensor.device().type(), config.implementation_index());
    if constexpr (kIsImplemented<Key, Device::Type::kNvidia, kProviderSlot>) {
      if (config.implementation_index() == kProviderSlot) {
        auto op = std::make_unique<Operator<Key, Device::Type::kNvidia, kProviderSlot>>(tensor, std::forward<Args>(args)...);
        op->set_config(config);
        return op;
      }
    }
    if constexpr (kIsImplemented<Key, Device::Type::kNvidia, 0>) {
      auto op = std::make_unique<Operator<Key, Device::Type::kNvidia, 0>>(tensor, std::forward<Args>(args)...);
      op->set_config(config);
      return op;
    } else {
      return nullptr;
    }
  }

  template <typename... Args>
  static std::unique_ptr<Front> Make(const Tensor tensor, Args&&... args) {
    return Make(Config{}, tensor, std::as_const(args)...);
  }

  template <typename... Args>
  static void Call(const Handle& handle, const Config& config, const Args&... args) {
    static thread_local std::unordered_map<std::string, std::unique_ptr<Front>> cache;
    static thread_local std::size_t generation{0};
    const auto now = cache_generation_.load(std::memory_order_relaxed);
    if (generation != now) {
      cache.clear();
      generation = now;
    }
    detail::KeyBytes key;
    key.Add(config.implementation_index());
    (key.Add(args), ...);
    auto bytes = key.Take();
    auto it = cache.find(bytes);
    if (it == cache.end()) it = cache.emplace(std::move(bytes), Make(config, args...)).first;
    if (detail::TraceCalls()) {
      const Tensor* first = detail::FirstTensor(args...);
      const auto device = first ? Device::StringFromType(first->device().type()) : std::string_view{"unknown"};
      std::fprintf(stderr,
                   "[INFINI_OPS_TRACE_CALLS] {\"operator_name\": \"%s\", \"device_type\": \"%.*s\", "
                   "\"implementation\": %zu}\n",
                   Key::kName, static_cast<int>(device.size()), device.data(), config.implementation_index());
    }
    (*it->second)(handle, args...);
  }

  template <typename... Args>
  static void Call(const Tensor tensor, const Args&... args) {
    Call(Handle{}, Config{}, tensor, args...);
  }

  template <typename... Args>
  void operator()(const Handle& handle, const Args&... args) {
    set_stream(handle.stream());
    set_workspace(handle.workspace());
    set_workspace_size_in_bytes(handle.workspace_size_in_bytes());
    static_cast<const Key&>(*this)(args...);
  }

  template <typename First, typename... Args,
            typename = std::enable_if_t<!std::is_base_of_v<Handle, std::decay_t<First>>>>
  void operator()(const First& first, const Args&... args) {
    (*this)(Handle{}, first, args...);
  }

 private:
  static void RequireBackend(Device::Type type, std::size_t index) {
    const bool known = (index == 0 && kIsImplemented<Key, Device::Type::kNvidia, 0>) ||
                       (index == kProviderSlot && kIsImplemented<Key, Device::Type::kNvidia, kProviderSlot>);
    if (type != Device::Type::kNvidia || !known) {
      const auto name = Device::StringFromType(type);
      std::fprintf(stderr, "`%s` has no implementation %zu for device `%.*s` (this build: nvidia, slot 0, and slot 16 for the Marlin GEMMs)\n",
                   Key::kName, index, static_cast<int>(name.size()), name.data());
      std::fflush(stderr);
      std::abort();
    }
  }

  static inline std::atomic<std::size_t> cache_generation_{0};
};

// Helpers shared by the operator descriptors.
inline bool SameDevice(const Tensor& a, const Tensor& b) { return a.device() == b.device(); }
inline bool SameMetadata(const Tensor& a, const Tensor& b) { return std::equal_to<Tensor>{}(a, b); }
inline bool SameMetadata(const std::optional<Tensor>& a, const std::optional<Tensor>& b) {
  return a.has_value() == b.has_value() && (!a || SameMetadata(*a, *b));
}

}  // namespace infini::ops

#endif  // INFINI_OPS_OPERATOR_H_
