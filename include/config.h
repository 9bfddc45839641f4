// Geometry-independent operator configuration (src/config.h:11-29 of the reference).
#ifndef INFINI_OPS_CONFIG_H_
#define INFINI_OPS_CONFIG_H_

#include <cstddef>
#include <memory>

namespace infini::ops {

class Config {
 public:
  virtual ~Config() = default;
  virtual std::unique_ptr<Config> Clone() const { return std::make_unique<Config>(*this); }

  std::size_t implementation_index() const { return implementation_index_; }
  void set_implementation_index(std::size_t index) { implementation_index_ = index; }

 private:
  std::size_t implementation_index_{0};
};

}  // namespace infini::ops

#endif
