// Per-call runtime resources: stream, optional workspace (src/handle.h:10-41 of the reference).
#ifndef INFINI_OPS_HANDLE_H_
#define INFINI_OPS_HANDLE_H_

#include <cstddef>
#include <memory>

namespace infini::ops {

class Handle {
 public:
  virtual ~Handle() = default;
  virtual std::unique_ptr<Handle> Clone() const { return std::make_unique<Handle>(*this); }

  void* stream() const { return stream_; }
  void* workspace() const { return workspace_; }
  std::size_t workspace_size_in_bytes() const { return workspace_size_in_bytes_; }

  void set_stream(void* stream) { stream_ = stream; }
  void set_workspace(void* workspace) { workspace_ = workspace; }
  void set_workspace_size_in_bytes(std::size_t bytes) { workspace_size_in_bytes_ = bytes; }

 private:
  void* stream_{nullptr};
  void* workspace_{nullptr};
  std::size_t workspace_size_in_bytes_{0};
};

}  // namespace infini::ops

#endif
