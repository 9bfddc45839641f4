// A C++ consumer of the operator API, as an application would write it: `#include <infini/ops.h>`,
// device buffers of its own, a Handle carrying its stream and a workspace whose previous content is
// arbitrary (filled with 0xFF here), then
//   GptqMarlinRepack::Call(handle, config, ...)            (static call through the descriptor cache)
//   MoeAlignBlockSize::Make(...) + (*op)(handle, ...)      (explicit descriptor; > 1024 ids, so the
//                                                           sort writes its histograms into the workspace)
//   MoeWna16MarlinGemm::Call / MarlinGemm::Call            (split-K counters in the SAME workspace)
//   SiluAndMul::MakeReturnValue + SiluAndMul::Call, MoeSum::Make + (*op)(handle, ...)
// Inputs are read from, and results written to, raw little-endian files in the directory given as
// argv[1]; the Python test that builds and runs this program prepares the inputs and checks the
// results against the oracle.  Mirrors the way tests/test_cpp_api.py of the reference exercises
// its C++ API with small compiled programs.
#include <cuda_runtime.h>
#include <infini/ops.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <string>
#include <vector>

using namespace infini::ops;

namespace {

std::string g_dir;

std::vector<char> ReadFile(const std::string& name) {
  std::ifstream in(g_dir + "/" + name, std::ios::binary);
  if (!in) {
    std::fprintf(stderr, "cannot read %s\n", name.c_str());
    std::exit(2);
  }
  return std::vector<char>((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
}

void Check(cudaError_t err, const char* what) {
  if (err != cudaSuccess) {
    std::fprintf(stderr, "%s: %s\n", what, cudaGetErrorString(err));
    std::exit(3);
  }
}

// An owning device tensor of the application: what `MakeReturnValue` is written for.
class Buffer {
 public:
  using Shape = Tensor::Shape;

  static Buffer Empty(const Shape& shape, DataType dtype, Device device) {
    Buffer b;
    b.shape_ = shape;
    b.dtype_ = dtype;
    b.device_ = device;
    size_t n = infini::rt::SizeOf(dtype);
    for (auto s : shape) n *= s;
    b.bytes_ = n;
    Check(cudaMalloc(&b.data_, n ? n : 1), "cudaMalloc");
    return b;
  }
  static Buffer FromFile(const std::string& name, const Shape& shape, DataType dtype) {
    Buffer b = Empty(shape, dtype, Device{Device::Type::kNvidia, 0});
    const auto host = ReadFile(name);
    if (host.size() != b.bytes_) {
      std::fprintf(stderr, "%s: %zu bytes, expected %zu\n", name.c_str(), host.size(), b.bytes_);
      std::exit(2);
    }
    Check(cudaMemcpy(b.data_, host.data(), b.bytes_, cudaMemcpyHostToDevice), "upload");
    return b;
  }
  void ToFile(const std::string& name) const {
    std::vector<char> host(bytes_);
    Check(cudaMemcpy(host.data(), data_, bytes_, cudaMemcpyDeviceToHost), "download");
    std::ofstream out(g_dir + "/" + name, std::ios::binary);
    out.write(host.data(), static_cast<std::streamsize>(host.size()));
  }
  const Shape& shape() const { return shape_; }
  DataType dtype() const { return dtype_; }
  Device device() const { return device_; }
  void* data() const { return data_; }
  size_t bytes() const { return bytes_; }
  Tensor view() const { return Tensor{data_, shape_, dtype_, device_}; }
  Tensor view(const Shape& as) const { return Tensor{data_, as, dtype_, device_}; }

 private:
  void* data_{nullptr};
  Shape shape_;
  DataType dtype_{DataType::kFloat32};
  Device device_;
  size_t bytes_{0};
};

}  // namespace

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  g_dir = argv[1];
  Check(cudaSetDevice(0), "cudaSetDevice");
  cudaStream_t stream;
  Check(cudaStreamCreate(&stream), "cudaStreamCreate");

  // geometry (kept in step with tests/test_cpp_consumer.py)
  constexpr size_t kTokens = 700, kExperts = 8, kTopK = 2, kHidden = 256, kInter = 128, kBlock = 16;
  constexpr size_t kRoutes = kTokens * kTopK;                     // 1400 ids: the multi-block sort path
  constexpr size_t kSorted = kRoutes + kExperts * (kBlock - 1);
  constexpr size_t kBlocks = (kSorted + kBlock - 1) / kBlock;
  constexpr int64_t kUint4B8 = 1125899907892224;

  // One workspace for every operator, deliberately dirty.
  const size_t workspace_bytes = size_t{64} << 20;
  void* workspace = nullptr;
  Check(cudaMalloc(&workspace, workspace_bytes), "cudaMalloc workspace");
  Check(cudaMemset(workspace, 0xFF, workspace_bytes), "fill workspace");
  Handle handle;
  handle.set_stream(stream);
  handle.set_workspace(workspace);
  handle.set_workspace_size_in_bytes(workspace_bytes);
  const Config config;

  // ---- weight preparation: one expert matrix at a time through the static call ----------------------
  auto gptq13 = Buffer::FromFile("w13_gptq.bin", {kExperts, kHidden / 8, 2 * kInter}, DataType::kInt32);
  auto gptq2 = Buffer::FromFile("w2_gptq.bin", {kExperts, kInter / 8, kHidden}, DataType::kInt32);
  auto w13 = Buffer::Empty({kExperts, kHidden / 16, 2 * 2 * kInter}, DataType::kInt32, gptq13.device());
  auto w2 = Buffer::Empty({kExperts, kInter / 16, 2 * kHidden}, DataType::kInt32, gptq13.device());
  auto no_perm = Buffer::Empty({0}, DataType::kInt32, gptq13.device());
  for (size_t e = 0; e < kExperts; ++e) {
    auto slice = [&](const Buffer& b, size_t rows, size_t cols) {
      return Tensor{static_cast<char*>(b.data()) + e * rows * cols * 4, Tensor::Shape{rows, cols}, DataType::kInt32, b.device()};
    };
    GptqMarlinRepack::Call(handle, config, slice(gptq13, kHidden / 8, 2 * kInter), no_perm.view(),
                           static_cast<int64_t>(kHidden), static_cast<int64_t>(2 * kInter), int64_t{4}, false,
                           slice(w13, kHidden / 16, 4 * kInter));
    GptqMarlinRepack::Call(handle, config, slice(gptq2, kInter / 8, kHidden), no_perm.view(), static_cast<int64_t>(kInter),
                           static_cast<int64_t>(kHidden), int64_t{4}, false, slice(w2, kInter / 16, 2 * kHidden));
  }
  w13.ToFile("w13_marlin.bin");

  // ---- routing: explicit descriptor, called through the handle ----------------------------------------
  auto ids = Buffer::FromFile("topk_ids.bin", {kTokens, kTopK}, DataType::kInt32);
  auto sorted = Buffer::Empty({kSorted}, DataType::kInt32, ids.device());
  auto expert_ids = Buffer::Empty({kBlocks}, DataType::kInt32, ids.device());
  auto npost = Buffer::Empty({1}, DataType::kInt32, ids.device());
  auto align = MoeAlignBlockSize::Make(ids.view(), std::nullopt, static_cast<int64_t>(kExperts),
                                       static_cast<int64_t>(kBlock), sorted.view(), expert_ids.view(), npost.view());
  (*align)(handle, ids.view(), std::optional<Tensor>{}, static_cast<int64_t>(kExperts), static_cast<int64_t>(kBlock),
           sorted.view(), expert_ids.view(), npost.view());
  sorted.ToFile("sorted.bin");

  // ---- expert GEMMs on the same (now partly overwritten) workspace ---------------------------------------
  auto x = Buffer::FromFile("x.bin", {kTokens, kHidden}, DataType::kBFloat16);
  auto s13 = Buffer::FromFile("s13.bin", {kExperts, kHidden / 128, 2 * kInter}, DataType::kBFloat16);
  auto s2 = Buffer::FromFile("s2.bin", {kExperts, kInter / 128, kHidden}, DataType::kBFloat16);
  auto tw = Buffer::FromFile("topk_weights.bin", {kRoutes}, DataType::kFloat32);
  auto locks = Buffer::Empty({432}, DataType::kInt32, x.device());
  Check(cudaMemset(locks.data(), 0, locks.bytes()), "clear locks");
  auto g = Buffer::Empty({kRoutes, 2 * kInter}, DataType::kBFloat16, x.device());
  MoeWna16MarlinGemm::Call(handle, config, x.view(), w13.view(), std::optional<Tensor>{}, s13.view(), std::optional<Tensor>{},
                           std::optional<Tensor>{}, std::optional<Tensor>{}, std::optional<Tensor>{}, std::optional<Tensor>{},
                           locks.view(), sorted.view(), expert_ids.view(), npost.view(), tw.view(),
                           static_cast<int64_t>(kBlock), static_cast<int64_t>(kTopK), false, kUint4B8,
                           static_cast<int64_t>(kTokens), static_cast<int64_t>(2 * kInter), static_cast<int64_t>(kHidden), true,
                           false, true, false, int64_t{-1}, int64_t{-1}, int64_t{-1}, g.view());
  g.ToFile("g.bin");

  // `MakeReturnValue` with the application's own tensor type, then the activation
  auto h = SiluAndMul::MakeReturnValue(g);
  SiluAndMul::Call(handle, config, g.view(), h.view());
  h.ToFile("h.bin");

  auto y = Buffer::Empty({kRoutes, kHidden}, DataType::kBFloat16, x.device());
  MoeWna16MarlinGemm::Call(handle, config, h.view(), w2.view(), std::optional<Tensor>{}, s2.view(), std::optional<Tensor>{},
                           std::optional<Tensor>{}, std::optional<Tensor>{}, std::optional<Tensor>{}, std::optional<Tensor>{},
                           locks.view(), sorted.view(), expert_ids.view(), npost.view(), tw.view(),
                           static_cast<int64_t>(kBlock), int64_t{1}, true, kUint4B8, static_cast<int64_t>(kRoutes),
                           static_cast<int64_t>(kHidden), static_cast<int64_t>(kInter), true, false, true, false, int64_t{-1},
                           int64_t{-1}, int64_t{-1}, y.view());
  y.ToFile("y.bin");

  auto out = Buffer::Empty({kTokens, kHidden}, DataType::kBFloat16, x.device());
  auto sum = MoeSum::Make(y.view({kTokens, kTopK, kHidden}), out.view());
  (*sum)(handle, y.view({kTokens, kTopK, kHidden}), out.view());
  out.ToFile("out.bin");

  // ---- a dense problem whose single column tile is split over many blocks along K --------------------------
  constexpr size_t kM = 16, kK = 8192, kN = 128;
  auto a = Buffer::FromFile("dense_a.bin", {kM, kK}, DataType::kFloat16);
  auto dw = Buffer::FromFile("dense_w.bin", {kK / 16, 2 * kN}, DataType::kInt32);
  auto ds = Buffer::FromFile("dense_s.bin", {kK / 128, kN}, DataType::kFloat16);
  auto dout = Buffer::Empty({kM, kN}, DataType::kFloat16, a.device());
  Check(cudaMemsetAsync(workspace, 0xFF, workspace_bytes, stream), "dirty the workspace again");
  MarlinGemm::Call(handle, config, a.view(), dw.view(), std::optional<Tensor>{}, ds.view(), std::optional<Tensor>{},
                   std::optional<Tensor>{}, std::optional<Tensor>{}, std::optional<Tensor>{}, std::optional<Tensor>{},
                   locks.view(), kUint4B8, static_cast<int64_t>(kM), static_cast<int64_t>(kN), static_cast<int64_t>(kK), true,
                   false, true, false, dout.view());
  dout.ToFile("dense_out.bin");

  Check(cudaStreamSynchronize(stream), "synchronize");
  std::printf("active slots: %zu\n", GptqMarlinRepack::active_implementation_indices(Device::Type::kNvidia).size());
  return 0;
}
