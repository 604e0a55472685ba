// Device checks of the fusilli:: C++ front end on a B200: the paths the reference's samples do
// not reach through the graph API of this backend — SDPA as a graph node, bf16 shapes that go to
// the tcgen05 kernels, artifact round trips into a second Graph, imported device buffers, a
// workspace-requiring plan, and the execute() guards. Expected values are computed here on the
// host in double precision from the same inputs.
#include <fusilli.h>

#include "utils.h"

#include <catch2/catch_test_macros.hpp>

#include <atomic>
#include <barrier>
#include <cmath>
#include <cstdint>
#include <memory>
#include <mutex>
#include <random>
#include <thread>
#include <vector>

using namespace fusilli;

namespace {

std::vector<bf16> randomBf16(size_t n, uint32_t seed, float scale) {
  std::mt19937 rng(seed);
  std::uniform_real_distribution<float> d(-scale, scale);
  std::vector<bf16> v(n);
  for (auto &x : v) x = bf16(d(rng));
  return v;
}

std::shared_ptr<Buffer> share(Buffer &&b) { return std::make_shared<Buffer>(std::move(b)); }

} // namespace

TEST_CASE("bf16 batched matmul with bias runs the tensor-core plan and matches a host sum", "[matmul]") {
  const int64_t b = 2, m = 256, k = 192, n = 384;
  FUSILLI_REQUIRE_ASSIGN(Handle handle, Handle::create(kDefaultBackend));
  Graph g;
  g.setName("cpp_matmul_bias").setIODataType(DataType::BFloat16).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto aT = g.tensor(TensorAttr().setName("a").setDim({b, m, k}).setStride({m * k, k, 1}));
  auto bT = g.tensor(TensorAttr().setName("b").setDim({b, k, n}).setStride({k * n, n, 1}));
  auto biasT = g.tensor(TensorAttr().setName("bias").setDim({1, 1, n}).setStride({n, n, 1}));
  MatmulAttr mm;
  mm.setName("mm");
  auto cT = g.matmul(aT, bT, mm);
  PointwiseAttr add;
  add.setName("add").setMode(PointwiseAttr::Mode::ADD);
  auto yT = g.pointwise(cT, biasT, add);
  yT->setOutput(true);
  FUSILLI_REQUIRE_OK(g.validate());
  FUSILLI_REQUIRE_OK(g.compile(handle, /*remove=*/true));
  FUSILLI_REQUIRE_ASSIGN(auto stats, g.readCompilationCacheFile(CachedAssetsType::Statistics));
  REQUIRE(stats.find("gemm_tcgen05") != std::string::npos);

  auto a = randomBf16(b * m * k, 1, 1.f), bb = randomBf16(b * k * n, 2, 1.f), bias = randomBf16(n, 3, 1.f);
  FUSILLI_REQUIRE_ASSIGN(auto aBuf, allocateBufferOfType(handle, aT, a));
  FUSILLI_REQUIRE_ASSIGN(auto bBuf, allocateBufferOfType(handle, bT, bb));
  FUSILLI_REQUIRE_ASSIGN(auto biasBuf, allocateBufferOfType(handle, biasT, bias));
  FUSILLI_REQUIRE_ASSIGN(auto yBuf, allocateBufferOfType(handle, yT, DataType::BFloat16, 0.0));
  FUSILLI_REQUIRE_ASSIGN(auto ws, g.getWorkspaceSize());
  FUSILLI_REQUIRE_ASSIGN(auto wsBuf, allocateWorkspace(handle, ws));
  Graph::VariantPack pack = {{aT, aBuf}, {bT, bBuf}, {biasT, biasBuf}, {yT, yBuf}};
  FUSILLI_REQUIRE_OK(g.execute(handle, pack, wsBuf));
  std::vector<bf16> y;
  FUSILLI_REQUIRE_OK(yBuf->read(handle, y));
  double worst = 0;
  for (int64_t bi = 0; bi < b; ++bi)
    for (int64_t i = 0; i < m; i += 7)
      for (int64_t j = 0; j < n; j += 5) {
        double acc = float(bias[j]);
        for (int64_t kk = 0; kk < k; ++kk) acc += double(float(a[(bi * m + i) * k + kk])) * double(float(bb[(bi * k + kk) * n + j]));
        const double got = float(y[(bi * m + i) * n + j]);
        worst = std::max(worst, std::abs(got - acc) / (1.0 + std::abs(acc)));
      }
  INFO("worst relative error " << worst);
  REQUIRE(worst < 1.0 / 128); // one bf16 rounding of the result
}

TEST_CASE("SDPA graph node: causal attention matches a host softmax", "[sdpa]") {
  const int64_t b = 1, h = 2, s = 256, d = 128;
  FUSILLI_REQUIRE_ASSIGN(Handle handle, Handle::create(kDefaultBackend));
  Graph g;
  g.setName("cpp_sdpa_causal").setIODataType(DataType::BFloat16).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto mk = [&](const char *name) {
    return g.tensor(TensorAttr().setName(name).setDim({b, h, s, d}).setStride({h * s * d, s * d, d, 1}));
  };
  auto qT = mk("q"), kT = mk("k"), vT = mk("v");
  SdpaAttr attr;
  attr.setName("attn").setIsCausal(true);
  auto oT = g.sdpa(qT, kT, vT, nullptr, attr);
  oT->setOutput(true);
  FUSILLI_REQUIRE_OK(g.validate());
  FUSILLI_REQUIRE_OK(g.compile(handle, /*remove=*/true));
  auto q = randomBf16(b * h * s * d, 11, 1.f), k = randomBf16(b * h * s * d, 12, 1.f), v = randomBf16(b * h * s * d, 13, 1.f);
  FUSILLI_REQUIRE_ASSIGN(auto qBuf, allocateBufferOfType(handle, qT, q));
  FUSILLI_REQUIRE_ASSIGN(auto kBuf, allocateBufferOfType(handle, kT, k));
  FUSILLI_REQUIRE_ASSIGN(auto vBuf, allocateBufferOfType(handle, vT, v));
  FUSILLI_REQUIRE_ASSIGN(auto oBuf, allocateBufferOfType(handle, oT, DataType::BFloat16, 0.0));
  FUSILLI_REQUIRE_ASSIGN(auto ws, g.getWorkspaceSize());
  FUSILLI_REQUIRE_ASSIGN(auto wsBuf, allocateWorkspace(handle, ws));
  Graph::VariantPack pack = {{qT, qBuf}, {kT, kBuf}, {vT, vBuf}, {oT, oBuf}};
  FUSILLI_REQUIRE_OK(g.execute(handle, pack, wsBuf));
  std::vector<bf16> o;
  FUSILLI_REQUIRE_OK(oBuf->read(handle, o));
  const double scale = 1.0 / std::sqrt(double(d));
  double worst = 0;
  for (int64_t hh = 0; hh < h; ++hh)
    for (int64_t i = 0; i < s; i += 17) {
      std::vector<double> p(i + 1);
      double mx = -1e300, sum = 0;
      for (int64_t j = 0; j <= i; ++j) {
        double acc = 0;
        for (int64_t t = 0; t < d; ++t) acc += double(float(q[(hh * s + i) * d + t])) * double(float(k[(hh * s + j) * d + t]));
        p[j] = acc * scale;
        mx = std::max(mx, p[j]);
      }
      for (auto &x : p) { x = std::exp(x - mx); sum += x; }
      for (int64_t t = 0; t < d; t += 9) {
        double acc = 0;
        for (int64_t j = 0; j <= i; ++j) acc += p[j] * double(float(v[(hh * s + j) * d + t]));
        acc /= sum;
        worst = std::max(worst, std::abs(double(float(o[(hh * s + i) * d + t])) - acc));
      }
    }
  INFO("worst absolute error " << worst);
  REQUIRE(worst < 2e-2);
}

TEST_CASE("artifact built without a device loads into a second graph and an imported buffer", "[artifact]") {
  const int64_t n = 4, c = 32, hw = 16, kk = 64;
  auto build = [&](Graph &g) {
    g.setName("cpp_conv_artifact").setIODataType(DataType::BFloat16).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
    auto x = g.tensor(TensorAttr().setName("x").setDim({n, c, hw, hw}).setStride({c * hw * hw, 1, c * hw, c}));
    auto w = g.tensor(TensorAttr().setName("w").setDim({kk, c, 3, 3}).setStride({c * 9, 1, c * 3, c}));
    ConvFPropAttr conv;
    conv.setName("conv").setPadding({1, 1}).setStride({1, 1}).setDilation({1, 1});
    auto y = g.convFProp(x, w, conv);
    PointwiseAttr relu;
    relu.setName("relu").setMode(PointwiseAttr::Mode::RELU_FWD);
    auto z = g.pointwise(y, relu);
    z->setOutput(true);
    return std::make_tuple(x, w, z);
  };
  Graph offline;
  build(offline);
  FUSILLI_REQUIRE_OK(offline.validate());
  FUSILLI_REQUIRE_ASSIGN(auto bytes, offline.compileToArtifact(Backend::CUDA, /*remove=*/true));

  FUSILLI_REQUIRE_ASSIGN(Handle handle, Handle::create(kDefaultBackend));
  Graph online;
  auto [xT, wT, zT] = build(online);
  auto notValidated = online.loadFromArtifact(handle, bytes);
  REQUIRE(notValidated.getCode() == ErrorCode::NotValidated);
  FUSILLI_REQUIRE_OK(online.validate());
  FUSILLI_REQUIRE_OK(online.loadFromArtifact(handle, bytes));

  // all-ones input and filter: interior outputs are 9*c, corners 4*c
  FUSILLI_REQUIRE_ASSIGN(auto xBuf, allocateBufferOfType(handle, xT, DataType::BFloat16, 1.0));
  FUSILLI_REQUIRE_ASSIGN(auto wBuf, allocateBufferOfType(handle, wT, DataType::BFloat16, 1.0));
  FUSILLI_REQUIRE_ASSIGN(auto owned, Buffer::allocateRaw(handle, size_t(n * kk * hw * hw) * sizeof(bf16)));
  // the output goes through an import of the raw device pointer, as an integration would do
  FUSILLI_REQUIRE_ASSIGN(auto imported, Buffer::import(handle, owned.devicePointer(), owned.sizeInBytes()));
  auto zBuf = share(std::move(imported));
  Graph::VariantPack pack = {{xT, xBuf}, {wT, wBuf}, {zT, zBuf}};

  // execute() before getWorkspaceSize() is refused, as in the reference
  auto early = online.execute(handle, pack, nullptr);
  REQUIRE(early.getCode() == ErrorCode::InvalidArgument);
  FUSILLI_REQUIRE_ASSIGN(auto ws, online.getWorkspaceSize());
  FUSILLI_REQUIRE_ASSIGN(auto wsBuf, allocateWorkspace(handle, ws));
  FUSILLI_REQUIRE_OK(online.execute(handle, pack, wsBuf));
  std::vector<bf16> z;
  FUSILLI_REQUIRE_OK(owned.read(handle, z));
  REQUIRE(z.size() == size_t(n * kk * hw * hw));
  auto at = [&](int64_t ni, int64_t ki, int64_t y, int64_t x) { return float(z[((ni * hw + y) * hw + x) * kk + ki]); };
  REQUIRE(at(0, 0, 0, 0) == 4.f * c);
  REQUIRE(at(1, 5, 0, 7) == 6.f * c);
  REQUIRE(at(3, 63, 8, 8) == 9.f * c);
  REQUIRE(at(2, 17, 15, 15) == 4.f * c);

  // a missing tensor in the variant pack is an error, not a crash
  Graph::VariantPack partial = {{xT, xBuf}, {zT, zBuf}};
  auto missing = online.execute(handle, partial, wsBuf);
  REQUIRE(missing.getCode() == ErrorCode::VariantPackError);
}

TEST_CASE("conv wgrad plan asks for a workspace and refuses to run without it", "[wgrad]") {
  const int64_t n = 8, c = 64, hw = 16, kk = 64;
  FUSILLI_REQUIRE_ASSIGN(Handle handle, Handle::create(kDefaultBackend));
  Graph g;
  g.setName("cpp_wgrad_workspace").setIODataType(DataType::BFloat16).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto dyT = g.tensor(TensorAttr().setName("dy").setDim({n, kk, hw, hw}).setStride({kk * hw * hw, 1, kk * hw, kk}));
  auto xT = g.tensor(TensorAttr().setName("x").setDim({n, c, hw, hw}).setStride({c * hw * hw, 1, c * hw, c}));
  ConvWGradAttr attr;
  attr.setName("wgrad").setPadding({1, 1}).setStride({1, 1}).setDilation({1, 1});
  auto dwT = g.convWGrad(dyT, xT, attr);
  dwT->setOutput(true).setDim({kk, c, 3, 3}).setStride({c * 9, 1, c * 3, c});
  FUSILLI_REQUIRE_OK(g.validate());
  FUSILLI_REQUIRE_OK(g.compile(handle, /*remove=*/true));
  FUSILLI_REQUIRE_ASSIGN(auto ws, g.getWorkspaceSize());
  REQUIRE(ws.has_value());
  FUSILLI_REQUIRE_ASSIGN(auto dyBuf, allocateBufferOfType(handle, dyT, DataType::BFloat16, 1.0));
  FUSILLI_REQUIRE_ASSIGN(auto xBuf, allocateBufferOfType(handle, xT, DataType::BFloat16, 1.0));
  FUSILLI_REQUIRE_ASSIGN(auto dwBuf, allocateBufferOfType(handle, dwT, DataType::BFloat16, 0.0));
  Graph::VariantPack pack = {{dyT, dyBuf}, {xT, xBuf}, {dwT, dwBuf}};
  if (*ws > 0) {
    auto refused = g.execute(handle, pack, nullptr);
    REQUIRE(refused.getCode() == ErrorCode::InvalidArgument);
  }
  FUSILLI_REQUIRE_ASSIGN(auto wsBuf, allocateWorkspace(handle, ws));
  FUSILLI_REQUIRE_OK(g.execute(handle, pack, wsBuf));
  std::vector<bf16> dw;
  FUSILLI_REQUIRE_OK(dwBuf->read(handle, dw));
  // all-ones dy and x: the centre tap sums every pixel of every image, a corner tap (hw-1)^2
  auto at = [&](int64_t ki, int64_t ci, int64_t r, int64_t s) { return float(dw[((ki * 3 + r) * 3 + s) * c + ci]); };
  REQUIRE(at(0, 0, 1, 1) == float(n * hw * hw));
  REQUIRE(at(63, 63, 0, 0) == float(n * (hw - 1) * (hw - 1)));
  REQUIRE(at(5, 9, 1, 0) == float(n * hw * (hw - 1)));
}

TEST_CASE("Comm: the fp32 weight-gradient partial lands in the exchange buffer and is summed and rounded there", "[comm]") {
  // One rank (world = 1) exercises the whole C++ path of a sharded run: the graph declares its dW as fp32
  // and binds it INTO the communicator's buffer, the fused sum rounds it once to bf16 in the same buffer.
  const int64_t n = 8, c = 64, hw = 16, kk = 64;
  const size_t elems = kk * c * 9;
  FUSILLI_REQUIRE_ASSIGN(Handle handle, Handle::create(kDefaultBackend));
  FUSILLI_REQUIRE_ASSIGN(Comm comm, Comm::create(handle, /*rank=*/0, /*world=*/1, elems * 4 + elems * 2));
  REQUIRE(comm.rank() == 0);
  REQUIRE(comm.world() == 1);
  REQUIRE(comm.bufferBytes() >= elems * 6);
  Graph g;
  g.setName("cpp_wgrad_comm").setIODataType(DataType::BFloat16).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto dyT = g.tensor(TensorAttr().setName("dy").setDim({n, kk, hw, hw}).setStride({kk * hw * hw, 1, kk * hw, kk}));
  auto xT = g.tensor(TensorAttr().setName("x").setDim({n, c, hw, hw}).setStride({c * hw * hw, 1, c * hw, c}));
  ConvWGradAttr attr;
  attr.setName("wgrad").setPadding({1, 1}).setStride({1, 1}).setDilation({1, 1});
  auto dwT = g.convWGrad(dyT, xT, attr);
  dwT->setOutput(true).setDataType(DataType::Float).setDim({kk, c, 3, 3}).setStride({c * 9, 1, c * 3, c});
  FUSILLI_REQUIRE_OK(g.validate());
  FUSILLI_REQUIRE_OK(g.compile(handle, /*remove=*/true));
  FUSILLI_REQUIRE_ASSIGN(auto ws, g.getWorkspaceSize());
  FUSILLI_REQUIRE_ASSIGN(auto dyBuf, allocateBufferOfType(handle, dyT, DataType::BFloat16, 1.0));
  FUSILLI_REQUIRE_ASSIGN(auto xBuf, allocateBufferOfType(handle, xT, DataType::BFloat16, 1.0));
  FUSILLI_REQUIRE_ASSIGN(auto dwView, comm.view(0, elems * 4));
  Graph::VariantPack pack = {{dyT, dyBuf}, {xT, xBuf}, {dwT, dwView}};
  FUSILLI_REQUIRE_ASSIGN(auto wsBuf, allocateWorkspace(handle, ws));
  FUSILLI_REQUIRE_OK(g.execute(handle, pack, wsBuf));
  FUSILLI_REQUIRE_OK(comm.sumFused(0, elems, elems * 4, DataType::BFloat16));
  FUSILLI_REQUIRE_ASSIGN(auto outView, comm.view(elems * 4, elems * 2));
  std::vector<bf16> dw;
  FUSILLI_REQUIRE_OK(outView->read(handle, dw));
  REQUIRE(dw.size() == elems);
  auto at = [&](int64_t ki, int64_t ci, int64_t r, int64_t s) { return float(dw[((ki * 3 + r) * 3 + s) * c + ci]); };
  REQUIRE(at(0, 0, 1, 1) == float(n * hw * hw));
  REQUIRE(at(63, 63, 0, 0) == float(n * (hw - 1) * (hw - 1)));
  // ranges that overlap or leave the buffer are refused before anything is launched
  REQUIRE(comm.sumFused(0, elems, elems * 2, DataType::BFloat16).getCode() == ErrorCode::InvalidArgument);
  REQUIRE(isError(comm.view(elems * 6, 4096)));
}

TEST_CASE("one plan with a dynamic batch serves channels-last buffers of several batch sizes", "[dynamic]") {
  const int64_t n = 8, c = 64, hw = 16, kk = 64;
  FUSILLI_REQUIRE_ASSIGN(Handle handle, Handle::create(kDefaultBackend));
  Graph g;
  g.setName("cpp_dynamic_conv").setIODataType(DataType::BFloat16).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto xT = g.tensor(TensorAttr().setName("x").setDim({n, c, hw, hw}).setStride({c * hw * hw, 1, c * hw, c}).setDynamicDims({0}));
  auto wT = g.tensor(TensorAttr().setName("w").setDim({kk, c, 3, 3}).setStride({c * 9, 1, c * 3, c}));
  ConvFPropAttr conv;
  conv.setName("conv").setPadding({1, 1}).setStride({1, 1}).setDilation({1, 1});
  auto yT = g.convFProp(xT, wT, conv);
  yT->setDynamicDims({0});
  PointwiseAttr relu;
  relu.setName("relu").setMode(PointwiseAttr::Mode::RELU_FWD);
  auto zT = g.pointwise(yT, relu);
  zT->setDynamicDims({0}).setOutput(true);
  FUSILLI_REQUIRE_OK(g.validate());
  FUSILLI_REQUIRE_OK(g.compile(handle, /*remove=*/true));
  FUSILLI_REQUIRE_ASSIGN(auto text, g.readCompilationCacheFile(CachedAssetsType::Input));
  REQUIRE(text.find("dynamic=1") != std::string::npos);
  FUSILLI_REQUIRE_ASSIGN(auto ws, g.getWorkspaceSize());
  FUSILLI_REQUIRE_ASSIGN(auto wsBuf, allocateWorkspace(handle, ws));
  FUSILLI_REQUIRE_ASSIGN(auto wBuf, allocateBufferOfType(handle, wT, DataType::BFloat16, 1.0));

  for (int64_t rn : {int64_t(1), int64_t(3), n, int64_t(3)}) {
    // buffer shapes are in physical (NHWC) order, as the reference's helpers allocate them
    const std::vector<size_t> xShape = {size_t(rn), size_t(hw), size_t(hw), size_t(c)};
    const std::vector<size_t> zShape = {size_t(rn), size_t(hw), size_t(hw), size_t(kk)};
    FUSILLI_REQUIRE_ASSIGN(auto xRaw, Buffer::allocate(handle, xShape, std::vector<bf16>(rn * c * hw * hw, bf16(1.0f))));
    FUSILLI_REQUIRE_ASSIGN(auto zRaw, Buffer::allocate(handle, zShape, std::vector<bf16>(rn * kk * hw * hw, bf16(-1.0f))));
    auto xBuf = share(std::move(xRaw)), zBuf = share(std::move(zRaw));
    Graph::VariantPack pack = {{xT, xBuf}, {wT, wBuf}, {zT, zBuf}};
    FUSILLI_REQUIRE_OK(g.execute(handle, pack, wsBuf));
    std::vector<bf16> z;
    FUSILLI_REQUIRE_OK(zBuf->read(handle, z));
    REQUIRE(z.size() == size_t(rn * kk * hw * hw));
    auto at = [&](int64_t ni, int64_t ki, int64_t y, int64_t x) { return float(z[((ni * hw + y) * hw + x) * kk + ki]); };
    REQUIRE(at(0, 0, 0, 0) == 4.f * c);
    REQUIRE(at(rn - 1, 63, 8, 8) == 9.f * c);
    REQUIRE(at(rn - 1, 17, 15, 15) == 4.f * c);
    REQUIRE(at(rn / 2, 5, 0, 7) == 6.f * c);
  }

  // an imported pointer with its shape works; without a shape a single dynamic dim follows from the size
  const int64_t rn = 2;
  FUSILLI_REQUIRE_ASSIGN(auto xOwned, Buffer::allocate(handle, {size_t(rn * c * hw * hw)}, std::vector<bf16>(rn * c * hw * hw, bf16(1.0f))));
  FUSILLI_REQUIRE_ASSIGN(auto zOwned, Buffer::allocateRaw(handle, size_t(rn * kk * hw * hw) * sizeof(bf16)));
  FUSILLI_REQUIRE_ASSIGN(auto xImp, Buffer::import(handle, xOwned.devicePointer(), xOwned.sizeInBytes(),
                                                   {size_t(rn), size_t(hw), size_t(hw), size_t(c)}));
  FUSILLI_REQUIRE_ASSIGN(auto zImp, Buffer::import(handle, zOwned.devicePointer(), zOwned.sizeInBytes()));
  Graph::VariantPack pack = {{xT, share(std::move(xImp))}, {wT, wBuf}, {zT, share(std::move(zImp))}};
  FUSILLI_REQUIRE_OK(g.execute(handle, pack, wsBuf));
  std::vector<bf16> z;
  FUSILLI_REQUIRE_OK(zOwned.read(handle, z));
  REQUIRE(float(z[((1 * hw + 8) * hw + 8) * kk + 9]) == 9.f * c);

  // an output buffer whose batch is not the input's is refused before anything is launched
  FUSILLI_REQUIRE_ASSIGN(auto wrong, Buffer::allocate(handle, {size_t(3), size_t(hw), size_t(hw), size_t(kk)},
                                                      std::vector<bf16>(3 * kk * hw * hw, bf16(0.0f))));
  pack[zT] = share(std::move(wrong));
  auto st = g.execute(handle, pack, wsBuf);
  REQUIRE(st.getCode() == ErrorCode::InvalidArgument);
  REQUIRE(st.getMessage().find("imply") != std::string::npos);
}

TEST_CASE("32 threads create handles at once; deviceId / stream on the CPU backend is an InvalidArgument", "[handle]") {
  // the reference's tests/test_handle.cpp:47-85, on the one backend that exists here
  constexpr int kNumThreads = 32;
  std::vector<std::thread> threads;
  std::vector<Handle> handles;
  handles.reserve(kNumThreads);
  std::barrier startBarrier(kNumThreads);
  std::atomic<bool> creationFailed{false};
  std::mutex handlesMutex;
  for (int i = 0; i < kNumThreads; ++i) {
    threads.emplace_back([&]() {
      startBarrier.arrive_and_wait();
      auto h = Handle::create(kDefaultBackend);
      if (isError(h)) {
        creationFailed.store(true);
        return;
      }
      std::lock_guard<std::mutex> lock(handlesMutex);
      handles.push_back(std::move(*h));
    });
  }
  for (auto &t : threads) t.join();
  REQUIRE(!creationFailed.load());
  REQUIRE(handles.size() == size_t(kNumThreads));
  auto withStream = Handle::create(Backend::CPU, /*deviceId=*/0, /*stream=*/0);
  REQUIRE(isError(withStream));
  REQUIRE(ErrorObject(withStream).getCode() == ErrorCode::InvalidArgument);
  auto withDevice = Handle::create(Backend::CPU, /*deviceId=*/0);
  REQUIRE(isError(withDevice));
  REQUIRE(ErrorObject(withDevice).getCode() == ErrorCode::InvalidArgument);
}
