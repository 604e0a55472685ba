// Host-only checks of the fusilli:: C++ front end of the B200 backend: graph building, name
// inference, validation errors, plan building without a device, cache files, and the error
// surface of Handle/Buffer when no CUDA device is usable. Nothing here launches a kernel.
//
// The behaviours checked are the reference's (include/fusilli/graph/graph.h:80-113 validate,
// :756-1193 builders; include/fusilli/backend/runtime.h:242-529 compile/execute guards).
#include <fusilli.h>

#include "utils.h"

#include <catch2/catch_test_macros.hpp>

#include <cstdlib>
#include <filesystem>
#include <fstream>
#include <string>

using namespace fusilli;

namespace {
TensorAttr nhwc(const std::string &name, int64_t n, int64_t c, int64_t h, int64_t w) {
  return TensorAttr().setName(name).setDim({n, c, h, w}).setStride({c * h * w, 1, c * w, c});
}
} // namespace

TEST_CASE("graph needs a name to validate", "[graph]") {
  Graph g;
  g.setIODataType(DataType::Float).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto st = g.validate();
  REQUIRE(isError(st));
  REQUIRE(st.getCode() == ErrorCode::AttributeNotSet);
  REQUIRE(st.getMessage() == "Graph name not set");
}

TEST_CASE("builders name nodes and outputs, outputs are virtual until marked", "[graph]") {
  Graph g;
  g.setName("naming").setIODataType(DataType::BFloat16).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto x = g.tensor(nhwc("", 2, 16, 8, 8));
  auto w = g.tensor(nhwc("", 32, 16, 3, 3));
  ConvFPropAttr conv;
  conv.setPadding({1, 1}).setStride({1, 1}).setDilation({1, 1});
  auto y = g.convFProp(x, w, conv);
  REQUIRE(y->isVirtual());
  REQUIRE(y->getName() == "conv_fprop_0_Y");
  REQUIRE(x->getName() == "conv_fprop_0_X");
  REQUIRE(w->getName() == "conv_fprop_0_W");
  PointwiseAttr relu;
  relu.setMode(PointwiseAttr::Mode::RELU_FWD);
  auto z = g.pointwise(y, relu);
  REQUIRE(z->getName() == "pointwise_1_OUT_0");
  z->setOutput(true);
  REQUIRE(!z->isVirtual());
  FUSILLI_REQUIRE_OK(g.validate());
  REQUIRE(y->getDim() == std::vector<int64_t>{2, 32, 8, 8});
  REQUIRE(z->getDim() == std::vector<int64_t>{2, 32, 8, 8});
  REQUIRE(z->getDataType() == DataType::BFloat16); // IO type on the graph boundary
  REQUIRE(y->getDataType() == DataType::Float);    // intermediate type on virtual tensors
  // channels-last input gives a channels-last inferred output
  REQUIRE(z->getStride() == std::vector<int64_t>{32 * 8 * 8, 1, 32 * 8, 32});
}

TEST_CASE("duplicate symbol names are rejected", "[graph]") {
  Graph g;
  g.setName("dups").setIODataType(DataType::Float).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto a = g.tensor(TensorAttr().setName("t").setDim({4, 8}).setStride({8, 1}));
  auto b = g.tensor(TensorAttr().setName("t").setDim({8, 4}).setStride({4, 1}));
  MatmulAttr mm;
  mm.setName("mm");
  g.matmul(a, b, mm)->setOutput(true);
  auto st = g.validate();
  REQUIRE(isError(st));
  REQUIRE(st.getCode() == ErrorCode::InvalidAttribute);
  REQUIRE(st.getMessage() == "Symbol name 't' already in use");
}

TEST_CASE("conv validation reports the reference's messages", "[conv]") {
  Graph g;
  g.setName("conv_errors").setIODataType(DataType::Float).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto x = g.tensor(nhwc("x", 2, 16, 8, 8));
  auto w = g.tensor(nhwc("w", 32, 16, 3, 3));
  SECTION("padding missing") {
    ConvFPropAttr conv;
    conv.setName("c").setStride({1, 1}).setDilation({1, 1});
    g.convFProp(x, w, conv)->setOutput(true);
    auto st = g.validate();
    REQUIRE(st.getCode() == ErrorCode::AttributeNotSet);
    REQUIRE(st.getMessage() == "Conv padding not set");
  }
  SECTION("channel mismatch") {
    auto w2 = g.tensor(nhwc("w2", 32, 5, 3, 3));
    ConvFPropAttr conv;
    conv.setName("c").setPadding({1, 1}).setStride({1, 1}).setDilation({1, 1});
    g.convFProp(x, w2, conv)->setOutput(true);
    auto st = g.validate();
    REQUIRE(isError(st));
    REQUIRE(st.getCode() == ErrorCode::InvalidAttribute);
  }
}

TEST_CASE("compile guards: not validated, wrong backend, not compiled", "[graph]") {
  Graph g;
  g.setName("guards").setIODataType(DataType::Float).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto a = g.tensor(TensorAttr().setName("a").setDim({4, 8}).setStride({8, 1}));
  auto b = g.tensor(TensorAttr().setName("b").setDim({8, 4}).setStride({4, 1}));
  MatmulAttr mm;
  mm.setName("mm");
  auto c = g.matmul(a, b, mm);
  c->setOutput(true);
  auto early = g.compileToArtifact(Backend::CUDA, /*remove=*/true);
  REQUIRE(isError(early));
  REQUIRE(ErrorObject(early).getCode() == ErrorCode::NotValidated);
  FUSILLI_REQUIRE_OK(g.validate());
  auto cpu = g.compileToArtifact(Backend::CPU, /*remove=*/true);
  REQUIRE(ErrorObject(cpu).getCode() == ErrorCode::NotImplemented);
  FUSILLI_REQUIRE_ASSIGN(auto ws, g.getWorkspaceSize());
  REQUIRE(!ws.has_value()); // nothing loaded yet
}

TEST_CASE("plans build without a device and land in the cache directory", "[graph][cache]") {
  const auto dir = std::filesystem::temp_directory_path() / "fusilli_b200_host_test_cache";
  std::filesystem::remove_all(dir);
  setenv("FUSILLI_CACHE_DIR", dir.c_str(), 1);
  {
    Graph g;
    g.setName("cache me").setIODataType(DataType::BFloat16).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
    auto a = g.tensor(TensorAttr().setName("a").setDim({2, 128, 64}).setStride({128 * 64, 64, 1}));
    auto b = g.tensor(TensorAttr().setName("b").setDim({2, 64, 256}).setStride({64 * 256, 256, 1}));
    auto bias = g.tensor(TensorAttr().setName("bias").setDim({1, 1, 256}).setStride({256, 256, 1}));
    MatmulAttr mm;
    mm.setName("mm");
    auto c = g.matmul(a, b, mm);
    PointwiseAttr add;
    add.setName("add").setMode(PointwiseAttr::Mode::ADD);
    auto y = g.pointwise(c, bias, add);
    y->setOutput(true);
    FUSILLI_REQUIRE_OK(g.validate());
    FUSILLI_REQUIRE_ASSIGN(auto bytes, g.compileToArtifact(Backend::CUDA, /*remove=*/true));
    REQUIRE(bytes.size() > 32);
    REQUIRE(std::string(bytes.begin(), bytes.begin() + 7) == "FB2PLAN");
    // the plan is checkable without a device and fuses the bias add into the contraction
    FUSILLI_REQUIRE_OK(fromStatus(fb_plan_check(bytes.data(), bytes.size())));
    const auto sub = dir / ".cache" / "fusilli" / "cache_me";
    REQUIRE(std::filesystem::exists(sub / FUSILLI_B200_OUTPUT_FILENAME));
    REQUIRE(std::filesystem::exists(sub / FUSILLI_B200_INPUT_FILENAME));
    FUSILLI_REQUIRE_ASSIGN(auto text, g.readCompilationCacheFile(CachedAssetsType::Input));
    REQUIRE(text.find("mm") != std::string::npos);
    // same graph again: served from the cache file, byte-identical
    FUSILLI_REQUIRE_ASSIGN(auto again, g.compileToArtifact(Backend::CUDA, /*remove=*/true));
    REQUIRE(again == bytes);
    // a corrupted artifact is refused
    auto bad = bytes;
    bad[bad.size() - 1] ^= 0x5a;
    REQUIRE(fb_plan_check(bad.data(), bad.size()) != FB_OK);
  }
  // remove=true cleans up after the graph goes away
  REQUIRE(!std::filesystem::exists(dir / ".cache" / "fusilli" / "cache_me" / FUSILLI_B200_OUTPUT_FILENAME));
  std::filesystem::remove_all(dir);
  unsetenv("FUSILLI_CACHE_DIR");
}

TEST_CASE("in-process compile cache: hit only for the same instance, name, plan input and command", "[graph][cache]") {
  // The rules of the reference's Graph::validateCache (include/fusilli/graph/graph.h:557-644). A hit is
  // made visible by tampering with the cached output file: a hit returns the tampered bytes, a miss a
  // freshly built plan.
  const auto dir = std::filesystem::temp_directory_path() / "fusilli_b200_host_test_cache_rules";
  std::filesystem::remove_all(dir);
  setenv("FUSILLI_CACHE_DIR", dir.c_str(), 1);
  auto build = [](Graph &g, const std::string &name, int64_t cols) {
    g.setName(name).setIODataType(DataType::Float).setComputeDataType(DataType::Float);
    auto a = g.tensor(TensorAttr().setName("a").setDim({4, cols}).setStride({cols, 1}));
    auto b = g.tensor(TensorAttr().setName("b").setDim({4, cols}).setStride({cols, 1}));
    PointwiseAttr add;
    add.setName("add").setMode(PointwiseAttr::Mode::ADD);
    auto y = g.pointwise(a, b, add);
    y->setName("y").setOutput(true);
    return y;
  };
  auto tamper = [&](const std::string &sub) {
    std::ofstream f(dir / ".cache" / "fusilli" / sub / FUSILLI_B200_OUTPUT_FILENAME, std::ios::binary | std::ios::trunc);
    f << "TAMPERED";
  };
  auto isTampered = [](const std::vector<uint8_t> &v) { return std::string(v.begin(), v.end()) == "TAMPERED"; };
  {
    Graph g;
    build(g, "rules_one", 8);
    FUSILLI_REQUIRE_OK(g.validate());
    // 1. nothing cached for this instance yet: miss, a real plan
    FUSILLI_REQUIRE_ASSIGN(auto first, g.compileToArtifact(Backend::CUDA, /*remove=*/false));
    REQUIRE(fb_plan_check(first.data(), first.size()) == FB_OK);
    // 2. same instance, same name, same plan input, same command: hit (the file's bytes come back)
    tamper("rules_one");
    FUSILLI_REQUIRE_ASSIGN(auto second, g.compileToArtifact(Backend::CUDA, /*remove=*/false));
    REQUIRE(isTampered(second));
    // 3. the name (and therefore every cache path) changed: miss, built again under the new name
    g.setName("rules_two");
    FUSILLI_REQUIRE_ASSIGN(auto third, g.compileToArtifact(Backend::CUDA, /*remove=*/false));
    REQUIRE(fb_plan_check(third.data(), third.size()) == FB_OK);
    REQUIRE(std::filesystem::exists(dir / ".cache" / "fusilli" / "rules_two" / FUSILLI_B200_OUTPUT_FILENAME));
    // 4. the command on file differs from the one this build would run: miss
    tamper("rules_two");
    {
      std::ofstream f(dir / ".cache" / "fusilli" / "rules_two" / FUSILLI_B200_COMMAND_FILENAME, std::ios::trunc);
      f << "some other compiler --flags\n";
    }
    FUSILLI_REQUIRE_ASSIGN(auto fourth, g.compileToArtifact(Backend::CUDA, /*remove=*/false));
    REQUIRE(!isTampered(fourth));
    // 5. the plan input on file differs from the one generated now: miss
    tamper("rules_two");
    {
      std::ofstream f(dir / ".cache" / "fusilli" / "rules_two" / FUSILLI_B200_INPUT_FILENAME, std::ios::app);
      f << "tensor extra\n";
    }
    FUSILLI_REQUIRE_ASSIGN(auto fifth, g.compileToArtifact(Backend::CUDA, /*remove=*/false));
    REQUIRE(!isTampered(fifth));
    REQUIRE(fifth == third);
  }
  {
    // 6. another instance with the same name and the same graph does not inherit the cache
    tamper("rules_two");
    Graph other;
    build(other, "rules_two", 8);
    FUSILLI_REQUIRE_OK(other.validate());
    FUSILLI_REQUIRE_ASSIGN(auto fresh, other.compileToArtifact(Backend::CUDA, /*remove=*/false));
    REQUIRE(!isTampered(fresh));
    // 7. same instance and name, different graph contents (the generated plan input differs): miss
    Graph wider;
    build(wider, "rules_three", 8);
    FUSILLI_REQUIRE_OK(wider.validate());
    FUSILLI_REQUIRE_ASSIGN(auto w1, wider.compileToArtifact(Backend::CUDA, /*remove=*/false));
    Graph wider2;
    build(wider2, "rules_three", 16);
    FUSILLI_REQUIRE_OK(wider2.validate());
    FUSILLI_REQUIRE_ASSIGN(auto w2, wider2.compileToArtifact(Backend::CUDA, /*remove=*/false));
    REQUIRE(w1 != w2);
  }
  std::filesystem::remove_all(dir);
  unsetenv("FUSILLI_CACHE_DIR");
}

TEST_CASE("execute before compile is NotCompiled; CPU and AMDGPU handles are NotImplemented", "[backend]") {
  auto cpu = Handle::create(Backend::CPU);
  REQUIRE(isError(cpu));
  REQUIRE(ErrorObject(cpu).getCode() == ErrorCode::NotImplemented);
  auto amd = Handle::create(Backend::AMDGPU);
  REQUIRE(isError(amd));
  REQUIRE(ErrorObject(amd).getCode() == ErrorCode::NotImplemented);
}

TEST_CASE("unsupported node kinds fail loudly at plan build, never fall back", "[graph]") {
  Graph g;
  g.setName("f64_matmul").setIODataType(DataType::Double).setComputeDataType(DataType::Double).setIntermediateDataType(DataType::Double);
  auto a = g.tensor(TensorAttr().setName("a").setDim({4, 8}).setStride({8, 1}));
  auto b = g.tensor(TensorAttr().setName("b").setDim({8, 4}).setStride({4, 1}));
  MatmulAttr mm;
  mm.setName("mm");
  g.matmul(a, b, mm)->setOutput(true);
  FUSILLI_REQUIRE_OK(g.validate());
  auto r = g.compileToArtifact(Backend::CUDA, /*remove=*/true);
  REQUIRE(isError(r));
}

TEST_CASE("graphs with dynamic dims build plans without a device", "[graph][dynamic]") {
  Graph g;
  g.setName("dynamic_rows").setIODataType(DataType::Float).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto a = g.tensor(TensorAttr().setName("a").setDim({64, 32}).setStride({32, 1}).setDynamicDims({0}));
  auto b = g.tensor(TensorAttr().setName("b").setDim({32, 16}).setStride({16, 1}));
  MatmulAttr mm;
  mm.setName("mm");
  auto c = g.matmul(a, b, mm);
  c->setDynamicDims({0}).setOutput(true);
  FUSILLI_REQUIRE_OK(g.validate());
  FUSILLI_REQUIRE_ASSIGN(auto bytes, g.compileToArtifact(Backend::CUDA, /*remove=*/true));
  FUSILLI_REQUIRE_OK(fromStatus(fb_plan_check(bytes.data(), bytes.size())));
  // specialising for 5 rows gives the plan of the graph declared with 5 rows
  // argument order: outputs by name, then inputs by name -> mm_C, a, b
  int64_t dims[3 * FB_MAX_RANK] = {};
  for (auto &d : dims) d = 1;
  dims[0] = 5, dims[1] = 16;
  dims[FB_MAX_RANK] = 5, dims[FB_MAX_RANK + 1] = 32;
  dims[2 * FB_MAX_RANK] = 32, dims[2 * FB_MAX_RANK + 1] = 16;
  uint8_t *out = nullptr;
  size_t n = 0;
  FUSILLI_REQUIRE_OK(fromStatus(fb_plan_specialize(bytes.data(), bytes.size(), dims, 3, &out, &n)));
  std::vector<uint8_t> shaped(out, out + n);
  fb_bytes_free(out);
  Graph five;
  five.setName("dynamic_rows").setIODataType(DataType::Float).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto a5 = five.tensor(TensorAttr().setName("a").setDim({5, 32}).setStride({32, 1}).setDynamicDims({0}));
  auto b5 = five.tensor(TensorAttr().setName("b").setDim({32, 16}).setStride({16, 1}));
  MatmulAttr mm5;
  mm5.setName("mm");
  auto c5 = five.matmul(a5, b5, mm5);
  c5->setDynamicDims({0}).setOutput(true);
  FUSILLI_REQUIRE_OK(five.validate());
  FUSILLI_REQUIRE_ASSIGN(auto direct, five.compileToArtifact(Backend::CUDA, /*remove=*/true));
  REQUIRE(shaped == direct);
  // a static dim that differs is refused
  dims[FB_MAX_RANK + 1] = 40;
  REQUIRE(fb_plan_specialize(bytes.data(), bytes.size(), dims, 3, &out, &n) == FB_INVALID_ARGUMENT);
}

TEST_CASE("custom ops are accepted by the builders and refused when the plan is built", "[custom_op]") {
  Graph g;
  g.setName("custom").setIODataType(DataType::Float).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
  auto a = g.tensor(TensorAttr().setDim({4, 8}).setStride({8, 1}));
  CustomOpAttr attr;
  attr.setMlir("func.func private @{FUNC_NAME}() { return }").setNumOutputs(2);
  auto outs = g.customOp({a}, attr);
  REQUIRE(outs.size() == 2);
  REQUIRE(a->getName() == "custom_op_0_IN_0");
  REQUIRE(outs[1]->getName() == "custom_op_0_OUT_1");
  REQUIRE(outs[0]->isVirtual());
  for (auto &o : outs) o->setDim({4, 8}).setStride({8, 1}).setDataType(DataType::Float).setOutput(true);
  FUSILLI_REQUIRE_OK(g.validate());
  auto r = g.compileToArtifact(Backend::CUDA, /*remove=*/true);
  REQUIRE(isError(r));
  REQUIRE(ErrorObject(r).getCode() == ErrorCode::NotImplemented);
  REQUIRE(ErrorObject(r).getMessage().find("custom_op_0") != std::string::npos);

  SECTION("missing MLIR") {
    Graph h;
    h.setName("custom_bad").setIODataType(DataType::Float).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
    auto x = h.tensor(TensorAttr().setName("x").setDim({4}).setStride({1}));
    CustomOpAttr bad;
    bad.setName("op").setNumOutputs(1);
    h.customOp({x}, bad)[0]->setDim({4}).setStride({1}).setOutput(true);
    auto st = h.validate();
    REQUIRE(st.getCode() == ErrorCode::AttributeNotSet);
    REQUIRE(st.getMessage() == "CustomOp MLIR not set");
  }
  SECTION("no outputs") {
    Graph h;
    h.setName("custom_bad").setIODataType(DataType::Float).setComputeDataType(DataType::Float).setIntermediateDataType(DataType::Float);
    auto x = h.tensor(TensorAttr().setName("x").setDim({4}).setStride({1}));
    CustomOpAttr bad;
    bad.setName("op").setMlir("x");
    h.customOp({x}, bad);
    auto st = h.validate();
    REQUIRE(st.getCode() == ErrorCode::AttributeNotSet);
    REQUIRE(st.getMessage() == "CustomOp outputs not set");
  }
}
