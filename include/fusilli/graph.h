// fusilli::Graph on the B200 backend: builders, validate(), compile(handle) /
// compileToArtifact(backend) / loadFromArtifact(handle, bytes), getWorkspaceSize(),
// execute(handle, variantPack, workspace), readCompilationCacheFile().
//
// Same surface, guards and messages as the reference's include/fusilli/graph/graph.h:75-468 and
// include/fusilli/backend/runtime.h:242-529. Where the reference emits MLIR and runs the IREE
// compiler, compileToArtifact() flattens the validated graph into the C ABI's fb_graph_desc and
// calls fb_plan_build (no device needed); loadFromArtifact() calls fb_plan_load; execute() is one
// fb_plan_execute, asynchronous on the handle's stream.
#ifndef FUSILLI_GRAPH_H
#define FUSILLI_GRAPH_H

#include <algorithm>
#include <array>
#include <cctype>
#include <cstdlib>
#include <filesystem>
#include <fstream>
#include <memory>
#include <optional>
#include <set>
#include <span>
#include <sstream>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "backend.h"
#include "nodes.h"

namespace fusilli {

// ---- compile cache files: ${FUSILLI_CACHE_DIR or HOME}/.cache/fusilli/<graph>/<file> ---------
// (reference include/fusilli/support/cache.h:71-347)
enum class CachedAssetsType : uint8_t { Input, Output, Command, Statistics };

class CacheFile {
public:
  static std::filesystem::path getCacheDir() {
    const char *env = std::getenv("FUSILLI_CACHE_DIR");
    std::string base = env ? env : "";
    if (base.empty()) {
      const char *home = std::getenv("HOME");
      base = home ? home : "";
    }
    return std::filesystem::path(base) / ".cache" / "fusilli";
  }
  static std::filesystem::path getPath(const std::string &graphName, const std::string &fileName) {
    std::string clean;
    for (char c : graphName) {
      if (c == ' ') c = '_';
      if (std::isalnum(static_cast<unsigned char>(c)) || c == '_') clean.push_back(c);
    }
    if (clean.empty()) clean = "unnamed_graph";
    return getCacheDir() / clean / fileName;
  }
  static ErrorOr<CacheFile> create(const std::string &graphName, const std::string &fileName, bool remove) {
    const auto path = getPath(graphName, fileName);
    std::error_code ec;
    std::filesystem::create_directories(path.parent_path(), ec);
    FUSILLI_RETURN_ERROR_IF(bool(ec), ErrorCode::FileSystemFailure,
                            "Failed to create cache directory: " + path.parent_path().string() + " - " + ec.message());
    std::ofstream f(path, std::ios::binary);
    FUSILLI_RETURN_ERROR_IF(!f.is_open(), ErrorCode::FileSystemFailure, "Failed to create file: " + path.string());
    return ok(CacheFile(path, remove));
  }
  // An existing cache file; never removed by this object.
  static ErrorOr<CacheFile> open(const std::string &graphName, const std::string &fileName) {
    const auto path = getPath(graphName, fileName);
    FUSILLI_RETURN_ERROR_IF(!std::filesystem::exists(path), ErrorCode::FileSystemFailure,
                            "File does not exist: " + path.string());
    return ok(CacheFile(path, false));
  }
  ErrorObject write(const std::string &content) {
    std::ofstream f(path, std::ios::out | std::ios::binary);
    FUSILLI_RETURN_ERROR_IF(!f.is_open(), ErrorCode::FileSystemFailure, "Failed to open file: " + path.string());
    f << content;
    FUSILLI_RETURN_ERROR_IF(!f.good(), ErrorCode::FileSystemFailure, "Failed to write to file: " + path.string());
    return ok();
  }
  ErrorOr<std::string> read() const {
    std::ifstream f(path, std::ios::binary);
    FUSILLI_RETURN_ERROR_IF(!f.is_open(), ErrorCode::FileSystemFailure, "Failed to open file: " + path.string());
    std::ostringstream ss;
    ss << f.rdbuf();
    return ok(ss.str());
  }
  CacheFile(CacheFile &&o) noexcept : path(std::move(o.path)), remove_(std::exchange(o.remove_, false)) { o.path.clear(); }
  CacheFile &operator=(CacheFile &&o) noexcept {
    if (this != &o) {
      drop();
      path = std::move(o.path);
      remove_ = std::exchange(o.remove_, false);
      o.path.clear();
    }
    return *this;
  }
  CacheFile(const CacheFile &) = delete;
  CacheFile &operator=(const CacheFile &) = delete;
  ~CacheFile() { drop(); }
  std::filesystem::path path;

private:
  CacheFile(std::filesystem::path p, bool remove) : path(std::move(p)), remove_(remove) {}
  void drop() {
    if (remove_ && !path.empty()) {
      std::error_code ec;
      std::filesystem::remove(path, ec);
      // leave no empty per-graph directory behind
      const auto dir = path.parent_path();
      if (std::filesystem::exists(dir, ec) && std::filesystem::is_empty(dir, ec)) std::filesystem::remove(dir, ec);
    }
  }
  bool remove_ = false;
};

struct CachedAssets {
  CacheFile input, output, command, statistics;
};

#define FUSILLI_B200_INPUT_FILENAME "fusilli-b200-graph.txt"
#define FUSILLI_B200_OUTPUT_FILENAME "fusilli-b200-plan.bin"
#define FUSILLI_B200_COMMAND_FILENAME "fusilli-b200-command.txt"
#define FUSILLI_B200_STATISTICS_FILENAME "fusilli-b200-statistics.json"

class Graph {
public:
  using VariantPack = std::unordered_map<std::shared_ptr<TensorAttr>, std::shared_ptr<Buffer>>;

  Graph() = default;
  Graph(const Graph &) = delete;
  Graph &operator=(const Graph &) = delete;
  Graph(Graph &&o) noexcept { *this = std::move(o); }
  Graph &operator=(Graph &&o) noexcept {
    if (this != &o) {
      clearRuntimeState();
      context = o.context;
      nodes_ = std::move(o.nodes_);
      inputs_ = std::move(o.inputs_);
      outputs_ = std::move(o.outputs_);
      validated_ = o.validated_;
      plan_ = std::exchange(o.plan_, nullptr);
      artifact_ = std::move(o.artifact_);
      workspaceSize_ = o.workspaceSize_;
      loadedBackend_ = o.loadedBackend_;
      argTensors_ = std::move(o.argTensors_);
      cache_ = std::move(o.cache_);
      o.cache_.reset();
      cachedDescription_ = std::move(o.cachedDescription_);
      cachedRemove_ = o.cachedRemove_;
    }
    return *this;
  }
  ~Graph() { clearRuntimeState(); }

  Context context;

  // ---- context ---------------------------------------------------------------------------
  const std::string &getName() const { return context.getName(); }
  Graph &setName(const std::string &n) { context.setName(n); return *this; }
  Graph &setIODataType(DataType t) { context.setIODataType(t); return *this; }
  Graph &setComputeDataType(DataType t) { context.setComputeDataType(t); return *this; }
  Graph &setIntermediateDataType(DataType t) { context.setIntermediateDataType(t); return *this; }

  // ---- builders (reference graph.h:756-1193: auto names, virtual outputs) ----------------------
  TensorPtr tensor(const TensorAttr &t) {
    auto p = std::make_shared<TensorAttr>(t);
    inputs_.push_back(p);
    return p;
  }
  TensorPtr convFProp(const TensorPtr &x, const TensorPtr &w, ConvFPropAttr &a) {
    autoName(a, "conv_fprop", {{"X", x}, {"W", w}});
    auto y = outputTensor(a.getName() + "_Y");
    a.setX(x).setW(w).setY(y);
    nodes_.push_back(std::make_unique<ConvFPropNode>(std::move(a), context));
    return y;
  }
  TensorPtr convWGrad(const TensorPtr &dy, const TensorPtr &x, ConvWGradAttr &a) {
    autoName(a, "conv_wgrad", {{"DY", dy}, {"X", x}});
    auto dw = outputTensor(a.getName() + "_DW");
    a.setDY(dy).setX(x).setDW(dw);
    nodes_.push_back(std::make_unique<ConvWGradNode>(std::move(a), context));
    return dw;
  }
  TensorPtr convDGrad(const TensorPtr &dy, const TensorPtr &w, ConvDGradAttr &a) {
    autoName(a, "conv_dgrad", {{"DY", dy}, {"W", w}});
    auto dx = outputTensor(a.getName() + "_DX");
    a.setDY(dy).setW(w).setDX(dx);
    nodes_.push_back(std::make_unique<ConvDGradNode>(std::move(a), context));
    return dx;
  }
  TensorPtr matmul(const TensorPtr &a_, const TensorPtr &b, MatmulAttr &a) {
    autoName(a, "matmul", {{"A", a_}, {"B", b}});
    auto c = outputTensor(a.getName() + "_C");
    a.setA(a_).setB(b).setC(c);
    nodes_.push_back(std::make_unique<MatmulNode>(std::move(a), context));
    return c;
  }
  TensorPtr sdpa(const TensorPtr &q, const TensorPtr &k, const TensorPtr &v, const TensorPtr &mask, SdpaAttr &a) {
    autoName(a, "sdpa", {{"Q", q}, {"K", k}, {"V", v}, {"MASK", mask}});
    auto o = outputTensor(a.getName() + "_O");
    a.setQ(q).setK(k).setV(v).setO(o);
    if (mask) a.setMASK(mask);
    nodes_.push_back(std::make_unique<SdpaNode>(std::move(a), context));
    return o;
  }
  std::array<TensorPtr, 3> layernorm(const TensorPtr &x, const TensorPtr &scale, const TensorPtr &bias,
                                     LayernormAttr &a) {
    autoName(a, "layernorm", {{"X", x}, {"SCALE", scale}, {"BIAS", bias}, {"EPSILON", a.getEpsilon()}});
    auto y = outputTensor(a.getName() + "_Y");
    TensorPtr m, v;
    if (a.getForwardPhase() == NormFwdPhase::TRAINING) {
      m = outputTensor(a.getName() + "_MEAN");
      v = outputTensor(a.getName() + "_INV_VARIANCE");
    }
    a.setX(x).setSCALE(scale).setBIAS(bias).setY(y).setMEAN(m).setINV_VARIANCE(v);
    nodes_.push_back(std::make_unique<LayerNormNode>(std::move(a), context));
    return {y, m, v};
  }
  std::array<TensorPtr, 3> batchnorm(const TensorPtr &x, const TensorPtr &scale, const TensorPtr &bias,
                                     const TensorPtr &mean, const TensorPtr &var, BatchnormAttr &a) {
    autoName(a, "batchnorm", {{"X", x}, {"SCALE", scale}, {"BIAS", bias}, {"MEAN", mean}, {"VAR", var},
                              {"EPSILON", a.getEpsilon()}, {"MOMENTUM", a.getMomentum()}});
    auto y = outputTensor(a.getName() + "_Y");
    TensorPtr sm, si;
    if (a.getForwardPhase() == NormFwdPhase::TRAINING) {
      sm = outputTensor(a.getName() + "_SAVED_MEAN");
      si = outputTensor(a.getName() + "_SAVED_INV_VARIANCE");
    }
    a.setX(x).setSCALE(scale).setBIAS(bias).setMEAN(mean).setVAR(var).setY(y).setSAVED_MEAN(sm).setSAVED_INV_VARIANCE(si);
    nodes_.push_back(std::make_unique<BatchNormNode>(std::move(a), context));
    return {y, sm, si};
  }
  std::array<TensorPtr, 2> rmsnorm(const TensorPtr &x, const TensorPtr &scale, RmsnormAttr &a) {
    autoName(a, "rmsnorm", {{"X", x}, {"SCALE", scale}, {"EPSILON", a.getEpsilon()}});
    auto y = outputTensor(a.getName() + "_Y");
    TensorPtr r;
    if (a.getForwardPhase() == NormFwdPhase::TRAINING) r = outputTensor(a.getName() + "_INV_RMS");
    a.setX(x).setSCALE(scale).setY(y).setINV_RMS(r);
    nodes_.push_back(std::make_unique<RmsNormNode>(std::move(a), context));
    return {y, r};
  }
  TensorPtr reduction(const TensorPtr &x, ReductionAttr &a) {
    autoName(a, "reduction", {{"X", x}});
    auto y = outputTensor(a.getName() + "_Y");
    a.setX(x).setY(y);
    nodes_.push_back(std::make_unique<ReductionNode>(std::move(a), context));
    return y;
  }
  // Accepted as in the reference (graph.h:1195-1227); compileToArtifact refuses graphs that hold one.
  std::vector<TensorPtr> customOp(std::vector<TensorPtr> ins, CustomOpAttr &a) {
    if (a.getName().empty()) a.setName("custom_op_" + std::to_string(nodes_.size()));
    for (size_t i = 0; i < ins.size(); ++i)
      if (ins[i] && ins[i]->getName().empty()) ins[i]->setName(a.getName() + "_IN_" + std::to_string(i));
    std::vector<TensorPtr> outs;
    for (size_t i = 0; i < a.getNumOutputs(); ++i) outs.push_back(outputTensor(a.getName() + "_OUT_" + std::to_string(i)));
    auto node = std::make_unique<CustomOpNode>(std::move(a), context);
    node->inputs = std::move(ins);
    node->outputs = outs;
    nodes_.push_back(std::move(node));
    return outs;
  }
  TensorPtr pointwise(const TensorPtr &in0, PointwiseAttr &a) { return addPointwise({in0, nullptr, nullptr}, 1, a); }
  TensorPtr pointwise(const TensorPtr &in0, const TensorPtr &in1, PointwiseAttr &a) {
    return addPointwise({in0, in1, nullptr}, 2, a);
  }
  TensorPtr pointwise(const TensorPtr &in0, const TensorPtr &in1, const TensorPtr &in2, PointwiseAttr &a) {
    return addPointwise({in0, in1, in2}, 3, a);
  }

#include "graph_impl.inc"
};

} // namespace fusilli

#endif // FUSILLI_GRAPH_H
