// Host cost of Graph::execute: a 1x1 bf16 convolution plan (one tensor-core kernel, two tensor maps)
// enqueued 1000 times back to back, timed with std::chrono around the enqueue loop only (the device
// drains afterwards). Run once as is and once with FUSILLI_B200_NO_LAUNCH_CACHE=1 to see what the
// tensor-map cache and the once-per-device shared-memory attribute save per call.
#include <fusilli.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <unordered_map>
#include <vector>

using namespace fusilli;

#define CHECK_OK(expr)                                                        \
  do {                                                                        \
    auto _e = ErrorObject(expr);                                              \
    if (isError(_e)) {                                                        \
      std::fprintf(stderr, "%s failed: %s\n", #expr, _e.getMessage().c_str()); \
      return 1;                                                               \
    }                                                                         \
  } while (0)

int main() {
  constexpr int64_t n = 8, c = 64, h = 56, w = 56, k = 64;
  auto handleOr = Handle::create(Backend::CUDA);
  if (isError(handleOr)) {
    std::fprintf(stderr, "no CUDA device\n");
    return 1;
  }
  Handle handle = std::move(*handleOr);
  Graph g;
  g.setName("host_execute_latency").setIODataType(DataType::BFloat16).setComputeDataType(DataType::Float)
      .setIntermediateDataType(DataType::BFloat16);
  auto x = g.tensor(TensorAttr().setName("x").setDim({n, c, h, w}).setStride({c * h * w, 1, c * w, c}));
  auto wt = g.tensor(TensorAttr().setName("w").setDim({k, c, 1, 1}).setStride({c, 1, c, c}));
  ConvFPropAttr attr;
  attr.setPadding({0, 0}).setStride({1, 1}).setDilation({1, 1}).setName("conv");
  auto y = g.convFProp(x, wt, attr);
  y->setName("y").setOutput(true);
  CHECK_OK(g.validate());
  CHECK_OK(g.compile(handle, /*remove=*/true));
  auto bufOf = [&](size_t elems) { return Buffer::allocateRaw(handle, elems * 2); };
  auto xb = bufOf(n * c * h * w), wb = bufOf(k * c), yb = bufOf(n * k * h * w);
  if (isError(xb) || isError(wb) || isError(yb)) return 1;
  std::unordered_map<std::shared_ptr<TensorAttr>, std::shared_ptr<Buffer>> pack = {
      {x, std::make_shared<Buffer>(std::move(*xb))},
      {wt, std::make_shared<Buffer>(std::move(*wb))},
      {y, std::make_shared<Buffer>(std::move(*yb))}};
  auto ws = g.getWorkspaceSize();
  if (isError(ws)) return 1;
  for (int i = 0; i < 20; ++i) CHECK_OK(g.execute(handle, pack, nullptr));
  fb_device_sync(handle.device());
  constexpr int calls = 1000;
  const auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < calls; ++i) CHECK_OK(g.execute(handle, pack, nullptr));
  const auto t1 = std::chrono::steady_clock::now();
  fb_device_sync(handle.device());
  const auto t2 = std::chrono::steady_clock::now();
  const double enqueue_us = std::chrono::duration<double, std::micro>(t1 - t0).count() / calls;
  const double total_us = std::chrono::duration<double, std::micro>(t2 - t0).count() / calls;
  const char *e = std::getenv("FUSILLI_B200_NO_LAUNCH_CACHE");
  std::printf("{\"launch_cache\": %s, \"calls\": %d, \"host_us_per_execute\": %.2f, \"us_per_execute_incl_device\": %.2f}\n",
              (e && e[0] == '1') ? "false" : "true", calls, enqueue_us, total_us);
  return 0;
}
