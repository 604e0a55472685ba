// Internal definitions shared by the host side of libfusilli_b200.so:
// status/error plumbing, the device/buffer objects behind the opaque C handles,
// and the kernel plan (the lowered form of a validated Fusilli graph).
#ifndef FB_COMMON_H
#define FB_COMMON_H

#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/fusilli_b200.h"
#include "kernels/device_types.h"

#define FB_EXPORT extern "C" __attribute__((visibility("default")))

namespace fb {

// Records `msg` as the calling thread's last error and returns `code`.
fb_status fail(fb_status code, const std::string &msg);
void clear_error();

#define FB_CUDA_OK(expr)                                                       \
  do {                                                                         \
    cudaError_t _e = (expr);                                                   \
    if (_e != cudaSuccess)                                                     \
      return fb::fail(FB_RUNTIME_FAILURE, std::string(#expr) + ": " +          \
                                              cudaGetErrorString(_e));         \
  } while (0)

#define FB_REQUIRE(cond, code, msg)                                            \
  do {                                                                         \
    if (!(cond)) return fb::fail((code), (msg));                               \
  } while (0)

size_t dtype_size(int32_t dtype); // 0 for unsupported and for sub-byte types
size_t dtype_bits(int32_t dtype); // 0 for unsupported types; 4 for Int4 (matmul operands only)
const char *dtype_name(int32_t dtype);

} // namespace fb

struct fb_device {
  int ordinal = 0;
  cudaStream_t stream = nullptr;
  bool owns_stream = false;
  int sm_count = 0;
  uint32_t *error_word = nullptr; // device word set by kernels whose waits ran out
  // One reference for the handle itself plus one per live buffer: closing the
  // handle before its buffers must not pull the stream out from under them.
  std::atomic<int> refs{1};
};

struct fb_buffer {
  void *ptr = nullptr;
  size_t bytes = 0;
  bool owned = false;
  int ordinal = 0;
  fb_device *dev = nullptr; // retained; its stream orders the allocation and the free
  std::atomic<int> refs{1};
};

namespace fb {

// ---- plan -------------------------------------------------------------------

struct TensorInfo {
  std::string name;
  int32_t dtype = 0, role = 0, rank = 0, arg_index = -1;
  int64_t dims[FB_MAX_RANK] = {0};
  int64_t strides[FB_MAX_RANK] = {0};
  double scalar = 0.0;
  uint32_t dynamic_mask = 0; // bit k: logical dim k takes its extent at execute
  int64_t ws_offset = -1; // >= 0: materialised in the workspace at this byte offset
  int64_t phys_elems() const; // elements of the dense physical buffer
  size_t phys_bytes() const;  // its size; sub-byte elements are packed, rounded up to a byte
};

struct NodeInfo {
  std::string name;
  fb_node_desc d; // d.name is not valid after load; use `name`
};

enum StepKind : int32_t {
  STEP_POINTWISE = 1, // standalone elementwise kernel
  STEP_REDUCTION = 2,
  STEP_NORM = 3,      // layernorm / rmsnorm
  STEP_CONTRACT = 4,  // conv fprop/dgrad/wgrad or matmul (+ fused epilogue)
  STEP_SDPA = 5,
  STEP_BATCHNORM = 6, // training: partial statistics, merge, apply; inference: apply
};

enum Engine : int32_t {
  ENGINE_SIMT = 0,    // CUDA-core kernels: any dtype/stride the op allows
  ENGINE_TCGEN05 = 1, // tcgen05/TMEM/TMA kernels: 16-bit operands, aligned shapes
  ENGINE_TCGEN05_SPLIT = 2, // fp32 forward convolution as bf16 piece products on tcgen05 (fp32-grade results)
};

constexpr int kMaxEpilogueOps = 6;

// One fused pointwise op applied to the running value `v` of a contraction.
struct EpilogueOpInfo {
  int32_t mode = 0;      // FB_PW_*
  int32_t operand = -1;  // tensor id of the other input, -1 for unary
  int32_t value_is_in1 = 0; // running value is IN_1 (operand is IN_0)
  int32_t out_tensor = -1;  // tensor whose dtype the result is rounded to
  float fparams[4] = {1.f, 1.f, 20.f, 1.f};
};

struct Step {
  int32_t kind = 0;
  int32_t engine = ENGINE_SIMT;
  int32_t node = -1;     // index of the (first) node this step executes
  int32_t out_tensor = -1; // tensor written by the step (after the epilogue)
  int32_t num_epilogue = 0;
  EpilogueOpInfo epilogue[kMaxEpilogueOps];
  int32_t split_k = 1;      // STEP_CONTRACT wgrad: partial sums in the workspace
  int64_t scratch_offset = -1; // workspace byte offset of this step's scratch
  int64_t scratch_bytes = 0;
};

struct Plan {
  std::string name;
  std::vector<TensorInfo> tensors;
  std::vector<NodeInfo> nodes;
  std::vector<Step> steps;
  int32_t num_args = 0;
  size_t workspace_bytes = 0;
  std::vector<int32_t> arg_tensor; // arg index -> tensor id
  bool has_dynamic_dims() const {
    for (const TensorInfo &t : tensors)
      if (t.dynamic_mask) return true;
    return false;
  }
};

// Lowers tensors+nodes (already filled in `plan`) to steps; FB_NOT_IMPLEMENTED
// for graphs the kernels cannot run.
fb_status lower(Plan &plan);
// `base` with the dynamic dims of its bound tensors replaced by `arg_dims` (FB_MAX_RANK logical
// extents per argument), the dims of virtual tensors derived from the nodes' shape rules, dense
// strides regenerated, and the steps lowered again for the concrete shape.
fb_status specialize(const Plan &base, const int64_t *arg_dims, Plan &out);
fb_status serialize(const Plan &plan, std::vector<uint8_t> &out);
fb_status deserialize(const uint8_t *bytes, size_t n, Plan &plan);
std::string stats_json(const Plan &plan);
const char *step_kernel_name(const Plan &plan, const Step &s);

// Launchers (defined next to their kernels). `ptr(t)` resolves a tensor id to its
// device pointer for this execute call.
struct ExecContext {
  const Plan *plan;
  fb_device *dev;
  void *const *args;
  uint8_t *workspace;
  void *tensor_ptr(int32_t id) const;
  TensorRef ref(int32_t id) const; // pointer + dtype + dims + strides
};

fb_status launch_pointwise(const ExecContext &cx, const Step &s);
fb_status launch_reduction(const ExecContext &cx, const Step &s);
fb_status launch_norm(const ExecContext &cx, const Step &s);
fb_status launch_contract_simt(const ExecContext &cx, const Step &s);
fb_status launch_sdpa_simt(const ExecContext &cx, const Step &s);
fb_status launch_gemm_tc(const ExecContext &cx, const Step &s);
fb_status launch_conv_tc(const ExecContext &cx, const Step &s);
fb_status launch_sdpa_tc(const ExecContext &cx, const Step &s);
fb_status launch_conv_wgrad_tc(const ExecContext &cx, const Step &s);
fb_status launch_batchnorm(const ExecContext &cx, const Step &s);
fb_status launch_conv_split_f32(const ExecContext &cx, const Step &s);
// Workspace the batch-statistics pass needs (0 in inference); *splits = slices of the reduction.
int64_t batchnorm_scratch_bytes(const Plan &p, const Step &s, int32_t *splits);

// Eligibility checks used by the lowering (pure host logic, no device).
bool gemm_tc_eligible(const Plan &p, const Step &s);
bool conv_tc_eligible(const Plan &p, const Step &s);
bool sdpa_tc_eligible(const Plan &p, const Step &s);
bool conv_wgrad_tc_eligible(const Plan &p, const Step &s);
bool conv_split_f32_eligible(const Plan &p, const Step &s);
int64_t conv_split_f32_scratch_bytes(const Plan &p, const Step &s);
int64_t conv_wgrad_tc_scratch_bytes(const Plan &p, const Step &s, int32_t *slices);
// Kernel launches one execute of this step issues.
int step_launches(const Plan &p, const Step &s);

// Fills the device-side epilogue description of a contraction step.
fb_status build_epilogue(const ExecContext &cx, const Step &s, EpilogueDev &out);

} // namespace fb

#endif // FB_COMMON_H
