// Device, buffer and plan entry points of the C ABI (host side).
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "common.h"

namespace fb {

static thread_local std::string g_last_error;

fb_status fail(fb_status code, const std::string &msg) {
  g_last_error = msg;
  return code;
}
void clear_error() { g_last_error.clear(); }

size_t dtype_size(int32_t dt) {
  switch (dt) {
  case FB_DT_HALF:
  case FB_DT_BFLOAT16:
  case FB_DT_INT16: return 2;
  case FB_DT_FLOAT:
  case FB_DT_INT32: return 4;
  case FB_DT_INT64: return 8;
  case FB_DT_UINT8:
  case FB_DT_INT8:
  case FB_DT_BOOLEAN: return 1;
  default: return 0; // Double, FP8E5M2: no kernels; Int4: see dtype_bits
  }
}

size_t dtype_bits(int32_t dt) { return dt == FB_DT_INT4 ? 4 : dtype_size(dt) * 8; }

const char *dtype_name(int32_t dt) {
  static const char *names[] = {"notset", "f16", "bf16", "f32",  "f64",  "ui8", "si4",
                                "si8",    "si16", "si32", "si64", "i1",  "f8E5M2"};
  return (dt >= 0 && dt <= FB_DT_FP8E5M2) ? names[dt] : "?";
}

// Elements the buffer must hold: one past the offset of the last element. For a dense tensor in
// any dim order this is the product of the dims; with padded strides (a matmul operand whose
// leading stride exceeds its row length) it is larger, and the size check must see that.
int64_t TensorInfo::phys_elems() const {
  int64_t last = 0;
  for (int i = 0; i < rank; ++i)
    if (strides[i] != 0) last += (dims[i] - 1) * strides[i];
  return last + 1;
}

size_t TensorInfo::phys_bytes() const { return ((size_t)phys_elems() * dtype_bits(dtype) + 7) / 8; }

void *ExecContext::tensor_ptr(int32_t id) const {
  const TensorInfo &t = plan->tensors[id];
  if (t.arg_index >= 0) return args[t.arg_index];
  if (t.ws_offset >= 0) return workspace + t.ws_offset;
  return nullptr;
}

TensorRef ExecContext::ref(int32_t id) const {
  TensorRef r;
  memset(&r, 0, sizeof(r));
  if (id < 0) return r;
  const TensorInfo &t = plan->tensors[id];
  r.ptr = tensor_ptr(id);
  r.dtype = t.dtype;
  r.rank = t.rank;
  for (int i = 0; i < t.rank; ++i) {
    r.dims[i] = t.dims[i];
    r.strides[i] = t.strides[i];
  }
  return r;
}

} // namespace fb

using namespace fb;

struct fb_plan {
  Plan plan;
  int ordinal = 0;
  // Plans lowered again for concrete extents of the dynamic dims, keyed by the extents of all
  // arguments. Bounded: shapes past the limit replace the whole set. Entries are shared: a caller
  // holds its own reference for the length of its execute, so dropping the set under it is safe.
  std::mutex mu;
  std::map<std::vector<int64_t>, std::shared_ptr<const Plan>> shaped;
  static constexpr size_t kMaxShaped = 64;
};

FB_EXPORT int32_t fb_abi_version(void) { return FB_ABI_VERSION; }

FB_EXPORT const char *fb_last_error(void) { return g_last_error.c_str(); }

FB_EXPORT int32_t fb_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// ---- device --------------------------------------------------------------------

static std::mutex g_device_mutex;

FB_EXPORT fb_status fb_device_open(int32_t ordinal, void *ext_stream, fb_device **out) {
  clear_error();
  FB_REQUIRE(out != nullptr, FB_INVALID_ARGUMENT, "fb_device_open: out is NULL");
  *out = nullptr;
  std::lock_guard<std::mutex> lock(g_device_mutex);
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    cudaGetLastError();
    return fail(FB_RUNTIME_FAILURE,
                "fb_device_open: no usable CUDA device (this library has no CPU execution path)");
  }
  FB_REQUIRE(ordinal >= 0 && ordinal < n, FB_RUNTIME_FAILURE,
             "fb_device_open: device ordinal " + std::to_string(ordinal) + " out of range (" +
                 std::to_string(n) + " devices)");
  cudaDeviceProp prop;
  FB_CUDA_OK(cudaGetDeviceProperties(&prop, ordinal));
  FB_REQUIRE(prop.major == 10, FB_RUNTIME_FAILURE,
             std::string("fb_device_open: device '") + prop.name + "' is compute capability " +
                 std::to_string(prop.major) + "." + std::to_string(prop.minor) +
                 "; this library is built for sm_100a only");
  FB_CUDA_OK(cudaSetDevice(ordinal));
  fb_device *d = new fb_device();
  d->ordinal = ordinal;
  d->sm_count = prop.multiProcessorCount;
  if (ext_stream) {
    d->stream = static_cast<cudaStream_t>(ext_stream);
    d->owns_stream = false;
  } else {
    cudaError_t se = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking);
    if (se != cudaSuccess) {
      delete d;
      return fail(FB_RUNTIME_FAILURE, std::string("cudaStreamCreate: ") + cudaGetErrorString(se));
    }
    d->owns_stream = true;
  }
  cudaError_t me = cudaMalloc(&d->error_word, sizeof(uint32_t));
  if (me == cudaSuccess) me = cudaMemset(d->error_word, 0, sizeof(uint32_t));
  if (me != cudaSuccess) {
    if (d->owns_stream) cudaStreamDestroy(d->stream);
    delete d;
    return fail(FB_RUNTIME_FAILURE, std::string("cudaMalloc(error word): ") + cudaGetErrorString(me));
  }
  *out = d;
  return FB_OK;
}

static void device_unref(fb_device *dev) {
  if (dev->refs.fetch_sub(1) != 1) return;
  cudaSetDevice(dev->ordinal);
  cudaStreamSynchronize(dev->stream);
  if (dev->error_word) cudaFree(dev->error_word);
  if (dev->owns_stream) cudaStreamDestroy(dev->stream);
  delete dev;
}

FB_EXPORT fb_status fb_device_close(fb_device *dev) {
  clear_error();
  if (!dev) return FB_OK;
  cudaSetDevice(dev->ordinal);
  cudaStreamSynchronize(dev->stream);
  device_unref(dev); // destroyed once the last buffer created on it is released
  return FB_OK;
}

FB_EXPORT fb_status fb_device_sync(fb_device *dev) {
  clear_error();
  FB_REQUIRE(dev != nullptr, FB_INVALID_ARGUMENT, "fb_device_sync: device is NULL");
  FB_CUDA_OK(cudaSetDevice(dev->ordinal));
  FB_CUDA_OK(cudaStreamSynchronize(dev->stream));
  return FB_OK;
}

FB_EXPORT void *fb_device_stream(fb_device *dev) { return dev ? dev->stream : nullptr; }
FB_EXPORT int32_t fb_device_ordinal(fb_device *dev) { return dev ? dev->ordinal : -1; }

FB_EXPORT fb_status fb_device_kernel_error(fb_device *dev, uint32_t *error_word) {
  clear_error();
  FB_REQUIRE(dev && error_word, FB_INVALID_ARGUMENT, "fb_device_kernel_error: NULL argument");
  FB_CUDA_OK(cudaSetDevice(dev->ordinal));
  FB_CUDA_OK(cudaMemcpyAsync(error_word, dev->error_word, sizeof(uint32_t), cudaMemcpyDeviceToHost,
                             dev->stream));
  FB_CUDA_OK(cudaStreamSynchronize(dev->stream));
  return FB_OK;
}

// ---- buffers -----------------------------------------------------------------

FB_EXPORT fb_status fb_buffer_alloc(fb_device *dev, size_t bytes, fb_buffer **out) {
  clear_error();
  FB_REQUIRE(dev && out, FB_INVALID_ARGUMENT, "fb_buffer_alloc: NULL argument");
  *out = nullptr;
  FB_REQUIRE(bytes > 0, FB_RUNTIME_FAILURE, "fb_buffer_alloc: cannot allocate zero-size buffer");
  FB_CUDA_OK(cudaSetDevice(dev->ordinal));
  void *p = nullptr;
  FB_CUDA_OK(cudaMallocAsync(&p, bytes, dev->stream));
  fb_buffer *b = new fb_buffer();
  b->ptr = p;
  b->bytes = bytes;
  b->owned = true;
  b->ordinal = dev->ordinal;
  b->dev = dev;
  dev->refs.fetch_add(1);
  *out = b;
  return FB_OK;
}

FB_EXPORT fb_status fb_buffer_wrap(fb_device *dev, void *dptr, size_t bytes, fb_buffer **out) {
  clear_error();
  FB_REQUIRE(dev && out, FB_INVALID_ARGUMENT, "fb_buffer_wrap: NULL argument");
  *out = nullptr;
  FB_REQUIRE(dptr != nullptr, FB_RUNTIME_FAILURE, "fb_buffer_wrap: device pointer is NULL");
  FB_REQUIRE(bytes > 0, FB_RUNTIME_FAILURE, "fb_buffer_wrap: zero-size buffer");
  fb_buffer *b = new fb_buffer();
  b->ptr = dptr;
  b->bytes = bytes;
  b->owned = false;
  b->ordinal = dev->ordinal;
  b->dev = dev;
  dev->refs.fetch_add(1);
  *out = b;
  return FB_OK;
}

FB_EXPORT fb_status fb_buffer_retain(fb_buffer *buf) {
  clear_error();
  FB_REQUIRE(buf != nullptr, FB_INVALID_ARGUMENT, "fb_buffer_retain: buffer is NULL");
  buf->refs.fetch_add(1);
  return FB_OK;
}

FB_EXPORT fb_status fb_buffer_release(fb_buffer *buf) {
  clear_error();
  if (!buf) return FB_OK;
  if (buf->refs.fetch_sub(1) == 1) {
    if (buf->owned && buf->ptr) {
      cudaSetDevice(buf->ordinal);
      // Ordered after the work already queued on the stream it was allocated on.
      cudaFreeAsync(buf->ptr, buf->dev->stream);
    }
    device_unref(buf->dev);
    delete buf;
  }
  return FB_OK;
}

FB_EXPORT fb_status fb_buffer_h2d(fb_device *dev, fb_buffer *buf, const void *src, size_t bytes) {
  clear_error();
  FB_REQUIRE(dev && buf && src, FB_INVALID_ARGUMENT, "fb_buffer_h2d: NULL argument");
  FB_REQUIRE(bytes <= buf->bytes, FB_INVALID_ARGUMENT,
             "fb_buffer_h2d: copy of " + std::to_string(bytes) + " bytes exceeds buffer size " +
                 std::to_string(buf->bytes));
  FB_CUDA_OK(cudaSetDevice(dev->ordinal));
  FB_CUDA_OK(cudaMemcpyAsync(buf->ptr, src, bytes, cudaMemcpyHostToDevice, dev->stream));
  // Pageable sources are staged before the call returns; pinned sources are not, so
  // wait for those: the caller may reuse `src` as soon as this returns.
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, src) == cudaSuccess && attr.type == cudaMemoryTypeHost) {
    FB_CUDA_OK(cudaStreamSynchronize(dev->stream));
  } else {
    cudaGetLastError();
  }
  return FB_OK;
}

FB_EXPORT fb_status fb_buffer_d2h(fb_device *dev, fb_buffer *buf, void *dst, size_t bytes) {
  clear_error();
  FB_REQUIRE(dev && buf && dst, FB_INVALID_ARGUMENT, "fb_buffer_d2h: NULL argument");
  FB_REQUIRE(bytes <= buf->bytes, FB_INVALID_ARGUMENT,
             "fb_buffer_d2h: read of " + std::to_string(bytes) + " bytes exceeds buffer size " +
                 std::to_string(buf->bytes));
  FB_CUDA_OK(cudaSetDevice(dev->ordinal));
  FB_CUDA_OK(cudaMemcpyAsync(dst, buf->ptr, bytes, cudaMemcpyDeviceToHost, dev->stream));
  FB_CUDA_OK(cudaStreamSynchronize(dev->stream));
  return FB_OK;
}

FB_EXPORT void *fb_buffer_ptr(fb_buffer *buf) { return buf ? buf->ptr : nullptr; }
FB_EXPORT size_t fb_buffer_size(fb_buffer *buf) { return buf ? buf->bytes : 0; }

// ---- plan -------------------------------------------------------------------

static fb_status plan_from_desc(const fb_graph_desc *g, Plan &p) {
  FB_REQUIRE(g != nullptr, FB_INVALID_ARGUMENT, "fb_plan_build: graph is NULL");
  FB_REQUIRE(g->num_tensors > 0 && g->num_nodes > 0 && g->tensors && g->nodes,
             FB_INVALID_ARGUMENT, "fb_plan_build: graph has no tensors or no nodes");
  p.name = g->name ? g->name : "";
  p.tensors.resize(g->num_tensors);
  int max_arg = -1;
  for (int i = 0; i < g->num_tensors; ++i) {
    const fb_tensor_desc &d = g->tensors[i];
    TensorInfo &t = p.tensors[i];
    t.name = d.name ? d.name : "";
    t.dtype = d.dtype;
    t.role = d.role;
    t.rank = d.rank;
    t.arg_index = d.arg_index;
    t.scalar = d.scalar_value;
    FB_REQUIRE(d.rank >= 1 && d.rank <= FB_MAX_RANK, FB_INVALID_ARGUMENT,
               "fb_plan_build: tensor '" + t.name + "' has unsupported rank " + std::to_string(d.rank));
    for (int k = 0; k < d.rank; ++k) {
      t.dims[k] = d.dims[k];
      t.strides[k] = d.strides[k];
      FB_REQUIRE(d.dims[k] >= 1 && d.strides[k] >= 0, FB_INVALID_ARGUMENT,
                 "fb_plan_build: tensor '" + t.name + "' has a non-positive dim or negative stride");
    }
    t.dynamic_mask = d.dynamic_mask;
    FB_REQUIRE(d.rank >= 32 || (d.dynamic_mask >> d.rank) == 0, FB_INVALID_ARGUMENT,
               "fb_plan_build: tensor '" + t.name + "' marks a dim past its rank as dynamic");
    for (int k = 0; k < d.rank; ++k)
      FB_REQUIRE(!(d.dynamic_mask >> k & 1) || (d.strides[k] != 0 && d.role != FB_TENSOR_SCALAR),
                 FB_INVALID_ARGUMENT,
                 "fb_plan_build: tensor '" + t.name + "' has a dynamic dim with a broadcast stride");
    bool bound = d.role == FB_TENSOR_INPUT || d.role == FB_TENSOR_OUTPUT;
    FB_REQUIRE(bound == (d.arg_index >= 0), FB_INVALID_ARGUMENT,
               "fb_plan_build: tensor '" + t.name + "' role and arg_index disagree");
    if (d.arg_index > max_arg) max_arg = d.arg_index;
  }
  p.num_args = max_arg + 1;
  p.arg_tensor.assign(p.num_args, -1);
  for (int i = 0; i < g->num_tensors; ++i) {
    int a = p.tensors[i].arg_index;
    if (a >= 0) {
      FB_REQUIRE(p.arg_tensor[a] < 0, FB_INVALID_ARGUMENT,
                 "fb_plan_build: arg_index " + std::to_string(a) + " used twice");
      p.arg_tensor[a] = i;
    }
  }
  for (int a = 0; a < p.num_args; ++a)
    FB_REQUIRE(p.arg_tensor[a] >= 0, FB_INVALID_ARGUMENT,
               "fb_plan_build: arg_index " + std::to_string(a) + " is not assigned");
  p.nodes.resize(g->num_nodes);
  for (int i = 0; i < g->num_nodes; ++i) {
    p.nodes[i].d = g->nodes[i];
    p.nodes[i].name = g->nodes[i].name ? g->nodes[i].name : "";
    p.nodes[i].d.name = nullptr;
    for (int k = 0; k < FB_MAX_NODE_INPUTS; ++k)
      FB_REQUIRE(g->nodes[i].inputs[k] < g->num_tensors, FB_INVALID_ARGUMENT,
                 "fb_plan_build: node input tensor id out of range");
    for (int k = 0; k < FB_MAX_NODE_OUTPUTS; ++k)
      FB_REQUIRE(g->nodes[i].outputs[k] < g->num_tensors, FB_INVALID_ARGUMENT,
                 "fb_plan_build: node output tensor id out of range");
  }
  return FB_OK;
}

FB_EXPORT fb_status fb_plan_build(const fb_graph_desc *graph, uint8_t **bytes, size_t *num_bytes) {
  clear_error();
  FB_REQUIRE(bytes && num_bytes, FB_INVALID_ARGUMENT, "fb_plan_build: NULL output argument");
  *bytes = nullptr;
  *num_bytes = 0;
  Plan p;
  fb_status st = plan_from_desc(graph, p);
  if (st != FB_OK) return st;
  st = lower(p);
  if (st != FB_OK) return st;
  std::vector<uint8_t> blob;
  st = serialize(p, blob);
  if (st != FB_OK) return st;
  uint8_t *out = static_cast<uint8_t *>(malloc(blob.size()));
  FB_REQUIRE(out != nullptr, FB_INTERNAL_ERROR, "fb_plan_build: out of host memory");
  memcpy(out, blob.data(), blob.size());
  *bytes = out;
  *num_bytes = blob.size();
  return FB_OK;
}

FB_EXPORT void fb_bytes_free(uint8_t *bytes) { free(bytes); }

FB_EXPORT fb_status fb_plan_specialize(const uint8_t *bytes, size_t num_bytes, const int64_t *arg_dims,
                                       int32_t num_args, uint8_t **out_bytes, size_t *out_num_bytes) {
  clear_error();
  FB_REQUIRE(out_bytes && out_num_bytes, FB_INVALID_ARGUMENT, "fb_plan_specialize: NULL output argument");
  *out_bytes = nullptr;
  *out_num_bytes = 0;
  FB_REQUIRE(bytes != nullptr && num_bytes > 0, FB_RUNTIME_FAILURE, "fb_plan_specialize: empty artifact");
  Plan base, shaped;
  fb_status st = deserialize(bytes, num_bytes, base);
  if (st != FB_OK) return st;
  FB_REQUIRE(num_args == base.num_args, FB_VARIANT_PACK_ERROR,
             "fb_plan_specialize: expected dims of " + std::to_string(base.num_args) + " buffers, got " +
                 std::to_string(num_args));
  st = specialize(base, arg_dims, shaped);
  if (st != FB_OK) return st;
  std::vector<uint8_t> blob;
  st = serialize(shaped, blob);
  if (st != FB_OK) return st;
  uint8_t *out = static_cast<uint8_t *>(malloc(blob.size()));
  FB_REQUIRE(out != nullptr, FB_INTERNAL_ERROR, "fb_plan_specialize: out of host memory");
  memcpy(out, blob.data(), blob.size());
  *out_bytes = out;
  *out_num_bytes = blob.size();
  return FB_OK;
}

FB_EXPORT fb_status fb_plan_load(fb_device *dev, const uint8_t *bytes, size_t num_bytes,
                                 fb_plan **out) {
  clear_error();
  FB_REQUIRE(out != nullptr, FB_INVALID_ARGUMENT, "fb_plan_load: out is NULL");
  *out = nullptr;
  FB_REQUIRE(dev != nullptr, FB_INVALID_ARGUMENT, "fb_plan_load: device is NULL");
  FB_REQUIRE(bytes != nullptr && num_bytes > 0, FB_RUNTIME_FAILURE, "fb_plan_load: empty artifact");
  fb_plan *p = new fb_plan();
  fb_status st = deserialize(bytes, num_bytes, p->plan);
  if (st != FB_OK) {
    delete p;
    return st;
  }
  p->ordinal = dev->ordinal;
  *out = p;
  return FB_OK;
}

FB_EXPORT fb_status fb_plan_check(const uint8_t *bytes, size_t num_bytes) {
  clear_error();
  FB_REQUIRE(bytes != nullptr && num_bytes > 0, FB_RUNTIME_FAILURE, "fb_plan_check: empty artifact");
  Plan p;
  return deserialize(bytes, num_bytes, p);
}

FB_EXPORT fb_status fb_plan_free(fb_plan *plan) {
  clear_error();
  delete plan;
  return FB_OK;
}

FB_EXPORT fb_status fb_plan_workspace_size(fb_plan *plan, size_t *bytes) {
  clear_error();
  FB_REQUIRE(plan && bytes, FB_INVALID_ARGUMENT, "fb_plan_workspace_size: NULL argument");
  *bytes = plan->plan.workspace_bytes;
  return FB_OK;
}

FB_EXPORT fb_status fb_plan_num_args(fb_plan *plan, int32_t *num_args) {
  clear_error();
  FB_REQUIRE(plan && num_args, FB_INVALID_ARGUMENT, "fb_plan_num_args: NULL argument");
  *num_args = plan->plan.num_args;
  return FB_OK;
}

FB_EXPORT fb_status fb_plan_num_launches(fb_plan *plan, int32_t *num_launches) {
  clear_error();
  FB_REQUIRE(plan && num_launches, FB_INVALID_ARGUMENT, "fb_plan_num_launches: NULL argument");
  int n = 0;
  for (const Step &s : plan->plan.steps) n += step_launches(plan->plan, s);
  *num_launches = n;
  return FB_OK;
}

FB_EXPORT fb_status fb_plan_stats_json(fb_plan *plan, char *buf, size_t cap, size_t *needed) {
  clear_error();
  FB_REQUIRE(plan && needed, FB_INVALID_ARGUMENT, "fb_plan_stats_json: NULL argument");
  std::string s = stats_json(plan->plan);
  *needed = s.size() + 1;
  if (buf && cap >= s.size() + 1) memcpy(buf, s.c_str(), s.size() + 1);
  return FB_OK;
}

static fb_status execute_plan(const fb_plan *plan, const Plan &p, fb_device *dev, void *const *args,
                              const size_t *arg_bytes, int32_t num_args, void *workspace,
                              size_t workspace_bytes) {
  FB_REQUIRE(dev->ordinal == plan->ordinal, FB_INVALID_ARGUMENT,
             "fb_plan_execute: plan was loaded for device " + std::to_string(plan->ordinal) +
                 " but executed on device " + std::to_string(dev->ordinal));
  FB_REQUIRE(num_args == p.num_args, FB_VARIANT_PACK_ERROR,
             "fb_plan_execute: expected " + std::to_string(p.num_args) + " buffers, got " +
                 std::to_string(num_args));
  FB_REQUIRE(args != nullptr || num_args == 0, FB_INVALID_ARGUMENT, "fb_plan_execute: args is NULL");
  for (int a = 0; a < num_args; ++a) {
    const TensorInfo &t = p.tensors[p.arg_tensor[a]];
    FB_REQUIRE(args[a] != nullptr, FB_VARIANT_PACK_ERROR,
               "fb_plan_execute: buffer for tensor '" + t.name + "' is NULL");
    if (arg_bytes) {
      size_t need = t.phys_bytes();
      FB_REQUIRE(arg_bytes[a] >= need, FB_INVALID_ARGUMENT,
                 "fb_plan_execute: buffer for tensor '" + t.name + "' has " +
                     std::to_string(arg_bytes[a]) + " bytes, needs " + std::to_string(need));
    }
  }
  if (p.workspace_bytes > 0) {
    FB_REQUIRE(workspace != nullptr, FB_INVALID_ARGUMENT,
               "Workspace buffer required but not provided (size=" +
                   std::to_string(p.workspace_bytes) + " bytes)");
    FB_REQUIRE(workspace_bytes >= p.workspace_bytes, FB_INVALID_ARGUMENT,
               "Workspace buffer too small: provided " + std::to_string(workspace_bytes) +
                   " bytes, required " + std::to_string(p.workspace_bytes) + " bytes");
  }
  FB_CUDA_OK(cudaSetDevice(dev->ordinal));
  ExecContext cx{&p, dev, args, static_cast<uint8_t *>(workspace)};
  for (const Step &s : p.steps) {
    fb_status st = FB_OK;
    switch (s.kind) {
    case STEP_POINTWISE: st = launch_pointwise(cx, s); break;
    case STEP_REDUCTION: st = launch_reduction(cx, s); break;
    case STEP_NORM: st = launch_norm(cx, s); break;
    case STEP_BATCHNORM: st = launch_batchnorm(cx, s); break;
    case STEP_CONTRACT:
      if (s.engine == ENGINE_TCGEN05_SPLIT) {
        st = launch_conv_split_f32(cx, s);
      } else if (s.engine == ENGINE_TCGEN05) {
        const int op = p.nodes[s.node].d.op;
        st = op == FB_OP_MATMUL ? launch_gemm_tc(cx, s)
                                : (op == FB_OP_CONV_WGRAD ? launch_conv_wgrad_tc(cx, s) : launch_conv_tc(cx, s));
      }
      else
        st = launch_contract_simt(cx, s);
      break;
    case STEP_SDPA:
      st = (s.engine == ENGINE_TCGEN05) ? launch_sdpa_tc(cx, s) : launch_sdpa_simt(cx, s);
      break;
    default: st = fail(FB_INTERNAL_ERROR, "fb_plan_execute: unknown step kind");
    }
    if (st != FB_OK) return st;
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess)
      return fail(FB_RUNTIME_FAILURE, std::string("kernel launch failed (") +
                                          step_kernel_name(p, s) + "): " + cudaGetErrorString(le));
  }
  return FB_OK;
}

FB_EXPORT fb_status fb_plan_execute(fb_plan *plan, fb_device *dev, void *const *args,
                                    const size_t *arg_bytes, int32_t num_args, void *workspace,
                                    size_t workspace_bytes) {
  clear_error();
  FB_REQUIRE(plan && dev, FB_INVALID_ARGUMENT, "fb_plan_execute: NULL plan or device");
  return execute_plan(plan, plan->plan, dev, args, arg_bytes, num_args, workspace, workspace_bytes);
}

// The plan for these extents: the loaded one when they are its own, else a specialisation (kept).
static fb_status shaped_plan(fb_plan *plan, const int64_t *arg_dims, int32_t num_args,
                             std::shared_ptr<const Plan> *out) {
  const Plan &base = plan->plan;
  FB_REQUIRE(num_args == base.num_args, FB_VARIANT_PACK_ERROR,
             "expected " + std::to_string(base.num_args) + " buffers, got " + std::to_string(num_args));
  FB_REQUIRE(arg_dims != nullptr || num_args == 0, FB_INVALID_ARGUMENT, "arg_dims is NULL");
  bool same = true;
  std::vector<int64_t> key;
  for (int a = 0; a < num_args; ++a) {
    const TensorInfo &t = base.tensors[base.arg_tensor[a]];
    for (int k = 0; k < t.rank; ++k) {
      const int64_t v = arg_dims[(size_t)a * FB_MAX_RANK + k];
      key.push_back(v);
      same = same && v == t.dims[k];
    }
  }
  if (same) {
    // the loaded plan itself: aliasing pointer without ownership (it lives as long as `plan`)
    *out = std::shared_ptr<const Plan>(std::shared_ptr<const Plan>(), &base);
    return FB_OK;
  }
  std::lock_guard<std::mutex> lock(plan->mu);
  auto it = plan->shaped.find(key);
  if (it == plan->shaped.end()) {
    auto sp = std::make_shared<Plan>();
    fb_status st = specialize(base, arg_dims, *sp);
    if (st != FB_OK) return st;
    if (plan->shaped.size() >= fb_plan::kMaxShaped) plan->shaped.clear();
    it = plan->shaped.emplace(std::move(key), std::shared_ptr<const Plan>(std::move(sp))).first;
  }
  *out = it->second;
  return FB_OK;
}

FB_EXPORT fb_status fb_plan_execute_shaped(fb_plan *plan, fb_device *dev, void *const *args,
                                           const size_t *arg_bytes, const int64_t *arg_dims,
                                           int32_t num_args, void *workspace, size_t workspace_bytes) {
  clear_error();
  FB_REQUIRE(plan && dev, FB_INVALID_ARGUMENT, "fb_plan_execute_shaped: NULL plan or device");
  std::shared_ptr<const Plan> p;
  fb_status st = shaped_plan(plan, arg_dims, num_args, &p);
  if (st != FB_OK) return st;
  return execute_plan(plan, *p, dev, args, arg_bytes, num_args, workspace, workspace_bytes);
}

FB_EXPORT fb_status fb_plan_workspace_size_shaped(fb_plan *plan, const int64_t *arg_dims, int32_t num_args,
                                                  size_t *bytes) {
  clear_error();
  FB_REQUIRE(plan && bytes, FB_INVALID_ARGUMENT, "fb_plan_workspace_size_shaped: NULL argument");
  std::shared_ptr<const Plan> p;
  fb_status st = shaped_plan(plan, arg_dims, num_args, &p);
  if (st != FB_OK) return st;
  *bytes = p->workspace_bytes;
  return FB_OK;
}
